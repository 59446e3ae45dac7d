"""Deep Gradient Compression on top of the engine's sparse codec.

The reference contains only DGC's selector (``dgc_body.h``), not wired into its module.
Everything that makes it DGC is added here and in ``csrc/kernels/dgc.cu``:

* momentum correction and momentum factor masking (velocity ``u``, accumulator ``v``),
* local gradient clipping (per bucket, threshold scaled by ``world ** -0.5``),
* sparsity warm-up: the kept fraction falls exponentially from 25 % to the target over the
  first ``warmup_steps`` steps in four stages (75 %, 93.75 %, 98.4375 %, 99.6 % sparsity,
  then the target), as in the DGC paper,
* a fused AdamW (or SGD) update applied to the averaged sparse gradient.
"""
from __future__ import annotations

from typing import List, Optional

import torch.nn as nn

from .ddp import CompressedDataParallel, CompressionConfig


def warmup_schedule(target_keep: float, warmup_steps: int, stages: int = 4) -> List[tuple]:
    """[(first_step, keep_fraction)]: keep 25 %, 6.25 %, 1.5625 %, 0.39 % ... then the target."""
    sched = []
    if warmup_steps > 0:
        per = max(1, warmup_steps // stages)
        for s in range(stages):
            keep = max(target_keep, 0.25 ** (s + 1))
            sched.append((s * per, keep))
    sched.append((warmup_steps, target_keep))
    return sched


class DGCDataParallel(CompressedDataParallel):
    def __init__(self, module: nn.Module, keep_fraction: float = 0.001, *, sample_rate: float = 0.01,
                 warmup_steps: int = 400, momentum_correction: float = 0.9, clip_norm: float = 1.0,
                 lr: float = 1e-4, weight_decay: float = 0.01, optimizer: str = "adamw",
                 bucket_mb: float = 25.0, seed: int = 1, start_step: int = 0,
                 graph_capturable: bool = False, trace: bool = False, transport: str = "p2p", **kw):
        # start_step: position in the warm-up schedule of the first step (resuming a run, or
        # measuring the steady state without running the warm-up first)
        self.start_step = int(start_step)
        self.schedule = warmup_schedule(keep_fraction, warmup_steps)
        max_keep = max(k for _, k in self.schedule)
        cfg = CompressionConfig("dgc", keep_fraction=max_keep, sample_rate=sample_rate, bucket_mb=bucket_mb,
                                seed=seed, momentum_correction=momentum_correction > 0,
                                dgc_momentum=momentum_correction, clip_norm=clip_norm,
                                graph_capturable=graph_capturable, trace=trace, transport=transport)
        super().__init__(module, cfg, lr=lr, momentum=0.0, weight_decay=weight_decay, fused_sgd=True,
                         optimizer=optimizer, **kw)
        self.target_keep = keep_fraction
        self._apply_schedule(self.start_step)

    def keep_fraction_at(self, step: int) -> float:
        keep = self.schedule[0][1]
        for first, k in self.schedule:
            if step >= first:
                keep = k
        return keep

    def _apply_schedule(self, step: int) -> None:
        self.engine.set_keep_fraction(self.keep_fraction_at(step))

    def begin_step(self) -> None:
        self._apply_schedule(self.start_step + self.engine.steps)
        super().begin_step()

    def end_capture(self) -> int:
        """A captured step keeps the sparsity it was captured with: only the steady state (after the
        warm-up schedule) may be replayed from a graph."""
        step = self.start_step + self.engine.steps - 1      # the step that was just captured
        if self.keep_fraction_at(step) != self.target_keep:
            raise RuntimeError("DGC: capture the training step after the sparsity warm-up "
                               f"(step {step} of {self.schedule[-1][0]})")
        return super().end_capture()
