"""Whole forward + backward of a data-parallel wrapper captured in one CUDA graph.

At the batch sizes this framework is benchmarked on (64 images or 32 sequences per GPU) a
B200 finishes the kernels of a training step faster than eager PyTorch can launch them: the
step time is the host's, not the device's.  ``GraphedTrainStep`` captures the model's forward,
loss and backward once (static input buffers, gradients accumulating into the wrapper's flat
gradient buffer exactly as in eager mode) and replays them with a single launch per step.  The
gradient exchange itself stays outside the graph: its kernels take the step's epoch (flag
values, slot parity, rounding seed) as arguments, which a replayed graph could not change.
After the replay every bucket is handed to the engine at once; on NVLink the exchange of a
whole model is a few hundred microseconds, so losing the overlap with backward costs less
than the launch gaps it removes.

The reference has no training loop (its caller drives ``submit_task`` per tensor,
ref hp_cuda.cpp:776-853); this is part of the data-parallel layer built on top of the codecs.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedTrainStep:
    """``loss = step(*inputs)`` runs one full training step: copy the inputs into the captured
    buffers, replay forward + backward, exchange and apply the gradients.

    ``fn(module, *inputs)`` must return the scalar loss (it chooses its own autocast).
    ``ddp`` is any wrapper of this package (``begin_step`` / ``step`` / ``grad_buffers``).
    The returned loss tensor is the graph's static output: read it before the next call.
    """

    def __init__(self, ddp, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        self.ddp = ddp
        self.fn = fn
        self.static_inputs = [t.clone() for t in example_inputs]
        saved = [g.clone() for g in ddp.grad_buffers()]
        ddp.hooks_enabled = False
        try:
            side = torch.cuda.Stream(device=self.static_inputs[0].device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):      # lets cuDNN pick its algorithms outside the capture
                    fn(ddp.module, *self.static_inputs).backward()
            torch.cuda.current_stream().wait_stream(side)
            self._restore(saved)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.loss = fn(ddp.module, *self.static_inputs)
                self.loss.backward()
            self._restore(saved)
        finally:
            ddp.hooks_enabled = True

    def _restore(self, saved) -> None:
        with torch.no_grad():
            for g, s in zip(self.ddp.grad_buffers(), saved):
                g.copy_(s)

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self.ddp.begin_step()
        self.ddp.hooks_enabled = False       # nothing fires during a replay; guards an eager fallback
        try:
            self.graph.replay()
        finally:
            self.ddp.hooks_enabled = True
        self.ddp.step()
        return self.loss
