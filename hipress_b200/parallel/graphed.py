"""A training step replayed from one CUDA graph.

At the batch sizes this framework is benchmarked on (64 images or 32 sequences per GPU) a
B200 finishes the kernels of a training step faster than eager PyTorch can launch them: the
step time is the host's, not the device's.  ``GraphedTrainStep`` captures the step once
(static input buffers, gradients accumulating into the wrapper's flat gradient buffer exactly
as in eager mode) and replays it with a single launch.

Two capture scopes:

* **Whole step** (wrappers created with ``graph_capturable=True``: TBQ, TernGrad, ECQ, GradDrop,
  DGC and the dense codec with a fused optimizer, and PowerSGD).  The engine keeps the step's epoch -- flag
  values, slot parity, rounding / sampling seed, AdamW's step count -- in device memory, advanced
  by a one-thread kernel at the start of the step, so nothing in its launches changes from step
  to step.  The capture then contains
  ``begin_step``, forward, backward *with the gradient hooks firing* and ``step``: every bucket
  is compressed, pushed to the peers, unpacked and applied on the engine's side streams as soon
  as its gradients exist, overlapping the rest of backward, exactly as in eager mode.  PowerSGD
  alternates between two accumulator sets by epoch parity; its step is captured once per parity
  (``capture_variants``) and the two graphs, which share one memory pool, are replayed in turn.
* **Forward + backward only** (every other wrapper).  The exchange takes host-side arguments
  per step and stays outside the graph; all buckets are handed to the engine right after the
  replay.  On NVLink the exchange of a whole model costs a few hundred microseconds, less than
  the launch gaps removed.

The reference has no training loop (its caller drives ``submit_task`` per tensor,
ref hp_cuda.cpp:776-853); this is part of the data-parallel layer built on top of the codecs.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedTrainStep:
    """``loss = step(*inputs)`` runs one full training step: copy the inputs into the captured
    buffers, replay, and (forward + backward scope only) exchange and apply the gradients.

    ``fn(module, *inputs)`` must return the scalar loss (it chooses its own autocast).
    ``ddp`` is any wrapper of this package (``begin_step`` / ``step`` / ``grad_buffers``).
    The returned loss tensor is the graph's static output: read it before the next call.
    """

    def __init__(self, ddp, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        self.ddp = ddp
        self.fn = fn
        self.whole_step = bool(getattr(ddp, "graph_capturable", False))
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
            self.variants = int(getattr(ddp, "capture_variants", 1)) if self.whole_step else 1
            self.graphs, self.losses = [], []
            if self.whole_step:
                ddp.hooks_enabled = True
                pool = None
                for v in range(self.variants):
                    if self.variants > 1:
                        ddp.begin_capture_variant(v)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        ddp.begin_step()
                        loss = fn(ddp.module, *self.static_inputs)
                        loss.backward()
                        ddp.step()
                    # nothing ran: the step issued during the capture comes back out of the counters
                    self.launches_per_step = ddp.end_capture()
                    pool = g.pool()
                    self.graphs.append(g)
                    self.losses.append(loss)
                    self._restore(saved)
            else:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    loss = fn(ddp.module, *self.static_inputs)
                    loss.backward()
                self.graphs.append(g)
                self.losses.append(loss)
            self.graph, self.loss = self.graphs[0], self.losses[0]
            self._restore(saved)
        except BaseException:
            # a failed capture must leave the wrapper usable for eager steps
            if hasattr(ddp, "_in_step"):
                ddp._in_step = False
            try:
                self._restore(saved)
            except RuntimeError:
                pass                    # the original error is the one to report
            raise
        finally:
            ddp.hooks_enabled = True

    def _restore(self, saved) -> None:
        with torch.no_grad():
            for g, s in zip(self.ddp.grad_buffers(), saved):
                g.copy_(s)

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        for dst, src in zip(self.static_inputs, inputs):
            dst.copy_(src, non_blocking=True)
        if self.whole_step:
            v = self.ddp.next_variant() if self.variants > 1 else 0
            self.graphs[v].replay()
            self.ddp.note_replay(self.launches_per_step)
            return self.losses[v]
        self.ddp.begin_step()
        self.ddp.hooks_enabled = False       # nothing fires during a replay; guards an eager fallback
        try:
            self.graph.replay()
        finally:
            self.ddp.hooks_enabled = True
        self.ddp.step()
        return self.loss
