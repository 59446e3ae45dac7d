"""Uncompressed baseline: flat 25 MB buckets all-reduced with NCCL, then this framework's
fused SGD-momentum kernel.  Same wrapper interface as ``CompressedDataParallel`` so that a
benchmark can swap the synchroniser and nothing else.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _C
from .ddp import _view_like, plan_buckets, ALIGN


class NcclDataParallel(nn.Module):
    def __init__(self, module: nn.Module, *, lr: float = 0.1, momentum: float = 0.9,
                 weight_decay: float = 0.0, bucket_mb: float = 25.0, optimizer: str = "sgd",
                 betas=(0.9, 0.999), eps: float = 1e-8,
                 process_group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.module = module
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.device = self.params[0].device
        bucket_elems = max(ALIGN, int(bucket_mb * (1 << 20) / 4) // ALIGN * ALIGN)
        self.plan = plan_buckets([p.numel() for p in self.params], bucket_elems)
        n = self.plan.total
        self.flat_param = torch.zeros(n, device=self.device)
        self.flat_grad = torch.zeros(n, device=self.device)
        self.flat_momentum = torch.zeros(n, device=self.device)
        self.optimizer, self.betas, self.eps = optimizer, betas, eps
        self.flat_second = torch.zeros(n, device=self.device) if optimizer == "adamw" else None
        with torch.no_grad():
            for p, off in zip(self.params, self.plan.offsets):
                view = _view_like(self.flat_param[off:off + p.numel()], p)
                view.copy_(p.data)
                p.data = view
                p.grad = _view_like(self.flat_grad[off:off + p.numel()], p)
        if self.world > 1:
            dist.broadcast(self.flat_param, src=0, group=process_group)
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.pending = [b[2] for b in self.plan.buckets]
        self.handles = []
        self.comm_stream = torch.cuda.Stream(device=self.device)
        self.steps = 0
        self.launches = 0
        self.hooks_enabled = True
        for i, p in enumerate(self.params):
            p.register_post_accumulate_grad_hook(self._make_hook(i))

    def _make_hook(self, index: int):
        def hook(_p):
            if not self.hooks_enabled:
                return
            b = self.plan.param_bucket[index]
            self.pending[b] -= 1
            if self.pending[b] == 0:
                self._launch(b)
        return hook

    def _launch(self, b: int) -> None:
        off, numel, _ = self.plan.buckets[b]
        g = self.flat_grad[off:off + numel]
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            if self.world > 1:
                dist.all_reduce(g, group=self.group)
            if self.optimizer == "adamw":
                _C.adamw_apply(g, self.flat_param[off:off + numel], self.flat_momentum[off:off + numel],
                               self.flat_second[off:off + numel], 1.0 / self.world, self.lr, self.betas[0],
                               self.betas[1], self.eps, self.weight_decay, self.steps + 1, True)
            else:
                _C.sgd_apply(g, self.flat_param[off:off + numel], self.flat_momentum[off:off + numel],
                             1.0 / self.world, self.lr, self.momentum, self.weight_decay, self.steps == 0, True)
            self.launches += 1

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def begin_step(self) -> None:
        """Nothing to arm: buckets are counted down by the hooks and flushed by ``step``."""

    def grad_buffers(self):
        return [self.flat_grad]

    def step(self) -> None:
        for b, left in enumerate(self.pending):
            if left > 0:
                self._launch(b)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self.pending = [b[2] for b in self.plan.buckets]
        self.steps += 1            # the fused optimizer kernels left zeros in flat_grad

    def check(self) -> None:
        torch.cuda.synchronize()

    def metrics(self) -> Dict[str, float]:
        return {"kernel_launches": self.launches, "steps": self.steps, "buckets": len(self.plan.buckets)}
