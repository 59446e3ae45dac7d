"""Device-side timing helpers (CUDA events on the launching stream, max over ranks)."""
from __future__ import annotations

import torch
import torch.distributed as dist

_L2_FLUSH = {}


def flush_l2(device=None) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _L2_FLUSH.get(device)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        _L2_FLUSH[device] = buf
    buf.zero_()


class DeviceTimer:
    """``with DeviceTimer() as t: ...`` then ``t.ms`` (synchronises on both sides)."""

    def __init__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.stop = torch.cuda.Event(enable_timing=True)
        self.ms = 0.0

    def __enter__(self):
        torch.cuda.synchronize()
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.stop.record()
        torch.cuda.synchronize()
        self.ms = self.start.elapsed_time(self.stop)
        return False


def max_over_ranks(value: float, device=None) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], device=device or torch.device("cuda", torch.cuda.current_device()),
                     dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
