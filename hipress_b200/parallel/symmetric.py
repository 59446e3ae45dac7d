"""Symmetric memory across the ranks of one node.

Each rank allocates one buffer of the same size, exports a CUDA IPC handle,
all-gathers the handles through ``torch.distributed`` and maps every peer's
buffer, after which kernels can address ``base(r) + offset`` for any rank r and
store there over NVLink.  The reference has no transport: its payloads leave
through a CPU tensor for an external one (ref hp_cuda.cpp:307, 468, 616).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _C


class SymmetricMemory:
    """A ``bytes``-sized buffer on every rank, mapped everywhere."""

    def __init__(self, nbytes: int, device: Optional[torch.device] = None,
                 group: Optional[dist.ProcessGroup] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.nbytes = int(nbytes)
        self.buf = _C.SymmetricBuffer(self.nbytes, self.rank, self.world, self.device.index)
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, self.buf.export_handle(), group=group)
            self.buf.open_peers(handles)
            # nobody may store into a peer before that peer has zeroed and exported its buffer
            dist.barrier(group=group)

    def tensor(self, rank: int, byte_offset: int, numel: int, dtype: str = "float32") -> torch.Tensor:
        """A tensor over rank ``rank``'s buffer (peer memory when ``rank`` is not this rank)."""
        return self.buf.tensor(rank, int(byte_offset), int(numel), dtype, self.device.index)

    @classmethod
    def emulate(cls, nbytes: int, world: int, device: Optional[torch.device] = None) -> List["SymmetricMemory"]:
        """``world`` buffers on one device in one process, each seeing the others as its peers.

        For tests and single-GPU development of the multi-rank protocol: ranks are then driven
        one after another on one stream, never as kernels that wait on each other.
        """
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        out = []
        for r in range(world):
            m = cls.__new__(cls)
            m.device, m.rank, m.world, m.nbytes = device, r, world, int(nbytes)
            m.buf = _C.SymmetricBuffer(m.nbytes, r, world, device.index)
            out.append(m)
        bases = [m.buf.base(m.rank) for m in out]
        for m in out:
            m.buf.adopt_peers(bases)
        return out
