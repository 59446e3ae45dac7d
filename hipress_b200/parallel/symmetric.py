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
                 group: Optional[dist.ProcessGroup] = None, multicast: bool = False):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.nbytes = int(nbytes)
        self.multicast = False
        self._keep = None
        if multicast and self.world > 1 and self._try_multicast(group):
            return
        self.buf = _C.SymmetricBuffer(self.nbytes, self.rank, self.world, self.device.index)
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, self.buf.export_handle(), group=group)
            self.buf.open_peers(handles)
            # nobody may store into a peer before that peer has zeroed and exported its buffer
            dist.barrier(group=group)

    def _try_multicast(self, group) -> bool:
        """Allocate through torch's symmetric-memory allocator, which maps every peer's buffer and,
        where the GPUs sit behind an NVLink switch with multicast (NVLS), binds them to one
        multicast object: a store to ``multicast_ptr + offset`` lands at ``offset`` in every
        rank's buffer.  Returns False (and leaves nothing behind) when that is not available, so
        that the caller falls back to plain peer mappings."""
        self.multicast_note = ""
        try:
            import torch.distributed._symmetric_memory as tsm
            if not _C.multicast_supported(self.device.index):
                self.multicast_note = "CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED is 0 on this device"
                return False
            pg = group if group is not None else dist.group.WORLD
            t = tsm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            handle = tsm.rendezvous(t, group=pg)
            mc = int(handle.multicast_ptr or 0)
            if mc == 0:
                self.multicast_note = "the allocator returned no multicast mapping"
                return False
            t.zero_()
            torch.cuda.synchronize(self.device)
            bases = [int(p) for p in handle.buffer_ptrs]
            self.buf = _C.SymmetricBuffer(bases, mc, self.nbytes, self.rank, self.world)
            self._keep = (t, handle)     # the allocation must outlive every kernel that stores into it
            self.multicast = True
            dist.barrier(group=group)    # nobody stores into a peer before that peer has zeroed its buffer
            return True
        except Exception as exc:  # any failure of the optional path: plain peer mappings instead
            self.multicast_note = f"{type(exc).__name__}: {exc}"[:200]
            return False

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
