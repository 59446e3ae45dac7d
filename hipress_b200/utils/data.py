"""Synthetic inputs of the benchmark shapes, staged in pinned host memory."""
from __future__ import annotations

from typing import List, Tuple

import torch


def synthetic_images(batch: int, classes: int = 1000, hw: int = 224, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 NCHW images ~ N(0,1) and uniform labels, on the host."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, 3, hw, hw, generator=g)
    y = torch.randint(0, classes, (batch,), generator=g)
    return x, y


def synthetic_mlm(batch: int, seq: int = 128, vocab: int = 30522, mask_rate: float = 0.15,
                  seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token ids uniform over the vocabulary; 15 % of the positions are MLM targets
    (labels hold the original id there and -100 elsewhere; masked inputs become id 103)."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    k = max(1, int(round(seq * mask_rate)))
    labels = torch.full_like(ids, -100)
    for b in range(batch):
        pos = torch.randperm(seq, generator=g)[:k]
        labels[b, pos] = ids[b, pos]
        ids[b, pos] = 103
    return ids, labels


class PinnedBatches:
    """A small ring of distinct batches in pinned host memory; ``next(device)`` issues the
    host-to-device copies of one batch on the current stream and returns device tensors."""

    def __init__(self, batches: List[Tuple[torch.Tensor, ...]]):
        self.batches = [tuple(t.pin_memory() if torch.cuda.is_available() else t for t in b) for b in batches]
        self.i = 0
        self.bytes_per_batch = sum(t.numel() * t.element_size() for t in self.batches[0])

    def next(self, device) -> Tuple[torch.Tensor, ...]:
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return tuple(t.to(device, non_blocking=True) for t in b)


class Prefetcher:
    """Stages the *next* batch host-to-device on a side stream while the current step computes.

    ``next()`` returns device tensors of one batch.  Every batch is copied from pinned memory
    (each step's input does cross PCIe), but on a copy stream that runs alongside the previous
    step's kernels instead of in front of this step's.  The device buffers are a fixed ring
    allocated once: a slot is overwritten only after the consumer stream has passed the point
    where the batch it held was last used, which the ring learns at the following ``next()``.
    No allocator call happens per step (a per-step allocation would stall the pipeline: the
    host runs several steps ahead of the device).
    """

    def __init__(self, pinned: PinnedBatches, device, depth: int = 3):
        self.pinned = pinned
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device)
        proto = pinned.batches[0]
        self.ring = [tuple(torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in proto)
                     for _ in range(depth)]
        self.copied = [torch.cuda.Event() for _ in range(depth)]
        self.released = [None] * depth
        self.head = 0          # slot handed out by the next call
        self.last = None       # slot handed out by the previous call
        self._issue(self.head)

    def _issue(self, slot: int) -> None:
        b = self.pinned.batches[self.pinned.i % len(self.pinned.batches)]
        self.pinned.i += 1
        if self.released[slot] is not None:
            self.stream.wait_event(self.released[slot])
        with torch.cuda.stream(self.stream):
            for dst, src in zip(self.ring[slot], b):
                dst.copy_(src, non_blocking=True)
            self.copied[slot].record(self.stream)

    def next(self) -> Tuple[torch.Tensor, ...]:
        cur = torch.cuda.current_stream(self.device)
        if self.last is not None:
            # everything that used the previous batch has been enqueued by now
            ev = torch.cuda.Event()
            ev.record(cur)
            self.released[self.last] = ev
        slot = self.head
        cur.wait_event(self.copied[slot])
        self.last = slot
        self.head = (slot + 1) % len(self.ring)
        self._issue(self.head)
        return self.ring[slot]
