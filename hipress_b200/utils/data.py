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
