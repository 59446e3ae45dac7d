"""Synthetic data, device timing, clock sampling and metrics helpers."""
from .clocks import ClockSampler
from .data import PinnedBatches, Prefetcher, synthetic_images, synthetic_mlm
from .timing import DeviceTimer, flush_l2, max_over_ranks

__all__ = ["ClockSampler", "DeviceTimer", "PinnedBatches", "Prefetcher", "flush_l2", "max_over_ranks",
           "synthetic_images", "synthetic_mlm"]
