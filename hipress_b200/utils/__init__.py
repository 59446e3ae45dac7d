"""Synthetic data, device timing, clock sampling and metrics helpers."""
from .clocks import ClockSampler
from .data import PinnedBatches, synthetic_images, synthetic_mlm
from .timing import DeviceTimer, flush_l2, max_over_ranks

__all__ = ["ClockSampler", "DeviceTimer", "PinnedBatches", "flush_l2", "max_over_ranks",
           "synthetic_images", "synthetic_mlm"]
