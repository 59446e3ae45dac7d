"""Data parallelism: symmetric memory, bucket planning, the DDP wrapper, compressors."""
from .ddp import BucketPlan, CompressedDataParallel, CompressionConfig, plan_buckets, prefer_sharded
from .graphed import GraphedTrainStep
from .symmetric import SymmetricMemory

__all__ = ["BucketPlan", "CompressedDataParallel", "CompressionConfig", "GraphedTrainStep", "SymmetricMemory", "plan_buckets",
           "prefer_sharded"]
