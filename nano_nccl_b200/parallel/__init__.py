"""Data-parallel building blocks: bucket planning, a bucketed gradient all-reduce that runs on a
side stream, and a small DistributedDataParallel wrapper whose gradients live inside the buckets."""
from .bucket import BucketAllReducer, BucketPlan, CclBackend, TorchDistBackend  # noqa: F401
from .ddp import DistributedDataParallel  # noqa: F401
