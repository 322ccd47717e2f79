"""Synthetic tensor stacks shaped like real models (no weights are downloaded)."""
from .gpt2 import TinyGPT2, gpt2_small_shapes  # noqa: F401
