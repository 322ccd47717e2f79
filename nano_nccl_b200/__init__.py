"""nano_nccl_b200 — Python layer of b200ccl, a Blackwell-native collective library with the
capabilities of nano-nccl (AllReduce / ReduceScatter / AllGather over float, fp16, bf16 with
sum/avg/max/min), driven from PyTorch.

Layout: ``communicator`` (ctypes binding of the C++ communicator), ``ops`` (torch custom ops),
``parallel`` (bucketed gradient all-reduce, data-parallel wrapper), ``models`` (synthetic tensor
stacks shaped like real models, for benchmarks), ``utils`` (timing, clocks, simulator binding).
"""
from ._lib import B200CclError, lib_path, load  # noqa: F401
from .communicator import Communicator  # noqa: F401

__all__ = ["Communicator", "B200CclError", "load", "lib_path"]
__version__ = "0.1.0"
