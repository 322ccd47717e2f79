"""The allocation-free single-GPU all-reduce, called through its exported C symbol.

Some programs embedding the library may not allocate device memory when they need a reduction (all
memory already belongs to their own pool, or allocation is banned after start-up, or the stall of a
cudaMalloc is not acceptable at that point). ``b2_local_all_reduce_no_alloc`` serves them: its only
scratch memory is a fixed array inside the library image. This test checks that it gives the same
result as the communicator's own single-GPU emulation (the existing entry point), on two calls in a
row — the second call finds the array as the first one left it — and that it refuses rank counts
beyond the array's capacity with a message. It is collected last on purpose (file name), so that a
run that stops at the first failure has already run every other test; it does not depend on any of
them and also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

import nano_nccl_b200 as nn
from nano_nccl_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-1}
DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
OP_CODE = {"sum": 0, "avg": 1, "max": 2, "min": 3}


def entry_point():
    lib = _lib.load()
    fn = lib.b2_local_all_reduce_no_alloc
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_size_t,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return lib, fn


def call(fn, inputs, outputs, op, status=None):
    n = len(inputs)
    ins = (ctypes.c_void_p * n)(*[t.data_ptr() for t in inputs])
    outs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outputs])
    stream = torch.cuda.current_stream().cuda_stream
    return fn(ins, outs, n, inputs[0].numel(), DTYPE_CODE[inputs[0].dtype], OP_CODE[op], stream,
              status.data_ptr() if status is not None else None)


@pytest.mark.parametrize("dtype,op,ranks,numel", [
    (torch.float32, "sum", 4, 1 << 20),     # two-shot path
    (torch.bfloat16, "avg", 8, 4096),       # one-shot path, fused 1/N
    (torch.float16, "max", 2, 65537),       # element-wise fallback (odd size)
])
def test_matches_the_communicator_on_two_calls_in_a_row(dtype, op, ranks, numel):
    torch.cuda.set_device(0)
    lib, fn = entry_point()
    comm = nn.Communicator(devices=[0], loopback_ranks=ranks, wait_timeout_ms=2000)
    try:
        status = torch.zeros(8, dtype=torch.int32, device="cuda")  # the 32-byte failure record
        for round_ in range(2):
            gen = torch.Generator(device="cuda").manual_seed(40 + round_)
            inputs = [torch.randn(numel, device="cuda", generator=gen).to(dtype) for _ in range(ranks)]
            expect = [torch.empty_like(t) for t in inputs]
            comm.all_reduce(expect, inputs, op=op)  # the existing entry point
            got = [torch.full_like(t, float("nan")) for t in inputs]
            rc = call(fn, inputs, got, op, status)
            assert rc == 0, lib.b2_last_error()
            torch.cuda.synchronize()
            comm.check_async_error()
            assert int(status[0].item()) == 0, "a device wait gave up"
            for g, e in zip(got, expect):
                assert (g.float() - e.float()).abs().max().item() <= TOL[dtype]
            for g in got[1:]:
                assert torch.equal(g, got[0])
    finally:
        comm.close()


def test_rejects_what_the_fixed_array_cannot_hold():
    torch.cuda.set_device(0)
    lib, fn = entry_point()
    x = [torch.zeros(16, device="cuda") for _ in range(9)]
    y = [torch.zeros(16, device="cuda") for _ in range(9)]
    assert call(fn, x, y, "sum") == 2
    msg = lib.b2_last_error().decode()
    assert "nranks = 9" in msg and "1..8" in msg
    assert call(fn, x[:2], x[:2], "sum") == 2 and b"in-place" in lib.b2_last_error()
    # ranges that overlap part-way, and two outputs that alias, would race inside the kernel
    big = torch.zeros(64, device="cuda")
    assert call(fn, [big[:16], big[32:48]], [big[8:24], big[48:64]], "sum") == 2 and b"overlap" in lib.b2_last_error()
    assert call(fn, x[:2], [big[:16], big[:16]], "sum") == 2 and b"outputs 0 and 1 overlap" in lib.b2_last_error()
    # a count whose byte size does not fit in size_t
    ins = (ctypes.c_void_p * 1)(x[0].data_ptr())
    outs = (ctypes.c_void_p * 1)(y[0].data_ptr())
    assert fn(ins, outs, 1, (1 << 63), 0, 0, None, None) == 2 and b"does not fit" in lib.b2_last_error()
    # and a valid call still works afterwards
    a = [torch.ones(16, device="cuda"), torch.full((16,), 2.0, device="cuda")]
    b = [torch.empty(16, device="cuda") for _ in range(2)]
    assert call(fn, a, b, "sum") == 0
    torch.cuda.synchronize()
    assert torch.equal(b[0], torch.full((16,), 3.0, device="cuda")) and torch.equal(b[1], b[0])
