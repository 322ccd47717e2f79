"""GPU tests on ONE device: N ranks are emulated by one launch (rank = blockIdx.y), which runs
the same kernels as N real GPUs with every peer pointer on the same device. Numerics are compared
with a plain PyTorch fp32 reference of the same operation. Every device wait is bounded (2 s)."""
import ctypes

import pytest
import torch

import nano_nccl_b200 as nn
from nano_nccl_b200 import _lib

pytestmark = pytest.mark.gpu

DTYPES = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-1}


def make_inputs(ranks, numel, dtype, seed=0, normal=True):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for _ in range(ranks):
        x = torch.randn(numel, device="cuda", generator=gen) if normal else torch.rand(numel, device="cuda", generator=gen) * 2 - 1
        out.append(x.to(dtype))
    return out


def reference(inputs, op):
    stack = torch.stack([t.float() for t in inputs])
    if op == "sum":
        return stack.sum(0)
    if op == "avg":
        return stack.sum(0) / len(inputs)
    if op == "max":
        return stack.max(0).values
    return stack.min(0).values


@pytest.fixture(scope="module")
def comms():
    made = {}

    def get(ranks, **kw):
        key = (ranks, tuple(sorted(kw.items())))
        if key not in made:
            made[key] = nn.Communicator(devices=[0], loopback_ranks=ranks, wait_timeout_ms=2000, **kw)
        return made[key]

    yield get
    for c in made.values():
        c.close()


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("op", ["sum", "avg", "max", "min"])
def test_all_reduce_matrix(comms, ranks, dtype, op):
    comm = comms(ranks)
    for numel in (8, 4096, 262144 + 8, 1 << 20):
        inputs = make_inputs(ranks, numel, dtype, seed=numel)
        outputs = [torch.full_like(t, float("nan")) for t in inputs]
        comm.all_reduce(outputs, inputs, op=op)
        torch.cuda.synchronize()
        comm.check_async_error()
        ref = reference(inputs, op)
        for out in outputs:
            assert (out.float() - ref).abs().max().item() <= DTYPES[dtype], (numel, comm.last_call())
        for out in outputs[1:]:
            assert torch.equal(out, outputs[0]), "ranks must hold bit-identical results"


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_forced_algorithms_and_odd_sizes(comms, algo, dtype):
    comm = comms(4, algo=algo)
    # 65537 elements: not a multiple of 16 bytes → element-wise fallback path; 3 elements: tiny.
    for numel in (3, 65537, 262146, 1 << 18):
        inputs = make_inputs(4, numel, dtype, seed=7)
        outputs = [torch.empty_like(t) for t in inputs]
        comm.all_reduce(outputs, inputs, op="sum")
        torch.cuda.synchronize()
        comm.check_async_error()
        info = comm.last_call()
        assert info["algo"] == algo
        if numel == 65537:
            assert not info["vectorized"] or algo == "ring"
        ref = reference(inputs, "sum")
        for out in outputs:
            assert (out.float() - ref).abs().max().item() <= DTYPES[dtype]


@pytest.mark.parametrize("ranks", [2, 4, 8])
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_low_latency_all_reduce(comms, ranks, dtype):
    # The flag-in-data kernel: sizes that change from call to call (so the two slot parities and
    # the per-CTA call counters are exercised with different word ranges), every operator, in place.
    comm = comms(ranks, algo="ll")
    esz = torch.empty(0, dtype=dtype).element_size()
    sizes = [4 // esz, 4096 // esz + 2, (32 << 10) // esz, 2, 1026, 8 // esz, (128 << 10) // esz, (32 << 10) // esz]
    for i, numel in enumerate(sizes):
        op = ["sum", "avg", "max", "min"][i % 4]
        inputs = make_inputs(ranks, numel, dtype, seed=100 + i)
        ref = reference(inputs, op)
        if i % 2:
            outputs = inputs
            comm.all_reduce(outputs, op=op)
        else:
            outputs = [torch.full_like(t, float("nan")) for t in inputs]
            comm.all_reduce(outputs, inputs, op=op)
        torch.cuda.synchronize()
        comm.check_async_error()
        info = comm.last_call()
        assert info["algo"] == "ll" and info["grid"] == 8 and not info["staged_in"]
        for out in outputs:
            assert (out.float() - ref).abs().max().item() <= DTYPES[dtype], (numel, op)
        for out in outputs[1:]:
            assert torch.equal(out, outputs[0])


def test_low_latency_limits_and_mixing(comms):
    comm = comms(4, algo="ll")
    big = make_inputs(4, (128 << 10) // 4 + 1, torch.float32, seed=1)
    with pytest.raises(Exception, match="128 KiB"):
        comm.all_reduce([torch.empty_like(t) for t in big], big)
    odd = make_inputs(4, 3, torch.bfloat16, seed=1)  # 6 bytes: not a whole number of words
    with pytest.raises(Exception, match="4-byte"):
        comm.all_reduce([torch.empty_like(t) for t in odd], odd)
    # Refused calls leave the communicator usable, and the kernel mixes freely with the others.
    auto = comms(4)
    for numel in (256, 1 << 16, 512):
        inputs = make_inputs(4, numel, torch.float32, seed=numel)
        ref = reference(inputs, "sum")
        for c in (comm, auto) if numel <= 8192 else (auto,):
            outputs = [torch.empty_like(t) for t in inputs]
            c.all_reduce(outputs, inputs)
            torch.cuda.synchronize()
            c.check_async_error()
            for out in outputs:
                assert (out - ref).abs().max().item() <= DTYPES[torch.float32]


@pytest.mark.parametrize("ranks", [2, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_reduce_scatter_and_all_gather(comms, ranks, dtype):
    comm = comms(ranks)
    for block in (16, 1000, 1 << 16):
        inputs = make_inputs(ranks, block * ranks, dtype, seed=block)
        rs_out = [torch.empty(block, device="cuda", dtype=dtype) for _ in range(ranks)]
        comm.reduce_scatter(rs_out, inputs, op="avg")
        ag_in = [t[:block].contiguous() for t in inputs]
        ag_out = [torch.empty(block * ranks, device="cuda", dtype=dtype) for _ in range(ranks)]
        comm.all_gather(ag_out, ag_in)
        torch.cuda.synchronize()
        comm.check_async_error()
        ref = reference(inputs, "avg")
        for r in range(ranks):
            assert (rs_out[r].float() - ref[r * block:(r + 1) * block]).abs().max().item() <= DTYPES[dtype]
            assert torch.equal(ag_out[r], torch.cat(ag_in))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("op", ["max", "min"])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "ring", "ll"])
def test_nan_propagates_through_max_and_min(comms, dtype, op, algo):
    # NaNs injected on rank 1 at indices 3, 11, 19, 27 of a 32-element message (the reference's
    # tests/public_api.cu:166-230 pattern); every dtype must return NaN exactly there.
    comm = comms(4, algo=algo)
    inputs = make_inputs(4, 32, dtype, seed=5)
    for i in (3, 11, 19, 27):
        inputs[1][i] = float("nan")
    outputs = [torch.zeros_like(t) for t in inputs]
    comm.all_reduce(outputs, inputs, op=op)
    torch.cuda.synchronize()
    expect = torch.zeros(32, dtype=torch.bool, device="cuda")
    expect[[3, 11, 19, 27]] = True
    for out in outputs:
        assert torch.equal(torch.isnan(out), expect)


def test_symmetric_tensors_and_in_place(comms):
    comm = comms(4)
    sym_in = comm.empty(1 << 16, torch.bfloat16)
    assert isinstance(sym_in, list) and len(sym_in) == 4
    inputs = make_inputs(4, 1 << 16, torch.bfloat16, seed=3)
    for s, t in zip(sym_in, inputs):
        s.copy_(t)
    comm.all_reduce(sym_in, op="sum")  # in place on symmetric memory
    torch.cuda.synchronize()
    comm.check_async_error()
    assert comm.last_call()["algo"] != "oneshot"
    ref = reference(inputs, "sum")
    for s in sym_in:
        assert (s.float() - ref).abs().max().item() <= 1e-1


def test_argument_contract(comms):
    comm = comms(2)
    a = [torch.zeros(8, device="cuda"), torch.zeros(8, device="cuda")]
    b = [torch.zeros(8, device="cuda"), torch.zeros(8, device="cuda")]
    with pytest.raises(ValueError, match="one tensor per local rank"):
        comm.all_reduce(b[:1], a[:1])
    with pytest.raises(ValueError, match="in-place"):
        comm.reduce_scatter([a[0][:4], a[1][:4]], a)
    with pytest.raises(ValueError, match="unsupported dtype"):
        comm.all_reduce([t.double() for t in b], [t.double() for t in a])
    with pytest.raises(ValueError, match="world_size blocks"):
        comm.all_gather(b, a)
    # the communicator is still usable after rejected calls
    comm.all_reduce(b, a)
    torch.cuda.synchronize()
    comm.check_async_error()
    assert "transport" in comm.describe() and comm.transport == "p2p"


def test_back_to_back_without_sync_and_other_streams(comms):
    comm = comms(4)
    inputs = make_inputs(4, 1 << 14, torch.float32, seed=11)
    outs = [[torch.empty_like(t) for t in inputs] for _ in range(6)]
    side = torch.cuda.Stream()
    for i, o in enumerate(outs):
        comm.all_reduce(o, inputs, op="sum", stream=[side] * 4 if i % 2 else None)
    torch.cuda.synchronize()
    comm.check_async_error()
    ref = reference(inputs, "sum")
    for o in outs:
        for t in o:
            assert (t - ref).abs().max().item() <= 1e-5


@pytest.mark.parametrize("transport", ["shm", "socket", "rdma"])
def test_ring_over_host_and_network_edges(transport, monkeypatch):
    # shm: FIFOs and counters in mapped host memory. socket: every ring edge loops through TCP on
    # 127.0.0.1 with real proxy threads. rdma: every edge runs the RDMA proxies over the in-process
    # verbs backend. All on one GPU with emulated ranks.
    monkeypatch.setenv("B200CCL_RDMA_BACKEND", "fake")
    comm = nn.Communicator(devices=[0], loopback_ranks=4, transport=transport, wait_timeout_ms=5000, channels=2)
    try:
        assert comm.transport == transport
        for numel in (64, 100003, 1 << 20):
            inputs = make_inputs(4, numel, torch.float32, seed=numel)
            outputs = [torch.empty_like(t) for t in inputs]
            comm.all_reduce(outputs, inputs, op="avg")
            torch.cuda.synchronize()
            comm.check_async_error()
            assert comm.last_call()["algo"] == "ring"
            ref = reference(inputs, "avg")
            for out in outputs:
                assert (out - ref).abs().max().item() <= 1e-5
    finally:
        comm.close()


def test_rdma_write_plane_and_shared_progress(monkeypatch):
    monkeypatch.setenv("B200CCL_RDMA_BACKEND", "fake")
    monkeypatch.setenv("B200CCL_RDMA_USE_WRITE", "1")
    monkeypatch.setenv("B200CCL_RDMA_SHARED_PROGRESS", "1")
    comm = nn.Communicator(devices=[0], loopback_ranks=2, transport="rdma", wait_timeout_ms=5000, channels=2)
    try:
        inputs = make_inputs(2, 300000, torch.float16, seed=1)
        outputs = [torch.empty_like(t) for t in inputs]
        comm.all_reduce(outputs, inputs, op="sum")
        torch.cuda.synchronize()
        comm.check_async_error()
        ref = reference(inputs, "sum")
        for out in outputs:
            assert (out.float() - ref).abs().max().item() <= 1e-2
    finally:
        comm.close()


def test_bounded_wait_reports_instead_of_hanging():
    lib = _lib.load()
    out = (ctypes.c_int * 4)()
    waited = ctypes.c_double()
    lib.b2_selftest_wait.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.POINTER(ctypes.c_int),
                                     ctypes.POINTER(ctypes.c_double)]
    # A flag that nothing sets: the wait must run out after about 100 ms, record TIMEOUT (1) and raise abort.
    _lib.check(lib.b2_selftest_wait(0, 0, 100.0, out, ctypes.byref(waited)))
    assert out[0] == 0 and out[1] == 1 and out[2] == 99 and out[3] == 1
    assert 90.0 <= waited.value <= 1000.0
    # The host raises the abort word while a kernel waits with a 2 s limit: ends early as ABORTED (2).
    _lib.check(lib.b2_selftest_wait(1, 0, 2000.0, out, ctypes.byref(waited)))
    assert out[0] == 0 and out[1] in (1, 2)
    if out[1] == 2:
        assert waited.value < 2000.0
    # The device is still usable afterwards.
    assert torch.ones(4, device="cuda").sum().item() == 4


def test_release_acquire_publication():
    lib = _lib.load()
    ok = ctypes.c_int()
    _lib.check(lib.b2_selftest_publication(0, 50, ctypes.byref(ok)))
    assert ok.value == 1


def test_device_send_without_a_proxy():
    # The sending side of a network edge, as a kernel on its own: payload into a mapped host FIFO
    # slot, the slot's byte count, then the tail counter; the host plays the proxy (the reference's
    # tests/public_api.cu:515-585). Forty slices wrap the four-slot FIFO ten times, so credits matter.
    lib = _lib.load()
    ok = ctypes.c_int()
    _lib.check(lib.b2_selftest_direct_send(0, 40, ctypes.byref(ok)))
    assert ok.value == 1
    assert torch.ones(4, device="cuda").sum().item() == 4
