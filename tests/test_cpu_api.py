"""C interface pieces that work without a GPU: names/parsers, bandwidth formulas, the planner,
and loud failure when no device exists."""
import ctypes

import pytest

from nano_nccl_b200 import _lib


@pytest.fixture(scope="module")
def lib(native_build):
    return _lib.load()


def test_names_and_parsers(lib):
    v = ctypes.c_int()
    assert lib.b2_parse_dtype(b"bf16", ctypes.byref(v)) == 0 and v.value == 2
    assert lib.b2_parse_dtype(b"int8", ctypes.byref(v)) != 0
    assert lib.b2_parse_redop(b"min", ctypes.byref(v)) == 0 and v.value == 3
    assert lib.b2_parse_transport(b"socket", ctypes.byref(v)) != 0  # reported, never requested
    assert lib.b2_transport_name(3) == b"socket"
    assert lib.b2_parse_algo(b"ring_simple", ctypes.byref(v)) == 0 and lib.b2_algo_name(v.value) == b"ring"


def test_busbw(lib):
    assert lib.b2_busbw_gbs(0, 100.0, 8) == pytest.approx(175.0)
    assert lib.b2_busbw_gbs(1, 100.0, 8) == pytest.approx(87.5)
    assert lib.b2_busbw_gbs(2, 100.0, 2) == pytest.approx(50.0)


def _plan(lib, coll, count, flags, nranks=8, redop=0, forced=0):
    out = (ctypes.c_int * 5)()
    rc = lib.b2_make_plan(coll, 0, redop, nranks, count, flags, forced, out)
    return rc, list(out)


def test_planner(lib):
    WIDE, RD, WR, IMC, OMC, INPLACE, RING = 1, 2, 4, 8, 16, 32, 64
    rc, p = _plan(lib, 0, 1024, WIDE | RD | WR)
    assert rc == 0 and p[0] == 1 and p[2] == 0  # small → one-shot, no staging
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR)
    assert rc == 0 and p[0] == 2 and p[1] > 1  # large → two-shot on many CTAs
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR | IMC | OMC)
    assert rc == 0 and p[0] == 3  # symmetric + multicast → NVLS
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR | IMC | OMC, redop=2)
    assert rc == 0 and p[0] == 2  # max never uses the switch (NaN propagation is done in fp32 here)
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR | IMC | OMC, nranks=2)
    assert rc == 0 and p[0] == 2  # two ranks: direct peer access wins
    rc, p = _plan(lib, 0, 1 << 24, WIDE)
    assert rc == 0 and p[2] == 1 and p[3] == 1  # buffers of another process → staged both ways
    rc, p = _plan(lib, 0, 1024, WIDE | RD | WR | INPLACE)
    assert rc == 0 and p[0] == 2  # in place never one-shot on directly read buffers
    rc, p = _plan(lib, 0, 1024, WIDE | RD | WR | INPLACE, forced=1)
    assert rc == 2
    rc, p = _plan(lib, 0, 1024, WIDE | RING)
    assert rc == 0 and p[0] == 4
    rc, p = _plan(lib, 2, 1 << 20, WIDE | RD | WR)
    assert rc == 0 and p[4] == 0  # all_gather pushes when peers can be written
    rc, p = _plan(lib, 2, 1 << 20, WIDE)
    assert rc == 0 and p[4] == 1 and p[2] == 1  # else pulls from the staged inputs
    rc, p = _plan(lib, 0, 1 << 20, WIDE, forced=3)
    assert rc == 2 and b"nvls" in lib.b2_last_error()


def test_planner_low_latency(lib, monkeypatch):
    WIDE, RD, WR, WORD = 1, 2, 4, 128
    monkeypatch.delenv("B200CCL_LL_MAX_BYTES", raising=False)
    rc, p = _plan(lib, 0, 1024, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 1  # off unless asked for
    rc, p = _plan(lib, 0, 1024, WORD, forced=5)
    assert rc == 0 and p[0] == 5 and p[1] == 8 and p[2] == 0 and p[3] == 0  # no staging even for private buffers
    rc, p = _plan(lib, 0, 8192, WORD, forced=5)
    assert rc == 0 and p[0] == 5  # 32 KiB of floats still fits
    rc, p = _plan(lib, 0, 8193, WORD, forced=5)
    assert rc == 2 and b"32 KiB" in lib.b2_last_error()
    rc, p = _plan(lib, 0, 1024, WIDE, forced=5)
    assert rc == 2  # not 4-byte aligned
    rc, p = _plan(lib, 1, 1024, WIDE | RD | WR | WORD, forced=5)
    assert rc == 0 and p[0] != 5  # all_reduce only
    monkeypatch.setenv("B200CCL_LL_MAX_BYTES", "16K")
    rc, p = _plan(lib, 0, 4096, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 5
    rc, p = _plan(lib, 0, 4097 + 3, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] != 5  # above the threshold: the usual choice
    monkeypatch.setenv("B200CCL_LL_MAX_BYTES", "1M")  # clamped to the slot capacity
    rc, p = _plan(lib, 0, 8192, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 5
    rc, p = _plan(lib, 0, 16384, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] != 5


def test_no_gpu_is_a_loud_error(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    cfg = _lib.B2Config()
    lib.b2_config_default(ctypes.byref(cfg))
    devs = (ctypes.c_int * 1)(0)
    handle = ctypes.c_void_p()
    rc = lib.b2_comm_create(devs, 1, ctypes.byref(cfg), ctypes.byref(handle))
    assert rc != 0 and b"CUDA" in lib.b2_last_error()


def test_cta_cap_from_the_environment(lib, monkeypatch):
    WIDE, RD, WR, IMC, OMC = 1, 2, 4, 8, 16
    monkeypatch.delenv("B200CCL_MAX_CTAS", raising=False)
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR | IMC | OMC)
    assert rc == 0 and p[0] == 3 and p[1] == 64  # measured default for the multimem kernel
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR)
    assert rc == 0 and p[0] == 2 and p[1] == 128  # and for two-shot
    monkeypatch.setenv("B200CCL_MAX_CTAS", "16")  # leave SMs to kernels that run beside the collective
    for flags in (WIDE | RD | WR | IMC | OMC, WIDE | RD | WR):
        rc, p = _plan(lib, 0, 1 << 24, flags)
        assert rc == 0 and p[1] == 16
    cfg = _lib.B2Config()
    lib.b2_config_default(ctypes.byref(cfg))
    assert cfg.max_ctas == 0 and cfg.enable_nvls == 1
