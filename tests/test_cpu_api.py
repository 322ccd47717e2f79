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
    assert rc == 0 and p[0] == 5  # small messages: no barrier at all
    rc, p = _plan(lib, 0, 16384 + 4, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] != 5  # above 64 KiB: the usual choice
    monkeypatch.setenv("B200CCL_LL_MAX_BYTES", "0")
    rc, p = _plan(lib, 0, 1024, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 1  # switched off: one-shot
    monkeypatch.delenv("B200CCL_LL_MAX_BYTES")
    rc, p = _plan(lib, 0, 1024, WORD, forced=5)
    assert rc == 0 and p[0] == 5 and p[1] == 8 and p[2] == 0 and p[3] == 0  # no staging even for private buffers
    rc, p = _plan(lib, 0, 32768, WORD, forced=5)
    assert rc == 0 and p[0] == 5  # 128 KiB of floats still fits
    rc, p = _plan(lib, 0, 32769, WORD, forced=5)
    assert rc == 2 and b"128 KiB" in lib.b2_last_error()
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
    rc, p = _plan(lib, 0, 32768, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 5
    rc, p = _plan(lib, 0, 65536, WIDE | RD | WR | WORD)
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
    assert rc == 0 and p[0] == 3 and p[1] == 48  # measured default for the multimem kernel
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR)
    assert rc == 0 and p[0] == 2 and p[1] == 128  # and for two-shot
    monkeypatch.setenv("B200CCL_MAX_CTAS", "16")  # leave SMs to kernels that run beside the collective
    for flags in (WIDE | RD | WR | IMC | OMC, WIDE | RD | WR):
        rc, p = _plan(lib, 0, 1 << 24, flags)
        assert rc == 0 and p[1] == 16
    cfg = _lib.B2Config()
    lib.b2_config_default(ctypes.byref(cfg))
    assert cfg.max_ctas == 0 and cfg.enable_nvls == 1


def test_tuning_file(lib, monkeypatch, tmp_path):
    WIDE, RD, WR, IMC, OMC, WORD = 1, 2, 4, 8, 16, 128
    path = tmp_path / "b200.tuning"
    path.write_text("# measured on some machine\noneshot_max_bytes.8 = 64K   # eight ranks\nnvls_min_bytes = 1M\n"
                    "nvls_max_ctas = 40\nll_max_bytes = 4K\n\n")
    monkeypatch.setenv("B200CCL_TUNING_FILE", str(path))
    for var in ("B200CCL_MAX_CTAS", "B200CCL_LL_MAX_BYTES", "B200CCL_NVLS_MIN_BYTES", "B200CCL_ONESHOT_MAX_BYTES"):
        monkeypatch.delenv(var, raising=False)
    rc, p = _plan(lib, 0, 8192, WIDE | RD | WR | IMC | OMC)          # 32 KiB: one-shot now (default: multimem)
    assert rc == 0 and p[0] == 1
    rc, p = _plan(lib, 0, 8192, WIDE | RD | WR | IMC | OMC, nranks=4)  # other rank counts keep their default
    assert rc == 0 and p[0] == 2                                      # (8 KiB one-shot limit there, multimem from 1 MiB)
    rc, p = _plan(lib, 0, 1 << 24, WIDE | RD | WR | IMC | OMC)
    assert rc == 0 and p[0] == 3 and p[1] == 40
    rc, p = _plan(lib, 0, 512, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 5                                      # low-latency kernel switched on by the file
    monkeypatch.setenv("B200CCL_LL_MAX_BYTES", "0")                   # the environment still has the last word
    rc, p = _plan(lib, 0, 512, WIDE | RD | WR | WORD)
    assert rc == 0 and p[0] == 1
    path.write_text("nvls_min_bytes = 1M\nwarp_speed = 9\n")
    rc, p = _plan(lib, 0, 512, WIDE | RD | WR)
    assert rc == 2 and b"b200.tuning:2: unknown key 'warp_speed'" in lib.b2_last_error()
    path.write_text("oneshot_max_bytes.9 = 1K\n")
    rc, p = _plan(lib, 0, 512, WIDE | RD | WR)
    assert rc == 2 and b"must be 2..8" in lib.b2_last_error()
    monkeypatch.setenv("B200CCL_TUNING_FILE", str(tmp_path / "missing"))
    rc, p = _plan(lib, 0, 512, WIDE | RD | WR)
    assert rc == 2 and b"cannot be read" in lib.b2_last_error()


def test_tuning_file_from_tuner_tables():
    import json
    import os
    from nano_nccl_b200.tuning_file import derive_tuning, format_tuning
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tables = [json.load(open(os.path.join(root, "tuning", f"b200_n{n}_all_reduce_graph.json"))) for n in (8, 4)]
    values = derive_tuning(tables)
    assert values["oneshot_max_bytes.8"] == 8192 and values["oneshot_max_bytes.4"] == 8192  # what default_tuning() encodes
    assert 16 << 10 <= values["nvls_min_bytes"] <= 256 << 10
    # a synthetic table: ll wins up to 2 KiB, one-shot up to 8 KiB, two-shot in between, multimem from 1 MiB; 48 CTAs best
    rows = []
    for size in (1024, 2048, 4096, 8192, 65536, 1 << 20, 64 << 20):
        t = {"ll": 5 if size <= 2048 else 50, "oneshot": 8 if size <= 8192 else 80 + size / 1e4,
             "twoshot": 10 + size / 1e5, "nvls": 12 + size / 2e5 if size >= 1 << 20 else 14 + size / 1e5}
        for algo, us in t.items():
            if algo == "ll" and size > 131072:
                continue
            for ctas in (48, 64):
                rows.append({"collective": "all_reduce", "algo": algo, "requested": algo, "max_ctas": ctas, "bytes": size,
                             "time_us": us * (1.0 if ctas == 48 else 1.1)})
    values = derive_tuning([{"n_gpus": 8, "rows": rows}])
    assert values == {"oneshot_max_bytes.8": 8192, "ll_max_bytes": 2048, "nvls_min_bytes": 1 << 20, "nvls_max_ctas": 48,
                      "twoshot_max_ctas": 48}
    text = format_tuning(values, "synthetic")
    assert "ll_max_bytes = 2048\n" in text and text.startswith("# b200ccl tuning file")
