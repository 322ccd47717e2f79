"""CPU ring simulator: the plumbing configuration (4 ranks in one process, float32 sum, 1 Mi
elements per rank, uniform[-1,1) from seed = rank, 4 channels, Simple slice/step schedule with
step counters in host memory) checked against a host-summed reference, plus schedule coverage and
failure detection with a rank that stops (no GPU involved)."""
import ctypes

import pytest

from nano_nccl_b200 import _lib


def sim(lib, nranks=4, channels=4, redop=0, coll=0, count=1 << 20, fifo=4 << 20, stall_rank=-1, stall_after=0,
        timeout_ms=5000.0):
    cfg = (ctypes.c_longlong * 6)(nranks, channels, redop, coll, stall_rank, stall_after)
    oi = (ctypes.c_longlong * 7)()
    od = (ctypes.c_double * 2)()
    lib.b2_ring_sim.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.c_size_t, ctypes.c_size_t, ctypes.c_double,
                                ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_double)]
    rc = lib.b2_ring_sim(cfg, count, fifo, timeout_ms, oi, od)
    assert rc == 0, lib.b2_last_error()
    keys = ["wrong", "timed_out", "timeout_rank", "timeout_peer", "timeout_channel", "slices", "empty_slices"]
    res = dict(zip(keys, list(oi)))
    res["seconds"], res["max_abs"] = od[0], od[1]
    return res


@pytest.fixture(scope="module")
def lib(native_build):
    return _lib.load()


def test_plumbing_config(lib):
    r = sim(lib)
    assert r["wrong"] == 0 and not r["timed_out"] and r["max_abs"] <= 1e-5
    # 4 ranks x 4 channels, 2(n-1)+... : every thread ran 2*(n-1)+1 = 7 chunk ops... slices are counted, not guessed:
    assert r["slices"] > 0


@pytest.mark.parametrize("redop", [0, 1, 2, 3])
@pytest.mark.parametrize("nranks", [2, 3, 8])
def test_all_reduce_ops_and_ranks(lib, redop, nranks):
    r = sim(lib, nranks=nranks, redop=redop, count=70001, channels=3, fifo=64 << 10)
    assert r["wrong"] == 0 and not r["timed_out"]


@pytest.mark.parametrize("coll", [1, 2])
def test_reduce_scatter_and_all_gather(lib, coll):
    r = sim(lib, nranks=4, coll=coll, count=50001, channels=4, fifo=64 << 10)
    assert r["wrong"] == 0 and not r["timed_out"]


def test_small_fifo_wraps_many_times(lib):
    # 4 KiB FIFO = 8 steps of 128 floats: a 200k-element message wraps the FIFO hundreds of times.
    r = sim(lib, nranks=4, count=200000, channels=2, fifo=4096)
    assert r["wrong"] == 0 and r["slices"] > 1000


def test_empty_slices_are_elided(lib):
    # 5 elements over 4 channels and 4 ranks: most chunks and second slices are empty.
    r = sim(lib, nranks=4, count=5, channels=4)
    assert r["wrong"] == 0 and r["empty_slices"] > 0


def test_stopped_rank_is_detected(lib):
    # Rank 2 stops after 3 slices; its neighbours' bounded waits run out and name it.
    r = sim(lib, nranks=4, count=1 << 16, channels=2, fifo=64 << 10, stall_rank=2, stall_after=3, timeout_ms=300.0)
    assert r["timed_out"] == 1
    assert r["timeout_peer"] == 2 or r["timeout_rank"] != 2
    assert r["timeout_rank"] in (0, 1, 3)


def test_low_latency_protocol_sim():
    # The flag-in-data AllReduce on host threads: lengths change from call to call, one rank lags.
    from nano_nccl_b200.utils import ll_sim
    r = ll_sim([1, 1000, 7, 1024, 3, 512] * 10, nranks=8, ctas=2, redop="avg", slow_rank=3)
    assert r["wrong"] == 0 and not r["timed_out"] and r["max_lead"] <= 1
    r = ll_sim([64] * 8, nranks=4, stall_rank=1, stall_at_call=5, wait_timeout_ms=200.0)
    assert r["timed_out"] == 1 and r["timeout_peer"] == 1 and r["timeout_call"] == 5 and r["wrong"] == 0
    with pytest.raises(ValueError):
        ll_sim([4096], max_words=1024)
