import ctypes

from .. import _lib


def ring_sim(nranks=4, channels=4, count=1 << 20, redop="sum", collective="all_reduce", fifo_bytes=4 << 20,
             stall_rank=-1, stall_after_slices=0, wait_timeout_ms=5000.0):
    """Runs the CPU ring simulator (threads = ranks x channels, no GPU) and returns its result dict."""
    lib = _lib.load()
    ops = {"sum": 0, "avg": 1, "max": 2, "min": 3}
    colls = {"all_reduce": 0, "reduce_scatter": 1, "all_gather": 2}
    cfg = (ctypes.c_longlong * 6)(nranks, channels, ops[redop], colls[collective], stall_rank, stall_after_slices)
    oi = (ctypes.c_longlong * 7)()
    od = (ctypes.c_double * 2)()
    lib.b2_ring_sim.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.c_size_t, ctypes.c_size_t, ctypes.c_double,
                                ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_double)]
    _lib.check(lib.b2_ring_sim(cfg, count, fifo_bytes, wait_timeout_ms, oi, od))
    keys = ["wrong", "timed_out", "timeout_rank", "timeout_peer", "timeout_channel", "slices", "empty_slices"]
    res = dict(zip(keys, list(oi)))
    res["seconds"], res["max_abs_error"] = od[0], od[1]
    return res
