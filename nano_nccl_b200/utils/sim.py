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


def ll_sim(call_words, nranks=4, ctas=2, lanes=4, redop="sum", max_words=1024, slow_rank=-1, stall_rank=-1,
           stall_at_call=0, wait_timeout_ms=2000.0):
    """Runs the CPU simulator of the low-latency AllReduce protocol (threads = ranks x ctas, no GPU).
    ``call_words`` lists the length of every call in 4-byte words."""
    lib = _lib.load()
    ops = {"sum": 0, "avg": 1, "max": 2, "min": 3}
    cfg = (ctypes.c_longlong * 8)(nranks, ctas, lanes, ops[redop], max_words, slow_rank, stall_rank, stall_at_call)
    words = (ctypes.c_size_t * len(call_words))(*call_words)
    out = (ctypes.c_longlong * 6)()
    lib.b2_ll_sim.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_size_t), ctypes.c_int,
                              ctypes.c_double, ctypes.POINTER(ctypes.c_longlong)]
    _lib.check(lib.b2_ll_sim(cfg, words, len(call_words), wait_timeout_ms, out))
    keys = ["wrong", "timed_out", "timeout_rank", "timeout_peer", "timeout_call", "max_lead"]
    return dict(zip(keys, list(out)))
