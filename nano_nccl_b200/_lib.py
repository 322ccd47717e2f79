"""ctypes binding of libb200ccl.so (the C interface in include/b200ccl/c_api.h).

The shared library is built in-tree (nano_nccl_b200/lib/) by ``__graft_entry__.build()`` or
``cmake``; nothing here falls back to another implementation when it is missing.
"""
import ctypes
import os

_LIB = None


class B2Config(ctypes.Structure):
    _fields_ = [
        ("transport", ctypes.c_int),
        ("algo", ctypes.c_int),
        ("channels", ctypes.c_int),
        ("staging_bytes", ctypes.c_size_t),
        ("wait_timeout_ms", ctypes.c_double),
        ("loopback", ctypes.c_int),
        ("loopback_ranks", ctypes.c_int),
        ("enable_nvls", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
    ]


def lib_path():
    """libb200ccl.so beside this file. B200CCL_LIBRARY=check selects the checking variant
    (libb200ccl_check.so: test-only socket fault hook and device-side index checks compiled in);
    any other value is taken as a path."""
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
    choice = os.environ.get("B200CCL_LIBRARY", "")
    if choice == "check":
        return os.path.join(here, "libb200ccl_check.so")
    if choice:
        return choice
    return os.path.join(here, "libb200ccl.so")


def load():
    """Loads the library once and declares the argument types of every entry point."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `cmake -S . -B build -G Ninja && ninja -C build`")
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    vp, ci, cs = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.b2_last_error.restype = ctypes.c_char_p
    lib.b2_version.restype = ctypes.c_char_p
    for name in ("dtype", "redop", "transport", "algo"):
        getattr(lib, f"b2_parse_{name}").argtypes = [ctypes.c_char_p, ctypes.POINTER(ci)]
        getattr(lib, f"b2_{name}_name").argtypes = [ci]
        getattr(lib, f"b2_{name}_name").restype = ctypes.c_char_p
    lib.b2_busbw_gbs.argtypes = [ci, ctypes.c_double, ci]
    lib.b2_busbw_gbs.restype = ctypes.c_double
    lib.b2_config_default.argtypes = [ctypes.POINTER(B2Config)]
    lib.b2_config_default.restype = None
    lib.b2_bootstrap_create.argtypes = [ctypes.c_char_p, ci, ci, ci, ci, ctypes.POINTER(vp)]
    lib.b2_bootstrap_destroy.argtypes = [vp]
    lib.b2_bootstrap_destroy.restype = None
    lib.b2_bootstrap_barrier.argtypes = [vp]
    lib.b2_bootstrap_allgather.argtypes = [vp, vp, vp, cs]
    lib.b2_comm_create.argtypes = [ctypes.POINTER(ci), ci, ctypes.POINTER(B2Config), ctypes.POINTER(vp)]
    lib.b2_comm_create_bootstrap.argtypes = [vp, ctypes.POINTER(ci), ci, ctypes.POINTER(B2Config), ctypes.POINTER(vp)]
    lib.b2_comm_destroy.argtypes = [vp]
    lib.b2_comm_destroy.restype = None
    for name in ("local_ranks", "global_ranks", "first_rank", "transport", "nvls", "check_async_error"):
        getattr(lib, f"b2_comm_{name}").argtypes = [vp]
    lib.b2_comm_describe.argtypes = [vp, ctypes.c_char_p, cs]
    lib.b2_comm_describe.restype = cs
    lib.b2_collective.argtypes = [vp, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp), cs, ci, ci, ci]
    lib.b2_comm_last_call.argtypes = [vp, ctypes.POINTER(ci)]
    lib.b2_comm_ring_channel.argtypes = [vp, ci, ci, ctypes.POINTER(vp)]
    lib.b2_pointer_info.argtypes = [vp, ctypes.POINTER(ci)]
    lib.b2_comm_alloc_symmetric.argtypes = [vp, cs, ctypes.POINTER(vp)]
    lib.b2_comm_free_symmetric.argtypes = [vp, ctypes.POINTER(vp)]
    lib.b2_comm_register.argtypes = [vp, ctypes.POINTER(vp), cs]
    lib.b2_comm_unregister.argtypes = [vp, ctypes.POINTER(vp)]
    _LIB = lib
    return lib


class B200CclError(RuntimeError):
    pass


def check(code):
    if code != 0:
        msg = load().b2_last_error().decode("utf-8", "replace")
        if code == 2:
            raise ValueError(msg)
        raise B200CclError(msg)
