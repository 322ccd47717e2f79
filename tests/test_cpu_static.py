"""Source-level contracts, checked as text (the reference pins similar idioms with Python static
checks, e.g. tests/avg_scale_fusion_static.py): the avg scale is fused into the reducing kernels and
no output-wide scaling pass exists; device code never traps, asserts or spins without a bound; NCCL is
not linked into the product."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KERNELS = os.path.join(ROOT, "src", "kernels", "sm100")


def read(path):
    with open(path) as f:
        return f.read()


def kernel_sources():
    return {n: read(os.path.join(KERNELS, n)) for n in sorted(os.listdir(KERNELS)) if n.endswith((".cu", ".cuh", ".h"))}


def all_sources():
    out = {}
    for base in ("src", "include", "sim", "bench"):
        for d, _, files in os.walk(os.path.join(ROOT, base)):
            for n in files:
                if n.endswith((".cu", ".cuh", ".h", ".cc", ".py")):
                    out[os.path.join(d, n)] = read(os.path.join(d, n))
    return out


def test_avg_scale_is_fused_into_the_reduction():
    direct = read(os.path.join(KERNELS, "direct_collectives.cu"))
    ring = read(os.path.join(KERNELS, "ring_simple.cu"))
    assert re.search(r"acc\[e\]\s*\*=\s*a\.scale", direct), "direct kernels scale the accumulator before the single rounding"
    assert re.search(r"acc\[e\]\s*\*=\s*a\.scale", ring) and "kScale" in ring, "ring kernel scales at the pivot slice only"
    # the scale flag is set on the pivot / final-reduce chunk and nowhere else
    assert ring.count("| kScale") == 2
    for name, text in kernel_sources().items():
        assert not re.search(r"__global__[^;{]*\bscale\w*\s*\(", text), f"{name}: a stand-alone scaling kernel is not allowed"


def test_device_code_never_traps_or_spins_unbounded():
    for name, text in kernel_sources().items():
        assert "__trap" not in text and "asm(\"trap" not in text, name
        assert not re.search(r"\bassert\s*\(", text), f"{name}: no device assert"
        if name not in ("sync.cuh", "tma.cuh", "selftest.cu"):
            # every wait goes through the bounded helpers
            assert "ld_acquire_sys(" not in text or "wait_at_least" in text, name
            assert "mbar_try_wait(" not in text, f"{name}: use mbar_wait_bounded"
    sync = read(os.path.join(KERNELS, "sync.cuh"))
    assert "timeout_ns" in sync and "kStatusTimeout" in sync and "abort_flag" in sync


def test_nccl_is_not_linked_into_the_product():
    cmake = read(os.path.join(ROOT, "CMakeLists.txt"))
    assert "nccl" not in cmake.lower().replace("b200ccl", "").replace("nano_nccl", "").replace("nano-nccl", "")
    for path, text in all_sources().items():
        if path.endswith((".cu", ".cuh", ".cc", ".h")):
            assert "#include <nccl.h>" not in text and "ncclAllReduce" not in text, path


def test_step_counters_use_system_scope_release_acquire():
    sync = read(os.path.join(KERNELS, "sync.cuh"))
    assert "ld.acquire.sys.global.u64" in sync and "st.release.sys.global.u64" in sync
    ring = read(os.path.join(KERNELS, "ring_simple.cu"))
    # data stores of the whole CTA are ordered before the counter by a block barrier, then release
    publish = ring[ring.index("// Publish:"):]
    assert publish.index("__syncthreads()") < publish.index("st_release_sys(st.ch.recv_head") < publish.index("st_release_sys(st.ch.send_tail")
