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
    # the early credit of small slices is posted only after every thread holds its part of the slot
    early = ring[ring.index("if (early) {"):ring.index("auto combine_store")]
    assert early.index("ld16_volatile(") < early.index("__syncthreads_or(") < early.index("st_release_sys(st.ch.recv_head")


def test_low_latency_kernel_waits_are_bounded_and_flags_travel_with_the_data():
    ll = read(os.path.join(KERNELS, "ll_allreduce.cu"))
    # one 8-byte store carries data and call number; one 8-byte load polls them
    assert "st.relaxed.sys.global.v2.u32" in ll and "ld.relaxed.sys.global.v2.u32" in ll
    spin = ll[ll.index("while (pending != 0u)"):]
    spin = spin[:spin.index("float acc[")]
    # all sources' slots are loaded before the first comparison, so the polls overlap
    assert spin.index("ld_slot(") < spin.index("== flag")
    assert "abort_flag" in spin and "timeout_ns" in spin and "kStatusTimeout" in spin and spin.count("break;") >= 2
    assert "cooperative" in ll.lower(), "emulated ranks wait on one another: they must share one cooperative launch"


def test_bench_profiling_is_off_by_default_and_starts_after_warm_up():
    # Same contract as the reference's tests/bench_profiling_static.py: numbers never come from an
    # instrumented build, and the profiler window excludes warm-up.
    cmake = read(os.path.join(ROOT, "CMakeLists.txt"))
    assert re.search(r"option\(B200CCL_ENABLE_BENCH_PROFILING [^)]* OFF\)", cmake)
    assert re.search(r"option\(B200CCL_ENABLE_TIMELINE [^)]* OFF\)", cmake)
    runner = read(os.path.join(ROOT, "src", "collective", "bench_runner.cu"))
    assert runner.index("config.warmup_iters") < runner.index("ProfilerSession session")
    prof = read(os.path.join(ROOT, "src", "collective", "bench_profiling.h"))
    assert "#if defined(B200CCL_ENABLE_BENCH_PROFILING)" in prof and "cudaProfilerStart" in prof


def test_only_sm_100a_is_built():
    cmake = read(os.path.join(ROOT, "CMakeLists.txt"))
    assert cmake.count("-gencode") == 1 and "arch=compute_100a,code=sm_100a" in cmake and "-lineinfo" in cmake
    assert 'NOT B200CCL_CUDA_ARCH STREQUAL "100a"' in cmake and "FATAL_ERROR" in cmake
    entry = read(os.path.join(ROOT, "__graft_entry__.py"))
    assert "sm_100a" in entry or "cmake" in entry


def test_mpi_adapter_uses_the_c_api_only():
    # tests/mpi_c_api_link_static.py of the reference: no C++ bindings, C component only.
    adapter = read(os.path.join(ROOT, "src", "bootstrap", "mpi", "mpi_bootstrap.cc"))
    assert "MPI::" not in adapter and "mpicxx" not in adapter
    cmake = read(os.path.join(ROOT, "CMakeLists.txt"))
    assert "find_package(MPI REQUIRED COMPONENTS C)" in cmake and "MPI::MPI_C" in cmake and "MPI_CXX" not in cmake


def test_rdma_proxy_contracts():
    proxy = read(os.path.join(ROOT, "src", "transport", "rdma", "proxy.cc"))
    backend = read(os.path.join(ROOT, "src", "transport", "rdma", "verbs", "ibverbs_backend.cc"))
    header = read(os.path.join(ROOT, "src", "transport", "rdma", "verbs_backend.h"))
    gdr = read(os.path.join(ROOT, "src", "transport", "rdma", "gdr.cc"))
    # multi-flight with selective signalling; the queue pair never signals everything
    assert "max_flight()" in proxy and "kSignalEvery" in proxy and "window_full" in proxy and "burst_tail" in proxy
    assert "init.sq_sig_all = 0" in backend and "kMaxInlineData = 64" in header
    # the payload goes out straight from the FIFO slot: no bounce copy anywhere in the send path
    assert "wr.local_addr = fifo_.data + slot * fifo_.slot_bytes" in proxy and "wr.lkey = fifo_.mr.lkey" in proxy
    send_path = proxy[proxy.index("// 2. Post what the kernel has published"):proxy.index("qp_->post_send(wr);")]
    assert "memcpy" not in send_path
    # zero-byte slices never reach the network
    assert proxy.count("zero_payload_posts_.fetch_add") >= 2
    # WRITE plane: the grant is cleared at post time and goes inline; payloads carry their size as immediate data
    assert "WrOpcode::RdmaWriteWithImm" in proxy and "wr.imm = bytes" in proxy and "wr.inline_data = true" in proxy
    assert proxy.index("wr.imm = bytes") < proxy.index("__atomic_store_n(&grant.ready, 0u") < proxy.index("qp_->post_send(wr);")
    # device-memory FIFOs: registration failure is an error, never a silent host fallback
    gdr_branch = gdr[gdr.index("FifoPlacement::Gdr"):gdr.index("} else {")]
    assert "register_device_memory" in gdr_branch and "host_" not in gdr_branch
    assert "ibv_reg_dmabuf_mr" in backend and "unavailable" in backend


def test_transport_kinds_and_parser_contract():
    types_h = read(os.path.join(ROOT, "include", "b200ccl", "types.h"))
    assert re.search(r"enum class TransportKind[^}]*Socket[^}]*Rdma[^}]*Mixed", types_h)
    types_cc = read(os.path.join(ROOT, "src", "core", "types.cc"))
    parse = types_cc[types_cc.index("bool parse_transport"):]
    parse = parse[:parse.index("\n}\n")]
    assert '"rdma"' in parse and '"socket"' not in parse and '"mixed"' not in parse
