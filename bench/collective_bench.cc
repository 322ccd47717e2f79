// Command-line benchmark. Flags and table columns follow nano-nccl's
// nano_nccl_all_reduce_bench (benchmarks/all_reduce_bench.cu:50-58 usage, 395-411 table); added
// are --collective, --nranks, --loopback, --symmetric, --graph, --data and --json. Exit status is
// non-zero when any row has #wrong != 0, as in the reference (all_reduce_bench.cu:414-419).
#include "b200ccl/bench.h"
#include "b200ccl/bootstrap.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

using namespace b200ccl;

namespace {

void usage(const char* argv0) {
    std::fprintf(stderr,
                 "Usage: %s [--collective all_reduce|reduce_scatter|all_gather] [--algo auto|oneshot|twoshot|nvls|ring]\n"
                 "          [--dtype float|fp16|bf16] [--redop sum|avg|max|min] [--transport auto|shm|p2p|rdma]\n"
                 "          [--nranks N] [--loopback] [--symmetric] [--graph] [--data uniform|normal]\n"
                 "          [-b bytes] [-e bytes] [-f factor] [-w warmup] [-n iters] [--json file]\n"
                 "          [--world W --rank R --addr HOST:PORT [--device D]]   one process per GPU: start W copies,\n"
                 "          ranks 0..W-1, all naming rank 0's address; inputs are the constant rank+1 (--symmetric allowed)\n",
                 argv0);
}

bool size_arg(const char* text, std::size_t* out) {
    char* end = nullptr;
    const unsigned long long v = std::strtoull(text, &end, 10);
    if (end == text) return false;
    std::size_t mult = 1;
    if (*end == 'K' || *end == 'k') mult = 1024;
    else if (*end == 'M' || *end == 'm') mult = 1024 * 1024;
    else if (*end == 'G' || *end == 'g') mult = 1024ull * 1024 * 1024;
    else if (*end != '\0') return false;
    *out = static_cast<std::size_t>(v) * mult;
    return true;
}

}  // namespace

int main(int argc, char** argv) {
    BenchConfig cfg;
    std::string json_path, addr = "127.0.0.1:29400";
    int world = 1, rank = 0, device = -1;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : nullptr; };
        bool ok = true;
        if (a == "--algo") { const char* v = next(); ok = v; if (v) cfg.algo = v; }
        else if (a == "--collective") { const char* v = next(); ok = v && parse_collective(v, &cfg.collective); }
        else if (a == "--dtype") { const char* v = next(); ok = v && parse_dtype(v, &cfg.dtype); }
        else if (a == "--redop") { const char* v = next(); ok = v && parse_redop(v, &cfg.redop); }
        else if (a == "--transport") { const char* v = next(); ok = v && parse_transport(v, &cfg.transport); }
        else if (a == "--nranks") { const char* v = next(); ok = v; if (v) cfg.nranks = std::atoi(v); }
        else if (a == "--loopback") cfg.loopback = true;
        else if (a == "--symmetric") cfg.symmetric = true;
        else if (a == "--graph") cfg.graph = true;
        else if (a == "--data") { const char* v = next(); ok = v && (!std::strcmp(v, "uniform") || !std::strcmp(v, "normal")); if (ok) cfg.uniform_data = !std::strcmp(v, "uniform"); }
        else if (a == "-b") { const char* v = next(); ok = v && size_arg(v, &cfg.min_bytes); }
        else if (a == "-e") { const char* v = next(); ok = v && size_arg(v, &cfg.max_bytes); }
        else if (a == "-f") { const char* v = next(); ok = v; if (v) cfg.factor = std::atoi(v); }
        else if (a == "-w") { const char* v = next(); ok = v; if (v) cfg.warmup_iters = std::atoi(v); }
        else if (a == "-n") { const char* v = next(); ok = v; if (v) cfg.iters = std::atoi(v); }
        else if (a == "--json") { const char* v = next(); ok = v; if (v) json_path = v; }
        else if (a == "--world") { const char* v = next(); ok = v; if (v) world = std::atoi(v); }
        else if (a == "--rank") { const char* v = next(); ok = v; if (v) rank = std::atoi(v); }
        else if (a == "--device") { const char* v = next(); ok = v; if (v) device = std::atoi(v); }
        else if (a == "--addr") { const char* v = next(); ok = v; if (v) addr = v; }
        else ok = false;
        if (!ok) { usage(argv[0]); return 2; }
    }
    Algo algo;
    if (!parse_algo(cfg.algo.c_str(), &algo)) { usage(argv[0]); return 2; }

    std::vector<BenchResult> results;
    int rc = 0;
    const bool distributed = world > 1;
    try {
        if (distributed) {
            const auto colon = addr.rfind(':');
            if (colon == std::string::npos || rank < 0 || rank >= world) { usage(argv[0]); return 2; }
            auto bootstrap = create_tcp_bootstrap(addr.substr(0, colon), std::atoi(addr.c_str() + colon + 1), rank, world);
            rc = run_distributed_bench(*bootstrap, device >= 0 ? device : rank, cfg, &results);
        } else {
            rc = run_collective_bench(cfg, &results);
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "bench failed: %s\n", e.what());
        rc = 1;
    }
    if (distributed && rank != 0) return rc;  // every process holds the same rows; rank 0 prints them
    std::printf("# b200ccl collective_bench\n");
    std::printf("# collective %s algo %s dtype %s redop %s transport %s nGpus %d warmup iters: %d iters: %d validation: 1 timing: device events, max over ranks\n",
                collective_name(cfg.collective), cfg.algo.c_str(), dtype_name(cfg.dtype), redop_name(cfg.redop),
                transport_name(cfg.transport), results.empty() ? cfg.nranks : results[0].nranks, cfg.warmup_iters, cfg.iters);
    std::printf("# %14s %8s %8s %10s %12s %12s %10s %10s %10s %8s %12s\n", "algo", "dtype", "redop", "transport", "size(B)",
                "count", "time(us)", "algbw", "busbw", "#wrong", "max_abs");
    for (const auto& r : results)
        std::printf("%16s %8s %8s %10s %12zu %12zu %10.2f %10.2f %10.2f %8lld %12.6g\n", r.algo.c_str(), dtype_name(r.dtype),
                    redop_name(r.redop), transport_name(r.transport), r.bytes, r.count, r.time_us, r.algbw, r.busbw, r.wrong,
                    r.max_abs_error);
    if (!json_path.empty()) {
        if (FILE* f = std::fopen(json_path.c_str(), "w")) {
            std::fprintf(f, "[\n");
            for (std::size_t i = 0; i < results.size(); ++i) {
                const auto& r = results[i];
                std::fprintf(f,
                             "  {\"collective\": \"%s\", \"algo\": \"%s\", \"dtype\": \"%s\", \"redop\": \"%s\", \"transport\": \"%s\", "
                             "\"nranks\": %d, \"bytes\": %zu, \"count\": %zu, \"time_us\": %.3f, \"algbw_gbs\": %.3f, \"busbw_gbs\": %.3f, "
                             "\"wrong\": %lld, \"max_abs\": %.6g}%s\n",
                             collective_name(r.collective), r.algo.c_str(), dtype_name(r.dtype), redop_name(r.redop),
                             transport_name(r.transport), r.nranks, r.bytes, r.count, r.time_us, r.algbw, r.busbw, r.wrong,
                             r.max_abs_error, i + 1 < results.size() ? "," : "");
            }
            std::fprintf(f, "]\n");
            std::fclose(f);
        }
    }
    int exit_code = rc;
    for (const auto& r : results)
        if (r.wrong != 0) exit_code = 1;
    return exit_code;
}
