#include "b200ccl/types.h"

#include <cstring>
#include <stdexcept>

namespace b200ccl {

const char* dtype_name(DType d) {
    switch (d) {
        case DType::Float: return "float";
        case DType::Float16: return "fp16";
        case DType::BFloat16: return "bf16";
    }
    return "unknown";
}

const char* redop_name(RedOp r) {
    switch (r) {
        case RedOp::Sum: return "sum";
        case RedOp::Avg: return "avg";
        case RedOp::Max: return "max";
        case RedOp::Min: return "min";
    }
    return "unknown";
}

const char* transport_name(TransportKind t) {
    switch (t) {
        case TransportKind::Auto: return "auto";
        case TransportKind::Shm: return "shm";
        case TransportKind::P2p: return "p2p";
        case TransportKind::Socket: return "socket";
        case TransportKind::Rdma: return "rdma";
        case TransportKind::Mixed: return "mixed";
    }
    return "unknown";
}

const char* algo_name(Algo a) {
    switch (a) {
        case Algo::Auto: return "auto";
        case Algo::OneShot: return "oneshot";
        case Algo::TwoShot: return "twoshot";
        case Algo::Nvls: return "nvls";
        case Algo::Ring: return "ring";
        case Algo::LowLatency: return "ll";
        case Algo::Copy: return "copy";
        case Algo::Pipeline: return "pipeline";
    }
    return "unknown";
}

const char* collective_name(Collective c) {
    switch (c) {
        case Collective::AllReduce: return "all_reduce";
        case Collective::ReduceScatter: return "reduce_scatter";
        case Collective::AllGather: return "all_gather";
    }
    return "unknown";
}

namespace {
template <typename E>
bool parse_from(const char* text, E* out, const std::pair<const char*, E>* table, int n) {
    if (!text || !out) return false;
    for (int i = 0; i < n; ++i) {
        if (std::strcmp(text, table[i].first) == 0) {
            *out = table[i].second;
            return true;
        }
    }
    return false;
}
}  // namespace

bool parse_dtype(const char* text, DType* out) {
    static const std::pair<const char*, DType> t[] = {
        {"float", DType::Float}, {"fp32", DType::Float}, {"fp16", DType::Float16},
        {"half", DType::Float16}, {"bf16", DType::BFloat16}};
    return parse_from(text, out, t, 5);
}

bool parse_redop(const char* text, RedOp* out) {
    static const std::pair<const char*, RedOp> t[] = {
        {"sum", RedOp::Sum}, {"avg", RedOp::Avg}, {"max", RedOp::Max}, {"min", RedOp::Min}};
    return parse_from(text, out, t, 4);
}

bool parse_transport(const char* text, TransportKind* out) {
    static const std::pair<const char*, TransportKind> t[] = {{"auto", TransportKind::Auto},
                                                              {"shm", TransportKind::Shm},
                                                              {"p2p", TransportKind::P2p},
                                                              {"rdma", TransportKind::Rdma}};
    return parse_from(text, out, t, 4);
}

bool parse_algo(const char* text, Algo* out) {
    static const std::pair<const char*, Algo> t[] = {
        {"auto", Algo::Auto},       {"oneshot", Algo::OneShot}, {"twoshot", Algo::TwoShot},
        {"nvls", Algo::Nvls},       {"ring", Algo::Ring},       {"ring_simple", Algo::Ring},
        {"ll", Algo::LowLatency},   {"pipeline", Algo::Pipeline}};
    return parse_from(text, out, t, 8);
}

bool parse_collective(const char* text, Collective* out) {
    static const std::pair<const char*, Collective> t[] = {
        {"all_reduce", Collective::AllReduce},         {"allreduce", Collective::AllReduce},
        {"reduce_scatter", Collective::ReduceScatter}, {"reducescatter", Collective::ReduceScatter},
        {"all_gather", Collective::AllGather},         {"allgather", Collective::AllGather}};
    return parse_from(text, out, t, 6);
}

std::size_t dtype_size(DType d) { return d == DType::Float ? 4 : 2; }

float dtype_default_epsilon(DType d) {
    switch (d) {
        case DType::Float: return 1e-5f;
        case DType::Float16: return 1e-2f;
        case DType::BFloat16: return 1e-1f;
    }
    return 0.0f;
}

std::vector<std::size_t> make_sizes(std::size_t min_bytes, std::size_t max_bytes, int factor) {
    if (min_bytes == 0 || factor < 2 || max_bytes < min_bytes)
        throw std::invalid_argument("make_sizes: need 0 < min <= max and factor >= 2");
    std::vector<std::size_t> sizes;
    for (std::size_t b = min_bytes; b <= max_bytes; b *= static_cast<std::size_t>(factor)) {
        sizes.push_back(b);
        if (b > max_bytes / static_cast<std::size_t>(factor)) break;
    }
    return sizes;
}

double algbw_gbs(std::size_t bytes, double time_us) {
    return time_us > 0 ? static_cast<double>(bytes) / (time_us * 1e3) : 0.0;
}

double all_reduce_busbw_gbs(double algbw, int nranks) {
    return nranks > 0 ? algbw * 2.0 * (nranks - 1) / nranks : 0.0;
}

double busbw_gbs(Collective c, double algbw, int nranks) {
    if (nranks <= 0) return 0.0;
    if (c == Collective::AllReduce) return all_reduce_busbw_gbs(algbw, nranks);
    return algbw * (nranks - 1) / nranks;
}

}  // namespace b200ccl
