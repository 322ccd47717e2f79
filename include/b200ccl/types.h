// Public value types of the library: element types, reduction operators, transports,
// algorithms, benchmark records and the bandwidth formulas used in every report.
//
// Parity: covers what nano-nccl declares in include/nano_nccl/types.h:31-122. The rank
// count, channel count and block size, compile-time constants there (types.h:13-28),
// are run-time values here; only upper bounds are fixed at compile time.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace b200ccl {

// Upper bounds (one NVSwitch domain holds at most eight B200s).
constexpr int kMaxRanks = 8;
constexpr int kMaxChannels = 32;   // ring/Simple channels per rank
constexpr int kDefaultChannels = 8;
constexpr int kDefaultBlockThreads = 512;

enum class DType : int { Float = 0, Float16 = 1, BFloat16 = 2 };
enum class RedOp : int { Sum = 0, Avg = 1, Max = 2, Min = 3 };
enum class TransportKind : int { Auto = 0, Shm = 1, P2p = 2, Socket = 3, Rdma = 4, Mixed = 5 };
enum class Collective : int { AllReduce = 0, ReduceScatter = 1, AllGather = 2 };

// How a collective is carried out on the device.
//   OneShot  every rank reads every peer's whole input and reduces it (latency bound sizes)
//   TwoShot  rank r reduces shard r from all peers, then stores it into every peer's output
//   Nvls     NVSwitch multicast: multimem.ld_reduce on the own shard, multimem.st broadcast
//   Ring     ring over per-edge Simple-protocol FIFOs (works over SHM / socket / RDMA edges)
//   LowLatency  flag-in-data exchange without barriers for messages up to 128 KiB (AllReduce only)
//   Copy     one rank only: the collective is a device-to-device copy (TMA bulk copies); reported, never requested
//   Pipeline AllReduce of buffers that peers cannot address: copy into the staging arena, reduce and copy out
//            run as a tile pipeline inside one kernel (TMA bulk copies for the local tiles)
enum class Algo : int { Auto = 0, OneShot = 1, TwoShot = 2, Nvls = 3, Ring = 4, LowLatency = 5, Copy = 6, Pipeline = 7 };

const char* dtype_name(DType d);
const char* redop_name(RedOp r);
const char* transport_name(TransportKind t);
const char* algo_name(Algo a);
const char* collective_name(Collective c);

// Each parser returns false and leaves *out untouched when the text is not a known name.
// parse_transport does not accept "socket" or "mixed": neither can be requested, they are
// only ever reported (same contract as nano-nccl types.h:47-53).
bool parse_dtype(const char* text, DType* out);
bool parse_redop(const char* text, RedOp* out);
bool parse_transport(const char* text, TransportKind* out);
bool parse_algo(const char* text, Algo* out);
bool parse_collective(const char* text, Collective* out);

std::size_t dtype_size(DType d);
// Absolute tolerance used when results are verified (1e-5 / 1e-2 / 1e-1, traits.h:20,29,38).
float dtype_default_epsilon(DType d);

struct BenchConfig {
    std::string algo = "auto";  // auto|oneshot|twoshot|nvls|ring|ll  ("ring_simple" = ring)
    Collective collective = Collective::AllReduce;
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
    TransportKind transport = TransportKind::Auto;
    std::size_t min_bytes = 262144;
    std::size_t max_bytes = 67108864;
    int factor = 4;
    int warmup_iters = 5;
    int iters = 20;
    float epsilon = 0.0f;        // 0 → dtype default
    int nranks = 0;              // 0 → every visible GPU
    bool loopback = false;       // all ranks emulated on device 0 by one launch
    bool symmetric = false;      // buffers taken from the communicator's symmetric heap
    bool uniform_data = true;    // uniform[-1,1) seeded per rank; false → N(0,1)
    bool graph = false;          // capture the timed batch into CUDA graphs and time their replay
};

struct BenchResult {
    std::string algo;
    Collective collective = Collective::AllReduce;
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
    TransportKind transport = TransportKind::Auto;
    int nranks = 0;
    std::size_t bytes = 0;   // per-rank message bytes (AllReduce: whole buffer; RS/AG: one shard)
    std::size_t count = 0;
    double time_us = 0.0;    // device time, max over ranks, mean over iterations
    double algbw = 0.0;
    double busbw = 0.0;
    long long wrong = 0;     // number of wrong ELEMENTS over all ranks
    float max_abs_error = 0.0f;
};

std::vector<std::size_t> make_sizes(std::size_t min_bytes, std::size_t max_bytes, int factor);
double algbw_gbs(std::size_t bytes, double time_us);
// busbw = algbw * 2(n-1)/n for AllReduce, algbw * (n-1)/n for ReduceScatter / AllGather,
// where `bytes` is the full (n-shard) buffer for RS/AG.
double all_reduce_busbw_gbs(double algbw, int nranks);
double busbw_gbs(Collective c, double algbw, int nranks);

}  // namespace b200ccl
