// Per-call planning: which algorithm, how many CTAs, and whether a buffer must pass through
// the staging arena. Pure functions of the call shape, so that every rank (and every process)
// reaches the same decision without talking, and so that the logic is testable without a GPU.
//
// nano-nccl has a single algorithm and a fixed 4-CTA launch, so it has no counterpart; its
// nearest relative is the per-edge transport plan (src/transport/p2p/p2p_topology.h:13-36).
#pragma once

#include "b200ccl/types.h"

#include <cstddef>
#include <string>

namespace b200ccl::sched {

struct CallShape {
    Collective collective = Collective::AllReduce;
    DType dtype = DType::Float;
    RedOp redop = RedOp::Sum;
    int nranks = 1;
    std::size_t count = 0;       // the API's `count`
    bool wide = false;           // every pointer 16-byte aligned and every block a multiple of 16 bytes
    bool word_aligned = false;   // every pointer 4-byte aligned and the message a multiple of 4 bytes
    bool peers_read_input = false;    // peers can load this call's input directly
    bool peers_write_output = false;  // peers can store into this call's output directly
    bool input_multicast = false;     // input has a multicast alias (NVLS ld_reduce possible)
    bool output_multicast = false;    // output has a multicast alias (NVLS broadcast possible)
    bool staging_multicast = false;   // the staging arena has a multicast alias (staged NVLS possible)
    bool in_place = false;
    bool ring_only = false;      // transport without all-pairs peer access: ring is the only choice
    int max_ctas = 64;
};

struct Plan {
    Algo algo = Algo::TwoShot;
    int grid = 1;
    bool stage_in = false;
    bool stage_out = false;
    int gather_mode = 0;  // AllGather: 0 push, 1 pull, 2 nvls
    // Pipeline: bytes of one tile (CTA b owns tiles b, b + grid, ...) and whether its reduce stage
    // goes through the switch (multimem) or over plain peer loads and stores.
    std::size_t tile_bytes = 0;
    bool pipe_nvls = false;
    std::string error;    // non-empty → the request cannot be satisfied (forced algo impossible)
};

// Crossover points. Defaults come from measurements on 8×B200; each can be overridden by
// environment (B200CCL_ONESHOT_MAX_BYTES, B200CCL_NVLS_MIN_BYTES, B200CCL_MAX_CTAS).
struct Tuning {
    std::size_t oneshot_max_bytes[kMaxRanks + 1];  // per nranks: AllReduce sizes up to this use one-shot
    std::size_t nvls_min_bytes = 0;                // NVLS from this size up (when available)
    int max_ctas = 128;                            // hard cap for every algorithm (B200CCL_MAX_CTAS)
    int nvls_max_ctas = 64;                        // more CTAs than this slowed the multimem kernels down
    int nvls_staged_max_ctas = 64;                 // when the same CTAs also copy the message in and out of the arena
    int twoshot_max_ctas = 128;
    int nvls_unroll = 2;                           // multimem loads in flight per thread (B200CCL_NVLS_UNROLL)
    std::size_t bytes_per_cta = 0;                 // work given to one CTA before another is added
    std::size_t oneshot_bytes_per_cta = 0;         // one-shot reads every peer's copy: spread it thinner
    // AllReduce messages up to this size use the low-latency kernel (0 = only when asked for;
    // B200CCL_LL_MAX_BYTES; never above 128 KiB).
    std::size_t ll_max_bytes = 0;
    // Up to four ranks the flag-in-data kernel carries less traffic per rank and stays ahead longer
    // (B200CCL_LL_MAX_BYTES sets both limits).
    std::size_t ll_max_bytes_upto4 = 0;
    // Peer two-shot AllReduce moves 32 bytes per access (ld/st.global.v8, sm_100) where alignment allows
    // (B200CCL_WIDE32=0 keeps 16-byte accesses).
    bool wide32 = true;
    // Threads per CTA of the direct kernels (B200CCL_BLOCK_THREADS; the reference fixes its 512 at build
    // time, include/nano_nccl/types.h:23-28). Fewer threads per CTA on more CTAs leave room on every SM
    // for the CTAs of a matmul that runs beside the collective.
    int block_threads = 512;
    // AllReduce of buffers that peers cannot address: from this size up the copy into the staging arena,
    // the reduction and the copy out run as a tile pipeline in one kernel (B200CCL_PIPELINE_MIN_BYTES;
    // below it: copy, barrier, reduce, barrier, copy). Every CTA gets the same number of tiles of about
    // pipeline_tile_bytes (never under 32 KiB); at most pipeline_max_ctas CTAs.
    std::size_t pipeline_min_bytes = 0;
    std::size_t pipeline_min_bytes_upto4 = 0;  // the same threshold for up to four ranks (B200CCL_PIPELINE_MIN_BYTES sets both)
    int pipeline_nvls_unroll = 1;              // multimem loads in flight per reducer thread (B200CCL_PIPELINE_NVLS_UNROLL)
    std::size_t pipeline_tile_bytes = 0;
    int pipeline_max_ctas = 96;        // reduce stage through the switch (multimem)
    int pipeline_peer_max_ctas = 128;  // reduce stage over peer loads and stores
};
Tuning default_tuning();
// default_tuning(), then the file named by B200CCL_TUNING_FILE (if set), then the B200CCL_* variables.
Tuning tuning_from_env();
// Applies a tuning file to `base`. One `key = value` per line, `#` starts a comment; byte counts take
// K/M/G suffixes. Keys: oneshot_max_bytes (all rank counts) or oneshot_max_bytes.<nranks>, nvls_min_bytes,
// max_ctas, nvls_max_ctas, twoshot_max_ctas, nvls_unroll, bytes_per_cta, oneshot_bytes_per_cta, ll_max_bytes, ll_max_bytes_upto4,
// wide32, block_threads,
// pipeline_min_bytes, pipeline_min_bytes_upto4, pipeline_tile_bytes, pipeline_max_ctas, pipeline_peer_max_ctas,
// pipeline_nvls_unroll.
// `python -m nano_nccl_b200.tuner --emit-tuning FILE` writes such a file from its measurements.
// Throws std::invalid_argument naming the file and line on an unknown key or a bad value.
Tuning tuning_from_text(const std::string& text, const Tuning& base, const std::string& origin);
Tuning tuning_from_file(const std::string& path, const Tuning& base);

Plan make_plan(const CallShape& shape, Algo forced, const Tuning& tuning);

// Bytes moved through the API per rank: count*size for AllReduce, the full count*nranks*size
// buffer for ReduceScatter (input) and AllGather (output).
std::size_t message_bytes(const CallShape& shape);

}  // namespace b200ccl::sched
