// Plain-data structures shared by host launch code and the sm_100a kernels.
//
// nano-nccl passes per-channel FIFO and counter pointers of the two ring neighbours
// (src/transport/simple/protocol.h:26-71). The direct kernels here instead receive, for every
// buffer, a table with the address of EVERY rank's copy, because through NVSwitch each peer is
// one hop away and is loaded from / stored to directly.
#pragma once

#include "b200ccl/types.h"

#include <cstdint>

namespace b200ccl::dev {

constexpr int kMaxCtas = 160;       // flag rows per rank; one row per CTA index (148 SMs on B200)
constexpr int kBlockThreads = 512;  // direct kernels
constexpr int kRingMaxChannels = 32;
constexpr int kLlCtas = 8;                  // the low-latency kernel always runs this many CTAs per rank
constexpr unsigned kLlMaxBytes = 128u << 10; // largest message it takes
constexpr unsigned kLlMaxWords = kLlMaxBytes / 4;

// Per-rank control block. It lives in symmetric memory: every rank can store into every other
// rank's block; each rank polls only its own.
struct ControlBlock {
    // barrier[cta][src]: last barrier epoch that CTA `cta` of rank `src` has arrived at.
    // Written remotely by `src` (release, system scope), polled locally (acquire).
    unsigned long long barrier[kMaxCtas][kMaxRanks];
    // epoch[cta]: how many barriers CTA `cta` of THIS rank has passed since the communicator
    // was created. Never reset, never written by a peer; kept on the device so that a captured
    // CUDA graph replays correctly.
    unsigned long long epoch[kMaxCtas];
    // Non-zero → every wait on this rank gives up. Set by a peer whose wait ran out, or by the host.
    unsigned int abort_flag;
    // 0 until this rank's first failure has been recorded (device-local atomic; the status
    // record itself is then written with plain stores into host memory).
    unsigned int fail_once;
    // plan_hash[src]: fingerprint of the plan (algorithm, grid, pack width, staging) that rank `src`
    // launched its current direct collective with. Written remotely by CTA 0 of `src` just before its
    // first barrier signal; compared after that barrier, so that ranks whose plans differ end with a
    // diagnostic instead of running out their waits.
    unsigned long long plan_hash[kMaxRanks];
    unsigned int pad_[14];
    // Low-latency AllReduce: calls seen so far by each of its (fixed number of) CTAs. Local only.
    unsigned long long ll_epoch[kLlCtas];
    // Ring/Simple step counters. *_tail / *_head follow nano-nccl's ownership rule
    // (src/transport/p2p/p2p_step_counters.h:32-35): recv_tail and send_head are polled by this
    // rank and written by its neighbours; base steps persist progress between launches.
    unsigned long long ring_recv_tail[kRingMaxChannels];  // written by previous rank
    unsigned long long ring_send_head[kRingMaxChannels];  // written by next rank
    unsigned long long ring_send_base[kRingMaxChannels];  // local
    unsigned long long ring_recv_base[kRingMaxChannels];  // local
};

enum StatusCode : unsigned int {
    kStatusOk = 0,
    kStatusTimeout = 1,   // a bounded wait ran out
    kStatusAborted = 2,   // abort flag seen while waiting
    kStatusBadArgs = 3,   // index/bounds self-check failed (debug builds)
    kStatusPlanMismatch = 4,  // a peer launched this collective with a different plan
};

// One per local rank, in pinned mapped host memory: the host reads it without touching the device.
struct Status {
    unsigned int code;     // first failure wins (see ControlBlock::fail_once)
    unsigned int cta;
    unsigned int peer;     // rank that was waited for
    unsigned int where;    // kernel-specific site id
    unsigned long long epoch;      // barrier epoch or ring step that was waited for
    unsigned long long waited_ns;
};

enum ShardMode : int {
    kShardWhole = 0,   // one shard: the whole range (one-shot AllReduce, per-rank local reduce)
    kShardSplit = 1,   // range split into nranks contiguous shards (two-shot AllReduce)
    kShardBlocks = 2,  // nranks blocks of `len` each, strides given (ReduceScatter)
};

// Arguments of the direct (one-shot / two-shot / NVLS) kernels. Lengths and offsets are in
// PACKS: 16-byte vectors on the vector path, single elements on the scalar path.
struct CollArgs {
    const void* in[kMaxRanks];   // every rank's input as addressed from this rank
    void* out[kMaxRanks];        // every rank's output
    ControlBlock* ctrl[kMaxRanks];
    Status* status;
    const void* user_in;   // non-null → copy user_in into in[rank] first (staged input)
    void* user_out;        // non-null → copy out[rank] into user_out last (staged output)
    const void* mc_in;     // multicast alias of `in`  (NVLS kernels)
    void* mc_out;          // multicast alias of `out`
    unsigned long long len;         // packs: whole range (Whole/Split) or one block (Blocks)
    unsigned long long in_stride;   // Blocks: distance between blocks in `in`
    unsigned long long uin_stride;  // Blocks: distance between blocks in `user_in`
    unsigned long long timeout_ns;
    unsigned long long plan_hash;   // see ControlBlock::plan_hash; 0 = no check
    // Debug builds: extents in packs of in[p] / out[p] (0 = unknown); an index beyond them is
    // recorded as kStatusBadArgs and the access is skipped.
    unsigned long long in_extent;
    unsigned long long out_extent;
    float scale;        // multiplies the reduced value (1/N for avg, 1 otherwise)
    int rank;
    int nranks;
    int shard_mode;     // ShardMode
    int store_all;      // 1 → store the reduced pack into every rank's `out`; 0 → own only
};

// AllGather moves bytes only.
struct GatherArgs {
    const void* in[kMaxRanks];   // pull mode: every rank's input
    void* out[kMaxRanks];        // push mode: every rank's output
    ControlBlock* ctrl[kMaxRanks];
    Status* status;
    const void* user_in;   // pull mode staged input (copied into in[rank] first), else null
    void* mc_out;          // NVLS: multicast alias of out
    unsigned long long len;         // packs per rank
    unsigned long long out_stride;  // packs between consecutive ranks' blocks in the output
    unsigned long long timeout_ns;
    unsigned long long plan_hash;   // see ControlBlock::plan_hash; 0 = no check
    int rank;
    int nranks;
    int mode;        // 0 push (store own block into every out), 1 pull (load every in), 2 nvls
    int pack_bytes;  // 16, 4, 2 or 1
};

// Low-latency (flag-in-data) AllReduce. Every rank owns a receive area of
// 2 parities x nranks sources x kLlMaxWords slots of 8 bytes {4 data bytes, 4-byte call number}.
struct LlArgs {
    const void* in;              // local input (any device memory of this rank)
    void* out;                   // local output
    unsigned long long* area[kMaxRanks];  // every rank's receive area
    ControlBlock* own_ctrl;
    ControlBlock* ctrl[kMaxRanks];        // to raise every rank's abort word when a wait runs out
    Status* status;
    unsigned long long timeout_ns;
    unsigned int nwords;         // 4-byte words in the message
    float scale;
    int rank;
    int nranks;
};

// Arguments of every emulated rank, passed by value to a loopback launch.
template <typename A>
struct LoopPack {
    A r[kMaxRanks];
};

}  // namespace b200ccl::dev
