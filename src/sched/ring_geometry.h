// Geometry of the ring + Simple protocol: how a message is cut into channel parts, chunks and
// slices, and how slices map to FIFO steps. Header-only, usable on host and device, so that the
// kernels, the host launch code and the CPU simulator compute the same schedule.
//
// Parity: nano-nccl src/transport/simple/protocol.h:16-24 (kFifoSteps 8, kSliceSteps 2,
// kChunkSteps 4, 16-byte vectors), src/transport/simple/geometry.h:9-27 and
// src/collective/all_reduce/ring_simple_geometry.h:10-47 (channel part, 512-byte chunk grain,
// clamp at the end of a part, ring edge numbering). Channel count and FIFO size are run-time
// values here.
#pragma once

#include <cstddef>

#if defined(__CUDACC__)
#define B2_GEOM __host__ __device__ constexpr
#else
#define B2_GEOM constexpr
#endif

namespace b200ccl::ring {

constexpr int kFifoSteps = 8;    // steps a FIFO holds
constexpr int kSliceSteps = 2;   // steps one slice occupies; counters advance by this per slice
constexpr int kChunkSteps = 4;   // steps one chunk may occupy → kChunkSteps/kSliceSteps slices per chunk
constexpr int kSlicesPerChunk = kChunkSteps / kSliceSteps;
constexpr std::size_t kVectorBytes = 16;
constexpr std::size_t kGrainBytes = 512;               // chunk sizes are multiples of this
constexpr std::size_t kDefaultFifoBytes = 4u << 20;    // per channel and edge

B2_GEOM std::size_t div_up(std::size_t v, std::size_t d) { return (v + d - 1) / d; }
B2_GEOM std::size_t align_up(std::size_t v, std::size_t a) { return div_up(v, a) * a; }
B2_GEOM std::size_t min_sz(std::size_t a, std::size_t b) { return a < b ? a : b; }

// Directed edge e goes from rank e to rank (e+1) % n. -1 when (src,dst) is not a ring edge.
B2_GEOM int edge_index(int src, int dst, int nranks) { return dst == (src + 1) % nranks ? src : -1; }

// Elements one FIFO step holds.
B2_GEOM std::size_t step_elems(std::size_t fifo_bytes, std::size_t elem_size) {
    return fifo_bytes / kFifoSteps / elem_size;
}

struct Part {
    std::size_t offset;  // first element of the channel's part
    std::size_t count;   // elements in the part
};

// Channel c of `channels` owns elements [count*c/channels, count*(c+1)/channels).
B2_GEOM Part channel_part(std::size_t count, int channel, int channels) {
    const std::size_t b = count * static_cast<std::size_t>(channel) / static_cast<std::size_t>(channels);
    const std::size_t e = count * static_cast<std::size_t>(channel + 1) / static_cast<std::size_t>(channels);
    return Part{b, e - b};
}

// AllReduce: the part is cut into nranks chunks of this many elements (a multiple of 512 bytes),
// capped by what kChunkSteps FIFO steps can hold; the part is walked in windows of nranks chunks.
B2_GEOM std::size_t all_reduce_chunk_elems(std::size_t part_count, int nranks, std::size_t elem_size,
                                           std::size_t step_elems_) {
    if (part_count == 0) return 0;
    const std::size_t ideal = align_up(div_up(part_count, static_cast<std::size_t>(nranks)), kGrainBytes / elem_size);
    return min_sz(ideal, step_elems_ * kChunkSteps);
}

// ReduceScatter / AllGather: every block is walked in chunks of this many elements.
B2_GEOM std::size_t block_chunk_elems(std::size_t part_count, std::size_t elem_size, std::size_t step_elems_) {
    if (part_count == 0) return 0;
    return min_sz(align_up(part_count, kGrainBytes / elem_size), step_elems_ * kChunkSteps);
}

// Elements of a chunk that starts at `chunk_offset` inside a range of `range_count` elements.
B2_GEOM std::size_t clamp_elems(std::size_t chunk_elems, std::size_t range_count, std::size_t chunk_offset) {
    if (chunk_offset >= range_count) return 0;
    return min_sz(chunk_elems, range_count - chunk_offset);
}

// A chunk of n elements travels as up to kSlicesPerChunk slices of this many elements: half the
// chunk rounded up to whole 16-byte vectors, never more than kSliceSteps steps hold. Slices past
// the end of the chunk are empty and are skipped by sender and receiver alike (no wait, no post,
// no step), which keeps both sides' counters aligned.
B2_GEOM std::size_t slice_elems(std::size_t n, std::size_t elem_size, std::size_t step_elems_) {
    const std::size_t vec = kVectorBytes / elem_size;
    const std::size_t half = align_up(div_up(n, static_cast<std::size_t>(kSlicesPerChunk)), vec);
    return min_sz(half == 0 ? vec : half, step_elems_ * kSliceSteps);
}

// Sender may write the slice at `step` when head + kFifoSteps >= step + kSliceSteps.
B2_GEOM bool send_credit_ok(unsigned long long head, unsigned long long step) {
    return head + kFifoSteps >= step + kSliceSteps;
}
// Receiver may read the slice at `step` when tail >= step + kSliceSteps.
B2_GEOM bool recv_ready_ok(unsigned long long tail, unsigned long long step) { return tail >= step + kSliceSteps; }
// First element of the FIFO slot used by `step`.
B2_GEOM std::size_t slot_offset(unsigned long long step, std::size_t step_elems_) {
    return static_cast<std::size_t>(step % kFifoSteps) * step_elems_;
}

static_assert(kFifoSteps % kSliceSteps == 0, "a slice never wraps around the FIFO");
static_assert(kChunkSteps % kSliceSteps == 0, "a chunk is a whole number of slices");
static_assert(kFifoSteps / kSliceSteps == 4, "four slices in flight per channel and edge");

}  // namespace b200ccl::ring
