// Ring/Simple geometry: constants, part/chunk/slice arithmetic, credit rule, and the property
// that the slices of every (channel, window, chunk) tile the message exactly once.
// Modelled on the static_assert block of the reference's tests/simple_protocol.cu:38-104.
#include "check.h"
#include "sched/ring_geometry.h"

#include <vector>

using namespace b200ccl::ring;

static_assert(kFifoSteps == 8 && kSliceSteps == 2 && kChunkSteps == 4, "protocol constants");
static_assert(kSlicesPerChunk == 2, "two slices per chunk");
static_assert(div_up(10, 4) == 3 && align_up(10, 4) == 12, "rounding");
static_assert(edge_index(3, 0, 4) == 3 && edge_index(0, 2, 4) == -1, "edge numbering");
static_assert(step_elems(4u << 20, 4) == 131072, "4 MiB FIFO holds 8 steps of 128 Ki floats");
static_assert(channel_part(1000, 0, 4).offset == 0 && channel_part(1000, 3, 4).offset == 750, "parts");
static_assert(channel_part(1000, 3, 4).count == 250, "parts");
static_assert(all_reduce_chunk_elems(1000, 4, 4, 131072) == 256, "chunk = ceil(1000/4)=250 → 512-byte grain = 128 floats → 256");
static_assert(all_reduce_chunk_elems(0, 4, 4, 131072) == 0, "empty part");
static_assert(all_reduce_chunk_elems(1u << 30, 4, 4, 131072) == 4 * 131072, "capped by kChunkSteps steps");
static_assert(clamp_elems(256, 1000, 768) == 232 && clamp_elems(256, 1000, 1024) == 0, "clamp at the end of a part");
static_assert(slice_elems(256, 4, 131072) == 128, "half a chunk");
static_assert(slice_elems(6, 4, 131072) == 4, "rounded up to a 16-byte vector");
static_assert(slice_elems(8u << 20, 4, 131072) == 2 * 131072, "capped by kSliceSteps steps");
static_assert(send_credit_ok(0, 6) && !send_credit_ok(0, 8) && send_credit_ok(2, 8), "four slices in flight");
static_assert(recv_ready_ok(2, 0) && !recv_ready_ok(1, 0), "data is ready when tail passed the slice");
static_assert(slot_offset(10, 100) == 200, "slot = step mod 8");

int main() {
    // Every element of a message is covered exactly once by the AllReduce schedule of one rank's
    // "pivot" chunks taken over all ranks, for awkward sizes too.
    const std::size_t counts[] = {1, 7, 256, 1000, 65537, 262146 / 4, 1u << 20};
    for (std::size_t count : counts) {
        for (int nranks : {2, 3, 4, 8}) {
            for (int channels : {1, 4, 8}) {
                const std::size_t se = step_elems(1u << 20, 4);
                std::vector<int> hits(count, 0);
                std::size_t nonempty = 0, empty = 0;
                for (int c = 0; c < channels; ++c) {
                    const Part part = channel_part(count, c, channels);
                    const std::size_t cs = all_reduce_chunk_elems(part.count, nranks, 4, se);
                    for (std::size_t w0 = 0; cs > 0 && w0 < part.count; w0 += cs * nranks) {
                        for (int k = 0; k < nranks; ++k) {
                            const std::size_t off = w0 + k * cs;
                            const std::size_t len = clamp_elems(cs, part.count, off);
                            const std::size_t sl = slice_elems(len, 4, se);
                            for (int s = 0; s < kSlicesPerChunk; ++s) {
                                const std::size_t so = s * sl, sn = clamp_elems(sl, len, so);
                                sn ? ++nonempty : ++empty;
                                T_CHECK(sn <= se * kSliceSteps);
                                for (std::size_t i = 0; i < sn; ++i) ++hits[part.offset + off + so + i];
                            }
                        }
                    }
                }
                for (std::size_t i = 0; i < count; ++i) T_CHECK(hits[i] == 1);
                T_CHECK(nonempty > 0);
                (void)empty;
            }
        }
    }
    // Block schedule (ReduceScatter / AllGather).
    for (std::size_t count : counts) {
        const std::size_t se = step_elems(1u << 20, 2);
        std::vector<int> hits(count, 0);
        for (int c = 0; c < 4; ++c) {
            const Part part = channel_part(count, c, 4);
            const std::size_t cs = block_chunk_elems(part.count, 2, se);
            for (std::size_t w0 = 0; cs > 0 && w0 < part.count; w0 += cs) {
                const std::size_t len = clamp_elems(cs, part.count, w0);
                for (std::size_t i = 0; i < len; ++i) ++hits[part.offset + w0 + i];
            }
        }
        for (std::size_t i = 0; i < count; ++i) T_CHECK(hits[i] == 1);
    }
    std::puts("geometry ok");
    return 0;
}
