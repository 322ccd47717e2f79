// Single-rank collectives: a device-to-device copy at HBM speed.
//
// One persistent CTA per SM, launched as a programmatic dependent of the kernel before it; one
// elected thread per CTA drives a ring of shared-memory tiles with
// TMA bulk copies: global -> shared (completion on an mbarrier), then shared -> global (bulk
// group). No other thread touches the data, so the copy costs no registers and no load/store
// instructions, and a slot is refilled as soon as the store that drained it has read it.
// Only this GPU's own memory is read or written, and no copy carries a multicast qualifier.
//
// The reference has no single-rank configuration (its rank count is a build-time constant of at
// least two, include/nano_nccl/types.h:13-16); this is what the run-time rank count degenerates to.
#include "kernels/sm100/local_copy.h"

#include "kernels/sm100/sync.cuh"
#include "kernels/sm100/tma.cuh"

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

using u64 = unsigned long long;

// Four stages of 27 KiB: enough loads in flight per SM for HBM, and small enough that the CTAs of
// the NEXT copy in the stream fit on the SM beside this one's (see the dependent launch below).
constexpr int kStages = 4;
constexpr unsigned kTile = 27648;
constexpr unsigned kPolls = 1u << 20;  // bound on waiting for an own bulk copy

struct CopyShared {
    alignas(128) unsigned char tile[kStages][kTile];
    alignas(8) u64 full[kStages];
};

__global__ void __launch_bounds__(32) bulk_copy_kernel(const unsigned char* src, unsigned char* dst, u64 bytes, Status* status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    CopyShared& sm = *reinterpret_cast<CopyShared*>(smem_raw);
    if (threadIdx.x != 0) return;
    const u64 ntiles = (bytes + kTile - 1) / kTile;
    if (blockIdx.x >= ntiles) return;
    const u64 mine = (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x;  // tiles blockIdx.x, +grid, +2 grid, ...
    for (int s = 0; s < kStages; ++s) mbar_init(&sm.full[s], 1);
    mbar_fence_init();
    // Programmatic dependent launch: the next kernel in the stream may be scheduled now, so that its
    // launch latency overlaps this kernel; this kernel in turn touches global memory only after the
    // kernel before it has completed and its writes are visible. Both are no-ops for a kernel that
    // was not launched with the attribute.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    auto tile_offset = [&](u64 i) { return (blockIdx.x + i * (u64)gridDim.x) * (u64)kTile; };
    auto tile_bytes = [&](u64 i) {
        const u64 off = tile_offset(i);
        return (unsigned)(bytes - off < kTile ? bytes - off : kTile);
    };
    auto load = [&](u64 i) {
        const int s = (int)(i % kStages);
        const unsigned n = tile_bytes(i);
        mbar_arrive_expect_tx(&sm.full[s], n);
        tma_load_bulk(sm.tile[s], src + tile_offset(i), n, &sm.full[s]);
    };

    const u64 ahead = mine < (u64)kStages ? mine : (u64)kStages;
    for (u64 i = 0; i < ahead; ++i) load(i);
    u64 loaded = ahead;
    bool ok = true;
    u64 i = 0;
    for (; i < mine; ++i) {
        const int s = (int)(i % kStages);
        if (!mbar_wait_bounded(&sm.full[s], (unsigned)((i / kStages) & 1), kPolls)) {
            ok = false;
            break;
        }
        tma_store_bulk(dst + tile_offset(i), sm.tile[s], tile_bytes(i));
        tma_commit_group();
        // The slot drained by the PREVIOUS store is free once that store has read it; waiting for
        // all groups but the newest leaves the store just issued in flight.
        if (i >= 1 && loaded < mine) {
            tma_wait_group_read<1>();
            load(loaded++);  // loaded == i - 1 + kStages: the slot of tile i - 1
        }
    }
    if (!ok) {
        if (status != nullptr) {  // CTAs that fail together write the same kind of record: no latch needed
            status->cta = blockIdx.x;
            status->peer = 0;
            status->where = 40u;
            status->epoch = i;
            __threadfence_system();
            status->code = kStatusTimeout;  // written last: a non-zero code means "record complete"
        }
        // Loads still in flight write this CTA's shared memory: give each a bounded chance to land.
        for (u64 k = i + 1; k < loaded; ++k) mbar_wait_bounded(&sm.full[k % kStages], (unsigned)((k / kStages) & 1), kPolls);
    }
    tma_wait_group_all();  // stores read shared memory until they complete
}

}  // namespace

cudaError_t launch_local_copy(const void* src, void* dst, unsigned long long bytes, int max_ctas, Status* status,
                              cudaStream_t stream) {
    if (bytes == 0 || bytes % 16 != 0 || (reinterpret_cast<std::uintptr_t>(src) | reinterpret_cast<std::uintptr_t>(dst)) % 16 != 0)
        return cudaErrorInvalidValue;
    int device = 0, sms = 0;
    cudaError_t st = cudaGetDevice(&device);
    if (st == cudaSuccess) st = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (st != cudaSuccess) return st;
    const u64 ntiles = (bytes + kTile - 1) / kTile;
    int grid = max_ctas > 0 ? (max_ctas < sms ? max_ctas : sms) : sms;
    if ((u64)grid > ntiles) grid = (int)ntiles;
    // The attribute belongs to the current device's copy of the function.
    st = cudaFuncSetAttribute(bulk_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(CopyShared));
    if (st != cudaSuccess) return st;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid, 1, 1);
    config.blockDim = dim3(32, 1, 1);
    config.dynamicSmemBytes = sizeof(CopyShared);
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, bulk_copy_kernel, static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst),
                              static_cast<u64>(bytes), status);
}

}  // namespace b200ccl::kernels
