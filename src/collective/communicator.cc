// Communicator implementation: group layout, transport resolution, symmetric control/staging
// memory, per-call planning and kernel launch, completion tracking, the asynchronous error
// latch and teardown.
//
// Parity: nano-nccl src/collective/all_reduce/communicator.cu:150-1286 (Communicator::Impl).
// Kept behaviours: argument contract and diagnostics (832-859), asynchronous enqueue on caller
// streams, ordering of successive collectives of one communicator, latched first error that
// rejects new work (239, 260-269), destruction that waits for work in flight (202-236,
// 1129-1147). Replaced: the ring launch with per-edge FIFO wiring (965-1099) becomes a plan
// (sched/plan.h) over direct peer load/store kernels; the N×N cudaStreamWaitEvent serialisation
// (878-892) is not needed because the kernels themselves meet in per-CTA barriers, so only each
// rank's own previous launch is waited for.
#include "b200ccl/communicator.h"

#include "b200ccl/bootstrap.h"
#include "collective/ring_engine.h"
#include "collective/validate.h"
#include "core/check.h"
#include "core/env.h"
#include "kernels/sm100/dev_types.h"
#include "kernels/sm100/direct_collectives.h"
#include "kernels/sm100/ll_allreduce.h"
#include "kernels/sm100/local_copy.h"
#include "kernels/sm100/staged_pipeline.h"
#include "mem/ipc_window.h"
#include "mem/symmetric.h"
#include "sched/plan.h"
#include "sched/transport_plan.h"
#include "topo/topology.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <sstream>
#include <stdexcept>

namespace b200ccl {

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<std::uintptr_t>(p) & 15u) == 0; }

struct Located {
    int region = -1;  // index into windows_, or -1
    std::size_t offset = 0;
};

// FNV-1a over the facts of a launch that every rank must share; never 0 (0 means "no check").
unsigned long long plan_fingerprint(std::initializer_list<unsigned long long> facts) {
    unsigned long long h = 1469598103934665603ull;
    for (unsigned long long f : facts) {
        for (int b = 0; b < 8; ++b) {
            h ^= (f >> (8 * b)) & 0xffull;
            h *= 1099511628211ull;
        }
    }
    return h == 0 ? 1 : h;
}

}  // namespace

class Communicator::Impl {
public:
    Impl(const CommunicatorConfig& config, Bootstrap* bootstrap);
    ~Impl();

    void run(Collective collective, const CollectiveArgs& args);
    void check_async_error() const;
    int local_rank_count() const noexcept { return static_cast<int>(local_.size()); }
    int global_rank_count() const noexcept { return nranks_; }
    int first_global_rank() const noexcept { return local_.empty() ? 0 : local_[0].grank; }
    // One kind when every ring edge has it, else mixed (e.g. peer memory inside processes, sockets between them).
    TransportKind transport() const noexcept { return ring_plan_.resolved_kind(resolved_); }
    bool nvls_available() const noexcept { return alloc_ && alloc_->multicast_supported(); }
    std::vector<void*> alloc_symmetric(std::size_t bytes);
    void free_symmetric(const std::vector<void*>& ptrs);
    void register_buffers(const std::vector<void*>& ptrs, std::size_t bytes);
    void unregister_buffers(const std::vector<void*>& ptrs);
    void release_window(const std::vector<void*>& ptrs, const char* what);
    CallInfo last_call() const noexcept { return last_; }
    std::vector<const void*> ring_channel_pointers(int local_rank, int channel) const {
        if (!ring_) throw std::runtime_error("ring_channel_pointers: no ring collective has run on this communicator yet");
        const dev::RingChannelView v = ring_->channel_view(local_rank, channel);
        return {v.send_fifo, v.recv_fifo, v.send_tail, v.send_head, v.recv_tail, v.recv_head, v.send_base, v.recv_base};
    }
    std::string describe() const;

private:
    struct Local {
        int grank = 0;
        int device = 0;
        dev::Status* status = nullptr;  // pinned, mapped
        cudaEvent_t done = nullptr;
        bool launched = false;
        cudaStream_t last_stream = nullptr;
        bool last_in_capture = false;  // the completion event was last recorded inside a stream capture
    };

    void resolve_transport();
    void ensure_staging(const CollectiveArgs& args);
    void allocate_staging();
    // The two halves of rank p's staging arena (checking builds put a page of canary bytes before
    // the first and after the second) and their multicast aliases.
    char* stage_in_ptr(int p) const { return static_cast<char*>(stage_->rank_ptr(p)) + stage_guard_; }
    char* stage_out_ptr(int p) const { return stage_in_ptr(p) + staging_half_; }
    char* stage_mc_in() const { return static_cast<char*>(stage_->multicast_ptr()) + stage_guard_; }
    char* stage_mc_out() const { return stage_mc_in() + staging_half_; }
    void check_canaries() const;
    Located locate(const void* p, std::size_t bytes, int grank) const;
    void wait_previous(Local& l, cudaStream_t stream);
    void record_done(Local& l, cudaStream_t stream);
    // in_loc / out_loc: where each local rank's buffer lies; null when the buffers of this call do
    // not sit at one common offset of one window (then the window's peer addresses say nothing
    // about the other ranks' buffers and must not be used).
    void launch_all_reduce(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                           const std::vector<Located>* in_loc, const std::vector<Located>* out_loc);
    void launch_reduce_scatter(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                               const std::vector<Located>* in_loc);
    void launch_all_gather(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                           const std::vector<Located>* in_loc, const std::vector<Located>* out_loc);
    void fill_common(dev::CollArgs& a, const Local& l) const;
    void launch_reduce_ranks(const CollectiveArgs& args, std::vector<dev::CollArgs>& per_rank, int pack_bytes,
                             bool nvls, int grid);
    void launch_gather_ranks(const CollectiveArgs& args, std::vector<dev::GatherArgs>& per_rank, int grid);
    void launch_low_latency(const CollectiveArgs& args);
    void launch_pipeline(const CollectiveArgs& args, const sched::Plan& plan);
    bool direct_peer_pointers() const { return loopback_ || (!multiprocess_ && resolved_ == TransportKind::P2p); }
    void poison(const std::string& why) const {
        if (latched_.empty()) latched_ = why;
    }

    int nranks_ = 0;
    bool loopback_ = false;
    bool multiprocess_ = false;
    Bootstrap* bootstrap_ = nullptr;
    TransportKind requested_ = TransportKind::Auto;
    // P2p: every local ring edge uses peer memory (and the direct algorithms are available); Shm:
    // every edge uses host memory; Mixed: some of each; Socket / Rdma: as requested.
    TransportKind resolved_ = TransportKind::P2p;
    bool peer_memory_ = false;                    // every pair of local GPUs can address each other: symmetric memory exists
    std::vector<TransportKind> local_edge_kind_;  // per ring edge e -> e+1 (global numbering); meaningful for edges inside this process
    Algo forced_algo_ = Algo::Auto;
    unsigned long long timeout_ns_ = 0;
    std::size_t staging_half_ = 0;
    std::size_t stage_guard_ = 0;  // bytes of canary before and after the arena (checking builds), else 0
    int channels_ = kDefaultChannels;
    sched::Tuning tuning_;
    sched::ProcessLayout layout_;
    sched::RingTransportPlan ring_plan_;
    topo::TopologyReport topo_;
    std::vector<Local> local_;
    std::unique_ptr<mem::SymmetricAllocator> alloc_;
    std::unique_ptr<mem::SymmetricRegion> ctrl_;
    std::unique_ptr<mem::SymmetricRegion> stage_;
    std::unique_ptr<mem::SymmetricRegion> pipe_flags_;  // dev::PipeFlags per rank, allocated with the arena
    std::vector<dev::PipeStats*> pipe_stats_;           // per local rank, device memory (B200CCL_PIPELINE_STATS=1)
    std::unique_ptr<mem::SymmetricRegion> ll_area_;  // receive slots of the low-latency kernel (first use)
    // A window is a buffer that exists on every rank and that every rank can address: a symmetric
    // allocation (with a multicast alias where available) or a registered ordinary buffer.
    struct Window {
        std::size_t bytes = 0;  // 0 = released
        std::vector<void*> ptr;  // per global rank
        void* mc = nullptr;
        std::unique_ptr<mem::SymmetricRegion> region;
        std::unique_ptr<mem::IpcWindow> ipc;
    };
    std::vector<Window> windows_;
    mem::GroupDesc group_;
    std::unique_ptr<RingEngine> ring_;
    CallInfo last_;
    mutable std::string latched_;
};

// ---------------------------------------------------------------------------------------------

Communicator::Impl::Impl(const CommunicatorConfig& config, Bootstrap* bootstrap)
    : bootstrap_(bootstrap) {
    int visible = 0;
    {
        const cudaError_t st = cudaGetDeviceCount(&visible);
        if (st != cudaSuccess) {
            (void)cudaGetLastError();
            throw std::runtime_error(std::string("no usable CUDA device: ") + cudaGetErrorString(st));
        }
    }
    validate_config(config, visible);
    loopback_ = config.loopback;
    multiprocess_ = bootstrap != nullptr && bootstrap->size() > 1;
    if (!multiprocess_) bootstrap_ = nullptr;
    if (loopback_ && multiprocess_) throw std::invalid_argument("loopback emulation is single-process only");
    requested_ = config.transport;
    forced_algo_ = config.algo;
    if (const char* a = env::get("B200CCL_ALGO", "NANO_NCCL_ALGO")) {
        if (!parse_algo(a, &forced_algo_))
            throw std::invalid_argument(std::string("B200CCL_ALGO: unknown algorithm '") + a + "'");
    }
    const double timeout_ms =
        config.wait_timeout_ms > 0 ? config.wait_timeout_ms : env::get_double("B200CCL_WAIT_TIMEOUT_MS", 10000.0);
    timeout_ns_ = static_cast<unsigned long long>(timeout_ms * 1e6);
    staging_half_ = config.staging_bytes > 0 ? config.staging_bytes / 2
                                             : env::get_bytes("B200CCL_STAGING_BYTES", std::size_t(256) << 20) / 2;
    staging_half_ = std::max<std::size_t>(staging_half_ / 4096 * 4096, 4096);
    // 0: decided below, once the transport is known.
    channels_ = config.channels > 0 ? config.channels : static_cast<int>(env::get_int("B200CCL_NCHANNELS", 0, "NANO_NCCL_NCHANNELS"));
    tuning_ = sched::tuning_from_env();
    if (config.max_ctas > 0) {  // an explicit cap applies to every algorithm
        tuning_.max_ctas = tuning_.nvls_max_ctas = tuning_.nvls_staged_max_ctas = tuning_.twoshot_max_ctas =
            std::min(config.max_ctas, dev::kMaxCtas);
    }

    // Rank layout: ranks are contiguous per process, in bootstrap order
    // (MPI_Allgather + MPI_Exscan in mpi_communicator.cc:134-155).
    int first = 0;
    if (loopback_) {
        nranks_ = config.loopback_ranks;
    } else if (multiprocess_) {
        const int mine = static_cast<int>(config.devices.size());
        std::vector<int> counts(bootstrap_->size());
        bootstrap_->allgather(&mine, counts.data(), sizeof(int));
        for (int p = 0; p < bootstrap_->size(); ++p) {
            if (p < bootstrap_->rank()) first += counts[p];
            layout_.first_rank.push_back(nranks_);
            layout_.rank_count.push_back(counts[p]);
            nranks_ += counts[p];
        }
    } else {
        nranks_ = static_cast<int>(config.devices.size());
    }
    if (layout_.first_rank.empty()) {
        layout_.first_rank = {0};
        layout_.rank_count = {nranks_};
    }
    layout_.nranks = nranks_;
    if (nranks_ < 1 || nranks_ > kMaxRanks)
        throw std::invalid_argument("communicator needs between 1 and " + std::to_string(kMaxRanks) +
                                    " ranks in total, got " + std::to_string(nranks_));
    const int nlocal = loopback_ ? nranks_ : static_cast<int>(config.devices.size());
    local_.resize(nlocal);
    for (int i = 0; i < nlocal; ++i) {
        local_[i].grank = first + i;
        local_[i].device = loopback_ ? config.devices[0] : config.devices[i];
    }

    topo_ = topo::discover(config.devices);
    resolve_transport();
    if (channels_ <= 0) {
        // One ring CTA moves about 8 GB/s over NVLink, so peer-memory rings want many channels (8 GPUs, 64 MiB:
        // 272 GB/s with 32, 193 with 16); host-memory edges are limited by the host path and do best with few
        // (8 GPUs: 11.7 GB/s with 4, 10.3 with 8, 9.2 with 16); network edges keep a proxy thread pair per channel.
        channels_ = resolved_ == TransportKind::P2p ? 32
                    : (resolved_ == TransportKind::Shm || resolved_ == TransportKind::Mixed) ? 4 : kDefaultChannels;
        // Emulated ranks share one GPU and one cooperative launch: all their channel CTAs must be resident at once.
        if (loopback_) channels_ = std::min(channels_, std::max(1, 64 / nranks_));
    }
    channels_ = std::max(1, std::min(channels_, kMaxChannels));
    {
        // Per-edge view of the ring: edges inside a process use peer memory or host memory, decided
        // edge by edge; edges between processes use exported peer memory unless a network transport
        // was asked for; a single process that asked for socket/rdma loops every edge through it.
        const bool net = resolved_ == TransportKind::Socket || resolved_ == TransportKind::Rdma;
        ring_plan_ = sched::make_ring_transport_plan(layout_, TransportKind::P2p, net ? resolved_ : TransportKind::P2p,
                                                     net && !multiprocess_);
        if (!(net && !multiprocess_)) {
            for (int e = 0; e < static_cast<int>(ring_plan_.edge_kinds.size()); ++e) {
                const bool inside = layout_.owner_of(e) == layout_.owner_of((e + 1) % nranks_);
                if (inside && local_edge_kind_[e] == TransportKind::Shm) ring_plan_.edge_kinds[e] = TransportKind::Shm;
            }
        }
    }

    // Peer-mapped (symmetric) memory needs every pair of GPUs to address each other. Without it
    // only the ring runs, over per-edge FIFOs in the receiver's memory or in mapped host memory.
    if (peer_memory_) {
        mem::GroupDesc group;
        group.nranks = nranks_;
        group.bootstrap = bootstrap_;
        group.want_multicast = config.enable_nvls && resolved_ == TransportKind::P2p;
        group.loopback = loopback_;
        for (const auto& l : local_) group.local.push_back({l.grank, l.device});
        group_ = group;
        alloc_.reset(new mem::SymmetricAllocator(group));
        ctrl_ = alloc_->allocate(sizeof(dev::ControlBlock), "control");
        // Allocation is collective (and clears memory, which synchronises the device), so what the
        // small-message path needs exists before the first call rather than inside it.
        if (nranks_ >= 2) ll_area_ = alloc_->allocate(kernels::ll_area_bytes(nranks_), "low-latency slots");
        // Between processes any call may need the staging arena (ordinary tensors of another process
        // cannot be addressed), and which call does is a per-rank fact: allocating it on first use
        // would leave a rank that needs it waiting, inside a collective allocation, for ranks that do not.
        if (multiprocess_ && nranks_ >= 2) {
            allocate_staging();
        }
    }

    for (auto& l : local_) {
        DeviceGuard guard(l.device);
        B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&l.status), sizeof(dev::Status),
                              cudaHostAllocMapped | cudaHostAllocPortable));
        std::memset(l.status, 0, sizeof(dev::Status));
        B2_CUDA(cudaEventCreateWithFlags(&l.done, cudaEventDisableTiming));
    }
    if (env::get_bool("B200CCL_PIPELINE_STATS", false)) {
        for (auto& l : local_) {
            DeviceGuard guard(l.device);
            // Device memory, read back at destruction: atomics into mapped host memory cross PCIe one by
            // one, and system-scope releases on the same SM wait behind them.
            dev::PipeStats* st = nullptr;
            B2_CUDA(cudaMalloc(reinterpret_cast<void**>(&st), sizeof(dev::PipeStats)));
            B2_CUDA(cudaMemset(st, 0, sizeof(dev::PipeStats)));
            pipe_stats_.push_back(st);
        }
    }
    // (The ring engine, its FIFOs and any network edges are built on the first call that needs them.)
    log_info("communicator: %d ranks (%d local, first %d), transport %s, nvls %s", nranks_, nlocal, first,
             transport_name(resolved_), nvls_available() ? "yes" : "no");
}

namespace {

// "0-1,2-3" -> pairs; "0,2" -> single numbers. Test hooks only; malformed text is an error.
std::vector<std::pair<int, int>> parse_pairs(const char* text, const char* what) {
    std::vector<std::pair<int, int>> out;
    if (text == nullptr) return out;
    std::stringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ',')) {
        if (item.empty()) continue;
        char* end = nullptr;
        const long a = std::strtol(item.c_str(), &end, 10);
        long b = a;
        if (*end == '-') b = std::strtol(end + 1, &end, 10);
        if (end == item.c_str() || *end != '\0' || a < 0 || b < 0)
            throw std::invalid_argument(std::string(what) + ": cannot parse '" + item + "'");
        out.emplace_back(static_cast<int>(a), static_cast<int>(b));
    }
    return out;
}

}  // namespace

// Decides, per ring edge inside this process, between peer memory and host memory.
// Parity: nano-nccl resolve_ring_transport (src/transport/p2p/p2p_topology.cu:191-233): `auto`
// looks at each edge, `p2p` must hold on every edge or fail, `shm` is uniform. Its `auto` also
// demands a direct GPU-to-GPU NVLink (:53-90) and so picks SHM behind an NVSwitch; here peer
// access in both directions is enough.
void Communicator::Impl::resolve_transport() {
    std::vector<int> devs;
    for (const auto& l : local_)
        if (std::find(devs.begin(), devs.end(), l.device) == devs.end()) devs.push_back(l.device);
    // B200CCL_NO_PEER_PAIRS=a-b[,c-d]: treat these device pairs as unable to address each other
    // (exercises the mixed plan on a machine where every pair can).
    const auto denied = parse_pairs(env::get("B200CCL_NO_PEER_PAIRS"), "B200CCL_NO_PEER_PAIRS");
    auto pair_ok = [&](int a, int b, std::string* why) {
        if (a == b) return true;
        for (const auto& d : denied) {
            if ((d.first == a && d.second == b) || (d.first == b && d.second == a)) {
                if (why) *why = "device " + std::to_string(a) + " cannot access device " + std::to_string(b) + " (B200CCL_NO_PEER_PAIRS)";
                return false;
            }
        }
        int ab = 0, ba = 0;
        B2_CUDA(cudaDeviceCanAccessPeer(&ab, a, b));
        B2_CUDA(cudaDeviceCanAccessPeer(&ba, b, a));
        if (!(ab && ba) && why) *why = "device " + std::to_string(ab ? b : a) + " cannot access device " + std::to_string(ab ? a : b);
        return ab && ba;
    };
    std::string why;
    bool all_pairs = true;
    for (int a : devs)
        for (int b : devs)
            if (a < b && !pair_ok(a, b, all_pairs ? &why : nullptr)) all_pairs = false;
    auto device_of = [&](int grank) {
        for (const auto& l : local_)
            if (l.grank == grank) return l.device;
        return -1;
    };
    local_edge_kind_.assign(static_cast<std::size_t>(std::max(nranks_, 1)), TransportKind::P2p);
    auto edges_by_access = [&]() {
        bool any_shm = false;
        for (int e = 0; e < nranks_; ++e) {
            const int a = device_of(e), b = device_of((e + 1) % nranks_);
            if (a < 0 || b < 0) continue;  // an edge that leaves this process
            if (!pair_ok(a, b, nullptr)) {
                local_edge_kind_[e] = TransportKind::Shm;
                any_shm = true;
            }
        }
        return any_shm;
    };
    switch (requested_) {
        case TransportKind::Auto: {
            if (multiprocess_ && !all_pairs) throw std::runtime_error("transport auto between processes needs peer access among this process's GPUs: " + why);
            bool any_shm = edges_by_access();
            // B200CCL_SHM_EDGES=e[,e]: these ring edges use host memory although peer memory would do.
            for (const auto& f : parse_pairs(env::get("B200CCL_SHM_EDGES"), "B200CCL_SHM_EDGES")) {
                if (f.first >= nranks_) throw std::invalid_argument("B200CCL_SHM_EDGES: no ring edge " + std::to_string(f.first));
                if (device_of(f.first) >= 0 && device_of((f.first + 1) % nranks_) >= 0) {
                    local_edge_kind_[f.first] = TransportKind::Shm;
                    any_shm = true;
                }
            }
            bool any_p2p = false;
            for (int e = 0; e < nranks_; ++e)
                if (device_of(e) >= 0 && device_of((e + 1) % nranks_) >= 0 && local_edge_kind_[e] == TransportKind::P2p) any_p2p = true;
            resolved_ = !any_shm ? TransportKind::P2p : (any_p2p ? TransportKind::Mixed : TransportKind::Shm);
            if (any_shm) log_info("auto transport: %s ring edges use host memory%s%s", any_p2p ? "some" : "all", why.empty() ? "" : ": ", why.c_str());
            break;
        }
        case TransportKind::P2p:
            if (!all_pairs) throw std::runtime_error("transport p2p requested but " + why);
            resolved_ = TransportKind::P2p;
            break;
        case TransportKind::Shm:
            if (multiprocess_) throw std::invalid_argument("transport shm needs all ranks in one process");
            local_edge_kind_.assign(local_edge_kind_.size(), TransportKind::Shm);
            resolved_ = TransportKind::Shm;
            break;
        case TransportKind::Socket:
        case TransportKind::Rdma:
            // Multi-process: the ring edges between processes use the network transport. Single
            // process: every ring edge loops through it (TCP on the loopback interface, or the
            // in-process verbs backend), which tests the whole path on one host. Edges inside a
            // process still need peer access for the FIFOs of local edges.
            if (!all_pairs) throw std::runtime_error(std::string("transport ") + transport_name(requested_) + ": " + why);
            resolved_ = requested_;
            break;
        default: throw std::invalid_argument("bad transport");
    }
    // Symmetric memory (and with it every direct algorithm) needs all pairs.
    peer_memory_ = all_pairs && resolved_ != TransportKind::Shm;
    if (peer_memory_ && devs.size() >= 2 && !mem::enable_all_peer_access(devs, &why))
        throw std::runtime_error("enabling peer access failed: " + why);
}

Communicator::Impl::~Impl() {
    // Work in flight is waited for (destroying a communicator with unsynchronised streams is
    // allowed, as in tests/public_api.cu:904-916 of the reference).
    for (auto& l : local_) {
        if (l.launched && l.done && !l.last_in_capture) {
            const cudaError_t st = cudaEventSynchronize(l.done);
            if (st != cudaSuccess) {
                (void)cudaGetLastError();
                log_warn("waiting for rank %d's last collective failed: %s", l.grank, cudaGetErrorString(st));
            }
        }
    }
    for (std::size_t i = 0; i < pipe_stats_.size(); ++i) {
        dev::PipeStats t;
        std::memset(&t, 0, sizeof(t));
        {
            DeviceGuard guard(local_[i].device);
            if (cudaMemcpy(&t, pipe_stats_[i], sizeof(t), cudaMemcpyDeviceToHost) != cudaSuccess) (void)cudaGetLastError();
        }
        if (t.calls != 0) {
            int khz = 0;  // the counters are SM cycles; convert with the SM clock the device reports
            cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, local_[i].device);
            const double ns_per_cycle = khz > 0 ? 1e6 / static_cast<double>(khz) : 1.0;
            const double per_tile = ns_per_cycle * 1e-3 / static_cast<double>(t.tiles ? t.tiles : 1);
            std::fprintf(stderr,
                         "pipeline stats v1 rank=%d cta_calls=%llu tiles=%llu per-tile us: in_wait_slot=%.2f in_copy=%.2f red_wait=%.2f "
                         "red_work=%.2f out_wait=%.2f out_copy=%.2f kernel_ms_total=%.3f\n",
                         local_[i].grank, t.calls, t.tiles, t.in_wait_slot_ns * per_tile, t.in_copy_ns * per_tile,
                         t.red_wait_ns * per_tile, t.red_work_ns * per_tile, t.out_wait_ns * per_tile, t.out_copy_ns * per_tile,
                         t.kernel_ns * ns_per_cycle * 1e-6);
        }
        {
            DeviceGuard guard(local_[i].device);
            cudaFree(pipe_stats_[i]);
        }
    }
    ring_.reset();
    windows_.clear();
    pipe_flags_.reset();
    stage_.reset();
    ll_area_.reset();
    ctrl_.reset();
    for (auto& l : local_) {
        if (l.done) cudaEventDestroy(l.done);
        if (l.status) cudaFreeHost(l.status);
    }
}

void Communicator::Impl::check_async_error() const {
    if (latched_.empty()) check_canaries();
    if (latched_.empty() && ring_) {
        // The root cause first: a failed proxy raises the abort word, and the kernels that leave
        // their waits because of it only record the echo ("aborted").
        const std::string e = ring_->async_error();
        if (!e.empty()) latched_ = e;
    }
    if (latched_.empty()) {
        for (const auto& l : local_) {
            const volatile dev::Status* s = l.status;
            if (s && s->code != dev::kStatusOk) {
                std::ostringstream os;
                if (s->code == dev::kStatusPlanMismatch) {
                    os << "ranks disagree on the plan: rank " << l.grank << " and rank " << s->peer
                       << " launched this collective with different algorithms, grids, pack widths or staging; every rank "
                          "must pass the same count and dtype, and buffers of the same kind (symmetric, registered or plain) "
                          "and alignment";
                } else if (s->code == dev::kStatusBadArgs) {
                    os << "device self-check failed: rank " << l.grank << " cta " << s->cta << " computed index " << s->epoch
                       << " beyond the buffer extent at site " << s->where << "; the access was skipped";
                } else {
                    const char* what = s->code == dev::kStatusTimeout ? "device wait timed out" : "device wait aborted";
                    os << what << ": rank " << l.grank << " cta " << s->cta << " waited "
                       << static_cast<double>(s->waited_ns) * 1e-6 << " ms for rank " << s->peer << " at site " << s->where
                       << " (epoch/step " << s->epoch << ")";
                }
                latched_ = os.str();
                break;
            }
        }
    }
    if (!latched_.empty()) throw std::runtime_error(latched_);
}

void Communicator::Impl::ensure_staging(const CollectiveArgs& args) {
    if (stage_) return;
    // The arena is allocated on the first call that needs it. That allocation is collective between
    // processes and synchronises the device, neither of which a stream capture survives.
    for (cudaStream_t stream : args.streams) {
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st == cudaStreamCaptureStatusActive)
            throw std::runtime_error("the staging arena must be allocated outside a stream capture: run one collective on "
                                     "buffers of this kind before capturing, or use symmetric or registered buffers");
    }
    allocate_staging();
}

namespace {
constexpr unsigned char kCanaryByte = 0xA5;
}

void Communicator::Impl::allocate_staging() {
#if defined(B200CCL_DEBUG_BOUNDS)
    stage_guard_ = 4096;
#endif
    stage_ = alloc_->allocate(staging_half_ * 2 + 2 * stage_guard_, "staging");
    pipe_flags_ = alloc_->allocate(sizeof(dev::PipeFlags), "pipeline flags");
    if (stage_guard_ != 0) {
        for (const auto& l : local_) {
            DeviceGuard guard(l.device);
            char* base = static_cast<char*>(stage_->rank_ptr(l.grank));
            B2_CUDA(cudaMemset(base, kCanaryByte, stage_guard_));
            B2_CUDA(cudaMemset(base + stage_guard_ + 2 * staging_half_, kCanaryByte, stage_guard_));
        }
        for (const auto& l : local_) {
            DeviceGuard guard(l.device);
            B2_CUDA(cudaDeviceSynchronize());
        }
        if (bootstrap_) bootstrap_->barrier();
    }
}

// Checking builds: the canary pages around the arena must still hold their pattern. A kernel that
// indexed past a half of the arena (on this rank or, through peer stores, from another) shows here.
void Communicator::Impl::check_canaries() const {
    if (stage_guard_ == 0 || !stage_) return;
    std::vector<unsigned char> host(stage_guard_);
    for (const auto& l : local_) {
        DeviceGuard guard(l.device);
        char* base = static_cast<char*>(stage_->rank_ptr(l.grank));
#if defined(B200CCL_DEBUG_BOUNDS)
        // Test hook: overwrite one canary byte from the host, as a stray store would.
        if (env::get_bool("B200CCL_DEBUG_SMASH_CANARY", false)) B2_CUDA(cudaMemset(base + stage_guard_ + 2 * staging_half_ + 17, 0, 1));
#endif
        for (int side = 0; side < 2; ++side) {
            const char* from = side == 0 ? base : base + stage_guard_ + 2 * staging_half_;
            B2_CUDA(cudaMemcpy(host.data(), from, stage_guard_, cudaMemcpyDeviceToHost));
            for (std::size_t i = 0; i < stage_guard_; ++i) {
                if (host[i] != kCanaryByte) {
                    poison("staging arena canary overwritten: rank " + std::to_string(l.grank) + ", byte " + std::to_string(i) +
                           (side == 0 ? " of the page before the arena" : " of the page after the arena"));
                    return;
                }
            }
        }
    }
}

Located Communicator::Impl::locate(const void* p, std::size_t bytes, int grank) const {
    const char* q = static_cast<const char*>(p);
    for (std::size_t i = 0; i < windows_.size(); ++i) {
        const Window& w = windows_[i];
        if (w.bytes == 0) continue;
        const char* b = static_cast<const char*>(w.ptr[grank]);
        if (q >= b && q + bytes <= b + w.bytes) return {static_cast<int>(i), static_cast<std::size_t>(q - b)};
    }
    return {};
}

std::vector<void*> Communicator::Impl::alloc_symmetric(std::size_t bytes) {
    check_async_error();
    if (!alloc_) throw std::runtime_error("symmetric memory is not available with transport shm");
    Window w;
    w.region = alloc_->allocate(bytes, "user");
    w.bytes = w.region->bytes();
    w.mc = w.region->multicast_ptr();
    for (int g = 0; g < nranks_; ++g) w.ptr.push_back(w.region->rank_ptr(g));
    std::vector<void*> out;
    for (const auto& l : local_) out.push_back(w.ptr[l.grank]);
    windows_.push_back(std::move(w));
    return out;
}

void Communicator::Impl::release_window(const std::vector<void*>& ptrs, const char* what) {
    if (ptrs.empty()) return;
    for (auto& w : windows_) {
        if (w.bytes != 0 && w.ptr[local_[0].grank] == ptrs[0]) {
            for (auto& l : local_)
                if (l.launched && !l.last_in_capture) B2_CUDA(cudaEventSynchronize(l.done));
            if (bootstrap_) bootstrap_->barrier();  // no peer may still be using it
            w.bytes = 0;
            w.region.reset();
            w.ipc.reset();
            return;
        }
    }
    throw std::invalid_argument(std::string(what) + ": pointer does not name a live window of this communicator");
}

void Communicator::Impl::free_symmetric(const std::vector<void*>& ptrs) { release_window(ptrs, "free_symmetric"); }

void Communicator::Impl::register_buffers(const std::vector<void*>& ptrs, std::size_t bytes) {
    check_async_error();
    if (ptrs.size() != local_.size()) throw std::invalid_argument("register_buffers: one pointer per local rank");
    if (bytes == 0) throw std::invalid_argument("register_buffers: size must be positive");
    if (!multiprocess_) return;  // one process: every device buffer is already peer-addressable
    if (!alloc_) throw std::runtime_error("register_buffers: not available without peer-mapped memory (transport shm)");
    Window w;
    w.ipc = mem::IpcWindow::create(group_, ptrs, bytes);
    w.bytes = bytes;
    for (int g = 0; g < nranks_; ++g) w.ptr.push_back(w.ipc->rank_ptr(g));
    windows_.push_back(std::move(w));
}

void Communicator::Impl::unregister_buffers(const std::vector<void*>& ptrs) {
    if (!multiprocess_) return;
    release_window(ptrs, "unregister_buffers");
}

void Communicator::Impl::wait_previous(Local& l, cudaStream_t stream) {
    if (!l.launched || l.last_stream == stream) return;
    // An event recorded outside a capture cannot be waited for inside one, and the other way
    // round; across that boundary the caller's own ordering (capture begin/end, graph launch) holds.
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    B2_CUDA(cudaStreamIsCapturing(stream, &st));
    const bool capturing = st == cudaStreamCaptureStatusActive;
    if (capturing != l.last_in_capture) return;
    B2_CUDA(cudaStreamWaitEvent(stream, l.done, 0));
}

void Communicator::Impl::record_done(Local& l, cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    B2_CUDA(cudaStreamIsCapturing(stream, &st));
    B2_CUDA(cudaEventRecord(l.done, stream));
    l.launched = true;
    l.last_stream = stream;
    l.last_in_capture = st == cudaStreamCaptureStatusActive;
}

void Communicator::Impl::fill_common(dev::CollArgs& a, const Local& l) const {
    std::memset(&a, 0, sizeof(a));
    for (int p = 0; p < nranks_; ++p) a.ctrl[p] = static_cast<dev::ControlBlock*>(ctrl_->rank_ptr(p));
    a.status = l.status;
    a.timeout_ns = timeout_ns_;
    a.scale = 1.0f;
    a.rank = l.grank;
    a.nranks = nranks_;
}

void Communicator::Impl::launch_reduce_ranks(const CollectiveArgs& args, std::vector<dev::CollArgs>& per_rank,
                                             int pack_bytes, bool nvls, int grid) {
    kernels::LaunchConfig cfg;
    cfg.grid = std::min(grid, dev::kMaxCtas);
    cfg.block = tuning_.block_threads;
    cfg.nvls_unroll = tuning_.nvls_unroll;
    if (loopback_) cfg.grid = std::min(cfg.grid, std::max(1, 128 / nranks_));  // one cooperative launch: keep it resident
    for (auto& a : per_rank) {
        // Everything that must be equal on every rank for the kernels to meet: a rank that planned
        // differently (another buffer kind, alignment or size) is told so by the first barrier.
        a.plan_hash = plan_fingerprint({static_cast<unsigned long long>(last_.collective), static_cast<unsigned long long>(last_.algo),
                                        static_cast<unsigned long long>(cfg.grid), static_cast<unsigned long long>(pack_bytes),
                                        a.len, static_cast<unsigned long long>(a.shard_mode), static_cast<unsigned long long>(a.store_all),
                                        a.user_in != nullptr, a.user_out != nullptr, static_cast<unsigned long long>(args.dtype),
                                        static_cast<unsigned long long>(args.redop), nvls});
    }
    try {
        if (loopback_) {
            DeviceGuard guard(local_[0].device);
            cfg.stream = args.streams[0];
            cfg.loop_ranks = nranks_;
            for (auto& l : local_) wait_previous(l, cfg.stream);
            B2_CUDA(kernels::launch_reduce(args.dtype, args.redop, pack_bytes, nvls, per_rank.data(), cfg));
            for (auto& l : local_) record_done(l, cfg.stream);
        } else {
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                cfg.stream = args.streams[i];
                wait_previous(local_[i], cfg.stream);
                B2_CUDA(kernels::launch_reduce(args.dtype, args.redop, pack_bytes, nvls, &per_rank[i], cfg));
                record_done(local_[i], cfg.stream);
            }
        }
    } catch (const std::exception& e) {
        poison(std::string("launch failed: ") + e.what());
        throw;
    }
    last_.grid = cfg.grid;
    last_.block = cfg.block;
}

void Communicator::Impl::launch_gather_ranks(const CollectiveArgs& args, std::vector<dev::GatherArgs>& per_rank,
                                             int grid) {
    kernels::LaunchConfig cfg;
    cfg.grid = std::min(grid, dev::kMaxCtas);
    cfg.block = tuning_.block_threads;
    if (loopback_) cfg.grid = std::min(cfg.grid, std::max(1, 128 / nranks_));
    for (auto& a : per_rank)
        a.plan_hash = plan_fingerprint({static_cast<unsigned long long>(Collective::AllGather), static_cast<unsigned long long>(cfg.grid),
                                        a.len, a.out_stride, static_cast<unsigned long long>(a.mode),
                                        static_cast<unsigned long long>(a.pack_bytes), a.user_in != nullptr});
    try {
        if (loopback_) {
            DeviceGuard guard(local_[0].device);
            cfg.stream = args.streams[0];
            cfg.loop_ranks = nranks_;
            for (auto& l : local_) wait_previous(l, cfg.stream);
            B2_CUDA(kernels::launch_gather(per_rank.data(), cfg));
            for (auto& l : local_) record_done(l, cfg.stream);
        } else {
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                cfg.stream = args.streams[i];
                wait_previous(local_[i], cfg.stream);
                B2_CUDA(kernels::launch_gather(&per_rank[i], cfg));
                record_done(local_[i], cfg.stream);
            }
        }
    } catch (const std::exception& e) {
        poison(std::string("launch failed: ") + e.what());
        throw;
    }
    last_.grid = cfg.grid;
    last_.block = cfg.block;
}

// ---------------------------------------------------------------------------------------------

void Communicator::Impl::run(Collective collective, const CollectiveArgs& args) {
    check_async_error();
    validate_collective_args(collective, args, local_rank_count(), args.allow_in_place);
    const std::size_t esz = dtype_size(args.dtype);
    const std::size_t n = static_cast<std::size_t>(nranks_);
    const std::size_t in_bytes = args.count * esz * (collective == Collective::ReduceScatter ? n : 1);
    const std::size_t out_bytes = args.count * esz * (collective == Collective::AllGather ? n : 1);

    // Where do the buffers live?
    std::vector<Located> in_loc(local_.size()), out_loc(local_.size());
    bool in_sym = true, out_sym = true, in_place = false;
    for (std::size_t i = 0; i < local_.size(); ++i) {
        in_loc[i] = locate(args.send_buffers[i], in_bytes, local_[i].grank);
        out_loc[i] = locate(args.recv_buffers[i], out_bytes, local_[i].grank);
        in_sym &= in_loc[i].region >= 0 && in_loc[i].region == in_loc[0].region && in_loc[i].offset == in_loc[0].offset;
        out_sym &= out_loc[i].region >= 0 && out_loc[i].region == out_loc[0].region && out_loc[i].offset == out_loc[0].offset;
        in_place |= args.send_buffers[i] == args.recv_buffers[i];
    }

    // 16-byte path: every pointer aligned, every block a whole number of 16-byte packs.
    bool wide = (args.count * esz) % 16 == 0;
    for (std::size_t i = 0; i < local_.size(); ++i)
        wide &= aligned16(args.send_buffers[i]) && aligned16(args.recv_buffers[i]);
    if (multiprocess_) {
        // Ranks in other processes are not visible here; their buffers must follow the same
        // rule. Symmetric buffers do by construction (same offset); for staged buffers only the
        // local copy loops touch user memory, so a rank-local decision would make kernels
        // disagree on the pack size: keep the decision a function of the count alone there.
        if (!(in_sym && out_sym)) {
            bool local_aligned = true;
            for (std::size_t i = 0; i < local_.size(); ++i)
                local_aligned &= aligned16(args.send_buffers[i]) && aligned16(args.recv_buffers[i]);
            if (!local_aligned)
                throw std::invalid_argument(std::string(collective_name(collective)) +
                                            ": buffers of a multi-process communicator must be 16-byte aligned");
            wide = (args.count * esz) % 16 == 0;
        }
    }

    sched::CallShape shape;
    shape.collective = collective;
    shape.dtype = args.dtype;
    shape.redop = args.redop;
    shape.nranks = nranks_;
    shape.count = args.count;
    shape.wide = wide;
    shape.word_aligned = (args.count * esz) % 4 == 0 && args.count > 0;
    for (std::size_t i = 0; i < local_.size(); ++i)
        shape.word_aligned &= reinterpret_cast<std::uintptr_t>(args.send_buffers[i]) % 4 == 0 &&
                              reinterpret_cast<std::uintptr_t>(args.recv_buffers[i]) % 4 == 0;
    shape.in_place = in_place;
    shape.peers_read_input = direct_peer_pointers() || in_sym;
    shape.peers_write_output = direct_peer_pointers() || out_sym;
    shape.input_multicast = in_sym && windows_[in_loc[0].region].mc != nullptr;
    shape.output_multicast = out_sym && windows_[out_loc[0].region].mc != nullptr;
    shape.ring_only = resolved_ != TransportKind::P2p;  // shm, mixed, socket, rdma: only the ring crosses those edges
    shape.max_ctas = tuning_.max_ctas;
    shape.staging_multicast = alloc_ && alloc_->multicast_supported() && (!stage_ || stage_->multicast_ptr() != nullptr);
    sched::Plan plan = sched::make_plan(shape, forced_algo_, tuning_);
    if (plan.error.empty() && plan.algo == Algo::Nvls && (plan.stage_in || plan.stage_out)) {
        // The staging arena is allocated on first use; every rank learns together (the binding is
        // agreed between processes) whether it got a multicast alias. Without one, plan again.
        ensure_staging(args);
        if (stage_->multicast_ptr() == nullptr) {
            shape.staging_multicast = false;
            plan = sched::make_plan(shape, forced_algo_, tuning_);
        }
    }
    if (!plan.error.empty()) throw std::invalid_argument(std::string(collective_name(collective)) + ": " + plan.error);

    last_ = CallInfo{};
    last_.collective = collective;
    last_.algo = plan.algo;
    last_.staged_in = plan.stage_in;
    last_.staged_out = plan.stage_out;
    last_.vectorized = wide;
    log_trace("%s count=%zu dtype=%s op=%s → %s grid=%d stage_in=%d stage_out=%d wide=%d", collective_name(collective),
              args.count, dtype_name(args.dtype), redop_name(args.redop), algo_name(plan.algo), plan.grid,
              plan.stage_in, plan.stage_out, wide);

    if (plan.algo == Algo::Ring) {
        if (!ring_) {
            RingEngineConfig rc;
            rc.nranks = nranks_;
            rc.channels = channels_;
            rc.timeout_ns = timeout_ns_;
            rc.edge_kinds = ring_plan_.edge_kinds;
            rc.loopback = loopback_;
            if (resolved_ == TransportKind::Socket || resolved_ == TransportKind::Rdma) rc.net_kind = resolved_;
            for (const auto& l : local_) rc.local.push_back({l.grank, l.device});
            for (const auto& l : local_) rc.status.push_back(l.status);
            ring_.reset(new RingEngine(rc, alloc_.get(), ctrl_.get(), bootstrap_));
        }
        try {
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                wait_previous(local_[i], args.streams[loopback_ ? 0 : i]);
            }
            ring_->launch(collective, args);
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                record_done(local_[i], args.streams[loopback_ ? 0 : i]);
            }
        } catch (const std::invalid_argument&) {
            throw;
        } catch (const std::exception& e) {
            poison(std::string("ring launch failed: ") + e.what());
            throw;
        }
        last_.grid = ring_->channels();
        last_.block = ring_->block_threads();
        return;
    }

    if (plan.algo == Algo::LowLatency) {
        launch_low_latency(args);
        return;
    }
    if (plan.algo == Algo::Copy) {
        // One rank: input and output hold `count` elements for every collective.
        Local& l = local_[0];
        DeviceGuard guard(l.device);
        cudaStream_t stream = args.streams[0];
        try {
            wait_previous(l, stream);
            if (args.send_buffers[0] != args.recv_buffers[0])
                B2_CUDA(kernels::launch_local_copy(args.send_buffers[0], args.recv_buffers[0], args.count * esz, plan.grid,
                                                   l.status, stream));
            record_done(l, stream);
        } catch (const std::exception& e) {
            poison(std::string("launch failed: ") + e.what());
            throw;
        }
        last_.grid = plan.grid;
        last_.block = 32;
        return;
    }
    if (plan.stage_in || plan.stage_out) ensure_staging(args);
    if (plan.algo == Algo::Pipeline) {
        launch_pipeline(args, plan);
        return;
    }
    switch (collective) {
        case Collective::AllReduce: launch_all_reduce(args, plan, wide, in_sym ? &in_loc : nullptr, out_sym ? &out_loc : nullptr); break;
        case Collective::ReduceScatter: launch_reduce_scatter(args, plan, wide, in_sym ? &in_loc : nullptr); break;
        case Collective::AllGather: launch_all_gather(args, plan, wide, in_sym ? &in_loc : nullptr, out_sym ? &out_loc : nullptr); break;
    }
}

// Low-latency AllReduce: the ranks exchange {data, call number} words through receive areas in
// symmetric memory; the user's buffers are only touched by their own rank.
void Communicator::Impl::launch_low_latency(const CollectiveArgs& args) {
    if (!ll_area_) throw std::runtime_error("low-latency all_reduce needs peer-mapped memory");
    std::vector<dev::LlArgs> per(local_.size());
    for (std::size_t i = 0; i < local_.size(); ++i) {
        dev::LlArgs& a = per[i];
        std::memset(&a, 0, sizeof(a));
        a.in = args.send_buffers[i];
        a.out = args.recv_buffers[i];
        for (int p = 0; p < nranks_; ++p) {
            a.area[p] = static_cast<unsigned long long*>(ll_area_->rank_ptr(p));
            a.ctrl[p] = static_cast<dev::ControlBlock*>(ctrl_->rank_ptr(p));
        }
        a.own_ctrl = a.ctrl[local_[i].grank];
        a.status = local_[i].status;
        a.timeout_ns = timeout_ns_;
        a.nwords = static_cast<unsigned>(args.count * dtype_size(args.dtype) / 4);
        a.scale = args.redop == RedOp::Avg ? 1.0f / static_cast<float>(nranks_) : 1.0f;
        a.rank = local_[i].grank;
        a.nranks = nranks_;
    }
    try {
        if (loopback_) {
            DeviceGuard guard(local_[0].device);
            cudaStream_t stream = args.streams[0];
            for (auto& l : local_) wait_previous(l, stream);
            B2_CUDA(kernels::launch_ll_all_reduce(args.dtype, args.redop, per.data(), nranks_, stream));
            for (auto& l : local_) record_done(l, stream);
        } else {
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                wait_previous(local_[i], args.streams[i]);
                B2_CUDA(kernels::launch_ll_all_reduce(args.dtype, args.redop, &per[i], 0, args.streams[i]));
                record_done(local_[i], args.streams[i]);
            }
        }
    } catch (const std::exception& e) {
        poison(std::string("launch failed: ") + e.what());
        throw;
    }
    last_.grid = dev::kLlCtas;
    last_.block = dev::kBlockThreads;
}

// Pipelined staged AllReduce: one launch per rank, whatever the message size (the arena is a ring).
void Communicator::Impl::launch_pipeline(const CollectiveArgs& args, const sched::Plan& plan) {
    const std::size_t bytes = args.count * dtype_size(args.dtype);
    kernels::PipeLaunch cfg;
    cfg.grid = std::min(plan.grid, dev::kMaxCtas);
    if (loopback_) {
        // One cooperative launch plays every rank: all its CTAs must be resident at once.
        int device = local_[0].device, sms = 0;
        B2_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        cfg.grid = std::min(cfg.grid, std::max(1, sms / nranks_ - 1));  // the peer-load variant fits one CTA per SM
    }
    // Tiles and slots must fit the arena half: grid * slots * tile <= half, with at least two slots.
    std::size_t tile = plan.tile_bytes;
    while (tile > 4096 && static_cast<std::size_t>(cfg.grid) * 2 * tile > staging_half_) tile /= 2;
    tile = tile / 16 * 16;
    if (tile == 0 || static_cast<std::size_t>(cfg.grid) * 2 * tile > staging_half_)
        throw std::invalid_argument("all_reduce: the staging arena is too small for the tile pipeline (B200CCL_STAGING_BYTES)");
    const int slots = static_cast<int>(std::min<std::size_t>(4, staging_half_ / (static_cast<std::size_t>(cfg.grid) * tile)));
    cfg.nvls = plan.pipe_nvls && !loopback_ && stage_->multicast_ptr() != nullptr;
    cfg.nvls_unroll = tuning_.pipeline_nvls_unroll;
    std::vector<dev::PipeArgs> per(local_.size());
    for (std::size_t i = 0; i < local_.size(); ++i) {
        dev::PipeArgs& a = per[i];
        std::memset(&a, 0, sizeof(a));
        a.user_in = args.send_buffers[i];
        a.user_out = args.recv_buffers[i];
        for (int p = 0; p < nranks_; ++p) {
            a.arena_in[p] = stage_in_ptr(p);
            a.arena_out[p] = stage_out_ptr(p);
            a.ctrl[p] = static_cast<dev::ControlBlock*>(ctrl_->rank_ptr(p));
            a.flags[p] = static_cast<dev::PipeFlags*>(pipe_flags_->rank_ptr(p));
        }
        if (cfg.nvls) {
            a.mc_in = stage_mc_in();
            a.mc_out = stage_mc_out();
        }
        a.status = local_[i].status;
        a.stats = pipe_stats_.empty() ? nullptr : pipe_stats_[i];
        a.bytes = bytes;
        a.tile_bytes = tile;
        a.timeout_ns = timeout_ns_;
        a.scale = args.redop == RedOp::Avg ? 1.0f / static_cast<float>(nranks_) : 1.0f;
        a.rank = local_[i].grank;
        a.nranks = nranks_;
        a.slots = slots;
        a.plan_hash = plan_fingerprint({static_cast<unsigned long long>(Algo::Pipeline), static_cast<unsigned long long>(cfg.grid), bytes, tile,
                                        static_cast<unsigned long long>(slots), cfg.nvls, static_cast<unsigned long long>(args.dtype),
                                        static_cast<unsigned long long>(args.redop)});
    }
    try {
        if (loopback_) {
            DeviceGuard guard(local_[0].device);
            cfg.stream = args.streams[0];
            cfg.loop_ranks = nranks_;
            for (auto& l : local_) wait_previous(l, cfg.stream);
            B2_CUDA(kernels::launch_staged_pipeline(args.dtype, args.redop, per.data(), cfg));
            for (auto& l : local_) record_done(l, cfg.stream);
        } else {
            for (std::size_t i = 0; i < local_.size(); ++i) {
                DeviceGuard guard(local_[i].device);
                cfg.stream = args.streams[i];
                wait_previous(local_[i], cfg.stream);
                B2_CUDA(kernels::launch_staged_pipeline(args.dtype, args.redop, &per[i], cfg));
                record_done(local_[i], cfg.stream);
            }
        }
    } catch (const std::exception& e) {
        poison(std::string("launch failed: ") + e.what());
        throw;
    }
    last_.grid = cfg.grid;
    last_.block = 512;
    last_.pack_bytes = 16;
}

void Communicator::Impl::launch_all_reduce(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                                           const std::vector<Located>* in_win, const std::vector<Located>* out_win) {
    const std::size_t esz = dtype_size(args.dtype);
    const bool direct = direct_peer_pointers();
    const bool nvls = plan.algo == Algo::Nvls;
    const bool oneshot = plan.algo == Algo::OneShot;
    // 256-bit accesses for the peer two-shot loop when every rank can tell, from facts all ranks
    // share, that the peer-visible addresses are 32-byte aligned: the arena is; windows are used at
    // one common offset; a single process sees every pointer. (Shard boundaries are counted in
    // packs, so all ranks must use the same pack.)
    bool wide32 = wide && tuning_.wide32 && plan.algo == Algo::TwoShot && (args.count * esz) % 32 == 0;
    auto aligned32 = [](const void* p) { return (reinterpret_cast<std::uintptr_t>(p) & 31u) == 0; };
    if (wide32 && !plan.stage_in) {
        if (in_win != nullptr) wide32 = aligned32(static_cast<const char*>(windows_[(*in_win)[0].region].ptr[0]) + (*in_win)[0].offset);
        else for (const void* p : args.send_buffers) wide32 = wide32 && aligned32(p);
    }
    if (wide32 && !plan.stage_out) {
        if (out_win != nullptr) wide32 = aligned32(static_cast<const char*>(windows_[(*out_win)[0].region].ptr[0]) + (*out_win)[0].offset);
        else for (const void* p : args.recv_buffers) wide32 = wide32 && aligned32(p);
    }
    const std::size_t pack = wide32 ? 32 : (wide ? 16 : esz);
    const std::size_t total_packs = args.count * esz / pack;
    const bool staged = plan.stage_in || plan.stage_out;
    const std::size_t cap_packs = staged ? staging_half_ / pack : total_packs;

    for (std::size_t done = 0; done < total_packs; done += cap_packs) {
        const std::size_t len = std::min(cap_packs, total_packs - done);
        const std::size_t off = done * pack;
        std::vector<dev::CollArgs> per(local_.size());
        for (std::size_t i = 0; i < local_.size(); ++i) {
            dev::CollArgs& a = per[i];
            fill_common(a, local_[i]);
            a.len = len;
            a.shard_mode = oneshot ? dev::kShardWhole : dev::kShardSplit;
            a.store_all = oneshot ? 0 : 1;
            if (args.redop == RedOp::Avg) a.scale = 1.0f / static_cast<float>(nranks_);
            for (int p = 0; p < nranks_; ++p) {
                // input table
                if (plan.stage_in) a.in[p] = stage_in_ptr(p);
                else if (in_win != nullptr)
                    a.in[p] = static_cast<const char*>(windows_[(*in_win)[i].region].ptr[p]) + (*in_win)[i].offset + off;
                else if (direct) a.in[p] = static_cast<const char*>(args.send_buffers[p]) + off;
                // output table
                if (plan.stage_out) a.out[p] = stage_out_ptr(p);
                else if (oneshot) a.out[p] = nullptr;
                else if (out_win != nullptr)
                    a.out[p] = static_cast<char*>(windows_[(*out_win)[i].region].ptr[p]) + (*out_win)[i].offset + off;
                else if (direct) a.out[p] = static_cast<char*>(args.recv_buffers[p]) + off;
            }
            if (oneshot) a.out[local_[i].grank] = static_cast<char*>(args.recv_buffers[i]) + off;
            if (plan.stage_in) a.user_in = static_cast<const char*>(args.send_buffers[i]) + off;
            if (plan.stage_out) a.user_out = static_cast<char*>(args.recv_buffers[i]) + off;
            a.in_extent = a.out_extent = len;  // what in[p] and out[p] address, in packs (checking builds compare against it)
#if defined(B200CCL_DEBUG_BOUNDS)
            // Test hook of the checking build: pretend the buffers are this many packs shorter, as a
            // wrong length computation on the host would; the kernel must record it and skip the accesses.
            a.in_extent -= std::min<std::size_t>(len, env::get_bytes("B200CCL_DEBUG_SHRINK_EXTENT", 0));
#endif
            if (nvls) {
                a.mc_in = plan.stage_in ? static_cast<const char*>(stage_mc_in())
                                        : static_cast<const char*>(windows_[(*in_win)[i].region].mc) + (*in_win)[i].offset + off;
                a.mc_out = plan.stage_out ? stage_mc_out()
                                          : static_cast<char*>(windows_[(*out_win)[i].region].mc) + (*out_win)[i].offset + off;
            }
        }
        last_.pack_bytes = static_cast<int>(pack);
        launch_reduce_ranks(args, per, static_cast<int>(pack), nvls, plan.grid);
    }
}

void Communicator::Impl::launch_reduce_scatter(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                                               const std::vector<Located>* in_win) {
    const std::size_t esz = dtype_size(args.dtype);
    const std::size_t pack = wide ? 16 : esz;
    const std::size_t block_packs = args.count * esz / pack;  // one rank's block
    const std::size_t cap_packs = plan.stage_in ? std::max<std::size_t>(staging_half_ / pack / nranks_, 1) : block_packs;
    const bool direct = direct_peer_pointers();
    const bool nvls = plan.algo == Algo::Nvls;

    for (std::size_t done = 0; done < block_packs; done += cap_packs) {
        const std::size_t len = std::min(cap_packs, block_packs - done);
        const std::size_t off = done * pack;
        std::vector<dev::CollArgs> per(local_.size());
        for (std::size_t i = 0; i < local_.size(); ++i) {
            dev::CollArgs& a = per[i];
            fill_common(a, local_[i]);
            a.len = len;
            a.shard_mode = dev::kShardBlocks;
            a.store_all = 0;
            a.in_stride = plan.stage_in ? len : block_packs;
            a.uin_stride = block_packs;
            if (args.redop == RedOp::Avg) a.scale = 1.0f / static_cast<float>(nranks_);
            for (int p = 0; p < nranks_; ++p) {
                if (plan.stage_in) a.in[p] = stage_in_ptr(p);
                else if (in_win != nullptr)
                    a.in[p] = static_cast<const char*>(windows_[(*in_win)[i].region].ptr[p]) + (*in_win)[i].offset + off;
                else if (direct) a.in[p] = static_cast<const char*>(args.send_buffers[p]) + off;
            }
            a.out[local_[i].grank] = static_cast<char*>(args.recv_buffers[i]) + off;
            a.in_extent = a.in_stride * static_cast<std::size_t>(nranks_ - 1) + len;
            a.out_extent = len;
            if (plan.stage_in) a.user_in = static_cast<const char*>(args.send_buffers[i]) + off;
            if (nvls) a.mc_in = static_cast<const char*>(windows_[(*in_win)[i].region].mc) + (*in_win)[i].offset + off;
        }
        launch_reduce_ranks(args, per, static_cast<int>(pack), nvls, plan.grid);
    }
}

void Communicator::Impl::launch_all_gather(const CollectiveArgs& args, const sched::Plan& plan, bool wide,
                                           const std::vector<Located>* in_win, const std::vector<Located>* out_win) {
    const std::size_t esz = dtype_size(args.dtype);
    const std::size_t bytes = args.count * esz;
    std::size_t pack = wide ? 16 : (bytes % 4 == 0 ? 4 : 2);
    if (!wide && pack == 4) {
        for (std::size_t i = 0; i < local_.size(); ++i)
            if ((reinterpret_cast<std::uintptr_t>(args.send_buffers[i]) | reinterpret_cast<std::uintptr_t>(args.recv_buffers[i])) & 3u)
                pack = esz;
        if (multiprocess_) pack = esz;  // alignment of remote buffers is unknown: stay with elements
    }
    const std::size_t block_packs = bytes / pack;
    const std::size_t cap_packs = plan.stage_in ? staging_half_ / pack : block_packs;
    const bool direct = direct_peer_pointers();

    for (std::size_t done = 0; done < block_packs; done += cap_packs) {
        const std::size_t len = std::min(cap_packs, block_packs - done);
        const std::size_t off = done * pack;
        std::vector<dev::GatherArgs> per(local_.size());
        for (std::size_t i = 0; i < local_.size(); ++i) {
            dev::GatherArgs& a = per[i];
            std::memset(&a, 0, sizeof(a));
            for (int p = 0; p < nranks_; ++p) a.ctrl[p] = static_cast<dev::ControlBlock*>(ctrl_->rank_ptr(p));
            a.status = local_[i].status;
            a.timeout_ns = timeout_ns_;
            a.rank = local_[i].grank;
            a.nranks = nranks_;
            a.mode = plan.gather_mode;
            a.pack_bytes = static_cast<int>(pack);
            a.len = len;
            a.out_stride = block_packs;
            for (int p = 0; p < nranks_; ++p) {
                if (plan.gather_mode == 1) {  // pull: need everyone's input
                    if (plan.stage_in) a.in[p] = stage_in_ptr(p);
                    else if (in_win != nullptr)
                        a.in[p] = static_cast<const char*>(windows_[(*in_win)[i].region].ptr[p]) + (*in_win)[i].offset + off;
                    else if (direct) a.in[p] = static_cast<const char*>(args.send_buffers[p]) + off;
                } else if (plan.gather_mode == 0) {  // push: need everyone's output
                    if (out_win != nullptr)
                        a.out[p] = static_cast<char*>(windows_[(*out_win)[i].region].ptr[p]) + (*out_win)[i].offset + off;
                    else if (direct) a.out[p] = static_cast<char*>(args.recv_buffers[p]) + off;
                }
            }
            if (plan.gather_mode != 1) a.in[local_[i].grank] = static_cast<const char*>(args.send_buffers[i]) + off;
            if (plan.gather_mode != 0) a.out[local_[i].grank] = static_cast<char*>(args.recv_buffers[i]) + off;
            if (plan.stage_in) a.user_in = static_cast<const char*>(args.send_buffers[i]) + off;
            if (plan.gather_mode == 2)
                a.mc_out = static_cast<char*>(windows_[(*out_win)[i].region].mc) + (*out_win)[i].offset + off;
        }
        launch_gather_ranks(args, per, plan.grid);
    }
}

std::string Communicator::Impl::describe() const {
    std::ostringstream os;
    os << "b200ccl communicator: " << nranks_ << " ranks, " << local_.size() << " local"
       << (loopback_ ? " (loopback emulation)" : "") << (multiprocess_ ? " (multi-process)" : "") << "\n";
    os << "transport: requested " << transport_name(requested_) << ", resolved " << transport_name(resolved_) << "\n";
    if (alloc_)
        os << "memory: " << (alloc_->uses_vmm() ? "virtual memory management" : "cudaMalloc + peer access")
           << "; NVLS multicast "
           << (alloc_->multicast_supported() ? "available" : ("unavailable (" + alloc_->multicast_reason() + ")")) << "\n";
    else
        os << "memory: mapped host memory only (shm)\n";
    for (const auto& l : local_) os << "rank " << l.grank << ": device " << l.device << "\n";
    os << topo_.text;
    os << ring_plan_.describe();
    return os.str();
}

// ---------------------------------------------------------------------------------------------

Communicator::Communicator(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
Communicator::Communicator(Communicator&&) noexcept = default;
Communicator& Communicator::operator=(Communicator&&) noexcept = default;
Communicator::~Communicator() = default;

void Communicator::all_reduce(const CollectiveArgs& args) { impl_->run(Collective::AllReduce, args); }
void Communicator::reduce_scatter(const CollectiveArgs& args) { impl_->run(Collective::ReduceScatter, args); }
void Communicator::all_gather(const CollectiveArgs& args) { impl_->run(Collective::AllGather, args); }
void Communicator::check_async_error() const { impl_->check_async_error(); }
int Communicator::local_rank_count() const noexcept { return impl_->local_rank_count(); }
int Communicator::global_rank_count() const noexcept { return impl_->global_rank_count(); }
int Communicator::first_global_rank() const noexcept { return impl_->first_global_rank(); }
TransportKind Communicator::transport() const noexcept { return impl_->transport(); }
bool Communicator::nvls_available() const noexcept { return impl_->nvls_available(); }
std::vector<void*> Communicator::alloc_symmetric(std::size_t bytes) { return impl_->alloc_symmetric(bytes); }
void Communicator::register_buffers(const std::vector<void*>& ptrs, std::size_t bytes) { impl_->register_buffers(ptrs, bytes); }
void Communicator::unregister_buffers(const std::vector<void*>& ptrs) { impl_->unregister_buffers(ptrs); }
void Communicator::free_symmetric(const std::vector<void*>& ptrs) { impl_->free_symmetric(ptrs); }
CallInfo Communicator::last_call() const noexcept { return impl_->last_call(); }
std::vector<const void*> Communicator::ring_channel_pointers(int local_rank, int channel) const {
    return impl_->ring_channel_pointers(local_rank, channel);
}
std::string Communicator::describe() const { return impl_->describe(); }

std::unique_ptr<Communicator> create_communicator(const CommunicatorConfig& config) {
    return std::unique_ptr<Communicator>(
        new Communicator(std::unique_ptr<Communicator::Impl>(new Communicator::Impl(config, nullptr))));
}

std::unique_ptr<Communicator> create_communicator_from_bootstrap(Bootstrap& bootstrap,
                                                                 const CommunicatorConfig& config) {
    return std::unique_ptr<Communicator>(
        new Communicator(std::unique_ptr<Communicator::Impl>(new Communicator::Impl(config, &bootstrap))));
}

}  // namespace b200ccl
