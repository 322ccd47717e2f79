#include "collective/ring_engine.h"

#include "core/buffers.h"
#include "core/check.h"
#include "core/env.h"
#include "core/numa.h"
#include "kernels/sm100/ring_simple.h"
#include "sched/ring_geometry.h"
#include "transport/net_edge.h"

#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace b200ccl {

struct RingEngine::State {
    RingEngineConfig cfg;
    std::size_t fifo_bytes = ring::kDefaultFifoBytes;
    Bootstrap* bootstrap = nullptr;
    // Peer-to-peer edges with all-pairs symmetric memory: every rank's incoming FIFOs
    // (channels × fifo_bytes) in its own memory, counters in the communicator's control blocks.
    std::unique_ptr<mem::SymmetricRegion> fifo_region;
    const mem::SymmetricRegion* ctrl = nullptr;
    // Without symmetric memory: a private control block per local rank (its neighbours store into
    // it through pairwise peer access) and, for a rank whose incoming edge is P2p, a plain device FIFO.
    std::vector<DeviceBuffer<dev::ControlBlock>> own_ctrl;
    std::vector<DeviceBuffer<unsigned char>> dev_fifo;
    // Host (SHM) edges: FIFO and counters of edge e, channel c at index e*channels + c.
    std::vector<MappedBuffer<unsigned char>> host_fifo;
    MappedU64Array host_counters;  // [(e*channels + c)*2 + {0 tail, 1 head}]
    // Network edges (socket / RDMA) of this process, by direction.
    std::unique_ptr<transport::NetEdgeSet> net;
    std::vector<std::vector<dev::RingChannel>> wiring;   // per local rank: [channels], host copy
    std::vector<DeviceBuffer<dev::RingChannel>> tables;  // per local rank: [channels]
    MappedBuffer<dev::RingTurnaroundStats> stats;        // [local rank][channel], optional
};

namespace {
int local_index_of(const RingEngineConfig& cfg, int grank) {
    for (std::size_t i = 0; i < cfg.local.size(); ++i)
        if (cfg.local[i].global_rank == grank) return static_cast<int>(i);
    return -1;
}

void enable_pair(int a, int b) {
    if (a == b) return;
    for (int k = 0; k < 2; ++k) {
        DeviceGuard guard(k == 0 ? a : b);
        const cudaError_t st = cudaDeviceEnablePeerAccess(k == 0 ? b : a, 0);
        if (st == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
        else B2_CUDA(st);
    }
}
}  // namespace

RingEngine::RingEngine(const RingEngineConfig& config, mem::SymmetricAllocator* alloc, const mem::SymmetricRegion* ctrl,
                       Bootstrap* bootstrap)
    : state_(new State()) {
    State& s = *state_;
    s.cfg = config;
    s.ctrl = ctrl;
    s.bootstrap = bootstrap;
    const int n = config.nranks, C = config.channels;
    if (n < 2) throw std::invalid_argument("ring needs at least two ranks");
    if (C < 1 || C > dev::kRingMaxChannels) throw std::invalid_argument("ring channel count out of range");
    if (s.cfg.edge_kinds.empty()) s.cfg.edge_kinds.assign(n, TransportKind::P2p);
    if (static_cast<int>(s.cfg.edge_kinds.size()) != n) throw std::invalid_argument("ring needs one transport kind per edge");
    s.fifo_bytes = env::get_bytes("B200CCL_FIFO_BUFF_BYTES", ring::kDefaultFifoBytes, "NANO_NCCL_FIFO_BUFF_BYTES");
    const std::size_t quantum = ring::kFifoSteps * ring::kGrainBytes;
    if (s.fifo_bytes < quantum || s.fifo_bytes % quantum != 0)
        throw std::invalid_argument("FIFO size must be a positive multiple of " + std::to_string(quantum) + " bytes");

    const bool net = config.net_kind != TransportKind::Auto;
    const bool symmetric = alloc != nullptr && ctrl != nullptr;
    auto is_shm = [&](int e) { return s.cfg.edge_kinds[e] == TransportKind::Shm; };
    bool any_shm = false, any_p2p = false;
    for (int e = 0; e < n; ++e) (is_shm(e) ? any_shm : any_p2p) = true;
    if (!symmetric && (bootstrap != nullptr || net))
        throw std::invalid_argument("a ring that leaves this process needs peer-mapped memory");

    if (symmetric) {
        // Every rank's incoming FIFOs in one symmetric region (unused by a rank whose incoming edge is SHM).
        if (any_p2p || net) s.fifo_region = alloc->allocate(static_cast<std::size_t>(C) * s.fifo_bytes, "ring-fifo");
    } else {
        for (const auto& l : config.local) {
            s.own_ctrl.emplace_back(l.device, 1);
            s.own_ctrl.back().zero();
        }
        s.dev_fifo.resize(config.local.size());
        for (int e = 0; e < n; ++e) {
            if (is_shm(e)) continue;
            // P2p edge e -> e+1 without symmetric memory: FIFO on the receiver (p2p_fifo.cu:123-125 of
            // the reference), peer access for this pair only (p2p_topology.cu:247-262).
            const int src = local_index_of(config, e), dst = local_index_of(config, (e + 1) % n);
            if (src < 0 || dst < 0) throw std::invalid_argument("ring edge without a local endpoint");
            if (!config.loopback) enable_pair(config.local[src].device, config.local[dst].device);
            s.dev_fifo[dst].reset(config.local[dst].device, static_cast<std::size_t>(C) * s.fifo_bytes);
        }
    }
    if (any_shm) {
        // SHM: one FIFO per edge and channel in mapped host memory on the RECEIVER's NUMA node
        // (nano-nccl communicator.cu:915-934); its two counters in mapped host memory too.
        s.host_fifo.resize(static_cast<std::size_t>(n) * C);
        for (int e = 0; e < n; ++e) {
            if (!is_shm(e)) continue;
            const int dst_local = local_index_of(config, (e + 1) % n);
            const int node = dst_local >= 0 ? numa::gpu_node(config.local[dst_local].device) : -1;
            for (int c = 0; c < C; ++c) s.host_fifo[e * C + c].reset(s.fifo_bytes, node);
        }
        s.host_counters.reset(static_cast<std::size_t>(n) * C * 2);
    }
    if (net) {
        transport::NetEdgeConfig nc;
        nc.kind = config.net_kind;
        nc.nranks = n;
        nc.channels = C;
        nc.fifo_bytes = s.fifo_bytes;
        nc.local = config.local;
        nc.all_edges = bootstrap == nullptr;  // single process: every edge loops through the transport
        s.net = transport::create_net_edges(nc, bootstrap);
    }
    if (env::get_bool("B200CCL_RING_TURNAROUND", false)) s.stats.reset(config.local.size() * C);

    auto ctrl_of = [&](int grank) -> dev::ControlBlock* {
        if (symmetric) return static_cast<dev::ControlBlock*>(ctrl->rank_ptr(grank));
        return s.own_ctrl[local_index_of(config, grank)].get();
    };
    auto fifo_of = [&](int grank, int c) -> char* {
        char* base = symmetric ? static_cast<char*>(s.fifo_region->rank_ptr(grank))
                               : reinterpret_cast<char*>(s.dev_fifo[local_index_of(config, grank)].get());
        return base + static_cast<std::size_t>(c) * s.fifo_bytes;
    };

    // Wire every local rank's channel table, edge by edge.
    for (std::size_t i = 0; i < config.local.size(); ++i) {
        const int r = config.local[i].global_rank;
        const int next = (r + 1) % n, prev = (r + n - 1) % n;
        const int out_e = r, in_e = prev;  // edge e goes e → e+1
        std::vector<dev::RingChannel> table(C);
        for (int c = 0; c < C; ++c) {
            dev::RingChannel ch;
            std::memset(&ch, 0, sizeof(ch));
            dev::ControlBlock* mine = ctrl_of(r);
            if (is_shm(out_e)) {
                ch.send_fifo = s.host_fifo[out_e * C + c].get();
                ch.send_tail = &s.host_counters[(out_e * C + c) * 2 + 0];
                ch.send_head = &s.host_counters[(out_e * C + c) * 2 + 1];
            } else if (!s.net || s.net->send_half(r, c) == nullptr) {
                ch.send_fifo = fifo_of(next, c);
                ch.send_tail = &ctrl_of(next)->ring_recv_tail[c];  // publish into the next rank
                ch.send_head = &mine->ring_send_head[c];           // poll locally
            }
            if (is_shm(in_e)) {
                ch.recv_fifo = s.host_fifo[in_e * C + c].get();
                ch.recv_tail = &s.host_counters[(in_e * C + c) * 2 + 0];
                ch.recv_head = &s.host_counters[(in_e * C + c) * 2 + 1];
            } else if (!s.net || s.net->recv_half(r, c) == nullptr) {
                ch.recv_fifo = fifo_of(r, c);
                ch.recv_tail = &mine->ring_recv_tail[c];               // poll locally
                ch.recv_head = &ctrl_of(prev)->ring_send_head[c];      // publish into the previous rank
            }
            ch.send_base = &mine->ring_send_base[c];
            ch.recv_base = &mine->ring_recv_base[c];
            if (s.net) {
                // Edges that leave this process go through host FIFOs served by proxy threads.
                if (const transport::NetHalf* h = s.net->send_half(r, c)) {
                    ch.send_fifo = h->fifo;
                    ch.send_tail = h->tail;
                    ch.send_head = h->head;
                    ch.send_sizes = h->sizes;
                    ch.abort_word = s.net->abort_word();
                }
                if (const transport::NetHalf* h = s.net->recv_half(r, c)) {
                    ch.recv_fifo = h->fifo;
                    ch.recv_tail = h->tail;
                    ch.recv_head = h->head;
                    ch.abort_word = s.net->abort_word();
                }
            }
            if (s.stats.get()) ch.stats = &s.stats[i * C + c];
            table[c] = ch;
        }
        s.tables.emplace_back(config.local[i].device, static_cast<std::size_t>(C));
        DeviceGuard guard(config.local[i].device);
        B2_CUDA(cudaMemcpy(s.tables.back().get(), table.data(), sizeof(dev::RingChannel) * C, cudaMemcpyHostToDevice));
        s.wiring.push_back(std::move(table));
    }
    if (s.net) s.net->start();
    if (bootstrap) bootstrap->barrier();
    log_info("ring engine: %d channels, %zu-byte FIFOs, edges:%s%s%s", C, s.fifo_bytes, any_p2p ? " peer-to-peer" : "",
             any_shm ? " host" : "", s.net ? " network" : "");
}

dev::RingChannelView RingEngine::channel_view(int local_index, int channel) const {
    const State& s = *state_;
    if (local_index < 0 || local_index >= static_cast<int>(s.wiring.size()) || channel < 0 || channel >= s.cfg.channels)
        throw std::invalid_argument("ring channel view: index out of range");
    const dev::RingChannel& ch = s.wiring[local_index][channel];
    dev::RingChannelView v;
    v.send_fifo = ch.send_fifo;
    v.recv_fifo = ch.recv_fifo;
    v.send_tail = ch.send_tail;
    v.send_head = ch.send_head;
    v.recv_tail = ch.recv_tail;
    v.recv_head = ch.recv_head;
    v.send_base = ch.send_base;
    v.recv_base = ch.recv_base;
    return v;
}

RingEngine::~RingEngine() {
    State& s = *state_;
    if (s.net) s.net->stop();
    if (s.stats.get()) {
        const int C = s.cfg.channels;
        for (std::size_t i = 0; i < s.cfg.local.size(); ++i) {
            for (int c = 0; c < C; ++c) {
                const dev::RingTurnaroundStats& t = s.stats[i * C + c];
                std::fprintf(stderr,
                             "ring turnaround v1 rank=%d channel=%d slices=%llu empty=%llu wait_recv_ms=%.3f wait_send_ms=%.3f "
                             "compute_ms=%.3f post_ms=%.3f\n",
                             s.cfg.local[i].global_rank, c, t.slices, t.empty_slices, t.wait_recv_ns * 1e-6,
                             t.wait_send_ns * 1e-6, t.compute_ns * 1e-6, t.post_ns * 1e-6);
            }
        }
    }
}

int RingEngine::channels() const { return state_->cfg.channels; }
int RingEngine::block_threads() const { return kernels::ring_block_threads(); }
std::string RingEngine::async_error() const { return state_->net ? state_->net->first_error() : std::string(); }

void RingEngine::launch(Collective collective, const CollectiveArgs& args) {
    State& s = *state_;
    const std::size_t esz = dtype_size(args.dtype);
    bool wide = (args.count * esz) % 16 == 0;
    for (std::size_t i = 0; i < s.cfg.local.size(); ++i)
        wide &= ((reinterpret_cast<std::uintptr_t>(args.send_buffers[i]) | reinterpret_cast<std::uintptr_t>(args.recv_buffers[i])) & 15u) == 0;
    if (s.bootstrap && !wide && (args.count * esz) % 16 == 0)
        throw std::invalid_argument("ring: buffers of a multi-process communicator must be 16-byte aligned");
    std::vector<dev::RingArgs> per(s.cfg.local.size());
    for (std::size_t i = 0; i < s.cfg.local.size(); ++i) {
        dev::RingArgs& a = per[i];
        std::memset(&a, 0, sizeof(a));
        a.input = args.send_buffers[i];
        a.output = args.recv_buffers[i];
        a.channels = s.tables[i].get();
        a.own_ctrl = s.ctrl != nullptr ? static_cast<dev::ControlBlock*>(s.ctrl->rank_ptr(s.cfg.local[i].global_rank))
                                       : s.own_ctrl[i].get();
        a.status = s.cfg.status[i];
        a.count = args.count;
        a.step_elems = ring::step_elems(s.fifo_bytes, esz);
        a.timeout_ns = s.cfg.timeout_ns;
        a.scale = args.redop == RedOp::Avg ? 1.0f / static_cast<float>(s.cfg.nranks) : 1.0f;
        a.rank = s.cfg.local[i].global_rank;
        a.nranks = s.cfg.nranks;
        a.nchannels = s.cfg.channels;
        a.collective = static_cast<int>(collective);
        a.wide = wide ? 1 : 0;
    }
    kernels::RingLaunch cfg;
    if (s.cfg.loopback) {
        DeviceGuard guard(s.cfg.local[0].device);
        cfg.stream = args.streams[0];
        cfg.loop_ranks = s.cfg.nranks;
        B2_CUDA(kernels::launch_ring(args.dtype, args.redop, per.data(), cfg));
    } else {
        for (std::size_t i = 0; i < s.cfg.local.size(); ++i) {
            DeviceGuard guard(s.cfg.local[i].device);
            cfg.stream = args.streams[i];
            B2_CUDA(kernels::launch_ring(args.dtype, args.redop, &per[i], cfg));
        }
    }
}

}  // namespace b200ccl
