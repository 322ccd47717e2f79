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
    // Peer-to-peer edges: every rank's incoming FIFOs (channels × fifo_bytes) in its own memory.
    std::unique_ptr<mem::SymmetricRegion> fifo_region;
    const mem::SymmetricRegion* ctrl = nullptr;
    // Host (SHM) edges: FIFO and counters of edge e, channel c at index e*channels + c.
    std::vector<MappedBuffer<unsigned char>> host_fifo;
    MappedU64Array host_counters;  // [(e*channels + c)*2 + {0 tail, 1 head}]
    MappedU64Array host_base;      // [(rank*channels + c)*2 + {0 send, 1 recv}]
    std::vector<DeviceBuffer<dev::ControlBlock>> own_ctrl;  // host mode: one private block per local rank
    // Network edges (socket / RDMA) of this process, by direction.
    std::unique_ptr<transport::NetEdgeSet> net;
    std::vector<DeviceBuffer<dev::RingChannel>> tables;  // per local rank: [channels]
    MappedBuffer<dev::RingTurnaroundStats> stats;        // [local rank][channel], optional
};

namespace {
int local_index_of(const RingEngineConfig& cfg, int grank) {
    for (std::size_t i = 0; i < cfg.local.size(); ++i)
        if (cfg.local[i].global_rank == grank) return static_cast<int>(i);
    return -1;
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
    s.fifo_bytes = env::get_bytes("B200CCL_FIFO_BUFF_BYTES", ring::kDefaultFifoBytes, "NANO_NCCL_FIFO_BUFF_BYTES");
    const std::size_t quantum = ring::kFifoSteps * ring::kGrainBytes;
    if (s.fifo_bytes < quantum || s.fifo_bytes % quantum != 0)
        throw std::invalid_argument("FIFO size must be a positive multiple of " + std::to_string(quantum) + " bytes");

    const bool host = config.use_host_fifo;
    const bool net = config.net_kind != TransportKind::Auto;
    if (!host) {
        if (!alloc || !ctrl) throw std::invalid_argument("peer-to-peer ring needs symmetric memory");
        s.fifo_region = alloc->allocate(static_cast<std::size_t>(C) * s.fifo_bytes, "ring-fifo");
    } else {
        // SHM: one FIFO per edge and channel in mapped host memory on the RECEIVER's NUMA node
        // (nano-nccl communicator.cu:915-934), counters and base steps in mapped host memory too.
        s.host_fifo.resize(static_cast<std::size_t>(n) * C);
        for (int e = 0; e < n; ++e) {
            const int dst_local = local_index_of(config, (e + 1) % n);
            const int node = dst_local >= 0 ? numa::gpu_node(config.local[dst_local].device) : -1;
            for (int c = 0; c < C; ++c) s.host_fifo[e * C + c].reset(s.fifo_bytes, node);
        }
        s.host_counters.reset(static_cast<std::size_t>(n) * C * 2);
        s.host_base.reset(static_cast<std::size_t>(n) * C * 2);
        for (const auto& l : config.local) {
            s.own_ctrl.emplace_back(l.device, 1);
            s.own_ctrl.back().zero();
        }
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

    // Wire every local rank's channel table.
    for (std::size_t i = 0; i < config.local.size(); ++i) {
        const int r = config.local[i].global_rank;
        const int next = (r + 1) % n, prev = (r + n - 1) % n;
        std::vector<dev::RingChannel> table(C);
        for (int c = 0; c < C; ++c) {
            dev::RingChannel ch;
            std::memset(&ch, 0, sizeof(ch));
            if (host) {
                const int out_e = r, in_e = prev;  // edge e goes e → e+1
                ch.send_fifo = s.host_fifo[out_e * C + c].get();
                ch.recv_fifo = s.host_fifo[in_e * C + c].get();
                ch.send_tail = &s.host_counters[(out_e * C + c) * 2 + 0];
                ch.send_head = &s.host_counters[(out_e * C + c) * 2 + 1];
                ch.recv_tail = &s.host_counters[(in_e * C + c) * 2 + 0];
                ch.recv_head = &s.host_counters[(in_e * C + c) * 2 + 1];
                ch.send_base = &s.host_base[(r * C + c) * 2 + 0];
                ch.recv_base = &s.host_base[(r * C + c) * 2 + 1];
            } else {
                auto* mine = static_cast<dev::ControlBlock*>(ctrl->rank_ptr(r));
                auto* nxt = static_cast<dev::ControlBlock*>(ctrl->rank_ptr(next));
                auto* prv = static_cast<dev::ControlBlock*>(ctrl->rank_ptr(prev));
                ch.send_fifo = static_cast<char*>(s.fifo_region->rank_ptr(next)) + static_cast<std::size_t>(c) * s.fifo_bytes;
                ch.recv_fifo = static_cast<char*>(s.fifo_region->rank_ptr(r)) + static_cast<std::size_t>(c) * s.fifo_bytes;
                ch.send_tail = &nxt->ring_recv_tail[c];  // publish into the next rank
                ch.send_head = &mine->ring_send_head[c];  // poll locally
                ch.recv_tail = &mine->ring_recv_tail[c];  // poll locally
                ch.recv_head = &prv->ring_send_head[c];   // publish into the previous rank
                ch.send_base = &mine->ring_send_base[c];
                ch.recv_base = &mine->ring_recv_base[c];
            }
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
    }
    if (s.net) s.net->start();
    if (bootstrap) bootstrap->barrier();
    log_info("ring engine: %d channels, %zu-byte FIFOs, %s edges%s", C, s.fifo_bytes, host ? "host" : "peer-to-peer",
             s.net ? " + network edges" : "");
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
        a.own_ctrl = s.cfg.use_host_fifo ? s.own_ctrl[i].get()
                                         : static_cast<dev::ControlBlock*>(s.ctrl->rank_ptr(s.cfg.local[i].global_rank));
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
