// RDMA edge set: one reliable-connection queue pair, one registered FIFO (pinned host memory, or
// device memory with GDR) and, on the WRITE plane, one clear-to-send ring per ring edge, channel
// and direction; proxies driven by a progress engine.
//
// Set-up order follows nano-nccl communicator.cu:490-785: create queue pairs and register
// memory; exchange the 64-byte peer records (all of them are published before any is read, so
// loopback pairs cannot deadlock); connect (RTR → RTS); receive proxies prepare first; only after
// every process has done so do send proxies start.
#include "core/check.h"
#include "sched/ring_geometry.h"
#include "transport/net_edge.h"
#include "transport/rdma/gdr.h"
#include "transport/rdma/progress.h"

#include <cstdio>
#include <map>

namespace b200ccl::transport {

namespace {

using namespace b200ccl::transport::rdma;

struct Half {
    bool sender = false;
    ProxyIdentity id;
    int device = 0;
    std::unique_ptr<RegisteredFifo> fifo;
    MappedU64Array counters;  // [0] tail, [1] head
    MappedU32Array sizes;
    std::unique_ptr<CompletionQueue> cq;
    std::unique_ptr<QueuePair> qp;
    MappedBuffer<RdmaCtsSlot> cts_ring;  // sender only, WRITE plane
    MemoryRegion cts_mr;
    RdmaPeerInfo local{}, remote{};
    NetHalf view;
    std::unique_ptr<RdmaProxy> proxy;
    std::unique_ptr<ProxyTimeline> timeline;
};

class RdmaEdgeSet final : public NetEdgeSet {
public:
    RdmaEdgeSet(const NetEdgeConfig& cfg, Bootstrap* bs) : cfg_(cfg), bs_(bs), abort_(1) {
        backend_ = create_backend();
        plane_ = data_plane_from_env();
        placement_ = fifo_placement_from_env();
        errors_ = std::make_shared<AsyncErrorState>("rdma", abort_.get());
        const int n = cfg.nranks, C = cfg.channels;
        const int nproc = bs ? bs->size() : 1, me = bs ? bs->rank() : 0;
        struct Range { int first, count; };
        Range mine{cfg.local.front().global_rank, static_cast<int>(cfg.local.size())};
        std::vector<Range> ranges(nproc);
        if (bs) bs->allgather(&mine, ranges.data(), sizeof(Range));
        else ranges[0] = mine;
        std::vector<int> owner(n, -1);
        for (int p = 0; p < nproc; ++p)
            for (int k = 0; k < ranges[p].count; ++k) owner[ranges[p].first + k] = p;
        if (backend_->name() == "fake" && nproc > 1)
            throw std::runtime_error("rdma: the fake backend connects queue pairs of one process only");

        const std::size_t step_bytes = cfg.fifo_bytes / ring::kFifoSteps;
        const std::size_t cts_slots = ring::kFifoSteps / ring::kSliceSteps;
        auto make_half = [&](bool sender, int src, int dst, int c, int device) {
            auto h = std::unique_ptr<Half>(new Half());
            h->sender = sender;
            h->id = ProxyIdentity{src, dst, c};
            h->device = device;
            h->fifo.reset(new RegisteredFifo(backend_, placement_, cfg.fifo_bytes, device));
            const int node = numa::gpu_node(device);
            h->counters.reset(2, node);
            h->sizes.reset(ring::kFifoSteps, node);
            h->cq = backend_->create_cq(32);
            h->qp = backend_->create_qp(h->cq.get(), 16, 16);
            h->qp->fill_local_info(&h->local);
            if (sender && plane_ == DataPlane::WriteCts) {
                h->cts_ring.reset(cts_slots, node);
                h->cts_mr = backend_->register_memory(h->cts_ring.get(), cts_slots * sizeof(RdmaCtsSlot));
                h->local.cts_fifo_addr = reinterpret_cast<std::uint64_t>(h->cts_ring.get());
                h->local.cts_fifo_rkey = h->cts_mr.rkey;
                h->local.cts_fifo_slots = static_cast<std::uint32_t>(cts_slots);
            }
            if (!sender) {
                h->local.recv_fifo_addr = reinterpret_cast<std::uint64_t>(h->fifo->data());
                h->local.recv_fifo_rkey = h->fifo->region().rkey;
                h->local.recv_fifo_bytes = static_cast<std::uint32_t>(cfg.fifo_bytes);
            }
            h->view.fifo = h->fifo->data();
            h->view.tail = &h->counters[0];
            h->view.head = &h->counters[1];
            h->view.sizes = h->sizes.get();
            return h;
        };
        for (const auto& l : cfg.local) {
            const int r = l.global_rank, next = (r + 1) % n, prev = (r + n - 1) % n;
            if (cfg.all_edges || owner[next] != me)
                for (int c = 0; c < C; ++c) send_[{r, c}] = make_half(true, r, next, c, l.device);
            if (cfg.all_edges || owner[prev] != me)
                for (int c = 0; c < C; ++c) recv_[{r, c}] = make_half(false, prev, r, c, l.device);
        }

        // Publish every local record, then read the partners'. Records are indexed by
        // (edge source rank, channel, direction): the send half of edge r pairs with the
        // receive half held by rank r+1.
        const std::size_t per_rank = static_cast<std::size_t>(C) * 2;
        std::vector<RdmaPeerInfo> mine_tbl(static_cast<std::size_t>(n) * per_rank), all_tbl;
        for (auto& kv : send_) mine_tbl[(kv.second->id.source_rank * C + kv.first.second) * 2 + 0] = kv.second->local;
        for (auto& kv : recv_) mine_tbl[(kv.second->id.source_rank * C + kv.first.second) * 2 + 1] = kv.second->local;
        if (bs) {
            std::vector<RdmaPeerInfo> gathered(mine_tbl.size() * nproc);
            bs->allgather(mine_tbl.data(), gathered.data(), mine_tbl.size() * sizeof(RdmaPeerInfo));
            all_tbl.assign(mine_tbl.size(), RdmaPeerInfo{});
            for (int p = 0; p < nproc; ++p)
                for (std::size_t i = 0; i < mine_tbl.size(); ++i)
                    if (gathered[p * mine_tbl.size() + i].qpn != 0) all_tbl[i] = gathered[p * mine_tbl.size() + i];
        } else {
            all_tbl = mine_tbl;
        }
        std::string err;
        try {
            for (auto& kv : send_) {
                Half& h = *kv.second;
                h.remote = all_tbl[(h.id.source_rank * C + h.id.channel) * 2 + 1];
                if (h.remote.qpn == 0) throw std::runtime_error("rdma: no receive half published for edge " + std::to_string(h.id.source_rank));
                h.qp->connect(h.remote);
            }
            for (auto& kv : recv_) {
                Half& h = *kv.second;
                h.remote = all_tbl[(h.id.source_rank * C + h.id.channel) * 2 + 0];
                if (h.remote.qpn == 0) throw std::runtime_error("rdma: no send half published for edge " + std::to_string(h.id.source_rank));
                h.qp->connect(h.remote);
            }
        } catch (const std::exception& e) {
            err = e.what();
        }
        const std::string all_err = bs ? bs->error_consensus(err) : err;
        if (!all_err.empty()) throw std::runtime_error("rdma edge setup failed: " + all_err);

        const bool timeline = timeline_enabled_from_env();
        engine_.reset(new ProgressEngine(shared_progress_from_env(), numa::gpu_node(cfg.local.front().device)));
        auto fifo_of = [&](Half& h) {
            RdmaFifo f;
            f.data = static_cast<std::uint8_t*>(h.fifo->data());
            f.slot_bytes = step_bytes;
            f.slot_count = ring::kFifoSteps;
            f.slot_sizes = h.sizes.get();
            f.step_increment = ring::kSliceSteps;
            f.mr = h.fifo->region();
            return f;
        };
        for (auto& kv : recv_) {
            Half& h = *kv.second;
            CtsRemoteRing cts{h.remote.cts_fifo_addr, h.remote.cts_fifo_rkey, h.remote.cts_fifo_slots};
            h.proxy.reset(new RdmaRecvProxy(h.qp.get(), h.cq.get(), fifo_of(h), h.view.head, h.view.tail, h.id, plane_, cts, errors_));
        }
        for (auto& kv : send_) {
            Half& h = *kv.second;
            CtsLocalRing cts{h.cts_ring.get(), h.cts_ring.count()};
            h.proxy.reset(new RdmaSendProxy(h.qp.get(), h.cq.get(), fifo_of(h), h.view.head, h.view.tail, h.id, plane_, cts, errors_));
        }
        for (auto* m : {&recv_, &send_}) {
            for (auto& kv : *m) {
                Half& h = *kv.second;
                if (timeline) {
                    h.timeline.reset(new ProxyTimeline(std::string(h.sender ? "send" : "recv") + " source=" + std::to_string(h.id.source_rank) +
                                                       " destination=" + std::to_string(h.id.destination_rank) + " channel=" +
                                                       std::to_string(h.id.channel)));
                    h.proxy->set_timeline(h.timeline.get());
                }
                engine_->add(h.proxy.get());
            }
        }
    }

    ~RdmaEdgeSet() override {
        stop();
        for (auto* m : {&recv_, &send_})
            for (auto& kv : *m) {
                if (kv.second->timeline) std::fputs(kv.second->timeline->dump().c_str(), stderr);
                if (kv.second->cts_mr.addr) backend_->deregister(kv.second->cts_mr);
            }
    }

    const NetHalf* send_half(int r, int c) const override {
        auto it = send_.find({r, c});
        return it == send_.end() ? nullptr : &it->second->view;
    }
    const NetHalf* recv_half(int r, int c) const override {
        auto it = recv_.find({r, c});
        return it == recv_.end() ? nullptr : &it->second->view;
    }
    const unsigned int* abort_word() const override { return abort_.get(); }

    void start() override {
        engine_->start_receivers();
        if (bs_) bs_->barrier();  // every receiver everywhere is ready before any sender starts
        engine_->start_senders();
    }

    void stop() override {
        if (stopped_) return;
        stopped_ = true;
        if (!errors_->has_error()) {
            for (auto& kv : send_) {
                auto* sp = static_cast<RdmaSendProxy*>(kv.second->proxy.get());
                for (int spin = 0; spin < 2000000 && !sp->drained(); ++spin) sched_yield();
            }
        }
        if (engine_) engine_->stop();
    }

    std::string first_error() const override { return errors_->message(); }

private:
    NetEdgeConfig cfg_;
    Bootstrap* bs_;
    MappedU32Array abort_;
    std::shared_ptr<VerbsBackend> backend_;
    DataPlane plane_ = DataPlane::SendRecv;
    FifoPlacement placement_ = FifoPlacement::HostPinned;
    std::shared_ptr<AsyncErrorState> errors_;
    std::map<std::pair<int, int>, std::unique_ptr<Half>> send_, recv_;
    std::unique_ptr<ProgressEngine> engine_;
    bool stopped_ = false;
};

}  // namespace

std::unique_ptr<NetEdgeSet> create_rdma_edges(const NetEdgeConfig& config, Bootstrap* bootstrap) {
    return std::unique_ptr<NetEdgeSet>(new RdmaEdgeSet(config, bootstrap));
}

}  // namespace b200ccl::transport
