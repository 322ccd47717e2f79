// Socket edge set: connects every ring edge that leaves this process over TCP and runs its
// proxies. Listener creation uses error consensus: if any process cannot set up its listener,
// every process throws the same message (nano-nccl mpi_communicator.cc:38-75). The process with
// the lower bootstrap rank connects, the higher one accepts; each connection starts with a HELLO
// that is checked against the expected (source, destination, channel) set and for duplicates
// (mpi_communicator.cc:210-247).
#include "core/buffers.h"
#include "core/check.h"
#include "sched/ring_geometry.h"
#include "transport/net_edge.h"
#include "transport/socket/proxy.h"

#include <map>
#include <set>
#include <tuple>

namespace b200ccl::transport {

namespace {

using namespace b200ccl::transport::socket;

struct Half {
    MappedBuffer<unsigned char> fifo;
    MappedU64Array counters;  // [0] tail, [1] head
    MappedU32Array sizes;     // per FIFO step
    NetHalf view;
    Fd connection;
    ProxyIdentity id;
    int numa_node = 0;
};

class SocketEdgeSet final : public NetEdgeSet {
public:
    SocketEdgeSet(const NetEdgeConfig& cfg, Bootstrap* bs) : cfg_(cfg), bs_(bs), abort_(1) {
        errors_ = std::make_shared<AsyncErrorState>("socket", abort_.get());
        const int n = cfg.nranks, C = cfg.channels;
        // Which process owns which rank.
        struct Range { int first, count; };
        const int nproc = bs ? bs->size() : 1, me = bs ? bs->rank() : 0;
        Range mine{cfg.local.front().global_rank, static_cast<int>(cfg.local.size())};
        std::vector<Range> ranges(nproc);
        if (bs) bs->allgather(&mine, ranges.data(), sizeof(Range));
        else ranges[0] = mine;
        std::vector<int> owner(n, -1);
        for (int p = 0; p < nproc; ++p)
            for (int k = 0; k < ranges[p].count; ++k) owner[ranges[p].first + k] = p;
        // The process of the sending rank opens the connection when its bootstrap rank is not
        // higher than the receiver's (equal = loopback inside one process); else the receiver's does.
        auto sender_connects = [&](int src, int dst) { return owner[src] <= owner[dst]; };

        // Listener with consensus.
        std::string err;
        try {
            listener_ = Listener::create(socket_ifname_from_env());
        } catch (const std::exception& e) {
            err = std::string("socket listener setup failed: ") + e.what();
        }
        const std::string all_err = bs ? bs->error_consensus(err) : err;
        if (!all_err.empty()) throw std::runtime_error("socket listener setup failed on " + all_err);
        std::vector<SocketAddress> addrs(nproc);
        if (bs) bs->allgather(&listener_.address(), addrs.data(), sizeof(SocketAddress));
        else addrs[0] = listener_.address();

        // Halves of this process.
        const std::size_t step_bytes = cfg.fifo_bytes / ring::kFifoSteps;
        auto make_half = [&](int src, int dst, int c, int device) {
            auto h = std::unique_ptr<Half>(new Half());
            h->numa_node = numa::gpu_node(device);
            h->fifo.reset(cfg.fifo_bytes, h->numa_node);
            h->counters.reset(2, h->numa_node);
            h->sizes.reset(ring::kFifoSteps, h->numa_node);
            h->view.fifo = h->fifo.get();
            h->view.tail = &h->counters[0];
            h->view.head = &h->counters[1];
            h->view.sizes = h->sizes.get();
            h->id = ProxyIdentity{src, dst, c};
            (void)step_bytes;
            return h;
        };
        int expected_accepts = 0;
        std::set<std::tuple<int, int, int>> expected;  // (src, dst, channel) of connections to accept
        for (const auto& l : cfg.local) {
            const int r = l.global_rank, next = (r + 1) % n, prev = (r + n - 1) % n;
            if (cfg.all_edges || owner[next] != me)
                for (int c = 0; c < C; ++c) send_[{r, c}] = make_half(r, next, c, l.device);
            if (cfg.all_edges || owner[prev] != me)
                for (int c = 0; c < C; ++c) recv_[{r, c}] = make_half(prev, r, c, l.device);
        }
        // Connect or accept, per edge and channel.
        const int timeout_ms = 30000;
        for (auto& kv : send_) {
            Half& h = *kv.second;
            if (sender_connects(h.id.source_rank, h.id.destination_rank))
                h.connection = connect_with_hello(addrs[owner[h.id.destination_rank]], h.id.channel, h.id.source_rank,
                                                  h.id.destination_rank, timeout_ms);
            else { expected.insert({h.id.source_rank, h.id.destination_rank, h.id.channel}); ++expected_accepts; }
        }
        for (auto& kv : recv_) {
            Half& h = *kv.second;
            if (!sender_connects(h.id.source_rank, h.id.destination_rank))
                h.connection = connect_with_hello(addrs[owner[h.id.source_rank]], h.id.channel, h.id.source_rank,
                                                  h.id.destination_rank, timeout_ms);
            else { expected.insert({h.id.source_rank, h.id.destination_rank, h.id.channel}); ++expected_accepts; }
        }
        std::string accept_err;
        try {
            for (int k = 0; k < expected_accepts; ++k) {
                auto got = listener_.accept_hello(timeout_ms);
                const WireHello& hello = got.second;
                const auto key = std::make_tuple(static_cast<int>(hello.source_rank), static_cast<int>(hello.destination_rank),
                                                 static_cast<int>(hello.channel));
                if (!expected.count(key))
                    throw std::runtime_error("unexpected or duplicate socket hello source=" + std::to_string(hello.source_rank) +
                                             " destination=" + std::to_string(hello.destination_rank) + " channel=" +
                                             std::to_string(hello.channel));
                expected.erase(key);
                // The accepting half is the one that did not connect.
                Half* h = nullptr;
                if (sender_connects(static_cast<int>(hello.source_rank), static_cast<int>(hello.destination_rank))) {
                    auto r = recv_.find({static_cast<int>(hello.destination_rank), static_cast<int>(hello.channel)});
                    if (r != recv_.end()) h = r->second.get();
                } else {
                    auto s = send_.find({static_cast<int>(hello.source_rank), static_cast<int>(hello.channel)});
                    if (s != send_.end()) h = s->second.get();
                }
                if (!h) throw std::runtime_error("socket hello matches no local edge");
                h->connection = std::move(got.first);
            }
        } catch (const std::exception& e) {
            accept_err = e.what();
        }
        const std::string all_accept = bs ? bs->error_consensus(accept_err) : accept_err;
        if (!all_accept.empty()) throw std::runtime_error("socket edge setup failed on " + all_accept);

        // Proxies.
        for (auto& kv : send_) {
            Half& h = *kv.second;
            ProxyFifo f{h.fifo.get(), step_bytes, static_cast<std::size_t>(ring::kFifoSteps), h.sizes.get(),
                        static_cast<std::size_t>(ring::kSliceSteps)};
            send_proxies_.emplace_back(new SendProxy(std::move(h.connection), f, SendControl{h.view.head, h.view.tail}, h.id,
                                                     h.numa_node, errors_));
        }
        for (auto& kv : recv_) {
            Half& h = *kv.second;
            ProxyFifo f{h.fifo.get(), step_bytes, static_cast<std::size_t>(ring::kFifoSteps), h.sizes.get(),
                        static_cast<std::size_t>(ring::kSliceSteps)};
            recv_proxies_.emplace_back(new RecvProxy(std::move(h.connection), f, RecvControl{h.view.head, h.view.tail}, h.id,
                                                     h.numa_node, errors_));
        }
    }

    ~SocketEdgeSet() override { stop(); }

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
        // Receivers are up before any sender may write (communicator.cu:749-784 of the reference).
        for (auto& p : recv_proxies_) p->start();
        if (bs_) bs_->barrier();
        for (auto& p : send_proxies_) p->start();
    }

    void stop() override {
        if (stopped_) return;
        stopped_ = true;
        if (!errors_->has_error())
            for (auto& p : send_proxies_) p->drain();
        for (auto& p : send_proxies_) p->stop();
        for (auto& p : recv_proxies_) p->stop();
        for (auto& p : send_proxies_) p->shutdown();
        for (auto& p : recv_proxies_) p->shutdown();
        for (auto& p : send_proxies_) p->join();
        for (auto& p : recv_proxies_) p->join();
    }

    std::string first_error() const override { return errors_->message(); }

private:
    NetEdgeConfig cfg_;
    Bootstrap* bs_;
    MappedU32Array abort_;
    std::shared_ptr<AsyncErrorState> errors_;
    Listener listener_;
    std::map<std::pair<int, int>, std::unique_ptr<Half>> send_, recv_;  // key (local rank's global id, channel)
    std::vector<std::unique_ptr<SendProxy>> send_proxies_;
    std::vector<std::unique_ptr<RecvProxy>> recv_proxies_;
    bool stopped_ = false;
};

}  // namespace

std::unique_ptr<NetEdgeSet> create_socket_edges(const NetEdgeConfig& config, Bootstrap* bootstrap) {
    return std::unique_ptr<NetEdgeSet>(new SocketEdgeSet(config, bootstrap));
}

}  // namespace b200ccl::transport
