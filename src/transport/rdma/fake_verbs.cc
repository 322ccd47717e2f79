#include "transport/rdma/fake_verbs.h"

#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <stdexcept>
#include <vector>

namespace b200ccl::transport::rdma {

namespace {
struct FakeCq;
struct FakeQp;
}  // namespace

struct FakeVerbs::Impl {
    std::mutex mu;
    std::uint32_t next_key = 0x1000;
    std::uint32_t next_qpn = 100;
    std::map<std::uint32_t, MemoryRegion> regions;  // by rkey
    std::map<std::uint32_t, FakeQp*> qps;           // by qpn
    std::uint64_t sends = 0, signaled = 0, inlined = 0, recvs = 0, regs = 0;
    std::uint64_t fail_at = 0;
    int fail_status = 0;
};

namespace {

struct FakeCq : CompletionQueue {
    std::shared_ptr<FakeVerbs::Impl> impl;
    std::deque<Completion> done;
    int poll(int max_entries, Completion* out) override {
        std::lock_guard<std::mutex> lock(impl->mu);
        int n = 0;
        while (n < max_entries && !done.empty()) {
            out[n++] = done.front();
            done.pop_front();
        }
        return n;
    }
};

struct PendingSend {
    SendWr wr;
    std::vector<unsigned char> inline_copy;
    bool failed = false;
    int status = 0;
};

struct FakeQp : QueuePair {
    std::shared_ptr<FakeVerbs::Impl> impl;
    FakeCq* cq = nullptr;
    std::uint32_t qpn = 0;
    FakeQp* peer = nullptr;
    bool connected = false;
    bool broken = false;
    std::deque<RecvWr> recv_queue;
    std::deque<PendingSend> send_queue;  // in order; the head may wait for a receive at the peer
    int max_send = 0, max_recv = 0;

    ~FakeQp() override {
        std::lock_guard<std::mutex> lock(impl->mu);
        impl->qps.erase(qpn);
        if (peer) peer->peer = nullptr;
    }

    void fill_local_info(RdmaPeerInfo* info) const override {
        info->qpn = qpn;
        info->psn = qpn * 7 + 1;
        info->lid = 1;
        info->gid_index = 0;
        info->active_mtu = 5;
        std::memset(info->gid, 0, sizeof(info->gid));
        info->gid[15] = static_cast<std::uint8_t>(qpn);
    }

    void connect(const RdmaPeerInfo& remote) override {
        std::lock_guard<std::mutex> lock(impl->mu);
        (void)negotiate_path_mtu(5, remote.active_mtu);
        auto it = impl->qps.find(remote.qpn);
        if (it == impl->qps.end()) throw std::runtime_error("fake verbs: unknown remote qpn " + std::to_string(remote.qpn));
        peer = it->second;
        connected = true;
    }

    // Caller holds impl->mu.
    bool in_region(std::uint64_t addr, std::uint32_t len, std::uint32_t rkey) const {
        auto it = impl->regions.find(rkey);
        if (it == impl->regions.end()) return false;
        const auto base = reinterpret_cast<std::uint64_t>(it->second.addr);
        return addr >= base && addr + len <= base + it->second.length;
    }

    void complete_send(const PendingSend& p, int status) {
        if (p.wr.signaled || status != 0) {
            Completion c;
            c.wr_id = p.wr.wr_id;
            c.status = status;
            c.opcode = p.wr.opcode == WrOpcode::Send ? WcOpcode::Send : WcOpcode::RdmaWrite;
            cq->done.push_back(c);
        }
    }

    // Delivers queued sends in order while their needs are met. Caller holds impl->mu.
    void pump() {
        while (!send_queue.empty() && !broken) {
            PendingSend& p = send_queue.front();
            if (p.failed) {
                complete_send(p, p.status);
                broken = true;  // an RC queue pair stops after an error
                send_queue.pop_front();
                break;
            }
            if (!peer || !peer->connected) break;
            const void* src = p.wr.inline_data ? p.inline_copy.data() : p.wr.local_addr;
            const bool needs_recv = p.wr.opcode != WrOpcode::RdmaWrite;
            if (needs_recv && peer->recv_queue.empty()) break;  // receiver not ready: retried later
            if (p.wr.opcode == WrOpcode::Send) {
                const RecvWr r = peer->recv_queue.front();
                peer->recv_queue.pop_front();
                Completion rc;
                rc.wr_id = r.wr_id;
                rc.opcode = WcOpcode::Recv;
                if (p.wr.length > r.length) {
                    rc.status = 1;  // local length error at the receiver
                    peer->cq->done.push_back(rc);
                    complete_send(p, 9);
                    broken = true;
                    send_queue.pop_front();
                    break;
                }
                if (p.wr.length) std::memcpy(r.addr, src, p.wr.length);
                rc.byte_len = p.wr.length;
                peer->cq->done.push_back(rc);
            } else {
                if (!in_region(p.wr.remote_addr, p.wr.length, p.wr.rkey)) {
                    complete_send(p, 10);  // remote access error
                    broken = true;
                    send_queue.pop_front();
                    break;
                }
                if (p.wr.length) std::memcpy(reinterpret_cast<void*>(p.wr.remote_addr), src, p.wr.length);
                if (p.wr.opcode == WrOpcode::RdmaWriteWithImm) {
                    const RecvWr r = peer->recv_queue.front();
                    peer->recv_queue.pop_front();
                    Completion rc;
                    rc.wr_id = r.wr_id;
                    rc.opcode = WcOpcode::RecvRdmaWithImm;
                    rc.byte_len = p.wr.length;
                    rc.imm = p.wr.imm;
                    peer->cq->done.push_back(rc);
                }
            }
            complete_send(p, 0);
            send_queue.pop_front();
        }
    }

    void post_send(const SendWr& wr) override {
        std::lock_guard<std::mutex> lock(impl->mu);
        if (!connected) throw std::runtime_error("fake verbs: post_send on an unconnected queue pair");
        if (broken) {
            // A queue pair in the error state accepts work requests and flushes them with errors.
            Completion c;
            c.wr_id = wr.wr_id;
            c.status = 5;  // flushed
            c.opcode = wr.opcode == WrOpcode::Send ? WcOpcode::Send : WcOpcode::RdmaWrite;
            cq->done.push_back(c);
            return;
        }
        if (static_cast<int>(send_queue.size()) >= max_send) throw std::runtime_error("fake verbs: send queue full");
        if (wr.inline_data && wr.length > kMaxInlineData) throw std::runtime_error("fake verbs: inline data too long");
        PendingSend p;
        p.wr = wr;
        if (wr.inline_data) p.inline_copy.assign(static_cast<const unsigned char*>(wr.local_addr),
                                                 static_cast<const unsigned char*>(wr.local_addr) + wr.length);
        ++impl->sends;
        if (wr.signaled) ++impl->signaled;
        if (wr.inline_data) ++impl->inlined;
        if (impl->fail_at != 0 && impl->sends == impl->fail_at) {
            p.failed = true;
            p.status = impl->fail_status;
        }
        send_queue.push_back(std::move(p));
        pump();
    }

    void post_recv(const RecvWr& wr) override {
        std::lock_guard<std::mutex> lock(impl->mu);
        if (static_cast<int>(recv_queue.size()) >= max_recv) throw std::runtime_error("fake verbs: receive queue full");
        recv_queue.push_back(wr);
        ++impl->recvs;
        if (peer) peer->pump();
    }
};

}  // namespace

FakeVerbs::FakeVerbs() : impl_(std::make_shared<Impl>()) {}
FakeVerbs::~FakeVerbs() = default;

MemoryRegion FakeVerbs::register_memory(void* addr, std::size_t length) {
    std::lock_guard<std::mutex> lock(impl_->mu);
    MemoryRegion mr;
    mr.addr = addr;
    mr.length = length;
    mr.lkey = mr.rkey = impl_->next_key++;
    mr.handle = mr.rkey;
    impl_->regions[mr.rkey] = mr;
    ++impl_->regs;
    return mr;
}

MemoryRegion FakeVerbs::register_device_memory(void* addr, std::size_t length) {
    if (!allow_device_registration) throw std::runtime_error("rdma gdr: device memory registration unavailable");
    return register_memory(addr, length);
}

void FakeVerbs::deregister(const MemoryRegion& mr) {
    std::lock_guard<std::mutex> lock(impl_->mu);
    impl_->regions.erase(mr.rkey);
}

std::unique_ptr<CompletionQueue> FakeVerbs::create_cq(int) {
    auto cq = std::unique_ptr<FakeCq>(new FakeCq());
    cq->impl = impl_;
    return cq;
}

std::unique_ptr<QueuePair> FakeVerbs::create_qp(CompletionQueue* cq, int max_send_wr, int max_recv_wr) {
    std::lock_guard<std::mutex> lock(impl_->mu);
    auto qp = std::unique_ptr<FakeQp>(new FakeQp());
    qp->impl = impl_;
    qp->cq = static_cast<FakeCq*>(cq);
    qp->qpn = impl_->next_qpn++;
    qp->max_send = max_send_wr;
    qp->max_recv = max_recv_wr;
    impl_->qps[qp->qpn] = qp.get();
    return qp;
}

void FakeVerbs::fail_send_number(std::uint64_t n, int status) {
    std::lock_guard<std::mutex> lock(impl_->mu);
    impl_->fail_at = n;
    impl_->fail_status = status;
}
std::uint64_t FakeVerbs::sends_posted() const { std::lock_guard<std::mutex> l(impl_->mu); return impl_->sends; }
std::uint64_t FakeVerbs::signaled_sends() const { std::lock_guard<std::mutex> l(impl_->mu); return impl_->signaled; }
std::uint64_t FakeVerbs::inline_sends() const { std::lock_guard<std::mutex> l(impl_->mu); return impl_->inlined; }
std::uint64_t FakeVerbs::recvs_posted() const { std::lock_guard<std::mutex> l(impl_->mu); return impl_->recvs; }
std::uint64_t FakeVerbs::registrations() const { std::lock_guard<std::mutex> l(impl_->mu); return impl_->regs; }

}  // namespace b200ccl::transport::rdma
