// The libibverbs backend of the RDMA transport (src/transport/rdma/verbs/ibverbs_backend.cc),
// compiled against the stand-in verbs header of this folder and run over its in-process loopback
// fabric: device / port / GID selection and their error messages, the INIT → RTR → RTS attribute
// masks (the stand-in refuses a transition whose mask lacks a required attribute), both data planes
// of the real send / receive proxies (four slices, credit back-pressure, ring wrap, shared and
// dedicated progress threads), RoCE addressing, a mis-wired pair, memory registration and a leak
// count at the end. No HCA, no GPU. Modelled on the reference's tests/rdma_bootstrap.cu (two RC
// queue pairs on one endpoint) and tests/rdma_proxy_test.cc:454-726.
#include "../check.h"
#include "transport/rdma/progress.h"
#include "transport/rdma/proxy.h"
#include "transport/rdma/verbs_backend.h"

#include <infiniband/verbs.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace b200ccl::transport::rdma {
std::shared_ptr<VerbsBackend> create_ibverbs_backend();
}

using namespace b200ccl::transport;
using namespace b200ccl::transport::rdma;

namespace {

constexpr std::size_t kSlots = 8, kSlotBytes = 64, kInc = 2;

struct Side {
    std::vector<std::uint8_t> data = std::vector<std::uint8_t>(kSlots * kSlotBytes, 0);
    unsigned int sizes[kSlots] = {0};
    unsigned long long head = 0, tail = 0;
    MemoryRegion mr;
    std::unique_ptr<CompletionQueue> cq;
    std::unique_ptr<QueuePair> qp;
    RdmaFifo fifo() { return RdmaFifo{data.data(), kSlotBytes, kSlots, sizes, kInc, mr}; }
};

struct Link {
    std::shared_ptr<VerbsBackend> verbs = create_ibverbs_backend();
    Side s, r;
    std::vector<RdmaCtsSlot> cts = std::vector<RdmaCtsSlot>(kSlots / kInc);
    MemoryRegion cts_mr;
    std::shared_ptr<AsyncErrorState> errors = std::make_shared<AsyncErrorState>("rdma");
    std::unique_ptr<RdmaSendProxy> send;
    std::unique_ptr<RdmaRecvProxy> recv;

    explicit Link(DataPlane plane) {
        T_CHECK(verbs->name() == "ibverbs");
        for (Side* side : {&s, &r}) {
            side->mr = verbs->register_memory(side->data.data(), side->data.size());
            side->cq = verbs->create_cq(32);
            side->qp = verbs->create_qp(side->cq.get(), 16, 16);
        }
        std::memset(cts.data(), 0, cts.size() * sizeof(RdmaCtsSlot));
        cts_mr = verbs->register_memory(cts.data(), cts.size() * sizeof(RdmaCtsSlot));
        RdmaPeerInfo si{}, ri{};
        s.qp->fill_local_info(&si);
        r.qp->fill_local_info(&ri);
        T_CHECK(si.qpn != ri.qpn && si.active_mtu == 5 && si.gid[0] == 0xfe);
        s.qp->connect(ri);
        r.qp->connect(si);
        send.reset(new RdmaSendProxy(s.qp.get(), s.cq.get(), s.fifo(), &s.head, &s.tail, ProxyIdentity{4, 5, 1}, plane,
                                     CtsLocalRing{cts.data(), cts.size()}, errors));
        recv.reset(new RdmaRecvProxy(r.qp.get(), r.cq.get(), r.fifo(), &r.head, &r.tail, ProxyIdentity{4, 5, 1}, plane,
                                     CtsRemoteRing{reinterpret_cast<std::uint64_t>(cts.data()), cts_mr.rkey, cts.size()}, errors, false));
        recv->prepare();
    }
    ~Link() {
        send.reset();
        recv.reset();
        verbs->deregister(cts_mr);
        for (Side* side : {&s, &r}) {
            side->qp.reset();
            side->cq.reset();
            verbs->deregister(side->mr);
        }
    }
    void pump(int rounds = 8) {
        for (int i = 0; i < rounds; ++i) {
            recv->progress();
            send->progress();
        }
    }
    void publish(unsigned slice, unsigned bytes) {
        const std::size_t slot = (slice * kInc) % kSlots;
        for (unsigned i = 0; i < bytes; ++i) s.data[slot * kSlotBytes + i] = static_cast<std::uint8_t>(slice * 31 + i);
        s.sizes[slot] = bytes;
        __atomic_store_n(&s.tail, (slice + 1) * kInc, __ATOMIC_RELEASE);
    }
    bool arrived(unsigned slice, unsigned bytes) {
        const std::size_t slot = (slice * kInc) % kSlots;
        if (__atomic_load_n(&r.tail, __ATOMIC_ACQUIRE) < (slice + 1) * kInc) return false;
        if (r.sizes[slot] != bytes) return false;
        for (unsigned i = 0; i < bytes; ++i)
            if (r.data[slot * kSlotBytes + i] != static_cast<std::uint8_t>(slice * 31 + i)) return false;
        return true;
    }
    void consume(unsigned slice) { __atomic_store_n(&r.head, (slice + 1) * kInc, __ATOMIC_RELEASE); }
};

void discovery_errors() {
    fake_ibv_reset();
    fake_ibv_set_device_count(0);
    t_expect_throw([] { create_ibverbs_backend(); }, "no RDMA device found", "no device");
    fake_ibv_reset();
    fake_ibv_set_port(IBV_PORT_DOWN, IBV_LINK_LAYER_INFINIBAND, 7, IBV_MTU_4096);
    t_expect_throw([] { create_ibverbs_backend(); }, "port 1 is not ACTIVE", "port down");
    fake_ibv_reset();
    setenv("B200CCL_RDMA_IFNAME", "no-such-interface0", 1);
    t_expect_throw([] { create_ibverbs_backend(); }, "no device matches interface 'no-such-interface0'", "interface");
    unsetenv("B200CCL_RDMA_IFNAME");
    setenv("NANO_NCCL_RDMA_GID_INDEX", "99", 1);
    t_expect_throw([] { create_ibverbs_backend(); }, "ibv_query_gid failed", "gid index");
    setenv("NANO_NCCL_RDMA_GID_INDEX", "3", 1);
    {
        auto verbs = create_ibverbs_backend();
        auto cq = verbs->create_cq(8);
        auto qp = verbs->create_qp(cq.get(), 4, 4);
        RdmaPeerInfo info{};
        qp->fill_local_info(&info);
        T_CHECK(info.gid_index == 3 && info.gid[15] == 0x13 && info.lid == 7);
    }
    unsetenv("NANO_NCCL_RDMA_GID_INDEX");
    T_CHECK(fake_ibv_get_counters().live_objects == 0);  // every failed or finished attempt released what it held
}

void four_slices(DataPlane plane) {
    fake_ibv_reset();
    Link l(plane);
    for (unsigned s = 0; s < 4; ++s) l.publish(s, 48 + s);
    l.pump();
    for (unsigned s = 0; s < 4; ++s) T_CHECK(l.arrived(s, 48 + s));
    T_CHECK(l.send->posts() == 4 && l.send->zero_payload_posts() == 0);
    T_CHECK(__atomic_load_n(&l.s.head, __ATOMIC_ACQUIRE) == 8 && !l.errors->has_error() && l.send->drained());
    const fake_ibv_counters c = fake_ibv_get_counters();
    if (plane == DataPlane::SendRecv) T_CHECK(c.sends == 4 && c.signaled >= 1 && c.signaled < 4 && c.rdma_writes == 0);
    if (plane == DataPlane::WriteCts) T_CHECK(c.inline_sends == 4 && c.rdma_writes == 8);  // four grants + four payloads
}

void back_pressure_and_wrap(DataPlane plane) {
    fake_ibv_reset();
    Link l(plane);
    for (unsigned s = 0; s < 4; ++s) l.publish(s, 32);
    l.pump();
    for (unsigned s = 0; s < 4; ++s) T_CHECK(l.arrived(s, 32));
    l.publish(4, 20);  // no credit: must stall (no grant, or a receiver-not-ready retry)
    l.pump(32);
    if (plane == DataPlane::WriteCts) T_CHECK(l.send->posts() == 4);
    if (plane == DataPlane::SendRecv) T_CHECK(fake_ibv_get_counters().rnr_waits > 0);
    T_CHECK(__atomic_load_n(&l.r.tail, __ATOMIC_ACQUIRE) == 8 && __atomic_load_n(&l.s.head, __ATOMIC_ACQUIRE) == 8);
    l.consume(0);
    l.pump(32);
    T_CHECK(l.send->posts() == 5 && l.arrived(4, 20));
    unsigned produced = 5, consumed = 1;
    for (; produced < 40; ++produced) {  // ten times round the ring: the send queue must keep being released
        l.consume(consumed++);
        l.publish(produced, 10 + produced % 50);
        l.pump(16);
        T_CHECK(l.arrived(produced, 10 + produced % 50));
    }
    T_CHECK(!l.errors->has_error());
}

void progress_threads(bool shared) {
    fake_ibv_reset();
    Link l(DataPlane::WriteCts);
    ProgressEngine engine(shared);
    engine.add(l.send.get());
    engine.add(l.recv.get());
    engine.start_receivers();
    engine.start_senders();
    for (unsigned s = 0; s < 12; ++s) {
        l.publish(s, 50);
        const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(5);
        while (!l.arrived(s, 50) && std::chrono::steady_clock::now() < end) std::this_thread::yield();
        T_CHECK(l.arrived(s, 50));
        l.consume(s);
    }
    engine.stop();
    T_CHECK(!l.errors->has_error());
}

void roce_needs_a_global_route() {
    fake_ibv_reset();
    fake_ibv_set_port(IBV_PORT_ACTIVE, IBV_LINK_LAYER_ETHERNET, 0, IBV_MTU_1024);
    Link* l = nullptr;
    // active_mtu 1024 = 3 is what both ends report; Link checks for 5, so build the pieces by hand here.
    auto verbs = create_ibverbs_backend();
    auto cq_a = verbs->create_cq(8), cq_b = verbs->create_cq(8);
    auto a = verbs->create_qp(cq_a.get(), 4, 4), b = verbs->create_qp(cq_b.get(), 4, 4);
    RdmaPeerInfo ia{}, ib{};
    a->fill_local_info(&ia);
    b->fill_local_info(&ib);
    T_CHECK(ia.lid == 0 && ia.active_mtu == 3);
    a->connect(ib);  // the stand-in refuses RTR on Ethernet without is_global: no exception = a GRH was set
    b->connect(ia);
    char out[16] = "RDMA_BOOT_OK", in[16] = {0};
    MemoryRegion mo = verbs->register_memory(out, sizeof(out)), mi = verbs->register_memory(in, sizeof(in));
    b->post_recv(RecvWr{77, in, sizeof(in), mi.lkey});
    SendWr w;
    w.wr_id = 5;
    w.local_addr = out;
    w.length = 13;
    w.lkey = mo.lkey;
    w.signaled = true;
    a->post_send(w);
    Completion c[2];
    T_CHECK(cq_b->poll(2, c) == 1 && c[0].wr_id == 77 && c[0].status == 0 && c[0].opcode == WcOpcode::Recv && c[0].byte_len == 13);
    T_CHECK(cq_a->poll(2, c) == 1 && c[0].wr_id == 5 && c[0].status == 0 && c[0].opcode == WcOpcode::Send);
    T_CHECK(std::strcmp(in, "RDMA_BOOT_OK") == 0);
    // RDMA WRITE WITH IMM: the immediate travels in network byte order and comes back in host order.
    b->post_recv(RecvWr{78, in, 1, mi.lkey});
    std::memcpy(out, "second", 7);
    w.wr_id = 6;
    w.opcode = WrOpcode::RdmaWriteWithImm;
    w.length = 7;
    w.remote_addr = reinterpret_cast<std::uint64_t>(in);
    w.rkey = mi.rkey;
    w.imm = 0x01020304u;
    a->post_send(w);
    T_CHECK(cq_b->poll(2, c) == 1 && c[0].wr_id == 78 && c[0].opcode == WcOpcode::RecvRdmaWithImm && c[0].imm == 0x01020304u &&
            c[0].byte_len == 7);
    T_CHECK(cq_a->poll(2, c) == 1 && c[0].opcode == WcOpcode::RdmaWrite);
    T_CHECK(std::strcmp(in, "second") == 0);
    // A write outside the registered range completes in error instead of touching memory.
    w.wr_id = 7;
    w.opcode = WrOpcode::RdmaWrite;
    w.remote_addr = reinterpret_cast<std::uint64_t>(in) + 12;
    a->post_send(w);
    T_CHECK(cq_a->poll(2, c) == 1 && c[0].wr_id == 7 && c[0].status == IBV_WC_REM_ACCESS_ERR);
    t_expect_throw([&] { a->post_send(w); }, "ibv_post_send failed", "send on a broken queue pair");
    verbs->deregister(mo);
    verbs->deregister(mi);
    (void)l;
}

void miswired_pair_fails_with_a_completion() {
    fake_ibv_reset();
    auto verbs = create_ibverbs_backend();
    auto cq_a = verbs->create_cq(8), cq_b = verbs->create_cq(8);
    auto a = verbs->create_qp(cq_a.get(), 4, 4), b = verbs->create_qp(cq_b.get(), 4, 4);
    RdmaPeerInfo ia{}, ib{};
    a->fill_local_info(&ia);
    b->fill_local_info(&ib);
    ia.psn ^= 1u;  // b will expect the wrong first packet number from a
    a->connect(ib);
    b->connect(ia);
    char buf[8] = {0};
    MemoryRegion m = verbs->register_memory(buf, sizeof(buf));
    b->post_recv(RecvWr{1, buf, 8, m.lkey});
    SendWr w;
    w.wr_id = 2;
    w.local_addr = buf;
    w.length = 4;
    w.lkey = m.lkey;
    w.signaled = true;
    a->post_send(w);
    Completion c[2];
    T_CHECK(cq_a->poll(2, c) == 1 && c[0].status == IBV_WC_RETRY_EXC_ERR);
    // Host memory registers; "device" registration falls back from dma-buf to a plain registration
    // (the stand-in accepts any address, as a peer-memory module would for device memory).
    MemoryRegion d = verbs->register_device_memory(buf, sizeof(buf));
    T_CHECK(d.rkey != 0 && d.rkey != m.rkey);
    verbs->deregister(d);
    verbs->deregister(m);
}

}  // namespace

int main() {
    discovery_errors();
    four_slices(DataPlane::SendRecv);
    four_slices(DataPlane::WriteCts);
    back_pressure_and_wrap(DataPlane::SendRecv);
    back_pressure_and_wrap(DataPlane::WriteCts);
    progress_threads(false);
    progress_threads(true);
    roce_needs_a_global_route();
    miswired_pair_fails_with_a_completion();
    T_CHECK(fake_ibv_get_counters().live_objects == 0);
    std::puts("ibverbs backend ok");
    return 0;
}
