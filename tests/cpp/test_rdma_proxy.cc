// RDMA proxies against the in-process verbs backend (no HCA, no GPU): wire structure layout,
// MTU negotiation, environment parsing, and both data planes — four slices, zero-byte elision,
// multi-flight with selective signalling, clear-to-send back-pressure, ring wrap, error
// completions, shared and dedicated progress. Failures are injected on the host (an error
// completion from the fake backend).
// Modelled on the reference's tests/rdma_protocol.cc and tests/rdma_proxy_test.cc:454-726.
#include "check.h"
#include "transport/rdma/fake_verbs.h"
#include "transport/rdma/gdr.h"
#include "transport/rdma/progress.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

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
    std::shared_ptr<FakeVerbs> verbs = std::make_shared<FakeVerbs>();
    Side s, r;
    std::vector<RdmaCtsSlot> cts = std::vector<RdmaCtsSlot>(kSlots / kInc);
    MemoryRegion cts_mr;
    std::shared_ptr<AsyncErrorState> errors = std::make_shared<AsyncErrorState>("rdma");
    std::unique_ptr<RdmaSendProxy> send;
    std::unique_ptr<RdmaRecvProxy> recv;

    explicit Link(DataPlane plane, bool elide = false, bool prepare_now = true) {
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
        s.qp->connect(ri);
        r.qp->connect(si);
        send.reset(new RdmaSendProxy(s.qp.get(), s.cq.get(), s.fifo(), &s.head, &s.tail, ProxyIdentity{4, 5, 1}, plane,
                                     CtsLocalRing{cts.data(), cts.size()}, errors));
        recv.reset(new RdmaRecvProxy(r.qp.get(), r.cq.get(), r.fifo(), &r.head, &r.tail, ProxyIdentity{4, 5, 1}, plane,
                                     CtsRemoteRing{reinterpret_cast<std::uint64_t>(cts.data()), cts_mr.rkey, cts.size()}, errors, elide));
        if (prepare_now) recv->prepare();
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

void structures_and_env() {
    T_CHECK(sizeof(RdmaPeerInfo) == 64 && sizeof(RdmaCtsSlot) == 32);
    T_CHECK(wr_id_for_step(42) == 42 && step_of_wr_id(42) == 42);
    T_CHECK(negotiate_path_mtu(5, 3) == 3 && negotiate_path_mtu(2, 4) == 2);
    t_expect_throw([] { negotiate_path_mtu(0, 3); }, "out of range", "mtu low");
    t_expect_throw([] { negotiate_path_mtu(3, 9); }, "out of range", "mtu high");
    T_CHECK(AsyncErrorState::format("rdma", ProxyIdentity{1, 2, 3}, 8, "boom") == "rdma proxy source=1 destination=2 channel=3 step=8: boom");
    unsetenv("B200CCL_RDMA_USE_WRITE"); unsetenv("NANO_NCCL_RDMA_USE_WRITE");
    T_CHECK(data_plane_from_env() == DataPlane::SendRecv);
    setenv("NANO_NCCL_RDMA_USE_WRITE", "on", 1);
    T_CHECK(data_plane_from_env() == DataPlane::WriteCts);
    setenv("B200CCL_RDMA_USE_WRITE", "maybe", 1);
    t_expect_throw([] { data_plane_from_env(); }, "0/1/true/false/on/off", "strict boolean");
    unsetenv("B200CCL_RDMA_USE_WRITE"); unsetenv("NANO_NCCL_RDMA_USE_WRITE");
    setenv("B200CCL_RDMA_GDR", "1", 1);
    T_CHECK(fifo_placement_from_env() == FifoPlacement::Gdr);
    unsetenv("B200CCL_RDMA_GDR");
    T_CHECK(fifo_placement_from_env() == FifoPlacement::HostPinned && !shared_progress_from_env());
    T_CHECK(create_backend("fake")->name() == "fake");
    t_expect_throw([] { create_backend("quantum"); }, "unknown backend", "backend name");
}

void four_slices(DataPlane plane) {
    Link l(plane);
    for (unsigned s = 0; s < 4; ++s) l.publish(s, 48 + s);
    l.pump();
    for (unsigned s = 0; s < 4; ++s) T_CHECK(l.arrived(s, 48 + s));
    T_CHECK(l.send->posts() == 4 && l.send->zero_payload_posts() == 0);
    T_CHECK(__atomic_load_n(&l.s.head, __ATOMIC_ACQUIRE) == 8 && !l.errors->has_error() && l.send->drained());
    // Multi-flight with selective signalling: four sends in one burst need fewer than four signals.
    if (plane == DataPlane::SendRecv) T_CHECK(l.verbs->signaled_sends() >= 1 && l.verbs->signaled_sends() < 4);
    if (plane == DataPlane::WriteCts) T_CHECK(l.verbs->inline_sends() == 4);  // the four grants went inline
}

void zero_byte_elision() {
    Link l(DataPlane::SendRecv, /*elide=*/true, /*prepare_now=*/false);
    const unsigned sizes[4] = {40, 0, 24, 0};
    for (unsigned s = 0; s < 4; ++s) l.r.sizes[(s * kInc) % kSlots] = sizes[s];  // what the receiver expects
    l.recv->prepare();
    for (unsigned s = 0; s < 4; ++s) {
        l.publish(s, sizes[s]);
        l.pump();
    }
    T_CHECK(l.send->posts() == 2 && l.send->zero_payload_posts() == 2);
    T_CHECK(l.recv->zero_payload_posts() == 2);
    T_CHECK(__atomic_load_n(&l.s.head, __ATOMIC_ACQUIRE) == 8 && __atomic_load_n(&l.r.tail, __ATOMIC_ACQUIRE) == 8);
    T_CHECK(l.arrived(0, 40) && l.arrived(2, 24) && l.verbs->sends_posted() == 2);
}

void back_pressure_and_wrap(DataPlane plane) {
    Link l(plane);
    // Generation 1 fills all four slices of the FIFO; the receiver's kernel consumes nothing yet.
    for (unsigned s = 0; s < 4; ++s) l.publish(s, 32);
    l.pump();
    for (unsigned s = 0; s < 4; ++s) T_CHECK(l.arrived(s, 32));
    // Generation 2 is published by the sending kernel but must stall: no credit, no grant.
    l.publish(4, 20);
    l.pump(32);
    // WRITE plane: without a grant nothing is posted. SEND plane: the send is posted but the
    // connection holds it back (receiver-not-ready retry) because no receive is posted.
    if (plane == DataPlane::WriteCts) T_CHECK(l.send->posts() == 4);
    T_CHECK(__atomic_load_n(&l.r.tail, __ATOMIC_ACQUIRE) == 8);
    T_CHECK(__atomic_load_n(&l.s.head, __ATOMIC_ACQUIRE) == 8);
    // One slice is consumed → exactly one more may flow, into the reused slot (ring wrap).
    l.consume(0);
    l.pump(32);
    T_CHECK(l.send->posts() == 5 && l.arrived(4, 20));
    // Walk the ring three more times to exercise grant reuse with changing step tags.
    unsigned produced = 5, consumed = 1;
    for (; produced < 17; ++produced) {
        l.consume(consumed++);
        l.publish(produced, 10 + produced);
        l.pump(16);
        T_CHECK(l.arrived(produced, 10 + produced));
    }
    T_CHECK(!l.errors->has_error());
    if (plane == DataPlane::WriteCts)
        for (const auto& g : l.cts) T_CHECK(g.ready == 0 || g.step_tag >= 17 * kInc - kSlots);
}

void error_completion_is_latched() {
    Link l(DataPlane::SendRecv);
    l.verbs->fail_send_number(2, 12);  // the second send completes with an error status
    for (unsigned s = 0; s < 3; ++s) l.publish(s, 16);
    l.pump(16);
    T_CHECK(l.errors->has_error());
    const std::string msg = l.errors->message();
    T_CHECK(msg.find("rdma proxy source=4 destination=5 channel=1") != std::string::npos);
    T_CHECK(msg.find("status 12") != std::string::npos);
    T_CHECK(!l.send->progress() && !l.recv->progress());  // a failed edge does no further work
}

void oversized_payload_is_rejected() {
    Link l(DataPlane::SendRecv);
    l.s.sizes[0] = kInc * kSlotBytes + 1;
    __atomic_store_n(&l.s.tail, kInc, __ATOMIC_RELEASE);
    l.pump(2);
    T_CHECK(l.errors->has_error() && l.errors->message().find("exceeds") != std::string::npos);
    T_CHECK(l.verbs->sends_posted() == 0);
}

void progress_engine(bool shared) {
    Link l(DataPlane::WriteCts);
    ProgressEngine engine(shared);
    engine.add(l.send.get());
    engine.add(l.recv.get());
    engine.start_receivers();
    engine.start_senders();
    T_CHECK(engine.thread_count() == (shared ? 1u : 2u));
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

void registered_fifo() {
    auto verbs = std::make_shared<FakeVerbs>();
    verbs->allow_device_registration = false;
    // A GDR request that cannot be met must fail rather than fall back to host memory. Building
    // the device buffer itself needs a GPU, so only the host placement is constructed here.
    t_expect_throw([&] { verbs->register_device_memory(reinterpret_cast<void*>(0x1000), 4096); }, "unavailable", "gdr");
    const std::uint64_t before = verbs->registrations();
    int devices = 0;
    if (cudaGetDeviceCount(&devices) != cudaSuccess) devices = 0;
    if (devices > 0) {  // pinned host memory comes from the CUDA runtime
        RegisteredFifo fifo(verbs, FifoPlacement::HostPinned, 4096, -1);
        T_CHECK(fifo.data() != nullptr && fifo.region().length == 4096 && verbs->registrations() == before + 1);
    }
}

}  // namespace

int main() {
    structures_and_env();
    four_slices(DataPlane::SendRecv);
    four_slices(DataPlane::WriteCts);
    zero_byte_elision();
    back_pressure_and_wrap(DataPlane::SendRecv);
    back_pressure_and_wrap(DataPlane::WriteCts);
    error_completion_is_latched();
    oversized_payload_is_rejected();
    progress_engine(false);
    progress_engine(true);
    registered_fifo();
    std::puts("rdma proxy ok");
    return 0;
}
