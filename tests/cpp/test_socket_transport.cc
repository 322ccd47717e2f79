// Socket transport without a GPU or a network: framing, HELLO, and real send/receive proxies
// joined by socketpair(AF_UNIX) with plain host memory as FIFO. Failures are made on the host:
// a closed descriptor, an oversized header, an injected send failure.
// Modelled on the reference's tests/socket_protocol_test.cc:74-289.
#include "check.h"
#include "transport/socket/proxy.h"

#include <chrono>
#include <cstring>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>
#include <vector>

using namespace b200ccl::transport;
using namespace b200ccl::transport::socket;

namespace {

struct Pair {
    Fd a, b;
    Pair() {
        int sv[2];
        T_CHECK(::socketpair(AF_UNIX, SOCK_STREAM, 0, sv) == 0);
        a = Fd(sv[0]);
        b = Fd(sv[1]);
    }
};

struct HostFifo {
    static constexpr std::size_t kSlots = 8, kSlotBytes = 64, kInc = 2;
    std::vector<std::uint8_t> data = std::vector<std::uint8_t>(kSlots * kSlotBytes, 0);
    unsigned int sizes[kSlots] = {0};
    unsigned long long head = 0, tail = 0;
    ProxyFifo view() { return ProxyFifo{data.data(), kSlotBytes, kSlots, sizes, kInc}; }
};

bool wait_until(const std::function<bool()>& pred, int ms = 5000) {
    const auto end = std::chrono::steady_clock::now() + std::chrono::milliseconds(ms);
    while (std::chrono::steady_clock::now() < end) {
        if (pred()) return true;
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    return pred();
}

unsigned long long load(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
void store(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

void framing() {
    Pair p;
    const char payload[] = "abcdefg";
    send_slice(p.a.get(), payload, 7);
    unsigned char raw[11];
    recv_all(p.b.get(), raw, sizeof(raw));
    T_CHECK(raw[0] == 0 && raw[1] == 0 && raw[2] == 0 && raw[3] == 7);  // big-endian length
    T_CHECK(std::memcmp(raw + 4, payload, 7) == 0);

    // a zero-byte slice is a header only and keeps the stream in step
    send_slice(p.a.get(), nullptr, 0);
    send_slice(p.a.get(), payload, 3);
    char buf[16] = {0};
    T_CHECK(recv_slice(p.b.get(), buf, sizeof(buf)) == 0);
    T_CHECK(recv_slice(p.b.get(), buf, sizeof(buf)) == 3 && std::memcmp(buf, "abc", 3) == 0);

    // an oversized header is rejected before any payload byte is copied
    send_slice(p.a.get(), payload, 7);
    char small[4] = {'x', 'x', 'x', 'x'};
    t_expect_throw([&] { recv_slice(p.b.get(), small, sizeof(small)); }, "oversized", "oversize");
    T_CHECK(small[0] == 'x' && small[3] == 'x');

    // a closed peer is reported as such
    Pair q;
    q.a.reset();
    t_expect_throw([&] { char c; recv_all(q.b.get(), &c, 1); }, "peer closed", "eof");
}

void hello() {
    Pair p;
    send_hello(p.a.get(), 3, 5, 6);
    const WireHello h = recv_hello(p.b.get());
    T_CHECK(h.magic == kHelloMagic && h.version == 1 && h.channel == 3 && h.source_rank == 5 && h.destination_rank == 6);
    WireHello bad{};
    bad.magic = 0x12345678;
    send_all(p.a.get(), &bad, sizeof(bad));
    t_expect_throw([&] { recv_hello(p.b.get()); }, "magic", "bad magic");

    // real TCP on the loopback interface
    Listener l = Listener::create("");
    std::thread client([&] { Fd fd = connect_with_hello(l.address(), 1, 0, 1, 5000); char c = 'k'; send_all(fd.get(), &c, 1); });
    auto got = l.accept_hello(5000);
    T_CHECK(got.second.channel == 1 && got.second.source_rank == 0 && got.second.destination_rank == 1);
    char c = 0;
    recv_all(got.first.get(), &c, 1);
    T_CHECK(c == 'k');
    client.join();
    t_expect_throw([] { interface_ipv4_be("no-such-interface-0"); }, "exactly one usable IPv4", "interface");
}

void proxies_move_slices() {
    Pair p;
    HostFifo src, dst;
    auto errors = std::make_shared<AsyncErrorState>("socket");
    SendProxy sp(std::move(p.a), src.view(), SendControl{&src.head, &src.tail}, ProxyIdentity{0, 1, 0}, -1, errors);
    RecvProxy rp(std::move(p.b), dst.view(), RecvControl{&dst.head, &dst.tail}, ProxyIdentity{0, 1, 0}, -1, errors);
    rp.start();
    sp.start();
    // Six slices: more than the four the FIFO holds, so credit must flow back.
    for (unsigned s = 0; s < 6; ++s) {
        const unsigned long long step = s * HostFifo::kInc;
        T_CHECK(wait_until([&] { return load(&src.head) + HostFifo::kSlots >= step + HostFifo::kInc; }));
        const std::size_t slot = step % HostFifo::kSlots;
        const unsigned bytes = s == 3 ? 0 : 40 + s;  // one empty payload
        for (unsigned i = 0; i < bytes; ++i) src.data[slot * HostFifo::kSlotBytes + i] = static_cast<std::uint8_t>(s * 16 + i);
        src.sizes[slot] = bytes;
        store(&src.tail, step + HostFifo::kInc);
        // consumer side
        T_CHECK(wait_until([&] { return load(&dst.tail) >= step + HostFifo::kInc; }));
        T_CHECK(dst.sizes[slot] == bytes);
        for (unsigned i = 0; i < bytes; ++i) T_CHECK(dst.data[slot * HostFifo::kSlotBytes + i] == static_cast<std::uint8_t>(s * 16 + i));
        store(&dst.head, step + HostFifo::kInc);
    }
    sp.drain();
    T_CHECK(load(&src.head) == 12 && sp.slices() == 6 && rp.slices() == 6 && !errors->has_error());
    sp.stop(); rp.stop(); sp.shutdown(); rp.shutdown(); sp.join(); rp.join();
}

void closed_peer_is_reported_with_identity() {
    Pair p;
    HostFifo dst;
    unsigned int abort_word = 0;
    auto errors = std::make_shared<AsyncErrorState>("socket", &abort_word);
    RecvProxy rp(std::move(p.b), dst.view(), RecvControl{&dst.head, &dst.tail}, ProxyIdentity{7, 8, 2}, -1, errors);
    rp.start();
    p.a.reset();  // the peer goes away
    T_CHECK(wait_until([&] { return errors->has_error(); }));
    const std::string msg = errors->message();
    T_CHECK(msg.find("socket proxy source=7 destination=8 channel=2 step=0") != std::string::npos);
    T_CHECK(msg.find("peer closed") != std::string::npos);
    T_CHECK(__atomic_load_n(&abort_word, __ATOMIC_ACQUIRE) == 1u);
    // only the first failure is kept
    errors->record_failure(ProxyIdentity{1, 2, 3}, 9, "later");
    T_CHECK(errors->message() == msg);
    rp.join();
}

void protocol_error_stops_the_other_side() {
    Pair p;
    HostFifo src, dst;
    auto recv_errors = std::make_shared<AsyncErrorState>("socket");
    auto send_errors = std::make_shared<AsyncErrorState>("socket");
    // The receiver's slots are smaller than what the sender will announce.
    ProxyFifo small = dst.view();
    small.slot_bytes = 8;
    SendProxy sp(std::move(p.a), src.view(), SendControl{&src.head, &src.tail}, ProxyIdentity{0, 1, 0}, -1, send_errors);
    RecvProxy rp(std::move(p.b), small, RecvControl{&dst.head, &dst.tail}, ProxyIdentity{0, 1, 0}, -1, recv_errors);
    rp.start();
    sp.start();
    src.sizes[0] = 100;
    store(&src.tail, 2);
    T_CHECK(wait_until([&] { return recv_errors->has_error(); }));
    T_CHECK(recv_errors->message().find("oversized") != std::string::npos);
    // the sender notices on its next slice because the receiver shut the connection down
    for (unsigned s = 1; s < 4 && !send_errors->has_error(); ++s) {
        src.sizes[(s * 2) % 8] = 100;
        store(&src.tail, (s + 1) * 2);
        wait_until([&] { return send_errors->has_error() || load(&src.head) >= (s + 1) * 2; }, 1000);
    }
    T_CHECK(send_errors->has_error());
    sp.join(); rp.join();
}

void injected_send_failure() {
    Pair p;
    HostFifo src, dst;
    unsigned int abort_word = 0;
    auto errors = std::make_shared<AsyncErrorState>("socket", &abort_word);
    SendProxy sp(std::move(p.a), src.view(), SendControl{&src.head, &src.tail}, ProxyIdentity{2, 3, 1}, -1, errors);
    sp.fail_after_slices_for_testing(2);
    sp.start();
    for (unsigned s = 0; s < 3; ++s) {
        src.sizes[(s * 2) % 8] = 16;
        store(&src.tail, (s + 1) * 2);
    }
    T_CHECK(wait_until([&] { return errors->has_error(); }));
    T_CHECK(errors->message().find("socket") != std::string::npos && errors->message().find("step=4") != std::string::npos);
    T_CHECK(load(&src.head) == 4 && abort_word == 1u);
    sp.join();
}

}  // namespace

int main() {
    framing();
    hello();
    proxies_move_slices();
    closed_peer_is_reported_with_identity();
    protocol_error_stops_the_other_side();
    injected_send_failure();
    std::puts("socket transport ok");
    return 0;
}
