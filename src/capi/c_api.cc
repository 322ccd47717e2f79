#include "b200ccl/c_api.h"

#include "b200ccl/bootstrap.h"
#include "b200ccl/communicator.h"
#include "kernels/sm100/selftest.h"
#include "core/check.h"
#include "sched/plan.h"
#include "sim/ll_sim.h"
#include "sim/ring_sim.h"

#include <cstring>
#include <exception>
#include <stdexcept>
#include <string>

using namespace b200ccl;

struct b2_comm {
    std::unique_ptr<Communicator> comm;
};
struct b2_bootstrap {
    std::unique_ptr<Bootstrap> bs;
};

namespace {
thread_local std::string g_error;
}  // namespace

namespace b200ccl::kernels {
// Lets entry points defined beside the kernels report through b2_last_error().
void set_last_error_message(const std::string& message) { g_error = message; }
}  // namespace b200ccl::kernels

namespace {

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::invalid_argument& e) {
        g_error = e.what();
        return 2;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    } catch (...) {
        g_error = "unknown failure";
        return 1;
    }
}

CommunicatorConfig to_config(const int* devices, int ndev, const b2_config* c) {
    CommunicatorConfig cfg;
    cfg.devices.assign(devices, devices + ndev);
    if (c) {
        cfg.transport = static_cast<TransportKind>(c->transport);
        cfg.algo = static_cast<Algo>(c->algo);
        cfg.channels = c->channels;
        cfg.staging_bytes = c->staging_bytes;
        cfg.wait_timeout_ms = c->wait_timeout_ms;
        cfg.loopback = c->loopback != 0;
        cfg.loopback_ranks = c->loopback_ranks;
        cfg.enable_nvls = c->enable_nvls != 0;
        cfg.max_ctas = c->max_ctas;
    }
    return cfg;
}
}  // namespace

extern "C" {

const char* b2_last_error(void) { return g_error.c_str(); }
const char* b2_version(void) { return "0.1.0"; }

int b2_parse_dtype(const char* t, int* out) { DType v; if (!parse_dtype(t, &v)) return 2; *out = static_cast<int>(v); return 0; }
int b2_parse_redop(const char* t, int* out) { RedOp v; if (!parse_redop(t, &v)) return 2; *out = static_cast<int>(v); return 0; }
int b2_parse_transport(const char* t, int* out) { TransportKind v; if (!parse_transport(t, &v)) return 2; *out = static_cast<int>(v); return 0; }
int b2_parse_algo(const char* t, int* out) { Algo v; if (!parse_algo(t, &v)) return 2; *out = static_cast<int>(v); return 0; }
const char* b2_dtype_name(int v) { return dtype_name(static_cast<DType>(v)); }
const char* b2_redop_name(int v) { return redop_name(static_cast<RedOp>(v)); }
const char* b2_transport_name(int v) { return transport_name(static_cast<TransportKind>(v)); }
const char* b2_algo_name(int v) { return algo_name(static_cast<Algo>(v)); }
double b2_busbw_gbs(int collective, double algbw, int nranks) {
    return busbw_gbs(static_cast<Collective>(collective), algbw, nranks);
}

void b2_config_default(b2_config* cfg) {
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->transport = static_cast<int>(TransportKind::Auto);
    cfg->algo = static_cast<int>(Algo::Auto);
    cfg->enable_nvls = 1;
}

int b2_bootstrap_create(const char* addr, int port, int rank, int size, int timeout_ms, b2_bootstrap** out) {
    return guarded([&] {
        auto bs = create_tcp_bootstrap(addr ? addr : "127.0.0.1", port, rank, size, timeout_ms > 0 ? timeout_ms : 60000);
        *out = new b2_bootstrap{std::move(bs)};
    });
}
void b2_bootstrap_destroy(b2_bootstrap* bs) { delete bs; }
int b2_bootstrap_barrier(b2_bootstrap* bs) { return guarded([&] { bs->bs->barrier(); }); }
int b2_bootstrap_allgather(b2_bootstrap* bs, const void* in, void* out, size_t bytes) {
    return guarded([&] { bs->bs->allgather(in, out, bytes); });
}

int b2_comm_create(const int* devices, int ndev, const b2_config* cfg, b2_comm** out) {
    return guarded([&] { *out = new b2_comm{create_communicator(to_config(devices, ndev, cfg))}; });
}
int b2_comm_create_bootstrap(b2_bootstrap* bs, const int* devices, int ndev, const b2_config* cfg, b2_comm** out) {
    return guarded([&] { *out = new b2_comm{create_communicator_from_bootstrap(*bs->bs, to_config(devices, ndev, cfg))}; });
}
void b2_comm_destroy(b2_comm* comm) { delete comm; }

int b2_comm_local_ranks(const b2_comm* c) { return c->comm->local_rank_count(); }
int b2_comm_global_ranks(const b2_comm* c) { return c->comm->global_rank_count(); }
int b2_comm_first_rank(const b2_comm* c) { return c->comm->first_global_rank(); }
int b2_comm_transport(const b2_comm* c) { return static_cast<int>(c->comm->transport()); }
int b2_comm_nvls(const b2_comm* c) { return c->comm->nvls_available() ? 1 : 0; }
size_t b2_comm_describe(const b2_comm* c, char* buf, size_t cap) {
    const std::string s = c->comm->describe();
    if (buf && cap) {
        const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        std::memcpy(buf, s.data(), n);
        buf[n] = '\0';
    }
    return s.size();
}
int b2_comm_check_async_error(const b2_comm* c) { return guarded([&] { c->comm->check_async_error(); }); }

int b2_collective(b2_comm* c, int collective, const void* const* send, void* const* recv, void* const* streams,
                  size_t count, int dtype, int redop, int allow_in_place) {
    return guarded([&] {
        const int n = c->comm->local_rank_count();
        CollectiveArgs a;
        a.send_buffers.assign(send, send + n);
        a.recv_buffers.assign(recv, recv + n);
        for (int i = 0; i < n; ++i) a.streams.push_back(static_cast<cudaStream_t>(streams[i]));
        a.count = count;
        a.dtype = static_cast<DType>(dtype);
        a.redop = static_cast<RedOp>(redop);
        a.allow_in_place = allow_in_place != 0;
        switch (collective) {
            case 0: c->comm->all_reduce(a); break;
            case 1: c->comm->reduce_scatter(a); break;
            case 2: c->comm->all_gather(a); break;
            default: throw std::invalid_argument("unknown collective id");
        }
    });
}

int b2_comm_last_call(const b2_comm* c, int out[7]) {
    const CallInfo i = c->comm->last_call();
    out[0] = static_cast<int>(i.algo);
    out[1] = i.grid;
    out[2] = i.block;
    out[3] = i.staged_in;
    out[4] = i.staged_out;
    out[5] = i.vectorized;
    out[6] = i.pack_bytes;
    return 0;
}

int b2_comm_ring_channel(const b2_comm* c, int local_rank, int channel, const void* out[8]) {
    return guarded([&] {
        const auto v = c->comm->ring_channel_pointers(local_rank, channel);
        for (size_t i = 0; i < 8 && i < v.size(); ++i) out[i] = v[i];
    });
}

int b2_pointer_info(const void* ptr, int out[2]) {
    return guarded([&] {
        cudaPointerAttributes attr;
        B2_CUDA(cudaPointerGetAttributes(&attr, ptr));
        out[0] = static_cast<int>(attr.type);
        out[1] = attr.device;
    });
}

int b2_comm_alloc_symmetric(b2_comm* c, size_t bytes, void** ptrs) {
    return guarded([&] {
        auto v = c->comm->alloc_symmetric(bytes);
        for (size_t i = 0; i < v.size(); ++i) ptrs[i] = v[i];
    });
}
int b2_comm_free_symmetric(b2_comm* c, void* const* ptrs) {
    return guarded([&] {
        std::vector<void*> v(ptrs, ptrs + c->comm->local_rank_count());
        c->comm->free_symmetric(v);
    });
}

int b2_comm_register(b2_comm* c, void* const* ptrs, size_t bytes) {
    return guarded([&] {
        std::vector<void*> v(ptrs, ptrs + c->comm->local_rank_count());
        c->comm->register_buffers(v, bytes);
    });
}
int b2_comm_unregister(b2_comm* c, void* const* ptrs) {
    return guarded([&] {
        std::vector<void*> v(ptrs, ptrs + c->comm->local_rank_count());
        c->comm->unregister_buffers(v);
    });
}

int b2_make_plan(int collective, int dtype, int redop, int nranks, size_t count, unsigned flags, int forced_algo,
                 int out[5]) {
    return guarded([&] {
        sched::CallShape s;
        s.collective = static_cast<Collective>(collective);
        s.dtype = static_cast<DType>(dtype);
        s.redop = static_cast<RedOp>(redop);
        s.nranks = nranks;
        s.count = count;
        s.wide = flags & 1u;
        s.peers_read_input = flags & 2u;
        s.peers_write_output = flags & 4u;
        s.input_multicast = flags & 8u;
        s.output_multicast = flags & 16u;
        s.in_place = flags & 32u;
        s.ring_only = flags & 64u;
        s.word_aligned = flags & 128u;
        s.max_ctas = 0;  // the tuning decides
        const sched::Plan p = sched::make_plan(s, static_cast<Algo>(forced_algo), sched::tuning_from_env());
        if (!p.error.empty()) throw std::invalid_argument(p.error);
        out[0] = static_cast<int>(p.algo);
        out[1] = p.grid;
        out[2] = p.stage_in;
        out[3] = p.stage_out;
        out[4] = p.gather_mode;
    });
}

int b2_ll_sim(const long long cfg[8], const size_t* call_words, int ncalls, double wait_timeout_ms, long long out[6]) {
    return guarded([&] {
        sim::LlSimConfig c;
        c.nranks = static_cast<int>(cfg[0]);
        c.ctas = static_cast<int>(cfg[1]);
        c.lanes = static_cast<int>(cfg[2]);
        c.redop = static_cast<RedOp>(cfg[3]);
        c.max_words = static_cast<std::size_t>(cfg[4]);
        c.slow_rank = static_cast<int>(cfg[5]);
        c.stall_rank = static_cast<int>(cfg[6]);
        c.stall_at_call = static_cast<int>(cfg[7]);
        c.wait_timeout_ms = wait_timeout_ms;
        c.call_words.assign(call_words, call_words + (ncalls > 0 ? ncalls : 0));
        const sim::LlSimResult r = sim::run_ll_sim(c);
        if (r.wrong < 0) throw std::invalid_argument(r.message);
        out[0] = r.wrong;
        out[1] = r.timed_out;
        out[2] = r.timeout_rank;
        out[3] = r.timeout_peer;
        out[4] = r.timeout_call;
        out[5] = r.max_lead;
    });
}

int b2_ring_sim(const long long cfg[6], size_t count, size_t fifo_bytes, double wait_timeout_ms, long long out_i[7],
                double out_d[2]) {
    return guarded([&] {
        sim::RingSimConfig c;
        c.nranks = static_cast<int>(cfg[0]);
        c.channels = static_cast<int>(cfg[1]);
        c.redop = static_cast<RedOp>(cfg[2]);
        c.collective = static_cast<Collective>(cfg[3]);
        c.stall_rank = static_cast<int>(cfg[4]);
        c.stall_after_slices = cfg[5];
        c.count = count;
        c.fifo_bytes = fifo_bytes;
        c.wait_timeout_ms = wait_timeout_ms;
        const sim::RingSimResult r = sim::run_ring_sim(c);
        if (r.wrong < 0) throw std::invalid_argument(r.message);
        out_i[0] = r.wrong;
        out_i[1] = r.timed_out;
        out_i[2] = r.timeout_rank;
        out_i[3] = r.timeout_peer;
        out_i[4] = r.timeout_channel;
        out_i[5] = static_cast<long long>(r.slices);
        out_i[6] = static_cast<long long>(r.empty_slices);
        out_d[0] = r.seconds;
        out_d[1] = r.max_abs_error;
    });
}

int b2_selftest_wait(int kind, int device, double timeout_ms, int out[4], double* waited_ms) {
    return guarded([&] {
        const kernels::SelfTestResult r = kind == 0 ? kernels::selftest_wait_timeout(device, timeout_ms)
                                                    : kernels::selftest_abort(device, timeout_ms);
        out[0] = r.wait_ok;
        out[1] = static_cast<int>(r.status_code);
        out[2] = static_cast<int>(r.where);
        out[3] = r.abort_raised ? 1 : 0;
        *waited_ms = r.waited_ms;
    });
}

int b2_selftest_direct_send(int device, int slices, int* ok) {
    return guarded([&] { *ok = kernels::selftest_direct_send(device, slices) ? 1 : 0; });
}

int b2_selftest_publication(int device, int rounds, int* ok) {
    return guarded([&] { *ok = kernels::selftest_publication(device, rounds) ? 1 : 0; });
}

}  // extern "C"
