/* C interface of the library, for callers that cannot use the C++ classes (Python through
 * ctypes, other runtimes). Every function returns 0 on success and a non-zero code on failure;
 * b2_last_error() then holds the message of the calling thread's last failure.
 *
 * nano-nccl has no C or Python surface (its product is C++ only); this layer is what the
 * PyTorch package of this project is built on. */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2_comm b2_comm;            /* a Communicator */
typedef struct b2_bootstrap b2_bootstrap;  /* a TCP rendezvous */

const char* b2_last_error(void);
const char* b2_version(void);

/* enums mirror b200ccl::DType / RedOp / TransportKind / Algo / Collective */
int b2_parse_dtype(const char* text, int* out);
int b2_parse_redop(const char* text, int* out);
int b2_parse_transport(const char* text, int* out);
int b2_parse_algo(const char* text, int* out);
const char* b2_dtype_name(int v);
const char* b2_redop_name(int v);
const char* b2_transport_name(int v);
const char* b2_algo_name(int v);
double b2_busbw_gbs(int collective, double algbw, int nranks);

typedef struct b2_config {
    int transport;          /* TransportKind */
    int algo;               /* Algo */
    int channels;           /* 0 = default */
    size_t staging_bytes;   /* 0 = default */
    double wait_timeout_ms; /* 0 = default */
    int loopback;           /* 1 = emulate loopback_ranks ranks on devices[0] */
    int loopback_ranks;
    int enable_nvls;
    int max_ctas;           /* 0 = default; CTAs one collective may occupy per GPU */
} b2_config;
void b2_config_default(b2_config* cfg);

int b2_bootstrap_create(const char* addr, int port, int rank, int size, int timeout_ms, b2_bootstrap** out);
void b2_bootstrap_destroy(b2_bootstrap* bs);
int b2_bootstrap_barrier(b2_bootstrap* bs);
int b2_bootstrap_allgather(b2_bootstrap* bs, const void* in, void* out, size_t bytes);

/* Single process owning `ndev` GPUs. */
int b2_comm_create(const int* devices, int ndev, const b2_config* cfg, b2_comm** out);
/* One process of a group; the bootstrap must outlive the communicator. */
int b2_comm_create_bootstrap(b2_bootstrap* bs, const int* devices, int ndev, const b2_config* cfg, b2_comm** out);
void b2_comm_destroy(b2_comm* comm);

int b2_comm_local_ranks(const b2_comm* comm);
int b2_comm_global_ranks(const b2_comm* comm);
int b2_comm_first_rank(const b2_comm* comm);
int b2_comm_transport(const b2_comm* comm);
int b2_comm_nvls(const b2_comm* comm);
/* Copies at most cap-1 bytes of the description; returns the full length. */
size_t b2_comm_describe(const b2_comm* comm, char* buf, size_t cap);
int b2_comm_check_async_error(const b2_comm* comm);

/* collective: 0 all_reduce, 1 reduce_scatter, 2 all_gather. Arrays have one entry per local
 * rank; streams are cudaStream_t values. */
int b2_collective(b2_comm* comm, int collective, const void* const* send, void* const* recv,
                  void* const* streams, size_t count, int dtype, int redop, int allow_in_place);
/* What the last call resolved to: algo, grid, block, staged_in, staged_out, vectorized, pack_bytes. */
int b2_comm_last_call(const b2_comm* comm, int out[7]);
/* Ring wiring of one local rank's channel: send_fifo, recv_fifo, send_tail, send_head, recv_tail,
 * recv_head, send_base, recv_base. Fails until a ring collective has run. */
int b2_comm_ring_channel(const b2_comm* comm, int local_rank, int channel, const void* out[8]);
/* Where an address lives, from cudaPointerGetAttributes: out[0] = 0 unknown, 1 host (pinned or
 * mapped), 2 device, 3 managed; out[1] = the device that owns it (for host memory: the device whose
 * context registered it). */
int b2_pointer_info(const void* ptr, int out[2]);

/* Symmetric heap: `ptrs` receives one pointer per local rank. Collective over all processes. */
int b2_comm_alloc_symmetric(b2_comm* comm, size_t bytes, void** ptrs);
int b2_comm_free_symmetric(b2_comm* comm, void* const* ptrs);
/* Registration of ordinary device buffers (one pointer per local rank, `bytes` each). Collective. */
int b2_comm_register(b2_comm* comm, void* const* ptrs, size_t bytes);
int b2_comm_unregister(b2_comm* comm, void* const* ptrs);

/* Planner (pure function, no GPU needed): out = {algo, grid, stage_in, stage_out, gather_mode}.
 * flags bits: 1 wide, 2 peers_read_input, 4 peers_write_output, 8 input_multicast,
 * 16 output_multicast, 32 in_place, 64 ring_only, 128 word_aligned. The tuning is the default one
 * with the B200CCL_* overrides of the environment. Returns 2 with a message when impossible. */
int b2_make_plan(int collective, int dtype, int redop, int nranks, size_t count, unsigned flags, int forced_algo,
                 int out[5]);

/* CPU ring simulator (no GPU needed). cfg: {nranks, channels, redop, collective, stall_rank,
 * stall_after_slices}; out_i: {wrong, timed_out, timeout_rank, timeout_peer, timeout_channel,
 * slices, empty_slices}; out_d: {seconds, max_abs_error}. */
int b2_ring_sim(const long long cfg[6], size_t count, size_t fifo_bytes, double wait_timeout_ms, long long out_i[7],
                double out_d[2]);

/* CPU simulator of the low-latency AllReduce protocol (no GPU needed). cfg: {nranks, ctas, lanes, redop,
 * max_words, slow_rank, stall_rank, stall_at_call}; call_words[ncalls]: words per call;
 * out: {wrong, timed_out, timeout_rank, timeout_peer, timeout_call, max_lead}. */
int b2_ll_sim(const long long cfg[8], const size_t* call_words, int ncalls, double wait_timeout_ms, long long out[6]);

/* Single-GPU self-tests of the signalling primitives (bounded; they cannot hang the device).
 * kind 0: a wait on a flag nothing sets must time out; kind 1: the host raises the abort word
 * while a kernel waits. out = {wait_ok, status_code, where, abort_raised}; *waited_ms as measured
 * on the device. */
int b2_selftest_wait(int kind, int device, double timeout_ms, int out[4], double* waited_ms);
/* A kernel writes a payload then releases a counter in mapped host memory; the host acquires the
 * counter and must see the payload. *ok = 1 when every round held. */
int b2_selftest_publication(int device, int rounds, int* ok);
/* A kernel publishes `slices` ring slices (payload, byte count, tail) into a mapped host FIFO with no
 * proxy thread; the host consumes them and returns credits. *ok = 1 when every slot was consistent. */
int b2_selftest_direct_send(int device, int slices, int* ok);

#ifdef __cplusplus
}
#endif
