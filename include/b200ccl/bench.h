// In-process benchmark of the collectives: per size it fills seeded inputs on the devices,
// warms up, times a batch with CUDA events on every rank's stream (maximum over ranks), verifies
// every element against a recomputed fp32 reference and reports algbw/busbw/#wrong.
//
// Parity: nano-nccl include/nano_nccl/all_reduce.h:10-11 (run_all_reduce_bench) and
// src/collective/all_reduce/ring_simple.cu:110-291. Differences: timing is on the device, not
// the host clock; #wrong counts elements, not ranks; ReduceScatter and AllGather are covered.
#pragma once

#include "b200ccl/communicator.h"

#include <vector>

namespace b200ccl {

class Bootstrap;

// Returns 0 on success (results appended), non-zero when the run could not be made.
int run_collective_bench(const BenchConfig& config, std::vector<BenchResult>* results);
// One process per GPU, joined by `bootstrap`: constant inputs of value global_rank + 1, a barrier
// before the timed batch, the slowest rank's device time, every rank's wrong elements, and one
// return value agreed between all processes (the MPI variant of the reference's benchmark,
// benchmarks/all_reduce_bench.cu:84-316). Every process appends the same rows to `results`.
int run_distributed_bench(Bootstrap& bootstrap, int device, const BenchConfig& config, std::vector<BenchResult>* results);
// Same name as the reference's entry point; AllReduce only.
int run_all_reduce_bench(const BenchConfig& config, std::vector<BenchResult>* results);

// Device-side helpers used by the bench and by tests (launched on `stream` of the current device).
// fill: element i of `buf` = round_to_dtype(datagen::value(uniform, seed, rank, first_index + i)).
void bench_fill(void* buf, std::size_t count, DType dtype, bool uniform, std::uint64_t seed, int rank,
                std::uint64_t first_index, cudaStream_t stream);
// verify: recomputes, for elements [0,count) of `out`, the reduction over `nranks` ranks of the
// generated inputs at index first_index+i (collective-specific index maps are handled by the
// caller through first_index), and adds the number of elements off by more than eps to *wrong
// and the largest absolute error (as float bits) to *max_abs_bits. AllGather: pass
// src_rank >= 0 to compare against that single rank's data instead of a reduction.
void bench_verify(const void* out, std::size_t count, DType dtype, RedOp redop, bool uniform, std::uint64_t seed,
                  int nranks, int src_rank, std::uint64_t first_index, float eps, unsigned long long* wrong,
                  unsigned int* max_abs_bits, cudaStream_t stream);

}  // namespace b200ccl
