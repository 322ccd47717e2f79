#!/usr/bin/env bash
# Builds the UNMODIFIED reference (nano-nccl) for sm_100 at 2, 4 and 8 ranks and puts its
# stock benchmark binary under baseline/_ref/bin/. The reference fixes its rank count at
# compile time, so one binary per rank count is needed. The source tree is copied to a
# scratch directory first because the build writes beside the sources.
#
# Two things the image lacks are supplied from outside the reference's code:
#   * libnuma: a header + static stub whose numa_available() returns -1, which turns the
#     reference's NUMA calls into no-ops (its own fallback path); GPU code is unaffected.
#   * libnvidia-ml at link time: the CUDA toolkit's stub; the driver's library is used at run time.
#
# Beside each benchmark binary it builds ref_e2e_n<N>, the harness of ref_e2e_driver.cu, against the
# same unmodified static library.
#
# usage: baseline/build_reference.sh <reference_source_dir> [out_dir]
set -euo pipefail
REF=${1:?usage: build_reference.sh <reference_source_dir> [out_dir]}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=${2:-$HERE/_ref}
WORK=$(mktemp -d /tmp/ref_build.XXXXXX)
trap 'rm -rf "$WORK"' EXIT

cp -r "$REF" "$WORK/src"
mkdir -p "$WORK/shim" "$OUT/bin"
cat > "$WORK/shim/numa.h" <<'EOF'
#pragma once
/* Stand-in for libnuma on an image that does not ship it: reports "NUMA unavailable". */
#ifdef __cplusplus
extern "C" {
#endif
struct bitmask { unsigned long size; unsigned long* maskp; };
int numa_available(void);
void numa_set_preferred(int node);
struct bitmask* numa_allocate_cpumask(void);
void numa_free_cpumask(struct bitmask* b);
int numa_node_to_cpus(int node, struct bitmask* mask);
unsigned int numa_bitmask_weight(const struct bitmask* b);
int numa_sched_setaffinity(int pid, struct bitmask* mask);
void* numa_alloc_onnode(unsigned long size, int node);
void numa_free(void* p, unsigned long size);
int numa_max_node(void);
#ifdef __cplusplus
}
#endif
EOF
cat > "$WORK/shim/numa.c" <<'EOF'
#include "numa.h"
#include <stdlib.h>
int numa_available(void) { return -1; }
void numa_set_preferred(int node) { (void)node; }
struct bitmask* numa_allocate_cpumask(void) { return 0; }
void numa_free_cpumask(struct bitmask* b) { (void)b; }
int numa_node_to_cpus(int node, struct bitmask* mask) { (void)node; (void)mask; return -1; }
unsigned int numa_bitmask_weight(const struct bitmask* b) { (void)b; return 0; }
int numa_sched_setaffinity(int pid, struct bitmask* mask) { (void)pid; (void)mask; return -1; }
void* numa_alloc_onnode(unsigned long size, int node) { (void)node; return malloc(size); }
void numa_free(void* p, unsigned long size) { (void)size; free(p); }
int numa_max_node(void) { return 0; }
EOF
gcc -O2 -fPIC -c "$WORK/shim/numa.c" -o "$WORK/shim/numa.o"
ar rcs "$WORK/shim/libnuma.a" "$WORK/shim/numa.o"

for n in 2 4 8; do
  cmake -S "$WORK/src" -B "$WORK/b$n" -G Ninja \
    -DCMAKE_BUILD_TYPE=Release -DBUILD_TESTING=OFF \
    -DNANO_NCCL_NRANKS=$n -DNANO_NCCL_CUDA_ARCH=100 \
    -DNUMA_LIB="$WORK/shim/libnuma.a" \
    -DNVML_LIB=/usr/local/cuda/lib64/stubs/libnvidia-ml.so \
    -DCMAKE_CUDA_FLAGS="-I$WORK/shim" -DCMAKE_CXX_FLAGS="-I$WORK/shim" \
    > "$WORK/cmake_$n.log" 2>&1 || { tail -30 "$WORK/cmake_$n.log"; exit 1; }
  ninja -C "$WORK/b$n" nano_nccl_all_reduce_bench > "$WORK/ninja_$n.log" 2>&1 \
    || { tail -40 "$WORK/ninja_$n.log"; exit 1; }
  cp "$WORK/b$n/benchmarks/nano_nccl_all_reduce_bench" "$OUT/bin/nano_nccl_all_reduce_bench_n$n"
  echo "built $OUT/bin/nano_nccl_all_reduce_bench_n$n"
  # Harness over the reference's public API for the end-to-end measurement (see ref_e2e_driver.cu).
  nvcc -O3 -std=c++17 -arch=sm_100 -I"$WORK/src/include" -I"$WORK/src/src" -I"$WORK/shim" \
    -DNANO_NCCL_NRANKS=$n -DNANO_NCCL_NCHANNELS=4 -DNANO_NCCL_BLOCK_THREADS=512 -DNANO_NCCL_FIFO_BUFF_BYTES=33554432 \
    "$HERE/ref_e2e_driver.cu" "$WORK/b$n/src/libnano_nccl.a" "$WORK/shim/libnuma.a" \
    -L/usr/local/cuda/lib64/stubs -lnvidia-ml -lpthread -o "$OUT/bin/ref_e2e_n$n" \
    > "$WORK/driver_$n.log" 2>&1 || { tail -30 "$WORK/driver_$n.log"; exit 1; }
  echo "built $OUT/bin/ref_e2e_n$n"
done
