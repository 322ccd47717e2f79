/* b2_local_all_reduce_no_alloc — an all-reduce over buffers that all live on ONE GPU, for callers
 * that must not allocate.
 *
 * This entry point has no counterpart in the reference library (nano-nccl); it is an addition of
 * this project.
 *
 * Who needs it. Some programs that embed this library are not free to call cudaMalloc (or any
 * routine that allocates on their behalf) at the moment they want to reduce something:
 *   - a server that handed every byte of device memory to its own pool at start-up, so that a
 *     later cudaMalloc either fails or takes memory the pool was sized to own;
 *   - a latency-sensitive loop, where cudaMalloc/cudaFree would stall the device behind an
 *     implicit synchronisation at an unpredictable point;
 *   - code that runs under a "no allocation after initialisation" rule (real-time or safety
 *     reviews often impose one).
 * The communicator's own entry points are of no use to them: creating a communicator allocates
 * control blocks, staging memory and events. This function does the same reduction as a
 * communicator in single-GPU emulation mode does, with the same kernel, but the only scratch memory
 * it touches is a fixed array that is part of the library image.
 *
 * What it computes. `nranks` input buffers and `nranks` output buffers of `count` elements, all on
 * the current device. Every output receives the element-wise reduction (sum, avg, max, min; fp32
 * accumulation for fp16/bf16; NaN-propagating max/min) of all inputs. Inputs and outputs must not
 * overlap: any two byte ranges that share a byte (an input with an output, or two outputs) are
 * rejected, as is a count whose byte size overflows size_t. Work is enqueued on `stream`; the call
 * returns without waiting for it.
 *
 * Scratch. One control block per emulated rank (barrier flags, per-CTA epochs, abort word) in a
 * file-scope `static __device__` array of B2_NO_ALLOC_MAX_RANKS blocks, about 13 KiB each, roughly
 * 104 KiB in total. Every GPU on which the library is loaded holds that array until the process
 * exits, whether or not this function is ever called.
 *
 * Limits and errors. nranks must be between 1 and B2_NO_ALLOC_MAX_RANKS (8); larger values are
 * rejected with a message (see b2_last_error) and nothing is launched. count must be positive.
 * Return value: 0 on success, 2 for a rejected argument, 1 for a CUDA failure.
 *
 * Set-up. The first call on a device resolves the array's device address (with that device
 * current) and remembers it; do that first call before starting any stream capture on that device.
 * Later calls on the same device do no set-up.
 *
 * Sharing. All calls on one device use the same array, and the array keeps what the previous call
 * left in it. Each call therefore begins by clearing the array on `stream`. Two calls whose work
 * overlaps on the GPU (different streams without an ordering between them, or two host threads)
 * would race on the array: order them.
 *
 * Failure of a wait. The emulated ranks meet in barriers inside one cooperative launch, which the
 * driver only accepts when all of its blocks can be resident, so the bounded waits are not
 * expected to run out. If one does (after `B2_NO_ALLOC_WAIT_MS`), the kernel ends early and, when
 * `status_record` is not null, writes a 32-byte record there whose first 32-bit word is non-zero
 * (1 = timed out, 2 = aborted). `status_record` is caller-owned memory that the device can write
 * (device memory or mapped host memory), cleared by the caller beforehand; pass null to skip it.
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_NO_ALLOC_MAX_RANKS 8
#define B2_NO_ALLOC_WAIT_MS 2000

/* dtype: 0 float, 1 fp16, 2 bf16. redop: 0 sum, 1 avg, 2 max, 3 min. stream: a cudaStream_t. */
int b2_local_all_reduce_no_alloc(const void* const* inputs, void* const* outputs, int nranks, size_t count, int dtype,
                                 int redop, void* stream, void* status_record);

#ifdef __cplusplus
}
#endif
