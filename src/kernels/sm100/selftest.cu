// Small self-tests of the signalling primitives, callable on any single GPU. None of them can
// hang or fault the device: every wait is bounded and ends with a status record.
//   * wait timeout: a warp waits for a flag that nothing sets; the wait must run out and say so.
//   * abort: the host raises the abort word while a warp waits; the wait must end as "aborted".
//   * publication: a kernel writes a payload and then releases a step counter in mapped host
//     memory; a host thread that acquires the counter must already see the payload.
//   * direct send: a kernel does what the ring kernel's sending side does on a network edge (payload
//     into a slot of a mapped host FIFO, the slot's byte count, then the tail counter) with NO proxy
//     thread running; the host, playing the proxy, must find tail, byte count and payload consistent
//     for every slot as the steps wrap around the FIFO.
// Modelled on the reference's tests/simple_protocol.cu:110-173 (publication),
// tests/public_api.cu:433-513 (abort unblocks the waits) and :515-585 (device direct_send without a proxy).
#include "kernels/sm100/selftest.h"

#include "core/check.h"
#include "kernels/sm100/sync.cuh"

#include <chrono>
#include <cstring>
#include <thread>

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

__global__ void wait_kernel(const unsigned long long* flag, unsigned long long want, ControlBlock* own, Status* status,
                            unsigned long long timeout_ns, unsigned int* started, int* ok_out) {
    if (threadIdx.x == 0) {
        if (started) {
            *started = 1u;
            __threadfence_system();
        }
        ControlBlock* ctrl[1] = {own};
        const bool ok = wait_at_least(flag, want, own, timeout_ns, status, ctrl, 1, 0u, 99u);
        *ok_out = ok ? 1 : 0;
    }
}

__global__ void publish_kernel(unsigned int* payload, int n, unsigned long long* step, unsigned long long value) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) payload[i] = 0xC0DE0000u + i;
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(step, value);
}

// The publish half of a ring slice on a network edge, in the order the ring kernel uses: payload
// stores by all threads, block barrier, then ONE thread writes the slot's byte count and releases
// the tail (src/kernels/sm100/ring_simple.cu, "Publish").
__global__ void direct_send_kernel(unsigned int* fifo, unsigned int slot_words, unsigned int* slot_sizes, int slots, int steps_per_slice,
                                   unsigned long long first_step, int slices, unsigned long long* tail,
                                   const unsigned long long* head, ControlBlock* own, Status* status, unsigned long long timeout_ns) {
    __shared__ int s_ok;
    unsigned long long step = first_step;
    for (int k = 0; k < slices; ++k) {
        // credit: the slot may be written once the consumer (here: the host) has freed it
        if (threadIdx.x == 0) {
            const unsigned long long fifo_steps = (unsigned long long)slots * steps_per_slice;
            const unsigned long long want = step + steps_per_slice >= fifo_steps ? step + steps_per_slice - fifo_steps : 0ull;
            s_ok = wait_at_least(head, want, own, timeout_ns, status, nullptr, 0, 0u, 98u) ? 1 : 0;
        }
        __syncthreads();
        if (!s_ok) return;
        const unsigned int slot = (unsigned int)((step / steps_per_slice) % slots);
        const unsigned int words = slot_words - (unsigned int)(k % 3);  // payload sizes vary from slice to slice
        for (unsigned int i = threadIdx.x; i < words; i += blockDim.x) fifo[slot * slot_words + i] = (unsigned int)(step * 7919u) + i;
        __syncthreads();
        if (threadIdx.x == 0) {
            slot_sizes[slot] = words * 4u;
            st_release_sys(tail, step + steps_per_slice);
        }
        step += steps_per_slice;
    }
}

struct Scratch {
    ControlBlock* ctrl = nullptr;
    Status* status = nullptr;       // mapped host
    unsigned long long* flag = nullptr;
    unsigned int* started = nullptr;  // mapped host
    int* ok = nullptr;                // mapped host
    cudaStream_t stream = nullptr;
    Scratch() {
        B2_CUDA(cudaMalloc(&ctrl, sizeof(ControlBlock)));
        B2_CUDA(cudaMemset(ctrl, 0, sizeof(ControlBlock)));
        B2_CUDA(cudaMalloc(&flag, sizeof(unsigned long long)));
        B2_CUDA(cudaMemset(flag, 0, sizeof(unsigned long long)));
        B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&status), sizeof(Status), cudaHostAllocMapped));
        B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&started), sizeof(unsigned int), cudaHostAllocMapped));
        B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&ok), sizeof(int), cudaHostAllocMapped));
        std::memset(status, 0, sizeof(Status));
        *started = 0;
        *ok = -1;
        B2_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    }
    ~Scratch() {
        cudaStreamDestroy(stream);
        cudaFree(ctrl);
        cudaFree(flag);
        cudaFreeHost(status);
        cudaFreeHost(started);
        cudaFreeHost(ok);
    }
};

}  // namespace

SelfTestResult selftest_wait_timeout(int device, double timeout_ms) {
    DeviceGuard guard(device);
    Scratch s;
    wait_kernel<<<1, 32, 0, s.stream>>>(s.flag, 1ull, s.ctrl, s.status, static_cast<unsigned long long>(timeout_ms * 1e6),
                                        nullptr, s.ok);
    B2_CUDA(cudaGetLastError());
    B2_CUDA(cudaStreamSynchronize(s.stream));
    SelfTestResult r;
    r.wait_ok = *s.ok;
    r.status_code = s.status->code;
    r.waited_ms = static_cast<double>(s.status->waited_ns) * 1e-6;
    r.where = s.status->where;
    unsigned int abort_seen = 0;
    B2_CUDA(cudaMemcpy(&abort_seen, &s.ctrl->abort_flag, sizeof(abort_seen), cudaMemcpyDeviceToHost));
    r.abort_raised = abort_seen != 0;
    return r;
}

SelfTestResult selftest_abort(int device, double timeout_ms) {
    DeviceGuard guard(device);
    Scratch s;
    wait_kernel<<<1, 32, 0, s.stream>>>(s.flag, 1ull, s.ctrl, s.status, static_cast<unsigned long long>(timeout_ms * 1e6),
                                        s.started, s.ok);
    B2_CUDA(cudaGetLastError());
    // Raise the abort word once the kernel says it is waiting (or after a grace period: the
    // kernel's own time limit ends the wait in any case).
    const auto t0 = std::chrono::steady_clock::now();
    while (__atomic_load_n(s.started, __ATOMIC_ACQUIRE) == 0u &&
           std::chrono::steady_clock::now() - t0 < std::chrono::milliseconds(static_cast<long>(timeout_ms / 2)))
        std::this_thread::yield();
    cudaStream_t side;
    B2_CUDA(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
    const unsigned int one = 1;
    B2_CUDA(cudaMemcpyAsync(&s.ctrl->abort_flag, &one, sizeof(one), cudaMemcpyHostToDevice, side));
    B2_CUDA(cudaStreamSynchronize(side));
    B2_CUDA(cudaStreamSynchronize(s.stream));
    cudaStreamDestroy(side);
    SelfTestResult r;
    r.wait_ok = *s.ok;
    r.status_code = s.status->code;
    r.waited_ms = static_cast<double>(s.status->waited_ns) * 1e-6;
    r.where = s.status->where;
    r.abort_raised = true;
    return r;
}

bool selftest_publication(int device, int rounds) {
    DeviceGuard guard(device);
    constexpr int kWords = 1024;
    unsigned int* payload = nullptr;
    unsigned long long* step = nullptr;
    B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&payload), kWords * sizeof(unsigned int), cudaHostAllocMapped));
    B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&step), sizeof(unsigned long long), cudaHostAllocMapped));
    *step = 0;  // cudaHostAlloc does not clear memory
    cudaStream_t stream;
    B2_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    bool good = true;
    for (int round = 1; round <= rounds && good; ++round) {
        std::memset(payload, 0, kWords * sizeof(unsigned int));
        publish_kernel<<<1, 256, 0, stream>>>(payload, kWords, step, static_cast<unsigned long long>(round));
        B2_CUDA(cudaGetLastError());
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(5);
        while (__atomic_load_n(step, __ATOMIC_ACQUIRE) < static_cast<unsigned long long>(round)) {
            if (std::chrono::steady_clock::now() > deadline) { good = false; break; }
        }
        // The counter is visible: so must be every payload word written before it.
        for (int i = 0; good && i < kWords; ++i) good = payload[i] == 0xC0DE0000u + i;
        B2_CUDA(cudaStreamSynchronize(stream));
    }
    cudaStreamDestroy(stream);
    cudaFreeHost(payload);
    cudaFreeHost(step);
    return good;
}

bool selftest_direct_send(int device, int slices) {
    DeviceGuard guard(device);
    constexpr int kSlots = 4, kStepsPerSlice = 2;
    constexpr unsigned int kSlotWords = 512;
    Scratch s;
    unsigned int *fifo = nullptr, *sizes = nullptr;
    unsigned long long* counters = nullptr;  // [0] tail (device publishes), [1] head (host frees)
    B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&fifo), kSlots * kSlotWords * sizeof(unsigned int), cudaHostAllocMapped));
    B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&sizes), kSlots * sizeof(unsigned int), cudaHostAllocMapped));
    B2_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&counters), 2 * sizeof(unsigned long long), cudaHostAllocMapped));
    std::memset(fifo, 0, kSlots * kSlotWords * sizeof(unsigned int));
    std::memset(sizes, 0, kSlots * sizeof(unsigned int));
    counters[0] = counters[1] = 0;
    direct_send_kernel<<<1, 128, 0, s.stream>>>(fifo, kSlotWords, sizes, kSlots, kStepsPerSlice, 0ull, slices, &counters[0], &counters[1],
                                                s.ctrl, s.status, 5000000000ull);
    B2_CUDA(cudaGetLastError());
    bool good = true;
    unsigned long long step = 0;
    for (int k = 0; k < slices && good; ++k) {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(5);
        while (__atomic_load_n(&counters[0], __ATOMIC_ACQUIRE) < step + kStepsPerSlice) {
            if (std::chrono::steady_clock::now() > deadline) { good = false; break; }
        }
        if (!good) break;
        // What a send proxy would do now: read the slot's size and payload, then return the credit.
        const unsigned int slot = static_cast<unsigned int>((step / kStepsPerSlice) % kSlots);
        const unsigned int words = kSlotWords - static_cast<unsigned int>(k % 3);
        good = sizes[slot] == words * 4u;
        for (unsigned int i = 0; good && i < words; ++i) good = fifo[slot * kSlotWords + i] == static_cast<unsigned int>(step * 7919u) + i;
        step += kStepsPerSlice;
        __atomic_store_n(&counters[1], step, __ATOMIC_RELEASE);
    }
    if (!good) {  // let the kernel's bounded wait end at once rather than after its time limit
        const unsigned int one = 1;
        cudaStream_t side;
        B2_CUDA(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
        B2_CUDA(cudaMemcpyAsync(&s.ctrl->abort_flag, &one, sizeof(one), cudaMemcpyHostToDevice, side));
        B2_CUDA(cudaStreamSynchronize(side));
        cudaStreamDestroy(side);
    }
    B2_CUDA(cudaStreamSynchronize(s.stream));
    good = good && s.status->code == kStatusOk;
    cudaFreeHost(fifo);
    cudaFreeHost(sizes);
    cudaFreeHost(counters);
    return good;
}

}  // namespace b200ccl::kernels
