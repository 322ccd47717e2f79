// RAII holders for streams, events and instantiated graphs.
// Parity: nano-nccl src/core/stream.h:11-133 (Stream non-blocking, Event without timing,
// GraphExec). Here GraphExec is used: the benchmark can replay a captured batch of collectives.
#pragma once

#include "core/check.h"

#include <utility>

namespace b200ccl {

class Stream {
public:
    explicit Stream(int device) : device_(device) {
        DeviceGuard guard(device);
        B2_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    }
    ~Stream() { if (stream_) cudaStreamDestroy(stream_); }
    Stream(Stream&& o) noexcept : stream_(o.stream_), device_(o.device_) { o.stream_ = nullptr; }
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    cudaStream_t get() const { return stream_; }
    int device() const { return device_; }
    void synchronize() const { DeviceGuard guard(device_); B2_CUDA(cudaStreamSynchronize(stream_)); }
private:
    cudaStream_t stream_ = nullptr;
    int device_ = 0;
};

class Event {
public:
    explicit Event(int device, bool timing = false) : device_(device) {
        DeviceGuard guard(device);
        B2_CUDA(cudaEventCreateWithFlags(&event_, timing ? cudaEventDefault : cudaEventDisableTiming));
    }
    ~Event() { if (event_) cudaEventDestroy(event_); }
    Event(Event&& o) noexcept : event_(o.event_), device_(o.device_) { o.event_ = nullptr; }
    Event(const Event&) = delete;
    Event& operator=(const Event&) = delete;
    cudaEvent_t get() const { return event_; }
    void record(cudaStream_t s) const { DeviceGuard guard(device_); B2_CUDA(cudaEventRecord(event_, s)); }
    bool done() const {
        const cudaError_t st = cudaEventQuery(event_);
        if (st == cudaErrorNotReady) { (void)cudaGetLastError(); return false; }
        B2_CUDA(st);
        return true;
    }
private:
    cudaEvent_t event_ = nullptr;
    int device_ = 0;
};

class GraphExec {
public:
    GraphExec() = default;
    explicit GraphExec(cudaGraph_t graph) { B2_CUDA(cudaGraphInstantiate(&exec_, graph, 0)); }
    ~GraphExec() { if (exec_) cudaGraphExecDestroy(exec_); }
    GraphExec(GraphExec&& o) noexcept : exec_(o.exec_) { o.exec_ = nullptr; }
    GraphExec& operator=(GraphExec&& o) noexcept { std::swap(exec_, o.exec_); return *this; }
    GraphExec(const GraphExec&) = delete;
    GraphExec& operator=(const GraphExec&) = delete;
    void launch(cudaStream_t s) const { B2_CUDA(cudaGraphLaunch(exec_, s)); }
    explicit operator bool() const { return exec_ != nullptr; }
private:
    cudaGraphExec_t exec_ = nullptr;
};

}  // namespace b200ccl
