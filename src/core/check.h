// Error helpers: CUDA runtime / driver status → std::runtime_error with call text and place.
// Counterpart of CUDA_CHECK_THROW in nano-nccl src/core/buffer.h:22-31.
#pragma once

#include <cuda_runtime.h>

#include <sstream>
#include <stdexcept>
#include <string>

namespace b200ccl {

[[noreturn]] inline void throw_cuda(cudaError_t st, const char* what, const char* file, int line) {
    std::ostringstream os;
    os << what << " failed: " << cudaGetErrorName(st) << " (" << cudaGetErrorString(st) << ") at "
       << file << ":" << line;
    throw std::runtime_error(os.str());
}

#define B2_CUDA(expr)                                                        \
    do {                                                                     \
        cudaError_t b2_st_ = (expr);                                         \
        if (b2_st_ != cudaSuccess) ::b200ccl::throw_cuda(b2_st_, #expr, __FILE__, __LINE__); \
    } while (0)

// For destructors and cleanup paths: report, never throw.
#define B2_CUDA_WARN(expr)                                                              \
    do {                                                                                \
        cudaError_t b2_st_ = (expr);                                                    \
        if (b2_st_ != cudaSuccess)                                                      \
            ::b200ccl::log_warn("%s failed: %s at %s:%d", #expr, cudaGetErrorString(b2_st_), \
                                __FILE__, __LINE__);                                    \
    } while (0)

#define B2_REQUIRE(cond, msg)                                  \
    do {                                                       \
        if (!(cond)) throw std::invalid_argument(std::string(msg)); \
    } while (0)

void log_warn(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
void log_info(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
void log_trace(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
int log_level();  // 0 none, 1 warn, 2 info, 3 trace  (B200CCL_DEBUG=WARN|INFO|TRACE)

// Scoped cudaSetDevice that restores the previous device.
class DeviceGuard {
public:
    explicit DeviceGuard(int device) {
        B2_CUDA(cudaGetDevice(&prev_));
        if (prev_ != device) B2_CUDA(cudaSetDevice(device));
        cur_ = device;
    }
    ~DeviceGuard() {
        if (prev_ != cur_) cudaSetDevice(prev_);
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;

private:
    int prev_ = 0;
    int cur_ = 0;
};

}  // namespace b200ccl
