// Single-GPU self-tests of the bounded wait, the abort flag and release/acquire publication.
#pragma once

namespace b200ccl::kernels {

struct SelfTestResult {
    int wait_ok = -1;            // 1 the wait was satisfied, 0 it gave up
    unsigned int status_code = 0;  // dev::StatusCode recorded by the kernel
    unsigned int where = 0;
    double waited_ms = 0.0;
    bool abort_raised = false;
};

SelfTestResult selftest_wait_timeout(int device, double timeout_ms);
SelfTestResult selftest_abort(int device, double timeout_ms);
bool selftest_publication(int device, int rounds);
// Device-side "send" of `slices` slices into a mapped host FIFO with no proxy thread: the host plays
// the proxy and checks tail, byte count and payload of every slot, returning credits as it goes.
bool selftest_direct_send(int device, int slices);

}  // namespace b200ccl::kernels
