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

}  // namespace b200ccl::kernels
