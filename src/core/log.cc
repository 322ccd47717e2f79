// Levelled logging to stderr. nano-nccl has no log levels (it prints errors only); this adds
// B200CCL_DEBUG=WARN|INFO|TRACE so that the chosen transport per edge and the algorithm per
// call can be seen without a debugger.
#include "core/check.h"
#include "core/env.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <unistd.h>

namespace b200ccl {

int log_level() {
    static const int level = [] {
        const char* v = env::get("B200CCL_DEBUG", "NANO_NCCL_DEBUG");
        if (!v) return 1;
        if (!strcasecmp(v, "NONE") || !strcmp(v, "0")) return 0;
        if (!strcasecmp(v, "WARN")) return 1;
        if (!strcasecmp(v, "INFO")) return 2;
        if (!strcasecmp(v, "TRACE")) return 3;
        return 1;
    }();
    return level;
}

static void vlog(const char* tag, const char* fmt, va_list ap) {
    char buf[2048];
    std::vsnprintf(buf, sizeof(buf), fmt, ap);
    std::fprintf(stderr, "[b200ccl %s pid=%d] %s\n", tag, static_cast<int>(getpid()), buf);
}

void log_warn(const char* fmt, ...) {
    if (log_level() < 1) return;
    va_list ap; va_start(ap, fmt); vlog("WARN", fmt, ap); va_end(ap);
}
void log_info(const char* fmt, ...) {
    if (log_level() < 2) return;
    va_list ap; va_start(ap, fmt); vlog("INFO", fmt, ap); va_end(ap);
}
void log_trace(const char* fmt, ...) {
    if (log_level() < 3) return;
    va_list ap; va_start(ap, fmt); vlog("TRACE", fmt, ap); va_end(ap);
}

}  // namespace b200ccl
