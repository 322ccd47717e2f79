// Minimal assertion helpers for the native test programs (exit code 0 = pass, 77 = skip).
#pragma once

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <stdexcept>
#include <string>

#define T_CHECK(cond)                                                                  \
    do {                                                                               \
        if (!(cond)) {                                                                 \
            std::fprintf(stderr, "CHECK FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                              \
        }                                                                              \
    } while (0)

// Runs f, requires that it throws and that the message contains `needle`.
inline void t_expect_throw(const std::function<void()>& f, const std::string& needle, const char* what) {
    try {
        f();
    } catch (const std::exception& e) {
        if (std::string(e.what()).find(needle) == std::string::npos) {
            std::fprintf(stderr, "%s: message '%s' lacks '%s'\n", what, e.what(), needle.c_str());
            std::exit(1);
        }
        return;
    }
    std::fprintf(stderr, "%s: expected an exception containing '%s'\n", what, needle.c_str());
    std::exit(1);
}
