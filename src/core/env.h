// Environment knobs. Every variable is read through these helpers so that a malformed value
// is an error, not a silent default (nano-nccl parses its booleans the same strict way,
// src/transport/rdma/rdma_proxy.cc:131-142). Names use the B200CCL_ prefix; where a
// nano-nccl variable has the same meaning its NANO_NCCL_ spelling is accepted too.
#pragma once

#include <cstddef>
#include <string>

namespace b200ccl::env {

// Returns nullptr when neither `name` nor `compat_name` is set.
const char* get(const char* name, const char* compat_name = nullptr);
bool get_bool(const char* name, bool dflt, const char* compat_name = nullptr);   // 0/1/true/false/on/off
long long get_int(const char* name, long long dflt, const char* compat_name = nullptr);
double get_double(const char* name, double dflt, const char* compat_name = nullptr);
std::size_t get_bytes(const char* name, std::size_t dflt, const char* compat_name = nullptr);  // 64K, 32M, 1G
std::string get_string(const char* name, const std::string& dflt, const char* compat_name = nullptr);

bool parse_bool(const std::string& text, bool* out);
bool parse_bytes(const std::string& text, std::size_t* out);

}  // namespace b200ccl::env
