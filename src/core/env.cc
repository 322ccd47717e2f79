#include "core/env.h"

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <stdexcept>

namespace b200ccl::env {

const char* get(const char* name, const char* compat_name) {
    const char* v = std::getenv(name);
    if (v && *v) return v;
    if (compat_name) {
        v = std::getenv(compat_name);
        if (v && *v) return v;
    }
    return nullptr;
}

bool parse_bool(const std::string& text, bool* out) {
    std::string t(text);
    std::transform(t.begin(), t.end(), t.begin(), [](unsigned char c) { return std::tolower(c); });
    if (t == "1" || t == "true" || t == "on") { *out = true; return true; }
    if (t == "0" || t == "false" || t == "off") { *out = false; return true; }
    return false;
}

bool parse_bytes(const std::string& text, std::size_t* out) {
    if (text.empty()) return false;
    char* end = nullptr;
    const double v = std::strtod(text.c_str(), &end);
    if (end == text.c_str() || v < 0) return false;
    double mult = 1;
    std::string suffix(end);
    std::transform(suffix.begin(), suffix.end(), suffix.begin(),
                   [](unsigned char c) { return std::toupper(c); });
    if (suffix == "" || suffix == "B") mult = 1;
    else if (suffix == "K" || suffix == "KB" || suffix == "KIB") mult = 1024.0;
    else if (suffix == "M" || suffix == "MB" || suffix == "MIB") mult = 1024.0 * 1024;
    else if (suffix == "G" || suffix == "GB" || suffix == "GIB") mult = 1024.0 * 1024 * 1024;
    else return false;
    *out = static_cast<std::size_t>(v * mult);
    return true;
}

bool get_bool(const char* name, bool dflt, const char* compat_name) {
    const char* v = get(name, compat_name);
    if (!v) return dflt;
    bool out = dflt;
    if (!parse_bool(v, &out))
        throw std::invalid_argument(std::string(name) + " must be one of 0/1/true/false/on/off, got '" + v + "'");
    return out;
}

long long get_int(const char* name, long long dflt, const char* compat_name) {
    const char* v = get(name, compat_name);
    if (!v) return dflt;
    char* end = nullptr;
    const long long out = std::strtoll(v, &end, 10);
    if (end == v || *end != '\0')
        throw std::invalid_argument(std::string(name) + " must be an integer, got '" + v + "'");
    return out;
}

double get_double(const char* name, double dflt, const char* compat_name) {
    const char* v = get(name, compat_name);
    if (!v) return dflt;
    char* end = nullptr;
    const double out = std::strtod(v, &end);
    if (end == v || *end != '\0')
        throw std::invalid_argument(std::string(name) + " must be a number, got '" + v + "'");
    return out;
}

std::size_t get_bytes(const char* name, std::size_t dflt, const char* compat_name) {
    const char* v = get(name, compat_name);
    if (!v) return dflt;
    std::size_t out = dflt;
    if (!parse_bytes(v, &out))
        throw std::invalid_argument(std::string(name) + " must be a byte count such as 32M, got '" + v + "'");
    return out;
}

std::string get_string(const char* name, const std::string& dflt, const char* compat_name) {
    const char* v = get(name, compat_name);
    return v ? std::string(v) : dflt;
}

}  // namespace b200ccl::env
