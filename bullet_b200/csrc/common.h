// Shared host helpers: the per-thread error string behind b200_last_error().
#pragma once
#include <cstdarg>
#include <cstdio>

namespace b200 {

inline char* error_buffer() {
    static thread_local char buf[512] = "";
    return buf;
}

// Records a formatted message for the calling thread and returns `code`.
inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace b200
