// Levelled stderr logging and assertion macros. SLIME_LOG_LEVEL: 0 = errors only,
// 1 = warnings and info, 2 = debug. SLIME_LOG_MUTEX=1 serialises lines from threads.
#pragma once

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>

#include "env.h"

namespace slime {

inline std::mutex& log_mutex()
{
    static std::mutex m;
    return m;
}

template<typename... Args>
inline std::string log_concat(Args&&... args)
{
    std::ostringstream os;
    (void)std::initializer_list<int>{((os << args), 0)...};
    return os.str();
}

inline void log_emit(const char* tag, const char* color, const char* file, int line, const std::string& msg)
{
    const bool                   lock = engine_env().log_mutex != 0;
    std::unique_lock<std::mutex> g(log_mutex(), std::defer_lock);
    if (lock) g.lock();
    const char* base = file;
    for (const char* p = file; *p; ++p)
        if (*p == '/') base = p + 1;
    fprintf(stderr, "%s[%s]\033[0m %s:%d %s\n", color, tag, base, line, msg.c_str());
}

}  // namespace slime

#define SLIME_LOG_AT(level, tag, color, ...)                                                                            \
    do {                                                                                                                \
        if (::slime::engine_env().log_level >= (level))                                                                 \
            ::slime::log_emit(tag, color, __FILE__, __LINE__, ::slime::log_concat(__VA_ARGS__));                        \
    } while (0)

#define SLIME_LOG_ERROR(...) SLIME_LOG_AT(0, "ERROR", "\033[1;31m", __VA_ARGS__)
#define SLIME_LOG_WARN(...) SLIME_LOG_AT(1, "WARN", "\033[1;33m", __VA_ARGS__)
#define SLIME_LOG_INFO(...) SLIME_LOG_AT(1, "INFO", "\033[1;32m", __VA_ARGS__)
#define SLIME_LOG_DEBUG(...) SLIME_LOG_AT(2, "DEBUG", "\033[1;36m", __VA_ARGS__)

// Unlike the reference's SLIME_ABORT (which ends the process), a failed check raises an
// exception that reaches Python as RuntimeError, so one bad call cannot take a server down.
#define SLIME_ASSERT(cond, ...)                                                                                        \
    do {                                                                                                                \
        if (!(cond)) {                                                                                                  \
            std::string _m = ::slime::log_concat("assertion failed: " #cond " ", __VA_ARGS__);                          \
            SLIME_LOG_ERROR(_m);                                                                                        \
            throw std::runtime_error(_m);                                                                               \
        }                                                                                                               \
    } while (0)

#define SLIME_FAIL(...)                                                                                                 \
    do {                                                                                                                \
        std::string _m = ::slime::log_concat(__VA_ARGS__);                                                              \
        SLIME_LOG_ERROR(_m);                                                                                            \
        throw std::runtime_error(_m);                                                                                   \
    } while (0)
