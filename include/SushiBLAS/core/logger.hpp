// core/logger.hpp -- SB_LOG_* / SB_THROW_IF / SB_ASSERT with the reference's call syntax
// (include/SushiBLAS/core/logger.hpp:212-323: std::format-style messages; SB_THROW_IF logs and
// throws std::runtime_error).  Minimal on purpose: one synchronous line to stderr, enabled by
// the environment variable SUSHI_LOG (error|warn|info|debug); silent by default so that nothing
// is formatted inside timed regions.  The reference's asynchronous logger thread is not rebuilt.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <format>
#include <stdexcept>
#include <string>

namespace SushiBLAS
{
    namespace Core
    {
        enum class LogLevel : int { NONE = 0, ERROR = 1, WARN = 2, INFO = 3, DEBUG = 4 };

        inline LogLevel log_level()
        {
            static const LogLevel level = [] {
                const char* e = std::getenv("SUSHI_LOG");
                if (!e) return LogLevel::NONE;
                if (!std::strcmp(e, "debug")) return LogLevel::DEBUG;
                if (!std::strcmp(e, "info")) return LogLevel::INFO;
                if (!std::strcmp(e, "warn")) return LogLevel::WARN;
                if (!std::strcmp(e, "error")) return LogLevel::ERROR;
                return LogLevel::NONE;
            }();
            return level;
        }

        inline void log_line(const char* tag, const std::string& msg)
        {
            std::fprintf(stderr, "[SushiBLAS %s] %s\n", tag, msg.c_str());
        }
    } // namespace Core
} // namespace SushiBLAS

#define SB_LOG_AT(level, tag, fmt, ...)                                                        \
    do {                                                                                       \
        if (static_cast<int>(::SushiBLAS::Core::log_level()) >= static_cast<int>(level))       \
            ::SushiBLAS::Core::log_line(tag, std::format(fmt __VA_OPT__(,) __VA_ARGS__));      \
    } while (0)

#define SB_LOG_ERROR(fmt, ...) SB_LOG_AT(::SushiBLAS::Core::LogLevel::ERROR, "ERROR", fmt __VA_OPT__(,) __VA_ARGS__)
#define SB_LOG_WARN(fmt, ...)  SB_LOG_AT(::SushiBLAS::Core::LogLevel::WARN,  "WARN",  fmt __VA_OPT__(,) __VA_ARGS__)
#define SB_LOG_INFO(fmt, ...)  SB_LOG_AT(::SushiBLAS::Core::LogLevel::INFO,  "INFO",  fmt __VA_OPT__(,) __VA_ARGS__)
#define SB_LOG_DEBUG(fmt, ...) SB_LOG_AT(::SushiBLAS::Core::LogLevel::DEBUG, "DEBUG", fmt __VA_OPT__(,) __VA_ARGS__)

#define SB_ASSERT(condition, msg)                                                              \
    do {                                                                                       \
        if (!(condition)) {                                                                    \
            std::fprintf(stderr, "[SushiBLAS] assertion failed: %s (%s:%d)\n", msg, __FILE__, __LINE__); \
            std::abort();                                                                      \
        }                                                                                      \
    } while (0)

#define SB_THROW_IF(condition, fmt, ...)                                                       \
    do {                                                                                       \
        if (condition) {                                                                       \
            std::string sb_msg_ = std::format(fmt __VA_OPT__(,) __VA_ARGS__);                  \
            SB_LOG_ERROR("Runtime exception: {}", sb_msg_);                                    \
            throw std::runtime_error(sb_msg_);                                                 \
        }                                                                                      \
    } while (0)
