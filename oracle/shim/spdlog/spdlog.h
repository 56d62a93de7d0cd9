// Stand-in for spdlog, used only to compile the reference's own sources into the
// test-only checker library (oracle/_ref). Every logging call is a no-op.
// This is test infrastructure; nothing in the product includes it.
#pragma once
#include <memory>
#include <string>
#include "../fmt/format.h"  // the real spdlog drags {fmt} in; callers rely on that

namespace spdlog {
namespace level {
enum level_enum { trace, debug, info, warn, err, critical, off };
}
class logger {
public:
    void set_level(level::level_enum) {}
    void set_pattern(const std::string&) {}
    template <typename... A> void trace(A&&...) {}
    template <typename... A> void debug(A&&...) {}
    template <typename... A> void info(A&&...) {}
    template <typename... A> void warn(A&&...) {}
    template <typename... A> void error(A&&...) {}
    template <typename... A> void critical(A&&...) {}
};
inline std::shared_ptr<logger>& registry_slot() {
    static std::shared_ptr<logger> slot;
    return slot;
}
inline std::shared_ptr<logger> get(const std::string&) { return registry_slot(); }
inline void set_default_logger(std::shared_ptr<logger> l) { registry_slot() = std::move(l); }
template <typename... A> inline void trace(A&&...) {}
template <typename... A> inline void debug(A&&...) {}
template <typename... A> inline void info(A&&...) {}
template <typename... A> inline void warn(A&&...) {}
template <typename... A> inline void error(A&&...) {}
template <typename... A> inline void critical(A&&...) {}
}  // namespace spdlog

#define SPDLOG_LOGGER_TRACE(lg, ...) ((void)0)
#define SPDLOG_LOGGER_DEBUG(lg, ...) ((void)0)
#define SPDLOG_LOGGER_INFO(lg, ...) ((void)0)
#define SPDLOG_LOGGER_WARN(lg, ...) ((void)0)
#define SPDLOG_LOGGER_ERROR(lg, ...) ((void)0)
#define SPDLOG_LOGGER_CRITICAL(lg, ...) ((void)0)
