// Stand-in for spdlog's colour sink header (see ../spdlog.h): test-only, no-op.
#pragma once
#include "../spdlog.h"
namespace spdlog {
inline std::shared_ptr<logger> stdout_color_mt(const std::string&) {
    auto l = std::make_shared<logger>();
    registry_slot() = l;
    return l;
}
}  // namespace spdlog
