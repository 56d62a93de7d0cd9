// Stand-in for {fmt}: forwards to std::format (C++20). Test-only, see ../spdlog/spdlog.h.
#pragma once
#include <format>
namespace fmt {
using std::format;
}
