// Minimal stand-in for {fmt}: the reference's error helper formats a message
// with it on a path this build never takes.
#pragma once
#include <string>
namespace fmt {
template <typename... Args>
inline std::string format(const char* f, Args&&...) { return std::string(f); }
}  // namespace fmt
