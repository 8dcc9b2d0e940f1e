// Minimal stand-in for spdlog: a logger type whose calls do nothing.
#pragma once
#include <memory>
#include <string>
namespace spdlog {
struct logger {
  template <typename... Args> void critical(Args&&...) {}
  template <typename... Args> void error(Args&&...) {}
  template <typename... Args> void info(Args&&...) {}
  template <typename... Args> void debug(Args&&...) {}
};
}  // namespace spdlog
