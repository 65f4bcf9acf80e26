// Provider failover order and the AIMD concurrency window, shared by the provider broker and
// the generation router (reference: harness/providers/src/lib.rs Failover, Aimd).
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "common.hpp"

namespace pbn {

struct AimdConfig {
  uint32_t min_window = 1, max_window = 32, increase = 1;
  double decrease = 0.5;
  uint64_t latency_limit_ms = 30000;
};

class Aimd {
 public:
  explicit Aimd(AimdConfig c) : cfg_(c), window_(std::max<uint32_t>(c.min_window, 1)) {}
  uint32_t window() const { return window_; }
  void on_success(uint64_t latency_ms) {
    if (latency_ms > cfg_.latency_limit_ms) return on_429();   // too slow counts as a push-back
    const uint64_t w = static_cast<uint64_t>(window_) + cfg_.increase;
    window_ = static_cast<uint32_t>(std::min<uint64_t>(w, cfg_.max_window));
  }
  void on_429() {
    const double scaled = static_cast<double>(window_) * cfg_.decrease;
    uint32_t floored = 0;
    if (std::isfinite(scaled)) floored = static_cast<uint32_t>(std::min(std::max(std::floor(scaled), 0.0), 4294967295.0));
    const uint32_t shrunk = floored >= window_ ? (window_ > 0 ? window_ - 1 : 0) : floored;
    window_ = std::max(shrunk, cfg_.min_window);
  }
  void on_outage() { on_429(); }

 private:
  AimdConfig cfg_;
  uint32_t window_;
};

class Failover {
 public:
  explicit Failover(std::vector<std::string> p) : providers_(std::move(p)) {}
  const std::string& current() const {
    for (const auto& p : providers_)
      if (!is_down(p)) return p;
    throw Error("NoProvider", "no provider available");
  }
  void mark_down(const std::string& id) {
    known(id);
    if (!is_down(id)) down_.push_back(id);
  }
  void mark_up(const std::string& id) {
    known(id);
    std::vector<std::string> keep;
    for (auto& d : down_)
      if (d != id) keep.push_back(d);
    down_ = keep;
  }
  uint64_t wait_backoff_ms() const { return 100ull << std::min<size_t>(down_.size(), 8); }
  const std::vector<std::string>& providers() const { return providers_; }
  const std::vector<std::string>& down() const { return down_; }

 private:
  bool is_down(const std::string& id) const {
    for (auto& d : down_)
      if (d == id) return true;
    return false;
  }
  void known(const std::string& id) const {
    for (auto& p : providers_)
      if (p == id) return;
    throw Error("NotFound", "not found: " + id);
  }
  std::vector<std::string> providers_, down_;
};

}  // namespace pbn
