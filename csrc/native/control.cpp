// Elastic data-parallel controller, rung bookkeeping and the scaling-law fit.
//
// Behavioural parity with the reference control crate: replica life cycle
// Live / Draining / Dead / Quarantined / Spare / Healing (control/src/lib.rs:71-123),
// gradient accumulation = ceil(tokens_per_step / (n_live * microbatch_tokens))
// (:208-226), straggler and health events drain a replica (:322-334, :571-574),
// spare healing with staged weight shards installed at a step boundary (:339-481),
// SDC majority vote that quarantines the offender's whole rack (:483-568, :713-751),
// collective watchdog on an injected clock (:576-630), loss-spike policy with a
// paging window (:633-653); RungRun (control/src/rung.rs:191-298) and the log-log
// least-squares scaling fit (control/src/scale.rs:112-252).
//
// Every clock is injected by the caller (milliseconds); nothing here reads wall time,
// touches a GPU or blocks, so failure handling is testable on the host alone.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <map>
#include <optional>
#include <set>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace control {

enum class ReplicaState { Live, Draining, Dead, Quarantined, Spare, Healing };
enum class HealthKind { Xid, Ecc, Nvlink, NicFlap, Thermal, WatchdogTimeout };

struct WeightShard {
  std::string name;
  std::string bytes;
};
struct ReplicaSpec {
  std::string id;
  std::string rack;
  bool spare = false;
};
struct ElasticConfig {
  uint64_t tokens_per_step = 0;
  uint64_t microbatch_tokens = 1;
  uint64_t sdc_period_steps = 0;
  uint64_t straggler_timeout_ms = 0;
  uint64_t collective_watchdog_ms = 0;
  uint64_t page_window_steps = 10000;
};
struct SpikeReport {
  std::string rollback_checkpoint_id;
  std::string skipped_shard;
  bool page = false;
};
struct HealthEvent {
  std::string replica, rank;
  HealthKind kind = HealthKind::Xid;
  uint64_t now_ms = 0;
  std::string detail;
};

class Controller {
 public:
  Controller(ElasticConfig cfg, const std::vector<ReplicaSpec>& specs) : cfg_(cfg) {
    if (cfg_.microbatch_tokens == 0) throw Error("Message", "microbatch_tokens must be greater than 0");
    size_t live = 0;
    for (const auto& s : specs) {
      if (table_.count(s.id)) throw Error("Message", "duplicate replica id: " + s.id);
      Rec r;
      r.rack = s.rack;
      r.state = s.spare ? ReplicaState::Spare : ReplicaState::Live;
      live += s.spare ? 0 : 1;
      order_.push_back(s.id);
      table_[s.id] = std::move(r);
    }
    if (live == 0) throw Error("NoLiveReplicas", "no live replicas remain");
  }

  std::vector<std::string> live_replicas() const {
    std::vector<std::string> out;
    for (const auto& id : order_)
      if (table_.at(id).state == ReplicaState::Live) out.push_back(id);
    return out;
  }
  ReplicaState replica_state(const std::string& id) const { return rec(id).state; }
  size_t n_live() const { return live_replicas().size(); }
  uint64_t grad_accumulation() const {
    const uint64_t n = n_live();
    if (cfg_.tokens_per_step == 0 || n == 0) return 0;
    const uint64_t per = n * cfg_.microbatch_tokens;
    if (per == 0) return 0;
    return (cfg_.tokens_per_step + per - 1) / per;
  }
  uint64_t effective_tokens_per_step() const {
    const unsigned __int128 v = static_cast<unsigned __int128>(n_live()) * cfg_.microbatch_tokens *
                                grad_accumulation();
    if (v > UINT64_MAX) throw Error("Message", "effective_tokens_per_step overflow");
    return static_cast<uint64_t>(v);
  }

  void fail_replica(const std::string& id) {
    require_live(id);
    drain(id);
  }
  void observe_step_time(const std::string& id, uint64_t /*step*/, uint64_t duration_ms) {
    require_live(id);
    if (duration_ms > cfg_.straggler_timeout_ms) drain(id);
  }
  void report_health(const HealthEvent& ev) {
    require_live(ev.replica);
    health_log_.push_back(ev);
    drain(ev.replica);
  }
  size_t health_events() const { return health_log_.size(); }

  // -- spare healing -------------------------------------------------------
  void heal_spare(const std::string& spare, const std::string& source) {
    if (rec(spare).state != ReplicaState::Spare) throw Error("NotSpare", "replica is not a spare: " + spare);
    require_live(source);
    Rec& r = table_[spare];
    r.state = ReplicaState::Healing;
    r.heal_source = source;
    r.staged.clear();
  }
  std::string heal_source(const std::string& spare) const {
    const Rec& r = rec(spare);
    if (r.state != ReplicaState::Healing || !r.heal_source)
      throw Error("NoHealInProgress", "no heal in progress: " + spare);
    return *r.heal_source;
  }
  void offer_weight_copy(const std::string& spare, const std::string& source,
                         const std::vector<WeightShard>& shards) {
    if (rec(spare).state != ReplicaState::Healing)
      throw Error("NoHealInProgress", "no heal in progress: " + spare);
    require_live(source);
    Rec& r = table_[spare];
    if (!r.heal_source) throw Error("NoHealInProgress", "no heal in progress: " + spare);
    if (*r.heal_source != source)
      throw Error("HealSourceMismatch", "heal source mismatch spare=" + spare + " expected=" +
                                            *r.heal_source + " got=" + source);
    std::set<std::string> names;
    for (const auto& s : r.staged) names.insert(s.name);
    for (const auto& s : shards) {
      if (s.name.empty()) throw Error("EmptyWeightShardName", "empty weight shard name");
      if (!names.insert(s.name).second)
        throw Error("DuplicateWeightShard", "duplicate weight shard name: " + s.name);
    }
    r.staged.insert(r.staged.end(), shards.begin(), shards.end());
  }
  void rejoin(const std::string& id, uint64_t step) {
    if (rec(id).state != ReplicaState::Healing) throw Error("NotSpare", "replica is not a spare: " + id);
    Rec& r = table_[id];
    r.installed = std::make_pair(step, std::move(r.staged));
    r.staged.clear();
    r.heal_source.reset();
    r.state = ReplicaState::Live;
  }
  std::vector<WeightShard> healed_weight_shards(const std::string& id) const {
    const Rec& r = rec(id);
    if (!r.installed) throw Error("WeightCopyNotInstalled", "weight copy not installed: " + id);
    return r.installed->second;
  }

  // -- silent data corruption ----------------------------------------------
  void report_shard_hash(const std::string& replica, const std::string& shard, const std::string& hex,
                         uint64_t step) {
    require_live(replica);
    hashes_[{step, replica, shard}] = hex;
  }
  void check_sdc(uint64_t step) {
    if (cfg_.sdc_period_steps == 0 || step % cfg_.sdc_period_steps != 0) return;
    const auto live = live_replicas();
    if (live.empty()) return;
    std::set<std::string> shards;
    for (const auto& kv : hashes_)
      if (std::get<0>(kv.first) == step &&
          std::find(live.begin(), live.end(), std::get<1>(kv.first)) != live.end())
        shards.insert(std::get<2>(kv.first));
    if (shards.empty()) throw Error("MissingHash", "missing SDC hash replica=" + live[0] + " shard=");
    for (const auto& shard : shards) {
      std::vector<std::pair<std::string, std::string>> reports;
      std::map<std::string, size_t> votes;
      for (const auto& id : live) {
        auto it = hashes_.find({step, id, shard});
        if (it == hashes_.end())
          throw Error("MissingHash", "missing SDC hash replica=" + id + " shard=" + shard);
        reports.emplace_back(id, it->second);
        ++votes[it->second];
      }
      std::string expected = reports.front().second;  // no majority: first reporter wins
      for (const auto& v : votes)
        if (v.second > reports.size() / 2) {
          expected = v.first;
          break;
        }
      for (const auto& rp : reports)
        if (rp.second != expected) quarantine_rack_of(rp.first, shard, expected, rp.second);
    }
  }

  // -- collective watchdog -------------------------------------------------
  void begin_collective(const std::string& name, const std::string& replica, uint64_t now_ms) {
    require_live(replica);
    for (const auto& c : open_)
      if (c.name == name && c.replica == replica)
        throw Error("Message", "collective already open: " + name);
    open_.push_back({name, replica, now_ms});
  }
  void end_collective(const std::string& name, const std::string& replica, uint64_t /*now_ms*/) {
    require_live(replica);
    open_.erase(std::remove_if(open_.begin(), open_.end(),
                               [&](const Open& c) { return c.name == name && c.replica == replica; }),
                open_.end());
  }
  void tick(uint64_t now_ms) {
    for (const auto& id : std::vector<std::string>(order_)) {
      if (table_[id].state != ReplicaState::Live) continue;
      bool overdue = false;
      for (const auto& c : open_)
        if (c.replica == id && now_ms >= c.begin_ms && now_ms - c.begin_ms > cfg_.collective_watchdog_ms)
          overdue = true;
      if (overdue) drain(id);
    }
  }
  size_t open_collectives() const { return open_.size(); }

  // -- loss spikes ---------------------------------------------------------
  SpikeReport on_loss_spike(uint64_t step, const std::string& shard, const std::string& last_ckpt) {
    bool page = false;
    if (last_spike_) page = (step >= *last_spike_ ? step - *last_spike_ : 0) < cfg_.page_window_steps;
    if (page) ++pages_;
    last_spike_ = step;
    skipped_.push_back(shard);
    return SpikeReport{last_ckpt, shard, page};
  }
  std::vector<std::string> skipped_shards() const { return skipped_; }
  uint64_t pages() const { return pages_; }

 private:
  struct Rec {
    std::string rack;
    ReplicaState state = ReplicaState::Live;
    std::optional<std::string> heal_source;
    std::vector<WeightShard> staged;
    std::optional<std::pair<uint64_t, std::vector<WeightShard>>> installed;
  };
  struct Open {
    std::string name, replica;
    uint64_t begin_ms;
  };
  const Rec& rec(const std::string& id) const {
    auto it = table_.find(id);
    if (it == table_.end()) throw Error("ReplicaNotFound", "replica not found: " + id);
    return it->second;
  }
  void require_live(const std::string& id) const {
    switch (rec(id).state) {
      case ReplicaState::Live: return;
      case ReplicaState::Quarantined: throw Error("Quarantined", "replica quarantined: " + id);
      default: throw Error("NotLive", "replica is not live: " + id);
    }
  }
  void forget_collectives(const std::string& id) {
    open_.erase(std::remove_if(open_.begin(), open_.end(), [&](const Open& c) { return c.replica == id; }),
                open_.end());
  }
  void drain(const std::string& id) {
    if (n_live() <= 1) throw Error("NoLiveReplicas", "no live replicas remain");
    table_[id].state = ReplicaState::Dead;
    forget_collectives(id);
  }
  [[noreturn]] void quarantine_rack_of(const std::string& offender, const std::string& shard,
                                       const std::string& expected, const std::string& got) {
    const std::string rack = rec(offender).rack;
    size_t live_on_rack = 0;
    for (const auto& id : order_)
      if (table_[id].rack == rack && table_[id].state == ReplicaState::Live) ++live_on_rack;
    if (n_live() > live_on_rack) {  // never quarantine the last live rack
      for (const auto& id : order_)
        if (table_[id].rack == rack) {
          table_[id].state = ReplicaState::Quarantined;
          forget_collectives(id);
        }
    }
    throw Error("HashMismatch", "SDC hash mismatch replica=" + offender + " shard=" + shard +
                                    " expected=" + expected + " got=" + got);
  }

  ElasticConfig cfg_;
  std::vector<std::string> order_;
  std::map<std::string, Rec> table_;
  std::map<std::tuple<uint64_t, std::string, std::string>, std::string> hashes_;
  std::vector<Open> open_;
  std::vector<HealthEvent> health_log_;
  std::vector<std::string> skipped_;
  uint64_t pages_ = 0;
  std::optional<uint64_t> last_spike_;
};

// ---------------------------------------------------------------------------
// rungs
// ---------------------------------------------------------------------------
struct RungSpec {
  int id = 0;  // 0..3
  uint64_t active_params = 0, total_params = 0, tokens = 0, gpus = 0;
};
static RungSpec rung_spec(int id) {
  static const RungSpec table[4] = {
      {0, 100000000ull, 1000000000ull, 20000000000ull, 64},
      {1, 1000000000ull, 15000000000ull, 200000000000ull, 1000},
      {2, 8000000000ull, 120000000000ull, 1500000000000ull, 5000},
      {3, 40000000000ull, 700000000000ull, 6000000000000ull, 15000}};
  if (id < 0 || id > 3) throw Error("Message", "rung id must be 0..3");
  return table[id];
}
struct RungConfig {
  RungSpec spec;
  uint64_t token_budget = 0, tokens_per_step = 0;
  std::string tokenizer_hash;
  uint64_t seed = 0;
};
struct RungCheckpoint {
  uint64_t step = 0, tokens_seen = 0;
  std::vector<double> loss_curve;
  std::string tokenizer_hash;
  uint64_t seed = 0, token_budget = 0, tokens_per_step = 0;
  int rung = 0;
};
struct RungStepReport {
  uint64_t step, tokens_seen;
  double loss;
  bool done;
};
static void validate_rung_config(const RungConfig& c) {
  if (c.spec.id != 0) throw Error("NotRung0", "RungRun is rung 0 only");
  if (c.token_budget == 0 || c.token_budget > c.spec.tokens)
    throw Error("InvalidBudget", "token_budget must be > 0 and <= spec.tokens");
  if (c.tokens_per_step == 0) throw Error("InvalidTokensPerStep", "tokens_per_step must be > 0");
  if (c.tokenizer_hash.empty()) throw Error("EmptyTokenizerHash", "tokenizer_hash must be non-empty");
}
class RungRun {
 public:
  explicit RungRun(RungConfig c) : cfg_(std::move(c)) { validate_rung_config(cfg_); }
  static RungRun resume(RungConfig c, const RungCheckpoint& k) {
    validate_rung_config(c);
    if (k.tokenizer_hash != c.tokenizer_hash)
      throw Error("TokenizerChanged", "tokenizer hash changed; the tokenizer is frozen before rung 0");
    if (k.seed != c.seed || k.token_budget != c.token_budget || k.tokens_per_step != c.tokens_per_step ||
        k.rung != c.spec.id)
      throw Error("CheckpointMismatch", "checkpoint does not match this config");
    if (k.tokens_seen > c.token_budget)
      throw Error("ResumePastBudget", "checkpoint tokens_seen exceeds token_budget");
    RungRun r(std::move(c));
    r.step_ = k.step;
    r.seen_ = k.tokens_seen;
    r.curve_ = k.loss_curve;
    return r;
  }
  RungStepReport step(double loss) {
    if (!std::isfinite(loss)) throw Error("NonFiniteLoss", "loss must be finite");
    if (done()) throw Error("AlreadyDone", "rung already consumed its token_budget");
    seen_ += std::min(cfg_.tokens_per_step, cfg_.token_budget - seen_);
    ++step_;
    curve_.push_back(loss);
    return {step_, seen_, loss, done()};
  }
  RungCheckpoint checkpoint() const {
    return {step_, seen_, curve_, cfg_.tokenizer_hash, cfg_.seed, cfg_.token_budget,
            cfg_.tokens_per_step, cfg_.spec.id};
  }
  bool done() const { return seen_ >= cfg_.token_budget; }
  uint64_t step_index() const { return step_; }
  uint64_t tokens_seen() const { return seen_; }
  uint64_t remaining_tokens() const { return cfg_.token_budget > seen_ ? cfg_.token_budget - seen_ : 0; }
  const std::vector<double>& loss_curve() const { return curve_; }
  const RungConfig& config() const { return cfg_; }

 private:
  RungConfig cfg_;
  uint64_t step_ = 0, seen_ = 0;
  std::vector<double> curve_;
};

// ---------------------------------------------------------------------------
// scaling law  L = A * C^-alpha,  C = 6 * active_params * tokens
// ---------------------------------------------------------------------------
struct RungObservation {
  RungSpec spec;
  double loss = 0;
};
struct ScalingFit {
  double a = 0, alpha = 0;
  double predict(uint64_t active, uint64_t tokens) const {
    if (active == 0 || tokens == 0) throw Error("InvalidCompute", "active_params and tokens must be > 0");
    const double p = a * std::pow(6.0 * double(active) * double(tokens), -alpha);
    if (!std::isfinite(p)) throw Error("NonFinitePrediction", "prediction must be finite");
    return p;
  }
  double predict_spec(const RungSpec& s) const {
    if (s.id == 0) throw Error("Rung0NotUsed", "rung 0 is not a scaling-law point");
    return predict(s.active_params, s.tokens);
  }
  double predict_flagship() const { return predict(400000000000ull, 180000000000000ull); }
};
static void validate_observation(const RungObservation& o) {
  if (o.spec.id == 0) throw Error("Rung0NotUsed", "rung 0 is not a scaling-law point");
  if (o.spec.active_params == 0 || o.spec.tokens == 0)
    throw Error("InvalidCompute", "active_params and tokens must be > 0");
  if (!std::isfinite(o.loss)) throw Error("NonFiniteLoss", "loss must be finite");
  if (o.loss <= 0) throw Error("NonPositiveLoss", "loss must be > 0");
}
static ScalingFit fit(const std::vector<RungObservation>& obs) {
  for (const auto& o : obs) validate_observation(o);
  for (size_t i = 0; i < obs.size(); ++i)
    for (size_t j = 0; j < i; ++j)
      if (obs[i].spec.id == obs[j].spec.id) throw Error("DuplicateRung", "duplicate rung in the fit");
  if (obs.size() < 2) throw Error("NeedTwoRungs", "need at least two rungs from 1 to 3");
  std::vector<double> xs, ys, cs;
  for (const auto& o : obs) {
    const double c = 6.0 * double(o.spec.active_params) * double(o.spec.tokens);
    if (!std::isfinite(c) || !std::isfinite(std::log(c)) || !std::isfinite(std::log(o.loss)))
      throw Error("DegenerateFit", "rungs do not determine a unique (A, alpha)");
    for (double prev : cs)
      if (prev == c) throw Error("DegenerateFit", "rungs do not determine a unique (A, alpha)");
    cs.push_back(c);
    xs.push_back(std::log(c));
    ys.push_back(std::log(o.loss));
  }
  double mx = 0, my = 0;
  for (size_t i = 0; i < xs.size(); ++i) {
    mx += xs[i];
    my += ys[i];
  }
  mx /= xs.size();
  my /= ys.size();
  double num = 0, den = 0;
  for (size_t i = 0; i < xs.size(); ++i) {
    num += (xs[i] - mx) * (ys[i] - my);
    den += (xs[i] - mx) * (xs[i] - mx);
  }
  if (den == 0 || !std::isfinite(den)) throw Error("DegenerateFit", "rungs do not determine a unique (A, alpha)");
  const double slope = num / den;
  return {std::exp(my - slope * mx), -slope};
}
static bool should_stop(double predicted, double observed) {
  if (!std::isfinite(predicted) || predicted <= 0)
    throw Error("InvalidPredicted", "predicted loss must be finite and > 0");
  if (!std::isfinite(observed)) throw Error("InvalidObserved", "observed loss must be finite");
  return observed >= predicted * 1.05;
}

}  // namespace control

void bind_control(py::module_& m) {
  using namespace control;
  py::enum_<ReplicaState>(m, "ReplicaState")
      .value("Live", ReplicaState::Live).value("Draining", ReplicaState::Draining)
      .value("Dead", ReplicaState::Dead).value("Quarantined", ReplicaState::Quarantined)
      .value("Spare", ReplicaState::Spare).value("Healing", ReplicaState::Healing);
  py::enum_<HealthKind>(m, "HealthKind")
      .value("Xid", HealthKind::Xid).value("Ecc", HealthKind::Ecc).value("Nvlink", HealthKind::Nvlink)
      .value("NicFlap", HealthKind::NicFlap).value("Thermal", HealthKind::Thermal)
      .value("WatchdogTimeout", HealthKind::WatchdogTimeout);
  py::class_<WeightShard>(m, "WeightShard")
      .def(py::init([](std::string n, py::bytes b) { return WeightShard{std::move(n), std::string(b)}; }))
      .def_readwrite("name", &WeightShard::name)
      .def_property_readonly("bytes", [](const WeightShard& s) { return py::bytes(s.bytes); });
  py::class_<ReplicaSpec>(m, "ReplicaSpec")
      .def(py::init([](std::string id, std::string rack, bool spare) {
             return ReplicaSpec{std::move(id), std::move(rack), spare};
           }),
           py::arg("id"), py::arg("rack"), py::arg("spare") = false)
      .def_readwrite("id", &ReplicaSpec::id).def_readwrite("rack", &ReplicaSpec::rack)
      .def_readwrite("spare", &ReplicaSpec::spare);
  py::class_<ElasticConfig>(m, "ElasticConfig")
      .def(py::init([](uint64_t tps, uint64_t mb, uint64_t sdc, uint64_t strag, uint64_t wd, uint64_t pw) {
             return ElasticConfig{tps, mb, sdc, strag, wd, pw};
           }),
           py::arg("tokens_per_step"), py::arg("microbatch_tokens"), py::arg("sdc_period_steps") = 0,
           py::arg("straggler_timeout_ms") = 60000, py::arg("collective_watchdog_ms") = 60000,
           py::arg("page_window_steps") = 10000)
      .def_readwrite("tokens_per_step", &ElasticConfig::tokens_per_step)
      .def_readwrite("microbatch_tokens", &ElasticConfig::microbatch_tokens)
      .def_readwrite("sdc_period_steps", &ElasticConfig::sdc_period_steps)
      .def_readwrite("straggler_timeout_ms", &ElasticConfig::straggler_timeout_ms)
      .def_readwrite("collective_watchdog_ms", &ElasticConfig::collective_watchdog_ms)
      .def_readwrite("page_window_steps", &ElasticConfig::page_window_steps);
  py::class_<SpikeReport>(m, "SpikeReport")
      .def_readonly("rollback_checkpoint_id", &SpikeReport::rollback_checkpoint_id)
      .def_readonly("skipped_shard", &SpikeReport::skipped_shard)
      .def_readonly("page", &SpikeReport::page);
  py::class_<HealthEvent>(m, "HealthEvent")
      .def(py::init([](std::string replica, std::string rank, HealthKind kind, uint64_t now, std::string d) {
             return HealthEvent{std::move(replica), std::move(rank), kind, now, std::move(d)};
           }),
           py::arg("replica"), py::arg("rank"), py::arg("kind"), py::arg("now_ms") = 0,
           py::arg("detail") = "");
  py::class_<Controller>(m, "Controller")
      .def(py::init<ElasticConfig, const std::vector<ReplicaSpec>&>())
      .def("live_replicas", &Controller::live_replicas)
      .def("replica_state", &Controller::replica_state)
      .def("n_live", &Controller::n_live)
      .def("grad_accumulation", &Controller::grad_accumulation)
      .def("effective_tokens_per_step", &Controller::effective_tokens_per_step)
      .def("fail_replica", &Controller::fail_replica)
      .def("observe_step_time", &Controller::observe_step_time)
      .def("report_health", &Controller::report_health)
      .def("health_events", &Controller::health_events)
      .def("heal_spare", &Controller::heal_spare)
      .def("heal_source", &Controller::heal_source)
      .def("offer_weight_copy", &Controller::offer_weight_copy)
      .def("rejoin", &Controller::rejoin)
      .def("healed_weight_shards", &Controller::healed_weight_shards)
      .def("report_shard_hash", &Controller::report_shard_hash)
      .def("check_sdc", &Controller::check_sdc)
      .def("begin_collective", &Controller::begin_collective)
      .def("end_collective", &Controller::end_collective)
      .def("tick", &Controller::tick)
      .def("open_collectives", &Controller::open_collectives)
      .def("on_loss_spike", &Controller::on_loss_spike)
      .def("skipped_shards", &Controller::skipped_shards)
      .def("pages", &Controller::pages);
  py::class_<RungSpec>(m, "RungSpec")
      .def(py::init([](int id, uint64_t a, uint64_t t, uint64_t tok, uint64_t g) {
             return RungSpec{id, a, t, tok, g};
           }),
           py::arg("id"), py::arg("active_params"), py::arg("total_params"), py::arg("tokens"),
           py::arg("gpus"))
      .def_readwrite("id", &RungSpec::id).def_readwrite("active_params", &RungSpec::active_params)
      .def_readwrite("total_params", &RungSpec::total_params).def_readwrite("tokens", &RungSpec::tokens)
      .def_readwrite("gpus", &RungSpec::gpus);
  m.def("rung_spec", &rung_spec);
  m.def("rung_0_spec", [] { return rung_spec(0); });
  py::class_<RungConfig>(m, "RungConfig")
      .def(py::init([](RungSpec s, uint64_t budget, uint64_t tps, std::string th, uint64_t seed) {
             return RungConfig{s, budget, tps, std::move(th), seed};
           }),
           py::arg("spec"), py::arg("token_budget"), py::arg("tokens_per_step"),
           py::arg("tokenizer_hash"), py::arg("seed") = 0)
      .def_readwrite("spec", &RungConfig::spec).def_readwrite("token_budget", &RungConfig::token_budget)
      .def_readwrite("tokens_per_step", &RungConfig::tokens_per_step)
      .def_readwrite("tokenizer_hash", &RungConfig::tokenizer_hash).def_readwrite("seed", &RungConfig::seed);
  py::class_<RungCheckpoint>(m, "RungCheckpoint")
      .def(py::init<>())
      .def_readwrite("step", &RungCheckpoint::step).def_readwrite("tokens_seen", &RungCheckpoint::tokens_seen)
      .def_readwrite("loss_curve", &RungCheckpoint::loss_curve)
      .def_readwrite("tokenizer_hash", &RungCheckpoint::tokenizer_hash)
      .def_readwrite("seed", &RungCheckpoint::seed).def_readwrite("token_budget", &RungCheckpoint::token_budget)
      .def_readwrite("tokens_per_step", &RungCheckpoint::tokens_per_step)
      .def_readwrite("rung", &RungCheckpoint::rung);
  py::class_<RungStepReport>(m, "RungStepReport")
      .def_readonly("step", &RungStepReport::step).def_readonly("tokens_seen", &RungStepReport::tokens_seen)
      .def_readonly("loss", &RungStepReport::loss).def_readonly("done", &RungStepReport::done);
  m.def("validate_rung_config", &validate_rung_config);
  py::class_<RungRun>(m, "RungRun")
      .def(py::init<RungConfig>())
      .def_static("resume", &RungRun::resume)
      .def("step", &RungRun::step).def("checkpoint", &RungRun::checkpoint).def("done", &RungRun::done)
      .def("step_index", &RungRun::step_index).def("tokens_seen", &RungRun::tokens_seen)
      .def("remaining_tokens", &RungRun::remaining_tokens).def("loss_curve", &RungRun::loss_curve)
      .def("config", &RungRun::config);
  py::class_<RungObservation>(m, "RungObservation")
      .def(py::init([](RungSpec s, double l) { return RungObservation{s, l}; }));
  py::class_<ScalingFit>(m, "ScalingFit")
      .def_property_readonly("a", [](const ScalingFit& f) { return f.a; })
      .def_property_readonly("alpha", [](const ScalingFit& f) { return f.alpha; })
      .def("predict", &ScalingFit::predict).def("predict_spec", &ScalingFit::predict_spec)
      .def("predict_flagship", &ScalingFit::predict_flagship);
  m.def("fit", &fit);
  m.def("should_stop", &should_stop);
  m.def("compute_flops", [](uint64_t a, uint64_t t) {
    if (a == 0 || t == 0) throw Error("InvalidCompute", "active_params and tokens must be > 0");
    return 6.0 * double(a) * double(t);
  });
  m.def("predict_held_out", [](const std::vector<RungObservation>& train, const RungSpec& held) {
    for (const auto& o : train)
      if (o.spec.id == held.id) throw Error("HeldOutInTrain", "held-out rung was in the train set");
    return fit(train).predict_spec(held);
  });
}
