// RL orchestration components:
//
//   coordinator  asynchronous RL bookkeeping: integer policy versions, a staleness-bounded batch
//                queue, weight publication and per-rack sync, trainer/engine log-prob parity
//                with a sticky HALT, and the rollout/trainer rack split (65 % of GPUs to
//                rollouts by default, one rack moved per rebalance)
//                (reference: rl/coordinator/src/lib.rs:32-41, 160-177, 179-557)
//   multiagent   episode topologies (50/20/15/10/5 mix by integer draw), rosters, private
//                inboxes, a shared scratch-pad, latent-memo dropout, credit records, one token
//                budget charged across all agents of an episode, distil-back rule
//                (reference: rl/multiagent/src/lib.rs:35-62, 202-627)
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cmath>
#include <deque>
#include <map>
#include <set>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

// ---------------------------------------------------------------------------- coordinator
struct CoordConfig {
  uint64_t max_staleness = 4, rollout_numer = 65, rollout_denom = 100;
  double parity_threshold = 1e-3;
  size_t queue_high = 8, min_rollout_racks = 1, min_trainer_racks = 1;
};
struct RolloutBatch {
  std::string id, prompt_id;
  uint64_t policy_version = 0;
  uint32_t n_samples = 0;
  bool routing_present = false;
};
struct Rack {
  uint64_t gpus = 0;
  bool rollout = false;
  std::optional<uint64_t> version;   // rollout racks only
};

uint64_t staleness(uint64_t trainer, uint64_t batch) {
  if (batch > trainer) throw Error("FromTheFuture", "batch policy version is ahead of the trainer");
  return trainer - batch;
}

class Coordinator {
 public:
  Coordinator(CoordConfig cfg, std::vector<std::pair<std::string, uint64_t>> racks) : cfg_(cfg) {
    if (racks.empty()) throw Error("EmptyFleet", "no racks in the fleet");
    std::set<std::string> seen;
    for (auto& r : racks)
      if (!seen.insert(r.first).second) throw Error("DuplicateRack", "duplicate rack id: " + r.first);
    for (auto& r : racks)
      if (r.second == 0) throw Error("Message", "rack " + r.first + " has 0 gpus; each rack must have gpus > 0");
    if (cfg.rollout_denom == 0 || cfg.rollout_numer > cfg.rollout_denom)
      throw Error("BadSplit", "rollout_denom must be greater than 0");
    if (racks.size() < cfg.min_rollout_racks + cfg.min_trainer_racks)
      throw Error("NotEnoughRacks", "not enough racks for min_rollout_racks + min_trainer_racks");
    std::sort(racks.begin(), racks.end());
    const size_t n = racks.size();
    for (auto& r : racks) total_ = total_ > UINT64_MAX - r.second ? UINT64_MAX : total_ + r.second;
    const uint64_t target = this->target();
    size_t n_rollout = 0;
    unsigned __int128 running = 0;
    for (size_t i = 0; i < n; ++i) {   // smallest ids first, while under the target share
      const unsigned __int128 next = running + racks[i].second;
      if (next <= target && n - i - 1 >= cfg.min_trainer_racks) {
        running = next;
        ++n_rollout;
      } else {
        break;
      }
    }
    while (n_rollout < cfg.min_rollout_racks && n - n_rollout > cfg.min_trainer_racks) ++n_rollout;
    for (size_t i = 0; i < n; ++i) {
      Rack r;
      r.gpus = racks[i].second;
      r.rollout = i < n_rollout;
      if (r.rollout) r.version = 0;
      order_.push_back(racks[i].first);
      racks_[racks[i].first] = r;
    }
  }

  bool halted() const { return halted_; }
  uint64_t trainer_version() const { return trainer_; }
  uint64_t rack_version(const std::string& id) const {
    const Rack& r = lookup(id);
    if (!r.version) throw Error("NotRollout", "rack is not a rollout rack: " + id);
    return *r.version;
  }
  std::string rack_role(const std::string& id) const { return lookup(id).rollout ? "rollout" : "trainer"; }
  std::pair<uint64_t, uint64_t> split_gpus() const { return {gpu_sum(true), gpu_sum(false)}; }
  size_t n_role(bool rollout) const {
    size_t n = 0;
    for (auto& kv : racks_) n += kv.second.rollout == rollout ? 1 : 0;
    return n;
  }
  size_t queue_depth() const { return queue_.size(); }

  // At most one rack changes side: starved trainers -> more rollout; a backlog -> more
  // trainer; otherwise toward the target GPU share. Minimum rack counts are floors.
  std::optional<std::pair<std::string, std::string>> rebalance() {
    guard();
    const size_t depth = queue_.size();
    if (depth == 0)
      if (auto id = move(false)) return std::make_pair(*id, std::string("rollout"));
    if (cfg_.queue_high > 0 && depth >= cfg_.queue_high)
      if (auto id = move(true)) return std::make_pair(*id, std::string("trainer"));
    const uint64_t ro = gpu_sum(true), tgt = target();
    if (ro < tgt) {
      if (auto id = move(false)) return std::make_pair(*id, std::string("rollout"));
    } else if (ro > tgt) {
      if (auto id = move(true)) return std::make_pair(*id, std::string("trainer"));
    }
    return std::nullopt;
  }
  void enqueue_batch(const RolloutBatch& b) {
    guard();
    if (b.n_samples == 0) throw Error("EmptyGroup", "n_samples must be greater than 0");
    if (b.id.empty()) throw Error("Message", "batch id must be non-empty");
    if (b.prompt_id.empty()) throw Error("Message", "prompt id must be non-empty");
    for (auto& q : queue_)
      if (q.id == b.id) throw Error("DuplicateBatch", "duplicate batch id: " + b.id);
    queue_.push_back(b);
  }
  // Too-stale batches at the head are dropped, then the next one is handed out.
  std::optional<RolloutBatch> consume_batch() {
    guard();
    size_t drop = 0;
    for (auto& b : queue_) {
      if (staleness(trainer_, b.policy_version) > cfg_.max_staleness) ++drop;
      else break;
    }
    for (size_t i = 0; i < drop; ++i) queue_.pop_front();
    if (queue_.empty()) return std::nullopt;
    RolloutBatch b = queue_.front();
    queue_.pop_front();
    return b;
  }
  void publish_weights(uint64_t v) {
    guard();
    if (v != trainer_ + 1) throw Error("NotNextVersion", "policy version must be trainer_version + 1");
    trainer_ = v;
  }
  void sync_rack(const std::string& id, uint64_t v) {
    guard();
    auto it = racks_.find(id);
    if (it == racks_.end()) throw Error("RackNotFound", "rack not found: " + id);
    if (!it->second.rollout) throw Error("NotRollout", "rack is not a rollout rack: " + id);
    if (v != trainer_) throw Error("Unpublished", "policy version " + std::to_string(v) + " was not published");
    it->second.version = v;
  }
  // max |trainer_logp - engine_logp|; above the threshold RL halts and stays halted.
  std::tuple<uint64_t, double, size_t> run_parity(uint64_t v, const std::vector<std::pair<double, double>>& s) {
    guard();
    if (v != trainer_) throw Error("Unpublished", "policy version " + std::to_string(v) + " was not published");
    for (auto& x : s)
      if (!std::isfinite(x.first) || !std::isfinite(x.second)) throw Error("InvalidLogprob", "invalid log-prob");
    double worst = 0.0;
    for (auto& x : s) worst = std::max(worst, std::fabs(x.first - x.second));
    if (worst > cfg_.parity_threshold) {
      halted_ = true;
      throw Error("ParityHalt", "parity drift version=" + std::to_string(v) + " max_abs_err=" + std::to_string(worst) +
                                    " threshold=" + std::to_string(cfg_.parity_threshold));
    }
    return std::make_tuple(v, worst, s.size());
  }

 private:
  void guard() const {
    if (halted_) throw Error("Halted", "RL halted after parity drift");
  }
  const Rack& lookup(const std::string& id) const {
    auto it = racks_.find(id);
    if (it == racks_.end()) throw Error("RackNotFound", "rack not found: " + id);
    return it->second;
  }
  uint64_t gpu_sum(bool rollout) const {
    uint64_t s = 0;
    for (auto& kv : racks_)
      if (kv.second.rollout == rollout) s = s > UINT64_MAX - kv.second.gpus ? UINT64_MAX : s + kv.second.gpus;
    return s;
  }
  uint64_t target() const {
    return static_cast<uint64_t>(static_cast<unsigned __int128>(total_) * cfg_.rollout_numer / cfg_.rollout_denom);
  }
  // move the lexicographically smallest rack of one side to the other
  std::optional<std::string> move(bool from_rollout) {
    if (n_role(from_rollout) <= (from_rollout ? cfg_.min_rollout_racks : cfg_.min_trainer_racks)) return std::nullopt;
    for (auto& id : order_) {
      Rack& r = racks_.at(id);
      if (r.rollout != from_rollout) continue;
      r.rollout = !from_rollout;
      if (r.rollout) r.version = 0;
      else r.version.reset();
      return id;
    }
    return std::nullopt;
  }
  CoordConfig cfg_;
  std::vector<std::string> order_;
  std::map<std::string, Rack> racks_;
  uint64_t trainer_ = 0, total_ = 0;
  bool halted_ = false;
  std::deque<RolloutBatch> queue_;
};

// ----------------------------------------------------------------------------- multiagent
const char* const kTopologies[] = {"single", "orchestrator_subs", "parallel_aggregate", "proposer_solver",
                                   "author_reviewer"};
constexpr uint32_t kDefaultWeights[] = {50, 20, 15, 10, 5};
constexpr uint32_t kMaxSubs = 99;

struct MultiConfig {
  uint32_t w[5] = {50, 20, 15, 10, 5};
  uint32_t keep_numer = 50, keep_denom = 100, default_n_subs = 2;
};

std::string topology_by_weights(uint64_t draw, const uint32_t* w) {
  const uint64_t u = draw % 100;
  uint64_t acc = 0;
  for (int i = 0; i < 5; ++i) {
    acc += w[i];
    if (u < acc) return kTopologies[i];
  }
  throw Error("BadMix", "topology weights must sum to 100");
}

std::string two(uint32_t i) {
  char b[16];
  std::snprintf(b, sizeof b, "%02u", i);
  return b;
}

std::vector<std::pair<std::string, std::string>> roster(const std::string& topo, uint32_t n_subs) {
  std::vector<std::pair<std::string, std::string>> out;
  auto width = [&](bool need) {
    if (need ? !(n_subs >= 1 && n_subs <= kMaxSubs) : n_subs != 0) throw Error("BadWidth", "bad sub-agent count");
  };
  if (topo == "single") {
    width(false);
    out = {{"solo", "solo"}};
  } else if (topo == "orchestrator_subs") {
    width(true);
    out.push_back({"orchestrator", "orchestrator"});
    for (uint32_t i = 0; i < n_subs; ++i) out.push_back({"sub-" + two(i), "sub_agent"});
  } else if (topo == "parallel_aggregate") {
    width(true);
    for (uint32_t i = 0; i < n_subs; ++i) out.push_back({"attempt-" + two(i), "attempt"});
    out.push_back({"aggregator", "aggregator"});
  } else if (topo == "proposer_solver") {
    width(false);
    out = {{"proposer", "proposer"}, {"solver", "solver"}};
  } else if (topo == "author_reviewer") {
    width(false);
    out = {{"author", "author"}, {"reviewer", "reviewer"}};
  } else {
    throw Error("Message", "unknown topology " + topo);
  }
  return out;
}

struct AgentMessage {
  std::string from, to, text;
  std::optional<std::vector<double>> latent_memo;
};

struct Episode {
  std::string topology;
  uint64_t budget = 0, used = 0;
  std::vector<std::pair<std::string, std::string>> roster;
  std::string scratch;
  std::map<std::string, std::vector<AgentMessage>> inboxes;
  std::vector<std::pair<std::string, std::vector<std::string>>> credit;
  std::map<std::string, uint64_t> by;
  bool has(const std::string& a) const {
    for (auto& r : roster)
      if (r.first == a) return true;
    return false;
  }
};

class Multiagent {
 public:
  explicit Multiagent(MultiConfig c) : cfg_(c) {
    uint64_t sum = 0;
    for (uint32_t x : c.w) sum += x;
    if (sum != 100 || c.w[0] < 50 || c.keep_denom == 0 || c.keep_numer > c.keep_denom || c.default_n_subs < 1 ||
        c.default_n_subs > kMaxSubs)
      throw Error("BadMix", "bad topology mix");
  }
  std::string sample_topology(uint64_t draw) const { return topology_by_weights(draw, cfg_.w); }
  std::vector<std::pair<std::string, std::string>> spawn_episode(const std::string& id, const std::string& task,
                                                                 const std::string& topo, uint32_t n_subs,
                                                                 uint64_t budget) {
    if (id.empty() || task.empty()) throw Error("EmptyId", "empty id");
    if (eps_.count(id)) throw Error("DuplicateEpisode", "duplicate episode " + id);
    auto r = roster(topo, n_subs);
    if (budget == 0)
      throw Error("Message", "token_budget must be > 0 (budget parity charges every agent against one cap)");
    Episode e;
    e.topology = topo;
    e.budget = budget;
    e.roster = r;
    for (auto& a : r) {
      e.inboxes[a.first];
      e.by[a.first] = 0;
    }
    eps_[id] = e;
    return r;
  }
  const Episode& ep(const std::string& id) const {
    auto it = eps_.find(id);
    if (it == eps_.end()) throw Error("UnknownEpisode", "unknown episode " + id);
    return it->second;
  }
  Episode& ep(const std::string& id) { return const_cast<Episode&>(static_cast<const Multiagent*>(this)->ep(id)); }
  void scratch_append(const std::string& id, const std::string& agent, const std::string& text) {
    Episode& e = ep(id);
    if (!e.has(agent)) throw Error("UnknownAgent", "unknown agent " + agent);
    e.scratch += text;
  }
  // A latent memo rides along only when keep_draw % denom < numer (dropout, default 50 %).
  AgentMessage send_message(const std::string& id, AgentMessage m, uint64_t keep_draw) {
    Episode& e = ep(id);
    if (!e.has(m.from)) throw Error("UnknownAgent", "unknown agent " + m.from);
    if (!e.has(m.to)) throw Error("UnknownAgent", "unknown agent " + m.to);
    if (m.latent_memo && !(keep_draw % cfg_.keep_denom < cfg_.keep_numer)) m.latent_memo.reset();
    e.inboxes[m.to].push_back(m);
    return m;
  }
  std::vector<AgentMessage> inbox(const std::string& id, const std::string& agent) const {
    const Episode& e = ep(id);
    if (!e.has(agent)) throw Error("UnknownAgent", "unknown agent " + agent);
    return e.inboxes.at(agent);
  }
  void record_credit(const std::string& id, const std::string& parent, const std::vector<std::string>& used) {
    Episode& e = ep(id);
    if (!e.has(parent)) throw Error("UnknownAgent", "unknown agent " + parent);
    for (auto& u : used)
      if (!e.has(u)) throw Error("UnknownAgent", "unknown agent " + u);
    e.credit.push_back({parent, used});
  }
  // One cap for the whole episode: a multi-agent run gets no more tokens than a single agent.
  uint64_t charge_tokens(const std::string& id, const std::string& agent, uint64_t n) {
    Episode& e = ep(id);
    if (!e.has(agent)) throw Error("UnknownAgent", "unknown agent " + agent);
    if (n > UINT64_MAX - e.used || e.used + n > e.budget) throw Error("BudgetExceeded", "token budget exceeded");
    e.used += n;
    e.by[agent] += n;
    return e.used;
  }
  uint64_t tokens_used_by(const std::string& id, const std::string& agent) const {
    const Episode& e = ep(id);
    if (!e.has(agent)) throw Error("UnknownAgent", "unknown agent " + agent);
    return e.by.at(agent);
  }

 private:
  MultiConfig cfg_;
  std::map<std::string, Episode> eps_;
};

}  // namespace

void bind_rl_core(py::module_& m) {
  auto cm = m.def_submodule("coordinator", "asynchronous RL coordinator");
  cm.attr("MAX_STALENESS") = 4;
  cm.attr("GROUP_SIZE") = 16;
  cm.attr("DEFAULT_ROLLOUT_NUMER") = 65;
  cm.attr("DEFAULT_ROLLOUT_DENOM") = 100;
  cm.def("staleness", &staleness);
  py::class_<CoordConfig>(cm, "CoordinatorConfig")
      .def(py::init([](uint64_t ms, uint64_t nu, uint64_t de, double pt, size_t qh, size_t mr, size_t mt) {
             CoordConfig c;
             c.max_staleness = ms;
             c.rollout_numer = nu;
             c.rollout_denom = de;
             c.parity_threshold = pt;
             c.queue_high = qh;
             c.min_rollout_racks = mr;
             c.min_trainer_racks = mt;
             return c;
           }),
           py::arg("max_staleness") = 4, py::arg("rollout_numer") = 65, py::arg("rollout_denom") = 100,
           py::arg("parity_threshold") = 1e-3, py::arg("queue_high") = 8, py::arg("min_rollout_racks") = 1,
           py::arg("min_trainer_racks") = 1);
  py::class_<RolloutBatch>(cm, "RolloutBatch")
      .def(py::init([](std::string id, std::string prompt, uint64_t v, uint32_t n, bool routing) {
             return RolloutBatch{std::move(id), std::move(prompt), v, n, routing};
           }),
           py::arg("id"), py::arg("prompt_id"), py::arg("policy_version"), py::arg("n_samples") = 16,
           py::arg("routing_present") = false)
      .def_readonly("id", &RolloutBatch::id)
      .def_readonly("prompt_id", &RolloutBatch::prompt_id)
      .def_readonly("policy_version", &RolloutBatch::policy_version)
      .def_readonly("n_samples", &RolloutBatch::n_samples)
      .def_readonly("routing_present", &RolloutBatch::routing_present);
  py::class_<Coordinator>(cm, "Coordinator")
      .def(py::init<CoordConfig, std::vector<std::pair<std::string, uint64_t>>>(), py::arg("config"), py::arg("racks"))
      .def("state", [](const Coordinator& c) { return std::string(c.halted() ? "halted" : "running"); })
      .def("halted", &Coordinator::halted)
      .def("trainer_version", &Coordinator::trainer_version)
      .def("rack_version", &Coordinator::rack_version)
      .def("rack_role", &Coordinator::rack_role)
      .def("split_gpus", &Coordinator::split_gpus)
      .def("n_rollout_racks", [](const Coordinator& c) { return c.n_role(true); })
      .def("n_trainer_racks", [](const Coordinator& c) { return c.n_role(false); })
      .def("queue_depth", &Coordinator::queue_depth)
      .def("rebalance", &Coordinator::rebalance)
      .def("enqueue_batch", &Coordinator::enqueue_batch)
      .def("consume_batch", &Coordinator::consume_batch)
      .def("publish_weights", &Coordinator::publish_weights)
      .def("sync_rack", &Coordinator::sync_rack)
      .def("run_parity", &Coordinator::run_parity);

  auto mm = m.def_submodule("multiagent", "multi-agent episode bookkeeping");
  mm.attr("TOPOLOGIES") = std::vector<std::string>(std::begin(kTopologies), std::end(kTopologies));
  mm.attr("MAX_N_SUBS") = kMaxSubs;
  mm.def("topology_weight", [](const std::string& t) {
    for (int i = 0; i < 5; ++i)
      if (t == kTopologies[i]) return kDefaultWeights[i];
    throw Error("Message", "unknown topology " + t);
  });
  mm.def("topology_from_draw", [](uint64_t d) { return topology_by_weights(d, kDefaultWeights); });
  mm.def("roster", &roster);
  py::class_<MultiConfig>(mm, "MultiConfig")
      .def(py::init([](std::vector<uint32_t> w, uint32_t kn, uint32_t kd, uint32_t subs) {
             if (w.size() != 5) throw Error("BadMix", "five weights");
             MultiConfig c;
             for (int i = 0; i < 5; ++i) c.w[i] = w[i];
             c.keep_numer = kn;
             c.keep_denom = kd;
             c.default_n_subs = subs;
             return c;
           }),
           py::arg("weights") = std::vector<uint32_t>{50, 20, 15, 10, 5}, py::arg("latent_keep_numer") = 50,
           py::arg("latent_keep_denom") = 100, py::arg("default_n_subs") = 2);
  py::class_<AgentMessage>(mm, "Message")
      .def(py::init([](std::string f, std::string t, std::string text, std::optional<std::vector<double>> memo) {
             return AgentMessage{std::move(f), std::move(t), std::move(text), std::move(memo)};
           }),
           py::arg("sender"), py::arg("to"), py::arg("text"), py::arg("latent_memo") = py::none())
      .def_readonly("sender", &AgentMessage::from)
      .def_readonly("to", &AgentMessage::to)
      .def_readonly("text", &AgentMessage::text)
      .def_readonly("latent_memo", &AgentMessage::latent_memo);
  py::class_<Multiagent>(mm, "Multiagent")
      .def(py::init<MultiConfig>(), py::arg("config") = MultiConfig{})
      .def("sample_topology", &Multiagent::sample_topology)
      .def("spawn_episode", &Multiagent::spawn_episode, py::arg("id"), py::arg("task"), py::arg("topology"),
           py::arg("n_subs"), py::arg("token_budget"))
      .def("agents", [](const Multiagent& x, const std::string& id) { return x.ep(id).roster; })
      .def("topology_of", [](const Multiagent& x, const std::string& id) { return x.ep(id).topology; })
      .def("scratch_read", [](const Multiagent& x, const std::string& id) { return x.ep(id).scratch; })
      .def("scratch_append", &Multiagent::scratch_append)
      .def("send_message", &Multiagent::send_message)
      .def("inbox", &Multiagent::inbox)
      .def("record_credit", &Multiagent::record_credit)
      .def("credit", [](const Multiagent& x, const std::string& id) { return x.ep(id).credit; })
      .def("charge_tokens", &Multiagent::charge_tokens)
      .def("tokens_used", [](const Multiagent& x, const std::string& id) { return x.ep(id).used; })
      .def("tokens_used_by", &Multiagent::tokens_used_by)
      .def("distill_back", [](const Multiagent&, const std::string& task, uint64_t budget, double multi,
                              double single) -> py::object {
        if (!std::isfinite(multi) || !std::isfinite(single)) throw Error("InvalidReward", "invalid reward");
        if (multi > single) return py::make_tuple(task, budget);
        return py::none();
      });
}
