// Control-plane components on the Raft group:
//
//   raft       bindings of raft.hpp (Cluster, LocalGroup)
//   providers  model-provider transport guards: response validation, AIMD concurrency window,
//              failover with backoff, token broker that commits the refresh token to Raft
//              before it issues an access token
//              (reference: harness/providers/src/lib.rs:98-185, 188-243, 245-344)
//   ops        quorum-signed release roll-out: propose -> shadow -> apply one node at a time ->
//              promote or roll back, with status text / JSON and a tiny CLI
//              (reference: harness/ops/src/lib.rs:26-39, 172-184, 188-508, 525-760)
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cmath>

#include "cas.hpp"
#include "providers.hpp"
#include "raft.hpp"

namespace py = pybind11;
using namespace pbn;
using raft::Cluster;

namespace {

// ------------------------------------------------------------------------------ providers
std::string lower(std::string s) {
  for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  return s;
}

bool args_truncated(const Json& call) {
  const Json* fn = call.is_object() ? call.find("function") : nullptr;
  if (fn == nullptr || !fn->is_object()) return true;
  const Json* a = fn->find("arguments");
  if (a == nullptr || a->is_null()) return true;
  if (a->is_string()) {
    try {
      Json::parse(a->as_string());
      return false;
    } catch (const Error&) {
      return true;
    }
  }
  return !(a->is_object() || a->is_array());
}

bool truncated_tool_call(const Json& choice) {
  if (!choice.is_object()) return false;
  const Json* fr = choice.find("finish_reason");
  if (fr == nullptr || !fr->is_string() || fr->as_string() != "length") return false;
  const Json* tc = choice.find("tool_calls");
  if (tc == nullptr) {
    const Json* msg = choice.find("message");
    if (msg != nullptr && msg->is_object()) tc = msg->find("tool_calls");
  }
  if (tc == nullptr) return false;
  if (!tc->is_array()) return true;
  if (tc->arr().empty()) return false;
  for (const Json& c : tc->arr())
    if (args_truncated(c)) return true;
  return false;
}

// Returns the parsed body, or throws InvalidResponse with `.kind` = the fault name.
Json validate_response(const std::string& body) {
  if (body.size() == 10 && lower(body) == "rate_limit")
    throw Error("RateLimitText", "invalid response: RateLimitText");
  Json v;
  try {
    v = Json::parse(body);
  } catch (const Error&) {
    throw Error("MalformedJson", "invalid response: MalformedJson");
  }
  if (!v.is_object()) throw Error("MalformedJson", "invalid response: MalformedJson");
  if (const Json* e = v.find("error"); e && e->is_string() && lower(e->as_string()) == "rate_limit")
    throw Error("RateLimitText", "invalid response: RateLimitText");
  const Json* ch = v.find("choices");
  if (ch == nullptr || !ch->is_array() || ch->arr().empty())
    throw Error("EmptyCompletion", "invalid response: EmptyCompletion");
  for (const Json& c : ch->arr())
    if (truncated_tool_call(c)) throw Error("TruncatedToolCall", "invalid response: TruncatedToolCall");
  return v;
}

struct AccessToken {
  std::string provider, token;
  uint64_t expires_at = 0;
};

// ------------------------------------------------------------------------------------ ops
struct Signature {
  std::string human, bytes;
};
struct Release {
  std::string version, digest, commit;
  std::vector<Signature> signatures;
  Json to_json() const {
    Json o = Json::object();
    o["version"] = version;
    o["digest"] = digest;
    o["commit"] = commit;
    Json s = Json::array();
    for (auto& g : signatures) {
      Json x = Json::object();
      x["human"] = g.human;
      Json b = Json::array();
      for (unsigned char c : g.bytes) b.arr().push_back(Json(static_cast<uint64_t>(c)));
      x["bytes"] = b;
      s.arr().push_back(x);
    }
    o["signatures"] = s;
    return o;
  }
  static Release from_json(const Json& v) {
    Release r;
    r.version = v.at("version").as_string();
    r.digest = v.at("digest").as_string();
    r.commit = v.at("commit").as_string();
    for (const Json& x : v.at("signatures").arr()) {
      Signature g;
      g.human = x.at("human").as_string();
      for (const Json& b : x.at("bytes").arr()) g.bytes.push_back(static_cast<char>(b.as_u64()));
      r.signatures.push_back(g);
    }
    return r;
  }
};

size_t quorum_count(const Release& r) {
  std::set<std::string> seen;
  for (auto& s : r.signatures)
    if (!s.bytes.empty()) seen.insert(s.human);
  return seen.size();
}

struct NodeStatus {
  std::string id, applied;
  bool healthy = true;
  bool shadow = false;
};

class Ops {
 public:
  static std::unique_ptr<Ops> create(const std::string& dir, size_t quorum) {
    if (::mkdir(dir.c_str(), 0777) != 0) throw Error("Io", dir + ": " + std::strerror(errno));
    auto o = std::unique_ptr<Ops>(new Ops(dir, quorum));
    o->log_ = EventLog::create(dir + "/log");
    return o;
  }
  static std::unique_ptr<Ops> open(const std::string& dir, size_t quorum) {
    auto o = std::unique_ptr<Ops>(new Ops(dir, quorum));
    o->log_ = EventLog::open(dir + "/log");
    for (const LogEvent& e : o->log_->events()) o->apply(e);
    return o;
  }

  void propose(const Release& rel, const std::string& artifact, CasStore& store, uint64_t now) {
    if (!(kind_ == "idle" || kind_ == "refused" || kind_ == "rolled_back" || kind_ == "current"))
      throw wrong("idle|current|refused|rolled_back");
    const std::string got = sha256_hex(artifact);
    if (got != rel.digest) throw Error("DigestMismatch", "digest mismatch: expected " + rel.digest + " got " + got);
    const size_t have = quorum_count(rel);
    if (have < quorum_) {
      Json p = Json::object();
      p["release"] = rel.to_json();
      p["reason"] = "need " + std::to_string(quorum_) + " human signatures, have " + std::to_string(have);
      p["have"] = uint64_t(have);
      p["need"] = uint64_t(quorum_);
      event("ops.refuse", p, now);
      throw Error("NoQuorum", "no quorum: have " + std::to_string(have) + ", need " + std::to_string(quorum_));
    }
    store.put(artifact);
    store.pin(rel.digest, "kernel.shadow");
    event("ops.propose", rel.to_json(), now);
  }
  void start_shadow(CasStore& store, uint64_t now) {
    if (kind_ != "proposed") throw wrong("proposed");
    if (release_) {
      try {
        store.pin(release_->digest, "kernel.shadow");
      } catch (const Error& e) {
        if (e.kind != "DuplicatePin") throw;
      }
    }
    Json p = Json::object();
    p["node"] = "shadow";
    event("ops.shadow", p, now);
  }
  void shadow_pass(uint64_t now) {
    if (kind_ != "shadowing") throw wrong("shadowing");
    Json p = Json::object();
    p["pass"] = true;
    event("ops.shadow_result", p, now);
  }
  void shadow_fail(const std::string& reason, CasStore& store, uint64_t now) {
    if (kind_ != "shadowing") throw wrong("shadowing");
    unpin_quiet(store, "kernel.shadow");
    Json p = Json::object();
    p["pass"] = false;
    p["reason"] = reason;
    event("ops.shadow_result", p, now);
  }
  void apply_one(const std::string& node, uint64_t now) {
    if (!(shadow_passed_ && (kind_ == "shadowing" || kind_ == "rolling"))) throw wrong("shadow_pass");
    live_or_throw(node);
    Json p = Json::object();
    p["node"] = node;
    event("ops.apply", p, now);
  }
  void promote(Cluster& cluster, CasStore& store, uint64_t now) {
    if (!shadow_passed_) throw wrong("shadow_pass");
    if (!all_live_applied()) throw wrong("all live applied and healthy");
    if (!release_) throw wrong("release");
    unpin_quiet(store, "kernel.shadow");
    if (current_digest_) {
      unpin_quiet(store, "kernel.current");
      unpin_quiet(store, "kernel.previous");
      store.pin(*current_digest_, "kernel.previous");
    }
    store.pin(release_->digest, "kernel.current");
    cluster.set_kernel_version(release_->version);
    Json p = Json::object();
    p["version"] = release_->version;
    event("ops.promote", p, now);
  }
  void rollback(const std::string& reason, Cluster& cluster, CasStore& store, uint64_t now) {
    if (!(kind_ == "proposed" || kind_ == "shadowing" || kind_ == "rolling" || kind_ == "current"))
      throw wrong("proposed|shadowing|rolling|current");
    const bool from_current = kind_ == "current";
    unpin_quiet(store, "kernel.shadow");
    if (from_current) {
      unpin_quiet(store, "kernel.current");
      if (previous_digest_) {
        unpin_quiet(store, "kernel.previous");
        store.pin(*previous_digest_, "kernel.current");
      }
      cluster.set_kernel_version(previous_version_);
    }
    Json p = Json::object();
    p["reason"] = reason;
    p["from_current"] = from_current;
    event("ops.rollback", p, now);
  }
  void mark_unhealthy(const std::string& node, const std::string& reason, Cluster& cluster, CasStore& store,
                      uint64_t now) {
    if (!(kind_ == "proposed" || kind_ == "shadowing" || kind_ == "rolling" || kind_ == "current"))
      throw wrong("proposed|shadowing|rolling|current");
    live_or_throw(node);
    Json p = Json::object();
    p["node"] = node;
    p["reason"] = reason;
    event("ops.unhealthy", p, now);
    rollback(reason, cluster, store, now);
  }

  std::string state_name() const {
    if (kind_ == "rolling" || kind_ == "rolled_back" || kind_ == "refused") return kind_ + ":" + detail_;
    return kind_;
  }
  std::vector<NodeStatus> status_nodes(const Cluster& cluster) const {
    const std::string& kv = cluster.state().kernel_version;
    std::vector<NodeStatus> out;
    for (const auto& m : cluster.state().membership) {
      NodeStatus s{m.id, kv, true, false};
      for (const auto& n : nodes_)
        if (!n.shadow && n.id == m.id) {
          s.applied = n.applied;
          s.healthy = n.healthy;
        }
      out.push_back(s);
    }
    for (const auto& n : nodes_)
      if (n.shadow) out.push_back(n);
    return out;
  }
  std::string status_text(const Cluster& cluster) const {
    std::string s = "kernel_version: " + cluster.state().kernel_version + "\nstate: " + state_name() + "\n";
    s += "release: " + (release_ ? release_->version : std::string("none")) + "\nnodes:\n";
    for (const auto& n : status_nodes(cluster))
      s += "  " + n.id + " applied=" + n.applied + " healthy=" + (n.healthy ? "true" : "false") +
           " role=" + (n.shadow ? "shadow" : "live") + "\n";
    return s;
  }
  std::string status_json(const Cluster& cluster) const {
    Json o = Json::object();
    o["kernel_version"] = cluster.state().kernel_version;
    Json ns = Json::array();
    for (const auto& n : status_nodes(cluster)) {
      Json x = Json::object();
      x["id"] = n.id;
      x["applied"] = n.applied;
      x["healthy"] = n.healthy;
      x["role"] = n.shadow ? "shadow" : "live";
      ns.arr().push_back(x);
    }
    o["nodes"] = ns;
    o["release"] = release_ ? release_->to_json() : Json();
    if (kind_ == "rolling") {
      Json in = Json::object(), st = Json::object();
      in["node"] = detail_;
      st["rolling"] = in;
      o["state"] = st;
    } else if (kind_ == "rolled_back" || kind_ == "refused") {
      Json in = Json::object(), st = Json::object();
      in["reason"] = detail_;
      st[kind_] = in;
      o["state"] = st;
    } else {
      o["state"] = kind_;
    }
    return o.dump();
  }
  std::string cli(const std::vector<std::string>& args, const Cluster& cluster) const {
    bool json = false;
    std::optional<std::string> cmd;
    for (const auto& a : args) {
      if (a == "--json") {
        json = true;
        continue;
      }
      if (cmd) throw Error("Other", "unexpected argument " + a);
      cmd = a;
    }
    if (!cmd) throw Error("Other", "missing command");
    if (*cmd != "status") throw Error("Other", "unknown command " + *cmd);
    return json ? status_json(cluster) : status_text(cluster);
  }
  const EventLog& log() const { return *log_; }
  const std::optional<Release>& release() const { return release_; }
  const std::string& kernel_version() const { return kernel_version_; }

 private:
  Ops(std::string dir, size_t quorum) : dir_(std::move(dir)), quorum_(quorum) {
    for (size_t i = 0; i < raft::kMinVoters; ++i) nodes_.push_back({std::to_string(i), "0", true, false});
  }
  Error wrong(const std::string& needed) const {
    return Error("WrongState", "wrong state: current " + state_name() + ", needed " + needed);
  }
  void live_or_throw(const std::string& node) const {
    for (const auto& n : nodes_)
      if (n.id == node) {
        if (n.shadow) throw wrong("live");
        return;
      }
    throw Error("NotFound", "not found: " + node);
  }
  static void unpin_quiet(CasStore& s, const std::string& name) {
    try {
      s.unpin(name);
    } catch (const Error& e) {
      if (e.kind != "NotFound") throw;
    }
  }
  bool all_live_applied() const {
    if (!release_) return false;
    bool any = false;
    for (const auto& n : nodes_)
      if (!n.shadow) {
        any = true;
        if (n.applied != release_->version || !n.healthy) return false;
      }
    return any;
  }
  void event(const char* type, const Json& payload, uint64_t now) {
    LogAppend a;
    a.event_type = type;
    a.payload = payload;
    char ms[8];
    std::snprintf(ms, sizeof ms, "%03u", static_cast<unsigned>(now % 1000));
    a.timestamp = std::to_string(now / 1000) + "." + ms + "Z";
    apply(log_->append(a));
  }
  void drop_shadow() {
    std::vector<NodeStatus> keep;
    for (auto& n : nodes_)
      if (!n.shadow) keep.push_back(n);
    nodes_ = keep;
  }
  void reset_live() {
    for (auto& n : nodes_)
      if (!n.shadow) {
        n.applied = kernel_version_;
        n.healthy = true;
      }
  }
  void rolled_back(const std::string& reason) {
    shadow_passed_ = false;
    drop_shadow();
    reset_live();
    kind_ = "rolled_back";
    detail_ = reason;
  }
  void apply(const LogEvent& e) {
    const std::string& t = e.event_type;
    auto str = [&](const char* k, const char* dflt) {
      const Json* v = e.payload.is_object() ? e.payload.find(k) : nullptr;
      return v && v->is_string() ? v->as_string() : std::string(dflt);
    };
    if (t == "ops.propose") {
      release_ = Release::from_json(e.payload);
      shadow_passed_ = false;
      kind_ = "proposed";
    } else if (t == "ops.refuse") {
      if (const Json* r = e.payload.find("release")) release_ = Release::from_json(*r);
      kind_ = "refused";
      detail_ = str("reason", "no quorum");
    } else if (t == "ops.shadow") {
      bool have = false;
      for (auto& n : nodes_) have = have || n.shadow;
      if (!have) nodes_.push_back({"shadow", release_ ? release_->version : kernel_version_, true, true});
      kind_ = "shadowing";
    } else if (t == "ops.shadow_result") {
      const Json* p = e.payload.find("pass");
      if (p && p->is_bool() && p->as_bool()) shadow_passed_ = true;
      else rolled_back(str("reason", "shadow failed"));
    } else if (t == "ops.apply") {
      const std::string id = str("node", "");
      for (auto& n : nodes_)
        if (!n.shadow && n.id == id) {
          n.applied = release_ ? release_->version : std::string();
          n.healthy = true;
        }
      kind_ = "rolling";
      detail_ = id;
    } else if (t == "ops.promote") {
      if (release_) {
        previous_version_ = kernel_version_;
        kernel_version_ = release_->version;
        if (current_digest_) previous_digest_ = current_digest_;
        current_digest_ = release_->digest;
      }
      drop_shadow();
      shadow_passed_ = false;
      kind_ = "current";
    } else if (t == "ops.rollback") {
      const Json* fc = e.payload.find("from_current");
      const bool from_current = fc && fc->is_bool() ? fc->as_bool() : kind_ == "current";
      if (from_current) {
        current_digest_ = previous_digest_;
        previous_digest_.reset();
        kernel_version_ = previous_version_;
      }
      rolled_back(str("reason", "rollback"));
    } else if (t == "ops.unhealthy") {
      const std::string id = str("node", "");
      for (auto& n : nodes_)
        if (!n.shadow && n.id == id) n.healthy = false;
    }
  }

  std::string dir_;
  size_t quorum_;
  std::unique_ptr<EventLog> log_;
  std::string kind_ = "idle", detail_;
  std::optional<Release> release_;
  std::vector<NodeStatus> nodes_;
  bool shadow_passed_ = false;
  std::string kernel_version_ = "0", previous_version_ = "0";
  std::optional<std::string> current_digest_, previous_digest_;
};

py::dict lease_dict(const raft::RoleLease& l) {
  py::dict d;
  d["role"] = raft::role_name(l.role);
  d["holder"] = l.holder;
  d["attempt"] = l.attempt;
  d["expires_at"] = l.expires_at;
  return d;
}
raft::Role role_of(const std::string& s) {
  if (s == "coordinator") return raft::Role::Coordinator;
  if (s == "token_broker") return raft::Role::TokenBroker;
  throw Error("Other", "unknown role " + s);
}

}  // namespace

void bind_harness_control(py::module_& m) {
  using namespace raft;
  auto rm = m.def_submodule("raft", "in-process Raft control plane");
  rm.attr("MIN_VOTERS") = kMinVoters;
  py::class_<ClusterConfig>(rm, "ClusterConfig")
      .def(py::init([](uint64_t p, uint32_t mh) {
             ClusterConfig c;
             c.heartbeat_period_ms = p;
             c.missed_heartbeats = mh;
             return c;
           }),
           py::arg("heartbeat_period_ms") = 15000, py::arg("missed_heartbeats") = 2)
      .def("lease_ttl_ms", &ClusterConfig::lease_ttl_ms);
  py::class_<NodeInfo>(rm, "NodeInfo")
      .def(py::init([](std::string id, std::string addr, bool always_on, bool trusted) {
             return NodeInfo{std::move(id), std::move(addr), always_on, trusted};
           }),
           py::arg("id"), py::arg("addr") = "", py::arg("always_on") = true, py::arg("trusted") = true)
      .def_readonly("id", &NodeInfo::id)
      .def_readonly("addr", &NodeInfo::addr)
      .def_readonly("always_on", &NodeInfo::always_on)
      .def_readonly("trusted", &NodeInfo::trusted);
  py::class_<Cluster, std::shared_ptr<Cluster>>(rm, "Cluster")
      .def_static("bootstrap", [](const std::string& d, const NodeInfo& n, ClusterConfig c) {
                    return Cluster::bootstrap(d, n, c);
                  }, py::arg("dir"), py::arg("this"), py::arg("config") = ClusterConfig{})
      .def_static("open", [](const std::string& d, const std::string& id, ClusterConfig c) {
                    return Cluster::open(d, id, c);
                  }, py::arg("dir"), py::arg("this_id"), py::arg("config") = ClusterConfig{})
      .def("is_leader", &Cluster::is_leader)
      .def_property_readonly("this_id", &Cluster::this_id)
      .def_property_readonly("term", &Cluster::term)
      .def_property_readonly("log_len", &Cluster::log_len)
      .def("add_voter", &Cluster::add_voter)
      .def("add_worker", &Cluster::add_worker)
      .def("remove_node", &Cluster::remove_node)
      .def("claim_role", [](Cluster& c, const std::string& role, const std::string& node, uint64_t now) {
        return lease_dict(c.claim_role(role_of(role), node, now));
      })
      .def("heartbeat_role", [](Cluster& c, const std::string& role, const std::string& node, uint64_t now) {
        return lease_dict(c.heartbeat_role(role_of(role), node, now));
      })
      .def("expire_roles", [](Cluster& c, uint64_t now) {
        std::vector<std::string> out;
        for (Role r : c.expire_roles(now)) out.push_back(role_name(r));
        return out;
      })
      .def("commit_token", [](Cluster& c, py::bytes blob) {
        const TokenRecord t = c.commit_token(std::string(blob));
        return py::make_tuple(t.generation, py::bytes(t.blob));
      })
      .def("set_kernel_version", &Cluster::set_kernel_version)
      .def("state", [](const Cluster& c) {
        const ControlState& s = c.state();
        py::dict d;
        py::list mem;
        for (auto& mbr : s.membership) mem.append(py::cast(mbr));
        d["membership"] = mem;
        d["coordinator"] = s.coordinator ? py::object(lease_dict(*s.coordinator)) : py::none();
        d["token_broker"] = s.token_broker ? py::object(lease_dict(*s.token_broker)) : py::none();
        d["kernel_version"] = s.kernel_version;
        d["token"] = s.token ? py::object(py::make_tuple(s.token->generation, py::bytes(s.token->blob))) : py::none();
        return d;
      });
  py::class_<LocalGroup>(rm, "LocalGroup")
      .def_static("start", [](size_t n, const std::string& base, ClusterConfig c) {
                    return std::make_unique<LocalGroup>(n, base, c);
                  }, py::arg("n"), py::arg("base_dir"), py::arg("config") = ClusterConfig{})
      .def("__len__", &LocalGroup::size)
      .def("get", &LocalGroup::get)
      .def("partition", &LocalGroup::partition)
      .def("heal", &LocalGroup::heal)
      .def("crash", &LocalGroup::crash)
      .def("restart", &LocalGroup::restart)
      .def("tick", &LocalGroup::tick)
      .def("leader", &LocalGroup::leader);

  auto pm = m.def_submodule("providers", "provider transport guards, AIMD, failover, token broker");
  pm.def("validate_response", [](py::bytes body) { return validate_response(std::string(body)).dump(); });
  py::class_<AimdConfig>(pm, "AimdConfig")
      .def(py::init([](uint32_t mn, uint32_t mx, uint32_t inc, double dec, uint64_t lat) {
             return AimdConfig{mn, mx, inc, dec, lat};
           }),
           py::arg("min_window") = 1, py::arg("max_window") = 32, py::arg("increase") = 1,
           py::arg("decrease") = 0.5, py::arg("latency_limit_ms") = 30000);
  py::class_<Aimd>(pm, "Aimd")
      .def(py::init<AimdConfig>(), py::arg("config") = AimdConfig{})
      .def_property_readonly("window", &Aimd::window)
      .def("on_success", &Aimd::on_success)
      .def("on_429", &Aimd::on_429)
      .def("on_outage", &Aimd::on_outage);
  py::class_<Failover>(pm, "Failover")
      .def(py::init<std::vector<std::string>>())
      .def("current", &Failover::current)
      .def("mark_down", &Failover::mark_down)
      .def("mark_up", &Failover::mark_up)
      .def("wait_backoff_ms", &Failover::wait_backoff_ms)
      .def_property_readonly("providers", &Failover::providers)
      .def_property_readonly("down", &Failover::down);
  py::class_<AccessToken>(pm, "AccessToken")
      .def_readonly("provider", &AccessToken::provider)
      .def_readonly("token", &AccessToken::token)
      .def_readonly("expires_at", &AccessToken::expires_at);
  // The refresh blob is committed to the Raft log before the access token exists, so a
  // broker that dies right after issuing never strands a token nobody else can refresh.
  pm.def("broker_refresh", [](Cluster& cluster, const std::string& provider, uint64_t access_ttl_ms,
                              py::bytes refresh_blob, uint64_t now) {
    if (!cluster.is_leader()) throw Error("NotBroker", "not the token broker");
    const std::string blob = refresh_blob;
    TokenRecord rec;
    try {
      rec = cluster.commit_token(blob);
    } catch (const Error& e) {
      throw Error("Raft", e.what());
    }
    AccessToken t{provider, sha256_hex(blob), now > UINT64_MAX - access_ttl_ms ? UINT64_MAX : now + access_ttl_ms};
    return py::make_tuple(py::make_tuple(rec.generation, py::bytes(rec.blob)), t);
  }, py::arg("cluster"), py::arg("provider"), py::arg("access_ttl_ms"), py::arg("refresh_blob"), py::arg("now"));

  auto om = m.def_submodule("ops", "quorum-signed release roll-out");
  om.attr("DEFAULT_QUORUM") = 2;
  om.attr("PIN_CURRENT") = "kernel.current";
  om.attr("PIN_PREVIOUS") = "kernel.previous";
  om.attr("PIN_SHADOW") = "kernel.shadow";
  py::class_<Release>(om, "Release")
      .def(py::init([](std::string version, std::string digest, std::string commit,
                       std::vector<std::pair<std::string, py::bytes>> sigs) {
             Release r{std::move(version), std::move(digest), std::move(commit), {}};
             for (auto& s : sigs) r.signatures.push_back({s.first, std::string(s.second)});
             return r;
           }),
           py::arg("version"), py::arg("digest"), py::arg("commit"), py::arg("signatures"))
      .def_readonly("version", &Release::version)
      .def_readonly("digest", &Release::digest);
  om.def("has_quorum", [](const Release& r, size_t q) { return quorum_count(r) >= q; }, py::arg("release"),
         py::arg("quorum") = 2);
  py::class_<Ops>(om, "Ops")
      .def_static("create", &Ops::create, py::arg("dir"), py::arg("quorum") = 2)
      .def_static("open", &Ops::open, py::arg("dir"), py::arg("quorum") = 2)
      .def("propose", [](Ops& o, const Release& r, py::bytes art, CasStore& s, uint64_t now) {
        o.propose(r, std::string(art), s, now);
      })
      .def("start_shadow", &Ops::start_shadow)
      .def("shadow_pass", &Ops::shadow_pass)
      .def("shadow_fail", &Ops::shadow_fail)
      .def("apply_one", &Ops::apply_one)
      .def("promote", &Ops::promote)
      .def("rollback", &Ops::rollback)
      .def("mark_unhealthy", &Ops::mark_unhealthy)
      .def_property_readonly("state", &Ops::state_name)
      .def_property_readonly("kernel_version", &Ops::kernel_version)
      .def("status_text", &Ops::status_text)
      .def("status_json", &Ops::status_json)
      .def("cli", &Ops::cli)
      .def("event_types", [](const Ops& o) {
        std::vector<std::string> out;
        for (const LogEvent& e : o.log().events()) out.push_back(e.event_type);
        return out;
      });
}
