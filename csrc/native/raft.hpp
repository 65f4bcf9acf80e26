// In-process Raft control plane: replicated log, terms and votes, apply on commit, a
// partitionable message bus, and the control state it guards (membership, the Coordinator and
// TokenBroker role leases, the committed refresh token, the kernel version).
//
// Behavioural contract of the reference's harness/raft crate (harness/raft/src/lib.rs:23-27,
// 131-402; harness/raft/src/inner.rs:84-350, 438-960): mutations are accepted only by the
// leader and only while it reaches a majority of the voters; ephemeral workers never vote;
// at least three voters once the group has ever had three; every node persists its term, vote,
// log and applied state to <dir>/state.json by write-to-temp + rename; a restarted node comes
// back as a follower; isolated nodes receive neither votes nor entries.
#pragma once

#include <map>
#include <set>

#include "common.hpp"

namespace pbn {
namespace raft {

constexpr size_t kMinVoters = 3;

struct NodeInfo {
  std::string id, addr;
  bool always_on = true;   // kind: always_on | ephemeral
  bool trusted = true;
  Json to_json() const {
    Json o = Json::object();
    o["id"] = id;
    o["addr"] = addr;
    o["kind"] = always_on ? "always_on" : "ephemeral";
    o["trusted"] = trusted;
    return o;
  }
  static NodeInfo from_json(const Json& v) {
    return {v.at("id").as_string(), v.at("addr").as_string(), v.at("kind").as_string() == "always_on",
            v.at("trusted").as_bool()};
  }
};

enum class Role { Coordinator, TokenBroker };
inline const char* role_name(Role r) { return r == Role::Coordinator ? "coordinator" : "token_broker"; }

struct RoleLease {
  Role role = Role::Coordinator;
  std::string holder;
  uint64_t attempt = 0, expires_at = 0;
  Json to_json() const {
    Json o = Json::object();
    o["role"] = role_name(role);
    o["holder"] = holder;
    o["attempt"] = attempt;
    o["expires_at"] = expires_at;
    return o;
  }
  static RoleLease from_json(const Json& v) {
    RoleLease l;
    l.role = v.at("role").as_string() == "coordinator" ? Role::Coordinator : Role::TokenBroker;
    l.holder = v.at("holder").as_string();
    l.attempt = v.at("attempt").as_u64();
    l.expires_at = v.at("expires_at").as_u64();
    return l;
  }
};

struct TokenRecord {
  uint64_t generation = 0;
  std::string blob;
};

struct ControlState {
  std::vector<NodeInfo> membership;
  std::optional<RoleLease> coordinator, token_broker;
  std::string kernel_version = "0";   // a fresh group runs kernel "0" until a release is committed
  std::optional<TokenRecord> token;
};

struct ClusterConfig {
  uint64_t heartbeat_period_ms = 15000;
  uint32_t missed_heartbeats = 2;
  uint64_t lease_ttl_ms() const {
    const unsigned __int128 p = static_cast<unsigned __int128>(heartbeat_period_ms) *
                                (missed_heartbeats < 1 ? 1 : missed_heartbeats);
    return p > UINT64_MAX ? UINT64_MAX : static_cast<uint64_t>(p);
  }
};

// A replicated command, kept as JSON so the log persists as written.
struct Entry {
  uint64_t term = 0;
  Json cmd;
};

struct Machine {
  ControlState st;
  uint64_t coord_attempt = 0, broker_attempt = 0;
  bool ever_min = false;

  size_t voters() const {
    size_t n = 0;
    for (auto& m : st.membership) n += m.always_on ? 1 : 0;
    return n;
  }
  bool is_voter(const std::string& id) const {
    for (auto& m : st.membership)
      if (m.id == id && m.always_on) return true;
    return false;
  }
  const NodeInfo* find(const std::string& id) const {
    for (auto& m : st.membership)
      if (m.id == id) return &m;
    return nullptr;
  }
  std::optional<RoleLease>& slot(Role r) { return r == Role::Coordinator ? st.coordinator : st.token_broker; }
  const std::optional<RoleLease>& slot(Role r) const {
    return r == Role::Coordinator ? st.coordinator : st.token_broker;
  }

  void apply(const Json& c) {
    const std::string op = c.at("op").as_string();
    if (op == "add_voter" || op == "add_worker") {
      const NodeInfo n = NodeInfo::from_json(c.at("node"));
      if (find(n.id) == nullptr) {
        st.membership.push_back(n);
        if (op == "add_voter" && voters() >= kMinVoters) ever_min = true;
      }
    } else if (op == "remove_node") {
      const std::string id = c.at("id").as_string();
      std::vector<NodeInfo> keep;
      for (auto& m : st.membership)
        if (m.id != id) keep.push_back(m);
      st.membership = keep;
      if (st.coordinator && st.coordinator->holder == id) st.coordinator.reset();
      if (st.token_broker && st.token_broker->holder == id) st.token_broker.reset();
    } else if (op == "claim_role") {
      const RoleLease l = RoleLease::from_json(c.at("lease"));
      slot(l.role) = l;
      coord_attempt = c.at("coord_attempt").as_u64();
      broker_attempt = c.at("broker_attempt").as_u64();
    } else if (op == "heartbeat_role") {
      const RoleLease l = RoleLease::from_json(c.at("lease"));
      slot(l.role) = l;
    } else if (op == "expire_roles") {
      auto get = [&](const char* k) -> std::optional<RoleLease> {
        const Json& v = c.at(k);
        if (v.is_null()) return std::nullopt;
        return RoleLease::from_json(v);
      };
      st.coordinator = get("coordinator");
      st.token_broker = get("token_broker");
    } else if (op == "commit_token") {
      TokenRecord t;
      t.generation = c.at("generation").as_u64();
      for (const Json& b : c.at("blob").arr()) t.blob.push_back(static_cast<char>(b.as_u64()));
      st.token = t;
    } else if (op == "set_kernel") {
      st.kernel_version = c.at("version").as_string();
    }
  }

  Json snapshot() const {
    Json o = Json::object();
    Json mem = Json::array();
    for (auto& m : st.membership) mem.arr().push_back(m.to_json());
    o["membership"] = mem;
    o["coordinator"] = st.coordinator ? st.coordinator->to_json() : Json();
    o["token_broker"] = st.token_broker ? st.token_broker->to_json() : Json();
    o["kernel_version"] = st.kernel_version;
    if (st.token) {
      Json t = Json::object();
      t["generation"] = st.token->generation;
      Json b = Json::array();
      for (unsigned char c : st.token->blob) b.arr().push_back(Json(static_cast<uint64_t>(c)));
      t["blob"] = b;
      o["token"] = t;
    } else {
      o["token"] = Json();
    }
    o["coord_attempt"] = coord_attempt;
    o["broker_attempt"] = broker_attempt;
    o["ever_reached_min_voters"] = ever_min;
    return o;
  }
  void restore(const Json& o) {
    st = ControlState{};
    for (const Json& m : o.at("membership").arr()) st.membership.push_back(NodeInfo::from_json(m));
    if (!o.at("coordinator").is_null()) st.coordinator = RoleLease::from_json(o.at("coordinator"));
    if (!o.at("token_broker").is_null()) st.token_broker = RoleLease::from_json(o.at("token_broker"));
    st.kernel_version = o.at("kernel_version").as_string();
    if (!o.at("token").is_null()) {
      TokenRecord t;
      t.generation = o.at("token").at("generation").as_u64();
      for (const Json& b : o.at("token").at("blob").arr()) t.blob.push_back(static_cast<char>(b.as_u64()));
      st.token = t;
    }
    coord_attempt = o.at("coord_attempt").as_u64();
    broker_attempt = o.at("broker_attempt").as_u64();
    ever_min = o.at("ever_reached_min_voters").as_bool();
  }
};

struct Node {
  std::string dir, id;
  ClusterConfig cfg;
  uint64_t term = 0;
  std::optional<std::string> voted_for;
  std::vector<Entry> log;
  uint64_t commit = 0, applied = 0;
  bool leader = false;
  Machine m;

  uint64_t last_index() const { return log.size(); }
  uint64_t last_term() const { return log.empty() ? 0 : log.back().term; }

  void persist() const {
    Json o = m.snapshot();
    o["current_term"] = term;
    o["voted_for"] = voted_for ? Json(*voted_for) : Json();
    Json l = Json::array();
    for (auto& e : log) {
      Json x = Json::object();
      x["term"] = e.term;
      x["cmd"] = e.cmd;
      l.arr().push_back(x);
    }
    o["log"] = l;
    o["commit_index"] = commit;
    o["last_applied"] = applied;
    const std::string text = o.dump_pretty();
    const std::string tmp = dir + "/state.json.tmp", path = dir + "/state.json";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (f == nullptr) throw Error("Other", tmp + ": " + std::strerror(errno));
    const bool ok = std::fwrite(text.data(), 1, text.size(), f) == text.size();
    std::fclose(f);
    if (!ok || ::rename(tmp.c_str(), path.c_str()) != 0) throw Error("Other", "persist failed: " + path);
  }
  static Node load(const std::string& dir, const std::string& id, ClusterConfig cfg) {
    if (!dir_exists(dir)) throw Error("Other", "open missing dir: " + dir);
    Json o;
    try {
      o = Json::parse(read_file(dir + "/state.json"));
    } catch (const Error& e) {
      throw Error("Other", e.what());
    }
    Node n;
    n.dir = dir;
    n.id = id;
    n.cfg = cfg;
    n.term = o.at("current_term").as_u64();
    if (!o.at("voted_for").is_null()) n.voted_for = o.at("voted_for").as_string();
    for (const Json& e : o.at("log").arr()) n.log.push_back({e.at("term").as_u64(), e.at("cmd")});
    n.applied = o.at("last_applied").as_u64();
    n.commit = std::min(o.at("commit_index").as_u64(), n.applied);
    n.leader = false;
    n.m.restore(o);
    return n;
  }
  void apply_committed() {
    while (applied < commit) {
      m.apply(log[applied].cmd);
      ++applied;
    }
  }
};

// The shared medium of one process: all live nodes and who is cut off.
struct Bus {
  std::map<std::string, Node> nodes;
  std::set<std::string> isolated;

  std::vector<std::string> reachable(const std::string& from) const {
    if (!nodes.count(from)) return {};
    if (isolated.count(from)) return {from};
    std::vector<std::string> out;
    for (auto& kv : nodes)
      if (!isolated.count(kv.first)) out.push_back(kv.first);
    return out;
  }
  bool has_majority(const std::string& from) const {
    auto it = nodes.find(from);
    if (it == nodes.end()) return false;
    const size_t total = it->second.m.voters();
    if (total == 0) return false;
    size_t acks = 0;
    for (auto& id : reachable(from)) acks += it->second.m.is_voter(id) ? 1 : 0;
    return acks * 2 > total;
  }
  bool is_leader(const std::string& id) const {
    auto it = nodes.find(id);
    return it != nodes.end() && it->second.leader;
  }
  void gate(const std::string& id) const {
    if (!is_leader(id) || !has_majority(id)) throw Error("NotLeader", "not leader");
  }

  static void install(Node& peer, const std::vector<Entry>& lead) {
    size_t i = 0;
    while (i < peer.log.size() && i < lead.size() && peer.log[i].term == lead[i].term) ++i;
    if (i < peer.log.size()) {
      peer.log.resize(i);
      peer.commit = std::min<uint64_t>(peer.commit, i);
      peer.applied = std::min<uint64_t>(peer.applied, i);
    }
    for (; i < lead.size(); ++i) peer.log.push_back(lead[i]);
  }

  void replicate(const std::string& lid) {
    auto it = nodes.find(lid);
    if (it == nodes.end() || !it->second.leader) return;
    const std::vector<Entry> llog = it->second.log;
    const uint64_t lterm = it->second.term, last = it->second.last_index();
    const size_t total = it->second.m.voters();
    std::set<std::string> voters;
    for (auto& mb : it->second.m.st.membership)
      if (mb.always_on) voters.insert(mb.id);
    const auto reach = reachable(lid);
    for (auto& pid : reach) {
      if (pid == lid) continue;
      Node& p = nodes.at(pid);
      if (lterm < p.term) continue;
      p.term = lterm;
      p.voted_for = lid;
      p.leader = false;
      install(p, llog);
    }
    size_t acks = 0;
    for (auto& pid : reach)
      if (nodes.at(pid).log.size() >= last && voters.count(pid)) ++acks;
    if (total > 0 && acks * 2 > total) nodes.at(lid).commit = last;
    const uint64_t commit = nodes.at(lid).commit;
    for (auto& pid : reach) {
      Node& n = nodes.at(pid);
      n.commit = std::max<uint64_t>(n.commit, std::min<uint64_t>(commit, n.log.size()));
      n.apply_committed();
      n.persist();
    }
  }

  void append_commit(const std::string& lid, const Json& cmd) {
    gate(lid);
    Node& l = nodes.at(lid);
    l.log.push_back({l.term, cmd});
    replicate(lid);
    if (nodes.at(lid).applied < nodes.at(lid).last_index()) throw Error("NotLeader", "not leader");
  }

  void elect() {
    for (auto& kv : nodes)
      if (isolated.count(kv.first)) kv.second.leader = false;
    std::vector<std::string> conn;
    for (auto& kv : nodes)
      if (!isolated.count(kv.first)) conn.push_back(kv.first);
    if (conn.empty()) return;
    // most complete log wins; ties go to the smallest id
    auto better = [&](const std::string& a, const std::string& b) {
      const Node &x = nodes.at(a), &y = nodes.at(b);
      if (x.last_term() != y.last_term()) return x.last_term() > y.last_term();
      if (x.last_index() != y.last_index()) return x.last_index() > y.last_index();
      return a < b;
    };
    std::string best = conn[0];
    for (auto& id : conn)
      if (better(id, best)) best = id;
    const Machine& view = nodes.at(best).m;
    const size_t total = view.voters();
    std::vector<std::string> cv;
    for (auto& id : conn)
      if (view.is_voter(id)) cv.push_back(id);
    if (total == 0 || cv.size() * 2 <= total) {
      for (auto& id : conn) nodes.at(id).leader = false;
      return;
    }
    for (auto& id : cv)
      if (nodes.at(id).leader) {          // a sitting leader among the majority stays
        for (auto& o : conn)
          if (o != id) nodes.at(o).leader = false;
        return;
      }
    std::string win = cv[0];
    for (auto& id : cv)
      if (better(id, win)) win = id;
    uint64_t t = 0;
    for (auto& id : conn) t = std::max(t, nodes.at(id).term);
    t = t == UINT64_MAX ? t : t + 1;
    for (auto& id : conn) {
      Node& n = nodes.at(id);
      n.term = t;
      n.voted_for = win;
      n.leader = id == win;
      n.persist();
    }
  }

  std::vector<Role> expire_roles(const std::string& from, uint64_t now) {
    gate(from);
    const Machine& m = nodes.at(from).m;
    std::vector<Role> dropped;
    auto c = m.st.coordinator;
    auto b = m.st.token_broker;
    if (c && c->expires_at <= now) {
      c.reset();
      dropped.push_back(Role::Coordinator);
    }
    if (b && b->expires_at <= now) {
      b.reset();
      dropped.push_back(Role::TokenBroker);
    }
    if (dropped.empty()) return dropped;
    Json cmd = Json::object();
    cmd["op"] = "expire_roles";
    cmd["coordinator"] = c ? c->to_json() : Json();
    cmd["token_broker"] = b ? b->to_json() : Json();
    append_commit(from, cmd);
    return dropped;
  }

  void tick(uint64_t now) {
    elect();
    std::vector<std::string> leaders;
    for (auto& kv : nodes)
      if (kv.second.leader) leaders.push_back(kv.first);
    for (auto& lid : leaders) {
      if (isolated.count(lid)) continue;
      replicate(lid);
      if (has_majority(lid)) expire_roles(lid, now);
    }
  }
};

// One node's handle on the group.
class Cluster {
 public:
  Cluster(std::shared_ptr<Bus> bus, std::string id) : bus_(std::move(bus)), id_(std::move(id)) {}

  static std::shared_ptr<Cluster> bootstrap(const std::string& dir, const NodeInfo& self, ClusterConfig cfg) {
    if (!self.always_on) throw Error("EphemeralVoter", "ephemeral node " + self.id + " cannot be a voter");
    if (!self.trusted) throw Error("Untrusted", "untrusted node " + self.id);
    if (file_exists(dir) || dir_exists(dir)) throw Error("Other", "bootstrap dir exists: " + dir);
    make_dirs(dir);
    Node n;
    n.dir = dir;
    n.id = self.id;
    n.cfg = cfg;
    n.term = 1;
    n.voted_for = self.id;
    n.leader = true;
    n.m.st.membership.push_back(self);
    n.persist();
    auto bus = std::make_shared<Bus>();
    bus->nodes[self.id] = n;
    return std::make_shared<Cluster>(bus, self.id);
  }
  static std::shared_ptr<Cluster> open(const std::string& dir, const std::string& id, ClusterConfig cfg,
                                       std::shared_ptr<Bus> bus = nullptr) {
    if (!bus) bus = std::make_shared<Bus>();
    bus->nodes[id] = Node::load(dir, id, cfg);
    return std::make_shared<Cluster>(bus, id);
  }

  const ControlState& state() const { return node().m.st; }
  bool is_leader() const { return bus_->is_leader(id_); }
  const std::string& this_id() const { return id_; }
  uint64_t term() const { return node().term; }
  size_t log_len() const { return node().log.size(); }

  void add_voter(const NodeInfo& n) {
    bus_->gate(id_);
    const Machine& m = node().m;
    if (m.find(n.id)) throw Error("Duplicate", "duplicate node " + n.id);
    if (!n.always_on) throw Error("EphemeralVoter", "ephemeral node " + n.id + " cannot be a voter");
    if (!n.trusted) throw Error("Untrusted", "untrusted node " + n.id);
    Json c = Json::object();
    c["op"] = "add_voter";
    c["node"] = n.to_json();
    bus_->append_commit(id_, c);
  }
  void add_worker(const NodeInfo& n) {
    bus_->gate(id_);
    if (node().m.find(n.id)) throw Error("Duplicate", "duplicate node " + n.id);
    if (n.always_on) throw Error("Other", "always-on node " + n.id + " must use add_voter");
    Json c = Json::object();
    c["op"] = "add_worker";
    c["node"] = n.to_json();
    bus_->append_commit(id_, c);
  }
  void remove_node(const std::string& id) {
    bus_->gate(id_);
    const Machine& m = node().m;
    const NodeInfo* n = m.find(id);
    if (n == nullptr) throw Error("NotFound", "not found: " + id);
    if (n->always_on) {
      const size_t would = m.voters() - 1;
      if (m.ever_min && would < kMinVoters)
        throw Error("TooFewVoters", "need at least 3 voters, have " + std::to_string(would));
      if (would < 1) throw Error("TooFewVoters", "need at least 3 voters, have 0");
    }
    Json c = Json::object();
    c["op"] = "remove_node";
    c["id"] = id;
    bus_->append_commit(id_, c);
  }
  RoleLease claim_role(Role role, const std::string& who, uint64_t now) {
    bus_->gate(id_);
    const Machine& m = node().m;
    const NodeInfo* n = m.find(who);
    if (n == nullptr) throw Error("NotFound", "not found: " + who);
    if (!n->trusted) throw Error("Untrusted", "untrusted node " + who);
    const auto& cur = m.slot(role);
    if (cur && cur->expires_at > now)
      throw Error("NotClaimable", std::string("role not claimable: ") + role_name(role));
    const uint64_t ca = m.coord_attempt + (role == Role::Coordinator ? 1 : 0);
    const uint64_t ba = m.broker_attempt + (role == Role::TokenBroker ? 1 : 0);
    RoleLease l;
    l.role = role;
    l.holder = who;
    l.attempt = role == Role::Coordinator ? ca : ba;
    const uint64_t ttl = node().cfg.lease_ttl_ms();
    l.expires_at = now > UINT64_MAX - ttl ? UINT64_MAX : now + ttl;
    Json c = Json::object();
    c["op"] = "claim_role";
    c["lease"] = l.to_json();
    c["coord_attempt"] = ca;
    c["broker_attempt"] = ba;
    bus_->append_commit(id_, c);
    return l;
  }
  RoleLease heartbeat_role(Role role, const std::string& who, uint64_t now) {
    bus_->gate(id_);
    const auto& cur = node().m.slot(role);
    if (!cur || cur->holder != who)
      throw Error("NotHolder", std::string("not holder: role=") + role_name(role) + " node=" + who);
    RoleLease l = *cur;
    const uint64_t ttl = node().cfg.lease_ttl_ms();
    l.expires_at = now > UINT64_MAX - ttl ? UINT64_MAX : now + ttl;
    Json c = Json::object();
    c["op"] = "heartbeat_role";
    c["lease"] = l.to_json();
    bus_->append_commit(id_, c);
    return l;
  }
  std::vector<Role> expire_roles(uint64_t now) { return bus_->expire_roles(id_, now); }
  TokenRecord commit_token(const std::string& blob) {
    bus_->gate(id_);
    TokenRecord t;
    t.generation = (node().m.st.token ? node().m.st.token->generation : 0) + 1;
    t.blob = blob;
    Json c = Json::object();
    c["op"] = "commit_token";
    c["generation"] = t.generation;
    Json b = Json::array();
    for (unsigned char ch : blob) b.arr().push_back(Json(static_cast<uint64_t>(ch)));
    c["blob"] = b;
    bus_->append_commit(id_, c);
    return t;
  }
  void set_kernel_version(const std::string& v) {
    bus_->gate(id_);
    Json c = Json::object();
    c["op"] = "set_kernel";
    c["version"] = v;
    bus_->append_commit(id_, c);
  }
  std::shared_ptr<Bus> bus() const { return bus_; }

 private:
  const Node& node() const {
    auto it = bus_->nodes.find(id_);
    if (it == bus_->nodes.end()) throw Error("NotFound", "not found: " + id_);
    return it->second;
  }
  std::shared_ptr<Bus> bus_;
  std::string id_;
};

// N always-on voters "0".."n-1" on one bus, with partition / heal / crash / restart / tick.
class LocalGroup {
 public:
  LocalGroup(size_t n, const std::string& base, ClusterConfig cfg) : base_(base), cfg_(cfg) {
    if (n < kMinVoters) throw Error("TooFewVoters", "need at least 3 voters, have " + std::to_string(n));
    std::vector<NodeInfo> members;
    for (size_t i = 0; i < n; ++i) members.push_back({std::to_string(i), "local://" + std::to_string(i), true, true});
    bus_ = std::make_shared<Bus>();
    for (size_t i = 0; i < n; ++i) {
      const std::string dir = base + "/" + std::to_string(i);
      if (file_exists(dir) || dir_exists(dir)) throw Error("Other", "start dir exists: " + dir);
      make_dirs(dir);
      Node node;
      node.dir = dir;
      node.id = members[i].id;
      node.cfg = cfg;
      node.m.st.membership = members;
      node.m.ever_min = n >= kMinVoters;
      node.persist();
      bus_->nodes[node.id] = node;
      nodes_.push_back(std::make_shared<Cluster>(bus_, node.id));
    }
    isolated_.assign(n, false);
  }
  size_t size() const { return nodes_.size(); }
  std::shared_ptr<Cluster> get(size_t i) {
    if (i >= nodes_.size() || !nodes_[i]) throw Error("NotFound", "not found: " + std::to_string(i));
    return nodes_[i];
  }
  void partition(const std::vector<size_t>& iso) {
    for (size_t i : iso)
      if (i >= nodes_.size()) throw Error("NotFound", "not found: " + std::to_string(i));
    isolated_.assign(nodes_.size(), false);
    for (size_t i : iso) isolated_[i] = true;
    sync();
  }
  void heal() {
    isolated_.assign(nodes_.size(), false);
    sync();
  }
  void crash(size_t i) {
    if (i >= nodes_.size() || !nodes_[i]) throw Error("NotFound", "not found: " + std::to_string(i));
    bus_->nodes.erase(std::to_string(i));
    nodes_[i].reset();
  }
  void restart(size_t i) {
    if (i >= nodes_.size()) throw Error("NotFound", "not found: " + std::to_string(i));
    if (nodes_[i]) throw Error("Other", "node " + std::to_string(i) + " is not crashed");
    nodes_[i] = Cluster::open(base_ + "/" + std::to_string(i), std::to_string(i), cfg_, bus_);
    sync();
  }
  void tick(uint64_t now) {
    sync();
    bus_->tick(now);
  }
  // index of the current leader among live nodes, or -1
  int leader() const {
    for (size_t i = 0; i < nodes_.size(); ++i)
      if (nodes_[i] && nodes_[i]->is_leader()) return static_cast<int>(i);
    return -1;
  }

 private:
  void sync() {
    bus_->isolated.clear();
    for (size_t i = 0; i < isolated_.size(); ++i)
      if (isolated_[i]) bus_->isolated.insert(std::to_string(i));
  }
  std::string base_;
  ClusterConfig cfg_;
  std::shared_ptr<Bus> bus_;
  std::vector<std::shared_ptr<Cluster>> nodes_;
  std::vector<bool> isolated_;
};

}  // namespace raft
}  // namespace pbn
