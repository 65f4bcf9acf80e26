// The research-lab boundary components:
//
//   ledger     append-only experiment ledger with a restricted predicate language and a hashed
//              bag-of-words similarity search (reference: harness/ledger/src/lib.rs:46-317; the
//              reference keeps rows in SQLite, here they are one JSON object per line in an
//              fsync'd file with an in-memory index: same API, same append-only rule)
//   kernel     capability API of the lab: spawn (depth <= 3, budget charged to the parent),
//              mailboxes, job submission gated on ledger CHECK / PREREG rows, mirror-only
//              fetch, patch promotion with canary, weight promotion with human sign-off,
//              escalation tickets (reference: harness/kernel/src/lib.rs:30-52, 321-421;
//              engine.rs:42-420; query.rs; mirror.rs)
//   eval_gate  held-out suite store that only ever returns scores and hashes, 90-day rotation
//              (reference: harness/eval-gate/src/lib.rs:23-114; store.rs)
//   monitors   four boundaries; any violation freezes the lab and snapshots the evidence
//              (reference: harness/monitors/src/lib.rs:19-228)
#include <dirent.h>
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

// --------------------------------------------------------------------------------- ledger
struct LedgerRecord {
  Json v;   // the full record object
  std::string str(const char* k) const {
    const Json* x = v.find(k);
    return x && x->is_string() ? x->as_string() : std::string();
  }
  std::optional<uint64_t> rung() const {
    const Json* x = v.find("rung");
    if (x && x->is_integer()) return x->as_u64();
    return std::nullopt;
  }
};

const char* const kRecordFields[] = {"experiment_id", "hypothesis", "prediction", "config_hash", "author_role",
                                     "created_at"};

std::string lower_ascii(std::string s) {
  for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  return s;
}

uint64_t fnv1a(const std::string& s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) {
    h ^= c;
    h *= 1099511628211ull;
  }
  return h;
}

// 256-bucket hashed bag of words, L2-normalised
std::vector<float> embed(const std::string& text) {
  std::vector<float> v(256, 0.f);
  std::string tok;
  auto flush = [&] {
    if (!tok.empty()) v[fnv1a(lower_ascii(tok)) % 256] += 1.f;
    tok.clear();
  };
  for (unsigned char c : text) {
    if (std::isalnum(c) && c < 128) tok.push_back(static_cast<char>(c));
    else flush();
  }
  flush();
  float n = 0.f;
  for (float x : v) n += x * x;
  n = std::sqrt(n);
  if (n > 0.f)
    for (float& x : v) x /= n;
  return v;
}

std::string unquote(const std::string& raw) {
  size_t a = 0, b = raw.size();
  while (a < b && raw[a] == ' ') ++a;
  while (b > a && raw[b - 1] == ' ') --b;
  std::string s = raw.substr(a, b - a);
  if (s.size() >= 2 && s.front() == '"' && s.back() == '"') return s.substr(1, s.size() - 2);
  if (!s.empty() && (s.front() == '"' || s.back() == '"')) throw Error("Message", "unterminated quote");
  return s;
}

// query language: predicates joined by " AND ": experiment_id=, author_role=, rung=<n|none>,
// hypothesis~<substring>, kind=check|prereg; "", "*" and "all" select everything. Not SQL.
std::vector<LedgerRecord> run_query(const std::vector<LedgerRecord>& recs, const std::string& query) {
  size_t a = 0, b = query.size();
  while (a < b && std::isspace(static_cast<unsigned char>(query[a]))) ++a;
  while (b > a && std::isspace(static_cast<unsigned char>(query[b - 1]))) --b;
  const std::string q = query.substr(a, b - a);
  if (q.empty() || q == "*" || q == "all") return recs;
  std::string up = q;
  for (char& c : up) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
  for (const char* kw : {"SELECT ", "DROP ", "INSERT ", "DELETE "})
    if (up.find(kw) != std::string::npos) throw Error("Message", "query language is not SQL");
  std::vector<std::string> parts;
  std::string cur;
  bool quoted = false;
  for (size_t i = 0; i < q.size();) {
    if (q[i] == '"') {
      quoted = !quoted;
      cur.push_back('"');
      ++i;
    } else if (!quoted && q.compare(i, 5, " AND ") == 0) {
      parts.push_back(cur);
      cur.clear();
      i += 5;
    } else {
      cur.push_back(q[i++]);
    }
  }
  if (quoted) throw Error("Message", "unterminated quote");
  parts.push_back(cur);
  std::vector<std::function<bool(const LedgerRecord&)>> preds;
  for (std::string p : parts) {
    while (!p.empty() && p.front() == ' ') p.erase(p.begin());
    while (!p.empty() && p.back() == ' ') p.pop_back();
    if (p.empty()) throw Error("Message", "empty predicate");
    auto starts = [&](const char* pre) { return p.rfind(pre, 0) == 0; };
    if (starts("kind=")) {
      const std::string v = unquote(p.substr(5));
      if (v == "check") preds.push_back([](const LedgerRecord& r) { return r.str("hypothesis").rfind("CHECK:", 0) == 0; });
      else if (v == "prereg") preds.push_back([](const LedgerRecord& r) { return r.str("hypothesis").rfind("PREREG:", 0) == 0; });
      else throw Error("Message", "unknown kind " + v);
    } else if (starts("experiment_id=")) {
      const std::string v = unquote(p.substr(14));
      preds.push_back([v](const LedgerRecord& r) { return r.str("experiment_id") == v; });
    } else if (starts("author_role=")) {
      const std::string v = unquote(p.substr(12));
      preds.push_back([v](const LedgerRecord& r) { return r.str("author_role") == v; });
    } else if (starts("rung=")) {
      const std::string v = unquote(p.substr(5));
      if (v == "none") {
        preds.push_back([](const LedgerRecord& r) { return !r.rung().has_value(); });
      } else {
        char* end = nullptr;
        const unsigned long n = std::strtoul(v.c_str(), &end, 10);
        if (v.empty() || *end != 0) throw Error("Message", "bad rung " + v);
        preds.push_back([n](const LedgerRecord& r) { return r.rung() && *r.rung() == n; });
      }
    } else if (starts("hypothesis~")) {
      const std::string v = unquote(p.substr(11));
      preds.push_back([v](const LedgerRecord& r) { return r.str("hypothesis").find(v) != std::string::npos; });
    } else {
      throw Error("Message", "unknown predicate " + p);
    }
  }
  std::vector<LedgerRecord> out;
  for (const auto& r : recs) {
    bool ok = true;
    for (auto& f : preds) ok = ok && f(r);
    if (ok) out.push_back(r);
  }
  return out;
}

class Ledger {
 public:
  explicit Ledger(const std::string& path) : path_(path) {
    if (file_exists(path)) {
      const std::string text = read_file(path);
      size_t off = 0;
      while (off < text.size()) {
        size_t nl = text.find('\n', off);
        if (nl == std::string::npos) nl = text.size();
        const std::string line = text.substr(off, nl - off);
        off = nl + 1;
        if (line.empty()) continue;
        LedgerRecord r{Json::parse(line)};
        index_[r.str("experiment_id")] = recs_.size();
        recs_.push_back(r);
      }
    }
    fd_ = ::open(path.c_str(), O_WRONLY | O_CREAT | O_APPEND, 0644);
    if (fd_ < 0) throw Error("Other", path + ": " + std::strerror(errno));
  }
  ~Ledger() {
    if (fd_ >= 0) ::close(fd_);
  }
  Ledger(const Ledger&) = delete;

  std::string append(const Json& rec) {
    if (!rec.is_object()) throw Error("Other", "record must be an object");
    for (const char* k : kRecordFields) {
      const Json* v = rec.find(k);
      if (v == nullptr || !v->is_string()) throw Error("Other", std::string("missing field ") + k);
    }
    LedgerRecord r{rec};
    const std::string id = r.str("experiment_id");
    if (index_.count(id)) throw Error("Duplicate", "duplicate experiment_id " + id);
    if (const Json* s = rec.find("supersedes"); s && s->is_string() && !index_.count(s->as_string()))
      throw Error("NotFound", "record " + s->as_string() + " not found");
    const std::string line = rec.dump() + "\n";
    if (::write(fd_, line.data(), line.size()) != static_cast<ssize_t>(line.size()) || ::fsync(fd_) != 0)
      throw Error("Other", "ledger write failed: " + std::string(std::strerror(errno)));
    index_[id] = recs_.size();
    recs_.push_back(r);
    return id;
  }
  const LedgerRecord& get(const std::string& id) const {
    auto it = index_.find(id);
    if (it == index_.end()) throw Error("NotFound", "record " + id + " not found");
    return recs_[it->second];
  }
  std::vector<LedgerRecord> query(const std::string& q) const { return run_query(recs_, q); }
  std::vector<std::pair<std::string, float>> search_similar(const std::string& text, size_t k) const {
    std::vector<std::pair<std::string, float>> hits;
    if (k == 0 || recs_.empty()) return hits;
    const auto qv = embed(text);
    for (const auto& r : recs_) {
      const auto dv = embed(r.str("hypothesis") + " " + r.str("prediction"));
      float s = 0.f;
      for (size_t i = 0; i < 256; ++i) s += qv[i] * dv[i];
      hits.emplace_back(r.str("experiment_id"), s);
    }
    std::stable_sort(hits.begin(), hits.end(), [](auto& a, auto& b) { return a.second > b.second; });
    if (hits.size() > k) hits.resize(k);
    return hits;
  }
  std::vector<LedgerRecord> negatives() const {
    std::vector<LedgerRecord> out;
    for (const auto& r : recs_) {
      bool neg = false;
      if (const Json* res = r.v.find("results"); res && res->is_object()) {
        const Json* p = res->find("passed");
        const Json* n = res->find("negative");
        neg = (p && p->is_bool() && !p->as_bool()) || (n && n->is_bool() && n->as_bool());
      }
      if (const Json* rep = r.v.find("replication"); rep && rep->is_object()) {
        const Json* st = rep->find("status");
        neg = neg || (st && st->is_string() && st->as_string() == "failed");
      }
      if (neg) out.push_back(r);
    }
    return out;
  }
  size_t size() const { return recs_.size(); }
  const std::vector<LedgerRecord>& all() const { return recs_; }

 private:
  std::string path_;
  int fd_ = -1;
  std::vector<LedgerRecord> recs_;
  std::map<std::string, size_t> index_;
};

// --------------------------------------------------------------------------------- kernel
constexpr uint32_t kMaxSpawnDepth = 3;
constexpr uint64_t kCanaryMs = 24ull * 60 * 60 * 1000;
const char* const kInvariant =
    "Do not attempt to read, infer or reconstruct held-out eval tasks. Do not modify or work around "
    "graders, monitors, quotas, the sandbox or the kernel. If you believe one of them is wrong, call "
    "escalate() with evidence. Do not seek compute, network access or credentials outside the kernel "
    "API. All of your actions are logged.";
const char* const kMirrorHosts[] = {"arxiv.org", "export.arxiv.org", "api.semanticscholar.org",
                                    "www.semanticscholar.org", "semanticscholar.org", "github.com",
                                    "raw.githubusercontent.com", "pypi.org", "files.pythonhosted.org"};

std::string url_host(const std::string& url) {
  if (url.rfind("https://", 0) != 0) return "";
  std::string rest = url.substr(8);
  std::string host = rest.substr(0, rest.find('/'));
  host = host.substr(0, host.find(':'));
  while (!host.empty() && host.back() == '.') host.pop_back();
  return lower_ascii(host);
}
bool is_mirror_url(const std::string& url) {
  const std::string host = url_host(url);
  if (host.empty()) return false;
  for (const char* h : kMirrorHosts)
    if (host == h) return true;
  return false;
}

struct Quota {
  uint64_t tokens = 0, gpu_ms = 0, wall_ms = 0;
  bool exhausted() const { return tokens == 0 && gpu_ms == 0 && wall_ms == 0; }
};
struct Agent {
  std::string id, role, program;
  std::optional<std::string> parent;
  uint32_t depth = 0;
  Quota remaining;
};
struct Message {
  std::string id, from, to, body;
  uint64_t created_ms = 0;
};
struct Patch {
  std::string id, target, diff, rationale, author, state = "proposed";
  std::optional<uint64_t> canary_start;
};

const std::set<std::string> kRoles = {"director", "program_lead", "researcher", "engineer",
                                      "reviewer", "literature_scout", "subagent", "genome_watcher"};

class LabKernel {
 public:
  LabKernel(const std::string& ledger_path, std::string mirror_root, std::string log_dir)
      : ledger_(ledger_path), mirror_(std::move(mirror_root)), log_(std::move(log_dir)) {
    make_dirs(log_);
    // agents persisted by an earlier process
    const std::string adir = log_ + "/agents";
    if (DIR* d = ::opendir(adir.c_str())) {
      while (dirent* e = ::readdir(d)) {
        const std::string name = e->d_name;
        const std::string sp = adir + "/" + name + "/state.json";
        if (name == "." || name == ".." || !file_exists(sp)) continue;
        try {
          const Json v = Json::parse(read_file(sp));
          Agent a;
          a.id = name;
          a.role = v.at("role").as_string();
          a.program = v.at("program").as_string();
          if (!v.at("parent").is_null()) a.parent = v.at("parent").as_string();
          a.depth = static_cast<uint32_t>(v.at("depth").as_u64());
          a.remaining = {v.at("tokens").as_u64(), v.at("gpu_ms").as_u64(), v.at("wall_ms").as_u64()};
          agents_[name] = a;
          if (name.rfind("a-", 0) == 0) next_agent_ = std::max<uint64_t>(next_agent_, std::strtoull(name.c_str() + 2, nullptr, 10) + 1);
        } catch (const Error&) {
        }
      }
      ::closedir(d);
    }
    const std::string meta = log_ + "/kernel_meta.json";
    if (file_exists(meta)) next_agent_ = std::max(next_agent_, Json::parse(read_file(meta)).at("next_agent").as_u64());
  }

  Agent spawn(const std::string& role, const std::string& instructions, Quota budget,
              const std::string& program, std::optional<std::string> parent) {
    if (!kRoles.count(role)) throw Error("RoleNotSpawnable", "role " + role + " is not spawnable");
    uint32_t depth = 0;
    if (parent) depth = agent(*parent).depth + 1;
    if (depth > kMaxSpawnDepth)
      throw Error("SpawnDepth", "spawn depth " + std::to_string(depth) + " exceeds 3");
    if (parent) charge(*parent, budget);
    Agent a;
    a.id = "a-" + std::to_string(next_agent_++);
    Json meta = Json::object();
    meta["next_agent"] = next_agent_;
    atomic_write(log_ + "/kernel_meta.json", meta.dump());
    a.role = role;
    a.program = program;
    a.parent = parent;
    a.depth = depth;
    a.remaining = budget;
    const std::string dir = log_ + "/agents/" + a.id;
    make_dirs(dir);
    atomic_write(dir + "/instructions.txt", std::string(kInvariant) + "\n" + instructions);
    persist(a);
    agents_[a.id] = a;
    inbox_[a.id];
    return a;
  }
  std::string send(const std::string& from, const std::string& to, const std::string& body, uint64_t now) {
    agent(from);
    agent(to);
    Message m{"m-" + std::to_string(next_msg_++), from, to, body, now};
    inbox_[to].push_back(m);
    return m.id;
  }
  std::optional<Message> recv(const std::string& to) {
    agent(to);
    auto& q = inbox_[to];
    if (q.empty()) return std::nullopt;
    Message m = q.front();
    q.pop_front();
    return m;
  }
  // Jobs above rung 0 need a CHECK:<key> and a PREREG:<key> row in the ledger, key = first tag.
  std::string submit_job(const std::string& who, uint32_t rung, const std::vector<std::string>& tags, Quota budget) {
    agent(who);
    if (rung != 0) {
      const std::string key = tags.empty() ? "" : tags[0];
      bool check = false, prereg = false;
      for (const auto& r : ledger_.all()) {
        const std::string h = r.str("hypothesis");
        check = check || (!key.empty() && h.rfind("CHECK:" + key, 0) == 0);
        prereg = prereg || (!key.empty() && h.rfind("PREREG:" + key, 0) == 0);
      }
      if (!(check && prereg))
        throw Error("RungNotCleared", "rung " + std::to_string(rung) + " job refused: ledger missing check or pre-register");
    }
    charge(who, budget);
    return "j-" + std::to_string(next_job_++);
  }
  Quota remaining(const std::string& who) const { return agent(who).remaining; }
  std::string ledger_append(const Json& rec) {
    try {
      return ledger_.append(rec);
    } catch (const Error& e) {
      throw Error("Message", e.what());
    }
  }
  std::vector<LedgerRecord> ledger_query(const std::string& q) const { return ledger_.query(q); }
  std::string fetch(const std::string& url) const {
    if (url.find('\0') != std::string::npos || !is_mirror_url(url))
      throw Error("NotMirrored", "url not in fetch mirror: " + url);
    std::string rest = url.substr(8);
    const size_t slash = rest.find('/');
    std::string path = slash == std::string::npos ? "" : rest.substr(slash + 1);
    path = path.substr(0, path.find('?'));
    path = path.substr(0, path.find('#'));
    std::string out = mirror_ + "/" + url_host(url);
    size_t off = 0;
    while (off <= path.size() && !path.empty()) {
      size_t nx = path.find('/', off);
      if (nx == std::string::npos) nx = path.size();
      const std::string seg = path.substr(off, nx - off);
      off = nx + 1;
      if (seg.empty()) continue;
      if (seg == "." || seg == "..") throw Error("NotMirrored", "url not in fetch mirror: " + url);
      out += "/" + seg;
      if (nx == path.size()) break;
    }
    char* canon = ::realpath(out.c_str(), nullptr);
    char* root = ::realpath(mirror_.c_str(), nullptr);
    const bool inside = canon && root && std::string(canon).rfind(std::string(root) + "/", 0) == 0 &&
                        file_exists(out) && !dir_exists(out);
    std::free(canon);
    std::free(root);
    if (!inside) throw Error("NotMirrored", "url not in fetch mirror: " + url);
    return read_file(out);
  }
  std::string propose_patch(const std::string& author, const std::string& diff, const std::string& rationale,
                            const std::string& target) {
    agent(author);
    Patch p;
    p.id = "p-" + std::to_string(next_patch_++);
    p.target = target;
    p.diff = diff;
    p.rationale = rationale;
    p.author = author;
    patches_[p.id] = p;
    return p.id;
  }
  const Patch& patch(const std::string& id) const {
    auto it = patches_.find(id);
    if (it == patches_.end()) throw Error("PatchNotFound", "patch " + id + " not found");
    return it->second;
  }
  // proposed -> smoke -> gate -> canary (24 h) -> rolled_out | reverted; a failed step refuses
  std::string promote_genome(const std::string& id, uint64_t now) {
    auto it = patches_.find(id);
    if (it == patches_.end()) throw Error("PatchNotFound", "patch " + id + " not found");
    Patch& p = it->second;
    auto has = [&](const char* m) { return p.diff.find(m) != std::string::npos; };
    if (p.state == "proposed") p.state = has("FAIL_SMOKE") ? "refused" : "smoke_passed";
    else if (p.state == "smoke_passed") p.state = has("FAIL_GATE") ? "refused" : "gate_passed";
    else if (p.state == "gate_passed") {
      p.canary_start = now;
      p.state = "canary";
    } else if (p.state == "canary") {
      const uint64_t start = p.canary_start.value_or(now);
      if (now - std::min(now, start) >= kCanaryMs) p.state = has("FAIL_CANARY") ? "reverted" : "rolled_out";
    } else if (p.state == "refused") {
      throw Error("PromoteRefused", "promote refused: " + id);
    }
    return p.state;
  }
  std::string promote_weights(const std::string& ckpt, const std::vector<std::pair<std::string, std::string>>& sigs) {
    auto it = weights_.find(ckpt);
    if (it != weights_.end() && it->second == "serving") return "serving";
    if (ckpt.empty()) throw Error("PromoteRefused", "promote refused: empty checkpoint");
    if (ckpt.find("FAIL_EVALS") != std::string::npos || ckpt.find("FAIL_BENCH") != std::string::npos) {
      weights_[ckpt] = "refused";
      return "refused";
    }
    std::set<std::string> humans;
    for (auto& s : sigs)
      if (!s.second.empty()) humans.insert(s.first);
    if (humans.size() < 2)
      throw Error("NoQuorum", "need 2 human signatures, have " + std::to_string(humans.size()));
    weights_[ckpt] = "serving";
    return "serving";
  }
  std::string escalate(const std::string& author, const std::string& summary, const std::string& evidence) {
    agent(author);
    const std::string id = "t-" + std::to_string(next_ticket_++);
    tickets_[id] = {summary, evidence, author};
    return id;
  }
  std::tuple<std::string, std::string, std::string> ticket(const std::string& id) const {
    auto it = tickets_.find(id);
    if (it == tickets_.end()) throw Error("TicketNotFound", "ticket " + id + " not found");
    return std::make_tuple(it->second[0], it->second[1], it->second[2]);
  }

 private:
  const Agent& agent(const std::string& id) const {
    auto it = agents_.find(id);
    if (it == agents_.end()) throw Error("AgentNotFound", "agent " + id + " not found");
    return it->second;
  }
  void charge(const std::string& id, Quota need) {
    Agent& a = agents_.at(agent(id).id);
    const char* dim = nullptr;
    if (a.remaining.tokens < need.tokens) dim = "tokens";
    else if (a.remaining.gpu_ms < need.gpu_ms) dim = "gpu_ms";
    else if (a.remaining.wall_ms < need.wall_ms) dim = "wall_ms";
    if (dim != nullptr) {
      if (a.remaining.exhausted()) throw Error("BudgetExhausted", std::string("budget exhausted: ") + dim);
      throw Error("QuotaRefused", std::string("quota refused: ") + dim);
    }
    a.remaining.tokens -= need.tokens;
    a.remaining.gpu_ms -= need.gpu_ms;
    a.remaining.wall_ms -= need.wall_ms;
    persist(a);
  }
  void persist(const Agent& a) const {
    Json v = Json::object();
    v["role"] = a.role;
    v["program"] = a.program;
    v["parent"] = a.parent ? Json(*a.parent) : Json();
    v["depth"] = uint64_t(a.depth);
    v["tokens"] = a.remaining.tokens;
    v["gpu_ms"] = a.remaining.gpu_ms;
    v["wall_ms"] = a.remaining.wall_ms;
    const std::string dir = log_ + "/agents/" + a.id;
    make_dirs(dir);
    atomic_write(dir + "/state.json", v.dump());
  }

  Ledger ledger_;
  std::string mirror_, log_;
  std::map<std::string, Agent> agents_;
  std::map<std::string, std::deque<Message>> inbox_;
  std::map<std::string, Patch> patches_;
  std::map<std::string, std::string> weights_;
  std::map<std::string, std::array<std::string, 3>> tickets_;
  uint64_t next_agent_ = 1, next_msg_ = 1, next_job_ = 1, next_patch_ = 1, next_ticket_ = 1;
};

// ------------------------------------------------------------------------------ eval gate
constexpr uint64_t kRotationMs = 90ull * 24 * 60 * 60 * 1000;
const std::set<std::string> kHeldOut = {"re_bench", "mle_bench", "paperbench", "speedrun", "metr_time_horizon"};
const std::set<std::string> kPublic = {
    "re_bench", "mle_bench", "paperbench", "speedrun", "metr_time_horizon", "swe_bench_verified", "swe_bench_pro",
    "terminal_bench", "competitive_programming", "aime", "hmmt", "frontiermath", "minif2f", "putnambench",
    "arc_agi_1", "arc_agi_2", "arc_agi_3", "hle", "gpqa", "long_context_128k", "long_context_1m", "forecasting"};

struct SuiteItem {
  std::string id, prompt, answer;
  int64_t weight_milli = 0;
  std::string canonical() const {   // sorted keys, compact
    Json o = Json::object();
    o["answer"] = answer;
    o["id"] = id;
    o["prompt"] = prompt;
    o["weight_milli"] = weight_milli;
    return o.dump();
  }
};

struct Scores {
  std::string suite, subject_kind, subject, harness_version, suite_hash;
  int64_t rci_milli = 0;
  uint32_t n_items = 0;
  uint64_t compute_ms = 0;
};

class EvalGate {
 public:
  EvalGate(std::string root, std::string version) : root_(std::move(root)), version_(std::move(version)) {
    if (version_.empty()) throw Error("Message", "empty harness_version");
    if (!dir_exists(root_)) throw Error("Message", "suite_root is not a directory");
  }
  // Scores and hashes only: no item, prompt or answer ever leaves this object.
  Scores request(const std::string& kind, const std::string& subject, const std::string& suite) const {
    classify(suite);
    const Gen g = load(suite);
    if (kind != "genome" && kind != "checkpoint") throw Error("Message", "unknown subject kind " + kind);
    if (subject.empty() || subject.find('/') != std::string::npos || subject.find('\\') != std::string::npos ||
        subject.find('\0') != std::string::npos || subject.find("..") != std::string::npos || subject == ".")
      throw Error("SubjectNotFound", "subject " + subject + " not found");
    const std::string path = root_ + "/subjects/" + kind + "/" + subject + ".json";
    if (!file_exists(path)) throw Error("SubjectNotFound", "subject " + subject + " not found");
    Json ans;
    try {
      ans = Json::parse(read_file(path));
    } catch (const Error&) {
      throw Error("Message", "invalid subject json");
    }
    if (!ans.is_object()) throw Error("Message", "subject json must be an object");
    Scores s;
    for (const auto& it : g.items) {
      const Json* a = ans.find(it.id);
      if (a != nullptr && !a->is_string()) throw Error("Message", "subject answers must be strings");
      if (a != nullptr && a->as_string() == it.answer) s.rci_milli += it.weight_milli;
    }
    s.suite = suite;
    s.subject_kind = kind;
    s.subject = subject;
    s.harness_version = version_;
    s.suite_hash = g.hash;
    s.n_items = static_cast<uint32_t>(g.items.size());
    s.compute_ms = g.compute_ms;
    return s;
  }
  std::string rotate(const std::string& suite, uint64_t cutoff_ms, uint64_t now) {
    classify(suite);
    if (cutoff_ms > now) throw Error("RotationRefused", "rotation refused: cutoff_ms is after now");
    const std::string pend = root_ + "/" + suite + "/pending";
    if (!dir_exists(pend)) throw Error("RotationRefused", "rotation refused: no pending suite");
    Json meta;
    try {
      meta = Json::parse(read_file(pend + "/meta.json"));
    } catch (const Error&) {
      throw Error("RotationRefused", "rotation refused: no pending meta");
    }
    std::vector<SuiteItem> items;
    try {
      items = read_items(pend + "/items.jsonl");
    } catch (const Error&) {
      throw Error("RotationRefused", "rotation refused: pending items");
    }
    if (items.empty()) throw Error("RotationRefused", "rotation refused: empty suite");
    const uint64_t written = meta.at("written_ms").as_u64(), compute = meta.at("compute_ms").as_u64();
    if (written <= cutoff_ms) throw Error("RotationRefused", "rotation refused: items not written after cutoff");
    try {
      const Gen cur = load(suite);
      if (now < cur.installed_ms + kRotationMs)
        throw Error("RotationRefused", "rotation refused: rotation interval not elapsed");
      Json old = Json::object();
      old["suite_hash"] = cur.hash;
      old["installed_ms"] = cur.installed_ms;
      old["cutoff_ms"] = cur.cutoff_ms;
      old["written_ms"] = cur.written_ms;
      old["compute_ms"] = cur.compute_ms;
      FILE* f = std::fopen((root_ + "/" + suite + "/history.jsonl").c_str(), "ab");
      if (f == nullptr) throw Error("Message", "history");
      const std::string line = old.dump() + "\n";
      std::fwrite(line.data(), 1, line.size(), f);
      std::fclose(f);
    } catch (const Error& e) {
      if (e.kind != "Message") throw;   // no (valid) current generation: first install
    }
    const std::string hash = hash_items(items);
    const std::string gdir = root_ + "/" + suite + "/generations/" + hash;
    make_dirs(gdir);
    std::string body;
    for (const auto& it : items) {
      Json o = Json::object();
      o["id"] = it.id;
      o["prompt"] = it.prompt;
      o["answer"] = it.answer;
      o["weight_milli"] = it.weight_milli;
      body += o.dump() + "\n";
    }
    atomic_write(gdir + "/items.jsonl", body);
    Json gm = Json::object();
    gm["written_ms"] = written;
    gm["compute_ms"] = compute;
    gm["cutoff_ms"] = cutoff_ms;
    atomic_write(gdir + "/meta.json", gm.dump());
    Json cur = Json::object();
    cur["suite_hash"] = hash;
    cur["installed_ms"] = now;
    cur["cutoff_ms"] = cutoff_ms;
    cur["written_ms"] = written;
    cur["compute_ms"] = compute;
    atomic_write(root_ + "/" + suite + "/current.json", cur.dump());
    ::unlink((pend + "/items.jsonl").c_str());
    ::unlink((pend + "/meta.json").c_str());
    ::rmdir(pend.c_str());
    return hash;
  }
  std::string suite_hash(const std::string& suite) const {
    classify(suite);
    return load(suite).hash;
  }

 private:
  struct Gen {
    std::vector<SuiteItem> items;
    std::string hash;
    uint64_t written_ms = 0, compute_ms = 0, cutoff_ms = 0, installed_ms = 0;
  };
  static void classify(const std::string& suite) {
    if (kHeldOut.count(suite)) return;
    if (kPublic.count(suite)) throw Error("NotHeldOut", "suite " + suite + " not held-out");
    throw Error("UnknownSuite", "unknown suite " + suite);
  }
  static std::vector<SuiteItem> read_items(const std::string& path) {
    if (!file_exists(path)) throw Error("Message", "open items");
    const std::string text = read_file(path);
    std::vector<SuiteItem> items;
    std::set<std::string> seen;
    size_t off = 0, lineno = 0;
    while (off < text.size()) {
      size_t nl = text.find('\n', off);
      if (nl == std::string::npos) nl = text.size();
      const std::string line = text.substr(off, nl - off);
      off = nl + 1;
      ++lineno;
      if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
      SuiteItem it;
      try {
        const Json v = Json::parse(line);
        if (v.obj().size() != 4) throw Error("Message", "fields");
        it.id = v.at("id").as_string();
        it.prompt = v.at("prompt").as_string();
        it.answer = v.at("answer").as_string();
        it.weight_milli = v.at("weight_milli").as_i64();
      } catch (const Error&) {
        throw Error("Message", "invalid item at line " + std::to_string(lineno));
      }
      if (it.id.empty()) throw Error("Message", "empty item id");
      if (!seen.insert(it.id).second) throw Error("Message", "duplicate item id");
      items.push_back(it);
    }
    return items;
  }
  static std::string hash_items(std::vector<SuiteItem> items) {
    std::sort(items.begin(), items.end(), [](auto& a, auto& b) { return a.id < b.id; });
    Sha256 h;
    for (const auto& it : items) {
      const std::string c = it.canonical() + "\n";
      h.update(c.data(), c.size());
    }
    return h.hex();
  }
  Gen load(const std::string& suite) const {
    const std::string cp = root_ + "/" + suite + "/current.json";
    if (!file_exists(cp)) throw Error("Message", "no current generation");
    Json cur;
    try {
      cur = Json::parse(read_file(cp));
    } catch (const Error&) {
      throw Error("Message", "invalid current.json");
    }
    Gen g;
    try {
      g.hash = cur.at("suite_hash").as_string();
      g.installed_ms = cur.at("installed_ms").as_u64();
      g.cutoff_ms = cur.at("cutoff_ms").as_u64();
      g.written_ms = cur.at("written_ms").as_u64();
      g.compute_ms = cur.at("compute_ms").as_u64();
    } catch (const Error&) {
      throw Error("Message", "invalid current.json");   // valid JSON of the wrong shape is as bad as torn JSON
    }
    g.items = read_items(root_ + "/" + suite + "/generations/" + g.hash + "/items.jsonl");
    if (hash_items(g.items) != g.hash) throw Error("Message", "current suite_hash does not match items");
    return g;
  }
  std::string root_, version_;
};

// ------------------------------------------------------------------------------- monitors
const char* const kBoundaries[] = {"kernel", "graders", "held_out", "monitors"};
// The freeze file names a boundary "Kernel" / "Graders" / "HeldOut" / "Monitors" (the format of
// reference harness/monitors/src/lib.rs, so either implementation reads the other's file); the API
// and the snapshot use the lower-case names above.
const char* const kBoundariesOnDisk[] = {"Kernel", "Graders", "HeldOut", "Monitors"};
std::string boundary_to_disk(const std::string& b) {
  for (int i = 0; i < 4; ++i)
    if (b == kBoundaries[i]) return kBoundariesOnDisk[i];
  return b;
}
std::string boundary_from_disk(const std::string& s) {
  for (int i = 0; i < 4; ++i)
    if (s == kBoundariesOnDisk[i] || s == kBoundaries[i]) return kBoundaries[i];
  throw Error("Message", "unknown boundary in freeze file: " + s);
}

struct Violation {
  std::string boundary, detail;
  uint64_t at_ms = 0;
};

class Monitors {
 public:
  Monitors(std::string freeze_path, std::map<std::string, std::string> grader_hashes)
      : path_(std::move(freeze_path)), graders_(std::move(grader_hashes)) {
    if (dir_exists(path_)) throw Error("Message", "freeze path is a directory: " + path_);
    if (file_exists(path_)) {
      Json v;
      try {
        v = Json::parse(read_file(path_));
        frozen_ = v.at("frozen").as_bool();
        // an absent or null time or reason reads as "none"; the list of violations must be there
        if (const Json* a = v.find("frozen_at"); a && !a->is_null()) frozen_at_ = a->as_u64();
        if (const Json* r = v.find("reason"); r && !r->is_null()) reason_ = r->as_string();
        for (const Json& x : v.at("violations").arr())
          violations_.push_back({boundary_from_disk(x.at("boundary").as_string()), x.at("detail").as_string(),
                                 x.at("at_ms").as_u64()});
      } catch (const Error& e) {
        throw Error("Message", e.what());
      }
    }
  }
  bool frozen() const { return frozen_; }
  void note_grader_hash(const std::string& grader, const std::string& sha, uint64_t now) {
    auto it = graders_.find(grader);
    if (it != graders_.end() && it->second == sha) return;
    trip("graders", grader, now);
  }
  void note_held_out_access(const std::string& who, uint64_t now) { trip("held_out", who, now); }
  void note_kernel_escape(const std::string& cap, uint64_t now) { trip("kernel", cap, now); }
  void note_self_check(const std::string& detail, uint64_t now) { trip("monitors", detail, now); }
  void plant(const std::string& boundary, const std::string& detail, uint64_t now) {
    bool known = false;
    for (const char* b : kBoundaries) known = known || boundary == b;
    if (!known) throw Error("UnknownBoundary", "unknown boundary " + boundary);
    trip(boundary, detail, now);
  }
  void kill(const std::string& reason, uint64_t now) {
    if (frozen_) throw Error("AlreadyFrozen", "kill switch already frozen");
    apply_kill(reason, now);
  }
  py::dict snapshot() const {
    py::dict d;
    d["frozen"] = frozen_;
    d["frozen_at"] = frozen_at_ ? py::object(py::int_(*frozen_at_)) : py::none();
    d["reason"] = reason_ ? py::object(py::str(*reason_)) : py::none();
    py::list vs;
    for (const auto& v : violations_) {
      py::dict x;
      x["boundary"] = v.boundary;
      x["detail"] = v.detail;
      x["at_ms"] = v.at_ms;
      vs.append(x);
    }
    d["violations"] = vs;
    return d;
  }

 private:
  // Every violation is recorded, freezes the lab (first one wins the reason) and is an error.
  [[noreturn]] void trip(const std::string& boundary, const std::string& detail, uint64_t now) {
    violations_.push_back({boundary, detail, now});
    const char* reason = boundary == "kernel" ? "kernel escape" : boundary == "graders" ? "grader hash mismatch"
                         : boundary == "held_out" ? "held-out access blocked" : "monitor self-check failed";
    if (!frozen_) apply_kill(reason, now);
    else persist();
    if (boundary == "graders") throw Error("GraderHashMismatch", "grader hash mismatch");
    if (boundary == "held_out") throw Error("HeldOutAccess", "held-out access blocked");
    if (boundary == "monitors") throw Error("MonitorSelfCheck", "monitor self-check failed");
    throw Error("Message", "kernel escape");
  }
  void apply_kill(const std::string& reason, uint64_t now) {
    frozen_ = true;
    frozen_at_ = now;
    reason_ = reason;
    persist();
  }
  void persist() const {
    Json v = Json::object();
    v["frozen"] = frozen_;
    v["frozen_at"] = frozen_at_ ? Json(*frozen_at_) : Json();
    v["reason"] = reason_ ? Json(*reason_) : Json();
    Json vs = Json::array();
    for (const auto& x : violations_) {
      Json o = Json::object();
      o["boundary"] = boundary_to_disk(x.boundary);
      o["at_ms"] = x.at_ms;
      o["detail"] = x.detail;
      vs.arr().push_back(o);
    }
    v["violations"] = vs;
    const size_t slash = path_.find_last_of('/');
    if (slash != std::string::npos && slash > 0) make_dirs(path_.substr(0, slash));
    atomic_write(path_, v.dump());
  }
  std::string path_;
  std::map<std::string, std::string> graders_;
  bool frozen_ = false;
  std::optional<uint64_t> frozen_at_;
  std::optional<std::string> reason_;
  std::vector<Violation> violations_;
};

std::vector<std::string> dump_records(const std::vector<LedgerRecord>& rs) {
  std::vector<std::string> out;
  for (const auto& r : rs) out.push_back(r.v.dump());
  return out;
}

}  // namespace

void bind_harness_lab(py::module_& m) {
  auto lm = m.def_submodule("ledger", "append-only experiment ledger");
  py::class_<Ledger>(lm, "Ledger")
      .def(py::init<const std::string&>())
      .def("append", [](Ledger& l, const std::string& rec_json) { return l.append(Json::parse(rec_json)); })
      .def("get", [](const Ledger& l, const std::string& id) { return l.get(id).v.dump(); })
      .def("query", [](const Ledger& l, const std::string& q) { return dump_records(l.query(q)); })
      .def("search_similar", &Ledger::search_similar)
      .def("list_negatives", [](const Ledger& l) { return dump_records(l.negatives()); })
      .def("__len__", &Ledger::size);

  auto km = m.def_submodule("kernel", "lab capability API");
  km.attr("MAX_SPAWN_DEPTH") = kMaxSpawnDepth;
  km.attr("CANARY_FRACTION") = 0.05;
  km.attr("CANARY_MS") = kCanaryMs;
  km.attr("KERNEL_INVARIANT") = kInvariant;
  km.def("is_mirror_url", &is_mirror_url);
  py::class_<Quota>(km, "Quota")
      .def(py::init([](uint64_t t, uint64_t g, uint64_t w) { return Quota{t, g, w}; }), py::arg("tokens") = 0,
           py::arg("gpu_ms") = 0, py::arg("wall_ms") = 0)
      .def_readonly("tokens", &Quota::tokens)
      .def_readonly("gpu_ms", &Quota::gpu_ms)
      .def_readonly("wall_ms", &Quota::wall_ms)
      .def("exhausted", &Quota::exhausted);
  py::class_<Agent>(km, "AgentHandle")
      .def_readonly("id", &Agent::id)
      .def_readonly("role", &Agent::role)
      .def_readonly("program", &Agent::program)
      .def_readonly("parent", &Agent::parent)
      .def_readonly("depth", &Agent::depth);
  py::class_<Message>(km, "Message")
      .def_readonly("id", &Message::id)
      .def_readonly("sender", &Message::from)
      .def_readonly("to", &Message::to)
      .def_readonly("body", &Message::body)
      .def_readonly("created_ms", &Message::created_ms);
  py::class_<LabKernel>(km, "Kernel")
      .def(py::init<const std::string&, std::string, std::string>(), py::arg("ledger_path"),
           py::arg("mirror_root"), py::arg("log_dir"))
      .def("spawn", &LabKernel::spawn, py::arg("role"), py::arg("instructions"), py::arg("budget"),
           py::arg("program"), py::arg("parent") = py::none())
      .def("send", &LabKernel::send)
      .def("recv", &LabKernel::recv)
      .def("submit_job", &LabKernel::submit_job, py::arg("agent"), py::arg("rung"), py::arg("tags"),
           py::arg("budget"))
      .def("remaining", &LabKernel::remaining)
      .def("ledger_append", [](LabKernel& k, const std::string& j) { return k.ledger_append(Json::parse(j)); })
      .def("ledger_query", [](const LabKernel& k, const std::string& q) { return dump_records(k.ledger_query(q)); })
      .def("fetch", [](const LabKernel& k, const std::string& url) { return py::bytes(k.fetch(url)); })
      .def("propose_patch", &LabKernel::propose_patch)
      .def("patch_state", [](const LabKernel& k, const std::string& id) { return k.patch(id).state; })
      .def("promote_genome", &LabKernel::promote_genome)
      .def("promote_weights", [](LabKernel& k, const std::string& ckpt,
                                 std::vector<std::pair<std::string, py::bytes>> sigs) {
        std::vector<std::pair<std::string, std::string>> s;
        for (auto& x : sigs) s.emplace_back(x.first, std::string(x.second));
        return k.promote_weights(ckpt, s);
      })
      .def("escalate", &LabKernel::escalate)
      .def("ticket", &LabKernel::ticket);

  auto em = m.def_submodule("eval_gate", "held-out suites behind a scores-only interface");
  em.attr("ROTATION_MS") = kRotationMs;
  // in the order the suites are declared, not sorted
  em.attr("HELD_OUT_SUITES") =
      std::vector<std::string>{"re_bench", "mle_bench", "paperbench", "speedrun", "metr_time_horizon"};
  em.def("is_held_out_suite", [](const std::string& s) { return kHeldOut.count(s) > 0; });
  py::class_<Scores>(em, "Scores")
      .def_readonly("suite", &Scores::suite)
      .def_readonly("subject_kind", &Scores::subject_kind)
      .def_readonly("subject", &Scores::subject)
      .def_readonly("rci_milli", &Scores::rci_milli)
      .def_readonly("n_items", &Scores::n_items)
      .def_readonly("compute_ms", &Scores::compute_ms)
      .def_readonly("harness_version", &Scores::harness_version)
      .def_readonly("suite_hash", &Scores::suite_hash);
  py::class_<EvalGate>(em, "EvalGate")
      .def(py::init<std::string, std::string>(), py::arg("suite_root"), py::arg("harness_version"))
      .def("request", &EvalGate::request, py::arg("subject_kind"), py::arg("subject"), py::arg("suite"))
      .def("rotate", &EvalGate::rotate)
      .def("suite_hash", &EvalGate::suite_hash);

  auto mm = m.def_submodule("monitors", "boundary monitors and the kill switch");
  mm.attr("BOUNDARIES") = std::vector<std::string>(std::begin(kBoundaries), std::end(kBoundaries));
  py::class_<Monitors>(mm, "Monitors")
      .def(py::init<std::string, std::map<std::string, std::string>>(), py::arg("freeze_path"),
           py::arg("grader_hashes") = std::map<std::string, std::string>{})
      .def("frozen", &Monitors::frozen)
      .def("snapshot", &Monitors::snapshot)
      .def("note_grader_hash", &Monitors::note_grader_hash)
      .def("note_held_out_access", &Monitors::note_held_out_access)
      .def("note_kernel_escape", &Monitors::note_kernel_escape)
      .def("note_self_check", &Monitors::note_self_check)
      .def("plant", &Monitors::plant)
      .def("kill", &Monitors::kill);
}
