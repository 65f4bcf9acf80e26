// Host-side fault injection and the batch-scheduler client:
//
//   chaos   scenario runner over N event-log replicas and M process ids: 18 fault kinds, gates
//           D0..D5 and the 72 h (injected clock) soak, invariants = lost tasks / duplicated
//           outputs across surviving replicas. Everything happens on the host in files and
//           memory; it never touches a GPU.
//           (reference: harness/chaos/src/lib.rs:23-39, 64-140, 265-578, 860-1060)
//   slurm   Slurm through one `ssh <cluster> ...` child per command with a poll-based timeout
//           (kill on expiry): job-name file written before sbatch, allowed GPU counts, at most
//           two live fv- jobs, wait with cancel on budget, reap only recorded ids, rsync fetch.
//           (reference: harness/slurm/src/lib.rs:20-27, 120-252, 296-430)
#include <fcntl.h>
#include <poll.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <signal.h>
#include <sys/wait.h>

#include <chrono>
#include <map>
#include <set>
#include <thread>

#include "eventlog.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

// ---------------------------------------------------------------------------------- chaos
constexpr uint32_t kD0Kills = 1000;
constexpr uint64_t kSoakMs = 72ull * 60 * 60 * 1000;
constexpr int64_t kClockSkewMs = 30000;
const char* const kEpoch = "1970-01-01T00:00:00Z";

struct Fault {
  std::string kind;        // snake_case name, e.g. "kill", "partition", "token_expiry"
  std::string a, b;        // process / replica ids / provider / job, by kind
  bool asymmetric = false;
  int64_t delta_ms = 0;

  Json to_json() const {
    auto obj = [&](std::initializer_list<std::pair<const char*, Json>> kv) {
      Json in = Json::object();
      for (auto& p : kv) in[p.first] = p.second;
      Json out = Json::object();
      out[kind] = in;
      return out;
    };
    if (kind == "kill") return obj({{"process", a}});
    if (kind == "partition") return obj({{"from", a}, {"to", b}, {"asymmetric", asymmetric}});
    if (kind == "heal_partition") return obj({{"from", a}, {"to", b}});
    if (kind == "outage" || kind == "heal_outage" || kind == "rate_limit") return obj({{"provider", a}});
    if (kind == "disk_full" || kind == "disk_corrupt" || kind == "node_loss") return obj({{"replica", a}});
    if (kind == "clock_skew") return obj({{"replica", a}, {"delta_ms", Json(delta_ms)}});
    if (kind == "node_replace") return obj({{"old", a}, {"new", b}});
    if (kind == "job_preempt" || kind == "walltime_kill") return obj({{"job", a}});
    return Json(kind);   // token_expiry, token_rotate, hung_squeue, unhang_squeue, broker_death
  }
};

const std::set<std::string> kFaultKinds = {
    "kill", "partition", "heal_partition", "outage", "heal_outage", "disk_full", "disk_corrupt", "clock_skew",
    "token_expiry", "token_rotate", "node_loss", "node_replace", "job_preempt", "walltime_kill", "hung_squeue",
    "unhang_squeue", "broker_death", "rate_limit"};

struct Replica {
  std::string id;
  std::unique_ptr<EventLog> log;
  std::vector<std::tuple<std::string, std::optional<std::string>, std::optional<uint64_t>>> events;
  bool disk_full = false, corrupt = false, lost = false;
};

struct Invariants {
  uint64_t lost_tasks = 0, duplicated_outputs = 0;
  bool hold() const { return lost_tasks == 0 && duplicated_outputs == 0; }
};
struct RunReport {
  std::string gate;
  uint32_t faults_applied = 0;
  Invariants invariants;
  bool recovered = false;
};

struct Lcg {
  uint64_t s;
  uint64_t next() { return s = s * 6364136223846793005ull + 1; }
  size_t pick(size_t n) { return static_cast<size_t>(next()) % n; }
};

class World {
 public:
  World(const std::string& dir, size_t n_replicas, uint32_t n_processes, uint64_t seed, bool existing)
      : dir_(dir), seed_(seed) {
    if (n_replicas < 2) throw Error("TooFewReplicas", "need at least 2 replicas, have " + std::to_string(n_replicas));
    if (n_processes > 0) {
      processes_.push_back("coordinator");
      for (uint32_t i = 0; i + 1 < n_processes; ++i) processes_.push_back("worker-" + std::to_string(i));
    }
    if (!existing) {
      if (file_exists(dir) || dir_exists(dir)) throw Error("Other", "directory exists: " + dir);
      if (::mkdir(dir.c_str(), 0777) != 0 || ::mkdir((dir + "/replicas").c_str(), 0777) != 0)
        throw Error("Other", dir + ": " + std::strerror(errno));
      for (size_t i = 0; i < n_replicas; ++i) {
        Replica r;
        r.id = std::to_string(i);
        r.log = EventLog::create(rpath(r.id));
        replicas_.push_back(std::move(r));
      }
      return;
    }
    if (!dir_exists(dir)) throw Error("Other", "missing world dir: " + dir);
    for (size_t i = 0; i < n_replicas; ++i) {
      Replica r;
      r.id = std::to_string(i);
      // a restart must not paper over damage: the file has to be whole lines of valid events
      const std::string text = read_file(rpath(r.id) + "/events.jsonl");
      if (!text.empty() && text.back() != '\n') throw Error("Log", "torn or corrupt replica log");
      size_t off = 0;
      while (off < text.size()) {
        const size_t nl = text.find('\n', off);
        if (nl > off) LogEvent::parse(text.substr(off, nl - off));
        off = nl + 1;
      }
      r.log = EventLog::open(rpath(r.id));
      for (const LogEvent& e : r.log->events()) r.events.emplace_back(e.event_type, e.task_id, e.attempt);
      replicas_.push_back(std::move(r));
    }
    rebuild();
  }

  uint64_t now() const { return now_; }
  void advance(uint64_t ms) { now_ = now_ > UINT64_MAX - ms ? UINT64_MAX : now_ + ms; }
  std::vector<std::string> replicas() const {
    std::vector<std::string> out;
    for (auto& r : replicas_) out.push_back(r.id);
    return out;
  }
  const std::vector<std::string>& processes() const { return processes_; }
  std::string replica_dir(const std::string& id) const { return rpath(id); }
  uint64_t seed() const { return seed_; }

  void enqueue_task(const std::string& task, uint64_t now) {
    const int origin = enqueue_origin();
    if (origin < 0) throw Error("Other", "no writeable replica (killed: recover required)");
    Json p = Json::object();
    p["task_id"] = task;
    p["now"] = now;
    for (size_t i : destinations(origin)) append(i, "chaos.enqueued", task, std::nullopt, p);
    api_enqueued_.push_back(task);
  }
  void complete_task(const std::string& task, uint64_t attempt, const std::string& output, uint64_t now) {
    int origin = (replicas_.size() > 1 && can_write(1)) ? 1 : enqueue_origin();
    if (origin < 0) throw Error("Other", "no writeable replica (killed: recover required)");
    Json p = Json::object();
    p["task_id"] = task;
    p["attempt"] = attempt;
    p["output"] = output;
    p["now"] = now;
    for (size_t i : destinations(origin)) append(i, "chaos.completed", task, attempt, p);
    ++complete_counts_[{task, attempt}];
  }

  // Log the fault on every writable replica first, then change the simulated world.
  void inject(const Fault& f) {
    if (!kFaultKinds.count(f.kind)) throw Error("Other", "unknown fault " + f.kind);
    if (f.kind == "kill") {
      bool ok = false;
      for (auto& p : processes_) ok = ok || p == f.a;
      if (!ok) throw Error("NoProcess", "unknown process: " + f.a);
    }
    if (f.kind == "partition" || f.kind == "heal_partition") {
      index_of(f.a);
      index_of(f.b);
    }
    if (f.kind == "disk_full" || f.kind == "disk_corrupt" || f.kind == "clock_skew" || f.kind == "node_loss" ||
        f.kind == "node_replace")
      index_of(f.a);
    if (f.kind == "clock_skew" && (f.delta_ms > kClockSkewMs || f.delta_ms < -kClockSkewMs))
      throw Error("ClockSkewBound", "clock skew " + std::to_string(f.delta_ms) + " ms exceeds +-30000 ms");
    const Json payload = f.to_json().is_object() ? f.to_json() : [&] {
      Json o = Json::object();
      o["fault"] = f.kind;
      return o;
    }();
    for (size_t i = 0; i < replicas_.size(); ++i)
      if (can_write(i)) append(i, "chaos.fault", std::nullopt, std::nullopt, payload);
    if (f.kind == "kill") {
      for (auto& r : replicas_) r.log.reset();   // every in-memory handle dies with the process
    } else if (f.kind == "partition") {
      dropped_.insert({f.a, f.b});
      if (!f.asymmetric) dropped_.insert({f.b, f.a});
    } else if (f.kind == "heal_partition") {
      dropped_.erase({f.a, f.b});
      dropped_.erase({f.b, f.a});
    } else if (f.kind == "disk_full") {
      replicas_[index_of(f.a)].disk_full = true;
    } else if (f.kind == "disk_corrupt") {
      Replica& r = replicas_[index_of(f.a)];
      r.log.reset();
      r.corrupt = true;
      r.events.clear();
      const std::string path = rpath(f.a) + "/events.jsonl";
      FILE* fp = std::fopen(path.c_str(), "wb");
      if (fp == nullptr) throw Error("Disk", "disk: " + std::string(std::strerror(errno)));
      std::fputs("{broken hash chain\n", fp);
      std::fclose(fp);
    } else if (f.kind == "node_loss") {
      Replica& r = replicas_[index_of(f.a)];
      r.lost = true;
      r.log.reset();
    } else if (f.kind == "node_replace") {
      Replica& r = replicas_[index_of(f.a)];
      r.lost = true;
      r.log.reset();
      bool have = false;
      for (auto& x : replicas_) have = have || x.id == f.b;
      if (!have) {
        Replica n;
        n.id = f.b;
        n.log = EventLog::create(rpath(f.b));
        replicas_.push_back(std::move(n));
      }
    }
    // outages, token events, scheduler events, skew within bounds: recorded only
  }

  // Start-up is replay: reopen every closed, uncorrupted replica from disk.
  void recover() {
    for (size_t i = 0; i < replicas_.size(); ++i) {
      Replica& r = replicas_[i];
      if (r.corrupt) continue;
      if (!r.log) r.log = EventLog::open(rpath(r.id));
      r.lost = false;
      append(i, "chaos.recover", std::nullopt, std::nullopt, Json::object());
    }
  }

  Invariants invariants() const {
    std::set<std::string> completed;
    for (auto& r : replicas_) {
      if (r.corrupt || r.lost) continue;
      for (auto& e : r.events)
        if (std::get<0>(e) == "chaos.completed" && std::get<1>(e)) completed.insert(*std::get<1>(e));
    }
    Invariants inv;
    std::set<std::string> seen;
    for (auto& id : api_enqueued_)
      if (seen.insert(id).second && !completed.count(id)) ++inv.lost_tasks;
    for (auto& kv : complete_counts_) inv.duplicated_outputs += kv.second > 0 ? kv.second - 1 : 0;
    return inv;
  }
  size_t log_len(const std::string& id) const {
    const Replica& r = replicas_[index_of(id)];
    if (r.corrupt) throw Error("Disk", "disk: corrupt replica " + id);
    return r.events.size();
  }
  std::vector<std::string> replica_event_types(const std::string& id) const {
    const Replica& r = replicas_[index_of(id)];
    if (!r.log) throw Error("Other", "replica " + id + " unavailable");
    std::vector<std::string> out;
    for (const LogEvent& e : r.log->events()) out.push_back(e.event_type);
    return out;
  }

 private:
  std::string rpath(const std::string& id) const { return dir_ + "/replicas/" + id; }
  size_t index_of(const std::string& id) const {
    for (size_t i = 0; i < replicas_.size(); ++i)
      if (replicas_[i].id == id) return i;
    throw Error("NoReplica", "unknown replica: " + id);
  }
  bool can_write(size_t i) const {
    const Replica& r = replicas_[i];
    return r.log && !r.disk_full && !r.corrupt && !r.lost;
  }
  int enqueue_origin() const {
    for (size_t i = 0; i < replicas_.size(); ++i)
      if (can_write(i)) return static_cast<int>(i);
    return -1;
  }
  std::vector<size_t> destinations(size_t origin) const {
    std::vector<size_t> out;
    for (size_t i = 0; i < replicas_.size(); ++i) {
      if (!can_write(i)) continue;
      if (i == origin || !dropped_.count({replicas_[origin].id, replicas_[i].id})) out.push_back(i);
    }
    return out;
  }
  void append(size_t i, const char* type, std::optional<std::string> task, std::optional<uint64_t> attempt,
              const Json& payload) {
    Replica& r = replicas_[i];
    if (!r.log) return;
    LogAppend a;
    a.event_type = type;
    a.payload = payload;
    a.timestamp = kEpoch;
    a.task_id = task;
    a.attempt = attempt;
    a.node_id = r.id;
    try {
      r.log->append(a);
    } catch (const Error& e) {
      throw Error("Log", e.what());
    }
    r.events.emplace_back(type, task, attempt);
  }
  void rebuild() {
    api_enqueued_.clear();
    complete_counts_.clear();
    std::set<std::string> seen;
    for (auto& r : replicas_)
      for (auto& e : r.events)
        if (std::get<0>(e) == "chaos.enqueued" && std::get<1>(e) && seen.insert(*std::get<1>(e)).second)
          api_enqueued_.push_back(*std::get<1>(e));
    for (auto& r : replicas_) {
      std::map<std::pair<std::string, uint64_t>, uint64_t> local;
      for (auto& e : r.events)
        if (std::get<0>(e) == "chaos.completed" && std::get<1>(e) && std::get<2>(e))
          ++local[{*std::get<1>(e), *std::get<2>(e)}];
      for (auto& kv : local) complete_counts_[kv.first] = std::max(complete_counts_[kv.first], kv.second);
    }
  }

  std::string dir_;
  uint64_t seed_, now_ = 0;
  std::vector<Replica> replicas_;
  std::vector<std::string> processes_;
  std::set<std::pair<std::string, std::string>> dropped_;
  std::vector<std::string> api_enqueued_;
  std::map<std::pair<std::string, uint64_t>, uint64_t> complete_counts_;
};

Fault mk(const std::string& kind, const std::string& a = "", const std::string& b = "", bool asym = false,
         int64_t delta = 0) {
  Fault f;
  f.kind = kind;
  f.a = a;
  f.b = b;
  f.asymmetric = asym;
  f.delta_ms = delta;
  return f;
}

std::vector<Fault> faults_for(const std::string& gate) {
  if (gate == "D0") return {mk("kill", "coordinator")};
  if (gate == "D1") return {mk("kill", "coordinator"), mk("partition", "0", "1", false)};
  if (gate == "D2")
    return {mk("partition", "0", "1", true), mk("clock_skew", "0", "", false, kClockSkewMs),
            mk("clock_skew", "1", "", false, -kClockSkewMs), mk("node_loss", "0")};
  if (gate == "D3") return {mk("job_preempt", "job-0"), mk("walltime_kill", "job-0"), mk("hung_squeue")};
  if (gate == "D4") return {mk("broker_death"), mk("token_expiry"), mk("outage", "xai")};
  if (gate == "D5") return {mk("outage", "xai"), mk("outage", "openai")};
  if (gate == "Soak") {
    std::vector<Fault> all;
    for (const char* g : {"D0", "D1", "D2", "D3", "D4", "D5"})
      for (auto& f : faults_for(g)) all.push_back(f);
    return all;
  }
  throw Error("Other", "unknown gate " + gate);
}

// ids the world does not know fall back to its first process / replica
Fault bind(const World& w, Fault f) {
  auto proc = [&](const std::string& p) {
    for (auto& x : w.processes())
      if (x == p) return p;
    return w.processes().empty() ? p : w.processes()[0];
  };
  auto rep = [&](const std::string& r) {
    const auto ids = w.replicas();
    for (auto& x : ids)
      if (x == r) return r;
    return ids.empty() ? r : ids[0];
  };
  if (f.kind == "kill") f.a = proc(f.a);
  else if (f.kind == "partition" || f.kind == "heal_partition") {
    f.a = rep(f.a);
    f.b = rep(f.b);
  } else if (f.kind == "disk_full" || f.kind == "disk_corrupt" || f.kind == "clock_skew" || f.kind == "node_loss" ||
             f.kind == "node_replace")
    f.a = rep(f.a);
  return f;
}

RunReport finish(World& w, const std::string& gate, uint32_t applied, const std::vector<std::string>& tasks) {
  w.recover();
  for (auto& t : tasks) w.complete_task(t, 1, "ok", w.now());
  const Invariants inv = w.invariants();
  if (!inv.hold())
    throw Error("Invariant", "invariants failed: lost_tasks=" + std::to_string(inv.lost_tasks) +
                                 " duplicated_outputs=" + std::to_string(inv.duplicated_outputs));
  return RunReport{gate, applied, inv, true};
}

RunReport run_soak(World& w, uint64_t duration_ms, uint64_t seed) {
  const uint64_t start = w.now();
  std::vector<std::string> tasks;
  for (int i = 0; i < 4; ++i) {
    tasks.push_back("t" + std::to_string(i));
    w.enqueue_task(tasks.back(), w.now());
  }
  uint32_t applied = 0;
  const char* gates[] = {"D0", "D1", "D2", "D3", "D4", "D5"};
  const uint64_t slice = duration_ms / 6;
  for (const char* g : gates) {
    std::vector<Fault> faults;
    if (std::string(g) == "D0") {
      Lcg rng{seed};
      const auto& procs = w.processes();
      faults.push_back(mk("kill", procs.empty() ? "coordinator" : procs[rng.pick(procs.size())]));
    } else {
      for (auto& f : faults_for(g)) faults.push_back(bind(w, f));
    }
    for (auto& f : faults) {
      try {
        w.inject(f);
        ++applied;
      } catch (const Error&) {
      }
      if (f.kind == "kill") {
        try {
          w.recover();
        } catch (const Error&) {
        }
      }
    }
    w.advance(slice);
    try {
      w.recover();
    } catch (const Error&) {
    }
  }
  const auto ids = w.replicas();
  if (!ids.empty()) {
    try {
      w.inject(mk("disk_full", ids.back()));
      ++applied;
    } catch (const Error&) {
    }
  }
  const uint64_t elapsed = w.now() - start;
  if (elapsed < duration_ms) w.advance(duration_ms - elapsed);
  return finish(w, "Soak", applied, tasks);
}

RunReport run_gate(World& w, const std::string& gate) {
  if (gate == "Soak") return run_soak(w, kSoakMs, w.seed());
  const auto planned = faults_for(gate);   // validates the gate name
  std::vector<std::string> tasks;
  for (int i = 0; i < 4; ++i) {
    tasks.push_back("t" + std::to_string(i));
    w.enqueue_task(tasks.back(), w.now());
  }
  uint32_t applied = 0;
  if (gate == "D0") {
    Lcg rng{w.seed()};
    const auto procs = w.processes();
    for (uint32_t i = 0; i < kD0Kills; ++i) {
      w.inject(mk("kill", procs[rng.pick(procs.size())]));
      ++applied;
      w.recover();
    }
  } else {
    for (auto& f0 : planned) {
      const Fault f = bind(w, f0);
      w.inject(f);
      ++applied;
      if (f.kind == "kill") w.recover();
    }
    if (gate == "D1") w.advance(10000);   // let the dead coordinator's lease run out
  }
  return finish(w, gate, applied, tasks);
}

// ---------------------------------------------------------------------------------- slurm
struct SlurmConfig {
  std::string cluster = "ncshare", remote_root = "/work/prometheus", partition = "gpu", state_dir,
              gres_type = "b200";
  uint64_t query_timeout_ms = 45000;
  uint32_t max_concurrent = 2;
};

struct ProcResult {
  bool timed_out = false;
  int status = 0;
  std::string out, err;
};

// Run argv with stdout / stderr captured; poll for exit; kill the child when the budget ends.
ProcResult run_child(const std::vector<std::string>& argv, uint64_t timeout_ms) {
  int po[2], pe[2];
  if (::pipe(po) != 0 || ::pipe(pe) != 0) throw Error("Other", "pipe: " + std::string(std::strerror(errno)));
  const pid_t pid = ::fork();
  if (pid < 0) throw Error("Other", "fork: " + std::string(std::strerror(errno)));
  if (pid == 0) {
    ::dup2(po[1], 1);
    ::dup2(pe[1], 2);
    ::close(po[0]); ::close(po[1]); ::close(pe[0]); ::close(pe[1]);
    std::vector<char*> av;
    for (auto& s : argv) av.push_back(const_cast<char*>(s.c_str()));
    av.push_back(nullptr);
    ::execvp(av[0], av.data());
    ::_exit(127);
  }
  ::close(po[1]);
  ::close(pe[1]);
  ::fcntl(po[0], F_SETFL, O_NONBLOCK);
  ::fcntl(pe[0], F_SETFL, O_NONBLOCK);
  ProcResult r;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  auto drain = [&](int fd, std::string& dst) {
    char buf[4096];
    ssize_t n;
    while ((n = ::read(fd, buf, sizeof buf)) > 0) dst.append(buf, static_cast<size_t>(n));
  };
  bool done = false;
  while (!done) {
    drain(po[0], r.out);
    drain(pe[0], r.err);
    int st = 0;
    const pid_t w = ::waitpid(pid, &st, WNOHANG);
    if (w == pid) {
      r.status = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + WTERMSIG(st);
      done = true;
    } else if (std::chrono::steady_clock::now() >= deadline) {
      ::kill(pid, SIGKILL);   // exactly the child we started
      ::waitpid(pid, &st, 0);
      r.timed_out = true;
      done = true;
    } else {
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
  }
  drain(po[0], r.out);
  drain(pe[0], r.err);
  ::close(po[0]);
  ::close(pe[0]);
  return r;
}

std::string parse_state(const std::string& raw) {
  size_t a = raw.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) return "";
  size_t b = raw.find_first_of(" \t\r\n", a);
  std::string tok = raw.substr(a, b == std::string::npos ? std::string::npos : b - a);
  while (!tok.empty() && tok.back() == '+') tok.pop_back();
  for (char& c : tok) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
  static const std::map<std::string, std::string> names = {
      {"PENDING", "Pending"}, {"RUNNING", "Running"}, {"COMPLETED", "Completed"}, {"FAILED", "Failed"},
      {"CANCELLED", "Cancelled"}, {"CANCELED", "Cancelled"}, {"TIMEOUT", "Timeout"}, {"PREEMPTED", "Preempted"},
      {"NODE_FAIL", "NodeFail"}, {"OUT_OF_MEMORY", "OutOfMemory"}};
  auto it = names.find(tok);
  return it == names.end() ? "" : it->second;
}
bool is_terminal(const std::string& st) { return !(st == "Pending" || st == "Running" || st == "Unknown"); }

uint32_t count_live_fv(const std::string& squeue_out) {
  uint32_t n = 0;
  size_t off = 0;
  while (off < squeue_out.size()) {
    size_t nl = squeue_out.find('\n', off);
    if (nl == std::string::npos) nl = squeue_out.size();
    const std::string line = squeue_out.substr(off, nl - off);
    off = nl + 1;
    bool named = false, live = false;
    size_t p = 0;
    while (p < line.size()) {
      const size_t s = line.find_first_not_of(" \t", p);
      if (s == std::string::npos) break;
      size_t e = line.find_first_of(" \t", s);
      if (e == std::string::npos) e = line.size();
      std::string f = line.substr(s, e - s);
      p = e;
      named = named || f == "fv" || f.rfind("fv-", 0) == 0;
      for (char& c : f) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
      live = live || f == "R" || f == "PD" || f == "RUNNING" || f == "PENDING";
    }
    n += (named && live) ? 1 : 0;
  }
  return n;
}

class SlurmClient {
 public:
  explicit SlurmClient(SlurmConfig c) : cfg_(std::move(c)) {
    if (cfg_.state_dir.empty()) {
      const char* home = std::getenv("HOME");
      cfg_.state_dir = std::string(home ? home : ".") + "/.local/state/prometheus-slurm";
    }
  }
  std::string submit(const std::string& run_id, const std::string& suffix, const std::string& script,
                     const std::string& walltime, uint32_t gpus) {
    if (gpus != 1 && gpus != 2 && gpus != 4)
      throw Error("BadGpuCount", "gpus must be one of [1, 2, 4], got " + std::to_string(gpus));
    if (count_live_fv(remote({"squeue", "--noheader"})) >= cfg_.max_concurrent)
      throw Error("ConcurrentCap", "already " + std::to_string(cfg_.max_concurrent) + " live fv- jobs; refusing submit");
    const std::string name = "fv-" + suffix;
    // the name is on disk before the job exists, so a crash between the two can be cleaned up
    make_dirs(run_dir(run_id));
    atomic_write(run_dir(run_id) + "/job-name", name + "\n");
    if (!file_exists(job_ids_path(run_id))) atomic_write(job_ids_path(run_id), std::string());
    const std::string out = remote({"sbatch", "-J", name, "-t", walltime, "-p", cfg_.partition,
                                    "--gres=gpu:" + cfg_.gres_type + ":" + std::to_string(gpus), script});
    std::string id;
    size_t p = 0;
    while (p < out.size() && id.empty()) {
      const size_t s = out.find_first_not_of(" \t\r\n", p);
      if (s == std::string::npos) break;
      size_t e = out.find_first_of(" \t\r\n", s);
      if (e == std::string::npos) e = out.size();
      const std::string tok = out.substr(s, e - s);
      if (tok.find_first_not_of("0123456789") == std::string::npos) id = tok;
      p = e;
    }
    if (id.empty()) throw Error("Submit", "sbatch did not return a job id: " + out);
    FILE* f = std::fopen(job_ids_path(run_id).c_str(), "ab");
    if (f == nullptr) throw Error("Other", "open " + job_ids_path(run_id));
    std::fprintf(f, "%s\n", id.c_str());
    std::fclose(f);
    return id;
  }
  // Never hangs and never guesses: anything but a clean answer is "Unknown" (a timeout raises).
  std::string state(const std::string& id) {
    try {
      const std::string out = remote({"sacct", "-j", id, "-n", "-X", "-o", "State"});
      size_t off = 0;
      while (off < out.size()) {
        size_t nl = out.find('\n', off);
        if (nl == std::string::npos) nl = out.size();
        const std::string line = out.substr(off, nl - off);
        off = nl + 1;
        if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
        const std::string st = parse_state(line);
        return st.empty() ? "Unknown" : st;
      }
      return "Unknown";
    } catch (const Error& e) {
      if (e.kind == "QueryTimeout") throw;
      return "Unknown";
    }
  }
  std::string wait(const std::string& id, uint64_t budget_ms) {
    const auto start = std::chrono::steady_clock::now();
    for (;;) {
      std::string st;
      try {
        st = state(id);
      } catch (const Error& e) {
        if (e.kind != "QueryTimeout") throw;
        st = "Unknown";
      }
      if (is_terminal(st)) return st;
      const auto spent = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start).count();
      if (static_cast<uint64_t>(spent) >= budget_ms) {
        try {
          cancel(id);
        } catch (const Error&) {
        }
        return "Cancelled";
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(std::min<uint64_t>(50, budget_ms - spent)));
    }
  }
  void cancel(const std::string& id) { remote({"scancel", id}); }
  void fetch(const std::string& run_id, const std::string& dest) {
    make_dirs(dest);
    const ProcResult r = run_child({"rsync", "-a", cfg_.cluster + ":" + cfg_.remote_root + "/" + run_id + "/", dest},
                                   10ull * 60 * 1000);
    if (r.timed_out || r.status != 0) throw Error("Other", "rsync failed: status " + std::to_string(r.status));
  }
  // Cancels exactly the ids this client recorded for the run, nothing matched by name.
  void reap_tracked(const std::string& run_id) {
    const std::string path = job_ids_path(run_id);
    if (!file_exists(path)) return;
    const std::string text = read_file(path);
    size_t off = 0;
    while (off < text.size()) {
      size_t nl = text.find('\n', off);
      if (nl == std::string::npos) nl = text.size();
      std::string tok = text.substr(off, nl - off);
      off = nl + 1;
      while (!tok.empty() && std::isspace(static_cast<unsigned char>(tok.back()))) tok.pop_back();
      if (!tok.empty() && tok.find_first_not_of("0123456789") == std::string::npos) cancel(tok);
    }
  }
  std::string job_ids_path(const std::string& run_id) const { return run_dir(run_id) + "/job-ids"; }

 private:
  std::string run_dir(const std::string& run_id) const { return cfg_.state_dir + "/runs/" + run_id; }
  std::string remote(std::vector<std::string> cmd) {
    const char* ssh = std::getenv("PROMETHEUS_SLURM_SSH");
    std::vector<std::string> argv = {ssh ? ssh : "ssh", cfg_.cluster};
    const bool sbatch = !cmd.empty() && cmd[0] == "sbatch";
    for (auto& c : cmd) argv.push_back(c);
    const ProcResult r = run_child(argv, cfg_.query_timeout_ms);
    if (r.timed_out) throw Error("QueryTimeout", "squeue/sacct timed out after " + std::to_string(cfg_.query_timeout_ms) + " ms");
    if (r.status != 0) {
      const std::string detail = "status=" + std::to_string(r.status) + " stdout=" + r.out + " stderr=" + r.err;
      throw Error(sbatch ? "Submit" : "Other", sbatch ? "sbatch did not return a job id: " + detail : detail);
    }
    return r.out;
  }
  SlurmConfig cfg_;
};

}  // namespace

void bind_harness_faults(py::module_& m) {
  auto cm = m.def_submodule("chaos", "host-side fault injection over event-log replicas");
  cm.attr("D0_KILLS") = kD0Kills;
  cm.attr("SOAK_MS") = kSoakMs;
  cm.attr("CLOCK_SKEW_MS") = kClockSkewMs;
  cm.attr("MIN_REPLICAS") = 2;
  cm.attr("FAULT_KINDS") = std::vector<std::string>(kFaultKinds.begin(), kFaultKinds.end());
  py::class_<Fault>(cm, "Fault")
      .def(py::init(&mk), py::arg("kind"), py::arg("a") = "", py::arg("b") = "", py::arg("asymmetric") = false,
           py::arg("delta_ms") = 0)
      .def_readonly("kind", &Fault::kind)
      .def_readonly("a", &Fault::a)
      .def_readonly("b", &Fault::b)
      .def("to_json", [](const Fault& f) { return f.to_json().dump(); });
  py::class_<Invariants>(cm, "Invariants")
      .def_readonly("lost_tasks", &Invariants::lost_tasks)
      .def_readonly("duplicated_outputs", &Invariants::duplicated_outputs)
      .def("hold", &Invariants::hold);
  py::class_<RunReport>(cm, "RunReport")
      .def_readonly("gate", &RunReport::gate)
      .def_readonly("faults_applied", &RunReport::faults_applied)
      .def_readonly("invariants", &RunReport::invariants)
      .def_readonly("recovered", &RunReport::recovered);
  py::class_<World>(cm, "World")
      .def_static("create", [](const std::string& d, size_t nr, uint32_t np, uint64_t seed) {
                    return std::make_unique<World>(d, nr, np, seed, false);
                  }, py::arg("dir"), py::arg("n_replicas") = 2, py::arg("n_processes") = 4, py::arg("seed") = 0)
      .def_static("open", [](const std::string& d, size_t nr, uint32_t np, uint64_t seed) {
                    return std::make_unique<World>(d, nr, np, seed, true);
                  }, py::arg("dir"), py::arg("n_replicas") = 2, py::arg("n_processes") = 4, py::arg("seed") = 0)
      .def("now", &World::now)
      .def("advance", &World::advance)
      .def("replicas", &World::replicas)
      .def("processes", &World::processes)
      .def("replica_dir", &World::replica_dir)
      .def("enqueue_task", &World::enqueue_task)
      .def("complete_task", [](World& w, const std::string& t, uint64_t a, py::bytes out, uint64_t now) {
        w.complete_task(t, a, std::string(out), now);
      })
      .def("inject", &World::inject)
      .def("recover", &World::recover)
      .def("invariants", &World::invariants)
      .def("log_len", &World::log_len)
      .def("replica_event_types", &World::replica_event_types);
  cm.def("faults_for", &faults_for);
  cm.def("run_gate", &run_gate);
  cm.def("run_soak", &run_soak, py::arg("world"), py::arg("duration_ms") = kSoakMs, py::arg("seed") = 0);

  auto sm = m.def_submodule("slurm", "Slurm over ssh with bounded waits");
  sm.attr("JOB_PREFIX") = "fv";
  sm.attr("ALLOWED_GPUS") = std::vector<uint32_t>{1, 2, 4};
  sm.attr("MAX_CONCURRENT_JOBS") = 2;
  sm.attr("QUERY_TIMEOUT_MS") = 45000;
  sm.def("parse_state", [](const std::string& raw) -> py::object {
    const std::string s = parse_state(raw);
    return s.empty() ? py::none() : py::object(py::str(s));
  });
  sm.def("is_terminal", &is_terminal);
  sm.def("count_live_fv", &count_live_fv);
  py::class_<SlurmConfig>(sm, "ClientConfig")
      .def(py::init([](std::string cluster, std::string root, std::string part, std::string state, uint64_t to,
                       uint32_t mc, std::string gres) {
             SlurmConfig c;
             c.cluster = std::move(cluster);
             c.remote_root = std::move(root);
             c.partition = std::move(part);
             c.state_dir = std::move(state);
             c.query_timeout_ms = to;
             c.max_concurrent = mc;
             c.gres_type = std::move(gres);
             return c;
           }),
           py::arg("cluster") = "ncshare", py::arg("remote_root") = "/work/prometheus", py::arg("partition") = "gpu",
           py::arg("state_dir") = "", py::arg("query_timeout_ms") = 45000, py::arg("max_concurrent") = 2,
           py::arg("gres_type") = "b200");
  py::class_<SlurmClient>(sm, "Client")
      .def(py::init<SlurmConfig>())
      .def("submit", &SlurmClient::submit, py::arg("run_id"), py::arg("suffix"), py::arg("script"),
           py::arg("walltime"), py::arg("gpus"), py::call_guard<py::gil_scoped_release>())
      .def("state", &SlurmClient::state, py::call_guard<py::gil_scoped_release>())
      .def("wait", &SlurmClient::wait, py::call_guard<py::gil_scoped_release>())
      .def("cancel", &SlurmClient::cancel, py::call_guard<py::gil_scoped_release>())
      .def("fetch", &SlurmClient::fetch, py::call_guard<py::gil_scoped_release>())
      .def("reap_tracked", &SlurmClient::reap_tracked, py::call_guard<py::gil_scoped_release>())
      .def("job_ids_path", &SlurmClient::job_ids_path);
}
