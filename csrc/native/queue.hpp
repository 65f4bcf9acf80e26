// Lease queue: durable FIFO of work items with leases, heartbeats and attempt-keyed outputs.
//
// Same observable behaviour and on-disk layout as the reference's harness/leases crate
// (harness/leases/src/lib.rs:15-26, 126-397, 400-577): the event log at <dir>/log is the only
// source of truth (event types task.enqueued / claimed / heartbeat / expired / completed /
// failed / output, timestamps = the injected `now` in decimal), the in-memory tables are
// rebuilt by replaying it, outputs live at <dir>/outputs/<task>/<attempt> so a zombie worker
// of an older attempt can never overwrite a newer result.
#pragma once

#include <deque>
#include <functional>
#include <map>

#include "eventlog.hpp"

namespace pbn {

struct QueueConfig {
  uint64_t heartbeat_period_ms = 15000;
  uint32_t missed_heartbeats = 2;
  uint64_t lease_ttl_ms() const {
    const uint64_t m = missed_heartbeats < 1 ? 1 : missed_heartbeats;
    const unsigned __int128 p = static_cast<unsigned __int128>(heartbeat_period_ms) * m;
    return p > UINT64_MAX ? UINT64_MAX : static_cast<uint64_t>(p);
  }
};

enum class TaskState { Queued, Leased, Completed, Failed };
inline const char* task_state_name(TaskState s) {
  switch (s) {
    case TaskState::Queued: return "Queued";
    case TaskState::Leased: return "Leased";
    case TaskState::Completed: return "Completed";
    default: return "Failed";
  }
}

struct QueueTask {
  std::string id;
  Json payload;
  TaskState state = TaskState::Queued;
  uint64_t attempt = 0;
  std::optional<std::string> worker_id;
  std::optional<uint64_t> expires_at;
  std::optional<std::string> output_hash;
};

struct Lease {
  std::string task_id, worker_id;
  uint64_t attempt = 0, expires_at = 0;
};

inline uint64_t sat_add(uint64_t a, uint64_t b) { return a > UINT64_MAX - b ? UINT64_MAX : a + b; }

class LeaseQueue {
 public:
  static std::unique_ptr<LeaseQueue> create(const std::string& dir, QueueConfig cfg = {}) {
    if (::mkdir(dir.c_str(), 0777) != 0) throw Error("Other", dir + ": " + std::strerror(errno));
    auto q = std::unique_ptr<LeaseQueue>(new LeaseQueue(dir, cfg));
    q->log_ = EventLog::create(dir + "/log");
    return q;
  }
  static std::unique_ptr<LeaseQueue> open(const std::string& dir, QueueConfig cfg = {}) {
    auto q = std::unique_ptr<LeaseQueue>(new LeaseQueue(dir, cfg));
    try {
      q->log_ = EventLog::open(dir + "/log");
    } catch (const Error& e) {
      throw Error("Log", e.what());
    }
    for (const LogEvent& e : q->log_->events()) q->apply(e);
    return q;
  }

  std::string enqueue(const std::string& task_id, const Json& payload, uint64_t now) {
    if (tasks_.count(task_id)) throw Error("Duplicate", "duplicate: " + task_id);
    append("task.enqueued", task_id, std::nullopt, payload, std::nullopt, now);
    return task_id;
  }

  std::optional<Lease> claim(const std::string& worker, uint64_t now) {
    return claim_if(worker, now, [](const QueueTask&) { return true; });
  }

  // First queued task (FIFO order) accepted by `pred`; tasks it rejects stay untouched.
  std::optional<Lease> claim_if(const std::string& worker, uint64_t now,
                                const std::function<bool(const QueueTask&)>& pred) {
    expire_due(now);
    std::string id;
    bool found = false;
    for (const std::string& q : queued_) {
      if (pred(tasks_.at(q))) {
        id = q;
        found = true;
        break;
      }
    }
    if (!found) return std::nullopt;
    const uint64_t attempt = sat_add(tasks_.at(id).attempt, 1);
    const uint64_t expires = sat_add(now, cfg_.lease_ttl_ms());
    Json p = Json::object();
    p["worker_id"] = worker;
    p["expires_at"] = expires;
    append("task.claimed", id, attempt, p, worker, now);
    return Lease{id, worker, attempt, expires};
  }

  Lease heartbeat(const std::string& task, const std::string& worker, uint64_t attempt, uint64_t now) {
    require_holder(task, worker, attempt);
    const uint64_t expires = sat_add(now, cfg_.lease_ttl_ms());
    Json p = Json::object();
    p["expires_at"] = expires;
    append("task.heartbeat", task, attempt, p, worker, now);
    return Lease{task, worker, attempt, expires};
  }

  // Leases whose deadline has passed go back to the end of the queue.
  std::vector<std::string> expire_due(uint64_t now) {
    std::vector<std::pair<std::string, uint64_t>> due;
    for (const std::string& id : all_ids_) {
      const QueueTask& t = tasks_.at(id);
      if (t.state == TaskState::Leased && t.expires_at && *t.expires_at <= now)
        due.emplace_back(id, t.attempt);
    }
    std::vector<std::string> out;
    for (auto& d : due) {
      append("task.expired", d.first, d.second, Json::object(), std::nullopt, now);
      out.push_back(d.first);
    }
    return out;
  }

  void complete(const std::string& task, const std::string& worker, uint64_t attempt,
                const std::string& output, uint64_t now) {
    require_holder(task, worker, attempt);
    persist_output(task, attempt, output);
    Json p = Json::object();
    p["output_hash"] = sha256_hex(output);
    append("task.output", task, attempt, p, worker, now);
    append("task.completed", task, attempt, p, worker, now);
  }

  void fail(const std::string& task, const std::string& worker, uint64_t attempt,
            const std::string& reason, uint64_t now) {
    require_holder(task, worker, attempt);
    Json p = Json::object();
    p["reason"] = reason;
    append("task.failed", task, attempt, p, worker, now);
  }

  const QueueTask* get(const std::string& task) const {
    auto it = tasks_.find(task);
    return it == tasks_.end() ? nullptr : &it->second;
  }

  std::optional<std::string> get_output(const std::string& task, uint64_t attempt) const {
    if (!tasks_.count(task)) throw Error("NotFound", "not found: " + task);
    const std::string path = output_path(task, attempt);
    if (!file_exists(path)) return std::nullopt;
    return read_file(path);
  }

  static std::string checkpoint_branch(const std::string& task, uint64_t attempt) {
    return "task/" + task + "/attempt/" + std::to_string(attempt);
  }

  const EventLog& log() const { return *log_; }
  const std::string& dir() const { return dir_; }
  const QueueConfig& config() const { return cfg_; }
  size_t queued_len() const { return queued_.size(); }
  std::vector<std::string> queued_ids() const { return {queued_.begin(), queued_.end()}; }
  const std::vector<std::string>& all_ids() const { return all_ids_; }

 private:
  LeaseQueue(std::string dir, QueueConfig cfg) : dir_(std::move(dir)), cfg_(cfg) {}

  void require_holder(const std::string& task, const std::string& worker, uint64_t attempt) const {
    auto it = tasks_.find(task);
    if (it == tasks_.end()) throw Error("NotFound", "not found: " + task);
    const QueueTask& t = it->second;
    if (t.attempt != attempt)
      throw Error("StaleAttempt", "stale attempt: task=" + task + " attempt=" + std::to_string(attempt) +
                                      " current=" + std::to_string(t.attempt));
    if (t.state != TaskState::Leased || !t.worker_id || *t.worker_id != worker)
      throw Error("NotHolder", "not holder: task=" + task + " worker=" + worker +
                                   " attempt=" + std::to_string(attempt));
  }

  void append(const std::string& type, const std::string& task, std::optional<uint64_t> attempt,
              const Json& payload, std::optional<std::string> node, uint64_t now) {
    LogAppend a;
    a.event_type = type;
    a.payload = payload;
    a.timestamp = std::to_string(now);
    a.task_id = task;
    a.attempt = attempt;
    a.node_id = std::move(node);
    try {
      const LogEvent& e = log_->append(a);
      apply(e);
    } catch (const Error& e) {
      if (e.kind == "Duplicate" || e.kind == "Log") throw;
      throw Error("Log", e.what());
    }
  }

  QueueTask& task_mut(const std::string& id) {
    auto it = tasks_.find(id);
    if (it == tasks_.end()) throw Error("Log", "replay of unknown task " + id);
    return it->second;
  }
  void drop_queued(const std::string& id) {
    for (auto it = queued_.begin(); it != queued_.end();)
      it = (*it == id) ? queued_.erase(it) : it + 1;
  }

  void apply(const LogEvent& e) {
    if (!e.task_id)
      throw Error("Log", "event " + e.event_type + " seq " + std::to_string(e.seq) + " missing task_id");
    const std::string id = *e.task_id;
    const std::string& ty = e.event_type;
    auto u64_field = [&](const char* k) -> std::optional<uint64_t> {
      const Json* v = e.payload.find(k);
      if (v && v->is_integer()) return v->as_u64();
      return std::nullopt;
    };
    auto str_field = [&](const char* k) -> std::optional<std::string> {
      const Json* v = e.payload.find(k);
      if (v && v->is_string()) return v->as_string();
      return std::nullopt;
    };
    if (ty == "task.enqueued") {
      if (tasks_.count(id)) throw Error("Duplicate", "duplicate: " + id);
      QueueTask t;
      t.id = id;
      t.payload = e.payload;
      t.attempt = e.attempt.value_or(0);
      tasks_[id] = t;
      all_ids_.push_back(id);
      queued_.push_back(id);
    } else if (ty == "task.claimed") {
      QueueTask& t = task_mut(id);
      t.attempt = e.attempt ? *e.attempt : sat_add(t.attempt, 1);
      t.state = TaskState::Leased;
      t.worker_id = e.node_id ? e.node_id : str_field("worker_id");
      t.expires_at = u64_field("expires_at");
      drop_queued(id);
    } else if (ty == "task.heartbeat") {
      task_mut(id).expires_at = u64_field("expires_at");
    } else if (ty == "task.expired") {
      QueueTask& t = task_mut(id);
      t.state = TaskState::Queued;
      t.worker_id.reset();
      t.expires_at.reset();
      bool present = false;
      for (const auto& q : queued_) present = present || q == id;
      if (!present) queued_.push_back(id);
    } else if (ty == "task.output") {
      task_mut(id).output_hash = str_field("output_hash");
    } else if (ty == "task.completed") {
      QueueTask& t = task_mut(id);
      t.state = TaskState::Completed;
      t.expires_at.reset();
      if (auto h = str_field("output_hash")) t.output_hash = h;
      drop_queued(id);
    } else if (ty == "task.failed") {
      QueueTask& t = task_mut(id);
      t.state = TaskState::Failed;
      t.expires_at.reset();
      drop_queued(id);
    } else {
      throw Error("Log", "unknown event type " + ty + " at seq " + std::to_string(e.seq));
    }
  }

  std::string output_path(const std::string& task, uint64_t attempt) const {
    return dir_ + "/outputs/" + task + "/" + std::to_string(attempt);
  }
  void persist_output(const std::string& task, uint64_t attempt, const std::string& out) const {
    const std::string tdir = dir_ + "/outputs/" + task;
    make_dirs(tdir);
    const std::string path = tdir + "/" + std::to_string(attempt);
    const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) throw Error("Other", path + ": " + std::strerror(errno));
    size_t done = 0;
    while (done < out.size()) {
      const ssize_t w = ::write(fd, out.data() + done, out.size() - done);
      if (w < 0) {
        if (errno == EINTR) continue;
        ::close(fd);
        throw Error("Other", path + ": " + std::strerror(errno));
      }
      done += static_cast<size_t>(w);
    }
    ::fsync(fd);
    ::close(fd);
    fsync_dir(tdir);
    fsync_dir(dir_ + "/outputs");
  }

  std::string dir_;
  QueueConfig cfg_;
  std::unique_ptr<EventLog> log_;
  std::map<std::string, QueueTask> tasks_;
  std::vector<std::string> all_ids_;
  std::deque<std::string> queued_;
};

}  // namespace pbn
