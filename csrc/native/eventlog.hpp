// Durable hash-chained JSONL event log, the root dependency of the harness components.
//
// File format and semantics of the reference harness/log crate (harness/log/src/lib.rs):
// a directory holding `events.jsonl`, one event per line with the fields in the order
// schema_id, schema_version, seq, prev_hash, hash, timestamp, event_type, task_id, attempt,
// node_id, payload, payload_hash (:53-69); first seq 0, genesis prev-hash 64 zeros;
// payload_hash = sha256(canonical sorted-key compact JSON of the payload), hash =
// sha256("{seq}|{prev_hash}|{payload_hash}|{timestamp}|{event_type}") (:219-237); every
// append is flushed and fsync'd and rolled back on a write error (:262-272); open()
// replays and verifies the chain, truncates a torn last line, adds a missing trailing
// newline and fails closed on any broken link (:95-142, :274-351).
#pragma once

#include "common.hpp"

#include <optional>

namespace pbn {

struct LogEvent {
  uint64_t seq = 0;
  std::string prev_hash, hash, timestamp, event_type;
  std::optional<std::string> task_id;
  std::optional<uint64_t> attempt;
  std::optional<std::string> node_id;
  Json payload;
  std::string payload_hash;
  uint32_t schema_version = 1;

  std::string line() const {
    std::string out = "{\"schema_id\":\"prometheus.event_log\",\"schema_version\":";
    out += std::to_string(schema_version);
    out += ",\"seq\":" + std::to_string(seq);
    out += ",\"prev_hash\":";
    Json::write_string(out, prev_hash);
    out += ",\"hash\":";
    Json::write_string(out, hash);
    out += ",\"timestamp\":";
    Json::write_string(out, timestamp);
    out += ",\"event_type\":";
    Json::write_string(out, event_type);
    out += ",\"task_id\":";
    if (task_id) Json::write_string(out, *task_id); else out += "null";
    out += ",\"attempt\":";
    out += attempt ? std::to_string(*attempt) : std::string("null");
    out += ",\"node_id\":";
    if (node_id) Json::write_string(out, *node_id); else out += "null";
    out += ",\"payload\":";
    payload.write(out);
    out += ",\"payload_hash\":";
    Json::write_string(out, payload_hash);
    out += "}";
    return out;
  }
  static LogEvent parse(const std::string& text) {
    Json v;
    try {
      v = Json::parse(text);
    } catch (const Error& e) {
      throw Error("Corrupt", std::string("corrupt log: invalid json: ") + e.what());
    }
    LogEvent e;
    try {
      if (v.at("schema_id").as_string() != "prometheus.event_log")
        throw Error("Schema", "schema: schema_id " + v.at("schema_id").as_string());
      e.schema_version = static_cast<uint32_t>(v.at("schema_version").as_u64());
      e.seq = v.at("seq").as_u64();
      e.prev_hash = v.at("prev_hash").as_string();
      e.hash = v.at("hash").as_string();
      e.timestamp = v.at("timestamp").as_string();
      e.event_type = v.at("event_type").as_string();
      if (const Json* t = v.find("task_id")) if (!t->is_null()) e.task_id = t->as_string();
      if (const Json* a = v.find("attempt")) if (!a->is_null()) e.attempt = a->as_u64();
      if (const Json* n = v.find("node_id")) if (!n->is_null()) e.node_id = n->as_string();
      e.payload = v.at("payload");
      e.payload_hash = v.at("payload_hash").as_string();
    } catch (const Error& err) {
      if (err.kind == "Schema" && std::string(err.what()).rfind("schema:", 0) == 0) throw;
      throw Error("Corrupt", std::string("corrupt log: invalid json: ") + err.what());
    }
    return e;
  }
};

inline std::string log_payload_hash(const Json& payload) { return sha256_hex(payload.dump()); }
inline std::string log_event_hash(uint64_t seq, const std::string& prev, const std::string& ph,
                                  const std::string& ts, const std::string& type) {
  return sha256_hex(std::to_string(seq) + "|" + prev + "|" + ph + "|" + ts + "|" + type);
}
static const char* const kLogGenesis =
    "0000000000000000000000000000000000000000000000000000000000000000";

inline void verify_chain(const std::vector<LogEvent>& events) {
  std::string prev = kLogGenesis;
  for (size_t i = 0; i < events.size(); ++i) {
    const LogEvent& e = events[i];
    if (e.seq != i) throw Error("BrokenChain", "broken hash chain at seq " + std::to_string(e.seq));
    if (e.schema_version < 1 || e.schema_version > 1)
      throw Error("Schema", "schema: unknown schema_version " + std::to_string(e.schema_version));
    if (e.event_type.empty()) throw Error("Schema", "schema: event_type must be non-empty");
    if (e.prev_hash != prev) throw Error("BrokenChain", "broken hash chain at seq " + std::to_string(e.seq));
    if (e.payload_hash != log_payload_hash(e.payload))
      throw Error("Corrupt", "corrupt log: payload_hash mismatch at seq " + std::to_string(i));
    if (e.hash != log_event_hash(e.seq, e.prev_hash, e.payload_hash, e.timestamp, e.event_type))
      throw Error("Corrupt", "corrupt log: hash mismatch at seq " + std::to_string(i));
    prev = e.hash;
  }
}

struct LogAppend {
  std::string event_type;
  Json payload = Json::object();
  std::string timestamp;
  std::optional<std::string> task_id;
  std::optional<uint64_t> attempt;
  std::optional<std::string> node_id;
};

class EventLog {
 public:
  EventLog(const EventLog&) = delete;
  EventLog& operator=(const EventLog&) = delete;
  EventLog(EventLog&& o) noexcept : dir_(std::move(o.dir_)), events_(std::move(o.events_)), fd_(o.fd_) {
    o.fd_ = -1;
  }
  ~EventLog() {
    if (fd_ >= 0) ::close(fd_);
  }

  static std::unique_ptr<EventLog> create(const std::string& dir) {
    if (::mkdir(dir.c_str(), 0777) != 0)
      throw Error("Io", "io: create " + dir + ": " + std::strerror(errno));
    const std::string path = dir + "/events.jsonl";
    const int fd = ::open(path.c_str(), O_RDWR | O_CREAT | O_EXCL | O_APPEND, 0644);
    if (fd < 0) throw Error("Io", "io: " + path + ": " + std::strerror(errno));
    ::fsync(fd);
    fsync_dir(dir);
    const size_t slash = dir.find_last_of('/');
    if (slash != std::string::npos && slash > 0) fsync_dir(dir.substr(0, slash));
    return std::unique_ptr<EventLog>(new EventLog(dir, {}, fd));
  }

  static std::unique_ptr<EventLog> open(const std::string& dir) {
    if (!dir_exists(dir)) throw Error("Io", "io: log dir missing or not a directory: " + dir);
    const std::string path = dir + "/events.jsonl";
    const int fd = ::open(path.c_str(), O_RDWR | O_APPEND);
    if (fd < 0) throw Error("Io", "io: " + path + ": " + std::strerror(errno));
    std::string bytes;
    char buf[1 << 16];
    ssize_t n;
    while ((n = ::read(fd, buf, sizeof(buf))) > 0) bytes.append(buf, static_cast<size_t>(n));
    std::vector<LogEvent> events;
    size_t off = 0, complete_end = 0;
    bool needs_newline = false;
    try {
      while (off < bytes.size()) {
        const size_t nl = bytes.find('\n', off);
        if (nl != std::string::npos) {
          events.push_back(LogEvent::parse(bytes.substr(off, nl - off)));
          off = nl + 1;
          complete_end = off;
        } else {
          try {  // a last line without newline: keep it if it is a whole record, else it is torn
            events.push_back(LogEvent::parse(bytes.substr(off)));
            complete_end = bytes.size();
            needs_newline = true;
          } catch (const Error&) {
          }
          break;
        }
      }
      verify_chain(events);
    } catch (...) {
      ::close(fd);
      throw;
    }
    if (complete_end < bytes.size()) {
      if (::ftruncate(fd, static_cast<off_t>(complete_end)) != 0) {
        ::close(fd);
        throw Error("Io", "io: truncate failed");
      }
      ::fsync(fd);
    }
    if (needs_newline) {
      if (::write(fd, "\n", 1) != 1) {
        ::close(fd);
        throw Error("Io", "io: write failed");
      }
      ::fsync(fd);
    }
    return std::unique_ptr<EventLog>(new EventLog(dir, std::move(events), fd));
  }

  const LogEvent& append(const LogAppend& rec) {
    if (rec.event_type.empty()) throw Error("Schema", "schema: event_type must be non-empty");
    LogEvent e;
    e.seq = events_.size();
    e.prev_hash = events_.empty() ? kLogGenesis : events_.back().hash;
    e.payload = rec.payload;
    e.payload_hash = log_payload_hash(rec.payload);
    e.timestamp = rec.timestamp;
    e.event_type = rec.event_type;
    e.task_id = rec.task_id;
    e.attempt = rec.attempt;
    e.node_id = rec.node_id;
    e.hash = log_event_hash(e.seq, e.prev_hash, e.payload_hash, e.timestamp, e.event_type);
    const std::string line = e.line() + "\n";
    struct stat st;
    ::fstat(fd_, &st);
    const off_t start = st.st_size;
    size_t done = 0;
    bool ok = true;
    while (done < line.size()) {
      const ssize_t w = ::write(fd_, line.data() + done, line.size() - done);
      if (w < 0) {
        if (errno == EINTR) continue;
        ok = false;
        break;
      }
      done += static_cast<size_t>(w);
    }
    if (ok && ::fsync(fd_) != 0) ok = false;
    if (!ok) {
      const std::string msg = std::strerror(errno);
      if (::ftruncate(fd_, start) == 0) ::fsync(fd_);
      throw Error("Io", "io: append failed: " + msg);
    }
    events_.push_back(std::move(e));
    return events_.back();
  }

  size_t size() const { return events_.size(); }
  const std::vector<LogEvent>& events() const { return events_; }
  const LogEvent* get(uint64_t seq) const { return seq < events_.size() ? &events_[seq] : nullptr; }
  const std::string& dir() const { return dir_; }
  void verify() const { verify_chain(events_); }

 private:
  EventLog(std::string dir, std::vector<LogEvent> ev, int fd)
      : dir_(std::move(dir)), events_(std::move(ev)), fd_(fd) {}
  std::string dir_;
  std::vector<LogEvent> events_;
  int fd_;
};

}  // namespace pbn
