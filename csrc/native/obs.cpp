// Observability: kind-checked metrics, nested spans, a run registry with hash-chained
// events, loss-spike detection, step-stamped metric series with a JSONL sink, and
// dashboard snapshots.
//
// Behavioural parity with the reference obs crate (obs/src/lib.rs): Metrics (:104-158),
// Tracer with LIFO span discipline (:175-215), RunRegistry whose per-run event chain
// starts at seq 1 with a 64-zero genesis hash and hashes
// sha256("{seq}|{prev}|{payload_hash}|{timestamp}|{event_type}") over the canonical
// (sorted-key, compact) payload (:219-350), SpikeLog with a rolling-mean baseline and the
// Log / SkipShard / Rollback / Page actions (:388-554), MetricLog (:566-602) and
// snapshot (:604-674). Added here: an injectable clock for the tracer, durable JSONL
// output of the metric log, and event-chain verification.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <chrono>
#include <ctime>
#include <map>
#include <optional>
#include <set>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace obs {

using Labels = std::map<std::string, std::string>;
static const char* kGenesis = "0000000000000000000000000000000000000000000000000000000000000000";

enum class MetricKind { Counter, Gauge, Histogram };

class Metrics {
 public:
  void inc(const std::string& name, const Labels& l, double amount) {
    kind(name, MetricKind::Counter);
    series_[name][l] += amount;
  }
  void set(const std::string& name, const Labels& l, double value) {
    kind(name, MetricKind::Gauge);
    series_[name][l] = value;
  }
  void observe(const std::string& name, const Labels& l, double value) {
    kind(name, MetricKind::Histogram);
    series_[name][l] += value;
    ++counts_[name][l];
  }
  std::optional<double> get(const std::string& name, const Labels& l) const {
    auto it = series_.find(name);
    if (it == series_.end()) return std::nullopt;
    auto jt = it->second.find(l);
    if (jt == it->second.end()) return std::nullopt;
    return jt->second;
  }
  uint64_t count(const std::string& name, const Labels& l) const {
    auto it = counts_.find(name);
    if (it == counts_.end()) return 0;
    auto jt = it->second.find(l);
    return jt == it->second.end() ? 0 : jt->second;
  }
  std::vector<std::string> names() const {
    std::vector<std::string> out;
    for (const auto& kv : kinds_) out.push_back(kv.first);
    return out;
  }

 private:
  void kind(const std::string& name, MetricKind k) {
    auto it = kinds_.find(name);
    if (it == kinds_.end()) kinds_[name] = k;
    else if (it->second != k) throw Error("KindMismatch", "metric kind mismatch for " + name);
  }
  std::map<std::string, MetricKind> kinds_;
  std::map<std::string, std::map<Labels, double>> series_;
  std::map<std::string, std::map<Labels, uint64_t>> counts_;
};

// Nested spans. `end` must be called on the innermost open span. The clock is the
// steady clock unless `set_now_ms` injects one (tests, replay).
class Tracer {
 public:
  uint64_t start(const std::string& name) {
    stack_.push_back({name, now_ms(), ++next_id_});
    return next_id_;
  }
  double end(uint64_t span_id) {
    if (stack_.empty() || stack_.back().id != span_id)
      throw Error("Other", "span is not the innermost open span on this tracer");
    const double t0 = stack_.back().start_ms;
    stack_.pop_back();
    return now_ms() - t0;
  }
  std::optional<std::string> current() const {
    if (stack_.empty()) return std::nullopt;
    return stack_.back().name;
  }
  size_t depth() const { return stack_.size(); }
  void set_now_ms(std::optional<double> t) { injected_ = t; }

 private:
  double now_ms() const {
    if (injected_) return *injected_;
    return std::chrono::duration<double, std::milli>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
  }
  struct Open {
    std::string name;
    double start_ms;
    uint64_t id;
  };
  std::vector<Open> stack_;
  uint64_t next_id_ = 0;
  std::optional<double> injected_;
};

inline std::string payload_hash(const Json& payload) { return sha256_hex(payload.dump()); }
inline std::string event_hash(uint64_t seq, const std::string& prev, const std::string& phash,
                              const std::string& ts, const std::string& type) {
  return sha256_hex(std::to_string(seq) + "|" + prev + "|" + phash + "|" + ts + "|" + type);
}
inline std::string rfc3339_utc(uint64_t secs) {
  std::time_t t = static_cast<std::time_t>(secs);
  std::tm tm{};
  gmtime_r(&t, &tm);
  char buf[32];
  std::strftime(buf, sizeof(buf), "%Y-%m-%dT%H:%M:%SZ", &tm);
  return buf;
}

struct RunRecord {
  std::string run_id, kind, status = "pending", config_hash, created_at;
  std::optional<std::string> parent_run_id;
};
struct Event {
  uint64_t seq = 0;
  std::string prev_hash, hash, timestamp, event_type, payload_json, payload_hash;
  Json to_value() const {
    Json o = Json::object();
    o["schema_id"] = "prometheus.event_log";
    o["schema_version"] = uint64_t(1);
    o["seq"] = seq;
    o["prev_hash"] = prev_hash;
    o["hash"] = hash;
    o["timestamp"] = timestamp;
    o["event_type"] = event_type;
    o["payload"] = Json::parse(payload_json);
    o["payload_hash"] = payload_hash;
    o["task_id"] = Json();
    o["attempt"] = Json();
    o["node_id"] = Json();
    return o;
  }
};

class RunRegistry {
 public:
  void register_run(const RunRecord& r) {
    static const std::set<std::string> ok = {"pending", "running", "completed", "failed", "cancelled"};
    if (!ok.count(r.status)) throw Error("Other", "unknown run status " + r.status);
    if (runs_.count(r.run_id)) throw Error("DuplicateRun", "duplicate run " + r.run_id);
    runs_[r.run_id] = r;
  }
  RunRecord get(const std::string& id) const {
    auto it = runs_.find(id);
    if (it == runs_.end()) throw Error("UnknownRun", "unknown run " + id);
    return it->second;
  }
  void set_status(const std::string& id, const std::string& status) {
    static const std::set<std::string> ok = {"pending", "running", "completed", "failed", "cancelled"};
    if (!ok.count(status)) throw Error("Other", "unknown run status " + status);
    auto it = runs_.find(id);
    if (it == runs_.end()) throw Error("UnknownRun", "unknown run " + id);
    it->second.status = status;
  }
  std::vector<RunRecord> list() const {
    std::vector<RunRecord> out;
    for (const auto& kv : runs_) out.push_back(kv.second);
    return out;
  }
  Event append_event(const std::string& run, const std::string& type, const std::string& payload_json,
                     std::optional<std::string> timestamp) {
    if (!runs_.count(run)) throw Error("UnknownRun", "unknown run " + run);
    auto& chain = events_[run];
    Event e;
    e.seq = chain.empty() ? 1 : chain.back().seq + 1;
    e.prev_hash = chain.empty() ? kGenesis : chain.back().hash;
    e.timestamp = timestamp ? *timestamp : rfc3339_utc(static_cast<uint64_t>(std::time(nullptr)));
    const Json payload = Json::parse(payload_json);
    e.payload_json = payload.dump();
    e.payload_hash = payload_hash(payload);
    e.event_type = type;
    e.hash = event_hash(e.seq, e.prev_hash, e.payload_hash, e.timestamp, type);
    chain.push_back(e);
    return e;
  }
  std::vector<Event> events(const std::string& run) const {
    if (!runs_.count(run)) throw Error("UnknownRun", "unknown run " + run);
    auto it = events_.find(run);
    return it == events_.end() ? std::vector<Event>{} : it->second;
  }
  // True when the run's chain is continuous and every hash recomputes.
  bool verify(const std::string& run) const {
    std::string prev = kGenesis;
    uint64_t seq = 1;
    for (const auto& e : events(run)) {
      if (e.seq != seq || e.prev_hash != prev) return false;
      if (payload_hash(Json::parse(e.payload_json)) != e.payload_hash) return false;
      if (event_hash(e.seq, e.prev_hash, e.payload_hash, e.timestamp, e.event_type) != e.hash) return false;
      prev = e.hash;
      ++seq;
    }
    return true;
  }

 private:
  std::map<std::string, RunRecord> runs_;
  std::map<std::string, std::vector<Event>> events_;
};

struct SpikeEvent {
  uint64_t step;
  double loss, baseline;
  std::string shard_id, run_id;
};
struct SkipShardRecord {
  std::string shard_id;
  uint64_t step;
  std::string run_id, reason;
};
struct SpikeAction {
  std::string kind;  // log | skip_shard | rollback | page
  std::optional<SpikeEvent> event;
  std::string shard_id, message;
  uint64_t checkpoint_step = 0;
};

class SpikeLog {
 public:
  SpikeLog(uint64_t page_window, double rel_threshold, size_t baseline_window, uint64_t last_ckpt)
      : page_window_(page_window), thr_(rel_threshold), window_(baseline_window),
        last_checkpoint_step(last_ckpt) {}
  std::vector<SpikeAction> observe(uint64_t step, double loss, const std::string& shard,
                                   const std::string& run) {
    if (thr_ <= 0.0) throw Error("BadSpikeConfig", "spike config: relative_threshold must be > 0");
    if (window_ == 0) throw Error("BadSpikeConfig", "spike config: baseline_window must be > 0");
    if (!std::isfinite(loss)) throw Error("BadSpikeConfig", "spike config: loss must be finite");
    if (history_.size() < window_) {
      history_.push_back(loss);
      return {};
    }
    double base = 0;
    for (size_t i = history_.size() - window_; i < history_.size(); ++i) base += history_[i];
    base /= static_cast<double>(window_);
    const bool spike = base > 0.0 && loss > base * (1.0 + thr_);
    history_.push_back(loss);
    if (!spike) return {};
    bool page = false;
    for (const auto& p : spikes_) {
      const uint64_t dist = step > p.step ? step - p.step : p.step - step;
      if (dist <= page_window_) page = true;
    }
    SpikeEvent ev{step, loss, base, shard, run};
    spikes_.push_back(ev);
    skipped_.push_back({shard, step, run, "loss_spike"});
    std::vector<SpikeAction> acts(3);
    acts[0].kind = "log";
    acts[0].event = ev;
    acts[1].kind = "skip_shard";
    acts[1].shard_id = shard;
    acts[2].kind = "rollback";
    acts[2].checkpoint_step = last_checkpoint_step;
    if (page) {
      SpikeAction a;
      a.kind = "page";
      a.message = "page run_id=" + run + " step=" + std::to_string(step);
      acts.push_back(a);
    }
    return acts;
  }
  const std::vector<SkipShardRecord>& skipped_shards() const { return skipped_; }
  const std::vector<SpikeEvent>& spikes() const { return spikes_; }

 private:
  uint64_t page_window_;
  double thr_;
  size_t window_;

 public:
  uint64_t last_checkpoint_step;

 private:
  std::vector<SkipShardRecord> skipped_;
  std::vector<SpikeEvent> spikes_;
  std::vector<double> history_;
};

class MetricLog {
 public:
  void record(const std::string& name, const Labels& l, uint64_t step, double value) {
    data_[name][l][step] = value;
    if (sink_) {
      Json o = Json::object();
      o["name"] = name;
      o["step"] = step;
      o["value"] = value;
      Json lab = Json::object();
      for (const auto& kv : l) lab[kv.first] = kv.second;
      o["labels"] = lab;
      const std::string line = o.dump() + "\n";
      std::fwrite(line.data(), 1, line.size(), sink_);
      std::fflush(sink_);
    }
  }
  std::vector<std::pair<uint64_t, double>> series(const std::string& name, const Labels& l) const {
    if (data_.empty()) throw Error("EmptyHistory", "spike log is empty");
    auto it = data_.find(name);
    if (it == data_.end()) throw Error("UnknownMetric", "unknown metric " + name);
    auto jt = it->second.find(l);
    if (jt == it->second.end()) throw Error("UnknownMetric", "unknown metric " + name);
    return {jt->second.begin(), jt->second.end()};
  }
  void open_sink(const std::string& path) {
    close_sink();
    sink_ = std::fopen(path.c_str(), "ab");
    if (!sink_) throw Error("Other", "cannot open " + path);
  }
  void close_sink() {
    if (sink_) std::fclose(sink_);
    sink_ = nullptr;
  }
  ~MetricLog() { close_sink(); }

 private:
  std::map<std::string, std::map<Labels, std::map<uint64_t, double>>> data_;
  FILE* sink_ = nullptr;
};

struct Panel {
  std::string id, title, metric_name, kind;  // timeseries | gauge | table | log
};
struct Dashboard {
  std::string id, title;
  std::vector<Panel> panels;
};

// JSON snapshot {"dashboard_id", "generated_at", "panels": [{"panel_id", "points"}], "recent_spikes"}
static std::string snapshot(const Dashboard& d, const MetricLog& log, const std::vector<SpikeEvent>& spikes,
                            const std::string& generated_at) {
  Json out = Json::object();
  out["dashboard_id"] = d.id;
  out["generated_at"] = generated_at;
  Json panels = Json::array();
  for (const auto& p : d.panels) {
    Json ps = Json::object();
    ps["panel_id"] = p.id;
    Json pts = Json::array();
    if (p.kind == "timeseries" || p.kind == "gauge") {
      const auto series = log.series(p.metric_name, Labels{});
      if (series.empty()) throw Error("EmptyHistory", "spike log is empty");
      for (const auto& sv : series) {
        Json pt = Json::object();
        pt["step"] = sv.first;
        pt["value"] = sv.second;
        pts.push(pt);
      }
    } else if (p.kind != "table" && p.kind != "log") {
      throw Error("Other", "unknown panel kind " + p.kind);
    }
    ps["points"] = pts;
    panels.push(ps);
  }
  out["panels"] = panels;
  Json sp = Json::array();
  for (const auto& s : spikes) {
    Json e = Json::object();
    e["step"] = s.step;
    e["loss"] = s.loss;
    e["baseline"] = s.baseline;
    e["shard_id"] = s.shard_id;
    e["run_id"] = s.run_id;
    sp.push(e);
  }
  out["recent_spikes"] = sp;
  return out.dump();
}

}  // namespace obs

void bind_obs(py::module_& m) {
  using namespace obs;
  m.attr("GENESIS_HASH") = kGenesis;
  m.attr("PAGE_WINDOW_STEPS") = 10000;
  py::class_<Metrics>(m, "Metrics")
      .def(py::init<>())
      .def("inc", &Metrics::inc, py::arg("name"), py::arg("labels") = Labels{}, py::arg("amount") = 1.0)
      .def("set", &Metrics::set, py::arg("name"), py::arg("labels"), py::arg("value"))
      .def("observe", &Metrics::observe, py::arg("name"), py::arg("labels"), py::arg("value"))
      .def("get", &Metrics::get, py::arg("name"), py::arg("labels") = Labels{})
      .def("count", &Metrics::count, py::arg("name"), py::arg("labels") = Labels{})
      .def("names", &Metrics::names);
  py::class_<Tracer>(m, "Tracer")
      .def(py::init<>())
      .def("start", &Tracer::start)
      .def("end", &Tracer::end)
      .def("current", &Tracer::current)
      .def("depth", &Tracer::depth)
      .def("set_now_ms", &Tracer::set_now_ms);
  py::class_<RunRecord>(m, "RunRecord")
      .def(py::init([](std::string id, std::string kind, std::string status, std::string cfg,
                       std::string created, std::optional<std::string> parent) {
             return RunRecord{std::move(id), std::move(kind), std::move(status), std::move(cfg),
                              std::move(created), std::move(parent)};
           }),
           py::arg("run_id"), py::arg("kind"), py::arg("status") = "pending",
           py::arg("config_hash") = "", py::arg("created_at") = "", py::arg("parent_run_id") = py::none())
      .def_readwrite("run_id", &RunRecord::run_id).def_readwrite("kind", &RunRecord::kind)
      .def_readwrite("status", &RunRecord::status).def_readwrite("config_hash", &RunRecord::config_hash)
      .def_readwrite("created_at", &RunRecord::created_at)
      .def_readwrite("parent_run_id", &RunRecord::parent_run_id);
  py::class_<Event>(m, "Event")
      .def_readonly("seq", &Event::seq).def_readonly("prev_hash", &Event::prev_hash)
      .def_readonly("hash", &Event::hash).def_readonly("timestamp", &Event::timestamp)
      .def_readonly("event_type", &Event::event_type).def_readonly("payload_json", &Event::payload_json)
      .def_readonly("payload_hash", &Event::payload_hash)
      .def("to_json", [](const Event& e) { return e.to_value().dump(); });
  py::class_<RunRegistry>(m, "RunRegistry")
      .def(py::init<>())
      .def("register", &RunRegistry::register_run)
      .def("get", &RunRegistry::get)
      .def("set_status", &RunRegistry::set_status)
      .def("list", &RunRegistry::list)
      .def("append_event", &RunRegistry::append_event, py::arg("run_id"), py::arg("event_type"),
           py::arg("payload_json"), py::arg("timestamp") = py::none())
      .def("events", &RunRegistry::events)
      .def("verify", &RunRegistry::verify);
  m.def("payload_hash", [](const std::string& json) { return payload_hash(Json::parse(json)); });
  m.def("event_hash", &event_hash);
  m.def("rfc3339_utc", &rfc3339_utc);
  py::class_<SpikeEvent>(m, "SpikeEvent")
      .def_readonly("step", &SpikeEvent::step).def_readonly("loss", &SpikeEvent::loss)
      .def_readonly("baseline", &SpikeEvent::baseline).def_readonly("shard_id", &SpikeEvent::shard_id)
      .def_readonly("run_id", &SpikeEvent::run_id);
  py::class_<SkipShardRecord>(m, "SkipShardRecord")
      .def_readonly("shard_id", &SkipShardRecord::shard_id).def_readonly("step", &SkipShardRecord::step)
      .def_readonly("run_id", &SkipShardRecord::run_id).def_readonly("reason", &SkipShardRecord::reason);
  py::class_<SpikeAction>(m, "SpikeAction")
      .def_readonly("kind", &SpikeAction::kind).def_readonly("event", &SpikeAction::event)
      .def_readonly("shard_id", &SpikeAction::shard_id).def_readonly("message", &SpikeAction::message)
      .def_readonly("checkpoint_step", &SpikeAction::checkpoint_step);
  py::class_<SpikeLog>(m, "SpikeLog")
      .def(py::init<uint64_t, double, size_t, uint64_t>(), py::arg("page_window_steps") = 10000,
           py::arg("relative_threshold") = 0.5, py::arg("baseline_window") = 8,
           py::arg("last_checkpoint_step") = 0)
      .def("observe", &SpikeLog::observe, py::arg("step"), py::arg("loss"), py::arg("shard_id") = "",
           py::arg("run_id") = "")
      .def("skipped_shards", &SpikeLog::skipped_shards)
      .def("spikes", &SpikeLog::spikes)
      .def_readwrite("last_checkpoint_step", &SpikeLog::last_checkpoint_step);
  py::class_<MetricLog>(m, "MetricLog")
      .def(py::init<>())
      .def("record", &MetricLog::record, py::arg("name"), py::arg("labels"), py::arg("step"),
           py::arg("value"))
      .def("series", &MetricLog::series, py::arg("name"), py::arg("labels") = Labels{})
      .def("open_sink", &MetricLog::open_sink)
      .def("close_sink", &MetricLog::close_sink);
  py::class_<Panel>(m, "Panel")
      .def(py::init([](std::string id, std::string title, std::string metric, std::string kind) {
             return Panel{std::move(id), std::move(title), std::move(metric), std::move(kind)};
           }),
           py::arg("id"), py::arg("title"), py::arg("metric_name"), py::arg("kind") = "timeseries");
  py::class_<Dashboard>(m, "Dashboard")
      .def(py::init([](std::string id, std::string title, std::vector<Panel> panels) {
             return Dashboard{std::move(id), std::move(title), std::move(panels)};
           }));
  m.def("snapshot", &snapshot);
}
