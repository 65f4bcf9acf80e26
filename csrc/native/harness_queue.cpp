// Harness components built on the lease queue and the event log:
//
//   cas       replicated content-addressed blob store with named pins and GC
//             (reference: harness/cas/src/lib.rs:20-25, 88-300)
//   mesh      capability adverts, pull-claim by capability, signed freeze, watcher ring
//             (reference: harness/mesh/src/lib.rs:18-19, 33-80, 105-407)
//   pipeline  oracle -> implementers -> review -> merge state machine on a lease queue
//             (reference: harness/pipeline/src/lib.rs:16-29, 119-186, 189-640)
//
// and the Python bindings of these and of LeaseQueue (queue.hpp).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <set>

#include "cas.hpp"
#include "queue.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

// ----------------------------------------------------------------------------------- mesh
struct Capabilities {
  uint32_t gpus = 0, cpus = 1;
  bool kvm = false;
  std::vector<std::string> providers;
};
struct Advert {
  std::string node, key;
  Capabilities caps;
  uint64_t at = 0;
};
struct Freeze {
  std::string payload, signer, signature;   // signature: raw bytes
};
struct Watch {
  std::string watcher, watchee;
};

bool caps_satisfy(const Capabilities& caps, const Json& payload) {
  const Json* req = payload.is_object() ? payload.find("requires") : nullptr;
  if (req == nullptr) return true;
  if (!req->is_object()) return false;
  auto u = [&](const char* k) -> uint64_t {
    const Json* v = req->find(k);
    return v && v->is_integer() ? v->as_u64() : 0;
  };
  const Json* kv = req->find("kvm");
  const bool kvm = kv && kv->is_bool() && kv->as_bool();
  if (caps.gpus < u("gpus") || caps.cpus < u("cpus")) return false;
  if (kvm && !caps.kvm) return false;
  if (const Json* ps = req->find("providers"); ps && ps->is_array()) {
    for (const Json& p : ps->arr()) {
      if (!p.is_string()) continue;
      bool have = false;
      for (const auto& mine : caps.providers) have = have || mine == p.as_string();
      if (!have) return false;
    }
  }
  return true;
}

class Mesh {
 public:
  Mesh(std::string dir, std::string id, std::string key, bool trusted, bool must_exist)
      : dir_(std::move(dir)), id_(std::move(id)), key_(std::move(key)), trusted_(trusted) {
    if (must_exist) {
      if (!dir_exists(dir_)) throw Error("NotFound", "not found: " + dir_);
      const std::string f = dir_ + "/freeze.json";
      if (file_exists(f)) {
        const Json v = Json::parse(read_file(f));
        Freeze c;
        c.payload = v.at("payload").as_string();
        c.signer = v.at("signer").as_string();
        for (const Json& b : v.at("signature").arr()) c.signature.push_back(static_cast<char>(b.as_u64()));
        freeze_ = c;
        frozen_ = true;
      }
    } else {
      if (file_exists(dir_) || dir_exists(dir_)) throw Error("AlreadyExists", "already exists: " + dir_);
      if (::mkdir(dir_.c_str(), 0777) != 0) throw Error("Other", dir_ + ": " + std::strerror(errno));
    }
  }

  Advert advertise(const Capabilities& caps, uint64_t now) {
    if (frozen_) throw Error("Frozen", "mesh is frozen");
    Advert a{id_, key_, caps, now};
    upsert(a);
    return a;
  }
  std::optional<Lease> pull(LeaseQueue& q, uint64_t now) {
    if (!trusted_) throw Error("Untrusted", "untrusted node cannot pull");
    if (frozen_) throw Error("Frozen", "mesh is frozen");
    Capabilities caps;
    bool have = false;
    uint64_t best = 0;
    for (const Advert& a : adverts_)
      if (a.node == id_ && (!have || a.at >= best)) {
        caps = a.caps;
        best = a.at;
        have = true;
      }
    try {
      return q.claim_if(id_, now, [&](const QueueTask& t) { return caps_satisfy(caps, t.payload); });
    } catch (const Error& e) {
      throw Error("Other", e.what());
    }
  }
  void freeze(const Freeze& cmd) {
    if (cmd.signature != cmd.payload) throw Error("BadSignature", "bad freeze signature");
    apply_freeze(cmd);
  }
  void apply_freeze(const Freeze& cmd) {
    Json v = Json::object();
    v["payload"] = cmd.payload;
    v["signer"] = cmd.signer;
    Json sig = Json::array();
    for (unsigned char c : cmd.signature) sig.arr().push_back(Json(static_cast<uint64_t>(c)));
    v["signature"] = sig;
    const std::string text = v.dump();
    const std::string path = dir_ + "/freeze.json";
    const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) throw Error("Other", path + ": " + std::strerror(errno));
    if (::write(fd, text.data(), text.size()) != static_cast<ssize_t>(text.size())) {
      ::close(fd);
      throw Error("Other", "short write: " + path);
    }
    ::close(fd);
    frozen_ = true;
    freeze_ = cmd;
  }
  void upsert(const Advert& a) {
    for (Advert& e : adverts_)
      if (e.node == a.node) {
        e = a;
        return;
      }
    adverts_.push_back(a);
  }

  std::string dir_, id_, key_;
  bool trusted_;
  std::vector<Advert> adverts_;
  bool frozen_ = false;
  std::optional<Freeze> freeze_;
  std::vector<Watch> watches_;
};

// In-process mesh of always-on slots "0".."n-1" (not a network transport).
class LocalMesh {
 public:
  LocalMesh(size_t n, const std::string& base) {
    if (n < 3) throw Error("TooFewNodes", "need at least 3 nodes for a watcher ring, have " + std::to_string(n));
    make_dirs(base);
    std::vector<Watch> ring;
    for (size_t i = 0; i < n; ++i) {   // node i is watched by (i+1) % n and (i+2) % n
      ring.push_back({std::to_string((i + 1) % n), std::to_string(i)});
      ring.push_back({std::to_string((i + 2) % n), std::to_string(i)});
    }
    for (size_t i = 0; i < n; ++i) {
      auto node = std::make_shared<Mesh>(base + "/" + std::to_string(i), std::to_string(i),
                                         "key-" + std::to_string(i), true, false);
      node->watches_ = ring;
      nodes_.push_back(node);
    }
  }
  std::shared_ptr<Mesh> get(size_t i) {
    if (i >= nodes_.size()) throw Error("NotFound", "not found: " + std::to_string(i));
    return nodes_[i];
  }
  void partition(const std::vector<size_t>& isolated) { isolated_ = {isolated.begin(), isolated.end()}; }
  void heal() { isolated_.clear(); }
  // Gossip among connected nodes: newest advert per node wins; a freeze known to any
  // connected node reaches all of them (so a partitioned node honours it once healed).
  void tick(uint64_t) {
    std::vector<size_t> conn;
    for (size_t i = 0; i < nodes_.size(); ++i)
      if (!isolated_.count(i)) conn.push_back(i);
    std::map<std::string, Advert> best;
    for (size_t i : conn)
      for (const Advert& a : nodes_[i]->adverts_) {
        auto it = best.find(a.node);
        if (it != best.end() && it->second.at > a.at) continue;
        best[a.node] = a;
      }
    std::vector<Advert> merged;
    for (auto& kv : best) merged.push_back(kv.second);
    std::optional<Freeze> fr;
    for (size_t i : conn)
      if (!fr && nodes_[i]->frozen_) fr = nodes_[i]->freeze_;
    for (size_t i : conn) {
      nodes_[i]->adverts_ = merged;
      if (fr) nodes_[i]->apply_freeze(*fr);
    }
  }
  size_t size() const { return nodes_.size(); }

 private:
  std::vector<std::shared_ptr<Mesh>> nodes_;
  std::set<size_t> isolated_;
};

// ------------------------------------------------------------------------------- pipeline
const char* const kPlantedBad = "PLANTED_BAD_PATCH";
enum class Stage { Interface, Oracle, StubMustFail, Implement, Review, Merged, Blocked };
const char* stage_name(Stage s) {
  static const char* n[] = {"Interface", "Oracle", "StubMustFail", "Implement", "Review", "Merged", "Blocked"};
  return n[static_cast<int>(s)];
}
struct Candidate {
  std::string id, angle, patch;   // patch: raw bytes
};
struct Verdict {
  bool pick = false;
  std::string candidate;              // when pick
  std::vector<std::string> defects;   // when reject-all
  Json to_json() const {
    Json v = Json::object();
    if (pick) {
      v["Pick"] = candidate;
    } else {
      Json d = Json::array();
      for (auto& s : defects) d.arr().push_back(Json(s));
      Json inner = Json::object();
      inner["defects"] = d;
      v["RejectAll"] = inner;
    }
    return v;
  }
  static std::optional<Verdict> from_json(const Json& v) {
    if (!v.is_object()) return std::nullopt;
    Verdict out;
    if (const Json* p = v.find("Pick"); p && p->is_string()) {
      out.pick = true;
      out.candidate = p->as_string();
      return out;
    }
    if (const Json* r = v.find("RejectAll"); r && r->is_object()) {
      if (const Json* d = r->find("defects"); d && d->is_array())
        for (const Json& s : d->arr())
          if (s.is_string()) out.defects.push_back(s.as_string());
      return out;
    }
    return std::nullopt;
  }
};

bool is_planted_bad(const std::string& patch) { return patch.find(kPlantedBad) != std::string::npos; }

Verdict review(const std::vector<Candidate>& cands, const std::vector<bool>& ok) {
  if (cands.size() != ok.size())
    throw Error("Other", "tests_ok length " + std::to_string(ok.size()) + " != candidates " +
                             std::to_string(cands.size()));
  Verdict v;
  for (size_t i = 0; i < cands.size(); ++i)
    if (ok[i] && !is_planted_bad(cands[i].patch)) {
      v.pick = true;
      v.candidate = cands[i].id;
      return v;
    }
  if (cands.empty()) {
    v.defects.push_back("no candidates");
  } else {
    for (size_t i = 0; i < cands.size(); ++i) {
      if (is_planted_bad(cands[i].patch)) v.defects.push_back("candidate " + cands[i].id + " is planted-bad");
      else if (!ok[i]) v.defects.push_back("candidate " + cands[i].id + " tests failed");
    }
    if (v.defects.empty()) v.defects.push_back("no candidate qualified");
  }
  return v;
}

void merge_allowed(const Verdict& v, const std::vector<Candidate>& cands, const std::vector<bool>& ok) {
  if (cands.size() != ok.size())
    throw Error("Other", "tests_ok length " + std::to_string(ok.size()) + " != candidates " +
                             std::to_string(cands.size()));
  if (!v.pick) throw Error("Other", "verdict is RejectAll");
  for (size_t i = 0; i < cands.size(); ++i)
    if (cands[i].id == v.candidate) {
      if (is_planted_bad(cands[i].patch)) throw Error("PlantedBad", "planted bad patch cannot be picked");
      if (!ok[i]) throw Error("CandidateFailed", "candidate tests failed");
      return;
    }
  throw Error("NoCandidate", "no such candidate: " + v.candidate);
}

// task id = role/module/round[/op][/candidate]; payload = extra + {module, role}
std::pair<std::string, Json> work_payload(const std::string& module, const std::string& role, Json extra) {
  if (!extra.is_object()) {
    Json m = Json::object();
    m["extra"] = extra;
    extra = m;
  }
  extra["module"] = module;
  extra["role"] = role;
  uint64_t round = 0;
  // only a non-negative JSON integer names a round; a negative, fractional or textual one reads as round 0
  if (const Json* r = extra.find("round"); r && (r->kind == Json::UInt || (r->kind == Json::Int && r->i >= 0)))
    round = r->as_u64();
  std::string id = role + "/" + module + "/" + std::to_string(round);
  if (const Json* op = extra.find("op"); op && op->is_string()) id += "/" + op->as_string();
  if (const Json* c = extra.find("candidate"); c && c->is_string()) id += "/" + c->as_string();
  return {id, extra};
}

class Pipeline {
 public:
  Pipeline(const std::string& dir, std::string module, uint32_t n_impl, uint32_t max_rounds,
           QueueConfig qc, bool existing)
      : dir_(dir), module_(std::move(module)), n_impl_(n_impl), max_rounds_(max_rounds) {
    if (!existing) {
      if (file_exists(dir) || dir_exists(dir)) throw Error("Other", "directory exists: " + dir);
      if (::mkdir(dir.c_str(), 0777) != 0) throw Error("Other", dir + ": " + std::strerror(errno));
      queue_ = LeaseQueue::create(dir + "/queue", qc);
    } else {
      if (!dir_exists(dir)) throw Error("NotFound", "not found: pipeline dir missing: " + dir);
      queue_ = LeaseQueue::open(dir + "/queue", qc);
      replay();
    }
  }

  std::string start_oracle(uint64_t now) {
    require(Stage::Interface);
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    const std::string id = enqueue(work_payload(module_, "oracle", x), now);
    stage_ = Stage::Oracle;
    return id;
  }
  void record_oracle(bool passed_on_stub, uint64_t now) {
    require(Stage::Oracle);
    if (passed_on_stub) throw Error("StubPassed", "oracle tests passed the stub");
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    x["op"] = "record_oracle";
    x["passed_on_stub"] = false;
    enqueue(work_payload(module_, "pipeline", x), now);
    stub_failed_ = true;
    stage_ = Stage::StubMustFail;
  }
  std::vector<std::string> start_implementers(uint64_t now) {
    if (!stub_failed_) throw Error("StubNotFailed", "stub has not been shown to fail");
    require(Stage::StubMustFail);
    auto ids = enqueue_implementers(now);
    stage_ = Stage::Implement;
    return ids;
  }
  void submit_candidate(const Candidate& c, uint64_t now) {
    require(Stage::Implement);
    bool expected = false;
    for (auto& e : expected_) expected = expected || e == c.id;
    if (!expected) throw Error("NoCandidate", "no such candidate: " + c.id);
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    x["op"] = "submit_candidate";
    x["candidate"] = c.id;
    x["angle"] = c.angle;
    Json bytes = Json::array();
    for (unsigned char b : c.patch) bytes.arr().push_back(Json(static_cast<uint64_t>(b)));
    x["patch"] = bytes;
    auto item = work_payload(module_, "pipeline", x);
    if (queue_->get(item.first) != nullptr) {   // a resubmission gets a fresh task id
      const std::string base = item.first;
      for (uint32_t n = 1;; ++n) {
        const std::string tid = base + "#" + std::to_string(n);
        if (queue_->get(tid) == nullptr) {
          item.first = tid;
          break;
        }
      }
    }
    enqueue(item, now);
    upsert(c);
  }
  std::string start_review(uint64_t now) {
    require(Stage::Implement);
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    const std::string id = enqueue(work_payload(module_, "reviewer", x), now);
    stage_ = Stage::Review;
    return id;
  }
  Stage record_verdict(const Verdict& v, uint64_t now) {
    require(Stage::Review);
    if (v.pick) check_pick(v.candidate);
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    x["op"] = "record_verdict";
    x["verdict"] = v.to_json();
    enqueue(work_payload(module_, "pipeline", x), now);
    apply_verdict(v, now, true);
    return stage_;
  }
  void record_merge(const std::string& module, const std::string& spec_section, const std::string& commit,
                    uint32_t passed, uint32_t failed, const std::vector<std::string>& jobs, uint64_t now) {
    require(Stage::Merged);
    if (module != module_) throw Error("Other", "merge record module mismatch");
    if (!last_ || !last_->pick) throw Error("Other", "record_merge requires a Pick verdict");
    check_pick(last_->candidate);
    Json rec = Json::object();
    rec["module"] = module;
    rec["spec_section"] = spec_section;
    rec["commit"] = commit;
    rec["tests_passed"] = uint64_t(passed);
    rec["tests_failed"] = uint64_t(failed);
    Json j = Json::array();
    for (auto& s : jobs) j.arr().push_back(Json(s));
    rec["gpu_job_ids"] = j;
    Json x = Json::object();
    x["round"] = uint64_t(round_);
    x["op"] = "record_merge";
    x["record"] = rec;
    enqueue(work_payload(module_, "pipeline", x), now);
  }

  Stage stage() const { return stage_; }
  uint32_t round() const { return round_; }
  bool stub_failed() const { return stub_failed_; }
  const std::vector<Candidate>& candidates() const { return submitted_; }
  LeaseQueue& queue() { return *queue_; }
  const std::string& module() const { return module_; }

 private:
  void require(Stage want) const {
    if (stage_ != want)
      throw Error("WrongStage", std::string("wrong stage: expected ") + stage_name(want) + ", at " +
                                    stage_name(stage_));
  }
  void check_pick(const std::string& id) const {
    for (auto& c : submitted_)
      if (c.id == id) {
        if (is_planted_bad(c.patch)) throw Error("PlantedBad", "planted bad patch cannot be picked");
        return;
      }
    throw Error("NoCandidate", "no such candidate: " + id);
  }
  std::string enqueue(const std::pair<std::string, Json>& item, uint64_t now) {
    return queue_->enqueue(item.first, item.second, now);
  }
  std::vector<std::string> enqueue_implementers(uint64_t now) {
    expected_.clear();
    submitted_.clear();
    std::vector<std::string> ids;
    for (uint32_t i = 0; i < n_impl_; ++i) {
      Json x = Json::object();
      x["round"] = uint64_t(round_);
      x["candidate"] = std::to_string(i);
      ids.push_back(enqueue(work_payload(module_, "implementer", x), now));
      expected_.push_back(std::to_string(i));
    }
    return ids;
  }
  void apply_verdict(const Verdict& v, uint64_t now, bool live) {
    last_ = v;
    if (v.pick) {
      stage_ = Stage::Merged;
      return;
    }
    round_ = round_ == UINT32_MAX ? round_ : round_ + 1;
    submitted_.clear();
    expected_.clear();
    if (round_ >= max_rounds_) {
      stage_ = Stage::Blocked;
    } else {
      if (live) enqueue_implementers(now);
      stage_ = Stage::Implement;
    }
  }
  void upsert(const Candidate& c) {
    for (auto& s : submitted_)
      if (s.id == c.id) {
        s = c;
        return;
      }
    submitted_.push_back(c);
  }
  void replay() {
    for (const LogEvent& e : queue_->log().events()) {
      if (e.event_type != "task.enqueued") continue;
      const Json& p = e.payload;
      auto str = [&](const char* k) {
        const Json* v = p.is_object() ? p.find(k) : nullptr;
        return v && v->is_string() ? v->as_string() : std::string();
      };
      auto num = [&](const char* k) -> std::optional<uint64_t> {
        const Json* v = p.is_object() ? p.find(k) : nullptr;
        if (v && v->is_integer()) return v->as_u64();
        return std::nullopt;
      };
      const std::string role = str("role"), op = str("op");
      if (role == "oracle") {
        stage_ = Stage::Oracle;
        if (auto r = num("round")) round_ = static_cast<uint32_t>(*r);
      } else if (role == "pipeline" && op == "record_oracle") {
        const Json* v = p.find("passed_on_stub");
        if (!(v && v->is_bool() && v->as_bool())) {
          stub_failed_ = true;
          stage_ = Stage::StubMustFail;
        }
      } else if (role == "implementer") {
        if (auto r = num("round"); r && static_cast<uint32_t>(*r) != round_) {
          round_ = static_cast<uint32_t>(*r);
          expected_.clear();
          submitted_.clear();
        }
        const std::string c = str("candidate");
        if (p.find("candidate") != nullptr && p.find("candidate")->is_string()) {
          bool have = false;
          for (auto& x : expected_) have = have || x == c;
          if (!have) expected_.push_back(c);
        }
        stage_ = Stage::Implement;
      } else if (role == "pipeline" && op == "submit_candidate") {
        Candidate c;
        c.id = str("candidate");
        c.angle = str("angle");
        if (const Json* b = p.find("patch"); b && b->is_array())
          for (const Json& x : b->arr())
            if (x.is_integer()) c.patch.push_back(static_cast<char>(x.as_u64()));
        upsert(c);
      } else if (role == "reviewer") {
        stage_ = Stage::Review;
      } else if (role == "pipeline" && op == "record_verdict") {
        if (const Json* v = p.find("verdict"))
          if (auto verdict = Verdict::from_json(*v)) apply_verdict(*verdict, 0, false);
      } else if (role == "pipeline" && op == "record_merge") {
        stage_ = Stage::Merged;
      }
    }
  }

  std::string dir_, module_;
  uint32_t n_impl_, max_rounds_;
  std::unique_ptr<LeaseQueue> queue_;
  Stage stage_ = Stage::Interface;
  uint32_t round_ = 0;
  bool stub_failed_ = false;
  std::vector<std::string> expected_;
  std::vector<Candidate> submitted_;
  std::optional<Verdict> last_;
};

py::object lease_to_py(const std::optional<Lease>& l) {
  if (!l) return py::none();
  return py::cast(*l);
}

}  // namespace

void bind_harness_queue(py::module_& m) {
  // ---- leases
  auto lm = m.def_submodule("leases", "durable FIFO work queue with leases and attempt-keyed outputs");
  lm.attr("DEFAULT_HEARTBEAT_PERIOD_MS") = 15000;
  lm.attr("MISSED_HEARTBEATS") = 2;
  py::class_<QueueConfig>(lm, "QueueConfig")
      .def(py::init([](uint64_t period, uint32_t missed) {
             QueueConfig c;
             c.heartbeat_period_ms = period;
             c.missed_heartbeats = missed;
             return c;
           }),
           py::arg("heartbeat_period_ms") = 15000, py::arg("missed_heartbeats") = 2)
      .def_readwrite("heartbeat_period_ms", &QueueConfig::heartbeat_period_ms)
      .def_readwrite("missed_heartbeats", &QueueConfig::missed_heartbeats)
      .def("lease_ttl_ms", &QueueConfig::lease_ttl_ms);
  py::class_<Lease>(lm, "Lease")
      .def_readonly("task_id", &Lease::task_id)
      .def_readonly("worker_id", &Lease::worker_id)
      .def_readonly("attempt", &Lease::attempt)
      .def_readonly("expires_at", &Lease::expires_at);
  py::class_<QueueTask>(lm, "Task")
      .def_readonly("id", &QueueTask::id)
      .def_property_readonly("payload_json", [](const QueueTask& t) { return t.payload.dump(); })
      .def_property_readonly("state", [](const QueueTask& t) { return std::string(task_state_name(t.state)); })
      .def_readonly("attempt", &QueueTask::attempt)
      .def_readonly("worker_id", &QueueTask::worker_id)
      .def_readonly("expires_at", &QueueTask::expires_at)
      .def_readonly("output_hash", &QueueTask::output_hash);
  py::class_<LeaseQueue>(lm, "Queue")
      .def_static("create", [](const std::string& d, QueueConfig c) { return LeaseQueue::create(d, c); },
                  py::arg("dir"), py::arg("config") = QueueConfig{})
      .def_static("open", [](const std::string& d, QueueConfig c) { return LeaseQueue::open(d, c); },
                  py::arg("dir"), py::arg("config") = QueueConfig{})
      .def("enqueue", [](LeaseQueue& q, const std::string& id, const std::string& payload_json, uint64_t now) {
             return q.enqueue(id, Json::parse(payload_json), now);
           }, py::arg("task_id"), py::arg("payload_json") = "{}", py::arg("now") = 0)
      .def("claim", [](LeaseQueue& q, const std::string& w, uint64_t now) { return lease_to_py(q.claim(w, now)); })
      .def("claim_if", [](LeaseQueue& q, const std::string& w, uint64_t now, py::function pred) {
             return lease_to_py(q.claim_if(w, now, [&](const QueueTask& t) {
               return pred(py::cast(t, py::return_value_policy::reference)).cast<bool>();
             }));
           })
      .def("heartbeat", &LeaseQueue::heartbeat)
      .def("expire_due", &LeaseQueue::expire_due)
      .def("complete", [](LeaseQueue& q, const std::string& t, const std::string& w, uint64_t a, py::bytes out,
                          uint64_t now) { q.complete(t, w, a, std::string(out), now); })
      .def("fail", &LeaseQueue::fail)
      .def("get", [](const LeaseQueue& q, const std::string& t) -> py::object {
             const QueueTask* p = q.get(t);
             return p ? py::cast(*p) : py::none();
           })
      .def("get_output", [](const LeaseQueue& q, const std::string& t, uint64_t a) -> py::object {
             auto o = q.get_output(t, a);
             return o ? py::object(py::bytes(*o)) : py::none();
           })
      .def_static("checkpoint_branch", &LeaseQueue::checkpoint_branch)
      .def("queued_ids", &LeaseQueue::queued_ids)
      .def("event_types", [](const LeaseQueue& q) {
             std::vector<std::string> out;
             for (const LogEvent& e : q.log().events()) out.push_back(e.event_type);
             return out;
           })
      .def("log_len", [](const LeaseQueue& q) { return q.log().size(); })
      .def_property_readonly("dir", &LeaseQueue::dir);

  // ---- cas
  auto cm = m.def_submodule("cas", "replicated content-addressed store with pins and GC");
  cm.attr("MIN_REPLICAS") = kMinReplicas;
  py::class_<GcReport>(cm, "GcReport")
      .def_readonly("blobs_removed", &GcReport::blobs_removed)
      .def_readonly("bytes_freed", &GcReport::bytes_freed);
  py::class_<CasStore>(cm, "Store")
      .def_static("create", &CasStore::create, py::arg("dir"), py::arg("backends"),
                  py::arg("min_replicas") = kMinReplicas)
      .def_static("open", &CasStore::open, py::arg("dir"), py::arg("backends"),
                  py::arg("min_replicas") = kMinReplicas)
      .def("put", [](CasStore& s, py::bytes b) { return s.put(std::string(b)); })
      .def("get", [](const CasStore& s, const std::string& d) { return py::bytes(s.get(d)); })
      .def("pin", &CasStore::pin)
      .def("unpin", &CasStore::unpin)
      .def("gc", &CasStore::gc)
      .def("replica_count", &CasStore::replica_count)
      .def_property_readonly("pins", &CasStore::pins)
      .def("event_types", [](const CasStore& s) {
        std::vector<std::string> out;
        for (const LogEvent& e : s.log().events()) out.push_back(e.event_type);
        return out;
      });

  // ---- mesh
  auto mm = m.def_submodule("mesh", "capability adverts, pull-claim, signed freeze, watcher ring");
  mm.attr("MIN_WATCHERS") = 2;
  mm.attr("MIN_RING") = 3;
  py::class_<Capabilities>(mm, "Capabilities")
      .def(py::init([](uint32_t g, uint32_t c, bool k, std::vector<std::string> p) {
             return Capabilities{g, c, k, std::move(p)};
           }),
           py::arg("gpus") = 0, py::arg("cpus") = 1, py::arg("kvm") = false,
           py::arg("providers") = std::vector<std::string>{})
      .def_readwrite("gpus", &Capabilities::gpus)
      .def_readwrite("cpus", &Capabilities::cpus)
      .def_readwrite("kvm", &Capabilities::kvm)
      .def_readwrite("providers", &Capabilities::providers);
  py::class_<Advert>(mm, "Advert")
      .def_readonly("node", &Advert::node)
      .def_readonly("key", &Advert::key)
      .def_readonly("caps", &Advert::caps)
      .def_readonly("at", &Advert::at);
  py::class_<Watch>(mm, "Watch").def_readonly("watcher", &Watch::watcher).def_readonly("watchee", &Watch::watchee);
  py::class_<Freeze>(mm, "Freeze")
      .def(py::init([](std::string payload, std::string signer, py::bytes sig) {
             return Freeze{std::move(payload), std::move(signer), std::string(sig)};
           }),
           py::arg("payload"), py::arg("signer"), py::arg("signature"));
  py::class_<Mesh, std::shared_ptr<Mesh>>(mm, "Mesh")
      .def_static("create", [](const std::string& d, const std::string& id, const std::string& key, bool trusted) {
                    return std::make_shared<Mesh>(d, id, key, trusted, false);
                  }, py::arg("dir"), py::arg("this_id"), py::arg("this_key"), py::arg("trusted") = true)
      .def_static("open", [](const std::string& d, const std::string& id, const std::string& key, bool trusted) {
                    return std::make_shared<Mesh>(d, id, key, trusted, true);
                  }, py::arg("dir"), py::arg("this_id"), py::arg("this_key"), py::arg("trusted") = true)
      .def("advertise", &Mesh::advertise)
      .def("pull", [](Mesh& me, LeaseQueue& q, uint64_t now) { return lease_to_py(me.pull(q, now)); })
      .def("freeze", &Mesh::freeze)
      .def("is_frozen", [](const Mesh& me) { return me.frozen_; })
      .def_property_readonly("adverts", [](const Mesh& me) { return me.adverts_; })
      .def_property_readonly("watches", [](const Mesh& me) { return me.watches_; });
  mm.def("caps_satisfy", [](const Capabilities& c, const std::string& payload_json) {
    return caps_satisfy(c, Json::parse(payload_json));
  });
  py::class_<LocalMesh>(mm, "LocalMesh")
      .def_static("start", [](size_t n, const std::string& base) { return std::make_unique<LocalMesh>(n, base); })
      .def("__len__", &LocalMesh::size)
      .def("get", &LocalMesh::get)
      .def("partition", &LocalMesh::partition)
      .def("heal", &LocalMesh::heal)
      .def("tick", &LocalMesh::tick);

  // ---- pipeline
  auto pm = m.def_submodule("pipeline", "oracle -> implementers -> review -> merge on a lease queue");
  pm.attr("PLANTED_BAD_MARKER") = py::bytes(kPlantedBad);
  pm.attr("DEFAULT_N_IMPLEMENTERS") = 3;
  pm.attr("DEFAULT_MAX_ROUNDS") = 3;
  py::class_<Candidate>(pm, "Candidate")
      .def(py::init([](std::string id, std::string angle, py::bytes patch) {
             return Candidate{std::move(id), std::move(angle), std::string(patch)};
           }),
           py::arg("id"), py::arg("angle"), py::arg("patch"))
      .def_readonly("id", &Candidate::id)
      .def_readonly("angle", &Candidate::angle)
      .def_property_readonly("patch", [](const Candidate& c) { return py::bytes(c.patch); });
  py::class_<Verdict>(pm, "Verdict")
      .def_static("pick", [](std::string id) {
        Verdict v;
        v.pick = true;
        v.candidate = std::move(id);
        return v;
      })
      .def_static("reject_all", [](std::vector<std::string> defects) {
        Verdict v;
        v.defects = std::move(defects);
        return v;
      })
      .def_readonly("is_pick", &Verdict::pick)
      .def_readonly("candidate", &Verdict::candidate)
      .def_readonly("defects", &Verdict::defects)
      .def("to_json", [](const Verdict& v) { return v.to_json().dump(); });
  pm.def("is_planted_bad", [](py::bytes b) { return is_planted_bad(std::string(b)); });
  pm.def("review", &review);
  pm.def("merge_allowed", &merge_allowed);
  pm.def("work_payload", [](const std::string& module, const std::string& role, const std::string& extra_json) {
    auto it = work_payload(module, role, Json::parse(extra_json));
    return std::make_pair(it.first, it.second.dump());
  });
  py::class_<Pipeline>(pm, "Pipeline")
      .def_static("create", [](const std::string& d, const std::string& module, uint32_t n, uint32_t r, QueueConfig qc) {
                    return std::make_unique<Pipeline>(d, module, n, r, qc, false);
                  }, py::arg("dir"), py::arg("module"), py::arg("n_implementers") = 3,
                  py::arg("max_rounds") = 3, py::arg("queue_config") = QueueConfig{})
      .def_static("open", [](const std::string& d, const std::string& module, uint32_t n, uint32_t r, QueueConfig qc) {
                    return std::make_unique<Pipeline>(d, module, n, r, qc, true);
                  }, py::arg("dir"), py::arg("module"), py::arg("n_implementers") = 3,
                  py::arg("max_rounds") = 3, py::arg("queue_config") = QueueConfig{})
      .def("start_oracle", &Pipeline::start_oracle)
      .def("record_oracle", &Pipeline::record_oracle)
      .def("start_implementers", &Pipeline::start_implementers)
      .def("submit_candidate", &Pipeline::submit_candidate)
      .def("start_review", &Pipeline::start_review)
      .def("record_verdict", [](Pipeline& p, const Verdict& v, uint64_t now) {
        return std::string(stage_name(p.record_verdict(v, now)));
      })
      .def("record_merge", &Pipeline::record_merge, py::arg("module"), py::arg("spec_section"),
           py::arg("commit"), py::arg("tests_passed"), py::arg("tests_failed"), py::arg("gpu_job_ids"),
           py::arg("now"))
      .def_property_readonly("stage", [](const Pipeline& p) { return std::string(stage_name(p.stage())); })
      .def_property_readonly("round", &Pipeline::round)
      .def_property_readonly("stub_failed", &Pipeline::stub_failed)
      .def_property_readonly("candidates", &Pipeline::candidates)
      .def_property_readonly("module", &Pipeline::module)
      .def("queue", &Pipeline::queue, py::return_value_policy::reference_internal);
}
