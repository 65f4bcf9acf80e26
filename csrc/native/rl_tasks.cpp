// Task factories, the solve-rate filter and the tool-call horizon curriculum.
//
// Eight factories (code, swe, math, research, long_horizon, arc, forecast, open_ended) mint a
// `prometheus.task_spec` v1 plus the checker payload from catalog rows, round-robin. The
// solve-rate filter runs n attempts of an injected solver against the payload and keeps only
// tasks solved sometimes but not always. Nothing here reads a clock: `created_at` is supplied.
// Catalog rows and minted tasks cross the binding as JSON text.
// (reference: rl/tasks/src/lib.rs:29-75 constants, :213-260 spec, :330-395 filter,
//  :397-560 scoring, :562-590 horizon, :592-1132 factories, :1134-1500 mint functions)
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

constexpr uint32_t kStartToolCalls = 10;
constexpr double kRaiseThreshold = 0.5;
constexpr double kProbEps = 1e-12;
constexpr size_t kGridPassK = 2;
const char* const kHiddenTestPath = "/grader/hidden.py";
const char* const kHiddenTestBody = "# hidden\nprint(open('/workspace/out.txt').read())\n";
const char* const kPythonCode = "print(open('/workspace/out.txt').read())";

struct Kind {
  const char* name;
  const char* domain;
  const char* verifier_id;
  const char* verifier_kind;
  uint32_t horizon_s, max_tool_calls;
};
const Kind kKinds[] = {
    {"code", "code", "sandboxed-tests", "sandboxed_tests", 30, kStartToolCalls},
    {"swe", "code", "sandboxed-tests", "sandboxed_tests", 60, kStartToolCalls * 2},
    {"math", "math", "symbolic-math", "symbolic_math", 30, kStartToolCalls},
    {"research", "science", "research-numeric", "lean_kernel", 600, kStartToolCalls},
    {"long_horizon", "agent", "long-horizon", "lean_kernel", 3600, 2000},
    {"arc", "arc", "grid-match", "grid_match", 30, kStartToolCalls},
    {"forecast", "other", "market-resolution", "market_resolution", 30, kStartToolCalls},
    {"open_ended", "other", "open-ended-rubric", "lean_kernel", 30, kStartToolCalls},
};
const Kind& kind_of(const std::string& name) {
  for (const Kind& k : kKinds)
    if (name == k.name) return k;
  throw Error("Schema", "unknown factory kind " + name);
}

std::string fixed_double(double v) {   // shortest round-trip text without an exponent
  char buf[400];
  const auto res = std::to_chars(buf, buf + sizeof buf, v, std::chars_format::fixed);
  return std::string(buf, res.ptr);
}
std::string bool_text(bool b) { return b ? "true" : "false"; }
std::string le_bytes(double v) {
  uint64_t u;
  std::memcpy(&u, &v, 8);
  std::string b(8, '\0');
  for (int i = 0; i < 8; ++i) b[i] = static_cast<char>((u >> (8 * i)) & 0xFF);
  return b;
}

// ---- payload scoring ------------------------------------------------------------------
bool grid_ok(const Json& g) {
  if (!g.is_array() || g.arr().empty() || !g.arr()[0].is_array() || g.arr()[0].arr().empty()) return false;
  const size_t w = g.arr()[0].arr().size();
  for (const Json& row : g.arr()) {
    if (!row.is_array() || row.arr().size() != w) return false;
    for (const Json& c : row.arr())
      if (!c.is_integer() || c.as_i64() < 0 || c.as_i64() > 9) return false;
  }
  return true;
}
bool is_grid_shape(const Json& g) {   // array of arrays of small non-negative integers (may be ragged)
  if (!g.is_array()) return false;
  for (const Json& row : g.arr()) {
    if (!row.is_array()) return false;
    for (const Json& c : row.arr())
      if (!c.is_integer() || c.as_i64() < 0 || c.as_i64() > 255) return false;
  }
  return true;
}
std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
  while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
  return s.substr(a, b - a);
}
bool score_grid(const Json& expected, const std::string& attempt) {
  Json v;
  try {
    v = Json::parse(trim(attempt));
  } catch (const Error&) {
    return false;
  }
  std::vector<Json> predicted;
  bool as_list = v.is_array();
  if (as_list)
    for (const Json& g : v.arr()) as_list = as_list && is_grid_shape(g);
  if (as_list) {
    // an empty outer list parses as "no grids" in the three-level reading
    for (const Json& g : v.arr()) predicted.push_back(g);
  } else if (is_grid_shape(v)) {
    predicted.push_back(v);
  } else {
    return false;
  }
  if (predicted.size() > kGridPassK) return false;
  if (!grid_ok(expected)) return false;
  for (const Json& g : predicted)
    if (!grid_ok(g)) return false;
  for (const Json& g : predicted)
    if (g == expected) return true;
  return false;
}
bool parse_f64(const std::string& text, double& out) {
  const std::string s = trim(text);
  if (s.empty()) return false;
  char* end = nullptr;
  out = std::strtod(s.c_str(), &end);
  return end == s.c_str() + s.size();
}
double clamp_prob(double p) { return std::min(std::max(p, kProbEps), 1.0 - kProbEps); }
bool score_market(const Json& m, const std::string& attempt) {
  double p;
  if (!parse_f64(attempt, p) || !std::isfinite(p) || p < 0 || p > 1) return false;
  const double mp = m.at("market_p").as_double();
  if (!std::isfinite(mp) || mp < 0 || mp > 1) return false;
  const double a = clamp_prob(p), b = clamp_prob(mp);
  const double score = m.at("outcome").as_bool() ? std::log(a) - std::log(b) : std::log(1 - a) - std::log(1 - b);
  return score > 0;
}
bool score_research(const Json& r, const std::string& attempt) {
  double x;
  const double target = r.at("target").as_double();
  return parse_f64(attempt, x) && std::isfinite(x) && std::isfinite(target) && x == target;
}
const Json* opt(const Json& o, const char* key) {
  const Json* v = o.find(key);
  return (v == nullptr || v->is_null()) ? nullptr : v;
}
// math expected string, else code expected stdout, else grid
bool score_simple(const Json* math, const Json* code, const Json* grid, const std::string& attempt) {
  if (math != nullptr) return attempt == math->at("expected").as_string();
  if (code != nullptr) return attempt == code->at("expected_stdout").as_string();
  if (grid != nullptr) return score_grid(grid->at("expected"), attempt);
  return false;
}
bool score_long_horizon(const Json& t, const std::string& attempt) {
  Json v;
  try {
    v = Json::parse(trim(attempt));
    const auto& cps = v.at("checkpoints").arr();
    const std::string& fin = v.at("final").as_string();
    const auto& want = t.at("checkpoints").arr();
    if (cps.size() != want.size()) return false;
    for (size_t i = 0; i < want.size(); ++i)
      if (!score_simple(opt(want[i], "math"), opt(want[i], "code"), opt(want[i], "grid"), cps[i].as_string())) return false;
    return score_simple(opt(t, "final_math"), opt(t, "final_code"), nullptr, fin);
  } catch (const Error&) {
    return false;
  }
}
bool score_open_ended(const Json& t, const std::string& attempt) {
  Json scores;
  try {
    scores = Json::parse(trim(attempt));
    if (!scores.is_object()) return false;
    double num = 0, den = 0;
    for (const Json& c : t.at("rubric").at("criteria").arr()) {
      const Json* v = scores.find(c.at("id").as_string());
      if (v == nullptr || !v->is_number()) return false;
      const double x = v->as_double();
      if (!std::isfinite(x) || x < 0 || x > 1) return false;
      const double w = c.at("weight").as_double();
      num += w * x;
      den += w;
    }
    for (const auto& kv : scores.obj())
      if (!kv.second.is_number()) return false;
    return (den == 0 ? 0.0 : num / den) > 0.5;
  } catch (const Error&) {
    return false;
  }
}
bool score_attempt(const Json& task, const std::string& attempt) {
  if (const Json* m = opt(task, "math")) return attempt == m->at("expected").as_string();
  if (const Json* c = opt(task, "code")) return attempt == c->at("expected_stdout").as_string();
  if (const Json* g = opt(task, "grid")) return score_grid(g->at("expected"), attempt);
  if (const Json* m = opt(task, "market")) return score_market(*m, attempt);
  if (const Json* r = opt(task, "research")) return score_research(*r, attempt);
  if (const Json* l = opt(task, "long_horizon")) return score_long_horizon(*l, attempt);
  if (const Json* o = opt(task, "open_ended")) return score_open_ended(*o, attempt);
  throw Error("Unverifiable", "unverifiable: no D2 payload");
}

// ---- hidden-test hashes ---------------------------------------------------------------
std::string hidden_grid(const Json& cells) { return sha256_hex(cells.dump()); }
std::string simple_hidden(const Json* math, const Json* code, const Json* grid) {
  if (math != nullptr) return "math:" + math->at("expected").as_string();
  if (code != nullptr) return "code:" + code->at("expected_stdout").as_string();
  if (grid != nullptr) return "grid:" + hidden_grid(grid->at("expected"));
  return "";
}

// ---- factories ------------------------------------------------------------------------
class Factory {
 public:
  Factory(const std::string& kind, std::string id, const std::string& sources_json)
      : kind_(kind_of(kind)), id_(std::move(id)) {
    const Json rows = Json::parse(sources_json);
    for (const Json& r : rows.arr()) sources_.push_back(r);
  }
  const std::string& id() const { return id_; }
  std::string domain() const { return kind_.domain; }
  std::string kind() const { return kind_.name; }
  size_t size() const { return sources_.size(); }

  std::string mint(uint64_t /*now*/, const std::string& created_at) {
    if (sources_.empty()) throw Error("EmptyCatalog", "empty factory catalog");
    const Json& row = sources_[cursor_];
    const std::string& body = row.at("body").as_string();
    if (body.empty()) throw Error("EmptyStatement", "empty public statement");
    Json task = build(row, body, created_at);
    cursor_ = (cursor_ + 1) % sources_.size();
    return task.dump();
  }

 private:
  Json provenance(const Json& row) const {
    Json p = Json::object();
    p["source"] = row.at("source").as_string();
    for (const char* k : {"license", "url_hash", "snapshot_date", "collection_id", "author"})
      if (const Json* v = opt(row, k)) p[k] = v->as_string();
    return p;
  }
  Json build(const Json& row, const std::string& body, const std::string& created_at) const {
    const std::string name = kind_.name;
    const std::string& src_id = row.at("id").as_string();
    Json task = Json::object();
    Json env_image;   // null unless sandboxed
    std::string hidden;
    for (const char* k : {"code", "math", "grid", "market", "research", "long_horizon", "open_ended"}) task[k] = Json();
    if (name == "math") {
      const std::string expected = sha256_hex("math-expected:" + body);
      hidden = sha256_hex(expected);
      Json m = Json::object();
      m["expected"] = expected;
      task["math"] = m;
    } else if (name == "code" || name == "swe") {
      const bool swe = name == "swe";
      const std::string image_id = "img:" + id_ + ":" + src_id;
      Sha256 h;
      h.update(kHiddenTestPath, std::strlen(kHiddenTestPath));
      const char nul = 0;
      h.update(&nul, 1);
      h.update(kHiddenTestBody, std::strlen(kHiddenTestBody));
      hidden = h.hex();
      env_image = image_id;
      Json image = Json::object();
      image["id"] = image_id;
      Json hidden_tests = Json::object();
      hidden_tests[kHiddenTestPath] = kHiddenTestBody;
      image["hidden_tests"] = hidden_tests;
      Json agent = Json::object();
      if (swe) agent["/workspace/repo"] = body;
      image["agent_files"] = agent;
      image["hidden_tests_hash"] = hidden;
      Json run = Json::object();
      run["tool"] = "python";
      Json payload = Json::object();
      payload["code"] = kPythonCode;
      run["payload"] = payload;
      run["timeout_s"] = static_cast<uint64_t>(swe ? 10 : 5);
      Json mutant = Json::object();
      mutant["id"] = swe ? "wrong-patch" : "wrong-stdout";
      Json files = Json::object();
      files["/workspace/out.txt"] = swe ? "WRONG_SWE\n" : "WRONG\n";
      mutant["files"] = files;
      Json code = Json::object();
      code["image"] = image;
      code["run"] = run;
      code["expected_stdout"] = sha256_hex((swe ? "swe-stdout:" : "code-stdout:") + body);
      Json mutants = Json::array();
      mutants.push(mutant);
      code["mutants"] = mutants;
      task["code"] = code;
    } else if (name == "research") {
      const double target = row.at("target").as_double();
      hidden = sha256_hex(le_bytes(target));
      Json r = Json::object();
      r["kind"] = row.at("kind").as_string();
      const std::string& rk = r["kind"].as_string();
      if (rk != "speedrun" && rk != "paper_repro" && rk != "kaggle") throw Error("Schema", "unknown research kind " + rk);
      r["target"] = target;
      r["budget_gpu_minutes"] = opt(row, "budget_gpu_minutes") ? *opt(row, "budget_gpu_minutes") : Json();
      r["rubric"] = opt(row, "rubric") ? *opt(row, "rubric") : Json();
      task["research"] = r;
    } else if (name == "long_horizon") {
      Json t = Json::object();
      t["checkpoints"] = row.at("checkpoints");
      t["final_math"] = opt(row, "final_math") ? *opt(row, "final_math") : Json();
      t["final_code"] = opt(row, "final_code") ? *opt(row, "final_code") : Json();
      std::string buf;
      for (const Json& cp : t["checkpoints"].arr()) {
        buf += simple_hidden(opt(cp, "math"), opt(cp, "code"), opt(cp, "grid"));
        buf.push_back('\0');
      }
      buf += "final:" + simple_hidden(opt(t, "final_math"), opt(t, "final_code"), nullptr);
      hidden = sha256_hex(buf);
      task["long_horizon"] = t;
    } else if (name == "arc") {
      hidden = hidden_grid(row.at("expected"));
      Json g = Json::object();
      g["expected"] = row.at("expected");
      task["grid"] = g;
    } else if (name == "forecast") {
      const Json& m = row.at("market");
      hidden = sha256_hex(bool_text(m.at("outcome").as_bool()) + ":" + fixed_double(m.at("market_p").as_double()));
      task["market"] = m;
    } else {   // open_ended
      std::string buf;
      for (const Json& c : row.at("rubric").at("criteria").arr()) {
        buf += c.at("id").as_string();
        buf.push_back('\0');
        buf += c.at("prompt").as_string();
        buf.push_back('\0');
      }
      hidden = sha256_hex(buf);
      Json o = Json::object();
      o["rubric"] = row.at("rubric");
      task["open_ended"] = o;
    }
    Json spec = Json::object();
    spec["schema_id"] = "prometheus.task_spec";
    spec["schema_version"] = static_cast<uint64_t>(1);
    spec["task_id"] = id_ + ":" + src_id;
    spec["domain"] = kind_.domain;
    spec["split"] = "train";
    spec["statement_hash"] = sha256_hex(body);
    spec["hidden_tests_hash"] = hidden;
    spec["verifier_id"] = kind_.verifier_id;
    if (!env_image.is_null()) spec["env_image"] = env_image;
    spec["horizon_s"] = static_cast<uint64_t>(kind_.horizon_s);
    spec["max_tool_calls"] = static_cast<uint64_t>(kind_.max_tool_calls);
    spec["provenance"] = provenance(row);
    spec["created_at"] = created_at;
    task["spec"] = spec;
    task["verifier_kind"] = kind_.verifier_kind;
    task["verifier_id"] = kind_.verifier_id;
    task["statement"] = body;
    return task;
  }

  const Kind& kind_;
  std::string id_;
  std::vector<Json> sources_;
  size_t cursor_ = 0;
};

void schema_ok(const std::string& spec_json) {
  const Json s = Json::parse(spec_json);
  const std::string id = s.at("schema_id").as_string();
  const uint64_t v = s.at("schema_version").as_u64();
  if (id != "prometheus.task_spec" || v != 1) throw Error("Schema", "schema mismatch: " + id + " v" + std::to_string(v));
}

class ScriptedSolver {
 public:
  void insert(const std::string& statement, const std::string& reply) { replies_[statement] = reply; }
  std::string attempt(const std::string& statement, uint64_t) const {
    auto it = replies_.find(statement);
    if (it == replies_.end()) throw Error("Unverifiable", "unverifiable: no scripted attempt for " + statement);
    return it->second;
  }

 private:
  std::map<std::string, std::string> replies_;
};

struct SolveRate {
  uint32_t passed = 0, n = 0;
  double rate() const { return n == 0 ? 0.0 : static_cast<double>(passed) / n; }
  bool in_open_interval() const { return n > 0 && passed > 0 && passed < n; }
};

SolveRate probe(const std::function<std::string(const std::string&, uint64_t)>& solver, const std::string& task_json,
                uint32_t n, uint64_t now) {
  if (n == 0) throw Error("BadN", "solve-rate sample count must be > 0");
  const Json task = Json::parse(task_json);
  const std::string& statement = task.at("statement").as_string();
  SolveRate r{0, n};
  for (uint32_t i = 0; i < n; ++i)
    if (score_attempt(task, solver(statement, now))) ++r.passed;
  return r;
}
SolveRate keep(SolveRate r) {
  if (r.n == 0) throw Error("BadN", "solve-rate sample count must be > 0");
  if (r.passed == 0) throw Error("Impossible", "solve rate 0%");
  if (r.passed >= r.n) throw Error("Trivial", "solve rate 100%");
  return r;
}

class Horizon {
 public:
  uint32_t tool_calls() const { return tool_calls_; }
  void raise_if(double success_rate) {
    if (success_rate > kRaiseThreshold) tool_calls_ = tool_calls_ > UINT32_MAX / 2 ? UINT32_MAX : tool_calls_ * 2;
  }

 private:
  uint32_t tool_calls_ = kStartToolCalls;
};

}  // namespace

void bind_rl_tasks(py::module_& m) {
  auto tm = m.def_submodule("tasks", "task factories, solve-rate filter, horizon curriculum");
  tm.attr("SCHEMA_TASK_SPEC") = "prometheus.task_spec";
  tm.attr("SCHEMA_VERSION") = 1;
  tm.attr("START_TOOL_CALLS") = kStartToolCalls;
  tm.attr("RAISE_THRESHOLD") = kRaiseThreshold;
  {
    std::vector<std::string> names;
    for (const Kind& k : kKinds) names.push_back(k.name);
    tm.attr("FACTORY_KINDS") = names;
  }
  py::class_<Factory>(tm, "Factory")
      .def(py::init<const std::string&, std::string, const std::string&>(), py::arg("kind"), py::arg("id"),
           py::arg("sources_json"))
      .def_property_readonly("id", &Factory::id)
      .def_property_readonly("domain", &Factory::domain)
      .def_property_readonly("kind", &Factory::kind)
      .def("__len__", &Factory::size)
      .def("mint", &Factory::mint, py::arg("now"), py::arg("created_at"));
  tm.def("schema_ok", &schema_ok);
  tm.def("score_attempt", [](const std::string& task_json, const std::string& attempt) {
    return score_attempt(Json::parse(task_json), attempt);
  });
  py::class_<ScriptedSolver>(tm, "ScriptedSolver")
      .def(py::init<>())
      .def("insert", &ScriptedSolver::insert)
      .def("attempt", &ScriptedSolver::attempt, py::arg("statement"), py::arg("now") = 0)
      .def("__call__", &ScriptedSolver::attempt, py::arg("statement"), py::arg("now") = 0);
  py::class_<SolveRate>(tm, "SolveRate")
      .def(py::init([](uint32_t p, uint32_t n) { return SolveRate{p, n}; }))
      .def_readonly("passed", &SolveRate::passed)
      .def_readonly("n", &SolveRate::n)
      .def("rate", &SolveRate::rate)
      .def("in_open_interval", &SolveRate::in_open_interval);
  auto fm = tm.def_submodule("SolveRateFilter");
  fm.def("probe", &probe, py::arg("solver"), py::arg("task_json"), py::arg("n"), py::arg("now") = 0);
  fm.def("keep", &keep);
  py::class_<Horizon>(tm, "Horizon")
      .def(py::init<>())
      .def_property_readonly("tool_calls", &Horizon::tool_calls)
      .def("raise_if", &Horizon::raise_if);
}
