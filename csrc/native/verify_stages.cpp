// Verification stages V0..V10: the stage table, job-script rendering and the exit checkers.
//
// A stage passes only on what its job wrote into its output directory (`busbw_gbps` and
// `node_facts.txt` for V0, `<stage>.json` for the others); nobody's summary is taken as the
// criterion. GPU counts are those of one 8 x B200 box.
// (reference: verify/ncshare/src/lib.rs:37-284 stage table and API, check.rs:9-236 criteria,
//  parse.rs:6-33 nccl-tests parser, kvm.rs:6-76 node facts, render.rs:6-49 templates)
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

struct StageSpec {
  const char* name;
  int gpus;   // 0 = shared / soak
  const char* what;
  const char* exit;
};
const StageSpec kStages[] = {
    {"v0", 1, "environment: build inside the job, scheduler dry run, all-reduce bandwidth on one box and across two, /dev/kvm and NVMe facts, queue waits",
     "measured bus bandwidth recorded; known whether microVM sandboxes can run there"},
    {"v1", 1, "about 10M parameters in the flagship shape, every custom kernel",
     "kernel path vs independent fp32 reference logits within 1e-5; gradient checks pass; one batch is overfit"},
    {"v2", 8, "same model on 1 GPU vs EP=8, FSDP=8, PP=2 x 4, CP=2, then DP across two boxes",
     "loss equals single-device to 1e-6 relative in fp32 over 200 steps; routing identical"},
    {"v3", 8, "bf16 and FP8 at 0.1-0.5B for 2k-5k steps; NVFP4 by fake quantisation",
     "FP8 loss within 0.5% of bf16; NVFP4 checked for numerics only"},
    {"v4", 4, "a rank killed mid-step, elastic DP continues; in-memory checkpoint restore; injected bit flip; injected bad shard",
     "resumed run bitwise equal to the uninterrupted run; the SDC hash catches the flip; spike rollback skips the shard"},
    {"v5", 8, "0.1B / 1B MoE on 20B tokens; rung-1 shape at 10B tokens",
     "loss curve matches the ladder's small-scale fit; checkpoint / resume across job boundaries works"},
    {"v6", 4, "stage A then stage B compression at 0.1-0.5B on verified math; latent budget sweep 1x-8x",
     "curriculum trains without collapse; held-out accuracy rises with latent budget; thoughts decode to their steps"},
    {"v7", 8, "GSPO/DAPO loss, async staleness, routing replay, weight sync, parity halt, reward-hacking controls",
     "reward rises on a tiny verifiable task; an injected log-prob drift halts RL; a planted test-file write is flagged"},
    {"v8", 1, "serving fork loads a checkpoint; latent decode, recurrence buckets, MTP speculative decode, KV tiering",
     "serving vs training log-probs within threshold; tiered session restore matches unswapped output"},
    {"v9", 1, "one full research cycle through the Slurm backend",
     "a planted known-positive idea is found and replicated; a planted negative is recorded as negative"},
    {"v10", 0, "harness chaos suite while V5-V9 jobs run", "72 h with no lost task, no duplicated output, no dead token"},
};
constexpr double kLogitsMax = 1e-5, kLossRelMax = 1e-6, kFp8RelMax = 0.005, kSoakHoursMin = 72.0;

const StageSpec& stage_of(const std::string& s) {
  std::string low = s;
  if (!low.empty() && low[0] == 'V') low[0] = 'v';
  for (const StageSpec& st : kStages)
    if (low == st.name) return st;
  throw Error("UnknownStage", "unknown stage " + s);
}

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace(static_cast<unsigned char>(s[a]))) ++a;
  while (b > a && std::isspace(static_cast<unsigned char>(s[b - 1]))) --b;
  return s.substr(a, b - a);
}
std::vector<std::string> lines_of(const std::string& text) {
  std::vector<std::string> out;
  size_t off = 0;
  while (off <= text.size()) {
    size_t nl = text.find('\n', off);
    if (nl == std::string::npos) nl = text.size();
    out.push_back(text.substr(off, nl - off));
    off = nl + 1;
  }
  return out;
}
std::vector<std::string> columns(const std::string& line) {
  std::vector<std::string> out;
  std::string cur;
  for (unsigned char c : line) {
    if (std::isspace(c)) {
      if (!cur.empty()) out.push_back(cur);
      cur.clear();
    } else {
      cur.push_back(static_cast<char>(c));
    }
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}
bool parse_u64(const std::string& s) { return !s.empty() && s.find_first_not_of("0123456789") == std::string::npos; }
bool parse_f64(const std::string& s, double& v) {
  if (s.empty()) return false;
  char* end = nullptr;
  v = std::strtod(s.c_str(), &end);
  return end == s.c_str() + s.size();
}

// out-of-place bus bandwidth (GB/s) of the last data row of an all-reduce benchmark table:
//   size count type redop root time algbw busbw #wrong ...
double parse_busbw_gbps(const std::string& text) {
  if (trim(text).empty()) throw Error("Other", "verify: empty nccl stdout");
  bool found = false;
  double last = 0;
  for (const auto& raw : lines_of(text)) {
    const std::string line = trim(raw);
    if (line.empty() || line[0] == '#') continue;
    const auto cols = columns(line);
    double v;
    if (cols.size() < 9 || !parse_u64(cols[0]) || !parse_u64(cols[1]) || !parse_f64(cols[7], v) || !std::isfinite(v)) continue;
    last = v;
    found = true;
  }
  if (!found) throw Error("Other", "verify: no busbw data row");
  return last;
}

bool kvm_available(const std::string& facts) {
  if (trim(facts).empty()) throw Error("Other", "verify: empty node facts");
  int explicit_value = -1;
  bool char_device = false, absent = false, mentioned = false;
  for (const auto& raw : lines_of(facts)) {
    std::string line = trim(raw);
    if (line.empty() || line[0] == '#') continue;
    for (char& c : line) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    if (line.rfind("kvm:", 0) == 0) {
      mentioned = true;
      const std::string v = trim(line.substr(4));
      if (v == "yes" || v == "true" || v == "1" || v == "present") explicit_value = 1;
      else if (v == "no" || v == "false" || v == "0" || v == "absent") explicit_value = 0;
      else throw Error("Other", "verify: unrecognized kvm value: " + v);
      continue;
    }
    if (line.find("/dev/kvm") == std::string::npos) continue;
    mentioned = true;
    const auto cols = columns(line);
    const std::string first = cols.empty() ? "" : cols[0];
    if (!first.empty() && first[0] == 'c' && first.rfind("cannot", 0) != 0) char_device = true;   // ls -l mode string
    if (line.find("character device") != std::string::npos || line.find("character special") != std::string::npos) char_device = true;
    for (const char* w : {"no such file", "not found", "cannot stat", "missing", "absent"})
      if (line.find(w) != std::string::npos) absent = true;
  }
  if (explicit_value >= 0) return explicit_value == 1;
  if (char_device) return true;
  if (absent) return false;
  if (mentioned) throw Error("Other", "verify: kvm mentioned but not a character device and not an absence line");
  throw Error("Other", "verify: node facts do not mention kvm");
}

std::string replace_all(std::string s, const std::string& from, const std::string& to) {
  size_t pos = 0;
  while ((pos = s.find(from, pos)) != std::string::npos) {
    s.replace(pos, from.size(), to);
    pos += to.size();
  }
  return s;
}
std::string render(const std::string& path, const std::string& run_id, const std::string& walltime, const std::string& gpus) {
  if (run_id.empty()) throw Error("Other", "verify: empty run_id");
  if (walltime.empty()) throw Error("Other", "verify: empty walltime");
  if (!file_exists(path)) throw Error("Other", "verify: read template " + path);
  std::string t = read_file(path);
  t = replace_all(t, "{{RUN_ID}}", run_id);
  t = replace_all(t, "{{WALLTIME}}", walltime);
  if (!gpus.empty()) t = replace_all(t, "{{GPUS}}", gpus);
  return t;
}

bool is_dir(const std::string& p) {
  struct stat st{};
  return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
double need_f64(const Json& o, const char* key) {
  const Json* v = o.find(key);
  if (v == nullptr) throw Error("MissingOutput", std::string("missing output ") + key);
  if (!v->is_number()) throw Error("ExitFailed", std::string("exit criterion failed: ") + key + " is not a number");
  return v->as_double();
}
void need_true(const Json& o, const char* key) {
  const Json* v = o.find(key);
  if (v == nullptr) throw Error("MissingOutput", std::string("missing output ") + key);
  if (!v->is_bool()) throw Error("ExitFailed", std::string("exit criterion failed: ") + key + " is not a boolean");
  if (!v->as_bool()) throw Error("ExitFailed", std::string("exit criterion failed: ") + key + " is false");
}
void need_le(const Json& o, const char* key, double max) {
  const double got = need_f64(o, key);
  if (!(got <= max)) throw Error("ExitFailed", std::string("exit criterion failed: ") + key + " " + std::to_string(got) + " > " + std::to_string(max));
}
void need_zero(const Json& o, const char* key) {
  const double got = need_f64(o, key);
  if (got != 0.0) throw Error("ExitFailed", std::string("exit criterion failed: ") + key + " " + std::to_string(got) + " != 0");
}

void check_exit(const std::string& stage, const std::string& dir) {
  const StageSpec& st = stage_of(stage);
  if (!is_dir(dir)) throw Error("MissingOutput", "missing output output_dir " + dir);
  const std::string name = st.name;
  if (name == "v0") {
    if (!file_exists(dir + "/busbw_gbps")) throw Error("MissingOutput", "missing output busbw_gbps");
    const std::string text = read_file(dir + "/busbw_gbps");
    double v;
    if (parse_f64(trim(text), v)) {
      if (!std::isfinite(v)) throw Error("ExitFailed", "exit criterion failed: non-finite busbw");
    } else {
      try {
        v = parse_busbw_gbps(text);
      } catch (const Error&) {
        throw Error("ExitFailed", "exit criterion failed: busbw unparseable");
      }
    }
    if (!file_exists(dir + "/node_facts.txt")) throw Error("MissingOutput", "missing output node_facts.txt");
    try {
      kvm_available(read_file(dir + "/node_facts.txt"));   // either answer passes: it must be known
    } catch (const Error& e) {
      throw Error("ExitFailed", std::string("exit criterion failed: kvm facts: ") + e.what());
    }
    return;
  }
  const std::string file = name + ".json";
  if (!file_exists(dir + "/" + file)) throw Error("MissingOutput", "missing output " + file);
  Json o;
  try {
    o = Json::parse(read_file(dir + "/" + file));
  } catch (const Error& e) {
    throw Error("ExitFailed", "exit criterion failed: invalid json in " + file + ": " + e.what());
  }
  if (!o.is_object()) throw Error("ExitFailed", "exit criterion failed: " + file + " must be a JSON object");
  if (name == "v1") {
    need_f64(o, "logits_max_diff");
    need_true(o, "grad_ok");
    need_true(o, "overfit_ok");
    need_le(o, "logits_max_diff", kLogitsMax);
  } else if (name == "v2") {
    need_f64(o, "loss_rel_diff");
    need_true(o, "routing_identical");
    need_le(o, "loss_rel_diff", kLossRelMax);
  } else if (name == "v3") {
    need_f64(o, "fp8_loss_rel_diff");
    need_true(o, "nvfp4_numerics_ok");
    need_le(o, "fp8_loss_rel_diff", kFp8RelMax);
  } else if (name == "v4") {
    for (const char* k : {"resumed_bitwise_equal", "sdc_caught_flip", "spike_rollback_skipped_shard"}) need_true(o, k);
  } else if (name == "v5") {
    for (const char* k : {"loss_curve_matches_ladder", "checkpoint_resume_ok"}) need_true(o, k);
  } else if (name == "v6") {
    for (const char* k : {"curriculum_no_collapse", "accuracy_rises_with_latent_budget", "thoughts_decode"}) need_true(o, k);
  } else if (name == "v7") {
    for (const char* k : {"reward_rises", "logprob_drift_halted", "planted_write_flagged"}) need_true(o, k);
  } else if (name == "v8") {
    for (const char* k : {"logprob_within_threshold", "tiered_restore_matches"}) need_true(o, k);
  } else if (name == "v9") {
    for (const char* k : {"planted_positive_found", "planted_positive_replicated", "planted_negative_recorded"}) need_true(o, k);
  } else {   // v10
    const double hours = need_f64(o, "hours");
    need_f64(o, "lost_tasks");
    need_f64(o, "duplicated_outputs");
    need_f64(o, "dead_tokens");
    if (hours < kSoakHoursMin) throw Error("ExitFailed", "exit criterion failed: hours " + std::to_string(hours) + " < 72");
    need_zero(o, "lost_tasks");
    need_zero(o, "duplicated_outputs");
    need_zero(o, "dead_tokens");
  }
}

}  // namespace

void bind_verify_stages(py::module_& m) {
  auto vm = m.def_submodule("ncshare", "verification stages V0..V10: table, templates, exit checkers");
  vm.attr("JOB_PREFIX") = "fv";
  vm.attr("V0_2NODE_NODES") = 2;
  vm.attr("V0_2NODE_GPUS_PER_NODE") = 4;
  vm.attr("V1_INDEPENDENT_FORWARD") = "torch";
  {
    std::vector<std::string> names;
    for (const StageSpec& s : kStages) names.push_back(s.name);
    vm.attr("STAGES") = names;
  }
  vm.def("parse_stage", [](const std::string& s) { return std::string(stage_of(s).name); });
  vm.def("spec", [](const std::string& s) {
    const StageSpec& st = stage_of(s);
    py::dict d;
    d["stage"] = st.name;
    d["gpus"] = st.gpus == 0 ? py::object(py::none()) : py::object(py::int_(st.gpus));
    d["what"] = st.what;
    d["exit"] = st.exit;
    return d;
  });
  vm.def("render_job", [](const std::string& stage, const std::string& run_id, const std::string& walltime, uint32_t gpus,
                          const std::string& template_dir) {
    const StageSpec& st = stage_of(stage);
    if (gpus == 0) throw Error("Other", "verify: gpus must be > 0 (the soak template does not interpolate the count; pass any)");
    return render(template_dir + "/" + st.name + ".sh", run_id, walltime, std::to_string(gpus));
  }, py::arg("stage"), py::arg("run_id"), py::arg("walltime"), py::arg("gpus"), py::arg("template_dir"));
  vm.def("render_v0_2node", [](const std::string& run_id, const std::string& walltime, const std::string& template_dir) {
    return render(template_dir + "/v0-2node.sh", run_id, walltime, "");
  }, py::arg("run_id"), py::arg("walltime"), py::arg("template_dir"));
  vm.def("check_exit", &check_exit, py::arg("stage"), py::arg("output_dir"));
  vm.def("parse_busbw_gbps", &parse_busbw_gbps);
  vm.def("kvm_available", &kvm_available);
}
