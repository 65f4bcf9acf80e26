// Event log bindings, data-mixture arithmetic and the byte-fallback BPE tokenizer.
//
// Mixture: eight sources in a fixed order, weights summing to 1 +- 1e-9, mix hash =
// sha256 of the compact JSON {"mix_id","mix_bucket","phase","weights"} with weights in
// source order, decay re-weighting of the code / math / reasoning sources, drop-one-source
// ablations, inverse-CDF sampling (reference data/mixture/src/lib.rs:28-286).
//
// Tokenizer: ids 0-3 bos/eos/pad/unk, 4-259 raw bytes, 260-269 ARC colours, merges from
// 270; training picks the most frequent adjacent pair (ties: smallest (left, right));
// encoding repeatedly merges the lowest-rank adjacent pair, leftmost first; `vocab.jsonl`
// lists specials, bytes, colours, merges and a header as compact sorted-key JSON lines and
// its sha256 is the vocabulary hash; `tokenizer.json` is the pretty-printed contract
// (reference tokenizer/src/lib.rs:28-33, :158-307, :383-673).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <map>
#include <unordered_map>

#include "common.hpp"
#include "eventlog.hpp"

namespace py = pybind11;
using namespace pbn;

// ---------------------------------------------------------------------------
// mixture
// ---------------------------------------------------------------------------
namespace mixture {

static const std::vector<std::string> kSources = {
    "web", "code", "math_science_arxiv", "books_papers", "synthetic_rewrites",
    "synthetic_reasoning", "procedural_arc", "agentic_trajectories"};
static const std::vector<std::string> kDecaySources = {"code", "math_science_arxiv", "synthetic_reasoning"};

static int source_index(const std::string& s) {
  auto it = std::find(kSources.begin(), kSources.end(), s);
  if (it == kSources.end()) throw Error("UnknownSource", "unknown source " + s);
  return static_cast<int>(it - kSources.begin());
}

struct Mix {
  std::string mix_id, mix_bucket, phase = "pretrain";
  std::map<int, double> weights;  // keyed by source index = declaration order

  std::map<std::string, double> named() const {
    std::map<std::string, double> out;
    for (const auto& kv : weights) out[kSources[kv.first]] = kv.second;
    return out;
  }
};

static Mix make_mix(std::string id, std::string bucket, std::string phase,
                    const std::map<std::string, double>& w) {
  if (phase != "pretrain" && phase != "decay") throw Error("Config", "mix config: unknown phase " + phase);
  Mix m;
  m.mix_id = std::move(id);
  m.mix_bucket = std::move(bucket);
  m.phase = std::move(phase);
  for (const auto& kv : w) m.weights[source_index(kv.first)] = kv.second;
  return m;
}

static void validate(const Mix& m) {
  if (m.mix_id.empty()) throw Error("Config", "mix config: empty mix_id");
  if (m.mix_bucket.empty()) throw Error("Config", "mix config: empty mix_bucket");
  if (m.weights.empty()) throw Error("Config", "mix config: empty weights");
  double total = 0;
  for (const auto& kv : m.weights) {
    if (!std::isfinite(kv.second) || kv.second <= 0)
      throw Error("Config", "mix config: non-finite or non-positive weight " + kSources[kv.first]);
    total += kv.second;
  }
  if (!std::isfinite(total) || std::fabs(total - 1.0) > 1e-9)
    throw Error("Config", "mix config: weights must sum to 1");
}

static std::string canonical_json(const Mix& m) {
  std::string out = "{\"mix_id\":";
  Json::write_string(out, m.mix_id);
  out += ",\"mix_bucket\":";
  Json::write_string(out, m.mix_bucket);
  out += ",\"phase\":";
  Json::write_string(out, m.phase);
  out += ",\"weights\":{";
  bool first = true;
  for (const auto& kv : m.weights) {
    if (!std::isfinite(kv.second)) throw Error("Config", "mix config: non-finite weight");
    if (!first) out += ",";
    first = false;
    Json::write_string(out, kSources[kv.first]);
    out += ":";
    Json::write_double(out, kv.second);
  }
  out += "}}";
  return out;
}

static std::map<int, double> renormalize(std::map<int, double> w) {
  double total = 0;
  for (const auto& kv : w) total += kv.second;
  if (!std::isfinite(total) || total <= 0) throw Error("Config", "mix config: cannot renormalize weights");
  for (auto& kv : w) kv.second /= total;
  return w;
}

static Mix decay_reweight(const Mix& m, double factor) {
  validate(m);
  if (!std::isfinite(factor) || factor <= 1.0)
    throw Error("Config", "mix config: decay factor must be finite and > 1");
  Mix out = m;
  for (const auto& s : kDecaySources) {
    auto it = out.weights.find(source_index(s));
    if (it != out.weights.end()) it->second *= factor;
  }
  out.weights = renormalize(out.weights);
  out.phase = "decay";
  return out;
}

static Mix drop_source(const Mix& m, const std::string& source) {
  const int idx = source_index(source);
  if (!m.weights.count(idx)) throw Error("UnknownSource", "unknown source " + source);
  if (m.weights.size() == 1) throw Error("Config", "mix config: cannot drop the last source");
  validate(m);
  Mix out = m;
  out.weights.erase(idx);
  out.weights = renormalize(out.weights);
  return out;
}

static std::string sample_source(const Mix& m, double u) {
  if (!std::isfinite(u) || u < 0.0 || u >= 1.0) throw Error("Config", "mix config: u must be in [0, 1)");
  validate(m);
  double acc = 0;
  int last = -1;
  for (const auto& kv : m.weights) {
    acc += kv.second;
    last = kv.first;
    if (u < acc) return kSources[kv.first];
  }
  return kSources[last];
}

}  // namespace mixture

// ---------------------------------------------------------------------------
// tokenizer
// ---------------------------------------------------------------------------
namespace tok {

constexpr uint32_t kFirstByte = 4, kFirstArc = 260, kArcColors = 10, kFirstMerge = 270;

struct PairHash {
  size_t operator()(const std::pair<uint32_t, uint32_t>& p) const {
    return (static_cast<size_t>(p.first) << 32) ^ p.second;
  }
};

class Tokenizer {
 public:
  std::string tokenizer_id;
  uint32_t vocab_size = 0;
  bool byte_fallback = true;
  bool frozen = false;
  std::optional<std::string> frozen_at, corpus_hash;
  std::map<std::string, uint32_t> specials{{"bos", 0}, {"eos", 1}, {"pad", 2}, {"unk", 3}};
  uint32_t arc_start = kFirstArc, arc_end = kFirstArc + kArcColors;
  std::vector<std::pair<uint32_t, uint32_t>> merges;

  static Tokenizer train(const std::vector<std::string>& docs, const std::string& id, uint32_t vocab,
                         bool byte_fallback) {
    if (!byte_fallback) throw Error("Message", "byte_fallback must be true for algorithm byte_fallback_bpe");
    if (id.empty()) throw Error("Message", "tokenizer_id must be non-empty");
    if (vocab < kFirstMerge + 1)
      throw Error("VocabTooSmall", "vocab size " + std::to_string(vocab) +
                                       " is too small for specials, bytes, and ARC colors");
    Tokenizer t;
    t.tokenizer_id = id;
    t.vocab_size = vocab;
    std::vector<std::vector<uint32_t>> seqs;
    std::string blob;
    for (size_t i = 0; i < docs.size(); ++i) {
      if (i) blob += '\n';
      blob += docs[i];
      std::vector<uint32_t> s;
      for (unsigned char c : docs[i]) s.push_back(kFirstByte + c);
      seqs.push_back(std::move(s));
    }
    t.corpus_hash = sha256_hex(blob);
    for (uint32_t next = kFirstMerge; next < vocab; ++next) {
      std::unordered_map<std::pair<uint32_t, uint32_t>, uint64_t, PairHash> counts;
      for (const auto& s : seqs)
        for (size_t i = 0; i + 1 < s.size(); ++i) ++counts[{s[i], s[i + 1]}];
      if (counts.empty()) break;
      std::pair<uint32_t, uint32_t> best{};
      uint64_t best_n = 0;
      bool have = false;
      for (const auto& kv : counts)
        if (!have || kv.second > best_n || (kv.second == best_n && kv.first < best)) {
          best = kv.first;
          best_n = kv.second;
          have = true;
        }
      t.merges.push_back(best);
      for (auto& s : seqs) {
        std::vector<uint32_t> out;
        out.reserve(s.size());
        for (size_t i = 0; i < s.size();) {
          if (i + 1 < s.size() && s[i] == best.first && s[i + 1] == best.second) {
            out.push_back(next);
            i += 2;
          } else {
            out.push_back(s[i++]);
          }
        }
        s.swap(out);
      }
    }
    return t;
  }

  std::vector<uint32_t> encode_bytes(const std::string& bytes) const {
    std::vector<uint32_t> ids;
    for (unsigned char c : bytes) ids.push_back(kFirstByte + c);
    if (ids.empty() || merges.empty()) return ids;
    if (rank_.empty())
      for (size_t i = 0; i < merges.size(); ++i) rank_.emplace(merges[i], i);
    while (true) {
      size_t best_rank = SIZE_MAX, pos = 0;
      for (size_t i = 0; i + 1 < ids.size(); ++i) {
        auto it = rank_.find({ids[i], ids[i + 1]});
        if (it != rank_.end() && it->second < best_rank) {
          best_rank = it->second;
          pos = i;
        }
      }
      if (best_rank == SIZE_MAX) break;
      ids[pos] = kFirstMerge + static_cast<uint32_t>(best_rank);
      ids.erase(ids.begin() + static_cast<long>(pos) + 1);
    }
    return ids;
  }
  void expand(uint32_t id, std::string& out) const {
    if (id >= kFirstByte && id < kFirstByte + 256) {
      out += static_cast<char>(id - kFirstByte);
      return;
    }
    if (id < kFirstMerge || id - kFirstMerge >= merges.size())
      throw Error("UnknownId", "unknown token id " + std::to_string(id));
    expand(merges[id - kFirstMerge].first, out);
    expand(merges[id - kFirstMerge].second, out);
  }
  std::string decode_bytes(const std::vector<uint32_t>& ids) const {
    std::string out;
    for (uint32_t id : ids) expand(id, out);
    return out;
  }
  std::vector<uint32_t> encode_grid(const std::vector<uint8_t>& cells) const {
    std::vector<uint32_t> out;
    for (uint8_t c : cells) {
      if (c >= arc_end - arc_start) throw Error("BadColor", "grid color " + std::to_string(c) + " out of range");
      out.push_back(arc_start + c);
    }
    return out;
  }
  void freeze(const std::string& at) {
    if (frozen) {
      if (frozen_at && *frozen_at == at) return;
      throw Error("Frozen", "tokenizer is frozen");
    }
    frozen = true;
    frozen_at = at;
  }
  double tokens_per_word(const std::string& text) const {
    size_t words = 0;
    bool in = false;
    for (unsigned char c : text) {
      const bool ws = std::isspace(c);
      if (!ws && !in) ++words;
      in = !ws;
    }
    return words == 0 ? 0.0 : static_cast<double>(encode_bytes(text).size()) / words;
  }

  std::string vocab_jsonl() const {
    std::string out;
    auto line = [&](Json o) { out += o.dump() + "\n"; };
    for (const char* name : {"bos", "eos", "pad", "unk"}) {
      Json o = Json::object();
      o["id"] = uint64_t(specials.at(name));
      o["kind"] = "special";
      o["name"] = name;
      line(o);
    }
    for (uint32_t b = 0; b < 256; ++b) {
      Json o = Json::object();
      o["byte"] = uint64_t(b);
      o["id"] = uint64_t(kFirstByte + b);
      o["kind"] = "byte";
      line(o);
    }
    for (uint32_t c = 0; c < kArcColors; ++c) {
      Json o = Json::object();
      o["color"] = uint64_t(c);
      o["id"] = uint64_t(kFirstArc + c);
      o["kind"] = "arc";
      line(o);
    }
    for (size_t r = 0; r < merges.size(); ++r) {
      Json o = Json::object();
      o["id"] = uint64_t(kFirstMerge + r);
      o["kind"] = "merge";
      o["left"] = uint64_t(merges[r].first);
      o["right"] = uint64_t(merges[r].second);
      line(o);
    }
    Json h = Json::object();
    h["algorithm"] = "byte_fallback_bpe";
    h["byte_fallback"] = byte_fallback;
    h["kind"] = "header";
    h["tokenizer_id"] = tokenizer_id;
    h["vocab_size"] = uint64_t(vocab_size);
    line(h);
    return out;
  }
  std::string vocab_hash() const { return sha256_hex(vocab_jsonl()); }
  Json contract() const {
    Json o = Json::object();
    o["schema_id"] = "prometheus.tokenizer";
    o["schema_version"] = uint64_t(1);
    o["tokenizer_id"] = tokenizer_id;
    o["algorithm"] = "byte_fallback_bpe";
    o["vocab_size"] = uint64_t(vocab_size);
    o["byte_fallback"] = byte_fallback;
    Json sp = Json::object();
    for (const auto& kv : specials) sp[kv.first] = uint64_t(kv.second);
    o["special_tokens"] = sp;
    Json arc = Json::object();
    arc["start"] = uint64_t(arc_start);
    arc["end"] = uint64_t(arc_end);
    o["arc_grid_token_range"] = arc;
    o["vocab_hash"] = vocab_hash();
    o["frozen"] = frozen;
    if (frozen_at) o["frozen_at"] = *frozen_at;
    if (corpus_hash) o["corpus_hash"] = *corpus_hash;
    return o;
  }
  // Writes vocab.jsonl and tokenizer.json; returns the prometheus.vocab pointer as JSON.
  std::string save(const std::string& dir) const {
    make_dirs(dir);
    const std::string blob = vocab_jsonl();
    atomic_write(dir + "/vocab.jsonl", blob);
    atomic_write(dir + "/tokenizer.json", contract().dump_pretty());
    Json p = Json::object();
    p["schema_id"] = "prometheus.vocab";
    p["schema_version"] = uint64_t(1);
    p["tokenizer_id"] = tokenizer_id;
    p["vocab_size"] = uint64_t(vocab_size);
    Json sp = Json::object();
    for (const auto& kv : specials) sp[kv.first] = uint64_t(kv.second);
    p["special_token_ids"] = sp;
    Json art = Json::object();
    art["content_hash"] = sha256_hex(blob);
    art["bytes"] = uint64_t(blob.size());
    art["path"] = "vocab.jsonl";
    art["media_type"] = "application/jsonl";
    p["artifact"] = art;
    p["format"] = "jsonl";
    return p.dump();
  }
  static Tokenizer load(const std::string& dir) {
    Json c;
    std::string blob;
    try {
      c = Json::parse(read_file(dir + "/tokenizer.json"));
    } catch (const Error& e) {
      throw Error("Message", std::string("failed to load tokenizer.json: ") + e.what());
    }
    try {
      blob = read_file(dir + "/vocab.jsonl");
    } catch (const Error& e) {
      throw Error("Message", std::string("failed to load vocab.jsonl: ") + e.what());
    }
    Tokenizer t;
    t.tokenizer_id = c.at("tokenizer_id").as_string();
    t.vocab_size = static_cast<uint32_t>(c.at("vocab_size").as_u64());
    if (const Json* b = c.find("byte_fallback")) t.byte_fallback = b->as_bool();
    if (const Json* f = c.find("frozen")) t.frozen = f->as_bool();
    if (const Json* f = c.find("frozen_at")) if (f->is_string()) t.frozen_at = f->as_string();
    if (const Json* f = c.find("corpus_hash")) if (f->is_string()) t.corpus_hash = f->as_string();
    t.specials.clear();
    for (const auto& kv : c.at("special_tokens").obj()) t.specials[kv.first] = static_cast<uint32_t>(kv.second.as_u64());
    for (const char* need : {"bos", "eos", "pad", "unk"})
      if (!t.specials.count(need)) throw Error("Message", std::string("missing or invalid ") + need);
    t.arc_start = static_cast<uint32_t>(c.at("arc_grid_token_range").at("start").as_u64());
    t.arc_end = static_cast<uint32_t>(c.at("arc_grid_token_range").at("end").as_u64());
    size_t off = 0;
    while (off < blob.size()) {
      size_t nl = blob.find('\n', off);
      if (nl == std::string::npos) nl = blob.size();
      const std::string line = blob.substr(off, nl - off);
      off = nl + 1;
      if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
      const Json o = Json::parse(line);
      const Json* k = o.find("kind");
      if (k == nullptr || !k->is_string() || k->as_string() != "merge") continue;
      t.merges.emplace_back(static_cast<uint32_t>(o.at("left").as_u64()),
                            static_cast<uint32_t>(o.at("right").as_u64()));
    }
    // the contract names the hash of the vocabulary file it was written with: a file that was
    // edited or swapped afterwards does not load
    if (const Json* h = c.find("vocab_hash"))
      if (h->is_string() && h->as_string() != sha256_hex(blob))
        throw Error("Message", "vocab.jsonl does not match the vocab_hash in tokenizer.json");
    return t;
  }

 private:
  mutable std::unordered_map<std::pair<uint32_t, uint32_t>, size_t, PairHash> rank_;
};

}  // namespace tok

void bind_harness_core(py::module_& m) {
  // ---- event log ----
  auto log = m.def_submodule("log", "durable hash-chained JSONL event log");
  log.attr("GENESIS_PREV_HASH") = kLogGenesis;
  py::class_<LogEvent>(log, "Event")
      .def_readonly("seq", &LogEvent::seq).def_readonly("prev_hash", &LogEvent::prev_hash)
      .def_readonly("hash", &LogEvent::hash).def_readonly("timestamp", &LogEvent::timestamp)
      .def_readonly("event_type", &LogEvent::event_type).def_readonly("task_id", &LogEvent::task_id)
      .def_readonly("attempt", &LogEvent::attempt).def_readonly("node_id", &LogEvent::node_id)
      .def_readonly("payload_hash", &LogEvent::payload_hash)
      .def_property_readonly("payload_json", [](const LogEvent& e) { return e.payload.dump(); })
      .def("line", &LogEvent::line);
  py::class_<EventLog>(log, "EventLog")
      .def_static("create", &EventLog::create)
      .def_static("open", &EventLog::open)
      .def("append",
           [](EventLog& l, const std::string& type, const std::string& payload_json,
              const std::string& ts, std::optional<std::string> task, std::optional<uint64_t> attempt,
              std::optional<std::string> node) {
             LogAppend a;
             a.event_type = type;
             a.payload = Json::parse(payload_json);
             a.timestamp = ts;
             a.task_id = std::move(task);
             a.attempt = attempt;
             a.node_id = std::move(node);
             return l.append(a);
           },
           py::arg("event_type"), py::arg("payload_json") = "{}", py::arg("timestamp") = "",
           py::arg("task_id") = py::none(), py::arg("attempt") = py::none(),
           py::arg("node_id") = py::none())
      .def("__len__", &EventLog::size)
      .def("events", &EventLog::events)
      .def("get", [](const EventLog& l, uint64_t seq) -> std::optional<LogEvent> {
        const LogEvent* e = l.get(seq);
        return e ? std::optional<LogEvent>(*e) : std::nullopt;
      })
      .def("verify", &EventLog::verify)
      .def_property_readonly("dir", &EventLog::dir);
  log.def("payload_hash", [](const std::string& j) { return log_payload_hash(Json::parse(j)); });
  log.def("event_hash", &log_event_hash);

  // ---- mixture ----
  auto mx = m.def_submodule("mixture", "data mixture weights, hash, decay, ablations, sampling");
  using namespace mixture;
  mx.attr("SOURCES") = kSources;
  mx.attr("DECAY_SOURCES") = kDecaySources;
  mx.attr("WEIGHT_SUM_TOL") = 1e-9;
  py::class_<Mix>(mx, "Mix")
      .def(py::init(&make_mix), py::arg("mix_id"), py::arg("mix_bucket"), py::arg("phase"),
           py::arg("weights"))
      .def_readwrite("mix_id", &Mix::mix_id).def_readwrite("mix_bucket", &Mix::mix_bucket)
      .def_readwrite("phase", &Mix::phase)
      .def_property_readonly("weights", &Mix::named);
  mx.def("validate_mix", &validate);
  mx.def("canonical_json", &canonical_json);
  mx.def("mix_hash", [](const Mix& mm) { return sha256_hex(canonical_json(mm)); });
  mx.def("decay_reweight", &decay_reweight);
  mx.def("drop_source", &drop_source);
  mx.def("rung2_ablations", [](const Mix& base) {
    validate(base);
    if (base.weights.size() <= 1) throw Error("Config", "mix config: cannot drop the last source");
    std::vector<Mix> out;
    for (const auto& kv : base.weights) out.push_back(drop_source(base, kSources[kv.first]));
    return out;
  });
  mx.def("sample_source", &sample_source);
  mx.def("tokens_seen", [](std::optional<uint64_t> unique, uint32_t epochs) -> std::optional<uint64_t> {
    if (!unique) return std::nullopt;
    return *unique * epochs;
  });
  mx.def("flagship_catalog", [] {
    // (source, unique_tokens or None, epochs_min, epochs_max)
    std::vector<std::tuple<std::string, std::optional<uint64_t>, uint32_t, uint32_t>> c = {
        {"web", 20000000000000ull, 2, 3}, {"code", 4000000000000ull, 4, 4},
        {"math_science_arxiv", 1500000000000ull, 4, 4}, {"books_papers", std::nullopt, 2, 4},
        {"synthetic_rewrites", 40000000000000ull, 1, 1}, {"synthetic_reasoning", 10000000000000ull, 1, 1},
        {"procedural_arc", 2000000000000ull, 1, 1}, {"agentic_trajectories", 1000000000000ull, 1, 1}};
    return c;
  });

  // ---- tokenizer ----
  auto tk = m.def_submodule("tokenizer", "byte-fallback BPE tokenizer");
  using tok::Tokenizer;
  tk.attr("PRODUCTION_VOCAB_SIZE") = 256000;
  tk.attr("ARC_N_COLORS") = 10;
  py::class_<Tokenizer>(tk, "Tokenizer")
      .def_static("train", &Tokenizer::train, py::arg("docs"), py::arg("tokenizer_id"),
                  py::arg("vocab_size"), py::arg("byte_fallback") = true)
      .def_static("load", &Tokenizer::load)
      .def("save", &Tokenizer::save)
      .def("freeze", &Tokenizer::freeze)
      .def("encode", [](const Tokenizer& t, const std::string& s) { return t.encode_bytes(s); })
      .def("encode_bytes", [](const Tokenizer& t, py::bytes b) { return t.encode_bytes(std::string(b)); })
      .def("decode", [](const Tokenizer& t, const std::vector<uint32_t>& ids) {
        const std::string out = t.decode_bytes(ids);
        PyObject* u = PyUnicode_DecodeUTF8(out.data(), static_cast<Py_ssize_t>(out.size()), "strict");
        if (u == nullptr) {
          PyErr_Clear();
          throw Error("Message", "decoded bytes are not valid UTF-8");
        }
        return py::reinterpret_steal<py::str>(u);
      })
      .def("decode_bytes", [](const Tokenizer& t, const std::vector<uint32_t>& ids) {
        return py::bytes(t.decode_bytes(ids));
      })
      .def("encode_grid", &Tokenizer::encode_grid)
      .def("tokens_per_word", &Tokenizer::tokens_per_word)
      .def("vocab_jsonl", [](const Tokenizer& t) { return py::bytes(t.vocab_jsonl()); })
      .def("vocab_hash", &Tokenizer::vocab_hash)
      .def("to_contract", [](const Tokenizer& t) { return t.contract().dump(); })
      .def_readonly("tokenizer_id", &Tokenizer::tokenizer_id)
      .def_readonly("vocab_size", &Tokenizer::vocab_size)
      .def_readonly("frozen", &Tokenizer::frozen)
      .def_readonly("frozen_at", &Tokenizer::frozen_at)
      .def_readonly("corpus_hash", &Tokenizer::corpus_hash)
      .def_readonly("merges", &Tokenizer::merges)
      .def_readonly("special_tokens", &Tokenizer::specials);
  tk.def("baseline_byte_tokens_per_word", [](const std::string& text) {
    size_t words = 0;
    bool in = false;
    for (unsigned char c : text) {
      const bool ws = std::isspace(c);
      if (!ws && !in) ++words;
      in = !ws;
    }
    return words == 0 ? 0.0 : static_cast<double>(text.size()) / words;
  });
}
