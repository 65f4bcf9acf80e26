// Synthetic-data generation: style rewrites with a source-grounded fact check, rejection
// sampling of reasoning traces, procedural ARC-style grid families with dihedral x colour
// augmentation, and agentic trajectories in a sandbox.
//
// The generator, verifier, sandbox and token counter are callables handed in by the caller
// (the batch generation engine, a verifier registry, a sandbox pool, a tokenizer), so nothing
// here starts an engine or reads a clock.
// (reference: synth/src/lib.rs:78-563 rewrites, synth/src/reject.rs:18-402 rejection sampling,
//  synth/src/arc.rs:19-993 grid families, synth/src/agentic.rs:12-219 trajectories)
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <array>
#include <set>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

using GenFn = std::function<std::vector<std::string>(std::vector<std::string>, uint32_t, float)>;
using CountFn = std::function<uint32_t(const std::string&)>;

constexpr uint32_t kMaxTokens = 512, kMaxBatch = 8;
constexpr float kTemperature = 0.7f;

bool is_ws(unsigned char c) { return c == ' ' || (c >= 9 && c <= 13); }
std::vector<std::string> words(const std::string& s) {
  std::vector<std::string> out;
  std::string cur;
  for (unsigned char c : s) {
    if (is_ws(c)) {
      if (!cur.empty()) out.push_back(cur);
      cur.clear();
    } else {
      cur.push_back(static_cast<char>(c));
    }
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}
std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && is_ws(s[a])) ++a;
  while (b > a && is_ws(s[b - 1])) --b;
  return s.substr(a, b - a);
}
std::string lower(std::string s) {
  for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  return s;
}
size_t n_chars(const std::string& s) {   // UTF-8 code points
  size_t n = 0;
  for (unsigned char c : s) n += (c & 0xC0) != 0x80;
  return n;
}

std::vector<std::string> generate_chunked(const GenFn& gen, const std::vector<std::string>& prompts, uint32_t max_tokens,
                                          float temperature, size_t max_batch) {
  std::vector<std::string> out;
  for (size_t i = 0; i < prompts.size(); i += max_batch) {
    std::vector<std::string> chunk(prompts.begin() + i, prompts.begin() + std::min(prompts.size(), i + max_batch));
    const auto got = gen(chunk, max_tokens, temperature);
    if (got.size() != chunk.size())
      throw Error("LengthMismatch", "generator returned " + std::to_string(got.size()) + " completions for " +
                                        std::to_string(chunk.size()) + " prompts");
    out.insert(out.end(), got.begin(), got.end());
  }
  return out;
}
uint32_t token_count(const std::string& text, const CountFn& counter) {
  if (text.empty()) return 0;
  if (counter) return counter(text);
  return static_cast<uint32_t>(words(text).size());
}

// ------------------------------------------------------------------------------ rewrites
const char* const kStyles[] = {"encyclopedia", "textbook", "conversational", "news", "technical", "simplified"};
void check_style(const std::string& s) {
  for (const char* k : kStyles)
    if (s == k) return;
  throw Error("Message", "unknown style " + s);
}
std::string rewrite_prompt(const std::string& text, const std::string& style) {
  check_style(style);
  if (text.empty()) throw Error("EmptySource", "empty source");
  return "Rephrase the document in " + style + " style. Preserve every fact. Do not add facts.\n\nDocument:\n" + text;
}
std::vector<std::string> numbers_in(const std::string& text) {
  std::vector<std::string> out;
  size_t i = 0;
  auto digit = [&](size_t k) { return k < text.size() && text[k] >= '0' && text[k] <= '9'; };
  while (i < text.size()) {
    if (!digit(i)) {
      ++i;
      continue;
    }
    const size_t start = i;
    while (digit(i)) ++i;
    if (i < text.size() && text[i] == '.' && digit(i + 1)) {
      ++i;
      while (digit(i)) ++i;
    }
    out.push_back(text.substr(start, i - start));
  }
  return out;
}
std::vector<std::string> extract_claims(const std::string& text) {
  std::vector<std::string> out;
  std::string cur;
  auto flush = [&] {
    const std::string t = trim(cur);
    if (!t.empty()) out.push_back(t);
    cur.clear();
  };
  for (size_t i = 0; i < text.size(); ++i) {
    cur.push_back(text[i]);
    const char c = text[i];
    if ((c == '.' || c == '!' || c == '?') && i + 1 < text.size() && is_ws(text[i + 1])) {
      flush();
      while (i + 1 < text.size() && is_ws(text[i + 1])) ++i;
    }
  }
  flush();
  return out;
}
const std::set<std::string> kStop = {"that", "this", "with", "from", "they", "them", "have", "been", "were", "will", "would",
                                     "could", "should", "into", "over", "under", "than", "then", "when", "what", "which", "their"};
std::string check_claim(const std::string& source, const std::string& claim) {
  if (source.empty()) throw Error("EmptySource", "empty source");
  if (words(claim).empty()) return "not_in_source";
  const auto src_nums = numbers_in(source);
  if (!src_nums.empty()) {
    const std::set<std::string> have(src_nums.begin(), src_nums.end());
    for (const auto& n : numbers_in(claim))
      if (!have.count(n)) return "contradicted";
  }
  const auto src_tok = words(lower(source)), claim_tok = words(lower(claim));
  std::vector<std::string> content;
  for (const auto& t : claim_tok)
    if (n_chars(t) >= 4 && !kStop.count(t)) content.push_back(t);
  const std::set<std::string> content_set(content.begin(), content.end());
  for (size_t i = 0; i + 1 < src_tok.size(); ++i)
    if ((src_tok[i] == "not" || src_tok[i] == "no") && content_set.count(src_tok[i + 1])) return "contradicted";
  if (!content.empty()) {
    const std::set<std::string> src_set(src_tok.begin(), src_tok.end());
    for (const auto& w : content)
      if (!src_set.count(w)) return "not_in_source";
    return "supported";
  }
  auto joined = [](const std::vector<std::string>& v) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? " " : "") + v[i];
    return s;
  };
  return joined(src_tok).find(joined(claim_tok)) != std::string::npos ? "supported" : "not_in_source";
}
struct Claim {
  std::string text, verdict;
};
struct FactCheck {
  std::vector<Claim> claims;
  size_t count(const char* v) const {
    size_t n = 0;
    for (auto& c : claims) n += c.verdict == v;
    return n;
  }
};
FactCheck fact_check(const std::string& source, const std::string& rewrite) {
  if (source.empty()) throw Error("EmptySource", "empty source");
  FactCheck f;
  for (auto& t : extract_claims(rewrite)) f.claims.push_back({t, check_claim(source, t)});
  return f;
}
struct Rewrite {
  std::string source_id, style, text;
  uint32_t token_count = 0;
  FactCheck fact_check;
  bool accepted = false;
};
double precision(const std::vector<std::tuple<std::string, std::string, std::string>>& examples) {
  uint64_t tp = 0, fp = 0;
  for (auto& [source, claim, gold] : examples)
    if (check_claim(source, claim) == "supported") (gold == "supported" ? tp : fp) += 1;
  return tp + fp == 0 ? 0.0 : static_cast<double>(tp) / static_cast<double>(tp + fp);
}

class Orchestrator {
 public:
  Orchestrator(GenFn gen, uint32_t max_tokens, float temperature, uint32_t max_batch, std::vector<std::string> styles,
               CountFn counter)
      : gen_(std::move(gen)), counter_(std::move(counter)), max_tokens_(max_tokens), temperature_(temperature),
        max_batch_(max_batch), styles_(std::move(styles)) {
    for (auto& s : styles_) check_style(s);
    if (max_batch_ == 0) throw Error("Message", "max_batch must be > 0");
  }
  Rewrite rephrase(const std::string& source_id, const std::string& text, const std::string& style) const {
    const auto out = generate_chunked(gen_, {rewrite_prompt(text, style)}, max_tokens_, temperature_, 1);
    return finish(source_id, text, style, out[0]);
  }
  // docs: (source_id, text); result is docs-major, then styles
  std::vector<Rewrite> rephrase_many(const std::vector<std::pair<std::string, std::string>>& docs,
                                     std::optional<std::vector<std::string>> styles) const {
    if (docs.empty()) throw Error("EmptyBatch", "empty batch");
    const auto& use = styles ? *styles : styles_;
    std::vector<std::string> prompts;
    for (auto& d : docs)
      for (auto& s : use) prompts.push_back(rewrite_prompt(d.second, s));
    const auto outs = generate_chunked(gen_, prompts, max_tokens_, temperature_, max_batch_);
    std::vector<Rewrite> res;
    size_t k = 0;
    for (auto& d : docs)
      for (auto& s : use) res.push_back(finish(d.first, d.second, s, outs[k++]));
    return res;
  }

 private:
  Rewrite finish(const std::string& id, const std::string& src, const std::string& style, const std::string& completion) const {
    Rewrite r;
    r.source_id = id;
    r.style = style;
    r.text = completion;
    r.fact_check = fact_check(src, completion);
    r.accepted = r.fact_check.count("contradicted") == 0;
    r.token_count = token_count(completion, counter_);
    return r;
  }
  GenFn gen_;
  CountFn counter_;
  uint32_t max_tokens_;
  float temperature_;
  uint32_t max_batch_;
  std::vector<std::string> styles_;
};

// -------------------------------------------------------------------- rejection sampling
const char* const kDomains[] = {"math", "code", "lean", "grid", "market"};
struct Problem {
  std::string problem_id, domain, prompt, verifier_id;
};
struct Sample {
  std::string problem_id, text, answer;
  bool passed = false;
  uint32_t token_count = 0;
};
struct RejectionResult {
  std::string problem_id;
  uint32_t n_generated = 0, n_accepted = 0;
  std::vector<Sample> samples;
  double rate() const { return n_generated == 0 ? 0.0 : static_cast<double>(n_accepted) / n_generated; }
};
std::string solve_prompt(const Problem& p) {
  if (p.prompt.empty()) throw Error("EmptyPrompt", "empty prompt");
  return "Solve the following " + p.domain + " problem. Put the final answer after the reasoning.\n\nProblem:\n" + p.prompt;
}
std::vector<std::string> lines_of(const std::string& text) {
  std::vector<std::string> out;
  size_t off = 0;
  while (off < text.size()) {
    size_t nl = text.find('\n', off);
    if (nl == std::string::npos) nl = text.size();
    std::string line = text.substr(off, nl - off);
    if (!line.empty() && line.back() == '\r') line.pop_back();
    out.push_back(line);
    off = nl + 1;
  }
  return out;
}
// "answer" (any case), optional blanks, ':', optional blanks, then a non-empty rest
std::optional<std::string> answer_of_line(const std::string& line) {
  if (line.size() < 6 || lower(line.substr(0, 6)) != "answer") return std::nullopt;
  size_t i = 6;
  while (i < line.size() && is_ws(line[i])) ++i;
  if (i >= line.size() || line[i] != ':') return std::nullopt;
  ++i;
  while (i < line.size() && is_ws(line[i])) ++i;
  if (i >= line.size()) return std::nullopt;
  return trim(line.substr(i));
}
std::optional<std::string> last_fence(const std::string& text) {
  std::optional<std::string> last;
  size_t i = 0;
  while (i < text.size()) {
    const size_t open = text.find("```", i);
    if (open == std::string::npos) break;
    if (open != 0 && text[open - 1] != '\n') {
      i = open + 3;
      continue;
    }
    const size_t nl = text.find('\n', open + 3);
    if (nl == std::string::npos) break;
    const size_t close = text.find("```", nl + 1);
    if (close == std::string::npos) break;
    last = text.substr(nl + 1, close - nl - 1);
    i = close + 3;
  }
  return last;
}
std::string extract_answer(const std::string& raw) {
  size_t end = raw.size();
  while (end > 0 && is_ws(raw[end - 1])) --end;
  const std::string text = raw.substr(0, end);
  if (text.empty()) return "";
  const auto lines = lines_of(text);
  std::optional<std::string> ans;
  for (auto& l : lines)
    if (auto a = answer_of_line(l)) ans = a;
  if (ans) return *ans;
  if (auto f = last_fence(text)) return *f;
  for (size_t i = lines.size(); i-- > 0;)
    if (!trim(lines[i]).empty()) return lines[i];
  return "";
}
double verified_correct_rate(const std::vector<RejectionResult>& rs) {
  uint64_t g = 0, a = 0;
  for (auto& r : rs) {
    g += r.n_generated;
    a += r.n_accepted;
  }
  return g == 0 ? 0.0 : static_cast<double>(a) / static_cast<double>(g);
}

class RejectionSampler {
 public:
  using VerifyFn = std::function<bool(const Problem&, const std::string&)>;
  RejectionSampler(GenFn gen, VerifyFn verify, uint32_t n_samples, uint32_t max_tokens, float temperature, uint32_t max_batch,
                   CountFn counter)
      : gen_(std::move(gen)), verify_(std::move(verify)), counter_(std::move(counter)), n_samples_(n_samples),
        max_tokens_(max_tokens), temperature_(temperature), max_batch_(max_batch) {
    if (max_batch_ == 0) throw Error("Message", "max_batch must be > 0");
  }
  RejectionResult sample(const Problem& p, std::optional<uint32_t> n) const { return sample_many({p}, n, true)[0]; }
  std::vector<RejectionResult> sample_many(const std::vector<Problem>& problems, std::optional<uint32_t> n_opt,
                                           bool single = false) const {
    const uint32_t n = n_opt ? *n_opt : n_samples_;
    if (problems.empty()) throw Error("EmptyBatch", "empty batch");
    if (n == 0) throw Error("ZeroSamples", "n_samples must be > 0");
    (void)single;
    std::vector<std::string> prompts;
    for (auto& p : problems) {
      const std::string prompt = solve_prompt(p);
      prompts.insert(prompts.end(), n, prompt);
    }
    const auto outs = generate_chunked(gen_, prompts, max_tokens_, temperature_, max_batch_);
    std::vector<RejectionResult> res;
    size_t k = 0;
    for (auto& p : problems) {
      RejectionResult r;
      r.problem_id = p.problem_id;
      r.n_generated = n;
      for (uint32_t i = 0; i < n; ++i) {
        Sample s;
        s.problem_id = p.problem_id;
        s.text = outs[k++];
        s.answer = extract_answer(s.text);
        s.passed = verify_(p, s.answer);
        s.token_count = token_count(s.text, counter_);
        r.n_accepted += s.passed;
        r.samples.push_back(std::move(s));
      }
      res.push_back(std::move(r));
    }
    return res;
  }

 private:
  GenFn gen_;
  VerifyFn verify_;
  CountFn counter_;
  uint32_t n_samples_, max_tokens_;
  float temperature_;
  uint32_t max_batch_;
};

// --------------------------------------------------------------------------- ARC grids
using Cells = std::vector<std::vector<uint8_t>>;
constexpr int kColors = 10, kMaxGrid = 30, kMaxSampleDim = 8, kMaxPairAttempts = 10000;
const char* const kDihedral[] = {"identity", "rot90", "rot180", "rot270", "flip_h", "flip_v", "transpose", "anti_transpose"};
const char* const kFamilies[] = {"translate", "recolor", "crop", "tile", "gravity", "mirror", "scale", "border"};

const Cells& checked(const Cells& c) {
  if (c.empty() || c[0].empty()) throw Error("EmptyGrid", "empty grid");
  const size_t rows = c.size(), cols = c[0].size();
  if (rows > kMaxGrid || cols > kMaxGrid)
    throw Error("GridSize", "grid size " + std::to_string(rows) + "x" + std::to_string(cols) + " out of range");
  for (auto& row : c) {
    if (row.size() != cols) throw Error("JaggedGrid", "jagged grid");
    for (uint8_t v : row)
      if (v >= kColors) throw Error("BadColor", "ARC color " + std::to_string(v) + " out of range");
  }
  return c;
}
int dihedral_index(const std::string& name) {
  for (int i = 0; i < 8; ++i)
    if (name == kDihedral[i]) return i;
  throw Error("Message", "unknown dihedral " + name);
}
// Every element of D4 is "optionally transpose, then optionally flip rows, then optionally flip
// columns" of the source index; the table gives (transpose, flip source row, flip source col).
Cells dihedral(const Cells& src, int k) {
  if (k < 0 || k >= 8) throw Error("BadDihedral", "dihedral index " + std::to_string(k) + " out of range");
  checked(src);
  static const bool T[8] = {false, true, false, true, false, false, true, true};
  static const bool FR[8] = {false, true, true, false, false, true, false, true};
  static const bool FC[8] = {false, false, true, true, true, false, false, true};
  const size_t h = src.size(), w = src[0].size();
  const size_t oh = T[k] ? w : h, ow = T[k] ? h : w;
  Cells out(oh, std::vector<uint8_t>(ow));
  for (size_t r = 0; r < oh; ++r)
    for (size_t c = 0; c < ow; ++c) {
      size_t sr = T[k] ? c : r, sc = T[k] ? r : c;
      if (FR[k]) sr = h - 1 - sr;
      if (FC[k]) sc = w - 1 - sc;
      out[r][c] = src[sr][sc];
    }
  return out;
}
Cells color_perm(const Cells& src, const std::vector<uint8_t>& perm) {
  if (perm.size() != kColors) throw Error("BadPermutation", "color permutation is not a permutation of 0..10");
  bool seen[kColors] = {};
  for (uint8_t v : perm) {
    if (v >= kColors || seen[v]) throw Error("BadPermutation", "color permutation is not a permutation of 0..10");
    seen[v] = true;
  }
  Cells out = checked(src);
  for (auto& row : out)
    for (auto& c : row) c = perm[c];
  return out;
}

struct Pair {
  Cells input, output;
};
struct Task {
  std::string family_id;
  uint64_t seed = 0;
  std::vector<Pair> train;
  Pair test;
};
struct FamilySpec {
  std::string kind;
  std::map<std::string, int> params;
  std::string family_id() const {
    std::string s = kind;
    bool first = true;
    for (auto& kv : params) {
      s += (first ? ":" : ",") + kv.first + "=" + std::to_string(kv.second);
      first = false;
    }
    return s;
  }
  int get(const char* k) const { return params.at(k); }
};
void need_keys(const FamilySpec& s, std::initializer_list<const char*> keys) {
  if (s.params.size() != keys.size()) throw Error("UnknownFamily", "unknown family");
  for (const char* k : keys)
    if (!s.params.count(k)) throw Error("UnknownFamily", "unknown family");
}
void need(bool ok) {
  if (!ok) throw Error("UnknownFamily", "unknown family");
}
bool is_color(int v) { return v >= 0 && v < kColors; }
void validate(const FamilySpec& s) {
  const std::string& k = s.kind;
  if (k == "translate") {
    need_keys(s, {"dx", "dy", "bg"});
    need(is_color(s.get("bg")));
  } else if (k == "recolor") {
    need_keys(s, {"src", "dst"});
    need(is_color(s.get("src")) && is_color(s.get("dst")) && s.get("src") != s.get("dst"));
  } else if (k == "crop") {
    need_keys(s, {"bg"});
    need(is_color(s.get("bg")));
  } else if (k == "tile") {
    need_keys(s, {"nx", "ny"});
    need(s.get("nx") >= 1 && s.get("ny") >= 1 && s.get("nx") <= kMaxGrid && s.get("ny") <= kMaxGrid);
  } else if (k == "gravity") {
    need_keys(s, {"dir", "bg"});
    need(s.get("dir") >= 0 && s.get("dir") <= 3 && is_color(s.get("bg")));
  } else if (k == "mirror") {
    need_keys(s, {"dihedral"});
    need(s.get("dihedral") >= 0 && s.get("dihedral") < 8);
  } else if (k == "scale") {
    need_keys(s, {"factor"});
    need(s.get("factor") == 2 || s.get("factor") == 3);
  } else if (k == "border") {
    need_keys(s, {"color", "width"});
    need(is_color(s.get("color")) && (s.get("width") == 1 || s.get("width") == 2));
  } else {
    throw Error("Message", "unknown family " + k);
  }
}
size_t wrap_index(int64_t i, size_t n) {
  const int64_t m = static_cast<int64_t>(n);
  return static_cast<size_t>(((i % m) + m) % m);
}
Cells apply_family(const Cells& g, const FamilySpec& s) {
  validate(s);
  const size_t h = g.size(), w = g[0].size();
  const std::string& k = s.kind;
  Cells out;
  if (k == "translate") {
    const uint8_t bg = static_cast<uint8_t>(s.get("bg"));
    out.assign(h, std::vector<uint8_t>(w, bg));
    for (size_t r = 0; r < h; ++r)
      for (size_t c = 0; c < w; ++c)
        if (g[r][c] != bg)
          out[wrap_index(static_cast<int64_t>(r) + s.get("dy"), h)][wrap_index(static_cast<int64_t>(c) + s.get("dx"), w)] = g[r][c];
  } else if (k == "recolor") {
    out = g;
    for (auto& row : out)
      for (auto& c : row)
        if (c == s.get("src")) c = static_cast<uint8_t>(s.get("dst"));
  } else if (k == "crop") {
    const uint8_t bg = static_cast<uint8_t>(s.get("bg"));
    size_t r0 = h, r1 = 0, c0 = w, c1 = 0;
    for (size_t r = 0; r < h; ++r)
      for (size_t c = 0; c < w; ++c)
        if (g[r][c] != bg) {
          r0 = std::min(r0, r), r1 = std::max(r1, r), c0 = std::min(c0, c), c1 = std::max(c1, c);
        }
    if (r0 == h) return Cells{{bg}};
    for (size_t r = r0; r <= r1; ++r) out.emplace_back(g[r].begin() + c0, g[r].begin() + c1 + 1);
  } else if (k == "tile") {
    for (int y = 0; y < s.get("ny"); ++y)
      for (size_t r = 0; r < h; ++r) {
        std::vector<uint8_t> row;
        for (int x = 0; x < s.get("nx"); ++x) row.insert(row.end(), g[r].begin(), g[r].end());
        out.push_back(row);
      }
  } else if (k == "gravity") {
    const uint8_t bg = static_cast<uint8_t>(s.get("bg"));
    const int dir = s.get("dir");   // 0 down, 1 up, 2 left, 3 right
    out.assign(h, std::vector<uint8_t>(w, bg));
    if (dir <= 1) {
      for (size_t c = 0; c < w; ++c) {
        std::vector<uint8_t> objs;
        for (size_t r = 0; r < h; ++r)
          if (g[r][c] != bg) objs.push_back(g[r][c]);
        const size_t start = dir == 0 ? h - objs.size() : 0;
        for (size_t i = 0; i < objs.size(); ++i) out[start + i][c] = objs[i];
      }
    } else {
      for (size_t r = 0; r < h; ++r) {
        std::vector<uint8_t> objs;
        for (size_t c = 0; c < w; ++c)
          if (g[r][c] != bg) objs.push_back(g[r][c]);
        const size_t start = dir == 2 ? 0 : w - objs.size();
        for (size_t i = 0; i < objs.size(); ++i) out[r][start + i] = objs[i];
      }
    }
  } else if (k == "mirror") {
    out = dihedral(g, s.get("dihedral"));
  } else if (k == "scale") {
    const size_t f = static_cast<size_t>(s.get("factor"));
    out.assign(h * f, std::vector<uint8_t>(w * f));
    for (size_t r = 0; r < h * f; ++r)
      for (size_t c = 0; c < w * f; ++c) out[r][c] = g[r / f][c / f];
  } else {   // border
    const size_t bw = static_cast<size_t>(s.get("width"));
    out.assign(h + 2 * bw, std::vector<uint8_t>(w + 2 * bw, static_cast<uint8_t>(s.get("color"))));
    for (size_t r = 0; r < h; ++r)
      for (size_t c = 0; c < w; ++c) out[r + bw][c + bw] = g[r][c];
  }
  return checked(out);
}

struct SplitMix {
  uint64_t state;
  uint64_t next() {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  size_t below(size_t n) { return static_cast<size_t>(next() % n); }
};
std::pair<size_t, size_t> max_input_hw(const FamilySpec& s) {
  if (s.kind == "tile") return {kMaxGrid / s.get("ny"), kMaxGrid / s.get("nx")};
  if (s.kind == "scale") return {kMaxGrid / s.get("factor"), kMaxGrid / s.get("factor")};
  if (s.kind == "border") return {kMaxGrid - 2 * s.get("width"), kMaxGrid - 2 * s.get("width")};
  return {kMaxGrid, kMaxGrid};
}
Task generate_task(const FamilySpec& spec, uint64_t seed, uint32_t n_train) {
  validate(spec);
  if (n_train == 0) throw Error("EmptyTrain", "empty train");
  SplitMix rng{seed};
  auto [mh, mw] = max_input_hw(spec);
  mh = std::min<size_t>(mh, kMaxSampleDim);
  mw = std::min<size_t>(mw, kMaxSampleDim);
  std::vector<Pair> pairs;
  std::set<std::pair<Cells, Cells>> seen;
  int attempts = 0;
  while (pairs.size() < n_train + 1u) {
    if (++attempts > kMaxPairAttempts) throw Error("Message", "could not sample distinct pairs");
    const size_t h = 1 + rng.below(mh), w = 1 + rng.below(mw);
    Cells in(h, std::vector<uint8_t>(w));
    for (auto& row : in)
      for (auto& c : row) c = static_cast<uint8_t>(rng.below(kColors));
    Cells out = apply_family(in, spec);
    if (!seen.insert({in, out}).second) continue;
    pairs.push_back({std::move(in), std::move(out)});
  }
  Task t;
  t.family_id = spec.family_id();
  t.seed = seed;
  t.test = pairs.back();
  pairs.pop_back();
  t.train = std::move(pairs);
  return t;
}
std::vector<FamilySpec> parameter_grid() {
  std::vector<FamilySpec> g;
  auto add = [&](const char* kind, std::map<std::string, int> p) { g.push_back({kind, std::move(p)}); };
  for (int bg = 0; bg < kColors; ++bg)
    for (int dx = -3; dx <= 3; ++dx)
      for (int dy = -3; dy <= 3; ++dy) add("translate", {{"dx", dx}, {"dy", dy}, {"bg", bg}});
  for (int a = 0; a < kColors; ++a)
    for (int b = 0; b < kColors; ++b)
      if (a != b) add("recolor", {{"src", a}, {"dst", b}});
  for (int bg = 0; bg < kColors; ++bg) add("crop", {{"bg", bg}});
  for (int nx = 1; nx < 5; ++nx)
    for (int ny = 1; ny < 5; ++ny) add("tile", {{"nx", nx}, {"ny", ny}});
  for (int bg = 0; bg < kColors; ++bg)
    for (int dir = 0; dir < 4; ++dir) add("gravity", {{"dir", dir}, {"bg", bg}});
  for (int d = 0; d < 8; ++d) add("mirror", {{"dihedral", d}});
  for (int f : {2, 3}) add("scale", {{"factor", f}});
  for (int c = 0; c < kColors; ++c)
    for (int w : {1, 2}) add("border", {{"color", c}, {"width", w}});
  return g;
}
std::vector<FamilySpec> sample_family_specs(uint32_t n, uint64_t seed) {
  if (n == 0) return {};
  auto specs = parameter_grid();
  if (n > specs.size()) throw Error("Message", "requested more family specs than the parameter grid");
  SplitMix rng{seed};
  for (size_t i = 0; i < specs.size(); ++i) std::swap(specs[i], specs[i + rng.below(specs.size() - i)]);
  specs.resize(n);
  return specs;
}
Pair augment_pair(const Pair& p, int k, const std::vector<uint8_t>& perm) {
  return {color_perm(dihedral(p.input, k), perm), color_perm(dihedral(p.output, k), perm)};
}
Task augment_task(const Task& t, int k, const std::vector<uint8_t>& perm) {
  Task out;
  out.family_id = t.family_id;
  out.seed = t.seed;
  for (auto& p : t.train) out.train.push_back(augment_pair(p, k, perm));
  out.test = augment_pair(t.test, k, perm);
  return out;
}
struct Diversity {
  uint64_t n_tasks = 0, n_families = 0, unique_test_inputs = 0, unique_test_outputs = 0, unique_tasks = 0, unique_shapes = 0;
  std::array<uint64_t, 10> color_histogram{};
  double collision_rate = 0;
};
Diversity diversity_stats(const std::vector<Task>& tasks) {
  Diversity d;
  std::set<std::string> fams;
  std::set<Cells> tin, tout;
  std::set<std::pair<size_t, size_t>> shapes;
  std::set<std::tuple<std::vector<std::pair<Cells, Cells>>, Cells, Cells>> keys;
  auto acc = [&](const Cells& g) {
    shapes.insert({g.size(), g.empty() ? 0 : g[0].size()});
    for (auto& row : g)
      for (uint8_t c : row)
        if (c < 10) ++d.color_histogram[c];
  };
  for (auto& t : tasks) {
    fams.insert(t.family_id);
    tin.insert(t.test.input);
    tout.insert(t.test.output);
    std::vector<std::pair<Cells, Cells>> tr;
    for (auto& p : t.train) {
      tr.push_back({p.input, p.output});
      acc(p.input);
      acc(p.output);
    }
    keys.insert({tr, t.test.input, t.test.output});
    acc(t.test.input);
    acc(t.test.output);
  }
  d.n_tasks = tasks.size();
  d.n_families = fams.size();
  d.unique_test_inputs = tin.size();
  d.unique_test_outputs = tout.size();
  d.unique_tasks = keys.size();
  d.unique_shapes = shapes.size();
  d.collision_rate = tasks.empty() ? 0.0 : 1.0 - static_cast<double>(keys.size()) / static_cast<double>(tasks.size());
  return d;
}
std::vector<Task> corpus_sample(const std::vector<FamilySpec>& specs, uint64_t seed, uint32_t n_train, uint32_t n) {
  if (n == 0) throw Error("EmptyTasks", "empty tasks");
  if (specs.empty()) throw Error("UnknownFamily", "unknown family");
  if (n_train == 0) throw Error("EmptyTrain", "empty train");
  std::vector<Task> out;
  for (uint32_t i = 0; i < n; ++i) out.push_back(generate_task(specs[i % specs.size()], seed + i, n_train));
  return out;
}

// -------------------------------------------------------------------- agentic trajectories
struct Step {
  std::string tool, args, result;
};
struct Trajectory {
  std::string task_id, outcome;   // verified | failed | truncated
  std::vector<Step> steps;
};
using SandboxFn = std::function<std::string(const std::string&, const std::string&)>;

Trajectory run_trajectory(const GenFn& gen, const SandboxFn& sandbox, const std::string& task_id, const std::string& prompt,
                          uint32_t max_steps, uint32_t max_tokens, float temperature) {
  Trajectory t;
  t.task_id = task_id;
  t.outcome = "truncated";
  std::string context = prompt;
  for (uint32_t i = 0; i < max_steps; ++i) {
    const auto out = generate_chunked(gen, {context}, max_tokens, temperature, 1);
    const std::string call = trim(out[0]);
    if (call.empty()) {
      t.outcome = "failed";
      break;
    }
    size_t sp = 0;
    while (sp < call.size() && !is_ws(call[sp])) ++sp;
    Step s;
    s.tool = call.substr(0, sp);
    while (sp < call.size() && is_ws(call[sp])) ++sp;
    s.args = call.substr(sp);
    s.result = sandbox(s.tool, s.args);
    context += "\n" + s.tool + "\n" + s.args + "\n" + s.result;
    const bool submit = s.tool == "submit", verified = submit && s.result == "verified";
    t.steps.push_back(std::move(s));
    if (submit) {
      t.outcome = verified ? "verified" : "failed";
      break;
    }
  }
  return t;
}
std::vector<Trajectory> generate_one(const GenFn& gen, const SandboxFn& sb, const std::string& task_id, const std::string& prompt,
                                     uint32_t n, uint32_t max_steps, uint32_t max_tokens, float temperature) {
  if (n == 0) throw Error("ZeroSamples", "n_samples must be > 0");
  if (prompt.empty()) throw Error("EmptyPrompt", "empty prompt");
  std::vector<Trajectory> out;
  for (uint32_t i = 0; i < n; ++i) out.push_back(run_trajectory(gen, sb, task_id, prompt, max_steps, max_tokens, temperature));
  return out;
}

}  // namespace

void bind_synth(py::module_& m) {
  auto sm = m.def_submodule("synth", "synthetic data: rewrites, rejection sampling, ARC grids, agentic traces");
  sm.attr("SCHEMA_VERSION") = 1;
  sm.attr("DEFAULT_MAX_TOKENS") = kMaxTokens;
  sm.attr("DEFAULT_TEMPERATURE") = kTemperature;
  sm.attr("DEFAULT_MAX_BATCH") = kMaxBatch;
  sm.attr("DEFAULT_N_SAMPLES") = 8;
  sm.attr("STYLES") = std::vector<std::string>(std::begin(kStyles), std::end(kStyles));
  sm.attr("DOMAINS") = std::vector<std::string>(std::begin(kDomains), std::end(kDomains));

  sm.def("generate_prompt", &rewrite_prompt, py::arg("text"), py::arg("style"));
  sm.def("extract_claims", &extract_claims);
  sm.def("check_claim", &check_claim, py::arg("source"), py::arg("claim"));
  sm.def("token_count", [](const std::string& t, py::object counter) {
    return token_count(t, counter.is_none() ? CountFn() : py::cast<CountFn>(counter));
  }, py::arg("text"), py::arg("counter") = py::none());
  sm.def("precision", &precision);
  py::class_<Claim>(sm, "Claim").def_readonly("text", &Claim::text).def_readonly("verdict", &Claim::verdict);
  py::class_<FactCheck>(sm, "FactCheck")
      .def_readonly("claims", &FactCheck::claims)
      .def_property_readonly("n_supported", [](const FactCheck& f) { return f.count("supported"); })
      .def_property_readonly("n_contradicted", [](const FactCheck& f) { return f.count("contradicted"); })
      .def_property_readonly("n_not_in_source", [](const FactCheck& f) { return f.count("not_in_source"); });
  sm.def("fact_check", &fact_check, py::arg("source"), py::arg("rewrite"));
  sm.def("accept", [](const FactCheck& f) { return f.count("contradicted") == 0; });
  py::class_<Rewrite>(sm, "Rewrite")
      .def_readonly("source_id", &Rewrite::source_id)
      .def_readonly("style", &Rewrite::style)
      .def_readonly("text", &Rewrite::text)
      .def_readonly("token_count", &Rewrite::token_count)
      .def_readonly("fact_check", &Rewrite::fact_check)
      .def_readonly("accepted", &Rewrite::accepted);
  py::class_<Orchestrator>(sm, "Orchestrator")
      .def(py::init([](GenFn gen, uint32_t mt, float temp, uint32_t mb, std::optional<std::vector<std::string>> styles,
                       py::object counter) {
             return Orchestrator(std::move(gen), mt, temp, mb,
                                 styles ? *styles : std::vector<std::string>(std::begin(kStyles), std::end(kStyles)),
                                 counter.is_none() ? CountFn() : py::cast<CountFn>(counter));
           }),
           py::arg("generator"), py::arg("max_tokens") = kMaxTokens, py::arg("temperature") = kTemperature,
           py::arg("max_batch") = kMaxBatch, py::arg("styles") = py::none(), py::arg("tokenizer") = py::none())
      .def("rephrase", &Orchestrator::rephrase, py::arg("source_id"), py::arg("text"), py::arg("style"))
      .def("rephrase_many", &Orchestrator::rephrase_many, py::arg("docs"), py::arg("styles") = py::none());

  py::class_<Problem>(sm, "Problem")
      .def(py::init([](std::string id, std::string domain, std::string prompt, std::string verifier_id) {
             bool ok = false;
             for (const char* d : kDomains) ok = ok || domain == d;
             if (!ok) throw Error("Message", "unknown domain " + domain);
             return Problem{std::move(id), std::move(domain), std::move(prompt), std::move(verifier_id)};
           }),
           py::arg("problem_id"), py::arg("domain"), py::arg("prompt"), py::arg("verifier_id"))
      .def_readonly("problem_id", &Problem::problem_id)
      .def_readonly("domain", &Problem::domain)
      .def_readonly("prompt", &Problem::prompt)
      .def_readonly("verifier_id", &Problem::verifier_id);
  py::class_<Sample>(sm, "Sample")
      .def_readonly("problem_id", &Sample::problem_id)
      .def_readonly("text", &Sample::text)
      .def_readonly("answer", &Sample::answer)
      .def_readonly("passed", &Sample::passed)
      .def_readonly("token_count", &Sample::token_count);
  py::class_<RejectionResult>(sm, "RejectionResult")
      .def_readonly("problem_id", &RejectionResult::problem_id)
      .def_readonly("n_generated", &RejectionResult::n_generated)
      .def_readonly("n_accepted", &RejectionResult::n_accepted)
      .def_readonly("samples", &RejectionResult::samples)
      .def("verified_correct_rate", &RejectionResult::rate);
  sm.def("generate_solve_prompt", &solve_prompt);
  sm.def("extract_answer", &extract_answer);
  sm.def("verified_correct_rate", &verified_correct_rate);
  py::class_<RejectionSampler>(sm, "RejectionSampler")
      .def(py::init([](GenFn gen, RejectionSampler::VerifyFn verify, uint32_t n, uint32_t mt, float temp, uint32_t mb,
                       py::object counter) {
             return RejectionSampler(std::move(gen), std::move(verify), n, mt, temp, mb,
                                     counter.is_none() ? CountFn() : py::cast<CountFn>(counter));
           }),
           py::arg("generator"), py::arg("verifier"), py::arg("n_samples") = 8, py::arg("max_tokens") = kMaxTokens,
           py::arg("temperature") = kTemperature, py::arg("max_batch") = kMaxBatch, py::arg("tokenizer") = py::none())
      .def("sample", &RejectionSampler::sample, py::arg("problem"), py::arg("n") = py::none())
      .def("sample_many", [](const RejectionSampler& s, const std::vector<Problem>& ps, std::optional<uint32_t> n) {
        return s.sample_many(ps, n);
      }, py::arg("problems"), py::arg("n") = py::none());

  auto am = sm.def_submodule("arc", "procedural ARC-style grid families");
  am.attr("N_COLORS") = kColors;
  am.attr("MIN_GRID_SIZE") = 1;
  am.attr("MAX_GRID_SIZE") = kMaxGrid;
  am.attr("N_DIHEDRAL") = 8;
  am.attr("DEFAULT_N_TRAIN") = 3;
  am.attr("DIHEDRALS") = std::vector<std::string>(std::begin(kDihedral), std::end(kDihedral));
  am.attr("FAMILY_KINDS") = std::vector<std::string>(std::begin(kFamilies), std::end(kFamilies));
  am.def("validate_grid", [](const Cells& c) { return checked(c); });
  am.def("flatten", [](const Cells& c) {
    std::vector<uint8_t> out;
    for (auto& row : checked(c)) out.insert(out.end(), row.begin(), row.end());
    return py::bytes(reinterpret_cast<const char*>(out.data()), out.size());
  });
  am.def("dihedral_index", &dihedral_index);
  am.def("apply_dihedral", [](const Cells& c, py::object d) {
    return dihedral(c, py::isinstance<py::str>(d) ? dihedral_index(py::cast<std::string>(d)) : py::cast<int>(d));
  });
  am.def("apply_color_perm", &color_perm);
  py::class_<Pair>(am, "Pair")
      .def(py::init([](Cells i, Cells o) { return Pair{checked(i), checked(o)}; }))
      .def_readonly("input", &Pair::input)
      .def_readonly("output", &Pair::output);
  py::class_<Task>(am, "Task")
      .def_readonly("family_id", &Task::family_id)
      .def_readonly("seed", &Task::seed)
      .def_readonly("train", &Task::train)
      .def_readonly("test", &Task::test);
  py::class_<FamilySpec>(am, "FamilySpec")
      .def(py::init([](std::string kind, std::map<std::string, int> params) {
             bool ok = false;
             for (const char* k : kFamilies) ok = ok || kind == k;
             if (!ok) throw Error("Message", "unknown family " + kind);
             return FamilySpec{std::move(kind), std::move(params)};
           }))
      .def_readonly("kind", &FamilySpec::kind)
      .def_readonly("params", &FamilySpec::params)
      .def("family_id", &FamilySpec::family_id)
      .def("validate", [](const FamilySpec& s) { validate(s); })
      .def("apply", [](const FamilySpec& s, const Cells& g) { return apply_family(checked(g), s); })
      .def("generate", [](const FamilySpec& s, uint64_t seed, uint32_t n_train) { return generate_task(s, seed, n_train); },
           py::arg("seed"), py::arg("n_train") = 3);
  am.def("parameter_grid", &parameter_grid);
  am.def("sample_family_specs", &sample_family_specs, py::arg("n"), py::arg("seed"));
  am.def("augment_pair", [](const Pair& p, int k, const std::vector<uint8_t>& perm) { return augment_pair(p, k, perm); });
  am.def("augment_task", [](const Task& t, int k, const std::vector<uint8_t>& perm) { return augment_task(t, k, perm); });
  am.def("tokenize_grid", [](const std::function<std::vector<uint32_t>(py::bytes)>& enc, const Cells& c) {
    std::vector<uint8_t> flat;
    for (auto& row : checked(c)) flat.insert(flat.end(), row.begin(), row.end());
    return enc(py::bytes(reinterpret_cast<const char*>(flat.data()), flat.size()));
  });
  py::class_<Diversity>(am, "DiversityStats")
      .def_readonly("n_tasks", &Diversity::n_tasks)
      .def_readonly("n_families", &Diversity::n_families)
      .def_readonly("unique_test_inputs", &Diversity::unique_test_inputs)
      .def_readonly("unique_test_outputs", &Diversity::unique_test_outputs)
      .def_readonly("unique_tasks", &Diversity::unique_tasks)
      .def_readonly("color_histogram", &Diversity::color_histogram)
      .def_readonly("unique_shapes", &Diversity::unique_shapes)
      .def_readonly("collision_rate", &Diversity::collision_rate);
  am.def("diversity_stats", &diversity_stats);
  am.def("corpus_sample", &corpus_sample, py::arg("specs"), py::arg("seed"), py::arg("n_train"), py::arg("n"));

  auto gm = sm.def_submodule("agentic", "tool-calling trajectories in a sandbox");
  py::class_<Step>(gm, "Step").def_readonly("tool", &Step::tool).def_readonly("args", &Step::args).def_readonly("result", &Step::result);
  py::class_<Trajectory>(gm, "Trajectory")
      .def_readonly("task_id", &Trajectory::task_id)
      .def_readonly("steps", &Trajectory::steps)
      .def_readonly("outcome", &Trajectory::outcome);
  gm.def("generate_one", &generate_one, py::arg("generator"), py::arg("sandbox"), py::arg("task_id"), py::arg("prompt"),
         py::arg("n"), py::arg("max_steps"), py::arg("max_tokens") = kMaxTokens, py::arg("temperature") = kTemperature);
  gm.def("generate_batch",
         [](const GenFn& gen, const SandboxFn& sb, const std::vector<std::pair<std::string, std::string>>& tasks, uint32_t n,
            uint32_t max_steps, uint32_t max_tokens, float temperature) {
           if (tasks.empty()) throw Error("EmptyBatch", "empty batch");
           if (n == 0) throw Error("ZeroSamples", "n_samples must be > 0");
           for (auto& t : tasks)
             if (t.second.empty()) throw Error("EmptyPrompt", "empty prompt");
           std::vector<std::vector<Trajectory>> out;
           for (auto& t : tasks) out.push_back(generate_one(gen, sb, t.first, t.second, n, max_steps, max_tokens, temperature));
           return out;
         },
         py::arg("generator"), py::arg("sandbox"), py::arg("tasks"), py::arg("n"), py::arg("max_steps"),
         py::arg("max_tokens") = kMaxTokens, py::arg("temperature") = kTemperature);
  gm.def("outcome_verified_rate", [](const std::vector<Trajectory>& ts) {
    if (ts.empty()) return 0.0;
    size_t ok = 0;
    for (auto& t : ts) ok += t.outcome == "verified";
    return static_cast<double>(ok) / static_cast<double>(ts.size());
  });
  gm.def("keep_verified", [](const std::vector<Trajectory>& ts) {
    std::vector<Trajectory> out;
    for (auto& t : ts)
      if (t.outcome == "verified") out.push_back(t);
    return out;
  });
}
