// Data pipeline components and the batch generation engine:
//
//   extract      HTML / PDF / LaTeX -> text + sha256 (own tag walker; PDF text operators from
//                plain or Flate-compressed content streams; LaTeX comment stripping with math
//                kept verbatim)  (reference: data/extract/src/lib.rs:17-136, html.rs, latex.rs, pdf.rs)
//   dedup        normalise, paragraphs, exact dedup at document / paragraph grain, word-shingle
//                MinHash (hash = first 8 LE bytes of sha256(seed || shingle)), LSH band keys,
//                clusters keep the lowest content hash  (reference: data/dedup/src/lib.rs:36-437)
//   decontam     8-gram overlap index against eval items, method hash, shard scan, planted-item
//                check; embedding match is an explicit error  (reference: data/decontam/src/lib.rs:36-199)
//   classifiers  sharded scoring orchestrator with a journal, local FNV-hash scorer, agreement
//                gate against human labels  (reference: data/classifiers/src/lib.rs:18-30, 40-429)
//   serve        batch generation API of the local engine (deterministic hashed completions)
//                and the OpenAI-style body  (reference: serve/src/lib.rs:19-22, 130-227)
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <zlib.h>
#include <sys/stat.h>

#include <map>
#include <set>

#include "common.hpp"
#include "providers.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

std::string lower_ascii(std::string s) {
  for (char& c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
  return s;
}

// -------------------------------------------------------------------------------- extract
struct Extracted {
  std::string text, format, content_hash;
  std::optional<std::string> source;
  uint64_t bytes_in = 0;
};

bool valid_utf8(const std::string& s) {
  size_t i = 0;
  while (i < s.size()) {
    const unsigned char c = s[i];
    size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
    if (n == 0 || i + n > s.size()) return false;
    for (size_t j = 1; j < n; ++j)
      if ((static_cast<unsigned char>(s[i + j]) >> 6) != 2) return false;
    i += n;
  }
  return true;
}

const std::set<std::string> kSkipTags = {"script", "style", "noscript", "template"};
const std::set<std::string> kBlockTags = {
    "address", "article", "aside", "blockquote", "br", "dd", "div", "dl", "dt", "figcaption", "figure", "footer",
    "form", "h1", "h2", "h3", "h4", "h5", "h6", "header", "hr", "li", "main", "nav", "ol", "p", "pre", "section",
    "table", "tr", "ul"};
const std::set<std::string> kVoidTags = {"br", "hr", "img", "input", "meta", "link", "area", "base", "col", "embed",
                                         "source", "track", "wbr"};

void push_break(std::string& out) {
  if (!out.empty() && out.back() != '\n') out.push_back('\n');
}

void append_utf8(unsigned long cp, std::string& out) {
  if (cp < 0x80) out.push_back(static_cast<char>(cp));
  else if (cp < 0x800) {
    out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else if (cp < 0x10000) {
    out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else {
    out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  }
}

std::string decode_entities(const std::string& s) {
  static const std::map<std::string, unsigned long> named = {
#include "html_entities.inc"
      {"apos", 0x27}};
  std::string out;
  for (size_t i = 0; i < s.size();) {
    if (s[i] == '&') {
      const size_t semi = s.find(';', i);
      if (semi != std::string::npos && semi - i <= 10) {
        const std::string name = s.substr(i + 1, semi - i - 1);
        auto it = named.find(name);
        if (it != named.end()) {
          append_utf8(it->second, out);
          i = semi + 1;
          continue;
        }
        if (name.size() > 1 && name[0] == '#') {
          const bool hex = name[1] == 'x' || name[1] == 'X';
          char* end = nullptr;
          const unsigned long cp = std::strtoul(name.c_str() + (hex ? 2 : 1), &end, hex ? 16 : 10);
          if (*end == 0 && cp > 0 && cp < 0x110000) {
            append_utf8(cp, out);
            i = semi + 1;
            continue;
          }
        }
      }
    }
    out.push_back(s[i++]);
  }
  return out;
}

// Text of an HTML document: script / style / noscript / template content dropped, a line break
// around every block element, everything else concatenated in document order.
std::string extract_html(const std::string& src) {
  if (!valid_utf8(src)) throw Error("Unparseable", "unparseable html");
  std::string out;
  int skip_depth = 0;
  std::string skip_tag;
  size_t i = 0;
  while (i < src.size()) {
    if (src[i] != '<') {
      const size_t lt = src.find('<', i);
      const std::string text = src.substr(i, lt == std::string::npos ? std::string::npos : lt - i);
      if (skip_depth == 0) out += decode_entities(text);
      i = lt == std::string::npos ? src.size() : lt;
      continue;
    }
    if (src.compare(i, 4, "<!--") == 0) {
      const size_t end = src.find("-->", i + 4);
      i = end == std::string::npos ? src.size() : end + 3;
      continue;
    }
    const size_t gt = src.find('>', i);
    if (gt == std::string::npos) break;
    std::string tag = src.substr(i + 1, gt - i - 1);
    i = gt + 1;
    if (tag.empty() || tag[0] == '!' || tag[0] == '?') continue;
    const bool closing = tag[0] == '/';
    if (closing) tag.erase(0, 1);
    size_t e = 0;
    while (e < tag.size() && !std::isspace(static_cast<unsigned char>(tag[e])) && tag[e] != '/') ++e;
    const std::string name = lower_ascii(tag.substr(0, e));
    if (skip_depth > 0) {
      if (name == skip_tag) skip_depth += closing ? -1 : 1;
      continue;
    }
    if (!closing && kSkipTags.count(name)) {
      skip_depth = 1;
      skip_tag = name;
      continue;
    }
    if (kBlockTags.count(name)) push_break(out);
  }
  return out;
}

std::string inflate_bytes(const std::string& in) {
  z_stream zs{};
  if (inflateInit(&zs) != Z_OK) return {};
  zs.next_in = reinterpret_cast<Bytef*>(const_cast<char*>(in.data()));
  zs.avail_in = static_cast<uInt>(in.size());
  std::string out;
  char buf[1 << 14];
  int rc = Z_OK;
  while (rc == Z_OK) {
    zs.next_out = reinterpret_cast<Bytef*>(buf);
    zs.avail_out = sizeof buf;
    rc = inflate(&zs, Z_NO_FLUSH);
    if (rc != Z_OK && rc != Z_STREAM_END) {
      inflateEnd(&zs);
      return {};
    }
    out.append(buf, sizeof buf - zs.avail_out);
  }
  inflateEnd(&zs);
  return out;
}

// Text shown by the Tj / TJ / ' / " operators of one content stream.
void pdf_text_ops(const std::string& s, std::string& out) {
  std::vector<std::string> pending;   // string operands since the last operator
  size_t i = 0;
  while (i < s.size()) {
    const char c = s[i];
    if (c == '(') {
      std::string lit;
      int depth = 1;
      ++i;
      while (i < s.size() && depth > 0) {
        if (s[i] == '\\' && i + 1 < s.size()) {
          const char n = s[i + 1];
          if (n == 'n') lit.push_back('\n');
          else if (n == 'r') lit.push_back('\r');
          else if (n == 't') lit.push_back('\t');
          else if (n >= '0' && n <= '7') {
            int v = 0, k = 0;
            while (k < 3 && i + 1 < s.size() && s[i + 1] >= '0' && s[i + 1] <= '7') {
              v = v * 8 + (s[i + 1] - '0');
              ++i;
              ++k;
            }
            lit.push_back(static_cast<char>(v));
            ++i;
            continue;
          } else lit.push_back(n);
          i += 2;
        } else if (s[i] == '(') {
          ++depth;
          lit.push_back('(');
          ++i;
        } else if (s[i] == ')') {
          if (--depth > 0) lit.push_back(')');
          ++i;
        } else {
          lit.push_back(s[i++]);
        }
      }
      pending.push_back(lit);
    } else if (std::isalpha(static_cast<unsigned char>(c)) || c == '\'' || c == '"') {
      size_t e = i;
      while (e < s.size() && (std::isalpha(static_cast<unsigned char>(s[e])) || s[e] == '\'' || s[e] == '"' || s[e] == '*')) ++e;
      const std::string op = s.substr(i, e - i);
      if (op == "Tj" || op == "TJ" || op == "'" || op == "\"") {
        if (op != "Tj" && op != "TJ") push_break(out);
        for (auto& p : pending) out += p;
      } else if (op == "ET" || op == "Td" || op == "TD" || op == "T*") {
        push_break(out);
      }
      pending.clear();
      i = e;
    } else {
      ++i;
    }
  }
}

std::string extract_pdf(const std::string& bytes) {
  if (bytes.rfind("%PDF", 0) != 0) throw Error("Unparseable", "unparseable pdf");
  std::string out;
  size_t pos = 0;
  bool any_stream = false;
  while ((pos = bytes.find("stream", pos)) != std::string::npos) {
    if (pos >= 3 && bytes.compare(pos - 3, 3, "end") == 0) {
      pos += 6;
      continue;
    }
    size_t start = pos + 6;
    if (start < bytes.size() && bytes[start] == '\r') ++start;
    if (start < bytes.size() && bytes[start] == '\n') ++start;
    const size_t end = bytes.find("endstream", start);
    if (end == std::string::npos) break;
    any_stream = true;
    std::string body = bytes.substr(start, end - start);
    const size_t dict = bytes.rfind("<<", pos);
    const bool flate = dict != std::string::npos && bytes.substr(dict, pos - dict).find("FlateDecode") != std::string::npos;
    if (flate) {
      while (!body.empty() && (body.back() == '\n' || body.back() == '\r')) body.pop_back();
      body = inflate_bytes(body);
    }
    if (body.find("BT") != std::string::npos) pdf_text_ops(body, out);
    pos = end + 9;
  }
  if (!any_stream) throw Error("Unparseable", "unparseable pdf");
  return out;
}

std::string extract_latex(const std::string& src) {
  if (!valid_utf8(src)) throw Error("Unparseable", "unparseable latex");
  std::string out;
  for (size_t i = 0; i < src.size();) {
    if (src[i] == '%' && (i == 0 || src[i - 1] != '\\')) {
      while (i < src.size() && src[i] != '\n') ++i;
      continue;
    }
    out.push_back(src[i++]);
  }
  return out;
}

bool preserves_latex_math(const std::string& text) {
  if (text.find("$$") != std::string::npos) return true;
  for (const char* env : {"align", "align*", "alignat", "alignat*", "displaymath", "eqnarray", "eqnarray*", "equation",
                          "equation*", "flalign", "flalign*", "gather", "gather*", "math", "multline", "multline*"})
    if (text.find(std::string("\\begin{") + env + "}") != std::string::npos) return true;
  // an unescaped $ ... $ pair with something in between
  auto escaped = [&](size_t i) {
    size_t n = 0;
    while (i > n && text[i - 1 - n] == '\\') ++n;
    return n % 2 == 1;
  };
  for (size_t i = 0; i < text.size(); ++i)
    if (text[i] == '$' && !escaped(i))
      for (size_t j = i + 1; j < text.size(); ++j)
        if (text[j] == '$' && !escaped(j)) {
          if (j > i + 1) return true;
          break;
        }
  return false;
}

std::string format_from_path(const std::string& path) {
  const size_t dot = path.find_last_of('.');
  const std::string ext = lower_ascii(dot == std::string::npos ? path : path.substr(dot + 1));
  if (ext == "html" || ext == "htm" || ext == "xhtml") return "html";
  if (ext == "pdf") return "pdf";
  if (ext == "tex" || ext == "latex") return "latex";
  return "";
}
std::string format_from_media_type(const std::string& mt) {
  if (mt == "text/html" || mt == "application/xhtml+xml") return "html";
  if (mt == "application/pdf") return "pdf";
  if (mt == "application/x-latex" || mt == "application/x-tex" || mt == "text/x-latex" || mt == "text/x-tex") return "latex";
  return "";
}

Extracted extract(const std::string& bytes, const std::string& format) {
  if (bytes.empty()) throw Error("Empty", "empty input");
  Extracted d;
  if (format == "html") d.text = extract_html(bytes);
  else if (format == "pdf") d.text = extract_pdf(bytes);
  else if (format == "latex") d.text = extract_latex(bytes);
  else throw Error("Unsupported", "unsupported format " + format);
  d.format = format;
  d.content_hash = sha256_hex(d.text);
  d.bytes_in = bytes.size();
  return d;
}

// ---------------------------------------------------------------------------------- dedup
struct Doc {
  std::string id, text, content_hash;
};
struct DedupConfig {
  size_t shingle_size = 5, num_hashes = 128, bands = 32, rows = 4;
};
struct Cluster {
  std::string kept;
  std::vector<std::string> dropped;
};
struct DedupReport {
  std::vector<std::string> kept, dropped_exact, dropped_near;
  std::vector<Cluster> clusters;
};

// UTF-8 aware: drops zero-width code points, lowercases ASCII and Latin-1 / Greek / Cyrillic
// capitals, collapses Unicode whitespace runs to one space.
std::vector<uint32_t> decode_utf8(const std::string& s) {
  std::vector<uint32_t> out;
  for (size_t i = 0; i < s.size();) {
    const unsigned char c = s[i];
    uint32_t cp = c;
    size_t n = 1;
    if (c >= 0xF0 && i + 3 < s.size()) {
      cp = ((c & 7) << 18) | ((s[i + 1] & 0x3F) << 12) | ((s[i + 2] & 0x3F) << 6) | (s[i + 3] & 0x3F);
      n = 4;
    } else if (c >= 0xE0 && i + 2 < s.size()) {
      cp = ((c & 15) << 12) | ((s[i + 1] & 0x3F) << 6) | (s[i + 2] & 0x3F);
      n = 3;
    } else if (c >= 0xC0 && i + 1 < s.size()) {
      cp = ((c & 31) << 6) | (s[i + 1] & 0x3F);
      n = 2;
    }
    out.push_back(cp);
    i += n;
  }
  return out;
}
void encode_utf8(uint32_t cp, std::string& out) {
  if (cp < 0x80) out.push_back(static_cast<char>(cp));
  else if (cp < 0x800) {
    out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else if (cp < 0x10000) {
    out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else {
    out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  }
}
bool is_zero_width(uint32_t c) {
  return c == 0x200B || c == 0x200C || c == 0x200D || c == 0x2060 || c == 0xFEFF || c == 0x180E;
}
bool is_space_cp(uint32_t c) {
  return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) ||
         c == 0x2028 || c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
uint32_t lower_cp(uint32_t c) {
  if (c >= 'A' && c <= 'Z') return c + 32;
  if ((c >= 0xC0 && c <= 0xDE && c != 0xD7) || (c >= 0x391 && c <= 0x3A9 && c != 0x3A2) || (c >= 0x410 && c <= 0x42F)) return c + 32;
  if (c >= 0x400 && c <= 0x40F) return c + 80;
  if (c >= 0x100 && c <= 0x17F && c % 2 == 0 && !(c >= 0x138 && c <= 0x148) && c != 0x130 && c != 0x178) return c + 1;
  return c;
}
std::string lower_strip(const std::string& text) {
  std::string out;
  for (uint32_t c : decode_utf8(text))
    if (!is_zero_width(c)) encode_utf8(lower_cp(c), out);
  return out;
}
std::vector<std::string> split_ws(const std::string& text) {
  std::vector<std::string> words;
  std::string cur;
  for (uint32_t c : decode_utf8(text)) {
    if (is_space_cp(c)) {
      if (!cur.empty()) words.push_back(cur);
      cur.clear();
    } else {
      encode_utf8(c, cur);
    }
  }
  if (!cur.empty()) words.push_back(cur);
  return words;
}
std::string join(const std::vector<std::string>& w, size_t a, size_t b, const char* sep = " ") {
  std::string out;
  for (size_t i = a; i < b; ++i) out += (i > a ? sep : "") + w[i];
  return out;
}
std::string normalize(const std::string& text) {
  const auto w = split_ws(lower_strip(text));
  return join(w, 0, w.size());
}
std::vector<std::string> paragraphs(const std::string& text) {
  std::string s = lower_strip(text);
  std::string t;
  for (size_t i = 0; i < s.size(); ++i) {
    if (s[i] == '\r') {
      t.push_back('\n');
      if (i + 1 < s.size() && s[i + 1] == '\n') ++i;
    } else {
      t.push_back(s[i]);
    }
  }
  std::vector<std::string> out, cur;
  auto flush = [&] {
    if (cur.empty()) return;
    const auto w = split_ws(join(cur, 0, cur.size(), "\n"));
    cur.clear();
    if (!w.empty()) out.push_back(join(w, 0, w.size()));
  };
  size_t off = 0;
  while (off <= t.size()) {
    size_t nl = t.find('\n', off);
    if (nl == std::string::npos) nl = t.size();
    const std::string line = t.substr(off, nl - off);
    if (split_ws(line).empty()) flush();
    else cur.push_back(line);
    off = nl + 1;
  }
  flush();
  return out;
}
std::string exact_hash(const std::string& text) { return sha256_hex(normalize(text)); }
std::vector<std::string> shingles(const std::string& text, size_t n) {
  std::vector<std::string> out;
  if (n == 0) return out;
  const auto w = split_ws(normalize(text));
  if (w.size() < n) return out;
  for (size_t i = 0; i + n <= w.size(); ++i) out.push_back(join(w, i, i + n));
  return out;
}
uint64_t u64_le_sha256(const std::string& bytes) {
  Sha256 h;
  h.update(bytes.data(), bytes.size());
  const std::string hex = h.hex();
  uint64_t v = 0;
  for (int i = 7; i >= 0; --i) v = (v << 8) | std::stoul(hex.substr(2 * i, 2), nullptr, 16);
  return v;
}
std::string le64(uint64_t x) {
  std::string b(8, '\0');
  for (int i = 0; i < 8; ++i) b[i] = static_cast<char>((x >> (8 * i)) & 0xFF);
  return b;
}
std::vector<uint64_t> minhash_signature(const std::string& text, const DedupConfig& c) {
  const auto sh = shingles(text, c.shingle_size);
  const std::set<std::string> uniq(sh.begin(), sh.end());
  if (uniq.empty()) return std::vector<uint64_t>(c.num_hashes, UINT64_MAX);
  std::vector<uint64_t> sig;
  for (size_t i = 0; i < c.num_hashes; ++i) {
    uint64_t best = UINT64_MAX;
    for (const auto& s : uniq) best = std::min(best, u64_le_sha256(le64(i) + s));
    sig.push_back(best);
  }
  return sig;
}
void validate(const DedupConfig& c) {
  if (c.shingle_size == 0) throw Error("Config", "shingle_size must be > 0");
  if (c.bands == 0 || c.rows == 0) throw Error("Config", "bands and rows must be > 0");
  if (c.bands * c.rows != c.num_hashes) throw Error("Config", "num_hashes must equal bands * rows");
}
std::vector<uint64_t> lsh_band_keys(const std::vector<uint64_t>& sig, const DedupConfig& c) {
  validate(c);
  if (sig.size() != c.num_hashes) throw Error("Config", "signature length must equal num_hashes (bands * rows)");
  std::vector<uint64_t> keys;
  for (size_t b = 0; b < c.bands; ++b) {
    std::string buf;
    for (size_t r = 0; r < c.rows; ++r) buf += le64(sig[b * c.rows + r]);
    keys.push_back(u64_le_sha256(buf));
  }
  return keys;
}
bool keeper_less(const Doc& a, const Doc& b) {
  return std::tie(a.content_hash, a.id) < std::tie(b.content_hash, b.id);
}
DedupReport canonical(DedupReport r) {
  std::sort(r.kept.begin(), r.kept.end());
  std::sort(r.dropped_exact.begin(), r.dropped_exact.end());
  std::sort(r.dropped_near.begin(), r.dropped_near.end());
  for (auto& c : r.clusters) std::sort(c.dropped.begin(), c.dropped.end());
  std::sort(r.clusters.begin(), r.clusters.end(), [](auto& a, auto& b) { return a.kept < b.kept; });
  return r;
}
DedupReport dedup_exact(const std::vector<Doc>& docs, bool paragraph) {
  if (docs.empty()) throw Error("Other", "empty corpus");
  DedupReport r;
  if (!paragraph) {
    std::map<std::string, std::vector<size_t>> groups;
    for (size_t i = 0; i < docs.size(); ++i) groups[exact_hash(docs[i].text)].push_back(i);
    for (auto& kv : groups) {
      auto idx = kv.second;
      std::sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return keeper_less(docs[a], docs[b]); });
      r.kept.push_back(docs[idx[0]].id);
      for (size_t j = 1; j < idx.size(); ++j) r.dropped_exact.push_back(docs[idx[j]].id);
    }
    return canonical(r);
  }
  std::vector<size_t> order(docs.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return keeper_less(docs[a], docs[b]); });
  std::set<std::string> seen;
  for (size_t i : order) {
    std::vector<std::string> hs;
    for (auto& p : paragraphs(docs[i].text)) hs.push_back(exact_hash(p));
    bool dup = false;
    for (auto& h : hs) dup = dup || seen.count(h);
    if (dup) {
      r.dropped_exact.push_back(docs[i].id);
    } else {
      r.kept.push_back(docs[i].id);
      seen.insert(hs.begin(), hs.end());
    }
  }
  return canonical(r);
}
DedupReport dedup_near(const std::vector<Doc>& docs, const DedupConfig& c) {
  if (docs.empty()) throw Error("Other", "empty corpus");
  validate(c);
  const size_t n = docs.size();
  std::vector<size_t> parent(n);
  for (size_t i = 0; i < n; ++i) parent[i] = i;
  std::function<size_t(size_t)> find = [&](size_t x) {
    while (parent[x] != x) x = parent[x] = parent[parent[x]];
    return x;
  };
  std::vector<std::optional<std::vector<uint64_t>>> keys(n);
  for (size_t i = 0; i < n; ++i)
    if (!shingles(docs[i].text, c.shingle_size).empty()) keys[i] = lsh_band_keys(minhash_signature(docs[i].text, c), c);
  for (size_t b = 0; b < c.bands; ++b) {
    std::map<uint64_t, std::vector<size_t>> buckets;
    for (size_t i = 0; i < n; ++i)
      if (keys[i]) buckets[(*keys[i])[b]].push_back(i);
    for (auto& kv : buckets)
      for (size_t j = 1; j < kv.second.size(); ++j) parent[find(kv.second[j])] = find(kv.second[j - 1]);
  }
  std::map<size_t, std::vector<size_t>> comps;
  for (size_t i = 0; i < n; ++i) comps[find(i)].push_back(i);
  DedupReport r;
  for (auto& kv : comps) {
    auto m = kv.second;
    std::sort(m.begin(), m.end(), [&](size_t a, size_t b) { return keeper_less(docs[a], docs[b]); });
    r.kept.push_back(docs[m[0]].id);
    if (m.size() > 1) {
      Cluster cl;
      cl.kept = docs[m[0]].id;
      for (size_t j = 1; j < m.size(); ++j) cl.dropped.push_back(docs[m[j]].id);
      r.dropped_near.insert(r.dropped_near.end(), cl.dropped.begin(), cl.dropped.end());
      r.clusters.push_back(cl);
    }
  }
  return canonical(r);
}
std::vector<Doc> select_kept(const std::vector<Doc>& docs, const std::vector<std::string>& ids) {
  const std::set<std::string> want(ids.begin(), ids.end());
  std::vector<Doc> out;
  for (auto& d : docs)
    if (want.count(d.id)) out.push_back(d);
  return out;
}
DedupReport dedup_corpus(const std::vector<Doc>& docs, const DedupConfig& c) {
  if (docs.empty()) throw Error("Other", "empty corpus");
  validate(c);
  const DedupReport r_doc = dedup_exact(docs, false);
  const auto after_doc = select_kept(docs, r_doc.kept);
  const DedupReport r_para = dedup_exact(after_doc, true);
  const auto after_para = select_kept(after_doc, r_para.kept);
  DedupReport r_near = after_para.empty() ? DedupReport{} : dedup_near(after_para, c);
  DedupReport out;
  out.kept = r_near.kept;
  out.dropped_exact = r_doc.dropped_exact;
  out.dropped_exact.insert(out.dropped_exact.end(), r_para.dropped_exact.begin(), r_para.dropped_exact.end());
  out.dropped_near = r_near.dropped_near;
  out.clusters = r_near.clusters;
  return canonical(out);
}

// ------------------------------------------------------------------------------- decontam
struct EvalItem {
  std::string suite, id, text;
};
struct Hit {
  std::string suite, item_id, method;
};
struct DecontamReport {
  std::string status, method_hash;
  std::vector<std::string> against;
  std::vector<Hit> hits;
};
constexpr size_t kNgram = 8;

std::vector<std::string> ngrams(const std::string& text) {
  std::string low;
  for (uint32_t c : decode_utf8(text)) encode_utf8(lower_cp(c), low);
  const auto w = split_ws(low);
  std::vector<std::string> out;
  if (w.size() < kNgram) return out;
  for (size_t i = 0; i + kNgram <= w.size(); ++i) out.push_back(join(w, i, i + kNgram));
  return out;
}

class DecontamIndex {
 public:
  void add(const EvalItem& it) {
    for (auto& e : items_)
      if (e.suite == it.suite && e.id == it.id) throw Error("Config", "duplicate eval item " + it.suite + "/" + it.id);
    items_.push_back(it);
  }
  size_t size() const { return items_.size(); }
  std::string method_hash() const {
    need();
    auto ord = items_;
    std::sort(ord.begin(), ord.end(), [](auto& a, auto& b) { return std::tie(a.suite, a.id) < std::tie(b.suite, b.id); });
    Sha256 h;
    auto up = [&](const std::string& s) { h.update(s.data(), s.size()); };
    up("prometheus-decontam/v1\n");
    up("ngram_n=" + std::to_string(kNgram) + "\n");
    up("embed_model=\n");
    for (auto& it : ord) {
      up(it.suite);
      up(std::string(1, '\0'));
      up(it.id);
      up(std::string(1, '\0'));
      up(it.text);
      up("\n");
    }
    return h.hex();
  }
  std::vector<Hit> ngram_match(const std::string& text) const {
    need();
    const auto q = ngrams(text);
    const std::set<std::string> query(q.begin(), q.end());
    std::vector<Hit> hits;
    for (auto& it : items_)
      for (auto& g : ngrams(it.text))
        if (query.count(g)) {
          hits.push_back({it.suite, it.id, "ngram"});
          break;
        }
    return hits;
  }
  DecontamReport scan_shard(const std::vector<std::string>& texts) const {
    need();
    std::vector<Hit> hits;
    std::set<std::pair<std::string, std::string>> seen;
    for (auto& t : texts)
      for (auto& h : ngram_match(t))
        if (seen.insert({h.suite, h.item_id}).second) hits.push_back(h);
    DecontamReport r;
    r.status = hits.empty() ? "clean" : "flagged";
    std::set<std::string> suites;
    for (auto& it : items_) suites.insert(it.suite);
    r.against.assign(suites.begin(), suites.end());
    r.method_hash = method_hash();
    r.hits = hits;
    return r;
  }
  void need() const {
    if (items_.empty()) throw Error("MissingIndex", "decontamination index is empty");
  }

 private:
  std::vector<EvalItem> items_;
};

// ---------------------------------------------------------------------------- classifiers
uint64_t fnv1a64(const std::string& s) {
  uint64_t h = 0xcbf29ce484222325ull;
  for (unsigned char c : s) {
    h ^= c;
    h *= 0x100000001b3ull;
  }
  return h;
}
uint64_t mix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
float unit01(uint64_t h) { return static_cast<float>(static_cast<uint32_t>(h >> 40)) / 16777216.0f; }
std::pair<float, float> local_scores(uint64_t seed, const std::string& text) {
  const uint64_t h = fnv1a64(text);
  return {unit01(mix64(seed ^ mix64(h + 0x51))), unit01(mix64(seed ^ mix64(h + 0x53)))};
}
std::pair<float, float> scores_from_completion(const std::string& text) {
  const uint64_t h = fnv1a64(text);
  return {unit01(h), unit01(mix64(h))};
}

struct Prediction {
  std::string content_hash;
  float quality = 0, safety = 0;
};
struct HumanLabel {
  std::string content_hash;
  bool keep_quality = false, keep_safety = false;
};
struct ClfConfig {
  size_t shard_size = 32;
  float quality_threshold = 0.5f, safety_threshold = 0.5f, min_agreement = 1.0f;
};

float agreement(const std::vector<Prediction>& preds, const std::vector<HumanLabel>& labels, float qt, float st) {
  if (labels.empty()) throw Error("Empty", "no labels");
  size_t hits = 0;
  for (auto& lab : labels) {
    const Prediction* p = nullptr;
    for (auto& x : preds)
      if (x.content_hash == lab.content_hash) {
        p = &x;
        break;
      }
    if (p == nullptr) throw Error("MissingLabel", "no prediction for label " + lab.content_hash);
    if ((p->quality >= qt) == lab.keep_quality && (p->safety >= st) == lab.keep_safety) ++hits;
  }
  return static_cast<float>(hits) / static_cast<float>(labels.size());
}

class Orchestrator {
 public:
  Orchestrator(const std::string& dir, ClfConfig c, bool existing) : dir_(dir), cfg_(c) {
    if (c.shard_size == 0) throw Error("BadShardSize", "shard_size must be > 0");
    if (!existing) {
      if (::mkdir(dir.c_str(), 0777) != 0) throw Error("Other", dir + ": " + std::strerror(errno));
      return;
    }
    struct stat sb;
    if (::stat(dir.c_str(), &sb) != 0 || !S_ISDIR(sb.st_mode)) throw Error("Other", dir + ": not a directory");
    const std::string path = dir + "/events.jsonl";
    if (!file_exists(path)) return;
    const std::string text = read_file(path);
    size_t off = 0;
    while (off < text.size()) {
      size_t nl = text.find('\n', off);
      if (nl == std::string::npos) nl = text.size();
      const std::string line = text.substr(off, nl - off);
      off = nl + 1;
      if (line.empty()) continue;
      const Json v = Json::parse(line);
      if (v.at("event").as_string() == "clf.ingest") {
        const Json& d = v.at("doc");
        Extracted e;
        e.text = d.at("text").as_string();
        e.format = d.at("format").as_string();
        e.content_hash = d.at("content_hash").as_string();
        if (!d.at("source").is_null()) e.source = d.at("source").as_string();
        e.bytes_in = d.at("bytes_in").as_u64();
        docs_.push_back(e);
      } else {
        preds_.clear();
        for (const Json& p : v.at("predictions").arr())
          preds_.push_back({p.at("content_hash").as_string(), static_cast<float>(p.at("scores").at("quality").as_double()),
                            static_cast<float>(p.at("scores").at("safety").as_double())});
      }
    }
  }
  void ingest(const Extracted& doc) {
    for (auto& d : docs_)
      if (d.content_hash == doc.content_hash) throw Error("WrongState", "duplicate content_hash " + doc.content_hash);
    Json d = Json::object();
    d["text"] = doc.text;
    d["format"] = doc.format;
    d["source"] = doc.source ? Json(*doc.source) : Json();
    d["content_hash"] = doc.content_hash;
    d["bytes_in"] = doc.bytes_in;
    Json ev = Json::object();
    ev["event"] = "clf.ingest";
    ev["doc"] = d;
    journal(ev);
    docs_.push_back(doc);
  }
  std::vector<std::vector<Extracted>> shards() const {
    std::vector<std::vector<Extracted>> out;
    for (size_t i = 0; i < docs_.size(); i += cfg_.shard_size)
      out.emplace_back(docs_.begin() + i, docs_.begin() + std::min(docs_.size(), i + cfg_.shard_size));
    return out;
  }
  // scorer(texts, now) -> [(quality, safety)] per text, called once per shard
  std::vector<Prediction> run(const std::function<std::vector<std::pair<float, float>>(std::vector<std::string>, uint64_t)>& scorer,
                              uint64_t now) {
    if (docs_.empty()) throw Error("Empty", "no documents");
    std::vector<Prediction> out;
    for (auto& shard : shards()) {
      std::vector<std::string> texts;
      for (auto& d : shard) texts.push_back(d.text);
      const auto sc = scorer(texts, now);
      if (sc.size() != shard.size())
        throw Error("WrongState", "scorer returned " + std::to_string(sc.size()) + " scores for shard of " + std::to_string(shard.size()));
      for (size_t i = 0; i < shard.size(); ++i) out.push_back({shard[i].content_hash, sc[i].first, sc[i].second});
    }
    Json ps = Json::array();
    for (auto& p : out) {
      Json s = Json::object();
      s["quality"] = static_cast<double>(p.quality);
      s["safety"] = static_cast<double>(p.safety);
      Json x = Json::object();
      x["content_hash"] = p.content_hash;
      x["scores"] = s;
      ps.arr().push_back(x);
    }
    Json ev = Json::object();
    ev["event"] = "clf.score";
    ev["predictions"] = ps;
    journal(ev);
    preds_ = out;
    return out;
  }
  float agree(const std::vector<HumanLabel>& labels) const {
    return agreement(preds_, labels, cfg_.quality_threshold, cfg_.safety_threshold);
  }
  void gate(const std::vector<HumanLabel>& labels) const {
    const float got = agree(labels);
    if (got < cfg_.min_agreement)
      throw Error("GateFailed", "agreement gate failed: got " + std::to_string(got) + ", need " + std::to_string(cfg_.min_agreement));
  }
  const std::vector<Prediction>& predictions() const { return preds_; }
  size_t n_docs() const { return docs_.size(); }

 private:
  void journal(const Json& ev) const {
    FILE* f = std::fopen((dir_ + "/events.jsonl").c_str(), "ab");
    if (f == nullptr) throw Error("Other", dir_ + ": " + std::strerror(errno));
    const std::string line = ev.dump() + "\n";
    std::fwrite(line.data(), 1, line.size(), f);
    std::fclose(f);
  }
  std::string dir_;
  ClfConfig cfg_;
  std::vector<Extracted> docs_;
  std::vector<Prediction> preds_;
};

// ---------------------------------------------------------------------------------- serve
uint32_t fnv1a32(const std::string& s) {
  uint32_t h = 0x811c9dc5u;
  for (unsigned char c : s) {
    h ^= c;
    h *= 0x01000193u;
  }
  return h;
}
uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
std::string completion_text(const std::string& prompt, uint32_t max_tokens, float temperature) {
  if (max_tokens == 0) return "";
  uint32_t tbits;
  std::memcpy(&tbits, &temperature, 4);
  const uint32_t seed = fnv1a32(prompt) ^ (max_tokens * 0x9E3779B9u) ^ tbits;
  std::string out;
  for (uint32_t j = 0; j < max_tokens; ++j) {
    char buf[16];
    std::snprintf(buf, sizeof buf, "%08x", mix32(seed + (j + 1) * 0x85EBCA6Bu));
    out += (j ? " " : "") + std::string(buf);
  }
  return out;
}

class LocalEngine {
 public:
  LocalEngine(std::string model, uint32_t gpus, uint32_t max_batch, uint16_t port)
      : model_(std::move(model)), gpus_(gpus), max_batch_(max_batch), port_(port) {
    if (gpus != 1 && gpus != 2 && gpus != 4) throw Error("BadGpuCount", "gpus must be one of [1, 2, 4], got " + std::to_string(gpus));
  }
  bool is_up() const { return up_; }
  void mark_down() { up_ = false; }
  void mark_up() { up_ = true; }
  // [(prompt_index, text, finish_reason)]
  std::vector<std::tuple<size_t, std::string, std::string>> generate(const std::vector<std::string>& prompts,
                                                                     uint32_t max_tokens, float temperature) const {
    if (!up_) throw Error("EngineDown", "engine is down");
    if (prompts.empty()) throw Error("EmptyBatch", "empty batch");
    if (prompts.size() > max_batch_) throw Error("BatchTooLarge", "batch larger than " + std::to_string(max_batch_));
    std::vector<std::tuple<size_t, std::string, std::string>> out;
    for (size_t i = 0; i < prompts.size(); ++i) out.emplace_back(i, completion_text(prompts[i], max_tokens, temperature), "stop");
    return out;
  }
  std::string openai_body(const std::vector<std::tuple<size_t, std::string, std::string>>& completions) const {
    Json choices = Json::array();
    for (auto& c : completions) {
      Json msg = Json::object();
      msg["role"] = "assistant";
      msg["content"] = std::get<1>(c);
      Json ch = Json::object();
      ch["index"] = static_cast<uint64_t>(std::get<0>(c));
      ch["message"] = msg;
      ch["finish_reason"] = std::get<2>(c);
      choices.arr().push_back(ch);
    }
    Json body = Json::object();
    body["model"] = model_;
    body["choices"] = choices;
    return body.dump();
  }
  const std::string& model() const { return model_; }
  uint32_t gpus() const { return gpus_; }
  uint32_t max_batch() const { return max_batch_; }
  uint16_t port() const { return port_; }

 private:
  std::string model_;
  uint32_t gpus_, max_batch_;
  uint16_t port_;
  bool up_ = true;
};

// Generation routed through the provider failover order; the local engine is always the last
// resort (reference: serve/src/lib.rs:284-363).
constexpr const char* kLastResort = "sglang";

class Router {
 public:
  Router(std::vector<std::string> hosted, LocalEngine engine, AimdConfig aimd)
      : failover_(with_last_resort(std::move(hosted))), aimd_(aimd), engine_(std::move(engine)) {
    // the swarm starts wide open; outages shrink it
    while (aimd_.window() < aimd.max_window) {
      const uint32_t before = aimd_.window();
      aimd_.on_success(0);
      if (aimd_.window() <= before) break;
    }
  }
  void mark_down(const std::string& id) {
    bool already = false;
    for (auto& d : failover_.down()) already = already || d == id;
    const bool hosted_up = id != kLastResort && !already;
    failover_.mark_down(id);
    if (hosted_up) aimd_.on_outage();
  }
  void mark_up(const std::string& id) { failover_.mark_up(id); }
  std::vector<std::tuple<size_t, std::string, std::string>> generate(const std::vector<std::string>& prompts,
                                                                     uint32_t max_tokens, float temperature) const {
    std::string current;
    try {
      current = failover_.current();
    } catch (const Error& e) {
      if (e.kind == "NoProvider") throw Error("EngineDown", "engine is down");
      throw;
    }
    if (current != kLastResort) throw Error("Hosted", "hosted provider " + current + " has no local backend");
    return engine_.generate(prompts, max_tokens, temperature);
  }
  const Failover& failover() const { return failover_; }
  uint32_t window() const { return aimd_.window(); }
  LocalEngine& engine() { return engine_; }

 private:
  static std::vector<std::string> with_last_resort(std::vector<std::string> p) {
    if (p.empty() || p.back() != kLastResort) p.push_back(kLastResort);
    return p;
  }
  Failover failover_;
  Aimd aimd_;
  LocalEngine engine_;
};

struct Deployment {
  std::string job, endpoint, model;
  uint32_t gpus = 0;
};

// Submits the stock serving script through the Slurm client (any object with the client's
// submit / cancel methods); refuses a GPU count the client would refuse before any I/O.
class Deployer {
 public:
  Deployer(py::object client, std::string script) : client_(std::move(client)), script_(std::move(script)) {}
  Deployment submit(const LocalEngine& cfg, const std::string& run_id, const std::string& suffix,
                    const std::string& walltime) const {
    if (cfg.gpus() != 1 && cfg.gpus() != 2 && cfg.gpus() != 4)
      throw Error("BadGpuCount", "gpus must be one of [1, 2, 4], got " + std::to_string(cfg.gpus()));
    const std::string job = py::cast<std::string>(client_.attr("submit")(run_id, suffix, script_, walltime, cfg.gpus()));
    return Deployment{job, "http://127.0.0.1:" + std::to_string(cfg.port()), cfg.model(), cfg.gpus()};
  }
  void teardown(const Deployment& d) const { client_.attr("cancel")(d.job); }
  const std::string& script() const { return script_; }
  py::object client() const { return client_; }

 private:
  py::object client_;
  std::string script_;
};

}  // namespace

void bind_data_pipeline(py::module_& m) {
  auto xm = m.def_submodule("extract", "HTML / PDF / LaTeX text extraction");
  xm.attr("PARQUET_SCHEMA_VERSION") = 1;
  py::class_<Extracted>(xm, "ExtractedDocument")
      .def(py::init([](std::string text, std::string format, std::optional<std::string> source, uint64_t bytes_in) {
             Extracted d;
             d.content_hash = sha256_hex(text);
             d.text = std::move(text);
             d.format = std::move(format);
             d.source = std::move(source);
             d.bytes_in = bytes_in;
             return d;
           }),
           py::arg("text"), py::arg("format"), py::arg("source") = py::none(), py::arg("bytes_in") = 0)
      .def_readonly("text", &Extracted::text)
      .def_readonly("format", &Extracted::format)
      .def_readonly("source", &Extracted::source)
      .def_readonly("content_hash", &Extracted::content_hash)
      .def_readonly("bytes_in", &Extracted::bytes_in);
  xm.def("extract", [](py::bytes b, const std::string& fmt) { return extract(std::string(b), fmt); });
  xm.def("extract_from", [](py::bytes b, std::optional<std::string> path, std::optional<std::string> media_type) {
    std::string fmt = path ? format_from_path(*path) : "";
    if (fmt.empty() && media_type) fmt = format_from_media_type(*media_type);
    if (fmt.empty()) throw Error("Unsupported", "unsupported format");
    Extracted d = extract(std::string(b), fmt);
    d.source = path;
    return d;
  }, py::arg("data"), py::arg("path") = py::none(), py::arg("media_type") = py::none());
  xm.def("format_from_path", [](const std::string& p) -> py::object {
    const std::string f = format_from_path(p);
    return f.empty() ? py::none() : py::object(py::str(f));
  });
  xm.def("format_from_media_type", [](const std::string& p) -> py::object {
    const std::string f = format_from_media_type(p);
    return f.empty() ? py::none() : py::object(py::str(f));
  });
  xm.def("preserves_latex_math", &preserves_latex_math);

  auto dm = m.def_submodule("dedup", "exact and MinHash near-duplicate removal");
  py::class_<Doc>(dm, "Document")
      .def(py::init([](std::string id, std::string text, std::optional<std::string> hash) {
             Doc d{std::move(id), std::move(text), ""};
             d.content_hash = hash ? *hash : sha256_hex(d.text);
             return d;
           }),
           py::arg("id"), py::arg("text"), py::arg("content_hash") = py::none())
      .def_readonly("id", &Doc::id)
      .def_readonly("content_hash", &Doc::content_hash);
  py::class_<DedupConfig>(dm, "DedupConfig")
      .def(py::init([](size_t s, size_t n, size_t b, size_t r) { return DedupConfig{s, n, b, r}; }),
           py::arg("shingle_size") = 5, py::arg("num_hashes") = 128, py::arg("bands") = 32, py::arg("rows") = 4);
  py::class_<Cluster>(dm, "Cluster").def_readonly("kept", &Cluster::kept).def_readonly("dropped", &Cluster::dropped);
  py::class_<DedupReport>(dm, "DedupReport")
      .def_readonly("kept", &DedupReport::kept)
      .def_readonly("dropped_exact", &DedupReport::dropped_exact)
      .def_readonly("dropped_near", &DedupReport::dropped_near)
      .def_readonly("clusters", &DedupReport::clusters);
  dm.def("normalize", &normalize);
  dm.def("paragraphs", &paragraphs);
  dm.def("exact_hash", &exact_hash);
  dm.def("shingles", &shingles);
  dm.def("minhash_signature", &minhash_signature, py::arg("text"), py::arg("config") = DedupConfig{});
  dm.def("lsh_band_keys", &lsh_band_keys, py::arg("signature"), py::arg("config") = DedupConfig{});
  dm.def("dedup_exact", [](const std::vector<Doc>& d, const std::string& grain) {
    if (grain != "document" && grain != "paragraph") throw Error("Config", "grain must be document or paragraph");
    return dedup_exact(d, grain == "paragraph");
  }, py::arg("docs"), py::arg("grain") = "document");
  dm.def("dedup_near", &dedup_near, py::arg("docs"), py::arg("config") = DedupConfig{});
  dm.def("dedup_corpus", &dedup_corpus, py::arg("docs"), py::arg("config") = DedupConfig{});

  auto cm = m.def_submodule("decontam", "n-gram decontamination against eval suites");
  cm.attr("NGRAM_N") = kNgram;
  py::class_<EvalItem>(cm, "EvalItem")
      .def(py::init([](std::string s, std::string i, std::string t) { return EvalItem{std::move(s), std::move(i), std::move(t)}; }))
      .def_readonly("suite", &EvalItem::suite)
      .def_readonly("id", &EvalItem::id);
  py::class_<Hit>(cm, "Hit").def_readonly("suite", &Hit::suite).def_readonly("item_id", &Hit::item_id).def_readonly("method", &Hit::method);
  py::class_<DecontamReport>(cm, "Report")
      .def_readonly("status", &DecontamReport::status)
      .def_readonly("against", &DecontamReport::against)
      .def_readonly("method_hash", &DecontamReport::method_hash)
      .def_readonly("hits", &DecontamReport::hits);
  cm.def("ngrams", &ngrams);
  py::class_<DecontamIndex>(cm, "Index")
      .def(py::init<>())
      .def("add", &DecontamIndex::add)
      .def("__len__", &DecontamIndex::size)
      .def("method_hash", &DecontamIndex::method_hash)
      .def("ngram_match", &DecontamIndex::ngram_match)
      .def("embedding_match", [](const DecontamIndex& ix, const std::string&) {
        ix.need();
        throw Error("Config", "no embedder configured");
      })
      .def("scan_text", [](const DecontamIndex& ix, const std::string& t) { return ix.scan_shard({t}); })
      .def("scan_shard", &DecontamIndex::scan_shard)
      .def("planted_caught", [](const DecontamIndex& ix, const std::vector<EvalItem>& planted, const std::vector<std::string>& shard) {
        const DecontamReport r = ix.scan_shard(shard);
        for (auto& it : planted) {
          bool caught = false;
          for (auto& h : r.hits) caught = caught || (h.suite == it.suite && h.item_id == it.id);
          if (!caught) throw Error("PlantedMiss", "planted item not caught: " + it.id);
        }
      });

  auto fm = m.def_submodule("classifiers", "sharded quality / safety scoring with an agreement gate");
  fm.attr("DEFAULT_SHARD_SIZE") = 32;
  py::class_<ClfConfig>(fm, "ClassifierConfig")
      .def(py::init([](size_t s, float q, float sa, float a) { return ClfConfig{s, q, sa, a}; }), py::arg("shard_size") = 32,
           py::arg("quality_threshold") = 0.5f, py::arg("safety_threshold") = 0.5f, py::arg("min_agreement") = 1.0f);
  py::class_<Prediction>(fm, "Prediction")
      .def_readonly("content_hash", &Prediction::content_hash)
      .def_readonly("quality", &Prediction::quality)
      .def_readonly("safety", &Prediction::safety);
  py::class_<HumanLabel>(fm, "HumanLabel")
      .def(py::init([](std::string h, bool q, bool s) { return HumanLabel{std::move(h), q, s}; }));
  fm.def("local_scores", &local_scores, py::arg("seed"), py::arg("text"));
  fm.def("scores_from_completion", &scores_from_completion);
  fm.def("agreement", &agreement);
  py::class_<Orchestrator>(fm, "Orchestrator")
      .def_static("create", [](const std::string& d, ClfConfig c) { return std::make_unique<Orchestrator>(d, c, false); },
                  py::arg("dir"), py::arg("config") = ClfConfig{})
      .def_static("open", [](const std::string& d, ClfConfig c) { return std::make_unique<Orchestrator>(d, c, true); },
                  py::arg("dir"), py::arg("config") = ClfConfig{})
      .def("ingest", &Orchestrator::ingest)
      .def("shards", &Orchestrator::shards)
      .def("run", &Orchestrator::run)
      .def("run_local", [](Orchestrator& o, uint64_t seed, uint64_t now) {
        return o.run([seed](std::vector<std::string> texts, uint64_t) {
          std::vector<std::pair<float, float>> out;
          for (auto& t : texts) out.push_back(local_scores(seed, t));
          return out;
        }, now);
      })
      .def_property_readonly("predictions", &Orchestrator::predictions)
      .def("agreement", &Orchestrator::agree)
      .def("gate", &Orchestrator::gate)
      .def("__len__", &Orchestrator::n_docs);

  auto sm = m.def_submodule("serve", "batch generation engine");
  sm.attr("LAST_RESORT_ID") = "sglang";
  sm.attr("DEFAULT_MODEL") = "open-weights";
  sm.def("completion_text", &completion_text);
  py::class_<LocalEngine>(sm, "LocalEngine")
      .def(py::init<std::string, uint32_t, uint32_t, uint16_t>(), py::arg("model") = "open-weights", py::arg("gpus") = 1,
           py::arg("max_batch") = 8, py::arg("port") = 30000)
      .def("is_up", &LocalEngine::is_up)
      .def("mark_down", &LocalEngine::mark_down)
      .def("mark_up", &LocalEngine::mark_up)
      .def("generate", &LocalEngine::generate, py::arg("prompts"), py::arg("max_tokens"), py::arg("temperature") = 0.0f)
      .def("openai_body", [](const LocalEngine& e, const std::vector<std::tuple<size_t, std::string, std::string>>& c) {
        return py::bytes(e.openai_body(c));
      })
      .def_property_readonly("model", &LocalEngine::model)
      .def_property_readonly("gpus", &LocalEngine::gpus)
      .def_property_readonly("max_batch", &LocalEngine::max_batch)
      .def_property_readonly("port", &LocalEngine::port);
  py::class_<Router>(sm, "Router")
      .def(py::init<std::vector<std::string>, LocalEngine, AimdConfig>(), py::arg("hosted"), py::arg("engine"),
           py::arg("aimd") = AimdConfig{})
      .def("mark_down", &Router::mark_down)
      .def("mark_up", &Router::mark_up)
      .def("generate", &Router::generate, py::arg("prompts"), py::arg("max_tokens"), py::arg("temperature") = 0.0f)
      .def("last_resort", [](const Router&) { return std::string(kLastResort); })
      .def_property_readonly("providers", [](const Router& r) { return r.failover().providers(); })
      .def_property_readonly("down", [](const Router& r) { return r.failover().down(); })
      .def("current", [](const Router& r) { return r.failover().current(); })
      .def_property_readonly("window", &Router::window)
      .def_property_readonly("engine", &Router::engine, py::return_value_policy::reference_internal);
  py::class_<Deployment>(sm, "Deployment")
      .def_readonly("job", &Deployment::job)
      .def_readonly("endpoint", &Deployment::endpoint)
      .def_readonly("model", &Deployment::model)
      .def_readonly("gpus", &Deployment::gpus);
  py::class_<Deployer>(sm, "Deployer")
      .def(py::init<py::object, std::string>(), py::arg("client"), py::arg("script"))
      .def("submit", &Deployer::submit, py::arg("engine"), py::arg("run_id"), py::arg("suffix"), py::arg("walltime"))
      .def("teardown", &Deployer::teardown)
      .def_property_readonly("script", &Deployer::script)
      .def_property_readonly("client", &Deployer::client);
}
