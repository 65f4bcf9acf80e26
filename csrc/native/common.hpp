// Shared host-side utilities of the native systems library: SHA-256, a small
// JSON value type with canonical (sorted-key, compact) output, atomic file
// writes, and the error type every component throws.
#pragma once

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <charconv>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <variant>
#include <vector>

namespace pbn {

// Error with a stable machine-readable kind ("NotFound", "HashMismatch", ...) so the
// Python side can map kinds to exception subclasses.
struct Error : std::runtime_error {
  std::string kind;
  Error(std::string k, const std::string& msg) : std::runtime_error(msg), kind(std::move(k)) {}
};

// ---------------------------------------------------------------------------
// SHA-256 (FIPS 180-4)
// ---------------------------------------------------------------------------
class Sha256 {
 public:
  Sha256() { reset(); }
  void reset() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    std::memcpy(h_, init, sizeof(init));
    len_ = 0;
    fill_ = 0;
  }
  void update(const void* data, size_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    len_ += n;
    while (n > 0) {
      const size_t take = std::min(n, size_t(64) - fill_);
      std::memcpy(buf_ + fill_, p, take);
      fill_ += take;
      p += take;
      n -= take;
      if (fill_ == 64) {
        block(buf_);
        fill_ = 0;
      }
    }
  }
  std::string hex() {
    uint8_t pad[72] = {0x80};
    const uint64_t bits = len_ * 8;
    const size_t padlen = (fill_ < 56) ? (56 - fill_) : (120 - fill_);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
    update(pad, padlen);
    update(lenb, 8);
    static const char* digits = "0123456789abcdef";
    std::string out(64, '0');
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) {
        const uint8_t b = static_cast<uint8_t>(h_[i] >> (24 - 8 * j));
        out[i * 8 + j * 2] = digits[b >> 4];
        out[i * 8 + j * 2 + 1] = digits[b & 15];
      }
    return out;
  }

 private:
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4,
        0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe,
        0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f,
        0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7,
        0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc,
        0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b,
        0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116,
        0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
        0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
        0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) |
             (uint32_t(p[4 * i + 2]) << 8) | uint32_t(p[4 * i + 3]);
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h_[0], b = h_[1], c = h_[2], d = h_[3], e = h_[4], f = h_[5], g = h_[6],
             h = h_[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
      const uint32_t ch = (e & f) ^ (~e & g);
      const uint32_t t1 = h + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
      const uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h_[0] += a; h_[1] += b; h_[2] += c; h_[3] += d; h_[4] += e; h_[5] += f; h_[6] += g;
    h_[7] += h;
  }
  uint32_t h_[8];
  uint8_t buf_[64];
  uint64_t len_;
  size_t fill_;
};

inline std::string sha256_hex(const void* data, size_t n) {
  Sha256 s;
  s.update(data, n);
  return s.hex();
}
inline std::string sha256_hex(const std::string& s) { return sha256_hex(s.data(), s.size()); }

// ---------------------------------------------------------------------------
// JSON
// ---------------------------------------------------------------------------
struct Json;
using JsonArray = std::vector<Json>;
using JsonObject = std::map<std::string, Json>;  // sorted keys = canonical order

struct Json {
  enum Kind { Null, Bool, Int, UInt, Double, String, Array, Object } kind = Null;
  bool b = false;
  int64_t i = 0;
  uint64_t u = 0;
  double d = 0.0;
  std::string s;
  std::shared_ptr<JsonArray> a;
  std::shared_ptr<JsonObject> o;

  Json() = default;
  Json(std::nullptr_t) {}
  Json(bool v) : kind(Bool), b(v) {}
  Json(int v) : kind(Int), i(v) {}
  Json(int64_t v) : kind(Int), i(v) {}
  Json(uint32_t v) : kind(UInt), u(v) {}
  Json(uint64_t v) : kind(UInt), u(v) {}
  Json(double v) : kind(Double), d(v) {}
  Json(const char* v) : kind(String), s(v) {}
  Json(std::string v) : kind(String), s(std::move(v)) {}
  Json(JsonArray v) : kind(Array), a(std::make_shared<JsonArray>(std::move(v))) {}
  Json(JsonObject v) : kind(Object), o(std::make_shared<JsonObject>(std::move(v))) {}

  static Json object() { return Json(JsonObject{}); }
  static Json array() { return Json(JsonArray{}); }

  bool is_null() const { return kind == Null; }
  bool is_object() const { return kind == Object; }
  bool is_array() const { return kind == Array; }
  bool is_string() const { return kind == String; }
  bool is_bool() const { return kind == Bool; }
  bool is_number() const { return kind == Int || kind == UInt || kind == Double; }
  bool is_integer() const {
    return kind == Int || kind == UInt || (kind == Double && std::floor(d) == d && std::isfinite(d));
  }
  uint64_t as_u64() const {
    if (kind == UInt) return u;
    if (kind == Int && i >= 0) return static_cast<uint64_t>(i);
    if (kind == Double && d >= 0 && std::floor(d) == d) return static_cast<uint64_t>(d);
    throw Error("Schema", "expected an unsigned integer");
  }
  int64_t as_i64() const {
    if (kind == Int) return i;
    if (kind == UInt) return static_cast<int64_t>(u);
    if (kind == Double && std::floor(d) == d) return static_cast<int64_t>(d);
    throw Error("Schema", "expected an integer");
  }
  double as_double() const {
    if (kind == Double) return d;
    if (kind == Int) return static_cast<double>(i);
    if (kind == UInt) return static_cast<double>(u);
    throw Error("Schema", "expected a number");
  }
  const std::string& as_string() const {
    if (kind != String) throw Error("Schema", "expected a string");
    return s;
  }
  bool as_bool() const {
    if (kind != Bool) throw Error("Schema", "expected a boolean");
    return b;
  }
  const JsonArray& arr() const {
    if (kind != Array) throw Error("Schema", "expected an array");
    return *a;
  }
  JsonArray& arr() {
    if (kind != Array) throw Error("Schema", "expected an array");
    return *a;
  }
  const JsonObject& obj() const {
    if (kind != Object) throw Error("Schema", "expected an object");
    return *o;
  }
  JsonObject& obj() {
    if (kind != Object) throw Error("Schema", "expected an object");
    return *o;
  }
  bool has(const std::string& k) const { return kind == Object && o->count(k) > 0; }
  const Json& at(const std::string& k) const {
    auto it = obj().find(k);
    if (it == o->end()) throw Error("Schema", "missing field " + k);
    return it->second;
  }
  const Json* find(const std::string& k) const {
    if (kind != Object) return nullptr;
    auto it = o->find(k);
    return it == o->end() ? nullptr : &it->second;
  }
  Json& operator[](const std::string& k) { return obj()[k]; }
  void push(Json v) { arr().push_back(std::move(v)); }

  bool operator==(const Json& r) const {
    if (is_number() && r.is_number()) {
      if (kind != Double && r.kind != Double) {
        if ((kind == Int && i < 0) || (r.kind == Int && r.i < 0))
          return kind == Int && r.kind == Int ? i == r.i : false;
        return as_u64() == r.as_u64();
      }
      return as_double() == r.as_double();
    }
    if (kind != r.kind) return false;
    switch (kind) {
      case Null: return true;
      case Bool: return b == r.b;
      case String: return s == r.s;
      case Array: return *a == *r.a;
      case Object: return *o == *r.o;
      default: return false;
    }
  }
  bool operator!=(const Json& r) const { return !(*this == r); }

  // Compact text, keys in sorted order (what serde_json emits for a Value/Map).
  std::string dump() const {
    std::string out;
    write(out);
    return out;
  }
  // Two-space indented text (serde_json::to_string_pretty layout), keys sorted.
  std::string dump_pretty() const {
    std::string out;
    write_pretty(out, 0);
    return out;
  }
  void write_pretty(std::string& out, int depth) const {
    const std::string pad(static_cast<size_t>(depth + 1) * 2, ' ');
    const std::string close(static_cast<size_t>(depth) * 2, ' ');
    if (kind == Array) {
      if (a->empty()) { out += "[]"; return; }
      out += "[\n";
      for (size_t i = 0; i < a->size(); ++i) {
        out += pad;
        (*a)[i].write_pretty(out, depth + 1);
        out += i + 1 < a->size() ? ",\n" : "\n";
      }
      out += close + "]";
    } else if (kind == Object) {
      if (o->empty()) { out += "{}"; return; }
      out += "{\n";
      size_t i = 0;
      for (const auto& kv : *o) {
        out += pad;
        write_string(out, kv.first);
        out += ": ";
        kv.second.write_pretty(out, depth + 1);
        out += ++i < o->size() ? ",\n" : "\n";
      }
      out += close + "}";
    } else {
      write(out);
    }
  }
  void write(std::string& out) const {
    switch (kind) {
      case Null: out += "null"; break;
      case Bool: out += b ? "true" : "false"; break;
      case Int: out += std::to_string(i); break;
      case UInt: out += std::to_string(u); break;
      case Double: write_double(out, d); break;
      case String: write_string(out, s); break;
      case Array: {
        out += '[';
        bool first = true;
        for (const auto& v : *a) {
          if (!first) out += ',';
          first = false;
          v.write(out);
        }
        out += ']';
        break;
      }
      case Object: {
        out += '{';
        bool first = true;
        for (const auto& kv : *o) {
          if (!first) out += ',';
          first = false;
          write_string(out, kv.first);
          out += ':';
          kv.second.write(out);
        }
        out += '}';
        break;
      }
    }
  }
  static void write_double(std::string& out, double v) {
    if (!std::isfinite(v)) {
      out += "null";
      return;
    }
    char buf[64];
    auto res = std::to_chars(buf, buf + sizeof(buf), v);
    std::string t(buf, res.ptr);
    // shortest round-trip digits; make integral values read "1.0" and exponents "1e-7"
    const size_t e = t.find('e');
    if (e != std::string::npos) {
      std::string mant = t.substr(0, e), ex = t.substr(e + 1);
      bool neg = !ex.empty() && ex[0] == '-';
      if (!ex.empty() && (ex[0] == '-' || ex[0] == '+')) ex = ex.substr(1);
      while (ex.size() > 1 && ex[0] == '0') ex = ex.substr(1);
      t = mant + "e" + (neg ? "-" : "") + ex;
    } else if (t.find('.') == std::string::npos) {
      t += ".0";
    }
    out += t;
  }
  static void write_string(std::string& out, const std::string& v) {
    out += '"';
    for (unsigned char c : v) {
      switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\r': out += "\\r"; break;
        case '\t': out += "\\t"; break;
        case '\b': out += "\\b"; break;
        case '\f': out += "\\f"; break;
        default:
          if (c < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof(buf), "\\u%04x", c);
            out += buf;
          } else {
            out += static_cast<char>(c);
          }
      }
    }
    out += '"';
  }

  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json v = parse_value(text, pos, 0);
    skip_ws(text, pos);
    if (pos != text.size()) throw Error("Schema", "trailing characters after JSON value");
    return v;
  }

 private:
  static void skip_ws(const std::string& t, size_t& p) {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
  }
  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) {
      out += static_cast<char>(cp);
    } else if (cp < 0x800) {
      out += static_cast<char>(0xC0 | (cp >> 6));
      out += static_cast<char>(0x80 | (cp & 0x3F));
    } else if (cp < 0x10000) {
      out += static_cast<char>(0xE0 | (cp >> 12));
      out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
      out += static_cast<char>(0x80 | (cp & 0x3F));
    } else {
      out += static_cast<char>(0xF0 | (cp >> 18));
      out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
      out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
      out += static_cast<char>(0x80 | (cp & 0x3F));
    }
  }
  static uint32_t hex4(const std::string& t, size_t& p) {
    if (p + 4 > t.size()) throw Error("Schema", "bad \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      const char c = t[p++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else throw Error("Schema", "bad \\u escape");
    }
    return v;
  }
  static std::string parse_string(const std::string& t, size_t& p) {
    ++p;  // opening quote
    std::string out;
    while (true) {
      if (p >= t.size()) throw Error("Schema", "unterminated string");
      const char c = t[p++];
      if (c == '"') break;
      if (c == '\\') {
        if (p >= t.size()) throw Error("Schema", "bad escape");
        const char e = t[p++];
        switch (e) {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            uint32_t cp = hex4(t, p);
            if (cp >= 0xD800 && cp < 0xDC00 && p + 1 < t.size() && t[p] == '\\' &&
                t[p + 1] == 'u') {
              p += 2;
              const uint32_t lo = hex4(t, p);
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            append_utf8(out, cp);
            break;
          }
          default: throw Error("Schema", "bad escape");
        }
      } else {
        out += c;
      }
    }
    return out;
  }
  static Json parse_value(const std::string& t, size_t& p, int depth) {
    if (depth > 200) throw Error("Schema", "JSON nested too deeply");
    skip_ws(t, p);
    if (p >= t.size()) throw Error("Schema", "unexpected end of JSON");
    const char c = t[p];
    if (c == '{') {
      ++p;
      JsonObject o;
      skip_ws(t, p);
      if (p < t.size() && t[p] == '}') {
        ++p;
        return Json(std::move(o));
      }
      while (true) {
        skip_ws(t, p);
        if (p >= t.size() || t[p] != '"') throw Error("Schema", "expected object key");
        std::string k = parse_string(t, p);
        skip_ws(t, p);
        if (p >= t.size() || t[p] != ':') throw Error("Schema", "expected ':'");
        ++p;
        o[k] = parse_value(t, p, depth + 1);
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == '}') { ++p; break; }
        throw Error("Schema", "expected ',' or '}'");
      }
      return Json(std::move(o));
    }
    if (c == '[') {
      ++p;
      JsonArray a;
      skip_ws(t, p);
      if (p < t.size() && t[p] == ']') {
        ++p;
        return Json(std::move(a));
      }
      while (true) {
        a.push_back(parse_value(t, p, depth + 1));
        skip_ws(t, p);
        if (p < t.size() && t[p] == ',') { ++p; continue; }
        if (p < t.size() && t[p] == ']') { ++p; break; }
        throw Error("Schema", "expected ',' or ']'");
      }
      return Json(std::move(a));
    }
    if (c == '"') return Json(parse_string(t, p));
    if (t.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (t.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (t.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    // number
    const size_t start = p;
    if (p < t.size() && (t[p] == '-' || t[p] == '+')) ++p;
    bool is_float = false;
    while (p < t.size() && (std::isdigit(static_cast<unsigned char>(t[p])) || t[p] == '.' ||
                            t[p] == 'e' || t[p] == 'E' || t[p] == '-' || t[p] == '+')) {
      if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_float = true;
      ++p;
    }
    if (p == start) throw Error("Schema", "unexpected character in JSON");
    const std::string num = t.substr(start, p - start);
    if (!is_float) {
      if (num[0] == '-') {
        int64_t v = 0;
        auto r = std::from_chars(num.data(), num.data() + num.size(), v);
        if (r.ec == std::errc() && r.ptr == num.data() + num.size()) return Json(v);
      } else {
        uint64_t v = 0;
        auto r = std::from_chars(num.data(), num.data() + num.size(), v);
        if (r.ec == std::errc() && r.ptr == num.data() + num.size()) return Json(v);
      }
    }
    double dv = 0;
    auto r = std::from_chars(num.data(), num.data() + num.size(), dv);
    if (r.ec != std::errc() || r.ptr != num.data() + num.size())
      throw Error("Schema", "bad number " + num);
    return Json(dv);
  }
};

// ---------------------------------------------------------------------------
// files
// ---------------------------------------------------------------------------
inline bool file_exists(const std::string& path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}
inline bool dir_exists(const std::string& path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
inline void make_dirs(const std::string& path) {
  std::string cur;
  for (size_t i = 0; i <= path.size(); ++i) {
    if (i == path.size() || path[i] == '/') {
      if (!cur.empty() && !dir_exists(cur)) {
        if (::mkdir(cur.c_str(), 0777) != 0 && errno != EEXIST)
          throw Error("Message", "mkdir " + cur + ": " + std::strerror(errno));
      }
    }
    if (i < path.size()) cur += path[i];
  }
}
inline std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw Error("NotFound", path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}
inline void fsync_dir(const std::string& dir) {
  const int fd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
  if (fd >= 0) {
    ::fsync(fd);
    ::close(fd);
  }
}
// Write to a temp name in the same directory, fsync, rename over the target.
inline void atomic_write(const std::string& path, const void* data, size_t n) {
  static uint64_t counter = 0;
  const std::string tmp =
      path + ".tmp." + std::to_string(::getpid()) + "." + std::to_string(++counter);
  const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) throw Error("Message", "open " + tmp + ": " + std::strerror(errno));
  const uint8_t* p = static_cast<const uint8_t*>(data);
  size_t left = n;
  while (left > 0) {
    const ssize_t w = ::write(fd, p, left);
    if (w < 0) {
      if (errno == EINTR) continue;
      const std::string msg = std::strerror(errno);
      ::close(fd);
      ::unlink(tmp.c_str());
      throw Error("Message", "write " + tmp + ": " + msg);
    }
    p += w;
    left -= static_cast<size_t>(w);
  }
  ::fsync(fd);
  ::close(fd);
  if (::rename(tmp.c_str(), path.c_str()) != 0) {
    const std::string msg = std::strerror(errno);
    ::unlink(tmp.c_str());
    throw Error("Message", "rename " + tmp + ": " + msg);
  }
  const size_t slash = path.find_last_of('/');
  fsync_dir(slash == std::string::npos ? "." : path.substr(0, slash));
}
inline void atomic_write(const std::string& path, const std::string& data) {
  atomic_write(path, data.data(), data.size());
}

// Deterministic generator used wherever the reference seeds SplitMix64.
struct SplitMix64 {
  uint64_t state;
  explicit SplitMix64(uint64_t seed) : state(seed) {}
  uint64_t next() {
    state += 0x9E3779B97F4A7C15ull;
    uint64_t z = state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
};

}  // namespace pbn
