// Versioned JSON-schema validation at the module boundaries.
//
// A payload names its schema (`schema_id` = "prometheus.<short>", `schema_version` = n); the
// schema is `<root>/v<n>/<short>.schema.json`, shared definitions live in
// `<root>/v<n>/_defs.schema.json`. The validator implements the draft 2020-12 keywords the
// contract schemas use: type, const, enum, properties, required, additionalProperties,
// minProperties, items, minItems, minLength, minimum, maximum, pattern, format (date-time, date)
// and $ref into the document itself or into the shared definitions.
// (reference: crates/contracts/src/lib.rs:9-185 validate / migrate / current_version)
#include <dirent.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <regex>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace {

struct Ctx {
  const Json* doc;    // the schema document being applied
  const Json* defs;   // the shared definitions document
};

std::string type_of(const Json& v) {
  if (v.is_null()) return "null";
  if (v.is_bool()) return "boolean";
  if (v.is_string()) return "string";
  if (v.is_array()) return "array";
  if (v.is_object()) return "object";
  return v.is_integer() ? "integer" : "number";
}
bool type_matches(const std::string& want, const Json& v) {
  const std::string have = type_of(v);
  return want == have || (want == "number" && have == "integer");
}
size_t utf8_len(const std::string& s) {
  size_t n = 0;
  for (unsigned char c : s) n += (c & 0xC0) != 0x80;
  return n;
}
bool all_digits(const std::string& s, size_t a, size_t n) {
  if (a + n > s.size()) return false;
  for (size_t i = a; i < a + n; ++i)
    if (s[i] < '0' || s[i] > '9') return false;
  return true;
}
bool valid_date(const std::string& s, size_t off = 0) {
  if (!all_digits(s, off, 4) || s.size() < off + 10 || s[off + 4] != '-' || !all_digits(s, off + 5, 2) ||
      s[off + 7] != '-' || !all_digits(s, off + 8, 2))
    return false;
  const int y = std::stoi(s.substr(off, 4)), m = std::stoi(s.substr(off + 5, 2)), d = std::stoi(s.substr(off + 8, 2));
  static const int days[] = {31, 28, 31, 30, 31, 30, 31, 31, 30, 31, 30, 31};
  if (m < 1 || m > 12 || d < 1) return false;
  const bool leap = (y % 4 == 0 && y % 100 != 0) || y % 400 == 0;
  return d <= days[m - 1] + ((m == 2 && leap) ? 1 : 0);
}
bool valid_datetime(const std::string& s) {   // RFC 3339
  if (s.size() < 20 || !valid_date(s) || (s[10] != 'T' && s[10] != 't')) return false;
  if (!all_digits(s, 11, 2) || s[13] != ':' || !all_digits(s, 14, 2) || s[16] != ':' || !all_digits(s, 17, 2)) return false;
  if (std::stoi(s.substr(11, 2)) > 23 || std::stoi(s.substr(14, 2)) > 59 || std::stoi(s.substr(17, 2)) > 60) return false;
  size_t i = 19;
  if (i < s.size() && s[i] == '.') {
    size_t j = i + 1;
    while (j < s.size() && s[j] >= '0' && s[j] <= '9') ++j;
    if (j == i + 1) return false;
    i = j;
  }
  if (i >= s.size()) return false;
  if (s[i] == 'Z' || s[i] == 'z') return i + 1 == s.size();
  if (s[i] != '+' && s[i] != '-') return false;
  return s.size() == i + 6 && all_digits(s, i + 1, 2) && s[i + 3] == ':' && all_digits(s, i + 4, 2) &&
         std::stoi(s.substr(i + 1, 2)) <= 23 && std::stoi(s.substr(i + 4, 2)) <= 59;
}

const Json& resolve(const std::string& ref, const Ctx& c, const Json*& doc_out) {
  const size_t hash = ref.find('#');
  const std::string file = hash == std::string::npos ? ref : ref.substr(0, hash);
  const std::string frag = hash == std::string::npos ? "" : ref.substr(hash + 1);
  const Json* cur = file.empty() ? c.doc : c.defs;
  if (!file.empty() && file.find("_defs.schema.json") == std::string::npos)
    throw Error("Validation", "validation error: unresolved $ref " + ref);
  doc_out = cur;
  size_t off = 0;
  while (off < frag.size()) {
    size_t slash = frag.find('/', off);
    if (slash == std::string::npos) slash = frag.size();
    const std::string part = frag.substr(off, slash - off);
    off = slash + 1;
    if (part.empty()) continue;
    const Json* next = cur->find(part);
    if (next == nullptr) throw Error("Validation", "validation error: unresolved $ref " + ref);
    cur = next;
  }
  return *cur;
}

void check(const Json& schema, const Json& v, const Ctx& c, const std::string& path, std::vector<std::string>& errs,
           int depth = 0) {
  if (depth > 64) throw Error("Validation", "validation error: schema nested too deeply");
  if (schema.is_bool()) {
    if (!schema.as_bool()) errs.push_back(path + ": not allowed");
    return;
  }
  if (!schema.is_object()) return;
  if (const Json* ref = schema.find("$ref")) {
    const Json* doc = nullptr;
    const Json& target = resolve(ref->as_string(), c, doc);
    check(target, v, Ctx{doc, c.defs}, path, errs, depth + 1);
  }
  if (const Json* t = schema.find("type")) {
    bool ok = false;
    if (t->is_string()) ok = type_matches(t->as_string(), v);
    else
      for (const Json& x : t->arr()) ok = ok || type_matches(x.as_string(), v);
    if (!ok) {
      errs.push_back(path + ": " + v.dump() + " is not of type " + t->dump());
      return;   // the remaining keywords assume the type
    }
  }
  if (const Json* k = schema.find("const"))
    if (!(*k == v)) errs.push_back(path + ": " + k->dump() + " was expected");
  if (const Json* e = schema.find("enum")) {
    bool ok = false;
    for (const Json& x : e->arr()) ok = ok || x == v;
    if (!ok) errs.push_back(path + ": " + v.dump() + " is not one of " + e->dump());
  }
  if (v.is_number()) {
    if (const Json* m = schema.find("minimum"))
      if (v.as_double() < m->as_double()) errs.push_back(path + ": " + v.dump() + " is less than the minimum of " + m->dump());
    if (const Json* m = schema.find("maximum"))
      if (v.as_double() > m->as_double()) errs.push_back(path + ": " + v.dump() + " is greater than the maximum of " + m->dump());
  }
  if (v.is_string()) {
    const std::string& s = v.as_string();
    if (const Json* m = schema.find("minLength"))
      if (utf8_len(s) < m->as_u64()) errs.push_back(path + ": " + v.dump() + " is too short");
    if (const Json* p = schema.find("pattern")) {
      const std::regex re(p->as_string(), std::regex::ECMAScript);
      if (!std::regex_search(s, re)) errs.push_back(path + ": " + v.dump() + " does not match " + p->dump());
    }
    if (const Json* f = schema.find("format")) {
      const std::string& fmt = f->as_string();
      if ((fmt == "date-time" && !valid_datetime(s)) || (fmt == "date" && !(s.size() == 10 && valid_date(s))))
        errs.push_back(path + ": " + v.dump() + " is not a " + fmt);
    }
  }
  if (v.is_array()) {
    if (const Json* m = schema.find("minItems"))
      if (v.arr().size() < m->as_u64()) errs.push_back(path + ": array is too short");
    if (const Json* items = schema.find("items"))
      for (size_t i = 0; i < v.arr().size(); ++i) check(*items, v.arr()[i], c, path + "/" + std::to_string(i), errs, depth + 1);
  }
  if (v.is_object()) {
    const Json* props = schema.find("properties");
    if (const Json* req = schema.find("required"))
      for (const Json& r : req->arr())
        if (!v.has(r.as_string())) errs.push_back(path + ": " + r.dump() + " is a required property");
    if (const Json* m = schema.find("minProperties"))
      if (v.obj().size() < m->as_u64()) errs.push_back(path + ": object does not have enough properties");
    const Json* extra = schema.find("additionalProperties");
    for (const auto& kv : v.obj()) {
      const Json* sub = props != nullptr ? props->find(kv.first) : nullptr;
      if (sub != nullptr) {
        check(*sub, kv.second, c, path + "/" + kv.first, errs, depth + 1);
      } else if (extra != nullptr) {
        if (extra->is_bool()) {
          if (!extra->as_bool()) errs.push_back(path + ": additional property '" + kv.first + "' is not allowed");
        } else {
          check(*extra, kv.second, c, path + "/" + kv.first, errs, depth + 1);
        }
      }
    }
  }
}

std::string short_name(const std::string& id, uint64_t version) {
  const std::string prefix = "prometheus.";
  if (id.rfind(prefix, 0) != 0 || id.size() == prefix.size() || id.find('/') != std::string::npos)
    throw Error("UnknownSchema", "unknown schema " + id + " v" + std::to_string(version));
  return id.substr(prefix.size());
}
Json read_json(const std::string& path) {
  try {
    return Json::parse(read_file(path));
  } catch (const Error& e) {
    throw Error("Validation", std::string("validation error: ") + e.what());
  }
}

std::pair<std::string, uint64_t> payload_ref(const Json& payload) {
  if (!payload.is_object()) throw Error("Validation", "validation error: payload must be an object");
  const Json* id = payload.find("schema_id");
  if (id == nullptr) throw Error("Validation", "validation error: missing schema_id");
  if (!id->is_string()) throw Error("Validation", "validation error: schema_id must be a string");
  const Json* ver = payload.find("schema_version");
  if (ver == nullptr) throw Error("Validation", "validation error: missing schema_version");
  if (!ver->is_number() || !ver->is_integer()) throw Error("Validation", "validation error: schema_version must be an integer");
  if (ver->as_i64() < 0 || ver->as_i64() > 4294967295ll) throw Error("Validation", "validation error: schema_version must be a u32");
  return {id->as_string(), ver->as_u64()};
}

void validate(const std::string& payload_json, const std::string& root) {
  Json payload;
  try {
    payload = Json::parse(payload_json);
  } catch (const Error& e) {
    throw Error("Validation", std::string("validation error: ") + e.what());
  }
  const auto [id, version] = payload_ref(payload);
  const std::string dir = root + "/v" + std::to_string(version);
  const std::string path = dir + "/" + short_name(id, version) + ".schema.json";
  if (!file_exists(path)) throw Error("UnknownSchema", "unknown schema " + id + " v" + std::to_string(version));
  const Json schema = read_json(path), defs = read_json(dir + "/_defs.schema.json");
  std::vector<std::string> errs;
  check(schema, payload, Ctx{&schema, &defs}, "$", errs);
  if (!errs.empty()) {
    std::string msg = "validation error: ";
    for (size_t i = 0; i < errs.size(); ++i) msg += (i ? "; " : "") + errs[i];
    throw Error("Validation", msg);
  }
}

std::string migrate(const std::string& payload_json, uint32_t to_version) {
  const Json payload = Json::parse(payload_json);
  const Json* ver = payload.is_object() ? payload.find("schema_version") : nullptr;
  if (ver == nullptr || !ver->is_number() || !ver->is_integer() || ver->as_i64() < 0)
    throw Error("Validation", "validation error: schema_version must be an integer");
  if (ver->as_u64() == to_version) return payload.dump();
  throw Error("Migration", "no migration from v" + std::to_string(ver->as_u64()) + " to v" + std::to_string(to_version));
}

uint32_t current_version(const std::string& id, const std::string& root) {
  const std::string shortn = short_name(id, 0);
  DIR* d = ::opendir(root.c_str());
  if (d == nullptr) throw Error("Validation", "validation error: " + root + ": " + std::strerror(errno));
  int64_t best = -1;
  while (dirent* e = ::readdir(d)) {
    const std::string name = e->d_name;
    if (name.size() < 2 || name[0] != 'v' || name.find_first_not_of("0123456789", 1) != std::string::npos) continue;
    if (file_exists(root + "/" + name + "/" + shortn + ".schema.json")) best = std::max<int64_t>(best, std::stoll(name.substr(1)));
  }
  ::closedir(d);
  if (best < 0) throw Error("UnknownSchema", "unknown schema " + id + " v0");
  return static_cast<uint32_t>(best);
}

}  // namespace

void bind_contracts(py::module_& m) {
  auto cm = m.def_submodule("contracts", "versioned JSON-schema validation");
  cm.def("validate", &validate, py::arg("payload_json"), py::arg("schemas_root"));
  cm.def("migrate", &migrate, py::arg("payload_json"), py::arg("to_version"));
  cm.def("current_version", &current_version, py::arg("schema_id"), py::arg("schemas_root"));
  cm.def("valid_datetime", &valid_datetime);
}
