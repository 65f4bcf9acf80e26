// Replicated content-addressed blob store with named pins and garbage collection.
//
// Contract of the reference's harness/cas crate (harness/cas/src/lib.rs:20-25, 88-300): a blob
// is named by its sha256 and written to every backend directory; a put needs at least
// `min_replicas` successful copies; a get returns the first replica that re-hashes to its
// name; pins are named, logged to <dir>/log and replayed on open; gc removes every unpinned
// blob from every backend.
#pragma once

#include <dirent.h>

#include <map>
#include <set>

#include "eventlog.hpp"

namespace pbn {

constexpr size_t kMinReplicas = 2;
const char* const kCasTimestamp = "1970-01-01T00:00:00Z";

inline void list_files(const std::string& dir, std::vector<std::string>& out) {
  DIR* d = ::opendir(dir.c_str());
  if (d == nullptr) return;
  while (dirent* e = ::readdir(d)) {
    const std::string name = e->d_name;
    if (name == "." || name == "..") continue;
    const std::string path = dir + "/" + name;
    if (dir_exists(path)) list_files(path, out);
    else if (file_exists(path)) out.push_back(path);
  }
  ::closedir(d);
}

struct GcReport {
  uint64_t blobs_removed = 0, bytes_freed = 0;
};

class CasStore {
 public:
  static std::unique_ptr<CasStore> create(const std::string& dir, std::vector<std::string> backends,
                                          size_t min_replicas) {
    if (backends.size() < min_replicas)
      throw Error("TooFewBackends", "need at least " + std::to_string(kMinReplicas) +
                                        " backends, have " + std::to_string(backends.size()));
    if (file_exists(dir) || dir_exists(dir)) throw Error("Other", "already exists: " + dir);
    if (::mkdir(dir.c_str(), 0777) != 0) throw Error("Io", dir + ": " + std::strerror(errno));
    auto s = std::unique_ptr<CasStore>(new CasStore(dir, std::move(backends), min_replicas));
    s->log_ = EventLog::create(dir + "/log");
    return s;
  }
  static std::unique_ptr<CasStore> open(const std::string& dir, std::vector<std::string> backends,
                                        size_t min_replicas) {
    if (backends.size() < min_replicas)
      throw Error("TooFewBackends", "need at least " + std::to_string(kMinReplicas) +
                                        " backends, have " + std::to_string(backends.size()));
    auto s = std::unique_ptr<CasStore>(new CasStore(dir, std::move(backends), min_replicas));
    s->log_ = EventLog::open(dir + "/log");
    for (const LogEvent& e : s->log_->events()) {
      const Json* name = e.payload.find("name");
      if (e.event_type == "cas.pin") {
        const Json* dg = e.payload.find("digest");
        if (name && name->is_string() && dg && dg->is_string()) s->pins_[name->as_string()] = dg->as_string();
      } else if (e.event_type == "cas.unpin") {
        if (name && name->is_string()) s->pins_.erase(name->as_string());
      }
    }
    return s;
  }

  std::string put(const std::string& bytes) {
    const std::string hex = sha256_hex(bytes);
    size_t wrote = 0;
    for (const std::string& b : backends_) {
      const std::string path = b + "/" + hex;
      const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
      if (fd < 0) continue;
      size_t done = 0;
      bool ok = true;
      while (done < bytes.size()) {
        const ssize_t w = ::write(fd, bytes.data() + done, bytes.size() - done);
        if (w < 0) {
          if (errno == EINTR) continue;
          ok = false;
          break;
        }
        done += static_cast<size_t>(w);
      }
      if (ok && ::fsync(fd) != 0) ok = false;
      ::close(fd);
      if (ok) {
        fsync_dir(b);
        ++wrote;
      }
    }
    if (wrote < min_replicas_)
      throw Error("UnderReplicated", "put wrote " + std::to_string(wrote) + " replicas, need " +
                                         std::to_string(min_replicas_));
    Json p = Json::object();
    p["digest"] = hex;
    event("cas.put", p);
    return hex;
  }

  std::string get(const std::string& digest) const {
    std::optional<std::string> bad;
    for (const std::string& b : backends_) {
      const std::string path = b + "/" + digest;
      if (!file_exists(path)) continue;
      std::string bytes;
      try {
        bytes = read_file(path);
      } catch (const Error&) {
        continue;
      }
      const std::string got = sha256_hex(bytes);
      if (got == digest) return bytes;
      bad = got;
    }
    if (bad) throw Error("DigestMismatch", "digest mismatch: expected " + digest + " got " + *bad);
    throw Error("NotFound", "not found: " + digest);
  }

  size_t replica_count(const std::string& digest) const {
    size_t n = 0;
    for (const std::string& b : backends_) n += file_exists(b + "/" + digest) ? 1 : 0;
    return n;
  }

  void pin(const std::string& digest, const std::string& name) {
    if (replica_count(digest) == 0) throw Error("NotFound", "not found: " + digest);
    if (pins_.count(name)) throw Error("DuplicatePin", "duplicate pin " + name);
    Json p = Json::object();
    p["name"] = name;
    p["digest"] = digest;
    event("cas.pin", p);
    pins_[name] = digest;
  }
  void unpin(const std::string& name) {
    if (!pins_.count(name)) throw Error("NotFound", "not found: " + name);
    Json p = Json::object();
    p["name"] = name;
    event("cas.unpin", p);
    pins_.erase(name);
  }

  GcReport gc() {
    std::set<std::string> pinned;
    for (auto& kv : pins_) pinned.insert(kv.second);
    std::map<std::string, uint64_t> sizes;
    std::vector<std::string> doomed;
    for (const std::string& b : backends_) {
      std::vector<std::string> files;
      list_files(b, files);
      for (const std::string& path : files) {
        const std::string digest = path.substr(path.find_last_of('/') + 1);
        if (pinned.count(digest)) continue;
        struct stat st;
        sizes[digest] += ::stat(path.c_str(), &st) == 0 ? static_cast<uint64_t>(st.st_size) : 0;
        doomed.push_back(path);
      }
    }
    for (const std::string& path : doomed)
      if (::unlink(path.c_str()) != 0) throw Error("Io", path + ": " + std::strerror(errno));
    GcReport r;
    r.blobs_removed = sizes.size();
    for (auto& kv : sizes) r.bytes_freed += kv.second;
    Json p = Json::object();
    p["blobs_removed"] = r.blobs_removed;
    p["bytes_freed"] = r.bytes_freed;
    event("cas.gc", p);
    return r;
  }

  const std::map<std::string, std::string>& pins() const { return pins_; }
  const EventLog& log() const { return *log_; }
  const std::vector<std::string>& backends() const { return backends_; }

 private:
  CasStore(std::string dir, std::vector<std::string> backends, size_t min_replicas)
      : dir_(std::move(dir)), backends_(std::move(backends)), min_replicas_(min_replicas) {}
  void event(const char* type, const Json& payload) {
    LogAppend a;
    a.event_type = type;
    a.payload = payload;
    a.timestamp = kCasTimestamp;
    log_->append(a);
  }
  std::string dir_;
  std::vector<std::string> backends_;
  size_t min_replicas_;
  std::unique_ptr<EventLog> log_;
  std::map<std::string, std::string> pins_;
};


}  // namespace pbn
