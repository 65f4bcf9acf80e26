// Deterministic data loader: packing, seeded shuffle, resumable cursor.
//
// Byte/behaviour compatible with the reference loader (data/loader/src/lib.rs):
// same SplitMix64-driven Fisher-Yates order for (seed, epoch) (:204-217, :367-383),
// same three packing strategies (:247-365), same cursor accounting (:162-201) and
// the same JSON envelopes with sorted keys (:389-423). Batches are also exposed as
// contiguous row-major arrays so the trainer can copy them into pinned host memory
// without a per-token Python loop.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <optional>

#include "common.hpp"

namespace py = pybind11;
using namespace pbn;

namespace loader {

static const char* kEmptySha = "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855";
static const char* kPackingSchema = "prometheus.packing";
static const char* kStateSchema = "prometheus.loader_state";

struct Packing {
  std::string packing_id;
  uint32_t sequence_length = 0;
  std::string strategy = "concat_eos";  // concat_eos | document_mask | single_document
  bool eos_between_docs = true;
  uint32_t pad_id = 0;
  std::optional<uint32_t> drop_short_below;

  static void check_strategy(const std::string& s) {
    if (s != "concat_eos" && s != "document_mask" && s != "single_document")
      throw Error("UnknownStrategy", "unknown packing strategy " + s);
  }
  std::string to_json() const {
    check_strategy(strategy);
    Json o = Json::object();
    o["schema_id"] = kPackingSchema;
    o["schema_version"] = uint64_t(1);
    o["packing_id"] = packing_id;
    o["sequence_length"] = uint64_t(sequence_length);
    o["strategy"] = strategy;
    o["eos_between_docs"] = eos_between_docs;
    o["pad_id"] = uint64_t(pad_id);
    if (drop_short_below) o["drop_short_below"] = uint64_t(*drop_short_below);
    return o.dump();
  }
  static Packing from_json(const std::string& text) {
    const Json v = Json::parse(text);
    if (!v.is_object() || !v.has("schema_id") || !v.at("schema_id").is_string() ||
        v.at("schema_id").as_string() != kPackingSchema)
      throw Error("Message", std::string("expected schema_id ") + kPackingSchema);
    Packing p;
    if (v.has("strategy") && v.at("strategy").is_string()) check_strategy(v.at("strategy").as_string());
    p.packing_id = v.at("packing_id").as_string();
    p.sequence_length = static_cast<uint32_t>(v.at("sequence_length").as_u64());
    p.strategy = v.at("strategy").as_string();
    p.eos_between_docs = v.at("eos_between_docs").as_bool();
    p.pad_id = static_cast<uint32_t>(v.at("pad_id").as_u64());
    if (v.has("drop_short_below") && !v.at("drop_short_below").is_null())
      p.drop_short_below = static_cast<uint32_t>(v.at("drop_short_below").as_u64());
    return p;
  }
};

struct PackedSequence {
  std::vector<uint32_t> tokens;
  std::vector<uint8_t> mask;
  std::optional<std::vector<uint32_t>> document_ids;
  bool operator==(const PackedSequence& o) const {
    return tokens == o.tokens && mask == o.mask && document_ids == o.document_ids;
  }
};

struct LoaderState {
  uint32_t epoch = 0;
  uint64_t step = 0;
  uint64_t shuffle_seed = 0;
  uint32_t shard_index = 0;
  uint64_t shard_offset = 0;
  uint64_t consumed_token_count = 0;
  std::string data_mix_hash;
  std::string packing_remainder_hash = kEmptySha;

  Json to_value() const {
    Json o = Json::object();
    o["schema_id"] = kStateSchema;
    o["schema_version"] = uint64_t(1);
    o["epoch"] = uint64_t(epoch);
    o["step"] = step;
    o["shuffle_seed"] = shuffle_seed;
    o["shard_index"] = uint64_t(shard_index);
    o["shard_offset"] = shard_offset;
    o["consumed_token_count"] = consumed_token_count;
    o["data_mix_hash"] = data_mix_hash;
    o["packing_remainder_hash"] = packing_remainder_hash;
    return o;
  }
  std::string to_json() const { return to_value().dump(); }
  static LoaderState from_json(const std::string& text) {
    const Json v = Json::parse(text);
    if (!v.is_object() || !v.has("schema_id") || !v.at("schema_id").is_string() ||
        v.at("schema_id").as_string() != kStateSchema)
      throw Error("Message", std::string("expected schema_id ") + kStateSchema);
    LoaderState s;
    s.epoch = static_cast<uint32_t>(v.at("epoch").as_u64());
    s.step = v.at("step").as_u64();
    s.shuffle_seed = v.at("shuffle_seed").as_u64();
    s.shard_index = static_cast<uint32_t>(v.at("shard_index").as_u64());
    s.shard_offset = v.at("shard_offset").as_u64();
    s.consumed_token_count = v.at("consumed_token_count").as_u64();
    s.data_mix_hash = v.at("data_mix_hash").as_string();
    s.packing_remainder_hash = v.at("packing_remainder_hash").as_string();
    return s;
  }
  bool operator==(const LoaderState& o) const {
    return epoch == o.epoch && step == o.step && shuffle_seed == o.shuffle_seed &&
           shard_index == o.shard_index && shard_offset == o.shard_offset &&
           consumed_token_count == o.consumed_token_count && data_mix_hash == o.data_mix_hash &&
           packing_remainder_hash == o.packing_remainder_hash;
  }
};

// Permutation of 0..n for (seed, epoch): Fisher-Yates from the top, SplitMix64 draws.
std::vector<uint64_t> shuffle_order(uint64_t n, uint64_t seed, uint32_t epoch) {
  std::vector<uint64_t> order(n);
  for (uint64_t i = 0; i < n; ++i) order[i] = i;
  if (n <= 1) return order;
  SplitMix64 rng(seed ^ (0x9E3779B97F4A7C15ull * (uint64_t(epoch) + 1)));
  for (uint64_t i = n - 1; i >= 1; --i) {
    const uint64_t j = rng.next() % (i + 1);
    std::swap(order[i], order[j]);
  }
  return order;
}

// Streaming packer: tokens are appended with their document tag; a sequence is
// emitted whenever the window fills, the final partial window is padded.
class WindowPacker {
 public:
  WindowPacker(const Packing& p, bool tag_docs)
      : len_(p.sequence_length), pad_(p.pad_id), tag_(tag_docs) {}
  void add(uint32_t token, uint32_t doc) {
    cur_.tokens.push_back(token);
    cur_.mask.push_back(1);
    if (tag_) docs_.push_back(doc);
    if (cur_.tokens.size() == len_) flush(false);
  }
  std::vector<PackedSequence> done() {
    flush(true);
    return std::move(out_);
  }

 private:
  void flush(bool pad) {
    if (cur_.tokens.empty()) return;
    if (pad) {
      cur_.tokens.resize(len_, pad_);
      cur_.mask.resize(len_, 0);
      if (tag_) docs_.resize(len_, 0);
    }
    if (tag_) cur_.document_ids = std::move(docs_);
    out_.push_back(std::move(cur_));
    cur_ = PackedSequence{};
    docs_.clear();
  }
  size_t len_;
  uint32_t pad_;
  bool tag_;
  PackedSequence cur_;
  std::vector<uint32_t> docs_;
  std::vector<PackedSequence> out_;
};

std::vector<PackedSequence> pack(const std::vector<std::vector<uint32_t>>& docs,
                                 const Packing& packing, uint32_t eos_id) {
  Packing::check_strategy(packing.strategy);
  if (packing.sequence_length == 0) throw Error("BadSequenceLength", "sequence_length must be > 0");
  if (docs.empty()) throw Error("Empty", "empty");
  if (packing.strategy == "single_document") {
    std::vector<PackedSequence> out;
    uint64_t dropped = 0;
    const size_t len = packing.sequence_length;
    for (const auto& doc : docs) {
      if (packing.drop_short_below && doc.size() < *packing.drop_short_below) {
        ++dropped;
        continue;
      }
      const size_t take = std::min(doc.size(), len);
      PackedSequence s;
      s.tokens.assign(doc.begin(), doc.begin() + take);
      s.tokens.resize(len, packing.pad_id);
      s.mask.assign(take, 1);
      s.mask.resize(len, 0);
      out.push_back(std::move(s));
    }
    if (out.empty()) {
      if (dropped > 0) throw Error("DroppedShort", "all documents dropped as short");
      throw Error("Empty", "empty");
    }
    return out;
  }
  WindowPacker packer(packing, packing.strategy == "document_mask");
  for (size_t i = 0; i < docs.size(); ++i) {
    // the separator closes the previous document and carries its tag
    if (i > 0 && packing.eos_between_docs) packer.add(eos_id, static_cast<uint32_t>(i - 1));
    for (uint32_t t : docs[i]) packer.add(t, static_cast<uint32_t>(i));
  }
  return packer.done();
}

struct Batch {
  std::vector<std::vector<uint32_t>> tokens;
  std::vector<std::vector<uint8_t>> mask;
  LoaderState state;
};

class Loader {
 public:
  Loader(std::vector<PackedSequence> seqs, Packing packing, uint64_t seed, std::string mix_hash)
      : seqs_(std::move(seqs)), packing_(std::move(packing)) {
    state_.shuffle_seed = seed;
    state_.data_mix_hash = std::move(mix_hash);
  }
  static Loader from_state(std::vector<PackedSequence> seqs, Packing packing, LoaderState st) {
    Loader l(std::move(seqs), std::move(packing), st.shuffle_seed, st.data_mix_hash);
    l.state_ = std::move(st);
    return l;
  }
  const LoaderState& state() const { return state_; }
  size_t size() const { return seqs_.size(); }

  // Indices (into the sequence list) of the next batch; advances the cursor.
  std::vector<uint64_t> next_indices(size_t batch_size) {
    const uint64_t n = seqs_.size();
    if (n == 0) throw Error("Exhausted", "exhausted");
    uint32_t epoch = state_.epoch;
    uint64_t offset = state_.shard_offset;
    if (!(cache_valid_ && cache_epoch_ == epoch)) refill(epoch);
    std::vector<uint64_t> idx;
    idx.reserve(batch_size);
    uint64_t consumed = 0;
    for (size_t b = 0; b < batch_size; ++b) {
      const uint64_t i = order_[offset];
      idx.push_back(i);
      consumed += seqs_[i].tokens.size();
      if (++offset == n) {
        offset = 0;
        ++epoch;
        refill(epoch);
      }
    }
    const uint64_t raw = state_.shard_offset + batch_size;
    state_.epoch += static_cast<uint32_t>(raw / n);
    state_.shard_offset = raw % n;
    state_.step += 1;
    state_.consumed_token_count += consumed;
    return idx;
  }
  Batch next_batch(size_t batch_size) {
    Batch b;
    for (uint64_t i : next_indices(batch_size)) {
      b.tokens.push_back(seqs_[i].tokens);
      b.mask.push_back(seqs_[i].mask);
    }
    b.state = state_;
    return b;
  }
  const PackedSequence& seq(size_t i) const { return seqs_.at(i); }

 private:
  void refill(uint32_t epoch) {
    order_ = shuffle_order(seqs_.size(), state_.shuffle_seed, epoch);
    cache_epoch_ = epoch;
    cache_valid_ = true;
  }
  std::vector<PackedSequence> seqs_;
  Packing packing_;
  LoaderState state_;
  std::vector<uint64_t> order_;
  uint32_t cache_epoch_ = 0;
  bool cache_valid_ = false;
};

Batch reconstruct(const std::vector<PackedSequence>& seqs, const Packing& packing,
                  const LoaderState& state, size_t batch_size) {
  Loader l = Loader::from_state(seqs, packing, state);
  return l.next_batch(batch_size);
}

}  // namespace loader

void bind_loader(py::module_& m) {
  using namespace loader;
  py::class_<Packing>(m, "Packing")
      .def(py::init([](std::string id, uint32_t len, std::string strategy, bool eos, uint32_t pad,
                       std::optional<uint32_t> drop) {
             Packing::check_strategy(strategy);
             Packing p;
             p.packing_id = std::move(id);
             p.sequence_length = len;
             p.strategy = std::move(strategy);
             p.eos_between_docs = eos;
             p.pad_id = pad;
             p.drop_short_below = drop;
             return p;
           }),
           py::arg("packing_id"), py::arg("sequence_length"), py::arg("strategy") = "concat_eos",
           py::arg("eos_between_docs") = true, py::arg("pad_id") = 0,
           py::arg("drop_short_below") = py::none())
      .def_readwrite("packing_id", &Packing::packing_id)
      .def_readwrite("sequence_length", &Packing::sequence_length)
      .def_readwrite("strategy", &Packing::strategy)
      .def_readwrite("eos_between_docs", &Packing::eos_between_docs)
      .def_readwrite("pad_id", &Packing::pad_id)
      .def_readwrite("drop_short_below", &Packing::drop_short_below)
      .def("to_json", &Packing::to_json)
      .def_static("from_json", &Packing::from_json);
  py::class_<PackedSequence>(m, "PackedSequence")
      .def(py::init([](std::vector<uint32_t> t, std::vector<uint8_t> mk,
                       std::optional<std::vector<uint32_t>> d) {
             PackedSequence s;
             s.tokens = std::move(t);
             s.mask = std::move(mk);
             s.document_ids = std::move(d);
             return s;
           }),
           py::arg("tokens"), py::arg("mask"), py::arg("document_ids") = py::none())
      .def_readwrite("tokens", &PackedSequence::tokens)
      .def_readwrite("mask", &PackedSequence::mask)
      .def_readwrite("document_ids", &PackedSequence::document_ids)
      .def("__eq__", &PackedSequence::operator==);
  py::class_<LoaderState>(m, "LoaderState")
      .def(py::init<>())
      .def_readwrite("epoch", &LoaderState::epoch)
      .def_readwrite("step", &LoaderState::step)
      .def_readwrite("shuffle_seed", &LoaderState::shuffle_seed)
      .def_readwrite("shard_index", &LoaderState::shard_index)
      .def_readwrite("shard_offset", &LoaderState::shard_offset)
      .def_readwrite("consumed_token_count", &LoaderState::consumed_token_count)
      .def_readwrite("data_mix_hash", &LoaderState::data_mix_hash)
      .def_readwrite("packing_remainder_hash", &LoaderState::packing_remainder_hash)
      .def("to_json", &LoaderState::to_json)
      .def_static("from_json", &LoaderState::from_json)
      .def("__eq__", &LoaderState::operator==);
  py::class_<Batch>(m, "Batch")
      .def_readonly("tokens", &Batch::tokens)
      .def_readonly("mask", &Batch::mask)
      .def_readonly("state", &Batch::state);
  py::class_<Loader>(m, "Loader")
      .def(py::init<std::vector<PackedSequence>, Packing, uint64_t, std::string>(),
           py::arg("sequences"), py::arg("packing"), py::arg("shuffle_seed"),
           py::arg("data_mix_hash"))
      .def_static("from_state", &Loader::from_state)
      .def("state", &Loader::state)
      .def("__len__", &Loader::size)
      .def("next_batch", &Loader::next_batch)
      .def("next_indices", &Loader::next_indices)
      .def(
          "next_batch_arrays",
          [](Loader& l, size_t batch_size) {
            // (tokens int64 [B, S], mask float32 [B, S]); all sequences must share a length
            auto idx = l.next_indices(batch_size);
            const size_t S = l.seq(idx.at(0)).tokens.size();
            py::array_t<int64_t> tok({batch_size, S});
            py::array_t<float> msk({batch_size, S});
            auto t = tok.mutable_unchecked<2>();
            auto k = msk.mutable_unchecked<2>();
            for (size_t b = 0; b < batch_size; ++b) {
              const auto& s = l.seq(idx[b]);
              if (s.tokens.size() != S) throw Error("Message", "ragged sequences in a batch");
              for (size_t j = 0; j < S; ++j) {
                t(b, j) = s.tokens[j];
                k(b, j) = s.mask[j];
              }
            }
            return py::make_tuple(tok, msk);
          },
          py::arg("batch_size"));
  m.def("shuffle_order", &shuffle_order, py::arg("n"), py::arg("seed"), py::arg("epoch"));
  m.def("pack", &pack, py::arg("docs"), py::arg("packing"), py::arg("eos_id"));
  m.def("reconstruct", &reconstruct);
}
