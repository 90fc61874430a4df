// Checkpoint access: safetensors reader (mmap, zero copy) and writer, sharded-checkpoint index, Hugging Face
// hub-cache resolver, architecture detection from config.json, tensor-parallel shard descriptors.
// Weights are never converted here: callers get (dtype, shape, pointer into the mapping) and upload bytes as
// stored (quantised payloads and their scale tensors included).
// (same roles as src/loaders/safetensors.hpp, hf_cache.cpp, architecture.cpp:1-85, shardspec.hpp of the reference.)
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "rt/json.h"

namespace dgpp {
namespace loaders {

// ------------------------------------------------------------------------------------------- safetensors
inline int dtype_bits(const std::string& dt) {
  static const std::map<std::string, int> bits = {
      {"F64", 64}, {"I64", 64}, {"U64", 64}, {"F32", 32}, {"I32", 32}, {"U32", 32}, {"F16", 16}, {"BF16", 16},
      {"I16", 16}, {"U16", 16}, {"F8_E4M3", 8}, {"F8_E5M2", 8}, {"F8_E8M0", 8}, {"I8", 8}, {"U8", 8}, {"BOOL", 8},
      {"F4", 4}, {"F6_E2M3", 6}, {"F6_E3M2", 6}};
  auto it = bits.find(dt);
  if (it == bits.end()) throw std::runtime_error("safetensors: unknown dtype '" + dt + "'");
  return it->second;
}

struct TensorInfo {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range inside the data section
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
  uint64_t nbytes() const { return end - begin; }
};

class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd_ < 0) throw std::runtime_error("safetensors: cannot open " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw std::runtime_error("safetensors: " + path + " is too short"); }
    size_ = static_cast<uint64_t>(st.st_size);
    map_ = static_cast<unsigned char*>(mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
    if (map_ == MAP_FAILED) { ::close(fd_); throw std::runtime_error("safetensors: mmap failed for " + path); }
    try {
      parse();
    } catch (...) {
      munmap(map_, size_);
      ::close(fd_);
      throw;
    }
  }
  ~SafetensorsFile() {
    if (map_ && map_ != MAP_FAILED) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
  }
  SafetensorsFile(const SafetensorsFile&) = delete;
  SafetensorsFile& operator=(const SafetensorsFile&) = delete;

  const std::string& path() const { return path_; }
  const std::vector<TensorInfo>& tensors() const { return tensors_; }   // sorted by name
  const std::map<std::string, std::string>& metadata() const { return metadata_; }
  const TensorInfo* find(const std::string& name) const {
    auto it = std::lower_bound(tensors_.begin(), tensors_.end(), name,
                               [](const TensorInfo& t, const std::string& n) { return t.name < n; });
    return it != tensors_.end() && it->name == name ? &*it : nullptr;
  }
  const unsigned char* data(const TensorInfo& t) const { return map_ + data_off_ + t.begin; }
  uint64_t data_offset() const { return data_off_; }
  uint64_t file_size() const { return size_; }
  // Ask the kernel to read ahead / drop a tensor's pages (sequential cold loads, release after upload).
  void advise(const TensorInfo& t, bool will_need) const {
    const uint64_t page = 4096, a = (data_off_ + t.begin) / page * page, b = data_off_ + t.end;
    madvise(map_ + a, b - a, will_need ? MADV_WILLNEED : MADV_DONTNEED);
  }

 private:
  void parse() {
    uint64_t hlen = 0;
    memcpy(&hlen, map_, 8);  // little endian on every supported host
    if (hlen < 2 || hlen > size_ - 8 || hlen > (uint64_t(100) << 20))
      throw std::runtime_error("safetensors: bad header length in " + path_);
    data_off_ = 8 + hlen;
    const json::Value h = json::parse(reinterpret_cast<const char*>(map_ + 8), hlen, /*reject_duplicates=*/true);
    if (!h.is_object()) throw std::runtime_error("safetensors: header is not an object in " + path_);
    const uint64_t data_bytes = size_ - data_off_;
    for (const auto& kv : h.members()) {
      if (kv.first == "__metadata__") {
        if (kv.second.is_object())
          for (const auto& m : kv.second.members())
            if (m.second.is_string()) metadata_[m.first] = m.second.as_string();
        continue;
      }
      TensorInfo t;
      t.name = kv.first;
      t.dtype = kv.second.at("dtype").as_string();
      for (const auto& d : kv.second.at("shape").items()) {
        if (d.as_int() < 0) throw std::runtime_error("safetensors: negative dimension in " + t.name);
        t.shape.push_back(d.as_int());
      }
      const auto& off = kv.second.at("data_offsets").items();
      if (off.size() != 2) throw std::runtime_error("safetensors: data_offsets of " + t.name + " is not a pair");
      t.begin = static_cast<uint64_t>(off[0].as_int());
      t.end = static_cast<uint64_t>(off[1].as_int());
      if (t.begin > t.end || t.end > data_bytes)
        throw std::runtime_error("safetensors: tensor " + t.name + " lies outside the file");
      const uint64_t want = (static_cast<uint64_t>(t.numel()) * dtype_bits(t.dtype) + 7) / 8;
      if (want != t.nbytes())
        throw std::runtime_error("safetensors: tensor " + t.name + " has " + std::to_string(t.nbytes()) +
                                 " bytes, its dtype and shape need " + std::to_string(want));
      tensors_.push_back(std::move(t));
    }
    std::sort(tensors_.begin(), tensors_.end(), [](const TensorInfo& a, const TensorInfo& b) { return a.name < b.name; });
    for (size_t i = 1; i < tensors_.size(); ++i)
      if (tensors_[i].name == tensors_[i - 1].name) throw std::runtime_error("safetensors: duplicate tensor " + tensors_[i].name);
    // byte ranges must not overlap
    std::vector<std::pair<uint64_t, uint64_t>> ranges;
    for (const auto& t : tensors_)
      if (t.end > t.begin) ranges.emplace_back(t.begin, t.end);
    std::sort(ranges.begin(), ranges.end());
    for (size_t i = 1; i < ranges.size(); ++i)
      if (ranges[i].first < ranges[i - 1].second) throw std::runtime_error("safetensors: overlapping tensors in " + path_);
  }

  std::string path_;
  int fd_ = -1;
  unsigned char* map_ = nullptr;
  uint64_t size_ = 0, data_off_ = 0;
  std::vector<TensorInfo> tensors_;
  std::map<std::string, std::string> metadata_;
};

struct TensorToWrite {
  std::string name, dtype;
  std::vector<int64_t> shape;
  const void* data;
  uint64_t nbytes;
};

// Writes tensors in name order, data section aligned to 8 bytes (header padded with spaces).
inline void write_safetensors(const std::string& path, std::vector<TensorToWrite> tensors,
                              const std::map<std::string, std::string>& metadata = {}) {
  std::sort(tensors.begin(), tensors.end(), [](const TensorToWrite& a, const TensorToWrite& b) { return a.name < b.name; });
  json::Value h = json::Value::object();
  if (!metadata.empty()) {
    json::Value m = json::Value::object();
    for (const auto& kv : metadata) m.set(kv.first, kv.second);
    h.set("__metadata__", m);
  }
  uint64_t off = 0;
  for (const auto& t : tensors) {
    int64_t n = 1;
    json::Value shape = json::Value::array();
    for (int64_t d : t.shape) { n *= d; shape.push(d); }
    if ((static_cast<uint64_t>(n) * dtype_bits(t.dtype) + 7) / 8 != t.nbytes)
      throw std::runtime_error("write_safetensors: size of " + t.name + " does not match dtype and shape");
    json::Value e = json::Value::object();
    e.set("dtype", t.dtype);
    e.set("shape", shape);
    json::Value o = json::Value::array();
    o.push(off);
    o.push(off + t.nbytes);
    e.set("data_offsets", o);
    h.set(t.name, e);
    off += t.nbytes;
  }
  std::string hs = h.dump();
  while ((8 + hs.size()) % 8 != 0) hs.push_back(' ');
  const std::string tmp = path + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) throw std::runtime_error("write_safetensors: cannot create " + tmp);
  const uint64_t hlen = hs.size();
  bool ok = fwrite(&hlen, 8, 1, f) == 1 && fwrite(hs.data(), 1, hs.size(), f) == hs.size();
  for (const auto& t : tensors)
    if (ok && t.nbytes) ok = fwrite(t.data, 1, t.nbytes, f) == t.nbytes;
  ok = (fclose(f) == 0) && ok;
  if (!ok || rename(tmp.c_str(), path.c_str()) != 0) {
    remove(tmp.c_str());
    throw std::runtime_error("write_safetensors: write failed for " + path);
  }
}

inline bool file_exists(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}
inline bool dir_exists(const std::string& p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
inline std::string read_text(const std::string& path) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) throw std::runtime_error("cannot open " + path);
  std::string s;
  char buf[1 << 16];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) s.append(buf, n);
  fclose(f);
  return s;
}

// A checkpoint directory: model.safetensors, or model.safetensors.index.json + shards.  Files open lazily.
class Checkpoint {
 public:
  explicit Checkpoint(const std::string& dir) : dir_(dir) {
    const std::string idx = dir + "/model.safetensors.index.json";
    if (file_exists(idx)) {
      const json::Value j = json::parse(read_text(idx));
      for (const auto& kv : j.at("weight_map").members()) where_[kv.first] = kv.second.as_string();
    } else if (file_exists(dir + "/model.safetensors")) {
      auto f = std::make_shared<SafetensorsFile>(dir + "/model.safetensors");
      for (const auto& t : f->tensors()) where_[t.name] = "model.safetensors";
      files_["model.safetensors"] = f;
    } else {
      throw std::runtime_error("checkpoint: no model.safetensors or index in " + dir);
    }
  }
  const std::string& dir() const { return dir_; }
  std::vector<std::string> names() const {
    std::vector<std::string> n;
    for (const auto& kv : where_) n.push_back(kv.first);
    return n;
  }
  bool has(const std::string& name) const { return where_.count(name) != 0; }
  // (file, tensor) of a name; throws when absent.
  std::pair<std::shared_ptr<SafetensorsFile>, const TensorInfo*> get(const std::string& name) {
    auto it = where_.find(name);
    if (it == where_.end()) throw std::runtime_error("checkpoint: tensor '" + name + "' not found in " + dir_);
    auto& f = files_[it->second];
    if (!f) f = std::make_shared<SafetensorsFile>(dir_ + "/" + it->second);
    const TensorInfo* t = f->find(name);
    if (!t) throw std::runtime_error("checkpoint: index names '" + name + "' in " + it->second + " but the file lacks it");
    return {f, t};
  }

 private:
  std::string dir_;
  std::map<std::string, std::string> where_;
  std::map<std::string, std::shared_ptr<SafetensorsFile>> files_;
};

// ------------------------------------------------------------------------------------------- HF hub cache
// "org/name" (optionally "@revision") -> snapshot directory inside the hub cache; an existing directory is
// returned unchanged.  Cache root: $HF_HUB_CACHE, else $HF_HOME/hub, else ~/.cache/huggingface/hub.
inline std::string hub_cache_root() {
  if (const char* e = getenv("HF_HUB_CACHE")) return e;
  if (const char* e = getenv("HF_HOME")) return std::string(e) + "/hub";
  const char* home = getenv("HOME");
  return std::string(home ? home : ".") + "/.cache/huggingface/hub";
}
inline std::string resolve_model(const std::string& spec, const std::string& cache_root = "") {
  if (dir_exists(spec)) return spec;
  std::string repo = spec, rev = "main";
  const size_t at = spec.find('@');
  if (at != std::string::npos) { repo = spec.substr(0, at); rev = spec.substr(at + 1); }
  if (repo.empty() || std::count(repo.begin(), repo.end(), '/') != 1 || repo.find("..") != std::string::npos)
    throw std::runtime_error("resolve_model: '" + spec + "' is neither a directory nor an org/name repository id");
  std::string folder = "models--" + repo;
  folder.replace(folder.find('/'), 1, "--");
  const std::string base = (cache_root.empty() ? hub_cache_root() : cache_root) + "/" + folder;
  if (!dir_exists(base)) throw std::runtime_error("resolve_model: " + repo + " is not in the hub cache (" + base + ")");
  std::string commit = rev;
  const std::string ref = base + "/refs/" + rev;
  if (file_exists(ref)) {
    commit = read_text(ref);
    while (!commit.empty() && (commit.back() == '\n' || commit.back() == ' ' || commit.back() == '\r')) commit.pop_back();
  }
  const std::string snap = base + "/snapshots/" + commit;
  if (!dir_exists(snap)) throw std::runtime_error("resolve_model: snapshot " + commit + " of " + repo + " is missing");
  return snap;
}

// ------------------------------------------------------------------------------------------- architecture detect
enum class Family { Unknown, QwenHybrid, QwenFlashNext, Glm4, GlmFlash, GlmDsa, DeepSeekV4, DeepSeekV41, MiMo, MiniMax, Flint, Dory, DenseGqa };

inline const char* family_name(Family f) {
  switch (f) {
    case Family::QwenHybrid: return "qwen_hybrid";
    case Family::QwenFlashNext: return "qwen_flash_next";
    case Family::Glm4: return "glm4";
    case Family::GlmFlash: return "glm_flash";
    case Family::GlmDsa: return "glm_dsa";
    case Family::DeepSeekV4: return "deepseek_v4";
    case Family::DeepSeekV41: return "deepseek_v41";
    case Family::MiMo: return "mimo";
    case Family::MiniMax: return "minimax";
    case Family::Flint: return "flint";
    case Family::Dory: return "dory";
    case Family::DenseGqa: return "dense_gqa";
    default: return "unknown";
  }
}

// Decides from `architectures[0]` first, then `model_type`; multimodal wrappers are looked through
// (`text_config`).  Unknown models raise with both strings in the message.
inline Family detect_family(const json::Value& config) {
  const json::Value* cfg = &config;
  std::string arch;
  if (const json::Value* a = config.find("architectures"))
    if (a->is_array() && a->size() > 0 && a->at(0).is_string()) arch = a->at(0).as_string();
  std::string type = config.get_string("model_type");
  if (const json::Value* tc = config.find("text_config"))
    if (tc->is_object() && type.empty()) { cfg = tc; type = tc->get_string("model_type"); }
  auto lower = [](std::string s) { for (auto& c : s) c = static_cast<char>(tolower(c)); return s; };
  const std::string a = lower(arch), t = lower(type);
  auto has = [&](const char* needle) { return a.find(needle) != std::string::npos || t.find(needle) != std::string::npos; };
  if (has("flashnext") || has("flash_next")) return Family::QwenFlashNext;
  if (has("qwen3_5") || has("qwen3_8") || has("qwen35") || has("qwen3next") || has("qwen3_next")) return Family::QwenHybrid;
  if (has("glmdsa") || has("glm_dsa") || (has("glm") && cfg->has("index_topk"))) return Family::GlmDsa;
  if (has("glmflash") || has("glm_flash") || has("glm5")) return Family::GlmFlash;
  if (has("glm4") || has("glm")) return Family::Glm4;
  if (has("deepseekv41") || has("deepseek_v41") || has("deepseek_v4_1")) return Family::DeepSeekV41;
  if (has("deepseekv4") || has("deepseek_v4")) return Family::DeepSeekV4;
  if (has("mimo")) return Family::MiMo;
  if (has("minimax")) return Family::MiniMax;
  if (has("flint")) return Family::Flint;
  if (has("dory")) return Family::Dory;
  if (has("qwen3") || has("qwen2") || has("llama") || has("mistral")) return Family::DenseGqa;
  throw std::runtime_error("detect_family: unsupported architecture '" + arch + "' / model_type '" + type + "'");
}

// ------------------------------------------------------------------------------------------- shard specs
// How one checkpoint tensor maps onto a tensor-parallel (or expert-parallel) rank.
enum class Split { Replicated, Rows, Cols, Vocab, Expert };

struct ShardSpec {
  Split split = Split::Replicated;
  int world = 1, rank = 0;
  int64_t granule = 1;  // slices are multiples of this many rows / columns (heads, quant blocks)
};

struct Slice {
  int64_t begin = 0, end = 0;  // half-open, along the split axis
  int64_t size() const { return end - begin; }
};

// Even split of `extent` units of `granule` elements; the remainder goes to the lowest ranks one granule each
// (so vocab 151936 / 8 and odd head counts still shard).  Replicated returns the whole extent.
inline Slice shard_slice(const ShardSpec& s, int64_t extent) {
  if (s.split == Split::Replicated || s.world <= 1) return {0, extent};
  if (s.rank < 0 || s.rank >= s.world) throw std::runtime_error("shard_slice: rank outside world");
  if (s.granule <= 0 || extent % s.granule != 0)
    throw std::runtime_error("shard_slice: extent " + std::to_string(extent) + " is not a multiple of granule " + std::to_string(s.granule));
  const int64_t units = extent / s.granule, base = units / s.world, rem = units % s.world;
  const int64_t b = s.rank * base + std::min<int64_t>(s.rank, rem);
  const int64_t e = b + base + (s.rank < rem ? 1 : 0);
  return {b * s.granule, e * s.granule};
}

// Which experts a rank owns under expert parallelism (contiguous blocks, remainder to the lowest ranks).
inline Slice expert_slice(int experts, int world, int rank) {
  ShardSpec s;
  s.split = Split::Expert;
  s.world = world;
  s.rank = rank;
  return shard_slice(s, experts);
}

}  // namespace loaders
}  // namespace dgpp
