// Small runtime services: levelled logger, scoped JSONL trace spans, CRC-32C, progress / shutdown watchdogs,
// deployment-config parser with digest, KV memory plan.
// (same roles as src/common/log.hpp, src/core/trace.hpp, src/common/crc32c.hpp, src/serve/engine_watchdog.hpp,
//  shutdown_watchdog.hpp, cluster_config.cpp, src/engine/memory_plan.hpp of the reference.)
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/resource.h>
#include <sys/stat.h>
#include <unistd.h>

#include "rt/json.h"

namespace dgpp {

// ------------------------------------------------------------------------------------------- logging
enum class LogLevel { Trace = 0, Debug, Info, Warn, Error, Off };

class Logger {
 public:
  static Logger& get() {
    static Logger l;
    return l;
  }
  static LogLevel parse(const std::string& s, LogLevel dflt) {
    static const std::map<std::string, LogLevel> m = {{"trace", LogLevel::Trace}, {"debug", LogLevel::Debug},
                                                      {"info", LogLevel::Info},   {"warn", LogLevel::Warn},
                                                      {"error", LogLevel::Error}, {"off", LogLevel::Off}};
    std::string k;
    for (char c : s) k.push_back(static_cast<char>(tolower(c)));
    auto it = m.find(k);
    return it == m.end() ? dflt : it->second;
  }
  void set_level(LogLevel l) { level_.store(static_cast<int>(l)); }
  LogLevel level() const { return static_cast<LogLevel>(level_.load()); }
  void set_sink(std::function<void(const std::string&)> sink) {
    std::lock_guard<std::mutex> g(mu_);
    sink_ = std::move(sink);
  }
  void log(LogLevel l, const std::string& component, const std::string& msg) {
    if (static_cast<int>(l) < level_.load()) return;
    static const char* names[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR"};
    const auto now = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
    char head[96];
    snprintf(head, sizeof(head), "%lld.%03lld %-5s [%s] ", static_cast<long long>(now / 1000), static_cast<long long>(now % 1000),
             names[static_cast<int>(l)], component.c_str());
    const std::string line = std::string(head) + msg;
    std::lock_guard<std::mutex> g(mu_);
    if (sink_) sink_(line);
    else fprintf(stderr, "%s\n", line.c_str());
  }

 private:
  Logger() {
    const char* e = getenv("DGPP_LOG_LEVEL");
    level_.store(static_cast<int>(e ? parse(e, LogLevel::Info) : LogLevel::Info));
  }
  std::atomic<int> level_;
  std::mutex mu_;
  std::function<void(const std::string&)> sink_;
};

// ------------------------------------------------------------------------------------------- trace spans
// One JSON object per line: {"name":..., "ts_us":..., "dur_us":..., "tid":..., "args":{...}}.  Off unless a path is set
// (DGPP_TRACE=<file> at start-up or Trace::open).
class Trace {
 public:
  static Trace& get() {
    static Trace t;
    return t;
  }
  bool enabled() const { return f_ != nullptr; }
  void open(const std::string& path) {
    std::lock_guard<std::mutex> g(mu_);
    if (f_) fclose(f_);
    f_ = path.empty() ? nullptr : fopen(path.c_str(), "w");
  }
  void close() { open(""); }
  static int64_t now_us() {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
  }
  void emit(const std::string& name, int64_t ts_us, int64_t dur_us, const std::string& args_json = "{}") {
    if (!f_) return;
    json::Value v = json::Value::object();
    v.set("name", name);
    v.set("ts_us", ts_us);
    v.set("dur_us", dur_us);
    v.set("tid", static_cast<int64_t>(std::hash<std::thread::id>()(std::this_thread::get_id()) & 0xffff));
    std::string line = v.dump();
    line.insert(line.size() - 1, ",\"args\":" + args_json);
    std::lock_guard<std::mutex> g(mu_);
    if (f_) { fprintf(f_, "%s\n", line.c_str()); fflush(f_); }
  }

 private:
  Trace() {
    const char* e = getenv("DGPP_TRACE");
    if (e && *e) f_ = fopen(e, "w");
  }
  std::mutex mu_;
  FILE* f_ = nullptr;
};

class TraceSpan {
 public:
  explicit TraceSpan(std::string name, std::string args_json = "{}")
      : name_(std::move(name)), args_(std::move(args_json)), t0_(Trace::get().enabled() ? Trace::now_us() : 0) {}
  ~TraceSpan() {
    if (Trace::get().enabled()) Trace::get().emit(name_, t0_, Trace::now_us() - t0_, args_);
  }

 private:
  std::string name_, args_;
  int64_t t0_;
};

// ------------------------------------------------------------------------------------------- CRC-32C (Castagnoli)
inline uint32_t crc32c(const void* data, size_t n, uint32_t crc = 0) {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
      table[i] = c;
    }
    init = true;
  }
  crc = ~crc;
  const unsigned char* p = static_cast<const unsigned char*>(data);
  for (size_t i = 0; i < n; ++i) crc = table[(crc ^ p[i]) & 0xff] ^ (crc >> 8);
  return ~crc;
}

// ------------------------------------------------------------------------------------------- watchdogs
// The engine loop calls progress() whenever it completes a pass; a monitor thread fires `on_stall` once when no
// progress was seen for `deadline` while work was pending.  Atomics only on the hot side.
class EngineWatchdog {
 public:
  EngineWatchdog(std::chrono::milliseconds deadline, std::function<void(int64_t stalled_ms)> on_stall,
                 std::chrono::milliseconds poll = std::chrono::milliseconds(50))
      : deadline_(deadline), poll_(poll), on_stall_(std::move(on_stall)) {
    last_.store(now_ms());
    th_ = std::thread([this] { loop(); });
  }
  ~EngineWatchdog() {
    stop_.store(true);
    if (th_.joinable()) th_.join();
  }
  void progress() { last_.store(now_ms()); }
  void set_busy(bool busy) {
    if (busy && !busy_.load()) last_.store(now_ms());
    busy_.store(busy);
  }
  bool fired() const { return fired_.load(); }

 private:
  static int64_t now_ms() {
    return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
  }
  void loop() {
    while (!stop_.load()) {
      std::this_thread::sleep_for(poll_);
      if (!busy_.load() || fired_.load()) continue;
      const int64_t idle = now_ms() - last_.load();
      if (idle > deadline_.count()) {
        fired_.store(true);
        if (on_stall_) on_stall_(idle);
      }
    }
  }
  std::chrono::milliseconds deadline_, poll_;
  std::function<void(int64_t)> on_stall_;
  std::atomic<int64_t> last_{0};
  std::atomic<bool> busy_{false}, fired_{false}, stop_{false};
  std::thread th_;
};

// Armed at shutdown: if the process has not finished within `limit`, `on_timeout` runs (the server's emergency
// exit).  disarm() on a clean finish.
class ShutdownWatchdog {
 public:
  ShutdownWatchdog(std::chrono::milliseconds limit, std::function<void()> on_timeout)
      : th_([this, limit, on_timeout] {
          const auto end = std::chrono::steady_clock::now() + limit;
          while (!done_.load() && std::chrono::steady_clock::now() < end) std::this_thread::sleep_for(std::chrono::milliseconds(10));
          if (!done_.load()) { timed_out_.store(true); if (on_timeout) on_timeout(); }
        }) {}
  ~ShutdownWatchdog() {
    done_.store(true);
    if (th_.joinable()) th_.join();
  }
  void disarm() { done_.store(true); }
  bool timed_out() const { return timed_out_.load(); }

 private:
  std::atomic<bool> done_{false}, timed_out_{false};
  std::thread th_;
};

// ------------------------------------------------------------------------------------------- deployment config
// Flat JSON deployment description.  Unknown keys are errors (a typo must not silently fall back to a default);
// digest() is the CRC-32C of the canonical (sorted-key) dump, compared across ranks before serving.
struct ClusterConfig {
  std::string model;
  std::string host = "127.0.0.1";
  int port = 8000;
  int tensor_parallel = 1;
  int expert_parallel = 1;
  int max_concurrency = 8;
  int64_t max_context = 32768;
  int prefill_chunk = 2048;
  int prefill_group_max = 4;                // readers packed into one prefill pass (1 = one request per pass)
  bool mixed_pass = false;                  // a reader's chunk rides in the pass of the decode step
  std::string kv_dtype = "fp8";
  int64_t kv_headroom_mib = 4096;
  bool prefix_cache = true;
  int64_t prefix_min_tokens = 16;
  std::string scheduler_policy = "grow";
  int mtp_depth = 0;
  int sampling_candidates = 128;
  bool fuse_all_reduce = true;
  // Everything that changes what the engine computes or which kernels run is a key here (covered by digest()), never
  // an environment variable: ranks that disagree on one of these refuse to serve together.
  int engine_decode_splits = 0;             // split-KV factor of decode attention; 0 = one resident wave
  bool engine_fuse_combine = true;          // fold the split-KV partials inside the o projection's quantiser
  bool engine_l2_prefetch = false;          // GEMMs ask L2 for the next projection's weights
  std::string engine_fp4_splits = "auto";   // split-K policy of the block-scaled GEMM: auto | resident | legacy
  bool engine_cluster_splitk = false;       // split-K through distributed shared memory instead of the workspace
  bool engine_fp4_preload = true;           // weight half of the first ring stages issued before the grid dependency
  bool engine_layer_kernel = false;         // decode through the persistent decode-layer kernel
  bool engine_seq_parallel = true;          // tensor-parallel prefill keeps the residual stream sharded by token tile
  int engine_moe_prefill_terms = 3;         // residual NVFP4 terms of the activations in expert GEMMs at prefill sizes (1..3)
  int engine_mtp_depth = 0;                 // speculative decoding: MTP drafts per step (0 = off, up to 3)
  bool engine_pin_split_rows = false;       // split-K choices ignore one row vs several (plain == speculative bits)
  std::string log_level = "info";

  static ClusterConfig parse(const std::string& text) {
    const json::Value v = json::parse(text, /*reject_duplicates=*/true);
    if (!v.is_object()) throw std::runtime_error("config: the top level must be an object");
    static const std::set<std::string> known = {
        "model", "host", "port", "tensor_parallel", "expert_parallel", "max_concurrency", "max_context", "prefill_chunk", "prefill_group_max",
        "mixed_pass",
        "kv_dtype", "kv_headroom_mib", "prefix_cache", "prefix_min_tokens", "scheduler_policy", "mtp_depth",
        "sampling_candidates", "fuse_all_reduce", "log_level", "engine_decode_splits", "engine_fuse_combine",
        "engine_l2_prefetch", "engine_fp4_splits", "engine_cluster_splitk", "engine_fp4_preload", "engine_layer_kernel",
        "engine_seq_parallel", "engine_moe_prefill_terms", "engine_mtp_depth", "engine_pin_split_rows"};
    for (const auto& kv : v.members())
      if (!known.count(kv.first)) throw std::runtime_error("config: unknown key '" + kv.first + "'");
    ClusterConfig c;
    c.model = v.get_string("model");
    if (c.model.empty()) throw std::runtime_error("config: 'model' is required");
    c.host = v.get_string("host", c.host);
    c.port = static_cast<int>(v.get_int("port", c.port));
    c.tensor_parallel = static_cast<int>(v.get_int("tensor_parallel", 1));
    c.expert_parallel = static_cast<int>(v.get_int("expert_parallel", 1));
    c.max_concurrency = static_cast<int>(v.get_int("max_concurrency", c.max_concurrency));
    c.max_context = v.get_int("max_context", c.max_context);
    c.prefill_chunk = static_cast<int>(v.get_int("prefill_chunk", c.prefill_chunk));
    c.prefill_group_max = static_cast<int>(v.get_int("prefill_group_max", c.prefill_group_max));
    c.mixed_pass = v.get_bool("mixed_pass", false);
    c.kv_dtype = v.get_string("kv_dtype", c.kv_dtype);
    c.kv_headroom_mib = v.get_int("kv_headroom_mib", c.kv_headroom_mib);
    c.prefix_cache = v.get_bool("prefix_cache", true);
    c.prefix_min_tokens = v.get_int("prefix_min_tokens", c.prefix_min_tokens);
    c.scheduler_policy = v.get_string("scheduler_policy", c.scheduler_policy);
    c.mtp_depth = static_cast<int>(v.get_int("mtp_depth", 0));
    c.sampling_candidates = static_cast<int>(v.get_int("sampling_candidates", 128));
    c.fuse_all_reduce = v.get_bool("fuse_all_reduce", true);
    c.log_level = v.get_string("log_level", c.log_level);
    c.engine_decode_splits = static_cast<int>(v.get_int("engine_decode_splits", 0));
    c.engine_fuse_combine = v.get_bool("engine_fuse_combine", true);
    c.engine_l2_prefetch = v.get_bool("engine_l2_prefetch", false);
    c.engine_fp4_splits = v.get_string("engine_fp4_splits", c.engine_fp4_splits);
    c.engine_cluster_splitk = v.get_bool("engine_cluster_splitk", false);
    c.engine_fp4_preload = v.get_bool("engine_fp4_preload", true);
    c.engine_layer_kernel = v.get_bool("engine_layer_kernel", false);
    c.engine_seq_parallel = v.get_bool("engine_seq_parallel", true);
    c.engine_moe_prefill_terms = static_cast<int>(v.get_int("engine_moe_prefill_terms", 3));
    c.engine_mtp_depth = static_cast<int>(v.get_int("engine_mtp_depth", 0));
    c.engine_pin_split_rows = v.get_bool("engine_pin_split_rows", false);
    auto need = [](bool ok, const std::string& what) { if (!ok) throw std::runtime_error("config: " + what); };
    need(c.port > 0 && c.port < 65536, "port out of range");
    need(c.tensor_parallel == 1 || c.tensor_parallel == 2 || c.tensor_parallel == 4 || c.tensor_parallel == 8,
         "tensor_parallel must be 1, 2, 4 or 8");
    need(c.expert_parallel >= 1 && c.expert_parallel <= 8, "expert_parallel must be 1..8");
    need(c.max_concurrency >= 1 && c.max_concurrency <= 64, "max_concurrency must be 1..64");
    need(c.max_context >= 16, "max_context too small");
    need(c.prefill_chunk >= 16 && c.prefill_chunk % 16 == 0, "prefill_chunk must be a positive multiple of 16");
    need(c.prefill_group_max >= 1 && c.prefill_group_max <= 64, "prefill_group_max must be 1..64");
    need(c.kv_dtype == "fp8" || c.kv_dtype == "bf16", "kv_dtype must be fp8 or bf16");
    need(c.scheduler_policy == "grow" || c.scheduler_policy == "reserve", "scheduler_policy must be grow or reserve");
    need(c.mtp_depth >= 0 && c.mtp_depth <= 5, "mtp_depth must be 0..5");
    need(c.sampling_candidates >= 1 && c.sampling_candidates <= 256, "sampling_candidates must be 1..256");
    need(c.engine_decode_splits >= 0 && c.engine_decode_splits <= 64, "engine_decode_splits must be 0..64");
    need(c.engine_moe_prefill_terms >= 1 && c.engine_moe_prefill_terms <= 3, "engine_moe_prefill_terms must be 1..3");
    need(c.engine_mtp_depth >= 0 && c.engine_mtp_depth <= 3, "engine_mtp_depth must be 0..3");
    need(c.engine_fp4_splits == "auto" || c.engine_fp4_splits == "resident" || c.engine_fp4_splits == "legacy",
         "engine_fp4_splits must be auto, resident or legacy");
    return c;
  }
  json::Value to_json() const {
    json::Value v = json::Value::object();
    v.set("expert_parallel", expert_parallel); v.set("fuse_all_reduce", fuse_all_reduce); v.set("host", host);
    v.set("kv_dtype", kv_dtype); v.set("kv_headroom_mib", kv_headroom_mib); v.set("log_level", log_level);
    v.set("max_concurrency", max_concurrency); v.set("max_context", max_context); v.set("model", model);
    v.set("mtp_depth", mtp_depth); v.set("port", port); v.set("prefill_chunk", prefill_chunk); v.set("prefill_group_max", prefill_group_max);
    v.set("mixed_pass", mixed_pass);
    v.set("prefix_cache", prefix_cache); v.set("prefix_min_tokens", prefix_min_tokens);
    v.set("sampling_candidates", sampling_candidates); v.set("scheduler_policy", scheduler_policy);
    v.set("tensor_parallel", tensor_parallel);
    v.set("engine_decode_splits", engine_decode_splits); v.set("engine_fuse_combine", engine_fuse_combine);
    v.set("engine_l2_prefetch", engine_l2_prefetch); v.set("engine_fp4_splits", engine_fp4_splits);
    v.set("engine_cluster_splitk", engine_cluster_splitk); v.set("engine_fp4_preload", engine_fp4_preload);
    v.set("engine_layer_kernel", engine_layer_kernel);
    v.set("engine_seq_parallel", engine_seq_parallel); v.set("engine_moe_prefill_terms", engine_moe_prefill_terms);
    v.set("engine_mtp_depth", engine_mtp_depth); v.set("engine_pin_split_rows", engine_pin_split_rows);
    return v;
  }
  // Same on every rank iff the engine-relevant settings agree (host / port / log level are per process).
  uint32_t digest() const {
    json::Value v = to_json();
    json::Value f = json::Value::object();
    for (const auto& kv : v.members())
      if (kv.first != "host" && kv.first != "port" && kv.first != "log_level") f.set(kv.first, kv.second);
    const std::string s = f.dump();
    return crc32c(s.data(), s.size());
  }
};

// ------------------------------------------------------------------------------------------- memory plan
// How many KV blocks fit: free device memory minus head-room minus the activation workspace, divided by the bytes of
// one block across all layers.
struct MemoryPlan {
  int64_t kv_blocks = 0;
  int64_t kv_bytes = 0;
  int64_t tokens = 0;
};
inline MemoryPlan plan_kv(int64_t free_bytes, int64_t headroom_bytes, int64_t workspace_bytes, int layers, int kv_heads,
                          int head_dim, int block_tokens, bool fp8, int64_t max_blocks = -1) {
  const int64_t elem = fp8 ? 1 : 2;
  const int64_t per_block = static_cast<int64_t>(layers) * 2 * kv_heads * block_tokens * (head_dim * elem + (fp8 ? 4 : 0));
  const int64_t avail = free_bytes - headroom_bytes - workspace_bytes;
  MemoryPlan p;
  if (avail <= 0 || per_block <= 0) return p;
  p.kv_blocks = avail / per_block;
  if (max_blocks >= 0 && p.kv_blocks > max_blocks) p.kv_blocks = max_blocks;
  p.kv_bytes = p.kv_blocks * per_block;
  p.tokens = p.kv_blocks * block_tokens;
  return p;
}

// ------------------------------------------------------------------------------------------- process memory / residency
// What the host process holds and what of a file is in the page cache: resident and peak set, locked bytes against the
// memlock limit (pinned staging buffers count against it), and the resident fraction of a weight file (mincore over a
// private read-only mapping), so the launcher can tell a warm start from a cold one and the metrics page can show it.
// (same roles as src/common/process_memory.hpp, src/common/residency.hpp of the reference.)
struct ProcessMemory {
  int64_t rss_bytes = -1, peak_rss_bytes = -1, locked_bytes = -1, memlock_limit_bytes = -1;   // -1: unknown
};
inline ProcessMemory process_memory() {
  ProcessMemory m;
  if (FILE* f = std::fopen("/proc/self/status", "r")) {
    char line[256];
    while (std::fgets(line, sizeof(line), f)) {
      long long kb = 0;
      if (std::sscanf(line, "VmRSS: %lld kB", &kb) == 1) m.rss_bytes = kb * 1024;
      else if (std::sscanf(line, "VmHWM: %lld kB", &kb) == 1) m.peak_rss_bytes = kb * 1024;
      else if (std::sscanf(line, "VmLck: %lld kB", &kb) == 1) m.locked_bytes = kb * 1024;
    }
    std::fclose(f);
  }
  struct rlimit rl;
  if (getrlimit(RLIMIT_MEMLOCK, &rl) == 0)
    m.memlock_limit_bytes = rl.rlim_cur == RLIM_INFINITY ? INT64_MAX : static_cast<int64_t>(rl.rlim_cur);
  return m;
}
// Fraction of the file's pages that are in the page cache (0..1); -1 when the file cannot be examined.  `sample_every`
// > 1 looks at every n-th page only (large checkpoints).
inline double file_residency(const std::string& path, int64_t* size_out = nullptr) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return -1.0;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size <= 0) { ::close(fd); return st.st_size == 0 ? 1.0 : -1.0; }
  if (size_out) *size_out = static_cast<int64_t>(st.st_size);
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) return -1.0;
  const long page = sysconf(_SC_PAGESIZE);
  const size_t pages = (static_cast<size_t>(st.st_size) + page - 1) / page;
  std::vector<unsigned char> vec(pages);
  double frac = -1.0;
  if (mincore(p, static_cast<size_t>(st.st_size), vec.data()) == 0) {
    size_t in = 0;
    for (unsigned char b : vec) in += b & 1;
    frac = static_cast<double>(in) / static_cast<double>(pages);
  }
  munmap(p, static_cast<size_t>(st.st_size));
  return frac;
}

// Progress of the prefills in flight, for /metrics and for a stall report: tokens done / total per request and the
// time since the last advance.
class PrefillProgress {
 public:
  void begin(const std::string& id, int64_t total, int64_t now_ms) { items_[id] = Item{0, total, now_ms, now_ms}; }
  void advance(const std::string& id, int64_t done, int64_t now_ms) {
    auto it = items_.find(id);
    if (it == items_.end()) return;
    if (done > it->second.done) { it->second.done = done; it->second.last_ms = now_ms; }
  }
  void end(const std::string& id) { items_.erase(id); }
  struct Row { std::string id; int64_t done, total, started_ms, idle_ms; };
  std::vector<Row> snapshot(int64_t now_ms) const {
    std::vector<Row> rows;
    for (const auto& kv : items_) rows.push_back(Row{kv.first, kv.second.done, kv.second.total, kv.second.start_ms, now_ms - kv.second.last_ms});
    return rows;
  }
  // the request that has gone longest without an advance (empty id: none in flight)
  Row most_stalled(int64_t now_ms) const {
    Row worst{"", 0, 0, 0, -1};
    for (const auto& r : snapshot(now_ms)) if (r.idle_ms > worst.idle_ms) worst = r;
    return worst;
  }
 private:
  struct Item { int64_t done, total, start_ms, last_ms; };
  std::map<std::string, Item> items_;
};

}  // namespace dgpp
