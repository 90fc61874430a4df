// Serving control loops that are pure functions of what they are shown (no clocks inside): the adaptive prefill
// quantum, and the multi-rank operation journal that keeps every rank's scheduler in lock step.
//
// PrefillController: decides how many prompt tokens the next engine pass may prefill.  Targets: while requests are
// decoding, the gap between two decode passes should stay under `decode_gap_target_ms`; a waiting request should see
// its first token within `first_token_target_ms`.  The quantum starts at 256, grows while passes finish under the
// gap target, shrinks when they overshoot, never drops under `floor` and is `idle_floor` when nothing is decoding
// (nobody is waiting on a decode step, so the prompt gets the whole pass).  Under load (queue depth x remaining
// prompt) the first-token target wins: the quantum is raised to what the measured prefill rate needs.
// (reference counterpart: src/sched/prefill_latency.hpp.)
//
// Journal: rank 0 appends every scheduling input (submit / cancel / tick) with a running FNV-1a digest; followers
// replay the records in order and compare digests, so a divergence is caught at the first differing operation.
// (reference counterpart: src/serve/fabric_serve.cpp rank journal / op-stream digests.)
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <stdexcept>
#include <string>
#include <vector>

#include "rt/json.h"

namespace dgpp {

struct PrefillControlConfig {
  double decode_gap_target_ms = 1000.0;
  double first_token_target_ms = 3000.0;
  int64_t start = 256, floor = 64, idle_floor = 1024, ceiling = 8192, granule = 16;
};

class PrefillController {
 public:
  explicit PrefillController(PrefillControlConfig c = PrefillControlConfig()) : c_(c), quantum_(c.start) {}

  // One finished engine pass that prefilled `tokens` prompt tokens and took `pass_ms`; `decoding` = requests that
  // were waiting on this pass for their next token.
  void observe(int64_t tokens, double pass_ms, int decoding) {
    if (tokens > 0 && pass_ms > 0) {
      const double rate = tokens / pass_ms;                      // tokens per ms
      rate_ = have_rate_ ? 0.7 * rate_ + 0.3 * rate : rate;
      have_rate_ = true;
    }
    if (decoding <= 0 || tokens <= 0) return;
    if (pass_ms > c_.decode_gap_target_ms) quantum_ = std::max<int64_t>(c_.floor, round_down(quantum_ / 2));
    else if (pass_ms < 0.5 * c_.decode_gap_target_ms) quantum_ = std::min<int64_t>(c_.ceiling, round_down(quantum_ + quantum_ / 4 + c_.granule));
  }
  // Tokens the next pass may prefill.  waiting_tokens = prompt tokens not yet prefilled over all queued requests,
  // oldest_wait_ms = how long the oldest of them has been waiting.
  int64_t next(int decoding, int64_t waiting_tokens, double oldest_wait_ms) const {
    if (waiting_tokens <= 0) return 0;
    int64_t q = decoding > 0 ? quantum_ : std::max(quantum_, c_.idle_floor);
    if (have_rate_ && decoding > 0) {
      // passes left before the oldest request breaks its first-token target, at one decode gap per pass
      const double left_ms = std::max(c_.first_token_target_ms - oldest_wait_ms, c_.decode_gap_target_ms);
      const double passes = std::max(1.0, left_ms / c_.decode_gap_target_ms);
      const int64_t need = static_cast<int64_t>(waiting_tokens / passes) + 1;
      // never ask a pass for more than the gap target allows at the measured rate
      const int64_t cap = std::max<int64_t>(c_.floor, static_cast<int64_t>(rate_ * c_.decode_gap_target_ms));
      q = std::max(q, std::min(need, cap));
    }
    q = std::min<int64_t>(std::min(q, c_.ceiling), round_up(waiting_tokens));
    return std::max<int64_t>(round_down(q), std::min<int64_t>(c_.granule, waiting_tokens));
  }
  int64_t quantum() const { return quantum_; }
  double rate_tokens_per_ms() const { return have_rate_ ? rate_ : 0.0; }

 private:
  int64_t round_down(int64_t v) const { return std::max<int64_t>(c_.granule, v / c_.granule * c_.granule); }
  int64_t round_up(int64_t v) const { return (v + c_.granule - 1) / c_.granule * c_.granule; }
  PrefillControlConfig c_;
  int64_t quantum_;
  double rate_ = 0.0;
  bool have_rate_ = false;
};

// ------------------------------------------------------------------------------------------- operation journal
struct JournalRecord {
  uint64_t seq = 0;
  std::string op;        // "submit" | "cancel" | "tick"
  std::string id;
  std::vector<int32_t> tokens;   // submit: prompt ids
  int64_t arg = 0;               // submit: max_tokens; tick: the leader's scheduler op digest before the tick (low 63 bits)
  std::string extra;             // submit: the remaining request fields as JSON text (part of the digest)
  uint64_t digest = 0;           // running digest after this record

  // One line of newline-delimited JSON (the wire and file format); digests travel as decimal strings because
  // they use all 64 bits.
  std::string to_line() const {
    json::Value o = json::Value::object();
    o.set("seq", static_cast<int64_t>(seq));
    o.set("op", op);
    o.set("id", id);
    json::Value t = json::Value::array();
    for (int32_t v : tokens) t.push(static_cast<int64_t>(v));
    o.set("tokens", std::move(t));
    o.set("arg", arg);
    if (!extra.empty()) o.set("extra", extra);
    o.set("digest", std::to_string(digest));
    return o.dump();
  }
  static JournalRecord from_line(const std::string& line) {
    const json::Value o = json::parse(line, true);
    JournalRecord r;
    r.seq = static_cast<uint64_t>(o.at("seq").as_int());
    r.op = o.at("op").as_string();
    r.id = o.get_string("id");
    if (const json::Value* t = o.find("tokens"))
      for (const auto& v : t->items()) r.tokens.push_back(static_cast<int32_t>(v.as_int()));
    r.arg = o.get_int("arg");
    r.extra = o.get_string("extra");
    r.digest = std::stoull(o.at("digest").as_string());
    return r;
  }
};

class Journal {
 public:
  // Leader side.
  const JournalRecord& append(const std::string& op, const std::string& id, const std::vector<int32_t>& tokens, int64_t arg,
                              const std::string& extra = std::string()) {
    JournalRecord r;
    r.seq = next_seq_++;
    r.op = op; r.id = id; r.tokens = tokens; r.arg = arg; r.extra = extra;
    r.digest = digest_ = fold(digest_, r);
    log_.push_back(r);
    if (log_.size() > keep_) log_.pop_front();
    return log_.back();
  }
  // Follower side: records must arrive in order; a gap or a digest mismatch is a hard error.
  void replay(const JournalRecord& r) {
    if (r.seq != next_seq_) throw std::runtime_error("journal: expected record " + std::to_string(next_seq_) + ", got " + std::to_string(r.seq));
    const uint64_t d = fold(digest_, r);
    if (d != r.digest) throw std::runtime_error("journal: digest mismatch at record " + std::to_string(r.seq) + " (" + r.op + " " + r.id + ")");
    digest_ = d;
    ++next_seq_;
  }
  uint64_t digest() const { return digest_; }
  uint64_t next_seq() const { return next_seq_; }
  // Records from `seq` on (for a follower that reconnects); empty when they were already dropped.
  std::vector<JournalRecord> since(uint64_t seq) const {
    std::vector<JournalRecord> out;
    for (const auto& r : log_)
      if (r.seq >= seq) out.push_back(r);
    if (!out.empty() && out.front().seq != seq) out.clear();
    return out;
  }
  void set_keep(size_t n) { keep_ = n; }

 private:
  static uint64_t mix(uint64_t h, const void* p, size_t n) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
  }
  static uint64_t fold(uint64_t h, const JournalRecord& r) {
    if (h == 0) h = 1469598103934665603ull;
    h = mix(h, &r.seq, 8);
    h = mix(h, r.op.data(), r.op.size());
    h = mix(h, "\0", 1);
    h = mix(h, r.id.data(), r.id.size());
    h = mix(h, "\0", 1);
    h = mix(h, r.tokens.data(), r.tokens.size() * 4);
    h = mix(h, &r.arg, 8);
    h = mix(h, r.extra.data(), r.extra.size());
    return h;
  }
  std::deque<JournalRecord> log_;
  size_t keep_ = 1 << 16;
  uint64_t next_seq_ = 0, digest_ = 0;
};

}  // namespace dgpp
