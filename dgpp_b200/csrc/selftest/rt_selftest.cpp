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
#include "rt/jpeg.h"
#include "rt/webp.h"
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

// ---- JPEG decoder: two small files (sequential 4:2:0 with restart markers, progressive 4:2:0), then truncations and
// random byte damage of both: every input either decodes or throws, nothing reads or writes out of bounds
static const unsigned char kJpegSeq[] = {
    255, 216, 255, 224, 0, 16, 74, 70, 73, 70, 0, 1, 1, 0, 0, 1, 0, 1, 0, 0, 255, 219, 0, 67,
    0, 13, 9, 10, 11, 10, 8, 13, 11, 10, 11, 14, 14, 13, 15, 19, 32, 21, 19, 18, 18, 19, 39, 28,
    30, 23, 32, 46, 41, 49, 48, 46, 41, 45, 44, 51, 58, 74, 62, 51, 54, 70, 55, 44, 45, 64, 87, 65,
    70, 76, 78, 82, 83, 82, 50, 62, 90, 97, 90, 80, 96, 74, 81, 82, 79, 255, 219, 0, 67, 1, 14, 14,
    14, 19, 17, 19, 38, 21, 21, 38, 79, 53, 45, 53, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79,
    79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79,
    79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 255, 192, 0, 17, 8, 0, 20, 0, 24, 3,
    1, 34, 0, 2, 17, 1, 3, 17, 1, 255, 196, 0, 31, 0, 0, 1, 5, 1, 1, 1, 1, 1, 1, 0,
    0, 0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 255, 196, 0, 181, 16, 0,
    2, 1, 3, 3, 2, 4, 3, 5, 5, 4, 4, 0, 0, 1, 125, 1, 2, 3, 0, 4, 17, 5, 18, 33,
    49, 65, 6, 19, 81, 97, 7, 34, 113, 20, 50, 129, 145, 161, 8, 35, 66, 177, 193, 21, 82, 209, 240, 36,
    51, 98, 114, 130, 9, 10, 22, 23, 24, 25, 26, 37, 38, 39, 40, 41, 42, 52, 53, 54, 55, 56, 57, 58,
    67, 68, 69, 70, 71, 72, 73, 74, 83, 84, 85, 86, 87, 88, 89, 90, 99, 100, 101, 102, 103, 104, 105, 106,
    115, 116, 117, 118, 119, 120, 121, 122, 131, 132, 133, 134, 135, 136, 137, 138, 146, 147, 148, 149, 150, 151, 152, 153,
    154, 162, 163, 164, 165, 166, 167, 168, 169, 170, 178, 179, 180, 181, 182, 183, 184, 185, 186, 194, 195, 196, 197, 198,
    199, 200, 201, 202, 210, 211, 212, 213, 214, 215, 216, 217, 218, 225, 226, 227, 228, 229, 230, 231, 232, 233, 234, 241,
    242, 243, 244, 245, 246, 247, 248, 249, 250, 255, 196, 0, 31, 1, 0, 3, 1, 1, 1, 1, 1, 1, 1, 1,
    1, 0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 255, 196, 0, 181, 17, 0,
    2, 1, 2, 4, 4, 3, 4, 7, 5, 4, 4, 0, 1, 2, 119, 0, 1, 2, 3, 17, 4, 5, 33, 49,
    6, 18, 65, 81, 7, 97, 113, 19, 34, 50, 129, 8, 20, 66, 145, 161, 177, 193, 9, 35, 51, 82, 240, 21,
    98, 114, 209, 10, 22, 36, 52, 225, 37, 241, 23, 24, 25, 26, 38, 39, 40, 41, 42, 53, 54, 55, 56, 57,
    58, 67, 68, 69, 70, 71, 72, 73, 74, 83, 84, 85, 86, 87, 88, 89, 90, 99, 100, 101, 102, 103, 104, 105,
    106, 115, 116, 117, 118, 119, 120, 121, 122, 130, 131, 132, 133, 134, 135, 136, 137, 138, 146, 147, 148, 149, 150, 151,
    152, 153, 154, 162, 163, 164, 165, 166, 167, 168, 169, 170, 178, 179, 180, 181, 182, 183, 184, 185, 186, 194, 195, 196,
    197, 198, 199, 200, 201, 202, 210, 211, 212, 213, 214, 215, 216, 217, 218, 226, 227, 228, 229, 230, 231, 232, 233, 234,
    242, 243, 244, 245, 246, 247, 248, 249, 250, 255, 221, 0, 4, 0, 1, 255, 218, 0, 12, 3, 1, 0, 2, 17,
    3, 17, 0, 63, 0, 189, 7, 136, 29, 97, 206, 58, 117, 226, 176, 245, 15, 17, 57, 147, 1, 70, 61, 125,
    43, 164, 142, 194, 193, 163, 225, 151, 29, 171, 46, 235, 76, 178, 50, 245, 21, 131, 196, 210, 173, 83, 217, 211,
    142, 129, 143, 150, 25, 97, 226, 220, 89, 255, 208, 110, 151, 174, 72, 64, 37, 78, 125, 104, 173, 93, 55, 78,
    176, 84, 193, 96, 114, 59, 154, 42, 37, 67, 7, 77, 218, 113, 212, 236, 192, 213, 195, 58, 43, 221, 103, 255,
    209, 205, 181, 185, 151, 102, 55, 145, 199, 175, 214, 169, 92, 220, 76, 126, 111, 49, 187, 255, 0, 65, 69, 21,
    223, 148, 70, 60, 205, 216, 245, 115, 56, 175, 171, 199, 67, 255, 210, 198, 180, 187, 157, 83, 112, 144, 209, 69,
    20, 241, 255, 0, 198, 103, 210, 96, 35, 31, 96, 180, 63, 255, 217,
};
static const unsigned char kJpegProg[] = {
    255, 216, 255, 224, 0, 16, 74, 70, 73, 70, 0, 1, 1, 0, 0, 1, 0, 1, 0, 0, 255, 219, 0, 67,
    0, 13, 9, 10, 11, 10, 8, 13, 11, 10, 11, 14, 14, 13, 15, 19, 32, 21, 19, 18, 18, 19, 39, 28,
    30, 23, 32, 46, 41, 49, 48, 46, 41, 45, 44, 51, 58, 74, 62, 51, 54, 70, 55, 44, 45, 64, 87, 65,
    70, 76, 78, 82, 83, 82, 50, 62, 90, 97, 90, 80, 96, 74, 81, 82, 79, 255, 219, 0, 67, 1, 14, 14,
    14, 19, 17, 19, 38, 21, 21, 38, 79, 53, 45, 53, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79,
    79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79,
    79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 79, 255, 194, 0, 17, 8, 0, 20, 0, 24, 3,
    1, 34, 0, 2, 17, 1, 3, 17, 1, 255, 196, 0, 24, 0, 1, 0, 3, 1, 0, 0, 0, 0, 0, 0,
    0, 0, 0, 0, 0, 0, 0, 2, 3, 4, 5, 255, 196, 0, 23, 1, 1, 1, 1, 1, 0, 0, 0, 0,
    0, 0, 0, 0, 0, 0, 0, 0, 3, 4, 0, 2, 255, 218, 0, 12, 3, 1, 0, 2, 16, 3, 16, 0,
    0, 1, 191, 15, 75, 41, 232, 181, 58, 110, 109, 5, 41, 48, 20, 127, 255, 196, 0, 26, 16, 0, 2, 2,
    3, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 2, 0, 3, 4, 17, 33, 255, 218, 0, 8,
    1, 1, 0, 1, 5, 2, 25, 28, 179, 35, 181, 94, 96, 68, 211, 86, 155, 174, 180, 138, 198, 51, 24, 172,
    103, 255, 196, 0, 29, 17, 0, 2, 2, 1, 5, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 3,
    0, 18, 2, 4, 19, 33, 35, 49, 255, 218, 0, 8, 1, 3, 1, 1, 63, 1, 121, 94, 216, 226, 35, 37,
    211, 201, 169, 29, 98, 32, 10, 79, 255, 196, 0, 29, 17, 0, 2, 2, 1, 5, 0, 0, 0, 0, 0, 0,
    0, 0, 0, 0, 0, 1, 2, 0, 3, 4, 17, 18, 19, 49, 50, 255, 218, 0, 8, 1, 2, 1, 1, 63,
    1, 228, 87, 109, 170, 33, 74, 87, 177, 49, 0, 214, 95, 238, 127, 255, 196, 0, 22, 16, 1, 1, 1, 0,
    0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 49, 32, 255, 218, 0, 8, 1, 1, 0, 6, 63,
    2, 221, 87, 255, 196, 0, 26, 16, 0, 3, 1, 0, 3, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0,
    0, 1, 49, 17, 16, 65, 81, 255, 218, 0, 8, 1, 1, 0, 1, 63, 33, 114, 45, 232, 120, 6, 233, 113,
    138, 170, 100, 165, 58, 23, 90, 63, 255, 218, 0, 12, 3, 1, 0, 2, 0, 3, 0, 0, 0, 16, 8, 231,
    254, 255, 196, 0, 24, 17, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 0,
    33, 17, 49, 255, 218, 0, 8, 1, 3, 1, 1, 63, 16, 42, 42, 88, 212, 94, 23, 39, 47, 255, 196, 0,
    24, 17, 0, 3, 1, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 17, 49, 33, 255,
    218, 0, 8, 1, 2, 1, 1, 63, 16, 121, 128, 105, 59, 22, 28, 54, 63, 255, 196, 0, 28, 16, 1, 0,
    2, 2, 3, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 0, 17, 33, 81, 49, 65, 113, 193, 255,
    218, 0, 8, 1, 1, 0, 1, 63, 16, 186, 87, 28, 226, 38, 128, 173, 234, 32, 21, 94, 230, 25, 71, 81,
    124, 201, 77, 67, 103, 108, 195, 220, 198, 253, 140, 244, 124, 37, 116, 167, 255, 217,
};

static void test_jpeg() {
  std::mt19937 rng(99);
  const std::pair<const unsigned char*, size_t> files[] = {{kJpegSeq, sizeof(kJpegSeq)}, {kJpegProg, sizeof(kJpegProg)}};
  for (const auto& f : files) {
    const auto img = dgpp::rt::jpeg::decode(f.first, f.second);
    CHECK(img.width == 24 && img.height == 20 && img.channels == 3 && img.pixels.size() == 24u * 20u * 3u);
    int ok = 0, refused = 0;
    for (size_t cut = 0; cut < f.second; cut += 3) {
      try { dgpp::rt::jpeg::decode(f.first, cut); ++ok; } catch (const std::runtime_error&) { ++refused; }
    }
    for (int it = 0; it < 3000; ++it) {
      std::vector<unsigned char> buf(f.first, f.first + f.second);
      const int hits = 1 + static_cast<int>(rng() % 4);
      for (int h = 0; h < hits; ++h) buf[rng() % buf.size()] = static_cast<unsigned char>(rng());
      try { dgpp::rt::jpeg::decode(buf.data(), buf.size()); ++ok; } catch (const std::runtime_error&) { ++refused; }
    }
    CHECK(ok > 0 && refused > 0);
  }
}

// two 24 x 20 lossless WebP files: a noisy gradient (predictor, cross-colour and subtract-green transforms, backward
// references) and a five-colour picture (colour indexing with packed pixels)
static const unsigned char kWebpPhoto[] = {
    82, 73, 70, 70, 32, 3, 0, 0, 87, 69, 66, 80, 86, 80, 56, 76, 19, 3, 0, 0, 47, 23, 192, 4,
    0, 1, 69, 109, 219, 64, 207, 74, 230, 207, 184, 59, 40, 68, 244, 127, 2, 164, 49, 241, 24, 40, 106, 219,
    136, 41, 128, 222, 30, 239, 227, 143, 239, 192, 176, 145, 36, 169, 205, 224, 137, 136, 108, 184, 255, 127, 29, 78,
    138, 21, 182, 109, 219, 240, 255, 115, 211, 221, 26, 69, 255, 195, 103, 182, 130, 104, 145, 21, 42, 255, 11, 250,
    206, 56, 16, 172, 220, 151, 190, 40, 105, 16, 47, 206, 133, 174, 231, 56, 28, 10, 229, 36, 33, 157, 220, 196,
    45, 128, 24, 128, 109, 219, 70, 150, 72, 0, 4, 148, 241, 255, 175, 109, 222, 128, 216, 54, 146, 35, 105, 186,
    92, 215, 154, 251, 207, 63, 218, 149, 32, 128, 109, 220, 54, 0, 8, 176, 237, 254, 255, 215, 83, 33, 34, 54,
    250, 127, 119, 85, 203, 183, 222, 183, 162, 115, 223, 239, 237, 127, 186, 254, 222, 238, 239, 95, 180, 30, 109, 235,
    239, 31, 235, 194, 99, 253, 126, 61, 217, 191, 247, 223, 211, 252, 196, 245, 104, 245, 101, 218, 160, 41, 88, 189,
    175, 149, 206, 73, 247, 244, 236, 215, 50, 153, 147, 59, 151, 154, 106, 155, 11, 161, 37, 157, 89, 238, 148, 92,
    68, 103, 197, 194, 122, 179, 238, 105, 174, 37, 5, 91, 146, 133, 244, 204, 144, 132, 135, 171, 22, 148, 163, 174,
    224, 237, 250, 254, 60, 100, 140, 142, 229, 251, 112, 52, 108, 142, 113, 167, 101, 209, 115, 39, 50, 187, 184, 140,
    180, 173, 148, 210, 230, 206, 96, 43, 165, 226, 186, 195, 85, 64, 6, 84, 117, 57, 131, 213, 93, 100, 163, 241,
    13, 101, 69, 128, 214, 109, 196, 17, 218, 238, 128, 57, 164, 204, 54, 45, 166, 24, 27, 79, 203, 197, 57, 152,
    125, 242, 114, 165, 91, 61, 49, 34, 136, 26, 17, 104, 152, 206, 211, 82, 205, 63, 116, 75, 221, 73, 67, 184,
    212, 217, 17, 122, 50, 233, 32, 47, 117, 234, 60, 74, 17, 38, 45, 41, 182, 111, 247, 246, 20, 91, 232, 139,
    61, 170, 118, 230, 77, 69, 120, 176, 226, 53, 179, 213, 41, 87, 238, 186, 214, 70, 176, 213, 177, 24, 27, 131,
    80, 97, 148, 167, 99, 21, 6, 17, 34, 186, 135, 209, 133, 141, 213, 35, 160, 229, 109, 223, 40, 218, 229, 2,
    70, 222, 90, 229, 201, 77, 97, 103, 39, 68, 15, 3, 80, 115, 253, 207, 192, 124, 175, 180, 138, 123, 236, 229,
    195, 76, 79, 209, 161, 63, 219, 88, 185, 57, 197, 108, 28, 27, 35, 204, 64, 130, 41, 189, 156, 33, 48, 19,
    53, 145, 52, 230, 112, 230, 74, 64, 208, 238, 76, 109, 69, 0, 212, 74, 80, 115, 136, 77, 197, 46, 184, 89,
    42, 77, 29, 178, 137, 176, 37, 240, 232, 197, 185, 231, 60, 172, 187, 224, 15, 149, 162, 222, 126, 216, 213, 205,
    152, 74, 164, 49, 226, 224, 6, 28, 137, 2, 105, 161, 5, 125, 20, 240, 250, 168, 4, 103, 145, 97, 194, 51,
    88, 52, 126, 217, 137, 53, 164, 208, 225, 142, 104, 174, 53, 136, 169, 85, 1, 59, 67, 81, 228, 90, 246, 156,
    133, 139, 195, 7, 219, 103, 23, 12, 137, 123, 46, 184, 84, 195, 195, 253, 180, 129, 229, 237, 132, 215, 207, 7,
    10, 238, 185, 104, 116, 152, 60, 136, 30, 194, 155, 105, 213, 71, 20, 176, 175, 88, 4, 135, 101, 20, 25, 111,
    102, 170, 88, 130, 112, 190, 135, 114, 0, 207, 245, 149, 252, 26, 0, 51, 39, 173, 180, 73, 209, 70, 57, 112,
    52, 23, 116, 100, 233, 152, 29, 123, 162, 254, 118, 86, 105, 83, 217, 47, 54, 71, 80, 99, 51, 32, 251, 242,
    11, 202, 213, 225, 47, 57, 27, 250, 146, 209, 39, 11, 148, 67, 221, 249, 215, 187, 54, 169, 116, 102, 108, 25,
    158, 109, 152, 136, 70, 215, 131, 241, 85, 113, 212, 51, 186, 174, 188, 206, 1, 215, 33, 16, 138, 99, 97, 241,
    26, 130, 19, 247, 222, 54, 52, 73, 123, 221, 179, 247, 69, 200, 208, 116, 24, 198, 92, 80, 91, 131, 2, 46,
    41, 237, 123, 117, 213, 97, 83, 140, 53, 174, 11, 103, 116, 95, 203, 92, 25, 109, 47, 144, 168, 166, 116, 244,
    154, 34, 126, 200, 222, 239, 33, 190, 130, 53, 189, 51, 181, 86, 163, 102, 213, 67, 215, 229, 140, 51, 196, 187,
    86, 28, 149, 98, 22, 250, 62, 156, 198, 115, 100, 210, 0, 213, 2, 0,
};
static const unsigned char kWebpPalette[] = {
    82, 73, 70, 70, 216, 0, 0, 0, 87, 69, 66, 80, 86, 80, 56, 76, 204, 0, 0, 0, 47, 23, 192, 4,
    0, 39, 64, 152, 109, 244, 29, 195, 96, 6, 119, 198, 103, 67, 144, 109, 147, 140, 97, 0, 51, 184, 230, 177,
    9, 178, 109, 4, 70, 48, 148, 73, 221, 253, 4, 243, 31, 234, 47, 128, 117, 125, 192, 32, 0, 144, 182, 178,
    80, 12, 128, 72, 0, 95, 0, 230, 8, 224, 33, 162, 255, 241, 218, 223, 73, 112, 221, 233, 101, 209, 0, 108,
    136, 250, 63, 222, 86, 184, 230, 230, 117, 238, 191, 57, 226, 28, 35, 193, 154, 14, 110, 108, 242, 55, 193, 54,
    246, 72, 222, 234, 157, 75, 3, 113, 211, 151, 14, 0, 93, 42, 19, 236, 165, 27, 83, 162, 79, 168, 109, 9,
    130, 125, 143, 235, 243, 109, 187, 67, 127, 166, 16, 226, 126, 149, 118, 86, 235, 109, 85, 141, 75, 110, 214, 254,
    152, 176, 149, 179, 7, 62, 177, 211, 137, 83, 95, 24, 199, 109, 110, 185, 204, 60, 121, 30, 196, 8, 213, 82,
    162, 3, 159, 23, 88, 58, 152, 36, 13, 85, 4, 177, 176, 136, 103, 155, 166, 149, 227, 11, 252, 29, 135, 30,
    34, 31, 94, 158, 5, 192, 157, 38,
};

static void test_webp() {
  std::mt19937 rng(123);
  const std::pair<const unsigned char*, size_t> files[] = {{kWebpPhoto, sizeof(kWebpPhoto)}, {kWebpPalette, sizeof(kWebpPalette)}};
  for (const auto& f : files) {
    const auto img = dgpp::rt::webp::decode(f.first, f.second);
    CHECK(img.width == 24 && img.height == 20 && img.rgba.size() == 24u * 20u * 4u);
    int ok = 0, refused = 0;
    for (size_t cut = 0; cut < f.second; cut += 3) {
      try { dgpp::rt::webp::decode(f.first, cut); ++ok; } catch (const std::runtime_error&) { ++refused; }
    }
    for (int it = 0; it < 6000; ++it) {
      std::vector<unsigned char> buf(f.first, f.first + f.second);
      const int hits = 1 + static_cast<int>(rng() % 4);
      for (int h = 0; h < hits; ++h) buf[20 + rng() % (buf.size() - 20)] = static_cast<unsigned char>(rng());
      try {
        const auto r = dgpp::rt::webp::decode(buf.data(), buf.size());
        CHECK(r.rgba.size() == static_cast<size_t>(r.width) * r.height * 4);
        ++ok;
      } catch (const std::runtime_error&) { ++refused; }
    }
    CHECK(ok > 0 && refused > 0);
  }
}

int main() {
  test_blocks();
  test_scheduler();
  test_json();
  test_grammar();
  test_crc_and_journal();
  test_jpeg();
  test_webp();
  if (g_fail) { std::fprintf(stderr, "selftest: %d check(s) failed\n", g_fail); return 1; }
  std::puts("rt selftest ok");
  return 0;
}
