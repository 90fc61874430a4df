// OpenAI-compatible request parsing / validation and response formatting (Chat Completions, Completions,
// Models), plus the stop-string scanner used while streaming.
//
// Validation answers HTTP 400 with {"error": {"message", "type": "invalid_request_error", "param", "code"}}
// naming the offending field; duplicate top-level fields are rejected; `max_tokens` and
// `max_completion_tokens` are mutually exclusive; `n` is 1..128; `stop` is 1..4 non-empty strings;
// `top_logprobs` is 0..20 and needs `logprobs`; `prompt_logprobs` is answered with code
// `unsupported_parameter`.  Extensions: top_k, min_p, repetition_penalty, ignore_eos, prefix_cache,
// prompt_cache_key (1..256 bytes), chat_template_kwargs, sse_ping_interval.
// (contract: docs/openai-compatibility.md:17-135, src/serve/generation_service.cpp of the reference.)
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "rt/json.h"

namespace dgpp {
namespace openai {

struct ApiError {
  int status = 400;
  std::string message, param, code, type = "invalid_request_error";
  std::string to_json() const;
};

struct Request {
  bool chat = true;
  std::string model;
  json::Value messages;              // chat: validated array of messages
  std::string prompt_text;           // completions: text prompt
  std::vector<int32_t> prompt_ids;   // completions: token-array prompt
  bool stream = false, include_usage = false;
  int64_t max_tokens = -1;           // -1: engine default
  int n = 1;
  double temperature = 1.0, top_p = 1.0, min_p = 0.0;
  int top_k = 0;
  double presence_penalty = 0.0, frequency_penalty = 0.0, repetition_penalty = 1.0;
  bool has_seed = false;
  int64_t seed = 0;
  std::vector<std::string> stop;
  bool logprobs = false;
  int top_logprobs = 0;
  std::map<int32_t, float> logit_bias;
  json::Value tools, tool_choice, response_format, chat_template_kwargs;
  bool parallel_tool_calls = true;
  bool ignore_eos = false, prefix_cache = true;
  std::string prompt_cache_key, reasoning_effort, user;
  double sse_ping_interval = 30.0;
};

// Throws ApiError.
Request parse_chat_request(const std::string& body);
Request parse_completion_request(const std::string& body);

struct Usage {
  int64_t prompt_tokens = 0, completion_tokens = 0, cached_tokens = 0;
};

struct TokenLogprob {
  std::string token;
  double logprob = 0;
  std::vector<std::pair<std::string, double>> top;
};

struct Choice {
  int index = 0;
  std::string text;            // assistant content (chat) or completion text
  std::string reasoning;       // optional reasoning_content
  std::string finish_reason;   // "stop" | "length" | "tool_calls" | "" (unfinished)
  json::Value tool_calls;      // array or null
  std::vector<TokenLogprob> logprobs;
  bool has_logprobs = false;
};

std::string completion_json(bool chat, const std::string& id, const std::string& model, int64_t created,
                            const std::vector<Choice>& choices, const Usage& usage);
// One SSE event ("data: {...}\n\n").  role_delta: first chunk of a chat choice carries {"role":"assistant"}.
std::string chunk_event(bool chat, const std::string& id, const std::string& model, int64_t created, int index,
                        const std::string& delta_text, bool role_delta, const std::string& finish_reason,
                        const json::Value* tool_calls_delta = nullptr, const TokenLogprob* logprob = nullptr);
std::string usage_event(bool chat, const std::string& id, const std::string& model, int64_t created, const Usage& usage);
std::string error_event(const ApiError& e);
inline std::string done_event() { return "data: [DONE]\n\n"; }
std::string models_json(const std::vector<std::string>& ids, int64_t created);

// Incremental stop-string scanner: feed decoded text, get the text that is safe to emit (nothing that could
// still turn into a stop string is released).  After a hit, `stopped()` is true and the stop string itself is
// never emitted.
class StopScanner {
 public:
  explicit StopScanner(std::vector<std::string> stops) : stops_(std::move(stops)) {}
  std::string feed(const std::string& text);
  std::string flush();  // end of generation without a hit: release the held-back tail
  bool stopped() const { return stopped_; }

 private:
  std::vector<std::string> stops_;
  std::string held_;
  bool stopped_ = false;
};

}  // namespace openai
}  // namespace dgpp
