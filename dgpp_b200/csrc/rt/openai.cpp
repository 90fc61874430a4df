#include "rt/openai.h"

#include <algorithm>
#include <cmath>

namespace dgpp {
namespace openai {

using json::Value;

std::string ApiError::to_json() const {
  Value e = Value::object();
  e.set("message", message);
  e.set("type", type);
  e.set("param", param.empty() ? Value() : Value(param));
  e.set("code", code.empty() ? Value() : Value(code));
  Value root = Value::object();
  root.set("error", e);
  return root.dump();
}

namespace {

[[noreturn]] void bad(const std::string& param, const std::string& msg, const std::string& code = "") {
  ApiError e;
  e.message = msg;
  e.param = param;
  e.code = code;
  throw e;
}

Value parse_body(const std::string& body) {
  try {
    Value v = json::parse(body, /*reject_duplicates=*/true);
    if (!v.is_object()) bad("", "request body must be a JSON object");
    return v;
  } catch (const json::ParseError& pe) {
    bad("", std::string("invalid JSON body: ") + pe.what());
  }
}

double number(const Value& root, const char* k, double dflt, double lo, double hi) {
  const Value* v = root.find(k);
  if (!v || v->is_null()) return dflt;
  if (!v->is_number()) bad(k, std::string("'") + k + "' must be a number");
  const double d = v->as_double();
  if (!(d >= lo && d <= hi)) bad(k, std::string("'") + k + "' is out of range");
  return d;
}
int64_t integer(const Value& root, const char* k, int64_t dflt, int64_t lo, int64_t hi) {
  const Value* v = root.find(k);
  if (!v || v->is_null()) return dflt;
  if (!v->is_number() || std::floor(v->as_double()) != v->as_double()) bad(k, std::string("'") + k + "' must be an integer");
  const int64_t i = v->as_int();
  if (i < lo || i > hi) bad(k, std::string("'") + k + "' is out of range");
  return i;
}
bool boolean(const Value& root, const char* k, bool dflt) {
  const Value* v = root.find(k);
  if (!v || v->is_null()) return dflt;
  if (!v->is_bool()) bad(k, std::string("'") + k + "' must be a boolean");
  return v->as_bool();
}

void common_fields(const Value& root, Request& r) {
  if (const Value* m = root.find("model")) {
    if (!m->is_string()) bad("model", "'model' must be a string");
    r.model = m->as_string();
  }
  r.stream = boolean(root, "stream", false);
  if (const Value* so = root.find("stream_options")) {
    if (!so->is_null()) {
      if (!so->is_object()) bad("stream_options", "'stream_options' must be an object");
      r.include_usage = boolean(*so, "include_usage", false);
    }
  }
  const bool has_mt = root.has("max_tokens") && !root.at("max_tokens").is_null();
  const bool has_mct = root.has("max_completion_tokens") && !root.at("max_completion_tokens").is_null();
  if (has_mt && has_mct) bad("max_tokens", "'max_tokens' and 'max_completion_tokens' are mutually exclusive");
  if (has_mt) r.max_tokens = integer(root, "max_tokens", -1, 1, 1 << 30);
  if (has_mct) r.max_tokens = integer(root, "max_completion_tokens", -1, 1, 1 << 30);
  r.n = static_cast<int>(integer(root, "n", 1, 1, 128));
  r.temperature = number(root, "temperature", 1.0, 0.0, 2.0);
  r.top_p = number(root, "top_p", 1.0, 0.0, 1.0);
  r.min_p = number(root, "min_p", 0.0, 0.0, 1.0);
  r.top_k = static_cast<int>(integer(root, "top_k", 0, 0, 1 << 24));
  r.presence_penalty = number(root, "presence_penalty", 0.0, -2.0, 2.0);
  r.frequency_penalty = number(root, "frequency_penalty", 0.0, -2.0, 2.0);
  r.repetition_penalty = number(root, "repetition_penalty", 1.0, 0.01, 100.0);
  if (const Value* s = root.find("seed")) {
    if (!s->is_null()) {
      r.has_seed = true;
      r.seed = integer(root, "seed", 0, INT64_MIN, INT64_MAX);
    }
  }
  if (const Value* st = root.find("stop")) {
    if (st->is_string()) {
      if (st->as_string().empty()) bad("stop", "'stop' strings must be non-empty");
      r.stop.push_back(st->as_string());
    } else if (st->is_array()) {
      if (st->size() > 4) bad("stop", "'stop' accepts at most 4 strings");
      for (const Value& s : st->items()) {
        if (!s.is_string() || s.as_string().empty()) bad("stop", "'stop' strings must be non-empty strings");
        r.stop.push_back(s.as_string());
      }
    } else if (!st->is_null()) {
      bad("stop", "'stop' must be a string or an array of strings");
    }
  }
  if (const Value* lb = root.find("logit_bias")) {
    if (!lb->is_null()) {
      if (!lb->is_object()) bad("logit_bias", "'logit_bias' must be an object");
      for (const auto& kv : lb->members()) {
        char* end = nullptr;
        const long id = strtol(kv.first.c_str(), &end, 10);
        if (!end || *end || id < 0) bad("logit_bias", "'logit_bias' keys must be token ids");
        if (!kv.second.is_number() || std::fabs(kv.second.as_double()) > 100.0)
          bad("logit_bias", "'logit_bias' values must be numbers in [-100, 100]");
        r.logit_bias[static_cast<int32_t>(id)] = static_cast<float>(kv.second.as_double());
      }
    }
  }
  if (root.has("prompt_logprobs") && !root.at("prompt_logprobs").is_null())
    bad("prompt_logprobs", "'prompt_logprobs' is not supported", "unsupported_parameter");
  r.ignore_eos = boolean(root, "ignore_eos", false);
  r.prefix_cache = boolean(root, "prefix_cache", true);
  if (const Value* k = root.find("prompt_cache_key")) {
    if (!k->is_null()) {
      if (!k->is_string() || k->as_string().empty() || k->as_string().size() > 256)
        bad("prompt_cache_key", "'prompt_cache_key' must be a string of 1..256 bytes");
      r.prompt_cache_key = k->as_string();
    }
  }
  r.sse_ping_interval = number(root, "sse_ping_interval", 30.0, 1.0, 3600.0);
  if (const Value* u = root.find("user")) {
    if (u->is_string()) r.user = u->as_string();
  }
}

}  // namespace

Request parse_chat_request(const std::string& body) {
  const Value root = parse_body(body);
  Request r;
  r.chat = true;
  common_fields(root, r);
  const Value* msgs = root.find("messages");
  if (!msgs || !msgs->is_array() || msgs->size() == 0) bad("messages", "'messages' must be a non-empty array");
  Value out = Value::array();
  int idx = 0;
  for (const Value& m : msgs->items()) {
    const std::string where = "messages[" + std::to_string(idx) + "]";
    if (!m.is_object()) bad(where, where + " must be an object");
    const std::string role = m.get_string("role");
    if (role != "system" && role != "developer" && role != "user" && role != "assistant" && role != "tool")
      bad(where + ".role", where + ".role must be one of system, developer, user, assistant, tool");
    Value mm = Value::object();
    mm.set("role", role == "developer" ? std::string("system") : role);
    const Value* c = m.find("content");
    if (c && c->is_string()) {
      mm.set("content", c->as_string());
    } else if (c && c->is_array()) {
      // text parts are joined in order; other part types are passed through for multimodal frontends
      std::string text;
      Value parts = Value::array();
      bool only_text = true;
      for (const Value& part : c->items()) {
        if (!part.is_object()) bad(where + ".content", where + ".content parts must be objects");
        const std::string type = part.get_string("type");
        if (type == "text") {
          if (!part.has("text") || !part.at("text").is_string()) bad(where + ".content", "text parts need a 'text' string");
          text += part.at("text").as_string();
        } else if (type == "image_url" || type == "input_audio" || type == "video_url" || type == "file") {
          only_text = false;
        } else {
          bad(where + ".content", "unknown content part type '" + type + "'");
        }
        parts.push(part);
      }
      mm.set("content", text);
      if (!only_text) mm.set("parts", parts);
    } else if (!c || c->is_null()) {
      if (role != "assistant") bad(where + ".content", where + ".content is required");
      mm.set("content", "");
    } else {
      bad(where + ".content", where + ".content must be a string or an array of parts");
    }
    if (role == "tool") {
      if (!m.has("tool_call_id") || !m.at("tool_call_id").is_string())
        bad(where + ".tool_call_id", "tool messages need a 'tool_call_id'");
      mm.set("tool_call_id", m.at("tool_call_id"));
    }
    if (const Value* tc = m.find("tool_calls")) {
      if (!tc->is_null()) {
        if (!tc->is_array()) bad(where + ".tool_calls", "'tool_calls' must be an array");
        mm.set("tool_calls", *tc);
      }
    }
    if (const Value* nm = m.find("name")) {
      if (nm->is_string()) mm.set("name", *nm);
    }
    if (const Value* rc = m.find("reasoning_content")) {
      if (rc->is_string()) mm.set("reasoning_content", *rc);
    }
    out.push(mm);
    ++idx;
  }
  r.messages = out;
  r.logprobs = boolean(root, "logprobs", false);
  r.top_logprobs = static_cast<int>(integer(root, "top_logprobs", 0, 0, 20));
  if (r.top_logprobs > 0 && !r.logprobs) bad("top_logprobs", "'top_logprobs' requires 'logprobs': true");
  if (const Value* tools = root.find("tools")) {
    if (!tools->is_null()) {
      if (!tools->is_array()) bad("tools", "'tools' must be an array");
      if (tools->size() > 128) bad("tools", "at most 128 tools are supported");
      int ti = 0;
      for (const Value& t : tools->items()) {
        const std::string where = "tools[" + std::to_string(ti++) + "]";
        if (!t.is_object() || t.get_string("type") != "function" || !t.has("function") || !t.at("function").is_object())
          bad(where, where + " must be {\"type\": \"function\", \"function\": {...}}");
        if (t.at("function").get_string("name").empty()) bad(where + ".function.name", "function tools need a name");
      }
      r.tools = *tools;
    }
  }
  if (const Value* tc = root.find("tool_choice")) {
    if (tc->is_string()) {
      const std::string& s = tc->as_string();
      if (s != "auto" && s != "none" && s != "required") bad("tool_choice", "'tool_choice' must be auto, none, required or a named tool");
    } else if (tc->is_object()) {
      const std::string type = tc->get_string("type");
      if (type != "function" && type != "allowed_tools") bad("tool_choice", "unknown tool_choice type");
    } else if (!tc->is_null()) {
      bad("tool_choice", "'tool_choice' must be a string or an object");
    }
    r.tool_choice = *tc;
  }
  r.parallel_tool_calls = boolean(root, "parallel_tool_calls", true);
  if (const Value* rf = root.find("response_format")) {
    if (!rf->is_null()) {
      if (!rf->is_object()) bad("response_format", "'response_format' must be an object");
      const std::string type = rf->get_string("type");
      if (type != "text" && type != "json_object" && type != "json_schema")
        bad("response_format.type", "'response_format.type' must be text, json_object or json_schema");
      if (type == "json_schema" && (!rf->has("json_schema") || !rf->at("json_schema").is_object()))
        bad("response_format.json_schema", "'json_schema' response formats need a 'json_schema' object");
      r.response_format = *rf;
    }
  }
  if (const Value* k = root.find("chat_template_kwargs")) {
    if (!k->is_null()) {
      if (!k->is_object()) bad("chat_template_kwargs", "'chat_template_kwargs' must be an object");
      r.chat_template_kwargs = *k;
    }
  }
  if (const Value* re = root.find("reasoning_effort")) {
    if (re->is_string()) {
      static const char* ok[] = {"none", "minimal", "low", "medium", "high", "max"};
      bool found = false;
      for (const char* o : ok) found |= re->as_string() == o;
      if (!found) bad("reasoning_effort", "'reasoning_effort' must be one of none, minimal, low, medium, high, max");
      r.reasoning_effort = re->as_string();
    }
  }
  return r;
}

Request parse_completion_request(const std::string& body) {
  const Value root = parse_body(body);
  Request r;
  r.chat = false;
  common_fields(root, r);
  const Value* p = root.find("prompt");
  if (!p) bad("prompt", "'prompt' is required");
  if (p->is_string()) {
    r.prompt_text = p->as_string();
  } else if (p->is_array() && p->size() > 0 && p->at(size_t(0)).is_number()) {
    for (const Value& t : p->items()) {
      if (!t.is_number() || t.as_int() < 0) bad("prompt", "token-array prompts must hold non-negative integers");
      r.prompt_ids.push_back(static_cast<int32_t>(t.as_int()));
    }
  } else if (p->is_array() && p->size() == 1 && p->at(size_t(0)).is_string()) {
    r.prompt_text = p->at(size_t(0)).as_string();
  } else {
    bad("prompt", "'prompt' must be a string, a single-element array of strings or an array of token ids");
  }
  if (const Value* lp = root.find("logprobs")) {
    if (!lp->is_null()) {
      r.top_logprobs = static_cast<int>(integer(root, "logprobs", 0, 0, 20));
      r.logprobs = true;
    }
  }
  return r;
}

// ------------------------------------------------------------------ formatting
namespace {

Value logprob_value(const TokenLogprob& lp) {
  Value v = Value::object();
  v.set("token", lp.token);
  v.set("logprob", lp.logprob);
  Value bytes = Value::array();
  for (unsigned char c : lp.token) bytes.push(Value(static_cast<int>(c)));
  v.set("bytes", bytes);
  Value top = Value::array();
  for (const auto& t : lp.top) {
    Value e = Value::object();
    e.set("token", t.first);
    e.set("logprob", t.second);
    top.push(e);
  }
  v.set("top_logprobs", top);
  return v;
}

Value usage_value(const Usage& u) {
  Value v = Value::object();
  v.set("prompt_tokens", u.prompt_tokens);
  v.set("completion_tokens", u.completion_tokens);
  v.set("total_tokens", u.prompt_tokens + u.completion_tokens);
  Value d = Value::object();
  d.set("cached_tokens", u.cached_tokens);
  v.set("prompt_tokens_details", d);
  return v;
}

}  // namespace

std::string completion_json(bool chat, const std::string& id, const std::string& model, int64_t created,
                            const std::vector<Choice>& choices, const Usage& usage) {
  Value root = Value::object();
  root.set("id", id);
  root.set("object", chat ? "chat.completion" : "text_completion");
  root.set("created", created);
  root.set("model", model);
  Value arr = Value::array();
  for (const Choice& c : choices) {
    Value ch = Value::object();
    ch.set("index", c.index);
    if (chat) {
      Value msg = Value::object();
      msg.set("role", "assistant");
      msg.set("content", (c.tool_calls.is_array() && c.text.empty()) ? Value() : Value(c.text));
      if (!c.reasoning.empty()) msg.set("reasoning_content", c.reasoning);
      if (c.tool_calls.is_array()) msg.set("tool_calls", c.tool_calls);
      ch.set("message", msg);
    } else {
      ch.set("text", c.text);
    }
    if (c.has_logprobs) {
      Value lp = Value::object();
      Value content = Value::array();
      for (const auto& t : c.logprobs) content.push(logprob_value(t));
      lp.set("content", content);
      ch.set("logprobs", lp);
    } else {
      ch.set("logprobs", Value());
    }
    ch.set("finish_reason", c.finish_reason.empty() ? Value() : Value(c.finish_reason));
    arr.push(ch);
  }
  root.set("choices", arr);
  root.set("usage", usage_value(usage));
  return root.dump();
}

std::string chunk_event(bool chat, const std::string& id, const std::string& model, int64_t created, int index,
                        const std::string& delta_text, bool role_delta, const std::string& finish_reason,
                        const Value* tool_calls_delta, const TokenLogprob* logprob) {
  Value root = Value::object();
  root.set("id", id);
  root.set("object", chat ? "chat.completion.chunk" : "text_completion");
  root.set("created", created);
  root.set("model", model);
  Value ch = Value::object();
  ch.set("index", index);
  if (chat) {
    Value delta = Value::object();
    if (role_delta) delta.set("role", "assistant");
    if (!delta_text.empty() || role_delta) delta.set("content", delta_text);
    if (tool_calls_delta) delta.set("tool_calls", *tool_calls_delta);
    ch.set("delta", delta);
  } else {
    ch.set("text", delta_text);
  }
  if (logprob) {
    Value lp = Value::object();
    Value content = Value::array();
    content.push(logprob_value(*logprob));
    lp.set("content", content);
    ch.set("logprobs", lp);
  } else {
    ch.set("logprobs", Value());
  }
  ch.set("finish_reason", finish_reason.empty() ? Value() : Value(finish_reason));
  Value arr = Value::array();
  arr.push(ch);
  root.set("choices", arr);
  return "data: " + root.dump() + "\n\n";
}

std::string usage_event(bool chat, const std::string& id, const std::string& model, int64_t created, const Usage& usage) {
  Value root = Value::object();
  root.set("id", id);
  root.set("object", chat ? "chat.completion.chunk" : "text_completion");
  root.set("created", created);
  root.set("model", model);
  root.set("choices", Value::array());
  root.set("usage", usage_value(usage));
  return "data: " + root.dump() + "\n\n";
}

std::string error_event(const ApiError& e) { return "data: " + e.to_json() + "\n\n"; }

std::string models_json(const std::vector<std::string>& ids, int64_t created) {
  Value root = Value::object();
  root.set("object", "list");
  Value arr = Value::array();
  for (const std::string& id : ids) {
    Value m = Value::object();
    m.set("id", id);
    m.set("object", "model");
    m.set("created", created);
    m.set("owned_by", "dgpp_b200");
    arr.push(m);
  }
  root.set("data", arr);
  return root.dump();
}

// ------------------------------------------------------------------ stop scanner
std::string StopScanner::feed(const std::string& text) {
  if (stopped_) return std::string();
  held_ += text;
  if (stops_.empty()) {
    std::string out;
    out.swap(held_);
    return out;
  }
  // earliest full match
  size_t hit = std::string::npos;
  for (const std::string& s : stops_) {
    const size_t p = held_.find(s);
    if (p != std::string::npos && p < hit) hit = p;
  }
  if (hit != std::string::npos) {
    stopped_ = true;
    std::string out = held_.substr(0, hit);
    held_.clear();
    return out;
  }
  // keep the longest tail that is a proper prefix of some stop string
  size_t keep = 0;
  for (const std::string& s : stops_) {
    const size_t maxk = std::min(s.size() - 1, held_.size());
    for (size_t k = maxk; k > keep; --k) {
      if (held_.compare(held_.size() - k, k, s, 0, k) == 0) { keep = k; break; }
    }
  }
  std::string out = held_.substr(0, held_.size() - keep);
  held_.erase(0, held_.size() - keep);
  return out;
}

std::string StopScanner::flush() {
  std::string out;
  if (!stopped_) out.swap(held_);
  held_.clear();
  return out;
}

}  // namespace openai
}  // namespace dgpp
