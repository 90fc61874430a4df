// Streaming parser of generated tool calls: splits the model's text into plain content and complete tool calls
// while the text arrives in arbitrary pieces.
//
// Formats
//   JsonTags   <tool_call>{"name": "f", "arguments": {...}}</tool_call>            (Qwen / Hermes style)
//   ArgTags    <tool_call>f\n<arg_key>k</arg_key>\n<arg_value>v</arg_value>...</tool_call>   (GLM markers; a value
//              that parses as JSON is kept as JSON, anything else becomes a string)
// Content outside the tags is released as soon as it cannot be the beginning of an opening tag.  A call is emitted
// when its closing tag has arrived (name, arguments as one JSON text, running index, generated id).  A body that is
// not a valid call, or text still open at finish(), is returned as content: nothing the model wrote is dropped.
// (reference counterpart: src/text/tool_parser.cpp, formats kQwenXml / kGlmMarkers.)
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "rt/json.h"

namespace dgpp {
namespace tools {

enum class Format { JsonTags, ArgTags };

struct Event {
  bool is_call = false;
  std::string text;        // content
  int index = 0;           // tool call number within the response
  std::string id, name, arguments;
};

class ToolParser {
 public:
  explicit ToolParser(Format f, std::string id_prefix = "call_") : fmt_(f), id_prefix_(std::move(id_prefix)) {}

  std::vector<Event> feed(const std::string& piece) {
    buf_ += piece;
    std::vector<Event> out;
    for (;;) {
      if (!inside_) {
        if (skip_newline_ && !buf_.empty()) {
          if (buf_[0] == '\n') buf_.erase(0, 1);
          skip_newline_ = false;
        }
        const size_t p = buf_.find(kOpen);
        if (p == std::string::npos) {
          // keep the longest tail that is a proper prefix of the opening tag
          size_t hold = 0;
          const size_t lim = std::min(buf_.size(), sizeof(kOpen) - 2);
          for (size_t k = lim; k > 0; --k)
            if (buf_.compare(buf_.size() - k, k, kOpen, k) == 0) { hold = k; break; }
          emit_content(out, buf_.substr(0, buf_.size() - hold));
          buf_.erase(0, buf_.size() - hold);
          return out;
        }
        emit_content(out, buf_.substr(0, p));
        buf_.erase(0, p + sizeof(kOpen) - 1);
        inside_ = true;
      } else {
        const size_t p = buf_.find(kClose);
        if (p == std::string::npos) return out;
        const std::string body = buf_.substr(0, p);
        buf_.erase(0, p + sizeof(kClose) - 1);
        inside_ = false;
        Event e;
        if (parse_body(body, e)) {
          e.is_call = true;
          e.index = calls_++;
          e.id = id_prefix_ + std::to_string(e.index);
          out.push_back(std::move(e));
          skip_newline_ = true;   // one separator newline after a call is formatting, not content
        } else {
          emit_content(out, std::string(kOpen) + body + kClose);
        }
      }
    }
  }
  std::vector<Event> finish() {
    std::vector<Event> out;
    if (inside_) emit_content(out, std::string(kOpen) + buf_);
    else emit_content(out, buf_);
    buf_.clear();
    inside_ = false;
    return out;
  }
  int calls() const { return calls_; }

 private:
  static constexpr char kOpen[] = "<tool_call>";
  static constexpr char kClose[] = "</tool_call>";

  static void emit_content(std::vector<Event>& out, const std::string& text) {
    if (text.empty()) return;
    if (!out.empty() && !out.back().is_call) { out.back().text += text; return; }
    Event e;
    e.text = text;
    out.push_back(std::move(e));
  }
  static std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && (s[a] == ' ' || s[a] == '\n' || s[a] == '\r' || s[a] == '\t')) ++a;
    while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\n' || s[b - 1] == '\r' || s[b - 1] == '\t')) --b;
    return s.substr(a, b - a);
  }
  bool parse_body(const std::string& body, Event& e) const {
    if (fmt_ == Format::JsonTags) {
      try {
        const json::Value v = json::parse(trim(body));
        if (!v.is_object() || !v.has("name") || !v.at("name").is_string()) return false;
        e.name = v.at("name").as_string();
        const json::Value* a = v.find("arguments");
        if (!a) a = v.find("parameters");
        if (!a) e.arguments = "{}";
        else if (a->is_string()) e.arguments = a->as_string();     // already serialised by the model
        else e.arguments = a->dump();
        return !e.name.empty();
      } catch (const std::exception&) {
        return false;
      }
    }
    // ArgTags: first line = function name, then key / value tag pairs
    const std::string t = trim(body);
    const size_t first_tag = t.find("<arg_key>");
    e.name = trim(t.substr(0, first_tag == std::string::npos ? t.size() : first_tag));
    if (e.name.empty() || e.name.find('<') != std::string::npos) return false;
    json::Value args = json::Value::object();
    size_t p = first_tag;
    while (p != std::string::npos) {
      const size_t ke = t.find("</arg_key>", p);
      if (ke == std::string::npos) return false;
      const std::string key = trim(t.substr(p + 9, ke - p - 9));
      const size_t vs = t.find("<arg_value>", ke);
      const size_t ve = vs == std::string::npos ? std::string::npos : t.find("</arg_value>", vs);
      if (ve == std::string::npos) return false;
      const std::string raw = t.substr(vs + 11, ve - vs - 11);
      json::Value val;
      try {
        val = json::parse(trim(raw));
      } catch (const std::exception&) {
        val = json::Value(raw);
      }
      args.set(key, val);
      p = t.find("<arg_key>", ve);
    }
    e.arguments = args.dump();
    return true;
  }

  Format fmt_;
  std::string id_prefix_;
  std::string buf_;
  bool inside_ = false, skip_newline_ = false;
  int calls_ = 0;
};

// Renders the tool list the way the chat template expects it when it has no tools block of its own: one JSON
// object per line inside <tools></tools>.
inline std::string render_tools_block(const json::Value& tools) {
  std::string s = "<tools>\n";
  if (tools.is_array())
    for (const auto& t : tools.items()) s += t.dump() + "\n";
  return s + "</tools>";
}

}  // namespace tools
}  // namespace dgpp
