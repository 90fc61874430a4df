// Streaming parser of generated tool calls: splits the model's text into plain content and complete tool calls
// while the text arrives in arbitrary pieces.
//
// Formats
//   JsonTags   <tool_call>{"name": "f", "arguments": {...}}</tool_call>            (Qwen / Hermes style)
//   ArgTags    <tool_call>f\n<arg_key>k</arg_key>\n<arg_value>v</arg_value>...</tool_call>   (GLM markers; a value
//              that parses as JSON is kept as JSON, anything else becomes a string)
//   Dsml       <｜DSML｜tool_calls> <｜DSML｜invoke name="f"> <｜DSML｜parameter name="k" string="true|false">v</｜DSML｜parameter>
//              ... </｜DSML｜invoke> </｜DSML｜tool_calls>   (every invoke is one call; string="false" values are JSON; the
//              tool_calls wrapper tags are formatting and never reach the content).  Second dialect (`set_dsml_spaced`):
//              the marker is followed by a space and the block is "calls": <｜DSML｜ calls> <｜DSML｜ invoke name="ns::f">
//              <｜DSML｜ parameter name="k" ...>; a name may carry a "namespace::" prefix, which is dropped
//   NsXml      NS<tool_call> NS<invoke name="f"> NS<k>v NS</k> ... NS</invoke> ... NS</tool_call>   (MiniMax style: the
//              namespace marker NS, "]<]minimax[>[" by default, precedes every structural tag, so '<' and '&' inside
//              values are plain bytes; a block may hold several invokes = several calls; values nest: an object is
//              NS<key>...NS</key> children, an array NS<item>...NS</item> children.  A scalar takes its JSON type from
//              the tool's parameter schema when the tools were given (`set_tools`), else it is kept as a JSON literal
//              when it reads as a number / true / false / null and as a string otherwise)
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

enum class Format { JsonTags, ArgTags, Dsml, NsXml };

struct Event {
  bool is_call = false;
  std::string text;        // content
  int index = 0;           // tool call number within the response
  std::string id, name, arguments;
};

class ToolParser {
 public:
  explicit ToolParser(Format f, std::string id_prefix = "call_") : fmt_(f), id_prefix_(std::move(id_prefix)) {
    if (f == Format::Dsml) {
      open_ = "<\xef\xbd\x9c" "DSML\xef\xbd\x9c" "invoke";
      close_ = "</\xef\xbd\x9c" "DSML\xef\xbd\x9c" "invoke>";
      silent_ = {"<\xef\xbd\x9c" "DSML\xef\xbd\x9c" "tool_calls>", "</\xef\xbd\x9c" "DSML\xef\xbd\x9c" "tool_calls>"};
    } else if (f == Format::NsXml) {
      set_namespace("]<]minimax[>[");
    } else {
      open_ = "<tool_call>";
      close_ = "</tool_call>";
    }
  }

  // Dsml: the dialect whose marker is followed by a space and whose block is called "calls".
  void set_dsml_spaced(bool spaced) {
    const std::string m = std::string("\xef\xbd\x9c" "DSML\xef\xbd\x9c") + (spaced ? " " : "");
    const std::string block = spaced ? "calls" : "tool_calls";
    open_ = "<" + m + "invoke";
    close_ = "</" + m + "invoke>";
    silent_ = {"<" + m + block + ">", "</" + m + block + ">"};
    dsml_param_ = "<" + m + "parameter";
    dsml_param_end_ = "</" + m + "parameter>";
  }
  // NsXml: the namespace marker of the model's template.
  void set_namespace(const std::string& ns) {
    ns_ = ns;
    open_ = ns + "<tool_call>";
    close_ = ns + "</tool_call>";
  }
  // The request's tools (an OpenAI `tools` array): NsXml reads the parameter schemas for value types.
  void set_tools(const json::Value& tools) { tools_ = tools; }

  std::vector<Event> feed(const std::string& piece) {
    buf_ += piece;
    std::vector<Event> out;
    for (;;) {
      if (!inside_) {
        if (skip_newline_ && !buf_.empty()) {
          if (buf_[0] == '\n') buf_.erase(0, 1);
          skip_newline_ = false;
        }
        // earliest of: the opening tag of a call, a formatting-only tag of this format
        size_t p = buf_.find(open_);
        const std::string* silent = nullptr;
        for (const auto& t : silent_) {
          const size_t q = buf_.find(t);
          if (q != std::string::npos && (p == std::string::npos || q < p)) { p = q; silent = &t; }
        }
        if (p == std::string::npos) {
          // keep the longest tail that is a proper prefix of one of those tags
          size_t hold = 0;
          auto consider = [&](const std::string& tag) {
            const size_t lim = std::min(buf_.size(), tag.size() - 1);
            for (size_t k = lim; k > hold; --k)
              if (buf_.compare(buf_.size() - k, k, tag, 0, k) == 0) { hold = k; break; }
          };
          consider(open_);
          for (const auto& t : silent_) consider(t);
          size_t cut = buf_.size() - hold;
          // newlines that may turn out to separate the text from a formatting-only tag wait for what follows them
          if (!silent_.empty())
            while (cut > 0 && buf_[cut - 1] == '\n') --cut;
          emit_content(out, buf_.substr(0, cut));
          buf_.erase(0, cut);
          return out;
        }
        if (silent) {
          std::string before = buf_.substr(0, p);
          // the blank line that separates the answer text from the tool-call block is formatting too
          while (!before.empty() && before.back() == '\n') before.pop_back();
          emit_content(out, before);
          buf_.erase(0, p + silent->size());
          skip_newline_ = true;
          continue;
        }
        emit_content(out, buf_.substr(0, p));
        buf_.erase(0, p + open_.size());
        inside_ = true;
      } else {
        const size_t p = buf_.find(close_);
        if (p == std::string::npos) return out;
        const std::string body = buf_.substr(0, p);
        buf_.erase(0, p + close_.size());
        inside_ = false;
        if (fmt_ == Format::NsXml) {
          std::vector<Event> calls;
          if (parse_ns_block(body, calls)) {
            for (auto& c : calls) {
              c.is_call = true;
              c.index = calls_++;
              c.id = id_prefix_ + std::to_string(c.index);
              out.push_back(std::move(c));
            }
            skip_newline_ = true;
          } else {
            emit_content(out, open_ + body + close_);
          }
          continue;
        }
        Event e;
        if (parse_body(body, e)) {
          e.is_call = true;
          e.index = calls_++;
          e.id = id_prefix_ + std::to_string(e.index);
          out.push_back(std::move(e));
          skip_newline_ = true;   // one separator newline after a call is formatting, not content
        } else {
          emit_content(out, open_ + body + close_);
        }
      }
    }
  }
  std::vector<Event> finish() {
    std::vector<Event> out;
    if (inside_) emit_content(out, open_ + buf_);
    else emit_content(out, buf_);
    buf_.clear();
    inside_ = false;
    return out;
  }
  int calls() const { return calls_; }

 private:
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
    if (fmt_ == Format::Dsml) {
      // body:  name="f">  then parameter elements
      const std::string& kParam = dsml_param_;
      const std::string& kParamEnd = dsml_param_end_;
      auto attr = [](const std::string& head, const std::string& key, std::string* val) {
        const size_t a = head.find(key + "=\"");
        if (a == std::string::npos) return false;
        const size_t b = head.find('"', a + key.size() + 2);
        if (b == std::string::npos) return false;
        *val = head.substr(a + key.size() + 2, b - a - key.size() - 2);
        return true;
      };
      const size_t gt = body.find('>');
      if (gt == std::string::npos || !attr(body.substr(0, gt), "name", &e.name) || e.name.empty()) return false;
      const size_t nsep = e.name.rfind("::");
      if (nsep != std::string::npos && nsep + 2 < e.name.size()) e.name = e.name.substr(nsep + 2);   // "namespace::name"
      json::Value args = json::Value::object();
      size_t p = body.find(kParam, gt);
      while (p != std::string::npos) {
        const size_t he = body.find('>', p);
        const size_t pe = he == std::string::npos ? std::string::npos : body.find(kParamEnd, he);
        if (pe == std::string::npos) return false;
        const std::string head = body.substr(p, he - p);
        std::string key, is_str = "true";
        if (!attr(head, "name", &key)) return false;
        attr(head, "string", &is_str);
        const std::string raw = body.substr(he + 1, pe - he - 1);
        if (is_str == "false") {
          try { args.set(key, json::parse(trim(raw))); } catch (const std::exception&) { args.set(key, json::Value(raw)); }
        } else {
          args.set(key, json::Value(raw));
        }
        p = body.find(kParam, pe);
      }
      e.arguments = args.dump();
      return true;
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

  // ---- NsXml
  struct NsReader {
    const std::string& t;
    const std::string& ns;
    size_t pos = 0;
    bool accept(const std::string& s) {
      if (t.compare(pos, s.size(), s) != 0) return false;
      pos += s.size();
      return true;
    }
    void ws() {
      while (pos < t.size() && (t[pos] == ' ' || t[pos] == '\n' || t[pos] == '\r' || t[pos] == '\t')) ++pos;
    }
    static std::string type_of(const json::Value* schema) {
      if (!schema || !schema->is_object()) return "";
      const json::Value* ty = schema->find("type");
      if (ty && ty->is_string()) return ty->as_string();
      if (ty && ty->is_array())
        for (const auto& x : ty->items())
          if (x.is_string() && x.as_string() != "null") return x.as_string();
      if (schema->find("properties")) return "object";
      if (schema->find("items")) return "array";
      return "";
    }
    // the value between the current position and NS</close>; consumes the closing tag
    bool value(const std::string& close, const json::Value* schema, json::Value* out, int depth, bool root) {
      if (depth > 64) return false;
      const std::string closer = ns + "</" + close + ">";
      const std::string type = type_of(schema);
      size_t look = pos;
      while (look < t.size() && (t[look] == ' ' || t[look] == '\n' || t[look] == '\r' || t[look] == '\t')) ++look;
      const bool children = t.compare(look, ns.size() + 1, ns + "<") == 0 && t.compare(look, closer.size(), closer) != 0;
      const bool array = type == "array" ? (children || t.compare(look, closer.size(), closer) == 0)
                                         : (type.empty() && children && t.compare(look, ns.size() + 6, ns + "<item>") == 0);
      const bool object = !array && (root || (type == "object" && (children || t.compare(look, closer.size(), closer) == 0)) ||
                                     (type.empty() && children));
      if (array || object) {
        *out = array ? json::Value::array() : json::Value::object();
        for (;;) {
          ws();
          if (accept(closer)) return true;
          if (!accept(ns + "<")) return false;
          const size_t end = t.find('>', pos);
          if (end == std::string::npos || end == pos) return false;
          const std::string key = t.substr(pos, end - pos);
          if (key.find_first_of("<>/\"' \n\r\t") != std::string::npos) return false;
          if (array && key != "item") return false;
          if (!array && out->find(key)) return false;
          pos = end + 1;
          const json::Value* child = nullptr;
          if (schema && schema->is_object()) {
            if (array) {
              child = schema->find("items");
            } else {
              const json::Value* props = schema->find("properties");
              if (props && props->is_object()) child = props->find(key);
              if (!child) {
                const json::Value* extra = schema->find("additionalProperties");
                if (extra && extra->is_object()) child = extra;
              }
            }
          }
          json::Value v;
          if (!value(key, child, &v, depth + 1, false)) return false;
          if (array) out->push(std::move(v));
          else out->set(key, std::move(v));
        }
      }
      const size_t end = t.find(closer, pos);
      if (end == std::string::npos) return false;
      const std::string raw = t.substr(pos, end - pos);
      pos = end + closer.size();
      if (type == "string") { *out = json::Value(raw); return true; }
      // a JSON literal when it reads as one (always tried for the non-string types, and for untyped scalars only
      // numbers / true / false / null count)
      try {
        json::Value lit = json::parse(trim(raw));
        const bool scalar_lit = lit.is_number() || lit.is_bool() || lit.is_null();
        if (!type.empty() || scalar_lit) { *out = std::move(lit); return true; }
      } catch (const std::exception&) {
      }
      *out = json::Value(raw);
      return true;
    }
  };
  const json::Value* params_schema(const std::string& name) const {
    if (!tools_.is_array()) return nullptr;
    for (const auto& tool : tools_.items()) {
      const json::Value* fn = tool.is_object() ? tool.find("function") : nullptr;
      if (!fn || !fn->is_object()) continue;
      const json::Value* n = fn->find("name");
      if (n && n->is_string() && n->as_string() == name) return fn->find("parameters");
    }
    return nullptr;
  }
  bool parse_ns_block(const std::string& body, std::vector<Event>& calls) const {
    NsReader r{body, ns_};
    for (;;) {
      r.ws();
      if (r.pos == body.size()) return !calls.empty();
      if (!r.accept(ns_ + "<invoke name=\"")) return false;
      const size_t q = body.find('"', r.pos);
      if (q == std::string::npos || q == r.pos) return false;
      Event e;
      e.name = body.substr(r.pos, q - r.pos);
      if (e.name.find_first_of("<>\r\n") != std::string::npos) return false;
      r.pos = q;
      if (!r.accept("\">")) return false;
      json::Value args;
      if (!r.value("invoke", params_schema(e.name), &args, 0, true)) return false;
      e.arguments = args.dump();
      calls.push_back(std::move(e));
    }
  }

  Format fmt_;
  std::string dsml_param_ = "<\xef\xbd\x9c" "DSML\xef\xbd\x9c" "parameter";
  std::string dsml_param_end_ = "</\xef\xbd\x9c" "DSML\xef\xbd\x9c" "parameter>";
  std::string ns_;
  json::Value tools_;
  std::string id_prefix_;
  std::string open_, close_;
  std::vector<std::string> silent_;
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
