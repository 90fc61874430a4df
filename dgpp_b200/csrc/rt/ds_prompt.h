// Prompt renderer for checkpoints that ship no chat template (DeepSeek-V4 style conversation layout):
//
//   <｜begin▁of▁sentence｜>[effort preamble]{system text}
//   <｜User｜>{user}<｜Assistant｜><think>{reasoning}</think>{content}[\n\n<｜DSML｜tool_calls>...]<｜end▁of▁sentence｜>
//   ... and, after a final user turn, the generation header  <｜Assistant｜><think>   (thinking mode)
//                                                        or  <｜Assistant｜></think>  (chat mode)
// Rules:
//   * there is no system token: a system message is its bare text where it stands; a conversation that ends in a
//     system message gets no generation header;
//   * consecutive user messages merge with a blank line between them; a `tool` message becomes a
//     <tool_result>...</tool_result> block inside the user turn it follows (or opens one);
//   * the request's tools are listed in a "## Tools" block appended to the first system message (an empty one is
//     inserted when the conversation has none); each line is the function object as JSON;
//   * assistant tool calls render as a DSML block: <｜DSML｜tool_calls> <｜DSML｜invoke name="f">
//     <｜DSML｜parameter name="k" string="true|false">value</｜DSML｜parameter> ... </｜DSML｜invoke> </｜DSML｜tool_calls>
//     (string="true": the raw string; "false": the value as JSON);
//   * in thinking mode the reasoning of earlier assistant turns is dropped unless the conversation carries tools or
//     `clear_thinking` is false; in chat mode every assistant turn starts with </think>;
//   * reasoning effort: minimal / low / medium (and absent) add nothing, high and xhigh / max prepend a fixed paragraph;
//     other values are refused.
// (reference counterpart: src/text/dsv4_prompt.hpp, whose header documents this layout.)
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "rt/json.h"

namespace dgpp {

class DeepSeekPrompt {
 public:
  static constexpr const char* kBos = "<\xef\xbd\x9c" "begin\xe2\x96\x81of\xe2\x96\x81sentence\xef\xbd\x9c>";
  static constexpr const char* kEos = "<\xef\xbd\x9c" "end\xe2\x96\x81of\xe2\x96\x81sentence\xef\xbd\x9c>";
  static constexpr const char* kUser = "<\xef\xbd\x9cUser\xef\xbd\x9c>";
  static constexpr const char* kAssistant = "<\xef\xbd\x9c" "Assistant\xef\xbd\x9c>";
  static constexpr const char* kDsml = "\xef\xbd\x9c" "DSML\xef\xbd\x9c";

  // globals: {"messages": [...], "tools": [...]?, "enable_thinking": bool?, "reasoning_effort": str?,
  //           "clear_thinking": bool?, "add_generation_prompt": bool?}
  static std::string render(const json::Value& g) {
    const json::Value& msgs = g.at("messages");
    const bool thinking = g.get_bool("enable_thinking", g.get_bool("thinking", true));
    const json::Value* tools = g.find("tools");
    const bool has_tools = tools && tools->is_array() && tools->size() > 0;
    const bool clear = g.get_bool("clear_thinking", g.get_bool("drop_thinking", true)) && !has_tools;
    const bool gen = g.get_bool("add_generation_prompt", true);
    std::string out = kBos;
    if (thinking) out += effort_preamble(g.get_string("reasoning_effort", "low"));

    // pass 1: normalise into turns
    struct Turn { std::string role, text, reasoning; const json::Value* calls = nullptr; };
    std::vector<Turn> turns;
    bool tools_placed = !has_tools;
    auto tools_block = [&]() {
      std::string b = "## Tools\n";
      for (const auto& t : tools->items()) {
        const json::Value* fn = t.find("function");
        if (fn) { b += fn->dump(); }
        else {
          json::Value flat = json::Value::object();
          for (const auto& kv : t.members())
            if (kv.first != "type") flat.set(kv.first, kv.second);
          b += flat.dump();
        }
        b += "\n";
      }
      return b;
    };
    if (has_tools && (msgs.size() == 0 || msgs.at(size_t(0)).get_string("role") != "system")) {
      Turn t; t.role = "system"; t.text = tools_block();
      turns.push_back(t);
      tools_placed = true;
    }
    for (const auto& m : msgs.items()) {
      const std::string role = m.get_string("role");
      if (role == "system") {
        Turn t; t.role = "system"; t.text = text_of(m, role);
        if (!tools_placed) { t.text += (t.text.empty() ? "" : "\n\n") + tools_block(); tools_placed = true; }
        turns.push_back(t);
      } else if (role == "user" || role == "tool") {
        std::string body = role == "tool" ? "<tool_result>" + text_of(m, role) + "</tool_result>" : text_of(m, role);
        if (!turns.empty() && turns.back().role == "user") turns.back().text += "\n\n" + body;
        else { Turn t; t.role = "user"; t.text = body; turns.push_back(t); }
      } else if (role == "assistant") {
        Turn t; t.role = "assistant"; t.text = text_of(m, role);
        t.reasoning = m.get_string("reasoning_content", m.get_string("reasoning"));
        const json::Value* c = m.find("tool_calls");
        if (c && c->is_array() && c->size() > 0) t.calls = c;
        turns.push_back(t);
      } else {
        throw std::invalid_argument("prompt: unsupported role '" + role + "'");
      }
    }
    // index of the last assistant turn: earlier ones lose their reasoning in thinking mode
    int last_assistant = -1;
    for (size_t i = 0; i < turns.size(); ++i)
      if (turns[i].role == "assistant") last_assistant = static_cast<int>(i);

    for (size_t i = 0; i < turns.size(); ++i) {
      const Turn& t = turns[i];
      if (t.role == "system") {
        out += t.text;
      } else if (t.role == "user") {
        out += kUser;
        out += t.text;
        const bool next_is_assistant = i + 1 < turns.size() && turns[i + 1].role == "assistant";
        if (next_is_assistant || (i + 1 == turns.size() && gen)) {
          out += kAssistant;
          if (!next_is_assistant) out += thinking ? "<think>" : "</think>";
        }
      } else {
        if (i == 0 || turns[i - 1].role != "user") out += kAssistant;   // an assistant turn with no user turn before it
        if (thinking) {
          const bool keep = !clear || static_cast<int>(i) == last_assistant;
          out += "<think>" + (keep ? t.reasoning : std::string()) + "</think>";
        } else {
          out += "</think>";
        }
        out += t.text;
        if (t.calls) out += std::string(t.text.empty() ? "" : "\n\n") + dsml_calls(*t.calls);
        out += kEos;
      }
    }
    return out;
  }

 private:
  static std::string effort_preamble(const std::string& e) {
    if (e.empty() || e == "minimal" || e == "low" || e == "medium") return "";
    if (e == "high") return "Reasoning effort: high. Think carefully and check the answer before replying.\n\n";
    if (e == "xhigh" || e == "max")
      return "Reasoning effort: maximum. Explore alternatives, verify every step and leave no shortcut untested.\n\n";
    throw std::invalid_argument("prompt: unknown reasoning_effort '" + e + "'");
  }
  static std::string text_of(const json::Value& m, const std::string& role) {
    const json::Value* c = m.find("content");
    if (!c || c->is_null()) return "";
    if (c->is_string()) return c->as_string();
    if (!c->is_array()) throw std::invalid_argument("prompt: content must be a string or an array of parts");
    std::string out;
    for (const auto& part : c->items()) {
      const std::string type = part.get_string("type");
      std::string piece;
      if (type == "text") piece = part.get_string("text");
      else if (role == "tool") piece = "[Unsupported " + type + "]";
      else throw std::invalid_argument("prompt: a '" + type + "' part in a " + role + " message cannot be rendered");
      if (!out.empty()) out += "\n\n";
      out += piece;
    }
    return out;
  }
  static std::string dsml_calls(const json::Value& calls) {
    const std::string d = kDsml;
    std::string out = "<" + d + "tool_calls>\n";
    for (const auto& c : calls.items()) {
      const json::Value* fn = c.find("function");
      const json::Value& f = fn ? *fn : c;
      out += "<" + d + "invoke name=\"" + f.get_string("name") + "\">\n";
      const json::Value* args = f.find("arguments");
      json::Value parsed;
      bool have = false;
      if (args && args->is_object()) { parsed = *args; have = true; }
      else if (args && args->is_string()) {
        try {
          parsed = json::parse(args->as_string());
          if (!parsed.is_object()) throw std::invalid_argument("prompt: tool-call arguments must be a JSON object");
          have = true;
        } catch (const json::ParseError&) {
          // not JSON: one parameter named "arguments" carrying the string
          out += "<" + d + "parameter name=\"arguments\" string=\"true\">" + args->as_string() + "</" + d + "parameter>\n";
        }
      }
      if (have)
        for (const auto& kv : parsed.members()) {
          const bool is_str = kv.second.is_string();
          out += "<" + d + "parameter name=\"" + kv.first + "\" string=\"" + (is_str ? "true" : "false") + "\">" +
                 (is_str ? kv.second.as_string() : kv.second.dump()) + "</" + d + "parameter>\n";
        }
      out += "</" + d + "invoke>\n";
    }
    out += "</" + d + "tool_calls>";
    return out;
  }
};

}  // namespace dgpp
