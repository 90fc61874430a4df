// Interpreter for the Jinja subset that Hugging Face chat templates use.
//
// Supported: {{ expr }}, {% if/elif/else %}, {% for x in y [if cond] %} ... {% else %} with the `loop`
// object, {% set x = e %}, {% set ns.attr = e %}, block set, {% macro %} / calls, namespace(),
// raise_exception(), strftime_now(), whitespace control ({%- -%}), trim_blocks + lstrip_blocks (the
// settings transformers renders with), literals, lists, dicts, indexing / slicing / attribute access,
// method calls on strings / lists / dicts, filters, tests (`is defined`, `is none`, ...), the operators
// + - * / // % ~ == != < <= > >= in, not in, and / or / not, and the inline `a if c else b`.
// Execution limits (output bytes, loop iterations, call depth) stop hostile templates.
// (behavioural spec: src/text/chat_template.cpp:1-2251 of the reference.)
#pragma once
#include <memory>
#include <string>

#include "rt/json.h"

namespace dgpp {

struct TemplateLimits {
  size_t max_output_bytes = 64u << 20;
  size_t max_loop_iterations = 1u << 22;
  int max_depth = 64;
};

class TemplateError : public std::runtime_error {
 public:
  explicit TemplateError(const std::string& m) : std::runtime_error(m) {}
};

class ChatTemplate {
 public:
  // Parses the template source; throws TemplateError with a byte offset on syntax errors.
  explicit ChatTemplate(const std::string& source, TemplateLimits limits = TemplateLimits());
  ~ChatTemplate();
  ChatTemplate(ChatTemplate&&) noexcept;
  // Renders with the given context object (keys become template variables), e.g.
  // {"messages": [...], "add_generation_prompt": true, "bos_token": "...", "tools": [...]}.
  std::string render(const json::Value& context) const;

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

}  // namespace dgpp
