// Token-level constrained decoding of tool calls.
//
// The generated text is  <free text>  then zero or more calls
//     <tool_call>\n{"name": "<one of the request's tools>", "arguments": <JSON matching that tool's parameters>}\n</tool_call>
// separated by "\n".  The machine below walks that language byte by byte:
//   Text   free text.  Allowed only when the tool choice is "auto"; every byte is legal, a small matcher tracks how
//          much of the opening tag has been written, and completing it enters the call.
//   Open   the forced remainder of  <tool_call>\n{"name": "   (tool choice "required" / a named function start here)
//   Name   one of the tool names, matched as a set of candidates that shrinks byte by byte, ended by '"'
//   Mid    the literal  , "arguments":<space>
//   Args   the JSON pushdown machine over the chosen tool's parameter schema
//   Close  the literal  }\n</tool_call>
//   After  end of text, or "\n" + another call (when parallel calls are allowed)
// A wrapper turns the byte machine into vocabulary masks exactly like the JSON grammar does: a token is allowed when
// all of its bytes are, masks are cached by machine signature, the end-of-sequence ids are allowed where the text may
// stop.  With tool choice "auto" the Text phase allows every token, so an unconstrained answer costs nothing.
// (reference counterpart: src/text/tool_grammar.cpp -- Qwen XML / GLM marker grammars over the JSON machine.)
#pragma once
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "rt/json_grammar.h"

namespace dgpp {
namespace grammar {

struct ToolSpec {
  std::string name;
  std::shared_ptr<const Schema> parameters;   // compiled "parameters" schema (any object when absent)
};

enum class ToolChoice { Auto, Required };

class ToolCallMachine {
 public:
  ToolCallMachine(std::shared_ptr<const std::vector<ToolSpec>> tools, ToolChoice choice, bool parallel)
      : tools_(std::move(tools)), parallel_(parallel) {
    if (choice == ToolChoice::Required) { phase_ = Open; pos_ = 0; }
  }
  // May the text end here?
  bool can_finish() const { return phase_ == Text || phase_ == After; }
  bool in_call() const { return phase_ != Text && phase_ != After; }
  int calls() const { return calls_; }

  bool step(unsigned char c) {
    switch (phase_) {
      case Text: {
        // longest-prefix matcher on the opening tag (the tag has no proper border, so a mismatch restarts at 0 or 1)
        if (static_cast<unsigned char>(kOpenTag[pos_]) == c) {
          if (kOpenTag[++pos_] == 0) { phase_ = Open; pos_ = static_cast<int>(sizeof(kOpenTag) - 1); }
        } else {
          pos_ = static_cast<unsigned char>(kOpenTag[0]) == c ? 1 : 0;
        }
        return true;
      }
      case Open:
        if (static_cast<unsigned char>(kOpen[pos_]) != c) return false;
        if (kOpen[++pos_] == 0) { phase_ = Name; pos_ = 0; cand_.assign(tools_->size(), true); }
        return true;
      case Name: {
        if (c == '"') {
          for (size_t i = 0; i < tools_->size(); ++i)
            if (cand_[i] && (*tools_)[i].name.size() == static_cast<size_t>(pos_)) {
              tool_ = static_cast<int>(i);
              phase_ = Mid;
              pos_ = 0;
              return true;
            }
          return false;
        }
        bool any = false;
        for (size_t i = 0; i < tools_->size(); ++i) {
          const std::string& n = (*tools_)[i].name;
          cand_[i] = cand_[i] && static_cast<size_t>(pos_) < n.size() && static_cast<unsigned char>(n[pos_]) == c;
          any = any || cand_[i];
        }
        ++pos_;
        return any;
      }
      case Mid:
        if (static_cast<unsigned char>(kMid[pos_]) != c) return false;
        if (kMid[++pos_] == 0) {
          phase_ = Args;
          args_ = std::make_shared<Machine>((*tools_)[tool_].parameters);
        }
        return true;
      case Args: {
        if (!args_->done()) {
          // copy-on-write: trial copies of this machine share the inner machine until one of them advances it
          const bool could_end = args_->can_finish();
          if (args_.use_count() > 1) args_ = std::make_shared<Machine>(*args_);
          if (args_->step(c)) return true;
          if (!could_end) return false;
        }
        // the arguments value is complete: this byte belongs to the closing literal
        phase_ = Close;
        pos_ = 0;
        args_.reset();
        return step(c);
      }
      case Close:
        if (static_cast<unsigned char>(kClose[pos_]) != c) return false;
        if (kClose[++pos_] == 0) { phase_ = After; pos_ = 0; ++calls_; }
        return true;
      case After:
        if (!parallel_) return false;
        if (static_cast<unsigned char>(kAgain[pos_]) != c) return false;
        if (kAgain[++pos_] == 0) { phase_ = Open; pos_ = static_cast<int>(sizeof(kOpenTag) - 1); }
        return true;
    }
    return false;
  }
  bool feed(const std::string& bytes) {
    for (unsigned char c : bytes)
      if (!step(c)) return false;
    return true;
  }
  // Free text with no partial tag pending: every token is allowed (the wrapper's fast path).
  bool unconstrained() const { return phase_ == Text && pos_ == 0; }
  std::string signature() const {
    std::string s;
    s.push_back(static_cast<char>(phase_));
    s.append(reinterpret_cast<const char*>(&pos_), 4);
    s.push_back(static_cast<char>(tool_));
    if (phase_ == Name)
      for (bool b : cand_) s.push_back(b ? '1' : '0');
    if (phase_ == Args && args_) s += args_->signature();
    return s;
  }

 private:
  enum Phase : uint8_t { Text, Open, Name, Mid, Args, Close, After };
  static constexpr char kOpenTag[] = "<tool_call>";
  static constexpr char kOpen[] = "<tool_call>\n{\"name\": \"";
  static constexpr char kMid[] = ", \"arguments\": ";
  static constexpr char kClose[] = "}\n</tool_call>";
  static constexpr char kAgain[] = "\n<tool_call>";
  std::shared_ptr<const std::vector<ToolSpec>> tools_;
  bool parallel_;
  Phase phase_ = Text;
  int pos_ = 0, tool_ = -1, calls_ = 0;
  std::vector<bool> cand_;
  std::shared_ptr<Machine> args_;
};

class ToolTokenGrammar {
 public:
  ToolTokenGrammar(std::shared_ptr<const std::vector<ToolSpec>> tools, ToolChoice choice, bool parallel,
                   std::shared_ptr<const std::vector<std::string>> token_bytes, std::vector<int32_t> eos_ids)
      : machine_(std::move(tools), choice, parallel), tokens_(std::move(token_bytes)), eos_(std::move(eos_ids)),
        cache_(std::make_shared<std::unordered_map<std::string, std::vector<uint32_t>>>()) {}

  size_t words() const { return (tokens_->size() + 31) / 32; }
  bool complete() const { return machine_.can_finish(); }
  bool in_call() const { return machine_.in_call(); }
  int calls() const { return machine_.calls(); }
  const std::vector<uint32_t>& mask() {
    const std::string sig = machine_.unconstrained() ? std::string("*") : machine_.signature();
    auto it = cache_->find(sig);
    if (it != cache_->end()) return it->second;
    std::vector<uint32_t> m(words(), 0u);
    const size_t n = tokens_->size();
    for (size_t i = 0; i < n; ++i) {
      const std::string& b = (*tokens_)[i];
      if (b.empty()) continue;
      // free text: a token without '<' cannot touch the opening tag
      if (machine_.unconstrained() && b.find('<') == std::string::npos) { m[i >> 5] |= 1u << (i & 31); continue; }
      ToolCallMachine trial = machine_;
      if (trial.feed(b)) m[i >> 5] |= 1u << (i & 31);
    }
    if (machine_.can_finish())
      for (int32_t e : eos_)
        if (e >= 0 && static_cast<size_t>(e) < n) m[e >> 5] |= 1u << (e & 31);
    if (cache_->size() > 4096) cache_->clear();
    return cache_->emplace(sig, std::move(m)).first->second;
  }
  bool accept(int32_t token) {
    for (int32_t e : eos_)
      if (e == token) return machine_.can_finish();
    if (token < 0 || static_cast<size_t>(token) >= tokens_->size()) return false;
    const std::string& b = (*tokens_)[token];
    if (b.empty()) return false;
    return machine_.feed(b);
  }

 private:
  ToolCallMachine machine_;
  std::shared_ptr<const std::vector<std::string>> tokens_;
  std::vector<int32_t> eos_;
  std::shared_ptr<std::unordered_map<std::string, std::vector<uint32_t>>> cache_;
};

}  // namespace grammar
}  // namespace dgpp
