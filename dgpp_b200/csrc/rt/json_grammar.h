// Constrained decoding of JSON: a byte-level pushdown machine that accepts exactly the texts that are valid JSON
// (response_format json_object) or valid instances of a JSON-schema subset (json_schema), and the per-step token
// masks derived from it.
//
// Schema subset: type (object / array / string / number / integer / boolean / null, or a list of them),
// properties + required + additionalProperties (default true), items, minItems / maxItems, enum, const.
// Unknown keywords are ignored; a schema that uses anyOf / oneOf / allOf / $ref / pattern is rejected at compile
// time so that the caller can answer 400 instead of producing unconstrained text.
// Whitespace between tokens is limited to 4 consecutive blanks (a model cannot stall in whitespace).
// The machine is a value type: a trial run for a candidate token is a copy + a few byte steps.
// Masks are cached per machine signature (most steps revisit states such as "inside a string value").
// (reference counterparts: src/text/json_grammar.cpp JsonLexer / JsonSchema / JsonMachine / JsonTables.)
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "rt/json.h"
#include "rt/string_constraint.h"

namespace dgpp {
namespace grammar {

enum TypeBit { kObject = 1, kArray = 2, kString = 4, kNumber = 8, kInteger = 16, kBool = 32, kNull = 64, kAny = 127 };

struct SchemaNode {
  int types = kAny;
  std::vector<std::pair<std::string, int>> properties;   // name -> node index
  std::set<std::string> required;
  bool additional = true;
  int items = -1;                                         // node index or -1: any
  int64_t min_items = 0, max_items = -1;
  std::vector<std::string> literals;                      // enum / const, serialised JSON texts
  int str = -1;                                           // index of the string-body constraint (lengths, pattern, format)
  int64_t multiple_of = 0;                                // integer nodes: the value must be a multiple of this (0: off)
};

class Schema {
 public:
  Schema() { nodes_.push_back(SchemaNode()); }            // node 0: anything
  static Schema any_object() {
    Schema s;
    SchemaNode n;
    n.types = kObject;
    s.nodes_.push_back(n);
    s.root_ = 1;
    return s;
  }
  static Schema compile(const json::Value& v) {
    Schema s;
    s.root_ = s.add(v, 0);
    return s;
  }
  const SchemaNode& node(int i) const { return nodes_[i]; }
  const StringConstraint& str(int i) const { return strs_[i]; }
  int root() const { return root_; }

 private:
  int add(const json::Value& v, int depth) {
    if (depth > 32) throw std::runtime_error("json_schema: nesting deeper than 32");
    if (v.is_bool()) {
      if (!v.as_bool()) throw std::runtime_error("json_schema: 'false' schemas are not supported");
      return 0;
    }
    if (!v.is_object()) throw std::runtime_error("json_schema: a schema must be an object");
    for (const char* bad : {"anyOf", "oneOf", "allOf", "not", "$ref", "patternProperties", "if"})
      if (v.has(bad)) throw std::runtime_error(std::string("json_schema: keyword '") + bad + "' is not supported");
    SchemaNode n;
    if (const json::Value* t = v.find("type")) {
      n.types = 0;
      auto one = [&](const std::string& name) {
        if (name == "object") n.types |= kObject;
        else if (name == "array") n.types |= kArray;
        else if (name == "string") n.types |= kString;
        else if (name == "number") n.types |= kNumber | kInteger;
        else if (name == "integer") n.types |= kInteger;
        else if (name == "boolean") n.types |= kBool;
        else if (name == "null") n.types |= kNull;
        else throw std::runtime_error("json_schema: unknown type '" + name + "'");
      };
      if (t->is_string()) one(t->as_string());
      else if (t->is_array()) for (const auto& x : t->items()) one(x.as_string());
      else throw std::runtime_error("json_schema: 'type' must be a string or a list");
    } else if (v.has("properties") || v.has("required")) {
      n.types = kObject;
    } else if (v.has("items")) {
      n.types = kArray;
    }
    if (const json::Value* e = v.find("enum")) {
      if (!e->is_array() || e->size() == 0) throw std::runtime_error("json_schema: 'enum' must be a non-empty list");
      for (const auto& x : e->items()) n.literals.push_back(x.dump());
    }
    if (const json::Value* c = v.find("const")) n.literals.push_back(c->dump());
    if (n.literals.empty() && (n.types & kString) && (v.has("pattern") || v.has("minLength") || v.has("maxLength") || v.has("format"))) {
      std::string pat = v.get_string("pattern");
      if (pat.empty()) pat = StringConstraint::format_pattern(v.get_string("format"));   // unknown formats are annotations
      const int64_t lo = v.get_int("minLength", 0), hi = v.get_int("maxLength", -1);
      if (hi >= 0 && hi < lo) throw std::runtime_error("json_schema: maxLength below minLength");
      if (!pat.empty() || lo > 0 || hi >= 0) {
        try {
          strs_.push_back(StringConstraint::compile(pat, lo, hi));
        } catch (const std::runtime_error& e) {
          throw std::runtime_error(std::string("json_schema: ") + e.what());
        }
        n.str = static_cast<int>(strs_.size()) - 1;
      }
    }
    const int idx = static_cast<int>(nodes_.size());
    nodes_.push_back(n);
    if (const json::Value* p = v.find("properties")) {
      if (!p->is_object()) throw std::runtime_error("json_schema: 'properties' must be an object");
      for (const auto& kv : p->members()) {
        const int child = add(kv.second, depth + 1);
        nodes_[idx].properties.emplace_back(kv.first, child);
      }
    }
    if (const json::Value* r = v.find("required"))
      for (const auto& x : r->items()) nodes_[idx].required.insert(x.as_string());
    if (const json::Value* a = v.find("additionalProperties")) {
      if (a->is_bool()) nodes_[idx].additional = a->as_bool();
      else throw std::runtime_error("json_schema: 'additionalProperties' must be a boolean");
    }
    if (const json::Value* it = v.find("items")) nodes_[idx].items = add(*it, depth + 1);
    if (const json::Value* m = v.find("multipleOf")) {
      // supported where it can be enforced while the digits are written: integer values, integer divisor
      const double d = m->as_double();
      const int t = nodes_[idx].types;
      if (!((t & kInteger) && !(t & kNumber)) || d < 1 || d != static_cast<double>(static_cast<int64_t>(d)) || d > 1e15)
        throw std::runtime_error("json_schema: 'multipleOf' is supported for integer values with a positive integer divisor");
      nodes_[idx].multiple_of = static_cast<int64_t>(d);
    }
    nodes_[idx].min_items = v.get_int("minItems", 0);
    nodes_[idx].max_items = v.get_int("maxItems", -1);
    for (const auto& r : nodes_[idx].required) {
      bool known = nodes_[idx].additional;
      for (const auto& p : nodes_[idx].properties) known = known || p.first == r;
      if (!known) throw std::runtime_error("json_schema: required property '" + r + "' can never be written");
    }
    return idx;
  }
  std::vector<SchemaNode> nodes_;
  std::vector<StringConstraint> strs_;
  int root_ = 0;
};

// One level of the pushdown stack.
struct Frame {
  enum Kind : uint8_t { Value, ObjFirst, ObjKey, ObjColon, ObjValueDone, ArrFirst, ArrValueDone, Str, Num, Lit, Choice };
  Kind kind = Value;
  int node = 0;          // schema node of the value / container
  uint8_t sub = 0;       // Str: 0 body, 1 after backslash, 2..5 hex digits left + 1; Num: lexer state; Lit / Choice: offset
  bool is_key = false;   // Str: this string is an object key
  int count = 0;         // Arr: items so far; Choice: candidate bitmask; Lit: which literal (0 true, 1 false, 2 null)
  std::string text;      // ObjKey..ObjValueDone: '\n'-joined keys seen; Str key: key bytes so far (raw, unescaped only)
  int64_t aux = 0;       // Num under multipleOf: the digits so far modulo the divisor
};

class Machine {
 public:
  explicit Machine(std::shared_ptr<const Schema> schema) : schema_(std::move(schema)) {
    Frame f;
    f.kind = Frame::Value;
    f.node = schema_->root();
    stack_.push_back(f);
  }
  bool done() const { return stack_.empty(); }              // a complete top-level value has been read
  // A value is also complete when the only open frame is a number / choice that may end here.
  bool can_finish() const {
    if (stack_.empty()) return true;
    if (stack_.size() == 1) return ends_here(stack_.back());
    return false;
  }
  // Feeds one byte; false = the byte is not allowed here (the machine is then unusable).
  bool step(unsigned char c) {
    for (int guard = 0; guard < 8; ++guard) {
      if (stack_.empty()) {
        if (is_ws(c)) return ++ws_ <= 4;
        return false;
      }
      Frame& f = stack_.back();
      switch (f.kind) {
        case Frame::Value: return begin_value(c);
        case Frame::Str: return in_string(c);
        case Frame::Num:
          if (num_step(f, c)) return true;
          if (!num_final(f.sub) || (integer_only(f.node) && f.count) || !multiple_ok(f)) return false;
          stack_.pop_back();
          value_done();
          continue;                                          // re-dispatch c to the parent
        case Frame::Lit: {
          static const char* kLit[3] = {"true", "false", "null"};
          const char* s = kLit[f.count];
          if (s[f.sub] != static_cast<char>(c)) return false;
          if (s[++f.sub] == 0) { stack_.pop_back(); value_done(); }
          return true;
        }
        case Frame::Choice: {
          const auto& lits = schema_->node(f.node).literals;
          int next = 0;
          for (size_t i = 0; i < lits.size() && i < 31; ++i)
            if ((f.count >> i & 1) && f.sub < lits[i].size() && static_cast<unsigned char>(lits[i][f.sub]) == c) next |= 1 << i;
          if (next) { f.count = next; ++f.sub; ws_ = 0; return true; }
          if (!ends_here(f)) return false;
          stack_.pop_back();
          value_done();
          continue;
        }
        default: return between(c);
      }
    }
    return false;
  }
  bool feed(const std::string& bytes) {
    for (unsigned char c : bytes)
      if (!step(c)) return false;
    return true;
  }
  // Cache key: everything that decides the future.
  std::string signature() const {
    std::string s;
    s.push_back(static_cast<char>(ws_));
    for (const auto& f : stack_) {
      s.push_back(static_cast<char>(f.kind));
      s.append(reinterpret_cast<const char*>(&f.node), 4);
      s.push_back(static_cast<char>(f.sub));
      s.push_back(f.is_key ? 1 : 0);
      s.append(reinterpret_cast<const char*>(&f.count), 4);
      s.append(f.text);
      if (f.aux) s.append(reinterpret_cast<const char*>(&f.aux), 8);
      s.push_back('\x1f');
    }
    return s;
  }

 private:
  static bool is_ws(unsigned char c) { return c == ' ' || c == '\n' || c == '\t' || c == '\r'; }
  bool integer_only(int node) const {
    const int t = schema_->node(node).types;
    return (t & kInteger) && !(t & kNumber);
  }
  // Num lexer: 0 after '-', 1 after leading 0, 2 integer digits, 3 after '.', 4 fraction digits, 5 after e/E,
  // 6 after exponent sign, 7 exponent digits.  f.count = 1 once a '.', 'e' or 'E' was seen.
  static bool num_final(uint8_t s) { return s == 1 || s == 2 || s == 4 || s == 7; }
  bool multiple_ok(const Frame& f) const { return schema_->node(f.node).multiple_of <= 0 || f.aux == 0; }
  bool num_step(Frame& f, unsigned char c) {
    const bool digit = c >= '0' && c <= '9';
    const int64_t mo = schema_->node(f.node).multiple_of;
    if (mo > 0 && digit && (f.sub == 0 || f.sub == 2)) f.aux = (f.aux * 10 + (c - '0')) % mo;   // integer digits only
    switch (f.sub) {
      case 0: if (c == '0') { f.sub = 1; return true; } if (digit) { f.sub = 2; return true; } return false;
      case 1: break;
      case 2: if (digit) return true; break;
      case 3: if (digit) { f.sub = 4; return true; } return false;
      case 4: if (digit) return true; if (c == 'e' || c == 'E') { f.sub = 5; return true; } return false;
      case 5: if (c == '+' || c == '-') { f.sub = 6; return true; } if (digit) { f.sub = 7; return true; } return false;
      case 6: if (digit) { f.sub = 7; return true; } return false;
      case 7: return digit;
    }
    // states 1 and 2: fraction or exponent may follow
    if (integer_only(f.node)) return false;
    if (c == '.') { f.sub = 3; f.count = 1; return true; }
    if (c == 'e' || c == 'E') { f.sub = 5; f.count = 1; return true; }
    return false;
  }
  bool ends_here(const Frame& f) const {
    if (f.kind == Frame::Num) return num_final(f.sub) && multiple_ok(f);
    if (f.kind == Frame::Choice) {
      const auto& lits = schema_->node(f.node).literals;
      for (size_t i = 0; i < lits.size() && i < 31; ++i)
        if ((f.count >> i & 1) && lits[i].size() == f.sub) return true;
    }
    return false;
  }
  bool begin_value(unsigned char c) {
    if (is_ws(c)) return ++ws_ <= 4;
    ws_ = 0;
    Frame& f = stack_.back();
    const SchemaNode& n = schema_->node(f.node);
    if (!n.literals.empty()) {
      f.kind = Frame::Choice;
      f.sub = 0;
      f.count = static_cast<int>((1u << (n.literals.size() < 31 ? n.literals.size() : 31)) - 1);
      return step(c);
    }
    const int t = n.types;
    if (c == '{' && (t & kObject)) { f.kind = Frame::ObjFirst; f.text.clear(); return true; }
    if (c == '[' && (t & kArray)) { f.kind = Frame::ArrFirst; f.count = 0; return true; }
    if (c == '"' && (t & kString)) {
      f.kind = Frame::Str; f.sub = 0; f.is_key = false; f.count = 0;
      f.text = n.str >= 0 ? schema_->str(n.str).initial() : std::string();
      return true;
    }
    if ((c == '-' || (c >= '0' && c <= '9')) && (t & (kNumber | kInteger))) {
      f.kind = Frame::Num;
      f.count = 0;
      f.sub = c == '-' ? 0 : (c == '0' ? 1 : 2);
      f.aux = (n.multiple_of > 0 && c > '0' && c <= '9') ? (c - '0') % n.multiple_of : 0;
      return true;
    }
    if ((c == 't' || c == 'f') && (t & kBool)) { f.kind = Frame::Lit; f.count = c == 't' ? 0 : 1; f.sub = 1; return true; }
    if (c == 'n' && (t & kNull)) { f.kind = Frame::Lit; f.count = 2; f.sub = 1; return true; }
    return false;
  }
  // One decoded character byte of a constrained string value: length limits (in code points) and the pattern NFA.
  bool body_byte(Frame& f, const StringConstraint& sc, unsigned char c) {
    if ((c & 0xC0) != 0x80) {
      if (sc.max_len >= 0 && f.count + 1 > sc.max_len) return false;
      ++f.count;
    }
    return sc.step(f.text, c);
  }
  bool in_string(unsigned char c) {
    Frame& f = stack_.back();
    const int sci = f.is_key ? -1 : schema_->node(f.node).str;
    if (f.sub == 1) {                                       // after a backslash
      if (c == 'u') {
        if (sci >= 0) return false;                         // constrained bodies take the character itself
        f.sub = 5;
        return !f.is_key || key_free();
      }
      static const std::string esc = "\"\\/bfnrt";
      const size_t which = esc.find(static_cast<char>(c));
      if (which == std::string::npos) return false;
      f.sub = 0;
      if (sci >= 0) {
        static const char decoded[] = {'"', '\\', '/', '\b', '\f', '\n', '\r', '\t'};
        return body_byte(f, schema_->str(sci), static_cast<unsigned char>(decoded[which]));
      }
      return !f.is_key || key_free();                       // escaped keys only where any key is allowed
    }
    if (f.sub >= 2) {                                       // hex digits of \uXXXX
      const bool hex = (c >= '0' && c <= '9') || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F');
      if (!hex) return false;
      f.sub = f.sub == 2 ? 0 : f.sub - 1;
      return true;
    }
    if (c == '\\') {
      if (sci >= 0) {
        // a backslash is viable only if one of the escapes it can start is
        const StringConstraint& sc = schema_->str(sci);
        bool any = false;
        for (unsigned char d : {'"', '\\', '/', '\b', '\f', '\n', '\r', '\t'}) {
          Frame trial = f;
          if (body_byte(trial, sc, d)) { any = true; break; }
        }
        if (!any) return false;
      }
      f.sub = 1;
      return true;
    }
    if (c < 0x20) return false;
    if (c == '"') {
      if (f.is_key) {
        const std::string key = f.text;
        stack_.pop_back();
        Frame& obj = stack_.back();
        if (!key_allowed(obj, key, /*complete=*/true)) return false;
        obj.text += key;
        obj.text.push_back('\n');
        obj.kind = Frame::ObjColon;
        return true;
      }
      if (sci >= 0) {
        const StringConstraint& sc = schema_->str(sci);
        if (f.count < sc.min_len || !sc.accepting(f.text)) return false;
      }
      stack_.pop_back();
      value_done();
      return true;
    }
    if (f.is_key) {
      f.text.push_back(static_cast<char>(c));
      return key_allowed(stack_[stack_.size() - 2], f.text, /*complete=*/false);
    }
    if (sci >= 0) return body_byte(f, schema_->str(sci), c);
    return true;
  }
  bool key_free() const { return schema_->node(stack_[stack_.size() - 2].node).additional; }
  static bool seen(const Frame& obj, const std::string& key) {
    size_t p = 0;
    while (p < obj.text.size()) {
      const size_t e = obj.text.find('\n', p);
      if (obj.text.compare(p, e - p, key) == 0 && e - p == key.size()) return true;
      p = e + 1;
    }
    return false;
  }
  bool key_allowed(const Frame& obj, const std::string& key, bool complete) const {
    const SchemaNode& n = schema_->node(obj.node);
    if (complete && seen(obj, key)) return false;           // duplicate keys are never produced
    if (n.additional) return true;
    for (const auto& p : n.properties) {
      if (complete ? p.first == key : p.first.compare(0, key.size(), key) == 0) {
        if (complete || !seen(obj, p.first)) return true;
      }
    }
    return false;
  }
  int child_node(const Frame& obj) const {
    // node of the value that follows the last key
    const size_t e = obj.text.size() - 1, b = obj.text.rfind('\n', e - 1);
    const std::string key = obj.text.substr(b == std::string::npos ? 0 : b + 1, e - (b == std::string::npos ? 0 : b + 1));
    for (const auto& p : schema_->node(obj.node).properties)
      if (p.first == key) return p.second;
    return 0;
  }
  bool required_done(const Frame& obj) const {
    for (const auto& r : schema_->node(obj.node).required)
      if (!seen(obj, r)) return false;
    return true;
  }
  void value_done() {
    ws_ = 0;
    if (stack_.empty()) return;
    Frame& p = stack_.back();
    if (p.kind == Frame::ObjColon) p.kind = Frame::ObjValueDone;     // (set by push_value below)
    else if (p.kind == Frame::ArrFirst || p.kind == Frame::ArrValueDone) { p.kind = Frame::ArrValueDone; ++p.count; }
  }
  void push_value(int node) {
    Frame v;
    v.kind = Frame::Value;
    v.node = node;
    stack_.push_back(v);
  }
  bool between(unsigned char c) {
    if (is_ws(c)) return ++ws_ <= 4;
    ws_ = 0;
    Frame& f = stack_.back();
    const SchemaNode& n = schema_->node(f.node);
    switch (f.kind) {
      case Frame::ObjFirst:
      case Frame::ObjKey:
        if (c == '}' && f.kind == Frame::ObjFirst) {
          if (!required_done(f)) return false;
          stack_.pop_back();
          value_done();
          return true;
        }
        if (c == '"') {
          // a key may start only if some key is still possible
          bool any = n.additional;
          for (const auto& p : n.properties) any = any || !seen(f, p.first);
          if (!any) return false;
          Frame k;
          k.kind = Frame::Str;
          k.is_key = true;
          stack_.push_back(k);
          return true;
        }
        return false;
      case Frame::ObjColon:
        if (c != ':') return false;
        {
          const int child = child_node(f);
          push_value(child);                                 // parent stays ObjColon until the value completes
        }
        return true;
      case Frame::ObjValueDone:
        if (c == ',') {
          bool any = n.additional;
          for (const auto& p : n.properties) any = any || !seen(f, p.first);
          if (!any) return false;
          f.kind = Frame::ObjKey;
          return true;
        }
        if (c == '}') {
          if (!required_done(f)) return false;
          stack_.pop_back();
          value_done();
          return true;
        }
        return false;
      case Frame::ArrFirst:
        if (c == ']') {
          if (n.min_items > 0) return false;
          stack_.pop_back();
          value_done();
          return true;
        }
        if (n.max_items == 0) return false;
        push_value(n.items < 0 ? 0 : n.items);
        return step(c);
      case Frame::ArrValueDone:
        if (c == ',') {
          if (n.max_items >= 0 && f.count >= n.max_items) return false;
          push_value(n.items < 0 ? 0 : n.items);
          return true;
        }
        if (c == ']') {
          if (f.count < n.min_items) return false;
          stack_.pop_back();
          value_done();
          return true;
        }
        return false;
      default: return false;
    }
  }

  std::shared_ptr<const Schema> schema_;
  std::vector<Frame> stack_;
  int ws_ = 0;
};

// Token-level view: which vocabulary entries may come next.
class TokenGrammar {
 public:
  // token_bytes[i] = raw bytes of token i (empty = never allowed, e.g. special tokens); eos_ids are allowed
  // exactly when the value is complete.
  TokenGrammar(std::shared_ptr<const Schema> schema, std::shared_ptr<const std::vector<std::string>> token_bytes,
               std::vector<int32_t> eos_ids)
      : machine_(std::move(schema)), tokens_(std::move(token_bytes)), eos_(std::move(eos_ids)),
        cache_(std::make_shared<std::unordered_map<std::string, std::vector<uint32_t>>>()) {}

  size_t words() const { return (tokens_->size() + 31) / 32; }
  bool complete() const { return machine_.can_finish(); }
  const std::vector<uint32_t>& mask() {
    const std::string sig = machine_.signature();
    auto it = cache_->find(sig);
    if (it != cache_->end()) return it->second;
    std::vector<uint32_t> m(words(), 0u);
    const size_t n = tokens_->size();
    for (size_t i = 0; i < n; ++i) {
      const std::string& b = (*tokens_)[i];
      if (b.empty()) continue;
      Machine trial = machine_;
      if (trial.feed(b)) m[i >> 5] |= 1u << (i & 31);
    }
    if (machine_.can_finish())
      for (int32_t e : eos_)
        if (e >= 0 && static_cast<size_t>(e) < n) m[e >> 5] |= 1u << (e & 31);
    if (cache_->size() > 4096) cache_->clear();
    return cache_->emplace(sig, std::move(m)).first->second;
  }
  // Advances by a sampled token; false when the token was not allowed.
  bool accept(int32_t token) {
    for (int32_t e : eos_)
      if (e == token) return machine_.can_finish();
    if (token < 0 || static_cast<size_t>(token) >= tokens_->size()) return false;
    const std::string& b = (*tokens_)[token];
    if (b.empty()) return false;
    return machine_.feed(b);
  }

 private:
  Machine machine_;
  std::shared_ptr<const std::vector<std::string>> tokens_;
  std::vector<int32_t> eos_;
  std::shared_ptr<std::unordered_map<std::string, std::vector<uint32_t>>> cache_;
};

}  // namespace grammar
}  // namespace dgpp
