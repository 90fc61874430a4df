// Small JSON DOM: strict parser (UTF-8, \uXXXX with surrogate pairs, duplicate-key detection on
// request) and a compact emitter.  Used by the tokenizer / chat-template loaders, the config
// parser, the safetensors header reader and the HTTP service.
// (same role as src/loaders/minijson.hpp of the reference.)
#pragma once
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace dgpp {
namespace json {

struct ParseError : std::runtime_error {
  size_t offset;
  ParseError(const std::string& m, size_t off) : std::runtime_error(m + " at byte " + std::to_string(off)), offset(off) {}
};

class Value;
typedef std::vector<std::pair<std::string, Value>> Members;  // insertion-ordered object

class Value {
 public:
  enum Type { Null, Bool, Int, Double, String, Array, Object };
  Value() : type_(Null) {}
  Value(std::nullptr_t) : type_(Null) {}
  Value(bool b) : type_(Bool), b_(b) {}
  Value(int v) : type_(Int), i_(v) {}
  Value(int64_t v) : type_(Int), i_(v) {}
  Value(uint64_t v) : type_(Int), i_(static_cast<int64_t>(v)) {}
  Value(double v) : type_(Double), d_(v) {}
  Value(const char* s) : type_(String), s_(s) {}
  Value(const std::string& s) : type_(String), s_(s) {}
  Value(std::string&& s) : type_(String), s_(std::move(s)) {}
  static Value array() { Value v; v.type_ = Array; return v; }
  static Value object() { Value v; v.type_ = Object; return v; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Null; }
  bool is_bool() const { return type_ == Bool; }
  bool is_int() const { return type_ == Int; }
  bool is_number() const { return type_ == Int || type_ == Double; }
  bool is_string() const { return type_ == String; }
  bool is_array() const { return type_ == Array; }
  bool is_object() const { return type_ == Object; }

  bool as_bool() const { need(Bool); return b_; }
  int64_t as_int() const {
    if (type_ == Double && std::floor(d_) == d_) return static_cast<int64_t>(d_);
    need(Int);
    return i_;
  }
  double as_double() const {
    if (type_ == Int) return static_cast<double>(i_);
    need(Double);
    return d_;
  }
  const std::string& as_string() const { need(String); return s_; }
  const std::vector<Value>& items() const { need(Array); return a_; }
  std::vector<Value>& items() { need(Array); return a_; }
  const Members& members() const { need(Object); return o_; }
  Members& members() { need(Object); return o_; }
  size_t size() const { return type_ == Array ? a_.size() : (type_ == Object ? o_.size() : 0); }

  const Value* find(const std::string& key) const {
    if (type_ != Object) return nullptr;
    for (const auto& kv : o_)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  Value* find(const std::string& key) {
    return const_cast<Value*>(static_cast<const Value*>(this)->find(key));
  }
  bool has(const std::string& key) const { return find(key) != nullptr; }
  const Value& at(const std::string& key) const {
    const Value* v = find(key);
    if (!v) throw std::runtime_error("missing key '" + key + "'");
    return *v;
  }
  const Value& at(size_t i) const { need(Array); return a_.at(i); }
  Value& set(const std::string& key, Value v) {
    if (type_ == Null) type_ = Object;
    need(Object);
    for (auto& kv : o_)
      if (kv.first == key) { kv.second = std::move(v); return kv.second; }
    o_.emplace_back(key, std::move(v));
    return o_.back().second;
  }
  void push(Value v) {
    if (type_ == Null) type_ = Array;
    need(Array);
    a_.push_back(std::move(v));
  }
  // typed getters with defaults
  std::string get_string(const std::string& k, const std::string& d = "") const {
    const Value* v = find(k);
    return v && v->is_string() ? v->s_ : d;
  }
  int64_t get_int(const std::string& k, int64_t d = 0) const {
    const Value* v = find(k);
    return v && v->is_number() ? v->as_int() : d;
  }
  double get_double(const std::string& k, double d = 0) const {
    const Value* v = find(k);
    return v && v->is_number() ? v->as_double() : d;
  }
  bool get_bool(const std::string& k, bool d = false) const {
    const Value* v = find(k);
    return v && v->is_bool() ? v->b_ : d;
  }
  bool operator==(const Value& o) const {
    if (type_ != o.type_) {
      if (is_number() && o.is_number()) return as_double() == o.as_double();
      return false;
    }
    switch (type_) {
      case Null: return true;
      case Bool: return b_ == o.b_;
      case Int: return i_ == o.i_;
      case Double: return d_ == o.d_;
      case String: return s_ == o.s_;
      case Array: return a_ == o.a_;
      case Object: return o_ == o.o_;
    }
    return false;
  }
  bool operator!=(const Value& o) const { return !(*this == o); }

  std::string dump(int indent = -1) const {
    std::string out;
    dump_to(out, indent, 0);
    return out;
  }
  void dump_to(std::string& out, int indent = -1, int depth = 0) const;

 private:
  void need(Type t) const {
    if (type_ != t) throw std::runtime_error(std::string("json: expected ") + name(t) + ", have " + name(type_));
  }
  static const char* name(Type t) {
    static const char* n[] = {"null", "bool", "int", "double", "string", "array", "object"};
    return n[t];
  }
  Type type_;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  std::vector<Value> a_;
  Members o_;
};

inline void escape_to(std::string& out, const std::string& s, bool ensure_ascii = false) {
  out.push_back('"');
  for (size_t i = 0; i < s.size(); ++i) {
    unsigned char c = static_cast<unsigned char>(s[i]);
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      case '\b': out += "\\b"; break;
      case '\f': out += "\\f"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else if (ensure_ascii && c >= 0x80) {
          // decode one UTF-8 sequence
          uint32_t cp = 0;
          int n = (c >= 0xF0) ? 3 : (c >= 0xE0) ? 2 : (c >= 0xC0) ? 1 : 0;
          cp = n == 3 ? (c & 7) : n == 2 ? (c & 15) : n == 1 ? (c & 31) : c;
          for (int k = 0; k < n && i + 1 < s.size(); ++k) cp = (cp << 6) | (static_cast<unsigned char>(s[++i]) & 63);
          char buf[16];
          if (cp >= 0x10000) {
            cp -= 0x10000;
            snprintf(buf, sizeof(buf), "\\u%04x\\u%04x", 0xD800 + (cp >> 10), 0xDC00 + (cp & 0x3FF));
          } else {
            snprintf(buf, sizeof(buf), "\\u%04x", cp);
          }
          out += buf;
        } else {
          out.push_back(static_cast<char>(c));
        }
    }
  }
  out.push_back('"');
}

inline void Value::dump_to(std::string& out, int indent, int depth) const {
  auto nl = [&](int d) {
    if (indent >= 0) {
      out.push_back('\n');
      out.append(static_cast<size_t>(indent * d), ' ');
    }
  };
  switch (type_) {
    case Null: out += "null"; break;
    case Bool: out += b_ ? "true" : "false"; break;
    case Int: out += std::to_string(i_); break;
    case Double: {
      if (!std::isfinite(d_)) { out += "null"; break; }
      char buf[40];
      snprintf(buf, sizeof(buf), "%.17g", d_);
      // prefer the shortest representation that round-trips
      for (int p = 1; p < 17; ++p) {
        char b2[40];
        snprintf(b2, sizeof(b2), "%.*g", p, d_);
        if (strtod(b2, nullptr) == d_) { snprintf(buf, sizeof(buf), "%s", b2); break; }
      }
      out += buf;
      bool has_dot = false;
      for (const char* p = buf; *p; ++p)
        if (*p == '.' || *p == 'e' || *p == 'E' || *p == 'n' || *p == 'i') has_dot = true;
      if (!has_dot) out += ".0";
      break;
    }
    case String: escape_to(out, s_); break;
    case Array:
      out.push_back('[');
      for (size_t i = 0; i < a_.size(); ++i) {
        if (i) out.push_back(',');
        nl(depth + 1);
        a_[i].dump_to(out, indent, depth + 1);
      }
      if (!a_.empty()) nl(depth);
      out.push_back(']');
      break;
    case Object:
      out.push_back('{');
      for (size_t i = 0; i < o_.size(); ++i) {
        if (i) out.push_back(',');
        nl(depth + 1);
        escape_to(out, o_[i].first);
        out.push_back(':');
        if (indent >= 0) out.push_back(' ');
        o_[i].second.dump_to(out, indent, depth + 1);
      }
      if (!o_.empty()) nl(depth);
      out.push_back('}');
      break;
  }
}

class Parser {
 public:
  Parser(const char* p, size_t n, bool reject_duplicates) : p_(p), n_(n), dup_(reject_duplicates) {}
  Value parse_document() {
    ws();
    Value v = parse_value(0);
    ws();
    if (i_ != n_) fail("trailing characters");
    return v;
  }

 private:
  [[noreturn]] void fail(const std::string& m) { throw ParseError("json: " + m, i_); }
  void ws() {
    while (i_ < n_ && (p_[i_] == ' ' || p_[i_] == '\t' || p_[i_] == '\n' || p_[i_] == '\r')) ++i_;
  }
  Value parse_value(int depth) {
    if (depth > 256) fail("nesting too deep");
    if (i_ >= n_) fail("unexpected end");
    char c = p_[i_];
    if (c == '{') return parse_object(depth);
    if (c == '[') return parse_array(depth);
    if (c == '"') return Value(parse_string());
    if (c == 't') { lit("true"); return Value(true); }
    if (c == 'f') { lit("false"); return Value(false); }
    if (c == 'n') { lit("null"); return Value(); }
    return parse_number();
  }
  void lit(const char* s) {
    size_t l = strlen_(s);
    if (i_ + l > n_ || std::string(p_ + i_, l) != s) fail("bad literal");
    i_ += l;
  }
  static size_t strlen_(const char* s) { size_t l = 0; while (s[l]) ++l; return l; }
  Value parse_number() {
    size_t s = i_;
    bool is_double = false;
    if (i_ < n_ && p_[i_] == '-') ++i_;
    if (i_ >= n_ || !(p_[i_] >= '0' && p_[i_] <= '9')) fail("bad number");
    if (p_[i_] == '0') { ++i_; } else { while (i_ < n_ && p_[i_] >= '0' && p_[i_] <= '9') ++i_; }
    if (i_ < n_ && p_[i_] == '.') {
      is_double = true;
      ++i_;
      if (i_ >= n_ || !(p_[i_] >= '0' && p_[i_] <= '9')) fail("bad fraction");
      while (i_ < n_ && p_[i_] >= '0' && p_[i_] <= '9') ++i_;
    }
    if (i_ < n_ && (p_[i_] == 'e' || p_[i_] == 'E')) {
      is_double = true;
      ++i_;
      if (i_ < n_ && (p_[i_] == '+' || p_[i_] == '-')) ++i_;
      if (i_ >= n_ || !(p_[i_] >= '0' && p_[i_] <= '9')) fail("bad exponent");
      while (i_ < n_ && p_[i_] >= '0' && p_[i_] <= '9') ++i_;
    }
    std::string t(p_ + s, i_ - s);
    if (!is_double) {
      errno = 0;
      char* end = nullptr;
      long long v = strtoll(t.c_str(), &end, 10);
      if (errno == 0 && end && *end == 0) return Value(static_cast<int64_t>(v));
    }
    return Value(strtod(t.c_str(), nullptr));
  }
  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 63))); }
    else if (cp < 0x10000) {
      out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 63)));
      out.push_back(static_cast<char>(0x80 | (cp & 63)));
    } else {
      out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 63)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 63)));
      out.push_back(static_cast<char>(0x80 | (cp & 63)));
    }
  }
  uint32_t hex4() {
    if (i_ + 4 > n_) fail("bad \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      char c = p_[i_++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string parse_string() {
    ++i_;  // opening quote
    std::string out;
    for (;;) {
      if (i_ >= n_) fail("unterminated string");
      unsigned char c = static_cast<unsigned char>(p_[i_++]);
      if (c == '"') break;
      if (c < 0x20) fail("control character in string");
      if (c != '\\') { out.push_back(static_cast<char>(c)); continue; }
      if (i_ >= n_) fail("bad escape");
      char e = p_[i_++];
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF) {
            if (i_ + 2 <= n_ && p_[i_] == '\\' && p_[i_ + 1] == 'u') {
              i_ += 2;
              uint32_t lo = hex4();
              if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
              else { utf8(out, 0xFFFD); cp = lo; }
            } else {
              cp = 0xFFFD;
            }
          } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
            cp = 0xFFFD;
          }
          utf8(out, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
    return out;
  }
  Value parse_array(int depth) {
    ++i_;
    Value v = Value::array();
    ws();
    if (i_ < n_ && p_[i_] == ']') { ++i_; return v; }
    for (;;) {
      ws();
      v.push(parse_value(depth + 1));
      ws();
      if (i_ >= n_) fail("unterminated array");
      if (p_[i_] == ',') { ++i_; continue; }
      if (p_[i_] == ']') { ++i_; break; }
      fail("expected , or ]");
    }
    return v;
  }
  Value parse_object(int depth) {
    ++i_;
    Value v = Value::object();
    ws();
    if (i_ < n_ && p_[i_] == '}') { ++i_; return v; }
    for (;;) {
      ws();
      if (i_ >= n_ || p_[i_] != '"') fail("expected string key");
      std::string k = parse_string();
      ws();
      if (i_ >= n_ || p_[i_] != ':') fail("expected :");
      ++i_;
      ws();
      Value item = parse_value(depth + 1);
      if (dup_ && v.has(k)) fail("duplicate key '" + k + "'");
      v.members().emplace_back(std::move(k), std::move(item));
      ws();
      if (i_ >= n_) fail("unterminated object");
      if (p_[i_] == ',') { ++i_; continue; }
      if (p_[i_] == '}') { ++i_; break; }
      fail("expected , or }");
    }
    return v;
  }
  const char* p_;
  size_t n_;
  size_t i_ = 0;
  bool dup_;
};

inline Value parse(const std::string& s, bool reject_duplicates = false) {
  return Parser(s.data(), s.size(), reject_duplicates).parse_document();
}
inline Value parse(const char* p, size_t n, bool reject_duplicates = false) {
  return Parser(p, n, reject_duplicates).parse_document();
}

}  // namespace json
}  // namespace dgpp
