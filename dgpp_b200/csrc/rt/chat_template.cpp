#include "rt/chat_template.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <ctime>
#include <functional>
#include <map>
#include <sstream>
#include <vector>

namespace dgpp {
namespace {

// ====================================================================== values
struct Val;
typedef std::shared_ptr<Val> VP;
struct Macro;

struct Val {
  enum T { Undefined, None, Bool, Int, Float, Str, List, Dict, MacroT } t = Undefined;
  bool b = false;
  int64_t i = 0;
  double f = 0;
  std::string s;
  std::vector<VP> list;
  std::vector<std::pair<std::string, VP>> dict;  // insertion ordered; also used by namespace()
  std::shared_ptr<Macro> macro;
};

VP mk(Val::T t) { auto v = std::make_shared<Val>(); v->t = t; return v; }
VP mk_bool(bool b) { auto v = mk(Val::Bool); v->b = b; return v; }
VP mk_int(int64_t i) { auto v = mk(Val::Int); v->i = i; return v; }
VP mk_float(double f) { auto v = mk(Val::Float); v->f = f; return v; }
VP mk_str(std::string s) { auto v = mk(Val::Str); v->s = std::move(s); return v; }
VP undefined() { return mk(Val::Undefined); }
VP none() { return mk(Val::None); }

VP from_json(const json::Value& j) {
  switch (j.type()) {
    case json::Value::Null: return none();
    case json::Value::Bool: return mk_bool(j.as_bool());
    case json::Value::Int: return mk_int(j.as_int());
    case json::Value::Double: return mk_float(j.as_double());
    case json::Value::String: return mk_str(j.as_string());
    case json::Value::Array: {
      auto v = mk(Val::List);
      for (const auto& e : j.items()) v->list.push_back(from_json(e));
      return v;
    }
    case json::Value::Object: {
      auto v = mk(Val::Dict);
      for (const auto& kv : j.members()) v->dict.emplace_back(kv.first, from_json(kv.second));
      return v;
    }
  }
  return none();
}

json::Value to_json(const VP& v) {
  switch (v->t) {
    case Val::Undefined: case Val::None: case Val::MacroT: return json::Value();
    case Val::Bool: return json::Value(v->b);
    case Val::Int: return json::Value(v->i);
    case Val::Float: return json::Value(v->f);
    case Val::Str: return json::Value(v->s);
    case Val::List: {
      json::Value a = json::Value::array();
      for (const auto& e : v->list) a.push(to_json(e));
      return a;
    }
    case Val::Dict: {
      json::Value o = json::Value::object();
      for (const auto& kv : v->dict) o.set(kv.first, to_json(kv.second));
      return o;
    }
  }
  return json::Value();
}

bool truthy(const VP& v) {
  switch (v->t) {
    case Val::Undefined: case Val::None: return false;
    case Val::Bool: return v->b;
    case Val::Int: return v->i != 0;
    case Val::Float: return v->f != 0;
    case Val::Str: return !v->s.empty();
    case Val::List: return !v->list.empty();
    case Val::Dict: return !v->dict.empty();
    case Val::MacroT: return true;
  }
  return false;
}

std::string fmt_float(double f) {
  if (std::floor(f) == f && std::fabs(f) < 1e16) {
    std::ostringstream o;
    o << static_cast<int64_t>(f) << ".0";
    return o.str();
  }
  char buf[40];
  for (int p = 1; p <= 17; ++p) {
    snprintf(buf, sizeof(buf), "%.*g", p, f);
    if (strtod(buf, nullptr) == f) break;
  }
  return buf;
}

// python-style tojson with ", " and ": " separators (what transformers' tojson filter prints)
void py_json(const VP& v, std::string& out, int indent, int depth) {
  auto nl = [&](int d) {
    if (indent > 0) { out.push_back('\n'); out.append(static_cast<size_t>(indent * d), ' '); }
  };
  switch (v->t) {
    case Val::Undefined: case Val::None: case Val::MacroT: out += "null"; break;
    case Val::Bool: out += v->b ? "true" : "false"; break;
    case Val::Int: out += std::to_string(v->i); break;
    case Val::Float: out += fmt_float(v->f); break;
    case Val::Str: json::escape_to(out, v->s); break;
    case Val::List:
      out.push_back('[');
      for (size_t k = 0; k < v->list.size(); ++k) {
        if (k) out += indent > 0 ? "," : ", ";
        nl(depth + 1);
        py_json(v->list[k], out, indent, depth + 1);
      }
      if (!v->list.empty()) nl(depth);
      out.push_back(']');
      break;
    case Val::Dict:
      out.push_back('{');
      for (size_t k = 0; k < v->dict.size(); ++k) {
        if (k) out += indent > 0 ? "," : ", ";
        nl(depth + 1);
        json::escape_to(out, v->dict[k].first);
        out += ": ";
        py_json(v->dict[k].second, out, indent, depth + 1);
      }
      if (!v->dict.empty()) nl(depth);
      out.push_back('}');
      break;
  }
}

std::string repr(const VP& v);
std::string to_text(const VP& v) {
  switch (v->t) {
    case Val::Undefined: return "";
    case Val::None: return "None";
    case Val::Bool: return v->b ? "True" : "False";
    case Val::Int: return std::to_string(v->i);
    case Val::Float: return fmt_float(v->f);
    case Val::Str: return v->s;
    case Val::List: case Val::Dict: return repr(v);
    case Val::MacroT: return "<macro>";
  }
  return "";
}
std::string repr(const VP& v) {
  if (v->t == Val::Str) {
    std::string o = "'";
    for (char c : v->s) {
      if (c == '\'' || c == '\\') o.push_back('\\');
      if (c == '\n') { o += "\\n"; continue; }
      o.push_back(c);
    }
    return o + "'";
  }
  if (v->t == Val::List) {
    std::string o = "[";
    for (size_t k = 0; k < v->list.size(); ++k) { if (k) o += ", "; o += repr(v->list[k]); }
    return o + "]";
  }
  if (v->t == Val::Dict) {
    std::string o = "{";
    for (size_t k = 0; k < v->dict.size(); ++k) {
      if (k) o += ", ";
      o += "'" + v->dict[k].first + "': " + repr(v->dict[k].second);
    }
    return o + "}";
  }
  return to_text(v);
}

VP dict_get(const VP& d, const std::string& k) {
  for (const auto& kv : d->dict)
    if (kv.first == k) return kv.second;
  return nullptr;
}
void dict_set(const VP& d, const std::string& k, VP v) {
  for (auto& kv : d->dict)
    if (kv.first == k) { kv.second = std::move(v); return; }
  d->dict.emplace_back(k, std::move(v));
}

bool is_num(const VP& v) { return v->t == Val::Int || v->t == Val::Float || v->t == Val::Bool; }
double num(const VP& v) { return v->t == Val::Float ? v->f : (v->t == Val::Bool ? (v->b ? 1.0 : 0.0) : static_cast<double>(v->i)); }

bool equals(const VP& a, const VP& b) {
  if (is_num(a) && is_num(b)) return num(a) == num(b);
  if (a->t != b->t) {
    const bool an = a->t == Val::None || a->t == Val::Undefined, bn = b->t == Val::None || b->t == Val::Undefined;
    return an && bn && a->t == b->t;
  }
  switch (a->t) {
    case Val::Str: return a->s == b->s;
    case Val::List:
      if (a->list.size() != b->list.size()) return false;
      for (size_t k = 0; k < a->list.size(); ++k) if (!equals(a->list[k], b->list[k])) return false;
      return true;
    case Val::Dict:
      if (a->dict.size() != b->dict.size()) return false;
      for (const auto& kv : a->dict) { VP o = dict_get(b, kv.first); if (!o || !equals(kv.second, o)) return false; }
      return true;
    default: return true;
  }
}

// ====================================================================== lexer
enum Tok { T_EOF, T_NAME, T_INT, T_FLOAT, T_STR, T_OP };
struct Token { Tok t; std::string s; size_t pos; };

struct ExprLexer {
  const std::string& src;
  size_t i, end;
  ExprLexer(const std::string& s, size_t b, size_t e) : src(s), i(b), end(e) {}
  [[noreturn]] void fail(const std::string& m, size_t at) const {
    throw TemplateError("template: " + m + " at byte " + std::to_string(at));
  }
  Token next() {
    while (i < end && isspace(static_cast<unsigned char>(src[i]))) ++i;
    if (i >= end) return {T_EOF, "", i};
    const size_t p = i;
    const char c = src[i];
    if (isalpha(static_cast<unsigned char>(c)) || c == '_') {
      while (i < end && (isalnum(static_cast<unsigned char>(src[i])) || src[i] == '_')) ++i;
      return {T_NAME, src.substr(p, i - p), p};
    }
    if (isdigit(static_cast<unsigned char>(c))) {
      bool fl = false;
      while (i < end && (isdigit(static_cast<unsigned char>(src[i])) || src[i] == '_')) ++i;
      if (i + 1 < end && src[i] == '.' && isdigit(static_cast<unsigned char>(src[i + 1]))) {
        fl = true; ++i;
        while (i < end && isdigit(static_cast<unsigned char>(src[i]))) ++i;
      }
      if (i < end && (src[i] == 'e' || src[i] == 'E')) {
        size_t k = i + 1;
        if (k < end && (src[k] == '+' || src[k] == '-')) ++k;
        if (k < end && isdigit(static_cast<unsigned char>(src[k]))) { fl = true; i = k; while (i < end && isdigit(static_cast<unsigned char>(src[i]))) ++i; }
      }
      std::string t = src.substr(p, i - p);
      t.erase(std::remove(t.begin(), t.end(), '_'), t.end());
      return {fl ? T_FLOAT : T_INT, t, p};
    }
    if (c == '"' || c == '\'') {
      ++i;
      std::string out;
      while (i < end && src[i] != c) {
        if (src[i] == '\\' && i + 1 < end) {
          const char e = src[i + 1];
          i += 2;
          switch (e) {
            case 'n': out.push_back('\n'); break;
            case 't': out.push_back('\t'); break;
            case 'r': out.push_back('\r'); break;
            case '\\': out.push_back('\\'); break;
            case '\'': out.push_back('\''); break;
            case '"': out.push_back('"'); break;
            default: out.push_back('\\'); out.push_back(e);
          }
        } else {
          out.push_back(src[i++]);
        }
      }
      if (i >= end) fail("unterminated string", p);
      ++i;
      return {T_STR, out, p};
    }
    static const char* two[] = {"==", "!=", "<=", ">=", "//", "**"};
    for (const char* o : two)
      if (i + 1 < end && src[i] == o[0] && src[i + 1] == o[1]) { i += 2; return {T_OP, o, p}; }
    ++i;
    return {T_OP, std::string(1, c), p};
  }
};

// ====================================================================== AST
struct Expr;
typedef std::shared_ptr<Expr> EP;
struct Expr {
  enum K { Lit, Name, Attr, Index, Slice, Call, Filter, Test, Unary, Binary, Cond, ListE, DictE } k;
  VP lit;
  std::string name;            // Name / Attr / Filter / Test / op
  EP a, b, c;                  // operands
  std::vector<EP> args;
  std::vector<std::pair<std::string, EP>> kwargs;
  std::vector<std::pair<EP, EP>> pairs;
  bool negate = false;
  size_t pos = 0;
};

struct Node;
typedef std::shared_ptr<Node> NP;
struct Node {
  enum K { Text, Output, If, For, Set, SetBlock, MacroDef, CallBlock, Break, Continue } k;
  std::string text;
  EP expr;                                  // Output / Set value / For iterable
  std::vector<std::pair<EP, std::vector<NP>>> branches;  // If: (cond or null, body)
  std::vector<std::string> targets;         // For loop vars / Set target / macro params
  std::string attr;                         // Set ns.attr
  EP filter_cond;                           // For ... if cond
  std::vector<NP> body, else_body;
  std::vector<std::pair<std::string, EP>> defaults;  // macro defaults
  bool recursive = false;
};

struct Macro {
  std::string name;
  std::vector<std::string> params;
  std::vector<std::pair<std::string, EP>> defaults;
  std::vector<NP> body;
};

// ====================================================================== parser
struct Piece { bool is_tag; bool is_expr; size_t b, e; std::string text; };

class Parser {
 public:
  explicit Parser(const std::string& src) : src_(src) { split(); }
  std::vector<NP> parse() {
    std::vector<NP> out = block({});
    if (pi_ < pieces_.size()) fail("unexpected tag", pieces_[pi_].b);
    return out;
  }

 private:
  [[noreturn]] void fail(const std::string& m, size_t at) const {
    throw TemplateError("template: " + m + " at byte " + std::to_string(at));
  }
  // Splits source into text / {{ }} / {% %} pieces applying {#..#} removal, '-' whitespace control,
  // trim_blocks (newline after a tag removed) and lstrip_blocks (indentation before a tag removed).
  void split() {
    size_t i = 0;
    std::string text;
    bool trim_next_newline = false, strip_next = false;
    auto flush_text = [&](bool rstrip, bool lstrip_line) {
      std::string t = text;
      text.clear();
      if (rstrip) {
        while (!t.empty() && isspace(static_cast<unsigned char>(t.back()))) t.pop_back();
      } else if (lstrip_line) {
        size_t k = t.size();
        while (k > 0 && (t[k - 1] == ' ' || t[k - 1] == '\t')) --k;
        if (k == 0 ? at_line_start_ : t[k - 1] == '\n') t.resize(k);
      }
      if (!t.empty()) {
        at_line_start_ = t.back() == '\n';
        pieces_.push_back({false, false, 0, 0, t});
      }
    };
    while (i < src_.size()) {
      if (src_[i] == '{' && i + 1 < src_.size() && (src_[i + 1] == '{' || src_[i + 1] == '%' || src_[i + 1] == '#')) {
        const char kind = src_[i + 1];
        const char* close = kind == '{' ? "}}" : (kind == '%' ? "%}" : "#}");
        size_t e = src_.find(close, i + 2);
        if (e == std::string::npos) fail("unterminated tag", i);
        size_t b = i + 2;
        bool lstrip = false, rstrip_after = false, no_lstrip = false;
        if (b < e && src_[b] == '-') { lstrip = true; ++b; }
        else if (b < e && src_[b] == '+') { no_lstrip = true; ++b; }
        size_t ee = e;
        if (ee > b && src_[ee - 1] == '-') { rstrip_after = true; --ee; }
        flush_text(lstrip, kind != '{' && !no_lstrip);
        if (kind != '#') pieces_.push_back({true, kind == '{', b, ee, ""});
        i = e + 2;
        strip_next = rstrip_after;
        trim_next_newline = kind != '{' && !rstrip_after;
        if (kind != '{') at_line_start_ = false;
        // apply right-side whitespace handling to the upcoming text
        if (strip_next) {
          while (i < src_.size() && isspace(static_cast<unsigned char>(src_[i]))) ++i;
          at_line_start_ = i > 0 && src_[i - 1] == '\n';
        } else if (trim_next_newline) {
          if (i < src_.size() && src_[i] == '\n') { ++i; at_line_start_ = true; }
          else if (i + 1 < src_.size() && src_[i] == '\r' && src_[i + 1] == '\n') { i += 2; at_line_start_ = true; }
        }
        continue;
      }
      text.push_back(src_[i++]);
    }
    flush_text(false, false);
  }

  // ---- expression parsing (precedence climbing)
  struct TS {
    std::vector<Token> toks;
    size_t i = 0;
    const Token& peek() const { return toks[i]; }
    Token take() { return toks[i++]; }
    bool is_op(const char* o) const { return toks[i].t == T_OP && toks[i].s == o; }
    bool is_name(const char* n) const { return toks[i].t == T_NAME && toks[i].s == n; }
  };
  TS lex(size_t b, size_t e) {
    TS ts;
    ExprLexer lx(src_, b, e);
    for (;;) {
      Token t = lx.next();
      ts.toks.push_back(t);
      if (t.t == T_EOF) break;
    }
    return ts;
  }
  EP mk(Expr::K k, size_t pos) { auto e = std::make_shared<Expr>(); e->k = k; e->pos = pos; return e; }

  EP parse_expr(TS& ts) { return parse_cond(ts); }
  EP parse_cond(TS& ts) {
    EP a = parse_or(ts);
    if (ts.is_name("if")) {
      const size_t p = ts.take().pos;
      EP c = parse_or(ts);
      EP e = mk(Expr::Cond, p);
      e->a = a; e->b = c;
      if (ts.is_name("else")) { ts.take(); e->c = parse_cond(ts); }
      return e;
    }
    return a;
  }
  EP bin(const std::string& op, EP a, EP b, size_t p) { EP e = mk(Expr::Binary, p); e->name = op; e->a = a; e->b = b; return e; }
  EP parse_or(TS& ts) {
    EP a = parse_and(ts);
    while (ts.is_name("or")) { size_t p = ts.take().pos; a = bin("or", a, parse_and(ts), p); }
    return a;
  }
  EP parse_and(TS& ts) {
    EP a = parse_not(ts);
    while (ts.is_name("and")) { size_t p = ts.take().pos; a = bin("and", a, parse_not(ts), p); }
    return a;
  }
  EP parse_not(TS& ts) {
    if (ts.is_name("not")) { size_t p = ts.take().pos; EP e = mk(Expr::Unary, p); e->name = "not"; e->a = parse_not(ts); return e; }
    return parse_cmp(ts);
  }
  EP parse_cmp(TS& ts) {
    EP a = parse_add(ts);
    for (;;) {
      if (ts.peek().t == T_OP && (ts.peek().s == "==" || ts.peek().s == "!=" || ts.peek().s == "<" || ts.peek().s == ">" ||
                                  ts.peek().s == "<=" || ts.peek().s == ">=")) {
        Token o = ts.take();
        a = bin(o.s, a, parse_add(ts), o.pos);
      } else if (ts.is_name("in")) {
        size_t p = ts.take().pos;
        a = bin("in", a, parse_add(ts), p);
      } else if (ts.is_name("not") && ts.toks[ts.i + 1].t == T_NAME && ts.toks[ts.i + 1].s == "in") {
        size_t p = ts.take().pos; ts.take();
        EP e = mk(Expr::Unary, p); e->name = "not"; e->a = bin("in", a, parse_add(ts), p);
        a = e;
      } else if (ts.is_name("is")) {
        size_t p = ts.take().pos;
        EP e = mk(Expr::Test, p);
        if (ts.is_name("not")) { ts.take(); e->negate = true; }
        if (ts.peek().t != T_NAME) fail("expected test name", ts.peek().pos);
        e->name = ts.take().s;
        e->a = a;
        // optional argument: `is divisibleby(3)` or `is divisibleby 3`
        if (ts.is_op("(")) { ts.take(); while (!ts.is_op(")")) { e->args.push_back(parse_expr(ts)); if (ts.is_op(",")) ts.take(); } ts.take(); }
        else if (ts.peek().t == T_INT || ts.peek().t == T_STR) e->args.push_back(parse_primary(ts));
        a = e;
      } else break;
    }
    return a;
  }
  EP parse_add(TS& ts) {
    EP a = parse_mul(ts);
    while (ts.is_op("+") || ts.is_op("-") || ts.is_op("~")) { Token o = ts.take(); a = bin(o.s, a, parse_mul(ts), o.pos); }
    return a;
  }
  EP parse_mul(TS& ts) {
    EP a = parse_unary(ts);
    while (ts.is_op("*") || ts.is_op("/") || ts.is_op("//") || ts.is_op("%")) { Token o = ts.take(); a = bin(o.s, a, parse_unary(ts), o.pos); }
    return a;
  }
  EP parse_unary(TS& ts) {
    if (ts.is_op("-") || ts.is_op("+")) { Token o = ts.take(); EP e = mk(Expr::Unary, o.pos); e->name = o.s; e->a = parse_unary(ts); return e; }
    return parse_postfix(ts);
  }
  void parse_call_args(TS& ts, EP call) {
    ts.take();  // (
    while (!ts.is_op(")")) {
      if (ts.peek().t == T_EOF) fail("unterminated call", ts.peek().pos);
      if (ts.peek().t == T_NAME && ts.toks[ts.i + 1].t == T_OP && ts.toks[ts.i + 1].s == "=") {
        std::string k = ts.take().s; ts.take();
        call->kwargs.emplace_back(k, parse_expr(ts));
      } else {
        call->args.push_back(parse_expr(ts));
      }
      if (ts.is_op(",")) ts.take();
    }
    ts.take();
  }
  EP parse_postfix(TS& ts) {
    EP a = parse_primary(ts);
    for (;;) {
      if (ts.is_op(".")) {
        size_t p = ts.take().pos;
        if (ts.peek().t != T_NAME && ts.peek().t != T_INT) fail("expected attribute name", ts.peek().pos);
        EP e = mk(Expr::Attr, p); e->a = a; e->name = ts.take().s; a = e;
      } else if (ts.is_op("[")) {
        size_t p = ts.take().pos;
        EP lo, hi, st;
        bool slice = false;
        if (!ts.is_op(":")) lo = parse_expr(ts);
        if (ts.is_op(":")) {
          slice = true; ts.take();
          if (!ts.is_op("]") && !ts.is_op(":")) hi = parse_expr(ts);
          if (ts.is_op(":")) { ts.take(); if (!ts.is_op("]")) st = parse_expr(ts); }
        }
        if (!ts.is_op("]")) fail("expected ]", ts.peek().pos);
        ts.take();
        if (slice) { EP e = mk(Expr::Slice, p); e->a = a; e->args = {lo, hi, st}; a = e; }
        else { EP e = mk(Expr::Index, p); e->a = a; e->b = lo; a = e; }
      } else if (ts.is_op("(")) {
        EP e = mk(Expr::Call, ts.peek().pos); e->a = a; parse_call_args(ts, e); a = e;
      } else if (ts.is_op("|")) {
        size_t p = ts.take().pos;
        if (ts.peek().t != T_NAME) fail("expected filter name", ts.peek().pos);
        EP e = mk(Expr::Filter, p); e->a = a; e->name = ts.take().s;
        if (ts.is_op("(")) parse_call_args(ts, e);
        a = e;
      } else break;
    }
    return a;
  }
  EP parse_primary(TS& ts) {
    Token t = ts.take();
    switch (t.t) {
      case T_INT: { EP e = mk(Expr::Lit, t.pos); e->lit = mk_int(strtoll(t.s.c_str(), nullptr, 10)); return e; }
      case T_FLOAT: { EP e = mk(Expr::Lit, t.pos); e->lit = mk_float(strtod(t.s.c_str(), nullptr)); return e; }
      case T_STR: {
        EP e = mk(Expr::Lit, t.pos);
        std::string s = t.s;
        while (ts.peek().t == T_STR) s += ts.take().s;  // adjacent literals concatenate
        e->lit = mk_str(s);
        return e;
      }
      case T_NAME: {
        if (t.s == "true" || t.s == "True") { EP e = mk(Expr::Lit, t.pos); e->lit = mk_bool(true); return e; }
        if (t.s == "false" || t.s == "False") { EP e = mk(Expr::Lit, t.pos); e->lit = mk_bool(false); return e; }
        if (t.s == "none" || t.s == "None") { EP e = mk(Expr::Lit, t.pos); e->lit = none(); return e; }
        EP e = mk(Expr::Name, t.pos); e->name = t.s; return e;
      }
      case T_OP:
        if (t.s == "(") {
          EP e = parse_expr(ts);
          if (ts.is_op(",")) {  // tuple -> list
            EP l = mk(Expr::ListE, t.pos); l->args.push_back(e);
            while (ts.is_op(",")) { ts.take(); if (ts.is_op(")")) break; l->args.push_back(parse_expr(ts)); }
            e = l;
          }
          if (!ts.is_op(")")) fail("expected )", ts.peek().pos);
          ts.take();
          return e;
        }
        if (t.s == "[") {
          EP l = mk(Expr::ListE, t.pos);
          while (!ts.is_op("]")) {
            if (ts.peek().t == T_EOF) fail("unterminated list", t.pos);
            l->args.push_back(parse_expr(ts));
            if (ts.is_op(",")) ts.take();
          }
          ts.take();
          return l;
        }
        if (t.s == "{") {
          EP d = mk(Expr::DictE, t.pos);
          while (!ts.is_op("}")) {
            if (ts.peek().t == T_EOF) fail("unterminated dict", t.pos);
            EP k = parse_expr(ts);
            if (!ts.is_op(":")) fail("expected :", ts.peek().pos);
            ts.take();
            d->pairs.emplace_back(k, parse_expr(ts));
            if (ts.is_op(",")) ts.take();
          }
          ts.take();
          return d;
        }
        fail("unexpected '" + t.s + "'", t.pos);
      default: fail("unexpected end of expression", t.pos);
    }
  }
  EP full_expr(TS& ts) {
    EP e = parse_expr(ts);
    if (ts.peek().t != T_EOF) fail("unexpected '" + ts.peek().s + "'", ts.peek().pos);
    return e;
  }

  // ---- statements
  std::string tag_word(const Piece& p) {
    ExprLexer lx(src_, p.b, p.e);
    Token t = lx.next();
    return t.t == T_NAME ? t.s : "";
  }
  std::vector<NP> block(const std::vector<std::string>& stop) {
    std::vector<NP> out;
    while (pi_ < pieces_.size()) {
      const Piece& p = pieces_[pi_];
      if (!p.is_tag) {
        auto n = std::make_shared<Node>(); n->k = Node::Text; n->text = p.text; out.push_back(n); ++pi_;
        continue;
      }
      if (p.is_expr) {
        TS ts = lex(p.b, p.e);
        auto n = std::make_shared<Node>(); n->k = Node::Output; n->expr = full_expr(ts); out.push_back(n); ++pi_;
        continue;
      }
      const std::string w = tag_word(p);
      if (std::find(stop.begin(), stop.end(), w) != stop.end()) return out;
      ++pi_;
      TS ts = lex(p.b, p.e);
      ts.take();  // the keyword
      if (w == "if") out.push_back(parse_if(ts));
      else if (w == "for") out.push_back(parse_for(ts));
      else if (w == "set") out.push_back(parse_set(ts, p));
      else if (w == "macro") out.push_back(parse_macro(ts));
      else if (w == "break") { auto n = std::make_shared<Node>(); n->k = Node::Break; out.push_back(n); }
      else if (w == "continue") { auto n = std::make_shared<Node>(); n->k = Node::Continue; out.push_back(n); }
      else if (w == "generation" || w == "endgeneration") { /* transformers' assistant-mask markers: no output */ }
      else fail("unknown tag '" + w + "'", p.b);
    }
    if (!stop.empty()) fail("missing {% " + stop.back() + " %}", src_.size());
    return out;
  }
  void expect_tag(const std::string& w) {
    if (pi_ >= pieces_.size() || tag_word(pieces_[pi_]) != w) fail("expected {% " + w + " %}", pi_ < pieces_.size() ? pieces_[pi_].b : src_.size());
    ++pi_;
  }
  NP parse_if(TS& ts) {
    auto n = std::make_shared<Node>();
    n->k = Node::If;
    EP cond = full_expr(ts);
    for (;;) {
      std::vector<NP> body = block({"elif", "else", "endif"});
      n->branches.emplace_back(cond, body);
      const Piece& p = pieces_[pi_];
      const std::string w = tag_word(p);
      ++pi_;
      if (w == "endif") break;
      if (w == "else") {
        std::vector<NP> eb = block({"endif"});
        n->branches.emplace_back(nullptr, eb);
        expect_tag("endif");
        break;
      }
      TS t2 = lex(p.b, p.e);
      t2.take();
      cond = full_expr(t2);
    }
    return n;
  }
  NP parse_for(TS& ts) {
    auto n = std::make_shared<Node>();
    n->k = Node::For;
    for (;;) {
      if (ts.peek().t != T_NAME) fail("expected loop variable", ts.peek().pos);
      n->targets.push_back(ts.take().s);
      if (ts.is_op(",")) { ts.take(); continue; }
      break;
    }
    if (!ts.is_name("in")) fail("expected 'in'", ts.peek().pos);
    ts.take();
    n->expr = parse_or(ts);
    if (ts.is_name("if")) { ts.take(); n->filter_cond = parse_expr(ts); }
    if (ts.is_name("recursive")) { ts.take(); n->recursive = true; }
    if (ts.peek().t != T_EOF) fail("unexpected '" + ts.peek().s + "' in for", ts.peek().pos);
    n->body = block({"else", "endfor"});
    if (tag_word(pieces_[pi_]) == "else") { ++pi_; n->else_body = block({"endfor"}); }
    expect_tag("endfor");
    return n;
  }
  NP parse_set(TS& ts, const Piece& p) {
    auto n = std::make_shared<Node>();
    if (ts.peek().t != T_NAME) fail("expected name after set", ts.peek().pos);
    n->targets.push_back(ts.take().s);
    if (ts.is_op(".")) { ts.take(); n->attr = ts.take().s; }
    while (ts.is_op(",")) { ts.take(); n->targets.push_back(ts.take().s); }
    if (ts.is_op("=")) {
      ts.take();
      n->k = Node::Set;
      EP e = parse_expr(ts);
      if (ts.is_op(",")) {  // tuple on the right-hand side
        EP l = mk(Expr::ListE, p.b); l->args.push_back(e);
        while (ts.is_op(",")) { ts.take(); l->args.push_back(parse_expr(ts)); }
        e = l;
      }
      if (ts.peek().t != T_EOF) fail("unexpected '" + ts.peek().s + "' in set", ts.peek().pos);
      n->expr = e;
    } else {
      n->k = Node::SetBlock;
      n->body = block({"endset"});
      expect_tag("endset");
    }
    return n;
  }
  NP parse_macro(TS& ts) {
    auto n = std::make_shared<Node>();
    n->k = Node::MacroDef;
    n->text = ts.take().s;
    if (!ts.is_op("(")) fail("expected ( after macro name", ts.peek().pos);
    ts.take();
    while (!ts.is_op(")")) {
      if (ts.peek().t != T_NAME) fail("expected parameter name", ts.peek().pos);
      std::string nm = ts.take().s;
      n->targets.push_back(nm);
      if (ts.is_op("=")) { ts.take(); n->defaults.emplace_back(nm, parse_expr(ts)); }
      if (ts.is_op(",")) ts.take();
    }
    n->body = block({"endmacro"});
    expect_tag("endmacro");
    return n;
  }

  const std::string& src_;
  std::vector<Piece> pieces_;
  size_t pi_ = 0;
  bool at_line_start_ = true;
};

// ====================================================================== interpreter
struct LoopControl { enum K { Break, Continue } k; };

class Interp {
 public:
  Interp(const TemplateLimits& lim) : lim_(lim) { scopes_.emplace_back(); }
  void set_global(const std::string& k, VP v) { scopes_[0][k] = std::move(v); }
  std::string run(const std::vector<NP>& nodes) {
    std::string out;
    exec(nodes, out);
    return out;
  }

 private:
  [[noreturn]] void fail(const std::string& m, size_t pos) const {
    throw TemplateError("template: " + m + " at byte " + std::to_string(pos));
  }
  VP lookup(const std::string& n) const {
    for (size_t k = scopes_.size(); k-- > 0;) {
      auto it = scopes_[k].find(n);
      if (it != scopes_[k].end()) return it->second;
    }
    return undefined();
  }
  void emit(std::string& out, const std::string& s) {
    if (out.size() + s.size() > lim_.max_output_bytes) throw TemplateError("template: output limit exceeded");
    out += s;
  }
  void exec(const std::vector<NP>& nodes, std::string& out) {
    for (const NP& n : nodes) {
      switch (n->k) {
        case Node::Text: emit(out, n->text); break;
        case Node::Output: emit(out, to_text(eval(n->expr))); break;
        case Node::If:
          for (const auto& br : n->branches)
            if (!br.first || truthy(eval(br.first))) { exec(br.second, out); break; }
          break;
        case Node::For: exec_for(n, out); break;
        case Node::Set: {
          VP v = eval(n->expr);
          if (!n->attr.empty()) {
            VP ns = lookup(n->targets[0]);
            if (ns->t != Val::Dict) throw TemplateError("template: cannot set attribute on a non-namespace");
            dict_set(ns, n->attr, v);
          } else if (n->targets.size() == 1) {
            scopes_.back()[n->targets[0]] = v;
          } else {
            if (v->t != Val::List || v->list.size() != n->targets.size()) throw TemplateError("template: cannot unpack in set");
            for (size_t k = 0; k < n->targets.size(); ++k) scopes_.back()[n->targets[k]] = v->list[k];
          }
          break;
        }
        case Node::SetBlock: {
          std::string buf;
          exec(n->body, buf);
          scopes_.back()[n->targets[0]] = mk_str(buf);
          break;
        }
        case Node::MacroDef: {
          auto m = std::make_shared<Macro>();
          m->name = n->text; m->params = n->targets; m->defaults = n->defaults; m->body = n->body;
          VP v = mk(Val::MacroT);
          v->macro = m;
          scopes_.back()[n->text] = v;
          break;
        }
        case Node::Break: throw LoopControl{LoopControl::Break};
        case Node::Continue: throw LoopControl{LoopControl::Continue};
        case Node::CallBlock: break;
      }
    }
  }
  std::vector<VP> iterate(const VP& v, size_t pos) {
    std::vector<VP> items;
    if (v->t == Val::List) items = v->list;
    else if (v->t == Val::Dict) for (const auto& kv : v->dict) items.push_back(mk_str(kv.first));
    else if (v->t == Val::Str) {
      for (size_t i = 0; i < v->s.size();) {
        unsigned char c = static_cast<unsigned char>(v->s[i]);
        size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
        items.push_back(mk_str(v->s.substr(i, n)));
        i += n;
      }
    } else if (v->t == Val::Undefined || v->t == Val::None) {
      if (v->t == Val::None) fail("cannot iterate over none", pos);
    } else fail("value is not iterable", pos);
    return items;
  }
  void exec_for(const NP& n, std::string& out) {
    std::vector<VP> items = iterate(eval(n->expr), n->expr->pos);
    if (n->filter_cond) {
      std::vector<VP> kept;
      for (const VP& it : items) {
        scopes_.emplace_back();
        bind_targets(n, it);
        const bool keep = truthy(eval(n->filter_cond));
        scopes_.pop_back();
        if (keep) kept.push_back(it);
      }
      items.swap(kept);
    }
    if (items.empty()) { exec(n->else_body, out); return; }
    for (size_t k = 0; k < items.size(); ++k) {
      if (++iterations_ > lim_.max_loop_iterations) throw TemplateError("template: loop iteration limit exceeded");
      scopes_.emplace_back();
      bind_targets(n, items[k]);
      VP loop = mk(Val::Dict);
      dict_set(loop, "index0", mk_int(static_cast<int64_t>(k)));
      dict_set(loop, "index", mk_int(static_cast<int64_t>(k) + 1));
      dict_set(loop, "revindex", mk_int(static_cast<int64_t>(items.size() - k)));
      dict_set(loop, "revindex0", mk_int(static_cast<int64_t>(items.size() - k) - 1));
      dict_set(loop, "first", mk_bool(k == 0));
      dict_set(loop, "last", mk_bool(k + 1 == items.size()));
      dict_set(loop, "length", mk_int(static_cast<int64_t>(items.size())));
      dict_set(loop, "previtem", k > 0 ? items[k - 1] : undefined());
      dict_set(loop, "nextitem", k + 1 < items.size() ? items[k + 1] : undefined());
      scopes_.back()["loop"] = loop;
      bool brk = false;
      try {
        exec(n->body, out);
      } catch (const LoopControl& lc) {
        brk = lc.k == LoopControl::Break;
      }
      scopes_.pop_back();
      if (brk) break;
    }
  }
  void bind_targets(const NP& n, const VP& item) {
    if (n->targets.size() == 1) { scopes_.back()[n->targets[0]] = item; return; }
    if (item->t != Val::List || item->list.size() != n->targets.size()) throw TemplateError("template: cannot unpack loop item");
    for (size_t k = 0; k < n->targets.size(); ++k) scopes_.back()[n->targets[k]] = item->list[k];
  }

  // ---------------------------------------------------------------- expressions
  VP eval(const EP& e) {
    switch (e->k) {
      case Expr::Lit: return e->lit;
      case Expr::Name: return lookup(e->name);
      case Expr::ListE: {
        VP l = mk(Val::List);
        for (const EP& a : e->args) l->list.push_back(eval(a));
        return l;
      }
      case Expr::DictE: {
        VP d = mk(Val::Dict);
        for (const auto& kv : e->pairs) dict_set(d, to_text(eval(kv.first)), eval(kv.second));
        return d;
      }
      case Expr::Attr: return get_attr(eval(e->a), e->name);
      case Expr::Index: return get_item(eval(e->a), eval(e->b), e->pos);
      case Expr::Slice: return slice(eval(e->a), e);
      case Expr::Cond:
        if (truthy(eval(e->b))) return eval(e->a);
        return e->c ? eval(e->c) : undefined();
      case Expr::Unary: {
        VP a = eval(e->a);
        if (e->name == "not") return mk_bool(!truthy(a));
        if (!is_num(a)) fail("unary operator on a non-number", e->pos);
        if (e->name == "-") return a->t == Val::Float ? mk_float(-a->f) : mk_int(-a->i);
        return a;
      }
      case Expr::Binary: return binary(e);
      case Expr::Test: {
        const bool r = test(e);
        return mk_bool(e->negate ? !r : r);
      }
      case Expr::Filter: return filter(e);
      case Expr::Call: return call(e);
    }
    return undefined();
  }
  VP get_attr(const VP& o, const std::string& name) {
    if (o->t == Val::Dict) {
      VP v = dict_get(o, name);
      if (v) return v;
    }
    return undefined();
  }
  VP get_item(const VP& o, const VP& k, size_t pos) {
    if (o->t == Val::Dict) {
      VP v = dict_get(o, to_text(k));
      return v ? v : undefined();
    }
    if (o->t == Val::List || o->t == Val::Str) {
      if (k->t != Val::Int) fail("index must be an integer", pos);
      int64_t n = o->t == Val::List ? static_cast<int64_t>(o->list.size()) : static_cast<int64_t>(o->s.size());
      int64_t i = k->i < 0 ? k->i + n : k->i;
      if (i < 0 || i >= n) return undefined();
      return o->t == Val::List ? o->list[static_cast<size_t>(i)] : mk_str(std::string(1, o->s[static_cast<size_t>(i)]));
    }
    return undefined();
  }
  VP slice(const VP& o, const EP& e) {
    int64_t n = o->t == Val::List ? static_cast<int64_t>(o->list.size()) : (o->t == Val::Str ? static_cast<int64_t>(o->s.size()) : -1);
    if (n < 0) fail("cannot slice this value", e->pos);
    int64_t step = e->args[2] ? eval(e->args[2])->i : 1;
    if (step == 0) fail("slice step cannot be zero", e->pos);
    auto bound = [&](const EP& x, int64_t dflt) {
      if (!x) return dflt;
      VP v = eval(x);
      if (v->t == Val::None || v->t == Val::Undefined) return dflt;
      int64_t i = v->i < 0 ? v->i + n : v->i;
      if (step > 0) return std::max<int64_t>(0, std::min(i, n));
      return std::max<int64_t>(-1, std::min(i, n - 1));
    };
    int64_t lo = bound(e->args[0], step > 0 ? 0 : n - 1), hi = bound(e->args[1], step > 0 ? n : -1);
    VP r = mk(o->t);
    for (int64_t i = lo; step > 0 ? i < hi : i > hi; i += step) {
      if (o->t == Val::List) r->list.push_back(o->list[static_cast<size_t>(i)]);
      else r->s.push_back(o->s[static_cast<size_t>(i)]);
    }
    return r;
  }
  bool contains(const VP& item, const VP& box, size_t pos) {
    if (box->t == Val::Str) return item->t == Val::Str && box->s.find(item->s) != std::string::npos;
    if (box->t == Val::List) { for (const VP& x : box->list) if (equals(x, item)) return true; return false; }
    if (box->t == Val::Dict) return dict_get(box, to_text(item)) != nullptr;
    if (box->t == Val::Undefined || box->t == Val::None) return false;
    fail("'in' needs a container", pos);
  }
  VP binary(const EP& e) {
    const std::string& op = e->name;
    if (op == "and") { VP a = eval(e->a); return truthy(a) ? eval(e->b) : a; }
    if (op == "or") { VP a = eval(e->a); return truthy(a) ? a : eval(e->b); }
    VP a = eval(e->a), b = eval(e->b);
    if (op == "==") return mk_bool(equals(a, b));
    if (op == "!=") return mk_bool(!equals(a, b));
    if (op == "in") return mk_bool(contains(a, b, e->pos));
    if (op == "~") return mk_str(to_text(a) + to_text(b));
    if (op == "<" || op == ">" || op == "<=" || op == ">=") {
      int c;
      if (is_num(a) && is_num(b)) c = num(a) < num(b) ? -1 : (num(a) > num(b) ? 1 : 0);
      else if (a->t == Val::Str && b->t == Val::Str) c = a->s.compare(b->s) < 0 ? -1 : (a->s == b->s ? 0 : 1);
      else fail("cannot compare these values", e->pos);
      return mk_bool(op == "<" ? c < 0 : op == ">" ? c > 0 : op == "<=" ? c <= 0 : c >= 0);
    }
    if (op == "+") {
      if (a->t == Val::Str && b->t == Val::Str) return mk_str(a->s + b->s);
      if (a->t == Val::List && b->t == Val::List) { VP r = mk(Val::List); r->list = a->list; r->list.insert(r->list.end(), b->list.begin(), b->list.end()); return r; }
    }
    if (op == "*" && a->t == Val::Str && b->t == Val::Int) { std::string s; for (int64_t k = 0; k < b->i; ++k) s += a->s; return mk_str(s); }
    if (op == "%" && a->t == Val::Str) return mk_str(a->s);  // printf-style formatting is not supported; keep the text
    if (!is_num(a) || !is_num(b)) fail("arithmetic on non-numbers ('" + op + "')", e->pos);
    const bool fl = a->t == Val::Float || b->t == Val::Float;
    if (op == "+") return fl ? mk_float(num(a) + num(b)) : mk_int(a->i + b->i);
    if (op == "-") return fl ? mk_float(num(a) - num(b)) : mk_int(a->i - b->i);
    if (op == "*") return fl ? mk_float(num(a) * num(b)) : mk_int(a->i * b->i);
    if (op == "/") { if (num(b) == 0) fail("division by zero", e->pos); return mk_float(num(a) / num(b)); }
    if (op == "//") {
      if (num(b) == 0) fail("division by zero", e->pos);
      if (fl) return mk_float(std::floor(num(a) / num(b)));
      int64_t q = a->i / b->i;
      if ((a->i % b->i != 0) && ((a->i < 0) != (b->i < 0))) --q;
      return mk_int(q);
    }
    if (op == "%") {
      if (num(b) == 0) fail("modulo by zero", e->pos);
      if (fl) return mk_float(num(a) - std::floor(num(a) / num(b)) * num(b));
      int64_t r = a->i % b->i;
      if (r != 0 && ((r < 0) != (b->i < 0))) r += b->i;
      return mk_int(r);
    }
    fail("unknown operator " + op, e->pos);
  }
  bool test(const EP& e) {
    VP a = eval(e->a);
    const std::string& n = e->name;
    if (n == "defined") return a->t != Val::Undefined;
    if (n == "undefined") return a->t == Val::Undefined;
    if (n == "none") return a->t == Val::None;
    if (n == "string") return a->t == Val::Str;
    if (n == "boolean") return a->t == Val::Bool;
    if (n == "true") return a->t == Val::Bool && a->b;
    if (n == "false") return a->t == Val::Bool && !a->b;
    if (n == "number") return a->t == Val::Int || a->t == Val::Float;
    if (n == "integer") return a->t == Val::Int;
    if (n == "float") return a->t == Val::Float;
    if (n == "mapping") return a->t == Val::Dict;
    if (n == "sequence") return a->t == Val::List || a->t == Val::Str || a->t == Val::Dict;
    if (n == "iterable") return a->t == Val::List || a->t == Val::Str || a->t == Val::Dict;
    if (n == "callable") return a->t == Val::MacroT;
    if (n == "odd") return a->t == Val::Int && (a->i % 2 != 0);
    if (n == "even") return a->t == Val::Int && (a->i % 2 == 0);
    if (n == "divisibleby") return a->t == Val::Int && !e->args.empty() && eval(e->args[0])->i != 0 && a->i % eval(e->args[0])->i == 0;
    if (n == "equalto" || n == "eq") return !e->args.empty() && equals(a, eval(e->args[0]));
    if (n == "in") return !e->args.empty() && contains(a, eval(e->args[0]), e->pos);
    fail("unknown test '" + n + "'", e->pos);
  }
  static std::string strip(const std::string& s, const std::string& chars, bool l, bool r) {
    auto is = [&](char c) { return chars.empty() ? isspace(static_cast<unsigned char>(c)) != 0 : chars.find(c) != std::string::npos; };
    size_t b = 0, e = s.size();
    if (l) while (b < e && is(s[b])) ++b;
    if (r) while (e > b && is(s[e - 1])) --e;
    return s.substr(b, e - b);
  }
  VP arg(const EP& e, size_t k, const char* kw = nullptr) {
    if (k < e->args.size()) return eval(e->args[k]);
    if (kw) for (const auto& kv : e->kwargs) if (kv.first == kw) return eval(kv.second);
    return nullptr;
  }
  VP filter(const EP& e) {
    VP a = eval(e->a);
    const std::string& n = e->name;
    if (n == "trim" || n == "strip") return mk_str(strip(to_text(a), "", true, true));
    if (n == "tojson") {
      VP ind = arg(e, 0, "indent");
      std::string out;
      py_json(a, out, ind && ind->t == Val::Int ? static_cast<int>(ind->i) : 0, 0);
      return mk_str(out);
    }
    if (n == "length" || n == "count") {
      if (a->t == Val::Str) {
        int64_t c = 0;
        for (unsigned char ch : a->s) if ((ch & 0xC0) != 0x80) ++c;
        return mk_int(c);
      }
      if (a->t == Val::List) return mk_int(static_cast<int64_t>(a->list.size()));
      if (a->t == Val::Dict) return mk_int(static_cast<int64_t>(a->dict.size()));
      return mk_int(0);
    }
    if (n == "lower") { std::string s = to_text(a); for (auto& c : s) c = static_cast<char>(tolower(static_cast<unsigned char>(c))); return mk_str(s); }
    if (n == "upper") { std::string s = to_text(a); for (auto& c : s) c = static_cast<char>(toupper(static_cast<unsigned char>(c))); return mk_str(s); }
    if (n == "capitalize") { std::string s = to_text(a); for (auto& c : s) c = static_cast<char>(tolower(static_cast<unsigned char>(c))); if (!s.empty()) s[0] = static_cast<char>(toupper(static_cast<unsigned char>(s[0]))); return mk_str(s); }
    if (n == "title") {
      std::string s = to_text(a);
      bool start = true;
      for (auto& c : s) { c = static_cast<char>(start ? toupper(static_cast<unsigned char>(c)) : tolower(static_cast<unsigned char>(c))); start = !isalnum(static_cast<unsigned char>(c)); }
      return mk_str(s);
    }
    if (n == "string") return mk_str(to_text(a));
    if (n == "safe" || n == "escape" || n == "e") return a;
    if (n == "int") {
      if (a->t == Val::Int) return a;
      if (a->t == Val::Float) return mk_int(static_cast<int64_t>(a->f));
      if (a->t == Val::Bool) return mk_int(a->b);
      if (a->t == Val::Str) { char* end = nullptr; long long v = strtoll(a->s.c_str(), &end, 10); if (end && end != a->s.c_str()) return mk_int(v); }
      VP d = arg(e, 0, "default");
      return d ? d : mk_int(0);
    }
    if (n == "float") { if (is_num(a)) return mk_float(num(a)); if (a->t == Val::Str) return mk_float(strtod(a->s.c_str(), nullptr)); return mk_float(0); }
    if (n == "abs") { if (a->t == Val::Float) return mk_float(std::fabs(a->f)); return mk_int(a->i < 0 ? -a->i : a->i); }
    if (n == "list") { VP l = mk(Val::List); l->list = iterate(a, e->pos); return l; }
    if (n == "first") { auto it = iterate(a, e->pos); return it.empty() ? undefined() : it.front(); }
    if (n == "last") { auto it = iterate(a, e->pos); return it.empty() ? undefined() : it.back(); }
    if (n == "reverse") { VP l = mk(Val::List); l->list = iterate(a, e->pos); std::reverse(l->list.begin(), l->list.end()); return l; }
    if (n == "default" || n == "d") {
      VP d = arg(e, 0, "default_value");
      VP boolean = arg(e, 1, "boolean");
      const bool use = a->t == Val::Undefined || (boolean && truthy(boolean) && !truthy(a));
      return use ? (d ? d : mk_str("")) : a;
    }
    if (n == "join") {
      VP sep = arg(e, 0, "d");
      VP attr = nullptr;
      for (const auto& kv : e->kwargs) if (kv.first == "attribute") attr = eval(kv.second);
      std::string s;
      bool first = true;
      for (const VP& x : iterate(a, e->pos)) {
        if (!first && sep) s += to_text(sep);
        first = false;
        s += to_text(attr ? get_attr(x, to_text(attr)) : x);
      }
      return mk_str(s);
    }
    if (n == "replace") {
      VP from = arg(e, 0), to = arg(e, 1);
      std::string s = to_text(a);
      if (!from || !to || from->s.empty()) return mk_str(s);
      std::string out;
      size_t i = 0;
      for (;;) {
        size_t k = s.find(from->s, i);
        if (k == std::string::npos) { out += s.substr(i); break; }
        out += s.substr(i, k - i) + to->s;
        i = k + from->s.size();
      }
      return mk_str(out);
    }
    if (n == "items" || n == "dictsort") {
      VP l = mk(Val::List);
      if (a->t == Val::Dict) {
        for (const auto& kv : a->dict) { VP p = mk(Val::List); p->list = {mk_str(kv.first), kv.second}; l->list.push_back(p); }
        if (n == "dictsort") std::sort(l->list.begin(), l->list.end(), [](const VP& x, const VP& y) { return x->list[0]->s < y->list[0]->s; });
      }
      return l;
    }
    if (n == "keys") { VP l = mk(Val::List); if (a->t == Val::Dict) for (const auto& kv : a->dict) l->list.push_back(mk_str(kv.first)); return l; }
    if (n == "unique") {
      VP l = mk(Val::List);
      for (const VP& x : iterate(a, e->pos)) { bool seen = false; for (const VP& y : l->list) if (equals(x, y)) seen = true; if (!seen) l->list.push_back(x); }
      return l;
    }
    if (n == "sort") {
      VP l = mk(Val::List);
      l->list = iterate(a, e->pos);
      std::stable_sort(l->list.begin(), l->list.end(), [](const VP& x, const VP& y) {
        if (is_num(x) && is_num(y)) return num(x) < num(y);
        return to_text(x) < to_text(y);
      });
      return l;
    }
    if (n == "sum") { double s = 0; bool fl = false; for (const VP& x : iterate(a, e->pos)) { s += num(x); fl |= x->t == Val::Float; } return fl ? mk_float(s) : mk_int(static_cast<int64_t>(s)); }
    if (n == "min" || n == "max") {
      auto it = iterate(a, e->pos);
      if (it.empty()) return undefined();
      VP best = it[0];
      for (const VP& x : it) if (n == "min" ? num(x) < num(best) : num(x) > num(best)) best = x;
      return best;
    }
    if (n == "map") {
      VP attr = nullptr;
      for (const auto& kv : e->kwargs) if (kv.first == "attribute") attr = eval(kv.second);
      VP l = mk(Val::List);
      for (const VP& x : iterate(a, e->pos)) {
        if (attr) l->list.push_back(get_attr(x, to_text(attr)));
        else if (!e->args.empty()) {
          // map('filtername')
          EP f = std::make_shared<Expr>();
          f->k = Expr::Filter; f->name = to_text(eval(e->args[0])); f->pos = e->pos;
          EP lit = std::make_shared<Expr>(); lit->k = Expr::Lit; lit->lit = x; f->a = lit;
          l->list.push_back(filter(f));
        } else l->list.push_back(x);
      }
      return l;
    }
    if (n == "selectattr" || n == "rejectattr" || n == "select" || n == "reject") {
      const bool by_attr = n == "selectattr" || n == "rejectattr";
      const bool want = n == "selectattr" || n == "select";
      VP l = mk(Val::List);
      size_t ai = 0;
      std::string attr = by_attr && !e->args.empty() ? to_text(eval(e->args[ai++])) : "";
      std::string tname = ai < e->args.size() ? to_text(eval(e->args[ai++])) : "";
      VP targ = ai < e->args.size() ? eval(e->args[ai]) : nullptr;
      for (const VP& x : iterate(a, e->pos)) {
        VP v = by_attr ? get_attr(x, attr) : x;
        bool r;
        if (tname.empty()) r = truthy(v);
        else {
          EP t = std::make_shared<Expr>(); t->k = Expr::Test; t->name = tname; t->pos = e->pos;
          EP lit = std::make_shared<Expr>(); lit->k = Expr::Lit; lit->lit = v; t->a = lit;
          if (targ) { EP al = std::make_shared<Expr>(); al->k = Expr::Lit; al->lit = targ; t->args.push_back(al); }
          r = test(t);
        }
        if (r == want) l->list.push_back(x);
      }
      return l;
    }
    if (n == "indent") {
      VP w = arg(e, 0, "width");
      const std::string pad(static_cast<size_t>(w ? w->i : 4), ' ');
      VP firstp = arg(e, 1, "first");
      std::string s = to_text(a), out;
      bool at_start = true, is_first = true;
      for (char c : s) {
        if (at_start && c != '\n' && !(is_first && !(firstp && truthy(firstp)))) out += pad;
        at_start = false;
        out.push_back(c);
        if (c == '\n') { at_start = true; is_first = false; }
      }
      return mk_str(out);
    }
    if (n == "round") { VP p = arg(e, 0, "precision"); double m = std::pow(10.0, p ? static_cast<double>(p->i) : 0.0); return mk_float(std::round(num(a) * m) / m); }
    fail("unknown filter '" + n + "'", e->pos);
  }
  VP call_macro(const std::shared_ptr<Macro>& m, const EP& e) {
    if (++depth_ > lim_.max_depth) throw TemplateError("template: call depth limit exceeded");
    std::map<std::string, VP> scope;
    for (size_t k = 0; k < m->params.size(); ++k) {
      VP v;
      if (k < e->args.size()) v = eval(e->args[k]);
      for (const auto& kv : e->kwargs) if (kv.first == m->params[k]) v = eval(kv.second);
      if (!v) for (const auto& d : m->defaults) if (d.first == m->params[k]) v = eval(d.second);
      scope[m->params[k]] = v ? v : undefined();
    }
    scopes_.push_back(std::move(scope));
    std::string out;
    exec(m->body, out);
    scopes_.pop_back();
    --depth_;
    return mk_str(out);
  }
  VP call(const EP& e) {
    // method call?
    if (e->a->k == Expr::Attr) {
      VP obj = eval(e->a->a);
      const std::string& m = e->a->name;
      if (obj->t == Val::Dict) {
        VP member = dict_get(obj, m);
        if (member && member->t == Val::MacroT) return call_macro(member->macro, e);
        if (m == "items") { VP l = mk(Val::List); for (const auto& kv : obj->dict) { VP p = mk(Val::List); p->list = {mk_str(kv.first), kv.second}; l->list.push_back(p); } return l; }
        if (m == "keys") { VP l = mk(Val::List); for (const auto& kv : obj->dict) l->list.push_back(mk_str(kv.first)); return l; }
        if (m == "values") { VP l = mk(Val::List); for (const auto& kv : obj->dict) l->list.push_back(kv.second); return l; }
        if (m == "get") { VP k = arg(e, 0); VP v = k ? dict_get(obj, to_text(k)) : nullptr; if (v) return v; VP d = arg(e, 1); return d ? d : none(); }
        if (m == "update") { VP o = arg(e, 0); if (o && o->t == Val::Dict) for (const auto& kv : o->dict) dict_set(obj, kv.first, kv.second); return none(); }
      }
      if (obj->t == Val::Str) {
        const std::string& s = obj->s;
        VP a0 = arg(e, 0);
        if (m == "strip") return mk_str(strip(s, a0 ? a0->s : "", true, true));
        if (m == "lstrip") return mk_str(strip(s, a0 ? a0->s : "", true, false));
        if (m == "rstrip") return mk_str(strip(s, a0 ? a0->s : "", false, true));
        if (m == "startswith") return mk_bool(a0 && s.compare(0, a0->s.size(), a0->s) == 0);
        if (m == "endswith") return mk_bool(a0 && s.size() >= a0->s.size() && s.compare(s.size() - a0->s.size(), a0->s.size(), a0->s) == 0);
        if (m == "upper" || m == "lower" || m == "title" || m == "capitalize") {
          EP f = std::make_shared<Expr>(); f->k = Expr::Filter; f->name = m; f->a = e->a->a; f->pos = e->pos;
          return filter(f);
        }
        if (m == "replace") { EP f = std::make_shared<Expr>(); f->k = Expr::Filter; f->name = "replace"; f->a = e->a->a; f->args = e->args; f->pos = e->pos; return filter(f); }
        if (m == "find") return mk_int(a0 ? static_cast<int64_t>(s.find(a0->s) == std::string::npos ? -1 : static_cast<int64_t>(s.find(a0->s))) : -1);
        if (m == "split") {
          VP l = mk(Val::List);
          VP mx = arg(e, 1);
          int64_t maxsplit = mx ? mx->i : -1;
          if (!a0 || a0->t != Val::Str || a0->s.empty()) {
            std::istringstream is(s);
            std::string w;
            while (is >> w) l->list.push_back(mk_str(w));
          } else {
            size_t i = 0;
            for (;;) {
              size_t k = (maxsplit >= 0 && static_cast<int64_t>(l->list.size()) >= maxsplit) ? std::string::npos : s.find(a0->s, i);
              if (k == std::string::npos) { l->list.push_back(mk_str(s.substr(i))); break; }
              l->list.push_back(mk_str(s.substr(i, k - i)));
              i = k + a0->s.size();
            }
          }
          return l;
        }
        if (m == "join") { std::string out; bool first = true; if (a0) for (const VP& x : iterate(a0, e->pos)) { if (!first) out += s; first = false; out += to_text(x); } return mk_str(out); }
      }
      if (obj->t == Val::List) {
        if (m == "append") { VP v = arg(e, 0); if (v) obj->list.push_back(v); return none(); }
        if (m == "pop") { if (obj->list.empty()) fail("pop from empty list", e->pos); VP v = obj->list.back(); obj->list.pop_back(); return v; }
        if (m == "index") { VP v = arg(e, 0); for (size_t k = 0; k < obj->list.size(); ++k) if (v && equals(obj->list[k], v)) return mk_int(static_cast<int64_t>(k)); fail("value not in list", e->pos); }
      }
      fail("unknown method '" + m + "'", e->pos);
    }
    if (e->a->k == Expr::Name) {
      const std::string& f = e->a->name;
      VP bound = lookup(f);
      if (bound->t == Val::MacroT) return call_macro(bound->macro, e);
      if (f == "namespace") {
        VP ns = mk(Val::Dict);
        for (const auto& kv : e->kwargs) dict_set(ns, kv.first, eval(kv.second));
        return ns;
      }
      if (f == "dict") {
        VP d = mk(Val::Dict);
        for (const auto& kv : e->kwargs) dict_set(d, kv.first, eval(kv.second));
        return d;
      }
      if (f == "raise_exception") { VP m = arg(e, 0); throw TemplateError("template raised: " + (m ? to_text(m) : std::string())); }
      if (f == "range") {
        VP a0 = arg(e, 0), a1 = arg(e, 1), a2 = arg(e, 2);
        int64_t lo = a1 ? a0->i : 0, hi = a1 ? a1->i : (a0 ? a0->i : 0), st = a2 ? a2->i : 1;
        if (st == 0) fail("range step cannot be zero", e->pos);
        VP l = mk(Val::List);
        for (int64_t i = lo; st > 0 ? i < hi : i > hi; i += st) {
          if (l->list.size() > lim_.max_loop_iterations) throw TemplateError("template: range too large");
          l->list.push_back(mk_int(i));
        }
        return l;
      }
      if (f == "strftime_now") {
        VP fm = arg(e, 0);
        char buf[256];
        time_t t = time(nullptr);
        struct tm tmv;
        localtime_r(&t, &tmv);
        strftime(buf, sizeof(buf), fm ? fm->s.c_str() : "%Y-%m-%d", &tmv);
        return mk_str(buf);
      }
      fail("unknown function '" + f + "'", e->pos);
    }
    fail("value is not callable", e->pos);
  }

  TemplateLimits lim_;
  std::vector<std::map<std::string, VP>> scopes_;
  size_t iterations_ = 0;
  int depth_ = 0;
};

}  // namespace

struct ChatTemplate::Impl {
  std::vector<NP> nodes;
  TemplateLimits limits;
};

ChatTemplate::ChatTemplate(const std::string& source, TemplateLimits limits) : impl_(new Impl) {
  impl_->limits = limits;
  impl_->nodes = Parser(source).parse();
}
ChatTemplate::~ChatTemplate() = default;
ChatTemplate::ChatTemplate(ChatTemplate&&) noexcept = default;

std::string ChatTemplate::render(const json::Value& context) const {
  Interp in(impl_->limits);
  if (context.is_object())
    for (const auto& kv : context.members()) in.set_global(kv.first, from_json(kv.second));
  return in.run(impl_->nodes);
}

}  // namespace dgpp
