// Constraints on the body of a JSON string value: minLength / maxLength, `pattern` (a regular-expression subset) and
// `format` (a few fixed shapes expressed as patterns).  The constraint is a byte-level Thompson NFA that the JSON
// machine advances with every decoded character of the string; the set of live NFA states travels in the machine's
// frame, so the vocabulary mask of a partially written string is exact: a token is allowed only if some completion
// of the string can still match.
//
// Regular-expression subset: literals, `.`, escapes \d \w \s \D \W \S and escaped punctuation, classes [a-z0-9_] and
// negated classes, groups ( ) and (?: ), alternation |, quantifiers * + ? {m} {m,} {m,n} (bounded counts are expanded,
// at most 64 copies), anchors ^ at the start and $ at the end.  As in JSON Schema a pattern without anchors may match
// anywhere in the string.  Characters are bytes: a non-ASCII character counts one per UTF-8 byte for `.` / negated
// classes and for the length limits (documented deviation; ASCII strings are exact).
// Formats: date (YYYY-MM-DD), time (hh:mm:ss with optional fraction and zone), date-time, uuid, ipv4.
// Inside a constrained string the escapes \" \\ \/ \b \f \n \r \t are decoded before they reach the NFA; \uXXXX is
// not accepted there (the character can be written directly).
// (reference counterpart: src/text/string_constraint.cpp.)
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace dgpp {
namespace grammar {

class StringConstraint {
 public:
  static constexpr int kMaxStates = 1024;

  int64_t min_len = 0, max_len = -1;
  bool has_pattern = false;

  // Compiles `pattern` (may be empty: lengths only).  Throws std::runtime_error on syntax outside the subset.
  static StringConstraint compile(const std::string& pattern, int64_t min_len, int64_t max_len) {
    StringConstraint c;
    c.min_len = min_len;
    c.max_len = max_len;
    if (!pattern.empty()) {
      c.has_pattern = true;
      Parser p{pattern, 0, &c};
      std::string src = pattern;
      const bool head = !src.empty() && src[0] == '^';
      const bool tail = src.size() >= 1 && src.back() == '$' && (src.size() < 2 || src[src.size() - 2] != '\\');
      p.src = src.substr(head ? 1 : 0, src.size() - (head ? 1 : 0) - (tail ? 1 : 0));
      Frag f = p.alternation();
      if (p.pos != p.src.size()) throw std::runtime_error("pattern: unbalanced ')' or trailing input");
      if (!head) f = c.concat(c.star(c.any()), f);
      if (!tail) f = c.concat(f, c.star(c.any()));
      c.accept_ = c.add_state(State::Accept);
      c.patch(f.out, c.accept_);
      c.start_ = f.start;
      if (static_cast<int>(c.states_.size()) > kMaxStates) throw std::runtime_error("pattern: too many states");
    }
    return c;
  }
  static std::string format_pattern(const std::string& fmt) {
    if (fmt == "date") return "^\\d{4}-\\d{2}-\\d{2}$";
    if (fmt == "time") return "^\\d{2}:\\d{2}:\\d{2}(\\.\\d+)?(Z|[+-]\\d{2}:\\d{2})?$";
    if (fmt == "date-time") return "^\\d{4}-\\d{2}-\\d{2}[Tt ]\\d{2}:\\d{2}:\\d{2}(\\.\\d+)?(Z|[+-]\\d{2}:\\d{2})$";
    if (fmt == "uuid") return "^[0-9a-fA-F]{8}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{12}$";
    if (fmt == "ipv4") return "^\\d{1,3}\\.\\d{1,3}\\.\\d{1,3}\\.\\d{1,3}$";
    return "";
  }

  // ---- run-time: the live state set is a byte string (bitset) kept by the caller
  std::string initial() const {
    std::string set;
    if (!has_pattern) return set;
    set.assign((states_.size() + 7) / 8, '\0');
    add_closure(set, start_);
    return set;
  }
  // Advances `set` by one byte; false = no state survives.
  bool step(std::string& set, unsigned char c) const {
    if (!has_pattern) return true;
    std::string next(set.size(), '\0');
    bool any = false;
    for (size_t i = 0; i < states_.size(); ++i) {
      if (!(set[i >> 3] >> (i & 7) & 1)) continue;
      const State& s = states_[i];
      if (s.kind == State::Byte && s.cls[c >> 6] >> (c & 63) & 1) {
        add_closure(next, s.out);
        any = true;
      }
    }
    set.swap(next);
    return any;
  }
  bool accepting(const std::string& set) const {
    if (!has_pattern) return true;
    return set[accept_ >> 3] >> (accept_ & 7) & 1;
  }

 private:
  struct State {
    enum Kind : uint8_t { Byte, Split, Accept } kind = Byte;
    uint64_t cls[4] = {0, 0, 0, 0};   // Byte: the accepted bytes
    int out = -1, out2 = -1;          // Split: two epsilon targets
  };
  struct Frag {
    int start;
    std::vector<int*> out;            // dangling arrows (pointers stay valid: states_ is reserved up front)
  };
  std::vector<State> states_;
  int start_ = 0, accept_ = 0;

  StringConstraint() { states_.reserve(kMaxStates + 8); }
  int add_state(State::Kind k) {
    if (static_cast<int>(states_.size()) >= kMaxStates) throw std::runtime_error("pattern: too many states");
    State s;
    s.kind = k;
    states_.push_back(s);
    return static_cast<int>(states_.size()) - 1;
  }
  void patch(const std::vector<int*>& outs, int target) {
    for (int* p : outs) *p = target;
  }
  Frag byte_class(const uint64_t cls[4]) {
    const int i = add_state(State::Byte);
    for (int k = 0; k < 4; ++k) states_[i].cls[k] = cls[k];
    return Frag{i, {&states_[i].out}};
  }
  Frag any() {
    uint64_t cls[4] = {~0ull, ~0ull, ~0ull, ~0ull};
    cls[0] &= ~(1ull << '\n');
    return byte_class(cls);
  }
  Frag concat(Frag a, Frag b) {
    patch(a.out, b.start);
    return Frag{a.start, b.out};
  }
  Frag alt(Frag a, Frag b) {
    const int i = add_state(State::Split);
    states_[i].out = a.start;
    states_[i].out2 = b.start;
    Frag f{i, a.out};
    f.out.insert(f.out.end(), b.out.begin(), b.out.end());
    return f;
  }
  Frag star(Frag a) {
    const int i = add_state(State::Split);
    states_[i].out = a.start;
    patch(a.out, i);
    return Frag{i, {&states_[i].out2}};
  }
  Frag plus(Frag a) {
    const int i = add_state(State::Split);
    states_[i].out = a.start;
    patch(a.out, i);
    return Frag{a.start, {&states_[i].out2}};
  }
  Frag quest(Frag a) {
    const int i = add_state(State::Split);
    states_[i].out = a.start;
    Frag f{i, a.out};
    f.out.push_back(&states_[i].out2);
    return f;
  }
  Frag empty() {
    const int i = add_state(State::Split);          // a split whose second arrow stays unused (-1)
    return Frag{i, {&states_[i].out}};
  }
  void add_closure(std::string& set, int s) const {
    if (s < 0 || (set[s >> 3] >> (s & 7) & 1)) return;
    set[s >> 3] = static_cast<char>(set[s >> 3] | (1 << (s & 7)));
    if (states_[s].kind == State::Split) {
      add_closure(set, states_[s].out);
      add_closure(set, states_[s].out2);
    }
  }

  struct Parser {
    std::string src;
    size_t pos;
    StringConstraint* c;

    bool more() const { return pos < src.size(); }
    Frag alternation() {
      Frag f = sequence();
      while (more() && src[pos] == '|') {
        ++pos;
        f = c->alt(f, sequence());
      }
      return f;
    }
    Frag sequence() {
      bool have = false;
      Frag f{0, {}};
      while (more() && src[pos] != '|' && src[pos] != ')') {
        Frag a = repeat();
        f = have ? c->concat(f, a) : a;
        have = true;
      }
      return have ? f : c->empty();
    }
    // Re-parses the same atom text to build another copy (bounded repetition).
    Frag atom_at(size_t at, size_t* end) {
      const size_t save = pos;
      pos = at;
      Frag a = atom();
      *end = pos;
      pos = save;
      return a;
    }
    Frag repeat() {
      const size_t at = pos;
      Frag a = atom();
      const size_t end = pos;
      if (!more()) return a;
      const char q = src[pos];
      if (q == '*') { ++pos; return c->star(a); }
      if (q == '+') { ++pos; return c->plus(a); }
      if (q == '?') { ++pos; return c->quest(a); }
      if (q == '{') {
        size_t p = pos + 1;
        auto num = [&](int* v) {
          bool any = false;
          *v = 0;
          while (p < src.size() && src[p] >= '0' && src[p] <= '9') { *v = *v * 10 + (src[p] - '0'); ++p; any = true; }
          return any;
        };
        int lo = 0, hi = -2;
        if (!num(&lo)) return a;                                  // a literal '{'
        if (p < src.size() && src[p] == ',') {
          ++p;
          if (!num(&hi)) hi = -1;                                 // {m,}
        } else {
          hi = lo;
        }
        if (p >= src.size() || src[p] != '}') throw std::runtime_error("pattern: malformed {m,n}");
        pos = p + 1;
        if (lo > 64 || hi > 64 || (hi >= 0 && hi < lo)) throw std::runtime_error("pattern: repetition count outside 0..64");
        // a{lo,hi} = lo copies, then (hi - lo) optional copies or a star
        size_t e2;
        bool have = lo > 0;
        Frag f = a;                                               // first copy (used when lo > 0)
        for (int i = 1; i < lo; ++i) f = c->concat(f, atom_at(at, &e2));
        if (hi == -1) {
          Frag s = c->star(lo > 0 ? atom_at(at, &e2) : a);
          f = have ? c->concat(f, s) : s;
          have = true;
        } else {
          for (int i = lo; i < hi; ++i) {
            Frag o = c->quest((i == 0) ? a : atom_at(at, &e2));
            f = have ? c->concat(f, o) : o;
            have = true;
          }
        }
        (void)end;
        return have ? f : c->empty();
      }
      return a;
    }
    static void set_bit(uint64_t cls[4], unsigned char b) { cls[b >> 6] |= 1ull << (b & 63); }
    static void set_range(uint64_t cls[4], int a, int b) { for (int x = a; x <= b; ++x) set_bit(cls, static_cast<unsigned char>(x)); }
    static bool klass(char e, uint64_t cls[4]) {
      uint64_t t[4] = {0, 0, 0, 0};
      const char l = static_cast<char>(e | 0x20);
      if (l == 'd') set_range(t, '0', '9');
      else if (l == 'w') { set_range(t, '0', '9'); set_range(t, 'a', 'z'); set_range(t, 'A', 'Z'); set_bit(t, '_'); }
      else if (l == 's') { for (char ch : std::string(" \t\n\r\f\v")) set_bit(t, static_cast<unsigned char>(ch)); }
      else return false;
      const bool neg = e >= 'A' && e <= 'Z';
      for (int k = 0; k < 4; ++k) cls[k] |= neg ? ~t[k] : t[k];
      return true;
    }
    Frag atom() {
      if (!more()) throw std::runtime_error("pattern: unexpected end");
      const char ch = src[pos++];
      uint64_t cls[4] = {0, 0, 0, 0};
      if (ch == '(') {
        if (pos + 1 < src.size() && src[pos] == '?' && src[pos + 1] == ':') pos += 2;
        else if (more() && src[pos] == '?') throw std::runtime_error("pattern: only (?: ) groups are supported");
        Frag f = alternation();
        if (!more() || src[pos] != ')') throw std::runtime_error("pattern: missing ')'");
        ++pos;
        return f;
      }
      if (ch == '.') return c->any();
      if (ch == '[') {
        bool neg = false;
        if (more() && src[pos] == '^') { neg = true; ++pos; }
        bool first = true;
        while (more() && (src[pos] != ']' || first)) {
          first = false;
          unsigned char a = static_cast<unsigned char>(src[pos++]);
          if (a == '\\') {
            if (!more()) throw std::runtime_error("pattern: dangling backslash");
            const char e = src[pos++];
            if (klass(e, cls)) continue;
            a = e == 'n' ? '\n' : e == 't' ? '\t' : e == 'r' ? '\r' : static_cast<unsigned char>(e);
          }
          if (pos + 1 < src.size() && src[pos] == '-' && src[pos + 1] != ']') {
            unsigned char b = static_cast<unsigned char>(src[pos + 1]);
            pos += 2;
            if (b == '\\') { if (!more()) throw std::runtime_error("pattern: dangling backslash"); b = static_cast<unsigned char>(src[pos++]); }
            if (b < a) throw std::runtime_error("pattern: reversed range in a class");
            set_range(cls, a, b);
          } else {
            set_bit(cls, a);
          }
        }
        if (!more()) throw std::runtime_error("pattern: missing ']'");
        ++pos;
        if (neg) for (int k = 0; k < 4; ++k) cls[k] = ~cls[k];
        return c->byte_class(cls);
      }
      if (ch == '\\') {
        if (!more()) throw std::runtime_error("pattern: dangling backslash");
        const char e = src[pos++];
        if (klass(e, cls)) return c->byte_class(cls);
        if (e == 'b' || e == 'B' || (e >= '1' && e <= '9')) throw std::runtime_error("pattern: \\b and back-references are not supported");
        set_bit(cls, e == 'n' ? '\n' : e == 't' ? '\t' : e == 'r' ? '\r' : static_cast<unsigned char>(e));
        return c->byte_class(cls);
      }
      if (ch == '*' || ch == '+' || ch == '?' || ch == ')') throw std::runtime_error("pattern: nothing to repeat");
      if (ch == '^' || ch == '$') throw std::runtime_error("pattern: anchors are supported at the ends only");
      set_bit(cls, static_cast<unsigned char>(ch));
      return c->byte_class(cls);
    }
  };
};

}  // namespace grammar
}  // namespace dgpp
