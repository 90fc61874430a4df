#include "rt/tokenizer.h"

#include <algorithm>
#include <queue>
#include <stdexcept>

#include "rt/json.h"
#include "rt/prefix_cache.h"  // fnv1a_bytes
#include "rt/unicode_tables.h"

namespace dgpp {

namespace {

// ------------------------------------------------------------------ UTF-8 helpers
inline int utf8_len(unsigned char c) {
  if (c < 0x80) return 1;
  if ((c >> 5) == 6) return 2;
  if ((c >> 4) == 14) return 3;
  if ((c >> 3) == 30) return 4;
  return 1;
}

// Decodes one code point at s[i]; invalid bytes decode as themselves (length 1).
inline uint32_t decode_cp(const std::string& s, size_t i, int* len) {
  const unsigned char c = static_cast<unsigned char>(s[i]);
  int n = utf8_len(c);
  if (i + n > s.size()) n = 1;
  uint32_t cp = c;
  if (n == 2) cp = ((c & 31u) << 6) | (static_cast<unsigned char>(s[i + 1]) & 63u);
  else if (n == 3) cp = ((c & 15u) << 12) | ((static_cast<unsigned char>(s[i + 1]) & 63u) << 6) | (static_cast<unsigned char>(s[i + 2]) & 63u);
  else if (n == 4) cp = ((c & 7u) << 18) | ((static_cast<unsigned char>(s[i + 1]) & 63u) << 12) |
                        ((static_cast<unsigned char>(s[i + 2]) & 63u) << 6) | (static_cast<unsigned char>(s[i + 3]) & 63u);
  *len = n;
  return cp;
}

inline void append_cp(std::string& out, uint32_t cp) {
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

template <size_t N>
inline bool in_ranges(const uint32_t (&tab)[N][2], int count, uint32_t cp) {
  int lo = 0, hi = count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (cp < tab[mid][0]) hi = mid - 1;
    else if (cp > tab[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
inline bool is_letter(uint32_t cp) {
  if (cp < 128) return (cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z');
  return in_ranges(unicode::kLetters, unicode::kLetters_count, cp);
}
inline bool is_number(uint32_t cp) {
  if (cp < 128) return cp >= '0' && cp <= '9';
  return in_ranges(unicode::kNumbers, unicode::kNumbers_count, cp);
}
inline bool is_space(uint32_t cp) {
  if (cp < 128) return cp == ' ' || (cp >= 9 && cp <= 13) || (cp >= 28 && cp <= 31);
  return in_ranges(unicode::kSpaces, unicode::kSpaces_count, cp);
}

// ------------------------------------------------------------------ GPT-2 byte <-> code point table
struct ByteTable {
  uint32_t to_cp[256];
  std::unordered_map<uint32_t, uint8_t> to_byte;
  ByteTable() {
    bool printable[256] = {false};
    for (int b = '!'; b <= '~'; ++b) printable[b] = true;
    for (int b = 0xA1; b <= 0xAC; ++b) printable[b] = true;
    for (int b = 0xAE; b <= 0xFF; ++b) printable[b] = true;
    int n = 0;
    for (int b = 0; b < 256; ++b) {
      to_cp[b] = printable[b] ? static_cast<uint32_t>(b) : 256u + static_cast<uint32_t>(n++);
      to_byte[to_cp[b]] = static_cast<uint8_t>(b);
    }
  }
};
const ByteTable& byte_table() {
  static const ByteTable t;
  return t;
}

std::string map_bytes(const std::string& raw) {
  std::string out;
  const ByteTable& t = byte_table();
  for (unsigned char c : raw) append_cp(out, t.to_cp[c]);
  return out;
}
// Printable token string -> raw bytes; false when a code point is outside the table (added tokens).
bool unmap_bytes(const std::string& mapped, std::string* raw) {
  const ByteTable& t = byte_table();
  raw->clear();
  for (size_t i = 0; i < mapped.size();) {
    int n;
    const uint32_t cp = decode_cp(mapped, i, &n);
    auto it = t.to_byte.find(cp);
    if (it == t.to_byte.end()) return false;
    raw->push_back(static_cast<char>(it->second));
    i += static_cast<size_t>(n);
  }
  return true;
}

// ------------------------------------------------------------------ pre-tokenizer scanners
struct Cp {
  uint32_t cp;
  uint32_t off;  // byte offset
  uint8_t len;
};

std::vector<Cp> to_cps(const std::string& s) {
  std::vector<Cp> v;
  v.reserve(s.size());
  for (size_t i = 0; i < s.size();) {
    int n;
    const uint32_t cp = decode_cp(s, i, &n);
    v.push_back({cp, static_cast<uint32_t>(i), static_cast<uint8_t>(n)});
    i += static_cast<size_t>(n);
  }
  return v;
}

inline uint32_t lower_ascii(uint32_t c) { return (c >= 'A' && c <= 'Z') ? c + 32 : c; }

// Length (in code points) of a contraction starting at i ('s 't 're 've 'm 'll 'd), else 0.
size_t contraction(const std::vector<Cp>& v, size_t i, bool icase) {
  if (v[i].cp != '\'' || i + 1 >= v.size()) return 0;
  auto at = [&](size_t k) { return icase ? lower_ascii(v[k].cp) : v[k].cp; };
  const uint32_t a = at(i + 1);
  if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
  if (i + 2 < v.size()) {
    const uint32_t b = at(i + 2);
    if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
  }
  return 0;
}

void split_gpt2(const std::string& s, std::vector<std::string>& out) {
  const std::vector<Cp> v = to_cps(s);
  const size_t n = v.size();
  size_t i = 0;
  auto emit = [&](size_t a, size_t b) {
    const size_t o0 = v[a].off, o1 = b < n ? v[b].off : s.size();
    out.emplace_back(s, o0, o1 - o0);
  };
  while (i < n) {
    size_t c = contraction(v, i, false);
    if (c) { emit(i, i + c); i += c; continue; }
    size_t j = i;
    const bool sp = v[j].cp == ' ' && j + 1 < n;
    const size_t k = sp ? j + 1 : j;
    if (k < n && is_letter(v[k].cp)) {
      size_t e = k;
      while (e < n && is_letter(v[e].cp)) ++e;
      emit(i, e); i = e; continue;
    }
    if (k < n && is_number(v[k].cp)) {
      size_t e = k;
      while (e < n && is_number(v[e].cp)) ++e;
      emit(i, e); i = e; continue;
    }
    if (k < n && !is_space(v[k].cp) && !is_letter(v[k].cp) && !is_number(v[k].cp)) {
      size_t e = k;
      while (e < n && !is_space(v[e].cp) && !is_letter(v[e].cp) && !is_number(v[e].cp)) ++e;
      emit(i, e); i = e; continue;
    }
    // whitespace run: \s+(?!\S) leaves the last space to prefix the next word
    size_t e = i;
    while (e < n && is_space(v[e].cp)) ++e;
    if (e < n && e - i > 1) --e;
    if (e == i) e = i + 1;
    emit(i, e);
    i = e;
  }
}

// Cl100k / Qwen2 family.  max_digits = 3 (cl100k, llama3) or 1 (qwen2).
void split_cl100k(const std::string& s, int max_digits, std::vector<std::string>& out) {
  const std::vector<Cp> v = to_cps(s);
  const size_t n = v.size();
  size_t i = 0;
  auto emit = [&](size_t a, size_t b) {
    const size_t o0 = v[a].off, o1 = b < n ? v[b].off : s.size();
    out.emplace_back(s, o0, o1 - o0);
  };
  auto is_nl = [](uint32_t c) { return c == '\r' || c == '\n'; };
  while (i < n) {
    size_t c = contraction(v, i, true);
    if (c) { emit(i, i + c); i += c; continue; }
    // [^\r\n\p{L}\p{N}]?\p{L}+
    {
      size_t k = i;
      if (!is_nl(v[k].cp) && !is_letter(v[k].cp) && !is_number(v[k].cp) && k + 1 < n && is_letter(v[k + 1].cp)) ++k;
      if (is_letter(v[k].cp)) {
        size_t e = k;
        while (e < n && is_letter(v[e].cp)) ++e;
        emit(i, e); i = e; continue;
      }
    }
    // \p{N}{1,max}
    if (is_number(v[i].cp)) {
      size_t e = i;
      while (e < n && is_number(v[e].cp) && e - i < static_cast<size_t>(max_digits)) ++e;
      emit(i, e); i = e; continue;
    }
    //  ?[^\s\p{L}\p{N}]+[\r\n]*
    {
      size_t k = i;
      if (v[k].cp == ' ' && k + 1 < n) ++k;
      if (k < n && !is_space(v[k].cp) && !is_letter(v[k].cp) && !is_number(v[k].cp)) {
        size_t e = k;
        while (e < n && !is_space(v[e].cp) && !is_letter(v[e].cp) && !is_number(v[e].cp)) ++e;
        while (e < n && is_nl(v[e].cp)) ++e;
        emit(i, e); i = e; continue;
      }
    }
    // \s*[\r\n]+  : longest run of whitespace that ends with a newline
    if (is_space(v[i].cp)) {
      size_t e = i, last_nl = 0;
      bool has_nl = false;
      while (e < n && is_space(v[e].cp)) {
        if (is_nl(v[e].cp)) { has_nl = true; last_nl = e + 1; }
        ++e;
      }
      if (has_nl) { emit(i, last_nl); i = last_nl; continue; }
      // \s+(?!\S) | \s+
      if (e < n && e - i > 1) --e;
      emit(i, e); i = e; continue;
    }
    emit(i, i + 1);
    ++i;
  }
}

// ------------------------------------------------------------------ NFC
const unicode::Decomp* find_decomp(uint32_t cp) {
  int lo = 0, hi = unicode::kDecomp_count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (unicode::kDecomp[mid].cp == cp) return &unicode::kDecomp[mid];
    if (unicode::kDecomp[mid].cp < cp) lo = mid + 1; else hi = mid - 1;
  }
  return nullptr;
}
uint8_t combining_class(uint32_t cp) {
  int lo = 0, hi = unicode::kCcc_count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (unicode::kCcc[mid].cp == cp) return unicode::kCcc[mid].cls;
    if (unicode::kCcc[mid].cp < cp) lo = mid + 1; else hi = mid - 1;
  }
  return 0;
}
uint32_t compose_pair(uint32_t a, uint32_t b) {
  // Hangul LV / LVT
  if (a >= 0x1100 && a < 0x1113 && b >= 0x1161 && b < 0x1176) return 0xAC00 + ((a - 0x1100) * 21 + (b - 0x1161)) * 28;
  if (a >= 0xAC00 && a < 0xD7A4 && (a - 0xAC00) % 28 == 0 && b > 0x11A7 && b < 0x11C3) return a + (b - 0x11A7);
  int lo = 0, hi = unicode::kComp_count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    const auto& c = unicode::kComp[mid];
    if (c.a == a && c.b == b) return c.cp;
    if (c.a < a || (c.a == a && c.b < b)) lo = mid + 1; else hi = mid - 1;
  }
  return 0;
}
void decompose(uint32_t cp, std::vector<uint32_t>& out) {
  if (cp >= 0xAC00 && cp < 0xD7A4) {  // Hangul syllable
    const uint32_t s = cp - 0xAC00;
    out.push_back(0x1100 + s / 588);
    out.push_back(0x1161 + (s % 588) / 28);
    if (s % 28) out.push_back(0x11A7 + s % 28);
    return;
  }
  const unicode::Decomp* d = find_decomp(cp);
  if (!d) { out.push_back(cp); return; }
  decompose(d->a, out);
  if (d->b) decompose(d->b, out);
}

}  // namespace

std::string Tokenizer::normalize_nfc(const std::string& s) {
  bool ascii = true;
  for (unsigned char c : s) if (c >= 0x80) { ascii = false; break; }
  if (ascii) return s;
  std::vector<uint32_t> d;
  for (size_t i = 0; i < s.size();) {
    int n;
    decompose(decode_cp(s, i, &n), d);
    i += static_cast<size_t>(n);
  }
  // canonical ordering
  for (size_t i = 1; i < d.size(); ++i) {
    const uint8_t c = combining_class(d[i]);
    if (!c) continue;
    size_t j = i;
    while (j > 0 && combining_class(d[j - 1]) > c) { std::swap(d[j], d[j - 1]); --j; }
  }
  // composition
  std::vector<uint32_t> out;
  size_t starter = static_cast<size_t>(-1);
  uint8_t last_cc = 0;
  for (size_t i = 0; i < d.size(); ++i) {
    const uint8_t cc = combining_class(d[i]);
    if (starter != static_cast<size_t>(-1)) {
      // a character combines with the last starter unless something of equal or higher class (or
      // another starter) stands between them
      const bool adjacent = out.size() - 1 == starter;
      const bool unblocked = adjacent || (cc != 0 && last_cc < cc);
      if (unblocked) {
        const uint32_t c = compose_pair(out[starter], d[i]);
        if (c) { out[starter] = c; continue; }
      }
    }
    if (cc == 0) starter = out.size();
    last_cc = cc;
    out.push_back(d[i]);
  }
  std::string r;
  for (uint32_t cp : out) append_cp(r, cp);
  return r;
}

// ------------------------------------------------------------------ construction
void Tokenizer::finish() {
  added_first_byte_.assign(256, 0);
  added_max_len_ = 0;
  added_lookup_.clear();
  for (const AddedToken& a : added_) {
    if (a.content.empty()) continue;
    added_lookup_[a.content] = a.id;
    added_first_byte_[static_cast<unsigned char>(a.content[0])] = 1;
    added_max_len_ = std::max(added_max_len_, a.content.size());
    if (a.id >= static_cast<int32_t>(id_to_bytes_.size())) {
      id_to_bytes_.resize(static_cast<size_t>(a.id) + 1);
      special_.resize(static_cast<size_t>(a.id) + 1, 0);
    }
    id_to_bytes_[a.id] = a.content;
    special_[a.id] = a.special ? 1 : 0;
  }
}

Tokenizer Tokenizer::byte_level(const std::vector<std::pair<std::string, std::string>>& merges,
                                const std::vector<AddedToken>& added, SplitPattern pattern) {
  Tokenizer t;
  t.pattern_ = pattern;
  int32_t next = 0;
  for (int b = 0; b < 256; ++b) {
    std::string raw(1, static_cast<char>(b));
    t.vocab_[map_bytes(raw)] = next++;
    t.id_to_bytes_.push_back(raw);
  }
  int32_t rank = 0;
  for (const auto& m : merges) {
    const std::string l = map_bytes(m.first), r = map_bytes(m.second);
    t.merge_rank_[l + '\x01' + r] = rank++;
    const std::string joined = l + r;
    if (!t.vocab_.count(joined)) {
      t.vocab_[joined] = next++;
      t.id_to_bytes_.push_back(m.first + m.second);
    }
  }
  t.special_.assign(t.id_to_bytes_.size(), 0);
  t.added_ = added;
  t.finish();
  return t;
}

Tokenizer Tokenizer::from_json(const std::string& text) {
  const json::Value root = json::parse(text);
  Tokenizer t;
  const json::Value& model = root.at("model");
  if (model.get_string("type", "BPE") != "BPE") throw std::runtime_error("tokenizer: only BPE models are supported");
  t.ignore_merges_ = model.get_bool("ignore_merges", false);
  const json::Value& vocab = model.at("vocab");
  int32_t max_id = -1;
  for (const auto& kv : vocab.members()) max_id = std::max<int32_t>(max_id, static_cast<int32_t>(kv.second.as_int()));
  t.id_to_bytes_.assign(static_cast<size_t>(max_id) + 1, std::string());
  t.special_.assign(static_cast<size_t>(max_id) + 1, 0);
  for (const auto& kv : vocab.members()) {
    const int32_t id = static_cast<int32_t>(kv.second.as_int());
    t.vocab_[kv.first] = id;
    std::string raw;
    t.id_to_bytes_[id] = unmap_bytes(kv.first, &raw) ? raw : kv.first;
  }
  int32_t rank = 0;
  for (const json::Value& m : model.at("merges").items()) {
    std::string l, r;
    if (m.is_string()) {
      const std::string& s = m.as_string();
      const size_t sp = s.find(' ');
      if (sp == std::string::npos) throw std::runtime_error("tokenizer: malformed merge '" + s + "'");
      l = s.substr(0, sp);
      r = s.substr(sp + 1);
    } else {
      l = m.at(size_t(0)).as_string();
      r = m.at(size_t(1)).as_string();
    }
    t.merge_rank_[l + '\x01' + r] = rank++;
  }
  if (const json::Value* added = root.find("added_tokens")) {
    for (const json::Value& a : added->items())
      t.added_.push_back({a.get_string("content"), static_cast<int32_t>(a.get_int("id")), a.get_bool("special", false)});
  }
  // normaliser
  if (const json::Value* norm = root.find("normalizer")) {
    std::string dump = norm->dump();
    if (dump.find("\"NFC\"") != std::string::npos) t.nfc_ = true;
  }
  // pre-tokeniser: recognise the pinned patterns by their distinguishing fragments
  t.pattern_ = SplitPattern::Gpt2;
  if (const json::Value* pre = root.find("pre_tokenizer")) {
    const std::string dump = pre->dump();
    if (dump.find("\\\\p{N}{1,3}") != std::string::npos) t.pattern_ = SplitPattern::Cl100k;
    else if (dump.find("(?i:") != std::string::npos) t.pattern_ = SplitPattern::Qwen2;
    else if (dump.find("ByteLevel") != std::string::npos || dump.find("'s|'t") != std::string::npos) t.pattern_ = SplitPattern::Gpt2;
    else if (pre->is_null()) t.pattern_ = SplitPattern::Whole;
  }
  t.finish();
  return t;
}

// ------------------------------------------------------------------ encoding
std::vector<std::string> Tokenizer::pre_tokenize(const std::string& text) const {
  std::vector<std::string> out;
  switch (pattern_) {
    case SplitPattern::Gpt2: split_gpt2(text, out); break;
    case SplitPattern::Cl100k: split_cl100k(text, 3, out); break;
    case SplitPattern::Qwen2: split_cl100k(text, 1, out); break;
    case SplitPattern::Whole: if (!text.empty()) out.push_back(text); break;
  }
  return out;
}

void Tokenizer::encode_word(const std::string& word, std::vector<int32_t>& out) const {
  auto hit = cache_.find(word);
  if (hit != cache_.end()) {
    out.insert(out.end(), hit->second.begin(), hit->second.end());
    return;
  }
  const std::string mapped = map_bytes(word);
  std::vector<int32_t> ids;
  auto whole = vocab_.find(mapped);
  if (ignore_merges_ && whole != vocab_.end()) {
    ids.push_back(whole->second);
  } else {
    // symbols as a doubly linked list; a heap of (rank, position, generation) candidate merges
    struct Sym { std::string s; int prev, next; bool alive; };
    std::vector<Sym> sym;
    for (size_t i = 0; i < mapped.size();) {
      const int n = utf8_len(static_cast<unsigned char>(mapped[i]));
      sym.push_back({mapped.substr(i, static_cast<size_t>(n)), static_cast<int>(sym.size()) - 1,
                     static_cast<int>(sym.size()) + 1, true});
      i += static_cast<size_t>(n);
    }
    if (!sym.empty()) sym.back().next = -1;
    struct Cand { int32_t rank; int left; size_t len_l, len_r; };
    auto cmp = [](const Cand& a, const Cand& b) { return a.rank != b.rank ? a.rank > b.rank : a.left > b.left; };
    std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> heap(cmp);
    auto push = [&](int l) {
      if (l < 0) return;
      const int r = sym[l].next;
      if (r < 0) return;
      auto it = merge_rank_.find(sym[l].s + '\x01' + sym[r].s);
      if (it != merge_rank_.end()) heap.push({it->second, l, sym[l].s.size(), sym[r].s.size()});
    };
    for (int i = 0; i + 1 < static_cast<int>(sym.size()); ++i) push(i);
    while (!heap.empty()) {
      const Cand c = heap.top();
      heap.pop();
      const int l = c.left;
      if (!sym[l].alive) continue;
      const int r = sym[l].next;
      if (r < 0 || !sym[r].alive || sym[l].s.size() != c.len_l || sym[r].s.size() != c.len_r) continue;
      sym[l].s += sym[r].s;
      sym[r].alive = false;
      sym[l].next = sym[r].next;
      if (sym[r].next >= 0) sym[sym[r].next].prev = l;
      push(sym[l].prev);
      push(l);
    }
    for (int i = sym.empty() ? -1 : 0; i >= 0; i = sym[i].next) {
      auto it = vocab_.find(sym[i].s);
      if (it != vocab_.end()) {
        ids.push_back(it->second);
      } else {
        // unknown symbol: fall back to its single bytes (always present in byte-level vocabularies)
        std::string raw;
        unmap_bytes(sym[i].s, &raw);
        for (unsigned char b : raw) {
          auto bt = vocab_.find(map_bytes(std::string(1, static_cast<char>(b))));
          if (bt != vocab_.end()) ids.push_back(bt->second);
        }
      }
    }
  }
  if (cache_.size() < 200000) cache_[word] = ids;
  out.insert(out.end(), ids.begin(), ids.end());
}

void Tokenizer::encode_segment(const std::string& text, std::vector<int32_t>& out) const {
  if (text.empty()) return;
  const std::string norm = nfc_ ? normalize_nfc(text) : text;
  for (const std::string& w : pre_tokenize(norm)) encode_word(w, out);
}

std::vector<int32_t> Tokenizer::encode(const std::string& text, bool allow_special) const {
  std::vector<int32_t> out;
  if (added_.empty()) {
    encode_segment(text, out);
    return out;
  }
  size_t seg = 0, i = 0;
  while (i < text.size()) {
    if (added_first_byte_[static_cast<unsigned char>(text[i])]) {
      // longest added token starting here
      size_t best = 0;
      int32_t best_id = -1;
      const size_t maxl = std::min(added_max_len_, text.size() - i);
      for (size_t l = maxl; l >= 1; --l) {
        auto it = added_lookup_.find(text.substr(i, l));
        if (it != added_lookup_.end() && (allow_special || !special_[it->second])) { best = l; best_id = it->second; break; }
      }
      if (best) {
        encode_segment(text.substr(seg, i - seg), out);
        out.push_back(best_id);
        i += best;
        seg = i;
        continue;
      }
    }
    ++i;
  }
  encode_segment(text.substr(seg), out);
  return out;
}

const std::string& Tokenizer::token_bytes(int32_t id) const {
  if (id < 0 || id >= static_cast<int32_t>(id_to_bytes_.size())) return empty_;
  return id_to_bytes_[id];
}

int32_t Tokenizer::token_to_id(const std::string& token) const {
  auto a = added_lookup_.find(token);
  if (a != added_lookup_.end()) return a->second;
  auto it = vocab_.find(map_bytes(token));
  return it == vocab_.end() ? -1 : it->second;
}

bool Tokenizer::is_special(int32_t id) const {
  return id >= 0 && id < static_cast<int32_t>(special_.size()) && special_[id];
}

std::string Tokenizer::decode(const std::vector<int32_t>& ids, bool skip_special) const {
  std::string out;
  for (int32_t id : ids) {
    if (skip_special && is_special(id)) continue;
    out += token_bytes(id);
  }
  return out;
}

uint64_t Tokenizer::fingerprint() const {
  uint64_t h = kFnvSeed;
  std::vector<std::pair<std::string, int32_t>> v(vocab_.begin(), vocab_.end());
  std::sort(v.begin(), v.end());
  for (const auto& kv : v) {
    h = fnv1a_bytes(h, kv.first.data(), kv.first.size());
    h = fnv1a_bytes(h, &kv.second, sizeof(kv.second));
  }
  std::vector<std::pair<std::string, int32_t>> m(merge_rank_.begin(), merge_rank_.end());
  std::sort(m.begin(), m.end());
  for (const auto& kv : m) {
    h = fnv1a_bytes(h, kv.first.data(), kv.first.size());
    h = fnv1a_bytes(h, &kv.second, sizeof(kv.second));
  }
  return h;
}

// ------------------------------------------------------------------ streaming decode
static size_t complete_utf8_prefix(const std::string& s) {
  // length of the longest prefix that does not end inside a multi-byte sequence
  size_t n = s.size();
  size_t back = 0;
  while (back < 4 && back < n) {
    const unsigned char c = static_cast<unsigned char>(s[n - 1 - back]);
    if ((c & 0xC0) == 0x80) { ++back; continue; }
    if (c >= 0xC0) {
      const size_t need = static_cast<size_t>(utf8_len(c));
      if (need > back + 1) return n - 1 - back;  // lead byte without all its continuation bytes
    }
    break;
  }
  return n;
}

std::string StreamDecoder::push(int32_t id) {
  if (skip_special_ && tok_->is_special(id)) return std::string();
  pending_ += tok_->token_bytes(id);
  const size_t ok = complete_utf8_prefix(pending_);
  std::string out = pending_.substr(0, ok);
  pending_.erase(0, ok);
  return out;
}

std::string StreamDecoder::flush() {
  std::string out;
  out.swap(pending_);
  return out;
}

}  // namespace dgpp
