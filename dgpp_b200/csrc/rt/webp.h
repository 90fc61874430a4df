// WebP decoder for inline image inputs: the LOSSLESS bitstream (VP8L chunk, plain or inside the extended VP8X
// container).  Output: interleaved 8-bit RGBA (alpha 255 when the file carries none).  Lossy (VP8) and animated files are
// refused with a message that names the reason.
//
// VP8L in brief (bits are read least-significant first):
//   header     0x2f, 14 bits width - 1, 14 bits height - 1, alpha hint, 3 version bits (0)
//   transforms up to four, each kind once: predictor (per-block choice of 14 spatial predictors), cross-colour (per-block
//              red / blue corrections from green and red), subtract-green, colour indexing (palette, pixels packed 8 / 4 /
//              2 / 1 per word when the palette is small); their parameter images use the same entropy coding
//   pixels     ARGB, entropy coded with five prefix codes per group (green + length + cache index, red, blue, alpha,
//              distance); groups are picked per block by an optional entropy image; backward references use LZ77 with
//              the 120 nearest (dx, dy) offsets as short codes; an optional colour cache holds recent pixels by hash
// The decoder below follows that order: read everything into an ARGB word image, then undo the transforms in reverse.
// Every read is bounds-checked (past the end the reader supplies zeros and flags the stream as truncated, which the
// caller turns into an error), every table index is validated, sizes are capped.
// (reference counterpart: src/serve/image_inputs.cpp, which decodes WebP through a third-party single-file library.)
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace dgpp::rt::webp {

struct Image {
  int width = 0, height = 0;
  std::vector<uint8_t> rgba;   // rows of width * 4 bytes
};

namespace detail {

[[noreturn]] inline void fail(const std::string& why) { throw std::runtime_error("webp: " + why); }

struct BitReader {
  const uint8_t* p;
  size_t n, pos = 0;     // pos in bits
  bool overrun = false;
  BitReader(const uint8_t* d, size_t size) : p(d), n(size) {}
  uint32_t bits(int count) {     // count <= 25
    uint32_t v = 0;
    for (int i = 0; i < count; ++i, ++pos) {
      const size_t byte = pos >> 3;
      if (byte >= n) { overrun = true; continue; }
      v |= static_cast<uint32_t>((p[byte] >> (pos & 7)) & 1u) << i;
    }
    return v;
  }
  // up to 16 bits without consuming them (zeros past the end)
  uint32_t peek16() const {
    uint32_t v = 0;
    const size_t byte = pos >> 3;
    for (int i = 0; i < 4; ++i)
      if (byte + i < n) v |= static_cast<uint32_t>(p[byte + i]) << (8 * i);
    return (v >> (pos & 7)) & 0xFFFFu;
  }
  void skip(int count) {
    pos += static_cast<size_t>(count);
    if ((pos + 7) / 8 > n + 1) overrun = true;
  }
};

// Canonical prefix code, codes assigned in increasing (length, symbol) order and read LSB-first: a direct table over
// the next kRoot bits for short codes, a bit-by-bit walk for longer ones.
struct PrefixCode {
  static constexpr int kRoot = 8, kMaxLen = 15;
  int single = -1;                       // a code with one symbol reads no bits
  std::vector<uint16_t> fast;            // (len << 12 is too small for 15-bit symbols) -> two tables
  std::vector<uint8_t> fast_len;
  std::vector<int> count;                // codes per length
  std::vector<int> first_code, first_index;
  std::vector<uint16_t> sorted;          // symbols in (length, symbol) order

  void build(const std::vector<uint8_t>& lengths) {
    const int n = static_cast<int>(lengths.size());
    count.assign(kMaxLen + 1, 0);
    int used = 0, last = -1;
    for (int s = 0; s < n; ++s) {
      if (lengths[static_cast<size_t>(s)] > kMaxLen) fail("prefix code length out of range");
      if (lengths[static_cast<size_t>(s)]) { ++count[lengths[static_cast<size_t>(s)]]; ++used; last = s; }
    }
    single = -1;
    if (used == 0) { single = 0; return; }                 // an unused alphabet: any read yields symbol 0
    if (used == 1) { single = last; return; }
    // completeness (Kraft sum == 1)
    long long left = 1;
    for (int len = 1; len <= kMaxLen; ++len) {
      left = left * 2 - count[len];
      if (left < 0) fail("over-subscribed prefix code");
    }
    if (left != 0) fail("incomplete prefix code");
    first_code.assign(kMaxLen + 2, 0);
    first_index.assign(kMaxLen + 2, 0);
    int code = 0, index = 0;
    for (int len = 1; len <= kMaxLen; ++len) {
      first_code[len] = code;
      first_index[len] = index;
      code = (code + count[len]) << 1;
      index += count[len];
    }
    sorted.assign(static_cast<size_t>(used), 0);
    std::vector<int> next(first_index.begin(), first_index.end());
    for (int s = 0; s < n; ++s)
      if (lengths[static_cast<size_t>(s)]) sorted[static_cast<size_t>(next[lengths[static_cast<size_t>(s)]]++)] = static_cast<uint16_t>(s);
    // direct table: the stream carries a code most-significant bit first, i.e. bit-reversed in an LSB-first word
    fast.assign(1u << kRoot, 0);
    fast_len.assign(1u << kRoot, 0);
    for (int len = 1; len <= kRoot; ++len)
      for (int i = 0; i < count[len]; ++i) {
        const int c = first_code[len] + i;
        uint32_t rev = 0;
        for (int b = 0; b < len; ++b) rev |= static_cast<uint32_t>((c >> (len - 1 - b)) & 1) << b;
        for (uint32_t hi = 0; hi < (1u << (kRoot - len)); ++hi) {
          fast[rev | (hi << len)] = sorted[static_cast<size_t>(first_index[len] + i)];
          fast_len[rev | (hi << len)] = static_cast<uint8_t>(len);
        }
      }
  }

  int read(BitReader& br) const {
    if (single >= 0) return single;
    const uint32_t w = br.peek16();
    const uint8_t l = fast_len[w & ((1u << kRoot) - 1)];
    if (l) {
      br.skip(l);
      return fast[w & ((1u << kRoot) - 1)];
    }
    int code = 0;
    for (int len = 1; len <= kMaxLen; ++len) {
      code = (code << 1) | static_cast<int>((w >> (len - 1)) & 1u);
      if (len > kRoot && count[len] && code - first_code[len] < count[len] && code >= first_code[len]) {
        br.skip(len);
        return sorted[static_cast<size_t>(first_index[len] + code - first_code[len])];
      }
    }
    br.overrun = true;       // (cannot happen for a complete code; a damaged table was refused in build)
    br.skip(kMaxLen);
    return 0;
  }
};

constexpr int kCodeLengthOrder[19] = {17, 18, 0, 1, 2, 3, 4, 5, 16, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15};

inline void read_prefix_code(BitReader& br, int alphabet, PrefixCode& out) {
  std::vector<uint8_t> lengths(static_cast<size_t>(alphabet), 0);
  if (br.bits(1)) {                          // simple code: one or two symbols
    const int n = static_cast<int>(br.bits(1)) + 1;
    const int first_bits = br.bits(1) ? 8 : 1;
    const int s0 = static_cast<int>(br.bits(first_bits));
    if (s0 >= alphabet) fail("simple prefix code symbol out of range");
    lengths[static_cast<size_t>(s0)] = 1;
    if (n == 2) {
      const int s1 = static_cast<int>(br.bits(8));
      if (s1 >= alphabet) fail("simple prefix code symbol out of range");
      lengths[static_cast<size_t>(s1)] = 1;
    }
  } else {
    std::vector<uint8_t> cl(19, 0);
    const int ncl = 4 + static_cast<int>(br.bits(4));
    if (ncl > 19) fail("too many code length codes");
    for (int i = 0; i < ncl; ++i) cl[static_cast<size_t>(kCodeLengthOrder[i])] = static_cast<uint8_t>(br.bits(3));
    PrefixCode clc;
    clc.build(cl);
    int max_symbol = alphabet;
    if (br.bits(1)) {
      const int nbits = 2 + 2 * static_cast<int>(br.bits(3));
      max_symbol = 2 + static_cast<int>(br.bits(nbits));
      if (max_symbol > alphabet) fail("prefix code reads more symbols than its alphabet has");
    }
    int prev = 8, s = 0;
    while (s < alphabet) {
      if (max_symbol-- == 0) break;
      if (br.overrun) fail("truncated prefix code");
      const int c = clc.read(br);
      if (c < 16) {
        lengths[static_cast<size_t>(s++)] = static_cast<uint8_t>(c);
        if (c) prev = c;
      } else {
        const int extra = c == 16 ? 2 : (c == 17 ? 3 : 7);
        const int base = c == 18 ? 11 : 3;
        const int rep = base + static_cast<int>(br.bits(extra));
        if (s + rep > alphabet) fail("code length run past the alphabet");
        const uint8_t v = c == 16 ? static_cast<uint8_t>(prev) : 0;
        for (int i = 0; i < rep; ++i) lengths[static_cast<size_t>(s++)] = v;
      }
    }
  }
  out.build(lengths);
}

// the 120 short distance codes: (dx, dy) with dy rows up and dx columns left (negative dx: to the right on the row above)
constexpr int8_t kDistanceMap[120][2] = {
    {0, 1},  {1, 0},  {1, 1},  {-1, 1}, {0, 2},  {2, 0},  {1, 2},  {-1, 2}, {2, 1},  {-2, 1}, {2, 2},  {-2, 2},
    {0, 3},  {3, 0},  {1, 3},  {-1, 3}, {3, 1},  {-3, 1}, {2, 3},  {-2, 3}, {3, 2},  {-3, 2}, {0, 4},  {4, 0},
    {1, 4},  {-1, 4}, {4, 1},  {-4, 1}, {3, 3},  {-3, 3}, {2, 4},  {-2, 4}, {4, 2},  {-4, 2}, {0, 5},  {3, 4},
    {-3, 4}, {4, 3},  {-4, 3}, {5, 0},  {1, 5},  {-1, 5}, {5, 1},  {-5, 1}, {2, 5},  {-2, 5}, {5, 2},  {-5, 2},
    {4, 4},  {-4, 4}, {3, 5},  {-3, 5}, {5, 3},  {-5, 3}, {0, 6},  {6, 0},  {1, 6},  {-1, 6}, {6, 1},  {-6, 1},
    {2, 6},  {-2, 6}, {6, 2},  {-6, 2}, {4, 5},  {-4, 5}, {5, 4},  {-5, 4}, {3, 6},  {-3, 6}, {6, 3},  {-6, 3},
    {0, 7},  {7, 0},  {1, 7},  {-1, 7}, {5, 5},  {-5, 5}, {7, 1},  {-7, 1}, {4, 6},  {-4, 6}, {6, 4},  {-6, 4},
    {2, 7},  {-2, 7}, {7, 2},  {-7, 2}, {3, 7},  {-3, 7}, {7, 3},  {-7, 3}, {5, 6},  {-5, 6}, {6, 5},  {-6, 5},
    {8, 0},  {4, 7},  {-4, 7}, {7, 4},  {-7, 4}, {8, 1},  {8, 2},  {6, 6},  {-6, 6}, {8, 3},  {5, 7},  {-5, 7},
    {7, 5},  {-7, 5}, {8, 4},  {6, 7},  {-6, 7}, {7, 6},  {-7, 6}, {8, 5},  {7, 7},  {-7, 7}, {8, 6},  {8, 7}};

inline int lz77_value(BitReader& br, int prefix) {
  if (prefix < 4) return prefix + 1;
  const int extra = (prefix - 2) >> 1;
  const int offset = (2 + (prefix & 1)) << extra;
  return offset + static_cast<int>(br.bits(extra)) + 1;
}

struct Group {
  PrefixCode green, red, blue, alpha, dist;
};

}  // namespace detail

class LosslessDecoder {
 public:
  static constexpr int kMaxSide = 8192;      // refused before anything of that size is allocated

  LosslessDecoder(const uint8_t* data, size_t size) : br_(data, size) {}

  Image run() {
    using detail::fail;
    if (br_.bits(8) != 0x2f) fail("bad lossless signature");
    width_ = static_cast<int>(br_.bits(14)) + 1;
    height_ = static_cast<int>(br_.bits(14)) + 1;
    br_.bits(1);                                   // alpha hint (the pixels say what they are)
    if (br_.bits(3) != 0) fail("unknown lossless version");
    if (width_ > kMaxSide || height_ > kMaxSide) fail("image side above " + std::to_string(kMaxSide));
    // transforms, in stream order
    int xsize = width_;
    bool seen[4] = {false, false, false, false};
    while (br_.bits(1)) {
      Transform t;
      t.type = static_cast<int>(br_.bits(2));
      if (seen[t.type]) fail("a transform appears twice");
      seen[t.type] = true;
      t.xsize = xsize;
      if (t.type == 0 || t.type == 1) {
        t.bits = static_cast<int>(br_.bits(3)) + 2;
        const int bw = (xsize + (1 << t.bits) - 1) >> t.bits, bh = (height_ + (1 << t.bits) - 1) >> t.bits;
        t.data = decode_stream(bw, bh, false);
      } else if (t.type == 3) {
        const int colors = static_cast<int>(br_.bits(8)) + 1;
        t.data = decode_stream(colors, 1, false);
        for (int i = 1; i < colors; ++i) t.data[static_cast<size_t>(i)] = add_pixels(t.data[static_cast<size_t>(i)], t.data[static_cast<size_t>(i - 1)]);
        t.bits = colors <= 2 ? 3 : (colors <= 4 ? 2 : (colors <= 16 ? 1 : 0));
        xsize = (xsize + (1 << t.bits) - 1) >> t.bits;
      }
      transforms_.push_back(std::move(t));
      if (br_.overrun) fail("truncated transform data");
    }
    std::vector<uint32_t> argb = decode_stream(xsize, height_, true);
    if (br_.overrun) fail("truncated pixel data");
    for (size_t i = transforms_.size(); i-- > 0;) argb = inverse(transforms_[i], argb);
    Image img;
    img.width = width_;
    img.height = height_;
    img.rgba.resize(static_cast<size_t>(width_) * height_ * 4);
    for (size_t i = 0; i < static_cast<size_t>(width_) * height_; ++i) {
      const uint32_t v = argb[i];
      img.rgba[4 * i] = static_cast<uint8_t>(v >> 16);
      img.rgba[4 * i + 1] = static_cast<uint8_t>(v >> 8);
      img.rgba[4 * i + 2] = static_cast<uint8_t>(v);
      img.rgba[4 * i + 3] = static_cast<uint8_t>(v >> 24);
    }
    return img;
  }

 private:
  struct Transform {
    int type = 0, bits = 0, xsize = 0;
    std::vector<uint32_t> data;
  };
  detail::BitReader br_;
  int width_ = 0, height_ = 0;
  std::vector<Transform> transforms_;

  static uint32_t add_pixels(uint32_t a, uint32_t b) {      // per-channel sums modulo 256
    const uint32_t ag = (a & 0xff00ff00u) + (b & 0xff00ff00u);
    const uint32_t rb = (a & 0x00ff00ffu) + (b & 0x00ff00ffu);
    return (ag & 0xff00ff00u) | (rb & 0x00ff00ffu);
  }

  // One entropy-coded ARGB image of xsize x ysize; `main` = the picture itself (may carry an entropy image).
  std::vector<uint32_t> decode_stream(int xsize, int ysize, bool main) {
    using detail::fail;
    int cache_bits = 0;
    if (br_.bits(1)) {
      cache_bits = static_cast<int>(br_.bits(4));
      if (cache_bits < 1 || cache_bits > 11) fail("colour cache size out of range");
    }
    int prefix_bits = 0, groups = 1;
    std::vector<uint32_t> entropy;
    int ew = 0;
    if (main && br_.bits(1)) {
      prefix_bits = static_cast<int>(br_.bits(3)) + 2;
      ew = (xsize + (1 << prefix_bits) - 1) >> prefix_bits;
      const int eh = (ysize + (1 << prefix_bits) - 1) >> prefix_bits;
      entropy = decode_stream(ew, eh, false);
      for (auto& v : entropy) {
        v = (v >> 8) & 0xffffu;
        groups = std::max(groups, static_cast<int>(v) + 1);
      }
      if (groups > 4096) fail("too many prefix code groups");      // bounds the table memory (a few KB per group)
    }
    const int cache_size = cache_bits ? 1 << cache_bits : 0;
    std::vector<detail::Group> g(static_cast<size_t>(groups));
    for (auto& grp : g) {
      detail::read_prefix_code(br_, 256 + 24 + cache_size, grp.green);
      detail::read_prefix_code(br_, 256, grp.red);
      detail::read_prefix_code(br_, 256, grp.blue);
      detail::read_prefix_code(br_, 256, grp.alpha);
      detail::read_prefix_code(br_, 40, grp.dist);
      if (br_.overrun) fail("truncated prefix codes");
    }
    std::vector<uint32_t> cache(static_cast<size_t>(cache_size), 0);
    auto cache_put = [&](uint32_t v) {
      if (cache_bits) cache[static_cast<size_t>((0x1e35a7bdu * v) >> (32 - cache_bits))] = v;
    };
    const size_t total = static_cast<size_t>(xsize) * ysize;
    std::vector<uint32_t> px(total, 0);
    size_t pos = 0;
    int x = 0, y = 0;
    while (pos < total) {
      if (br_.overrun) fail("truncated pixel data");
      const detail::Group& grp = entropy.empty() ? g[0] : g[entropy[static_cast<size_t>(y >> prefix_bits) * ew + (x >> prefix_bits)]];
      const int s = grp.green.read(br_);
      if (s < 256) {
        const uint32_t r = static_cast<uint32_t>(grp.red.read(br_)), b = static_cast<uint32_t>(grp.blue.read(br_)),
                       a = static_cast<uint32_t>(grp.alpha.read(br_));
        const uint32_t v = (a << 24) | (r << 16) | (static_cast<uint32_t>(s) << 8) | b;
        px[pos++] = v;
        cache_put(v);
        if (++x == xsize) { x = 0; ++y; }
      } else if (s < 256 + 24) {
        const int length = detail::lz77_value(br_, s - 256);
        const int dcode = detail::lz77_value(br_, grp.dist.read(br_));
        int64_t dist;
        if (dcode > 120) {
          dist = dcode - 120;
        } else {
          const int dx = detail::kDistanceMap[dcode - 1][0], dy = detail::kDistanceMap[dcode - 1][1];
          dist = static_cast<int64_t>(dy) * xsize + dx;
          if (dist < 1) dist = 1;
        }
        if (dist > static_cast<int64_t>(pos)) fail("backward reference before the first pixel");
        if (static_cast<size_t>(length) > total - pos) fail("backward reference runs past the image");
        for (int i = 0; i < length; ++i) {
          const uint32_t v = px[pos - static_cast<size_t>(dist)];
          px[pos++] = v;
          cache_put(v);
        }
        x += length;
        while (x >= xsize) { x -= xsize; ++y; }
      } else {
        const int idx = s - (256 + 24);
        if (idx >= cache_size) fail("colour cache index out of range");
        const uint32_t v = cache[static_cast<size_t>(idx)];
        px[pos++] = v;
        cache_put(v);
        if (++x == xsize) { x = 0; ++y; }
      }
    }
    return px;
  }

  // ---- inverse transforms
  static int clamp255(int v) { return v < 0 ? 0 : (v > 255 ? 255 : v); }
  static uint32_t avg2(uint32_t a, uint32_t b) { return (((a ^ b) & 0xfefefefeu) >> 1) + (a & b); }
  static uint32_t select(uint32_t L, uint32_t T, uint32_t TL) {
    int pl = 0, pt = 0;      // Manhattan distances of (L + T - TL) to T and to L
    for (int sh = 0; sh < 32; sh += 8) {
      const int l = static_cast<int>((L >> sh) & 255), t = static_cast<int>((T >> sh) & 255), tl = static_cast<int>((TL >> sh) & 255);
      pl += std::abs(t - tl);    // |p - L| = |T - TL|
      pt += std::abs(l - tl);    // |p - T| = |L - TL|
    }
    return pl < pt ? L : T;
  }
  static uint32_t clamp_add_sub_full(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t out = 0;
    for (int sh = 0; sh < 32; sh += 8)
      out |= static_cast<uint32_t>(clamp255(static_cast<int>((a >> sh) & 255) + static_cast<int>((b >> sh) & 255) -
                                            static_cast<int>((c >> sh) & 255))) << sh;
    return out;
  }
  static uint32_t clamp_add_sub_half(uint32_t a, uint32_t b) {
    uint32_t out = 0;
    for (int sh = 0; sh < 32; sh += 8) {
      const int av = static_cast<int>((a >> sh) & 255), bv = static_cast<int>((b >> sh) & 255);
      out |= static_cast<uint32_t>(clamp255(av + (av - bv) / 2)) << sh;
    }
    return out;
  }
  static uint32_t predict(int mode, uint32_t L, uint32_t T, uint32_t TR, uint32_t TL) {
    switch (mode) {
      case 0: return 0xff000000u;
      case 1: return L;
      case 2: return T;
      case 3: return TR;
      case 4: return TL;
      case 5: return avg2(avg2(L, TR), T);
      case 6: return avg2(L, TL);
      case 7: return avg2(L, T);
      case 8: return avg2(TL, T);
      case 9: return avg2(T, TR);
      case 10: return avg2(avg2(L, TL), avg2(T, TR));
      case 11: return select(L, T, TL);
      case 12: return clamp_add_sub_full(L, T, TL);
      case 13: return clamp_add_sub_half(avg2(L, T), TL);
      default: return 0xff000000u;     // modes 14, 15 are reserved: treated as black
    }
  }

  std::vector<uint32_t> inverse(const Transform& t, std::vector<uint32_t>& in) const {
    const int w = t.xsize, h = height_;
    if (t.type == 2) {                                   // add green to red and blue
      for (auto& v : in) {
        const uint32_t g = (v >> 8) & 255;
        v = (v & 0xff00ff00u) | ((((v >> 16) + g) & 255) << 16) | ((v + g) & 255);
      }
      return std::move(in);
    }
    if (t.type == 0) {                                   // spatial prediction
      const int bw = (w + (1 << t.bits) - 1) >> t.bits;
      for (int y = 0; y < h; ++y)
        for (int x = 0; x < w; ++x) {
          const size_t i = static_cast<size_t>(y) * w + x;
          uint32_t pred;
          if (y == 0) pred = x == 0 ? 0xff000000u : in[i - 1];
          else if (x == 0) pred = in[i - w];
          else {
            const int mode = static_cast<int>((t.data[static_cast<size_t>(y >> t.bits) * bw + (x >> t.bits)] >> 8) & 15);
            // in memory order the top-right neighbour of the last column is the first pixel of the current row,
            // which is what the format prescribes there
            const uint32_t TR = in[i - w + 1];
            pred = predict(mode, in[i - 1], in[i - w], TR, in[i - w - 1]);
          }
          in[i] = add_pixels(in[i], pred);
        }
      return std::move(in);
    }
    if (t.type == 1) {                                   // cross-colour
      const int bw = (w + (1 << t.bits) - 1) >> t.bits;
      auto delta = [](int8_t m, int8_t c) { return (static_cast<int>(m) * static_cast<int>(c)) >> 5; };
      for (int y = 0; y < h; ++y)
        for (int x = 0; x < w; ++x) {
          const uint32_t e = t.data[static_cast<size_t>(y >> t.bits) * bw + (x >> t.bits)];
          const int8_t g2r = static_cast<int8_t>(e & 255), g2b = static_cast<int8_t>((e >> 8) & 255), r2b = static_cast<int8_t>((e >> 16) & 255);
          uint32_t& v = in[static_cast<size_t>(y) * w + x];
          const int8_t g = static_cast<int8_t>((v >> 8) & 255);
          int r = static_cast<int>((v >> 16) & 255), b = static_cast<int>(v & 255);
          r = (r + delta(g2r, g)) & 255;
          b = (b + delta(g2b, g)) & 255;
          b = (b + delta(r2b, static_cast<int8_t>(r))) & 255;
          v = (v & 0xff00ff00u) | (static_cast<uint32_t>(r) << 16) | static_cast<uint32_t>(b);
        }
      return std::move(in);
    }
    // colour indexing: `in` is (xsize packed) x h indices in the green channel
    const int pw = (w + (1 << t.bits) - 1) >> t.bits;
    const int per = 1 << t.bits, bits_per = 8 >> t.bits;
    std::vector<uint32_t> out(static_cast<size_t>(w) * h);
    for (int y = 0; y < h; ++y)
      for (int x = 0; x < w; ++x) {
        const uint32_t packed = (in[static_cast<size_t>(y) * pw + (x >> t.bits)] >> 8) & 255;
        const uint32_t idx = t.bits ? (packed >> ((x & (per - 1)) * bits_per)) & ((1u << bits_per) - 1) : packed;
        out[static_cast<size_t>(y) * w + x] = idx < t.data.size() ? t.data[idx] : 0u;
      }
    return out;
  }
};

// RIFF container: plain lossless file, or the extended form whose image chunk is lossless.
inline Image decode(const uint8_t* data, size_t size) {
  using detail::fail;
  if (size < 20 || std::memcmp(data, "RIFF", 4) != 0 || std::memcmp(data + 8, "WEBP", 4) != 0) fail("not a RIFF / WEBP file");
  size_t pos = 12;
  while (pos + 8 <= size) {
    const uint32_t len = static_cast<uint32_t>(data[pos + 4]) | (static_cast<uint32_t>(data[pos + 5]) << 8) |
                         (static_cast<uint32_t>(data[pos + 6]) << 16) | (static_cast<uint32_t>(data[pos + 7]) << 24);
    const uint8_t* body = data + pos + 8;
    if (len > size - pos - 8) fail("truncated chunk");
    if (std::memcmp(data + pos, "VP8L", 4) == 0) return LosslessDecoder(body, len).run();
    if (std::memcmp(data + pos, "VP8 ", 4) == 0) fail("lossy (VP8) files are not supported: send PNG, JPEG or lossless WebP");
    if (std::memcmp(data + pos, "ANIM", 4) == 0 || std::memcmp(data + pos, "ANMF", 4) == 0) fail("animated files are not supported");
    pos += 8 + static_cast<size_t>(len) + (len & 1);       // VP8X, ICCP, EXIF, ALPH ... are skipped
  }
  fail("no image chunk");
}

}  // namespace dgpp::rt::webp
