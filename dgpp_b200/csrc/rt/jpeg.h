// JPEG decoder for inline image inputs: baseline and extended sequential (SOF0 / SOF1, 8-bit) and progressive (SOF2)
// Huffman streams, 1 or 3 components (grey, YCbCr per JFIF, RGB when an Adobe marker says so), any sampling factors
// up to 4, restart intervals, 8- and 16-bit quantisation tables.  Output: interleaved 8-bit grey or RGB.
//
// Structure: every scan decodes into a coefficient store (int16 per component, blocks padded to whole MCUs), which is
// what the progressive refinement passes need; sequential files take the same route.  After the last scan each block
// is dequantised and transformed (separable float inverse DCT, rounded once), chroma planes are brought to full
// resolution (triangle filter for the common 2x factors, as libjpeg's default upsampler does, so that results stay
// within a level or two of it; replication for other factors) and converted to RGB.
// Not handled (refused with a message): arithmetic coding, lossless / hierarchical processes, 12-bit samples, 4
// components (CMYK / YCCK).
// (reference counterpart: src/serve/image_inputs.cpp, which decodes through a third-party single-header library.)
#pragma once

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace dgpp::rt::jpeg {

struct Image {
  int width = 0, height = 0, channels = 0;
  std::vector<uint8_t> pixels;  // rows of width * channels bytes
};

namespace detail {

[[noreturn]] inline void fail(const std::string& why) { throw std::runtime_error("jpeg: " + why); }

constexpr uint8_t kZigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                                 41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                                 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

// Canonical Huffman table: codes of length <= kFast resolve through one lookup, longer ones through the per-length
// (first code, first index) pairs.
struct Huffman {
  static constexpr int kFast = 9;
  bool present = false;
  uint8_t symbols[256] = {};
  int32_t maxcode[18] = {};   // largest code of each length, left-aligned to 16 bits, +1; maxcode[17] = sentinel
  int32_t delta[17] = {};     // symbol index = code + delta[len]
  uint16_t fast[1 << kFast] = {};  // (len << 8) | symbol, 0 = not a short code

  void build(const uint8_t counts[16], const uint8_t* syms, int n) {
    std::memcpy(symbols, syms, static_cast<size_t>(n));
    std::fill(std::begin(fast), std::end(fast), uint16_t{0});
    int code = 0, k = 0;
    for (int len = 1; len <= 16; ++len) {
      delta[len] = k - code;
      for (int i = 0; i < counts[len - 1]; ++i, ++k, ++code) {
        if (len <= kFast) {
          const int first = code << (kFast - len);
          for (int j = 0; j < (1 << (kFast - len)); ++j) fast[first + j] = static_cast<uint16_t>((len << 8) | symbols[k]);
        }
      }
      if (code > (1 << len)) fail("Huffman table assigns more codes than a length has");
      maxcode[len] = code << (16 - len);
      code <<= 1;
    }
    maxcode[17] = INT32_MAX;
    present = true;
  }
};

// Entropy-coded segment reader: removes 0xFF00 stuffing, stops at any other marker (which it keeps for the caller)
// and then supplies zero bits, as the standard prescribes for a truncated segment.
struct BitReader {
  const uint8_t* p;
  const uint8_t* end;
  uint32_t acc = 0;   // bits, most significant first
  int have = 0;
  int marker = 0;     // marker byte met inside the segment (0 = none yet)

  BitReader(const uint8_t* b, const uint8_t* e) : p(b), end(e) {}

  void fill() {
    while (have <= 24) {
      uint32_t byte = 0;
      if (!marker && p < end) {
        byte = *p++;
        if (byte == 0xFF) {
          while (p < end && *p == 0xFF) ++p;     // fill bytes
          const uint8_t next = p < end ? *p++ : 0xD9;
          if (next != 0) {
            marker = next;
            byte = 0;
          }
        }
      }
      acc |= byte << (24 - have);
      have += 8;
    }
  }
  int bit() {
    if (have < 1) fill();
    const int b = static_cast<int>(acc >> 31);
    acc <<= 1;
    --have;
    return b;
  }
  int bits(int n) {      // n in 0..16
    if (n == 0) return 0;
    if (have < n) fill();
    const int v = static_cast<int>(acc >> (32 - n));
    acc <<= n;
    have -= n;
    return v;
  }
  // value of an n-bit magnitude field with the sign convention of the standard (EXTEND)
  int extend(int n) {
    if (n == 0) return 0;
    const int v = bits(n);
    return v < (1 << (n - 1)) ? v - (1 << n) + 1 : v;
  }
  int symbol(const Huffman& h) {
    if (have < 16) fill();
    const uint16_t f = h.fast[acc >> (32 - Huffman::kFast)];
    if (f) {
      const int len = f >> 8;
      acc <<= len;
      have -= len;
      return f & 0xFF;
    }
    const int32_t top = static_cast<int32_t>(acc >> 16);
    int len = Huffman::kFast + 1;
    while (len <= 16 && top >= h.maxcode[len]) ++len;
    if (len > 16) fail("bad Huffman code");
    const int code = static_cast<int>(acc >> (32 - len));
    acc <<= len;
    have -= len;
    const int idx = code + h.delta[len];
    if (idx < 0 || idx > 255) fail("bad Huffman code");
    return h.symbols[idx];
  }
  // drop the bits of the current byte and take the restart marker that must follow
  void restart() {
    acc = 0;
    have = 0;
    if (!marker) {      // the marker was not reached through fill(): look for it in the bytes
      while (p + 1 < end && !(p[0] == 0xFF && p[1] != 0 && p[1] != 0xFF)) ++p;
      if (p + 1 < end) {
        marker = p[1];
        p += 2;
      }
    }
    if (marker >= 0xD0 && marker <= 0xD7) marker = 0;   // consumed; anything else ends the scan (zeros follow)
  }
};

struct Component {
  int id = 0, h = 1, v = 1, tq = 0;
  int td = 0, ta = 0;          // Huffman selectors of the current scan
  int bw = 0, bh = 0;          // blocks per row / column of the store (padded to whole MCUs)
  int pred = 0;                // DC predictor
  std::vector<int16_t> coef;   // bw * bh * 64, natural (not zigzag) order
  std::vector<uint8_t> plane;  // bw * 8 by bh * 8 samples after the inverse transform
};

inline uint8_t clamp8(float v) {
  const int i = static_cast<int>(std::lrintf(v));
  return static_cast<uint8_t>(i < 0 ? 0 : (i > 255 ? 255 : i));
}

// Separable float inverse DCT of one dequantised block, level shift and clamp included.
inline void idct_block(const float* in, uint8_t* out, int stride) {
  static const std::array<float, 64> basis = [] {
    std::array<float, 64> b{};
    for (int x = 0; x < 8; ++x)
      for (int u = 0; u < 8; ++u)
        b[static_cast<size_t>(x * 8 + u)] = (u == 0 ? std::sqrt(0.125f) : 0.5f) *
                                            std::cos((2.0f * static_cast<float>(x) + 1.0f) * static_cast<float>(u) * 3.14159265358979323846f / 16.0f);
    return b;
  }();
  float tmp[64];
  for (int v = 0; v < 8; ++v)          // rows: tmp[v][x] = sum_u basis[x][u] in[v][u]
    for (int x = 0; x < 8; ++x) {
      float s = 0.f;
      for (int u = 0; u < 8; ++u) s += basis[static_cast<size_t>(x * 8 + u)] * in[v * 8 + u];
      tmp[v * 8 + x] = s;
    }
  for (int y = 0; y < 8; ++y)
    for (int x = 0; x < 8; ++x) {
      float s = 0.f;
      for (int v = 0; v < 8; ++v) s += basis[static_cast<size_t>(y * 8 + v)] * tmp[v * 8 + x];
      out[y * stride + x] = clamp8(s + 128.f);
    }
}

}  // namespace detail

class Decoder {
 public:
  Decoder(const uint8_t* data, size_t size) : begin_(data), end_(data + size) {}

  Image run() {
    using detail::fail;
    const uint8_t* p = begin_;
    if (end_ - p < 4 || p[0] != 0xFF || p[1] != 0xD8) fail("missing SOI marker");
    p += 2;
    bool done = false;
    while (!done) {
      // next marker (fill bytes allowed)
      while (p < end_ && *p != 0xFF) ++p;
      while (p < end_ && *p == 0xFF) ++p;
      if (p >= end_) break;
      const int m = *p++;
      if (m == 0xD9) break;                                 // EOI
      if (m == 0x00 || m == 0x01 || (m >= 0xD0 && m <= 0xD7)) continue;  // stuffed byte / standalone markers
      if (end_ - p < 2) fail("truncated segment");
      const int len = (p[0] << 8) | p[1];
      if (len < 2 || end_ - p < len) fail("truncated segment");
      const uint8_t* s = p + 2;
      const uint8_t* e = p + len;
      p = e;
      switch (m) {
        case 0xDB: read_dqt(s, e); break;
        case 0xC4: read_dht(s, e); break;
        case 0xC0: case 0xC1: case 0xC2: read_sof(s, e, m == 0xC2); break;
        case 0xDD:
          if (e - s < 2) fail("bad DRI");
          restart_interval_ = (s[0] << 8) | s[1];
          break;
        case 0xEE:                                          // Adobe: transform flag in byte 11
          if (e - s >= 12 && std::memcmp(s, "Adobe", 5) == 0) adobe_transform_ = s[11];
          break;
        case 0xDA:
          p = read_scan(s, e);
          break;
        case 0xC3: case 0xC5: case 0xC6: case 0xC7: case 0xCB: case 0xCD: case 0xCE: case 0xCF:
          fail("lossless / hierarchical processes are not supported");
        case 0xC9: case 0xCA:
          fail("arithmetic coding is not supported");
        default: break;                                     // APPn, COM and anything else: skipped
      }
    }
    if (comps_.empty()) fail("no frame header");
    if (!saw_scan_) fail("no scan");
    return finish();
  }

 private:
  const uint8_t* begin_;
  const uint8_t* end_;
  uint16_t quant_[4][64] = {};
  bool quant_set_[4] = {};
  detail::Huffman dc_[4], ac_[4];
  std::vector<detail::Component> comps_;
  int width_ = 0, height_ = 0, hmax_ = 1, vmax_ = 1, mcus_x_ = 0, mcus_y_ = 0;
  bool progressive_ = false, saw_scan_ = false;
  int restart_interval_ = 0, adobe_transform_ = -1;
  int eobrun_ = 0;

  void read_dqt(const uint8_t* s, const uint8_t* e) {
    while (s < e) {
      const int pq = *s >> 4, tq = *s & 15;
      ++s;
      if (tq > 3 || pq > 1) detail::fail("bad quantisation table header");
      if (e - s < 64 * (pq + 1)) detail::fail("truncated quantisation table");
      for (int i = 0; i < 64; ++i) {
        const int v = pq ? ((s[0] << 8) | s[1]) : s[0];
        s += pq + 1;
        quant_[tq][detail::kZigzag[i]] = static_cast<uint16_t>(v);
      }
      quant_set_[tq] = true;
    }
  }

  void read_dht(const uint8_t* s, const uint8_t* e) {
    while (s < e) {
      const int tc = *s >> 4, th = *s & 15;
      ++s;
      if (tc > 1 || th > 3 || e - s < 16) detail::fail("bad Huffman table header");
      int n = 0;
      for (int i = 0; i < 16; ++i) n += s[i];
      if (n > 256 || e - s < 16 + n) detail::fail("truncated Huffman table");
      (tc ? ac_[th] : dc_[th]).build(s, s + 16, n);
      s += 16 + n;
    }
  }

  void read_sof(const uint8_t* s, const uint8_t* e, bool progressive) {
    using detail::fail;
    if (!comps_.empty()) fail("more than one frame");
    if (e - s < 6) fail("truncated frame header");
    if (s[0] != 8) fail("only 8-bit samples are supported");
    height_ = (s[1] << 8) | s[2];
    width_ = (s[3] << 8) | s[4];
    const int n = s[5];
    if (width_ <= 0 || height_ <= 0) fail("empty image (a DNL-defined height is not supported)");
    if (static_cast<int64_t>(width_) * height_ > (int64_t{1} << 28)) fail("image too large");
    if (n != 1 && n != 3) fail("only 1 or 3 components are supported (got " + std::to_string(n) + ")");
    if (e - s < 6 + 3 * n) fail("truncated frame header");
    progressive_ = progressive;
    comps_.resize(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) {
      auto& c = comps_[static_cast<size_t>(i)];
      c.id = s[6 + 3 * i];
      c.h = s[7 + 3 * i] >> 4;
      c.v = s[7 + 3 * i] & 15;
      c.tq = s[8 + 3 * i];
      if (c.h < 1 || c.h > 4 || c.v < 1 || c.v > 4 || c.tq > 3) fail("bad component parameters");
      hmax_ = std::max(hmax_, c.h);
      vmax_ = std::max(vmax_, c.v);
    }
    if (n == 1) comps_[0].h = comps_[0].v = hmax_ = vmax_ = 1;   // a single component is never interleaved
    mcus_x_ = (width_ + 8 * hmax_ - 1) / (8 * hmax_);
    mcus_y_ = (height_ + 8 * vmax_ - 1) / (8 * vmax_);
    for (auto& c : comps_) {
      c.bw = mcus_x_ * c.h;
      c.bh = mcus_y_ * c.v;
      c.coef.assign(static_cast<size_t>(c.bw) * c.bh * 64, 0);
    }
  }

  // ---- block decoders (coefficients in natural order)
  void block_sequential(detail::BitReader& br, detail::Component& c, int16_t* blk) {
    const int t = br.symbol(dc_[c.td]);
    if (t > 11) detail::fail("bad DC category");
    c.pred = std::clamp(c.pred + br.extend(t), -32768, 32767);
    blk[0] = static_cast<int16_t>(c.pred);
    const detail::Huffman& h = ac_[c.ta];
    for (int k = 1; k < 64;) {
      const int rs = br.symbol(h);
      const int r = rs >> 4, sz = rs & 15;
      if (sz == 0) {
        if (r != 15) break;          // EOB
        k += 16;
        continue;
      }
      k += r;
      if (k > 63) detail::fail("AC coefficient index out of range");
      blk[detail::kZigzag[k++]] = static_cast<int16_t>(br.extend(sz));
    }
  }

  void block_dc_first(detail::BitReader& br, detail::Component& c, int16_t* blk, int al) {
    const int t = br.symbol(dc_[c.td]);
    if (t > 11) detail::fail("bad DC category");
    c.pred = std::clamp(c.pred + br.extend(t), -32768, 32767);
    blk[0] = static_cast<int16_t>(c.pred * (1 << al));
  }

  void block_ac_first(detail::BitReader& br, const detail::Huffman& h, int16_t* blk, int ss, int se, int al) {
    if (eobrun_ > 0) {
      --eobrun_;
      return;
    }
    for (int k = ss; k <= se;) {
      const int rs = br.symbol(h);
      const int r = rs >> 4, sz = rs & 15;
      if (sz == 0) {
        if (r < 15) {
          eobrun_ = (1 << r) - 1;
          if (r) eobrun_ += br.bits(r);
          break;
        }
        k += 16;
        continue;
      }
      k += r;
      if (k > se) detail::fail("AC coefficient index out of range");
      blk[detail::kZigzag[k++]] = static_cast<int16_t>(br.extend(sz) * (1 << al));
    }
  }

  void block_ac_refine(detail::BitReader& br, const detail::Huffman& h, int16_t* blk, int ss, int se, int al) {
    const int p1 = 1 << al, m1 = -(1 << al);
    int k = ss;
    if (eobrun_ == 0) {
      for (; k <= se;) {
        const int rs = br.symbol(h);
        int r = rs >> 4;
        const int sz = rs & 15;
        int value = 0;
        if (sz == 0) {
          if (r < 15) {
            eobrun_ = 1 << r;
            if (r) eobrun_ += br.bits(r);
            break;                 // the rest of the band is handled as part of the run below
          }
        } else {
          if (sz != 1) detail::fail("bad refinement symbol");
          value = br.bit() ? p1 : m1;
        }
        // skip r zero-history coefficients, refining the non-zero ones that are passed on the way
        for (; k <= se; ++k) {
          int16_t& co = blk[detail::kZigzag[k]];
          if (co != 0) {
            if (br.bit() && (co & p1) == 0) co = static_cast<int16_t>(co + (co >= 0 ? p1 : m1));
          } else {
            if (r == 0) {
              if (value) co = static_cast<int16_t>(value);
              ++k;
              break;
            }
            --r;
          }
        }
      }
    }
    if (eobrun_ > 0) {
      for (; k <= se; ++k) {
        int16_t& co = blk[detail::kZigzag[k]];
        if (co != 0 && br.bit() && (co & p1) == 0) co = static_cast<int16_t>(co + (co >= 0 ? p1 : m1));
      }
      --eobrun_;
    }
  }

  // ---- one scan; returns the position after its entropy-coded data
  const uint8_t* read_scan(const uint8_t* s, const uint8_t* e) {
    using detail::fail;
    if (comps_.empty()) fail("scan before the frame header");
    if (e - s < 1) fail("truncated scan header");
    const int n = s[0];
    if (n < 1 || n > static_cast<int>(comps_.size()) || e - s < 4 + 2 * n) fail("bad scan header");
    std::vector<detail::Component*> sc;
    for (int i = 0; i < n; ++i) {
      detail::Component* found = nullptr;
      for (auto& c : comps_)
        if (c.id == s[1 + 2 * i]) found = &c;
      if (!found) fail("scan names an unknown component");
      found->td = s[2 + 2 * i] >> 4;
      found->ta = s[2 + 2 * i] & 15;
      if (found->td > 3 || found->ta > 3) fail("bad table selector");
      sc.push_back(found);
    }
    const int ss = s[1 + 2 * n], se = s[2 + 2 * n], ah = s[3 + 2 * n] >> 4, al = s[3 + 2 * n] & 15;
    if (progressive_) {
      if (ss > se || se > 63 || (ss == 0 && se != 0) || (ss > 0 && n != 1) || al > 13) fail("bad progressive scan parameters");
    } else if (ss != 0 || se != 63 || ah != 0 || al != 0) {
      fail("bad sequential scan parameters");
    }
    for (auto* c : sc) {
      const bool need_dc = !progressive_ || (ss == 0 && ah == 0);
      const bool need_ac = !progressive_ || ss > 0;
      if (need_dc && !dc_[c->td].present) fail("scan uses an undefined DC table");
      if (need_ac && !ac_[c->ta].present) fail("scan uses an undefined AC table");
      c->pred = 0;
    }
    eobrun_ = 0;
    saw_scan_ = true;
    detail::BitReader br(e, end_);

    auto decode_block = [&](detail::Component& c, int bx, int by) {
      int16_t* blk = &c.coef[(static_cast<size_t>(by) * c.bw + bx) * 64];
      if (!progressive_) block_sequential(br, c, blk);
      else if (ss == 0 && ah == 0) block_dc_first(br, c, blk, al);
      else if (ss == 0) { if (br.bit()) blk[0] = static_cast<int16_t>(blk[0] | (1 << al)); }
      else if (ah == 0) block_ac_first(br, ac_[c.ta], blk, ss, se, al);
      else block_ac_refine(br, ac_[c.ta], blk, ss, se, al);
    };
    auto restart_if_due = [&](int64_t unit, int64_t units) {
      if (restart_interval_ && (unit + 1) % restart_interval_ == 0 && unit + 1 < units) {
        br.restart();
        for (auto* c : sc) c->pred = 0;
        eobrun_ = 0;
      }
    };

    if (n == 1) {
      // non-interleaved: the component's own blocks, only those that cover the image
      detail::Component& c = *sc[0];
      const int w = (((width_ * c.h + hmax_ - 1) / hmax_) + 7) / 8;
      const int h = (((height_ * c.v + vmax_ - 1) / vmax_) + 7) / 8;
      const int64_t units = static_cast<int64_t>(w) * h;
      int64_t u = 0;
      for (int by = 0; by < h; ++by)
        for (int bx = 0; bx < w; ++bx, ++u) {
          decode_block(c, bx, by);
          restart_if_due(u, units);
        }
    } else {
      const int64_t units = static_cast<int64_t>(mcus_x_) * mcus_y_;
      int64_t u = 0;
      for (int my = 0; my < mcus_y_; ++my)
        for (int mx = 0; mx < mcus_x_; ++mx, ++u) {
          for (auto* c : sc)
            for (int v = 0; v < c->v; ++v)
              for (int h = 0; h < c->h; ++h) decode_block(*c, mx * c->h + h, my * c->v + v);
          restart_if_due(u, units);
        }
    }
    // position of the marker that ended the entropy-coded data
    if (br.marker) {
      const uint8_t* q = br.p - 2;
      return q < e ? e : q;
    }
    return br.p;
  }

  // ---- coefficients -> samples -> pixels
  // One full-resolution row of a component: `out` gets `width_` samples of image row y.
  void upsampled_row(const detail::Component& c, int y, std::vector<uint8_t>& out) const {
    const int stride = c.bw * 8;
    const int cw = (width_ * c.h + hmax_ - 1) / hmax_;      // samples of the component that carry image data
    const int ch = (height_ * c.v + vmax_ - 1) / vmax_;
    const int fx = hmax_ / c.h, fy = vmax_ / c.v;
    const bool exact = hmax_ % c.h == 0 && vmax_ % c.v == 0;
    auto row = [&](int r) { return &c.plane[static_cast<size_t>(std::clamp(r, 0, ch - 1)) * stride]; };
    if (exact && fx == 1 && fy == 1) {
      std::memcpy(out.data(), row(y), static_cast<size_t>(width_));
      return;
    }
    if (exact && fx == 2 && fy == 1) {
      // triangle filter along the row: 3/4 of the nearer sample, 1/4 of the further one
      const uint8_t* r = row(y);
      for (int x = 0; x < width_; ++x) {
        const int i = x >> 1;
        const int near_ = r[std::min(i, cw - 1)];
        const int far_ = r[std::clamp((x & 1) ? i + 1 : i - 1, 0, cw - 1)];
        out[static_cast<size_t>(x)] = static_cast<uint8_t>((3 * near_ + far_ + ((x & 1) ? 2 : 1)) >> 2);
      }
      return;
    }
    if (exact && fx == 2 && fy == 2) {
      // the same filter in both directions: 9/16, 3/16, 3/16, 1/16
      const int j = y >> 1;
      const uint8_t* r0 = row(j);
      const uint8_t* r1 = row((y & 1) ? j + 1 : j - 1);
      auto col = [&](int i) { return 3 * r0[std::clamp(i, 0, cw - 1)] + r1[std::clamp(i, 0, cw - 1)]; };
      for (int x = 0; x < width_; ++x) {
        const int i = x >> 1;
        const int near_ = col(i), far_ = col((x & 1) ? i + 1 : i - 1);
        out[static_cast<size_t>(x)] = static_cast<uint8_t>((3 * near_ + far_ + ((x & 1) ? 7 : 8)) >> 4);
      }
      return;
    }
    if (exact && fx == 1 && fy == 2) {
      const int j = y >> 1;
      const uint8_t* r0 = row(j);
      const uint8_t* r1 = row((y & 1) ? j + 1 : j - 1);
      for (int x = 0; x < width_; ++x)
        out[static_cast<size_t>(x)] = static_cast<uint8_t>((3 * r0[std::min(x, cw - 1)] + r1[std::min(x, cw - 1)] + ((y & 1) ? 2 : 1)) >> 2);
      return;
    }
    // other ratios: nearest sample
    const uint8_t* r = row(static_cast<int>(static_cast<int64_t>(y) * c.v / vmax_));
    for (int x = 0; x < width_; ++x)
      out[static_cast<size_t>(x)] = r[std::min(static_cast<int>(static_cast<int64_t>(x) * c.h / hmax_), cw - 1)];
  }

  Image finish() {
    for (auto& c : comps_) {
      if (!quant_set_[c.tq]) detail::fail("component uses an undefined quantisation table");
      const uint16_t* q = quant_[c.tq];
      const int stride = c.bw * 8;
      c.plane.assign(static_cast<size_t>(stride) * c.bh * 8, 0);
      float deq[64];
      for (int by = 0; by < c.bh; ++by)
        for (int bx = 0; bx < c.bw; ++bx) {
          const int16_t* blk = &c.coef[(static_cast<size_t>(by) * c.bw + bx) * 64];
          for (int i = 0; i < 64; ++i) deq[i] = static_cast<float>(blk[i]) * static_cast<float>(q[i]);
          detail::idct_block(deq, &c.plane[static_cast<size_t>(by) * 8 * stride + static_cast<size_t>(bx) * 8], stride);
        }
      c.coef.clear();
      c.coef.shrink_to_fit();
    }
    Image img;
    img.width = width_;
    img.height = height_;
    img.channels = comps_.size() == 1 ? 1 : 3;
    img.pixels.resize(static_cast<size_t>(width_) * height_ * img.channels);
    if (comps_.size() == 1) {
      const auto& c = comps_[0];
      for (int y = 0; y < height_; ++y)
        std::memcpy(&img.pixels[static_cast<size_t>(y) * width_], &c.plane[static_cast<size_t>(y) * c.bw * 8], static_cast<size_t>(width_));
      return img;
    }
    // three components: YCbCr unless an Adobe marker says "no transform" (or, without any marker, the component ids
    // spell R, G, B)
    bool rgb = adobe_transform_ == 0;
    if (adobe_transform_ < 0 && comps_[0].id == 'R' && comps_[1].id == 'G' && comps_[2].id == 'B') rgb = true;
    std::vector<uint8_t> r0(static_cast<size_t>(width_)), r1(r0.size()), r2(r0.size());
    for (int y = 0; y < height_; ++y) {
      upsampled_row(comps_[0], y, r0);
      upsampled_row(comps_[1], y, r1);
      upsampled_row(comps_[2], y, r2);
      uint8_t* o = &img.pixels[static_cast<size_t>(y) * width_ * 3];
      for (int x = 0; x < width_; ++x, o += 3) {
        if (rgb) {
          o[0] = r0[static_cast<size_t>(x)];
          o[1] = r1[static_cast<size_t>(x)];
          o[2] = r2[static_cast<size_t>(x)];
        } else {
          const float Y = r0[static_cast<size_t>(x)], cb = static_cast<float>(r1[static_cast<size_t>(x)]) - 128.f,
                      cr = static_cast<float>(r2[static_cast<size_t>(x)]) - 128.f;
          o[0] = detail::clamp8(Y + 1.402f * cr);
          o[1] = detail::clamp8(Y - 0.344136f * cb - 0.714136f * cr);
          o[2] = detail::clamp8(Y + 1.772f * cb);
        }
      }
    }
    return img;
  }
};

inline Image decode(const uint8_t* data, size_t size) { return Decoder(data, size).run(); }

}  // namespace dgpp::rt::jpeg
