// JPEG decoder (ITU-T T.81 sequential and progressive DCT, Huffman coding, 8-bit samples) for image inputs of chat requests.
//
// The reference decodes JPEG data URLs with nvJPEG on the GPU (kernels/oracle/bridge/vision.cpp:204-228) after the
// server recognised the format (crates/agens-server/src/vision.rs:126-135).  Here the decode runs on the host next to
// the PNG / PPM readers: one, three or four (Adobe CMYK / YCCK) components, any 1x / 2x sampling factors (4:4:4, 4:2:2, 4:4:0, 4:2:0), restart
// intervals, JFIF YCbCr or Adobe RGB colour, any number of scans: interleaved or one component per scan, and the
// progressive mode (spectral selection and successive approximation: DC / AC first and refinement scans with
// end-of-band runs).  Every scan writes into per-component coefficient buffers; dequantisation and the inverse DCT run
// once after the last scan.  Arithmetic-coded, lossless, hierarchical and 12-bit files are refused with a message.  Chroma is upsampled with the triangle filter common decoders use by default, so results stay within a
// few levels of theirs.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {

struct Huff {
  // canonical code tables: for code length l (1..16) the smallest code, the largest code and the index of its first symbol
  int mincode[17], maxcode[18], valptr[17];
  uint8_t vals[256];
  uint8_t look_len[256], look_sym[256];      // codes of up to 8 bits resolved by one table look-up
  bool present = false;
};

struct Comp {
  int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0;
  int bw = 0, bh = 0;                        // blocks per row / column (padded to whole MCUs)
  int nbw = 0, nbh = 0;                      // blocks per row / column that a scan of this component alone visits
  int pred = 0;
  std::vector<int16_t> coef;                 // bw * bh blocks of 64 coefficients (natural order), filled by the scans
  std::vector<uint8_t> plane;                // bw * 8 x bh * 8 samples
};

struct Dec {
  const uint8_t* p;
  const uint8_t* end;
  std::string err;
  int W = 0, H = 0, ncomp = 0;
  bool progressive = false, have_frame = false, adobe = false;
  int adobe_transform = -1;
  uint16_t qt[4][64];
  bool qt_ok[4] = {false, false, false, false};
  Huff dc[4], ac[4];
  Comp comp[4];
  int restart = 0;
  int hmax = 1, vmax = 1;
  // the scan being decoded
  Comp* scan_comp[4] = {nullptr, nullptr, nullptr, nullptr};
  int scan_n = 0, ss = 0, se = 63, ah = 0, al = 0;
  int eobrun = 0;
  bool planes_ready = false;
  // bit reader
  uint32_t acc = 0;
  int nbits = 0;
  bool hit_marker = false;
};

const uint8_t kZigzag[64] = {0,  1,  8,  16, 9,  2,  3,  10, 17, 24, 32, 25, 18, 11, 4,  5,  12, 19, 26, 33, 40, 48,
                             41, 34, 27, 20, 13, 6,  7,  14, 21, 28, 35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23,
                             30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

bool fail(Dec& d, const char* m) {
  if (d.err.empty()) d.err = m;
  return false;
}

int u16(const uint8_t* q) { return (q[0] << 8) | q[1]; }

bool build_huff(Dec& d, Huff& h, const uint8_t* counts, const uint8_t* vals, int nvals) {
  int code = 0, k = 0;
  for (int l = 1; l <= 16; ++l) {
    h.valptr[l] = k;
    h.mincode[l] = code;
    k += counts[l - 1];
    code += counts[l - 1];
    h.maxcode[l] = counts[l - 1] ? code - 1 : -1;
    if (code > (1 << l)) return fail(d, "jpeg: bad Huffman table");
    code <<= 1;
  }
  h.maxcode[17] = 0x7fffffff;
  if (k != nvals || nvals > 256) return fail(d, "jpeg: bad Huffman table");
  std::memcpy(h.vals, vals, nvals);
  std::memset(h.look_len, 0, sizeof h.look_len);
  code = 0;
  k = 0;
  for (int l = 1; l <= 8; ++l) {
    for (int i = 0; i < counts[l - 1]; ++i, ++k, ++code) {
      const int first = code << (8 - l), n = 1 << (8 - l);
      for (int j = 0; j < n; ++j) { h.look_len[first + j] = (uint8_t)l; h.look_sym[first + j] = vals[k]; }
    }
    code <<= 1;
  }
  h.present = true;
  return true;
}

// Entropy-coded bytes: 0xFF 0x00 is a data byte 0xFF; any other marker ends the segment (zeros are fed from then on).
void fill(Dec& d) {
  while (d.nbits <= 24) {
    uint32_t b = 0;
    if (!d.hit_marker && d.p < d.end) {
      b = *d.p;
      if (b == 0xFF) {
        if (d.p + 1 < d.end && d.p[1] == 0x00) {
          d.p += 2;
        } else {
          d.hit_marker = true;
          b = 0;
        }
      } else {
        ++d.p;
      }
    }
    d.acc |= b << (24 - d.nbits);
    d.nbits += 8;
  }
}
int get_bits(Dec& d, int n) {
  if (n == 0) return 0;
  if (d.nbits < n) fill(d);
  const int v = (int)(d.acc >> (32 - n));
  d.acc <<= n;
  d.nbits -= n;
  return v;
}
int decode_sym(Dec& d, const Huff& h) {
  if (d.nbits < 16) fill(d);
  const int top = (int)(d.acc >> 24);
  if (h.look_len[top]) {
    const int l = h.look_len[top];
    d.acc <<= l;
    d.nbits -= l;
    return h.look_sym[top];
  }
  int code = (int)(d.acc >> 23), l = 9;          // first nine bits
  for (; l <= 16; ++l) {
    if (h.maxcode[l] >= 0 && code <= h.maxcode[l] && code >= h.mincode[l]) break;
    code = (int)(d.acc >> (32 - (l + 1)));
  }
  if (l > 16) return -1;
  d.acc <<= l;
  d.nbits -= l;
  return h.vals[h.valptr[l] + code - h.mincode[l]];
}
int extend(int v, int n) { return v < (1 << (n - 1)) ? v - (1 << n) + 1 : v; }

// Inverse DCT of one dequantised block (separable, float), level shift and clamp.
struct IdctTable {
  float c[8][8];                             // c[x][u]
  float ct[8][8];                            // ct[u][x]: the same numbers with the output index innermost
  IdctTable() {
    for (int x = 0; x < 8; ++x)
      for (int u = 0; u < 8; ++u) ct[u][x] = c[x][u] = (u == 0 ? std::sqrt(0.125f) : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979323846f / 16.f);
  }
};
// Sums run over ascending u (then v) as in the plain triple loop, zero coefficients and all-zero rows left out (adding
// them changes nothing), the output index innermost so that the compiler can use vector registers.  A block with only
// its DC coefficient (most blocks of a smooth image) is one constant.
__attribute__((optimize("O3"))) void idct_store(const int* coef, uint8_t* out, int stride) {
  static const IdctTable table;              // initialised once, thread-safe
  const float (*c)[8] = table.c;
  const float (*ct)[8] = table.ct;
  unsigned rows = 0;                         // bit v: row v has a non-zero coefficient
  for (int v = 0; v < 8; ++v) {
    int any = 0;
    for (int u = 0; u < 8; ++u) any |= coef[v * 8 + u];
    if (any) rows |= 1u << v;
  }
  bool dc_only = rows <= 1u;
  if (dc_only) for (int u = 1; u < 8; ++u) dc_only = dc_only && coef[u] == 0;
  if (dc_only) {
    const float s = c[0][0] * (c[0][0] * (float)coef[0]);
    const int q = (int)std::lrintf(s + 128.f);
    const uint8_t px = (uint8_t)std::min(255, std::max(0, q));
    for (int y = 0; y < 8; ++y) std::memset(out + y * stride, px, 8);
    return;
  }
  float tmp[64];
  for (int v = 0; v < 8; ++v) {             // rows: over u
    if (!(rows >> v & 1u)) continue;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int u = 0; u < 8; ++u) {
      if (coef[v * 8 + u] == 0) continue;
      const float f = (float)coef[v * 8 + u];
      for (int x = 0; x < 8; ++x) acc[x] += ct[u][x] * f;
    }
    for (int x = 0; x < 8; ++x) tmp[v * 8 + x] = acc[x];
  }
  for (int y = 0; y < 8; ++y) {             // columns: over v
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int v = 0; v < 8; ++v) {
      if (!(rows >> v & 1u)) continue;
      const float f = c[y][v];
      for (int x = 0; x < 8; ++x) acc[x] += f * tmp[v * 8 + x];
    }
    for (int x = 0; x < 8; ++x) {
      const int q = (int)std::lrintf(acc[x] + 128.f);
      out[y * stride + x] = (uint8_t)std::min(255, std::max(0, q));
    }
  }
}

// ---- one block of one scan --------------------------------------------------------------------------------------------
// Sequential mode: the whole block.  Progressive mode: the DC coefficient (first pass / one refinement bit) or the band
// ss..se of AC coefficients (first pass with end-of-band runs / refinement with correction bits), T.81 annex G.
bool block_sequential(Dec& d, Comp& cp, int16_t* c) {
  const Huff& hd = d.dc[cp.td];
  const Huff& ha = d.ac[cp.ta];
  int t = decode_sym(d, hd);
  if (t < 0 || t > 11) return fail(d, "jpeg: bad DC code");
  cp.pred += t ? extend(get_bits(d, t), t) : 0;
  c[0] = (int16_t)cp.pred;
  for (int k = 1; k < 64;) {
    const int rs = decode_sym(d, ha);
    if (rs < 0) return fail(d, "jpeg: bad AC code");
    const int r = rs >> 4, s = rs & 15;
    if (s == 0) {
      if (r != 15) break;                  // end of block
      k += 16;
      continue;
    }
    k += r;
    if (k > 63) return fail(d, "jpeg: coefficient index out of range");
    c[kZigzag[k]] = (int16_t)extend(get_bits(d, s), s);
    ++k;
  }
  return true;
}

bool block_dc(Dec& d, Comp& cp, int16_t* c) {
  if (d.ah == 0) {
    int t = decode_sym(d, d.dc[cp.td]);
    if (t < 0 || t > 11) return fail(d, "jpeg: bad DC code");
    cp.pred += t ? extend(get_bits(d, t), t) : 0;
    c[0] = (int16_t)(cp.pred * (1 << d.al));
  } else if (get_bits(d, 1)) {
    c[0] = (int16_t)(c[0] | (1 << d.al));
  }
  return true;
}

bool block_ac_first(Dec& d, Comp& cp, int16_t* c) {
  if (d.eobrun > 0) { --d.eobrun; return true; }
  const Huff& ha = d.ac[cp.ta];
  for (int k = d.ss; k <= d.se; ++k) {
    const int rs = decode_sym(d, ha);
    if (rs < 0) return fail(d, "jpeg: bad AC code");
    const int r = rs >> 4, s = rs & 15;
    if (s) {
      k += r;
      if (k > d.se) return fail(d, "jpeg: coefficient index out of range");
      c[kZigzag[k]] = (int16_t)(extend(get_bits(d, s), s) * (1 << d.al));
    } else if (r == 15) {
      k += 15;
    } else {
      d.eobrun = (1 << r) - 1 + (r ? get_bits(d, r) : 0);      // this block ends the band, and so do the next eobrun blocks
      break;
    }
  }
  return true;
}

bool block_ac_refine(Dec& d, Comp& cp, int16_t* c) {
  const int p1 = 1 << d.al, m1 = -(1 << d.al);
  const Huff& ha = d.ac[cp.ta];
  auto correct = [&](int16_t& v) {         // one more bit of precision for a coefficient that is already non-zero
    if (get_bits(d, 1) && (v & p1) == 0) v = (int16_t)(v + (v >= 0 ? p1 : m1));
  };
  int k = d.ss;
  if (d.eobrun == 0) {
    for (; k <= d.se; ++k) {
      const int rs = decode_sym(d, ha);
      if (rs < 0) return fail(d, "jpeg: bad AC code");
      int r = rs >> 4, s = rs & 15;
      if (s) {
        if (s != 1) return fail(d, "jpeg: bad refinement code");
        s = get_bits(d, 1) ? p1 : m1;
      } else if (r != 15) {
        d.eobrun = (1 << r) + (r ? get_bits(d, r) : 0);
        break;
      }
      // pass over r coefficients that are still zero; the non-zero ones on the way take a correction bit each
      do {
        int16_t& v = c[kZigzag[k]];
        if (v != 0) correct(v);
        else if (--r < 0) break;
        ++k;
      } while (k <= d.se);
      if (s) {
        if (k > d.se) return fail(d, "jpeg: coefficient index out of range");
        c[kZigzag[k]] = (int16_t)s;
      }
    }
  }
  if (d.eobrun > 0) {
    for (; k <= d.se; ++k) {
      int16_t& v = c[kZigzag[k]];
      if (v != 0) correct(v);
    }
    --d.eobrun;
  }
  return true;
}

bool decode_one_block(Dec& d, Comp& cp, int16_t* c) {
  if (!d.progressive) return block_sequential(d, cp, c);
  if (d.ss == 0) return block_dc(d, cp, c);
  return d.ah == 0 ? block_ac_first(d, cp, c) : block_ac_refine(d, cp, c);
}

bool parse_headers(Dec& d, bool stop_at_frame) {
  if (d.end - d.p < 4 || d.p[0] != 0xFF || d.p[1] != 0xD8) return fail(d, "jpeg: no SOI marker");
  d.p += 2;
  while (d.p + 4 <= d.end) {
    if (d.p[0] != 0xFF) return fail(d, "jpeg: marker expected");
    while (d.p + 1 < d.end && d.p[1] == 0xFF) ++d.p;     // fill bytes
    if (d.p + 2 > d.end) break;
    const int m = d.p[1];
    d.p += 2;
    if (m == 0xD9) return fail(d, "jpeg: no scan before EOI");
    if (m >= 0xD0 && m <= 0xD7) continue;
    if (d.p + 2 > d.end) break;
    const int len = u16(d.p);
    if (len < 2 || d.p + len > d.end) return fail(d, "jpeg: truncated segment");
    const uint8_t* s = d.p + 2;
    const uint8_t* se = d.p + len;
    if (m == 0xC0 || m == 0xC1 || m == 0xC2) {
      if (se - s < 6) return fail(d, "jpeg: bad frame header");
      if (d.have_frame) return fail(d, "jpeg: more than one frame header");   // the caller sized its buffer by the first
      if (s[0] != 8) return fail(d, "jpeg: only 8-bit samples are supported");
      d.progressive = m == 0xC2;
      d.H = u16(s + 1);
      d.W = u16(s + 3);
      d.ncomp = s[5];
      if (d.W <= 0 || d.H <= 0) return fail(d, "jpeg: empty image");
      if (d.ncomp != 1 && d.ncomp != 3 && d.ncomp != 4) return fail(d, "jpeg: only grey, three- and four-component images are supported");
      if (se - s < 6 + 3 * d.ncomp) return fail(d, "jpeg: bad frame header");
      for (int i = 0; i < d.ncomp; ++i) {
        Comp& c = d.comp[i];
        c.id = s[6 + 3 * i];
        c.h = s[7 + 3 * i] >> 4;
        c.v = s[7 + 3 * i] & 15;
        c.tq = s[8 + 3 * i] & 3;
        if (c.h < 1 || c.h > 2 || c.v < 1 || c.v > 2) return fail(d, "jpeg: sampling factors other than 1 and 2 are not supported");
        d.hmax = std::max(d.hmax, c.h);
        d.vmax = std::max(d.vmax, c.v);
      }
      d.have_frame = true;
      if (stop_at_frame) return true;
      {
        const int mcu_w = 8 * d.hmax, mcu_h = 8 * d.vmax;
        const int mx = (d.W + mcu_w - 1) / mcu_w, my = (d.H + mcu_h - 1) / mcu_h;
        if (d.ncomp == 1) { d.comp[0].h = d.comp[0].v = 1; d.hmax = d.vmax = 1; }
        for (int i = 0; i < d.ncomp; ++i) {
          Comp& c = d.comp[i];
          c.bw = d.ncomp == 1 ? (d.W + 7) / 8 : mx * c.h;
          c.bh = d.ncomp == 1 ? (d.H + 7) / 8 : my * c.v;
          // a scan of this component alone covers the component's own size, not the padded one
          c.nbw = (((long)d.W * c.h + d.hmax - 1) / d.hmax + 7) / 8;
          c.nbh = (((long)d.H * c.v + d.vmax - 1) / d.vmax + 7) / 8;
          if ((long long)c.bw * c.bh > (1ll << 22)) return fail(d, "jpeg: image too large");
          c.coef.assign((size_t)c.bw * c.bh * 64, 0);
        }
      }
    } else if (m == 0xC3 || (m >= 0xC5 && m <= 0xCF && m != 0xC4 && m != 0xC8 && m != 0xCC)) {
      return fail(d, "jpeg: lossless, hierarchical and arithmetic-coded files are not supported");
    } else if (m == 0xC4) {
      while (s < se) {
        if (se - s < 17) return fail(d, "jpeg: bad Huffman segment");
        const int tc = s[0] >> 4, th = s[0] & 15;
        if (tc > 1 || th > 3) return fail(d, "jpeg: bad Huffman table id");
        int n = 0;
        for (int i = 0; i < 16; ++i) n += s[1 + i];
        if (se - s < 17 + n) return fail(d, "jpeg: bad Huffman segment");
        if (!build_huff(d, tc ? d.ac[th] : d.dc[th], s + 1, s + 17, n)) return false;
        s += 17 + n;
      }
    } else if (m == 0xDB) {
      while (s < se) {
        const int pq = s[0] >> 4, tq = s[0] & 15;
        if (tq > 3) return fail(d, "jpeg: bad quantisation table id");
        const int need = 1 + (pq ? 128 : 64);
        if (se - s < need) return fail(d, "jpeg: bad quantisation segment");
        for (int i = 0; i < 64; ++i) d.qt[tq][i] = pq ? (uint16_t)u16(s + 1 + 2 * i) : s[1 + i];
        d.qt_ok[tq] = true;
        s += need;
      }
    } else if (m == 0xDD) {
      if (se - s < 2) return fail(d, "jpeg: bad restart interval");
      d.restart = u16(s);
    } else if (m == 0xEE) {
      if (se - s >= 12 && std::memcmp(s, "Adobe", 5) == 0) { d.adobe = true; d.adobe_transform = s[11]; }
    } else if (m == 0xDA) {
      if (!d.have_frame) return fail(d, "jpeg: scan before frame header");
      const int ns = se > s ? s[0] : 0;
      if (ns < 1 || ns > d.ncomp || se - s < 1 + 2 * ns + 3) return fail(d, "jpeg: bad scan header");
      d.scan_n = ns;
      d.ss = s[1 + 2 * ns]; d.se = s[2 + 2 * ns]; d.ah = s[3 + 2 * ns] >> 4; d.al = s[3 + 2 * ns] & 15;
      if (!d.progressive) { d.ss = 0; d.se = 63; d.ah = d.al = 0; }
      else if (d.ss > d.se || d.se > 63 || (d.ss == 0 && d.se != 0) || (d.ss > 0 && ns != 1) || d.al > 13)
        return fail(d, "jpeg: bad progressive scan parameters");
      for (int i = 0; i < ns; ++i) {
        const int cid = s[1 + 2 * i];
        Comp* c = nullptr;
        for (int j = 0; j < d.ncomp; ++j)
          if (d.comp[j].id == cid) c = &d.comp[j];
        if (!c) return fail(d, "jpeg: scan names an unknown component");
        c->td = s[2 + 2 * i] >> 4;
        c->ta = s[2 + 2 * i] & 15;
        const bool need_dc = d.ss == 0 && d.ah == 0, need_ac = d.se > 0;
        if (c->td > 3 || c->ta > 3 || (need_dc && !d.dc[c->td].present) || (need_ac && !d.ac[c->ta].present))
          return fail(d, "jpeg: scan uses a table that was not defined");
        d.scan_comp[i] = c;
      }
      d.p += len;
      return true;                          // entropy-coded data follows
    }
    d.p += len;
  }
  return fail(d, "jpeg: no scan found");
}

// Entropy-coded data of the scan whose header parse_headers() just read.
bool decode_scan(Dec& d) {
  for (int i = 0; i < d.scan_n; ++i) d.scan_comp[i]->pred = 0;
  d.eobrun = 0;
  d.acc = 0; d.nbits = 0; d.hit_marker = false;
  const bool single = d.scan_n == 1;
  Comp& c0 = *d.scan_comp[0];
  const int mcu_w = 8 * d.hmax, mcu_h = 8 * d.vmax;
  // one component: its blocks in raster order; several: MCUs of h x v blocks per component
  const int nx = single ? c0.nbw : (d.W + mcu_w - 1) / mcu_w, ny = single ? c0.nbh : (d.H + mcu_h - 1) / mcu_h;
  int countdown = d.restart, next_rst = 0;
  for (int y = 0; y < ny; ++y)
    for (int x = 0; x < nx; ++x) {
      if (d.restart && countdown == 0) {
        // byte-align, expect RSTn
        d.acc = 0; d.nbits = 0;
        if (!d.hit_marker) {
          while (d.p + 1 < d.end && !(d.p[0] == 0xFF && d.p[1] != 0x00 && d.p[1] != 0xFF)) ++d.p;   // skip padding
        }
        if (d.p + 1 < d.end && d.p[0] == 0xFF && d.p[1] == 0xD0 + next_rst) {
          d.p += 2;
        } else {
          return fail(d, "jpeg: restart marker missing");
        }
        d.hit_marker = false;
        next_rst = (next_rst + 1) & 7;
        countdown = d.restart;
        for (int i = 0; i < d.scan_n; ++i) d.scan_comp[i]->pred = 0;
        d.eobrun = 0;
      }
      if (single) {
        if (!decode_one_block(d, c0, c0.coef.data() + ((size_t)y * c0.bw + x) * 64)) return false;
      } else {
        for (int i = 0; i < d.scan_n; ++i) {
          Comp& c = *d.scan_comp[i];
          for (int by = 0; by < c.v; ++by)
            for (int bx = 0; bx < c.h; ++bx)
              if (!decode_one_block(d, c, c.coef.data() + ((size_t)(y * c.v + by) * c.bw + (size_t)(x * c.h + bx)) * 64)) return false;
        }
      }
      if (d.restart) --countdown;
    }
  return true;
}

// After a scan: the markers and segments up to the next scan header.  Returns false at the end of the image.
bool next_scan(Dec& d) {
  // the bit reader stopped in front of a marker (or at the end of the data)
  while (d.p + 1 < d.end && !(d.p[0] == 0xFF && d.p[1] != 0x00 && d.p[1] != 0xFF && !(d.p[1] >= 0xD0 && d.p[1] <= 0xD7))) ++d.p;
  while (d.p + 4 <= d.end) {
    if (d.p[0] != 0xFF) { ++d.p; continue; }
    const int m = d.p[1];
    if (m == 0xFF) { ++d.p; continue; }
    d.p += 2;
    if (m == 0xD9) return false;
    if (m == 0x00 || (m >= 0xD0 && m <= 0xD7)) continue;
    const int len = u16(d.p);
    if (len < 2 || d.p + len > d.end) return false;         // truncated tail: keep what the earlier scans gave
    const uint8_t* s = d.p + 2;
    const uint8_t* se = d.p + len;
    if (m == 0xC4) {
      while (s < se) {
        if (se - s < 17) return fail(d, "jpeg: bad Huffman segment");
        const int tc = s[0] >> 4, th = s[0] & 15;
        if (tc > 1 || th > 3) return fail(d, "jpeg: bad Huffman table id");
        int n = 0;
        for (int i = 0; i < 16; ++i) n += s[1 + i];
        if (se - s < 17 + n) return fail(d, "jpeg: bad Huffman segment");
        if (!build_huff(d, tc ? d.ac[th] : d.dc[th], s + 1, s + 17, n)) return false;
        s += 17 + n;
      }
    } else if (m == 0xDB) {
      while (s < se) {
        const int pq = s[0] >> 4, tq = s[0] & 15;
        const int need = 1 + (pq ? 128 : 64);
        if (tq > 3 || se - s < need) return fail(d, "jpeg: bad quantisation segment");
        for (int i = 0; i < 64; ++i) d.qt[tq][i] = pq ? (uint16_t)u16(s + 1 + 2 * i) : s[1 + i];
        d.qt_ok[tq] = true;
        s += need;
      }
    } else if (m == 0xDD) {
      if (se - s >= 2) d.restart = u16(s);
    } else if (m == 0xDA) {
      const int ns = se > s ? s[0] : 0;
      if (ns < 1 || ns > d.ncomp || se - s < 1 + 2 * ns + 3) return fail(d, "jpeg: bad scan header");
      d.scan_n = ns;
      d.ss = s[1 + 2 * ns]; d.se = s[2 + 2 * ns]; d.ah = s[3 + 2 * ns] >> 4; d.al = s[3 + 2 * ns] & 15;
      if (!d.progressive) { d.ss = 0; d.se = 63; d.ah = d.al = 0; }
      else if (d.ss > d.se || d.se > 63 || (d.ss == 0 && d.se != 0) || (d.ss > 0 && ns != 1) || d.al > 13)
        return fail(d, "jpeg: bad progressive scan parameters");
      for (int i = 0; i < ns; ++i) {
        Comp* c = nullptr;
        for (int j = 0; j < d.ncomp; ++j)
          if (d.comp[j].id == s[1 + 2 * i]) c = &d.comp[j];
        if (!c) return fail(d, "jpeg: scan names an unknown component");
        c->td = s[2 + 2 * i] >> 4;
        c->ta = s[2 + 2 * i] & 15;
        const bool need_dc = d.ss == 0 && d.ah == 0, need_ac = d.se > 0;
        if (c->td > 3 || c->ta > 3 || (need_dc && !d.dc[c->td].present) || (need_ac && !d.ac[c->ta].present))
          return fail(d, "jpeg: scan uses a table that was not defined");
        d.scan_comp[i] = c;
      }
      d.p += len;
      return true;
    }
    d.p += len;
  }
  return false;
}

// Dequantise and transform every block once all scans are in.
bool finish_planes(Dec& d) {
  for (int i = 0; i < d.ncomp; ++i) {
    Comp& c = d.comp[i];
    if (!d.qt_ok[c.tq]) return fail(d, "jpeg: a component uses a quantisation table that was not defined");
    int qnat[64];
    for (int k = 0; k < 64; ++k) qnat[kZigzag[k]] = d.qt[c.tq][k];
    c.plane.assign((size_t)c.bw * 8 * c.bh * 8, 0);
    const int stride = c.bw * 8;
    int blk[64];
    for (int by = 0; by < c.bh; ++by)
      for (int bx = 0; bx < c.bw; ++bx) {
        const int16_t* src = c.coef.data() + ((size_t)by * c.bw + bx) * 64;
        for (int k = 0; k < 64; ++k) blk[k] = (int)src[k] * qnat[k];
        idct_store(blk, c.plane.data() + (size_t)by * 8 * stride + (size_t)bx * 8, stride);
      }
  }
  return true;
}

// All scans of the image.
bool decode_image(Dec& d) {
  do {
    if (!decode_scan(d)) return false;
  } while (next_scan(d));
  if (!d.err.empty()) return false;
  return finish_planes(d);
}

// Sample of a subsampled plane at full-resolution position (x, y): triangle filter (3/4, 1/4) along each halved axis,
// edge samples replicated.
inline float sample_up(const Comp& c, int x, int y, int hs, int vs, int W, int H) {
  const int stride = c.bw * 8, pw = (W + hs - 1) / hs, ph = (H + vs - 1) / vs;     // the component's own size
  auto at = [&](int xx, int yy) {
    xx = std::min(std::max(xx, 0), pw - 1);
    yy = std::min(std::max(yy, 0), ph - 1);
    return (float)c.plane[(size_t)yy * stride + xx];
  };
  if (hs == 1 && vs == 1) return at(x, y);
  int x0 = x, x1 = x, y0 = y, y1 = y;
  float wx = 0.f, wy = 0.f;                  // weight of the second sample
  if (hs == 2) { x0 = x >> 1; x1 = (x & 1) ? x0 + 1 : x0 - 1; wx = 0.25f; }
  if (vs == 2) { y0 = y >> 1; y1 = (y & 1) ? y0 + 1 : y0 - 1; wy = 0.25f; }
  const float a = at(x0, y0) * (1.f - wx) + at(x1, y0) * wx;
  const float b = at(x0, y1) * (1.f - wx) + at(x1, y1) * wx;
  return a * (1.f - wy) + b * wy;
}

// One full-resolution row of a component: the same arithmetic as sample_up() for every x, with the row addresses and
// weights taken once per row instead of once per pixel.
__attribute__((optimize("O3"))) void sample_row(const Comp& c, int y, int hs, int vs, int W, int H, float* out) {
  const int stride = c.bw * 8, pw = (W + hs - 1) / hs, ph = (H + vs - 1) / vs;
  auto clampi = [](int v, int hi) { return std::min(std::max(v, 0), hi); };
  if (hs == 1 && vs == 1) {
    const uint8_t* r = c.plane.data() + (size_t)clampi(y, ph - 1) * stride;
    for (int x = 0; x < W; ++x) out[x] = (float)r[x];                 // pw == W here
    return;
  }
  int y0 = y, y1 = y;
  float wy = 0.f;
  if (vs == 2) { y0 = y >> 1; y1 = (y & 1) ? y0 + 1 : y0 - 1; wy = 0.25f; }
  const uint8_t* r0 = c.plane.data() + (size_t)clampi(y0, ph - 1) * stride;
  const uint8_t* r1 = c.plane.data() + (size_t)clampi(y1, ph - 1) * stride;
  for (int x = 0; x < W; ++x) {
    int x0 = x, x1 = x;
    float wx = 0.f;
    if (hs == 2) { x0 = x >> 1; x1 = (x & 1) ? x0 + 1 : x0 - 1; wx = 0.25f; }
    x0 = clampi(x0, pw - 1); x1 = clampi(x1, pw - 1);
    const float a = (float)r0[x0] * (1.f - wx) + (float)r0[x1] * wx;
    const float b = (float)r1[x0] * (1.f - wx) + (float)r1[x1] * wx;
    out[x] = a * (1.f - wy) + b * wy;
  }
}

inline uint8_t clamp8(float v) { return (uint8_t)std::min(255, std::max(0, (int)std::lrintf(v))); }

void to_rgb(const Dec& d, uint8_t* rgb) {
  if (d.ncomp == 1) {
    const Comp& c = d.comp[0];
    for (int y = 0; y < d.H; ++y)
      for (int x = 0; x < d.W; ++x) {
        const uint8_t g = c.plane[(size_t)y * c.bw * 8 + x];
        uint8_t* o = rgb + ((size_t)y * d.W + x) * 3;
        o[0] = o[1] = o[2] = g;
      }
    return;
  }
  if (d.ncomp == 4) {
    // Adobe CMYK (transform 0) or YCCK (transform 2): the file holds the inverted ink values (255 = no ink); YCCK codes
    // the three colour inks as YCbCr.  RGB = colour ink value x black value / 255, the conversion common viewers use.
    const bool ycck = d.adobe && d.adobe_transform == 2;
    for (int y = 0; y < d.H; ++y)
      for (int x = 0; x < d.W; ++x) {
        float v[4];
        for (int i = 0; i < 4; ++i) {
          const Comp& c = d.comp[i];
          v[i] = sample_up(c, x, y, d.hmax / c.h, d.vmax / c.v, d.W, d.H);
        }
        if (ycck) {
          const float Y = v[0], cb = v[1] - 128.f, cr = v[2] - 128.f;
          v[0] = std::min(255.f, std::max(0.f, Y + 1.402f * cr));
          v[1] = std::min(255.f, std::max(0.f, Y - 0.344136f * cb - 0.714136f * cr));
          v[2] = std::min(255.f, std::max(0.f, Y + 1.772f * cb));
        }
        if (!d.adobe) { v[0] = 255.f - v[0]; v[1] = 255.f - v[1]; v[2] = 255.f - v[2]; v[3] = 255.f - v[3]; }   // plain CMYK: not inverted
        uint8_t* o = rgb + ((size_t)y * d.W + x) * 3;
        for (int i = 0; i < 3; ++i) o[i] = clamp8(v[i] * v[3] / 255.f);
      }
    return;
  }
  // three components: YCbCr unless an Adobe segment says the data is RGB (transform 0)
  const bool ycc = !(d.adobe && d.adobe_transform == 0);
  std::vector<float> rows((size_t)3 * d.W);
  float* v0 = rows.data();
  float* v1 = v0 + d.W;
  float* v2 = v1 + d.W;
  for (int y = 0; y < d.H; ++y) {
    for (int i = 0; i < 3; ++i) sample_row(d.comp[i], y, d.hmax / d.comp[i].h, d.vmax / d.comp[i].v, d.W, d.H, v0 + (size_t)i * d.W);
    uint8_t* o = rgb + (size_t)y * d.W * 3;
    if (ycc) {
      for (int x = 0; x < d.W; ++x, o += 3) {
        const float Y = v0[x], cb = v1[x] - 128.f, cr = v2[x] - 128.f;
        o[0] = clamp8(Y + 1.402f * cr);
        o[1] = clamp8(Y - 0.344136f * cb - 0.714136f * cr);
        o[2] = clamp8(Y + 1.772f * cb);
      }
    } else {
      for (int x = 0; x < d.W; ++x, o += 3) { o[0] = clamp8(v0[x]); o[1] = clamp8(v1[x]); o[2] = clamp8(v2[x]); }
    }
  }
}

thread_local std::string g_jpeg_err;

}  // namespace

// Height, width and component count of a JPEG file; 0 on success.
B2H_API int b2h_jpeg_info(const uint8_t* data, long n, int* h, int* w, int* comps) {
  Dec d;
  d.p = data;
  d.end = data + n;
  if (!parse_headers(d, true)) { g_jpeg_err = d.err; return 1; }
  *h = d.H; *w = d.W; *comps = d.ncomp;
  return 0;
}

// Decodes into rgb (h * w * 3 bytes, sizes from b2h_jpeg_info); 0 on success, else b2h_jpeg_error() says why.
B2H_API int b2h_jpeg_decode(const uint8_t* data, long n, uint8_t* rgb) {
  Dec d;
  d.p = data;
  d.end = data + n;
  if (!parse_headers(d, false) || !decode_image(d)) { g_jpeg_err = d.err.empty() ? "jpeg: decode failed" : d.err; return 1; }
  to_rgb(d, rgb);
  return 0;
}

B2H_API const char* b2h_jpeg_error() { return g_jpeg_err.c_str(); }
