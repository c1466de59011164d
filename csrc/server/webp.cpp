// WebP reader for image inputs of chat requests: the lossless format (VP8L), bare or inside the extended container
// (VP8X; the first frame of an animation).  Alpha is dropped (the vision tower takes RGB).  The lossy format (VP8) is
// recognised and refused with a message: it is not decoded here.
// The reference takes WebP through its image crate (crates/agens-server/src/vision.rs:126-135).
//
// VP8L in brief: a little-endian bit stream; up to four transforms (predictor, cross-colour, subtract-green, colour
// indexing) announced before the pixels; pixels entropy coded with five prefix codes per group (green + length +
// cache symbols, red, blue, alpha, distance), groups chosen per block through an "entropy image"; LZ77 backward
// references with a short-distance code table and an optional colour cache.  Sub-images (transform data, the entropy
// image, the palette) use the same pixel coding without transforms and without groups.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_werr;

struct Bits {
  const uint8_t* p;
  size_t n, pos = 0;     // bit position
  uint32_t read(int k) {
    uint32_t v = 0;
    for (int i = 0; i < k; ++i, ++pos) {
      if ((pos >> 3) >= n) throw std::runtime_error("webp: truncated bit stream");
      v |= (uint32_t)((p[pos >> 3] >> (pos & 7)) & 1) << i;
    }
    return v;
  }
};

// Canonical prefix code, decoded one bit at a time (the first bit read is the most significant bit of the code word).
struct Prefix {
  std::vector<uint16_t> sorted;         // symbols by (length, value)
  int count[16] = {0};
  int single = -1;                      // >= 0: the code has one symbol and takes no bits
  void build(const std::vector<int>& len) {
    int used = 0, last = -1;
    for (size_t s = 0; s < len.size(); ++s) if (len[s] > 0) { ++used; last = (int)s; }
    if (used == 0) throw std::runtime_error("webp: empty prefix code");
    if (used == 1) { single = last; return; }
    for (int i = 0; i < 16; ++i) count[i] = 0;
    for (int l : len) if (l > 0) { if (l > 15) throw std::runtime_error("webp: bad code length"); ++count[l]; }
    long left = 1;                       // the code must be complete
    for (int l = 1; l < 16; ++l) { left = left * 2 - count[l]; if (left < 0) throw std::runtime_error("webp: over-subscribed prefix code"); }
    if (left != 0) throw std::runtime_error("webp: incomplete prefix code");
    sorted.clear();
    for (int l = 1; l < 16; ++l)
      for (size_t s = 0; s < len.size(); ++s) if (len[s] == l) sorted.push_back((uint16_t)s);
  }
  int decode(Bits& b) const {
    if (single >= 0) return single;
    int code = 0, first = 0, index = 0;
    for (int l = 1; l < 16; ++l) {
      code |= (int)b.read(1);
      const int c = count[l];
      if (code - first < c) return sorted[index + (code - first)];
      index += c; first += c; first <<= 1; code <<= 1;
    }
    throw std::runtime_error("webp: bad prefix code word");
  }
};

const int kLengthOrder[19] = {17, 18, 0, 1, 2, 3, 4, 5, 16, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15};

Prefix read_prefix(Bits& b, int alphabet) {
  std::vector<int> len((size_t)alphabet, 0);
  if (b.read(1)) {                                        // simple code: one or two symbols
    const int n = (int)b.read(1) + 1;
    const int s0 = (int)b.read(b.read(1) ? 8 : 1);
    if (s0 >= alphabet) throw std::runtime_error("webp: symbol outside the alphabet");
    len[(size_t)s0] = 1;
    if (n == 2) {
      const int s1 = (int)b.read(8);
      if (s1 >= alphabet) throw std::runtime_error("webp: symbol outside the alphabet");
      len[(size_t)s1] = 1;
    }
  } else {
    std::vector<int> cl(19, 0);
    const int nc = (int)b.read(4) + 4;
    if (nc > 19) throw std::runtime_error("webp: bad code length count");
    for (int i = 0; i < nc; ++i) cl[(size_t)kLengthOrder[i]] = (int)b.read(3);
    Prefix lc;
    lc.build(cl);
    int max_symbol = alphabet;
    if (b.read(1)) {
      const int nb = 2 + 2 * (int)b.read(3);
      max_symbol = 2 + (int)b.read(nb);
      if (max_symbol > alphabet) throw std::runtime_error("webp: bad symbol count");
    }
    int sym = 0, prev = 8;
    while (sym < alphabet) {
      if (max_symbol-- == 0) break;
      const int c = lc.decode(b);
      if (c < 16) {
        len[(size_t)sym++] = c;
        if (c) prev = c;
      } else {
        static const int extra[3] = {2, 3, 7}, base[3] = {3, 3, 11};
        const int rep = (int)b.read(extra[c - 16]) + base[c - 16];
        if (sym + rep > alphabet) throw std::runtime_error("webp: code length run past the alphabet");
        const int v = c == 16 ? prev : 0;
        for (int i = 0; i < rep; ++i) len[(size_t)sym++] = v;
      }
    }
  }
  Prefix p;
  p.build(len);
  return p;
}

// (x offset, y offset) of the 120 short distance codes
const int8_t kNear[120][2] = {
    {0, 1},  {1, 0},  {1, 1},  {-1, 1}, {0, 2},  {2, 0},  {1, 2},  {-1, 2}, {2, 1},  {-2, 1}, {2, 2},  {-2, 2}, {0, 3},  {3, 0},  {1, 3},
    {-1, 3}, {3, 1},  {-3, 1}, {2, 3},  {-2, 3}, {3, 2},  {-3, 2}, {0, 4},  {4, 0},  {1, 4},  {-1, 4}, {4, 1},  {-4, 1}, {3, 3},  {-3, 3},
    {2, 4},  {-2, 4}, {4, 2},  {-4, 2}, {0, 5},  {3, 4},  {-3, 4}, {4, 3},  {-4, 3}, {5, 0},  {1, 5},  {-1, 5}, {5, 1},  {-5, 1}, {2, 5},
    {-2, 5}, {5, 2},  {-5, 2}, {4, 4},  {-4, 4}, {3, 5},  {-3, 5}, {5, 3},  {-5, 3}, {0, 6},  {6, 0},  {1, 6},  {-1, 6}, {6, 1},  {-6, 1},
    {2, 6},  {-2, 6}, {6, 2},  {-6, 2}, {4, 5},  {-4, 5}, {5, 4},  {-5, 4}, {3, 6},  {-3, 6}, {6, 3},  {-6, 3}, {0, 7},  {7, 0},  {1, 7},
    {-1, 7}, {5, 5},  {-5, 5}, {7, 1},  {-7, 1}, {4, 6},  {-4, 6}, {6, 4},  {-6, 4}, {2, 7},  {-2, 7}, {7, 2},  {-7, 2}, {3, 7},  {-3, 7},
    {7, 3},  {-7, 3}, {5, 6},  {-5, 6}, {6, 5},  {-6, 5}, {8, 0},  {4, 7},  {-4, 7}, {7, 4},  {-7, 4}, {8, 1},  {8, 2},  {6, 6},  {-6, 6},
    {8, 3},  {5, 7},  {-5, 7}, {7, 5},  {-7, 5}, {8, 4},  {6, 7},  {-6, 7}, {7, 6},  {-7, 6}, {8, 5},  {7, 7},  {-7, 7}, {8, 6},  {8, 7}};

int prefix_value(Bits& b, int sym) {          // length / distance symbols: small values direct, then (offset, extra bits)
  if (sym < 4) return sym + 1;
  const int extra = (sym - 2) >> 1;
  const int offset = (2 + (sym & 1)) << extra;
  return offset + (int)b.read(extra) + 1;
}

struct Group { Prefix green, red, blue, alpha, dist; };

int div_up(int a, int bits) { return (a + (1 << bits) - 1) >> bits; }

// One entropy-coded image of w x h ARGB pixels.  top: the main image (may carry an entropy image).
std::vector<uint32_t> decode_pixels(Bits& b, int w, int h, bool top) {
  int cache_bits = 0;
  if (b.read(1)) {
    cache_bits = (int)b.read(4);
    if (cache_bits < 1 || cache_bits > 11) throw std::runtime_error("webp: bad colour cache size");
  }
  std::vector<uint32_t> meta;
  int meta_bits = 0, meta_w = 0, n_groups = 1;
  if (top && b.read(1)) {
    meta_bits = (int)b.read(3) + 2;
    meta_w = div_up(w, meta_bits);
    meta = decode_pixels(b, meta_w, div_up(h, meta_bits), false);
    for (auto& m : meta) { m = (m >> 8) & 0xffff; if ((int)m + 1 > n_groups) n_groups = (int)m + 1; }
  }
  std::vector<Group> groups((size_t)n_groups);
  for (auto& g : groups) {
    g.green = read_prefix(b, 256 + 24 + (cache_bits ? 1 << cache_bits : 0));
    g.red = read_prefix(b, 256);
    g.blue = read_prefix(b, 256);
    g.alpha = read_prefix(b, 256);
    g.dist = read_prefix(b, 40);
  }
  std::vector<uint32_t> cache(cache_bits ? (size_t)1 << cache_bits : 0, 0);
  auto remember = [&](uint32_t px) { if (cache_bits) cache[(size_t)((0x1e35a7bdu * px) >> (32 - cache_bits))] = px; };
  const size_t total = (size_t)w * h;
  std::vector<uint32_t> out(total);
  size_t pos = 0;
  while (pos < total) {
    const int x = (int)(pos % (size_t)w), y = (int)(pos / (size_t)w);
    const Group& g = groups[meta.empty() ? 0 : meta[(size_t)(y >> meta_bits) * meta_w + (x >> meta_bits)]];
    const int s = g.green.decode(b);
    if (s < 256) {
      const uint32_t r = (uint32_t)g.red.decode(b), bl = (uint32_t)g.blue.decode(b), a = (uint32_t)g.alpha.decode(b);
      const uint32_t px = (a << 24) | (r << 16) | ((uint32_t)s << 8) | bl;
      out[pos++] = px;
      remember(px);
    } else if (s < 256 + 24) {
      const int len = prefix_value(b, s - 256);
      const int dcode = prefix_value(b, g.dist.decode(b));
      long dist;
      if (dcode > 120) dist = dcode - 120;
      else { dist = (long)kNear[dcode - 1][0] + (long)kNear[dcode - 1][1] * w; if (dist < 1) dist = 1; }
      if ((size_t)dist > pos || pos + (size_t)len > total) throw std::runtime_error("webp: backward reference outside the image");
      for (int i = 0; i < len; ++i, ++pos) { out[pos] = out[pos - (size_t)dist]; remember(out[pos]); }
    } else {
      const size_t key = (size_t)(s - 280);
      if (key >= cache.size()) throw std::runtime_error("webp: colour cache index out of range");
      out[pos] = cache[key];
      remember(out[pos]);
      ++pos;
    }
  }
  return out;
}

struct Transform { int type, bits, w_in; std::vector<uint32_t> data; };   // w_in: width of the image the transform was read for

uint32_t add_px(uint32_t a, uint32_t b) {                  // per channel, modulo 256
  return (((a & 0xff00ff00u) + (b & 0xff00ff00u)) & 0xff00ff00u) | (((a & 0x00ff00ffu) + (b & 0x00ff00ffu)) & 0x00ff00ffu);
}
uint32_t avg2(uint32_t a, uint32_t b) { return (((a ^ b) & 0xfefefefeu) >> 1) + (a & b); }
int clamp255(int v) { return v < 0 ? 0 : (v > 255 ? 255 : v); }
uint32_t select_px(uint32_t L, uint32_t T, uint32_t TL) {
  int pl = 0, pt = 0;
  for (int s = 0; s < 32; s += 8) {
    pl += std::abs((int)((T >> s) & 0xff) - (int)((TL >> s) & 0xff));
    pt += std::abs((int)((L >> s) & 0xff) - (int)((TL >> s) & 0xff));
  }
  return pl < pt ? L : T;
}
uint32_t clamp_add_sub_full(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t o = 0;
  for (int s = 0; s < 32; s += 8) o |= (uint32_t)clamp255((int)((a >> s) & 0xff) + (int)((b >> s) & 0xff) - (int)((c >> s) & 0xff)) << s;
  return o;
}
uint32_t clamp_add_sub_half(uint32_t a, uint32_t b) {
  uint32_t o = 0;
  for (int s = 0; s < 32; s += 8) {
    const int x = (int)((a >> s) & 0xff), y = (int)((b >> s) & 0xff);
    o |= (uint32_t)clamp255(x + (x - y) / 2) << s;
  }
  return o;
}

void undo_predictor(const Transform& t, std::vector<uint32_t>& px, int w, int h) {
  const int bw = div_up(w, t.bits);
  for (int y = 0; y < h; ++y)
    for (int x = 0; x < w; ++x) {
      const size_t i = (size_t)y * w + x;
      uint32_t pred;
      if (y == 0) pred = x == 0 ? 0xff000000u : px[i - 1];
      else if (x == 0) pred = px[i - (size_t)w];
      else {
        const uint32_t L = px[i - 1], T = px[i - (size_t)w], TL = px[i - (size_t)w - 1], TR = px[i - (size_t)w + 1];
        switch ((t.data[(size_t)(y >> t.bits) * bw + (x >> t.bits)] >> 8) & 0xf) {
          case 0: pred = 0xff000000u; break;
          case 1: pred = L; break;
          case 2: pred = T; break;
          case 3: pred = TR; break;
          case 4: pred = TL; break;
          case 5: pred = avg2(avg2(L, TR), T); break;
          case 6: pred = avg2(L, TL); break;
          case 7: pred = avg2(L, T); break;
          case 8: pred = avg2(TL, T); break;
          case 9: pred = avg2(T, TR); break;
          case 10: pred = avg2(avg2(L, TL), avg2(T, TR)); break;
          case 11: pred = select_px(L, T, TL); break;
          case 12: pred = clamp_add_sub_full(L, T, TL); break;
          case 13: pred = clamp_add_sub_half(avg2(L, T), TL); break;
          default: pred = 0xff000000u; break;
        }
      }
      px[i] = add_px(px[i], pred);
    }
}

int8_t s8(uint32_t v) { return (int8_t)(uint8_t)v; }
uint32_t cdelta(uint32_t t, uint32_t c) { return (uint32_t)(((int)s8(t) * (int)s8(c)) >> 5); }

void undo_cross_colour(const Transform& t, std::vector<uint32_t>& px, int w, int h) {
  const int bw = div_up(w, t.bits);
  for (int y = 0; y < h; ++y)
    for (int x = 0; x < w; ++x) {
      const uint32_t m = t.data[(size_t)(y >> t.bits) * bw + (x >> t.bits)];
      const uint32_t g2r = m & 0xff, g2b = (m >> 8) & 0xff, r2b = (m >> 16) & 0xff;
      uint32_t& p = px[(size_t)y * w + x];
      const uint32_t green = (p >> 8) & 0xff;
      uint32_t red = (p >> 16) & 0xff, blue = p & 0xff;
      red = (red + cdelta(g2r, green)) & 0xff;
      blue = (blue + cdelta(g2b, green) + cdelta(r2b, red)) & 0xff;
      p = (p & 0xff00ff00u) | (red << 16) | blue;
    }
}

void undo_subtract_green(std::vector<uint32_t>& px) {
  for (auto& p : px) {
    const uint32_t g = (p >> 8) & 0xff;
    p = (p & 0xff00ff00u) | ((((p >> 16) & 0xff) + g) & 0xff) << 16 | (((p & 0xff) + g) & 0xff);
  }
}

// px: w_packed x h indices (several per pixel when the palette is small) -> w x h colours
std::vector<uint32_t> undo_indexing(const Transform& t, const std::vector<uint32_t>& px, int w_packed, int w, int h) {
  std::vector<uint32_t> out((size_t)w * h);
  const int per = 1 << t.bits, bpp = 8 >> t.bits;
  const uint32_t mask = (1u << bpp) - 1;
  for (int y = 0; y < h; ++y)
    for (int x = 0; x < w; ++x) {
      const uint32_t packed = (px[(size_t)y * w_packed + (x / per)] >> 8) & 0xff;
      const uint32_t idx = t.bits ? (packed >> ((x % per) * bpp)) & mask : packed;
      out[(size_t)y * w + x] = idx < t.data.size() ? t.data[idx] : 0u;
    }
  return out;
}

// Finds the VP8L payload: a bare "VP8L" chunk, or the one inside a VP8X container (first frame of an animation).
const uint8_t* find_vp8l(const uint8_t* d, size_t n, size_t& len) {
  if (n < 20 || std::memcmp(d, "RIFF", 4) != 0 || std::memcmp(d + 8, "WEBP", 4) != 0) throw std::runtime_error("webp: bad header");
  size_t p = 12;
  bool lossy = false;
  while (p + 8 <= n) {
    const uint32_t sz = d[p + 4] | (d[p + 5] << 8) | (d[p + 6] << 16) | ((uint32_t)d[p + 7] << 24);
    const uint8_t* body = d + p + 8;
    if (p + 8 + (size_t)sz > n) throw std::runtime_error("webp: truncated chunk");
    if (std::memcmp(d + p, "VP8L", 4) == 0) { len = sz; return body; }
    if (std::memcmp(d + p, "VP8 ", 4) == 0) lossy = true;
    if (std::memcmp(d + p, "ANMF", 4) == 0 && sz > 16) {        // frame: 16 bytes of placement, then the frame's own chunks
      size_t q = 16;
      while (q + 8 <= sz) {
        const uint32_t fs = body[q + 4] | (body[q + 5] << 8) | (body[q + 6] << 16) | ((uint32_t)body[q + 7] << 24);
        if (q + 8 + (size_t)fs > sz) break;
        if (std::memcmp(body + q, "VP8L", 4) == 0) { len = fs; return body + q + 8; }
        if (std::memcmp(body + q, "VP8 ", 4) == 0) lossy = true;
        q += 8 + fs + (fs & 1);
      }
    }
    p += 8 + (size_t)sz + (sz & 1);
  }
  throw std::runtime_error(lossy ? "webp: the lossy format (VP8) is not supported, only lossless WebP" : "webp: no image data");
}

void vp8l_size(const uint8_t* v, size_t len, int& w, int& h) {
  if (len < 5 || v[0] != 0x2f) throw std::runtime_error("webp: bad lossless signature");
  const uint32_t bits = v[1] | (v[2] << 8) | (v[3] << 16) | ((uint32_t)v[4] << 24);
  w = (int)(bits & 0x3fff) + 1;
  h = (int)((bits >> 14) & 0x3fff) + 1;
  if ((bits >> 29) != 0) throw std::runtime_error("webp: unknown lossless version");
  if ((long long)w * h > (1ll << 28)) throw std::runtime_error("webp: image too large");
}

}  // namespace

B2H_API const char* b2h_webp_error() { return g_werr.c_str(); }

B2H_API int b2h_webp_info(const uint8_t* d, long n, int* h, int* w) {
  try {
    size_t len = 0;
    const uint8_t* v = find_vp8l(d, (size_t)n, len);
    vp8l_size(v, len, *w, *h);
    return 0;
  } catch (const std::exception& e) { g_werr = e.what(); return 1; }
}

B2H_API int b2h_webp_decode(const uint8_t* d, long n, uint8_t* rgb) {
  try {
    size_t len = 0;
    const uint8_t* v = find_vp8l(d, (size_t)n, len);
    int w, h;
    vp8l_size(v, len, w, h);
    Bits b{v + 5, len - 5};
    std::vector<Transform> tr;
    int cur_w = w;
    bool seen[4] = {false, false, false, false};
    while (b.read(1)) {
      Transform t;
      t.type = (int)b.read(2);
      if (seen[t.type]) throw std::runtime_error("webp: a transform appears twice");
      seen[t.type] = true;
      t.bits = 0;
      t.w_in = cur_w;
      if (t.type == 0 || t.type == 1) {
        t.bits = (int)b.read(3) + 2;
        t.data = decode_pixels(b, div_up(cur_w, t.bits), div_up(h, t.bits), false);
      } else if (t.type == 3) {
        const int colours = (int)b.read(8) + 1;
        t.bits = colours > 16 ? 0 : (colours > 4 ? 1 : (colours > 2 ? 2 : 3));
        t.data = decode_pixels(b, colours, 1, false);
        for (size_t i = 1; i < t.data.size(); ++i) t.data[i] = add_px(t.data[i], t.data[i - 1]);
        cur_w = div_up(cur_w, t.bits);
      }
      tr.push_back(std::move(t));
    }
    std::vector<uint32_t> px = decode_pixels(b, cur_w, h, true);
    for (size_t i = tr.size(); i-- > 0;) {
      const Transform& t = tr[i];
      if (t.type == 0) undo_predictor(t, px, cur_w, h);
      else if (t.type == 1) undo_cross_colour(t, px, cur_w, h);
      else if (t.type == 2) undo_subtract_green(px);
      else { px = undo_indexing(t, px, cur_w, t.w_in, h); cur_w = t.w_in; }
    }
    if (cur_w != w) throw std::runtime_error("webp: inconsistent transforms");
    for (size_t i = 0; i < (size_t)w * h; ++i) {
      rgb[3 * i] = (uint8_t)(px[i] >> 16); rgb[3 * i + 1] = (uint8_t)(px[i] >> 8); rgb[3 * i + 2] = (uint8_t)px[i];
    }
    return 0;
  } catch (const std::exception& e) { g_werr = e.what(); return 1; }
}
