// BMP and GIF (first frame) readers and the PNG scanline reconstruction for image inputs of chat requests, next to the
// PPM / JPEG / WebP readers.
//
// The reference accepts these formats through its image crate / nvJPEG path (crates/agens-server/src/vision.rs:126-135);
// here they are decoded on the host.  BMP: uncompressed 24 / 32-bit and 8-bit palettised, bottom-up or top-down.
// GIF: the first image of the file (87a / 89a), global or local colour table, interlaced or not, LZW decoded;
// transparency is ignored (the colour of the index is used), animation frames after the first are not read.
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_err;
int fail(const char* m) { g_err = m; return 1; }
uint32_t le16(const uint8_t* p) { return p[0] | (p[1] << 8); }
uint32_t le32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | ((uint32_t)p[3] << 24); }

struct BmpInfo { int w, h, bpp, off, ncolors, hdr; bool top_down; };

int bmp_parse(const uint8_t* d, long n, BmpInfo& b) {
  if (n < 54 || d[0] != 'B' || d[1] != 'M') return fail("bmp: bad header");
  b.off = (int)le32(d + 10);
  b.hdr = (int)le32(d + 14);
  if (b.hdr < 40) return fail("bmp: only BITMAPINFOHEADER and later are supported");
  const int32_t w = (int32_t)le32(d + 18), h = (int32_t)le32(d + 22);
  b.w = w;
  b.top_down = h < 0;
  b.h = h < 0 ? -h : h;
  b.bpp = (int)le16(d + 28);
  const uint32_t comp = le32(d + 30);
  if (comp != 0 && !(comp == 3 && b.bpp == 32)) return fail("bmp: compressed bitmaps are not supported");
  if (b.bpp != 24 && b.bpp != 32 && b.bpp != 8) return fail("bmp: only 8, 24 and 32 bits per pixel are supported");
  if (b.w <= 0 || b.h <= 0 || (long long)b.w * b.h > (1ll << 28)) return fail("bmp: bad size");
  b.ncolors = (int)le32(d + 46);
  if (b.bpp == 8 && b.ncolors == 0) b.ncolors = 256;
  const long stride = ((long)b.w * b.bpp + 31) / 32 * 4;
  if (b.off < 14 + b.hdr || b.off + stride * b.h > n) return fail("bmp: truncated");
  if (b.bpp == 8 && 14 + b.hdr + 4l * b.ncolors > n) return fail("bmp: truncated palette");
  return 0;
}

struct GifInfo { int w, h; };

}  // namespace

B2H_API const char* b2h_image_error() { return g_err.c_str(); }

B2H_API int b2h_bmp_info(const uint8_t* d, long n, int* h, int* w) {
  BmpInfo b;
  if (bmp_parse(d, n, b)) return 1;
  *h = b.h; *w = b.w;
  return 0;
}

B2H_API int b2h_bmp_decode(const uint8_t* d, long n, uint8_t* rgb) {
  BmpInfo b;
  if (bmp_parse(d, n, b)) return 1;
  const long stride = ((long)b.w * b.bpp + 31) / 32 * 4;
  const uint8_t* pal = d + 14 + b.hdr;
  for (int y = 0; y < b.h; ++y) {
    const uint8_t* row = d + b.off + stride * (b.top_down ? y : b.h - 1 - y);
    uint8_t* o = rgb + (size_t)y * b.w * 3;
    for (int x = 0; x < b.w; ++x) {
      if (b.bpp == 8) {
        const int i = row[x];
        if (i >= b.ncolors) return fail("bmp: palette index out of range");
        o[3 * x] = pal[4 * i + 2]; o[3 * x + 1] = pal[4 * i + 1]; o[3 * x + 2] = pal[4 * i];
      } else {
        const uint8_t* p = row + (size_t)x * (b.bpp / 8);
        o[3 * x] = p[2]; o[3 * x + 1] = p[1]; o[3 * x + 2] = p[0];
      }
    }
  }
  return 0;
}

// Logical screen size of a GIF (the decoded frame is painted onto a canvas of that size).
B2H_API int b2h_gif_info(const uint8_t* d, long n, int* h, int* w) {
  if (n < 13 || std::memcmp(d, "GIF8", 4) != 0 || (d[4] != '7' && d[4] != '9') || d[5] != 'a') return fail("gif: bad header");
  *w = (int)le16(d + 6);
  *h = (int)le16(d + 8);
  if (*w <= 0 || *h <= 0 || (long long)*w * *h > (1ll << 28)) return fail("gif: bad size");
  return 0;
}

B2H_API int b2h_gif_decode(const uint8_t* d, long n, uint8_t* rgb) {
  int H, W;
  if (b2h_gif_info(d, n, &H, &W)) return 1;
  const uint8_t* p = d + 13;
  const uint8_t* end = d + n;
  const uint8_t* gct = nullptr;
  int gct_n = 0;
  const int bg = d[11];
  if (d[10] & 0x80) {
    gct_n = 1 << ((d[10] & 7) + 1);
    if (p + 3 * gct_n > end) return fail("gif: truncated colour table");
    gct = p;
    p += 3 * gct_n;
  }
  // canvas starts as the background colour (black without a global table)
  for (long i = 0; i < (long)W * H; ++i) {
    const uint8_t* c = (gct && bg < gct_n) ? gct + 3 * bg : nullptr;
    rgb[3 * i] = c ? c[0] : 0; rgb[3 * i + 1] = c ? c[1] : 0; rgb[3 * i + 2] = c ? c[2] : 0;
  }
  while (p < end) {
    const uint8_t tag = *p++;
    if (tag == 0x3B) break;                               // trailer
    if (tag == 0x21) {                                    // extension: label, then sub-blocks
      if (p >= end) break;
      ++p;
      while (p < end && *p) p += 1 + *p;
      ++p;
      continue;
    }
    if (tag != 0x2C) return fail("gif: unexpected block");
    if (p + 9 > end) return fail("gif: truncated image descriptor");
    const int x0 = (int)le16(p), y0 = (int)le16(p + 2), w = (int)le16(p + 4), h = (int)le16(p + 6);
    const uint8_t flags = p[8];
    p += 9;
    const uint8_t* ct = gct;
    int ct_n = gct_n;
    if (flags & 0x80) {
      ct_n = 1 << ((flags & 7) + 1);
      if (p + 3 * ct_n > end) return fail("gif: truncated colour table");
      ct = p;
      p += 3 * ct_n;
    }
    if (!ct) return fail("gif: no colour table");
    if (w <= 0 || h <= 0 || x0 + w > W || y0 + h > H) return fail("gif: frame outside the screen");
    if (p >= end) return fail("gif: truncated");
    const int min_code = *p++;
    if (min_code < 2 || min_code > 8) return fail("gif: bad LZW code size");
    // gather the data sub-blocks
    std::vector<uint8_t> data;
    while (p < end && *p) {
      const int len = *p++;
      if (p + len > end) return fail("gif: truncated data");
      data.insert(data.end(), p, p + len);
      p += len;
    }
    // LZW
    const int clear = 1 << min_code, eoi = clear + 1;
    std::vector<uint16_t> prefix(4096);
    std::vector<uint8_t> suffix(4096), stack(4097);
    std::vector<uint8_t> idx((size_t)w * h, 0);
    int code_size = min_code + 1, next = eoi + 1, prev = -1;
    uint32_t acc = 0;
    int nb = 0;
    size_t out = 0, di = 0;
    for (int i = 0; i < clear; ++i) { prefix[i] = 0; suffix[i] = (uint8_t)i; }
    uint8_t first = 0;
    while (out < idx.size()) {
      while (nb < code_size && di < data.size()) { acc |= (uint32_t)data[di++] << nb; nb += 8; }
      if (nb < code_size) break;
      int code = (int)(acc & ((1u << code_size) - 1));
      acc >>= code_size;
      nb -= code_size;
      if (code == clear) { code_size = min_code + 1; next = eoi + 1; prev = -1; continue; }
      if (code == eoi) break;
      int sp = 0, cur = code;
      if (prev < 0) {
        if (code >= clear) return fail("gif: bad first code");
        idx[out++] = (uint8_t)code;
        first = (uint8_t)code;
        prev = code;
        continue;
      }
      if (code >= next) {                                 // the code being defined right now: prev string + its first symbol
        if (code > next) return fail("gif: bad LZW code");
        stack[sp++] = first;
        cur = prev;
      }
      while (cur >= clear) {
        if (cur >= 4096 || sp >= 4096) return fail("gif: bad LZW chain");
        stack[sp++] = suffix[cur];
        cur = prefix[cur];
      }
      stack[sp++] = (uint8_t)cur;
      first = (uint8_t)cur;
      if (next < 4096) {
        prefix[next] = (uint16_t)prev;
        suffix[next] = first;
        ++next;
        if (next == (1 << code_size) && code_size < 12) ++code_size;
      }
      prev = code;
      while (sp > 0 && out < idx.size()) idx[out++] = stack[--sp];
    }
    // paint (interlaced rows come in four passes)
    std::vector<int> rows(h);
    if (flags & 0x40) {
      int r = 0;
      const int start[4] = {0, 4, 2, 1}, step[4] = {8, 8, 4, 2};
      for (int ps = 0; ps < 4; ++ps)
        for (int y = start[ps]; y < h; y += step[ps]) rows[r++] = y;
    } else {
      for (int y = 0; y < h; ++y) rows[y] = y;
    }
    for (int r = 0; r < h; ++r)
      for (int x = 0; x < w; ++x) {
        const int i = idx[(size_t)r * w + x];
        if (i >= ct_n) continue;
        uint8_t* o = rgb + ((size_t)(y0 + rows[r]) * W + x0 + x) * 3;
        o[0] = ct[3 * i]; o[1] = ct[3 * i + 1]; o[2] = ct[3 * i + 2];
      }
    return 0;                                             // first frame only
  }
  return fail("gif: no image in the file");
}

// ---- PNG: scanline reconstruction ----------------------------------------------------------------------------------------
// The inflated IDAT stream (zlib runs in the caller) -> RGB: filter types 0..4, bit depths 1 / 2 / 4 / 8 / 16, colour types
// grey / RGB / palette / grey+alpha / RGBA (alpha dropped, 16-bit samples keep their high byte), Adam7 interlacing.
// pal: the PLTE entries (3 bytes each).  Returns 0 on success.
namespace {

inline int paeth(int a, int b, int c) {
  const int pa = std::abs(b - c), pb = std::abs(a - c), pc = std::abs(a + b - 2 * c);
  return pa <= pb && pa <= pc ? a : (pb <= pc ? b : c);
}

// One sub-image (the whole picture, or one Adam7 pass): pw x ph pixels whose scanlines start at raw; writes pixel (i, j) of
// it to rgb at (x0 + i * dx, y0 + j * dy).  Returns the bytes consumed, or -1.
long png_pass(const uint8_t* raw, long n, int pw, int ph, int depth, int ctype, const uint8_t* pal, int npal, uint8_t* rgb, int W,
              int x0, int y0, int dx, int dy) {
  static const int kCh[7] = {1, 0, 3, 1, 2, 0, 4};
  const int ch = kCh[ctype];
  const int bpp = std::max(1, ch * depth / 8);
  const long line = ((long)pw * ch * depth + 7) / 8;
  if (pw == 0 || ph == 0) return 0;
  if ((line + 1) * ph > n) return -1;
  std::vector<uint8_t> prev((size_t)line, 0), cur((size_t)line);
  for (int j = 0; j < ph; ++j) {
    const uint8_t* src = raw + (size_t)j * (line + 1);
    const int f = src[0];
    ++src;
    for (long i = 0; i < line; ++i) {
      const int a = i >= bpp ? cur[(size_t)(i - bpp)] : 0, b = prev[(size_t)i], c = i >= bpp ? prev[(size_t)(i - bpp)] : 0;
      int pr;
      switch (f) {
        case 0: pr = 0; break;
        case 1: pr = a; break;
        case 2: pr = b; break;
        case 3: pr = (a + b) >> 1; break;
        case 4: pr = paeth(a, b, c); break;
        default: return -1;
      }
      cur[(size_t)i] = (uint8_t)(src[i] + pr);
    }
    const int maxv = (1 << depth) - 1;
    for (int i = 0; i < pw; ++i) {
      auto sample = [&](int k) -> int {       // k-th sample of the pixel, as 8 bits (raw index for palette images)
        const long s = (long)i * ch + k;
        if (depth == 8) return cur[(size_t)s];
        if (depth == 16) return cur[(size_t)(2 * s)];
        const long bit = s * depth;
        const int v = (cur[(size_t)(bit >> 3)] >> (8 - depth - (bit & 7))) & maxv;
        return ctype == 3 ? v : v * 255 / maxv;
      };
      uint8_t* o = rgb + ((size_t)(y0 + j * dy) * W + (size_t)(x0 + i * dx)) * 3;
      if (ctype == 3) {
        const int idx = sample(0);
        if (idx < npal) { o[0] = pal[3 * idx]; o[1] = pal[3 * idx + 1]; o[2] = pal[3 * idx + 2]; }
        else { o[0] = o[1] = o[2] = 0; }
      } else if (ch <= 2) {
        o[0] = o[1] = o[2] = (uint8_t)sample(0);
      } else {
        o[0] = (uint8_t)sample(0); o[1] = (uint8_t)sample(1); o[2] = (uint8_t)sample(2);
      }
    }
    prev.swap(cur);
  }
  return (line + 1) * ph;
}

}  // namespace

B2H_API int b2h_png_unfilter(const uint8_t* raw, long n, int w, int h, int depth, int ctype, int interlace, const uint8_t* pal,
                             int npal, uint8_t* rgb) {
  if (w <= 0 || h <= 0 || (long long)w * h > (1ll << 28)) return fail("png: bad size");
  const bool depth_ok = (ctype == 0 && (depth == 1 || depth == 2 || depth == 4 || depth == 8 || depth == 16)) ||
                        (ctype == 3 && (depth == 1 || depth == 2 || depth == 4 || depth == 8)) ||
                        ((ctype == 2 || ctype == 4 || ctype == 6) && (depth == 8 || depth == 16));
  if (!depth_ok) return fail("png: bad colour type / bit depth");
  if (ctype == 3 && (!pal || npal <= 0)) return fail("png: palette image without a palette");
  if (interlace == 0) {
    if (png_pass(raw, n, w, h, depth, ctype, pal, npal, rgb, w, 0, 0, 1, 1) < 0) return fail("png: truncated or damaged image data");
    return 0;
  }
  if (interlace != 1) return fail("png: unknown interlace method");
  static const int kX0[7] = {0, 4, 0, 2, 0, 1, 0}, kY0[7] = {0, 0, 4, 0, 2, 0, 1}, kDx[7] = {8, 8, 4, 4, 2, 2, 1}, kDy[7] = {8, 8, 8, 4, 4, 2, 2};
  long off = 0;
  for (int p = 0; p < 7; ++p) {
    const int pw = (w - kX0[p] + kDx[p] - 1) / kDx[p], ph = (h - kY0[p] + kDy[p] - 1) / kDy[p];
    if (pw <= 0 || ph <= 0) continue;
    const long used = png_pass(raw + off, n - off, pw, ph, depth, ctype, pal, npal, rgb, w, kX0[p], kY0[p], kDx[p], kDy[p]);
    if (used < 0) return fail("png: truncated or damaged image data");
    off += used;
  }
  return 0;
}
