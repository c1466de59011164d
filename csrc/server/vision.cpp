// Image input, host side: smart_resize, antialiased bicubic resize, normalisation and patch layout, placeholder
// expansion and multi-axis rotary positions.  Pure C++ (no image library): pixels arrive as 8-bit RGB (raw or binary
// PPM; compressed formats are decoded by the caller), everything after that is arithmetic.
//
// Reference behaviour: crates/agens-server/src/vision.rs (smart_resize :88-107, expand :154-176, rope_positions
// :178-208) and kernels/oracle/bridge/vision.cpp preprocess (:234-256: antialiased bicubic in fp32, clamp, round to
// 8 bits, (x - 127.5) / 127.5, patches of 2 x 16 x 16 x 3 in merge-block order with the frame duplicated in time).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

// round half to even, as Python's round()
static long long py_round(double v) {
  const double f = std::floor(v);
  const double d = v - f;
  if (d > 0.5) return (long long)f + 1;
  if (d < 0.5) return (long long)f;
  return ((long long)f % 2 == 0) ? (long long)f : (long long)f + 1;
}

// Returns 0 and the target size, or -1 when the aspect ratio is beyond 200.
static int smart_resize(int h, int w, int factor, long long min_pixels, long long max_pixels, int* oh, int* ow) {
  if (h <= 0 || w <= 0) return -1;
  if ((double)std::max(h, w) / (double)std::min(h, w) > 200.0) return -1;
  long long hb = std::max<long long>(factor, py_round((double)h / factor) * factor);
  long long wb = std::max<long long>(factor, py_round((double)w / factor) * factor);
  if (hb * wb > max_pixels) {
    const double beta = std::sqrt((double)h * (double)w / (double)max_pixels);
    hb = std::max<long long>(factor, (long long)std::floor((double)h / beta / factor) * factor);
    wb = std::max<long long>(factor, (long long)std::floor((double)w / beta / factor) * factor);
  } else if (hb * wb < min_pixels) {
    const double beta = std::sqrt((double)min_pixels / ((double)h * (double)w));
    hb = (long long)std::ceil((double)h * beta / factor) * factor;
    wb = (long long)std::ceil((double)w * beta / factor) * factor;
  }
  *oh = (int)hb; *ow = (int)wb;
  return 0;
}

static inline float cubic(float x) {       // Keys kernel, a = -0.5
  const float a = -0.5f;
  x = std::fabs(x);
  if (x < 1.f) return ((a + 2.f) * x - (a + 3.f)) * x * x + 1.f;
  if (x < 2.f) return (((x - 5.f) * x + 8.f) * x - 4.f) * a;
  return 0.f;
}

struct Taps { std::vector<int> start, count; std::vector<float> w; int stride; };

// Antialiased taps: the kernel is stretched by the downscale factor, weights are normalised per output sample.
static Taps make_taps(int in, int out) {
  Taps t;
  const float scale = (float)in / (float)out;
  const float support = scale >= 1.f ? 2.f * scale : 2.f;
  const float invscale = scale >= 1.f ? 1.f / scale : 1.f;
  t.stride = (int)std::ceil(support) * 2 + 1;
  t.start.resize(out); t.count.resize(out); t.w.assign((size_t)out * t.stride, 0.f);
  for (int i = 0; i < out; ++i) {
    const float center = scale * ((float)i + 0.5f);
    const int xmin = std::max(0, (int)(center - support + 0.5f));
    const int xsize = std::min(in, (int)(center + support + 0.5f)) - xmin;
    float total = 0.f;
    for (int j = 0; j < xsize; ++j) {
      const float wv = cubic(((float)(j + xmin) - center + 0.5f) * invscale);
      t.w[(size_t)i * t.stride + j] = wv;
      total += wv;
    }
    for (int j = 0; j < xsize; ++j) t.w[(size_t)i * t.stride + j] /= total;
    t.start[i] = xmin; t.count[i] = xsize;
  }
  return t;
}

// src: [h][w][3] 8-bit.  dst: [3][oh][ow] fp32 (not yet rounded).  Horizontal pass, then vertical, both in fp32.
static void resize_bicubic_aa(const uint8_t* src, int h, int w, int oh, int ow, float* dst) {
  const Taps tx = make_taps(w, ow), ty = make_taps(h, oh);
  std::vector<float> tmp((size_t)3 * h * ow);
  for (int c = 0; c < 3; ++c)
    for (int y = 0; y < h; ++y)
      for (int x = 0; x < ow; ++x) {
        float s = 0.f;
        const float* wv = &tx.w[(size_t)x * tx.stride];
        const uint8_t* row = src + ((size_t)y * w + tx.start[x]) * 3 + c;
        for (int j = 0; j < tx.count[x]; ++j) s += wv[j] * (float)row[(size_t)j * 3];
        tmp[((size_t)c * h + y) * ow + x] = s;
      }
  for (int c = 0; c < 3; ++c)
    for (int y = 0; y < oh; ++y) {
      const float* wv = &ty.w[(size_t)y * ty.stride];
      for (int x = 0; x < ow; ++x) {
        float s = 0.f;
        for (int j = 0; j < ty.count[y]; ++j) s += wv[j] * tmp[((size_t)c * h + ty.start[y] + j) * ow + x];
        dst[((size_t)c * oh + y) * ow + x] = s;
      }
    }
}

// Rounds to 8 bits, normalises to [-1, 1] and lays the pixels out as patches.
// out: [gh*gw][3*2*P*P] fp32, rows in merge-block order (gh/2, gw/2, 2, 2), columns (channel, time 2, py, px).
static void patchify(const float* img, int oh, int ow, int P, float* out) {
  const int gh = oh / P, gw = ow / P;
  const int cols = 3 * 2 * P * P;
  for (int by = 0; by < gh / 2; ++by)
    for (int bx = 0; bx < gw / 2; ++bx)
      for (int iy = 0; iy < 2; ++iy)
        for (int ix = 0; ix < 2; ++ix) {
          const int gy = by * 2 + iy, gx = bx * 2 + ix;
          const size_t row = (((size_t)by * (gw / 2) + bx) * 2 + iy) * 2 + ix;
          float* o = out + row * cols;
          for (int c = 0; c < 3; ++c)
            for (int py = 0; py < P; ++py)
              for (int px = 0; px < P; ++px) {
                float v = img[((size_t)c * oh + gy * P + py) * ow + gx * P + px];
                v = std::nearbyint(std::min(255.f, std::max(0.f, v)));
                v = (v - 127.5f) / 127.5f;
                o[((size_t)(c * 2 + 0) * P + py) * P + px] = v;
                o[((size_t)(c * 2 + 1) * P + py) * P + px] = v;
              }
        }
}

}  // namespace b2

using namespace b2;

B2H_API int b2h_smart_resize(int h, int w, int factor, long long min_pixels, long long max_pixels, int* oh, int* ow) {
  return smart_resize(h, w, factor, min_pixels, max_pixels, oh, ow);
}

// rgb: [h][w][3]; resized: optional [3][oh][ow] fp32 (unrounded); patches: optional [gh*gw][3*2*P*P] fp32.
B2H_API int b2h_image_preprocess(const uint8_t* rgb, int h, int w, int oh, int ow, int patch, float* resized, float* patches) {
  if (!rgb || h <= 0 || w <= 0 || oh <= 0 || ow <= 0 || patch <= 0 || oh % (2 * patch) || ow % (2 * patch)) return -1;
  std::vector<float> img((size_t)3 * oh * ow);
  resize_bicubic_aa(rgb, h, w, oh, ow, img.data());
  if (resized) std::memcpy(resized, img.data(), img.size() * sizeof(float));
  if (patches) patchify(img.data(), oh, ow, patch, patches);
  return 0;
}

// Binary PPM (P6, maxval 255) header parse: returns the offset of the pixel data or -1.
B2H_API int b2h_ppm_header(const uint8_t* data, long n, int* h, int* w) {
  if (n < 11 || data[0] != 'P' || data[1] != '6') return -1;
  long p = 2;
  int vals[3], got = 0;
  while (got < 3 && p < n) {
    while (p < n && (data[p] == ' ' || data[p] == '\n' || data[p] == '\r' || data[p] == '\t')) ++p;
    if (p < n && data[p] == '#') { while (p < n && data[p] != '\n') ++p; continue; }
    int v = 0, digits = 0;
    while (p < n && data[p] >= '0' && data[p] <= '9') { v = v * 10 + (data[p] - '0'); ++p; ++digits; }
    if (!digits) return -1;
    vals[got++] = v;
  }
  if (got < 3 || vals[2] != 255 || p >= n) return -1;
  ++p;                                      // the single whitespace byte after maxval
  if ((long)vals[0] * vals[1] * 3 > n - p) return -1;
  *w = vals[0]; *h = vals[1];
  return (int)p;
}

// Replaces every `pad_id` of `ids` (one per image, in order) by counts[i] copies.  Returns the new length, or -1 when
// the number of placeholders and images differ or `cap` is too small.
B2H_API int b2h_expand_placeholders(const int* ids, int n, int pad_id, const int* counts, int n_images, int* out, int cap) {
  int k = 0, img = 0;
  for (int i = 0; i < n; ++i) {
    if (ids[i] == pad_id) {
      if (img >= n_images) return -1;
      for (int j = 0; j < counts[img]; ++j) { if (k >= cap) return -1; out[k++] = pad_id; }
      ++img;
    } else { if (k >= cap) return -1; out[k++] = ids[i]; }
  }
  return img == n_images ? k : -1;
}

// Multi-axis rotary positions [3][n] (time, height, width).  Text: all three = running position.  The tokens of an
// image with a merged grid of gh x gw start at running position s: token (r, c) gets (s, s + r, s + c); afterwards
// the running position advances by max(gh, gw).  Returns the final running position (next text position).
B2H_API int b2h_mrope_positions(const int* ids, int n, int pad_id, const int* grid_hw, int n_images, int* pos) {
  int run = 0, img = 0, i = 0;
  while (i < n) {
    if (ids[i] == pad_id) {
      if (img >= n_images) return -1;
      const int gh = grid_hw[2 * img], gw = grid_hw[2 * img + 1];
      for (int r = 0; r < gh; ++r)
        for (int c = 0; c < gw; ++c) {
          if (i >= n || ids[i] != pad_id) return -1;
          pos[i] = run; pos[n + i] = run + r; pos[2 * n + i] = run + c;
          ++i;
        }
      run += std::max(gh, gw);
      ++img;
    } else {
      pos[i] = pos[n + i] = pos[2 * n + i] = run;
      ++run; ++i;
    }
  }
  return run;
}
