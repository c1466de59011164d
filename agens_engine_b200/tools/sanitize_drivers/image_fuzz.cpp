// Damaged image files through the host decoders under AddressSanitizer / UBSan: seed files (a directory, argv[1]) are
// mutated argv[2] times with the generator seeded by argv[3]; PNG scanline reconstruction gets random geometry and
// bytes.  Built and run by tools/sanitize.py (fuzz-images) against a sanitizer build of the host library.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <dirent.h>
extern "C" {
int b2h_jpeg_info(const uint8_t*, long, int*, int*, int*);
int b2h_jpeg_decode(const uint8_t*, long, uint8_t*);
int b2h_webp_info(const uint8_t*, long, int*, int*);
int b2h_webp_decode(const uint8_t*, long, uint8_t*);
int b2h_bmp_info(const uint8_t*, long, int*, int*);
int b2h_bmp_decode(const uint8_t*, long, uint8_t*);
int b2h_gif_info(const uint8_t*, long, int*, int*);
int b2h_gif_decode(const uint8_t*, long, uint8_t*);
int b2h_png_unfilter(const uint8_t* raw, long n, int w, int h, int depth, int ctype, int interlace, const uint8_t* pal, int npal, uint8_t* out);
}
static uint64_t s = 88172645463325252ull;
static uint64_t rnd() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; }
static std::vector<uint8_t> readf(const std::string& p) {
  FILE* f = fopen(p.c_str(), "rb"); std::vector<uint8_t> v; uint8_t b[4096]; size_t n;
  while ((n = fread(b, 1, sizeof b, f)) > 0) v.insert(v.end(), b, b + n);
  fclose(f); return v;
}
static long ok = 0, bad = 0;
static void run(const std::string& ext, const std::vector<uint8_t>& in) {
  // exact-size copy so that ASan sees reads past the end
  uint8_t* d = (uint8_t*)malloc(in.size() ? in.size() : 1); memcpy(d, in.data(), in.size());
  long n = (long)in.size(); int h = 0, w = 0, c = 0, r;
  if (ext == "jpg") r = b2h_jpeg_info(d, n, &h, &w, &c);
  else if (ext == "webp") r = b2h_webp_info(d, n, &h, &w);
  else if (ext == "bmp") r = b2h_bmp_info(d, n, &h, &w);
  else r = b2h_gif_info(d, n, &h, &w);
  if (r == 0 && h > 0 && w > 0 && (long)h * w <= (1 << 22)) {
    uint8_t* out = (uint8_t*)malloc((size_t)h * w * 3);
    if (ext == "jpg") r = b2h_jpeg_decode(d, n, out);
    else if (ext == "webp") r = b2h_webp_decode(d, n, out);
    else if (ext == "bmp") r = b2h_bmp_decode(d, n, out);
    else r = b2h_gif_decode(d, n, out);
    free(out);
  } else if (r == 0) r = 1;
  (r == 0 ? ok : bad)++;
  free(d);
}
int main(int argc, char** argv) {
  std::string dir = argv[1]; long iters = atol(argv[2]); if (argc > 3) s ^= strtoull(argv[3], 0, 10) * 0x9E3779B97F4A7C15ull;
  std::vector<std::pair<std::string, std::vector<uint8_t>>> seeds;
  DIR* dp = opendir(dir.c_str()); dirent* e;
  while ((e = readdir(dp))) { std::string nm = e->d_name; auto p = nm.rfind('.'); if (p == std::string::npos || nm[0] == '.') continue;
    seeds.push_back({nm.substr(p + 1), readf(dir + "/" + nm)}); }
  for (auto& sd : seeds) run(sd.first, sd.second);
  printf("seeds ok=%ld bad=%ld\n", ok, bad);
  for (long it = 0; it < iters; ++it) {
    auto& sd = seeds[rnd() % seeds.size()];
    std::vector<uint8_t> m = sd.second;
    int k = 1 + rnd() % 4;
    for (int j = 0; j < k && !m.empty(); ++j) {
      switch (rnd() % 6) {
        case 0: m[rnd() % m.size()] = (uint8_t)rnd(); break;
        case 1: m[rnd() % m.size()] ^= 1u << (rnd() % 8); break;
        case 2: m.resize(rnd() % m.size()); break;
        case 3: { size_t a = rnd() % m.size(), l = rnd() % 16; for (size_t q = a; q < a + l && q < m.size(); ++q) m[q] = (rnd() & 1) ? 0xFF : 0; } break;
        case 4: { size_t a = rnd() % m.size(), b = rnd() % m.size(), l = rnd() % 64; for (size_t q = 0; q < l && a + q < m.size() && b + q < m.size(); ++q) m[a + q] = m[b + q]; } break;
        case 5: { size_t a = rnd() % m.size(); size_t l = rnd() % 32; m.erase(m.begin() + a, m.begin() + std::min(m.size(), a + l)); } break;
      }
    }
    run(sd.first, m);
  }
  // PNG scanline reconstruction: random geometry and random bytes
  for (long it = 0; it < iters / 4; ++it) {
    int w = 1 + rnd() % 40, h = 1 + rnd() % 40; static const int depths[] = {1, 2, 4, 8, 16, 3, 0}; static const int ct[] = {0, 2, 3, 4, 6, 5};
    int depth = depths[rnd() % 7], ctype = ct[rnd() % 6], inter = rnd() % 3;
    long n = rnd() % (w * h * 8 + 64); int npal = rnd() % 258;
    uint8_t* raw = (uint8_t*)malloc(n ? n : 1); for (long q = 0; q < n; ++q) raw[q] = (rnd() % 3 == 0) ? rnd() % 5 : (uint8_t)rnd();
    uint8_t* pal = (uint8_t*)malloc(npal * 3 + 1); for (int q = 0; q < npal * 3; ++q) pal[q] = (uint8_t)rnd();
    uint8_t* out = (uint8_t*)malloc((size_t)w * h * 3);
    int r = b2h_png_unfilter(raw, n, w, h, depth, ctype, inter, pal, npal, out);
    (r == 0 ? ok : bad)++;
    free(raw); free(pal); free(out);
  }
  printf("done ok=%ld bad=%ld\n", ok, bad);
}
