// Checkpoint core: safetensors reader/writer (mmap), SHA-256, SHA256SUMS verification in parallel, and validation of
// a dense-GQA checkpoint directory against the expected tensor manifest with per-linear format detection.
//
// Reference: crates/agens-core/src/safetensors.rs (reader, dtype set, serialize, advise_sequential) and
// crates/agens-core/src/weights.rs (manifest :35-107, Checkpoint::open :133-165, linear_format :176-187, validate
// :190-251, verify_sha256sums :286-309).  The container is kept (HF directory, safetensors shards + index, packed
// weights + scales); added are 2- and 3-bit streams, fp16 scales and an optional zero-point tensor.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#if defined(__x86_64__)
#include <immintrin.h>
#endif

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "json.hpp"

#define B2H_API extern "C" __attribute__((visibility("default")))

namespace b2 {

// ------------------------------------------------------------------------------------------------ safetensors
struct StTensor { std::string name, dtype; std::vector<long long> shape; long long begin = 0, end = 0; };

struct StFile {
  int fd = -1;
  uint8_t* base = nullptr;
  size_t size = 0, data_off = 0;
  std::vector<StTensor> tensors;
  std::map<std::string, int> index;
  std::string error;
  ~StFile() { if (base) munmap(base, size); if (fd >= 0) close(fd); }
};

static int dtype_size(const std::string& d) {
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "I64" || d == "F64" || d == "U64") return 8;
  if (d == "U8" || d == "I8" || d == "F8_E4M3" || d == "F8_E5M2" || d == "BOOL") return 1;
  return 0;
}

static StFile* st_open(const std::string& path, std::string& err) {
  auto f = new StFile();
  f->fd = open(path.c_str(), O_RDONLY);
  struct stat sb;
  if (f->fd < 0 || fstat(f->fd, &sb) != 0) { err = "cannot open " + path; delete f; return nullptr; }
  f->size = (size_t)sb.st_size;
  if (f->size < 8) { err = "file too small: " + path; delete f; return nullptr; }
  f->base = (uint8_t*)mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (f->base == MAP_FAILED) { f->base = nullptr; err = "mmap failed: " + path; delete f; return nullptr; }
  uint64_t hlen = 0;
  memcpy(&hlen, f->base, 8);
  if (hlen > f->size - 8 || hlen > (100u << 20)) { err = "bad header length in " + path; delete f; return nullptr; }
  f->data_off = 8 + (size_t)hlen;
  try {
    Json h = Json::parse(std::string((const char*)f->base + 8, (size_t)hlen));
    for (auto& kv : h.members()) {
      if (kv.first == "__metadata__") continue;
      StTensor t;
      t.name = kv.first;
      t.dtype = kv.second.at("dtype").as_string();
      for (auto& d : kv.second.at("shape").items()) t.shape.push_back(d.as_int());
      t.begin = kv.second.at("data_offsets")[0].as_int();
      t.end = kv.second.at("data_offsets")[1].as_int();
      long long n = 1;
      bool shape_ok = true;                                // no negative extents, no product beyond 63 bits
      for (auto d : t.shape) shape_ok = shape_ok && d >= 0 && !__builtin_mul_overflow(n, d, &n);
      if (!shape_ok || n > (1ll << 56) || t.begin < 0 || t.end < t.begin || (size_t)t.end > f->size - f->data_off || dtype_size(t.dtype) == 0 ||
          n * dtype_size(t.dtype) != t.end - t.begin) {
        err = "tensor " + t.name + ": offsets do not match dtype and shape";
        delete f;
        return nullptr;
      }
      f->index[t.name] = (int)f->tensors.size();
      f->tensors.push_back(std::move(t));
    }
  } catch (const std::exception& e) { err = std::string("bad safetensors header: ") + e.what(); delete f; return nullptr; }
  return f;
}

// ------------------------------------------------------------------------------------------------ SHA-256
#if defined(__x86_64__)
static const uint32_t kShaK[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
// The compression function on the CPU's SHA extensions (two rounds per instruction, the message schedule in two more):
// about six times the portable loop, which decides how long verifying a checkpoint of tens of gigabytes takes.  Chosen
// at run time; CPUs without the extension keep the portable code.
__attribute__((target("sha,sse4.1,ssse3"))) static void sha256_blocks_ni(uint32_t state[8], const uint8_t* data, size_t nblocks) {
  const __m128i swap = _mm_set_epi64x(0x0c0d0e0f08090a0bll, 0x0405060700010203ll);
  __m128i tmp = _mm_loadu_si128((const __m128i*)&state[0]);          // DCBA
  __m128i s1 = _mm_loadu_si128((const __m128i*)&state[4]);           // HGFE
  tmp = _mm_shuffle_epi32(tmp, 0xB1);                                 // CDAB
  s1 = _mm_shuffle_epi32(s1, 0x1B);                                   // EFGH
  __m128i s0 = _mm_alignr_epi8(tmp, s1, 8);                           // ABEF
  s1 = _mm_blend_epi16(s1, tmp, 0xF0);                                // CDGH
  while (nblocks--) {
    const __m128i save0 = s0, save1 = s1;
    __m128i m[4];
    for (int k = 0; k < 4; ++k) m[k] = _mm_shuffle_epi8(_mm_loadu_si128((const __m128i*)(data + 16 * k)), swap);
    for (int g = 0; g < 16; ++g) {
      __m128i msg = _mm_add_epi32(m[g & 3], _mm_loadu_si128((const __m128i*)(kShaK + 4 * g)));
      s1 = _mm_sha256rnds2_epu32(s1, s0, msg);
      msg = _mm_shuffle_epi32(msg, 0x0E);
      s0 = _mm_sha256rnds2_epu32(s0, s1, msg);
      if (g >= 3 && g < 15) {                                          // the four schedule words of group g + 1
        __m128i t = _mm_sha256msg1_epu32(m[(g + 1) & 3], m[(g + 2) & 3]);
        t = _mm_add_epi32(t, _mm_alignr_epi8(m[g & 3], m[(g + 3) & 3], 4));
        m[(g + 1) & 3] = _mm_sha256msg2_epu32(t, m[g & 3]);
      }
    }
    s0 = _mm_add_epi32(s0, save0);
    s1 = _mm_add_epi32(s1, save1);
    data += 64;
  }
  tmp = _mm_shuffle_epi32(s0, 0x1B);                                  // FEBA
  s1 = _mm_shuffle_epi32(s1, 0xB1);                                   // DCHG
  s0 = _mm_blend_epi16(tmp, s1, 0xF0);                                // DCBA
  s1 = _mm_alignr_epi8(s1, tmp, 8);                                   // HGFE
  _mm_storeu_si128((__m128i*)&state[0], s0);
  _mm_storeu_si128((__m128i*)&state[4], s1);
}
static bool sha_ni_available() {
  static const bool ok = __builtin_cpu_supports("sha") && __builtin_cpu_supports("sse4.1") && __builtin_cpu_supports("ssse3") &&
                         !std::getenv("B200E_NO_SHA_NI");         // the variable keeps the portable loop testable
  return ok;
}
#else
static bool sha_ni_available() { return false; }
static void sha256_blocks_ni(uint32_t*, const uint8_t*, size_t) {}
#endif

struct Sha256 {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t buf[64];
  size_t fill = 0;
  uint64_t total = 0;
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
        0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
        0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
        0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
        0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
        0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
      const uint32_t t1 = hh + S1 + ch + K[i] + w[i];
      const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
      const uint32_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    total += n;
    const bool ni = sha_ni_available();
    while (n) {
      if (fill == 0 && n >= 64) {
        if (ni) { const size_t nb = n / 64; sha256_blocks_ni(h, p, nb); p += nb * 64; n -= nb * 64; continue; }
        block(p); p += 64; n -= 64; continue;
      }
      const size_t k = std::min(n, 64 - fill);
      memcpy(buf + fill, p, k);
      fill += k; p += k; n -= k;
      if (fill == 64) { if (ni) sha256_blocks_ni(h, buf, 1); else block(buf); fill = 0; }
    }
  }
  std::string hex() {
    const uint64_t bits = total * 8;
    uint8_t pad[72] = {0x80};
    const size_t padlen = (fill < 56) ? 56 - fill : 120 - fill;
    uint8_t len[8];
    for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(pad, padlen);
    update(len, 8);
    char out[65];
    for (int i = 0; i < 8; ++i) snprintf(out + 8 * i, 9, "%08x", h[i]);
    return std::string(out, 64);
  }
};

static bool sha256_file(const std::string& path, std::string& hex) {
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) return false;
  posix_fadvise(fd, 0, 0, POSIX_FADV_SEQUENTIAL);
  Sha256 s;
  std::vector<uint8_t> buf(4 << 20);
  ssize_t n;
  while ((n = read(fd, buf.data(), buf.size())) > 0) s.update(buf.data(), (size_t)n);
  close(fd);
  hex = s.hex();
  return n == 0;
}

// Verifies every "<hex>  <file>" line of SHA256SUMS in `dir`, files hashed in parallel.
static Json verify_sums(const std::string& dir, int threads) {
  Json out = Json::object();
  std::ifstream f(dir + "/SHA256SUMS");
  if (!f) { out.set("error", "SHA256SUMS not found"); return out; }
  std::vector<std::pair<std::string, std::string>> items;
  std::string line;
  while (std::getline(f, line)) {
    if (line.size() < 66) continue;
    std::string hex = line.substr(0, 64), name = line.substr(64);
    while (!name.empty() && (name[0] == ' ' || name[0] == '*')) name.erase(0, 1);
    while (!name.empty() && (name.back() == '\r' || name.back() == ' ')) name.pop_back();
    items.emplace_back(hex, name);
  }
  std::vector<int> status(items.size(), 0);   // 1 ok, 2 mismatch, 3 unreadable
  std::atomic<size_t> next{0};
  auto work = [&]() {
    size_t i;
    while ((i = next.fetch_add(1)) < items.size()) {
      std::string hex;
      if (!sha256_file(dir + "/" + items[i].second, hex)) status[i] = 3;
      else status[i] = hex == items[i].first ? 1 : 2;
    }
  };
  std::vector<std::thread> pool;
  for (int t = 0; t < std::max(1, threads); ++t) pool.emplace_back(work);
  for (auto& t : pool) t.join();
  Json bad = Json::array();
  int ok = 0;
  for (size_t i = 0; i < items.size(); ++i) {
    if (status[i] == 1) ++ok;
    else { Json b = Json::object(); b.set("file", items[i].second); b.set("why", status[i] == 2 ? "digest mismatch" : "unreadable"); bad.push_back(b); }
  }
  out.set("files", (long long)items.size());
  out.set("ok", ok);
  out.set("bad", bad);
  return out;
}

// ------------------------------------------------------------------------------------------------ manifest / validation
static std::string read_text(const std::string& p) { std::ifstream f(p); std::stringstream s; s << f.rdbuf(); return s.str(); }

struct Found { std::string dtype; std::vector<long long> shape; std::string file; };

// Format of one linear from the tensors present: bf16 `weight`, or packed (`weight_packed` int32 [n, k*bits/32],
// `weight_scale` [n, k/group] bf16|fp16, optional `weight_zero_point` fp16 [n, k/group]).
static Json linear_format(const std::map<std::string, Found>& t, const std::string& prefix, long long n, long long k, std::string& err) {
  Json o = Json::object();
  auto w = t.find(prefix + ".weight");
  auto p = t.find(prefix + ".weight_packed");
  if (w != t.end() && p == t.end()) {
    if (w->second.dtype != "BF16" || w->second.shape != std::vector<long long>{n, k}) { err = prefix + ".weight: expected BF16 [" + std::to_string(n) + ", " + std::to_string(k) + "]"; return o; }
    o.set("format", "bf16");
    return o;
  }
  if (p == t.end()) { err = prefix + ": neither weight nor weight_packed present"; return o; }
  auto s = t.find(prefix + ".weight_scale");
  if (s == t.end()) { err = prefix + ".weight_scale missing"; return o; }
  if (p->second.dtype != "I32" || p->second.shape.size() != 2 || p->second.shape[0] != n) { err = prefix + ".weight_packed: expected I32 [n, k*bits/32]"; return o; }
  const long long words = p->second.shape[1];
  if ((words * 32) % k != 0) { err = prefix + ".weight_packed: width does not give an integral bit count"; return o; }
  const long long bits = words * 32 / k;
  if (bits < 2 || bits > 4) { err = prefix + ".weight_packed: " + std::to_string(bits) + " bits is not 2, 3 or 4"; return o; }
  if (s->second.shape.size() != 2 || s->second.shape[0] != n || s->second.shape[1] <= 0 || k % s->second.shape[1] != 0) { err = prefix + ".weight_scale: bad shape"; return o; }
  const long long group = k / s->second.shape[1];
  if (group != 64 && group != 128) { err = prefix + ".weight_scale: group size " + std::to_string(group) + " is not 64 or 128"; return o; }
  if (s->second.dtype != "BF16" && s->second.dtype != "F16") { err = prefix + ".weight_scale: expected BF16 or F16"; return o; }
  auto z = t.find(prefix + ".weight_zero_point");
  if (z != t.end() && (z->second.dtype != "F16" || z->second.shape != s->second.shape)) { err = prefix + ".weight_zero_point: expected F16 with the scale's shape"; return o; }
  o.set("format", "wq");
  o.set("bits", bits);
  o.set("group", group);
  o.set("asymmetric", z != t.end());
  o.set("scale_dtype", s->second.dtype);
  return o;
}

static Json validate_dir(const std::string& dir) {
  Json rep = Json::object();
  Json errors = Json::array();
  auto fail = [&](const std::string& e) { errors.push_back(e); };
  Json cfg;
  try { cfg = Json::parse(read_text(dir + "/config.json")); } catch (const std::exception& e) { fail(std::string("config.json: ") + e.what()); rep.set("errors", errors); rep.set("ok", false); return rep; }
  const long long L = cfg.get_int("num_hidden_layers", 0), d = cfg.get_int("hidden_size", 0), hq = cfg.get_int("num_attention_heads", 0);
  const long long hkv = cfg.get_int("num_key_value_heads", hq), ffn = cfg.get_int("intermediate_size", 0), vocab = cfg.get_int("vocab_size", 0);
  const long long hd = cfg.get_int("head_dim", hq ? d / hq : 0);
  if (L <= 0 || d <= 0 || hq <= 0 || hkv <= 0 || ffn <= 0 || vocab <= 0 || hq % hkv) fail("config.json: missing or inconsistent model dimensions");
  // shard list: index file or single file
  std::vector<std::string> shards;
  std::map<std::string, std::string> weight_map;
  {
    std::ifstream idx(dir + "/model.safetensors.index.json");
    if (idx) {
      try {
        Json j = Json::parse(read_text(dir + "/model.safetensors.index.json"));
        for (auto& kv : j.at("weight_map").members()) {
          weight_map[kv.first] = kv.second.as_string();
          if (std::find(shards.begin(), shards.end(), kv.second.as_string()) == shards.end()) shards.push_back(kv.second.as_string());
        }
      } catch (const std::exception& e) { fail(std::string("model.safetensors.index.json: ") + e.what()); }
    } else shards.push_back("model.safetensors");
  }
  std::map<std::string, Found> tensors;
  long long total_bytes = 0;
  for (auto& sh : shards) {
    std::string err;
    StFile* f = st_open(dir + "/" + sh, err);
    if (!f) { fail(err); continue; }
    for (auto& t : f->tensors) {
      if (!weight_map.empty()) {
        auto it = weight_map.find(t.name);
        if (it == weight_map.end()) fail("tensor " + t.name + " in " + sh + " is not in the index");
        else if (it->second != sh) fail("tensor " + t.name + ": index says " + it->second + ", found in " + sh);
      }
      tensors[t.name] = Found{t.dtype, t.shape, sh};
      total_bytes += t.end - t.begin;
    }
    delete f;
  }
  for (auto& kv : weight_map) if (!tensors.count(kv.first)) fail("tensor " + kv.first + " listed in the index is missing from " + kv.second);
  auto expect = [&](const std::string& name, const std::string& dtype, std::vector<long long> shape) {
    auto it = tensors.find(name);
    if (it == tensors.end()) { fail("missing tensor " + name); return; }
    if (it->second.dtype != dtype || it->second.shape != shape) fail(name + ": expected " + dtype + " of the manifest shape");
  };
  Json linears = Json::object();
  Json unexpected = Json::array();
  std::string root = "model.";
  // Text-model tensors live under `model.` (plain decoders) or `model.language_model.` (checkpoints that also carry a
  // vision tower; the reference's manifest uses that prefix: crates/agens-core/src/weights.rs:35-107).
  if (tensors.count("model.language_model.embed_tokens.weight")) root = "model.language_model.";
  std::set<std::string> used;
  auto expect_at = [&](const std::string& name, const std::string& dtype, std::vector<long long> shape) {
    used.insert(name);
    expect(name, dtype, shape);
  };
  auto linear_at = [&](const std::string& name, long long n, long long k) {
    std::string err;
    Json fmt = linear_format(tensors, name, n, k, err);
    if (!err.empty()) { fail(err); return; }
    linears.set(name, fmt);
    for (const char* suf : {".weight", ".weight_packed", ".weight_scale", ".weight_zero_point"})
      if (tensors.count(name + suf)) used.insert(name + suf);
  };
  if (errors.size() == 0) {
    expect_at(root + "embed_tokens.weight", "BF16", {vocab, d});
    expect_at(root + "norm.weight", "BF16", {d});
    const std::pair<const char*, std::pair<long long, long long>> lin[] = {
        {"self_attn.q_proj", {hq * hd, d}}, {"self_attn.k_proj", {hkv * hd, d}}, {"self_attn.v_proj", {hkv * hd, d}},
        {"self_attn.o_proj", {d, hq * hd}}, {"mlp.gate_proj", {ffn, d}}, {"mlp.up_proj", {ffn, d}}, {"mlp.down_proj", {d, ffn}}};
    for (long long l = 0; l < L; ++l) {
      const std::string p = root + "layers." + std::to_string(l) + ".";
      expect_at(p + "input_layernorm.weight", "BF16", {d});
      expect_at(p + "post_attention_layernorm.weight", "BF16", {d});
      // a q_proj with twice the rows carries an output gate (the reference's hybrid attention layers): the dense
      // family has no such gate, so say what it is instead of "bad shape"
      auto qp = tensors.find(p + "self_attn.q_proj.weight_packed");
      if (qp == tensors.end()) qp = tensors.find(p + "self_attn.q_proj.weight");
      if (qp != tensors.end() && qp->second.shape.size() == 2 && qp->second.shape[0] == 2 * hq * hd) {
        fail(p + "self_attn.q_proj has 2 x n_heads x head_dim rows (gated attention output): not a dense GQA layer");
        continue;
      }
      for (auto& e : lin) linear_at(p + e.first, e.second.first, e.second.second);
    }
    const bool tied = cfg.get_bool("tie_word_embeddings", false);
    if (!tied) linear_at("lm_head", vocab, d);
    for (auto& kv : tensors) {
      if (used.count(kv.first)) continue;
      const bool text = kv.first.rfind(root, 0) == 0 || kv.first.rfind("lm_head", 0) == 0;
      if (text) unexpected.push_back(kv.first);       // reported, not fatal (reference: weights.rs leftover report)
    }
  }
  rep.set("ok", errors.size() == 0);
  rep.set("errors", errors);
  rep.set("tensors", (long long)tensors.size());
  rep.set("shards", (long long)shards.size());
  rep.set("bytes", total_bytes);
  rep.set("linears", linears);
  rep.set("root", root);
  rep.set("unexpected", unexpected);
  return rep;
}

}  // namespace b2

using namespace b2;

static char* dup_str(const std::string& s) { char* p = (char*)malloc(s.size() + 1); memcpy(p, s.c_str(), s.size() + 1); return p; }

B2H_API void* b2h_st_open(const char* path, char* err, int err_cap) {
  std::string e;
  StFile* f = st_open(path, e);
  if (!f && err) snprintf(err, err_cap, "%s", e.c_str());
  return f;
}
B2H_API void b2h_st_close(void* f) { delete static_cast<StFile*>(f); }
B2H_API int b2h_st_count(void* f) { return (int)static_cast<StFile*>(f)->tensors.size(); }
// JSON description of tensor i: {"name", "dtype", "shape", "nbytes"}; free with b2h_free_str.
B2H_API char* b2h_st_info(void* fp, int i) {
  auto f = static_cast<StFile*>(fp);
  const StTensor& t = f->tensors[i];
  Json o = Json::object();
  o.set("name", t.name); o.set("dtype", t.dtype);
  Json sh = Json::array();
  for (auto d : t.shape) sh.push_back(d);
  o.set("shape", sh); o.set("nbytes", t.end - t.begin);
  return dup_str(o.dump());
}
B2H_API const void* b2h_st_data(void* fp, const char* name, long long* nbytes) {
  auto f = static_cast<StFile*>(fp);
  auto it = f->index.find(name);
  if (it == f->index.end()) return nullptr;
  const StTensor& t = f->tensors[it->second];
  if (nbytes) *nbytes = t.end - t.begin;
  return f->base + f->data_off + t.begin;
}
B2H_API void b2h_st_advise_sequential(void* fp) { auto f = static_cast<StFile*>(fp); madvise(f->base, f->size, MADV_SEQUENTIAL); }
B2H_API char* b2h_sha256_file(const char* path) { std::string h; return dup_str(sha256_file(path, h) ? h : std::string()); }
B2H_API char* b2h_sha256_bytes(const void* p, long long n) { Sha256 s; s.update((const uint8_t*)p, (size_t)n); return dup_str(s.hex()); }
B2H_API char* b2h_verify_sha256sums(const char* dir, int threads) { return dup_str(verify_sums(dir, threads).dump()); }
B2H_API char* b2h_validate_checkpoint(const char* dir) {
  try { return dup_str(validate_dir(dir).dump()); }
  catch (const std::exception& e) { Json o = Json::object(); o.set("ok", false); Json er = Json::array(); er.push_back(std::string(e.what())); o.set("errors", er); return dup_str(o.dump()); }
}
