// Weight layout tools for the FM (fragment-major) mixed-bit format: checkpoint container -> FM repack on the
// device, FM -> bf16 dequantisation (prefill GEMM operand, tests), and on-device random initialisation of a
// quantised linear directly in FM form (benchmarks with random-init weights of a named architecture).
// Counterparts in the reference: repack_kt_kernel / repack_wq_kernel / dequant_kt_kernel
// (kernels/src/w4_gemv.cu:441-464, :759) and the host quantisers quantize_wq / quantize_w4
// (crates/agens-cli/src/spec.rs:496-552).
#include "wq_gemv.cuh"

namespace b2 {
namespace {

__device__ __constant__ int kHiSrc[4][4] = {{0, 2, 4, 6}, {1, 3, 5, 7}, {8, 10, 12, 14}, {9, 11, 13, 15}};

struct FmPos {
  size_t rec;      // byte offset of the record (32 lanes x 16 B [+ 32 x 8 B]) inside the FM buffer
  int lane;        // lane inside the record
  int word, bit;   // low plane: 32-bit word of the lane's 16 bytes, bit position of the field's LSB
  int hword, hbit; // 3-bit high plane
};

__device__ __forceinline__ int fm_w_batch(int bits) { return bits == 3 ? 768 : (bits == 4 ? 1024 : 512); }
__device__ __forceinline__ int fm_block(int bits, int group) { return 2 * fm_w_batch(bits) + 2 * (128 / group) * 64; }

// Position of code (row r, column k) inside the FM layout.  Mirrors utils/quant.py::_slot_tables / pack_fm:
// blocks of (32-row panel, 128-k batch) = [2 row blocks x records][2 row blocks x groups x 16 rows x (scale, zero)].
__device__ __forceinline__ FmPos fm_pos(int r, int k, int bits, int group, int nbat) {
  const int ck = bits == 4 ? 64 : 128;
  const int panel = r >> 5, rbp = (r >> 4) & 1, rr = r & 15, g = rr & 7, rh = rr >> 3;
  const int batch = k >> 7, kb = k & 127;
  const int chunk = kb / ck, kk = kb - chunk * ck;
  const int step = kk >> 4, t = (kk >> 2) & 3, slot = kk & 3;
  FmPos p;
  p.rec = ((size_t)panel * nbat + batch) * fm_block(bits, group) + (size_t)rbp * fm_w_batch(bits) +
          (size_t)chunk * (bits == 3 ? 768 : 512);
  p.lane = g * 4 + t;
  const int hi16 = slot & 1;
  if (bits == 4) {
    p.word = step;
    p.bit = 4 * (slot >> 1) + 8 * rh + 16 * hi16;
    p.hword = 0; p.hbit = 0;
  } else {
    const int u = step >> 1, q = 2 * (step & 1) + (slot >> 1);
    p.word = u;
    p.bit = 2 * q + 8 * rh + 16 * hi16;
    p.hword = u >> 1;
    p.hbit = kHiSrc[2 * (u & 1) + rh][q] + 16 * hi16;
  }
  return p;
}

// Address of the (scale, zero) pair of (row r, group gi).
__device__ __forceinline__ size_t fm_sz_off(int r, int gi, int bits, int group, int nbat) {
  const int gpb = 128 / group;
  const int panel = r >> 5, rbp = (r >> 4) & 1, rr = r & 15;
  const int batch = gi / gpb, gl = gi - batch * gpb;
  return ((size_t)panel * nbat + batch) * fm_block(bits, group) + 2 * (size_t)fm_w_batch(bits) +
         ((size_t)(rbp * gpb + gl) * 16 + rr) * 4;
}

__device__ __forceinline__ void fm_store_code(uint8_t* wq, const FmPos& p, int bits, unsigned code) {
  uint32_t* rec = reinterpret_cast<uint32_t*>(wq + p.rec);
  const unsigned lo = bits == 3 ? (code & 3u) : code;
  atomicOr(rec + p.lane * 4 + p.word, lo << p.bit);
  if (bits == 3) atomicOr(rec + 128 + p.lane * 2 + p.hword, ((code >> 2) & 1u) << p.hbit);
}

__device__ __forceinline__ unsigned fm_load_code(const uint8_t* wq, const FmPos& p, int bits) {
  const uint32_t* rec = reinterpret_cast<const uint32_t*>(wq + p.rec);
  const unsigned lo_bits = bits == 3 ? 2 : bits;
  unsigned c = (rec[p.lane * 4 + p.word] >> p.bit) & ((1u << lo_bits) - 1u);
  if (bits == 3) c |= ((rec[128 + p.lane * 2 + p.hword] >> p.hbit) & 1u) << 2;
  return c;
}

__global__ void wq_dequant_kernel(const uint8_t* __restrict__ wq, int n, int k, int bits, int group,
                                  bf16* __restrict__ out, long ldo) {
  // one thread per 4 consecutive k of one row (the lane's 4 slots of one mma step)
  const long total = (long)n * (k >> 2);
  const int nbat = k >> 7;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / (k >> 2));
    const int k4 = (int)(idx - (long)r * (k >> 2)) << 2;
    const __half2 s = *reinterpret_cast<const __half2*>(wq + fm_sz_off(r, k4 / group, bits, group, nbat));
    const float sc = __low2float(s), zp = __high2float(s);
    __align__(8) bf16 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const FmPos p = fm_pos(r, k4 + i, bits, group, nbat);
      v[i] = __float2bfloat16_rn(((float)fm_load_code(wq, p, bits) - zp) * sc);
    }
    *reinterpret_cast<uint2*>(out + (size_t)r * ldo + k4) = *reinterpret_cast<const uint2*>(v);
  }
}

__global__ void wq_repack_kernel(const int32_t* __restrict__ packed, const void* __restrict__ scale, int scale_is_bf16,
                                 const __half* __restrict__ zero, int n, int k, int bits, int group,
                                 uint8_t* __restrict__ wq) {
  const long total = (long)n * k;
  const int nbat = k >> 7;
  const int ng = k / group;
  const int wpr = k * bits / 32;   // words per row of the bit stream
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / k), c = (int)(idx - (long)r * k);
    const long bitpos = (long)c * bits;
    const int w = (int)(bitpos >> 5), sh = (int)(bitpos & 31);
    const uint32_t* row = reinterpret_cast<const uint32_t*>(packed) + (size_t)r * wpr;
    uint64_t two = row[w];
    if (sh + bits > 32) two |= (uint64_t)row[w + 1] << 32;
    const unsigned code = (unsigned)(two >> sh) & ((1u << bits) - 1u);
    fm_store_code(wq, fm_pos(r, c, bits, group, nbat), bits, code);
    if (c % group == 0) {
      const int gi = c / group;
      float s;
      if (scale_is_bf16) s = __bfloat162float(reinterpret_cast<const bf16*>(scale)[(size_t)r * ng + gi]);
      else s = __half2float(reinterpret_cast<const __half*>(scale)[(size_t)r * ng + gi]);
      const float z = zero ? __half2float(zero[(size_t)r * ng + gi]) : (float)(1 << (bits - 1));
      *reinterpret_cast<__half2*>(wq + fm_sz_off(r, gi, bits, group, nbat)) = __floats2half2_rn(s, z);
    }
  }
}


// ---- FI layout ("fragment-major, integer"): the same blocks, records and (scale, zero) pairs as FM, but the codes of
// a lane are laid out for mma.m16n8k32 with 8-bit operands: one AND (plus one shift for every other register) turns a
// 32-bit word into four codes of ONE row as four bytes, i.e. one A register of the integer MMA.  For step s (32 k) of
// a 128-k batch, lane (g, t) holds registers r = 0..3: row g + 8 (r & 1), k = 32 s + 16 (r >> 1) + 4 t + byte.
//   4 bits: chunk s >> 1, word 2 (s & 1) + (r & 1), bit 8 byte + 4 (r >> 1)
//   2 bits: word s, bit 8 byte + 2 r;   3 bits: low plane as 2 bits, high bit in word s >> 1 at bit 8 byte + 4 (s & 1) + r
// The persistent decode-step kernel (step_kernel.cu) consumes this layout; everything else reads FM.
__device__ __forceinline__ FmPos fi_pos(int r, int k, int bits, int group, int nbat) {
  const int panel = r >> 5, rbp = (r >> 4) & 1, rr = r & 15, g = rr & 7, rh = rr >> 3;
  const int batch = k >> 7, kb = k & 127;
  const int s = kb >> 5, kl = kb & 31, half = kl >> 4, t = (kl >> 2) & 3, j = kl & 3;
  const int reg = rh + 2 * half;
  FmPos p;
  p.rec = ((size_t)panel * nbat + batch) * fm_block(bits, group) + (size_t)rbp * fm_w_batch(bits);
  p.lane = g * 4 + t;
  p.hword = 0; p.hbit = 0;
  if (bits == 4) {
    p.rec += (size_t)(s >> 1) * 512;
    p.word = 2 * (s & 1) + (reg & 1);
    p.bit = 8 * j + 4 * (reg >> 1);
  } else {
    p.word = s;
    p.bit = 8 * j + 2 * reg;
    p.hword = s >> 1;
    p.hbit = 8 * j + 4 * (s & 1) + reg;
  }
  return p;
}

// FM -> FI: one thread per code (a one-time conversion when a model opens the step kernel).
__global__ void wq_fm_to_fi_kernel(const uint8_t* __restrict__ fm, int n, int k, int bits, int group, uint8_t* __restrict__ fi) {
  const long total = (long)n * k;
  const int nbat = k >> 7;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / k), c = (int)(idx - (long)r * k);
    const unsigned code = fm_load_code(fm, fm_pos(r, c, bits, group, nbat), bits);
    fm_store_code(fi, fi_pos(r, c, bits, group, nbat), bits, code);
    if (c % group == 0) {
      const size_t off = fm_sz_off(r, c / group, bits, group, nbat);
      *reinterpret_cast<uint32_t*>(fi + off) = *reinterpret_cast<const uint32_t*>(fm + off);
    }
  }
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// Standard normal from a counter (Box-Muller on two 32-bit uniforms of one 64-bit hash).
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t idx) {
  const uint64_t h = splitmix64(seed ^ splitmix64(idx));
  const float u1 = ((float)(uint32_t)(h >> 32) + 1.0f) * (1.0f / 4294967296.0f);
  const float u2 = (float)(uint32_t)h * (1.0f / 4294967296.0f);
  return sqrtf(-2.0f * __logf(u1)) * __cosf(6.283185307f * u2);
}

// One thread per (row, group): draw the group's weights, pick asymmetric scale/zero, store codes in FM form.
__global__ void wq_random_kernel(uint8_t* __restrict__ wq, int n, int k, int bits, int group, float stddev,
                                 unsigned long long seed) {
  const int ng = k / group;
  const long total = (long)n * ng;
  const int nbat = k >> 7;
  const float qmax = (float)((1 << bits) - 1);
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / ng), gi = (int)(idx - (long)r * ng);
    const uint64_t base = (uint64_t)r * (uint64_t)k + (uint64_t)gi * group;
    float lo = 3.4e38f, hi = -3.4e38f;
    for (int i = 0; i < group; ++i) {
      const float w = stddev * normal_at(seed, base + i);
      lo = fminf(lo, w); hi = fmaxf(hi, w);
    }
    float s = (hi - lo) / qmax;
    if (!(s > 0.f)) s = 1.f;
    s = __half2float(__float2half_rn(s));
    const float z = __half2float(__float2half_rn(-lo / s));
    *reinterpret_cast<__half2*>(wq + fm_sz_off(r, gi, bits, group, nbat)) = __floats2half2_rn(s, z);
    for (int i = 0; i < group; ++i) {
      const float w = stddev * normal_at(seed, base + i);
      const float q = fminf(fmaxf(rintf(w / s + z), 0.f), qmax);
      fm_store_code(wq, fm_pos(r, gi * group + i, bits, group, nbat), bits, (unsigned)q);
    }
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

static inline int grid_for(long total, int threads) {
  long b = (total + threads - 1) / threads;
  return (int)(b > 148L * 16 ? 148L * 16 : (b < 1 ? 1 : b));
}

static inline size_t fm_bytes(int n, int k, int bits, int group) {
  const size_t wb = bits == 3 ? 768 : (bits == 4 ? 1024 : 512);
  return (size_t)(n / 32) * (k / 128) * (2 * wb + 2 * (128 / group) * 64);
}

static inline bool fm_ok(int n, int k, int bits, int group) {
  return n > 0 && k > 0 && n % 32 == 0 && k % 128 == 0 && (bits == 2 || bits == 3 || bits == 4) && (group == 64 || group == 128);
}

B2_API long b2_wq_bytes(int n, int k, int bits, int group) { return fm_ok(n, k, bits, group) ? (long)fm_bytes(n, k, bits, group) : -1; }

// FM -> bf16 [n][ldo].
B2_API int b2_wq_dequant(const uint8_t* wq, int n, int k, int bits, int group, bf16* out, long ldo, cudaStream_t stream) {
  if (!fm_ok(n, k, bits, group) || (ldo % 4)) return B2_ERR_ARG;
  wq_dequant_kernel<<<grid_for((long)n * (k / 4), 256), 256, 0, stream>>>(wq, n, k, bits, group, out, ldo);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

// Checkpoint bit stream (+ scale, optional zero point) -> FM.  Clears the destination first.
B2_API int b2_wq_repack(const int32_t* packed, const void* scale, int scale_is_bf16, const __half* zero, int n, int k,
                        int bits, int group, uint8_t* wq, cudaStream_t stream) {
  if (!fm_ok(n, k, bits, group)) return B2_ERR_ARG;
  if (cudaMemsetAsync(wq, 0, fm_bytes(n, k, bits, group), stream) != cudaSuccess) return B2_ERR_LAUNCH;
  wq_repack_kernel<<<grid_for((long)n * k, 256), 256, 0, stream>>>(packed, scale, scale_is_bf16, zero, n, k, bits, group, wq);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

// Random N(0, stddev) weights, asymmetric group quantisation, written directly in FM form.
B2_API int b2_wq_random(uint8_t* wq, int n, int k, int bits, int group, float stddev, unsigned long long seed,
                        cudaStream_t stream) {
  if (!fm_ok(n, k, bits, group)) return B2_ERR_ARG;
  if (cudaMemsetAsync(wq, 0, fm_bytes(n, k, bits, group), stream) != cudaSuccess) return B2_ERR_LAUNCH;
  wq_random_kernel<<<grid_for((long)n * (k / group), 128), 128, 0, stream>>>(wq, n, k, bits, group, stddev, seed);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

// FM -> FI (the integer-MMA layout of the decode-step kernel); `fi` has b2_wq_bytes(n, k, bits, group) bytes.
B2_API int b2_wq_fm_to_fi(const uint8_t* fm, int n, int k, int bits, int group, uint8_t* fi, cudaStream_t stream) {
  if (!fm_ok(n, k, bits, group) || !fm || !fi) return B2_ERR_ARG;
  if (cudaMemsetAsync(fi, 0, fm_bytes(n, k, bits, group), stream) != cudaSuccess) return B2_ERR_LAUNCH;
  wq_fm_to_fi_kernel<<<grid_for((long)n * k, 256), 256, 0, stream>>>(fm, n, k, bits, group, fi);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
