// Device-side sampling and speculative acceptance.
//
// One rule decides every sampled token (reference: kernels/m1/m1_model.cu:796-818): the token at absolute position n
// of a sequence with seed s is InvCDF_q(u(s, n)), where q is the filtered distribution (temperature, top-k, top-p,
// min-p) of that position's logits and u is the first uniform of Philox4x32-10 keyed by s at counter n.  Because the
// draw depends only on (seed, position, logits), a verify block samples every row exactly as a plain decode step would,
// so "a draft is accepted iff it equals the target's own sample" gives the plain sampling distribution and, with a
// seed, the same tokens with or without speculation and at any batch size.
//
// Implementation: one CTA per row.  Keys are the order-preserving integer images of the logits; top-k, top-p and the
// final inverse-CDF walk are radix descents over 8-bit digits (4 passes each) with 256-bin shared histograms of counts
// or probability mass; ties are broken by ascending token index.  All reductions run in a fixed order.
// Replaces samp_pos / samp_hist / samp_fast and accept_greedy / accept_sampled / bv_accept (m1_model.cu:476-579,
// 1099-1452, 1536).
#include "common.cuh"

namespace b2 {

struct SampleArgs {
  const float* logits; long ld; int vocab;      // [rows][ld], first `vocab` columns are valid
  const float* temperature;                      // per row; <= 0 means greedy
  const int* top_k;                              // per row; <= 0 means off
  const float* top_p;                            // per row; >= 1 means off
  const float* min_p;                            // per row; <= 0 means off
  const unsigned long long* seed;                // per row
  const int* position;                           // per row: absolute position of the token being sampled
  int* out;                                      // [rows]
};

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t key_of(float x) {      // larger float -> larger key
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Philox4x32-10, returns the first 32-bit output for (key = seed, counter = ctr).
__device__ uint32_t philox_first(unsigned long long seed, unsigned long long ctr) {
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ float block_reduce_sum(float v, float* sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < kThreads / 32; ++i) s += sh[i];
  __syncthreads();
  return s;
}
// Probability masses are fixed point (exp of a non-positive number times 2^31, so one mass fits 32 bits): integer sums
// do not depend on the order of the additions, so every threshold of the sampler is exactly reproducible.  A histogram
// bin is a (low, high) pair of 32-bit words: 32-bit shared-memory integer atomics are single instructions, where float
// and 64-bit ones are compare-and-swap loops; the carry into the high word is a second, rare, atomic.
__device__ __forceinline__ unsigned long long mass_of(float xv, float mx, float inv_t) {
  return (unsigned long long)(__expf((xv - mx) * inv_t) * 2147483648.f);
}
struct Hist { uint32_t lo[256], hi[256]; };
__device__ __forceinline__ void hist_add(Hist& h, uint32_t dig, unsigned long long v) {
  const uint32_t lo = (uint32_t)v;
  uint32_t hi = (uint32_t)(v >> 32);
  if (lo) { const uint32_t old = atomicAdd(&h.lo[dig], lo); hi += (old + lo < old) ? 1u : 0u; }
  if (hi) atomicAdd(&h.hi[dig], hi);
}
__device__ __forceinline__ unsigned long long hist_get(const Hist& h, int d) { return ((unsigned long long)h.hi[d] << 32) | h.lo[d]; }
__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ unsigned long long block_reduce_sum_u64(unsigned long long v, unsigned long long* sh) {
  v = warp_sum_u64(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long s = 0;
  for (int i = 0; i < kThreads / 32; ++i) s += sh[i];
  __syncthreads();
  return s;
}
__device__ float block_reduce_max(float v, float* sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = -INFINITY;
  for (int i = 0; i < kThreads / 32; ++i) s = fmaxf(s, sh[i]);
  __syncthreads();
  return s;
}

// One pass over a row: f(value, index, valid) for every element, the same number of calls on every thread (so f may
// use warp-wide primitives), with eight elements per thread in flight (two 16-byte loads) where the row allows it:
// with one element per iteration a pass is bound by the latency of its loads, not by bandwidth.
template <typename F>
__device__ __forceinline__ void scan_row(const float* x, int n, F f) {
  const int n4 = (reinterpret_cast<uintptr_t>(x) & 15) == 0 ? n >> 2 : 0;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int base = 0; base < n4; base += 2 * kThreads) {
    const int i0 = base + (int)threadIdx.x, i1 = i0 + kThreads;
    const bool v0 = i0 < n4, v1 = i1 < n4;
    const float4 a = v0 ? x4[i0] : zero;
    const float4 b = v1 ? x4[i1] : zero;
    f(a.x, 4 * i0, v0); f(a.y, 4 * i0 + 1, v0); f(a.z, 4 * i0 + 2, v0); f(a.w, 4 * i0 + 3, v0);
    f(b.x, 4 * i1, v1); f(b.y, 4 * i1 + 1, v1); f(b.z, 4 * i1 + 2, v1); f(b.w, 4 * i1 + 3, v1);
  }
  for (int base = 4 * n4; base < n; base += kThreads) {
    const int i = base + (int)threadIdx.x;
    f(i < n ? x[i] : 0.f, i, i < n);
  }
}

// Radix descent: finds the largest key prefix such that the mass of all elements with a strictly larger key is
// <= target (mass = probability or count).  On return *above = mass strictly above the final key, *at = mass of
// elements equal to the final key.  `keep_min`: elements with key < keep_min are ignored.
template <bool COUNT>
__device__ uint32_t radix_descend(const float* x, int n, float mx, float inv_t, uint32_t keep_min, unsigned long long target,
                                  Hist& hist, unsigned long long* above_out, unsigned long long* at_out) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long above = 0, at = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) { hist.lo[i] = 0; hist.hi[i] = 0; }
    __syncthreads();
    // Logits crowd into a few digits at the upper levels, where one shared-memory atomic per element would serialise
    // the warp: lanes that share a digit with at least seven others are summed in registers first and their leader
    // adds once; the rest add for themselves.
    const int lane = threadIdx.x & 31;
    scan_row(x, n, [&](float xv, int, bool valid) {
      const uint32_t k = key_of(xv);
      const bool on = valid && k >= keep_min && (k & mask) == prefix;
      const uint32_t dig = on ? (k >> shift) & 255u : 0xFFFFFFFFu;
      const unsigned long long v = !on ? 0ull : (COUNT ? 1ull : mass_of(xv, mx, inv_t));
      const unsigned peers = __match_any_sync(0xffffffffu, dig);
      const bool big = on && __popc(peers) >= 8;
      unsigned pending = __ballot_sync(0xffffffffu, big);
      while (pending) {
        const int leader = __ffs(pending) - 1;
        const unsigned grp = __shfl_sync(0xffffffffu, peers, leader);
        const unsigned long long sum = COUNT ? (unsigned long long)__popc(grp) : warp_sum_u64(((grp >> lane) & 1u) ? v : 0ull);
        if (lane == leader) hist_add(hist, dig, sum);
        pending &= ~grp;
      }
      if (on && !big) hist_add(hist, dig, v);
    });
    __syncthreads();
    // walk digits from high to low until the running mass passes the target (every thread does the same walk)
    int d = 255;
    unsigned long long run = above;
    for (; d > 0; --d) { const unsigned long long hd = hist_get(hist, d); if (run + hd > target) break; run += hd; }
    above = run;
    at = hist_get(hist, d);
    prefix |= (uint32_t)d << shift;
    mask |= 255u << shift;
    __syncthreads();
  }
  *above_out = above;
  *at_out = at;
  return prefix;
}

}  // namespace

// Determinism: counts and fixed-point masses are integers, so every histogram, threshold and the final walk are
// independent of the order in which threads add; equal keys are ordered by token index.
__global__ void __launch_bounds__(kThreads) sample_rows_kernel(const SampleArgs a) {
  __shared__ float sh[kThreads / 32];
  __shared__ unsigned long long sh64[kThreads / 32];
  __shared__ Hist hist;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const float* x = a.logits + (size_t)row * a.ld;
  const int n = a.vocab;
  float mx = -INFINITY;
  scan_row(x, n, [&](float xv, int, bool valid) { if (valid) mx = fmaxf(mx, xv); });
  mx = block_reduce_max(mx, sh);
  const float T = a.temperature ? a.temperature[row] : 0.f;
  const int topk = a.top_k ? a.top_k[row] : 0;
  if (T <= 0.f || topk == 1) {
    // greedy: lowest index among the maxima
    int best = 0x7fffffff;
    scan_row(x, n, [&](float xv, int i, bool valid) { if (valid && xv == mx) best = min(best, i); });
    __shared__ int sbest[kThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) sbest[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) { int b = sbest[0]; for (int i = 1; i < kThreads / 32; ++i) b = min(b, sbest[i]); a.out[row] = b; }
    return;
  }
  const float inv_t = 1.f / T;
  uint32_t keep_min = 0;          // smallest key that survives the filters
  // min-p: p >= min_p * p_max  <=>  x >= mx + T * ln(min_p)
  const float minp = a.min_p ? a.min_p[row] : 0.f;
  if (minp > 0.f) keep_min = max(keep_min, key_of(mx + T * __logf(minp)));
  // top-k: key of the k-th largest logit (ties at the threshold are all kept; the index rule orders them)
  if (topk > 1 && topk < n) {
    unsigned long long above, at;
    const uint32_t kth = radix_descend<true>(x, n, mx, inv_t, 0u, (unsigned long long)(topk - 1), hist, &above, &at);
    keep_min = max(keep_min, kth);
  }
  // top-p over what is left: smallest descending prefix whose mass reaches top_p * Z
  const float topp = a.top_p ? a.top_p[row] : 1.f;
  if (topp < 1.f) {
    unsigned long long z = 0;
    scan_row(x, n, [&](float xv, int, bool valid) { if (valid && key_of(xv) >= keep_min) z += mass_of(xv, mx, inv_t); });
    z = block_reduce_sum_u64(z, sh64);
    unsigned long long above, at;
    const uint32_t cut = radix_descend<false>(x, n, mx, inv_t, keep_min, (unsigned long long)((double)topp * (double)z), hist, &above, &at);
    keep_min = max(keep_min, cut);
  }
  // draw
  unsigned long long z = 0;
  scan_row(x, n, [&](float xv, int, bool valid) { if (valid && key_of(xv) >= keep_min) z += mass_of(xv, mx, inv_t); });
  z = block_reduce_sum_u64(z, sh64);                         // at least 2^31: the maximum always survives the filters
  const uint32_t r = philox_first(a.seed ? a.seed[row] : 0ull, (unsigned long long)(a.position ? a.position[row] : 0));
  const double u = ((double)(r >> 8) + 0.5) * (1.0 / 16777216.0);
  unsigned long long target = (unsigned long long)(u * (double)z);
  if (z > 0 && target >= z) target = z - 1;
  unsigned long long above, at;
  const uint32_t key = radix_descend<false>(x, n, mx, inv_t, keep_min, target, hist, &above, &at);
  // among the tokens that share the final key, walk by ascending index: the `want`-th of them wins
  const unsigned long long w = mass_of(__uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key), mx, inv_t);
  const unsigned long long rank64 = w > 0 && target > above ? (target - above) / w : 0ull;
  const int rank = (int)(rank64 > 1000000000ull ? 1000000000ull : rank64);
  float cnt = 0.f;
  scan_row(x, n, [&](float xv, int, bool valid) { cnt += valid && key_of(xv) == key ? 1.f : 0.f; });
  cnt = block_reduce_sum(cnt, sh);                          // exact: integers below 2^24
  const int want = min(rank, max((int)cnt - 1, 0));
  if ((int)cnt == 0) {                                       // rounding pushed the walk past the last bin: take the mode
    __shared__ int s_fb;
    if (threadIdx.x == 0) s_fb = 0x7fffffff;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kThreads) if (x[i] == mx) atomicMin(&s_fb, i);
    __syncthreads();
    if (threadIdx.x == 0) a.out[row] = s_fb;
    return;
  }
  if ((int)cnt == 1) {                                       // the usual case: one token owns the key
    scan_row(x, n, [&](float xv, int i, bool valid) { if (valid && key_of(xv) == key) a.out[row] = i; });
    return;
  }
  // smallest index I with (number of equal-key tokens at index <= I) == want + 1, by bisection over the index range
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    float c = 0.f;
    for (int i = threadIdx.x; i <= mid; i += kThreads) c += key_of(x[i]) == key ? 1.f : 0.f;
    c = block_reduce_sum(c, sh);
    if ((int)c >= want + 1) hi = mid; else lo = mid + 1;
  }
  if (threadIdx.x == 0) a.out[row] = lo;
}

// Longest-prefix acceptance for one or more verify blocks.  Block b covers rows [row0[b], row0[b] + cnt[b]): row 0 is
// the bonus token, rows 1.. are drafts.  target[r] is the model's own token (argmax or sample) after row r.
// Draft j + 1 is accepted iff it equals target[j].  Emits the accepted drafts followed by the target's next token.
__global__ void spec_accept_kernel(const int* __restrict__ ids, const int* __restrict__ target, const int* __restrict__ row0,
                                   const int* __restrict__ cnt, int n_blocks, int* __restrict__ n_emitted,
                                   int* __restrict__ emitted, int emitted_ld) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const int r0 = row0[b], c = cnt[b];
  int acc = 0;
  while (acc + 1 < c && ids[r0 + acc + 1] == target[r0 + acc]) ++acc;
  for (int j = 0; j < acc; ++j) emitted[(size_t)b * emitted_ld + j] = ids[r0 + j + 1];
  emitted[(size_t)b * emitted_ld + acc] = target[r0 + acc];
  n_emitted[b] = acc + 1;
}

}  // namespace b2

using namespace b2;

B2_API int b2_sample_rows(const SampleArgs* a, int rows, cudaStream_t st) {
  if (!a || rows <= 0 || a->vocab <= 0 || !a->logits || !a->out) return B2_ERR_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows); cfg.blockDim = dim3(kThreads); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, sample_rows_kernel, *a) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_spec_accept(const int* ids, const int* target, const int* row0, const int* cnt, int n_blocks, int* n_emitted,
                          int* emitted, int emitted_ld, cudaStream_t st) {
  if (n_blocks <= 0 || emitted_ld < 1) return B2_ERR_ARG;
  spec_accept_kernel<<<(n_blocks + 63) / 64, 64, 0, st>>>(ids, target, row0, cnt, n_blocks, n_emitted, emitted, emitted_ld);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
