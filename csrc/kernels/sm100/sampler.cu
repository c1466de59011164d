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
__device__ float block_reduce_max(float v, float* sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = -INFINITY;
  for (int i = 0; i < kThreads / 32; ++i) s = fmaxf(s, sh[i]);
  __syncthreads();
  return s;
}

// Radix descent: finds the largest key prefix such that the mass of all elements with a strictly larger key is
// <= target (mass = probability or count).  On return *above = mass strictly above the final key, *at = mass of
// elements equal to the final key.  `keep_min`: elements with key < keep_min are ignored.
template <bool COUNT>
__device__ uint32_t radix_descend(const float* x, int n, float mx, float inv_t, uint32_t keep_min, float target, float* hist,
                                  float* above_out, float* at_out) {
  uint32_t prefix = 0, mask = 0;
  float above = 0.f, at = 0.f;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const uint32_t k = key_of(x[i]);
      if (k >= keep_min && (k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], COUNT ? 1.f : __expf((x[i] - mx) * inv_t));
    }
    __syncthreads();
    // walk digits from high to low until the running mass passes the target (every thread does the same walk)
    int d = 255;
    float run = above;
    for (; d > 0; --d) { if (run + hist[d] > target) break; run += hist[d]; }
    above = run;
    at = hist[d];
    prefix |= (uint32_t)d << shift;
    mask |= 255u << shift;
    __syncthreads();
  }
  *above_out = above;
  *at_out = at;
  return prefix;
}

}  // namespace

// Note on determinism: shared-memory float atomics are order dependent in the last bits; thresholds that decide token
// identity are therefore taken on counts (exact) or compared with a margin-free walk whose only ambiguity is between
// equal keys, which the index rule resolves.  The probability-mass histograms feed only the top-p cut and the final
// walk; both compare against masses accumulated in the same pass, so a different summation order can move the draw
// only when u falls within one ulp-scale sliver of a bin boundary.
__global__ void __launch_bounds__(kThreads) sample_rows_kernel(const SampleArgs a) {
  __shared__ float sh[kThreads / 32];
  __shared__ float hist[256];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const float* x = a.logits + (size_t)row * a.ld;
  const int n = a.vocab;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < n; i += kThreads) mx = fmaxf(mx, x[i]);
  mx = block_reduce_max(mx, sh);
  const float T = a.temperature ? a.temperature[row] : 0.f;
  const int topk = a.top_k ? a.top_k[row] : 0;
  if (T <= 0.f || topk == 1) {
    // greedy: lowest index among the maxima
    int best = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += kThreads) if (x[i] == mx) best = min(best, i);
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
    float above, at;
    const uint32_t kth = radix_descend<true>(x, n, mx, inv_t, 0u, (float)topk - 0.5f, hist, &above, &at);
    keep_min = max(keep_min, kth);
  }
  // top-p over what is left: smallest descending prefix whose mass reaches top_p * Z
  const float topp = a.top_p ? a.top_p[row] : 1.f;
  if (topp < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < n; i += kThreads) if (key_of(x[i]) >= keep_min) z += __expf((x[i] - mx) * inv_t);
    z = block_reduce_sum(z, sh);
    float above, at;
    const uint32_t cut = radix_descend<false>(x, n, mx, inv_t, keep_min, topp * z, hist, &above, &at);
    keep_min = max(keep_min, cut);
  }
  // draw
  float z = 0.f;
  for (int i = threadIdx.x; i < n; i += kThreads) if (key_of(x[i]) >= keep_min) z += __expf((x[i] - mx) * inv_t);
  z = block_reduce_sum(z, sh);
  const uint32_t r = philox_first(a.seed ? a.seed[row] : 0ull, (unsigned long long)(a.position ? a.position[row] : 0));
  const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);
  const float target = fminf(u * z, z * (1.f - 1e-7f));
  float above, at;
  const uint32_t key = radix_descend<false>(x, n, mx, inv_t, keep_min, target, hist, &above, &at);
  // among the tokens that share the final key, walk by ascending index: the `want`-th of them wins
  const float w = __expf((__uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key) - mx) * inv_t);
  const int rank = w > 0.f ? (int)fminf(floorf(fmaxf(target - above, 0.f) / w), 1e9f) : 0;
  float cnt = 0.f;
  for (int i = threadIdx.x; i < n; i += kThreads) cnt += key_of(x[i]) == key ? 1.f : 0.f;
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
    for (int i = threadIdx.x; i < n; i += kThreads) if (key_of(x[i]) == key) a.out[row] = i;
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
