// Remaining pieces of the hybrid checkpoint family: mHC residual-stream boundary (mix with Sinkhorn-normalised 4x4
// stream matrix, combine), Engram n-gram hash gather, INT8 GEMV (lm_head / shortlist), INT8 KV row quantisation and
// block means for the KV tier, and the BCSA far branch (block scoring, top-k block selection in torch's
// (score desc, index asc) order, pooled K/V gather from the paged pool, far attention with (o, lse) merge).
//
// Replaces mhc_mix_kernel / mhc_combine_kernel (kernels/src/mhc.cu:61-109), engram_kernel (engram.cu:22),
// i8_gemv_kernel (i8_gemv.cu:33), quant_store_k / dequant_rows_k / block_mean_k (kv_tier.cu:32-86) and score_kernel,
// topk2_kernel, pool_kernel, fused_attend_kernel, combine_kernel (far_decode.cu:89-539).
#include <algorithm>

#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + __expf(-v)); }

// ---------------------------------------------------------------------------------------------------------------- mHC
// coef[t] = [pre(4) | post(4) | res(16 row-major)].  pre = sigmoid, post = 2 sigmoid, res = Sinkhorn(exp(.), iters).
__global__ void mhc_mix_kernel(const bf16* __restrict__ H, const float* __restrict__ dyn, const float* __restrict__ statics,
                               float* __restrict__ coef, bf16* __restrict__ x, int d, int iters) {
  __shared__ float c[24];
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    float r[16];
    for (int i = 0; i < 4; ++i) c[i] = sigmoidf(dyn[t * 24 + i] + statics[i]);
    for (int i = 4; i < 8; ++i) c[i] = 2.f * sigmoidf(dyn[t * 24 + i] + statics[i]);
    for (int i = 0; i < 16; ++i) r[i] = __expf(dyn[t * 24 + 8 + i] + statics[8 + i]);
    for (int it = 0; it < iters; ++it) {
      for (int a = 0; a < 4; ++a) { const float s = r[a * 4] + r[a * 4 + 1] + r[a * 4 + 2] + r[a * 4 + 3]; for (int b = 0; b < 4; ++b) r[a * 4 + b] /= s; }
      for (int b = 0; b < 4; ++b) { const float s = r[b] + r[4 + b] + r[8 + b] + r[12 + b]; for (int a = 0; a < 4; ++a) r[a * 4 + b] /= s; }
    }
    for (int i = 0; i < 16; ++i) c[8 + i] = r[i];
    for (int i = 0; i < 24; ++i) coef[t * 24 + i] = c[i];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int a = 0; a < 4; ++a) s += c[a] * __bfloat162float(H[((size_t)t * 4 + a) * d + i]);
    x[(size_t)t * d + i] = __float2bfloat16_rn(s);
  }
}

// H'[a] = sum_b res[a][b] H[b] + post[a] * y
__global__ void mhc_combine_kernel(const bf16* __restrict__ H, const bf16* __restrict__ y, const float* __restrict__ coef,
                                   bf16* __restrict__ Hout, int d) {
  const int t = blockIdx.x;
  const float* c = coef + t * 24;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float h[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) h[a] = __bfloat162float(H[((size_t)t * 4 + a) * d + i]);
    const float yy = __bfloat162float(y[(size_t)t * d + i]);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float s = c[4 + a] * yy;
#pragma unroll
      for (int b = 0; b < 4; ++b) s += c[8 + a * 4 + b] * h[b];
      Hout[((size_t)t * 4 + a) * d + i] = __float2bfloat16_rn(s);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------- Engram
// hist[t][j] = token id j steps back (j = 0 is the current token; -1 = before the start).  For every order n in
// 2 .. 1 + n_orders the n most recent ids are hashed (multiply-add chain over a 61-bit field) into a row of that
// order's table [rows][dim]; the table may live in mapped pinned host memory.
__global__ void engram_kernel(const int* __restrict__ hist, int hist_ld, const bf16* __restrict__ tables, long rows, int dim,
                              int n_orders, bf16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int o = 0; o < n_orders; ++o) {
    const int n = o + 2;
    unsigned long long h = 0x9E3779B97F4A7C15ull & ((1ull << 61) - 1);
    bool ok = true;
    for (int j = n - 1; j >= 0; --j) {
      const int id = hist[t * hist_ld + j];
      ok &= id >= 0;
      h = (h * 1000003ull + (unsigned long long)(id + 1) * 0x100000001B3ull) & ((1ull << 61) - 1);
    }
    const long row = (long)(h % (unsigned long long)rows);
    const bf16* src = tables + ((size_t)o * rows + row) * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
      out[((size_t)t * n_orders + o) * dim + i] = ok ? src[i] : __float2bfloat16_rn(0.f);
  }
}

// ------------------------------------------------------------------------------------------------------------ INT8
// y[m][n] = scale[n] * sum_k W[n][k] x[m][k]; one warp per output row, 16 weights per lane per step.
__global__ void i8_gemv_kernel(const int8_t* __restrict__ W, const float* __restrict__ scale, const bf16* __restrict__ x, long ldx,
                               float* __restrict__ y, long ldy, int n, int k, int m) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  for (int tok = 0; tok < m; ++tok) {
    float acc = 0.f;
    for (int c = lane * 16; c < k; c += 512) {
      const int4 wv = __ldg(reinterpret_cast<const int4*>(W + (size_t)row * k + c));
      const int8_t* w8 = reinterpret_cast<const int8_t*>(&wv);
      const uint4 x0 = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + c);
      const uint4 x1 = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + c + 8);
      const bf16* xa = reinterpret_cast<const bf16*>(&x0);
      const bf16* xb = reinterpret_cast<const bf16*>(&x1);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf((float)w8[i], __bfloat162float(xa[i]), acc);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf((float)w8[8 + i], __bfloat162float(xb[i]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)tok * ldy + row] = acc * scale[row];
  }
}

// per-row symmetric INT8: scale = amax / 127; one warp per row
__global__ void kv_quant_int8_kernel(const bf16* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scale, int rows, int d) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float amax = 0.f;
  for (int i = lane; i < d; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(x[(size_t)row * d + i])));
  amax = warp_max(amax);
  const float s = amax > 0.f ? amax / 127.f : 1.f;
  for (int i = lane; i < d; i += 32)
    q[(size_t)row * d + i] = (int8_t)max(-127, min(127, __float2int_rn(__bfloat162float(x[(size_t)row * d + i]) / s)));
  if (lane == 0) scale[row] = s;
}
__global__ void kv_dequant_int8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, bf16* __restrict__ x, long n, int d) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16_rn((float)q[i] * scale[i / d]);
}
// mean of `blk` consecutive rows, accumulated in fp32 in row order
__global__ void block_mean_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, long n_blocks, int blk, int d) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_blocks * d; i += (long)gridDim.x * blockDim.x) {
    const long b = i / d; const int c = (int)(i % d);
    float s = 0.f;
    for (int r = 0; r < blk; ++r) s += __bfloat162float(x[((size_t)b * blk + r) * d + c]);
    out[i] = __float2bfloat16_rn(s / (float)blk);
  }
}

// ---------------------------------------------------------------------------------------------------------------- BCSA
// score[b] = scale * sum_h w[h] * relu(qi[h] . kb[b]);  one warp per block
__global__ void bcsa_score_kernel(const bf16* __restrict__ qi, const float* __restrict__ w, const bf16* __restrict__ kb, float scale,
                                  float* __restrict__ score, int nb, int idxh, int di) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= nb) return;
  float total = 0.f;
  for (int h = 0; h < idxh; ++h) {
    float s = 0.f;
    for (int i = lane; i < di; i += 32) s += __bfloat162float(qi[h * di + i]) * __bfloat162float(kb[(size_t)b * di + i]);
    s = warp_sum(s);
    total += w[h] * fmaxf(s, 0.f);
  }
  if (lane == 0) score[b] = total * scale;
}

__device__ __forceinline__ uint32_t fkey(float x) { const uint32_t b = __float_as_uint(x); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }

// Top-k selection in (score desc, index asc) order by radix descent; one CTA.  Writes the k selected indices sorted
// by index ascending (the order the gather wants) and their count (min(k, n)).
__global__ void __launch_bounds__(1024) topk_blocks_kernel(const float* __restrict__ score, int n, int k, int* __restrict__ sel,
                                                           int* __restrict__ n_sel) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_above, s_cnt;
  if (k >= n) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) sel[i] = i;
    if (threadIdx.x == 0) *n_sel = n;
    return;
  }
  unsigned prefix = 0, mask = 0, above = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = fkey(score[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned run = above; int d = 255;
      for (; d > 0; --d) { if (run + hist[d] >= (unsigned)k) break; run += hist[d]; }
      s_above = run; s_prefix = prefix | ((unsigned)d << shift);
    }
    __syncthreads();
    above = s_above; prefix = s_prefix; mask |= 255u << shift;
    __syncthreads();
  }
  // keys > prefix are all selected; of the keys == prefix the lowest indices fill the rest
  const unsigned need_eq = (unsigned)k - above;
  if (threadIdx.x == 0) s_cnt = 0;
  __syncthreads();
  // selection flags are evaluated in index order chunk by chunk so that ties resolve by ascending index
  __shared__ unsigned s_eq_seen, s_out;
  if (threadIdx.x == 0) { s_eq_seen = 0; s_out = 0; }
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const uint32_t key = i < n ? fkey(score[i]) : 0u;
    const bool gt = i < n && key > prefix, eq = i < n && key == prefix;
    // ranks inside the chunk by warp ballots + per-warp prefix in shared memory
    __shared__ unsigned w_eq[32], w_sel[32];
    const unsigned lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const unsigned eq_b = __ballot_sync(0xffffffffu, eq);
    const unsigned eq_before_w = __popc(eq_b & ((1u << lane) - 1));
    if (lane == 0) w_eq[wid] = __popc(eq_b);
    __syncthreads();
    unsigned eq_before = s_eq_seen + eq_before_w;
    for (unsigned ww = 0; ww < wid; ++ww) eq_before += w_eq[ww];
    const bool take = gt || (eq && eq_before < need_eq);
    const unsigned tk_b = __ballot_sync(0xffffffffu, take);
    if (lane == 0) w_sel[wid] = __popc(tk_b);
    __syncthreads();
    unsigned pos = s_out + __popc(tk_b & ((1u << lane) - 1));
    for (unsigned ww = 0; ww < wid; ++ww) pos += w_sel[ww];
    if (take) sel[pos] = i;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned e = 0, t2 = 0;
      for (unsigned ww = 0; ww < (blockDim.x >> 5); ++ww) { e += w_eq[ww]; t2 += w_sel[ww]; }
      s_eq_seen += e; s_out += t2;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_sel = (int)s_out;
}

// Gathers the K and V rows of the selected blocks (blk tokens each) of one sequence from the paged pool into
// contiguous [n_sel * blk][hkv][hd] buffers.  One CTA per selected block.
__global__ void bcsa_gather_kernel(const bf16* __restrict__ kv_pool, const int* __restrict__ bt, const int* __restrict__ sel,
                                   const int* __restrict__ n_sel, int blk, int hkv, int hd, int page, bf16* __restrict__ kout,
                                   bf16* __restrict__ vout) {
  const int s = blockIdx.x;
  if (s >= *n_sel) return;
  const int b = sel[s];
  for (int r = 0; r < blk; ++r) {
    const int pos = b * blk + r;
    const int pg = bt[pos / page], in = pos % page;
    for (int i = threadIdx.x; i < hkv * hd; i += blockDim.x) {
      const int h = i / hd, c = i % hd;
      const size_t src = ((((size_t)pg * 2 + 0) * hkv + h) * page + in) * hd + c;
      const size_t srcv = ((((size_t)pg * 2 + 1) * hkv + h) * page + in) * hd + c;
      kout[((size_t)(s * blk + r) * hkv + h) * hd + c] = kv_pool[src];
      vout[((size_t)(s * blk + r) * hkv + h) * hd + c] = kv_pool[srcv];
    }
  }
}

// Far attention of one query token over the gathered rows, merged with the local branch: one warp per q head.
// local: o_loc [hq][hd] (normalised), lse_loc [hq] (natural log).  out = softmax-merge(local, far).
__global__ void bcsa_far_attend_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kf, const bf16* __restrict__ vf,
                                       const int* __restrict__ n_sel, int blk, int hq, int hkv, int hd, float scale,
                                       const float* __restrict__ o_loc, const float* __restrict__ lse_loc, bf16* __restrict__ out) {
  const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (head >= hq) return;
  const int kvh = head / (hq / hkv);
  const int nrow = *n_sel * blk;
  const int per = hd / 32;
  float qv[8], acc[8];
  for (int i = 0; i < per; ++i) { qv[i] = __bfloat162float(q[(size_t)head * hd + lane * per + i]); acc[i] = 0.f; }
  float mx = -INFINITY, l = 0.f;
  for (int r = 0; r < nrow; ++r) {
    float s = 0.f;
    for (int i = 0; i < per; ++i) s += qv[i] * __bfloat162float(kf[((size_t)r * hkv + kvh) * hd + lane * per + i]);
    s = warp_sum(s) * scale;
    const float mn = fmaxf(mx, s);
    const float corr = __expf(mx - mn), p = __expf(s - mn);
    l = l * corr + p;
    for (int i = 0; i < per; ++i) acc[i] = acc[i] * corr + p * __bfloat162float(vf[((size_t)r * hkv + kvh) * hd + lane * per + i]);
    mx = mn;
  }
  // merge with the local branch through log-sum-exp weights
  const float lse_f = nrow > 0 ? mx + __logf(l) : -INFINITY;
  const float lse_l = lse_loc ? lse_loc[head] : -INFINITY;
  const float m2 = fmaxf(lse_f, lse_l);
  const float wf = nrow > 0 ? __expf(lse_f - m2) : 0.f, wl = lse_loc ? __expf(lse_l - m2) : 0.f;
  const float inv = 1.f / (wf + wl);
  for (int i = 0; i < per; ++i) {
    const float of = nrow > 0 ? acc[i] / l : 0.f;
    const float ol = o_loc ? o_loc[(size_t)head * hd + lane * per + i] : 0.f;
    out[(size_t)head * hd + lane * per + i] = __float2bfloat16_rn((wf * of + wl * ol) * inv);
  }
}

}  // namespace
}  // namespace b2

using namespace b2;
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH)

B2_API int b2_mhc_mix(const bf16* H, const float* dyn, const float* statics, float* coef, bf16* x, int T, int d, int iters, cudaStream_t st) {
  if (T < 1 || d < 1) return B2_ERR_ARG;
  mhc_mix_kernel<<<T, 256, 0, st>>>(H, dyn, statics, coef, x, d, iters);
  return LAUNCH_OK();
}
B2_API int b2_mhc_combine(const bf16* H, const bf16* y, const float* coef, bf16* Hout, int T, int d, cudaStream_t st) {
  if (T < 1 || d < 1) return B2_ERR_ARG;
  mhc_combine_kernel<<<T, 256, 0, st>>>(H, y, coef, Hout, d);
  return LAUNCH_OK();
}
B2_API int b2_engram(const int* hist, int hist_ld, const bf16* tables, long rows, int dim, int n_orders, bf16* out, int T, cudaStream_t st) {
  if (T < 1 || rows < 1 || n_orders < 1 || hist_ld < n_orders + 1) return B2_ERR_ARG;
  engram_kernel<<<T, 128, 0, st>>>(hist, hist_ld, tables, rows, dim, n_orders, out);
  return LAUNCH_OK();
}
B2_API int b2_i8_gemv(const int8_t* W, const float* scale, const bf16* x, long ldx, float* y, long ldy, int n, int k, int m, cudaStream_t st) {
  if (n < 1 || k % 512 || m < 1) return B2_ERR_ARG;
  i8_gemv_kernel<<<(n + 7) / 8, 256, 0, st>>>(W, scale, x, ldx, y, ldy, n, k, m);
  return LAUNCH_OK();
}
B2_API int b2_kv_quant_int8(const bf16* x, int8_t* q, float* scale, int rows, int d, cudaStream_t st) {
  kv_quant_int8_kernel<<<(rows + 7) / 8, 256, 0, st>>>(x, q, scale, rows, d);
  return LAUNCH_OK();
}
B2_API int b2_kv_dequant_int8(const int8_t* q, const float* scale, bf16* x, long rows, int d, cudaStream_t st) {
  kv_dequant_int8_kernel<<<(int)std::min<long>((rows * d + 255) / 256, 4096), 256, 0, st>>>(q, scale, x, rows * d, d);
  return LAUNCH_OK();
}
B2_API int b2_block_mean(const bf16* x, bf16* out, long n_blocks, int blk, int d, cudaStream_t st) {
  block_mean_kernel<<<(int)std::min<long>((n_blocks * d + 255) / 256, 4096), 256, 0, st>>>(x, out, n_blocks, blk, d);
  return LAUNCH_OK();
}
B2_API int b2_bcsa_score(const bf16* qi, const float* w, const bf16* kb, float scale, float* score, int nb, int idxh, int di, cudaStream_t st) {
  if (nb < 1) return B2_ERR_ARG;
  bcsa_score_kernel<<<(nb + 7) / 8, 256, 0, st>>>(qi, w, kb, scale, score, nb, idxh, di);
  return LAUNCH_OK();
}
B2_API int b2_topk_blocks(const float* score, int n, int k, int* sel, int* n_sel, cudaStream_t st) {
  if (n < 1 || k < 1) return B2_ERR_ARG;
  topk_blocks_kernel<<<1, 1024, 0, st>>>(score, n, k, sel, n_sel);
  return LAUNCH_OK();
}
B2_API int b2_bcsa_gather(const bf16* kv_pool, const int* bt, const int* sel, const int* n_sel, int max_sel, int blk, int hkv, int hd,
                          int page, bf16* kout, bf16* vout, cudaStream_t st) {
  if (max_sel < 1) return B2_ERR_ARG;
  bcsa_gather_kernel<<<max_sel, 128, 0, st>>>(kv_pool, bt, sel, n_sel, blk, hkv, hd, page, kout, vout);
  return LAUNCH_OK();
}
B2_API int b2_bcsa_far_attend(const bf16* q, const bf16* kf, const bf16* vf, const int* n_sel, int blk, int hq, int hkv, int hd,
                              float scale, const float* o_loc, const float* lse_loc, bf16* out, cudaStream_t st) {
  if (hd % 32 || hd > 256 || hq % hkv) return B2_ERR_ARG;
  bcsa_far_attend_kernel<<<(hq + 3) / 4, 128, 0, st>>>(q, kf, vf, n_sel, blk, hq, hkv, hd, scale, o_loc, lse_loc, out);
  return LAUNCH_OK();
}
