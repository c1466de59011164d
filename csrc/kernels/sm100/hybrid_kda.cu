// KDA linear-attention layer pieces for the hybrid checkpoint family: causal depthwise conv update, gated delta-rule
// recurrence with an fp32 state per head, gated RMSNorm.  One set of kernels serves decode (T = 1), verify (T <= 8,
// state left untouched), commit (replay of the accepted prefix, count read from the device) and prefill (any T,
// sequential over tokens inside the kernel).
//
// Replaces conv_update_kernel, kda_decode_kernel, gated_rmsnorm_kernel, conv_multi_kernel, kda_multi*_kernel,
// kda_commit_all_kernel and kda_verify_fused_kernel (kernels/src/kda_decode.cu:92-561) and stands in for the chunked
// prefill cubins (kernels/src/kda_prefill.cu:258-416) with a token-sequential recurrence.
//
// Recurrence per head, state S [K][V] fp32, token inputs q, k in R^K (l2-normalised here, q scaled by K^-1/2),
// v in R^V, log-decay g in R^K (<= 0), beta in (0, 1):
//     S <- diag(exp(g)) S;   d = beta (v - k^T S);   S <- S + k d^T;   o = q^T S.
#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

// One thread per channel.  state: [dim][KW-1] fp32 (oldest first).  Tokens are processed in order; the state is
// written back after `n_commit` tokens (n_commit < 0: never; a device pointer overrides the host value).
template <int KW>
__global__ void conv_update_kernel(const bf16* __restrict__ x, long ldx, float* __restrict__ state, const bf16* __restrict__ w,
                                   const bf16* __restrict__ bias, bf16* __restrict__ out, long ldo, int T, int dim, int n_commit,
                                   const int* __restrict__ n_commit_dev, int apply_silu) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  if (n_commit_dev) n_commit = *n_commit_dev;
  float h[KW - 1], wk[KW];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) h[j] = state[(size_t)c * (KW - 1) + j];
#pragma unroll
  for (int j = 0; j < KW; ++j) wk[j] = __bfloat162float(w[(size_t)c * KW + j]);
  const float b = bias ? __bfloat162float(bias[c]) : 0.f;
  if (!out && n_commit <= 0) return;
  for (int t = 0; t < T; ++t) {
    const float xv = __bfloat162float(x[(size_t)t * ldx + c]);
    float y = b + wk[KW - 1] * xv;
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) y += wk[j] * h[j];
    if (out) out[(size_t)t * ldo + c] = __float2bfloat16_rn(apply_silu ? silu(y) : y);
#pragma unroll
    for (int j = 0; j < KW - 2; ++j) h[j] = h[j + 1];
    h[KW - 2] = xv;
    if (t + 1 == n_commit) {
#pragma unroll
      for (int j = 0; j < KW - 1; ++j) state[(size_t)c * (KW - 1) + j] = h[j];
    }
  }
}

// Grid (V / 32, heads); one warp per CTA; lane = one V column, whose K state entries live in registers.
template <int K>
__global__ void __launch_bounds__(32) kda_recurrent_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k,
                                                           const bf16* __restrict__ v, long ld_qk, long ld_v,
                                                           const float* __restrict__ g, const float* __restrict__ beta,
                                                           float* __restrict__ state, bf16* __restrict__ out, long ldo, int T,
                                                           int H, int V, int n_commit, const int* __restrict__ n_commit_dev,
                                                           int l2norm) {
  __shared__ float sq[K], sk[K], sg[K];
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.y, col = blockIdx.x * 32 + threadIdx.x, lane = threadIdx.x;
  if (n_commit_dev) n_commit = *n_commit_dev;
  float S[K];
  float* sp = state + ((size_t)head * K) * V + col;
#pragma unroll
  for (int j = 0; j < K; ++j) S[j] = sp[(size_t)j * V];
  const float qscale = rsqrtf((float)K);
  const int n_tok = out ? T : min(T, max(n_commit, 0));      // a commit pass stops at the accepted prefix
  for (int t = 0; t < n_tok; ++t) {
    float qq = 0.f, kk = 0.f;
    for (int j = lane; j < K; j += 32) {
      const float a = __bfloat162float(q[(size_t)t * ld_qk + (size_t)head * K + j]);
      const float b = __bfloat162float(k[(size_t)t * ld_qk + (size_t)head * K + j]);
      sq[j] = a; sk[j] = b;
      sg[j] = __expf(g[((size_t)t * H + head) * K + j]);
      qq += a * a; kk += b * b;
    }
    qq = warp_sum(qq); kk = warp_sum(kk);
    __syncwarp();
    const float qn = l2norm ? rsqrtf(qq + 1e-6f) * qscale : qscale;
    const float kn = l2norm ? rsqrtf(kk + 1e-6f) : 1.f;
    const float bt = beta[(size_t)t * H + head];
    const float vv = __bfloat162float(v[(size_t)t * ld_v + (size_t)head * V + col]);
    float pred = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { S[j] *= sg[j]; pred = fmaf(sk[j] * kn, S[j], pred); }
    const float d = bt * (vv - pred);
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) { S[j] = fmaf(sk[j] * kn, d, S[j]); o = fmaf(sq[j] * qn, S[j], o); }
    if (out) out[(size_t)t * ldo + (size_t)head * V + col] = __float2bfloat16_rn(o);
    __syncwarp();
    if (t + 1 == n_commit) {
#pragma unroll
      for (int j = 0; j < K; ++j) sp[(size_t)j * V] = S[j];
    }
  }
}

// out = rmsnorm(o) * w * sigmoid(gate); one warp per row of d elements.
__global__ void gated_rmsnorm_kernel(const bf16* __restrict__ o, long ld_o, const bf16* __restrict__ gate, long ld_g,
                                     const bf16* __restrict__ w, float eps, bf16* __restrict__ out, long ld_out, int rows, int d) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) { const float x = __bfloat162float(o[(size_t)row * ld_o + i]); ss += x * x; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)d + eps);
  for (int i = lane; i < d; i += 32) {
    const float x = __bfloat162float(o[(size_t)row * ld_o + i]) * inv * __bfloat162float(w[i]);
    const float gt = __bfloat162float(gate[(size_t)row * ld_g + i]);
    out[(size_t)row * ld_out + i] = __float2bfloat16_rn(x / (1.f + __expf(-gt)));
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

B2_API int b2_conv_update(const bf16* x, long ldx, float* state, const bf16* w, const bf16* bias, bf16* out, long ldo, int T, int dim,
                          int kw, int n_commit, const int* n_commit_dev, int apply_silu, cudaStream_t st) {
  if (kw != 4 || T < 1 || dim < 1) return B2_ERR_ARG;
  conv_update_kernel<4><<<(dim + 255) / 256, 256, 0, st>>>(x, ldx, state, w, bias, out, ldo, T, dim, n_commit, n_commit_dev, apply_silu);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_kda_recurrent(const bf16* q, const bf16* k, const bf16* v, long ld_qk, long ld_v, const float* g, const float* beta,
                            float* state, bf16* out, long ldo, int T, int H, int K, int V, int n_commit, const int* n_commit_dev,
                            int l2norm, cudaStream_t st) {
  if (K != 128 || V % 32 || T < 1 || H < 1) return B2_ERR_ARG;
  kda_recurrent_kernel<128><<<dim3(V / 32, H), 32, 0, st>>>(q, k, v, ld_qk, ld_v, g, beta, state, out, ldo, T, H, V, n_commit,
                                                            n_commit_dev, l2norm);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_gated_rmsnorm(const bf16* o, long ld_o, const bf16* gate, long ld_g, const bf16* w, float eps, bf16* out, long ld_out,
                            int rows, int d, cudaStream_t st) {
  if (rows < 1 || d < 1) return B2_ERR_ARG;
  gated_rmsnorm_kernel<<<(rows + 7) / 8, 256, 0, st>>>(o, ld_o, gate, ld_g, w, eps, out, ld_out, rows, d);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
