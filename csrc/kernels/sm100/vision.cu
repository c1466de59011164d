// Vision-encoder kernels: LayerNorm with bias, bias + GELU (+ residual) epilogue pass, 2-D rotary embedding on q/k and
// non-causal full attention over one image's patches.  The linears of the tower run on the tcgen05 GEMM
// (gemm_tc.cu); these kernels are the memory-bound glue and the attention.
//
// Replaces the ATen calls of the reference's vision bridge (kernels/oracle/bridge/vision.cpp:105-199: layer_norm,
// linear + gelu, rope_, scaled_dot_product_attention).
#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865476f)); }

// one warp per row
__global__ void layernorm_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w, const bf16* __restrict__ b, float eps,
                                 bf16* __restrict__ out, long ldo, int rows, int d) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s = 0.f;
  for (int i = lane; i < d; i += 32) s += __bfloat162float(x[(size_t)row * ldx + i]);
  const float mean = warp_sum(s) / (float)d;
  float v = 0.f;
  for (int i = lane; i < d; i += 32) { const float c = __bfloat162float(x[(size_t)row * ldx + i]) - mean; v += c * c; }
  const float inv = rsqrtf(warp_sum(v) / (float)d + eps);
  for (int i = lane; i < d; i += 32) {
    const float y = (__bfloat162float(x[(size_t)row * ldx + i]) - mean) * inv * __bfloat162float(w[i]) + (b ? __bfloat162float(b[i]) : 0.f);
    out[(size_t)row * ldo + i] = __float2bfloat16_rn(y);
  }
}

// y = act(x + bias) (+ resid); act: 0 none, 1 GELU(tanh), 2 GELU(erf)
__global__ void bias_act_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ bias, int act, const bf16* __restrict__ resid,
                                long ldr, bf16* __restrict__ out, long ldo, int rows, int d) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < (long)rows * d; i += (long)gridDim.x * blockDim.x) {
    const long r = i / d; const int c = (int)(i % d);
    float v = __bfloat162float(x[r * ldx + c]) + (bias ? __bfloat162float(bias[c]) : 0.f);
    if (act == 1) v = gelu_tanh(v); else if (act == 2) v = gelu_erf(v);
    if (resid) v += __bfloat162float(resid[r * ldr + c]);
    out[r * ldo + c] = __float2bfloat16_rn(v);
  }
}

// In-place rotary on the q and k thirds of qkv [N][3*H*hd]: x <- x cos + rotate_half(x) sin, fp32 math, cos/sin [N][hd].
__global__ void rope2d_kernel(bf16* __restrict__ qkv, long ld, const float* __restrict__ cs, const float* __restrict__ sn, int N, int H,
                              int hd) {
  const int half = hd / 2;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < (long)N * 2 * H * half; i += (long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    long r = i / half;
    const int h = (int)(r % H); r /= H;
    const int which = (int)(r % 2);
    const long n = r / 2;
    bf16* p = qkv + n * ld + (size_t)which * H * hd + (size_t)h * hd;
    const float a = __bfloat162float(p[j]), b = __bfloat162float(p[j + half]);
    const float c0 = cs[n * hd + j], s0 = sn[n * hd + j], c1 = cs[n * hd + j + half], s1 = sn[n * hd + j + half];
    p[j] = __float2bfloat16_rn(a * c0 - b * s0);
    p[j + half] = __float2bfloat16_rn(b * c1 + a * s1);
  }
}

// Non-causal attention over one sequence.  CTA = 8 warps = 8 query rows of one head; keys and values are staged in
// shared memory 32 rows at a time; each lane scores one key of the tile, then owns PER output dimensions.
template <int PER>
__global__ void __launch_bounds__(256) attn_full_kernel(const bf16* __restrict__ qkv, long ld, bf16* __restrict__ out, long ldo, int N,
                                                        int H, int hd, float scale) {
  constexpr int HDP = PER * 32;
  __shared__ float ks[32][HDP + 1], vs[32][HDP + 1];
  __shared__ float qs[8][HDP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int qrow = blockIdx.x * 8 + warp;
  const bool qok = qrow < N;
  for (int i = lane; i < HDP; i += 32)
    qs[warp][i] = (qok && i < hd) ? __bfloat162float(qkv[(size_t)qrow * ld + (size_t)head * hd + i]) * scale : 0.f;
  float acc[PER], mx = -INFINITY, l = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < N; k0 += 32) {
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * HDP; i += 256) {
      const int r = i / HDP, c = i % HDP;
      const bool ok = k0 + r < N && c < hd;
      ks[r][c] = ok ? __bfloat162float(qkv[(size_t)(k0 + r) * ld + (size_t)(H + head) * hd + c]) : 0.f;
      vs[r][c] = ok ? __bfloat162float(qkv[(size_t)(k0 + r) * ld + (size_t)(2 * H + head) * hd + c]) : 0.f;
    }
    __syncthreads();
    float s = 0.f;
    for (int c = 0; c < hd; ++c) s = fmaf(qs[warp][c], ks[lane][c], s);
    if (k0 + lane >= N) s = -INFINITY;
    const float mn = fmaxf(mx, warp_max(s));
    const float corr = __expf(mx - mn), p = __expf(s - mn);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] *= corr;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] = fmaf(pj, vs[j][lane + 32 * i], acc[i]);
    }
    mx = mn;
  }
  if (!qok) return;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = lane + 32 * i;
    if (c < hd) out[(size_t)qrow * ldo + (size_t)head * hd + c] = __float2bfloat16_rn(acc[i] * inv);
  }
}

}  // namespace
}  // namespace b2

using namespace b2;

B2_API int b2_layernorm(const bf16* x, long ldx, const bf16* w, const bf16* b, float eps, bf16* out, long ldo, int rows, int d, cudaStream_t st) {
  if (rows < 1 || d < 1) return B2_ERR_ARG;
  layernorm_kernel<<<(rows + 7) / 8, 256, 0, st>>>(x, ldx, w, b, eps, out, ldo, rows, d);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
B2_API int b2_bias_act(const bf16* x, long ldx, const bf16* bias, int act, const bf16* resid, long ldr, bf16* out, long ldo, int rows, int d,
                       cudaStream_t st) {
  if (rows < 1 || d < 1) return B2_ERR_ARG;
  const long n = (long)rows * d;
  bias_act_kernel<<<(int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256), 256, 0, st>>>(x, ldx, bias, act, resid, ldr, out, ldo, rows, d);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
B2_API int b2_rope2d(bf16* qkv, long ld, const float* cs, const float* sn, int N, int H, int hd, cudaStream_t st) {
  if (N < 1 || hd % 2) return B2_ERR_ARG;
  const long n = (long)N * H * hd;
  rope2d_kernel<<<(int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256), 256, 0, st>>>(qkv, ld, cs, sn, N, H, hd);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
B2_API int b2_attn_full(const bf16* qkv, long ld, bf16* out, long ldo, int N, int H, int hd, float scale, cudaStream_t st) {
  if (N < 1 || H < 1 || hd < 1 || hd > 128) return B2_ERR_ARG;
  const dim3 grid((N + 7) / 8, H);
  if (hd <= 64) attn_full_kernel<2><<<grid, 256, 0, st>>>(qkv, ld, out, ldo, N, H, hd, scale);
  else if (hd <= 96) attn_full_kernel<3><<<grid, 256, 0, st>>>(qkv, ld, out, ldo, N, H, hd, scale);
  else attn_full_kernel<4><<<grid, 256, 0, st>>>(qkv, ld, out, ldo, N, H, hd, scale);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
