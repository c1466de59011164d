// bf16 GEMV for linears kept in bf16 (checkpoints with LinearFormat bf16, the bf16 drafter): y[m, n] = x[m, k] * W[n, k]^T
// for up to eight token rows, fp32 accumulation, optional bf16 residual, bf16 or fp32 result.
// Reference counterpart: the batch-invariant bf16 GEMV family (kernels/src/bf16_gemv.cu:21, kernels/src/bi_gemv.cu:48-246).
//
// One warp owns one output row (up to four with more token rows) for all token rows: lane l reads the 16-byte pieces l, l + 32, ... of the weight row
// (and the same pieces of every token's activation row, which stay in L1 / L2), keeps one fp32 sum per token, and the
// warp adds the lanes' sums in a fixed xor tree.  The order of every addition depends on k only, never on the number
// of token rows or on a row's position in the batch: a token gets the same bits alone or among others.
// Memory bound by the weight stream (2 bytes per weight); four 16-byte loads are in flight per lane.
#include "common.cuh"

namespace b2 {
namespace {

constexpr int kBfWarps = 8;

// R weight rows per warp share every activation load (more token rows need more reuse: the activations come from L1 at
// M times the weight rate otherwise); U vectors per lane and round keep R * U = 4 weight loads in flight.  For one
// (row, token) pair the additions happen in the same order whatever M and R are.
template <int M, int R>
__global__ void __launch_bounds__(kBfWarps * 32) bf16_gemv_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w,
                                                                  long ldw, int n, int k, bf16* __restrict__ y, float* __restrict__ yf,
                                                                  long ldy, const bf16* __restrict__ resid, long ldr) {
  constexpr int U = 4 / R;
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * kBfWarps + warp) * R;
  if (row0 >= n) return;
  const uint4* wr[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wr[r] = reinterpret_cast<const uint4*>(w + (size_t)min(row0 + r, n - 1) * ldw);   // tail rows repeat the last row
  const int nvec = k >> 3;
  float acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < M; ++t) acc[r][t] = 0.f;
  auto fma8 = [&](const uint4 (&wv)[R], int v) {
    float wf[R][8];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bf16* wb = reinterpret_cast<const bf16*>(&wv[r]);
#pragma unroll
      for (int i = 0; i < 8; ++i) wf[r][i] = __bfloat162float(wb[i]);
    }
#pragma unroll
    for (int t = 0; t < M; ++t) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (size_t)t * ldx) + v);
      const bf16* xb = reinterpret_cast<const bf16*>(&xv);
      float xf[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) xf[i] = __bfloat162float(xb[i]);
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][t] = fmaf(wf[r][i], xf[i], acc[r][t]);
    }
  };
  int v = lane;
  for (; v + 32 * (U - 1) < nvec; v += 32 * U) {      // R * U independent weight loads per lane and round
    uint4 wv[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < R; ++r) wv[u][r] = ld_nc_v4(wr[r] + v + 32 * u);
#pragma unroll
    for (int u = 0; u < U; ++u) fma8(wv[u], v + 32 * u);
  }
  for (; v < nvec; v += 32) {
    uint4 wv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wv[r] = ld_nc_v4(wr[r] + v);
    fma8(wv, v);
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int t = 0; t < M; ++t) {
      float s = acc[r][t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const int row = row0 + r;
      if (lane == 0 && row < n) {
        if (resid) s += __bfloat162float(resid[(size_t)t * ldr + row]);
        if (y) y[(size_t)t * ldy + row] = __float2bfloat16(s);
        if (yf) yf[(size_t)t * ldy + row] = s;
      }
    }
}

template <typename... KArgs, typename... Args>
int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

}  // namespace

// x: bf16 [m, k] (row pitch ldx), W: bf16 [n, k] (row pitch ldw), 1 <= m <= 8, k a multiple of 8, rows 16-byte aligned.
// Exactly one of y (bf16) / yf (fp32) is written (both may be given); resid (bf16 [m, n]) is added before rounding.
B2_API int b2_bf16_gemv(const bf16* x, long ldx, const bf16* w, long ldw, int m, int n, int k, bf16* y, float* yf, long ldy,
                        const bf16* resid, long ldr, cudaStream_t st) {
  if (m < 1 || m > 8 || n <= 0 || k <= 0 || (k % 8) || (ldx % 8) || (ldw % 8) || (!y && !yf)) return B2_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return B2_ERR_ARG;
  const dim3 block(kBfWarps * 32);
  auto grid = [&](int rows_per_warp) { return dim3((n + kBfWarps * rows_per_warp - 1) / (kBfWarps * rows_per_warp)); };
  switch (m) {
    case 1: return launch_pdl(bf16_gemv_kernel<1, 1>, grid(1), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 2: return launch_pdl(bf16_gemv_kernel<2, 1>, grid(1), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 3: return launch_pdl(bf16_gemv_kernel<3, 2>, grid(2), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 4: return launch_pdl(bf16_gemv_kernel<4, 2>, grid(2), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 5: return launch_pdl(bf16_gemv_kernel<5, 4>, grid(4), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 6: return launch_pdl(bf16_gemv_kernel<6, 4>, grid(4), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    case 7: return launch_pdl(bf16_gemv_kernel<7, 4>, grid(4), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
    default: return launch_pdl(bf16_gemv_kernel<8, 4>, grid(4), block, st, x, ldx, w, ldw, n, k, y, yf, ldy, resid, ldr);
  }
}

}  // namespace b2
