// Small fused ops around the GEMV/GEMM kernels: embedding gather (+ first RMSNorm statistic), standalone
// RMSNorm / add+RMSNorm for the prefill path, RoPE + paged KV store, SwiGLU, argmax reduction, and the
// device-side step bookkeeping that keeps a decode step free of host input.
// Reference counterparts: embed_kernel / argmax_*_kernel (kernels/src/torch_ops.cu:50-167),
// rmsnorm_cute_kernel (kernels/src/rmsnorm.cu:115), qk_prep_kernel (kernels/src/rope.cu:109-189),
// silu_mul_kernel (kernels/src/fastmath/silu_mul.cu:10), decode_step_prep (kernels/m1/m1_model.cu:357).
#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float s = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) s += sh[i];   // fixed order on every thread
  __syncthreads();
  return s;
}

// h[tok] = E[ids[tok]] (or the substituted image row) ; ss[tok] = sum(h^2)
__global__ void embed_kernel(const int* __restrict__ ids, const bf16* __restrict__ table, int d, int vocab,
                             const bf16* __restrict__ sub_rows, const int* __restrict__ sub_index, bf16* __restrict__ h,
                             long ldh, float* __restrict__ ss, int* __restrict__ status) {
  __shared__ float sh[32];
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  int id = ids[tok];
  const bf16* src;
  if (sub_index && sub_index[tok] >= 0) {
    src = sub_rows + (size_t)sub_index[tok] * d;
  } else {
    if (id < 0 || id >= vocab) { if (threadIdx.x == 0) atomicExch(status, (int)B2_ERR_BOUNDS); id = 0; }
    src = table + (size_t)id * d;
  }
  float sq = 0.f;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + i);
    *reinterpret_cast<uint4*>(h + (size_t)tok * ldh + i) = v;
    const bf16* b = reinterpret_cast<const bf16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float f = __bfloat162float(b[j]); sq += f * f; }
  }
  sq = block_sum_256(sq, sh);
  if (threadIdx.x == 0 && ss) ss[tok] = sq;
}

// y = bf16(x * rsqrt(mean(x^2)+eps) * w) ; optional residual: x = bf16(x + r) first, written to xo.
__global__ void rmsnorm_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ r, long ldr,
                               bf16* __restrict__ xo, long ldxo, const bf16* __restrict__ w, float eps, int d,
                               bf16* __restrict__ y, long ldy) {
  __shared__ float sh[32];
  extern __shared__ __align__(16) uint8_t dyn[];
  float* row = reinterpret_cast<float*>(dyn);
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  float sq = 0.f;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + i);
    const bf16* b = reinterpret_cast<const bf16*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(b[j]);
    if (r) {
      const uint4 rv = *reinterpret_cast<const uint4*>(r + (size_t)tok * ldr + i);
      const bf16* rb = reinterpret_cast<const bf16*>(&rv);
      __align__(16) bf16 o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = __float2bfloat16_rn(f[j] + __bfloat162float(rb[j])); f[j] = __bfloat162float(o[j]); }
      *reinterpret_cast<uint4*>(xo + (size_t)tok * ldxo + i) = *reinterpret_cast<const uint4*>(o);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { row[i + j] = f[j]; sq += f[j] * f[j]; }
  }
  sq = block_sum_256(sq, sh);
  const float ir = rsqrtf(sq / (float)d + eps);
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const bf16* wb = reinterpret_cast<const bf16*>(&wv);
    __align__(16) bf16 o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(row[i + j] * ir * __bfloat162float(wb[j]));
    *reinterpret_cast<uint4*>(y + (size_t)tok * ldy + i) = *reinterpret_cast<const uint4*>(o);
  }
}

// Partial sums of squares of rows of h, in the layout the GEMV PRO_NORM prologue consumes ([part][ss_ld]).
__global__ void sumsq_kernel(const bf16* __restrict__ h, long ldh, int d, float* __restrict__ ss) {
  __shared__ float sh[32];
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  float sq = 0.f;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(h + (size_t)tok * ldh + i);
    const bf16* b = reinterpret_cast<const bf16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float f = __bfloat162float(b[j]); sq += f * f; }
  }
  sq = block_sum_256(sq, sh);
  if (threadIdx.x == 0) ss[tok] = sq;
}

// RoPE (NeoX pairing i <-> i + hd/2) on q and k of a fused qkv row, and the paged KV store.
// One warp per (token, head).  qkv row: [q heads | k heads | v heads] x hd.
// KV pool of one layer: [page][2][kv_head][page_size][hd].
__global__ void rope_kvstore_kernel(bf16* __restrict__ qkv, long ld, int n_tok, int hq, int hkv, int hd,
                                    const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                    const int* __restrict__ rope_pos, const int* __restrict__ tok_seq, const int* __restrict__ block_table, int bt_ld,
                                    bf16* __restrict__ kv_pool, int page_size, int n_pages, bf16* __restrict__ q_out,
                                    long ldq, int* __restrict__ status, const int* __restrict__ rope_pos3,
                                    const unsigned char* __restrict__ pair_axis) {
  pdl_wait();
  pdl_launch_dependents();
  const int warps_per_block = blockDim.x >> 5;
  const int wid = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = hq + 2 * hkv;
  if (wid >= n_tok * heads) return;
  const int tok = wid / heads, head = wid - tok * heads;
  const int pos = tok_pos[tok];                         // KV slot of the token inside its sequence
  const int rpos = rope_pos ? rope_pos[tok] : pos;      // rotary position (differs from the slot for tree drafts)
  bf16* src = qkv + (size_t)tok * ld + (size_t)head * hd;
  const int half = hd >> 1;
  bf16* dst;
  if (head < hq) {
    dst = q_out + (size_t)tok * ldq + (size_t)head * hd;
  } else {
    const int seq = tok_seq[tok];
    const int page = block_table[(size_t)seq * bt_ld + pos / page_size];
    if (page < 0 || page >= n_pages) { if (lane == 0) atomicExch(status, (int)B2_ERR_BOUNDS); return; }
    const int is_v = head >= hq + hkv;
    const int kvh = head - hq - (is_v ? hkv : 0);
    dst = kv_pool + ((((size_t)page * 2 + is_v) * hkv + kvh) * page_size + (pos % page_size)) * hd;
    if (is_v) {
      for (int i = lane * 2; i < hd; i += 64) *reinterpret_cast<uint32_t*>(dst + i) = *reinterpret_cast<const uint32_t*>(src + i);
      return;
    }
  }
  for (int i = lane * 2; i < half; i += 64) {
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(src + i);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(src + i + half);
    float s0, c0, s1, c1;
    // multi-axis rotary (image tokens): the position of frequency pair i comes from axis pair_axis[i] of
    // rope_pos3 [3][n_tok] (time, height, width); text tokens carry the same value on all three axes
    const int p0 = rope_pos3 ? rope_pos3[(size_t)pair_axis[i] * n_tok + tok] : rpos;
    const int p1 = rope_pos3 ? rope_pos3[(size_t)pair_axis[i + 1] * n_tok + tok] : rpos;
    sincosf((float)p0 * inv_freq[i], &s0, &c0);
    sincosf((float)p1 * inv_freq[i + 1], &s1, &c1);
    const float x0 = __low2float(lo), x1 = __high2float(lo), y0 = __low2float(hi), y1 = __high2float(hi);
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(x0 * c0 - y0 * s0, x1 * c1 - y1 * s1);
    *reinterpret_cast<__nv_bfloat162*>(dst + i + half) = __floats2bfloat162_rn(y0 * c0 + x0 * s0, y1 * c1 + x1 * s1);
  }
}

// act = bf16(silu(gate) * up) for a [T][2F] buffer laid out in the interleaved 8 gate / 8 up row blocks that the
// merged gate_up weight produces (see utils/quant.py::interleave_gate_up).
__global__ void swiglu_interleaved_kernel(const bf16* __restrict__ gu, long ldg, int f, bf16* __restrict__ act, long lda) {
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.y;
  for (int j = (blockIdx.x * blockDim.x + threadIdx.x) * 8; j < f; j += gridDim.x * blockDim.x * 8) {
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)tok * ldg + 2 * j);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)tok * ldg + 2 * j + 8);
    const bf16* gb = reinterpret_cast<const bf16*>(&gv);
    const bf16* ub = reinterpret_cast<const bf16*>(&uv);
    __align__(16) bf16 o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g = __bfloat162float(gb[i]);
      o[i] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * __bfloat162float(ub[i]));
    }
    *reinterpret_cast<uint4*>(act + (size_t)tok * lda + j) = *reinterpret_cast<const uint4*>(o);
  }
}

// Final argmax over per-panel partials [parts][ld] (value, index): lowest index wins ties, as torch.argmax does.
__global__ void argmax_final_kernel(const float* __restrict__ val, const int* __restrict__ idx, int parts, int ld,
                                    int* __restrict__ out_ids, float* __restrict__ out_val) {
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int p0 = threadIdx.x; p0 < parts; p0 += blockDim.x * 8) {   // eight loads in flight per thread
    float pv[8];
    int pi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int p = p0 + j * blockDim.x;
      pv[j] = p < parts ? val[(size_t)p * ld + tok] : -INFINITY;
      pi[j] = p < parts ? idx[(size_t)p * ld + tok] : 0x7fffffff;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (pv[j] > best || (pv[j] == best && pi[j] < bi)) { best = pv[j]; bi = pi[j]; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    out_ids[tok] = bi;
    if (out_val) out_val[tok] = best;
  }
}

// Plain row argmax of fp32 logits [rows][ld] over the first n_valid columns.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, long ld, int n_valid, int* __restrict__ out_ids) {
  const int tok = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n_valid; i += blockDim.x) {
    const float v = logits[(size_t)tok * ld + i];
    if (v > best) { best = v; bi = i; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    out_ids[tok] = bi;
  }
}

// Decode step bookkeeping on the device: every running sequence advances by one position; the token produced by
// the previous step becomes this step's input.  Keeps a captured decode graph free of host-written inputs.
__global__ void decode_step_prep_kernel(int n_seq, const int* __restrict__ last_ids, int* __restrict__ ids,
                                        int* __restrict__ seq_len, int* __restrict__ tok_pos, int* __restrict__ tok_seq,
                                        const int* __restrict__ slot_seq) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seq) return;
  const int seq = slot_seq ? slot_seq[i] : i;
  ids[i] = last_ids[i];
  tok_pos[i] = seq_len[seq];
  tok_seq[i] = seq;
  seq_len[seq] += 1;
}

__global__ void fill_u32_kernel(uint32_t* p, uint32_t v, long n) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) p[i] = v;
}

}  // namespace
}  // namespace b2

using namespace b2;

static inline int launch_ok() { return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH; }

template <typename... KArgs, typename... Args>
static int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_embed(const int* ids, int n_tok, const bf16* table, int d, int vocab, const bf16* sub_rows,
                    const int* sub_index, bf16* h, long ldh, float* ss, int* status, cudaStream_t st) {
  if (d % 8 || n_tok <= 0) return B2_ERR_ARG;
  return launch_pdl(embed_kernel, dim3(n_tok), dim3(256), 0, st, ids, table, d, vocab, sub_rows, sub_index, h, ldh, ss, status);
}

B2_API int b2_rmsnorm(const bf16* x, long ldx, const bf16* r, long ldr, bf16* xo, long ldxo, const bf16* w, float eps,
                      int n_tok, int d, bf16* y, long ldy, cudaStream_t st) {
  if (d % 8 || n_tok <= 0 || d > 16384) return B2_ERR_ARG;
  if (r && !xo) return B2_ERR_ARG;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536); attr = true; }
  return launch_pdl(rmsnorm_kernel, dim3(n_tok), dim3(256), (size_t)d * 4, st, x, ldx, r, ldr, xo, ldxo, w, eps, d, y, ldy);
}

B2_API int b2_sumsq(const bf16* h, long ldh, int n_tok, int d, float* ss, cudaStream_t st) {
  if (d % 8 || n_tok <= 0) return B2_ERR_ARG;
  return launch_pdl(sumsq_kernel, dim3(n_tok), dim3(256), 0, st, h, ldh, d, ss);
}

B2_API int b2_rope_kvstore(bf16* qkv, long ld, int n_tok, int hq, int hkv, int hd, const float* inv_freq,
                           const int* tok_pos, const int* rope_pos, const int* tok_seq, const int* block_table, int bt_ld,
                           bf16* kv_pool,
                           int page_size, int n_pages, bf16* q_out, long ldq, int* status, cudaStream_t st) {
  if (hd % 4 || hd > 256 || n_tok <= 0) return B2_ERR_ARG;
  const int warps = n_tok * (hq + 2 * hkv);
  return launch_pdl(rope_kvstore_kernel, dim3((warps + 7) / 8), dim3(256), 0, st, qkv, ld, n_tok, hq, hkv, hd, inv_freq,
                    tok_pos, rope_pos, tok_seq, block_table, bt_ld, kv_pool, page_size, n_pages, q_out, ldq, status,
                    (const int*)nullptr, (const unsigned char*)nullptr);
}

// Same with multi-axis rotary positions: rope_pos3 [3][n_tok], pair_axis [hd / 2] (axis 0..2 of every frequency pair).
B2_API int b2_rope_kvstore_m(bf16* qkv, long ld, int n_tok, int hq, int hkv, int hd, const float* inv_freq, const int* tok_pos,
                             const int* rope_pos3, const unsigned char* pair_axis, const int* tok_seq, const int* block_table,
                             int bt_ld, bf16* kv_pool, int page_size, int n_pages, bf16* q_out, long ldq, int* status,
                             cudaStream_t st) {
  if (hd % 4 || hd > 256 || n_tok <= 0 || !rope_pos3 || !pair_axis) return B2_ERR_ARG;
  const int warps = n_tok * (hq + 2 * hkv);
  return launch_pdl(rope_kvstore_kernel, dim3((warps + 7) / 8), dim3(256), 0, st, qkv, ld, n_tok, hq, hkv, hd, inv_freq,
                    tok_pos, (const int*)nullptr, tok_seq, block_table, bt_ld, kv_pool, page_size, n_pages, q_out, ldq, status,
                    rope_pos3, pair_axis);
}

B2_API int b2_swiglu_interleaved(const bf16* gu, long ldg, int n_tok, int f, bf16* act, long lda, cudaStream_t st) {
  if (f % 8 || n_tok <= 0) return B2_ERR_ARG;
  int gx = (f / 8 + 255) / 256;
  return launch_pdl(swiglu_interleaved_kernel, dim3(gx, n_tok), dim3(256), 0, st, gu, ldg, f, act, lda);
}

B2_API int b2_argmax_final(const float* val, const int* idx, int parts, int ld, int n_tok, int* out_ids, float* out_val,
                           cudaStream_t st) {
  if (n_tok <= 0 || parts <= 0) return B2_ERR_ARG;
  return launch_pdl(argmax_final_kernel, dim3(n_tok), dim3(1024), 0, st, val, idx, parts, ld, out_ids, out_val);
}

B2_API int b2_argmax_rows(const float* logits, long ld, int n_tok, int n_valid, int* out_ids, cudaStream_t st) {
  if (n_tok <= 0 || n_valid <= 0) return B2_ERR_ARG;
  argmax_rows_kernel<<<n_tok, 1024, 0, st>>>(logits, ld, n_valid, out_ids);
  return launch_ok();
}

B2_API int b2_decode_step_prep(int n_seq, const int* last_ids, int* ids, int* seq_len, int* tok_pos, int* tok_seq,
                               const int* slot_seq, cudaStream_t st) {
  if (n_seq <= 0) return B2_ERR_ARG;
  decode_step_prep_kernel<<<(n_seq + 127) / 128, 128, 0, st>>>(n_seq, last_ids, ids, seq_len, tok_pos, tok_seq, slot_seq);
  return launch_ok();
}

B2_API int b2_fill_u32(uint32_t* p, uint32_t v, long n, cudaStream_t st) {
  if (n <= 0) return B2_ERR_ARG;
  fill_u32_kernel<<<(int)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256), 256, 0, st>>>(p, v, n);
  return launch_ok();
}
