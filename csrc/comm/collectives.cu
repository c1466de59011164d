// Bounded push collectives over symmetric peer memory (NVLink P2P stores and local loads): all-reduce, all-gather,
// reduce-scatter, barrier and the vocab-parallel argmax combine.
//
// Reference counterparts: ar_kernel / push_ar_kernel / tp_push.cuh (kernels/src/tp_ar.cu:73-149, tp_push.cuh:97-148)
// and argmax_final_enc_kernel + argmax_combine_kernel (kernels/src/torch_ops.cu:141-165).  Differences by design:
// every wait is bounded and reports through a status word instead of spinning forever; sums are taken in rank order
// in fp32, so all ranks produce identical bits; there is no per-call host work (slots are chosen by the caller per
// call site), so the kernels can be captured in CUDA graphs.  The same inbox protocol is used by the fused
// GEMV -> all-reduce epilogue (wq_gemv.cu, EPI_TP_RESID).
#include "collectives.cuh"

namespace b2 {
namespace {

constexpr uint32_t kSentinel = 0x80000000u;   // -0.0f

__device__ __forceinline__ void st_peer_v4(float* p, float4 v) {
  asm volatile("st.volatile.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 ld_vol_v4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 sanitize(float4 v) {   // -0.0 -> +0.0 so that data never looks like the sentinel
  v.x += 0.f; v.y += 0.f; v.z += 0.f; v.w += 0.f;
  return v;
}
__device__ __forceinline__ bool arrived(const float4& v) {
  return (__float_as_uint(v.x) != kSentinel) & (__float_as_uint(v.y) != kSentinel) & (__float_as_uint(v.z) != kSentinel) &
         (__float_as_uint(v.w) != kSentinel);
}
// Poll one 16-byte unit until it holds no sentinel or the deadline passes.  Returns false on timeout (v zeroed).
__device__ __forceinline__ bool wait_unit(const float* p, float4& v, uint64_t t_start, unsigned long long timeout_ns) {
  unsigned spins = 0;
  while (true) {
    v = ld_vol_v4(p);
    if (arrived(v)) return true;
    if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > timeout_ns) break;
  }
  v = make_float4(0.f, 0.f, 0.f, 0.f);
  return false;
}
__device__ __forceinline__ void clear_unit(float* p) {
  const float n0 = __uint_as_float(kSentinel);
  *reinterpret_cast<float4*>(p) = make_float4(n0, n0, n0, n0);
}

// Re-arm the slot that no rank writes before its next use, over the extent the earlier call used (grid-stride).
__device__ __forceinline__ void rearm(const CommArgs& a) {
  if (a.clear_off < 0) return;
  const long nvec = a.clear_n >> 2;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float* clr = a.inbox[a.rank] + a.clear_off + (i << 2);
    for (int src = 0; src < a.size; ++src) clear_unit(clr + (long)src * a.slot_stride);
  }
}

// mode 0: all-reduce (n elements, every rank ends with the rank-ordered sum)
// mode 1: all-gather (n elements per rank, out[src * n + e])
// mode 2: reduce-scatter (input size * n elements; rank r ends with the sum of chunk r)
template <int MODE>
__global__ void push_collective_kernel(const CommArgs a, const float* __restrict__ in_f32, const bf16* __restrict__ in_bf16,
                                       long n, float* __restrict__ out_f32, bf16* __restrict__ out_bf16) {
  pdl_wait();
  pdl_launch_dependents();
  const long nvec = n >> 2;
  const uint64_t t_start = globaltimer_ns();
  bool timed_out = false;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long e = i << 2;
    // ---- push ----
    if (!a.skip_push) {
      for (int dst = 0; dst < a.size; ++dst) {
        const long src_e = MODE == 2 ? (long)dst * n + e : e;
        float4 v;
        if (in_f32) {
          v = *reinterpret_cast<const float4*>(in_f32 + src_e);
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(in_bf16 + src_e);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
          v = make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1]));
        }
        st_peer_v4(a.inbox[dst] + a.slot_off + (long)a.rank * a.slot_stride + e, sanitize(v));
      }
    }
    // ---- wait + combine ----
    const float* mine = a.inbox[a.rank] + a.slot_off + e;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int src = 0; src < a.size; ++src) {
      float4 v;
      if (!wait_unit(mine + (long)src * a.slot_stride, v, t_start, a.timeout_ns)) timed_out = true;
      if (MODE == 1) {
        *reinterpret_cast<float4*>(out_f32 + (long)src * n + e) = v;
      } else {
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    if (MODE != 1) {
      if (out_f32) *reinterpret_cast<float4*>(out_f32 + e) = s;
      if (out_bf16) {
        __nv_bfloat162 o[2] = {__floats2bfloat162_rn(s.x, s.y), __floats2bfloat162_rn(s.z, s.w)};
        *reinterpret_cast<uint2*>(out_bf16 + e) = *reinterpret_cast<const uint2*>(o);
      }
    }
  }
  rearm(a);
  if (timed_out) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
}

// Second half of a row-parallel linear whose GEMM epilogue already stored its fp32 partial tiles into the owners' inboxes
// (b2_gemm_bf16_push, slot A): sum my rows over the source ranks in rank order, write them as bf16 and push the sums to
// every peer (slot B); then take the peers' rows from slot B as they arrive.  One launch replaces reduce-scatter
// combine + all-gather + conversion.  Every unit is re-armed by the thread that read it, so the call needs no clearing
// pass; the caller rotates over three pairs of slots, so a slot is written again two calls after it was read.
// Rank r owns rows [r * rows_per, (r + 1) * rows_per) of the [total_rows, n_cols] result.
__global__ void collect_gather_kernel(const CommArgs a, long slot_b_off, int rows_per, int n_cols, int total_rows,
                                      bf16* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const uint64_t t_start = globaltimer_ns();
  bool timed_out = false;
  const long n_shard = (long)rows_per * n_cols;
  auto valid_units = [&](int r) -> long {
    long rows = (long)total_rows - (long)r * rows_per;
    rows = rows < 0 ? 0 : (rows > rows_per ? rows_per : rows);
    return rows * n_cols >> 2;
  };
  auto store_bf16 = [&](long flat, const float4& s) {
    __nv_bfloat162 o[2] = {__floats2bfloat162_rn(s.x, s.y), __floats2bfloat162_rn(s.z, s.w)};
    *reinterpret_cast<uint2*>(out + flat) = *reinterpret_cast<const uint2*>(o);
  };
  const long stride_t = (long)gridDim.x * blockDim.x, first = (long)blockIdx.x * blockDim.x + threadIdx.x;
  // ---- my rows: combine the partials of slot A, hand the sums on ----
  // All sources' units are requested before the first one is looked at, so a thread has `size` loads in flight; only a
  // unit that has not arrived yet is polled.
  float* mine_a = a.inbox[a.rank] + a.slot_off;
  for (long i = first, nv = valid_units(a.rank); i < nv; i += stride_t) {
    const long e = i << 2;
    float4 v[kCommMaxRanks];
#pragma unroll
    for (int src = 0; src < kCommMaxRanks; ++src)
      if (src < a.size) v[src] = ld_vol_v4(mine_a + (long)src * a.slot_stride + e);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int src = 0; src < kCommMaxRanks; ++src)
      if (src < a.size) {
        float* p = mine_a + (long)src * a.slot_stride + e;
        if (!arrived(v[src]) && !wait_unit(p, v[src], t_start, a.timeout_ns)) timed_out = true;
        clear_unit(p);
        s.x += v[src].x; s.y += v[src].y; s.z += v[src].z; s.w += v[src].w;
      }
    store_bf16((long)a.rank * n_shard + e, s);
    const float4 sv = sanitize(s);
    for (int dst = 0; dst < a.size; ++dst)
      if (dst != a.rank) st_peer_v4(a.inbox[dst] + slot_b_off + (long)a.rank * a.slot_stride + e, sv);
  }
  // ---- the peers' rows from slot B: four units of a peer in flight per thread ----
  float* mine_b = a.inbox[a.rank] + slot_b_off;
  for (int k = 1; k < a.size; ++k) {
    const int src = (a.rank + k) % a.size;
    float* base = mine_b + (long)src * a.slot_stride;
    const long nv = valid_units(src);
    for (long i = first; i < nv; i += 4 * stride_t) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * stride_t < nv) v[u] = ld_vol_v4(base + ((i + u * stride_t) << 2));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long iu = i + u * stride_t;
        if (iu < nv) {
          float* p = base + (iu << 2);
          if (!arrived(v[u]) && !wait_unit(p, v[u], t_start, a.timeout_ns)) timed_out = true;
          clear_unit(p);
          store_bf16((long)src * n_shard + (iu << 2), v[u]);
        }
      }
    }
  }
  if (timed_out) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
}

// Vocab-parallel argmax: every rank contributes (best value, best index) per token; all ranks pick the same winner
// (largest value, lowest index on ties).  One thread per token.
__global__ void argmax_combine_kernel(const CommArgs a, const float* __restrict__ val, const int* __restrict__ idx, int n_tok,
                                      int* __restrict__ out_idx, float* __restrict__ out_val) {
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x * blockDim.x + threadIdx.x;
  rearm(a);
  if (tok >= n_tok) return;
  const uint64_t t_start = globaltimer_ns();
  const long e = (long)tok * 4;
  if (!a.skip_push) {
    const float4 v = make_float4(val[tok] + 0.f, __int_as_float(idx[tok]), 0.f, 0.f);
    for (int dst = 0; dst < a.size; ++dst) st_peer_v4(a.inbox[dst] + a.slot_off + (long)a.rank * a.slot_stride + e, v);
  }
  const float* mine = a.inbox[a.rank] + a.slot_off + e;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  bool timed_out = false;
  for (int src = 0; src < a.size; ++src) {
    float4 v;
    if (!wait_unit(mine + (long)src * a.slot_stride, v, t_start, a.timeout_ns)) { timed_out = true; continue; }
    const int i = __float_as_int(v.y);
    if (v.x > best || (v.x == best && i < bi)) { best = v.x; bi = i; }
  }
  out_idx[tok] = bi;
  if (out_val) out_val[tok] = best;
  if (timed_out) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
}

template <typename... KArgs, typename... Args>
int launch_pdl_c(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

bool args_ok(const CommArgs* a, long n) {
  return a && a->size >= 1 && a->size <= kCommMaxRanks && a->rank >= 0 && a->rank < a->size && n > 0 && (n % 4) == 0 &&
         n <= a->slot_stride && (a->slot_off % 4) == 0 && (a->slot_stride % 4) == 0 && a->status &&
         (a->clear_off < 0 || (a->clear_n >= 0 && a->clear_n <= a->slot_stride && (a->clear_n % 4) == 0));
}
int grid_of(long nvec) {
  long b = (nvec + 255) / 256;
  return (int)(b > 296 ? 296 : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace b2

using namespace b2;

// out = sum over ranks of in (fp32 or bf16 input; fp32 and/or bf16 output); n % 4 == 0, n <= slot_stride.
B2_API int b2_comm_all_reduce(const CommArgs* a, const float* in_f32, const bf16* in_bf16, long n, float* out_f32,
                              bf16* out_bf16, cudaStream_t st) {
  if (!args_ok(a, n) || (!in_f32 == !in_bf16) || (!out_f32 && !out_bf16)) return B2_ERR_ARG;
  return launch_pdl_c(push_collective_kernel<0>, dim3(grid_of(n >> 2)), dim3(256), st, *a, in_f32, in_bf16, n, out_f32, out_bf16);
}

// out[src * n + e] = in of rank src.
B2_API int b2_comm_all_gather(const CommArgs* a, const float* in, long n, float* out, cudaStream_t st) {
  if (!args_ok(a, n) || !in || !out) return B2_ERR_ARG;
  return launch_pdl_c(push_collective_kernel<1>, dim3(grid_of(n >> 2)), dim3(256), st, *a, in, (const bf16*)nullptr, n, out,
                      (bf16*)nullptr);
}

// in holds size * n elements; rank r receives the sum over ranks of chunk r.
B2_API int b2_comm_reduce_scatter(const CommArgs* a, const float* in, long n, float* out, cudaStream_t st) {
  if (!args_ok(a, n) || (!in && !a->skip_push) || !out) return B2_ERR_ARG;   // skip_push: wait-and-combine only (the pushes came from a fused GEMM epilogue)
  return launch_pdl_c(push_collective_kernel<2>, dim3(grid_of(n >> 2)), dim3(256), st, *a, in, (const bf16*)nullptr, n, out,
                      (bf16*)nullptr);
}

// See collect_gather_kernel.  a->slot_off is slot A (the GEMM's partials), slot_b_off slot B (the gathered sums); out is
// bf16 [total_rows, n_cols] contiguous; rows_per * n_cols <= slot_stride, n_cols % 4 == 0.
B2_API int b2_comm_collect_gather(const CommArgs* a, long slot_b_off, int rows_per, int n_cols, int total_rows, bf16* out,
                                  cudaStream_t st) {
  if (!a || !a->status || !out || a->size < 1 || a->size > kCommMaxRanks || a->rank < 0 || a->rank >= a->size) return B2_ERR_ARG;
  if (rows_per <= 0 || n_cols <= 0 || (n_cols % 4) || total_rows <= 0 || (long)rows_per * a->size < total_rows) return B2_ERR_ARG;
  if ((long)rows_per * n_cols > a->slot_stride || (a->slot_off % 4) || (slot_b_off % 4) || (a->slot_stride % 4)) return B2_ERR_ARG;
  return launch_pdl_c(collect_gather_kernel, dim3(grid_of(((long)rows_per * n_cols) >> 2)), dim3(256), st, *a, slot_b_off, rows_per,
                      n_cols, total_rows, out);
}

// Barrier = all-gather of one unit whose result is discarded into the caller's 4 * size float scratch (status reports
// a missing rank).
B2_API int b2_comm_barrier(const CommArgs* a, cudaStream_t st) {
  if (!a || !a->status) return B2_ERR_ARG;
  static float* ones[16] = {nullptr};
  static float* sink[16] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return B2_ERR_ARG;
  if (!ones[dev]) {
    const float h[4] = {1.f, 1.f, 1.f, 1.f};
    if (cudaMalloc(&ones[dev], 16) != cudaSuccess || cudaMalloc(&sink[dev], 16 * kCommMaxRanks) != cudaSuccess) return B2_ERR_LAUNCH;
    cudaMemcpy(ones[dev], h, 16, cudaMemcpyHostToDevice);
  }
  return b2_comm_all_gather(a, ones[dev], 4, sink[dev], st);
}

B2_API int b2_comm_argmax_combine(const CommArgs* a, const float* val, const int* idx, int n_tok, int* out_idx, float* out_val,
                                  cudaStream_t st) {
  if (!a || n_tok <= 0 || (long)n_tok * 4 > a->slot_stride || !a->status) return B2_ERR_ARG;
  if (a->clear_off >= 0 && (a->clear_n < 0 || a->clear_n > a->slot_stride || (a->clear_n % 4))) return B2_ERR_ARG;
  long blocks = (n_tok + 255) / 256;
  const long cb = a->clear_off >= 0 ? (a->clear_n / 4 + 255) / 256 : 0;
  if (cb > blocks) blocks = cb > 64 ? 64 : cb;
  return launch_pdl_c(argmax_combine_kernel, dim3((unsigned)blocks), dim3(256), st, *a, val, idx, n_tok, out_idx, out_val);
}
