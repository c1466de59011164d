// Causal prefill attention over the paged KV cache on the 5th-generation tensor cores (tcgen05 + TMEM), head_dim 128.
//
// The reference's prefill attention is a flash kernel on mma.sync tiles (kernels/m1/m1_attn.cu:120-410, 64-row query
// tiles, K/V through cp.async).  Here a CTA owns one 128-row query tile = (128 / gq) consecutive tokens x the gq
// query heads of one KV head (GQA: the heads of a group share every K/V byte), the native M of tcgen05.mma, and walks
// the sequence in blocks of 64 keys:
//
//   S (128 x 64, fp32, TMEM)   = Q (smem, K-major, 128-byte swizzle)  x  K_blk^T (smem, K-major)      8 MMAs of k = 16
//   P = exp2(S * scale - m)    thread = row: tcgen05.ld of its 64 scores, online max / sum, bf16 P row written to
//                              shared memory in the swizzled A-operand layout
//   O_blk (128 x 128, TMEM)    = P (smem)  x  V_blk (smem as loaded, MN-major B operand)                4 MMAs of k = 16
//   O = O * exp2(m_old - m) + O_blk      in registers (128 fp32 per thread)
//
// K and V pages arrive with cp.async (16-token pages are contiguous 4 KB, so a block is four pages) straight into the
// swizzled operand layout; V needs no transpose because the B operand of P V is taken MN-major.  S is double-buffered
// in TMEM and K in shared memory: S(j + 1) is issued right behind P V(j), so the tensor core computes it while the
// threads fold O_blk(j) into O.  While one CTA runs its softmax the other resident CTA of the SM (96 KB of shared
// memory and 256 TMEM columns each) has the tensor core.
// Every wait on the tensor core is bounded; expiry sets the status word and the CTA leaves through the normal exit
// (TMEM is released).
#include "common.cuh"

namespace b2 {
namespace {

constexpr int HD = 128;
constexpr int BK = 64;                 // keys per block
constexpr int kPfThreads = 128;
constexpr int kPfTmemCols = 256;       // S of even / odd blocks at columns 0 / 64 (64 columns each), O_blk at column 128 (128 columns)
constexpr int SM_Q = 0;                // two 64-dim halves of [128 rows][128 B]
constexpr int SM_K = 32768;            // two K buffers, each two 64-dim halves of [64 keys][128 B]
constexpr int SM_V = SM_K + 32768;     // V, same layout as a K buffer
constexpr int SM_P = SM_V + 16384;     // P: [128 rows][128 B = 64 keys]
constexpr int SM_PF_BYTES = SM_P + 16384 + 1024;   // + slack for the 1024-byte alignment of the swizzle pattern

struct PfArgs {
  const bf16* q;          // [T][hq * 128]
  const bf16* kv_pool;    // [page][2][hkv][16][128]
  const int* bt;          // block-table row of the sequence
  bf16* out;              // [T][hq * 128]
  int T, pos0, hq, hkv, n_pages, bt_len;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void pf_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool pf_mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait (about two seconds); false = gave up.
__device__ __forceinline__ bool pf_mbar_wait(uint32_t bar, uint32_t parity) {
  if (pf_mbar_try(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (!pf_mbar_try(bar, parity)) {
    if (globaltimer_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}
// K-major operand, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t pf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D fp32, A / B bf16, A K-major, B K-major or (b_mn) MN-major, N / 8 and M / 16.
__host__ __device__ constexpr uint32_t pf_idesc(int m, int n, bool b_mn = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// MN-major operand, 128-byte swizzle: 64 elements of the MN dimension are contiguous (128 B); successive k rows are
// 128 B apart, 8-row groups `sbo` bytes apart, the next 64 MN elements `lbo` bytes away.
__device__ __forceinline__ uint64_t pf_desc_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void pf_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void pf_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void pf_tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void pf_tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16-byte asynchronous copy; `valid` false writes zeros (source size 0) without touching the source.
__device__ __forceinline__ void pf_cp16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
// 2^x on the special-function unit; 2^-inf = 0
__device__ __forceinline__ float pf_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pf_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace

__global__ void __launch_bounds__(kPfThreads, 2) attn_prefill_tc_kernel(const PfArgs a) {
  extern __shared__ __align__(1024) uint8_t pf_smem[];
  __shared__ __align__(8) uint64_t bar_s[2], bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;

  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t base = (smem_u32(pf_smem) + 1023u) & ~1023u;
  const int gq = a.hq / a.hkv;
  const int tt = 128 / gq;                                   // tokens per tile
  const int n_tiles = (a.T + tt - 1) / tt;
  const int tile = n_tiles - 1 - (int)blockIdx.x;            // longest tiles first
  const int kvh = blockIdx.y;
  const int tok0 = tile * tt;
  const int n_tok = min(tt, a.T - tok0);
  const int kv_len = a.pos0 + tok0 + n_tok;
  const int n_blocks = (kv_len + BK - 1) / BK;

  if (tid == 0) {
    pf_mbar_init(smem_u32(&bar_s[0]), 1);
    pf_mbar_init(smem_u32(&bar_s[1]), 1);
    pf_mbar_init(smem_u32(&bar_o), 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kPfTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_row = tmem_base + ((uint32_t)(warp * 32) << 16);     // this warp's 32 TMEM lanes
  pdl_wait();

  // this thread's row: token rt of the tile, query head rh of the group
  const int row = tid;
  const int rt = row / gq, rh = row - rt * gq;
  const bool row_valid = rt < n_tok;
  const int limit = a.pos0 + tok0 + rt;                      // last key this row may see

  // ---- Q tile: 128 rows x 256 B -> two swizzled halves
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int e = i * kPfThreads + tid;
    const int r = e >> 4, c = e & 15;
    const int t = r / gq, h = r - t * gq;
    const bool ok = t < n_tok;
    const bf16* src = a.q + ((size_t)(tok0 + (ok ? t : 0)) * a.hq + (size_t)kvh * gq + h) * HD + c * 8;
    pf_cp16(base + SM_Q + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4), src, ok);
  }

  // K (which = 0) or V (which = 1) of block j: 64 keys x 256 B as two 64-dim halves of [64 keys][128 B], 16-byte chunks
  // swizzled by key (K is the K-major B operand of S = Q K^T, V the MN-major B operand of O = P V).  This thread copies
  // chunk tid & 15 of keys 8 i + tid / 16; the block's four pages are looked up once; keys past kv_len are zero-filled.
  const int ld_key = tid >> 4, ld_c = tid & 15;
  auto load_block = [&](int j, int which, uint32_t dst_base) {
    int pages[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int pi = j * 4 + g;
      int page = 0;
      if (pi * 16 < kv_len) {
        page = pi < a.bt_len ? __ldg(a.bt + pi) : -1;
        if (page < 0 || page >= a.n_pages) { atomicExch(a.status, (int)B2_ERR_BOUNDS); page = 0; }
      }
      pages[g] = page;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int key = i * 8 + ld_key;
      const bool ok = j * BK + key < kv_len;
      const bf16* src = a.kv_pool + ((((size_t)pages[i >> 1] * 2 + which) * a.hkv + kvh) * 16 + (key & 15)) * HD + ld_c * 8;
      pf_cp16(dst_base + (ld_c >> 3) * 8192 + key * 128 + (((ld_c & 7) ^ (key & 7)) << 4), src, ok);
    }
  };
  auto commit = [] { asm volatile("cp.async.commit_group;" ::: "memory"); };
  constexpr uint32_t idesc_s = pf_idesc(128, BK), idesc_o = pf_idesc(128, HD, true);
  auto issue_s = [&](int j) {               // S(j) = Q K(j)^T into TMEM columns 64 (j & 1)
    const uint32_t kb = base + SM_K + (j & 1) * 16384;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint64_t dq = pf_desc(base + SM_Q + h * 16384), dk = pf_desc(kb + h * 8192);
#pragma unroll
      for (int k = 0; k < 4; ++k) pf_mma(tmem_base + 64u * (j & 1), dq + 2 * k, dk + 2 * k, idesc_s, (h | k) ? 1u : 0u);
    }
    pf_commit(smem_u32(&bar_s[j & 1]));
  };

  // prologue: Q + K(0) | K(1) | V(0) as three copy groups; S(0) is issued as soon as the first has landed
  if (n_blocks > 0) load_block(0, 0, base + SM_K);
  commit();
  if (n_blocks > 1) load_block(1, 0, base + SM_K + 16384);
  commit();
  if (n_blocks > 0) load_block(0, 1, base + SM_V);
  commit();
  asm volatile("cp.async.wait_group 2;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && n_blocks > 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    issue_s(0);
  }

  float o[HD];
#pragma unroll
  for (int i = 0; i < HD; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  bool failed = false;

#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    // 1. S(j) is complete: its K buffer takes K(j + 2)
    if (!failed && !pf_mbar_wait(smem_u32(&bar_s[j & 1]), (uint32_t)(j >> 1) & 1u)) { failed = true; atomicExch(&s_failed, 1); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (j + 2 < n_blocks) load_block(j + 2, 0, base + SM_K + (j & 1) * 16384);
    commit();
    // 2. softmax of this thread's row -> P
    float corr;
    {
      // raw scores; the softmax scale folds into the exponent: p = 2^(s * scale - m * scale), m = max of the raw scores
      float s[BK];
      {
        uint32_t r0[32], r1[32];
        pf_tmem_ld32_issue(tmem_row + 64u * (j & 1), r0);
        pf_tmem_ld32_issue(tmem_row + 64u * (j & 1) + 32u, r1);
        pf_tmem_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(r0[i]); s[32 + i] = __uint_as_float(r1[i]); }
      }
      const int kb = j * BK;
      if (!row_valid || kb + BK - 1 > limit) {
#pragma unroll
        for (int i = 0; i < BK; ++i)
          if (!row_valid || kb + i > limit) s[i] = -INFINITY;
      }
      // four independent chains for the maximum and for the sum: a warp has only one partner warp on its scheduler
      float mx4[4] = {m_run, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BK; i += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], s[i + u]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float mref = (mx == -INFINITY) ? 0.f : mx;      // a fully masked row: every p = 2^-inf = 0
      const float moff = -mref * a.scale_log2;
      corr = pf_ex2(fmaf(m_run, a.scale_log2, moff));
      m_run = mx;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[BK / 2];
#pragma unroll
      for (int i = 0; i < BK; i += 4) {
        const float p0 = pf_ex2(fmaf(s[i], a.scale_log2, moff)), p1 = pf_ex2(fmaf(s[i + 1], a.scale_log2, moff));
        const float p2 = pf_ex2(fmaf(s[i + 2], a.scale_log2, moff)), p3 = pf_ex2(fmaf(s[i + 3], a.scale_log2, moff));
        sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
        pk[i >> 1] = pf_pack(p0, p1);
        pk[(i >> 1) + 1] = pf_pack(p2, p3);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l_run = l_run * corr + sum;
      const uint32_t prow = base + SM_P + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((c ^ (row & 7)) << 4)), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                     "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3]) : "memory");
    }
    // 3. everything but the newest copy group has landed: K(j + 1) and V(j)
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (__syncthreads_or(failed ? 1 : 0)) break;            // a wait gave up: everyone leaves together
    // 4. O_blk = P V(j); then S(j + 1) right behind it, so that it runs while the threads fold O_blk into O
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t dp = pf_desc(base + SM_P);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        pf_mma(tmem_base + 128u, dp + 2 * k, pf_desc_mn(base + SM_V + k * 2048, 8192, 1024), idesc_o, k ? 1u : 0u);
      pf_commit(smem_u32(&bar_o));
      if (j + 1 < n_blocks) issue_s(j + 1);
    }
    // 5. O = O * corr + O_blk; the V buffer takes V(j + 1)
    if (!failed && !pf_mbar_wait(smem_u32(&bar_o), (uint32_t)j & 1u)) { failed = true; atomicExch(&s_failed, 1); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (j + 1 < n_blocks) load_block(j + 1, 1, base + SM_V);
    commit();
#pragma unroll
    for (int c0 = 0; c0 < HD; c0 += 64) {
      uint32_t r0[32], r1[32];
      pf_tmem_ld32_issue(tmem_row + 128u + (uint32_t)c0, r0);
      pf_tmem_ld32_issue(tmem_row + 160u + (uint32_t)c0, r1);
      pf_tmem_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        o[c0 + i] = fmaf(o[c0 + i], corr, __uint_as_float(r0[i]));
        o[c0 + 32 + i] = fmaf(o[c0 + 32 + i], corr, __uint_as_float(r1[i]));
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // ---- output row
  if (row_valid && !failed) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    bf16* dst = a.out + ((size_t)(tok0 + rt) * a.hq + (size_t)kvh * gq + rh) * HD;
#pragma unroll
    for (int c = 0; c < HD; c += 8) {
      uint4 w;
      w.x = pf_pack(o[c] * inv, o[c + 1] * inv);
      w.y = pf_pack(o[c + 2] * inv, o[c + 3] * inv);
      w.z = pf_pack(o[c + 4] * inv, o[c + 5] * inv);
      w.w = pf_pack(o[c + 6] * inv, o[c + 7] * inv);
      *reinterpret_cast<uint4*>(dst + c) = w;
    }
  }
  pdl_launch_dependents();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && s_failed && a.status) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPfTmemCols) : "memory");
  }
}

}  // namespace b2

using namespace b2;

// Causal attention of a prefill chunk: q [T][hq * 128] at positions pos0 .. pos0 + T - 1 of one sequence whose block
// table row is `bt` (bt_len entries); the KV pool already holds the chunk's own K / V.  head_dim 128, gq = hq / hkv
// a divisor of 128.
B2_API int b2_attn_prefill_tc(const void* q, const void* kv_pool, const int* bt, int bt_len, void* out, int T, int pos0, int hq, int hkv,
                              int n_pages, float scale, int* status, cudaStream_t stream) {
  if (T <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || 128 % (hq / hkv) || !status) return B2_ERR_ARG;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_PF_BYTES) != cudaSuccess) return B2_ERR_LAUNCH;
    attr_set = true;
  }
  PfArgs a;
  a.q = static_cast<const bf16*>(q);
  a.kv_pool = static_cast<const bf16*>(kv_pool);
  a.bt = bt;
  a.bt_len = bt_len;
  a.out = static_cast<bf16*>(out);
  a.T = T; a.pos0 = pos0; a.hq = hq; a.hkv = hkv; a.n_pages = n_pages;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  const int tt = 128 / (hq / hkv);
  dim3 grid((unsigned)((T + tt - 1) / tt), (unsigned)hkv, 1);
  attn_prefill_tc_kernel<<<grid, kPfThreads, SM_PF_BYTES, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
