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
//   O_blk (128 x 128, TMEM)    = P (smem)  x  V_blk (smem as V^T, K-major)                              4 MMAs of k = 16
//   O = O * exp2(m_old - m) + O_blk      in registers (128 fp32 per thread)
//
// K and V pages arrive with cp.async (16-token pages are contiguous 4 KB, so a block is four pages); V is transposed
// through ldmatrix.trans / stmatrix into the K-major layout the B operand wants.  While the tensor core works on one
// CTA's MMAs the other resident CTA of the SM (96 KB of shared memory and 256 TMEM columns each) runs its softmax.
// Every wait on the tensor core is bounded; expiry sets the status word and the CTA leaves through the normal exit
// (TMEM is released).
#include "common.cuh"

namespace b2 {
namespace {

constexpr int HD = 128;
constexpr int BK = 64;                 // keys per block
constexpr int kPfThreads = 128;
constexpr int kPfTmemCols = 256;       // S at column 0 (64 columns), O_blk at column 64 (128 columns)
constexpr int SM_Q = 0;                // two 64-dim halves of [128 rows][128 B]
constexpr int SM_K = 32768;            // two halves of [64 keys][128 B]
constexpr int SM_VR = SM_K + 16384;    // V as loaded: [64 keys][256 B], 16-byte chunks XOR-swizzled by key
constexpr int SM_VT = SM_VR + 16384;   // V^T: [128 dims][128 B = 64 keys]
constexpr int SM_P = SM_VT + 16384;    // P: [128 rows][128 B = 64 keys]
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
// D fp32, A / B bf16, both K-major, N / 8 and M / 16.
__host__ __device__ constexpr uint32_t pf_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
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
__device__ __forceinline__ void pf_ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pf_stsm_x4(uint32_t addr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
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
  __shared__ __align__(8) uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
    pf_mbar_init(smem_u32(&bar_s), 1);
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
  pdl_wait();

  // this thread's row: token t of the tile, query head h of the group
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
    const uint32_t dst = base + SM_Q + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4);
    pf_cp16(dst, src, ok);
  }

  // Pages of block j that this thread's copies touch (keys 8 i + tid / 16, i = 0..7: page i / 2 of the block's four).
  int pages[4];
  auto find_pages = [&](int j) {
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
  };
  // K (which = 0) or V (which = 1) of block j (whose pages find_pages looked up); keys past kv_len are zero-filled
  const int ld_key = tid >> 4, ld_c = tid & 15;
  auto load_block = [&](int j, int which) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int key = i * 8 + ld_key;
      const bool ok = j * BK + key < kv_len;
      const bf16* src = a.kv_pool + ((((size_t)pages[i >> 1] * 2 + which) * a.hkv + kvh) * 16 + (key & 15)) * HD + ld_c * 8;
      const uint32_t dst = which == 0 ? base + SM_K + (ld_c >> 3) * 8192 + key * 128 + (((ld_c & 7) ^ (key & 7)) << 4)
                                      : base + SM_VR + key * 256 + ((ld_c ^ (key & 7)) << 4);
      pf_cp16(dst, src, ok);
    }
  };
  if (n_blocks > 0) { find_pages(0); load_block(0, 0); load_block(0, 1); }
  asm volatile("cp.async.commit_group;" ::: "memory");

  float o[HD];
#pragma unroll
  for (int i = 0; i < HD; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  constexpr uint32_t idesc_s = pf_idesc(128, BK), idesc_o = pf_idesc(128, HD);
  bool failed = false;

#pragma unroll 1
  for (int j = 0; j < n_blocks; ++j) {
    const uint32_t par = (uint32_t)j & 1u;
    // A. K(j), V(j) (and Q) have landed; V -> V^T
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (__syncthreads_or(failed ? 1 : 0)) break;          // a wait gave up in the previous block: everyone leaves together
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int dc = warp * 4 + (u >> 1), k0 = (u & 1) * 32;              // 8-dim chunk, first key
      uint32_t r[4];
      {
        const int key = k0 + 8 * (lane >> 3) + (lane & 7);
        pf_ldsm_x4_t(base + SM_VR + key * 256 + ((dc ^ (key & 7)) << 4), r);
      }
      {
        const int d = dc * 8 + (lane & 7), kc = (k0 >> 3) + (lane >> 3);   // row of V^T, 8-key chunk
        pf_stsm_x4(base + SM_VT + d * 128 + ((kc ^ (d & 7)) << 4), r);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // B. S = Q K^T
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint64_t dq = pf_desc(base + SM_Q + h * 16384), dk = pf_desc(base + SM_K + h * 8192);
#pragma unroll
        for (int k = 0; k < 4; ++k) pf_mma(tmem_base, dq + 2 * k, dk + 2 * k, idesc_s, (h | k) ? 1u : 0u);
      }
      pf_commit(smem_u32(&bar_s));
    }
    // V(j + 1) may overwrite the raw V buffer now (everyone is past the transpose)
    if (j + 1 < n_blocks) { find_pages(j + 1); load_block(j + 1, 1); }
    // C. wait for S; then K(j + 1) may overwrite K
    if (!failed && !pf_mbar_wait(smem_u32(&bar_s), par)) { failed = true; atomicExch(&s_failed, 1); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (j + 1 < n_blocks) load_block(j + 1, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    // D. softmax of this thread's row
    float corr = 1.f;
    {
      float s[BK];
      {
        uint32_t r0[32], r1[32];
        pf_tmem_ld32_issue(tmem_base + ((uint32_t)(warp * 32) << 16) + 0u, r0);
        pf_tmem_ld32_issue(tmem_base + ((uint32_t)(warp * 32) << 16) + 32u, r1);
        pf_tmem_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = __uint_as_float(r0[i]) * a.scale_log2; s[32 + i] = __uint_as_float(r1[i]) * a.scale_log2; }
      }
      const int kb = j * BK;
      if (!row_valid || kb + BK - 1 > limit) {
#pragma unroll
        for (int i = 0; i < BK; ++i)
          if (!row_valid || kb + i > limit) s[i] = -INFINITY;
      }
      float mx = m_run;
#pragma unroll
      for (int i = 0; i < BK; ++i) mx = fmaxf(mx, s[i]);
      const float mref = (mx == -INFINITY) ? 0.f : mx;      // a fully masked row: every p = 2^-inf = 0
      corr = pf_ex2(m_run - mref);
      m_run = mx;
      float sum = 0.f;
      uint32_t pk[BK / 2];
#pragma unroll
      for (int i = 0; i < BK; i += 2) {
        const float p0 = pf_ex2(s[i] - mref), p1 = pf_ex2(s[i + 1] - mref);
        sum += p0 + p1;
        pk[i >> 1] = pf_pack(p0, p1);
      }
      l_run = l_run * corr + sum;
      const uint32_t prow = base + SM_P + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + ((c ^ (row & 7)) << 4)), "r"(pk[4 * c]), "r"(pk[4 * c + 1]),
                     "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3]) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // E. O_blk = P V
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t dp = pf_desc(base + SM_P), dv = pf_desc(base + SM_VT);
#pragma unroll
      for (int k = 0; k < 4; ++k) pf_mma(tmem_base + 64u, dp + 2 * k, dv + 2 * k, idesc_o, k ? 1u : 0u);
      pf_commit(smem_u32(&bar_o));
    }
    // F. O = O * corr + O_blk
    if (!failed && !pf_mbar_wait(smem_u32(&bar_o), par)) { failed = true; atomicExch(&s_failed, 1); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int c0 = 0; c0 < HD; c0 += 64) {
      uint32_t r0[32], r1[32];
      pf_tmem_ld32_issue(tmem_base + ((uint32_t)(warp * 32) << 16) + 64u + (uint32_t)c0, r0);
      pf_tmem_ld32_issue(tmem_base + ((uint32_t)(warp * 32) << 16) + 96u + (uint32_t)c0, r1);
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
