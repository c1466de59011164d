// Paged GQA attention for decode, batched decode and linear / tree verify (1..8 query tokens per sequence), sm_100a.
//
// Replaces the reference's FlashInfer instantiations for decode and multi-query verify (ak_attn_decode,
// ak_attn_decode_multi, ak_attn_decode_packed and their device-side planners, kernels/oracle/bcsa_local_oracle.cu:
// 262-695) and the small-window drafter/MTP attention kernels (kernels/m1/m1_draft.cu:153-340, m1_mtp.cu:225-279).
//
// Work item = (query group, kv head, 16-row tile, kv split) and is processed by ONE warp, sequentially over the
// pages of its split; splits are merged in split order by attn_merge_kernel.  The split size is an engine
// constant, so the arithmetic of a query row depends only on its own position: a row computed in an 8-token
// verify block is bit-identical to the same row computed by a plain decode step (the per-query plan rule the
// reference adopted in 1.3.3, CHANGELOG.md:203-205).  The q heads that share a kv head fill the M dimension of
// the mma tile (8 heads x 2 tokens per 16-row tile for the 32B model).
// KV pool of a layer: [page][2 (K,V)][kv_head][page_size = 16][head_dim] bf16; pages come from a block table.
#include "common.cuh"

namespace b2 {

struct AttnDecodeArgs {
  const bf16* q; long ldq;            // [n_tok][hq*hd], RoPE applied
  const bf16* kv_pool; int n_pages;
  const int* block_table; int bt_ld;  // [seq][bt_ld]
  const int* grp_tok0; const int* grp_cnt; int n_groups;   // consecutive tokens of one sequence
  const int* tok_pos; const int* tok_seq;
  const unsigned* tree_mask;          // optional [n_tok]: bit j set = token may attend the group's j-th token
  int hq, hkv;
  int split_keys, max_splits;
  float scale_log2;
  float* part_o;                      // [n_tok][hq][max_splits][hd]
  float* part_ml;                     // [n_tok][hq][max_splits][2]
  bf16* out; long ldo;                // [n_tok][hq*hd]
  int n_tok;
  int* status;
  // Tiered KV: a launch may cover only the splits [split_lo, split_hi) (0, 0 = all) and leave the merge to a later
  // launch (phase bit 0: split kernel, bit 1: merge kernel; 0 = both).  Partial results of several launches -- pages
  // resident on the GPU, page batches staged from pinned host memory -- land in their own split slots and are merged
  // once, in split order, so the result is bit-identical to an all-resident run.
  int split_lo, split_hi, phase;
  // 1: the four warps of a CTA take the four 16-row tiles of one (group, kv head, split) and share one K/V ring in
  // shared memory (prefill chunks and verify blocks, where a group has many rows); 0: every warp is its own item.
  int shared_kv;
};

namespace {

constexpr int kPage = 16;
constexpr int kStages = 3;      // CTA-shared ring (prefill chunks, verify blocks): 24 KB per CTA
constexpr int kStagesWarp = 2;  // per-warp rings (decode): 64 KB per 4-warp CTA; two CTAs per SM at 178 registers

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace

template <int HD, bool SHARED>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnDecodeArgs a) {
  constexpr int KS = HD / 16;          // k-steps of QK^T
  constexpr int NTO = HD / 8;          // n-tiles of O
  constexpr int ROWB = HD * 2;         // bytes per K/V row
  constexpr int CPR = ROWB / 16;       // 16-byte chunks per row
  constexpr int PAGE_B = kPage * ROWB; // bytes of one K (or V) page slab
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();
  pdl_launch_dependents();

  const int gq = a.hq / a.hkv;
  // decode the work item
  const int s_lo = a.split_hi > 0 ? a.split_lo : 0;
  const int s_n = a.split_hi > 0 ? a.split_hi - a.split_lo : a.max_splits;
  const int mt_max = (8 * gq + 15) / 16;             // tiles needed for the largest group (8 tokens)
  long item = SHARED ? (long)blockIdx.x : (long)blockIdx.x * 4 + warp;
  const int split = s_lo + (int)(item % s_n); item /= s_n;
  int mtile;
  if (SHARED) mtile = warp; else { mtile = (int)(item % mt_max); item /= mt_max; }
  const int kvh = (int)(item % a.hkv); item /= a.hkv;
  const int grp = (int)item;
  if (grp >= a.n_groups) return;                      // uniform over the CTA when SHARED
  const int tok0 = a.grp_tok0[grp], cnt = a.grp_cnt[grp];
  const bool tile_ok = mtile * 16 < cnt * gq;
  if (!SHARED && !tile_ok) return;
  const int seq = a.tok_seq[tok0];
  const int pos_first = a.tok_pos[tok0];
  const int kv_len = a.tok_pos[tok0 + cnt - 1] + 1;
  const int k_begin = split * a.split_keys;
  if (k_begin >= kv_len) return;
  const int k_end = min(kv_len, k_begin + a.split_keys);
  const int n_pg = (k_end - k_begin + kPage - 1) / kPage;

  // rows of this lane: r0 = g, r1 = g + 8
  int rtok[2], rhead[2], rpos[2];
  bool rvalid[2];
  unsigned rmask[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int R = mtile * 16 + g + 8 * i;
    const int tl = R / gq;
    rvalid[i] = tile_ok && tl < cnt;
    rtok[i] = tok0 + (rvalid[i] ? tl : 0);
    rhead[i] = kvh * gq + (R % gq);
    rpos[i] = rvalid[i] ? a.tok_pos[rtok[i]] : -1;
    rmask[i] = (a.tree_mask && rvalid[i]) ? a.tree_mask[rtok[i]] : 0xffffffffu;
  }

  constexpr int ST = SHARED ? kStages : kStagesWarp;
  uint8_t* wsm = smem + (SHARED ? (size_t)0 : (size_t)warp * ST * 2 * PAGE_B);
  const uint32_t wsm_u = smem_u32(wsm);
  const int* bt = a.block_table + (size_t)seq * a.bt_ld;
  if (bt[k_begin / kPage] == -2) return;   // split lives in the host tier: a staged launch fills its slot

  auto issue_page = [&](int pi) {
    const int stage = pi % ST;
    int page = bt[(k_begin / kPage) + pi];
    if (page < 0 || page >= a.n_pages) { atomicExch(a.status, (int)B2_ERR_BOUNDS); page = 0; }
    const uint8_t* kp = reinterpret_cast<const uint8_t*>(a.kv_pool) + (((size_t)page * 2 + 0) * a.hkv + kvh) * PAGE_B;
    const uint8_t* vp = reinterpret_cast<const uint8_t*>(a.kv_pool) + (((size_t)page * 2 + 1) * a.hkv + kvh) * PAGE_B;
    const uint32_t ks = wsm_u + stage * 2 * PAGE_B, vs = ks + PAGE_B;
#pragma unroll
    for (int c = SHARED ? (int)threadIdx.x : lane; c < kPage * CPR; c += SHARED ? 128 : 32) {
      const int row = c / CPR, cc = c % CPR;
      const uint32_t off = row * ROWB + ((cc ^ (row & 7)) << 4);
      cp_async16(ks + off, kp + (size_t)c * 16);
      cp_async16(vs + off, vp + (size_t)c * 16);
    }
  };

  // prefetch
#pragma unroll
  for (int pi = 0; pi < ST - 1; ++pi) {
    if (pi < n_pg) issue_page(pi);
    cp_async_commit();
  }

  // Q fragments
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t v0 = 0u, v1 = 0u;
      if (rvalid[i]) {
        const bf16* qp = a.q + (size_t)rtok[i] * a.ldq + (size_t)rhead[i] * HD + ks * 16 + 2 * t;
        v0 = *reinterpret_cast<const uint32_t*>(qp);
        v1 = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
      qa[ks][i] = v0;
      qa[ks][2 + i] = v1;
    }
  }

  float o[NTO][4];
#pragma unroll
  for (int n = 0; n < NTO; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  for (int pi = 0; pi < n_pg; ++pi) {
    if (pi + ST - 1 < n_pg) issue_page(pi + ST - 1);
    cp_async_commit();
    cp_async_wait<ST - 1>();
    if (SHARED) __syncthreads(); else __syncwarp();
    const int stage = pi % ST;
    const uint32_t ks_u = wsm_u + stage * 2 * PAGE_B, vs_u = ks_u + PAGE_B;
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b[4];
      const int j = lane >> 3;
      const int key = (j >> 1) * 8 + (lane & 7);
      const int cc = 2 * ks + (j & 1);
      ldsm_x4(ks_u + key * ROWB + ((cc ^ (key & 7)) << 4), b);
      mma_bf16_16816(s[0], qa[ks], b[0], b[1]);
      mma_bf16_16816(s[1], qa[ks], b[2], b[3]);
    }
    // scale + mask.  Lane holds keys kb + {2t, 2t+1} (tile 0) and kb + 8 + {2t, 2t+1} (tile 1) for rows g, g+8.
    const int kb = k_begin + pi * kPage;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i >> 1;
        const int key = kb + n * 8 + 2 * t + (i & 1);
        bool ok = key <= rpos[r];
        if (ok && key >= pos_first) ok = (rmask[r] >> (key - pos_first)) & 1u;   // inside the verify block: tree mask
        const float v = ok ? s[n][i] * a.scale_log2 : -INFINITY;
        s[n][i] = v;
        mx[r] = fmaxf(mx[r], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], psum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float mnew = fmaxf(mrow[r], mx[r]);
      corr[r] = (mnew == -INFINITY) ? 1.f : exp2f(mrow[r] - mnew);
      mrow[r] = mnew;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i >> 1;
        const float p = (s[n][i] == -INFINITY) ? 0.f : exp2f(s[n][i] - mrow[r]);
        s[n][i] = p;
        psum[r] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      lrow[r] = lrow[r] * corr[r] + psum[r];
    }
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    uint32_t pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = pack_bf16(s[0][2], s[0][3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int nn = 0; nn < NTO / 2; ++nn) {
      uint32_t b[4];
      const int j = lane >> 3;
      const int key = (j & 1) * 8 + (lane & 7);
      const int cc = 2 * nn + (j >> 1);
      ldsm_x4_t(vs_u + key * ROWB + ((cc ^ (key & 7)) << 4), b);
      mma_bf16_16816(o[2 * nn], pa, b[0], b[1]);
      mma_bf16_16816(o[2 * nn + 1], pa, b[2], b[3]);
    }
    if (SHARED) __syncthreads(); else __syncwarp();
  }
  cp_async_wait<0>();

  // partial result of this split
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (!rvalid[r]) continue;
    float* po = a.part_o + (((size_t)rtok[r] * a.hq + rhead[r]) * a.max_splits + split) * HD;
#pragma unroll
    for (int n = 0; n < NTO; ++n)
      *reinterpret_cast<float2*>(po + n * 8 + 2 * t) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
    if (t == 0) {
      float* pm = a.part_ml + (((size_t)rtok[r] * a.hq + rhead[r]) * a.max_splits + split) * 2;
      pm[0] = mrow[r];
      pm[1] = lrow[r];
    }
  }
}

// Combine the splits of every (token, q head).  Splits are taken in blocks of eight; block b belongs to lane set
// b % 8, every set adds its blocks' splits in ascending order, and the eight sets are added in set order at the end.
// WPI = 1: one warp per (token, head) keeps the eight sets in registers (prefill chunks, large batches).
// WPI = 8: eight warps per (token, head), one set each, joined through shared memory (decode and verify steps, where
// the items are few and the chain of dependent loads is what costs).  Both run the same additions in the same order,
// so a row's bits do not depend on which variant merged it.
template <int HD, int WPI>
__global__ void attn_merge_kernel(const AttnDecodeArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int PER = HD / 32;
  constexpr int SETS = 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int item = WPI == 1 ? blockIdx.x * (blockDim.x >> 5) + warp : blockIdx.x;
  const bool live = item < a.n_tok * a.hq;
  __shared__ float part[WPI == 1 ? 1 : SETS][HD + 32];
  float acc[WPI == 1 ? SETS : 1][PER], L[WPI == 1 ? SETS : 1];
#pragma unroll
  for (int w = 0; w < (WPI == 1 ? SETS : 1); ++w) {
    L[w] = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[w][i] = 0.f;
  }
  int tok = 0, head = 0;
  if (live) {
    tok = item / a.hq; head = item - tok * a.hq;
    const int ns = (a.tok_pos[tok] + a.split_keys) / a.split_keys;   // ceil((pos + 1) / split_keys)
    const float* po = a.part_o + ((size_t)tok * a.hq + head) * a.max_splits * HD;
    const float2* pm = reinterpret_cast<const float2*>(a.part_ml + ((size_t)tok * a.hq + head) * a.max_splits * 2);
    float M = -INFINITY;
    for (int s = lane; s < ns; s += 32) M = fmaxf(M, pm[s].x);
    M = warp_max(M);
    const int b0 = WPI == 1 ? 0 : warp, bstep = WPI == 1 ? 1 : SETS;
    for (int blk = b0; blk * 8 < ns; blk += bstep) {
      const int s0 = blk * 8;
      float2 ml[8];
      float pv[8][PER];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int s = s0 + j;
        ml[j] = s < ns ? pm[s] : make_float2(-INFINITY, 0.f);
#pragma unroll
        for (int i = 0; i < PER; ++i) pv[j][i] = s < ns ? po[(size_t)s * HD + lane * PER + i] : 0.f;
      }
      if (WPI == 1) {
#pragma unroll
        for (int w = 0; w < SETS; ++w) {
          if ((blk & (SETS - 1)) != w) continue;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (ml[j].x == -INFINITY) continue;
            const float wt = exp2f(ml[j].x - M);
            L[w] = fmaf(ml[j].y, wt, L[w]);
#pragma unroll
            for (int i = 0; i < PER; ++i) acc[w][i] = fmaf(pv[j][i], wt, acc[w][i]);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (ml[j].x == -INFINITY) continue;
          const float wt = exp2f(ml[j].x - M);
          L[0] = fmaf(ml[j].y, wt, L[0]);
#pragma unroll
          for (int i = 0; i < PER; ++i) acc[0][i] = fmaf(pv[j][i], wt, acc[0][i]);
        }
      }
    }
  }
  float o[PER], Ls;
  if (WPI == 1) {
    if (!live) return;
    Ls = L[0];
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = acc[0][i];
#pragma unroll
    for (int w = 1; w < SETS; ++w) {
      Ls = __fadd_rn(Ls, L[w]);
#pragma unroll
      for (int i = 0; i < PER; ++i) o[i] = __fadd_rn(o[i], acc[w][i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) part[warp][lane * PER + i] = acc[0][i];
    if (lane == 0) part[warp][HD] = L[0];
    __syncthreads();
    if (warp != 0 || !live) return;
    Ls = part[0][HD];
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = part[0][lane * PER + i];
#pragma unroll
    for (int w = 1; w < SETS; ++w) {
      Ls = __fadd_rn(Ls, part[w][HD]);
#pragma unroll
      for (int i = 0; i < PER; ++i) o[i] = __fadd_rn(o[i], part[w][lane * PER + i]);
    }
  }
  const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
  bf16* out = a.out + (size_t)tok * a.ldo + (size_t)head * HD + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; ++i) out[i] = __float2bfloat16_rn(__fmul_rn(o[i], inv));
}

}  // namespace b2

using namespace b2;

B2_API int b2_attn_decode_smem_bytes(int hd) { return 4 * kStagesWarp * 2 * kPage * hd * 2; }
static int attn_shared_smem_bytes(int hd) { return kStages * 2 * kPage * hd * 2; }

// Launches the split kernel and the merge kernel.  `max_groups_tiles` is not needed: the grid covers
// n_groups x hkv x tiles(8 tokens) x max_splits warp items.
B2_API int b2_attn_decode(const AttnDecodeArgs* args, int hd, cudaStream_t st) {
  const AttnDecodeArgs& a = *args;
  if (a.n_groups <= 0 || a.n_tok <= 0 || a.hq % a.hkv || a.split_keys % kPage || a.max_splits <= 0) return B2_ERR_ARG;
  if (hd != 128 && hd != 64) return B2_ERR_ARG;
  const int gq = a.hq / a.hkv;
  const int mt_max = (8 * gq + 15) / 16;
  if (a.split_hi > 0 && (a.split_lo < 0 || a.split_hi <= a.split_lo || a.split_hi > a.max_splits)) return B2_ERR_ARG;
  const int s_n = a.split_hi > 0 ? a.split_hi - a.split_lo : a.max_splits;
  const bool shared = a.shared_kv != 0 && mt_max <= 4;     // four warps = at most four row tiles per group
  const long items = shared ? (long)a.n_groups * a.hkv * s_n : (long)a.n_groups * a.hkv * mt_max * s_n;
  const bool run_split = a.phase == 0 || (a.phase & 1), run_merge = a.phase == 0 || (a.phase & 2);
  const int grid = shared ? (int)items : (int)((items + 3) / 4);
  const size_t smem = shared ? (size_t)attn_shared_smem_bytes(hd) : (size_t)b2_attn_decode_smem_bytes(hd);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  cudaError_t e = cudaSuccess;
  static bool attr_set = false;
  if (!attr_set) {
    const int big = b2_attn_decode_smem_bytes(128);
    cudaFuncSetAttribute(attn_decode_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attn_decode_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attn_decode_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    cudaFuncSetAttribute(attn_decode_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, big);
    attr_set = true;
  }
  if (!run_split) {
  } else if (hd == 128) {
    e = shared ? cudaLaunchKernelEx(&cfg, attn_decode_kernel<128, true>, a) : cudaLaunchKernelEx(&cfg, attn_decode_kernel<128, false>, a);
  } else {
    e = shared ? cudaLaunchKernelEx(&cfg, attn_decode_kernel<64, true>, a) : cudaLaunchKernelEx(&cfg, attn_decode_kernel<64, false>, a);
  }
  if (e != cudaSuccess) return B2_ERR_LAUNCH;
  if (!run_merge) return B2_OK;
  const int merge_items = a.n_tok * a.hq;
  const bool wide = merge_items <= 148 * 8;               // few items: eight warps per item shorten the load chain
  cfg.gridDim = dim3(wide ? merge_items : (merge_items + 7) / 8); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0;
  if (hd == 128) e = wide ? cudaLaunchKernelEx(&cfg, attn_merge_kernel<128, 8>, a) : cudaLaunchKernelEx(&cfg, attn_merge_kernel<128, 1>, a);
  else e = wide ? cudaLaunchKernelEx(&cfg, attn_merge_kernel<64, 8>, a) : cudaLaunchKernelEx(&cfg, attn_merge_kernel<64, 1>, a);
  return e == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
