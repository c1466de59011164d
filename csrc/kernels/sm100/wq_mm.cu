// Mixed-bit weight GEMM on the 5th-generation tensor cores for 9 .. 256 token rows (batched decode, big verify blocks,
// prefill chunks): y[tok][row] = sum_k W[row][k] x[tok][k], W stored as 2/3/4-bit codes in the FM layout of the GEMV.
//
// The weights are the M operand (128 rows per CTA), the tokens the N operand, so one tcgen05.mma covers 128 weight
// rows x all tokens x 16 k and the cost of a step hardly depends on the token count.  Per CTA (row tile, k slice):
//   warp 0      TMA: the fp16 activation tile [tokens][64 k] of every stage (128-byte swizzle, this CTA's own copy)
//   warp 1      one elected thread issues tcgen05.mma (kind f16, fp32 accumulator in TMEM) and commits stage releases
//   warps 2..17 dequantisers (two sets of eight alternating over the stages): each owns a 16-row block; it reads the lane's FM words straight from global memory
//               (prefetched one stage ahead), turns codes into fp16 weights scale * (code - zero) with two HFMA2 per
//               pair, and writes them into the stage's A tile in the same swizzled K-major layout TMA would produce
//   warps 2..5  afterwards read the accumulator with tcgen05.ld and run the epilogue (same variants as the GEMV:
//               store, residual + next-norm statistics, SwiGLU, fp32, argmax partials)
// Split-k partials meet in scratch memory; the CTA that arrives last adds them in slice order (deterministic, and
// independent of the token count).  Every wait is bounded; on expiry the CTA sets B2_ERR_TIMEOUT, frees its TMEM and
// returns.  Replaces dequant_kt_kernel + cuBLAS and w4_gemm_kernel / w4h_bt_kernel of the reference
// (kernels/m1/m1_model.cu:1875-1895, kernels/src/w4_gemv.cu, w4h.cu) for every m above the GEMV's range.
#include <cuda.h>

#include "common.cuh"

// The `dbg` bits of the argument block switch parts of the kernel off for measurements (results are then meaningless);
// production builds compile them out: only -DB2_MEASURE builds read the field.
#ifdef B2_MEASURE
#define B2_DBG(a, bit) ((a).dbg & (bit))
#else
#define B2_DBG(a, bit) 0
#endif

namespace b2 {

struct WqMmArgs {
  const uint8_t* wq; int n, k, m;
  int bits, group;
  int ks;                     // k slices: b2_wq_mm_ks(n, k)
  int n_pad;                  // token rows of the fp16 activation buffer: 32, 64, 128 or 256
  int stages;
  int epi;
  bf16* y; long ldy;
  const bf16* resid; long ldr;
  float* ss_out; int ss_ld;
  float* yf;
  float* amax_val; int* amax_idx; int n_valid;
  float* scratch; unsigned* counters;
  int* status;
  int dbg;                    // measurement aid (results meaningless): 1 no weight loads, 2 no proxy fence, 4 no dequant stores, 8 no MMA
};

namespace {

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2, EPI_F32 = 3, EPI_ARGMAX = 4 };
constexpr int BM = 128, BKS = 64;                // BKS: width of one 128-byte swizzle atom in fp16 elements
constexpr int A_SUB = BM * BKS * 2;              // 16 KB: 128 rows x 64 k
constexpr int A_STAGE = 2 * A_SUB;               // a stage covers one 128-k batch: two sub-tiles per operand
constexpr int kMmThreads = 576;                  // 18 warps: TMA, MMA, 2 x 8 dequantisers
constexpr int kDequantWarps = 8;
constexpr uint32_t kMagicH = 0x64006400u;        // two fp16 1024.0

__device__ __forceinline__ void mbar_init_m(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_m(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_m(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// try_wait with a suspend-time hint: the thread sleeps in hardware until the phase flips or the hint runs out, so a
// waiting warp issues few instructions (the tensor-core pipeline shares its issue slots with sixteen busy warps).
__device__ __forceinline__ bool mbar_try_wait_m(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000000u) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_m(uint32_t bar, uint32_t parity) {      // bounded: about two seconds
  if (mbar_try_wait_m(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  unsigned it = 0;
  while (!mbar_try_wait_m(bar, parity)) {
    if ((++it & 15u) == 0u && globaltimer_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d_m(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D fp32, A and B fp16 (format 0), both K-major
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_m(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32_m(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float siluf(float v) { return v / (1.f + __expf(-v)); }

template <int BITS> struct FmtM;
template <> struct FmtM<4> { static constexpr int CK = 64, REC = 512; };
template <> struct FmtM<2> { static constexpr int CK = 128, REC = 512; };
template <> struct FmtM<3> { static constexpr int CK = 128, REC = 768; };

struct RawW { uint4 lo0, lo1; uint2 hi; uint32_t sz[4]; };

}  // namespace

template <int BITS, int GROUP>
__global__ void __launch_bounds__(kMmThreads, 1) wq_mm_kernel(const __grid_constant__ CUtensorMap map_x, const WqMmArgs a) {
  constexpr int RPB = 128 / FmtM<BITS>::CK;
  constexpr int GPB = 128 / GROUP;
  constexpr int W_BATCH = RPB * FmtM<BITS>::REC;
  constexpr int BLK = 2 * W_BATCH + 2 * GPB * 64;
  extern __shared__ __align__(1024) uint8_t smem_m[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;
  __shared__ unsigned s_prev;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = a.stages;
  const int b_sub = a.n_pad * BKS * 2;
  const int b_stage = 2 * b_sub;
  const int stage_bytes = A_STAGE + b_stage;
  const uint32_t ring = (smem_u32(smem_m) + 1023u) & ~1023u;
  const int tile = blockIdx.x, slice = blockIdx.y;
  const int nbat = a.k / 128;
  const int kb0 = (nbat * slice) / a.ks, kb1 = (nbat * (slice + 1)) / a.ks;      // 128-k batches of this slice
  const int nkb = kb1 - kb0;
  const int npan = a.n / 32;
  // One accumulator for every token count: splitting the k steps over several TMEM regions measured no faster and
  // would make a row's summation order depend on how many rows travel with it.
  const int nacc = 1;
  const uint32_t tmem_cols = (uint32_t)(nacc * a.n_pad);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init_m(smem_u32(&full_bar[i]), 1 + kDequantWarps); mbar_init_m(smem_u32(&empty_bar[i]), 1); }
    mbar_init_m(smem_u32(&acc_bar), 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- activation tiles by TMA ----------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (kb >= S && !mbar_wait_m(smem_u32(&empty_bar[s]), ((kb / S) - 1) & 1)) { atomicExch(&s_failed, 1); break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        if (B2_DBG(a, 16)) { mbar_arrive_m(bar); continue; }
        mbar_expect_tx_m(bar, (uint32_t)b_stage);
        tma_load_2d_m(ring + s * stage_bytes + A_STAGE, &map_x, (kb0 + kb) * 128, 0, bar);
        tma_load_2d_m(ring + s * stage_bytes + A_STAGE + b_sub, &map_x, (kb0 + kb) * 128 + BKS, 0, bar);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = idesc_f16(BM, a.n_pad);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!mbar_wait_m(smem_u32(&full_bar[s]), (kb / S) & 1)) { atomicExch(&s_failed, 1); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = ring + s * stage_bytes, sb = sa + A_STAGE;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
          const uint64_t da = desc_sw128(sa + kh * A_SUB), db = desc_sw128(sb + kh * b_sub);
#pragma unroll
          for (int k = 0; k < BKS / 16; ++k) {
            const int q = kh * 4 + k, acc = q % nacc;
            if (!B2_DBG(a, 8)) umma_f16(tmem_base + (uint32_t)(acc * a.n_pad), da + 2 * k, db + 2 * k, idesc, (kb || q >= nacc) ? 1u : 0u);
          }
        }
        umma_commit_m(smem_u32(&empty_bar[s]));
      }
      umma_commit_m(smem_u32(&acc_bar));
    }
  } else {
    // ---------------- dequantisers: warp - 2 = 2 * panel + row block ----------------
    // two sets of eight warps alternate over the stages (set = stage parity), so that sixteen warps hide each other's
    // latencies; inside a set, warp = 2 * panel + row block
    const int dw = (warp - 2) & 7, kset = (warp - 2) >> 3;
    const int p = dw >> 1, rbk = dw & 1;
    const int g = lane >> 2, t = lane & 3;
    const int pan = tile * 4 + p;
    const bool pan_ok = pan < npan;
    const uint8_t* pbase = a.wq + (size_t)(pan_ok ? pan : 0) * nbat * BLK;
    auto load_raw = [&](int kb) -> RawW {
      RawW r;
      const uint8_t* blk = pbase + (size_t)(kb0 + kb) * BLK;
      r.lo1 = make_uint4(0u, 0u, 0u, 0u); r.hi = make_uint2(0u, 0u); r.sz[2] = r.sz[3] = 0u;
      if (B2_DBG(a, 1)) { r.lo0 = r.lo1 = make_uint4(kb, kb, kb, kb); r.sz[0] = r.sz[1] = r.sz[2] = r.sz[3] = 0x3C003C00u; return r; }
      r.lo0 = ld_nc_v4(blk + rbk * W_BATCH + lane * 16);
      if (BITS == 4) r.lo1 = ld_nc_v4(blk + rbk * W_BATCH + 512 + lane * 16);
      if (BITS == 3) r.hi = ld_nc_v2(blk + rbk * W_BATCH + 512 + lane * 8);
      const uint8_t* sz = blk + 2 * W_BATCH + rbk * GPB * 64 + g * 4;
#pragma unroll
      for (int gi = 0; gi < GPB; ++gi) { r.sz[2 * gi] = ld_nc_u32(sz + gi * 64); r.sz[2 * gi + 1] = ld_nc_u32(sz + gi * 64 + 32); }
      return r;
    };
    // tile address pieces of this lane: rows (p*32 + rbk*16 + g) and that + 8
    const uint32_t row_off = (uint32_t)((p * 4 + rbk * 2) * 1024 + g * 128);
    // the lane's fields of mma step j cover the four consecutive inputs 16 j + 4 t .. + 3 (first pair, second pair)
    uint32_t joff[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) joff[j] = (uint32_t)((((2 * j + (t >> 1)) ^ g) << 4) + ((t & 1) << 3));
    // Register ring of raw FM words, kPrefetch stages deep: enough loads in flight per warp to cover DRAM latency.
    constexpr int kPrefetch = 6;
    RawW ringw[kPrefetch];
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i)
      if (kset + 2 * i < nkb) ringw[i] = load_raw(kset + 2 * i);
    bool ok = true;
    for (int ibase = 0; kset + 2 * ibase < nkb && ok; ibase += kPrefetch) {
#pragma unroll
     for (int pi = 0; pi < kPrefetch; ++pi) {
      const int kb = kset + 2 * (ibase + pi);
      if (kb < nkb && ok) {
      const RawW cur = ringw[pi];
      if (kb + 2 * kPrefetch < nkb) ringw[pi] = load_raw(kb + 2 * kPrefetch);
      const int s = kb % S;
      if (kb >= S && !mbar_wait_m(smem_u32(&empty_bar[s]), ((kb / S) - 1) & 1)) { atomicExch(&s_failed, 1); ok = false; }
      if (ok) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
      // (scale, scale) and (-zero * scale) x 2 of rows g and g + 8, formed in fp16 (one rounding of the product, as
      // an fp32 product rounded once would give); a panel past the end of the matrix contributes zeros
      const int gi = GPB == 2 ? h : 0;
      const __half2 z0 = *reinterpret_cast<const __half2*>(&cur.sz[2 * gi]), z1 = *reinterpret_cast<const __half2*>(&cur.sz[2 * gi + 1]);
      const __half2 zero2 = __floats2half2_rn(0.f, 0.f);
      const __half2 s0h = pan_ok ? __low2half2(z0) : zero2, s1h = pan_ok ? __low2half2(z1) : zero2;
      const __half2 b0h = __hneg2(__hmul2(__high2half2(z0), s0h)), b1h = __hneg2(__hmul2(__high2half2(z1), s1h));
      const uint32_t sc0 = *reinterpret_cast<const uint32_t*>(&s0h), sc1 = *reinterpret_cast<const uint32_t*>(&s1h);
      const uint32_t bi0 = *reinterpret_cast<const uint32_t*>(&b0h), bi1 = *reinterpret_cast<const uint32_t*>(&b1h);
      const uint32_t sa = ring + s * stage_bytes + h * A_SUB + row_off;
      const uint4 lo = (BITS == 4 && h) ? cur.lo1 : cur.lo0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t r0, r1, r2, r3;
        float ic0, ic1;                       // 1 / c of the two field positions
        if (BITS == 4) {
          const uint32_t w = j == 0 ? lo.x : (j == 1 ? lo.y : (j == 2 ? lo.z : lo.w));
          const uint32_t w8 = w >> 8;
          r0 = lop3_and_or(w, 0x000F000Fu, kMagicH); r2 = lop3_and_or(w, 0x00F000F0u, kMagicH);
          r1 = lop3_and_or(w8, 0x000F000Fu, kMagicH); r3 = lop3_and_or(w8, 0x00F000F0u, kMagicH);
          ic0 = 1.f; ic1 = 1.f / 16.f;
        } else {
          const int u = 2 * h + (j >> 1);
          const uint32_t w = u == 0 ? lo.x : (u == 1 ? lo.y : (u == 2 ? lo.z : lo.w));
          const uint32_t w8 = w >> 8;
          const int q0 = 2 * (j & 1);
          const uint32_t m0 = 0x00030003u << (2 * q0), m1 = 0x00030003u << (2 * q0 + 2);
          r0 = lop3_and_or(w, m0, kMagicH); r2 = lop3_and_or(w, m1, kMagicH);
          r1 = lop3_and_or(w8, m0, kMagicH); r3 = lop3_and_or(w8, m1, kMagicH);
          if (BITS == 3) {
            const uint32_t hw = h ? cur.hi.y : cur.hi.x;
            const uint32_t h0 = (u & 1) ? (hw >> 6) : (hw << 2);
            const uint32_t h1 = (u & 1) ? (hw >> 7) : (hw << 1);
            const uint32_t b0 = 0x00040004u << (2 * q0), b1 = 0x00040004u << (2 * q0 + 2);
            r0 = lop3_or_and(r0, h0, b0); r2 = lop3_or_and(r2, h0, b1);
            r1 = lop3_or_and(r1, h1, b0); r3 = lop3_or_and(r3, h1, b1);
          }
          ic0 = q0 ? 1.f / 16.f : 1.f; ic1 = q0 ? 1.f / 64.f : 1.f / 4.f;
        }
        // code = (1024 + c code) / c - 1024 / c (exact), weight = code * scale - zero * scale.  fp16 bit patterns of
        // (1 / c, -1024 / c): c = 1: (1, -1024); 4: (0.25, -256); 16: (0.0625, -64); 64: (0.015625, -16)
        const uint32_t m0h = ic0 == 1.f ? 0x3C003C00u : 0x2C002C00u, a0h = ic0 == 1.f ? 0xE400E400u : 0xD400D400u;
        const uint32_t m1h = ic1 == 0.25f ? 0x34003400u : (ic1 == 1.f / 16.f ? 0x2C002C00u : 0x24002400u);
        const uint32_t a1h = ic1 == 0.25f ? 0xDC00DC00u : (ic1 == 1.f / 16.f ? 0xD400D400u : 0xCC00CC00u);
        r0 = hfma2_u(hfma2_u(r0, m0h, a0h), sc0, bi0);
        r2 = hfma2_u(hfma2_u(r2, m1h, a1h), sc0, bi0);
        r1 = hfma2_u(hfma2_u(r1, m0h, a0h), sc1, bi1);
        r3 = hfma2_u(hfma2_u(r3, m1h, a1h), sc1, bi1);
        const uint32_t off = joff[j];
        if (!B2_DBG(a, 4)) {
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(sa + off), "r"(r0), "r"(r2) : "memory");
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(sa + 1024u + off), "r"(r1), "r"(r3) : "memory");
        }
      }
      }
      if (!B2_DBG(a, 2)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive_m(smem_u32(&full_bar[s]));
      }
      }
     }
    }

    // ---------------- epilogue: warps 2..5 own TMEM lanes 32 * (warp % 4) ----------------
    if (warp < 6) {
      const bool acc_ok = mbar_wait_m(smem_u32(&acc_bar), 0);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!acc_ok) atomicExch(&s_failed, 1);
      const int lane_base = (warp & 3) * 32;
      const int rit = lane_base + lane;                   // row inside the tile
      const int row = tile * BM + rit;
      const bool row_ok = row < a.n;
      const int part = tile * 4 + (warp & 3);             // 32-row panel of this warp
      const bool good = acc_ok && !s_failed;
      const size_t tile_sz = (size_t)a.n_pad * BM;
      float* my_part = a.scratch + ((size_t)tile * a.ks + slice) * tile_sz;
      bool run_epi = good;
      if (a.ks > 1) {
        if (good) {
          for (int c0 = 0; c0 < a.m; c0 += 32) {
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.f;
            for (int ai = 0; ai < nacc; ++ai) {
              uint32_t r[32];
              tmem_ld32_m(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(ai * a.n_pad + c0), r);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(r[i]);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c0 + i < a.m) my_part[(size_t)(c0 + i) * BM + rit] = acc[i];
          }
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) s_prev = atomicInc(a.counters + tile, (unsigned)a.ks - 1u);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        run_epi = good && s_prev == (unsigned)a.ks - 1u;
        if (run_epi) __threadfence();
      }
      if (run_epi) {
        for (int c0 = 0; c0 < a.m; c0 += 32) {
          float v[32];
          if (a.ks > 1) {
            const float* base = a.scratch + (size_t)tile * a.ks * tile_sz + rit;
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
              float sum = 0.f;
              if (c0 + i < a.m)
                for (int sl = 0; sl < a.ks; ++sl) sum += __ldcg(base + (size_t)sl * tile_sz + (size_t)(c0 + i) * BM);
              v[i] = sum;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
            for (int ai = 0; ai < nacc; ++ai) {
              uint32_t r[32];
              tmem_ld32_m(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(ai * a.n_pad + c0), r);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += __uint_as_float(r[i]);
            }
          }
#pragma unroll 1
          for (int i = 0; i < 32; ++i) {
            const int tok = c0 + i;
            if (tok >= a.m) break;
            const float val = v[i];
            if (a.epi == EPI_STORE) {
              if (row_ok) a.y[(size_t)tok * a.ldy + row] = __float2bfloat16_rn(val);
            } else if (a.epi == EPI_F32) {
              if (row_ok) a.yf[(size_t)tok * a.ldy + row] = val;
            } else if (a.epi == EPI_RESID) {
              float sq = 0.f;
              if (row_ok) {
                const bf16 hb = __float2bfloat16_rn(val + __bfloat162float(a.resid[(size_t)tok * a.ldr + row]));
                a.y[(size_t)tok * a.ldy + row] = hb;
                const float hf = __bfloat162float(hb);
                sq = hf * hf;
              }
              sq = warp_sum(sq);
              if (lane == 0 && a.ss_out && part < npan) a.ss_out[(size_t)part * a.ss_ld + tok] = sq;
            } else if (a.epi == EPI_SWIGLU) {
              const float up = __shfl_down_sync(0xffffffffu, val, 8);
              if ((lane & 8) == 0 && row_ok)
                a.y[(size_t)tok * a.ldy + (size_t)part * 16 + (lane >> 4) * 8 + (lane & 7)] =
                    __float2bfloat16_rn(siluf(bf16r(val)) * bf16r(up));
            } else if (a.epi == EPI_ARGMAX) {
              if (a.yf && row_ok) a.yf[(size_t)tok * a.ldy + row] = val;
              float best = (row_ok && row < a.n_valid) ? val : -INFINITY;
              int bi = (row_ok && row < a.n_valid) ? row : 0x7fffffff;
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
              }
              if (lane == 0 && part < npan) { a.amax_val[(size_t)part * a.ss_ld + tok] = best; a.amax_idx[(size_t)part * a.ss_ld + tok] = bi; }
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && s_failed && a.status) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// x (bf16 [m][ldx], optionally RMS-normalised with statistics left by the previous epilogue) -> fp16 [n_pad][k], rows
// >= m zero.  One CTA per output row.
__global__ void __launch_bounds__(256) wq_mm_xprep_kernel(const bf16* __restrict__ x, long ldx, int m, int k, const float* __restrict__ ss_in,
                                                          int ss_parts, int ss_ld, const bf16* __restrict__ norm_w, float eps,
                                                          __half* __restrict__ out) {
  __shared__ float s_inv;
  pdl_wait();
  pdl_launch_dependents();
  const int tok = blockIdx.x;
  __half* o = out + (size_t)tok * k;
  if (tok >= m) {
    for (int i = threadIdx.x * 8; i < k; i += 256 * 8) *reinterpret_cast<uint4*>(o + i) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  float inv = 1.f;
  if (norm_w) {
    if (threadIdx.x < 32) {
      float s = 0.f;
      for (int p = threadIdx.x; p < ss_parts; p += 32) s += ss_in[(size_t)p * ss_ld + tok];
      s = warp_sum(s);
      if (threadIdx.x == 0) s_inv = rsqrtf(s / (float)k + eps);
    }
    __syncthreads();
    inv = s_inv;
  }
  for (int i = threadIdx.x * 8; i < k; i += 256 * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + i);
    const bf16* xb = reinterpret_cast<const bf16*>(&raw);
    __align__(16) __half hv[8];
    if (norm_w) {
      const uint4 wr = *reinterpret_cast<const uint4*>(norm_w + i);
      const bf16* wb = reinterpret_cast<const bf16*>(&wr);
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(bf16r(__bfloat162float(xb[j]) * inv * __bfloat162float(wb[j])));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) hv[j] = __float2half_rn(__bfloat162float(xb[j]));
    }
    *reinterpret_cast<uint4*>(o + i) = *reinterpret_cast<const uint4*>(hv);
  }
}

}  // namespace b2

using namespace b2;

typedef CUresult (*EncodeTiledFnM)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFnM encode_fn_m() {
  static EncodeTiledFnM fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnM>(p);
  }
  return fn;
}

// k slices of a linear for this kernel: a function of the shape only.  Enough CTAs to cover the SMs, slices of at
// least 512 inputs (four 128-k stages).
B2_API int b2_wq_mm_ks(int n, int k) {
  const int tiles = (n + BM - 1) / BM, nbat = k / 128;
  int best = 1;
  for (int ks = 1; ks <= nbat && ks <= 16; ++ks) {
    if (nbat % ks || nbat / ks < 4) continue;
    best = ks;
    if (tiles * ks >= 148) break;
  }
  return best;
}
B2_API int b2_wq_mm_npad(int m) { return m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)); }
B2_API long b2_wq_mm_scratch_floats(int n, int k, int n_pad) {
  const long tiles = (n + BM - 1) / BM;
  return tiles * b2_wq_mm_ks(n, k) * (long)n_pad * BM;
}

// x16: caller-provided fp16 [n_pad][k] staging buffer (16-byte aligned).  pro_norm: ss_in / norm_w given.
B2_API int b2_wq_mm(const WqMmArgs* args, const bf16* x, long ldx, const float* ss_in, int ss_parts, int ss_ld, const bf16* norm_w,
                    float eps, __half* x16, cudaStream_t st) {
  WqMmArgs a = *args;
  if (a.n <= 0 || a.n % 32 || a.k % 128 || a.m < 1 || a.m > 256 || (a.bits != 2 && a.bits != 3 && a.bits != 4) ||
      (a.group != 64 && a.group != 128) || !x || !x16 || (ldx % 8))
    return B2_ERR_ARG;
  a.n_pad = b2_wq_mm_npad(a.m);
  a.ks = b2_wq_mm_ks(a.n, a.k);
  if ((a.epi == EPI_RESID || a.epi == EPI_ARGMAX) && a.m > a.ss_ld) return B2_ERR_ARG;
  if (a.ks > 1 && (!a.scratch || !a.counters)) return B2_ERR_ARG;
  const int b_stage = 2 * a.n_pad * BKS * 2;
  int stages = (200 * 1024) / (A_STAGE + b_stage);
  a.stages = stages > 8 ? 8 : stages;
  if (a.stages < 2) return B2_ERR_ARG;
  EncodeTiledFnM fn = encode_fn_m();
  if (!fn) return B2_ERR_LAUNCH;
  CUtensorMap mx;
  cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.n_pad};
  cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
  cuuint32_t box[2] = {(cuuint32_t)BKS, (cuuint32_t)a.n_pad};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return B2_ERR_LAUNCH;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_pad); cfg.blockDim = dim3(256); cfg.stream = st; cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, wq_mm_xprep_kernel, x, ldx, a.m, a.k, ss_in, ss_parts, ss_ld, norm_w, eps, x16) != cudaSuccess)
      return B2_ERR_LAUNCH;
  }
  const size_t smem = (size_t)a.stages * (A_STAGE + b_stage) + 1024;
  void (*kern)(const CUtensorMap, const WqMmArgs) = nullptr;
  if (a.bits == 4) kern = a.group == 128 ? wq_mm_kernel<4, 128> : wq_mm_kernel<4, 64>;
  else if (a.bits == 3) kern = a.group == 128 ? wq_mm_kernel<3, 128> : wq_mm_kernel<3, 64>;
  else kern = a.group == 128 ? wq_mm_kernel<2, 128> : wq_mm_kernel<2, 64>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 205 * 1024) != cudaSuccess) return B2_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.n + BM - 1) / BM, a.ks, 1);
  cfg.blockDim = dim3(kMmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, mx, a) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
