// Fragment-major (FM) weight layout of the mixed 2/3/4-bit linears: record geometry, shared-memory fragment loads, code
// extraction for mma.m16n8k16 and the bounded mbarrier / bulk-copy helpers shared by the GEMV kernel (wq_gemv.cu) and
// the persistent decode-step kernel (step_kernel.cu).
#pragma once
#include "common.cuh"

namespace b2 {


constexpr uint32_t kMagic = 0x64006400u;   // two fp16 1024.0

template <int BITS> struct Fmt;
template <> struct Fmt<4> { static constexpr int CK = 64, REC = 512; };
template <> struct Fmt<2> { static constexpr int CK = 128, REC = 512; };
template <> struct Fmt<3> { static constexpr int CK = 128, REC = 768; };

// Weights of one 128-k batch of one 16-row block as held by a lane, plus the (scale, zero) pairs of its rows.
template <int BITS, int GROUP>
struct WFrag {
  static constexpr int RPB = 128 / Fmt<BITS>::CK;
  static constexpr int GPB = 128 / GROUP;
  uint4 lo[RPB];
  uint2 hi;                 // 3-bit only
  uint32_t sz[GPB][2];      // half2 (scale, zero) for rows g and g+8
};

// Geometry of the FM buffer and of a warp's shared-memory ring.  The buffer is a grid of blocks, one per (32-row
// panel, 128-k batch): [2 row blocks x records][2 row blocks x groups x 16 rows x (scale, zero)].  A ring stage holds
// the RB/2 blocks of one batch of a warp item and is filled by RB/2 cp.async.bulk copies that complete on the
// stage's mbarrier.  Every warp runs its own ring, so nothing inside the k loop synchronises the CTA.
template <int BITS, int GROUP, int RB>
struct Ring {
  static constexpr int RPB = 128 / Fmt<BITS>::CK;
  static constexpr int GPB = 128 / GROUP;
  static constexpr int W_BATCH = RPB * Fmt<BITS>::REC;     // weight bytes of one batch of one row block
  static constexpr int BLK = 2 * W_BATCH + 2 * GPB * 64;    // one (panel, batch) block
  static constexpr int STAGE = (RB / 2) * BLK;
  static constexpr int NST = (BITS == 4 ? 2 : (BITS == 3 ? 3 : 4)) * (RB == 2 ? 2 : 1);   // about 9 KB in flight per warp
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds and reports failure instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int BITS, int GROUP>
__device__ __forceinline__ void load_frag_smem(WFrag<BITS, GROUP>& f, const uint8_t* wrec, const uint8_t* szrec, int lane) {
  constexpr int REC = Fmt<BITS>::REC;
  constexpr int RPB = WFrag<BITS, GROUP>::RPB;
  constexpr int GPB = WFrag<BITS, GROUP>::GPB;
#pragma unroll
  for (int i = 0; i < RPB; ++i) f.lo[i] = *reinterpret_cast<const uint4*>(wrec + i * REC + lane * 16);
  if (BITS == 3) f.hi = *reinterpret_cast<const uint2*>(wrec + 512 + lane * 8);
#pragma unroll
  for (int g = 0; g < GPB; ++g) {
    f.sz[g][0] = *reinterpret_cast<const uint32_t*>(szrec + g * 64 + (lane >> 2) * 4);
    f.sz[g][1] = *reinterpret_cast<const uint32_t*>(szrec + g * 64 + 32 + (lane >> 2) * 4);
  }
}

__device__ __forceinline__ uint32_t u4_get(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// A fragments of mma step s (0..7) of the batch.
template <int BITS, int GROUP>
__device__ __forceinline__ void extract(const WFrag<BITS, GROUP>& f, int s, uint32_t (&a)[4]) {
  if (BITS == 4) {
    const uint32_t w = u4_get(f.lo[s >> 2], s & 3);
    const uint32_t w8 = w >> 8;
    a[0] = lop3_and_or(w, 0x000F000Fu, kMagic);    // row g,   slots 0,1  (c = 1)
    a[2] = lop3_and_or(w, 0x00F000F0u, kMagic);    // row g,   slots 2,3  (c = 16)
    a[1] = lop3_and_or(w8, 0x000F000Fu, kMagic);   // row g+8, slots 0,1
    a[3] = lop3_and_or(w8, 0x00F000F0u, kMagic);   // row g+8, slots 2,3
  } else {
    const int u = s >> 1;
    const uint32_t w = u4_get(f.lo[0], u);
    const uint32_t w8 = w >> 8;
    const int q0 = 2 * (s & 1);                      // field index of slots (0,1); slots (2,3) use q0 + 1
    const uint32_t m0 = 0x00030003u << (2 * q0);
    const uint32_t m1 = 0x00030003u << (2 * q0 + 2);
    a[0] = lop3_and_or(w, m0, kMagic);
    a[2] = lop3_and_or(w, m1, kMagic);
    a[1] = lop3_and_or(w8, m0, kMagic);
    a[3] = lop3_and_or(w8, m1, kMagic);
    if (BITS == 3) {
      // High bits: one shift per (word, row half) puts the four bits of that round right above their fields.
      const uint32_t h = (u >> 1) ? f.hi.y : f.hi.x;
      const uint32_t h0 = (u & 1) ? (h >> 6) : (h << 2);   // rounds 0 / 2 (row g)
      const uint32_t h1 = (u & 1) ? (h >> 7) : (h << 1);   // rounds 1 / 3 (row g+8)
      const uint32_t b0 = 0x00040004u << (2 * q0);
      const uint32_t b1 = 0x00040004u << (2 * q0 + 2);
      a[0] = lop3_or_and(a[0], h0, b0);
      a[2] = lop3_or_and(a[2], h0, b1);
      a[1] = lop3_or_and(a[1], h1, b0);
      a[3] = lop3_or_and(a[3], h1, b1);
    }
  }
}

// 1 / c of k position kk (0..127 inside a batch), and c itself.
template <int BITS>
__device__ __forceinline__ void slot_scale(int kk, float& cinv, float& c) {
  const int slot = kk & 3;
  if (BITS == 4) {
    c = (slot < 2) ? 1.f : 16.f;
  } else {
    const int sp = (kk >> 4) & 1;
    c = sp ? ((slot < 2) ? 16.f : 64.f) : ((slot < 2) ? 1.f : 4.f);
  }
  cinv = 1.f / c;
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

}  // namespace b2
