// Mixed 2/3/4-bit dequant GEMV for decode, verify and small batches (m <= 32 tokens), sm_100a.
//
// Replaces the reference's KT/KF/W4H GEMV family (kernels/src/w4_gemv.cu:280-2937, kernels/src/w4h.cu:140-553)
// with one kernel family over the fragment-major ("FM") weight layout:
//   * a lane's 16-byte load is exactly its m16n8k16 A fragments for rows g and g+8 of a 16-row block;
//   * one lop3 turns two codes into two fp16 numbers 1024 + c*code; the activation of that k slot is staged in
//     shared memory as x / c, and the 1024 offset and the zero point are removed once per group from
//     precomputed activation sums, so dequantisation costs about 0.6 integer instructions per weight;
//   * per-row arithmetic never depends on m, on the batch position of a token or on the launch shape: the k
//     range of every warp and the order of every reduction are functions of (n, k, ks) only.  This is the
//     batch-invariance contract of the reference (w4_gemv.cu:2640-2644) that makes speculative decoding
//     token-identical to plain greedy decoding.
// Prologue options fold RMSNorm into the activation staging; epilogue options fold the residual add (with the
// next norm's partial sums of squares), SwiGLU, argmax partials, or the tensor-parallel push all-reduce.
#include "wq_gemv.cuh"

namespace b2 {

namespace {

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

template <int BITS, int GROUP>
__device__ __forceinline__ void load_frag(WFrag<BITS, GROUP>& f, const uint8_t* wq, const __half2* sz, int rb, int nch,
                                          int ng, int kb /* batch index = k/128 */, int lane) {
  constexpr int REC = Fmt<BITS>::REC;
  constexpr int RPB = WFrag<BITS, GROUP>::RPB;
  constexpr int GPB = WFrag<BITS, GROUP>::GPB;
  const uint8_t* p = wq + ((size_t)rb * nch + (size_t)kb * RPB) * REC;
#pragma unroll
  for (int i = 0; i < RPB; ++i) f.lo[i] = ld_nc_v4(p + (size_t)i * REC + lane * 16);
  if (BITS == 3) f.hi = ld_nc_v2(p + 512 + lane * 8);
  const uint32_t* s = reinterpret_cast<const uint32_t*>(sz) + ((size_t)rb * ng + (size_t)kb * GPB) * 16 + (lane >> 2);
#pragma unroll
  for (int g = 0; g < GPB; ++g) {
    f.sz[g][0] = ld_nc_u32(s + g * 16);
    f.sz[g][1] = ld_nc_u32(s + g * 16 + 8);
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

}  // namespace

template <int BITS, int GROUP, int RB, int NT>
__global__ void __launch_bounds__(kGemvThreads) wq_gemv_kernel(const WqGemvArgs a) {
  constexpr int CK = Fmt<BITS>::CK;
  constexpr int GPB = 128 / GROUP;
  constexpr int PK = NT == 1 ? 512 : (NT == 2 ? 256 : 128);   // k positions staged per piece
  constexpr int XST = PK + 16;                                 // halfs per staged token row (bank spread)
  constexpr int ROWS = RB * 16;
  constexpr int MP = NT * 8;
  constexpr int NGP = PK / GROUP;

  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m = a.m;
  // carve shared memory
  float* inv_rms = reinterpret_cast<float*>(smem_raw);                       // [MP]
  float* red = inv_rms + MP;                                                 // [4][MP][ROWS]
  uint8_t* wbase = reinterpret_cast<uint8_t*>(red + 4 * MP * ROWS);
  const int xs_bytes = m * XST * 2;
  const int per_warp = xs_bytes + NGP * MP * 8;
  __half* xs = reinterpret_cast<__half*>(wbase + (size_t)warp * per_warp);   // [m][XST]
  float2* gsum = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(xs) + xs_bytes);   // [NGP][MP]

  const int nrb = a.n >> 4;
  const int nch = a.k / CK;
  const int ng = a.k / GROUP;
  const int panel = blockIdx.x;
  const int rb0 = panel * RB;

  // k range of this warp in 128-k batches (depends on k and ks only)
  const int nu = a.k >> 7;
  const int nsub = 4 * a.ks;
  const int sub = blockIdx.y * 4 + warp;
  const int u0 = (int)(((long)nu * sub) / nsub);
  const int u1 = (int)(((long)nu * (sub + 1)) / nsub);
  const int nb = u1 - u0;

  WFrag<BITS, GROUP> cur[RB], nxt[RB];
  int rbs[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) rbs[r] = min(rb0 + r, nrb - 1);   // tail panel: duplicate the last block, ignore it later
  // Weights do not depend on the previous kernel: start streaming before the dependency wait.
  if (nb > 0) {
#pragma unroll
    for (int r = 0; r < RB; ++r) load_frag<BITS, GROUP>(cur[r], a.wq, a.sz, rbs[r], nch, ng, u0, lane);
  }
  pdl_wait();
  pdl_launch_dependents();   // the next kernel may start prefetching its weights while this one runs

  if (a.pro == PRO_NORM) {
    for (int tok = warp; tok < m; tok += 4) {
      float s = 0.f;
      for (int p = lane; p < a.ss_parts; p += 32) s += a.ss_in[(size_t)p * a.ss_ld + tok];
      s = warp_sum(s);
      if (lane == 0) inv_rms[tok] = rsqrtf(s / (float)a.k + a.eps);
    }
  }
  __syncthreads();

  float y[RB][NT][4];
#pragma unroll
  for (int r = 0; r < RB; ++r)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) y[r][n][i] = 0.f;

  for (int b = 0; b < nb; ++b) {
    const int kb = u0 + b;
    if (b + 1 < nb) {
#pragma unroll
      for (int r = 0; r < RB; ++r) load_frag<BITS, GROUP>(nxt[r], a.wq, a.sz, rbs[r], nch, ng, kb + 1, lane);
    }
    const int pofs = (b * 128) % PK;
    if (pofs == 0) {
      // ---- stage the next piece of x for this warp: fp16(x / c) and the per-group sums ----
      __syncwarp();
      const int len = min(PK, (nb - b) * 128);
      const int k0 = kb * 128;
      const int nvec = len >> 3;
      for (int tok = 0; tok < m; ++tok) {
        for (int v0 = 0; v0 < nvec; v0 += 32) {
          const int v = v0 + lane;
          const bool act = v < nvec;
          float ssum = 0.f, xsum = 0.f;
          if (act) {
            const int k = k0 + v * 8;
            const uint4 raw = *reinterpret_cast<const uint4*>(a.x + (size_t)tok * a.ldx + k);
            const bf16* xb = reinterpret_cast<const bf16*>(&raw);
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(xb[i]);
            if (a.pro == PRO_NORM) {
              const uint4 wr = *reinterpret_cast<const uint4*>(a.norm_w + k);
              const bf16* wb = reinterpret_cast<const bf16*>(&wr);
              const float ir = inv_rms[tok];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = bf16_round(f[i] * ir * __bfloat162float(wb[i]));
            }
            __align__(16) __half h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float cinv, c;
              slot_scale<BITS>((v * 8 + i) & 127, cinv, c);
              h[i] = __float2half_rn(f[i] * cinv);
              const float hf = __half2float(h[i]);
              ssum += hf;
              xsum += hf * c;
            }
            *reinterpret_cast<uint4*>(xs + (size_t)tok * XST + v * 8) = *reinterpret_cast<const uint4*>(h);
          }
          // reduce over the GROUP/8 lanes that cover one group (fixed xor tree)
#pragma unroll
          for (int o = GROUP / 16; o > 0; o >>= 1) {
            ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
            xsum += __shfl_xor_sync(0xffffffffu, xsum, o);
          }
          if (act && (lane % (GROUP / 8)) == 0) gsum[((v * 8) / GROUP) * MP + tok] = make_float2(1024.f * ssum, xsum);
        }
      }
      __syncwarp();
    }
    // ---- one 128-k batch ----
#pragma unroll
    for (int gg = 0; gg < GPB; ++gg) {
      float acc[RB][NT][4];
#pragma unroll
      for (int r = 0; r < RB; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[r][n][i] = 0.f;
#pragma unroll
      for (int s8 = 0; s8 < 8 / GPB; ++s8) {
        const int s = gg * (8 / GPB) + s8;
        uint32_t bf[NT][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          bf[n][0] = 0u; bf[n][1] = 0u;
          const int tok = n * 8 + g;
          if (tok < m) {
            const uint2 v = *reinterpret_cast<const uint2*>(xs + (size_t)tok * XST + pofs + s * 16 + t * 4);
            bf[n][0] = v.x; bf[n][1] = v.y;
          }
        }
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          uint32_t af[4];
          extract<BITS, GROUP>(cur[r], s, af);
#pragma unroll
          for (int n = 0; n < NT; ++n) mma_f16_16816(acc[r][n], af, bf[n][0], bf[n][1]);
        }
      }
      // y += scale * (acc - 1024*sum(xs) - zero*sum(x))
      const int gi = (pofs / GROUP) + gg;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float2 q0 = gsum[gi * MP + n * 8 + 2 * t];
        const float2 q1 = gsum[gi * MP + n * 8 + 2 * t + 1];
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&cur[r].sz[gg][0]));
          const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&cur[r].sz[gg][1]));
          y[r][n][0] += s0.x * (acc[r][n][0] - q0.x - s0.y * q0.y);
          y[r][n][1] += s0.x * (acc[r][n][1] - q1.x - s0.y * q1.y);
          y[r][n][2] += s1.x * (acc[r][n][2] - q0.x - s1.y * q0.y);
          y[r][n][3] += s1.x * (acc[r][n][3] - q1.x - s1.y * q1.y);
        }
      }
    }
    if (b + 1 < nb) {
#pragma unroll
      for (int r = 0; r < RB; ++r) cur[r] = nxt[r];
    }
  }
  // tokens >= m were staged as zeros only implicitly (their B fragments were zero): gsum of those tokens is
  // uninitialised, so their y is garbage and is never read below.

  // ---- cross-warp reduction in warp order ----
#pragma unroll
  for (int r = 0; r < RB; ++r)
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int tok = n * 8 + 2 * t;
      float* base = red + ((size_t)warp * MP) * ROWS + r * 16 + g;
      base[(size_t)tok * ROWS] = y[r][n][0];
      base[(size_t)(tok + 1) * ROWS] = y[r][n][1];
      base[(size_t)tok * ROWS + 8] = y[r][n][2];
      base[(size_t)(tok + 1) * ROWS + 8] = y[r][n][3];
    }
  __syncthreads();
  float* fin = red;   // [tok][ROWS], reuses warp 0's slab after the sum
  {
    float v[(MP * ROWS + kGemvThreads - 1) / kGemvThreads];
    int c = 0;
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads, ++c)
      v[c] = ((red[idx] + red[MP * ROWS + idx]) + red[2 * MP * ROWS + idx]) + red[3 * MP * ROWS + idx];
    __syncthreads();
    c = 0;
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads, ++c) fin[idx] = v[c];
  }
  __syncthreads();

  // ---- split-k across CTAs: partials to scratch, the last CTA of the panel sums them in slice order ----
  if (a.ks > 1) {
    float* sp = a.scratch + ((size_t)panel * a.ks) * (size_t)(m * ROWS);
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads) sp[(size_t)blockIdx.y * (m * ROWS) + idx] = fin[idx];
    __threadfence();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
      const unsigned prev = atomicInc(a.counters + panel, (unsigned)a.ks - 1u);
      s_last = (prev == (unsigned)a.ks - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads) {
      float s = 0.f;
      for (int j = 0; j < a.ks; ++j) s += __ldcg(sp + (size_t)j * (m * ROWS) + idx);
      fin[idx] = s;
    }
    __syncthreads();
  }

  const int n0 = panel * ROWS;

  // ---- tensor-parallel push all-reduce of this panel ----
  if (a.epi == EPI_TP_RESID) {
    const TpPush& tp = a.tp;
    const int nvec = (m * ROWS) >> 2;
    if (!tp.skip_push) {
      for (int idx = threadIdx.x; idx < nvec * tp.size; idx += kGemvThreads) {
        const int dst = idx / nvec, e = (idx - dst * nvec) << 2;
        const int tok = e / ROWS, row = e - tok * ROWS;
        if (n0 + row >= a.n) continue;
        float4 v = *reinterpret_cast<const float4*>(fin + e);
        v.x += 0.f; v.y += 0.f; v.z += 0.f; v.w += 0.f;   // -0.0 -> +0.0: the sentinel never travels as data
        float* p = tp.inbox[dst] + tp.slot_off + (size_t)tp.rank * tp.slot_stride + (size_t)tok * a.n + n0 + row;
        asm volatile("st.volatile.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                     : "memory");
      }
    }
    __syncthreads();
    const float* mine = tp.inbox[tp.rank] + tp.slot_off;
    const uint64_t t_start = globaltimer_ns();
    for (int idx = threadIdx.x; idx < nvec; idx += kGemvThreads) {
      const int e = idx << 2;
      const int tok = e / ROWS, row = e - tok * ROWS;
      if (n0 + row >= a.n) continue;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int src = 0; src < tp.size; ++src) {
        const float* p = mine + (size_t)src * tp.slot_stride + (size_t)tok * a.n + n0 + row;
        float4 v;
        unsigned spins = 0;
        bool ok = false;
        while (true) {
          asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
          ok = (__float_as_uint(v.x) != 0x80000000u) & (__float_as_uint(v.y) != 0x80000000u) &
               (__float_as_uint(v.z) != 0x80000000u) & (__float_as_uint(v.w) != 0x80000000u);
          if (ok) break;
          if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > tp.timeout_ns) break;
        }
        if (!ok) {
          atomicExch(tp.status, (int)B2_ERR_TIMEOUT);
          v = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      *reinterpret_cast<float4*>(fin + e) = s;
    }
    // re-arm the slot that no rank writes before its next use
    if (tp.clear_off >= 0) {
      float* clr = tp.inbox[tp.rank] + tp.clear_off;
      const float neg0 = __uint_as_float(0x80000000u);
      for (int idx = threadIdx.x; idx < nvec * tp.size; idx += kGemvThreads) {
        const int src = idx / nvec, e = (idx - src * nvec) << 2;
        const int tok = e / ROWS, row = e - tok * ROWS;
        if (n0 + row >= a.n) continue;
        *reinterpret_cast<float4*>(clr + (size_t)src * tp.slot_stride + (size_t)tok * a.n + n0 + row) =
            make_float4(neg0, neg0, neg0, neg0);
      }
    }
    __syncthreads();
  }

  // ---- epilogues ----
  if (a.epi == EPI_STORE) {
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads) {
      const int tok = idx / ROWS, row = idx - tok * ROWS;
      if (n0 + row < a.n) a.y[(size_t)tok * a.ldy + n0 + row] = __float2bfloat16_rn(fin[idx]);
    }
  } else if (a.epi == EPI_F32) {
    for (int idx = threadIdx.x; idx < m * ROWS; idx += kGemvThreads) {
      const int tok = idx / ROWS, row = idx - tok * ROWS;
      if (n0 + row < a.n) a.yf[(size_t)tok * a.ldy + n0 + row] = fin[idx];
    }
  } else if (a.epi == EPI_RESID || a.epi == EPI_TP_RESID) {
    for (int tok = warp; tok < m; tok += 4) {
      float sq = 0.f;
#pragma unroll
      for (int row = lane; row < ROWS; row += 32) {
        if (n0 + row < a.n) {
          const float v = fin[tok * ROWS + row] + __bfloat162float(a.resid[(size_t)tok * a.ldr + n0 + row]);
          const bf16 hb = __float2bfloat16_rn(v);
          a.y[(size_t)tok * a.ldy + n0 + row] = hb;
          const float hf = __bfloat162float(hb);
          sq += hf * hf;
        }
      }
      sq = warp_sum(sq);
      if (lane == 0 && a.ss_out) a.ss_out[(size_t)panel * a.ss_ld + tok] = sq;
    }
  } else if (a.epi == EPI_SWIGLU) {
    constexpr int HR = ROWS / 2;
    for (int idx = threadIdx.x; idx < m * HR; idx += kGemvThreads) {
      const int tok = idx / HR, j = idx - tok * HR;
      const int blk = j >> 3, r = j & 7;
      if (n0 + blk * 16 < a.n) {
        const float gate = bf16_round(fin[tok * ROWS + blk * 16 + r]);
        const float up = bf16_round(fin[tok * ROWS + blk * 16 + 8 + r]);
        a.y[(size_t)tok * a.ldy + (size_t)panel * HR + j] = __float2bfloat16_rn(silu_f(gate) * up);
      }
    }
  } else if (a.epi == EPI_ARGMAX) {
    for (int tok = warp; tok < m; tok += 4) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int row = lane; row < ROWS; row += 32) {
        const int ni = n0 + row;
        if (ni < a.n) {
          const float v = fin[tok * ROWS + row];
          if (a.yf) a.yf[(size_t)tok * a.ldy + ni] = v;
          if (ni < a.n_valid && (v > best || (v == best && ni < bi))) { best = v; bi = ni; }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (lane == 0) {
        a.amax_val[(size_t)panel * a.ss_ld + tok] = best;
        a.amax_idx[(size_t)panel * a.ss_ld + tok] = bi;
      }
    }
  }
}

template <int BITS, int GROUP, int RB, int NT>
static int launch_one(const WqGemvArgs& a, cudaStream_t st) {
  constexpr int PK = NT == 1 ? 512 : (NT == 2 ? 256 : 128);
  constexpr int XST = PK + 16, ROWS = RB * 16, MP = NT * 8, NGP = PK / GROUP;
  const size_t smem = (size_t)MP * 4 + (size_t)4 * MP * ROWS * 4 + 4 * ((size_t)a.m * XST * 2 + (size_t)NGP * MP * 8);
  auto kern = wq_gemv_kernel<BITS, GROUP, RB, NT>;
  static bool attr_set = false;   // one flag per instantiation
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return B2_ERR_LAUNCH;
    attr_set = true;
  }
  const int nrb = a.n / 16;
  const int npanels = (nrb + RB - 1) / RB;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(npanels, a.ks, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, a) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

template <int BITS, int GROUP>
static int launch_bg(const WqGemvArgs& a, cudaStream_t st) {
  const int nt = (a.m + 7) / 8;
  if (a.rb == 4 && nt == 1) return launch_one<BITS, GROUP, 4, 1>(a, st);
  if (a.rb == 4 && nt == 2) return launch_one<BITS, GROUP, 4, 2>(a, st);
  if (a.rb == 2 && nt == 1) return launch_one<BITS, GROUP, 2, 1>(a, st);
  if (a.rb == 2 && nt == 2) return launch_one<BITS, GROUP, 2, 2>(a, st);
  if (a.rb == 2 && nt <= 4) return launch_one<BITS, GROUP, 2, 4>(a, st);
  return B2_ERR_ARG;
}

}  // namespace b2

using namespace b2;

B2_API long b2_wq_gemv_scratch_floats(int n, int rb, int ks, int m) {
  if (ks <= 1) return 0;
  const long npanels = (n / 16 + rb - 1) / rb;
  return npanels * ks * (long)m * rb * 16;
}

// Launches the GEMV described by *args on `stream`.  Returns a b2::Status; nothing is launched on B2_ERR_ARG.
B2_API int b2_wq_gemv(const WqGemvArgs* args, cudaStream_t stream) {
  WqGemvArgs a = *args;
  if (a.n <= 0 || a.k <= 0 || a.m <= 0 || a.m > 32) return B2_ERR_ARG;
  if (a.n % 16 || a.k % 128 || a.ks < 1) return B2_ERR_ARG;
  if (a.group != 64 && a.group != 128) return B2_ERR_ARG;
  if (a.rb != 2 && a.rb != 4) return B2_ERR_ARG;
  if (a.m > 16 && a.rb != 2) return B2_ERR_ARG;   // 17..32 tokens only with 32-row panels (register budget)
  if (a.ks > 1 && (!a.scratch || !a.counters)) return B2_ERR_ARG;
  if (a.epi == EPI_SWIGLU && (a.n % 32)) return B2_ERR_ARG;
  if ((a.ldx % 8) || (reinterpret_cast<uintptr_t>(a.x) & 15)) return B2_ERR_ARG;
  if (a.epi == EPI_TP_RESID && ((a.n % 4) || a.tp.size < 1 || a.tp.size > kMaxTp)) return B2_ERR_ARG;
  switch (a.bits * 1000 + a.group) {
    case 4128: return launch_bg<4, 128>(a, stream);
    case 4064: return launch_bg<4, 64>(a, stream);
    case 3128: return launch_bg<3, 128>(a, stream);
    case 3064: return launch_bg<3, 64>(a, stream);
    case 2128: return launch_bg<2, 128>(a, stream);
    case 2064: return launch_bg<2, 64>(a, stream);
  }
  return B2_ERR_ARG;
}
