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
#include <cstdlib>
#include "wq_gemv.cuh"
#include "wq_frag.cuh"

namespace b2 {


// Persistent kernel.  CTA c works on k slice (c % ks) of every item; its eight warps pull items of that slice from
// a ticket counter.  A warp item is (16*RB rows, k slice); the activation slice is staged once per CTA; partial
// results of the ks slices of an item meet in scratch memory, and the warp that arrives last sums them in slice
// order and runs the epilogue with one or two rows per lane.
template <int BITS, int GROUP, int RB, int NT>
__global__ void __launch_bounds__(kGemvThreads) wq_gemv_kernel(const WqGemvArgs a) {
  constexpr int GPB = 128 / GROUP;
  constexpr int MP = NT * 8;
  constexpr int ROWS = RB * 16;
  constexpr int RPL = RB / 2;                   // rows per lane in the epilogue
  using R = Ring<BITS, GROUP, RB>;
  constexpr int NST = R::NST;

  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m = a.m;
  const int npan = a.n >> 5;                    // 32-row panels of the FM buffer
  const int nitems = (npan + RPL - 1) / RPL;
  const int nbat = a.k >> 7;
  const int ks = a.ks;
  const int slice = blockIdx.x % ks;
  const int u0 = (int)(((long)nbat * slice) / ks);
  const int u1 = (int)(((long)nbat * (slice + 1)) / ks);
  const int nb = u1 - u0;                       // 128-k batches of this CTA's slice = ring stages per item
  const int nb_max = (nbat + ks - 1) / ks;
  const int XST = nb_max * 128 + 16;            // halfs per staged token row (row pitch = 32 B mod 128 B)

  // shared memory: [8 rings][mbarriers][inv_rms][8 x fin][xs][gsum]
  uint8_t* ring = smem_raw + (size_t)warp * NST * R::STAGE;
  uint8_t* after = smem_raw + (size_t)kGemvWarps * NST * R::STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after) + warp * NST;
  float* inv_rms = reinterpret_cast<float*>(after + kGemvWarps * NST * 8);
  float* fin = inv_rms + 32 + (size_t)warp * m * ROWS;                                   // [m][ROWS] per warp
  __half* xs = reinterpret_cast<__half*>(inv_rms + 32 + (size_t)kGemvWarps * m * ROWS);   // [m][XST]
  float2* gsum = reinterpret_cast<float2*>(xs + (size_t)m * XST);                         // [nb_max * GPB][MP]

  const uint32_t ring_u = smem_u32(ring);
  const uint32_t bars_u = smem_u32(bars);
  // Static, balanced schedule.  The (item, batch) units of a slice are laid out item-major and cut into V equal
  // contiguous ranges, one per virtual worker; V depends on the linear's shape only, so the cut points -- and with
  // them every summation order -- never depend on the token count or on how many CTAs are resident.  The warps of the
  // CTAs that share a slice take virtual workers round robin (normally exactly one each).
  const int wstride = (gridDim.x / ks) * kGemvWarps;
  const int wfirst = (blockIdx.x / ks) * kGemvWarps + warp;
  const int V = a.vworkers;
  const unsigned U = (unsigned)nitems * (unsigned)nb;          // host checks U * V < 2^32
  auto range_lo = [&](int v) -> unsigned { return ((unsigned)v * U) / (unsigned)V; };

#ifdef B2_MEASURE   // measurement builds only (B200E_NVCC_DEFS=-DB2_MEASURE): phase stamps and the bandwidth-probe mode
  unsigned long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * kGemvWarps + warp) * 8 : nullptr;
#else
  unsigned long long* tr = nullptr;
#endif
  auto stamp = [&](int i) { if (tr && lane == 0) tr[i] = globaltimer_ns(); };
  stamp(0);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NST; ++i) mbar_init(bars_u + i * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  unsigned prod = 0, cons = 0;     // stages issued / consumed by this warp since kernel start
  // producer cursor (lane 0): virtual worker, next unit and end of its range; item / batch of the next unit
  int p_v = wfirst;
  unsigned p_u = 0, p_end = 0;
  int p_item = 0, p_b = 0;
  auto p_load = [&]() {            // position the cursor on the first non-empty worker at or after p_v
    while (p_v < V) {
      p_u = range_lo(p_v); p_end = range_lo(p_v + 1);
      if (p_u < p_end) { p_item = (int)(p_u / (unsigned)nb); p_b = (int)(p_u - (unsigned)p_item * (unsigned)nb); return; }
      p_v += wstride;
    }
  };
  auto issue_one = [&]() -> bool { // lane 0 only; returns false when nothing is left to issue
    if (p_v >= V) return false;
    const int slot = prod % NST;
    const uint32_t bar = bars_u + slot * 8;
    mbar_expect_tx(bar, (uint32_t)R::STAGE);
    const uint32_t dst = ring_u + slot * R::STAGE;
#pragma unroll
    for (int pi = 0; pi < RPL; ++pi) {
      const int pan = min(p_item * RPL + pi, npan - 1);   // tail item: duplicate the last panel, ignored later
      bulk_g2s(dst + pi * R::BLK, a.wq + ((size_t)pan * nbat + (u0 + p_b)) * R::BLK, (uint32_t)R::BLK, bar);
    }
    ++prod;
    ++p_u;
    if (++p_b == nb) { p_b = 0; ++p_item; }
    if (p_u == p_end) { p_v += wstride; p_load(); }
    return true;
  };
  if (lane == 0 && nb > 0) p_load();
  // Weights do not depend on the previous kernel: start streaming before the dependency wait.
  if (lane == 0 && nb > 0) {
    while (prod - cons < (unsigned)NST && issue_one()) { }
  }
  __syncwarp();
  stamp(1);
  pdl_wait();
  pdl_launch_dependents();
  stamp(2);   // the next kernel may start prefetching its weights while this one runs

  // ---- stage the activation slice of this CTA: fp16(x / c) and the per-group sums ----
  if (a.pro == PRO_NORM) {
    for (int tok = warp; tok < m; tok += kGemvWarps) {
      // partial sums are fetched eight at a time so that their latencies overlap; the order of the adds is fixed
      float s = 0.f;
      for (int p0 = lane; p0 < a.ss_parts; p0 += 256) {
        float pv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int p = p0 + 32 * i;
          pv[i] = p < a.ss_parts ? a.ss_in[(size_t)p * a.ss_ld + tok] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) s += pv[i];
      }
      s = warp_sum(s);
      if (lane == 0) inv_rms[tok] = rsqrtf(s / (float)a.k + a.eps);
    }
    __syncthreads();
  }
  {
    const int nvec = nb * 16;
    const int k0 = u0 * 128;
    for (int tok = 0; tok < m; ++tok) {
      for (int v0 = 0; v0 < nvec; v0 += kGemvThreads) {
        const int v = v0 + threadIdx.x;
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
  }
  __syncthreads();
  stamp(3);

  bool failed = false;
  bool first_wait = true;
  for (int vw = wfirst; vw < V && nb > 0 && !failed; vw += wstride) {
   unsigned u = range_lo(vw);
   const unsigned u_end = range_lo(vw + 1);
   while (u < u_end && !failed) {
    // one fragment: the batches [b_lo, b_hi) of one item that fall into this worker's range
    const int cur = (int)(u / (unsigned)nb);
    const int b_lo = (int)(u - (unsigned)cur * (unsigned)nb);
    const int b_hi = min(nb, b_lo + (int)(u_end - u));
    u += (unsigned)(b_hi - b_lo);
    float y[RB][NT][4];
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) y[r][n][i] = 0.f;

#pragma unroll 1
    for (int b = b_lo; b < b_hi; ++b) {
      const int slot = cons % NST;
      if (!mbar_wait_bounded(bars_u + slot * 8, (cons / NST) & 1u)) {
        if (a.status) atomicExch(a.status, (int)B2_ERR_TIMEOUT);
        failed = true;
        break;
      }
      if (first_wait) { stamp(4); first_wait = false; }
      const uint8_t* stg = ring + slot * R::STAGE;
#ifdef B2_MEASURE
      if (a.debug == 1) {   // measurement aid: stream the weights, skip the arithmetic
        y[0][0][0] += (float)stg[lane];
        __syncwarp();
        ++cons;
        if (lane == 0) {
          while (prod - cons < (unsigned)NST && issue_one()) { }
        }
        continue;
      }
#endif
      WFrag<BITS, GROUP> cf[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r)
        load_frag_smem<BITS, GROUP>(cf[r], stg + (r >> 1) * R::BLK + (r & 1) * R::W_BATCH,
                                    stg + (r >> 1) * R::BLK + 2 * R::W_BATCH + (r & 1) * GPB * 64, lane);
      const __half* xrow = xs + b * 128 + t * 4;
#pragma unroll
      for (int gg = 0; gg < GPB; ++gg) {
        // accumulators start at -1024 * sum(x / c) of the group, so the mma result is sum(code * x) directly
        const int gi = b * GPB + gg;
        float2 q0[NT], q1[NT];
        float acc[RB][NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          q0[n] = gsum[gi * MP + n * 8 + 2 * t];
          q1[n] = gsum[gi * MP + n * 8 + 2 * t + 1];
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            acc[r][n][0] = -q0[n].x; acc[r][n][1] = -q1[n].x;
            acc[r][n][2] = -q0[n].x; acc[r][n][3] = -q1[n].x;
          }
        }
#pragma unroll
        for (int s8 = 0; s8 < 8 / GPB; ++s8) {
          const int s = gg * (8 / GPB) + s8;
          uint32_t bf[NT][2];
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            bf[n][0] = 0u; bf[n][1] = 0u;
            const int tok = n * 8 + g;
            if (tok < m) {
              const uint2 v = *reinterpret_cast<const uint2*>(xrow + (size_t)tok * XST + s * 16);
              bf[n][0] = v.x; bf[n][1] = v.y;
            }
          }
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            uint32_t af[4];
            extract<BITS, GROUP>(cf[r], s, af);
#pragma unroll
            for (int n = 0; n < NT; ++n) mma_f16_16816(acc[r][n], af, bf[n][0], bf[n][1]);
          }
        }
        // y += scale * (acc - zero * sum(x))
#pragma unroll
        for (int r = 0; r < RB; ++r) {
          const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&cf[r].sz[gg][0]));
          const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&cf[r].sz[gg][1]));
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            y[r][n][0] = fmaf(s0.x, fmaf(-s0.y, q0[n].y, acc[r][n][0]), y[r][n][0]);
            y[r][n][1] = fmaf(s0.x, fmaf(-s0.y, q1[n].y, acc[r][n][1]), y[r][n][1]);
            y[r][n][2] = fmaf(s1.x, fmaf(-s1.y, q0[n].y, acc[r][n][2]), y[r][n][2]);
            y[r][n][3] = fmaf(s1.x, fmaf(-s1.y, q1[n].y, acc[r][n][3]), y[r][n][3]);
          }
        }
      }
      // the slot is free again: keep the ring full (the cursor may already be in the next item)
      __syncwarp();
      ++cons;
      if (lane == 0) {
        while (prod - cons < (unsigned)NST && issue_one()) { }
      }
    }
    if (failed) break;

    // ---- item done: fragment layout -> RPL rows per lane (row = lane + 32 j) ----
    stamp(5);
    const int item = cur;
    const int n0 = item * ROWS;
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RB; ++r)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int tok = n * 8 + 2 * t;
        if (tok < m) {
          fin[(size_t)tok * ROWS + r * 16 + g] = y[r][n][0];
          fin[(size_t)tok * ROWS + r * 16 + g + 8] = y[r][n][2];
        }
        if (tok + 1 < m) {
          fin[(size_t)(tok + 1) * ROWS + r * 16 + g] = y[r][n][1];
          fin[(size_t)(tok + 1) * ROWS + r * 16 + g + 8] = y[r][n][3];
        }
      }
    __syncwarp();
    float v[RPL][MP];
#pragma unroll
    for (int j = 0; j < RPL; ++j)
#pragma unroll
      for (int tok = 0; tok < MP; ++tok) v[j][tok] = tok < m ? fin[tok * ROWS + j * 32 + lane] : 0.f;
    // Fragments of this item: workers v_first .. v_last of every slice.  Partials meet in scratch memory
    // [item][slice][fragment]; the last arriver sums them in (slice, fragment) order.
    const unsigned i_lo = (unsigned)cur * (unsigned)nb, i_hi = i_lo + (unsigned)nb - 1u;   // first / last unit of the item
    int v_first = (int)((i_lo * (unsigned)V) / U);
    while (range_lo(v_first + 1) <= i_lo) ++v_first;
    while (range_lo(v_first) > i_lo) --v_first;
    int v_last = (int)((i_hi * (unsigned)V) / U);
    while (range_lo(v_last + 1) <= i_hi) ++v_last;
    while (range_lo(v_last) > i_hi) --v_last;
    const int nfrag = v_last - v_first + 1;
    const int nparts = nfrag * ks;
    bool do_epi = true;
    if (nparts > 1) {
      const size_t fsz = (size_t)(m * ROWS);
      float* sp = a.scratch + ((size_t)item * ks) * a.fmax * fsz;
      float* mine = sp + ((size_t)slice * a.fmax + (vw - v_first)) * fsz;
#pragma unroll
      for (int j = 0; j < RPL; ++j)
#pragma unroll
        for (int tok = 0; tok < MP; ++tok)
          if (tok < m) mine[tok * ROWS + j * 32 + lane] = v[j][tok];
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      if (lane == 0) prev = atomicInc(a.counters + item, (unsigned)nparts - 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      do_epi = prev == (unsigned)nparts - 1u;
      if (do_epi) {
        __threadfence();
#pragma unroll
        for (int j = 0; j < RPL; ++j)
#pragma unroll
          for (int tok = 0; tok < MP; ++tok) {
            if (tok < m) {
              // (slice, fragment) order; eight loads in flight at a time
              float s = 0.f;
              for (int p0 = 0; p0 < nparts; p0 += 8) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int pidx = p0 + i;
                  const int sl = pidx / nfrag, f = pidx - sl * nfrag;
                  pv[i] = pidx < nparts ? __ldcg(sp + ((size_t)sl * a.fmax + f) * fsz + tok * ROWS + j * 32 + lane) : 0.f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) s += pv[i];
              }
              v[j][tok] = s;
            }
          }
      }
    }
    if (do_epi) {
#pragma unroll
      for (int j = 0; j < RPL; ++j) {
        const int row = n0 + j * 32 + lane;
        const bool row_ok = row < a.n;
        const int part = item * RPL + j;            // 32-row panel index: partial statistics are per panel
        if (a.epi == EPI_TP_RESID) {
          // push all-reduce of this panel: every rank writes its partial into every inbox, then sums its own inbox
          // in rank order once no sentinel is left
          const TpPush& tp = a.tp;
          if (row_ok) {
            if (!tp.skip_push) {
              for (int dst = 0; dst < tp.size; ++dst) {
                float* pb = tp.inbox[dst] + tp.slot_off + (size_t)tp.rank * tp.slot_stride + row;
#pragma unroll
                for (int tok = 0; tok < MP; ++tok)
                  if (tok < m) {
                    const float val = v[j][tok] + 0.f;   // -0.0 -> +0.0: the sentinel never travels as data
                    asm volatile("st.volatile.global.f32 [%0], %1;" ::"l"(pb + (size_t)tok * a.n), "f"(val) : "memory");
                  }
              }
            }
            const float* mine = tp.inbox[tp.rank] + tp.slot_off + row;
            const uint64_t t_start = globaltimer_ns();
#pragma unroll
            for (int tok = 0; tok < MP; ++tok) {
              if (tok < m) {
                float s = 0.f;
                for (int src = 0; src < tp.size; ++src) {
                  const float* pp = mine + (size_t)src * tp.slot_stride + (size_t)tok * a.n;
                  float val;
                  unsigned spins = 0;
                  bool ok;
                  while (true) {
                    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(val) : "l"(pp) : "memory");
                    ok = __float_as_uint(val) != 0x80000000u;
                    if (ok) break;
                    if ((++spins & 63u) == 0u && globaltimer_ns() - t_start > tp.timeout_ns) break;
                  }
                  if (!ok) { atomicExch(tp.status, (int)B2_ERR_TIMEOUT); val = 0.f; }
                  s += val;
                }
                v[j][tok] = s;
              }
            }
            if (tp.clear_off >= 0) {   // re-arm the slot that no rank writes before its next use
              float* clr = tp.inbox[tp.rank] + tp.clear_off + row;
              const float neg0 = __uint_as_float(0x80000000u);
              for (int src = 0; src < tp.size; ++src)
#pragma unroll
                for (int tok = 0; tok < MP; ++tok)
                  if (tok < m) clr[(size_t)src * tp.slot_stride + (size_t)tok * a.n] = neg0;
            }
          }
        }
        if (a.epi == EPI_STORE) {
#pragma unroll
          for (int tok = 0; tok < MP; ++tok)
            if (tok < m && row_ok) a.y[(size_t)tok * a.ldy + row] = __float2bfloat16_rn(v[j][tok]);
        } else if (a.epi == EPI_F32) {
#pragma unroll
          for (int tok = 0; tok < MP; ++tok)
            if (tok < m && row_ok) a.yf[(size_t)tok * a.ldy + row] = v[j][tok];
        } else if (a.epi == EPI_RESID || a.epi == EPI_TP_RESID) {
#pragma unroll
          for (int tok = 0; tok < MP; ++tok) {
            if (tok < m) {
              float sq = 0.f;
              if (row_ok) {
                const bf16 hb = __float2bfloat16_rn(v[j][tok] + __bfloat162float(a.resid[(size_t)tok * a.ldr + row]));
                a.y[(size_t)tok * a.ldy + row] = hb;
                const float hf = __bfloat162float(hb);
                sq = hf * hf;
              }
              sq = warp_sum(sq);
              if (lane == 0 && a.ss_out && part < npan) a.ss_out[(size_t)part * a.ss_ld + tok] = sq;
            }
          }
        } else if (a.epi == EPI_SWIGLU) {
          // lanes 0-7 / 16-23 hold gate rows, lanes 8-15 / 24-31 the matching up rows
#pragma unroll
          for (int tok = 0; tok < MP; ++tok) {
            if (tok < m) {
              const float up = __shfl_down_sync(0xffffffffu, v[j][tok], 8);
              if ((lane & 8) == 0 && row_ok) {
                const float gt = bf16_round(v[j][tok]);
                a.y[(size_t)tok * a.ldy + (size_t)part * 16 + (lane >> 4) * 8 + (lane & 7)] =
                    __float2bfloat16_rn(silu_f(gt) * bf16_round(up));
              }
            }
          }
        } else if (a.epi == EPI_ARGMAX) {
#pragma unroll
          for (int tok = 0; tok < MP; ++tok) {
            if (tok < m) {
              if (a.yf && row_ok) a.yf[(size_t)tok * a.ldy + row] = v[j][tok];
              float best = (row_ok && row < a.n_valid) ? v[j][tok] : -INFINITY;
              int bi = (row_ok && row < a.n_valid) ? row : 0x7fffffff;
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
              }
              if (lane == 0 && part < npan) {
                a.amax_val[(size_t)part * a.ss_ld + tok] = best;
                a.amax_idx[(size_t)part * a.ss_ld + tok] = bi;
              }
            }
          }
        }
      }
    }
   }
  }
  stamp(6);
  if (failed) {
    // Give copies still in flight a bounded chance to land before the CTA's shared memory is released.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { }
  }
}

template <int BITS, int GROUP, int RB, int NT>
static int launch_one(const WqGemvArgs& a, cudaStream_t st) {
  constexpr int MP = NT * 8;
  using R = Ring<BITS, GROUP, RB>;
  const int nbat = a.k / 128;
  const int nb_max = (nbat + a.ks - 1) / a.ks;
  const int xst = nb_max * 128 + 16;
  const size_t smem = (size_t)kGemvWarps * R::NST * R::STAGE + kGemvWarps * R::NST * 8 + 32 * 4 +
                      (size_t)kGemvWarps * a.m * RB * 16 * 4 + (size_t)a.m * xst * 2 + (size_t)nb_max * (128 / GROUP) * MP * 8;
  if (smem > 220 * 1024) return B2_ERR_ARG;
  auto kern = wq_gemv_kernel<BITS, GROUP, RB, NT>;
  static bool attr_set = false;   // one flag per instantiation
  static int sm_count = 0;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) return B2_ERR_LAUNCH;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    attr_set = true;
  }
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kGemvThreads, smem) != cudaSuccess || occ < 1) return B2_ERR_LAUNCH;
  static const int occ_cap = [] { const char* e = getenv("B200E_GEMV_OCC"); return e ? atoi(e) : 0; }();
  if (occ_cap > 0 && occ > occ_cap) occ = occ_cap;   // fewer resident CTAs leave room for the next kernel's prefetching CTAs
  const int npan = a.n / 32;
  const int nitems = (npan + RB / 2 - 1) / (RB / 2);
  // persistent grid of (CTAs per slice) x ks CTAs: every SM carries the same number of CTAs
  long cps = ((long)sm_count * occ) / a.ks;
  if (cps < 1) cps = 1;
  const long vcps = (a.vworkers + kGemvWarps - 1) / kGemvWarps;
  if (cps > vcps) cps = vcps;                                                     // never more warps than workers
  const long grid = cps * a.ks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
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
  if (nt == 1) return launch_one<BITS, GROUP, 2, 1>(a, st);
  if (nt == 2) return launch_one<BITS, GROUP, 2, 2>(a, st);
  if (nt <= 4) return launch_one<BITS, GROUP, 2, 4>(a, st);
  return B2_ERR_ARG;
}

}  // namespace b2

using namespace b2;

// Virtual workers per slice and the most fragments an item can be cut into, both functions of the shape only.
// kVirtualCtas is the resident-CTA count the schedule is laid out for (2 per SM on a 148-SM part).
static const int kVirtualCtas = 296;
B2_API int b2_wq_gemv_vworkers(int n, int k, int ks, int rb) {
  const long nitems = (n / 32 + rb / 2 - 1) / (rb / 2);
  const long U = nitems * (k / 128 / ks);
  long V = (long)(kVirtualCtas / ks) * kGemvWarps;
  if (V < 1) V = 1;
  // Small matrices: a worker owns at least kMinUnits (item, batch) units, so an item is cut into fewer fragments and
  // the hand-off (scratch round trip + ordered sum by the last arriver) stays short.  Shape-only, like everything here.
  static const long kMinUnits = [] { const char* e = getenv("B200E_GEMV_MIN_UNITS"); return e ? atol(e) : 4L; }();
  if (V > U / kMinUnits) V = U / kMinUnits;
  if (V < 1) V = 1;
  return (int)V;
}
B2_API int b2_wq_gemv_fmax(int n, int k, int ks, int rb) {
  const long nitems = (n / 32 + rb / 2 - 1) / (rb / 2);
  const long nb = k / 128 / ks;
  const long U = nitems * nb;
  const long V = b2_wq_gemv_vworkers(n, k, ks, rb);
  const long per = U / V;                       // every worker owns per or per + 1 units
  return (int)((nb + per - 1) / per + 1);
}
// Scratch floats for the split partials: [item][ks][fmax][m][rows per item].
B2_API long b2_wq_gemv_scratch_floats(int n, int k, int ks, int rb, int m) {
  const long nitems = (n / 32 + rb / 2 - 1) / (rb / 2);
  return nitems * ks * b2_wq_gemv_fmax(n, k, ks, rb) * (long)m * rb * 16;
}

// Launches the GEMV described by *args on `stream`.  Returns a b2::Status; nothing is launched on B2_ERR_ARG.
// Rows 17..32 tokens always use 32-row items (register budget), whatever args->rb says; per-row results do not
// depend on rb, because the k range and summation order of a row are fixed by (k, ks) alone.
B2_API int b2_wq_gemv(const WqGemvArgs* args, cudaStream_t stream) {
  const WqGemvArgs& a = *args;
  if (a.n <= 0 || a.k <= 0 || a.m <= 0 || a.m > 32) return B2_ERR_ARG;
  if (a.n % 32 || a.k % 128 || a.ks < 1 || a.ks > kMaxKs || a.ks > a.k / 128) return B2_ERR_ARG;
  if (a.group != 64 && a.group != 128) return B2_ERR_ARG;
  if (a.rb != 2 && a.rb != 4) return B2_ERR_ARG;
  if (!a.scratch || !a.counters) return B2_ERR_ARG;
  if (a.k / 128 % a.ks) return B2_ERR_ARG;
  if ((double)a.vworkers * (double)(a.n / 32) * (double)(a.k / 128 / a.ks) >= 4.0e9) return B2_ERR_ARG;   // 32-bit schedule arithmetic
  if (a.vworkers != b2_wq_gemv_vworkers(a.n, a.k, a.ks, a.rb) || a.fmax != b2_wq_gemv_fmax(a.n, a.k, a.ks, a.rb)) return B2_ERR_ARG;
  if ((a.ldx % 8) || (reinterpret_cast<uintptr_t>(a.x) & 15)) return B2_ERR_ARG;
  if (a.epi == EPI_TP_RESID && (a.tp.size < 1 || a.tp.size > kMaxTp)) return B2_ERR_ARG;
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
