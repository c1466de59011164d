// Persistent decode-step kernel, sm_100a: ONE cooperative launch runs a whole decode / verify step of the dense GQA
// decoder -- embedding, every layer (qkv, RoPE + KV store, paged attention, o_proj, gate/up, SwiGLU, down_proj), the
// lm_head and the argmax -- for up to eight token rows, on one GPU or on every GPU of a tensor-parallel group.
//
// The reference runs a step as a CUDA graph of several kernels per layer with programmatic-dependent-launch edges
// (kernels/m1/m1_model.cu:2544-2596 `layer`, :3071-3140 decode graphs, kernels/src/runtime.cu:198-228) and folds
// the tensor-parallel all-reduce into its push kernels (kernels/src/tp_ar.cu:160-227).  On a 148-SM part a step of
// the 32B model is bound by the ~450 kernel boundaries, not by the weights, so here the boundaries disappear:
//
//   * one CTA of 16 warps per SM stays resident for the whole step; phases are separated by grid barriers (one
//     release-add and a bounded acquire-poll per CTA), tensor-parallel phases by the same barrier across GPUs
//     (release-adds into every peer's counter over NVLink);
//   * every warp streams its statically known share of ALL the step's weights through a private cp.async.bulk ring
//     whose producer runs ahead across phase boundaries: while a barrier or the attention phase is in progress the
//     next linear's weights are already in flight or in shared memory;
//   * a linear is cut by contiguous block ranges over the CTAs (stream-k); the 16 warps of a CTA share one row panel
//     at a time and combine their k ranges through shared memory; a panel cut by a CTA boundary leaves one partial per
//     fragment in global memory.  The consumer ("finalize") stage adds the fragments in a fixed order and applies
//     what the reference does in separate kernels: RoPE + KV store, the split merge of attention, residual add,
//     SwiGLU, argmax;
//   * row-parallel linears under tensor parallelism write their fragments straight into every peer's exchange region
//     (plain stores over NVLink) and the finalize stage of every rank adds all ranks' fragments in rank order: the
//     GEMV -> all-reduce -> residual add -> next norm path is one kernel with no library collective.
//
// Batch invariance: the k range, the fragment cut and every summation order depend on the linear's shape and on the
// number of CTAs only, never on the number of rows; attention uses the fixed-size KV splits of attn_decode.cu.  A row
// of a verify block is therefore bit-identical to the same row of a plain decode step.
#include "step_kernel.cuh"
#include "wq_frag.cuh"

namespace b2 {
namespace {

constexpr int kRingBytes = 7168;           // weight bytes in flight per warp
constexpr int kRingBars = 16;              // units in flight per warp
constexpr int kRedTok = 20;                // floats between the token rows of a warp's partial tile (conflict-free)
constexpr int kRedWarp = kStepMaxRows * kRedTok;
constexpr int kAttnWarps = 6;              // warps of a CTA that run attention items (two 8 KB K/V stages each)
constexpr int kPage = 16;

constexpr int SM_RING = 0;
constexpr int SM_BARS = SM_RING + kStepWarps * kRingBytes;
constexpr int SM_MISC = SM_BARS + kStepWarps * kRingBars * 8;
constexpr int SM_MISC_BYTES = 2048;
constexpr int SM_WORK = SM_MISC + SM_MISC_BYTES;
constexpr int SM_XS_BYTES = kStepMaxRows * (kStepSliceK + 16) * 2;
constexpr int SM_GSUM = SM_WORK + SM_XS_BYTES;
constexpr int SM_GSUM_BYTES = (kStepSliceK / 128) * 2 * kStepMaxRows * 8;
constexpr int SM_RED = SM_GSUM + SM_GSUM_BYTES;
constexpr int SM_RED_BYTES = 2 * kStepWarps * kRedWarp * 4;
constexpr int SM_TOTAL = SM_RED + SM_RED_BYTES;
static_assert(kAttnWarps * 2 * 2 * kPage * 128 * 2 <= SM_TOTAL - SM_WORK, "attention stages alias the GEMV work area");
static_assert(SM_TOTAL <= 227 * 1024, "shared memory of one CTA");

// misc area (floats): [0,8) inv_rms, [8,136) per-warp sums, [136,264) argmax values, [264,392) argmax indices,
// [392,424) row description (ids, pos, seq, rope position)
constexpr int MI_WSUM = 8, MI_AV = 136, MI_AI = 264, MI_ROW = 392;

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
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

// ---------------------------------------------------------------------------------------------------- barriers
struct SyncState {
  unsigned local_target, cross_target;   // arrival counts the next barrier waits for (thread 0 of every CTA)
};

// Grid barrier.  Every CTA adds one to the counter with release semantics after its threads met at bar.sync, then
// polls with acquire loads until all CTAs of this epoch arrived.  The poll is bounded: on expiry (or when another
// wait already failed) the status word is set and the kernel runs to its end without waiting again.
__device__ __forceinline__ void grid_sync(const StepArgs& a, SyncState& ss) {
  __syncthreads();
  if (threadIdx.x == 0) {
    ss.local_target += gridDim.x;
    __threadfence();
    red_release_gpu(a.sync, 1u);
    if (ld_volatile_i32(a.status) == 0) {
      const uint64_t t0 = globaltimer_ns();
      unsigned spins = 0;
      while ((int)(ld_acquire_gpu(a.sync) - ss.local_target) < 0) {
        if ((++spins & 63u) == 0u) {
          if (ld_volatile_i32(a.status) != 0) break;
          if (globaltimer_ns() - t0 > a.timeout_ns) { atomicExch(a.status, (int)B2_ERR_TIMEOUT); break; }
        }
      }
    }
  }
  __syncthreads();
}

// The same barrier over all CTAs of all tensor-parallel ranks: one release-add into every rank's counter (word 0 of
// its exchange region), then a poll of the own counter.  With one rank it is the grid barrier.
__device__ __forceinline__ void cross_sync(const StepArgs& a, SyncState& ss) {
  if (a.tp_size <= 1) { grid_sync(a, ss); return; }
  __syncthreads();
  if (threadIdx.x == 0) {
    ss.cross_target += gridDim.x * (unsigned)a.tp_size;
    __threadfence_system();
    if (!a.skip_push)
      for (int r = 0; r < a.tp_size; ++r) red_release_sys(reinterpret_cast<unsigned*>(a.xreg[r]), 1u);
    if (ld_volatile_i32(a.status) == 0) {
      const unsigned* own = reinterpret_cast<const unsigned*>(a.xreg[a.tp_rank]);
      const uint64_t t0 = globaltimer_ns();
      unsigned spins = 0;
      while ((int)(ld_acquire_sys(own) - ss.cross_target) < 0) {
        if ((++spins & 63u) == 0u) {
          if (ld_volatile_i32(a.status) != 0) break;
          if (globaltimer_ns() - t0 > a.timeout_ns) { atomicExch(a.status, (int)B2_ERR_TIMEOUT); break; }
        }
      }
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------------- work split
struct Phase {
  StepLinear lin;
  int slice, ci;
  int bs0, nbs;          // first batch and batch count of this CTA's k slice
  unsigned lo, hi;       // this CTA's range of (panel, batch) blocks inside the slice, panel-major
  bool active;
};

// Field-wise copy of a StepLinear from global memory (four 16-byte loads; keeps the copy in registers).
__device__ __forceinline__ void fetch_linear(const StepLinear* src, StepLinear& L) {
  static_assert(sizeof(StepLinear) == 64, "StepLinear is read as four 16-byte words");
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  const uint4 a0 = __ldg(s4), a1 = __ldg(s4 + 1), a2 = __ldg(s4 + 2), a3 = __ldg(s4 + 3);
  L.wq = reinterpret_cast<const uint8_t*>(((unsigned long long)a0.y << 32) | (unsigned long long)a0.x);
  L.n = (int)a0.z; L.k = (int)a0.w;
  L.bits = (int)a1.x; L.group = (int)a1.y; L.npan = (int)a1.z; L.nbat = (int)a1.w;
  L.wbatch = (int)a2.x; L.szb = (int)a2.y; L.blk = (int)a2.z; L.ks = (int)a2.w;
  L.cps = (int)a3.x; L.fmax = (int)a3.y; L.pad = 0;
}

__device__ __forceinline__ void load_linear(const StepArgs& a, int phase, StepLinear& L) {
  if (phase >= 4 * a.n_layers) { L = a.lm_head; return; }
  const StepLayer* ly = a.layers + (phase >> 2);
  const int j = phase & 3;
  const StepLinear* src = j == 0 ? &ly->qkv : (j == 1 ? &ly->o : (j == 2 ? &ly->gate_up : &ly->down));
  fetch_linear(src, L);
}

__device__ __forceinline__ void split_phase(Phase& ph, int cta) {
  const StepLinear& L = ph.lin;
  ph.slice = cta / L.cps;
  ph.ci = cta - ph.slice * L.cps;
  ph.active = ph.slice < L.ks;
  ph.bs0 = 0; ph.nbs = 0; ph.lo = 0; ph.hi = 0;
  if (!ph.active) return;
  ph.bs0 = (L.nbat * ph.slice) / L.ks;
  ph.nbs = (L.nbat * (ph.slice + 1)) / L.ks - ph.bs0;
  const unsigned long long B = (unsigned long long)L.npan * (unsigned)ph.nbs;
  ph.lo = (unsigned)((B * (unsigned)ph.ci) / (unsigned)L.cps);
  ph.hi = (unsigned)((B * (unsigned)(ph.ci + 1)) / (unsigned)L.cps);
}

// Producer cursor of one warp (held by lane 0): walks the warp's units of every remaining linear of the step in the
// order the consumer will use them.  Warp w of a CTA takes row block (w & 1) of the batches b_lo + (w >> 1) + 8 i of
// every panel segment of the CTA's range.
struct Cursor {
  int phase, n_phases;
  Phase ph;
  unsigned p;
  int b, b_hi;
};

__device__ __forceinline__ void cursor_settle(Cursor& c, const StepArgs& a, int cta, int warp, bool fresh) {
  // `fresh`: c.ph was just loaded for c.phase and no segment is selected yet
  while (c.phase < c.n_phases) {
    if (fresh) {
      if (!c.ph.active || c.ph.lo >= c.ph.hi) {
        ++c.phase;
        if (c.phase < c.n_phases) { load_linear(a, c.phase, c.ph.lin); split_phase(c.ph, cta); }
        continue;
      }
      c.p = c.ph.lo / (unsigned)c.ph.nbs;
      const int b_lo = (int)(c.ph.lo - c.p * (unsigned)c.ph.nbs);
      c.b_hi = (int)min(c.ph.hi - c.p * (unsigned)c.ph.nbs, (unsigned)c.ph.nbs);
      c.b = b_lo + (warp >> 1);
      fresh = false;
    }
    if (c.b < c.b_hi) return;
    ++c.p;
    if (c.p * (unsigned)c.ph.nbs >= c.ph.hi) {
      ++c.phase;
      if (c.phase < c.n_phases) { load_linear(a, c.phase, c.ph.lin); split_phase(c.ph, cta); }
      fresh = true;
      continue;
    }
    c.b_hi = (int)min(c.ph.hi - c.p * (unsigned)c.ph.nbs, (unsigned)c.ph.nbs);
    c.b = warp >> 1;
  }
}

struct WRing {
  uint32_t base_u, bars_u;
  uint8_t* base;
  unsigned pidx, cidx;     // units issued (lane 0) / consumed (all lanes)
  int ppos, pfree;         // producer byte position and free bytes (lane 0)
  int cpos;                // consumer byte position (all lanes)
};

// Lane 0: issue bulk copies while the ring has room.
__device__ __forceinline__ void pump(WRing& r, Cursor& c, const StepArgs& a, int cta, int warp) {
  while (c.phase < c.n_phases) {
    const StepLinear& L = c.ph.lin;
    const int usz = L.wbatch + L.szb;
    if (r.pidx - r.cidx >= (unsigned)kRingBars) break;
    int pos = r.ppos, need = usz;
    if (pos + usz > kRingBytes) { need += kRingBytes - pos; pos = 0; }
    if (r.pfree < need) break;
    r.pfree -= need;
    const uint32_t bar = r.bars_u + (r.pidx % kRingBars) * 8;
    mbar_expect_tx(bar, (uint32_t)usz);
    const uint8_t* blkp = L.wq + ((size_t)c.p * L.nbat + (size_t)(c.ph.bs0 + c.b)) * L.blk;
    const int rb = warp & 1;
    bulk_g2s(r.base_u + pos, blkp + rb * L.wbatch, (uint32_t)L.wbatch, bar);
    bulk_g2s(r.base_u + pos + L.wbatch, blkp + 2 * L.wbatch + rb * L.szb, (uint32_t)L.szb, bar);
    r.ppos = pos + usz;
    ++r.pidx;
    c.b += 8;
    cursor_settle(c, a, cta, warp, false);
  }
}

// ---------------------------------------------------------------------------------------------------- GEMV phase
// One linear: stage this CTA's activation slice (optionally RMS-normalised) as fp16(x / c) with the per-group sums,
// then walk the panel segments of the CTA's block range.  Partial rows go to `a.part` (tp_off < 0) or into every
// rank's exchange region at float offset tp_off.
template <int BITS, int GROUP>
__device__ __forceinline__ void gemv_body(const StepArgs& a, const Phase& ph, uint8_t* smem, WRing& ring, Cursor& cur,
                                          const bf16* x, long ldx, const bf16* norm_w, long tp_off, bool& failed) {
  constexpr int GPB = 128 / GROUP;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;
  const int R = a.n_rows;
  const StepLinear& L = ph.lin;
  const int nbs = ph.nbs;
  const int XST = nbs * 128 + 16;
  __half* xs = reinterpret_cast<__half*>(smem + SM_WORK);
  float2* gsum = reinterpret_cast<float2*>(smem + SM_GSUM);
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
  float* inv_rms = misc;
  float* wsum = misc + MI_WSUM;

  if (norm_w) {
    const int nv = L.k >> 3;
    for (int tok = 0; tok < R; ++tok) {
      float s = 0.f;
      for (int v = tid; v < nv; v += kStepThreads) {
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)tok * ldx) + v);
        const bf16* xb = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float f = __bfloat162float(xb[i]); s = fmaf(f, f, s); }
      }
      s = warp_sum(s);
      if (lane == 0) wsum[tok * kStepWarps + warp] = s;
    }
    __syncthreads();
    if (tid < R) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kStepWarps; ++w) s += wsum[tid * kStepWarps + w];
      inv_rms[tid] = rsqrtf(s / (float)L.k + a.eps);
    }
    __syncthreads();
  }
  if (ph.active && nbs > 0) {
    const int nvec = nbs * 16;
    const int k0 = ph.bs0 * 128;
    for (int tok = 0; tok < R; ++tok) {
      for (int v0 = 0; v0 < nvec; v0 += kStepThreads) {
        const int v = v0 + tid;
        const bool act = v < nvec;
        float ssum = 0.f, xsum = 0.f;
        if (act) {
          const int k = k0 + v * 8;
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + k));
          const bf16* xb = reinterpret_cast<const bf16*>(&raw);
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(xb[i]);
          if (norm_w) {
            const uint4 wr = __ldg(reinterpret_cast<const uint4*>(norm_w + k));
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
#pragma unroll
        for (int o = GROUP / 16; o > 0; o >>= 1) {
          ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
          xsum += __shfl_xor_sync(0xffffffffu, xsum, o);
        }
        if (act && (lane % (GROUP / 8)) == 0) gsum[((v * 8) / GROUP) * kStepMaxRows + tok] = make_float2(1024.f * ssum, xsum);
      }
    }
  }
  __syncthreads();
  if (!ph.active) return;

  const unsigned Bsl = (unsigned)L.npan * (unsigned)nbs;
  const int nslots = L.ks * L.fmax;
  unsigned blk = ph.lo;
  int seg = 0;
  const int usz = L.wbatch + L.szb;
  while (blk < ph.hi) {
    const unsigned p = blk / (unsigned)nbs;
    const int b_lo = (int)(blk - p * (unsigned)nbs);
    const int b_hi = (int)min(ph.hi - p * (unsigned)nbs, (unsigned)nbs);
    float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int b = b_lo + (warp >> 1); b < b_hi; b += 8) {
      int freed = usz;
      if (ring.cpos + usz > kRingBytes) { freed += kRingBytes - ring.cpos; ring.cpos = 0; }
      if (!failed) {
        if (!mbar_wait_bounded(ring.bars_u + (ring.cidx % kRingBars) * 8, (ring.cidx / kRingBars) & 1u)) {
          atomicExch(a.status, (int)B2_ERR_TIMEOUT);
          failed = true;
        }
      }
      if (!failed) {
        const uint8_t* stg = ring.base + ring.cpos;
        WFrag<BITS, GROUP> cf;
        load_frag_smem<BITS, GROUP>(cf, stg, stg + L.wbatch, lane);
        const __half* xrow = xs + b * 128 + t * 4;
#pragma unroll
        for (int gg = 0; gg < GPB; ++gg) {
          const int gi = b * GPB + gg;
          const float2 q0 = gsum[gi * kStepMaxRows + 2 * t];
          const float2 q1 = gsum[gi * kStepMaxRows + 2 * t + 1];
          float acc[4] = {-q0.x, -q1.x, -q0.x, -q1.x};
#pragma unroll
          for (int s8 = 0; s8 < 8 / GPB; ++s8) {
            const int s = gg * (8 / GPB) + s8;
            uint2 bv = make_uint2(0u, 0u);
            if (g < R) bv = *reinterpret_cast<const uint2*>(xrow + (size_t)g * XST + s * 16);
            uint32_t af[4];
            extract<BITS, GROUP>(cf, s, af);
            mma_f16_16816(acc, af, bv.x, bv.y);
          }
          const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&cf.sz[gg][0]));
          const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&cf.sz[gg][1]));
          y[0] = fmaf(s0.x, fmaf(-s0.y, q0.y, acc[0]), y[0]);
          y[1] = fmaf(s0.x, fmaf(-s0.y, q1.y, acc[1]), y[1]);
          y[2] = fmaf(s1.x, fmaf(-s1.y, q0.y, acc[2]), y[2]);
          y[3] = fmaf(s1.x, fmaf(-s1.y, q1.y, acc[3]), y[3]);
        }
      }
      __syncwarp();
      ++ring.cidx;
      ring.cpos += usz;
      if (lane == 0) {
        ring.pfree += freed;
        if (!failed) pump(ring, cur, a, cta, warp);
      }
    }
    // the 16 warps' tiles of this segment meet in shared memory; eight warps carry each 16-row block
    float* red = reinterpret_cast<float*>(smem + SM_RED) + (seg & 1) * kStepWarps * kRedWarp;
    {
      float* mine = red + warp * kRedWarp;
      mine[(2 * t) * kRedTok + g] = y[0];
      mine[(2 * t + 1) * kRedTok + g] = y[1];
      mine[(2 * t) * kRedTok + g + 8] = y[2];
      mine[(2 * t + 1) * kRedTok + g + 8] = y[3];
    }
    __syncthreads();
    if (tid < 256) {
      const int row = tid & 31, tok = tid >> 5;
      if (tok < R) {
        const int rb = row >> 4, r16 = row & 15;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += red[(2 * j + rb) * kRedWarp + tok * kRedTok + r16];
        // fragment index of this CTA inside the panel = CTAs since the one that owns the panel's first block
        const unsigned first_owner = (((p * (unsigned)nbs) + 1u) * (unsigned)L.cps - 1u) / Bsl;
        const int f = ph.ci - (int)first_owner;
        const int f_end = (b_hi == nbs) ? L.fmax : f + 1;     // the last fragment also zeroes the unused slots
        const size_t col = (size_t)p * 32 + row;
        for (int ff = f; ff < f_end; ++ff) {
          const float val = ff == f ? s : 0.f;
          const size_t off = ((size_t)(ph.slice * L.fmax + ff) * R + tok) * L.n + col;
          if (tp_off < 0) {
            a.part[off] = val;
          } else {
            const size_t roff = (size_t)tp_off + (size_t)a.tp_rank * nslots * R * L.n + off;
            for (int d = 0; d < a.tp_size; ++d) a.xreg[d][roff] = val;
          }
        }
      }
    }
    blk = p * (unsigned)nbs + (unsigned)b_hi;
    ++seg;
  }
}

__device__ __forceinline__ void gemv_phase(const StepArgs& a, int phase, uint8_t* smem, WRing& ring, Cursor& cur,
                                           const bf16* x, long ldx, const bf16* norm_w, long tp_off, bool& failed) {
  Phase ph;
  load_linear(a, phase, ph.lin);
  split_phase(ph, blockIdx.x);
  switch (ph.lin.bits * 1000 + ph.lin.group) {
    case 4128: gemv_body<4, 128>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
    case 4064: gemv_body<4, 64>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
    case 3128: gemv_body<3, 128>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
    case 3064: gemv_body<3, 64>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
    case 2128: gemv_body<2, 128>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
    default: gemv_body<2, 64>(a, ph, smem, ring, cur, x, ldx, norm_w, tp_off, failed); break;
  }
}

// Sum of the fragments of output element (tok, col) of a linear, in (rank,) slice, fragment order.
__device__ __forceinline__ float sum_local(const StepArgs& a, const StepLinear& L, int tok, size_t col) {
  const int nslots = L.ks * L.fmax, R = a.n_rows;
  float s = 0.f;
  for (int sl = 0; sl < nslots; ++sl) s += __ldcg(a.part + ((size_t)sl * R + tok) * L.n + col);
  return s;
}
__device__ __forceinline__ float2 sum_local2(const StepArgs& a, const StepLinear& L, int tok, size_t col) {
  const int nslots = L.ks * L.fmax, R = a.n_rows;
  float2 s = make_float2(0.f, 0.f);
  for (int sl = 0; sl < nslots; ++sl) {
    const float2 v = __ldcg(reinterpret_cast<const float2*>(a.part + ((size_t)sl * R + tok) * L.n + col));
    s.x += v.x; s.y += v.y;
  }
  return s;
}

// ---------------------------------------------------------------------------------------------------- finalize stages
// h = embedding rows of the step's tokens
__device__ __forceinline__ void fin_embed(const StepArgs& a, const int* row_ids) {
  const int nv = a.d_model >> 3;
  const int total = a.n_rows * nv;
  for (int e = blockIdx.x * kStepThreads + threadIdx.x; e < total; e += gridDim.x * kStepThreads) {
    const int tok = e / nv, v = e - tok * nv;
    int id = row_ids[tok];
    if (id < 0 || id >= a.vocab) { atomicExch(a.status, (int)B2_ERR_BOUNDS); id = 0; }
    reinterpret_cast<uint4*>(a.h + (size_t)tok * a.d_model)[v] = __ldg(reinterpret_cast<const uint4*>(a.embed + (size_t)id * a.d_model) + v);
  }
}

// qkv fragments -> bf16 row -> RoPE on q and k -> q buffer / paged KV store.  One warp per (row, head).
__device__ __forceinline__ void fin_qkv(const StepArgs& a, const StepLayer* ly, const int* row_pos, const int* row_seq,
                                        const int* row_rope) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const StepLinear& L = ly->qkv;
  StepLinear Lc;
  fetch_linear(&L, Lc);
  bf16* kv_pool = ly->kv_pool;
  const int heads = a.hq + 2 * a.hkv;
  const int items = a.n_rows * heads;
  for (int it = warp * gridDim.x + blockIdx.x; it < items; it += gridDim.x * kStepWarps) {
    const int tok = it / heads, head = it - tok * heads;
    const int i = lane * 2;
    const size_t c0 = (size_t)head * 128 + i;
    float2 lo = sum_local2(a, Lc, tok, c0);
    float2 hi = sum_local2(a, Lc, tok, c0 + 64);
    lo.x = bf16_round(lo.x); lo.y = bf16_round(lo.y); hi.x = bf16_round(hi.x); hi.y = bf16_round(hi.y);
    const int pos = row_pos[tok];
    bf16* dst;
    if (head < a.hq) {
      dst = a.q + (size_t)tok * a.hq * 128 + (size_t)head * 128;
    } else {
      const int seq = row_seq[tok];
      const int page = a.block_table[(size_t)seq * a.bt_ld + pos / kPage];
      if (page < 0 || page >= a.n_pages) { if (lane == 0) atomicExch(a.status, (int)B2_ERR_BOUNDS); continue; }
      const int is_v = head >= a.hq + a.hkv;
      const int kvh = head - a.hq - (is_v ? a.hkv : 0);
      dst = kv_pool + ((((size_t)page * 2 + is_v) * a.hkv + kvh) * kPage + (pos % kPage)) * 128;
      if (is_v) {
        *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(lo.x, lo.y);
        *reinterpret_cast<__nv_bfloat162*>(dst + i + 64) = __floats2bfloat162_rn(hi.x, hi.y);
        continue;
      }
    }
    const int rpos = row_rope[tok];
    float s0, c0f, s1, c1f;
    sincosf((float)rpos * a.inv_freq[i], &s0, &c0f);
    sincosf((float)rpos * a.inv_freq[i + 1], &s1, &c1f);
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(lo.x * c0f - hi.x * s0, lo.y * c1f - hi.y * s1);
    *reinterpret_cast<__nv_bfloat162*>(dst + i + 64) = __floats2bfloat162_rn(hi.x * c0f + lo.x * s0, hi.y * c1f + lo.y * s1);
  }
}

// h = bf16(h + sum of the fragments of a row-parallel linear over all ranks)
__device__ __forceinline__ void fin_resid(const StepArgs& a, const StepLinear* Lg, long tp_off) {
  StepLinear L;
  fetch_linear(Lg, L);
  const int n = L.n, R = a.n_rows, nslots = L.ks * L.fmax;
  const int total = R * n;
  const float* own = tp_off >= 0 ? a.xreg[a.tp_rank] + tp_off : nullptr;
  for (int e = blockIdx.x * kStepThreads + threadIdx.x; e < total; e += gridDim.x * kStepThreads) {
    const int tok = e / n, c = e - tok * n;
    float s = 0.f;
    if (tp_off < 0) {
      s = sum_local(a, L, tok, (size_t)c);
    } else {
      for (int r = 0; r < a.tp_size; ++r)
        for (int sl = 0; sl < nslots; ++sl)
          s += __ldcg(own + (((size_t)r * nslots + sl) * R + tok) * n + c);
    }
    bf16* hp = a.h + (size_t)tok * a.d_model + c;
    const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(hp));
    *hp = __float2bfloat16_rn(s + __bfloat162float(__ushort_as_bfloat16(raw)));
  }
}

// act = bf16(silu(bf16 gate) * bf16 up); gate / up rows are interleaved in blocks of 8 inside every 16-row block
__device__ __forceinline__ void fin_swiglu(const StepArgs& a, const StepLinear* Lg) {
  StepLinear L;
  fetch_linear(Lg, L);
  const int f = L.n >> 1, R = a.n_rows;
  const int total = R * f;
  for (int e = blockIdx.x * kStepThreads + threadIdx.x; e < total; e += gridDim.x * kStepThreads) {
    const int tok = e / f, j = e - tok * f;
    const size_t grow = (size_t)(j >> 3) * 16 + (j & 7);
    const float gt = bf16_round(sum_local(a, L, tok, grow));
    const float up = bf16_round(sum_local(a, L, tok, grow + 8));
    a.act[(size_t)tok * f + j] = __float2bfloat16_rn(silu_f(gt) * up);
  }
}

// One attention work item (query group, kv head, 16-row tile, kv split) on one warp; the arithmetic of
// attn_decode_kernel<128, false> (attn_decode.cu) with a two-stage K/V ring in this warp's shared memory.
__device__ __forceinline__ void attn_item(const StepArgs& a, const bf16* kv_pool, long item, uint8_t* wsm, const int* row_pos,
                                       const int* row_seq) {
  constexpr int HD = 128, KS = HD / 16, NTO = HD / 8, ROWB = HD * 2, CPR = ROWB / 16, PAGE_B = kPage * ROWB, ST = 2;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int gq = a.hq / a.hkv;
  const int mt_max = (8 * gq + 15) / 16;
  const int split = (int)(item % a.max_splits); item /= a.max_splits;
  const int mtile = (int)(item % mt_max); item /= mt_max;
  const int kvh = (int)(item % a.hkv); item /= a.hkv;
  const int grp = (int)item;
  const int tok0 = a.grp_tok0[grp], cnt = a.grp_cnt[grp];
  if (mtile * 16 >= cnt * gq) return;
  const int seq = row_seq[tok0];
  const int pos_first = row_pos[tok0];
  const int kv_len = row_pos[tok0 + cnt - 1] + 1;
  const int k_begin = split * a.split_keys;
  if (k_begin >= kv_len) return;
  const int k_end = min(kv_len, k_begin + a.split_keys);
  const int n_pg = (k_end - k_begin + kPage - 1) / kPage;

  int rtok[2], rhead[2], rpos[2];
  bool rvalid[2];
  unsigned rmask[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int Rr = mtile * 16 + g + 8 * i;
    const int tl = Rr / gq;
    rvalid[i] = tl < cnt;
    rtok[i] = tok0 + (rvalid[i] ? tl : 0);
    rhead[i] = kvh * gq + (Rr % gq);
    rpos[i] = rvalid[i] ? row_pos[rtok[i]] : -1;
    rmask[i] = (a.tree_mask && rvalid[i]) ? a.tree_mask[rtok[i]] : 0xffffffffu;
  }
  const uint32_t wsm_u = smem_u32(wsm);
  const int* bt = a.block_table + (size_t)seq * a.bt_ld;

  auto issue_page = [&](int pi) {
    const int stage = pi % ST;
    int page = bt[(k_begin / kPage) + pi];
    if (page < 0 || page >= a.n_pages) { atomicExch(a.status, (int)B2_ERR_BOUNDS); page = 0; }
    const uint8_t* kp = reinterpret_cast<const uint8_t*>(kv_pool) + (((size_t)page * 2 + 0) * a.hkv + kvh) * PAGE_B;
    const uint8_t* vp = reinterpret_cast<const uint8_t*>(kv_pool) + (((size_t)page * 2 + 1) * a.hkv + kvh) * PAGE_B;
    const uint32_t ks = wsm_u + stage * 2 * PAGE_B, vs = ks + PAGE_B;
#pragma unroll
    for (int c = lane; c < kPage * CPR; c += 32) {
      const int row = c / CPR, cc = c % CPR;
      const uint32_t off = row * ROWB + ((cc ^ (row & 7)) << 4);
      cp_async16(ks + off, kp + (size_t)c * 16);
      cp_async16(vs + off, vp + (size_t)c * 16);
    }
  };
  if (0 < n_pg) issue_page(0);
  cp_async_commit();

  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t v0 = 0u, v1 = 0u;
      if (rvalid[i]) {
        const bf16* qp = a.q + (size_t)rtok[i] * a.hq * HD + (size_t)rhead[i] * HD + ks * 16 + 2 * t;
        v0 = __ldcg(reinterpret_cast<const unsigned*>(qp));
        v1 = __ldcg(reinterpret_cast<const unsigned*>(qp + 8));
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
    if (pi + 1 < n_pg) issue_page(pi + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
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
    const int kb = k_begin + pi * kPage;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i >> 1;
        const int key = kb + n * 8 + 2 * t + (i & 1);
        bool ok = key <= rpos[r];
        if (ok && key >= pos_first) ok = (rmask[r] >> (key - pos_first)) & 1u;
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
    __syncwarp();
  }
  cp_async_wait<0>();
  __syncwarp();
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

__device__ __forceinline__ void attn_phase(const StepArgs& a, const bf16* kv_pool, uint8_t* smem, const int* row_pos,
                                           const int* row_seq) {
  const int warp = threadIdx.x >> 5;
  if (warp >= kAttnWarps) return;
  const int gq = a.hq / a.hkv;
  const int mt_max = (8 * gq + 15) / 16;
  // splits that any row of this step can reach
  int max_pos = 0;
  for (int i = 0; i < a.n_rows; ++i) max_pos = max(max_pos, row_pos[i]);
  const int n_sp = min(a.max_splits, max_pos / a.split_keys + 1);
  const long per_grp = (long)a.hkv * mt_max;
  const long items = (long)a.n_groups * per_grp * n_sp;
  uint8_t* wsm = smem + SM_WORK + (size_t)warp * 2 * 2 * kPage * 128 * 2;
  for (long it = (long)warp * gridDim.x + blockIdx.x; it < items; it += (long)gridDim.x * kAttnWarps) {
    // item order: split fastest, so that the items of one (group, head) spread over the CTAs
    const long outer = it / n_sp;
    const int split = (int)(it - outer * n_sp);
    attn_item(a, kv_pool, outer * a.max_splits + split, wsm, row_pos, row_seq);
  }
}

// Merge of the attention splits of every (row, q head); the order of additions of attn_merge_kernel<128, 1>.
__device__ __forceinline__ void fin_merge(const StepArgs& a, const int* row_pos) {
  constexpr int HD = 128, PER = HD / 32, SETS = 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = a.n_rows * a.hq;
  for (int item = warp * gridDim.x + blockIdx.x; item < items; item += gridDim.x * kStepWarps) {
    const int tok = item / a.hq, head = item - tok * a.hq;
    const int ns = (row_pos[tok] + a.split_keys) / a.split_keys;
    const float* po = a.part_o + ((size_t)tok * a.hq + head) * a.max_splits * HD;
    const float2* pm = reinterpret_cast<const float2*>(a.part_ml + ((size_t)tok * a.hq + head) * a.max_splits * 2);
    float M = -INFINITY;
    for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(pm + s).x);
    M = warp_max(M);
    float acc[SETS][PER], Lw[SETS];
#pragma unroll
    for (int w = 0; w < SETS; ++w) {
      Lw[w] = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[w][i] = 0.f;
    }
    for (int blk = 0; blk * 8 < ns; ++blk) {
      const int s0 = blk * 8;
#pragma unroll
      for (int w = 0; w < SETS; ++w) {
        if ((blk & (SETS - 1)) != w) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int s = s0 + j;
          if (s >= ns) continue;
          const float2 ml = __ldcg(pm + s);
          if (ml.x == -INFINITY) continue;
          const float4 pv = __ldcg(reinterpret_cast<const float4*>(po + (size_t)s * HD + lane * PER));
          const float wt = exp2f(ml.x - M);
          Lw[w] = fmaf(ml.y, wt, Lw[w]);
          acc[w][0] = fmaf(pv.x, wt, acc[w][0]);
          acc[w][1] = fmaf(pv.y, wt, acc[w][1]);
          acc[w][2] = fmaf(pv.z, wt, acc[w][2]);
          acc[w][3] = fmaf(pv.w, wt, acc[w][3]);
        }
      }
    }
    float o[PER], Ls = Lw[0];
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = acc[0][i];
#pragma unroll
    for (int w = 1; w < SETS; ++w) {
      Ls = __fadd_rn(Ls, Lw[w]);
#pragma unroll
      for (int i = 0; i < PER; ++i) o[i] = __fadd_rn(o[i], acc[w][i]);
    }
    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
    bf16* out = a.attn + (size_t)tok * a.hq * HD + (size_t)head * HD + lane * PER;
    *reinterpret_cast<__nv_bfloat162*>(out) = __floats2bfloat162_rn(__fmul_rn(o[0], inv), __fmul_rn(o[1], inv));
    *reinterpret_cast<__nv_bfloat162*>(out + 2) = __floats2bfloat162_rn(__fmul_rn(o[2], inv), __fmul_rn(o[3], inv));
  }
}

// lm_head fragments -> (optional fp32 logits) -> per-CTA (max, argmax) of every row; lowest index wins ties
__device__ __forceinline__ void fin_argmax_cta(const StepArgs& a, uint8_t* smem) {
  const StepLinear& L = a.lm_head;
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
  float* sv = misc + MI_AV;
  int* si = reinterpret_cast<int*>(misc + MI_AI);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = a.n_rows;
  for (int tok = 0; tok < R; ++tok) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = blockIdx.x * kStepThreads + threadIdx.x; c < L.n; c += gridDim.x * kStepThreads) {
      const float v = sum_local(a, L, tok, (size_t)c);
      if (a.logits) a.logits[(size_t)tok * a.ld_logits + c] = v;
      if (c < a.lm_valid && (v > best || (v == best && c < bi))) { best = v; bi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp * kStepMaxRows + tok] = best; si[warp * kStepMaxRows + tok] = bi; }
  }
  __syncthreads();
  if (threadIdx.x < R) {
    const int tok = threadIdx.x;
    float best = sv[tok];
    int bi = si[tok];
    for (int w = 1; w < kStepWarps; ++w) {
      const float ov = sv[w * kStepMaxRows + tok];
      const int oi = si[w * kStepMaxRows + tok];
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    a.amax_val[(size_t)blockIdx.x * kStepMaxRows + tok] = best;
    a.amax_idx[(size_t)blockIdx.x * kStepMaxRows + tok] = bi;
  }
}

// CTA 0, warp = row: winner over the CTAs (then over the ranks)
__device__ __forceinline__ void argmax_over_ctas(const StepArgs& a, int tok, float& best, int& bi) {
  const int lane = threadIdx.x & 31;
  best = -INFINITY; bi = 0x7fffffff;
  for (int c = lane; c < (int)gridDim.x; c += 32) {
    const float ov = __ldcg(a.amax_val + (size_t)c * kStepMaxRows + tok);
    const int oi = __ldcg(a.amax_idx + (size_t)c * kStepMaxRows + tok);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (bi != 0x7fffffff) bi += a.lm_offset;
}

}  // namespace

__global__ void __launch_bounds__(kStepThreads, 1) step_kernel(const StepArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
  int* row_ids = reinterpret_cast<int*>(misc + MI_ROW);
  int* row_pos = row_ids + 8;
  int* row_seq = row_ids + 16;
  int* row_rope = row_ids + 24;

  WRing ring;
  ring.base = smem + SM_RING + (size_t)warp * kRingBytes;
  ring.base_u = smem_u32(ring.base);
  ring.bars_u = smem_u32(smem + SM_BARS) + warp * kRingBars * 8;
  ring.pidx = ring.cidx = 0;
  ring.ppos = ring.cpos = 0;
  ring.pfree = kRingBytes;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kRingBars; ++i) mbar_init(ring.bars_u + i * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  SyncState ss;
  ss.local_target = a.sync[1];
  ss.cross_target = a.sync[2];
  if (tid < kStepMaxRows) {
    int id = 0, pos = 0, seq = 0, rp = 0;
    if (tid < a.n_rows) {
      if (a.slot_seq) {
        seq = a.slot_seq[tid];
        id = a.last_ids[tid];
        pos = a.seq_len[seq];
        rp = pos;
        if (cta == 0) { a.ids[tid] = id; a.tok_pos[tid] = pos; a.tok_seq[tid] = seq; }
      } else {
        id = a.ids[tid]; pos = a.tok_pos[tid]; seq = a.tok_seq[tid];
        rp = a.rope_pos ? a.rope_pos[tid] : pos;
      }
    }
    row_ids[tid] = id; row_pos[tid] = pos; row_seq[tid] = seq; row_rope[tid] = rp;
  }
  __syncthreads();

  Cursor cur;
  cur.n_phases = 4 * a.n_layers + 1;
  cur.phase = 0;
  cur.p = 0; cur.b = 0; cur.b_hi = 0;
  if (lane == 0) {
    load_linear(a, 0, cur.ph.lin);
    split_phase(cur.ph, cta);
    cursor_settle(cur, a, cta, warp, true);
    pump(ring, cur, a, cta, warp);     // weights do not depend on anything: start streaming at once
  }
  __syncwarp();
  bool failed = false;

  fin_embed(a, row_ids);
  grid_sync(a, ss);
  const long d = a.d_model;
  const bool tp = a.tp_size > 1;
  for (int l = 0; l < a.n_layers; ++l) {
    const StepLayer* ly = a.layers + l;
    gemv_phase(a, 4 * l, smem, ring, cur, a.h, d, ly->ln1, -1, failed);
    grid_sync(a, ss);
    fin_qkv(a, ly, row_pos, row_seq, row_rope);
    grid_sync(a, ss);
    attn_phase(a, ly->kv_pool, smem, row_pos, row_seq);
    grid_sync(a, ss);
    fin_merge(a, row_pos);
    grid_sync(a, ss);
    gemv_phase(a, 4 * l + 1, smem, ring, cur, a.attn, (long)a.hq * 128, nullptr, tp ? a.x_off[0] : -1, failed);
    cross_sync(a, ss);
    fin_resid(a, &ly->o, tp ? a.x_off[0] : -1);
    grid_sync(a, ss);
    gemv_phase(a, 4 * l + 2, smem, ring, cur, a.h, d, ly->ln2, -1, failed);
    grid_sync(a, ss);
    fin_swiglu(a, &ly->gate_up);
    grid_sync(a, ss);
    gemv_phase(a, 4 * l + 3, smem, ring, cur, a.act, (long)a.ffn, nullptr, tp ? a.x_off[1] : -1, failed);
    cross_sync(a, ss);
    fin_resid(a, &ly->down, tp ? a.x_off[1] : -1);
    grid_sync(a, ss);
  }
  gemv_phase(a, 4 * a.n_layers, smem, ring, cur, a.h, d, a.final_norm, -1, failed);
  grid_sync(a, ss);
  fin_argmax_cta(a, smem);
  grid_sync(a, ss);
  // winners: CTA 0, one warp per row; under tensor parallelism every rank's candidate travels to every rank
  if (tp) {
    if (cta == 0 && warp < a.n_rows) {
      float best; int bi;
      argmax_over_ctas(a, warp, best, bi);
      if (lane == 0)
        for (int r = 0; r < a.tp_size; ++r) {
          float* slot = a.xreg[r] + a.x_amax + ((size_t)a.tp_rank * kStepMaxRows + warp) * 2;
          slot[0] = best;
          slot[1] = __int_as_float(bi);
        }
    }
    cross_sync(a, ss);
    if (cta == 0 && tid < a.n_rows) {
      float best = -INFINITY; int bi = 0x7fffffff;
      const float* own = a.xreg[a.tp_rank] + a.x_amax;
      for (int r = 0; r < a.tp_size; ++r) {
        const float ov = __ldcg(own + ((size_t)r * kStepMaxRows + tid) * 2);
        const int oi = __float_as_int(__ldcg(own + ((size_t)r * kStepMaxRows + tid) * 2 + 1));
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      a.out_ids[tid] = bi; a.out_val[tid] = best;
      if (a.slot_seq) { a.last_ids[tid] = bi; a.seq_len[row_seq[tid]] = row_pos[tid] + 1; }
    }
  } else if (cta == 0 && warp < a.n_rows) {
    float best; int bi;
    argmax_over_ctas(a, warp, best, bi);
    if (lane == 0) {
      a.out_ids[warp] = bi; a.out_val[warp] = best;
      if (a.slot_seq) { a.last_ids[warp] = bi; a.seq_len[row_seq[warp]] = row_pos[warp] + 1; }
    }
  }
  if (cta == 0 && tid == 0) { a.sync[1] = ss.local_target; a.sync[2] = ss.cross_target; }
  if (failed) {
    // give copies still in flight a bounded chance to land before the CTA's shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { }
  }
}

}  // namespace b2

using namespace b2;

// Work split of one linear over `ncta` CTAs (shape-only): k slices of at most kStepSliceK inputs, cps CTAs per slice
// (never more CTAs than blocks), and the most fragments a panel of a slice is cut into.
B2_API int b2_step_linear(const uint8_t* wq, int n, int k, int bits, int group, int ncta, StepLinear* out) {
  if (!out || n <= 0 || k <= 0 || n % 32 || k % 128 || ncta < 1) return B2_ERR_ARG;
  if ((bits != 2 && bits != 3 && bits != 4) || (group != 64 && group != 128)) return B2_ERR_ARG;
  StepLinear L = {};
  L.wq = wq; L.n = n; L.k = k; L.bits = bits; L.group = group;
  L.npan = n / 32; L.nbat = k / 128;
  const int rec = bits == 3 ? 768 : 512;
  const int rpb = bits == 4 ? 2 : 1;
  L.wbatch = rpb * rec;
  L.szb = (128 / group) * 64;
  L.blk = 2 * L.wbatch + 2 * L.szb;
  L.ks = (k + kStepSliceK - 1) / kStepSliceK;
  if (L.ks > L.nbat) L.ks = L.nbat;
  if (L.ks > ncta) return B2_ERR_ARG;
  const long nbs_min = L.nbat / L.ks, nbs_max = (L.nbat + L.ks - 1) / L.ks;
  const long bmin = (long)L.npan * nbs_min;
  long cps = ncta / L.ks;
  if (cps > bmin) cps = bmin;
  if (cps < 1) cps = 1;
  L.cps = (int)cps;
  const long per = bmin / cps;
  long fmax = (nbs_max + per - 1) / per + 1;
  if (fmax > nbs_max) fmax = nbs_max;
  L.fmax = (int)fmax;
  if ((double)L.npan * (double)nbs_max * (double)(cps + 1) >= 4.0e9) return B2_ERR_ARG;   // 32-bit block arithmetic
  *out = L;
  return B2_OK;
}

// Floats of the partial buffer one linear needs for `rows` token rows: [ks * fmax][rows][n].
B2_API long b2_step_part_floats(const StepLinear* lin, int rows) {
  return (long)lin->ks * lin->fmax * rows * lin->n;
}

B2_API int b2_step_smem_bytes() { return SM_TOTAL; }
B2_API int b2_step_args_bytes() { return (int)sizeof(StepArgs); }
B2_API int b2_step_layer_bytes() { return (int)sizeof(StepLayer); }

// CTAs of the persistent grid = SMs of the current device, provided one CTA fits per SM.
B2_API int b2_step_grid(int* ncta) {
  int dev = 0, sms = 0, occ = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B2_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (cudaFuncSetAttribute(step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, step_kernel, kStepThreads, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
  if (occ < 1 || !coop || sms < 1) return B2_ERR_LAUNCH;
  *ncta = sms;
  return B2_OK;
}

// Launches one step.  `ncta` must be the value the linears' work split was computed for (b2_step_grid).  The launch
// is cooperative, so all CTAs are resident together (the barriers inside the kernel rely on it).
B2_API int b2_step_launch(const StepArgs* args, int ncta, cudaStream_t stream) {
  const StepArgs& a = *args;
  if (a.n_rows < 1 || a.n_rows > kStepMaxRows || a.n_layers < 0 || ncta < 1) return B2_ERR_ARG;
  if (a.hq <= 0 || a.hkv <= 0 || a.hq % a.hkv || a.d_model % 8 || a.split_keys % kPage || a.max_splits <= 0) return B2_ERR_ARG;
  if (a.n_groups < 1 || a.n_groups > a.n_rows) return B2_ERR_ARG;
  if (a.tp_size < 1 || a.tp_size > kStepMaxTp || a.tp_rank < 0 || a.tp_rank >= a.tp_size) return B2_ERR_ARG;
  if (!a.sync || !a.status || !a.part || !a.h) return B2_ERR_ARG;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ncta, 1, 1);
  cfg.blockDim = dim3(kStepThreads, 1, 1);
  cfg.dynamicSmemBytes = SM_TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, step_kernel, a) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}
