// Persistent decode-step kernel, sm_100a: ONE cooperative launch runs a whole decode / verify step of the dense GQA
// decoder -- embedding, every layer (qkv, RoPE + KV store, paged attention, o_proj, gate/up, SwiGLU, down_proj), the
// lm_head and the argmax -- for up to sixteen token rows, on one GPU or on every GPU of a tensor-parallel group.
//
// The reference runs a step as a CUDA graph of several kernels per layer with programmatic-dependent-launch edges
// (kernels/m1/m1_model.cu:2544-2596 `layer`, :3071-3140 decode graphs, kernels/src/runtime.cu:198-228) and folds
// the tensor-parallel all-reduce into its push kernels (kernels/src/tp_ar.cu:160-227).  On a 148-SM part a step of
// the 32B model is bound by the ~450 kernel boundaries, not by the weights, so here the boundaries disappear:
//
//   * one CTA of 15 worker warps and one producer warp per SM stays resident for the whole step; phases are separated by grid barriers (one
//     release-add and a bounded acquire-poll per CTA), tensor-parallel phases by the same barrier across GPUs
//     (release-adds into every peer's counter over NVLink);
//   * every warp streams its statically known share of ALL the step's weights through a private cp.async.bulk ring
//     whose producer runs ahead across phase boundaries: while a barrier or the attention phase is in progress the
//     next linear's weights are already in flight or in shared memory;
//   * a linear is cut by contiguous block ranges over the CTAs (stream-k); the worker warps of a CTA share one row panel
//     at a time and combine their k ranges through shared memory; a panel cut by a CTA boundary leaves one partial per
//     fragment in global memory.  The consumer ("finalize") stage adds the fragments in a fixed order and applies
//     what the reference does in separate kernels: RoPE + KV store, the split merge of attention, residual add,
//     SwiGLU, argmax;
//   * row-parallel linears under tensor parallelism write their fragments straight into every peer's exchange region
//     (plain stores over NVLink) and the finalize stage of every rank adds all ranks' fragments in rank order: the
//     GEMV -> all-reduce -> residual add -> next norm path is one kernel with no library collective.
//
// Batch invariance: the k range, the fragment cut and every summation order depend on the linear's shape, the k slice
// and the number of CTAs only, never on the number of rows; attention uses the fixed-size KV splits of attn_decode.cu.
// A row of a verify block is therefore bit-identical to the same row of a plain decode step, as long as both use the
// same k slice: steps of up to eight rows stage slices of 5120 inputs, steps of nine to sixteen rows 2560 (their
// staged activations take twice the room per input), so rows are comparable bit for bit within each of the two classes.
#pragma once
#include "step_kernel.cuh"
#include "wq_frag.cuh"

namespace b2 {
namespace {

constexpr int kRingBars = 16;              // units in flight per warp
constexpr int kPage = 16;

// Shared memory of a CTA: [mbarriers | misc | work area | weight rings].  The work area (staged activations, group
// scalars, partial tiles; attention's K/V stages alias it) grows with the number of token rows, and the weight rings
// take everything that is left: a one-row decode step keeps about 11 KB of weights in flight per warp, an eight-row
// step 7 KB, a sixteen-row step 9 KB (its partial tiles live in global memory).  Ring depth changes no arithmetic.
constexpr int SM_TOTAL = 227328;
constexpr int SM_BARS = 0;
constexpr int SM_MISC = 2048;
constexpr int SM_MISC_BYTES = 3584;
constexpr int SM_WORK = SM_MISC + SM_MISC_BYTES;
// Warps of a CTA that run attention items and their 8 KB K/V page stages.  Base shape: three warps (six beyond four
// rows: the work area is that large anyway) with two stages each.  When the step has more split items than base warps
// in the grid, twice the warps run with one stage each in the same shared memory: a page costs a warp about 2 us of
// dependent tensor-core latency, so more warps in flight then beat a deeper pipeline per warp.
__host__ __device__ __forceinline__ int attn_warps(int rows) { return rows > 4 ? 6 : 3; }
__host__ __device__ __forceinline__ int attn_bytes(int rows) { return attn_warps(rows) * 2 * 2 * kPage * 128 * 2; }
constexpr int kTileFloats = kStepWarps * 2 * kStepMaxRows * 32;      // floats of one CTA's tiles in global memory
static_assert(kStepWarps * kRingBars * 8 <= SM_MISC, "mbarriers");
static_assert(SM_TOTAL <= 227 * 1024, "shared memory of one CTA");

__host__ __device__ __forceinline__ int token_sets(int rows) { return rows > 8 ? 4 : (rows > 4 ? 2 : 1); }

struct Lay {
  int xs_stride;      // bytes of staged activations per 128-k batch: token sets x four steps x 256 B
  int gstride;        // float2 entries per quantisation group in the group-scalar table (4 per token set)
  int gsum, tiles;    // byte offsets
  int ring, ring_w;   // offset of the rings and bytes per warp
};
__host__ __device__ __forceinline__ Lay make_lay(int rows, int slice_k) {
  Lay l;
  const int ns = token_sets(rows), maxb = slice_k / 128;
  l.xs_stride = ns * 1024;
  l.gstride = ns * 4;
  l.gsum = SM_WORK + maxb * l.xs_stride;
  l.tiles = l.gsum + maxb * 2 * l.gstride * 8;
  int end = l.tiles + (rows > kStepSmallRows ? 0 : kStepWarps * 2 * rows * 32 * 4);   // head and tail tile of every worker warp
  if (end < SM_WORK + attn_bytes(rows)) end = SM_WORK + attn_bytes(rows);
  l.ring = (end + 127) & ~127;
  l.ring_w = ((SM_TOTAL - l.ring) / kStepWarps) & ~63;
  return l;
}
static_assert(SM_WORK + (kStepSliceK / 128) * (2048 + 2 * 8 * 8) + kStepWarps * 2 * 8 * 32 * 4 + kStepWarps * 2304 * 3 <= SM_TOTAL,
              "an eight-row step still has three blocks per warp in flight");
static_assert(SM_WORK + (kStepSliceK / 256) * (4096 + 2 * 16 * 8) + kStepWarps * 2560 * 3 + 128 <= SM_TOTAL,
              "a sixteen-row step still has three blocks per warp in flight");
static_assert(SM_WORK + 6 * 2 * 2 * kPage * 128 * 2 + kStepWarps * 2560 * 3 + 128 <= SM_TOTAL,
              "the attention stages leave three blocks per warp in flight");

// misc area (floats): [0,16) inv_rms, [16,256) per-warp sums, [256,496) argmax values, [496,736) argmax indices,
// [736,800) row description (ids, pos, seq, rope position), [800,832) ring progress published to the producer warp,
// [832,862) panel index of every partial tile
constexpr int MI_WSUM = 16, MI_AV = 256, MI_AI = 496, MI_ROW = 736, MI_PUB = 800, MI_TILE = 832;   // MI_PUB: 2 words per worker warp
constexpr int MI_DESC = 864;               // [864,896): two 64-byte slots for the next linears' descriptors (16-byte aligned)
static_assert(MI_TILE + 2 * kStepWarps <= MI_DESC && (MI_DESC + 32) * 4 <= SM_MISC_BYTES && (MI_DESC * 4) % 16 == 0, "misc area");

// Barrier over the worker warps (the producer warp never takes part in a CTA barrier).
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kStepThreads) : "memory"); }

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
  unsigned ev;                           // trace builds: next stamp index
};
#ifdef B2_STEP_TRACE
#define B2_STAMP(a, ss) do { if ((a).trace && blockIdx.x == 0) (a).trace[(ss).ev++] = globaltimer_ns(); } while (0)
#else
#define B2_STAMP(a, ss) do { } while (0)
#endif

// Grid barrier.  Every CTA adds one to the counter with release semantics after its threads met at bar.sync, then
// polls with acquire loads until all CTAs of this epoch arrived.  The poll is bounded: on expiry (or when another
// wait already failed) the status word is set and the kernel runs to its end without waiting again.
__device__ __noinline__ void grid_sync(const StepArgs& a, SyncState& ss) {
  workers_sync();
  if (threadIdx.x == 0) {
    ss.local_target += gridDim.x;
    B2_STAMP(a, ss);
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
    B2_STAMP(a, ss);
  }
  workers_sync();
}

// The same barrier over all CTAs of all tensor-parallel ranks: one release-add into every rank's counter (word 0 of
// its exchange region), then a poll of the own counter.  With one rank it is the grid barrier.
__device__ __noinline__ void cross_sync(const StepArgs& a, SyncState& ss) {
  if (a.tp_size <= 1) { grid_sync(a, ss); return; }
  workers_sync();
  if (threadIdx.x == 0) {
    ss.cross_target += gridDim.x * (unsigned)a.tp_size;
    B2_STAMP(a, ss);
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
    B2_STAMP(a, ss);
  }
  workers_sync();
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
__device__ __forceinline__ void decode_linear(uint4 a0, uint4 a1, uint4 a2, uint4 a3, StepLinear& L);
__device__ __forceinline__ void fetch_linear(const StepLinear* src, StepLinear& L) {
  static_assert(sizeof(StepLinear) == 64, "StepLinear is read as four 16-byte words");
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  decode_linear(__ldg(s4), __ldg(s4 + 1), __ldg(s4 + 2), __ldg(s4 + 3), L);
}
__device__ __forceinline__ void decode_linear(uint4 a0, uint4 a1, uint4 a2, uint4 a3, StepLinear& L) {
  L.wq = reinterpret_cast<const uint8_t*>(((unsigned long long)a0.y << 32) | (unsigned long long)a0.x);
  L.n = (int)a0.z; L.k = (int)a0.w;
  L.bits = (int)a1.x; L.group = (int)a1.y; L.npan = (int)a1.z; L.nbat = (int)a1.w;
  L.wbatch = (int)a2.x; L.szb = (int)a2.y; L.blk = (int)a2.z; L.ks = (int)a2.w;
  L.cps = (int)a3.x; L.fmax = (int)a3.y; L.pad = 0;
}

__device__ __forceinline__ const StepLinear* linear_of(const StepArgs& a, int phase) {
  const StepLayer* ly = a.layers + (phase >> 2);
  const int j = phase & 3;
  return j == 0 ? &ly->qkv : (j == 1 ? &ly->o : (j == 2 ? &ly->gate_up : &ly->down));
}
__device__ __forceinline__ void load_linear(const StepArgs& a, int phase, StepLinear& L) {
  if (phase >= 4 * a.n_layers) { L = a.lm_head; return; }
  fetch_linear(linear_of(a, phase), L);
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

// Block range of worker warp w inside its CTA's range: the CTA's blocks are cut into kStepWarps contiguous pieces
// (stream-k at warp level), so the warps of a CTA carry the same number of blocks (+-1) and never wait for one another
// inside a phase.  A piece may start and end in the middle of a panel: the warp leaves at most two partial tiles
// (head and tail) in shared memory; panels that lie completely inside its piece are finished by the warp alone.
__device__ __forceinline__ void warp_range(const Phase& ph, int warp, unsigned& wlo, unsigned& whi) {
  const unsigned nblk = ph.hi - ph.lo;
  wlo = ph.lo + (unsigned)(((unsigned long long)nblk * (unsigned)warp) / kStepWarps);
  whi = ph.lo + (unsigned)(((unsigned long long)nblk * (unsigned)(warp + 1)) / kStepWarps);
}

// Producer cursor of one ring (one lane of the producer warp): the blocks of that worker warp, for every remaining
// linear of the step, in the order the worker consumes them.
struct Cursor {
  int phase, n_phases;
  Phase ph;
  unsigned blk, whi;
};

__device__ __noinline__ void cursor_settle(Cursor& c, const StepArgs& a, int cta, int warp, bool fresh) {
  // `fresh`: c.ph was just loaded for c.phase and the warp's range is not selected yet
  while (c.phase < c.n_phases) {
    if (fresh) {
      c.blk = c.whi = 0;
      if (c.ph.active && c.ph.lo < c.ph.hi) warp_range(c.ph, warp, c.blk, c.whi);
      fresh = false;
    }
    if (c.blk < c.whi) return;
    ++c.phase;
    if (c.phase < c.n_phases) { load_linear(a, c.phase, c.ph.lin); split_phase(c.ph, cta); }
    fresh = true;
  }
}

// Consumer side of one warp's weight ring.  The producer warp fills it; the consumer publishes how many units it
// has finished and how many ring bytes that released.
struct WRing {
  uint32_t bars_u;
  uint8_t* base;
  unsigned cidx;           // units consumed
  unsigned cbytes;         // ring bytes released (wrap skips included)
  int cpos;                // byte position of the next unit
  volatile unsigned* pub;  // [0] units consumed, [1] bytes released, as read by the producer warp
};

// The last warp of a CTA: lane i feeds the ring of worker warp i with bulk copies, for every linear of the step in
// order, as far ahead as the ring has room (across phase boundaries: while the workers sit in a barrier, a finalize
// stage or attention, the next linear's weights are already on their way).  One (32-row x 128-k) block = one
// contiguous copy.  The warp takes part in no
// barrier and ends when everything is issued (or when a failed wait set the status word).
__device__ __noinline__ void producer_loop(const StepArgs& a, uint8_t* smem, int cta, const Lay& lay) {
  const int kRingBytes = lay.ring_w;
  const int lane = threadIdx.x & 31;
  const bool owner = lane < kStepWarps;
  Cursor c;
  c.n_phases = 4 * a.n_layers + 1;
  c.phase = owner ? 0 : c.n_phases;
  c.blk = 0; c.whi = 0;
  unsigned pidx = 0, pbytes = 0;
  int ppos = 0;
  const uint32_t base_u = smem_u32(smem + lay.ring) + (owner ? lane : 0) * kRingBytes;
  const uint32_t bars_u = smem_u32(smem + SM_BARS) + (owner ? lane : 0) * kRingBars * 8;
  volatile unsigned* pub = reinterpret_cast<volatile unsigned*>(smem + SM_MISC) + MI_PUB + 2 * (owner ? lane : 0);
  if (owner) {
    load_linear(a, 0, c.ph.lin);
    split_phase(c.ph, cta);
    cursor_settle(c, a, cta, lane, true);
  }
  unsigned idle = 0;
  while (__any_sync(0xffffffffu, c.phase < c.n_phases)) {
    bool issued = false;
    if (c.phase < c.n_phases) {
      const StepLinear& L = c.ph.lin;
      const int usz = L.blk;
      int pos = ppos, need = usz;
      if (pos + usz > kRingBytes) { need += kRingBytes - pos; pos = 0; }
      const unsigned cidx = pub[0], cby = pub[1];
      if (pidx - cidx < (unsigned)kRingBars && (unsigned)kRingBytes - (pbytes - cby) >= (unsigned)need) {
        const uint32_t bar = bars_u + (pidx % kRingBars) * 8;
        mbar_expect_tx(bar, (uint32_t)usz);
        const unsigned pp = c.blk / (unsigned)c.ph.nbs, bb = c.blk - pp * (unsigned)c.ph.nbs;
        bulk_g2s(base_u + pos, L.wq + ((size_t)pp * L.nbat + (size_t)(c.ph.bs0 + bb)) * L.blk, (uint32_t)usz, bar);
        ppos = pos + usz;
        pbytes += (unsigned)need;
        ++pidx;
        ++c.blk;
        cursor_settle(c, a, cta, lane, false);
        issued = true;
      }
    }
    if (__any_sync(0xffffffffu, issued)) { idle = 0; continue; }
    if ((++idle & 15u) == 0u && ld_volatile_i32(a.status) != 0) break;     // a worker gave up: stop feeding
    __nanosleep(64);
  }
}

// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A registers of integer-MMA step s (32 k) of a batch from the FI layout (wq_tools.cu, fi_pos): register r holds four
// codes of row g + 8 (r & 1), k = 32 s + 16 (r >> 1) + 4 t + byte.
template <int BITS, int GROUP>
__device__ __forceinline__ void extract8(const WFrag<BITS, GROUP>& f, int s, uint32_t (&a)[4]) {
  if (BITS == 4) {
    const uint32_t w0 = u4_get(f.lo[s >> 1], 2 * (s & 1)), w1 = u4_get(f.lo[s >> 1], 2 * (s & 1) + 1);
    a[0] = w0 & 0x0F0F0F0Fu;
    a[1] = w1 & 0x0F0F0F0Fu;
    a[2] = (w0 >> 4) & 0x0F0F0F0Fu;
    a[3] = (w1 >> 4) & 0x0F0F0F0Fu;
  } else {
    const uint32_t w = u4_get(f.lo[0], s);
    a[0] = w & 0x03030303u;
    a[1] = (w >> 2) & 0x03030303u;
    a[2] = (w >> 4) & 0x03030303u;
    a[3] = (w >> 6) & 0x03030303u;
    if (BITS == 3) {
      // the third bit of register r sits at bit 8 byte + 4 (s & 1) + r of the high-plane word; one shift puts it on bit 2
      const uint32_t h = (s >> 1) ? f.hi.y : f.hi.x;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int q = 4 * (s & 1) + r;
        const uint32_t hs = q <= 2 ? (h << (2 - q)) : (h >> (q - 2));
        a[r] = lop3_and_or(hs, 0x04040404u, a[r]);
      }
    }
  }
}

// (y0, y1) += s_w * (s_x * acc - z_w * s_x * sum_x) for rows g, g + 8 and one token of one group;
// acc = 128 * (hi-limb sum) + (lo-limb sum), exact in int32.
__device__ __forceinline__ void gemv_scale(float& y0, float& y1, const int (&acc)[4], const uint32_t (&sz)[2], float2 q) {
  const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&sz[0]));
  const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&sz[1]));
  y0 = fmaf(s0.x, fmaf(-s0.y, q.y, (float)(acc[0] * 128 + acc[1]) * q.x), y0);
  y1 = fmaf(s1.x, fmaf(-s1.y, q.y, (float)(acc[2] * 128 + acc[3]) * q.x), y1);
}

// ---------------------------------------------------------------------------------------------------- GEMV phase
// Where a CTA's panel sums go.  One out-of-line copy of the store serves every store site of the kernel: the kernel's
// code has to stay small enough for the instruction cache, since each of its stages runs once per layer.
struct EmitCtx {
  unsigned nbs, cps, Bsl, hi;     // batches of the slice; CTAs per slice; blocks of the slice; end of this CTA's block range
  int ci, slice, fmax, n, R, nslots;
  long tp_off;
};

// Fragment slot of this CTA for panel p: float offset of (slot, token 0, first row of the panel) in the partial
// buffer, and how many slots after it the CTA zero-fills (the CTA that holds the panel's last block clears the slots
// that no fragment uses).  Computed once per panel, not per element.
struct PanelSlot { size_t base; int nzero; };
__device__ __forceinline__ PanelSlot panel_slot(const EmitCtx& c, unsigned p) {
  const unsigned first_owner = (((p * c.nbs) + 1u) * c.cps - 1u) / c.Bsl;
  const int f = c.ci - (int)first_owner;
  const int f_end = ((p + 1u) * c.nbs <= c.hi) ? c.fmax : f + 1;
  PanelSlot ps;
  ps.base = ((size_t)(c.slice * c.fmax + f) * c.R) * c.n + (size_t)p * 32;
  ps.nzero = f_end - f - 1;
  return ps;
}
// Partial sums go to the own partial buffer (tp_off < 0: one destination) or into every rank's exchange region at
// float offset tp_off (tp_size destinations, this rank's fragments after those of the lower ranks).
__device__ __forceinline__ int part_dests(const StepArgs& a, const EmitCtx& c) { return c.tp_off < 0 ? 1 : a.tp_size; }
__device__ __forceinline__ float* part_dest(const StepArgs& a, const EmitCtx& c, int d) {
  return c.tp_off < 0 ? a.part : a.xreg[d] + (size_t)c.tp_off + (size_t)a.tp_rank * c.nslots * c.R * c.n;
}
// Zero-fill of the unused slots of a panel by one warp (lane = row).
__device__ __forceinline__ void zero_slots(const StepArgs& a, const EmitCtx& c, const PanelSlot& ps, int tok_begin, int tok_step) {
  const int lane = threadIdx.x & 31;
  const size_t stride = (size_t)c.R * c.n;
#pragma unroll 1
  for (int d = 0; d < part_dests(a, c); ++d) {
    float* bp = part_dest(a, c, d);
#pragma unroll 1
    for (int z = 1; z <= ps.nzero; ++z)
#pragma unroll 1
      for (int tok = tok_begin; tok < c.R; tok += tok_step) bp[ps.base + z * stride + (size_t)tok * c.n + lane] = 0.f;
  }
}

// Activations reach a linear already staged: the stage that PRODUCES them (embedding, residual add, attention merge,
// SwiGLU) writes, next to the bf16 values, their fixed-point form in the layout the GEMV phases keep in shared
// memory, once for the whole grid; a GEMV phase then only copies its k slice.  (Quantising inside the GEMV phase made
// every CTA of a slice repeat the same conversion: tens of microseconds per layer at sixteen rows.)
//
// One warp, one (token, 128-k batch): lane i holds inputs k = 128 batch + 4 i + {0..3}.  Per quantisation group the
// inputs become 15-bit fixed point, x = s (128 hi + lo) with signed 8-bit limbs, written as columns (2 tok, 2 tok + 1)
// of the token's set in the B-operand order of mma.m16n8k32, plus (s, s * sum of the integers).  An RMS-normed input
// is staged WITHOUT its 1 / rms factor (a positive per-row scalar commutes with the group quantisation and with the
// linear): the consumer's finalize stage multiplies its sums by it.  `sq` is the lane's share of the row's sum of
// squares; the batch's total goes to a.psq[tok][batch].
__device__ __noinline__ void quant_store(const StepArgs& a, int xstride, int gstride, int group, int tok, int batch,
                                         float v0, float v1, float v2, float v3, bool want_sq, float sq, int nb) {
  const int lane = threadIdx.x & 31;
  float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
  if (group == 128) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float inv = amax > 0.f ? 16383.f / amax : 0.f;
  const int q0 = __float2int_rn(v0 * inv), q1 = __float2int_rn(v1 * inv), q2 = __float2int_rn(v2 * inv), q3 = __float2int_rn(v3 * inv);
  int isum = q0 + q1 + q2 + q3;
  if (group == 128) isum += __shfl_xor_sync(0xffffffffu, isum, 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) isum += __shfl_xor_sync(0xffffffffu, isum, o);
  const uint32_t hi = ((uint32_t)(q0 >> 7) & 0xFFu) | (((uint32_t)(q1 >> 7) & 0xFFu) << 8) | (((uint32_t)(q2 >> 7) & 0xFFu) << 16) |
                      (((uint32_t)(q3 >> 7) & 0xFFu) << 24);
  const uint32_t lo = ((uint32_t)q0 & 0x7Fu) | (((uint32_t)q1 & 0x7Fu) << 8) | (((uint32_t)q2 & 0x7Fu) << 16) | (((uint32_t)q3 & 0x7Fu) << 24);
  // k = 4 lane inside the batch: integer-MMA step lane / 8, half (lane / 4) & 1, thread-in-group lane & 3
  const int col = 2 * (tok & 3);
  uint8_t* base = a.xq + (size_t)batch * xstride + (tok >> 2) * 1024 + (lane >> 3) * 256 + ((lane >> 2) & 1) * 4;
  *reinterpret_cast<uint32_t*>(base + (col * 4 + (lane & 3)) * 8) = hi;
  *reinterpret_cast<uint32_t*>(base + ((col + 1) * 4 + (lane & 3)) * 8) = lo;
  if ((lane & (group / 4 - 1)) == 0) {
    const float sx = amax * (1.f / 16383.f);
    a.xg[((size_t)batch * (128 / group) + (lane * 4) / group) * gstride + tok] = make_float2(sx, sx * (float)isum);
  }
  if (want_sq) {
    sq = warp_sum(sq);
    if (lane == 0) a.psq[(size_t)tok * nb + batch] = sq;
  }
}

// Stage 1 of a linear: the CTA's k slice of the staged activations and of their group scalars, global -> shared.
__device__ __noinline__ void copy_staged(const StepArgs& a, const Phase& ph, Lay lay, bool want_scales) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x;
  if (want_scales) {
    // 1 / rms of every row from the per-batch sums of squares (fixed order), for the finalize stage after this linear
    float* inv_rms = reinterpret_cast<float*>(smem + SM_MISC);
    const int warp = tid >> 5, lane = tid & 31;
    const int nb = a.d_model >> 7;
    for (int tok = warp; tok < a.n_rows; tok += kStepWarps) {
      float s = 0.f;
      for (int b = lane; b < nb; b += 32) s += __ldcg(a.psq + (size_t)tok * nb + b);
      s = warp_sum(s);
      if (lane == 0) inv_rms[tok] = rsqrtf(s / (float)a.d_model + a.eps);
    }
  }
  if (ph.active && ph.nbs > 0) {
    const int gpb = 128 / ph.lin.group;
    const uint4* src = reinterpret_cast<const uint4*>(a.xq + (size_t)ph.bs0 * lay.xs_stride);
    uint4* dst = reinterpret_cast<uint4*>(smem + SM_WORK);
    const int nv = ph.nbs * (lay.xs_stride >> 4);
#pragma unroll 1
    for (int v = tid; v < nv; v += 4 * kStepThreads) {
      uint4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * kStepThreads < nv) r[u] = __ldcg(src + v + u * kStepThreads);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * kStepThreads < nv) dst[v + u * kStepThreads] = r[u];
    }
    const uint4* gs = reinterpret_cast<const uint4*>(a.xg + (size_t)ph.bs0 * gpb * lay.gstride);
    uint4* gd = reinterpret_cast<uint4*>(smem + lay.gsum);
    const int ng = ph.nbs * gpb * lay.gstride / 2;
    for (int v = tid; v < ng; v += kStepThreads) gd[v] = __ldcg(gs + v);
  }
  workers_sync();
}

// A finished panel of one warp (32 rows x R tokens in `tile`) goes to the CTA's fragment slot: lane = row.
__device__ __noinline__ void flush_panel(const StepArgs& a, const EmitCtx& ec, unsigned p, const float* tile, bool tile_global) {
  const int lane = threadIdx.x & 31;
  const int R = a.n_rows;
  const PanelSlot ps = panel_slot(ec, p);
#pragma unroll 1
  for (int tok0 = 0; tok0 < R; tok0 += 4) {
    // volatile: the tile may live in global memory, written by this warp past the L1 cache
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[u] = 0.f;
      if (tok0 + u < R) v[u] = *reinterpret_cast<const volatile float*>(tile + (tok0 + u) * 32 + lane);
    }
#pragma unroll 1
    for (int d = 0; d < part_dests(a, ec); ++d) {
      float* bp = part_dest(a, ec, d) + ps.base + lane;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (tok0 + u < R) bp[(size_t)(tok0 + u) * ec.n] = v[u];
    }
  }
  if (ps.nzero > 0) zero_slots(a, ec, ps, 0, 1);
}

// Stage 3 of a linear: partial tiles of one panel come from consecutive warps (tail of one, heads of the next ones), so
// the tile list in (warp, head / tail) order holds each panel as one run of consecutive entries.  A work item is
// (run, token quarter): lane = row of the panel, up to four tokens (tq, tq + 4, ...) whose tile values are added in
// list order (= k order) and stored into the CTA's fragment slot.  The panel's slot is computed once per item.
__device__ __noinline__ void reduce_tiles(const StepArgs& a, const EmitCtx& ec, const float* tiles, bool tiles_global) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = a.n_rows;
  const int tile_f = R * 32;
  const unsigned* tile_panel = reinterpret_cast<const unsigned*>(reinterpret_cast<const float*>(smem + SM_MISC) + MI_TILE);
  // run starts: a valid entry whose nearest valid predecessor holds another panel
  const unsigned mine = lane < 2 * kStepWarps ? tile_panel[lane] : 0xffffffffu;
  const unsigned valid = __ballot_sync(0xffffffffu, mine != 0xffffffffu);
  const unsigned before = valid & ((1u << lane) - 1u);
  const int prev = before ? 31 - __clz(before) : 0;
  const unsigned prev_p = __shfl_sync(0xffffffffu, mine, prev);
  const unsigned starts = __ballot_sync(0xffffffffu, mine != 0xffffffffu && (before == 0u || prev_p != mine));
  const int nruns = __popc(starts);
  // token chunks per run: many runs keep the warps busy by themselves (one chunk: all tokens' loads in flight at once),
  // few runs are split over the tokens
  int nq = nruns >= 12 ? 1 : (nruns >= 6 ? 2 : 4);
  if (nq > R) nq = R;
#pragma unroll 1
  for (int item = warp; item < nruns * nq; item += kStepWarps) {
    const int run = item / nq, tq = item - run * nq;
    const int i0 = __fns(starts, 0, run + 1);
    const unsigned later = starts & ~((2u << i0) - 1u);
    const int i1 = later ? __ffs(later) - 1 : 2 * kStepWarps;
    const unsigned p = __shfl_sync(0xffffffffu, mine, i0);
    float sum[kStepMaxRows];
#pragma unroll
    for (int u = 0; u < kStepMaxRows; ++u) sum[u] = 0.f;
#pragma unroll 1
    for (int i = i0; i < i1; ++i) {
      if (!((valid >> i) & 1u)) continue;
      const float* src = tiles + (size_t)i * tile_f + lane;
      float v[kStepMaxRows];
#pragma unroll
      for (int u = 0; u < kStepMaxRows; ++u) {
        const int tok = tq + nq * u;
        v[u] = 0.f;
        if (tok < R) v[u] = *reinterpret_cast<const volatile float*>(src + tok * 32);   // shared, or global past L1
      }
#pragma unroll
      for (int u = 0; u < kStepMaxRows; ++u) sum[u] += v[u];
    }
    const PanelSlot ps = panel_slot(ec, p);
#pragma unroll 1
    for (int d = 0; d < part_dests(a, ec); ++d) {
      float* bp = part_dest(a, ec, d) + ps.base + lane;
#pragma unroll
      for (int u = 0; u < kStepMaxRows; ++u) {
        const int tok = tq + nq * u;
        if (tok < R) bp[(size_t)tok * ec.n] = sum[u];
      }
    }
    if (ps.nzero > 0) zero_slots(a, ec, ps, tq, nq);
  }
}

template <int BITS, int GROUP, int NS>
__device__ __forceinline__ void gemv_body(const StepArgs& a, const Phase& ph, uint8_t* smem, const Lay& lay, WRing& ring,
                                          long tp_off, bool& failed, bool want_scales) {
  constexpr int GPB = 128 / GROUP;
  constexpr int SPG = 4 / GPB;               // integer-MMA steps per quantisation group
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;
  const int R = a.n_rows;
  const StepLinear& L = ph.lin;
  const int nbs = ph.nbs;
  const int kRingBytes = lay.ring_w;
  const int xstride = lay.xs_stride;
  const int gstride = lay.gstride;
  uint8_t* xs8 = smem + SM_WORK;                                       // [batch][token set][step][column][t][half][4]
  float2* gsum = reinterpret_cast<float2*>(smem + lay.gsum);          // [group][token] (s_x, s_x * sum_x)
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
#ifdef B2_STEP_TRACE
  long long tc_wait = 0, tc_comp = 0, tc_pump = 0, tc_red = 0, tc_units = 0;
  const long long tc_begin = clock64();
#define B2_TC(var, t0) var += clock64() - (t0)
#define B2_T0(name) const long long name = clock64()
#else
#define B2_TC(var, t0) do { } while (0)
#define B2_T0(name) do { } while (0)
#endif

  copy_staged(a, ph, lay, want_scales);
  if (!ph.active) return;
#ifdef B2_STEP_TRACE
  const long long tc_staged = clock64();
#endif

  const unsigned Bsl = (unsigned)L.npan * (unsigned)nbs;
  const int nslots = L.ks * L.fmax;
  const int usz = L.blk;
  // [warp][head | tail][token][32 rows]: in shared memory, or (more than eight rows) in this CTA's part of the global
  // tile scratch, written and read with L1-bypassing accesses on either side of a barrier of the worker warps
  const bool tiles_global = R > kStepSmallRows;
  float* tiles = tiles_global ? a.tile_scratch + (size_t)cta * kTileFloats : reinterpret_cast<float*>(smem + lay.tiles);
  unsigned* tile_panel = reinterpret_cast<unsigned*>(misc + MI_TILE);   // [warp][head | tail] panel of the tile, or none
  const int tile_f = R * 32;
  if (lane < 2) tile_panel[warp * 2 + lane] = 0xffffffffu;
  __syncwarp();

  EmitCtx ec;
  ec.nbs = (unsigned)nbs; ec.cps = (unsigned)L.cps; ec.Bsl = Bsl; ec.hi = ph.hi;
  ec.ci = ph.ci; ec.slice = ph.slice; ec.fmax = L.fmax; ec.n = L.n; ec.R = R; ec.nslots = nslots; ec.tp_off = tp_off;

  unsigned blk, whi;
  warp_range(ph, warp, blk, whi);
  int n_tiles = 0;
  B2_T0(tl0);
  while (blk < whi) {
    const unsigned p = blk / (unsigned)nbs;
    const int b0 = (int)(blk - p * (unsigned)nbs);
    const int b1 = (int)min(whi - p * (unsigned)nbs, (unsigned)nbs);
    float y[2][2 * NS];                       // [row block][2 set + (row g | row g + 8)], token t + 4 set
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int i = 0; i < 2 * NS; ++i) y[r][i] = 0.f;
#pragma unroll 1
    for (int b = b0; b < b1; ++b) {
      int freed = usz;
      if (ring.cpos + usz > kRingBytes) { freed += kRingBytes - ring.cpos; ring.cpos = 0; }
      B2_T0(tw0);
      if (!failed) {
        if (!mbar_wait_bounded(ring.bars_u + (ring.cidx % kRingBars) * 8, (ring.cidx / kRingBars) & 1u)) {
          atomicExch(a.status, (int)B2_ERR_TIMEOUT);
          failed = true;
        }
      }
      B2_TC(tc_wait, tw0);
      B2_T0(tc0);
      if (!failed) {
        const uint8_t* stg = ring.base + ring.cpos;
        // B operands: lane (g, t) feeds column g = (hi | lo) limb of token g / 2 of every token set.  Columns of tokens
        // past the last row hold whatever the staging area held before; a column only reaches its own outputs, and
        // those are never stored.
        const uint8_t* xb = xs8 + (size_t)b * xstride + (g * 4 + t) * 8;
        // both row blocks step by step: 2 NS independent integer-MMA chains in flight
        WFrag<BITS, GROUP> c0, c1;
        load_frag_smem<BITS, GROUP>(c0, stg, stg + 2 * L.wbatch, lane);
        load_frag_smem<BITS, GROUP>(c1, stg + L.wbatch, stg + 2 * L.wbatch + L.szb, lane);
#pragma unroll
        for (int gg = 0; gg < GPB; ++gg) {
          int acc[2][NS][4];
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int st = 0; st < NS; ++st)
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[r][st][i] = 0;
#pragma unroll
          for (int s8 = 0; s8 < SPG; ++s8) {
            const int s4 = gg * SPG + s8;
            uint32_t af0[4], af1[4];
            extract8<BITS, GROUP>(c0, s4, af0);
            extract8<BITS, GROUP>(c1, s4, af1);
#pragma unroll
            for (int st = 0; st < NS; ++st) {
              const uint2 bv = *reinterpret_cast<const uint2*>(xb + st * 1024 + s4 * 256);
              mma_u8s8_16832(acc[0][st], af0, bv.x, bv.y);
              mma_u8s8_16832(acc[1][st], af1, bv.x, bv.y);
            }
          }
#pragma unroll
          for (int st = 0; st < NS; ++st) {
            const float2 q = gsum[(b * GPB + gg) * gstride + t + 4 * st];
            gemv_scale(y[0][2 * st], y[0][2 * st + 1], acc[0][st], c0.sz[gg], q);
            gemv_scale(y[1][2 * st], y[1][2 * st + 1], acc[1][st], c1.sz[gg], q);
          }
        }
      }
      __syncwarp();
      B2_TC(tc_comp, tc0);
      B2_T0(tp0);
      ++ring.cidx;
      ring.cpos += usz;
      ring.cbytes += (unsigned)freed;
      if (lane == 0) {                      // the stage is free again: tell the producer warp
        __threadfence_block();
        ring.pub[1] = ring.cbytes;
        ring.pub[0] = ring.cidx;
      }
      B2_TC(tc_pump, tp0);
#ifdef B2_STEP_TRACE
      ++tc_units;
#endif
    }
    // the warp's sum over [b0, b1) of panel p goes to one of its two tiles: a piece that covers the whole panel is
    // final for this CTA and is flushed to the fragment slot at once (through the tail tile, which is still unused),
    // a head or tail piece stays in its tile for the reducer
    const bool full = b0 == 0 && b1 == nbs;
    float* mine = tiles + (size_t)(warp * 2 + (full ? 1 : n_tiles)) * tile_f;
#pragma unroll
    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
      for (int st = 0; st < NS; ++st)
        if (t + 4 * st < R) {
          float* d0 = mine + (t + 4 * st) * 32 + rb * 16 + g;
          if (tiles_global) { __stcg(d0, y[rb][2 * st]); __stcg(d0 + 8, y[rb][2 * st + 1]); }
          else { d0[0] = y[rb][2 * st]; d0[8] = y[rb][2 * st + 1]; }
        }
    __syncwarp();
    if (full) {
      flush_panel(a, ec, p, mine, tiles_global);
      __syncwarp();
    } else {
      if (lane == 0) tile_panel[warp * 2 + n_tiles] = p;
      ++n_tiles;
    }
    blk = p * (unsigned)nbs + (unsigned)b1;
  }
  B2_T0(tr0);
#ifdef B2_STEP_TRACE
  const long long tc_loop = tr0 - tl0, tc_pre = tl0 - tc_staged;
#endif
  workers_sync();
  reduce_tiles(a, ec, tiles, tiles_global);
  workers_sync();          // tiles and activations are reused by the next phase
  B2_TC(tc_red, tr0);
#ifdef B2_STEP_TRACE
  if (a.trace && blockIdx.x == 0 && lane == 0) {
    const long long tc_total = clock64() - tc_begin;
    unsigned long long* tr = a.trace + 4096 + ((size_t)a.trace[4095] * kStepWarps + warp) * 8;
    tr[0] = tc_staged - tc_begin; tr[1] = tc_wait; tr[2] = tc_comp; tr[3] = tc_pump; tr[4] = tc_red; tr[5] = tc_loop;
    tr[6] = tc_total; tr[7] = tc_pre;
  }
  workers_sync();
  if (a.trace && blockIdx.x == 0 && tid == 0) a.trace[4095] += 1;
#endif
}

// One copy of the format bodies serves the five call sites of the kernel (four linears per layer and the lm_head):
// inlined at every site the kernel would be five times as large and would miss the instruction cache at every stage.
template <int NS>
__device__ __noinline__ void gemv_phase(const StepArgs& a, int phase, Lay lay, WRing* ring_io, long tp_off, bool* failed_io) {
  extern __shared__ __align__(128) uint8_t smem[];
  WRing ring = *ring_io;
  bool failed = *failed_io;
  Phase ph;
  // The descriptor of this linear was copied to shared memory during the previous phase (its global load would sit in
  // front of everything else here); the first phase and the lm_head (kernel parameter) read theirs directly.  The
  // input is RMS-normed for qkv, gate / up and the lm_head: their finalize stages need the rows' 1 / rms.
  const bool want_scales = (phase & 1) == 0;
  uint4* dslot = reinterpret_cast<uint4*>(reinterpret_cast<float*>(smem + SM_MISC) + MI_DESC);
  if (phase == 0 || phase >= 4 * a.n_layers) {
    load_linear(a, phase, ph.lin);
  } else {
    const uint4* d4 = dslot + 4 * (phase & 1);
    decode_linear(d4[0], d4[1], d4[2], d4[3], ph.lin);
  }
  if (threadIdx.x < 4 && phase + 1 < 4 * a.n_layers) {
    cp_async16(smem_u32(dslot + 4 * ((phase + 1) & 1) + threadIdx.x), reinterpret_cast<const uint4*>(linear_of(a, phase + 1)) + threadIdx.x);
    cp_async_commit();
  }
  split_phase(ph, blockIdx.x);
#define B2_STEP_BODY(B, G) gemv_body<B, G, NS>(a, ph, smem, lay, ring, tp_off, failed, want_scales)
  switch (ph.lin.bits * 1000 + ph.lin.group) {
    case 4128: B2_STEP_BODY(4, 128); break;
    case 4064: B2_STEP_BODY(4, 64); break;
    case 3128: B2_STEP_BODY(3, 128); break;
    case 3064: B2_STEP_BODY(3, 64); break;
    case 2128: B2_STEP_BODY(2, 128); break;
    default: B2_STEP_BODY(2, 64); break;
  }
#undef B2_STEP_BODY
  if (threadIdx.x < 4) cp_async_wait<0>();      // the next descriptor has landed long ago; the stages' barriers publish it
  *ring_io = ring;
  *failed_io = failed;
}

// Sum of the fragments of output element (tok, col) of a linear, in (rank,) slice, fragment order.
__device__ __forceinline__ float sum_local(const StepArgs& a, const StepLinear& L, int tok, size_t col) {
  const int nslots = L.ks * L.fmax, R = a.n_rows;
  float s = 0.f;
  const float* p = a.part + (size_t)tok * L.n + col;
  const size_t st = (size_t)R * L.n;
#pragma unroll 1
  for (int sl = 0; sl < nslots; sl += 4) {      // four loads in flight; the sum keeps its order
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = sl + j < nslots ? __ldcg(p + (size_t)(sl + j) * st) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) if (sl + j < nslots) s += v[j];
  }
  return s;
}
__device__ __forceinline__ float2 sum_local2(const StepArgs& a, const StepLinear& L, int tok, size_t col) {
  const int nslots = L.ks * L.fmax, R = a.n_rows;
  float2 s = make_float2(0.f, 0.f);
  const float* p = a.part + (size_t)tok * L.n + col;
  const size_t st = (size_t)R * L.n;
#pragma unroll 1
  for (int sl = 0; sl < nslots; sl += 4) {
    float2 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = sl + j < nslots ? __ldcg(reinterpret_cast<const float2*>(p + (size_t)(sl + j) * st)) : make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j) if (sl + j < nslots) { s.x += v[j].x; s.y += v[j].y; }
  }
  return s;
}

// Four consecutive output elements at once (col a multiple of four).
__device__ __forceinline__ float4 sum_local4(const StepArgs& a, const StepLinear& L, int tok, size_t col) {
  const int nslots = L.ks * L.fmax, R = a.n_rows;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* p = a.part + (size_t)tok * L.n + col;
  const size_t st = (size_t)R * L.n;
#pragma unroll 1
  for (int sl = 0; sl < nslots; sl += 4) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      v[j] = sl + j < nslots ? __ldcg(reinterpret_cast<const float4*>(p + (size_t)(sl + j) * st)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (sl + j < nslots) { s.x += v[j].x; s.y += v[j].y; s.z += v[j].z; s.w += v[j].w; }
  }
  return s;
}

// ---------------------------------------------------------------------------------------------------- finalize stages
// The stages that produce the input of a linear work by (token, 128-column batch) items, one warp each, lane = four
// columns, and hand their values to quant_store.  `nw` is the RMS-norm weight of the consuming linear (or null),
// `group` its quantisation group.
// h = embedding rows of the step's tokens (and their staged form for the first qkv)
__device__ __noinline__ void fin_embed(const StepArgs& a, const int* row_ids, Lay lay, const bf16* nw, int group) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = a.d_model >> 7;
  const int items = a.n_rows * nb;
  for (int it = warp * gridDim.x + blockIdx.x; it < items; it += gridDim.x * kStepWarps) {
    const int tok = it / nb, b = it - tok * nb;
    int id = row_ids[tok];
    if (id < 0 || id >= a.vocab) { atomicExch(a.status, (int)B2_ERR_BOUNDS); id = 0; }
    const size_t c = (size_t)b * 128 + lane * 4;
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(a.embed + (size_t)id * a.d_model + c));
    *reinterpret_cast<uint2*>(a.h + (size_t)tok * a.d_model + c) = raw;
    const uint2 wr = __ldg(reinterpret_cast<const uint2*>(nw + c));
    const bf16* hb = reinterpret_cast<const bf16*>(&raw);
    const bf16* wb = reinterpret_cast<const bf16*>(&wr);
    float h[4], sq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { h[i] = __bfloat162float(hb[i]); sq = fmaf(h[i], h[i], sq); }
    quant_store(a, lay.xs_stride, lay.gstride, group, tok, b, h[0] * __bfloat162float(wb[0]), h[1] * __bfloat162float(wb[1]),
                h[2] * __bfloat162float(wb[2]), h[3] * __bfloat162float(wb[3]), true, sq, nb);
  }
}

// qkv fragments -> bf16 row -> RoPE on q and k -> q buffer / paged KV store.  One warp per (row, head).
__device__ __noinline__ void fin_qkv(const StepArgs& a, const StepLayer* ly, const int* row_pos, const int* row_seq,
                                        const int* row_rope) {
  extern __shared__ __align__(128) uint8_t smem[];
  const float* inv_rms = reinterpret_cast<const float*>(smem + SM_MISC);
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
    const float ir = inv_rms[tok];
    lo.x = bf16_round(lo.x * ir); lo.y = bf16_round(lo.y * ir); hi.x = bf16_round(hi.x * ir); hi.y = bf16_round(hi.y * ir);
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

// h = bf16(h + sum of the fragments of a row-parallel linear over all ranks), and its staged form for the next linear
__device__ __noinline__ void fin_resid(const StepArgs& a, const StepLinear* Lg, long tp_off, Lay lay, const bf16* nw, int group) {
  StepLinear L;
  fetch_linear(Lg, L);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = L.n, R = a.n_rows, nslots = L.ks * L.fmax;
  const int nb = n >> 7;
  const int items = R * nb;
  const float* own = tp_off >= 0 ? a.xreg[a.tp_rank] + tp_off : nullptr;
  for (int it = warp * gridDim.x + blockIdx.x; it < items; it += gridDim.x * kStepWarps) {
    const int tok = it / nb, b = it - tok * nb;
    const size_t c = (size_t)b * 128 + lane * 4;
    float4 s;
    if (tp_off < 0) {
      s = sum_local4(a, L, tok, c);
    } else {
      s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
      for (int r = 0; r < a.tp_size; ++r)
#pragma unroll 4
        for (int sl = 0; sl < nslots; ++sl) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(own + (((size_t)r * nslots + sl) * R + tok) * n + c));
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
    }
    bf16* hp = a.h + (size_t)tok * a.d_model + c;
    const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(hp));
    const bf16* hb = reinterpret_cast<const bf16*>(&raw);
    __nv_bfloat162 o01 = __floats2bfloat162_rn(s.x + __bfloat162float(hb[0]), s.y + __bfloat162float(hb[1]));
    __nv_bfloat162 o23 = __floats2bfloat162_rn(s.z + __bfloat162float(hb[2]), s.w + __bfloat162float(hb[3]));
    uint2 outw;
    outw.x = *reinterpret_cast<uint32_t*>(&o01);
    outw.y = *reinterpret_cast<uint32_t*>(&o23);
    *reinterpret_cast<uint2*>(hp) = outw;
    const uint2 wr = __ldg(reinterpret_cast<const uint2*>(nw + c));
    const bf16* wb = reinterpret_cast<const bf16*>(&wr);
    const float h0 = __low2float(o01), h1 = __high2float(o01), h2 = __low2float(o23), h3 = __high2float(o23);
    const float sq = fmaf(h0, h0, fmaf(h1, h1, fmaf(h2, h2, h3 * h3)));
    quant_store(a, lay.xs_stride, lay.gstride, group, tok, b, h0 * __bfloat162float(wb[0]), h1 * __bfloat162float(wb[1]),
                h2 * __bfloat162float(wb[2]), h3 * __bfloat162float(wb[3]), true, sq, nb);
  }
}

// act = bf16(silu(bf16 gate) * bf16 up) and its staged form for down_proj; gate / up rows are interleaved in blocks of 8
// inside every 16-row block, and the sums carry the 1 / rms of the normed input
__device__ __noinline__ void fin_swiglu(const StepArgs& a, const StepLinear* Lg, Lay lay, int group) {
  extern __shared__ __align__(128) uint8_t smem[];
  const float* inv_rms = reinterpret_cast<const float*>(smem + SM_MISC);
  StepLinear L;
  fetch_linear(Lg, L);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = L.n >> 1, R = a.n_rows;
  const int nb = f >> 7;
  const int items = R * nb;
  for (int it = warp * gridDim.x + blockIdx.x; it < items; it += gridDim.x * kStepWarps) {
    const int tok = it / nb, b = it - tok * nb;
    const int j = b * 128 + lane * 4;
    const size_t grow = (size_t)(j >> 3) * 16 + (j & 7);
    const float4 g4 = sum_local4(a, L, tok, grow);
    const float4 u4 = sum_local4(a, L, tok, grow + 8);
    const float ir = inv_rms[tok];
    const float gt[4] = {g4.x, g4.y, g4.z, g4.w}, up[4] = {u4.x, u4.y, u4.z, u4.w};
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = bf16_round(silu_f(bf16_round(gt[i] * ir)) * bf16_round(up[i] * ir));
    uint2 outw;
    __nv_bfloat162 o01 = __floats2bfloat162_rn(v[0], v[1]), o23 = __floats2bfloat162_rn(v[2], v[3]);
    outw.x = *reinterpret_cast<uint32_t*>(&o01);
    outw.y = *reinterpret_cast<uint32_t*>(&o23);
    *reinterpret_cast<uint2*>(a.act + (size_t)tok * f + j) = outw;
    quant_store(a, lay.xs_stride, lay.gstride, group, tok, b, v[0], v[1], v[2], v[3], false, 0.f, nb);
  }
}

// One attention work item (query group, kv head, 16-row tile, run of `spi` consecutive kv splits) on one warp: the
// pages of the run stream through one pipeline and the query fragments are loaded once, while every split still gets
// its own partial (accumulators restart at each split boundary), so the partials do not depend on the run length; the arithmetic of
// attn_decode_kernel<128, false> (attn_decode.cu) with an ST-stage K/V ring in this warp's shared memory.
// LOW8: every group of the step has at most eight (token, head) rows per KV head (plain decode rows with eight query
// heads per KV head), so rows 8..15 of the MMA tile are padding.  Their query fragments, scores and output
// accumulators are then not kept (zeros go in, the results are dropped): half the accumulator registers, which is what
// keeps this stage free of local-memory spills; rows 0..7 see exactly the same MMA operations either way.
template <bool LOW8>
__device__ __forceinline__ void mma_rows(float (&d)[LOW8 ? 2 : 4], const uint32_t (&a4)[4], uint32_t b0, uint32_t b1) {
  if (LOW8) {
    float t[4] = {d[0], d[1], 0.f, 0.f};
    mma_bf16_16816(t, a4, b0, b1);
    d[0] = t[0]; d[1] = t[1];
  } else {
    float t[4] = {d[0], d[1], d[LOW8 ? 0 : 2], d[LOW8 ? 1 : 3]};
    mma_bf16_16816(t, a4, b0, b1);
    d[0] = t[0]; d[1] = t[1]; d[LOW8 ? 0 : 2] = t[2]; d[LOW8 ? 1 : 3] = t[3];
  }
}

template <int ST, bool LOW8>
__device__ __forceinline__ void attn_item(const StepArgs& a, const bf16* kv_pool, long item, int split0, int spi, int mt_max,
                                          uint8_t* wsm, const int* row_pos, const int* row_seq) {
  constexpr int HD = 128, KS = HD / 16, NTO = HD / 8, ROWB = HD * 2, CPR = ROWB / 16, PAGE_B = kPage * ROWB;
  constexpr int NR = LOW8 ? 1 : 2;           // row halves of the tile that are kept (rows g, g + 8)
  constexpr int NA = LOW8 ? 2 : 4;           // accumulator registers per n-tile
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int gq = a.hq / a.hkv;
  const int mtile = (int)(item % mt_max); item /= mt_max;
  const int kvh = (int)(item % a.hkv); item /= a.hkv;
  const int grp = (int)item;
  const int tok0 = a.grp_tok0[grp], cnt = a.grp_cnt[grp];
  if (mtile * 16 >= cnt * gq) return;
  const int seq = row_seq[tok0];
  const int pos_first = row_pos[tok0];
  const int kv_len = row_pos[tok0 + cnt - 1] + 1;
  const int k_begin = split0 * a.split_keys;
  if (k_begin >= kv_len) return;
  const int k_end = min(kv_len, k_begin + spi * a.split_keys);
  const int n_pg = (k_end - k_begin + kPage - 1) / kPage;
  const int pps = a.split_keys / kPage;                      // pages per split

  int rtok[NR], rhead[NR], rpos[NR];
  bool rvalid[NR];
  unsigned rmask[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
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

  // page numbers of the whole run up front (at most 16 splits x 4 pages): lane i holds pages i and i + 32, so that the
  // page loop has no dependent global load in front of its copies
  const int pg_lo = lane < n_pg ? bt[(k_begin / kPage) + lane] : 0;
  const int pg_hi = lane + 32 < n_pg ? bt[(k_begin / kPage) + lane + 32] : 0;
  auto issue_page = [&](int pi) {
    const int stage = pi % ST;
    int page = pi < 32 ? __shfl_sync(0xffffffffu, pg_lo, pi) : (pi < 64 ? __shfl_sync(0xffffffffu, pg_hi, pi - 32) : bt[(k_begin / kPage) + pi]);
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
#pragma unroll
  for (int pi = 0; pi < ST - 1; ++pi) {
    if (pi < n_pg) issue_page(pi);
    cp_async_commit();
  }

  uint32_t qa[KS][2 * NR];                   // [ks][row half][k half]: A registers (a0, a2) of row g, (a1, a3) of row g + 8
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      uint32_t v0 = 0u, v1 = 0u;
      if (rvalid[i]) {
        const bf16* qp = a.q + (size_t)rtok[i] * a.hq * HD + (size_t)rhead[i] * HD + ks * 16 + 2 * t;
        v0 = __ldcg(reinterpret_cast<const unsigned*>(qp));
        v1 = __ldcg(reinterpret_cast<const unsigned*>(qp + 8));
      }
      qa[ks][2 * i] = v0;
      qa[ks][2 * i + 1] = v1;
    }
  }
  float o[NTO][NA];
#pragma unroll
  for (int n = 0; n < NTO; ++n)
#pragma unroll
    for (int i = 0; i < NA; ++i) o[n][i] = 0.f;
  float mrow[NR], lrow[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) { mrow[r] = -INFINITY; lrow[r] = 0.f; }

#ifdef B2_STEP_TRACE
  long long ta_issue = 0, ta_wait = 0, ta_comp = 0;
  const long long ta_begin = clock64();
#endif
  for (int pi = 0; pi < n_pg; ++pi) {
#ifdef B2_STEP_TRACE
    const long long tq0 = clock64();
#endif
    if (pi + ST - 1 < n_pg) issue_page(pi + ST - 1);
    cp_async_commit();
#ifdef B2_STEP_TRACE
    const long long tq1 = clock64();
#endif
    cp_async_wait<ST - 1>();
    __syncwarp();
#ifdef B2_STEP_TRACE
    const long long tq2 = clock64();
    ta_issue += tq1 - tq0; ta_wait += tq2 - tq1;
#endif
    const int stage = pi % ST;
    const uint32_t ks_u = wsm_u + stage * 2 * PAGE_B, vs_u = ks_u + PAGE_B;
    float s[2][NA];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < NA; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b[4];
      const int j = lane >> 3;
      const int key = (j >> 1) * 8 + (lane & 7);
      const int cc = 2 * ks + (j & 1);
      ldsm_x4(ks_u + key * ROWB + ((cc ^ (key & 7)) << 4), b);
      const uint32_t a4[4] = {qa[ks][0], LOW8 ? 0u : qa[ks][LOW8 ? 0 : 2], qa[ks][1], LOW8 ? 0u : qa[ks][LOW8 ? 1 : 3]};
      mma_rows<LOW8>(s[0], a4, b[0], b[1]);
      mma_rows<LOW8>(s[1], a4, b[2], b[3]);
    }
    const int kb = k_begin + pi * kPage;
    float mx[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) mx[r] = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < NA; ++i) {
        const int r = i >> 1;
        const int key = kb + n * 8 + 2 * t + (i & 1);
        bool ok = key <= rpos[r];
        if (ok && key >= pos_first) ok = (rmask[r] >> (key - pos_first)) & 1u;
        const float v = ok ? s[n][i] * a.scale_log2 : -INFINITY;
        s[n][i] = v;
        mx[r] = fmaxf(mx[r], v);
      }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[NR], psum[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      psum[r] = 0.f;
      const float mnew = fmaxf(mrow[r], mx[r]);
      corr[r] = (mnew == -INFINITY) ? 1.f : exp2f(mrow[r] - mnew);
      mrow[r] = mnew;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < NA; ++i) {
        const int r = i >> 1;
        const float p = (s[n][i] == -INFINITY) ? 0.f : exp2f(s[n][i] - mrow[r]);
        s[n][i] = p;
        psum[r] += p;
      }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      lrow[r] = lrow[r] * corr[r] + psum[r];
    }
#pragma unroll
    for (int n = 0; n < NTO; ++n)
#pragma unroll
      for (int i = 0; i < NA; ++i) o[n][i] *= corr[i >> 1];
    uint32_t pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = LOW8 ? 0u : pack_bf16(s[0][LOW8 ? 0 : 2], s[0][LOW8 ? 1 : 3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = LOW8 ? 0u : pack_bf16(s[1][LOW8 ? 0 : 2], s[1][LOW8 ? 1 : 3]);
#pragma unroll
    for (int nn = 0; nn < NTO / 2; ++nn) {
      uint32_t b[4];
      const int j = lane >> 3;
      const int key = (j & 1) * 8 + (lane & 7);
      const int cc = 2 * nn + (j >> 1);
      ldsm_x4_t(vs_u + key * ROWB + ((cc ^ (key & 7)) << 4), b);
      mma_rows<LOW8>(o[2 * nn], pa, b[0], b[1]);
      mma_rows<LOW8>(o[2 * nn + 1], pa, b[2], b[3]);
    }
    __syncwarp();
    // end of a split (or of the run): its partial goes out and the accumulators restart
    if ((pi + 1) % pps == 0 || pi + 1 == n_pg) {
      const int split = split0 + pi / pps;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
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
#pragma unroll
      for (int n = 0; n < NTO; ++n)
#pragma unroll
        for (int i = 0; i < NA; ++i) o[n][i] = 0.f;
#pragma unroll
      for (int r = 0; r < NR; ++r) { mrow[r] = -INFINITY; lrow[r] = 0.f; }
    }
#ifdef B2_STEP_TRACE
    ta_comp += clock64() - tq2;
#endif
  }
  cp_async_wait<0>();
  __syncwarp();
#ifdef B2_STEP_TRACE
  if (a.trace && blockIdx.x == 0 && lane == 0) {
    unsigned long long* tr = a.trace + 200000 + (threadIdx.x >> 5) * 8;
    tr[0] += (unsigned long long)ta_issue; tr[1] += (unsigned long long)ta_wait; tr[2] += (unsigned long long)ta_comp;
    tr[3] += (unsigned long long)n_pg; tr[4] += 1ull; tr[5] += (unsigned long long)(clock64() - ta_begin);
  }
#endif
}

template <int ST, bool LOW8>
__device__ __noinline__ void attn_phase_v(const StepArgs& a, const bf16* kv_pool, uint8_t* smem, const int* row_pos,
                                          const int* row_seq, int max_pos, int max_cnt, int* ctr) {
  const int warp = threadIdx.x >> 5;
  const int n_warps = attn_warps(a.n_rows) * (ST == 1 ? 2 : 1);
  if (warp >= n_warps) return;
  const int gq = a.hq / a.hkv;
  const int mt_max = (max_cnt * gq + 15) / 16;
  const int n_sp = min(a.max_splits, max_pos / a.split_keys + 1);
  const long per_grp = (long)a.hkv * mt_max;
  // An item sets up once (row description, page lookups, query fragments: a chain of a few microseconds), so long
  // contexts give an item a run of consecutive splits: about four items per attention warp of the grid, at most 16 splits.
  const long slots = (long)gridDim.x * n_warps;
  const long all_splits = (long)a.n_groups * per_grp * n_sp;
  int spi = (int)min(16l, max(1l, all_splits / (4 * slots)));
  const int n_run = (n_sp + spi - 1) / spi;
  const long items = (long)a.n_groups * per_grp * n_run;
  uint8_t* wsm = smem + SM_WORK + (size_t)warp * ST * 2 * kPage * 128 * 2;
  // Items are handed out by a counter (one per layer, back at zero when the kernel ends): which warp computes an item
  // does not change its result, and a warp that drew short items simply draws more.
  for (;;) {
    long it = 0;
    if ((threadIdx.x & 31) == 0) it = (long)atomicAdd(ctr, 1);
    it = __shfl_sync(0xffffffffu, it, 0);
    if (it >= items) break;
    // item order: run fastest, so that the items of one (group, head) spread over the CTAs
    const long outer = it / n_run;
    const int run = (int)(it - outer * n_run);
    attn_item<ST, LOW8>(a, kv_pool, outer, run * spi, min(spi, n_sp - run * spi), mt_max, wsm, row_pos, row_seq);
  }
}

__device__ __forceinline__ void attn_phase(const StepArgs& a, const bf16* kv_pool, uint8_t* smem, const int* row_pos,
                                           const int* row_seq, int* ctr) {
  // splits that any row of this step can reach, and rows of the largest group (one for plain decode rows)
  int max_pos = 0, max_cnt = 1;
  for (int i = 0; i < a.n_rows; ++i) max_pos = max(max_pos, row_pos[i]);
  for (int i = 0; i < a.n_groups; ++i) max_cnt = max(max_cnt, a.grp_cnt[i]);
  const int gq = a.hq / a.hkv;
  const long all_splits = (long)a.n_groups * a.hkv * ((max_cnt * gq + 15) / 16) * min(a.max_splits, max_pos / a.split_keys + 1);
  const bool wide = all_splits > (long)gridDim.x * attn_warps(a.n_rows);      // more items than base warps: one stage, twice the warps
  // plain decode rows with at most eight query heads per KV head: the upper half of every 16-row tile is padding
  const bool low8 = max_cnt * gq <= 8;
  if (wide) {
    if (low8) attn_phase_v<1, true>(a, kv_pool, smem, row_pos, row_seq, max_pos, max_cnt, ctr);
    else attn_phase_v<1, false>(a, kv_pool, smem, row_pos, row_seq, max_pos, max_cnt, ctr);
  } else {
    if (low8) attn_phase_v<2, true>(a, kv_pool, smem, row_pos, row_seq, max_pos, max_cnt, ctr);
    else attn_phase_v<2, false>(a, kv_pool, smem, row_pos, row_seq, max_pos, max_cnt, ctr);
  }
}

// Merge of the attention splits of every (row, q head): one warp per item, lane = four output dimensions; the
// splits are added in ascending order and their loads do not depend on one another, so they are all in flight at once.
__device__ __noinline__ void fin_merge(const StepArgs& a, const int* row_pos, Lay lay, int group) {
  constexpr int HD = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = a.n_rows * a.hq;
  for (int item = warp * gridDim.x + blockIdx.x; item < items; item += gridDim.x * kStepWarps) {
    const int tok = item / a.hq, head = item - tok * a.hq;
    const int ns = (row_pos[tok] + a.split_keys) / a.split_keys;
    const float* po = a.part_o + ((size_t)tok * a.hq + head) * a.max_splits * HD + lane * 4;
    const float2* pm = reinterpret_cast<const float2*>(a.part_ml + ((size_t)tok * a.hq + head) * a.max_splits * 2);
    float M = -INFINITY;
    for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(pm + s).x);
    M = warp_max(M);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float Ls = 0.f;
    for (int s0 = 0; s0 < ns; s0 += 8) {
      float2 ml[8];
      float4 pv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int sidx = min(s0 + j, ns - 1);
        ml[j] = __ldcg(pm + sidx);
        pv[j] = __ldcg(reinterpret_cast<const float4*>(po + (size_t)sidx * HD));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (s0 + j >= ns || ml[j].x == -INFINITY) continue;
        const float wt = exp2f(ml[j].x - M);
        Ls = fmaf(ml[j].y, wt, Ls);
        acc.x = fmaf(pv[j].x, wt, acc.x);
        acc.y = fmaf(pv[j].y, wt, acc.y);
        acc.z = fmaf(pv[j].z, wt, acc.z);
        acc.w = fmaf(pv[j].w, wt, acc.w);
      }
    }
    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
    bf16* out = a.attn + (size_t)tok * a.hq * HD + (size_t)head * HD + lane * 4;
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(__fmul_rn(acc.x, inv), __fmul_rn(acc.y, inv));
    const __nv_bfloat162 o23 = __floats2bfloat162_rn(__fmul_rn(acc.z, inv), __fmul_rn(acc.w, inv));
    *reinterpret_cast<__nv_bfloat162*>(out) = o01;
    *reinterpret_cast<__nv_bfloat162*>(out + 2) = o23;
    // one head = one 128-k batch of o_proj's input
    quant_store(a, lay.xs_stride, lay.gstride, group, tok, head, __low2float(o01), __high2float(o01), __low2float(o23), __high2float(o23),
                false, 0.f, a.hq);
  }
}

// lm_head fragments -> (optional fp32 logits) -> per-CTA (max, argmax) of every row; lowest index wins ties
__device__ __noinline__ void fin_argmax_cta(const StepArgs& a, uint8_t* smem) {
  const StepLinear& L = a.lm_head;
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
  float* sv = misc + MI_AV;
  int* si = reinterpret_cast<int*>(misc + MI_AI);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = a.n_rows;
  const float* inv_rms = misc;
  for (int tok = 0; tok < R; ++tok) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const float ir = inv_rms[tok];
    for (int c = blockIdx.x * kStepThreads + threadIdx.x; c < L.n; c += gridDim.x * kStepThreads) {
      const float v = sum_local(a, L, tok, (size_t)c) * ir;
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
  workers_sync();
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
__device__ __noinline__ void argmax_over_ctas(const StepArgs& a, int tok, float& best, int& bi) {
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

// NS = token sets of four rows the GEMV phases carry (1, 2 or 4): one instance of the kernel per value, each in a
// translation unit of its own (step_kernel_r4.cu, _r8.cu, _r16.cu), so that the three compile side by side.
template <int NS>
__global__ void __launch_bounds__(kStepBlock, 1) step_kernel(const __grid_constant__ StepArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  float* misc = reinterpret_cast<float*>(smem + SM_MISC);
  int* row_ids = reinterpret_cast<int*>(misc + MI_ROW);
  int* row_pos = row_ids + kStepMaxRows;
  int* row_seq = row_ids + 2 * kStepMaxRows;
  int* row_rope = row_ids + 3 * kStepMaxRows;

  if (warp < kStepWarps && lane == 0) {
    const uint32_t bars = smem_u32(smem + SM_BARS) + warp * kRingBars * 8;
#pragma unroll
    for (int i = 0; i < kRingBars; ++i) mbar_init(bars + i * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    volatile unsigned* pub = reinterpret_cast<volatile unsigned*>(misc) + MI_PUB + 2 * warp;
    pub[0] = 0u; pub[1] = 0u;
  }
  __syncthreads();          // the only CTA-wide barrier: rings are initialised before the producer warp starts
  const Lay lay = make_lay(a.n_rows, a.slice_k);
  if (warp == kStepWarps) {
    producer_loop(a, smem, cta, lay);     // weights do not depend on anything: start streaming at once
    return;
  }

  WRing ring;
  ring.base = smem + lay.ring + (size_t)warp * lay.ring_w;
  ring.bars_u = smem_u32(smem + SM_BARS) + warp * kRingBars * 8;
  ring.cidx = 0; ring.cbytes = 0; ring.cpos = 0;
  ring.pub = reinterpret_cast<volatile unsigned*>(misc) + MI_PUB + 2 * warp;
  SyncState ss;
  ss.local_target = a.sync[1];
  ss.cross_target = a.sync[2];
  ss.ev = 0;
  B2_STAMP(a, ss);
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
  workers_sync();
  bool failed = false;

  fin_embed(a, row_ids, lay, a.n_layers ? a.layers[0].ln1 : a.final_norm, a.n_layers ? a.layers[0].qkv.group : a.lm_head.group);
  grid_sync(a, ss);
  const bool tp = a.tp_size > 1;
  for (int l = 0; l < a.n_layers; ++l) {
    const StepLayer* ly = a.layers + l;
    gemv_phase<NS>(a, 4 * l, lay, &ring, -1, &failed);
    grid_sync(a, ss);
    fin_qkv(a, ly, row_pos, row_seq, row_rope);
    grid_sync(a, ss);
    attn_phase(a, ly->kv_pool, smem, row_pos, row_seq, a.attn_ctr + l);
    grid_sync(a, ss);
    if (cta == 0 && tid == 0) a.attn_ctr[l] = 0;          // every CTA is past its last draw: ready for the next launch
    fin_merge(a, row_pos, lay, ly->o.group);
    grid_sync(a, ss);
    gemv_phase<NS>(a, 4 * l + 1, lay, &ring, tp ? a.x_off[0] : -1, &failed);
    cross_sync(a, ss);
    fin_resid(a, &ly->o, tp ? a.x_off[0] : -1, lay, ly->ln2, ly->gate_up.group);
    grid_sync(a, ss);
    gemv_phase<NS>(a, 4 * l + 2, lay, &ring, -1, &failed);
    grid_sync(a, ss);
    fin_swiglu(a, &ly->gate_up, lay, ly->down.group);
    grid_sync(a, ss);
    gemv_phase<NS>(a, 4 * l + 3, lay, &ring, tp ? a.x_off[1] : -1, &failed);
    cross_sync(a, ss);
    {
      const bool last = l + 1 == a.n_layers;
      fin_resid(a, &ly->down, tp ? a.x_off[1] : -1, lay, last ? a.final_norm : ly[1].ln1, last ? a.lm_head.group : ly[1].qkv.group);
    }
    grid_sync(a, ss);
  }
  gemv_phase<NS>(a, 4 * a.n_layers, lay, &ring, -1, &failed);
  grid_sync(a, ss);
  fin_argmax_cta(a, smem);
  grid_sync(a, ss);
  // winners: CTA 0, one warp per row; under tensor parallelism every rank's candidate travels to every rank
  if (tp) {
    if (cta == 0)
      for (int tok = warp; tok < a.n_rows; tok += kStepWarps) {
        float best; int bi;
        argmax_over_ctas(a, tok, best, bi);
        if (lane == 0)
          for (int r = 0; r < a.tp_size; ++r) {
            float* slot = a.xreg[r] + a.x_amax + ((size_t)a.tp_rank * kStepMaxRows + tok) * 2;
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
  } else if (cta == 0) {
    for (int tok = warp; tok < a.n_rows; tok += kStepWarps) {
      float best; int bi;
      argmax_over_ctas(a, tok, best, bi);
      if (lane == 0) {
        a.out_ids[tok] = bi; a.out_val[tok] = best;
        if (a.slot_seq) { a.last_ids[tok] = bi; a.seq_len[row_seq[tok]] = row_pos[tok] + 1; }
      }
    }
  }
  if (cta == 0 && tid == 0) { a.sync[1] = ss.local_target; a.sync[2] = ss.cross_target; }
  if (failed) {
    // give copies still in flight a bounded chance to land before the CTA's shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) { }
  }
}


// Host side of one instance: occupancy check and cooperative launch.
template <int NS>
inline int step_prepare() {
  int occ = 0;
  if (cudaFuncSetAttribute(step_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, step_kernel<NS>, kStepBlock, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
  return occ >= 1 ? B2_OK : B2_ERR_LAUNCH;
}

template <int NS>
inline int step_launch_instance(const StepArgs& a, int ncta, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(step_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL) != cudaSuccess) return B2_ERR_LAUNCH;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ncta, 1, 1);
  cfg.blockDim = dim3(kStepBlock, 1, 1);
  cfg.dynamicSmemBytes = SM_TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, step_kernel<NS>, a) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

}  // namespace b2
