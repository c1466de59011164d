// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = A[M,K] * B[N,K]^T (+ residual), fp32 accumulation in TMEM.
//
// Prefill / large-batch linears: A = activations, B = weights dequantised to bf16 (wq_dequant) or bf16 weights.
// Replaces the reference's cuBLAS path for every prefill GEMM (kernels/src/bf16_linear.cu:54-110, engine call site
// kernels/m1/m1_model.cu:1875-1895).
//
// One CTA computes a 128 x 256 tile.  Warp 0 feeds a 4-stage shared-memory ring with TMA (cp.async.bulk.tensor, 128-byte
// swizzle, every CTA loads its own tiles); one elected thread of warp 1 issues tcgen05.mma (M 128, N 256, K 16 per instruction, operands
// read through shared-memory descriptors, accumulator = 256 TMEM columns) and commits stage releases and the final
// "accumulator ready" arrival to mbarriers; warps 2..5 read the accumulator back with tcgen05.ld (each warp owns the
// 32 TMEM lanes its warp id modulo 4 selects), add the optional residual, convert and store.
// Every mbarrier wait is bounded; on expiry the CTA records B2_ERR_TIMEOUT, still frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace b2 {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStagesG = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kGemmThreads = 192;             // 6 warps
constexpr int kTmemCols = 256;

__device__ __forceinline__ void mbar_init_g(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_g(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_g(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait (about two seconds); false = gave up.
__device__ __forceinline__ bool mbar_wait_g(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_g(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait_g(bar, parity)) {
    if (globaltimer_ns() - t0 > 2000000000ull) return false;
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                               // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D fp32, A/B bf16, both K-major, N / 8 and M / 16.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

struct GemmArgs {
  int M, N, K;
  bf16* D; long ldd;          // bf16 output (or null)
  float* Df;                  // fp32 output (or null), same ldd
  const bf16* R; long ldr;    // optional residual added in fp32 before rounding
  int* status;
  // Fused reduce-scatter (tensor-parallel row-parallel linears): the fp32 partial tile goes straight into the inbox slot
  // of the rank that owns its rows (rows_per_rank consecutive rows per rank), over NVLink for a peer, with plain stores,
  // while the other tiles are still being computed.  push[r] = rank r's inbox + slot + this rank's lane inside the slot.
  float* push[8];
  int push_ranks;             // 0: off
  int rows_per_rank;
};

}  // namespace

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_g[];
  __shared__ __align__(8) uint64_t full_bar[kStagesG], empty_bar[kStagesG], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1024-byte aligned base of the ring (the swizzle pattern is anchored at 1024-byte boundaries)
  const uint32_t ring = (smem_u32(smem_g) + 1023u) & ~1023u;
  // Tile order: groups of up to 16 row tiles sweep the column tiles together, row tile fastest, so that CTAs resident at
  // the same time share B tiles (weights) and the group's A rows stay in L2; B is then read from DRAM about once per
  // group instead of once per row tile.
  const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
  constexpr int kGroupM = 16;
  const int per_group = kGroupM * tiles_n;
  const int grp = (int)blockIdx.x / per_group;
  const int gm = min(kGroupM, tiles_m - grp * kGroupM);
  const int in_grp = (int)blockIdx.x - grp * per_group;
  const int tile_m = grp * kGroupM + in_grp % gm, tile_n = in_grp / gm;
  const int nkb = (g.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStagesG; ++i) { mbar_init_g(smem_u32(&full_bar[i]), 1); mbar_init_g(smem_u32(&empty_bar[i]), 1); }
    mbar_init_g(smem_u32(&acc_bar), 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % kStagesG;
        if (kb >= kStagesG && !mbar_wait_g(smem_u32(&empty_bar[s]), ((kb / kStagesG) - 1) & 1)) { atomicExch(&s_failed, 1); break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        mbar_expect_tx_g(bar, STAGE_BYTES);
        const uint32_t sa = ring + s * STAGE_BYTES, sb = sa + A_BYTES;
        tma_load_2d(sa, &map_a, kb * BK, tile_m * BM, bar);
        tma_load_2d(sb, &map_b, kb * BK, tile_n * BN, bar);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % kStagesG;
        if (!mbar_wait_g(smem_u32(&full_bar[s]), (kb / kStagesG) & 1)) { atomicExch(&s_failed, 1); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = ring + s * STAGE_BYTES, sb = sa + A_BYTES;
        const uint64_t da = make_desc_sw128(sa), db = make_desc_sw128(sb);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // advancing K by 16 bf16 = 32 bytes inside the 128-byte swizzle atom: +2 in the (>>4) start address field
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty_bar[s]));     // frees the stage once these MMAs have read it
      }
      umma_commit(smem_u32(&acc_bar));            // accumulator complete (arrives even after a failed wait)
    }
  } else {
    // ---------------- epilogue: warps 2..5, TMEM lanes 32 * (warp % 4) ----------------
    const bool ok = mbar_wait_g(smem_u32(&acc_bar), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!ok) atomicExch(&s_failed, 1);
    const int lane_base = (warp & 3) * 32;
    const int row = tile_m * BM + lane_base + lane;
    if (ok && !s_failed) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col = tile_n * BN + c0;
        if (row < g.M && col < g.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (g.R) {
            const bf16* rp = g.R + (size_t)row * g.ldr + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col + i < g.N) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rp + i);
                const bf16* rb = reinterpret_cast<const bf16*>(&rv);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i + j] += __bfloat162float(rb[j]);
              }
            }
          }
          if (g.D) {
            bf16* dp = g.D + (size_t)row * g.ldd + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col + i < g.N) {
                __align__(16) bf16 o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = __float2bfloat16_rn(v[i + j]);
                *reinterpret_cast<uint4*>(dp + i) = *reinterpret_cast<const uint4*>(o);
              }
            }
          }
          if (g.push_ranks) {
            const int owner = row / g.rows_per_rank;
            float* pp = g.push[owner] + (size_t)(row - owner * g.rows_per_rank) * g.N + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              if (col + i < g.N) {
                // + 0.f turns -0.0 into +0.0: the bit pattern of -0.0 marks a unit of the inbox that has not arrived
                asm volatile("st.volatile.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(pp + i), "f"(v[i] + 0.f), "f"(v[i + 1] + 0.f),
                             "f"(v[i + 2] + 0.f), "f"(v[i + 3] + 0.f) : "memory");
              }
          }
          if (g.Df) {
            float* fp = g.Df + (size_t)row * g.ldd + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              if (col + i < g.N) *reinterpret_cast<float4*>(fp + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && s_failed && g.status) atomicExch(g.status, (int)B2_ERR_TIMEOUT);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace b2

using namespace b2;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a row-major bf16 matrix [rows][cols] with leading dimension ld, boxes of box_rows x 64 columns.
static bool make_map(CUtensorMap* m, const void* ptr, long rows, long cols, long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// D (bf16 and/or fp32, leading dimension ldd) = A[M,K] (lda) * B[N,K]^T (ldb) + R (optional bf16 residual, ldr).
// Pointers must be 16-byte aligned, leading dimensions multiples of 8 elements, N a multiple of 8.
static int gemm_launch(const bf16* A, long lda, const bf16* B, long ldb, int M, int N, int K, bf16* D, float* Df, long ldd,
                       const bf16* R, long ldr, int* status, float* const* push, int push_ranks, int rows_per_rank, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (N % 8) || (lda % 8) || (ldb % 8) || (ldd % 8) || (R && (ldr % 8))) return B2_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return B2_ERR_ARG;
  if ((!D && !Df && push_ranks <= 0) || (reinterpret_cast<uintptr_t>(D) & 15) || (reinterpret_cast<uintptr_t>(Df) & 15)) return B2_ERR_ARG;
  CUtensorMap ma, mb;
  if (!make_map(&ma, A, M, K, lda, BM) || !make_map(&mb, B, N, K, ldb, BN)) return B2_ERR_LAUNCH;
  GemmArgs g{M, N, K, D, ldd, Df, R, ldr, status, {nullptr}, 0, 0};
  if (push_ranks > 0) {
    if (push_ranks > 8 || rows_per_rank <= 0 || (long)rows_per_rank * push_ranks < M) return B2_ERR_ARG;
    for (int r = 0; r < push_ranks; ++r) g.push[r] = push[r];
    g.push_ranks = push_ranks; g.rows_per_rank = rows_per_rank;
  }
  const size_t smem = (size_t)kStagesG * STAGE_BYTES + 1024;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return B2_ERR_LAUNCH;
    attr = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((N + BN - 1) / BN) * ((M + BM - 1) / BM), 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_tc_kernel, ma, mb, g) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_gemm_bf16(const bf16* A, long lda, const bf16* B, long ldb, int M, int N, int K, bf16* D, float* Df, long ldd,
                        const bf16* R, long ldr, int* status, cudaStream_t st) {
  return gemm_launch(A, lda, B, ldb, M, N, K, D, Df, ldd, R, ldr, status, nullptr, 0, 0, st);
}

// The same product with the reduce-scatter of a tensor-parallel row-parallel linear fused into the epilogue: every fp32
// partial tile is stored into the inbox slot (inbox[r] + slot_off + rank * slot_stride) of the rank r that owns its rows
// (rows_per_rank consecutive rows each; rows_per_rank * N <= slot_stride).  The owners then sum the slots in rank order
// with the wait-and-combine half of the push reduce-scatter (b2_comm_reduce_scatter with skip_push).
B2_API int b2_gemm_bf16_push(const bf16* A, long lda, const bf16* B, long ldb, int M, int N, int K, float* const* inbox, int ranks,
                             int rank, long slot_off, long slot_stride, int rows_per_rank, int* status, cudaStream_t st) {
  if (ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks || (long)rows_per_rank * N > slot_stride || (N % 4)) return B2_ERR_ARG;
  float* push[8];
  for (int r = 0; r < ranks; ++r) push[r] = inbox[r] + slot_off + (long)rank * slot_stride;
  return gemm_launch(A, lda, B, ldb, M, N, K, nullptr, nullptr, 8, nullptr, 0, status, push, ranks, rows_per_rank, st);
}
