// Argument block of the mixed-bit dequant GEMV family (wq_gemv.cu) and of its tensor-parallel variant.
#pragma once
#include "common.cuh"

namespace b2 {

enum GemvPro : int {
  PRO_PLAIN = 0,   // x is bf16 [m][ldx]
  PRO_NORM = 1,    // x = bf16(h * rsqrt(mean(h^2) + eps) * norm_w); mean from partial sums of squares
};
enum GemvEpi : int {
  EPI_STORE = 0,      // y bf16 [m][ldy]
  EPI_RESID = 1,      // y = bf16(acc + resid); partial sum of squares of y per panel -> ss_out
  EPI_SWIGLU = 2,     // rows g / g+8 of each 16-row block are (gate, up): y = bf16(silu(bf16 gate) * bf16 up), [m][n/2]
  EPI_F32 = 3,        // yf fp32 [m][ldy]
  EPI_ARGMAX = 4,     // per panel (max, argmax) of the fp32 result -> amax_val/amax_idx [panel][ss_ld]; optional yf
  EPI_TP_RESID = 5,   // tensor parallel: push the partial to every peer, sum all ranks in rank order, then EPI_RESID
};

constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kMaxTp = 8;
constexpr int kMaxKs = 64;            // most k slices a linear may be cut into

struct TpPush {
  // Lamport-style inboxes: inbox[r] is rank r's inbox region as mapped in this process (own region included).
  // A slot holds [src_rank][tok][n] fp32; a value of -0.0f means "not written yet".
  float* inbox[kMaxTp];
  int rank, size;
  long slot_off;         // float offset of the slot used by this call inside every inbox region
  long clear_off;        // float offset of the slot to re-arm (a slot no rank will write before its next use), -1: none
  long slot_stride;      // floats per source rank inside a slot (= tokens_cap * n)
  int* status;           // device status word (B2_ERR_TIMEOUT on wait expiry)
  unsigned long long timeout_ns;
  int skip_push;         // test hook: this rank does not push (peers then see the wait run out)
};

struct WqGemvArgs {
  const uint8_t* wq;     // FM blocks [n/32][k/128][2 x records | 2 x groups x 16 x (scale, zero)]
  int n, k, m;
  int bits, group;
  int ks;                // k slices (a function of the linear's shape only)
  int rb;                // row blocks per warp item: 2 (32 rows) or 4 (64 rows)
  int vworkers, fmax;    // b2_wq_gemv_vworkers / b2_wq_gemv_fmax of (n, k, ks, rb)
  int pro;
  const bf16* x; long ldx;
  const float* ss_in; int ss_parts; int ss_ld;
  const bf16* norm_w; float eps;
  int epi;
  bf16* y; long ldy;
  const bf16* resid; long ldr;
  float* ss_out;
  float* yf;
  float* amax_val; int* amax_idx; int n_valid;   // EPI_ARGMAX: rows >= n_valid never win
  float* scratch; unsigned* counters;   // split-k partials [item][ks][m][16*rb] and self-resetting panel counters
  int* status;           // device status word (B2_ERR_TIMEOUT when a bounded wait ran out)
  int debug;             // read by -DB2_MEASURE builds only: 1 = stream weights without arithmetic (bandwidth probe)
  TpPush tp;
  unsigned long long* trace;   // read by -DB2_MEASURE builds only: [CTA][warp][8] globaltimer stamps of the kernel's phases
};

}  // namespace b2

// Host entry points (C ABI).
B2_API int b2_wq_gemv(const b2::WqGemvArgs* args, cudaStream_t stream);
B2_API int b2_wq_gemv_vworkers(int n, int k, int ks, int rb);
B2_API int b2_wq_gemv_fmax(int n, int k, int ks, int rb);
B2_API long b2_wq_gemv_scratch_floats(int n, int k, int ks, int rb, int m);
B2_API long b2_wq_bytes(int n, int k, int bits, int group);
B2_API int b2_wq_dequant(const uint8_t* wq, int n, int k, int bits, int group, bf16* out, long ldo, cudaStream_t stream);
B2_API int b2_wq_repack(const int32_t* packed, const void* scale, int scale_is_bf16, const __half* zero, int n, int k,
                        int bits, int group, uint8_t* wq, cudaStream_t stream);
B2_API int b2_wq_random(uint8_t* wq, int n, int k, int bits, int group, float stddev, unsigned long long seed,
                        cudaStream_t stream);
