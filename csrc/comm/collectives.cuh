// Argument block of the bounded push collectives over symmetric peer memory (collectives.cu).
#pragma once
#include "../kernels/sm100/common.cuh"

namespace b2 {

constexpr int kCommMaxRanks = 8;

// A slot of a rank's inbox holds one contribution per source rank: [src][elems] fp32.  A value of -0.0f (bit pattern
// 0x80000000) means "not written yet" (Lamport-style: the payload carries its own arrival flag, no separate fence).
struct CommArgs {
  float* inbox[kCommMaxRanks];   // every rank's inbox region as mapped in this process (own region included)
  int rank, size;
  long slot_off;                 // float offset of this call's slot inside every region
  long clear_off;                // slot to re-arm with the sentinel (no rank writes it before its next use), -1: none
  long clear_n;                  // floats per source rank to re-arm there (the extent the earlier call used)
  long slot_stride;              // floats per source rank inside a slot
  int* status;                   // device status word: B2_ERR_TIMEOUT when a wait ran out
  unsigned long long timeout_ns;
  int skip_push;                 // test hook: behave like a rank whose message is lost
};

}  // namespace b2

B2_API int b2_comm_all_reduce(const b2::CommArgs* a, const float* in_f32, const bf16* in_bf16, long n, float* out_f32,
                              bf16* out_bf16, cudaStream_t st);
B2_API int b2_comm_all_gather(const b2::CommArgs* a, const float* in, long n_per_rank, float* out, cudaStream_t st);
B2_API int b2_comm_reduce_scatter(const b2::CommArgs* a, const float* in, long n_per_rank, float* out, cudaStream_t st);
B2_API int b2_comm_collect_gather(const b2::CommArgs* a, long slot_b_off, int rows_per, int n_cols, int total_rows, bf16* out,
                                  cudaStream_t st);
B2_API int b2_comm_barrier(const b2::CommArgs* a, cudaStream_t st);
B2_API int b2_comm_argmax_combine(const b2::CommArgs* a, const float* val, const int* idx, int n_tok, int* out_idx,
                                  float* out_val, cudaStream_t st);
