// Argument block of the persistent decode-step kernel (step_kernel.cu): one cooperative launch runs a whole decode /
// verify step of the dense GQA decoder -- every layer, the lm_head and the argmax -- for up to sixteen token rows.
#pragma once
#include "common.cuh"

namespace b2 {

constexpr int kStepWarps = 15;           // worker warps of a CTA
constexpr int kStepThreads = kStepWarps * 32;     // worker threads
constexpr int kStepBlock = kStepThreads + 32;    // plus the producer warp that feeds the workers' weight rings
constexpr int kStepMaxRows = 16;         // token rows of one step (up to four sets of four tokens = four n-8 mma tiles of (hi, lo) limb columns)
constexpr int kStepSmallRows = 8;        // steps of up to this many rows stage slices of kStepSliceK inputs, larger steps half of that
constexpr int kStepSliceK = 5120;        // most inputs of a linear that one CTA stages (k slice)
constexpr int kStepMaxTp = 8;

// One quantised linear in FM layout plus its shape-only work split over `ncta` CTAs (filled by b2_step_linear).
struct StepLinear {
  const uint8_t* wq;
  int n, k, bits, group;
  int npan, nbat;          // 32-row panels, 128-k batches
  int wbatch, szb, blk;    // bytes: weight record of one (16-row block, batch); its (scale, zero) pairs; one FM block
  int ks, cps;             // k slices; CTAs per slice (CTAs >= ks * cps idle in this linear's phase)
  int fmax;                // most fragments a (panel, slice) is cut into
  int pad;
};

struct StepLayer {
  StepLinear qkv, o, gate_up, down;
  const bf16* ln1;
  const bf16* ln2;
  bf16* kv_pool;           // [page][2][kv_head][16][128]
  void* pad;               // keeps every element of the device array 16-byte aligned (the linears are read as uint4)
};
static_assert(sizeof(StepLayer) % 16 == 0, "StepLayer array elements must stay 16-byte aligned");

struct StepArgs {
  const StepLayer* layers;   // device array [n_layers]
  int n_layers;
  StepLinear lm_head;
  const bf16* final_norm;
  const bf16* embed;         // [vocab][d_model]
  int vocab, d_model, hq, hkv, ffn;   // per-rank head counts / ffn width; head_dim is 128
  float eps;
  int lm_valid;              // lm_head rows >= lm_valid never win the argmax (padding of a vocabulary shard)
  int lm_offset;             // added to the winning row index (first vocabulary id of this rank's shard)

  // rows of this step
  int n_rows;                // 1..16
  int slice_k;               // k slice the linears' work split was computed for (b2_step_linear): 5120, or 2560 for more than 8 rows
  int* ids; int* tok_pos; int* tok_seq;       // [n_rows]
  const int* rope_pos;       // optional rotary positions (null: tok_pos)
  const int* grp_tok0; const int* grp_cnt; int n_groups;   // consecutive rows of one sequence
  const unsigned* tree_mask; // optional [n_rows]
  const int* block_table; int bt_ld; int n_pages;
  const float* inv_freq;     // [64]
  int split_keys, max_splits;
  float scale_log2;

  // decode mode (slot_seq != null): ids = last_ids, positions = seq_len[slot_seq[i]]; at the end seq_len advances and
  // last_ids receives the produced tokens
  const int* slot_seq; int* last_ids; int* seq_len;

  // workspaces (own device memory)
  float* part;               // GEMV partials [slot][row][n]
  float* tile_scratch;       // steps of more than 8 rows: [CTAs][15 warps][2][16][32] partial tiles (shared memory holds them otherwise)
  uint8_t* xq;               // staged activations of the next linear: [k / 128][token sets * 1024] bytes (fixed-point limbs)
  float2* xg;                // their group scalars: [k / group][4 * token sets] (scale, scale * integer sum)
  float* psq;                // sums of squares of the residual stream: [rows][d_model / 128]
  int* attn_ctr;             // [n_layers] work counters of the attention stages (zero between launches)
  bf16* h;                   // residual stream [rows][d_model]
  bf16* q;                   // [rows][hq * 128]
  bf16* attn;                // [rows][hq * 128]
  bf16* act;                 // [rows][ffn]
  float* part_o;             // [rows][hq][max_splits][128]
  float* part_ml;            // [rows][hq][max_splits][2]
  float* amax_val; int* amax_idx;   // [CTAs][16]
  float* logits; long ld_logits;    // optional fp32 logits of this rank's lm_head rows
  int* out_ids; float* out_val;     // [rows]
  unsigned* sync;            // [0] arrival counter of the grid barrier, [1] its base, [2] base of the cross-rank barrier
  int* status;
  unsigned long long timeout_ns;

  // tensor parallel: every rank's exchange region as mapped here.  Word 0 of a region is that rank's arrival counter
  // of the cross-rank barrier; partial sums of the row-parallel linears and the argmax candidates follow.
  int tp_rank, tp_size;
  float* xreg[kStepMaxTp];
  long x_off[2];             // float offsets of the two alternating partial areas (o_proj, down_proj)
  long x_amax;               // float offset of the argmax candidates [rank][16][2]
  int skip_push;             // test hook: this rank does not signal its peers (their bounded wait runs out)
  unsigned long long* trace; // builds with -DB2_STEP_TRACE only: CTA 0 stamps %globaltimer at every barrier (arrive, leave)
};

}  // namespace b2

B2_API int b2_step_linear(const uint8_t* wq, int n, int k, int bits, int group, int ncta, int slice_k, b2::StepLinear* out);
B2_API long b2_step_part_floats(const b2::StepLinear* lin, int rows);
B2_API int b2_step_smem_bytes();
B2_API int b2_step_args_bytes();    // sizeof(StepArgs) / sizeof(StepLayer): checked by the Python mirror of the structs
B2_API int b2_step_layer_bytes();
B2_API int b2_step_grid(int* ncta);
B2_API int b2_step_launch(const b2::StepArgs* args, int ncta, cudaStream_t stream);
