// Host side of the persistent decode-step kernel: work split of a linear, buffer sizes, grid size and the launch.
// The kernel itself is a template over the number of four-row token sets (step_kernel_impl.cuh), instantiated in
// step_kernel_r4.cu (1..4 rows), step_kernel_r8.cu (5..8) and step_kernel_r16.cu (9..16).
#include "step_kernel.cuh"

namespace b2 {
int step_smem_bytes();
int step_prepare_r4();
int step_prepare_r8();
int step_prepare_r16();
int step_launch_r4(const StepArgs& a, int ncta, cudaStream_t stream);
int step_launch_r8(const StepArgs& a, int ncta, cudaStream_t stream);
int step_launch_r16(const StepArgs& a, int ncta, cudaStream_t stream);
}  // namespace b2

using namespace b2;

// Work split of one linear over `ncta` CTAs (shape-only): k slices of at most `slice_k` inputs (kStepSliceK for steps
// of up to eight rows, half of it beyond), cps CTAs per slice (never more CTAs than blocks), and the most fragments a
// panel of a slice is cut into.
B2_API int b2_step_linear(const uint8_t* wq, int n, int k, int bits, int group, int ncta, int slice_k, StepLinear* out) {
  if (!out || n <= 0 || k <= 0 || n % 32 || k % 128 || ncta < 1) return B2_ERR_ARG;
  if (slice_k != kStepSliceK && slice_k != kStepSliceK / 2) return B2_ERR_ARG;
  if ((bits != 2 && bits != 3 && bits != 4) || (group != 64 && group != 128)) return B2_ERR_ARG;
  StepLinear L = {};
  L.wq = wq; L.n = n; L.k = k; L.bits = bits; L.group = group;
  L.npan = n / 32; L.nbat = k / 128;
  const int rec = bits == 3 ? 768 : 512;
  const int rpb = bits == 4 ? 2 : 1;
  L.wbatch = rpb * rec;
  L.szb = (128 / group) * 64;
  L.blk = 2 * L.wbatch + 2 * L.szb;
  L.ks = (k + slice_k - 1) / slice_k;
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

B2_API int b2_step_smem_bytes() { return step_smem_bytes(); }
B2_API int b2_step_args_bytes() { return (int)sizeof(StepArgs); }
B2_API int b2_step_layer_bytes() { return (int)sizeof(StepLayer); }

// CTAs of the persistent grid = SMs of the current device, provided one CTA of every instance fits per SM.
B2_API int b2_step_grid(int* ncta) {
  int dev = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B2_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (step_prepare_r4() != B2_OK || step_prepare_r8() != B2_OK || step_prepare_r16() != B2_OK) return B2_ERR_LAUNCH;
  if (!coop || sms < 1) return B2_ERR_LAUNCH;
  *ncta = sms;
  return B2_OK;
}

// Launches one step.  `ncta` must be the value the linears' work split was computed for (b2_step_grid).  The launch
// is cooperative, so all CTAs are resident together (the barriers inside the kernel rely on it).
B2_API int b2_step_launch(const StepArgs* args, int ncta, cudaStream_t stream) {
  const StepArgs& a = *args;
  if (a.n_rows < 1 || a.n_rows > kStepMaxRows || a.n_layers < 0 || ncta < 1) return B2_ERR_ARG;
  if (a.slice_k != kStepSliceK && a.slice_k != kStepSliceK / 2) return B2_ERR_ARG;
  if (a.n_rows > kStepSmallRows && (a.slice_k != kStepSliceK / 2 || !a.tile_scratch)) return B2_ERR_ARG;
  if (a.hq <= 0 || a.hkv <= 0 || a.hq % a.hkv || a.d_model % 8 || a.split_keys % 16 || a.max_splits <= 0) return B2_ERR_ARG;
  if (a.n_groups < 1 || a.n_groups > a.n_rows) return B2_ERR_ARG;
  if (a.tp_size < 1 || a.tp_size > kStepMaxTp || a.tp_rank < 0 || a.tp_rank >= a.tp_size) return B2_ERR_ARG;
  if (!a.sync || !a.status || !a.part || !a.h) return B2_ERR_ARG;
  if (a.n_rows <= 4) return step_launch_r4(a, ncta, stream);
  if (a.n_rows <= kStepSmallRows) return step_launch_r8(a, ncta, stream);
  return step_launch_r16(a, ncta, stream);
}
