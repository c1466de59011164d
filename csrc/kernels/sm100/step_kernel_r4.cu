// Instance of the persistent decode-step kernel for steps of one to four token rows (1 token set).
#include "step_kernel_impl.cuh"

namespace b2 {
int step_smem_bytes() { return SM_TOTAL; }
int step_prepare_r4() { return step_prepare<1>(); }
int step_launch_r4(const StepArgs& a, int ncta, cudaStream_t stream) { return step_launch_instance<1>(a, ncta, stream); }
}  // namespace b2
