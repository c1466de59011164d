// Instance of the persistent decode-step kernel for steps of five to eight token rows (2 token sets).
#include "step_kernel_impl.cuh"

namespace b2 {
int step_prepare_r8() { return step_prepare<2>(); }
int step_launch_r8(const StepArgs& a, int ncta, cudaStream_t stream) { return step_launch_instance<2>(a, ncta, stream); }
}  // namespace b2
