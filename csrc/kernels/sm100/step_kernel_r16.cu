// Instance of the persistent decode-step kernel for steps of nine to sixteen token rows (4 token sets).
#include "step_kernel_impl.cuh"

namespace b2 {
int step_prepare_r16() { return step_prepare<4>(); }
int step_launch_r16(const StepArgs& a, int ncta, cudaStream_t stream) { return step_launch_instance<4>(a, ncta, stream); }
}  // namespace b2
