// Instantiates the persistent decode-step kernel for K = 5 bits per weight.
#include "kernels_stack_impl.cuh"

namespace b200exl3 {
cudaError_t stack_dispatch_k5(const StackArgs& a, int cb, bool exact, const StackPlan& plan, cudaStream_t stream) {
    return stack_launch_k<5>(a, cb, exact, plan, stream);
}
}  // namespace b200exl3
