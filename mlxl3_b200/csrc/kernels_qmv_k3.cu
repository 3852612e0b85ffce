// Instantiates the fused linear-layer kernels for K = 3 bits per weight.
#include "kernels_qmv_impl.cuh"

namespace b200exl3 {
cudaError_t qmv_dispatch_k3(const QmvArgs& p, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    return qmv_launch_k<3>(p, cb, exact, plan, stream);
}
}  // namespace b200exl3
