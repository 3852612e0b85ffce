// Launch policy and K dispatch of the fused product kernels.
//
// The reference picks a split-K factor and tile width per shape for Apple GPUs
// (native/src/contracts.rs:1995-2012, native/src/linear.rs:899-919); only the meaning is kept
// (partials are summed in fp32 by the output rotation), the numbers are chosen for 148 SMs.
#include "kernels_qmv_impl.cuh"

#include <algorithm>

namespace b200exl3 {

cudaError_t qmv_dispatch_k1(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k2(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k3(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k4(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k5(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k6(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k7(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k8(const QmvParams&, int, bool, const QmvPlan&, cudaStream_t);

static int g_ctas_per_sm = 3;       // target resident CTAs per SM when choosing the split factor
static int g_force_splits = 0;      // > 0 overrides the heuristic (tuning and tests)

void qmv_set_tuning(int ctas_per_sm, int force_splits) {
    if (ctas_per_sm > 0) g_ctas_per_sm = ctas_per_sm;
    g_force_splits = force_splits > 0 ? force_splits : 0;
}

QmvPlan plan_qmv(int in, int out, int k, int64_t rows) {
    QmvPlan plan{};
    plan.warps = kQmvWarps;
    plan.col_blocks = out / 128;
    const int tiles_k = in / 16;
    const int units = tiles_k * 8;
    const int target = kSmCount * g_ctas_per_sm;
    int splits = g_force_splits > 0 ? g_force_splits : (target + plan.col_blocks / 2) / plan.col_blocks;
    // keep at least four tiles per warp so a CTA is not all prologue
    splits = std::min(splits, std::max(1, units / (kQmvWarps * 4)));
    splits = std::max(1, std::min(splits, tiles_k));
    plan.splits = splits;
    const int r = static_cast<int>(rows);
    size_t ring = static_cast<size_t>(kQmvWarps) * qmv_depth(k) * 64 * k * sizeof(uint32_t);
    size_t red = static_cast<size_t>(kQmvWarps / 2) * r * kQmvRedStride * sizeof(float);
    plan.smem_bytes = std::max(ring, red);
    return plan;
}

cudaError_t launch_qmv(const uint16_t* trellis, int in, int out, int k, int cb, const __half* xhat, int64_t rows,
                       bool exact, const QmvPlan& plan, float* partials, cudaStream_t stream) {
    if (rows <= 0 || rows > 32) return cudaErrorInvalidValue;
    QmvParams p{};
    p.trellis = reinterpret_cast<const uint32_t*>(trellis);
    p.xhat = xhat;
    p.partials = partials;
    p.in = in; p.out = out; p.rows = static_cast<int>(rows);
    p.tiles_k = in / 16; p.tiles_n = out / 16; p.splits = plan.splits;
    switch (k) {
        case 1: return qmv_dispatch_k1(p, cb, exact, plan, stream);
        case 2: return qmv_dispatch_k2(p, cb, exact, plan, stream);
        case 3: return qmv_dispatch_k3(p, cb, exact, plan, stream);
        case 4: return qmv_dispatch_k4(p, cb, exact, plan, stream);
        case 5: return qmv_dispatch_k5(p, cb, exact, plan, stream);
        case 6: return qmv_dispatch_k6(p, cb, exact, plan, stream);
        case 7: return qmv_dispatch_k7(p, cb, exact, plan, stream);
        case 8: return qmv_dispatch_k8(p, cb, exact, plan, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200exl3
