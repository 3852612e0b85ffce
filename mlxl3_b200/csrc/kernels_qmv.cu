// Launch policy and K dispatch of the fused linear-layer kernels.
//
// The reference picks a split-K factor and tile width per shape for Apple GPUs
// (native/src/contracts.rs:1995-2012, native/src/linear.rs:899-919); only the meaning is kept
// (partials are summed in fp32 before the output rotation), the numbers are chosen for 148 SMs.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>

namespace b200exl3 {

cudaError_t qmv_dispatch_k1(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k2(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k3(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k4(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k5(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k6(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k7(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k8(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);

static int g_ctas_per_sm = 2;       // CTAs per SM the grid is sized for (one wave)
static int g_force_splits = 0;      // > 0 overrides the heuristic (tuning and tests)
static int g_pdl = 0;               // programmatic dependent launch between consecutive layers

void qmv_set_tuning(int ctas_per_sm, int force_splits, int pdl) {
    if (ctas_per_sm > 0) g_ctas_per_sm = ctas_per_sm;
    g_force_splits = force_splits > 0 ? force_splits : 0;
    g_pdl = pdl > 0 ? 1 : 0;
}

static int xs_stride_for(int tiles_k, int splits) {
    // a CTA covers at most ceil(tiles_k*8/splits) tiles -> that many /8 input tiles (+1 for a ragged
    // start) -> 128-blocks (+1 for a ragged start); 8 halves of padding stagger the rows over the banks
    const int units = (tiles_k * 8 + splits - 1) / splits;
    const int tks = (units + 7) / 8 + 1;
    const int blocks = std::min((tks + 7) / 8 + 1, (tiles_k + 7) / 8);
    return blocks * 128 + 8;
}

QmvPlan plan_qmv(int in, int out, int k, int64_t rows) {
    QmvPlan plan{};
    plan.col_blocks = out / 128;
    const int tiles_k = in / 16;
    const int units = tiles_k * 8;
    const int r = static_cast<int>(std::min<int64_t>(rows, kQmvMaxRows));
    // register pressure grows with the number of 8-row blocks: 2 and 4 blocks fit 2 and 1 CTAs per SM
    const int resident = r <= 8 ? g_ctas_per_sm : (r <= 16 ? std::min(g_ctas_per_sm, 2) : 1);
    const int target = kSmCount * resident;
    int splits = g_force_splits > 0 ? g_force_splits : target / plan.col_blocks;      // floor: stay within one wave
    // keep at least four tiles per warp so a CTA is not all prologue and epilogue
    splits = std::min(splits, std::max(1, units / (kQmvWarps * 4)));
    splits = std::max(1, std::min(splits, tiles_k));
    const size_t ring = static_cast<size_t>(kQmvWarps) * qmv_depth(k) * 64 * k * sizeof(uint32_t);
    // the rotated activations of a CTA's input range must fit beside the ring
    const size_t budget = kQmvMaxSmemBytes - ring;
    while (splits < tiles_k && static_cast<size_t>(r) * xs_stride_for(tiles_k, splits) * sizeof(__half) > budget) ++splits;
    plan.splits = splits;
    plan.xs_stride = xs_stride_for(tiles_k, splits);
    const size_t xs = static_cast<size_t>(r) * plan.xs_stride * sizeof(__half);
    const size_t red = static_cast<size_t>(kQmvWarps / 2) * r * kQmvRedStride * sizeof(float);
    plan.smem_bytes = std::max(ring + xs, red);
    plan.pdl = g_pdl != 0;
    return plan;
}

size_t qmv_counter_bytes(int out) { return (static_cast<size_t>(out / 128) * sizeof(unsigned int) + 255) / 256 * 256; }

size_t qmv_partial_bytes(const QmvPlan& plan, int out, int64_t rows) {
    if (plan.splits <= 1) return 0;
    const int64_t r = std::min<int64_t>(rows, kQmvMaxRows);
    return (static_cast<size_t>(plan.splits) * r * out * sizeof(float) + 255) / 256 * 256;
}

cudaError_t launch_qmv(QmvArgs args, int k, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (args.rows <= 0 || args.rows > kQmvMaxRows) return cudaErrorInvalidValue;
    args.tiles_k = args.in / 16;
    args.tiles_n = args.out / 16;
    args.splits = plan.splits;
    args.xs_stride = plan.xs_stride;
    switch (k) {
        case 1: return qmv_dispatch_k1(args, cb, exact, plan, stream);
        case 2: return qmv_dispatch_k2(args, cb, exact, plan, stream);
        case 3: return qmv_dispatch_k3(args, cb, exact, plan, stream);
        case 4: return qmv_dispatch_k4(args, cb, exact, plan, stream);
        case 5: return qmv_dispatch_k5(args, cb, exact, plan, stream);
        case 6: return qmv_dispatch_k6(args, cb, exact, plan, stream);
        case 7: return qmv_dispatch_k7(args, cb, exact, plan, stream);
        case 8: return qmv_dispatch_k8(args, cb, exact, plan, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200exl3
