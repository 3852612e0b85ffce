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
static int g_force_grid = 0;        // > 0 overrides the grid size (tuning and tests)
static int g_pdl = 0;               // programmatic dependent launch between consecutive layers: 0 off, 1 late trigger, 2 early

void qmv_set_tuning(int ctas_per_sm, int force_grid, int pdl) {
    if (ctas_per_sm > 0) g_ctas_per_sm = ctas_per_sm;
    g_force_grid = force_grid > 0 ? force_grid : 0;
    g_pdl = pdl > 0 ? pdl : 0;
}

// halves per activation row kept in shared memory for a slice of at most `units` tiles of one block
static int xs_stride_for(int tiles_k, int64_t units) {
    // `units` tiles -> that many /8 input tiles (+1 for a ragged start) -> 128-blocks (+1 likewise);
    // 8 halves of padding stagger the rows over the banks
    const int64_t tks = (units + 7) / 8 + 1;
    const int blocks = static_cast<int>(std::min<int64_t>((tks + 7) / 8 + 1, (tiles_k + 7) / 8));
    return blocks * 128 + 8;
}

QmvPlan plan_qmv(int in, int out, int k, int64_t rows) {
    QmvPlan plan{};
    plan.col_blocks = out / 128;
    const int tiles_k = in / 16;
    const int64_t ub = static_cast<int64_t>(tiles_k) * 8;
    const int64_t total = ub * plan.col_blocks;
    const int r = static_cast<int>(std::min<int64_t>(rows, kQmvMaxRows));
    // register pressure grows with the number of 8-row blocks: 2 and 4 blocks fit 2 and 1 CTAs per SM
    const int resident = r <= 8 ? g_ctas_per_sm : (r <= 16 ? std::min(g_ctas_per_sm, 2) : 1);
    int64_t grid = g_force_grid > 0 ? g_force_grid : static_cast<int64_t>(kSmCount) * resident;
    // keep at least four tiles per warp so a CTA is not all prologue and epilogue
    grid = std::max<int64_t>(1, std::min(grid, total / (kQmvWarps * 4)));
    const size_t ring = static_cast<size_t>(kQmvWarps) * qmv_depth(k) * 64 * k * sizeof(uint32_t);
    // the rotated activations of a slice must fit beside the ring: more CTAs = shorter slices
    const size_t budget = kQmvMaxSmemBytes - ring;
    auto slice_units = [&](int64_t gr) { return std::min(ub, (total + gr - 1) / gr); };
    while (grid < total && static_cast<size_t>(r) * xs_stride_for(tiles_k, slice_units(grid)) * sizeof(__half) > budget)
        grid += kSmCount;
    grid = std::min(grid, total);
    plan.grid = static_cast<int>(grid);
    plan.max_pieces = static_cast<int>((grid + plan.col_blocks - 1) / plan.col_blocks + 1);
    plan.xs_stride = xs_stride_for(tiles_k, slice_units(grid));
    const size_t xs = static_cast<size_t>(r) * plan.xs_stride * sizeof(__half);
    const size_t red = static_cast<size_t>(kQmvWarps / 2) * r * kQmvRedStride * sizeof(float);
    plan.smem_bytes = std::max(ring + xs, red);
    plan.pdl = g_pdl != 0;
    plan.pdl_early = g_pdl == 2;
    return plan;
}

size_t qmv_counter_bytes(int out) { return (static_cast<size_t>(out / 128) * sizeof(unsigned int) + 255) / 256 * 256; }

size_t qmv_partial_bytes(const QmvPlan& plan, int out, int64_t rows) {
    const int64_t r = std::min<int64_t>(rows, kQmvMaxRows);
    return (static_cast<size_t>(plan.col_blocks) * plan.max_pieces * r * 128 * sizeof(float) + 255) / 256 * 256;
}

cudaError_t launch_qmv(QmvArgs args, int k, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (args.rows <= 0 || args.rows > kQmvMaxRows) return cudaErrorInvalidValue;
    args.tiles_k = args.in / 16;
    args.tiles_n = args.out / 16;
    args.max_pieces = plan.max_pieces;
    args.xs_stride = plan.xs_stride;
    args.pdl_early = plan.pdl_early ? 1 : 0;
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
