// Launch policy of the persistent decode-step kernel: one wave of CTAs that every layer of the step shares.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>
#include <atomic>

namespace b200exl3 {

cudaError_t stack_dispatch_k1(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k2(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k3(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k4(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k5(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k6(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k7(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);
cudaError_t stack_dispatch_k8(const StackArgs&, int, bool, const StackPlan&, cudaStream_t);

StackPlan plan_stack(int k, int rows, int n_ops) {
    StackPlan plan{};
    const int r = std::max(1, std::min(rows, kStackMaxRows));
    // per warp: [ring of packed rows | rotated activations | two staged result tiles]
    const size_t ring = static_cast<size_t>(kStackSlots) * stack_chunk_rows(k) * 64 * k * sizeof(uint32_t);
    plan.x_blocks = r == 1 ? kQmvXBlocks : 4;
    const size_t xs = static_cast<size_t>(r) * plan.x_blocks * 128 * sizeof(__half);
    const size_t stage = 2 * static_cast<size_t>(r) * kQmvRedStride * sizeof(float);
    plan.xs_offset = static_cast<int>(ring);
    plan.stage_offset = static_cast<int>(ring + xs);
    plan.warp_smem = static_cast<int>((ring + xs + stage + 15) / 16 * 16);
    plan.table_offset = plan.warp_smem * kStackWarps;
    plan.smem_bytes = static_cast<size_t>(plan.table_offset) + static_cast<size_t>(n_ops) * sizeof(StackOpLite);
    plan.grid = sm_count() * kStackCtasPerSm;                 // 16 warps per SM
    plan.cooperative = true;
    return plan;
}

bool plan_stack_op(const StackPlan& plan, StackOp& op) {
    if (op.in <= 0 || op.out <= 0 || op.in % 128 || op.out % 128) return false;
    op.tiles_k = op.in / 16;
    op.tiles_n = op.out / 16;
    op.col_blocks = op.out / 128;
    const int64_t ub = static_cast<int64_t>(op.tiles_k) * 8;
    const int64_t total = ub * op.col_blocks;
    if (total >= (int64_t(1) << 31)) return false;
    // the layer is dealt out in whole rows of 8 tiles; every warp of the grid takes part unless there are fewer rows than warps
    const int64_t rb = op.tiles_k, rt = rb * op.col_blocks;
    int64_t ctas = std::max<int64_t>(1, std::min<int64_t>(plan.grid, rt / kStackWarps));
    // a warp's range must stay within one column block's worth of rows (it then touches at most two blocks)
    const int64_t min_warps = (rt + rb - 2) / (rb - 1) + 1;
    ctas = std::max(ctas, (min_warps + kStackWarps - 1) / kStackWarps);
    if (ctas > plan.grid) return false;                       // wider than the grid can cover in one pass
    op.warps = static_cast<int>(ctas) * kStackWarps;
    op.narrow = static_cast<unsigned long long>(total + 1) * static_cast<unsigned long long>(op.warps) < 0xffffffffull ? 1 : 0;
    // whole warps per column block when that does not raise the largest share of rows (no warp then works on two blocks)
    const int64_t per_block = op.warps / op.col_blocks;
    if (per_block >= 1 && (rb + per_block - 1) / per_block <= (rt + op.warps - 1) / op.warps &&
        static_cast<unsigned long long>(op.warps + 1) * static_cast<unsigned long long>(op.col_blocks + 1) < 0xffffffffull)
        op.narrow |= 2;
    op.max_pieces = static_cast<int>((ctas + op.col_blocks - 1) / op.col_blocks + 1);
    return true;
}

cudaError_t launch_stack(const StackArgs& args, int k, int cb, bool exact, const StackPlan& plan, cudaStream_t stream) {
    if (args.rows <= 0 || args.rows > kStackMaxRows || args.n_ops <= 0 || args.n_ops > kStackMaxOps) return cudaErrorInvalidValue;
    switch (k) {
        case 1: return stack_dispatch_k1(args, cb, exact, plan, stream);
        case 2: return stack_dispatch_k2(args, cb, exact, plan, stream);
        case 3: return stack_dispatch_k3(args, cb, exact, plan, stream);
        case 4: return stack_dispatch_k4(args, cb, exact, plan, stream);
        case 5: return stack_dispatch_k5(args, cb, exact, plan, stream);
        case 6: return stack_dispatch_k6(args, cb, exact, plan, stream);
        case 7: return stack_dispatch_k7(args, cb, exact, plan, stream);
        case 8: return stack_dispatch_k8(args, cb, exact, plan, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200exl3
