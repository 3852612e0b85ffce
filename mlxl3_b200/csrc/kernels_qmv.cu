// Launch policy and K dispatch of the fused linear-layer kernels.
//
// The reference picks a split-K factor and tile width per shape for Apple GPUs
// (native/src/contracts.rs:1995-2012, native/src/linear.rs:899-919); only the meaning is kept
// (partials are summed in fp32 before the output rotation), the numbers are chosen for 148 SMs.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>
#include <atomic>

namespace b200exl3 {

cudaError_t qmv_dispatch_k1(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k2(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k3(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k4(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k5(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k6(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k7(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);
cudaError_t qmv_dispatch_k8(const QmvArgs&, int, bool, const QmvPlan&, cudaStream_t);

// Process-wide knobs; atomics because handles may be used from several threads while another thread sets an option.
static std::atomic<int> g_ctas_per_sm{2};   // CTAs per SM the grid is sized for (one wave)
static std::atomic<int> g_force_grid{0};    // > 0 overrides the grid size (tuning and tests)
static std::atomic<int> g_pdl{0};           // programmatic dependent launch between consecutive layers: 0 off, 1 late trigger, 2 early

bool pdl_enabled() { return g_pdl.load() != 0; }

int sm_count() {
    static std::atomic<int> cached[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        (void)cudaGetLastError();
        return kDefaultSmCount;
    }
    int n = cached[device].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return kDefaultSmCount;
    }
    cached[device].store(n, std::memory_order_relaxed);
    return n;
}

void qmv_set_tuning(int ctas_per_sm, int force_grid, int pdl) {
    if (ctas_per_sm > 0) g_ctas_per_sm = ctas_per_sm;
    g_force_grid = force_grid > 0 ? force_grid : 0;
    g_pdl = pdl > 0 ? pdl : 0;
}

static std::atomic<unsigned long long*> g_trace{nullptr};
void qmv_set_trace(unsigned long long* device_buffer) { g_trace = device_buffer; }

QmvPlan plan_qmv(int in, int out, int k, int64_t rows) {
    QmvPlan plan{};
    plan.col_blocks = out / 128;
    const int tiles_k = in / 16;
    const int64_t total = static_cast<int64_t>(tiles_k) * 8 * plan.col_blocks;
    const int r = static_cast<int>(std::min<int64_t>(rows, kQmvMaxRows));
    // two 8-row blocks need about twice the registers and shared memory: one CTA per SM
    const int resident = r <= 8 ? g_ctas_per_sm.load() : 1;
    const int forced = g_force_grid.load();
    int64_t grid = forced > 0 ? forced : static_cast<int64_t>(sm_count()) * resident;
    // the layer is dealt out in whole rows of 8 tiles: no more warps than rows
    const int64_t rb = tiles_k, rt = rb * plan.col_blocks;
    grid = std::max<int64_t>(1, std::min(grid, rt / kQmvWarps));
    // a warp's range must not exceed one column block (it then touches at most two blocks)
    const int64_t min_warps = (rt + rb - 2) / (rb - 1) + 1;
    grid = std::max(grid, (min_warps + kQmvWarps - 1) / kQmvWarps);
    plan.grid = static_cast<int>(grid);
    plan.max_pieces = static_cast<int>((grid + plan.col_blocks - 1) / plan.col_blocks + 1);
    plan.fused_rotation = r <= kQmvFusedRows;
    // per warp: [ring of packed rows | rotated activations | two staged result tiles]
    const size_t ring = static_cast<size_t>(qmv_chunk_rows(k)) * qmv_slots(k) * 64 * k * sizeof(uint32_t);
    const size_t xs = plan.fused_rotation ? static_cast<size_t>(r) * kQmvXBlocks * 128 * sizeof(__half) : 0;
    const size_t stage = 2 * static_cast<size_t>(r) * kQmvRedStride * sizeof(float);   // first and second block of a warp
    plan.xs_offset = static_cast<int>(ring);
    plan.stage_offset = static_cast<int>(ring + xs);
    plan.warp_smem = static_cast<int>((ring + xs + stage + 15) / 16 * 16);
    plan.smem_bytes = static_cast<size_t>(plan.warp_smem) * kQmvWarps;
    const int pdl = g_pdl.load();
    plan.pdl = pdl != 0;
    plan.pdl_early = pdl == 2;
    return plan;
}

size_t qmv_partial_bytes(const QmvPlan& plan, int out, int64_t rows) {
    const int64_t r = std::min<int64_t>(rows, kQmvMaxRows);
    return (static_cast<size_t>(plan.col_blocks) * plan.max_pieces * r * 128 * sizeof(float) + 255) / 256 * 256;
}

cudaError_t launch_qmv(QmvArgs args, int k, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (args.rows <= 0 || args.rows > kQmvMaxRows) return cudaErrorInvalidValue;
    args.tiles_k = args.in / 16;
    if (args.map_selected == nullptr) args.tiles_n = args.out / 16;   // the expert-mapped caller gives the bank's width
    args.max_pieces = plan.max_pieces;
    args.trace = g_trace.load();
    args.warp_smem = plan.warp_smem;
    args.xs_offset = plan.xs_offset;
    args.stage_offset = plan.stage_offset;
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
