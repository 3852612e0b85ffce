// Row-parallel layers across GPUs: the sum of the ranks' fp32 partial products and the output rotation
// in one kernel, over peer memory (NVLink), with no library collective.
//
// Reference behaviour kept: the partial products are the reference's split-K partials
// (native/src/linear.rs:978-982); they are added in fp32, in rank order on every rank (so all ranks
// hold bit-identical outputs), then rounded to fp16, rotated and scaled as in linear.rs:983-996.
//
// Protocol (one warp per unit = 128 columns of one row; all ranks run the same launches in the same
// order).  For its c-th use of a unit a rank
//   1. stores its 128 partial sums into slot [c & 1][own rank][unit] of every rank's inbox (peer stores),
//   2. fences system-wide and stores c into flag [own rank][unit] of every rank,
//   3. waits until its own flags [src][unit] have reached c for every src, sums the slots in rank order,
//      rotates and stores the output, and records c as done.
// A rank can run at most one call ahead of another (its next call cannot finish without the other's
// data), which is what the two slots per unit are for.  The wait is bounded (about four seconds): when it
// gives up the status word is set, later waits are skipped, and the kernel returns.
#include "hadamard.cuh"
#include "kernels.h"

namespace b200exl3 {

namespace {

constexpr int kTpWarps = 4;

__device__ __forceinline__ void store_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int load_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kTpWarps * 32)
tp_finish_kernel(TpArgs p) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = p.out >> 7;
    const int units = p.rows * blocks_per_row;
    const size_t slot_floats = static_cast<size_t>(p.max_units) * 128;
    float* const my_inbox = p.inbox[p.rank];
    unsigned int* const my_flags = p.flags[p.rank];
    for (int u = blockIdx.x * kTpWarps + (threadIdx.x >> 5); u < units; u += gridDim.x * kTpWarps) {
        const int row = u / blocks_per_row, col = (u - row * blocks_per_row) * 128 + lane * 4;
        const float4 mine = *reinterpret_cast<const float4*>(p.yhat + static_cast<size_t>(row) * p.out + col);
        unsigned int c = 0;
        if (lane == 0) c = p.done[u] + 1;
        c = __shfl_sync(0xffffffffu, c, 0);
        const size_t at = ((c & 1u) * p.world + p.rank) * slot_floats + static_cast<size_t>(u) * 128 + lane * 4;
        for (int r = 0; r < p.world; ++r) *reinterpret_cast<float4*>(p.inbox[r] + at) = mine;
        __threadfence_system();
        __syncwarp();
        if (lane < p.world) store_release_sys(p.flags[lane] + static_cast<size_t>(p.rank) * p.max_units + u, c);
        // every lane below `world` watches one source rank
        bool arrived = true;
        if (lane < p.world && *reinterpret_cast<volatile unsigned int*>(p.error) == 0) {
            const unsigned int* flag = my_flags + static_cast<size_t>(lane) * p.max_units + u;
            arrived = static_cast<int>(load_acquire_sys(flag) - c) >= 0;
            if (!arrived) {
                const unsigned long long t0 = global_ns();
                for (int i = 1; !arrived; ++i) {
                    arrived = static_cast<int>(load_acquire_sys(flag) - c) >= 0;
                    if (!arrived && (i & 255) == 0 && global_ns() - t0 > 4000000000ull) break;
                }
            }
        }
        if (!__all_sync(0xffffffffu, arrived)) {
            if (lane == 0) atomicExch(p.error, 4u);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int src = 0; src < p.world; ++src) {
            const float4 v = __ldcv(reinterpret_cast<const float4*>(
                my_inbox + ((c & 1u) * p.world + src) * slot_floats + static_cast<size_t>(u) * 128 + lane * 4));
            if (src == 0) acc = v;
            else { acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w); }
        }
        __half h[4] = {__float2half_rn(acc.x), __float2half_rn(acc.y), __float2half_rn(acc.z), __float2half_rn(acc.w)};
        warp_hadamard128_f16(h, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            store_from_half(p.y, p.y_dtype, static_cast<int64_t>(row) * p.out + col + j, __hmul_rn(h[j], p.svh[col + j]), p.bias, col + j);
        if (lane == 0) p.done[u] = c;
    }
}

}  // namespace

cudaError_t launch_tp_finish(const TpArgs& args, cudaStream_t stream) {
    const int units = args.rows * (args.out / 128);
    if (units <= 0 || units > args.max_units || args.world < 1 || args.world > kTpMaxWorld) return cudaErrorInvalidValue;
    // every rank must use the same grid: it only depends on the unit count
    const int grid = (units + kTpWarps - 1) / kTpWarps;
    tp_finish_kernel<<<grid < 4 * kSmCount ? grid : 4 * kSmCount, kTpWarps * 32, 0, stream>>>(args);
    return cudaGetLastError();
}

}  // namespace b200exl3
