// Row-parallel layers across GPUs: the sum of the ranks' fp32 partial products and the output rotation
// in one kernel, over peer memory (NVLink), with no library collective.
//
// Reference behaviour kept: the partial products are the reference's split-K partials
// (native/src/linear.rs:978-982); they are added in fp32, in rank order on every rank (so all ranks
// hold bit-identical outputs), then rounded to fp16, rotated and scaled as in linear.rs:983-996.
//
// The exchange itself (peer stores of {value, sequence} words, bounded wait, rank-ordered sum) is tp_exchange_unit.
#include "hadamard.cuh"
#include "kernels.h"
#include "tp_exchange.cuh"

namespace b200exl3 {

namespace {

constexpr int kTpWarps = 4;

__global__ void __launch_bounds__(kTpWarps * 32)
tp_finish_kernel(TpArgs p) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = p.out >> 7;
    const int units = p.rows * blocks_per_row;
    for (int u = blockIdx.x * kTpWarps + (threadIdx.x >> 5); u < units; u += gridDim.x * kTpWarps) {
        const int row = u / blocks_per_row, col = (u - row * blocks_per_row) * 128 + lane * 4;
        const float4 mine = *reinterpret_cast<const float4*>(p.yhat + static_cast<size_t>(row) * p.out + col);
        const float4 acc = tp_exchange_unit(p.peers, u, mine, lane);
        __half h[4] = {__float2half_rn(acc.x), __float2half_rn(acc.y), __float2half_rn(acc.z), __float2half_rn(acc.w)};
        warp_hadamard128_f16(h, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            store_from_half(p.y, p.y_dtype, static_cast<int64_t>(row) * p.out + col + j, __hmul_rn(h[j], p.svh[col + j]), p.bias, col + j);
    }
}

}  // namespace

cudaError_t launch_tp_finish(const TpArgs& args, cudaStream_t stream) {
    const int units = args.rows * (args.out / 128);
    if (units <= 0 || units > args.peers.max_units || args.peers.world < 1 || args.peers.world > kTpMaxWorld) return cudaErrorInvalidValue;
    // every rank must use the same grid: it only depends on the unit count
    const int grid = (units + kTpWarps - 1) / kTpWarps;
    tp_finish_kernel<<<grid < 4 * sm_count() ? grid : 4 * sm_count(), kTpWarps * 32, 0, stream>>>(args);
    return cudaGetLastError();
}

}  // namespace b200exl3
