// Input and output rotations of the EXL3 linear layer as stand-alone kernels
// (reference: native/src/linear.rs:855-861 and 978-996; native/shaders/_lane_prologue.metal,
// _lane_epilogue.metal, exl3.metal:204-235).  One warp per 128-block of one row.
#include "hadamard.cuh"
#include "kernels.h"

namespace b200exl3 {

__global__ void __launch_bounds__(256)
prepare_kernel(const void* __restrict__ x, int x_dtype, const __half* __restrict__ suh, int64_t scale_rows,
               int64_t rows, int in, __half* __restrict__ xhat, const __half* __restrict__ glu_up) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = in >> 7;
    const int64_t total = rows * blocks_per_row;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int64_t row = unit / blocks_per_row;
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        const __half* s = suh + (scale_rows == 1 ? 0 : row * in) + col;
        __align__(8) __half h[4];
        if (glu_up != nullptr) {
            // SwiGLU of two fp16 row sets as the input (x = gate rows): half(gate * sigmoid(gate)) * up, each product
            // rounded to half, the arithmetic of the stand-alone SwiGLU kernel and of the small-batch prologue
            const uint2 gv = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(x) + row * in + col);
            const uint2 uv = *reinterpret_cast<const uint2*>(glu_up + row * in + col);
            const __half2* gh = reinterpret_cast<const __half2*>(&gv);
            const __half2* uh = reinterpret_cast<const __half2*>(&uv);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float2 f = __half22float2(gh[j]);
                const __half2 sg = __floats2half2_rn(1.0f / (1.0f + expf(-f.x)), 1.0f / (1.0f + expf(-f.y)));
                const __half2 v = __hmul2_rn(__hmul2_rn(gh[j], sg), uh[j]);
                h[2 * j] = __hmul_rn(__low2half(v), s[2 * j]);
                h[2 * j + 1] = __hmul_rn(__high2half(v), s[2 * j + 1]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(load_as_half(x, x_dtype, row * in + col + j), s[j]);
        }
        warp_hadamard128_f16(h, lane);
        *reinterpret_cast<uint2*>(xhat + row * in + col) = *reinterpret_cast<uint2*>(h);
    }
}

__global__ void __launch_bounds__(256)
finish_kernel(const float* __restrict__ partials, int splits, int64_t split_stride, const __half* __restrict__ svh,
              int64_t scale_rows, const __half* __restrict__ bias, int64_t rows, int out, int y_dtype,
              void* __restrict__ y) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = out >> 7;
    const int64_t total = rows * blocks_per_row;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5)) {
        const int64_t row = unit / blocks_per_row;
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        const float* src = partials + row * out + col;
        float4 acc = *reinterpret_cast<const float4*>(src);
        for (int s0 = 1; s0 < splits; s0 += 8) {         // splits are added in order, in fp32; loads go out together
            float4 part[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) part[j] = *reinterpret_cast<const float4*>(src + (s0 + j) * split_stride);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) {
                    acc.x = __fadd_rn(acc.x, part[j].x); acc.y = __fadd_rn(acc.y, part[j].y);
                    acc.z = __fadd_rn(acc.z, part[j].z); acc.w = __fadd_rn(acc.w, part[j].w);
                }
        }
        __half h[4] = {__float2half_rn(acc.x), __float2half_rn(acc.y), __float2half_rn(acc.z), __float2half_rn(acc.w)};
        warp_hadamard128_f16(h, lane);
        const __half* s = svh + (scale_rows == 1 ? 0 : row * out) + col;
#pragma unroll
        for (int j = 0; j < 4; ++j) store_from_half(y, y_dtype, row * out + col + j, __hmul_rn(h[j], s[j]), bias, col + j);
    }
}

static unsigned grid_for(int64_t units) {
    int64_t blocks = (units + 7) / 8;
    int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

cudaError_t launch_prepare(const void* x, int x_dtype, const __half* suh, int64_t scale_rows, int64_t rows, int in,
                           __half* xhat, cudaStream_t stream, const __half* glu_up) {
    if (rows == 0) return cudaSuccess;
    if (glu_up != nullptr && x_dtype != kF16) return cudaErrorInvalidValue;
    return launch_dependent(prepare_kernel, dim3(grid_for(rows * (in / 128))), dim3(256), 0, stream, x, x_dtype, suh, scale_rows, rows, in, xhat,
                            glu_up);
}

cudaError_t launch_finish(const float* partials, int splits, int64_t split_stride, const __half* svh,
                          int64_t scale_rows, const __half* bias, int64_t rows, int out, int y_dtype, void* y,
                          cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    return launch_dependent(finish_kernel, dim3(grid_for(rows * (out / 128))), dim3(256), 0, stream, partials, splits, split_stride, svh,
                            scale_rows, bias, rows, out, y_dtype, y);
}

}  // namespace b200exl3
