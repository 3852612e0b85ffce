// Hadamard-128 rotation with the rounding points of the reference (MLX's fp16 hadamard_transform;
// native/shaders/exl3.metal:156-170, native/src/linear.rs:1383-1427): butterflies at strides
// 1,2,4,...,64 in fp32, every value rounded to fp16 after the stride-8 stage and after the
// stride-64 stage, then multiplied by 2^-3.5 in fp32 and rounded to fp16.
//
// One warp rotates one 128-block: lane l holds elements 4l..4l+3, so strides 1 and 2 are
// register-local and strides 4..64 are lane-xor shuffles 1..16.  The stage order is the
// reference's, which matters because fp32 addition is not associative.
#pragma once

#include "common.cuh"

namespace b200exl3 {

__device__ __forceinline__ float round_half(float v) { return __half2float(__float2half_rn(v)); }
// SiLU of the expert glue (native/src/moe.rs:486): the exponential is evaluated in fp32 (expf); the reference's Metal
// `exp` is a fast-math intrinsic whose last bits are not specified, so this glue is compared with a tolerance.
__device__ __forceinline__ float glu_silu(float v) { return __fdiv_rn(v, __fadd_rn(1.0f, expf(-v))); }

// round_mid / round_end: fp16 rounding after stride 8 / stride 64.  The MoE activation glue of the
// reference (native/src/moe.rs:27-53, SiLU models) clears both.
template <bool ROUND_MID, bool ROUND_END>
__device__ __forceinline__ void warp_hadamard128(float (&v)[4], int lane) {
    float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]);
    float a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a0, a2); v[1] = __fadd_rn(a1, a3);
    v[2] = __fsub_rn(a0, a2); v[3] = __fsub_rn(a1, a3);
#pragma unroll
    for (int bit = 1; bit <= 16; bit <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float peer = __shfl_xor_sync(0xffffffffu, v[j], bit);
            float r = (lane & bit) ? __fsub_rn(peer, v[j]) : __fadd_rn(v[j], peer);
            if ((bit == 2 && ROUND_MID) || (bit == 16 && ROUND_END)) r = round_half(r);
            v[j] = r;
        }
    }
}

// fp16 values in, fp16 values out (scale included): the transform applied to xhat and to the output.
__device__ __forceinline__ void warp_hadamard128_f16(__half (&h)[4], int lane) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __half2float(h[j]);
    warp_hadamard128<true, true>(v, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __float2half_rn(__fmul_rn(v[j], had_scale()));
}

}  // namespace b200exl3
