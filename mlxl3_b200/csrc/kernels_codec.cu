// Stand-alone, bit-exact codec kernels: trellis -> states -> fp16, and the whole-matrix
// reconstruction W[in, out] (reference: native/src/codec.rs:159-190, native/shaders/exl3.metal:85-114,
// native/shaders/lfm3_reconstruct.metal).  These use the per-state window formula, so they are an
// implementation independent of the lane-window reader inside the fused product kernels.
#include "codec.cuh"
#include "kernels.h"

namespace b200exl3 {

// One thread per state: states[tile*256 + t] and/or values[tile*256 + t] in kernel order.
__global__ void unpack_states_kernel(const uint16_t* __restrict__ packed, int64_t tiles, int k, int cb,
                                     uint16_t* __restrict__ states, __half* __restrict__ values) {
    int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= tiles * 256) return;
    uint32_t s = tile_state(packed + (e >> 8) * 16 * k, k, static_cast<int>(e & 255));
    if (states) states[e] = static_cast<uint16_t>(s);
    if (values) values[e] = decode_codeword_rt(s, cb);
}

__global__ void codebook_kernel(const uint16_t* __restrict__ states, int64_t n, int cb, __half* __restrict__ values) {
    int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < n) values[e] = decode_codeword_rt(states ? states[e] : static_cast<uint32_t>(e), cb);
}

// One CTA of 256 threads reconstructs a strip of 8 tiles: 16 rows x 128 columns of W.  Each warp
// decodes one tile into shared memory in row-major order; the CTA then writes 16-byte pieces so
// that every row segment (256 bytes) leaves as whole sectors.
__global__ void __launch_bounds__(256)
reconstruct_kernel(const uint16_t* __restrict__ trellis, int tiles_k, int tiles_n, int k, int cb,
                   __half* __restrict__ w) {
    __shared__ __align__(16) __half strip[16][128 + 8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strips_n = (tiles_n + 7) / 8;
    const int tk = blockIdx.x / strips_n;
    const int tn0 = (blockIdx.x % strips_n) * 8;
    const int tn = tn0 + warp;
    if (tn < tiles_n) {
        const uint16_t* tile = trellis + (static_cast<int64_t>(tk) * tiles_n + tn) * 16 * k;
        const int r = (lane & 3) * 2, c = lane >> 2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t s = tile_state(tile, k, lane * 8 + j);
            int row = r + (j & 1) + ((j & 2) ? 8 : 0);
            int col = c + ((j & 4) ? 8 : 0);
            strip[row][warp * 16 + col] = decode_codeword_rt(s, cb);
        }
    }
    __syncthreads();
    const int out = tiles_n * 16;
    const int row = threadIdx.x >> 4, piece = threadIdx.x & 15;      // 16 rows x 16 pieces of 8 halves
    const int col = tn0 * 16 + piece * 8;
    if (col < out) {
        uint4 v = *reinterpret_cast<const uint4*>(&strip[row][piece * 8]);
        *reinterpret_cast<uint4*>(w + (static_cast<int64_t>(tk) * 16 + row) * out + col) = v;
    }
}

cudaError_t launch_unpack_states(const uint16_t* packed, int64_t tiles, int k, int cb, uint16_t* states, __half* values,
                                 cudaStream_t stream) {
    if (tiles == 0) return cudaSuccess;
    int64_t n = tiles * 256;
    unpack_states_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(packed, tiles, k, cb, states, values);
    return cudaGetLastError();
}

cudaError_t launch_codebook(const uint16_t* states, int64_t n, int cb, __half* values, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    codebook_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(states, n, cb, values);
    return cudaGetLastError();
}

cudaError_t launch_reconstruct(const uint16_t* trellis, int tiles_k, int tiles_n, int k, int cb, __half* w,
                               cudaStream_t stream) {
    int64_t blocks = static_cast<int64_t>(tiles_k) * ((tiles_n + 7) / 8);
    if (blocks == 0) return cudaSuccess;
    reconstruct_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(trellis, tiles_k, tiles_n, k, cb, w);
    return cudaGetLastError();
}

}  // namespace b200exl3
