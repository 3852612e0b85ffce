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
// that every row segment (256 bytes) leaves as whole sectors.  QUADS selects the weight layout:
// false = checkpoint layout [tiles_k, tiles_n, 8K] words, true = quad layout [tiles_n/8, tiles_k, 2, 8K, 4].
template <bool QUADS>
__global__ void __launch_bounds__(256)
reconstruct_kernel(const uint32_t* __restrict__ trellis, int tiles_k, int tiles_n, int k, int cb,
                   __half* __restrict__ w) {
    __shared__ __align__(16) __half strip[16][128 + 8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int strips_n = (tiles_n + 7) / 8;
    const int tk = blockIdx.x / strips_n;
    const int tn0 = (blockIdx.x % strips_n) * 8;
    const int tn = tn0 + warp;
    if (tn < tiles_n) {
        const int64_t tile = static_cast<int64_t>(tk) * tiles_n + tn;
        const uint32_t* words = QUADS ? trellis + quad_row_offset(tk, tn >> 3, tiles_k, k) + ((tn >> 2) & 1) * (32 * k) + (tn & 3)
                                      : trellis + tile * (8 * k);
        const int r = (lane & 3) * 2, c = lane >> 2;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t s = tile_state_strided(words, QUADS ? 4 : 1, k, lane * 8 + j);
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

// One thread per 16-byte chunk of the quad layout: word w of four neighbouring tiles.  `quads` counts the source's
// groups of four tiles in checkpoint order (tile row, then column).
__global__ void repack_quads_kernel(const uint32_t* __restrict__ trellis, int64_t quads, int tiles_k, int tiles_n, int k,
                                    uint32_t* __restrict__ wq) {
    const int64_t chunk = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int nw = 8 * k;
    if (chunk >= quads * nw) return;
    const int64_t quad = chunk / nw;
    const int wi = static_cast<int>(chunk % nw);
    const uint32_t* src = trellis + quad * 4 * nw + wi;
    uint4 v = make_uint4(src[0], src[nw], src[2 * nw], src[3 * nw]);
    const int quads_n = tiles_n / 4;
    const int tk = static_cast<int>(quad / quads_n), qn = static_cast<int>(quad % quads_n);
    uint32_t* dst = wq + quad_row_offset(tk, qn >> 1, tiles_k, k) + (qn & 1) * (32 * k) + wi * 4;
    *reinterpret_cast<uint4*>(dst) = v;
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
    reconstruct_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const uint32_t*>(trellis), tiles_k, tiles_n, k, cb, w);
    return cudaGetLastError();
}

cudaError_t launch_reconstruct_quads(const uint32_t* wq, int tiles_k, int tiles_n, int k, int cb, __half* w,
                                     cudaStream_t stream) {
    int64_t blocks = static_cast<int64_t>(tiles_k) * ((tiles_n + 7) / 8);
    if (blocks == 0) return cudaSuccess;
    reconstruct_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(wq, tiles_k, tiles_n, k, cb, w);
    return cudaGetLastError();
}

cudaError_t launch_repack_quads(const uint32_t* trellis, int tiles_k, int tiles_n, int k, uint32_t* wq, cudaStream_t stream) {
    const int64_t quads = static_cast<int64_t>(tiles_k) * (tiles_n / 4);
    const int64_t chunks = quads * 8 * k;
    if (chunks == 0) return cudaSuccess;
    repack_quads_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, stream>>>(trellis, quads, tiles_k, tiles_n, k, wq);
    return cudaGetLastError();
}

}  // namespace b200exl3
