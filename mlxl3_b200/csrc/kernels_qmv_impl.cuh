// Fused trellis-decode x activation product for up to 32 activation rows (QMV and small-batch QMM).
//
// Reference behaviour replaced: native/shaders/_qmv_tile_kernel.metal (M = 1 and the MB row-sharing
// layouts) driven by native/src/linear.rs:934-955 and 1138-1175.  Output: fp32 partial sums
// partials[split, row, n] = sum_{k in split} float(xhat[row, k]) * W[k, n].
//
// Design (B200): the kernel is bound by HBM bandwidth and by the integer work of the decode, so
//  * packed trellis words are staged with 16-byte cp.async copies into a per-warp ring in shared
//    memory (no registers held by loads in flight, every byte read once);
//  * each warp decodes a 16x16 tile in registers: lane L owns states 8L..8L+7, which are exactly
//    the A-fragment of mma.m16n8k16 for W^T (rows = output columns, cols = inputs);
//  * the multiply by the activations runs on the tensor cores with the activation rows in the
//    n dimension, so 1..8 rows cost the same and the fp32 accumulators live in the MMA fragment;
//  * for codebooks 0 and 1 the weight is lo + hi of two fp16 halves; in the default "split" mode
//    the two halves are fed as two k elements against a duplicated activation, which removes the
//    fp16 add from the decode (x*(lo+hi) = x*lo + x*hi, accumulated in fp32).  "exact" mode adds
//    the halves first and reproduces the reference's fp16 weight bit for bit;
//  * work is cut into units of one tile; a CTA owns one 128-column block and one contiguous slice
//    of that block's tiles_k*8 units, and its warps own equal contiguous sub-slices, so the load
//    is balanced to one tile whatever the shape.
//
// Included by one small translation unit per K so the eight K values compile in parallel.
#pragma once

#include "codec.cuh"
#include "kernels.h"

namespace b200exl3 {

// rows of 8 tiles kept in flight per warp
__host__ __device__ constexpr int qmv_depth(int k) { return k <= 2 ? 8 : 4; }

constexpr int kQmvRedStride = 132;   // floats per reduced row: 128 + 4 keeps the fragment stores conflict-free

struct QmvParams {
    const uint32_t* trellis;   // [tiles_k, tiles_n, 8K] words
    const __half* xhat;        // [rows, in]
    float* partials;           // [splits, rows, out]
    int in, out, rows, tiles_k, tiles_n, splits;
};

template <int K>
__device__ __forceinline__ void qmv_issue_row(const uint32_t* __restrict__ trellis, int tiles_n, int tk, int tn0,
                                              int lo, int hi, uint32_t* slot, int lane) {
    constexpr int kChunksPerTile = 2 * K;                  // 16-byte chunks
    const char* src = reinterpret_cast<const char*>(trellis + (static_cast<int64_t>(tk) * tiles_n + tn0) * (8 * K));
    char* dst = reinterpret_cast<char*>(slot);
#pragma unroll
    for (int c = lane; c < 8 * kChunksPerTile; c += 32) {
        int tile = c / kChunksPerTile;
        if (tile >= lo && tile < hi) cp_async_16(dst + c * 16, src + c * 16);
    }
}

// MODE 0: codebook 0/1, split halves.  MODE 1: exact fp16 weights (all codebooks).
template <int K, int CB, int NB, int MODE, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
qmv_kernel(const QmvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kRowWords = 64 * K;                      // 8 tiles x 8K words
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int col_blocks = p.out >> 7;
    const int cblock = blockIdx.x % col_blocks;
    const int split = blockIdx.x / col_blocks;
    const int tn0 = cblock * 8;
    constexpr int DEPTH = qmv_depth(K);

    // unit range of this CTA, then of this warp
    const int units = p.tiles_k * 8;
    const int cta_u0 = static_cast<int>(static_cast<int64_t>(units) * split / p.splits);
    const int cta_u1 = static_cast<int>(static_cast<int64_t>(units) * (split + 1) / p.splits);
    const int cta_n = cta_u1 - cta_u0;
    const int u0 = cta_u0 + static_cast<int>(static_cast<int64_t>(cta_n) * warp / WARPS);
    const int u1 = cta_u0 + static_cast<int>(static_cast<int64_t>(cta_n) * (warp + 1) / WARPS);

    float acc[NB][8][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nb][t][i] = 0.0f;

    uint32_t* ring = reinterpret_cast<uint32_t*>(smem_raw) + static_cast<size_t>(warp) * DEPTH * kRowWords;

    if (u1 > u0) {
        const int tk_first = u0 >> 3, tk_last = (u1 - 1) >> 3;
        const int nrows = tk_last - tk_first + 1;
        for (int i = 0; i < DEPTH; ++i) {
            if (i < nrows) {
                int tk = tk_first + i;
                qmv_issue_row<K>(p.trellis, p.tiles_n, tk, tn0, max(u0 - 8 * tk, 0), min(u1 - 8 * tk, 8),
                                 ring + i * kRowWords, lane);
            }
            cp_async_commit();
        }
        int slot = 0;
        for (int r = 0; r < nrows; ++r) {
            const int tk = tk_first + r;
            // activation fragments for this input tile: rows nb*8+g, inputs 16tk + {2q,2q+1,2q+8,2q+9}
            uint32_t bx[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const int row = nb * 8 + g;
                uint32_t p0 = 0, p1 = 0;
                if (row < p.rows) {
                    const uint32_t* xr = reinterpret_cast<const uint32_t*>(p.xhat + static_cast<int64_t>(row) * p.in + tk * 16);
                    p0 = __ldg(xr + q);
                    p1 = __ldg(xr + q + 4);
                }
                if constexpr (MODE == 0) {
                    bx[nb][0] = prmt(p0, p0, 0x1010); bx[nb][1] = prmt(p0, p0, 0x3232);
                    bx[nb][2] = prmt(p1, p1, 0x1010); bx[nb][3] = prmt(p1, p1, 0x3232);
                } else {
                    bx[nb][0] = p0; bx[nb][1] = p1; bx[nb][2] = 0; bx[nb][3] = 0;
                }
            }
            // every iteration commits one group, so row r's group is complete once at most
            // DEPTH-1 newer groups are pending
            cp_async_wait<DEPTH - 1>();
            __syncwarp();
            const uint32_t* row_words = ring + slot * kRowWords;
            const int lo = max(u0 - 8 * tk, 0), hi = min(u1 - 8 * tk, 8);
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                if (t >= lo && t < hi) {
                    uint32_t st[8];
                    lane_states<K>(row_words + t * (8 * K), lane, st);
                    if constexpr (MODE == 0) {
                        uint32_t a[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = codeword_halves<CB>(st[j]);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            mma_16816(acc[nb][t], a[0], a[4], a[1], a[5], bx[nb][0], bx[nb][1]);
                            mma_16816(acc[nb][t], a[2], a[6], a[3], a[7], bx[nb][2], bx[nb][3]);
                        }
                    } else {
                        uint32_t a0, a1, a2, a3;
                        if constexpr (CB == 2) {
                            uint32_t s[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) s[j] = mul1_sum_bits(st[j]);
                            const __half2 inv = __half2half2(__ushort_as_half(0x1eee));
                            const __half2 bias = __half2half2(__ushort_as_half(0xc931));
                            auto pair = [&](uint32_t x, uint32_t y) {
                                uint32_t v = prmt(x, y, 0x5410);
                                __half2 w = __hfma2(*reinterpret_cast<__half2*>(&v), inv, bias);
                                return *reinterpret_cast<uint32_t*>(&w);
                            };
                            a0 = pair(s[0], s[1]); a1 = pair(s[4], s[5]); a2 = pair(s[2], s[3]); a3 = pair(s[6], s[7]);
                        } else {
                            uint32_t v[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = codeword_halves<CB>(st[j]);
                            auto pair = [&](uint32_t x, uint32_t y) {
                                uint32_t lo2 = prmt(x, y, 0x5410), hi2 = prmt(x, y, 0x7632);
                                __half2 w = __hadd2(*reinterpret_cast<__half2*>(&lo2), *reinterpret_cast<__half2*>(&hi2));
                                return *reinterpret_cast<uint32_t*>(&w);
                            };
                            a0 = pair(v[0], v[1]); a1 = pair(v[4], v[5]); a2 = pair(v[2], v[3]); a3 = pair(v[6], v[7]);
                        }
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) mma_16816(acc[nb][t], a0, a1, a2, a3, bx[nb][0], bx[nb][1]);
                    }
                }
            }
            __syncwarp();
            if (r + DEPTH < nrows) {
                int tkn = tk + DEPTH;
                qmv_issue_row<K>(p.trellis, p.tiles_n, tkn, tn0, max(u0 - 8 * tkn, 0), min(u1 - 8 * tkn, 8),
                                 ring + slot * kRowWords, lane);
            }
            cp_async_commit();
            slot = slot + 1 == DEPTH ? 0 : slot + 1;
        }
        cp_async_wait<0>();
    }

    // ---- deterministic tree reduction over the warps, then coalesced store of the partial sums ----
    __syncthreads();                                        // the ring is dead from here on
    float* red = reinterpret_cast<float*>(smem_raw);
    const int rows = p.rows;
    auto frag_store = [&](float* base) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    int row = nb * 8 + 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                    if (row < rows) base[row * kQmvRedStride + col] = acc[nb][t][i];
                }
    };
    auto frag_add = [&](const float* base) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    int row = nb * 8 + 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                    if (row < rows) acc[nb][t][i] = __fadd_rn(acc[nb][t][i], base[row * kQmvRedStride + col]);
                }
    };
    const int slab = rows * kQmvRedStride;
#pragma unroll
    for (int half = WARPS / 2; half >= 1; half >>= 1) {
        if (warp >= half && warp < 2 * half) frag_store(red + (warp - half) * slab);
        __syncthreads();
        if (warp < half) frag_add(red + warp * slab);
        __syncthreads();
    }
    if (warp == 0) frag_store(red);
    __syncthreads();
    float* dst = p.partials + static_cast<int64_t>(split) * rows * p.out + cblock * 128;
    for (int i = threadIdx.x; i < rows * 128; i += WARPS * 32) {
        int row = i >> 7, col = i & 127;
        dst[static_cast<int64_t>(row) * p.out + col] = red[row * kQmvRedStride + col];
    }
}

constexpr int kQmvWarps = 8;

template <int K, int CB, int NB, int MODE>
cudaError_t qmv_launch_one(const QmvParams& p, const QmvPlan& plan, cudaStream_t stream) {
    auto kernel = qmv_kernel<K, CB, NB, MODE, kQmvWarps>;
    if (plan.smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(plan.smem_bytes));
        if (e != cudaSuccess) return e;
    }
    kernel<<<static_cast<unsigned>(plan.col_blocks * plan.splits), kQmvWarps * 32, plan.smem_bytes, stream>>>(p);
    return cudaGetLastError();
}

template <int K, int CB, int MODE>
cudaError_t qmv_launch_nb(const QmvParams& p, const QmvPlan& plan, cudaStream_t stream) {
    if (p.rows <= 8) return qmv_launch_one<K, CB, 1, MODE>(p, plan, stream);
    if (p.rows <= 16) return qmv_launch_one<K, CB, 2, MODE>(p, plan, stream);
    return qmv_launch_one<K, CB, 4, MODE>(p, plan, stream);
}

template <int K>
cudaError_t qmv_launch_k(const QmvParams& p, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (cb == 2) return qmv_launch_nb<K, 2, 1>(p, plan, stream);
    if (cb == 0) return exact ? qmv_launch_nb<K, 0, 1>(p, plan, stream) : qmv_launch_nb<K, 0, 0>(p, plan, stream);
    return exact ? qmv_launch_nb<K, 1, 1>(p, plan, stream) : qmv_launch_nb<K, 1, 0>(p, plan, stream);
}

}  // namespace b200exl3
