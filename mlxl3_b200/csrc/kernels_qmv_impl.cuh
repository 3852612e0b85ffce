// Fused EXL3 linear layer for up to 32 activation rows (QMV and small-batch QMM) in ONE launch:
// input rotation -> trellis decode x activation product -> split reduction -> output rotation.
//
// Reference behaviour replaced: native/shaders/_qmv_tile_kernel.metal (M = 1 and the MB row-sharing
// layouts) with its prologue / epilogue kernels (_lane_prologue.metal, _lane_epilogue.metal), driven
// by native/src/linear.rs:847-996 and 1024-1216.
//
// Design (B200).  The layer is bound by HBM bandwidth and, at low K, by the integer work of the
// decode (about 30 instructions per 16x16 tile is the floor), so everything that is not decode is
// kept off the issue slots:
//  * weights live in a "quad" layout made once at load (4 neighbouring tiles interleaved word by
//    word), so one 16-byte shared-memory load gives a lane its stream word for four tiles;
//  * packed words are staged with 16-byte cp.async copies into a per-warp ring in shared memory,
//    issued before anything that depends on the activations;
//  * lane L owns states 8L..8L+7 of a tile, which are exactly the A-fragment of mma.m16n8k16 for
//    W^T; the product runs on the tensor cores with the activation rows in the n dimension, so
//    1..8 rows cost the same and the fp32 accumulators are the MMA fragment;
//  * codebooks 0/1: the weight is lo + hi of two fp16 halves of a 32-bit hash.  In the default
//    "split" mode the halves are fed as two k elements against a duplicated activation
//    (x*lo + x*hi in fp32), which removes the fp16 add; "exact" mode adds the halves first and
//    reproduces the reference's fp16 weight bit for bit;
//  * for K = 4 and K = 8 two states 16 bits apart share a register P = lo | hi << 16; then
//    b_hi = (P >> 16) * M + C,  T = P * M + (C + (C << 16)),  b_lo = T - (b_hi << 16)
//    hashes both without masking the low state (integer multiply-add pipe instead of the ALU pipe);
//  * a CTA owns one 128-column block and a contiguous slice of that block's tiles; its warps own
//    equal contiguous sub-slices (balanced to one tile).  The activations of the slice are rotated
//    into shared memory by the CTA itself; the last CTA to finish a column block sums the split
//    partials in a fixed order and applies the output rotation.
//
// Included by one small translation unit per K so the eight K values compile in parallel.
#pragma once

#include "codec.cuh"
#include "hadamard.cuh"
#include "kernels.h"

namespace b200exl3 {

// ---- hash of the eight states of a lane -------------------------------------------------------------

template <int CB>
__device__ __forceinline__ constexpr uint32_t hash_mul() { return CB == 0 ? 89226354u : (CB == 1 ? 0xcbac1fedu : 0x83dcd12du); }
template <int CB>
__device__ __forceinline__ constexpr uint32_t hash_add() { return CB == 0 ? 64248484u : 0u; }

// b[j] = state_j * M + C for the lane's states j = 0..7 (32-bit wrap-around).  (w0:w1:w2) are the
// stream words that end at the word holding the lane's last bit; `slack` bits of w2 lie past it.
template <int K, int CB>
__device__ __forceinline__ void lane_hashes(uint32_t w2, uint32_t w1, uint32_t w0, int slack, uint32_t (&b)[8]) {
    constexpr uint32_t M = hash_mul<CB>(), C = hash_add<CB>();
    if constexpr (K == 4 || K == 8) {
        uint32_t P[4];
        if constexpr (K == 4) {
            // states at bit offsets 0,4,...,28: P[p] = {offset 4p (state 7-p), offset 4p+16 (state 3-p)}
            P[0] = w2; P[1] = __funnelshift_r(w2, w1, 4); P[2] = __funnelshift_r(w2, w1, 8); P[3] = __funnelshift_r(w2, w1, 12);
        } else {
            // states at bit offsets 0,8,...,56: {0,16} {8,24} {32,48} {40,56} = states {7,5} {6,4} {3,1} {2,0}
            P[0] = w2; P[1] = __funnelshift_r(w2, w1, 8);
            P[2] = w1; P[3] = __funnelshift_r(w1, w0, 8);
        }
        constexpr uint32_t C2 = C + (C << 16);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t hi = P[p] >> 16;
            const uint32_t bh = hi * M + C;
            const uint32_t t = P[p] * M + C2;
            uint32_t bl;                                   // t - (bh << 16) as one multiply-add
            asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(bl) : "r"(bh), "r"(0xffff0000u), "r"(t));
            if constexpr (K == 4) {
                b[7 - p] = bl; b[3 - p] = bh;
            } else {
                const int jl = p == 0 ? 7 : (p == 1 ? 6 : (p == 2 ? 3 : 2));
                b[jl] = bl; b[jl - 2] = bh;
            }
        }
    } else {
        const uint32_t n2 = __funnelshift_r(w2, w1, slack);
        const uint32_t n1 = __funnelshift_r(w1, w0, slack);
        const uint32_t n0 = w0 >> slack;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = (7 - j) * K;
            uint32_t v;
            if (c + 16 <= 32) v = n2 >> c;
            else if (c < 32) v = __funnelshift_r(n2, n1, c);
            else if (c + 16 <= 64) v = n1 >> (c - 32);
            else if (c < 64) v = __funnelshift_r(n1, n0, c - 32);
            else v = n0 >> (c - 64);
            b[j] = (v & 0xffffu) * M + C;
        }
    }
}

// Per-lane geometry of the stream words, constant for the whole kernel.
template <int K>
struct LaneGeom {
    int i2, i1, i0, slack;     // word indices inside a tile; bits of word i2 that lie past the lane's last bit
    __device__ __forceinline__ explicit LaneGeom(int lane) {
        constexpr int NW = 8 * K;
        const int end = 8 * K * (lane + 1);
        i2 = (end - 1) >> 5;
        slack = ((i2 + 1) << 5) - end;
        i1 = i2 >= 1 ? i2 - 1 : i2 - 1 + NW;
        i0 = i2 >= 2 ? i2 - 2 : i2 - 2 + NW;
    }
};

// One tile: decode the lane's eight weights and issue the MMAs against the activation fragments.
// MODE 0: codebook 0/1, split halves (2 MMAs per 8 rows).  MODE 1: exact fp16 weights (1 MMA per 8 rows).
template <int K, int CB, int NB, int MODE>
__device__ __forceinline__ void tile_mma(uint32_t w2, uint32_t w1, uint32_t w0, int slack, const uint32_t (&bx)[NB][4],
                                         float (&acc)[NB][4]) {
    uint32_t b[8];
    lane_hashes<K, CB>(w2, w1, w0, slack, b);
    if constexpr (MODE == 0) {
        uint32_t a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = lop3_and_xor(b[j], 0x8fff8fffu, 0x3b603b60u);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            mma_16816(acc[nb], a[0], a[4], a[1], a[5], bx[nb][0], bx[nb][1]);
            mma_16816(acc[nb], a[2], a[6], a[3], a[7], bx[nb][2], bx[nb][3]);
        }
    } else {
        uint32_t a0, a1, a2, a3;
        if constexpr (CB == 2) {
            const __half2 inv = __half2half2(__ushort_as_half(0x1eee));
            const __half2 bias = __half2half2(__ushort_as_half(0xc931));
            auto pair = [&](uint32_t x, uint32_t y) {
                uint32_t v = prmt(__dp4a(x, 0x01010101u, 0x6400u), __dp4a(y, 0x01010101u, 0x6400u), 0x5410);
                __half2 w = __hfma2(*reinterpret_cast<__half2*>(&v), inv, bias);
                return *reinterpret_cast<uint32_t*>(&w);
            };
            a0 = pair(b[0], b[1]); a1 = pair(b[4], b[5]); a2 = pair(b[2], b[3]); a3 = pair(b[6], b[7]);
        } else {
            auto pair = [&](uint32_t x, uint32_t y) {
                x = lop3_and_xor(x, 0x8fff8fffu, 0x3b603b60u);
                y = lop3_and_xor(y, 0x8fff8fffu, 0x3b603b60u);
                uint32_t lo2 = prmt(x, y, 0x5410), hi2 = prmt(x, y, 0x7632);
                __half2 w = __hadd2_rn(*reinterpret_cast<__half2*>(&lo2), *reinterpret_cast<__half2*>(&hi2));
                return *reinterpret_cast<uint32_t*>(&w);
            };
            a0 = pair(b[0], b[1]); a1 = pair(b[4], b[5]); a2 = pair(b[2], b[3]); a3 = pair(b[6], b[7]);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_16816(acc[nb], a0, a1, a2, a3, bx[nb][0], bx[nb][1]);
    }
}

// All tiles [lo, hi) of one staged row.  FULL rows carry no per-tile tests.
template <int K, int CB, int NB, int MODE, bool FULL>
__device__ __forceinline__ void qmv_row(const uint32_t* __restrict__ row_words, const LaneGeom<K>& geom, int lo, int hi,
                                        const uint32_t (&bx)[NB][4], float (&acc)[8][NB][4]) {
#pragma unroll
    for (int quad = 0; quad < 2; ++quad) {
        if (FULL || (lo < 4 * quad + 4 && hi > 4 * quad)) {
            const uint4* qw = reinterpret_cast<const uint4*>(row_words + quad * (32 * K));
            const uint4 W2 = qw[geom.i2];
            const uint4 W1 = qw[geom.i1];
            uint4 W0 = make_uint4(0, 0, 0, 0);
            if constexpr (K >= 5) W0 = qw[geom.i0];
            const uint32_t w2[4] = {W2.x, W2.y, W2.z, W2.w}, w1[4] = {W1.x, W1.y, W1.z, W1.w},
                           w0[4] = {W0.x, W0.y, W0.z, W0.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (FULL || (quad * 4 + j >= lo && quad * 4 + j < hi))
                    tile_mma<K, CB, NB, MODE>(w2[j], w1[j], w0[j], geom.slack, bx, acc[quad * 4 + j]);
        }
    }
}

template <int K, int CB, int NB, int MODE>
__global__ void __launch_bounds__(kQmvWarps * 32)
qmv_kernel(const QmvArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = kQmvWarps;
    constexpr int DEPTH = qmv_depth(K);
    constexpr int kRowWords = 64 * K;                       // 2 quads x 8K words x 4 tiles
    constexpr int kRingBytes = WARPS * DEPTH * kRowWords * 4;
    constexpr uint32_t kRowBytes = kRowWords * 4;
    __shared__ int s_last;
    __shared__ __align__(8) uint64_t s_bar[WARPS][DEPTH];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int rows = p.rows;
    const int G = static_cast<int>(gridDim.x);
    const int bid = static_cast<int>(blockIdx.x);

    // All tiles of the layer in column-block-major order; unit = block * UB + (tk * 8 + tile-in-row).
    // CTA i owns units [T*i/G, T*(i+1)/G): the same number of tiles (+-1) for every CTA, so the
    // grid is one balanced wave whatever the shape.  A CTA may touch several column blocks, and a
    // block may be shared by several CTAs ("pieces").
    const int64_t UB = static_cast<int64_t>(p.tiles_k) * 8;
    const int64_t T = UB * (p.out >> 7);
    const int64_t my0 = T * bid / G, my1 = T * (bid + 1) / G;

    uint32_t* ring = reinterpret_cast<uint32_t*>(smem_raw) + static_cast<size_t>(warp) * DEPTH * kRowWords;
    __half* xs = reinterpret_cast<__half*>(smem_raw + kRingBytes);     // [rows][xs_stride]
    float* red = reinterpret_cast<float*>(smem_raw);                    // reused after the main loop
    uint64_t* bars = s_bar[warp];
    const size_t row_stride = static_cast<size_t>(p.tiles_n) * (32 * K);
    const LaneGeom<K> geom(lane);
    const int64_t tile_floats = static_cast<int64_t>(rows) * 128;

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) mbar_init(bars + i, 1);
        mbar_init_fence();
    }
    __syncwarp();
    int slot = 0;
    uint32_t parity = 0;
    bool copy_lost = false;
    bool first_block = true;

    for (int64_t cblock = my0 / UB; cblock * UB < my1; ++cblock) {
        // ---- this CTA's slice [cta_u0, cta_u1) of the block, then this warp's slice -----------------
        const int cta_u0 = static_cast<int>(max(my0, cblock * UB) - cblock * UB);
        const int cta_u1 = static_cast<int>(min(my1, (cblock + 1) * UB) - cblock * UB);
        const int cta_n = cta_u1 - cta_u0;
        const int u0 = cta_u0 + static_cast<int>(static_cast<int64_t>(cta_n) * warp / WARPS);
        const int u1 = cta_u0 + static_cast<int>(static_cast<int64_t>(cta_n) * (warp + 1) / WARPS);
        const int tk_first = u0 >> 3;
        const int nrows = u1 > u0 ? ((u1 - 1) >> 3) - tk_first + 1 : 0;
        const int tn0 = static_cast<int>(cblock) * 8;
        // CTA holding unit x: ceil((x+1)*G/T) - 1
        const int i_first = static_cast<int>(((cblock * UB + 1) * G - 1) / T);
        const int i_last = static_cast<int>((((cblock + 1) * UB) * G - 1) / T);
        const int pieces = i_last - i_first + 1;

        // ---- phase 0: start streaming weights (they do not depend on the previous kernel) ------------
        // Whole 8-tile rows are copied even when the warp owns only part of the first or last one:
        // one TMA copy per row, consecutive rows a fixed stride apart.
        const char* next_src =
            reinterpret_cast<const char*>(p.wq + (static_cast<int64_t>(tk_first) * p.tiles_n + tn0) * (8 * K));
        if (lane == 0) {
            // the slots may hold reduction scratch written through the generic proxy by the previous block
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
            for (int i = 0; i < DEPTH; ++i)
                if (i < nrows) {
                    const int sl = slot + i < DEPTH ? slot + i : slot + i - DEPTH;
                    mbar_expect_tx(bars + sl, kRowBytes);
                    bulk_copy_g2s(ring + sl * kRowWords, next_src + i * row_stride, kRowBytes, bars + sl);
                }
        }
        next_src += DEPTH * row_stride;
        if (first_block) {
            if (p.pdl_early) pdl_launch_dependents();
            pdl_wait();
            first_block = false;
        }

        // ---- phase 1: rotate (or fetch) the activations of this slice's input range into shared memory
        const int kb0 = (cta_u0 >> 3) >> 3;                              // first 128-block
        const int kb1 = (((cta_u1 - 1) >> 3) >> 3) + 1;                  // one past the last
        {
            const int nblk = kb1 - kb0;
            for (int unit = warp; unit < rows * nblk; unit += WARPS) {
                const int row = unit / nblk, blk = unit % nblk;
                const int col = (kb0 + blk) * 128 + lane * 4;
                __align__(8) __half h[4];
                if (p.xhat) {
                    *reinterpret_cast<uint2*>(h) = *reinterpret_cast<const uint2*>(p.xhat + static_cast<int64_t>(row) * p.in + col);
                } else {
                    __align__(8) __half sc[4];
                    *reinterpret_cast<uint2*>(sc) = *reinterpret_cast<const uint2*>(p.suh + col);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        h[j] = __hmul_rn(load_as_half(p.x, p.x_dtype, static_cast<int64_t>(row) * p.in + col + j), sc[j]);
                    warp_hadamard128_f16(h, lane);
                }
                *reinterpret_cast<uint2*>(xs + row * p.xs_stride + blk * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
            }
        }
        __syncthreads();

        // ---- phase 2: decode x activations ----------------------------------------------------------------
        float acc[8][NB][4];
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[t][nb][i] = 0.0f;

        // activation fragments of input tile tk: rows nb*8+g, inputs 16tk + {2q, 2q+1, 2q+8, 2q+9}
        const uint32_t* xfrag[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int row = min(nb * 8 + g, rows - 1);
            xfrag[nb] = reinterpret_cast<const uint32_t*>(xs + row * p.xs_stride + (tk_first * 16 - kb0 * 128)) + q;
        }
        const int lo_first = u0 & 7, hi_last = nrows > 0 ? ((u1 - 1) & 7) + 1 : 8;
        for (int r = 0; r < nrows; ++r) {
            uint32_t bx[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                uint32_t p0 = xfrag[nb][r * 8], p1 = xfrag[nb][r * 8 + 4];
                if (nb * 8 + g >= rows) { p0 = 0; p1 = 0; }
                if constexpr (MODE == 0) {
                    bx[nb][0] = prmt(p0, p0, 0x1010); bx[nb][1] = prmt(p0, p0, 0x3232);
                    bx[nb][2] = prmt(p1, p1, 0x1010); bx[nb][3] = prmt(p1, p1, 0x3232);
                } else {
                    bx[nb][0] = p0; bx[nb][1] = p1; bx[nb][2] = 0; bx[nb][3] = 0;
                }
            }
            if (!mbar_wait(bars + slot, parity)) copy_lost = true;
            const uint32_t* row_words = ring + slot * kRowWords;
            const int lo = r == 0 ? lo_first : 0, hi = r == nrows - 1 ? hi_last : 8;
            if (lo == 0 && hi == 8) qmv_row<K, CB, NB, MODE, true>(row_words, geom, 0, 8, bx, acc);
            else qmv_row<K, CB, NB, MODE, false>(row_words, geom, lo, hi, bx, acc);
            __syncwarp();                                       // every lane has read the slot
            if (lane == 0 && r + DEPTH < nrows) {
                mbar_expect_tx(bars + slot, kRowBytes);
                bulk_copy_g2s(ring + slot * kRowWords, next_src, kRowBytes, bars + slot);
            }
            next_src += row_stride;
            if (++slot == DEPTH) { slot = 0; parity ^= 1u; }
        }
        if (!p.pdl_early && (cblock + 1) * UB >= my1) pdl_launch_dependents();

        // ---- phase 3: deterministic tree reduction over the warps -------------------------------------------
        __syncthreads();                                        // ring and activations are dead from here on
        auto frag_store = [&](float* base) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = nb * 8 + 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                        if (row < rows) base[row * kQmvRedStride + col] = acc[t][nb][i];
                    }
        };
        auto frag_add = [&](const float* base) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = nb * 8 + 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                        if (row < rows) acc[t][nb][i] = __fadd_rn(acc[t][nb][i], base[row * kQmvRedStride + col]);
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

        // ---- phase 4: pieces of a block held by different CTAs; the last to arrive finishes the block ----
        bool finish = true;
        const float* piece_base = p.partials + cblock * p.max_pieces * tile_floats;
        if (pieces > 1) {
            float* dst = p.partials + (cblock * p.max_pieces + (bid - i_first)) * tile_floats;
            for (int i = threadIdx.x; i < rows * 128; i += WARPS * 32)
                __stcg(dst + i, red[(i >> 7) * kQmvRedStride + (i & 127)]);
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int prev = atomicAdd(p.counters + cblock, 1u);
                s_last = prev == static_cast<unsigned int>(pieces - 1);
            }
            __syncthreads();
            finish = s_last != 0;
            if (finish) {
                __threadfence();
                if (threadIdx.x == 0) p.counters[cblock] = 0;   // leave the scratch ready for the next call
            }
        }
        if (finish) {
            // one warp per activation row: sum the pieces in order, rotate, scale, store
            for (int row = warp; row < rows; row += WARPS) {
                float v[4];
                if (pieces > 1) {
                    const float* src = piece_base + row * 128 + lane * 4;
                    float4 a = __ldcg(reinterpret_cast<const float4*>(src));
                    for (int s0 = 1; s0 < pieces; s0 += 8) {
                        float4 part[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (s0 + j < pieces) part[j] = __ldcg(reinterpret_cast<const float4*>(src + (s0 + j) * tile_floats));
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (s0 + j < pieces) {
                                a.x = __fadd_rn(a.x, part[j].x); a.y = __fadd_rn(a.y, part[j].y);
                                a.z = __fadd_rn(a.z, part[j].z); a.w = __fadd_rn(a.w, part[j].w);
                            }
                    }
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = red[row * kQmvRedStride + lane * 4 + j];
                }
                const int col = static_cast<int>(cblock) * 128 + lane * 4;
                if (p.y == nullptr) {
                    *reinterpret_cast<float4*>(p.yhat + static_cast<int64_t>(row) * p.out + col) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                    __half h[4] = {__float2half_rn(v[0]), __float2half_rn(v[1]), __float2half_rn(v[2]), __float2half_rn(v[3])};
                    warp_hadamard128_f16(h, lane);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        store_from_half(p.y, p.y_dtype, static_cast<int64_t>(row) * p.out + col + j,
                                        __hmul_rn(h[j], p.svh[col + j]), p.bias, col + j);
                }
            }
        }
        __syncthreads();                                        // shared memory is reused by the next block
    }
    if (copy_lost && lane == 0) atomicExch(p.error, 1u);
}

template <int K, int CB, int NB, int MODE>
cudaError_t qmv_launch_one(const QmvArgs& p, const QmvPlan& plan, cudaStream_t stream) {
    auto kernel = qmv_kernel<K, CB, NB, MODE>;
    static bool attribute_set = false;                      // once per kernel: allow the largest carve-out
    if (!attribute_set) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQmvMaxSmemBytes);
        if (e != cudaSuccess) return e;
        attribute_set = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
    cfg.blockDim = dim3(kQmvWarps * 32);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = plan.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

template <int K, int CB, int MODE>
cudaError_t qmv_launch_nb(const QmvArgs& p, const QmvPlan& plan, cudaStream_t stream) {
    if (p.rows <= 8) return qmv_launch_one<K, CB, 1, MODE>(p, plan, stream);
    if (p.rows <= 16) return qmv_launch_one<K, CB, 2, MODE>(p, plan, stream);
    return qmv_launch_one<K, CB, 4, MODE>(p, plan, stream);
}

template <int K>
cudaError_t qmv_launch_k(const QmvArgs& p, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (cb == 2) return qmv_launch_nb<K, 2, 1>(p, plan, stream);
    if (cb == 0) return exact ? qmv_launch_nb<K, 0, 1>(p, plan, stream) : qmv_launch_nb<K, 0, 0>(p, plan, stream);
    return exact ? qmv_launch_nb<K, 1, 1>(p, plan, stream) : qmv_launch_nb<K, 1, 0>(p, plan, stream);
}

}  // namespace b200exl3
