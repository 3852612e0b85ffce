// Fused EXL3 linear layer for up to 16 activation rows (QMV and small-batch QMM) in ONE launch:
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
//  * packed words are staged by the TMA unit (one cp.async.bulk per row of 8 tiles) into a per-warp ring in
//    shared memory, issued before anything that depends on the activations;
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
//  * every warp is an independent worker: all tiles of the layer are ordered column-block-major and
//    split evenly over all warps of the grid (balanced to one tile for any shape, one wave).  A warp
//    rotates the activations of its own input range into shared memory, accumulates its tiles, and
//    writes its partial [rows, 128] tile; the last warp to arrive at a column block (arrival counter)
//    sums the partials in a fixed order and applies the output rotation.  No CTA-wide barrier exists.
//    With more than two activation rows the rotation is done once by a separate kernel instead.
//
// Included by one small translation unit per K so the eight K values compile in parallel.
#pragma once

#include "hadamard.cuh"
#include "tile_decode.cuh"
#include "kernels.h"

// The operators fused around a layer are compiled into instantiations of their own (kFused): 0 = none, 1 = those of
// a dense decoder (prologues 1..3, epilogues 1..2), 2 = all (the expert block's prologue 4 and epilogue 3 too).  With all
// of that code in it the plain kernel spilled 56 bytes and a 4096 -> 14336 layer took 22.4 instead of 21.2 us; the dense
// set alone does not spill, the expert set does (32..64 bytes).
#define QMV_PRO(p) ((kFused == 2 || (kFused == 1 && (p).prologue <= 3)) ? (p).prologue : 0)
#define QMV_EPI(p) ((kFused == 2 || (kFused == 1 && (p).epilogue <= 2)) ? (p).epilogue : 0)

namespace b200exl3 {

// One tile: decode the lane's eight weights and issue the MMAs against the activation fragments.
// MODE 0: codebook 0/1, split halves (2 MMAs per 8 rows).  MODE 1: exact fp16 weights (1 MMA per 8 rows).
template <int K, int CB, int NB, int MODE>
__device__ __forceinline__ void tile_mma(uint32_t w2, uint32_t w1, uint32_t w0, int slack, const uint32_t (&bx)[NB][4],
                                         float (&acc)[NB][4]) {
    if constexpr (MODE == 0) {
        uint32_t b[8], a[8];
        lane_hashes<K, CB>(w2, w1, w0, slack, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = lop3_and_xor(b[j], 0x8fff8fffu, 0x3b603b60u);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            mma_16816(acc[nb], a[0], a[4], a[1], a[5], bx[nb][0], bx[nb][1]);
            mma_16816(acc[nb], a[2], a[6], a[3], a[7], bx[nb][2], bx[nb][3]);
        }
    } else {
        uint32_t a0, a1, a2, a3;
        lane_weights_exact<K, CB>(w2, w1, w0, slack, a0, a1, a2, a3);
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

// group (fused projection) that owns 128-column block `cblock`
__device__ __forceinline__ int qmv_group_of(const QmvArgs& p, int cblock) {
    int grp = 0;
#pragma unroll 1
    while (grp + 1 < p.groups && cblock * 128 >= p.gcol0[grp + 1]) ++grp;
    return grp;
}

// ---- the rarely executed parts of the kernel: written small (no unrolling) so that they cost the
//      decode loop neither registers nor instruction-cache space -----------------------------------------

// Rotates the activations of input 128-blocks [kb0, kb0 + nblk) of every row into the warp's shared
// memory: xs[row][blk][128] = H128(half(half(x) * suh)).  The loads of the next block are issued before
// the butterflies of the current one.
__device__ __forceinline__ void qmv_rotate_chunk(const void* x, int x_dtype, const __half* suh, int in, int rows, int kb0,
                                                 int nblk, __half* xs, int lane) {
    constexpr int kXsHalves = kQmvXBlocks * 128;
    const int total = rows * nblk;
    auto fetch = [&](int unit, uint2& sv, __half (&xv)[4]) {
        const int row = unit / nblk, blk = unit - row * nblk;
        const int col = (kb0 + blk) * 128 + lane * 4;
        sv = *reinterpret_cast<const uint2*>(suh + col);
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[j] = load_as_half(x, x_dtype, static_cast<int64_t>(row) * in + col + j);
    };
    uint2 sv_next;
    __half xv_next[4];
    fetch(0, sv_next, xv_next);
#pragma unroll 1
    for (int unit = 0; unit < total; ++unit) {
        const uint2 sv = sv_next;
        __align__(8) __half h[4];
        const __half* sc = reinterpret_cast<const __half*>(&sv);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(xv_next[j], sc[j]);
        if (unit + 1 < total) fetch(unit + 1, sv_next, xv_next);
        warp_hadamard128_f16(h, lane);
        const int row = unit / nblk, blk = unit - row * nblk;
        *reinterpret_cast<uint2*>(xs + row * kXsHalves + blk * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
    }
    __syncwarp();
}

// Prologue 4: the SwiGLU glue of the expert block (native/src/moe.rs:438-533; SiLU path, both rotations without
// intermediate rounding) from the raw gate and up products of slot `slot`, for input blocks [kb0, kb0 + nblk) of the down
// product, into the warp's shared memory.  The arithmetic of glu_down_input_kernel, statement by statement.
__device__ __forceinline__ void qmv_rotate_chunk_glu(const QmvArgs& p, int64_t slot, int64_t expert, int kb0, int nblk, __half* xs, int lane) {
    const int hidden = p.in;
    const float scale = had_scale();
#pragma unroll 1
    for (int b = 0; b < nblk; ++b) {
        const int col = (kb0 + b) * 128 + lane * 4;
        const float4 graw = __ldcg(reinterpret_cast<const float4*>(p.pro_ygu + (slot * 2) * hidden + col));
        const float4 uraw = __ldcg(reinterpret_cast<const float4*>(p.pro_ygu + (slot * 2 + 1) * hidden + col));
        float gv[4] = {round_half(graw.x), round_half(graw.y), round_half(graw.z), round_half(graw.w)};
        float uv[4] = {round_half(uraw.x), round_half(uraw.y), round_half(uraw.z), round_half(uraw.w)};
        warp_hadamard128<false, false>(gv, lane);
        warp_hadamard128<false, false>(uv, lane);
        const __half* sg = p.pro_gu_svh + (expert * 2) * hidden + col;
        const __half* su = p.pro_gu_svh + (expert * 2 + 1) * hidden + col;
        const __half* sd = p.suh + expert * hidden + col;
        float d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gate = round_half(__fmul_rn(__fmul_rn(gv[j], scale), __half2float(sg[j])));
            const float up = round_half(__fmul_rn(__fmul_rn(uv[j], scale), __half2float(su[j])));
            float act = round_half(__fmul_rn(glu_silu(gate), up));
            if (col + j >= p.pro_logical) act = 0.0f;
            d[j] = round_half(__fmul_rn(act, __half2float(sd[j])));
        }
        warp_hadamard128<false, false>(d, lane);
        __align__(8) __half h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __float2half_rn(__fmul_rn(d[j], scale));
        *reinterpret_cast<uint2*>(xs + b * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
    }
    __syncwarp();
}

// 1 / rms of every row of x (+ residual), for the fused RMSNorm prologue: every warp adds the whole row in the same
// fixed order (lane partial sums over 8-element groups, then a shuffle tree), so all warps of the grid get the same bits.
__device__ __forceinline__ void qmv_row_inv_rms(const __half* x, const __half* residual, int in, int rows, float eps, int lane,
                                                float (&inv)[kQmvFusedRows]) {
#pragma unroll
    for (int row = 0; row < kQmvFusedRows; ++row) {
        inv[row] = 0.0f;
        if (row < rows) {
            float acc = 0.0f;
            for (int i = lane * 8; i < in; i += 256) {
                const uint4 xv = __ldcg(reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * in + i));
                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                uint4 rv = make_uint4(0, 0, 0, 0);
                if (residual != nullptr) rv = __ldcg(reinterpret_cast<const uint4*>(residual + static_cast<int64_t>(row) * in + i));
                const __half2* rh = reinterpret_cast<const __half2*>(&rv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(residual != nullptr ? __hadd2_rn(xh[j], rh[j]) : xh[j]);
                    acc = fmaf(f.x, f.x, acc);
                    acc = fmaf(f.y, f.y, acc);
                }
            }
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
            inv[row] = rsqrtf(acc / static_cast<float>(in) + eps);
        }
    }
}

// qmv_rotate_chunk with a fused prologue in front of the input scales: RMSNorm (after an optional residual add) or SwiGLU.
template <int kFused>
__device__ __forceinline__ void qmv_rotate_chunk_fused(const QmvArgs& p, const __half* suh, const float (&inv)[kQmvFusedRows], int rows, int kb0,
                                                       int nblk, bool store_sum, __half* xs, int lane) {
    constexpr int kXsHalves = kQmvXBlocks * 128;
    const __half* x = reinterpret_cast<const __half*>(p.x);
#pragma unroll 1
    for (int row = 0; row < rows; ++row) {
#pragma unroll 1
        for (int blk = 0; blk < nblk; ++blk) {
            const int col = (kb0 + blk) * 128 + lane * 4;
            const int64_t at = static_cast<int64_t>(row) * p.in + col;
            const uint2 xv = __ldcg(reinterpret_cast<const uint2*>(x + at));
            const uint2 sv = *reinterpret_cast<const uint2*>(suh + col);
            const __half2* xh = reinterpret_cast<const __half2*>(&xv);
            __align__(8) __half2 v[2];
            if (QMV_PRO(p) == 1 || QMV_PRO(p) == 3) {
                const uint2 wv = *reinterpret_cast<const uint2*>(p.pro_weight + col);
                const __half2* wh = reinterpret_cast<const __half2*>(&wv);
                __half2 s0 = xh[0], s1 = xh[1];
                if (QMV_PRO(p) == 1 && p.pro_aux != nullptr) {
                    const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(p.pro_aux + at));
                    const __half2* rh = reinterpret_cast<const __half2*>(&rv);
                    s0 = __hadd2_rn(s0, rh[0]);
                    s1 = __hadd2_rn(s1, rh[1]);
                }
                if (QMV_PRO(p) == 1 && store_sum && p.pro_sum != nullptr) {
                    __align__(8) __half2 keep[2] = {s0, s1};
                    *reinterpret_cast<uint2*>(p.pro_sum + at) = *reinterpret_cast<const uint2*>(keep);
                }
                const float2 f0 = __half22float2(s0), f1 = __half22float2(s1);
                v[0] = __hmul2_rn(wh[0], __floats2half2_rn(f0.x * inv[row], f0.y * inv[row]));
                v[1] = __hmul2_rn(wh[1], __floats2half2_rn(f1.x * inv[row], f1.y * inv[row]));
            } else {
                const uint2 uv = __ldcg(reinterpret_cast<const uint2*>(p.pro_aux + at));
                const __half2* uh = reinterpret_cast<const __half2*>(&uv);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float2 f = __half22float2(xh[j]);
                    const __half2 sg = __floats2half2_rn(1.0f / (1.0f + expf(-f.x)), 1.0f / (1.0f + expf(-f.y)));
                    v[j] = __hmul2_rn(__hmul2_rn(xh[j], sg), uh[j]);
                }
            }
            const __half2* sh = reinterpret_cast<const __half2*>(&sv);
            __align__(8) __half h[4];
            *reinterpret_cast<__half2*>(h) = __hmul2_rn(v[0], sh[0]);
            *reinterpret_cast<__half2*>(h + 2) = __hmul2_rn(v[1], sh[1]);
            warp_hadamard128_f16(h, lane);
            *reinterpret_cast<uint2*>(xs + row * kXsHalves + blk * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
        }
    }
    __syncwarp();
}

// The last warp of a CTA to stage its tile of column block `cblock`: adds the tiles of the warps that
// had work in the block (warp_mask) in warp order; if other CTAs share the block, publishes the
// sum as this CTA's piece and counts arrivals; the last CTA adds the pieces in piece order.  Whoever
// holds the complete sum applies the output rotation (or stores the raw sum).
template <int kFused>
__device__ __forceinline__ void qmv_finish_block(const QmvArgs& p, int cblock, unsigned int warp_mask, unsigned int second_mask,
                                              int pieces, int piece, const unsigned char* smem_base, int lane) {
    const int rows = p.rows;
    const int tile_floats = rows * 128;
    const float* piece_base = p.partials + static_cast<int64_t>(cblock) * p.max_pieces * tile_floats;
    float* piece_dst = p.partials + (static_cast<int64_t>(cblock) * p.max_pieces + piece) * tile_floats;
    const int stage_floats = rows * kQmvRedStride;
#pragma unroll 1
    for (int pass = 0; pass < (pieces > 1 ? 2 : 1); ++pass) {
        if (pass == 1) {
            __threadfence();
            __syncwarp();
            unsigned int prev = 0;
            if (lane == 0) prev = atomicAdd(p.counters + cblock, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev != static_cast<unsigned int>(pieces - 1)) return;       // not the last CTA of this block
            __threadfence();
            if (lane == 0) p.counters[cblock] = 0;              // leave the scratch ready for the next call
        }
        const bool complete = pass == 1 || pieces == 1;
#pragma unroll 1
        for (int row = 0; row < rows; ++row) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            if (pass == 0) {
                bool any = false;
#pragma unroll 1
                for (int w = 0; w < kQmvWarps; ++w) {
                    if (!((warp_mask >> w) & 1u)) continue;
                    // a warp stages the tile of its first block in buffer 0 and of its second block in buffer 1
                    const float4 t4 = *reinterpret_cast<const float4*>(
                        reinterpret_cast<const float*>(smem_base + static_cast<size_t>(w) * p.warp_smem + p.stage_offset) +
                        ((second_mask >> w) & 1u) * stage_floats + row * kQmvRedStride + lane * 4);
                    if (!any) { a = t4; any = true; }
                    else { a.x = __fadd_rn(a.x, t4.x); a.y = __fadd_rn(a.y, t4.y); a.z = __fadd_rn(a.z, t4.z); a.w = __fadd_rn(a.w, t4.w); }
                }
            } else {
                const float* src = piece_base + row * 128 + lane * 4;
                a = __ldcg(reinterpret_cast<const float4*>(src));
#pragma unroll 1
                for (int s0 = 1; s0 < pieces; s0 += 4) {         // loads of four pieces go out together
                    float4 part[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (s0 + j < pieces) part[j] = __ldcg(reinterpret_cast<const float4*>(src + (s0 + j) * tile_floats));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (s0 + j < pieces) {
                            a.x = __fadd_rn(a.x, part[j].x); a.y = __fadd_rn(a.y, part[j].y);
                            a.z = __fadd_rn(a.z, part[j].z); a.w = __fadd_rn(a.w, part[j].w);
                        }
                }
            }
            if (!complete) {
                __stcg(reinterpret_cast<float4*>(piece_dst + row * 128 + lane * 4), a);
                continue;
            }
            const int col = cblock * 128 + lane * 4;              // column in the concatenated output space
            if (p.yhat != nullptr && QMV_EPI(p) == 3) {
                // Expert-mapped down product, one row per slot: virtual block = (slot, block j of the expert's columns).
                // The block is rotated, scaled by the expert's output scales and the slot's routing weight and parked in
                // yhat; the last of a token's top_k slots to arrive adds them in slot order (the arithmetic and the order
                // of finish_and_reduce_kernel, so the same bits).
                const int slot = cblock / p.map_blocks, j = cblock - slot * p.map_blocks;
                const int width = p.map_blocks << 7, top_k = p.map_top_k;
                const int64_t expert = static_cast<int64_t>(min(p.map_selected[slot], static_cast<uint32_t>(p.map_experts - 1)));
                __half h[4] = {__float2half_rn(a.x), __float2half_rn(a.y), __float2half_rn(a.z), __float2half_rn(a.w)};
                warp_hadamard128_f16(h, lane);
                const uint2 svw = *reinterpret_cast<const uint2*>(p.svh + expert * width + j * 128 + lane * 4);
                const __half* sv = reinterpret_cast<const __half*>(&svw);
                float v[4];
                if (p.epi_score_f32) {
                    const float score = reinterpret_cast<const float*>(p.epi_scores)[slot];
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = __fmul_rn(__half2float(__hmul_rn(h[e], sv[e])), score);
                } else {
                    const __half score = reinterpret_cast<const __half*>(p.epi_scores)[slot];
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = __half2float(__hmul_rn(__hmul_rn(h[e], sv[e]), score));
                }
                __stcg(reinterpret_cast<float4*>(p.yhat + col), make_float4(v[0], v[1], v[2], v[3]));
                __threadfence();                                // the parked block before the arrival
                __syncwarp();
                const int token = slot / top_k;
                unsigned int* arrived = p.counters + p.epi_counter0 + token * p.map_blocks + j;
                unsigned int before = 0;
                if (lane == 0) before = atomicAdd(arrived, 1u);
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before != static_cast<unsigned int>(top_k - 1)) continue;
                __threadfence();
                if (lane == 0) *arrived = 0;                    // leave the scratch ready for the next call
                const float* parked = p.yhat + (static_cast<int64_t>(token) * top_k * p.map_blocks + j) * 128 + lane * 4;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                for (int t0 = 0; t0 < top_k; t0 += 4) {         // four loads in flight, added in slot order
                    float4 r[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (t0 + i < top_k) r[i] = __ldcg(reinterpret_cast<const float4*>(parked + static_cast<int64_t>(t0 + i) * width));
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (t0 + i >= top_k) continue;
                        const float f[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (t0 + i == 0) acc[e] = f[e];
                            else if (p.epi_score_f32) acc[e] = __fadd_rn(acc[e], f[e]);
                            else acc[e] = __half2float(__hadd_rn(__float2half_rn(acc[e]), __float2half_rn(f[e])));
                        }
                    }
                }
                const int64_t at = static_cast<int64_t>(token) * width + j * 128 + lane * 4;
                if (p.epi_score_f32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.gy[0]) + at) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                } else {
                    __align__(8) __half o16[4] = {__float2half_rn(acc[0]), __float2half_rn(acc[1]), __float2half_rn(acc[2]), __float2half_rn(acc[3])};
                    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.gy[0]) + at) = *reinterpret_cast<const uint2*>(o16);
                }
            } else if (p.yhat != nullptr) {
                *reinterpret_cast<float4*>(p.yhat + static_cast<int64_t>(row) * p.out + col) = a;
            } else {
                // a row shard of a tensor-parallel layer first adds the other ranks' sums for this block
                if (p.tp.world > 0) a = tp_exchange_unit(p.tp, (p.tp_row0 + row) * (p.out >> 7) + cblock, a, lane);
                __half h[4] = {__float2half_rn(a.x), __float2half_rn(a.y), __float2half_rn(a.z), __float2half_rn(a.w)};
                warp_hadamard128_f16(h, lane);
                __align__(8) __half sv[4];
                *reinterpret_cast<uint2*>(sv) = *reinterpret_cast<const uint2*>(p.svh + col);
                if (QMV_EPI(p) == 1) {
                    // residual add and the block's sum of squares for the next RMSNorm (fixed shuffle order)
                    const int64_t at = static_cast<int64_t>(row) * p.out + col;
                    const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(p.epi_residual + at));
                    const __half* rh = reinterpret_cast<const __half*>(&rv);
                    __align__(8) __half sum[4];
                    float sq = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __half y = __hmul_rn(h[j], sv[j]);
                        if (p.bias) y = __hadd_rn(y, p.bias[col + j]);
                        sum[j] = __hadd_rn(rh[j], y);
                        const float f = __half2float(sum[j]);
                        sq = fmaf(f, f, sq);
                    }
                    *reinterpret_cast<uint2*>(p.epi_sum + at) = *reinterpret_cast<const uint2*>(sum);
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
                    if (lane == 0) p.epi_sumsq[row * (p.out >> 7) + cblock] = sq;
                    continue;
                }
                const int grp = qmv_group_of(p, cblock);
                const int gcol = col - p.gcol0[grp];
                if (QMV_EPI(p) == 2) {
                    // [q | k | v] with 128-wide heads: this block is one head.  Rotary embedding of q and k heads (pairs
                    // (i, i + 64): lane L holds columns 4L..4L+3, its partner is lane L ^ 16), keys and values go
                    // straight into row `pos` of the caches.
                    int pos = __ldg(p.epi_pos);
                    pos = pos < 0 ? 0 : (pos >= p.epi_max_ctx ? p.epi_max_ctx - 1 : pos);
                    __align__(8) __half y[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        y[j] = __hmul_rn(h[j], sv[j]);
                        if (p.bias) y[j] = __hadd_rn(y[j], p.bias[col + j]);
                    }
                    if (grp < 2) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float mine = __half2float(y[j]);
                            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                            const int i = (lane & 15) * 4 + j;
                            const float inv_freq = exp2f(-p.epi_log2_theta * static_cast<float>(2 * i) / 128.0f);
                            float sn, cs;
                            sincosf(static_cast<float>(pos) * inv_freq, &sn, &cs);
                            const float a0 = lane < 16 ? mine : other, b0 = lane < 16 ? other : mine;
                            y[j] = __float2half_rn(lane < 16 ? a0 * cs - b0 * sn : a0 * sn + b0 * cs);
                        }
                    }
                    __half* dst = grp == 0 ? reinterpret_cast<__half*>(p.gy[0]) + gcol
                                           : (grp == 1 ? p.epi_k_cache : p.epi_v_cache) +
                                                 (static_cast<int64_t>(gcol >> 7) * p.epi_max_ctx + pos) * 128 + lane * 4;
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(y);
                    continue;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    store_from_half(p.gy[grp], p.y_dtype, static_cast<int64_t>(row) * p.gout[grp] + gcol + j,
                                    __hmul_rn(h[j], sv[j]), p.bias ? p.bias + (col - gcol) : nullptr, gcol + j);
            }
        }
    }
}

template <int K, int CB, int NB, int MODE, int kFused>
__global__ void __launch_bounds__(kQmvWarps * 32, NB == 1 ? 2 : 1)
qmv_kernel(const QmvArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = kQmvWarps;
    constexpr int R = qmv_chunk_rows(K);                    // rows per bulk copy (the rows of a column block are contiguous)
    constexpr int SLOTS = qmv_slots(K);                     // chunks in flight per warp
    constexpr int kRowWords = 64 * K;                       // 2 quads x 8K words x 4 tiles
    constexpr uint32_t kRowBytes = kRowWords * 4;
    constexpr int kXsHalves = kQmvXBlocks * 128;            // rotated activations kept per row and warp
    __shared__ __align__(8) uint64_t s_bar[WARPS][SLOTS];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int rows = p.rows;

    // All tiles of the layer are ordered column-block-major (unit = block * UB + tk * 8 + tile-in-row) and dealt out to
    // the W warps of the grid in whole rows of 8 tiles, so that no row is copied by two warps and no row is decoded with
    // a test per tile: warp w owns rows [RT*w/W, RT*(w+1)/W) of the RT rows (the same count +-1 for every warp, whatever
    // the shape) -- or, when that does not raise the largest share, every column block goes to a whole number of warps
    // (block c to warps [c W / C, (c + 1) W / C), which share its rows evenly), so that no warp works on two blocks (such
    // a warp stages, arrives and rotates activations twice; measured in the decode-step kernel: it finishes 1-2 us after
    // the others).  The eight warps of a CTA walk the same list of blocks, add their tiles up in shared memory, and CTAs
    // that share a block ("pieces") meet in global memory.
    // (the layer has fewer than 2^31 tiles; only the products with the warp count need 64 bits)
    const int W = static_cast<int>(gridDim.x) * WARPS;
    const int wid = static_cast<int>(blockIdx.x) * WARPS + warp;
    const int UB = p.tiles_k * 8;
    const int C = p.out >> 7;
    const int T = UB * C;
    const int RB = p.tiles_k, RT = RB * C;
    // a * b / d with a * b below (T + 1) * W: 32-bit when that fits (64-bit division is emulated and slow)
    const bool narrow = static_cast<unsigned long long>(T + 1) * static_cast<unsigned long long>(W) < 0xffffffffull;
    const int per_block = W / C;
    const bool aligned = per_block >= 1 && (RB + per_block - 1) / per_block <= (RT + W - 1) / W &&
                         static_cast<unsigned long long>(W + 1) * static_cast<unsigned long long>(C + 1) < 0xffffffffull;
    auto unit_begin = [=](int w) -> int {                    // first unit (tile) of warp w
        if (w >= W) return T;
        if (aligned) {
            const unsigned int c = ((static_cast<unsigned int>(w) + 1u) * C - 1u) / W;
            const unsigned int first = c * W / C, count = (c + 1u) * W / C - first;
            return 8 * static_cast<int>(c * RB + RB * (w - first) / count);
        }
        return 8 * (narrow ? static_cast<int>(static_cast<unsigned int>(RT) * static_cast<unsigned int>(w) / static_cast<unsigned int>(W))
                           : static_cast<int>(static_cast<unsigned long long>(RT) * w / W));
    };
    const int w0 = unit_begin(wid);
    const int w1 = unit_begin(wid + 1);

    unsigned char* mine = smem_raw + static_cast<size_t>(warp) * p.warp_smem;
    uint32_t* ring = reinterpret_cast<uint32_t*>(mine);                  // SLOTS chunks of R rows of packed words
    __half* xs = reinterpret_cast<__half*>(mine + p.xs_offset);          // [rows][kXsHalves] (fused rotation only)
    const int stage_floats = rows * kQmvRedStride;                       // one staged [rows][128] tile
    uint64_t* bars = s_bar[warp];
    constexpr size_t row_stride = 256 * K;                               // consecutive rows of a column block are contiguous
    const LaneGeom<K> geom(lane);
    const bool tracing = p.trace != nullptr && threadIdx.x == 0;
    if (tracing) p.trace[blockIdx.x * 8 + 0] = global_ns();

    // the unit ranges of the CTA's eight warps, for the block walk and the mask of contributing warps
    __shared__ int s_begin[WARPS + 1];
    __shared__ unsigned int s_arrived[WARPS + 2];            // per visited block: warps that staged their tile
    if (threadIdx.x <= WARPS)
        s_begin[threadIdx.x] = unit_begin(static_cast<int>(blockIdx.x) * WARPS + static_cast<int>(threadIdx.x));
    if (threadIdx.x < WARPS + 2) s_arrived[threadIdx.x] = 0;
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) mbar_init(bars + i, 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // barriers visible to the copy engine
    }
    __syncthreads();
    const int cta0 = s_begin[0];
    // A warp's range is at most one block long (the launch guarantees it), so it touches at most two
    // blocks and owns two staging buffers: nobody ever waits for anybody inside the CTA.
    if (w1 - w0 > UB) {
        if (threadIdx.x == 0) atomicExch(p.error, 2u);
        return;
    }
    int slot = 0;
    uint32_t parity = 0;
    bool copy_lost = false;
    bool first_chunk = true;
    bool have_inv = false;                       // fused RMSNorm prologue: the rows' 1 / rms, computed once per warp
    float inv_rms[kQmvFusedRows] = {};

    for (int cblock = w0 / UB; cblock * UB < w1; ++cblock) {
        // ---- this warp's segment [u0, u1) of the block ----------------------------------------------------
        const int u0 = max(w0, cblock * UB) - cblock * UB;
        const int u1 = min(w1, (cblock + 1) * UB) - cblock * UB;
        float* stage = reinterpret_cast<float*>(mine + p.stage_offset) + (cblock - w0 / UB) * stage_floats;
        int grp = qmv_group_of(p, cblock);
        int tn0 = cblock * 8;                               // first tile column of the block in the weight array
        bool active = true;
        int map_slot = 0, map_expert = 0;                   // expert-mapped: the slot of this block and its expert
        const void* x_rows = p.x;                           // activations and input scales this block's rotation reads
        int64_t suh_row = grp;
        if (p.map_selected != nullptr) {
            // The routes (and the slot count) are written by the previous kernel in the stream: under a programmatic
            // dependent launch they may be read only once that kernel's memory is visible, so this mode gives up
            // the early weight prefetch.
            if (first_chunk) {
                if (p.pdl_early) pdl_launch_dependents();
                pdl_wait();
                first_chunk = false;
            }
            // expert-mapped: virtual block -> (slot, projection, block of the expert's columns)
            const int sp = cblock / p.map_blocks, j = cblock - sp * p.map_blocks;
            const int slot = sp / p.map_proj, proj = sp - slot * p.map_proj;
            // unsigned clamp: an id of 2^31 or more must not turn into a negative index
            const int expert = static_cast<int>(min(p.map_selected[slot], static_cast<uint32_t>(p.map_experts - 1)));
            tn0 = (proj * p.map_stride_blocks + expert * p.map_blocks + j) * 8;
            map_slot = slot; map_expert = expert;
            grp = sp;                                       // rows of the rotated activations (stride: one slot)
            suh_row = static_cast<int64_t>(expert) * p.map_proj + proj;
            if (p.xhat == nullptr)
                x_rows = static_cast<const char*>(p.x) + static_cast<int64_t>(slot / p.map_top_k) * p.in * dtype_size(p.x_dtype);
            // slots past the device-side count hold nothing: no weights are read for them, zeros are reduced
            active = p.map_count == nullptr || slot < *p.map_count;
        }
        {
            const int tk_first = u0 >> 3, tk_last = (u1 - 1) >> 3;

            float acc[8][NB][4];
#pragma unroll
            for (int t = 0; t < 8; ++t)
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[t][nb][i] = 0.0f;

            // ---- phase 0: start streaming weights (they do not depend on the previous kernel) ----------------
            // The rows tk_first..tk_last of the block are contiguous in memory and are copied in chunks of up to R rows
            // (one bulk copy each), counted from tk_first; whole 8-tile rows are copied even when the warp owns only
            // part of the first or last one.
            const char* seg_src = reinterpret_cast<const char*>(p.wq + quad_row_offset(tk_first, tn0 >> 3, p.tiles_k, K));
            int req_tk = tk_first;                              // first row that has not been requested yet
            auto refill = [&](int s) {
                const int n = min(R, tk_last - req_tk + 1);
                if (lane == 0) {
                    mbar_expect_tx(bars + s, n * kRowBytes);
                    bulk_copy_g2s(ring + s * (R * kRowWords), seg_src + static_cast<size_t>(req_tk - tk_first) * row_stride, n * kRowBytes, bars + s);
                }
                req_tk += n;
            };
            if (active) {
#pragma unroll
                for (int i = 0; i < SLOTS; ++i)
                    if (req_tk <= tk_last) refill(slot + i < SLOTS ? slot + i : slot + i - SLOTS);
            }

            // The segment is walked in stretches whose inputs span at most kQmvXBlocks 128-blocks, so that
            // the rotated activations of a stretch fit the warp's shared memory.
            for (int tk0 = tk_first; active && tk0 <= tk_last;) {
                const int kb0 = tk0 >> 3;
                const int tk_end = min(tk_last + 1, (kb0 + kQmvXBlocks) * 8);
                const int nrows = tk_end - tk0;

                if (first_chunk) {
                    if (p.pdl_early) pdl_launch_dependents();
                    pdl_wait();
                    first_chunk = false;
                    if (tracing) p.trace[blockIdx.x * 8 + 1] = global_ns();
                }

                // ---- phase 1: rotate this chunk's activations into the warp's shared memory ------------
                if (p.xhat == nullptr) {
                    if (QMV_PRO(p) == 4) {
                        qmv_rotate_chunk_glu(p, map_slot, map_expert, kb0, ((tk_end - 1) >> 3) - kb0 + 1, xs, lane);
                    } else if (QMV_PRO(p) != 0) {
                        if (!have_inv && QMV_PRO(p) == 1) {
                            qmv_row_inv_rms(reinterpret_cast<const __half*>(p.x), p.pro_aux, p.in, rows, p.pro_eps, lane, inv_rms);
                            have_inv = true;
                        }
                        if (!have_inv && QMV_PRO(p) == 3) {
                            // the layer before left the sum of squares of every 128-block: add them in a fixed order
#pragma unroll
                            for (int row = 0; row < kQmvFusedRows; ++row)
                                if (row < rows) {
                                    float acc = 0.0f;
                                    for (int b = lane; b < (p.in >> 7); b += 32) acc += __ldcg(p.pro_sumsq + row * (p.in >> 7) + b);
#pragma unroll
                                    for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
                                    inv_rms[row] = rsqrtf(acc / static_cast<float>(p.in) + p.pro_eps);
                                }
                            have_inv = true;
                        }
                        qmv_rotate_chunk_fused<kFused>(p, p.suh + suh_row * p.in, inv_rms, rows, kb0, ((tk_end - 1) >> 3) - kb0 + 1, cblock == 0, xs, lane);
                    } else {
                        qmv_rotate_chunk(x_rows, p.x_dtype, p.suh + suh_row * p.in, p.in, rows, kb0,
                                         ((tk_end - 1) >> 3) - kb0 + 1, xs, lane);
                    }
                }
                if (tracing && tk0 == tk_first) p.trace[blockIdx.x * 8 + 2] = global_ns();

                // ---- phase 2: decode x activations ----------------------------------------------------------
                // activation fragments of input tile tk: rows nb*8+g, inputs 16tk + {2q, 2q+1, 2q+8, 2q+9}
                const uint32_t* xfrag[NB];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int row = min(nb * 8 + g, rows - 1);
                    if (p.xhat == nullptr)
                        xfrag[nb] = reinterpret_cast<const uint32_t*>(xs + row * kXsHalves + (tk0 * 16 - kb0 * 128)) + q;
                    else
                        xfrag[nb] = reinterpret_cast<const uint32_t*>(p.xhat + grp * p.xhat_group_stride + static_cast<int64_t>(row) * p.in + tk0 * 16) + q;
                }
                // The rows of the stretch are walked run by run (a run = the part of one chunk inside the stretch): the
                // barrier wait and the hand-back of the slot happen once per chunk, and the row loop tests nothing per
                // tile (a warp's range is whole rows).  Lanes whose activation row does not exist multiply the last
                // row again: column n of the product depends on column n of the activations only, and is never stored.
                auto fragments = [&](int r, uint32_t (&bx)[NB][4]) {
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const uint32_t p0 = xfrag[nb][r * 8], p1 = xfrag[nb][r * 8 + 4];
                        if constexpr (MODE == 0) {
                            bx[nb][0] = prmt(p0, p0, 0x1010); bx[nb][1] = prmt(p0, p0, 0x3232);
                            bx[nb][2] = prmt(p1, p1, 0x1010); bx[nb][3] = prmt(p1, p1, 0x3232);
                        } else {
                            bx[nb][0] = p0; bx[nb][1] = p1; bx[nb][2] = 0; bx[nb][3] = 0;
                        }
                    }
                };
#pragma unroll 1
                for (int r = 0; r < nrows;) {
                    const int tk = tk0 + r;
                    const int ri = (tk - tk_first) & (R - 1);                   // row inside its chunk
                    const int run = min(R - ri, nrows - r);
                    if (ri == 0 && !copy_lost && !mbar_wait(bars + slot, parity)) copy_lost = true;
                    const uint32_t* row_words = ring + (slot * R + ri) * kRowWords;
#pragma unroll 1
                    for (int j = 0; j < run; ++j) {
                        uint32_t bx[NB][4];
                        fragments(r + j, bx);
                        qmv_row<K, CB, NB, MODE, true>(row_words, geom, 0, 8, bx, acc);
                        row_words += kRowWords;
                    }
                    r += run;
                    if (ri + run == R || tk0 + r > tk_last) {                   // the chunk is consumed: its slot takes the next one
                        __syncwarp();                                           // every lane has read the slot
                        if (req_tk <= tk_last) refill(slot);
                        if (++slot == SLOTS) { slot = 0; parity ^= 1u; }
                    }
                }
                tk0 = tk_end;
            }

            if (first_chunk) {                                  // a warp whose block was skipped has not waited yet
                pdl_wait();
                first_chunk = false;
            }
            // ---- phase 3: stage the fragment as a [rows][128] tile in this warp's shared memory -----------
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = nb * 8 + 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                        if (row < rows) stage[row * kQmvRedStride + col] = acc[t][nb][i];
                    }
        }
        if (!p.pdl_early && (cblock + 1) * UB >= w1) pdl_launch_dependents();
        if (tracing) p.trace[blockIdx.x * 8 + 3] = global_ns();

        // ---- phase 4: the last warp of the CTA to arrive at this block adds the CTA's tiles, meets the
        //      other CTAs of the block, rotates and stores ---------------------------------------------------
        unsigned int mask = 0, second = 0;                      // warps with a tile here; ... as their 2nd block
#pragma unroll 1
        for (int w = 0; w < WARPS; ++w)
            if (min(s_begin[w + 1], (cblock + 1) * UB) > max(s_begin[w], cblock * UB)) {
                mask |= 1u << w;
                if (s_begin[w] / UB != cblock) second |= 1u << w;
            }
        __syncwarp();
        unsigned int prev = 0;
        if (lane == 0) {
            __threadfence_block();                              // the staged tile before the arrival
            prev = atomicAdd(&s_arrived[cblock - cta0 / UB], 1u);
        }
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (tracing) p.trace[blockIdx.x * 8 + 4] = global_ns();
        if (prev + 1 == static_cast<unsigned int>(__popc(mask))) {
            __threadfence_block();
            // first and last CTA with rows of this block: the inverse of unit_begin (warp holding row x: ceil((x+1)*W/RT) - 1)
            int i_first, i_last;
            if (aligned) {
                i_first = static_cast<int>(static_cast<unsigned int>(cblock) * W / C) / WARPS;
                i_last = (static_cast<int>(static_cast<unsigned int>(cblock + 1) * W / C) - 1) / WARPS;
            } else if (narrow) {
                i_first = static_cast<int>(((static_cast<unsigned int>(cblock * RB + 1) * W - 1u) / RT) / WARPS);
                i_last = static_cast<int>(((static_cast<unsigned int>((cblock + 1) * RB) * W - 1u) / RT) / WARPS);
            } else {
                i_first = static_cast<int>((((static_cast<int64_t>(cblock) * RB + 1) * W - 1) / RT) / WARPS);
                i_last = static_cast<int>(((static_cast<int64_t>(cblock + 1) * RB * W - 1) / RT) / WARPS);
            }
            qmv_finish_block<kFused>(p, cblock, mask, second, i_last - i_first + 1, static_cast<int>(blockIdx.x) - i_first, smem_raw,
                             lane);
            if (tracing) p.trace[blockIdx.x * 8 + 5] = global_ns();
        }
    }
    if (copy_lost && lane == 0) atomicExch(p.error, 1u);
}

template <int K, int CB, int NB, int MODE, int FUSED>
cudaError_t qmv_launch_one(const QmvArgs& p, const QmvPlan& plan, cudaStream_t stream) {
    auto kernel = qmv_kernel<K, CB, NB, MODE, FUSED>;
    static PerDeviceOnce attribute;                         // once per kernel and device: allow the largest carve-out
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQmvMaxSmemBytes);
        if (e != cudaSuccess) return e;
        attribute.mark();
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
    const int fused = (p.prologue == 4 || p.epilogue == 3) ? 2 : ((p.prologue != 0 || p.epilogue != 0) ? 1 : 0);
    if (p.rows <= 8) {
        if (fused == 2) return qmv_launch_one<K, CB, 1, MODE, 2>(p, plan, stream);
        return fused ? qmv_launch_one<K, CB, 1, MODE, 1>(p, plan, stream) : qmv_launch_one<K, CB, 1, MODE, 0>(p, plan, stream);
    }
    if (fused == 2) return qmv_launch_one<K, CB, 2, MODE, 2>(p, plan, stream);
    return fused ? qmv_launch_one<K, CB, 2, MODE, 1>(p, plan, stream) : qmv_launch_one<K, CB, 2, MODE, 0>(p, plan, stream);
}

template <int K>
cudaError_t qmv_launch_k(const QmvArgs& p, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream) {
    if (cb == 2) return qmv_launch_nb<K, 2, 1>(p, plan, stream);
    if (cb == 0) return exact ? qmv_launch_nb<K, 0, 1>(p, plan, stream) : qmv_launch_nb<K, 0, 0>(p, plan, stream);
    return exact ? qmv_launch_nb<K, 1, 1>(p, plan, stream) : qmv_launch_nb<K, 1, 0>(p, plan, stream);
}

}  // namespace b200exl3
