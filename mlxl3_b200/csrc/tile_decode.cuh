// Register-level decode of one 16x16 EXL3 tile by one warp, shared by the fused small-batch kernel
// and the tensor-core prefill kernel.
//
// Lane L owns states 8L..8L+7 of the tile = elements (rows 2q+{0,1,8,9}, columns g and g+8) of the
// weight tile W[16 inputs, 16 outputs] (q = L%4, g = L/4), which is the A-fragment of mma.m16n8k16
// for W^T (reference: native/src/codec.rs:126-138).
#pragma once

#include "codec.cuh"

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

// The lane's eight weights as the reference's bit-exact fp16 values, packed as the four A-fragment
// registers of W^T: a0 = (out g; in 2q,2q+1), a1 = (out g+8; in 2q,2q+1), a2 = (out g; in 2q+8,2q+9),
// a3 = (out g+8; in 2q+8,2q+9).
template <int K, int CB>
__device__ __forceinline__ void lane_weights_exact(uint32_t w2, uint32_t w1, uint32_t w0, int slack, uint32_t& a0,
                                                   uint32_t& a1, uint32_t& a2, uint32_t& a3) {
    uint32_t b[8];
    lane_hashes<K, CB>(w2, w1, w0, slack, b);
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
        // a weight is the fp16 sum of the two halves of its masked hash: two scalar adds that select their halves
        // (no repacking before them) and one merge -- one logic-pipe instruction less per pair than packing
        // (lo, lo) and (hi, hi) first
        auto pair = [&](uint32_t x, uint32_t y) {
            x = lop3_and_xor(x, 0x8fff8fffu, 0x3b603b60u);
            y = lop3_and_xor(y, 0x8fff8fffu, 0x3b603b60u);
            const __half2 hx = *reinterpret_cast<__half2*>(&x), hy = *reinterpret_cast<__half2*>(&y);
            const __half2 w = __halves2half2(__hadd_rn(__low2half(hx), __high2half(hx)), __hadd_rn(__low2half(hy), __high2half(hy)));
            return *reinterpret_cast<const uint32_t*>(&w);
        };
        a0 = pair(b[0], b[1]); a1 = pair(b[4], b[5]); a2 = pair(b[2], b[3]); a3 = pair(b[6], b[7]);
    }
}

}  // namespace b200exl3
