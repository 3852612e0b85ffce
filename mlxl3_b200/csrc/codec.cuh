// EXL3 trellis format on the device: state windows and the three procedural codebooks.
//
// Format (reference: native/src/codec.rs:34-71, native/shaders/exl3.metal:8-20, 72-83):
// a tile is 16*K uint16 = 8*K little-endian uint32 words, read as one circular stream of
// 256*K bits, most significant bit first inside each word.  State t (0..255) is the 16-bit
// window that ends at stream bit (t+1)*K.  Lane L of a warp owns states 8L..8L+7, which are
// the mma.m16n8k16 fragment elements (rows 2q+{0,1,8,9}, columns g and g+8; q = L%4, g = L/4)
// of the 16x16 weight tile (native/src/codec.rs:126-138).
#pragma once

#include "common.cuh"

namespace b200exl3 {

// ---- per-state window, any K, straight from the packed uint16 array (exl3.metal:72-83) ------------
__device__ __forceinline__ uint32_t tile_state(const uint16_t* __restrict__ tile, int k, int t) {
    int b0 = t * k + k + 256 * k - 16;
    int b1 = b0 + 16;
    int nw = 8 * k;
    int i0 = (b0 >> 5) % nw;
    int last = (b1 - 1) >> 5;
    int i1 = last % nw;
    int shift = ((last + 1) << 5) - b1;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(tile);
    uint64_t merged = (static_cast<uint64_t>(words[i0]) << 32) | words[i1];
    return static_cast<uint32_t>(merged >> shift) & 0xffffu;
}

// Same window with the tile's words `stride` apart (stride 4 = the quad layout of the fused kernels).
__device__ __forceinline__ uint32_t tile_state_strided(const uint32_t* __restrict__ words, int stride, int k, int t) {
    int b0 = t * k + k + 256 * k - 16;
    int b1 = b0 + 16;
    int nw = 8 * k;
    int i0 = (b0 >> 5) % nw;
    int last = (b1 - 1) >> 5;
    int i1 = last % nw;
    int shift = ((last + 1) << 5) - b1;
    uint64_t merged = (static_cast<uint64_t>(words[i0 * stride]) << 32) | words[i1 * stride];
    return static_cast<uint32_t>(merged >> shift) & 0xffffu;
}

// ---- codebooks ------------------------------------------------------------------------------------

// Codebooks 0 and 1: the 32-bit pattern whose two fp16 halves add up to the weight.
template <int CB>
__device__ __forceinline__ uint32_t codeword_halves(uint32_t state) {
    static_assert(CB == 0 || CB == 1, "half-pair form exists for codebooks 0 and 1 only");
    uint32_t b = CB == 0 ? state * 89226354u + 64248484u : state * 0xcbac1fedu;
    return lop3_and_xor(b, 0x8fff8fffu, 0x3b603b60u);
}

// Codebook 2: fp16 bit pattern of 1024 + (sum of the four bytes of state * 0x83DCD12D); the weight
// is fma(h, 0x1EEE, 0xC931) with one rounding.
__device__ __forceinline__ uint32_t mul1_sum_bits(uint32_t state) {
    uint32_t b = state * 0x83dcd12du;
    return __dp4a(b, 0x01010101u, 0x6400u);
}

// Bit-exact fp16 weight of one state (native/src/codec.rs:52-71).
template <int CB>
__device__ __forceinline__ __half decode_codeword(uint32_t state) {
    if constexpr (CB == 2) {
        __half h = __ushort_as_half(static_cast<unsigned short>(mul1_sum_bits(state)));
        return __hfma(h, __ushort_as_half(0x1eee), __ushort_as_half(0xc931));
    } else {
        uint32_t v = codeword_halves<CB>(state);
        return __hadd_rn(__ushort_as_half(static_cast<unsigned short>(v & 0xffffu)),
                      __ushort_as_half(static_cast<unsigned short>(v >> 16)));
    }
}

__device__ __forceinline__ __half decode_codeword_rt(uint32_t state, int cb) {
    if (cb == 0) return decode_codeword<0>(state);
    if (cb == 1) return decode_codeword<1>(state);
    return decode_codeword<2>(state);
}

}  // namespace b200exl3
