// Sum of one unit (128 columns of one row) of fp32 partial products over the ranks of a tensor-parallel
// group, through peer memory.  Used by the stand-alone exchange kernel and by the fused layer kernel.
//
// Protocol (all ranks issue the same calls in the same order; one warp per unit).  Every value travels in an
// 8-byte word together with the call's sequence number, written and read as ONE 64-bit scalar access, so one
// store publishes it and no fence is needed (measured here: 10.5 us per exchange with a fence-and-flag
// protocol).  For its c-th use of a unit a rank
//   1. stores {value, c} for its 128 partial sums into slot [c & 1][own rank][unit] of every rank's inbox,
//   2. polls its own inbox until every word of slots [c & 1][src][unit] carries c, for every src,
//   3. adds the values in rank order in fp32 (so every rank gets the same bits) and records c as done.
// A rank can run at most one call ahead of another (its next call cannot finish without the other's data),
// which is what the two slots per unit are for.  The wait is bounded (four seconds unless the "tp_wait_ms" option says otherwise): when it gives up
// the status word is set to 4, later waits give up after a few hundred polls, and the caller carries on with what
// it has (a wrong sum, flagged by the status).  The use counts of the ranks may then disagree: the context is
// reset on every rank (b200exl3_tp_reset) or rebuilt before it is used again.
#pragma once

#include "common.cuh"

namespace b200exl3 {

constexpr int kTpMaxWorld = 8;
constexpr int kTpUnitWords = 128;                 // 8-byte {value, sequence} words per unit and source

struct TpPeers {
    uint2* inbox[kTpMaxWorld];         // every rank's inbox [2, world, max_units, 128] words (own one at [rank])
    unsigned int* done;                // [max_units] uses completed by this rank
    unsigned int* error;               // status word
    int rank, world, max_units;        // world == 0: no exchange
    unsigned long long wait_ns;        // how long a rank polls for the others' words before it gives up
};

// One 64-bit scalar access each way: the memory model makes an aligned 8-byte scalar store single-copy atomic,
// so a reader sees the value and its sequence number together or not at all (a two-element vector access
// would be two independent 4-byte accesses and could be seen torn).
__device__ __forceinline__ void store_word(uint2* p, uint2 v) {
    const unsigned long long w = (static_cast<unsigned long long>(v.y) << 32) | v.x;
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 load_word(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
}

// `mine`: this rank's sums for columns 4*lane..4*lane+3 of unit u.  Returns the sum over ranks.
__device__ __forceinline__ float4 tp_exchange_unit(const TpPeers& t, int u, float4 mine, int lane) {
    const size_t slot_words = static_cast<size_t>(t.max_units) * kTpUnitWords;
    unsigned int c = 0;
    if (lane == 0) c = t.done[u] + 1;
    c = __shfl_sync(0xffffffffu, c, 0);
    const size_t parity = (c & 1u) * static_cast<size_t>(t.world) * slot_words;
    const size_t at = parity + t.rank * slot_words + static_cast<size_t>(u) * kTpUnitWords + lane * 4;
    const uint32_t bits[4] = {__float_as_uint(mine.x), __float_as_uint(mine.y), __float_as_uint(mine.z), __float_as_uint(mine.w)};
#pragma unroll 1
    for (int r = 0; r < t.world; ++r) {
        uint2* dst = t.inbox[r] + at;
#pragma unroll
        for (int j = 0; j < 4; ++j) store_word(dst + j, make_uint2(bits[j], c));
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool lost = false;
#pragma unroll 1
    for (int src = 0; src < t.world; ++src) {
        const uint2* from = t.inbox[t.rank] + parity + src * slot_words + static_cast<size_t>(u) * kTpUnitWords + lane * 4;
        uint2 w[4];
        bool ok = false;
        unsigned long long t0 = 0;
#pragma unroll 1
        for (int i = 0; !ok; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = load_word(from + j);
            ok = w[0].y == c && w[1].y == c && w[2].y == c && w[3].y == c;
            if (ok) break;
            // give up after the wait limit, or at once when an earlier wait of this rank already gave up
            if ((i & 255) == 255) {
                if (t0 == 0) t0 = global_ns();
                if (*reinterpret_cast<volatile unsigned int*>(t.error) != 0 || global_ns() - t0 > t.wait_ns) { lost = true; break; }
            }
        }
        const float v[4] = {__uint_as_float(w[0].x), __uint_as_float(w[1].x), __uint_as_float(w[2].x), __uint_as_float(w[3].x)};
        if (src == 0) acc = make_float4(v[0], v[1], v[2], v[3]);
        else { acc.x = __fadd_rn(acc.x, v[0]); acc.y = __fadd_rn(acc.y, v[1]); acc.z = __fadd_rn(acc.z, v[2]); acc.w = __fadd_rn(acc.w, v[3]); }
    }
    if (__any_sync(0xffffffffu, lost) && lane == 0) atomicExch(t.error, 4u);
    if (lane == 0) t.done[u] = c;
    return acc;
}

}  // namespace b200exl3
