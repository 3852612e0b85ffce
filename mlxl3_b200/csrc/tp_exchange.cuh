// Sum of one unit (128 columns of one row) of fp32 partial products over the ranks of a tensor-parallel
// group, through peer memory.  Used by the stand-alone exchange kernel and by the fused layer kernel.
//
// Protocol (all ranks issue the same calls in the same order; one warp per unit).  For its c-th use of a
// unit a rank
//   1. stores its 128 partial sums into slot [c & 1][own rank][unit] of every rank's inbox (peer stores),
//   2. fences system-wide and stores c into flag [own rank][unit] of every rank,
//   3. waits until its own flags [src][unit] have reached c for every src, and adds the slots in rank
//      order in fp32 (so every rank gets the same bits), then records c as done.
// A rank can run at most one call ahead of another (its next call cannot finish without the other's data),
// which is what the two slots per unit are for.  The wait is bounded (about four seconds): when it gives up
// the status word is set to 4, later waits are skipped, and the caller carries on with what it has.
#pragma once

#include "common.cuh"

namespace b200exl3 {

constexpr int kTpMaxWorld = 8;

struct TpPeers {
    float* inbox[kTpMaxWorld];         // every rank's inbox [2, world, max_units, 128] (own one at [rank])
    unsigned int* flags[kTpMaxWorld];  // every rank's arrival flags [world, max_units]
    unsigned int* done;                // [max_units] uses completed by this rank
    unsigned int* error;               // status word
    int rank, world, max_units;        // world == 0: no exchange
};

__device__ __forceinline__ void store_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int load_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// `mine`: this rank's sums for columns 4*lane..4*lane+3 of unit u.  Returns the sum over ranks.
__device__ __forceinline__ float4 tp_exchange_unit(const TpPeers& t, int u, float4 mine, int lane) {
    const size_t slot_floats = static_cast<size_t>(t.max_units) * 128;
    unsigned int c = 0;
    if (lane == 0) c = t.done[u] + 1;
    c = __shfl_sync(0xffffffffu, c, 0);
    const size_t at = ((c & 1u) * t.world + t.rank) * slot_floats + static_cast<size_t>(u) * 128 + lane * 4;
#pragma unroll 1
    for (int r = 0; r < t.world; ++r) *reinterpret_cast<float4*>(t.inbox[r] + at) = mine;
    __threadfence_system();
    __syncwarp();
    if (lane < t.world) store_release_sys(t.flags[lane] + static_cast<size_t>(t.rank) * t.max_units + u, c);
    bool arrived = true;                                   // every lane below `world` watches one source rank
    if (lane < t.world && *reinterpret_cast<volatile unsigned int*>(t.error) == 0) {
        const unsigned int* flag = t.flags[t.rank] + static_cast<size_t>(lane) * t.max_units + u;
        arrived = static_cast<int>(load_acquire_sys(flag) - c) >= 0;
        if (!arrived) {
            const unsigned long long t0 = global_ns();
#pragma unroll 1
            for (int i = 1; !arrived; ++i) {
                arrived = static_cast<int>(load_acquire_sys(flag) - c) >= 0;
                if (!arrived && (i & 255) == 0 && global_ns() - t0 > 4000000000ull) break;
            }
        }
    }
    if (!__all_sync(0xffffffffu, arrived) && lane == 0) atomicExch(t.error, 4u);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* mine_in = t.inbox[t.rank] + (c & 1u) * t.world * slot_floats + static_cast<size_t>(u) * 128 + lane * 4;
#pragma unroll 1
    for (int src = 0; src < t.world; ++src) {
        const float4 v = __ldcv(reinterpret_cast<const float4*>(mine_in + src * slot_floats));
        if (src == 0) acc = v;
        else { acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y); acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w); }
    }
    if (lane == 0) t.done[u] = c;
    return acc;
}

}  // namespace b200exl3
