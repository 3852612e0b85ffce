// Glue kernels of the grouped-expert SwiGLU block (reference: native/src/moe.rs).  One warp per
// 128-block; lane l holds elements 4l..4l+3, as in the stand-alone rotation kernels.
//
//   routed prepare    native/src/moe.rs:184-236   x row of the slot's token * gate/up input scales of the
//                                                  slot's expert, rotated (same rounding points as the
//                                                  plain input rotation); for small batches the expert kernel
//                                                  does this itself, the padded form below serves the sorted path
//   glu_down_input    native/src/moe.rs:438-533   SiLU path: both rotations without intermediate rounding
//   finish_and_reduce native/src/moe.rs:586-609   output rotation, expert output scales, routing weights,
//                                                  sum over the top_k slots of a token
#include "hadamard.cuh"
#include "kernels.h"

namespace b200exl3 {

namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ int expert_of(const uint32_t* selected, int64_t slot, int experts) {
    // an out-of-range id must not read out of bounds (unsigned compare: ids of 2^31 and more stay large)
    return static_cast<int>(min(selected[slot], static_cast<uint32_t>(experts - 1)));
}

__device__ __forceinline__ float silu(float v) { return glu_silu(v); }

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
glu_down_input_kernel(const float* __restrict__ ygu, const __half* __restrict__ gu_svh, const __half* __restrict__ down_suh,
                      const uint32_t* __restrict__ selected, int experts, int64_t slots, int hidden, int logical_hidden,
                      __half* __restrict__ xhat, const int* __restrict__ count) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = hidden >> 7;
    if (count != nullptr) slots = min(slots, static_cast<int64_t>(*count));
    const int64_t total = slots * blocks_per_row;
    const float scale = had_scale();
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int64_t slot = unit / blocks_per_row;
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        const int64_t expert = expert_of(selected, slot, experts);
        const float4 graw = *reinterpret_cast<const float4*>(ygu + (slot * 2) * hidden + col);
        const float4 uraw = *reinterpret_cast<const float4*>(ygu + (slot * 2 + 1) * hidden + col);
        float gv[4] = {round_half(graw.x), round_half(graw.y), round_half(graw.z), round_half(graw.w)};
        float uv[4] = {round_half(uraw.x), round_half(uraw.y), round_half(uraw.z), round_half(uraw.w)};
        warp_hadamard128<false, false>(gv, lane);
        warp_hadamard128<false, false>(uv, lane);
        const __half* sg = gu_svh + (expert * 2) * hidden + col;
        const __half* su = gu_svh + (expert * 2 + 1) * hidden + col;
        const __half* sd = down_suh + expert * hidden + col;
        float d[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gate = round_half(__fmul_rn(__fmul_rn(gv[j], scale), __half2float(sg[j])));
            const float up = round_half(__fmul_rn(__fmul_rn(uv[j], scale), __half2float(su[j])));
            float act = round_half(__fmul_rn(silu(gate), up));
            if (col + j >= logical_hidden) act = 0.0f;
            d[j] = round_half(__fmul_rn(act, __half2float(sd[j])));
        }
        warp_hadamard128<false, false>(d, lane);
        __align__(8) __half h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __float2half_rn(__fmul_rn(d[j], scale));
        *reinterpret_cast<uint2*>(xhat + slot * hidden + col) = *reinterpret_cast<uint2*>(h);
    }
}

template <bool F32>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
finish_and_reduce_kernel(const float* __restrict__ raw, const __half* __restrict__ down_svh,
                         const uint32_t* __restrict__ selected, int experts, const void* __restrict__ scores,
                         int64_t rows, int top_k, int out, void* __restrict__ y) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = out >> 7;
    const int64_t total = rows * blocks_per_row;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int64_t row = unit / blocks_per_row;
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        float acc32[4] = {0.f, 0.f, 0.f, 0.f};
        __half acc16[4];
        // the slots are added in order, but their loads go out four at a time (a token has few slots and few
        // 128-blocks: the latency of one slot after the other would be the whole kernel)
        for (int t0 = 0; t0 < top_k; t0 += 4) {
            float4 r[4];
            uint2 svw[4];
            float score32[4];
            __half score16[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (t0 + i >= top_k) continue;
                const int64_t slot = row * top_k + t0 + i;
                r[i] = *reinterpret_cast<const float4*>(raw + slot * out + col);
                svw[i] = *reinterpret_cast<const uint2*>(down_svh + static_cast<int64_t>(expert_of(selected, slot, experts)) * out + col);
                if (F32) score32[i] = reinterpret_cast<const float*>(scores)[slot];
                else score16[i] = reinterpret_cast<const __half*>(scores)[slot];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (t0 + i >= top_k) continue;
                __half h[4] = {__float2half_rn(r[i].x), __float2half_rn(r[i].y), __float2half_rn(r[i].z), __float2half_rn(r[i].w)};
                warp_hadamard128_f16(h, lane);
                const __half* sv = reinterpret_cast<const __half*>(&svw[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half scaled = __hmul_rn(h[j], sv[j]);
                    if (F32) {
                        // fp16 product promoted to the fp32 routing weight; the sum over slots stays in fp32
                        const float v = __fmul_rn(__half2float(scaled), score32[i]);
                        acc32[j] = t0 + i == 0 ? v : __fadd_rn(acc32[j], v);
                    } else {
                        const __half v = __hmul_rn(scaled, score16[i]);
                        acc16[j] = t0 + i == 0 ? v : __hadd_rn(acc16[j], v);
                    }
                }
            }
        }
        if (F32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row * out + col) = make_float4(acc32[0], acc32[1], acc32[2], acc32[3]);
        else *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(y) + row * out + col) = *reinterpret_cast<uint2*>(acc16);
    }
}

unsigned grid_for(int64_t units) {
    const int64_t blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

cudaError_t launch_glu_down_input(const float* ygu, const __half* gu_svh, const __half* down_suh, const uint32_t* selected,
                                  int experts, int64_t slots, int hidden, int logical_hidden, __half* xhat,
                                  cudaStream_t stream, const int* count) {
    if (slots == 0) return cudaSuccess;
    return launch_dependent(glu_down_input_kernel, dim3(grid_for(slots * (hidden / 128))), dim3(kWarpsPerBlock * 32), 0, stream, ygu, gu_svh,
                            down_suh, selected, experts, slots, hidden, logical_hidden, xhat, count);
}

cudaError_t launch_finish_and_reduce(const float* raw, const __half* down_svh, const uint32_t* selected, int experts,
                                     const void* scores, int score_dtype, int64_t rows, int top_k, int out, void* y,
                                     cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const unsigned grid = grid_for(rows * (out / 128));
    return launch_dependent(score_dtype == kF32 ? finish_and_reduce_kernel<true> : finish_and_reduce_kernel<false>, dim3(grid),
                            dim3(kWarpsPerBlock * 32), 0, stream, raw, down_svh, selected, experts, scores, rows, top_k, out, y);
}

}  // namespace b200exl3

// ---- expert-sorted form (many slots) ------------------------------------------------------------------------
namespace b200exl3 {

namespace {

constexpr uint32_t kNoSlot = 0xffffffffu;

// One CTA plans the whole batch: counts per expert, segments of seg_rows rows per expert in expert order, and the
// two maps between slots and padded rows.
__global__ void __launch_bounds__(1024)
route_plan_kernel(const uint32_t* __restrict__ selected, int64_t slots, int experts, int max_segments, int seg_rows,
                  int* __restrict__ seg_count, uint32_t* __restrict__ seg_expert, uint32_t* __restrict__ row_slot,
                  uint32_t* __restrict__ slot_row) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    extern __shared__ int s_mem[];
    int* count = s_mem;                 // [experts] rows per expert, then running position
    int* base = s_mem + experts;        // [experts + 1] first segment of each expert
    // expert of every slot, staged once (the walk below reads each of them once per expert)
    unsigned short* ids = reinterpret_cast<unsigned short*>(s_mem + 2 * experts + 1);
    for (int64_t s = threadIdx.x; s < slots; s += blockDim.x)
        ids[s] = static_cast<unsigned short>(min(selected[s], static_cast<uint32_t>(experts - 1)));
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int64_t r = threadIdx.x; r < static_cast<int64_t>(max_segments) * seg_rows; r += blockDim.x) row_slot[r] = kNoSlot;
    __syncthreads();
    // One warp per expert walks the slots in order, 32 at a time: a slot's position among its expert's rows is the
    // number of earlier slots with the same expert (ballot + population count), so the plan (and with it the
    // summation order of every row's products, which depends on the segment a row lands in) is the same on every call.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    {
        for (int e = warp; e < experts; e += warps) {
            int pos = 0;
            for (int64_t s0 = 0; s0 < slots; s0 += 32) {
                const int64_t s = s0 + lane;
                const bool mine = s < slots && ids[s] == e;
                const unsigned int votes = __ballot_sync(0xffffffffu, mine);
                if (mine) slot_row[s] = static_cast<uint32_t>(pos + __popc(votes & ((1u << lane) - 1u)));
                pos += __popc(votes);
            }
            if (lane == 0) count[e] = pos;
        }
    }
    __syncthreads();
    if (warp == 0) {
        // first segment of every expert: a running sum of the experts' segment counts, 32 experts per step of one warp
        int carry = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const int segs = e < experts ? (count[e] + seg_rows - 1) / seg_rows : 0;
            int incl = segs;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (e < experts) base[e] = carry + incl - segs;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            base[experts] = carry;
            seg_count[0] = min(carry, max_segments);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        for (int s = base[e]; s < base[e + 1] && s < max_segments; ++s) seg_expert[s] = static_cast<uint32_t>(e);
    for (int64_t s = threadIdx.x; s < slots; s += blockDim.x) {
        const int e = ids[s];
        const int pos = static_cast<int>(slot_row[s]);
        const int64_t row = static_cast<int64_t>(base[e] + pos / seg_rows) * seg_rows + pos % seg_rows;
        slot_row[s] = static_cast<uint32_t>(row);
        if (row < static_cast<int64_t>(max_segments) * seg_rows) row_slot[row] = static_cast<uint32_t>(s);
    }
}

// The same plan in three short passes (used whenever its table fits shared memory).  Slots are taken 32 at a time
// (a group): pass 1 counts, per group and expert, the slots of the group that chose the expert (match + population
// count: a slot's rank inside its group is the number of earlier lanes with the same expert); pass 2 turns the counts
// of every expert into running positions over the groups (one thread per expert); pass 3 gives every slot its row.
// The walk of the kernel above costs slots x experts / 32 warp steps (45 us for 2048 slots and 128 experts); this one
// costs slots / 32 + groups steps.  Same plan, bit for bit: position = number of earlier slots with the same expert.
__global__ void __launch_bounds__(1024)
route_plan_grouped_kernel(const uint32_t* __restrict__ selected, int64_t slots, int experts, int max_segments, int seg_rows,
                          int* __restrict__ seg_count, uint32_t* __restrict__ seg_expert, uint32_t* __restrict__ row_slot,
                          uint32_t* __restrict__ slot_row) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    extern __shared__ int s_mem[];
    int* count = s_mem;                 // [experts] rows per expert
    int* base = s_mem + experts;        // [experts + 1] first segment of each expert
    unsigned short* table = reinterpret_cast<unsigned short*>(s_mem + 2 * experts + 1);   // [groups][experts]: counts, then positions
    const int groups = static_cast<int>((slots + 31) / 32);
    // every slot's expert and its rank inside its group stay in shared memory between the passes
    unsigned short* slot_expert = table + static_cast<size_t>(groups) * experts;         // [groups * 32]
    unsigned char* slot_rank = reinterpret_cast<unsigned char*>(slot_expert + static_cast<size_t>(groups) * 32);   // [groups * 32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < groups * experts; i += blockDim.x) table[i] = 0;
    for (int64_t r = threadIdx.x; r < static_cast<int64_t>(max_segments) * seg_rows; r += blockDim.x) row_slot[r] = kNoSlot;
    __syncthreads();
    for (int g = warp; g < groups; g += warps) {
        const int64_t s = static_cast<int64_t>(g) * 32 + lane;
        const uint32_t e = s < slots ? min(selected[s], static_cast<uint32_t>(experts - 1)) : 0xffffffffu;
        const unsigned int same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (s < slots) {
            slot_expert[s] = static_cast<unsigned short>(e);
            slot_rank[s] = static_cast<unsigned char>(rank);                // rank inside the group, for pass 3
            if (rank == 0) table[g * experts + e] = static_cast<unsigned short>(__popc(same));
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int running = 0;
        for (int g = 0; g < groups; ++g) {
            const int c = table[g * experts + e];
            table[g * experts + e] = static_cast<unsigned short>(running);
            running += c;
        }
        count[e] = running;
    }
    __syncthreads();
    if (warp == 0) {
        // first segment of every expert: a running sum of the experts' segment counts, 32 experts per step of one warp
        int carry = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const int segs = e < experts ? (count[e] + seg_rows - 1) / seg_rows : 0;
            int incl = segs;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (e < experts) base[e] = carry + incl - segs;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            base[experts] = carry;
            seg_count[0] = min(carry, max_segments);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        for (int s = base[e]; s < base[e + 1] && s < max_segments; ++s) seg_expert[s] = static_cast<uint32_t>(e);
    for (int64_t s = threadIdx.x; s < slots; s += blockDim.x) {
        const int e = slot_expert[s];
        const int pos = table[(s >> 5) * experts + e] + static_cast<int>(slot_rank[s]);
        const int64_t row = static_cast<int64_t>(base[e] + pos / seg_rows) * seg_rows + pos % seg_rows;
        slot_row[s] = static_cast<uint32_t>(row);
        if (row < static_cast<int64_t>(max_segments) * seg_rows) row_slot[row] = static_cast<uint32_t>(s);
    }
}

// One warp per (slot, projection, 128-block): only rows that hold a slot are written.  Padding rows are left as they
// are: every activation row is multiplied on its own, and nothing downstream reads the products of a padding row.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
routed_prepare_padded_kernel(const void* __restrict__ x, int x_dtype, const __half* __restrict__ suh,
                             const uint32_t* __restrict__ seg_expert, const uint32_t* __restrict__ slot_row, int64_t slots,
                             int max_segments, int top_k, int proj, int in, int seg_rows, __half* __restrict__ xhat) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = in >> 7;
    const int64_t total = slots * proj * blocks_per_row;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        const int64_t sp = unit / blocks_per_row;                        // slot * proj + p
        const int64_t slot = sp / proj;
        const int p = static_cast<int>(sp - slot * proj);
        const int64_t prow = slot_row[slot];                             // segment * seg_rows + r
        const int64_t seg = prow / seg_rows;
        if (seg >= max_segments) continue;
        const int64_t out_row = (seg * proj + p) * seg_rows + (prow - seg * seg_rows);
        const __half* s = suh + (static_cast<int64_t>(seg_expert[seg]) * proj + p) * in + col;
        const int64_t token = slot / top_k;
        __align__(8) __half h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(load_as_half(x, x_dtype, token * in + col + j), s[j]);
        warp_hadamard128_f16(h, lane);
        *reinterpret_cast<uint2*>(xhat + out_row * in + col) = *reinterpret_cast<uint2*>(h);
    }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
glu_down_input_padded_kernel(const float* __restrict__ ygu, const __half* __restrict__ gu_svh, const __half* __restrict__ down_suh,
                             const uint32_t* __restrict__ seg_expert, const uint32_t* __restrict__ row_slot,
                             const int* __restrict__ seg_count, int max_segments, int hidden, int logical_hidden, int seg_rows,
                             __half* __restrict__ xhat) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = hidden >> 7;
    const int64_t total = static_cast<int64_t>(seg_count[0]) * seg_rows * blocks_per_row;
    const int64_t row_stride = static_cast<int64_t>(max_segments) * 2 * hidden;       // products are [seg_rows, segments * 2 * hidden]
    const float scale = had_scale();
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int64_t prow = unit / blocks_per_row;                      // segment * seg_rows + r
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        const int64_t seg = prow / seg_rows;
        const int r = static_cast<int>(prow - seg * seg_rows);
        __align__(8) __half h[4] = {__half(), __half(), __half(), __half()};
        if (row_slot[prow] != kNoSlot) {
            const int64_t expert = seg_expert[seg];
            const float4 graw = *reinterpret_cast<const float4*>(ygu + r * row_stride + (seg * 2) * hidden + col);
            const float4 uraw = *reinterpret_cast<const float4*>(ygu + r * row_stride + (seg * 2 + 1) * hidden + col);
            float gv[4] = {round_half(graw.x), round_half(graw.y), round_half(graw.z), round_half(graw.w)};
            float uv[4] = {round_half(uraw.x), round_half(uraw.y), round_half(uraw.z), round_half(uraw.w)};
            warp_hadamard128<false, false>(gv, lane);
            warp_hadamard128<false, false>(uv, lane);
            const __half* sg = gu_svh + (expert * 2) * hidden + col;
            const __half* su = gu_svh + (expert * 2 + 1) * hidden + col;
            const __half* sd = down_suh + expert * hidden + col;
            float d[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float gate = round_half(__fmul_rn(__fmul_rn(gv[j], scale), __half2float(sg[j])));
                const float up = round_half(__fmul_rn(__fmul_rn(uv[j], scale), __half2float(su[j])));
                float act = round_half(__fmul_rn(silu(gate), up));
                if (col + j >= logical_hidden) act = 0.0f;
                d[j] = round_half(__fmul_rn(act, __half2float(sd[j])));
            }
            warp_hadamard128<false, false>(d, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __float2half_rn(__fmul_rn(d[j], scale));
        }
        *reinterpret_cast<uint2*>(xhat + prow * hidden + col) = *reinterpret_cast<uint2*>(h);
    }
}

template <bool F32>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
finish_and_reduce_padded_kernel(const float* __restrict__ raw, const __half* __restrict__ down_svh,
                                const uint32_t* __restrict__ selected, const uint32_t* __restrict__ slot_row, int experts,
                                const void* __restrict__ scores, int64_t rows, int top_k, int out, int max_segments, int seg_rows,
                                void* __restrict__ y) {
    pdl_launch_dependents();                    // the kernel after this one may start; it waits for our memory itself
    pdl_wait();                                 // what the kernel before this one wrote is visible from here on
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = out >> 7;
    const int64_t total = rows * blocks_per_row;
    const int64_t row_stride = static_cast<int64_t>(max_segments) * out;              // products are [seg_rows, segments * out]
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int64_t row = unit / blocks_per_row;
        const int col = static_cast<int>(unit % blocks_per_row) * 128 + lane * 4;
        float acc32[4] = {0.f, 0.f, 0.f, 0.f};
        __half acc16[4];
        for (int t = 0; t < top_k; ++t) {
            const int64_t slot = row * top_k + t;
            const int64_t prow = slot_row[slot];
            const float4 r = *reinterpret_cast<const float4*>(raw + (prow % seg_rows) * row_stride + (prow / seg_rows) * out + col);
            __half h[4] = {__float2half_rn(r.x), __float2half_rn(r.y), __float2half_rn(r.z), __float2half_rn(r.w)};
            warp_hadamard128_f16(h, lane);
            const __half* sv = down_svh + static_cast<int64_t>(expert_of(selected, slot, experts)) * out + col;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half scaled = __hmul_rn(h[j], sv[j]);
                if (F32) {
                    const float v = __fmul_rn(__half2float(scaled), reinterpret_cast<const float*>(scores)[slot]);
                    acc32[j] = t == 0 ? v : __fadd_rn(acc32[j], v);
                } else {
                    const __half v = __hmul_rn(scaled, reinterpret_cast<const __half*>(scores)[slot]);
                    acc16[j] = t == 0 ? v : __hadd_rn(acc16[j], v);
                }
            }
        }
        if (F32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row * out + col) = make_float4(acc32[0], acc32[1], acc32[2], acc32[3]);
        else *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(y) + row * out + col) = *reinterpret_cast<uint2*>(acc16);
    }
}

}  // namespace

cudaError_t launch_route_plan(const uint32_t* selected, int64_t slots, int experts, int max_segments, int seg_rows, int* seg_count,
                              uint32_t* seg_expert, uint32_t* row_slot, uint32_t* slot_row, cudaStream_t stream) {
    if (experts > 65535 || slots >= 65535) return cudaErrorInvalidValue;              // positions are kept in 16 bits
    const size_t groups = static_cast<size_t>((slots + 31) / 32);
    const size_t grouped = (2 * static_cast<size_t>(experts) + 1) * sizeof(int) + groups * experts * sizeof(unsigned short) +
                           groups * 32 * (sizeof(unsigned short) + sizeof(unsigned char));
    if (grouped <= 48 * 1024) {
        return launch_dependent(route_plan_grouped_kernel, dim3(1), dim3(1024), grouped, stream, selected, slots, experts, max_segments,
                                seg_rows, seg_count, seg_expert, row_slot, slot_row);
    }
    const size_t smem = (2 * static_cast<size_t>(experts) + 1) * sizeof(int) + static_cast<size_t>(slots) * sizeof(unsigned short);
    if (smem > 48 * 1024) return cudaErrorInvalidValue;
    return launch_dependent(route_plan_kernel, dim3(1), dim3(1024), smem, stream, selected, slots, experts, max_segments, seg_rows,
                            seg_count, seg_expert, row_slot, slot_row);
}

cudaError_t launch_routed_prepare_padded(const void* x, int x_dtype, const __half* suh, const uint32_t* seg_expert,
                                         const uint32_t* slot_row, int64_t slots, int top_k, int proj, int max_segments,
                                         int seg_rows, int in, __half* xhat, cudaStream_t stream) {
    return launch_dependent(routed_prepare_padded_kernel, dim3(grid_for(slots * proj * (in / 128))), dim3(kWarpsPerBlock * 32), 0, stream, x,
                            x_dtype, suh, seg_expert, slot_row, slots, max_segments, top_k, proj, in, seg_rows, xhat);
}

cudaError_t launch_glu_down_input_padded(const float* ygu, const __half* gu_svh, const __half* down_suh,
                                         const uint32_t* seg_expert, const uint32_t* row_slot, const int* seg_count,
                                         int experts, int max_segments, int seg_rows, int hidden, int logical_hidden, __half* xhat,
                                         cudaStream_t stream) {
    (void)experts;
    return launch_dependent(glu_down_input_padded_kernel, dim3(grid_for(static_cast<int64_t>(max_segments) * seg_rows * (hidden / 128))),
                            dim3(kWarpsPerBlock * 32), 0, stream, ygu, gu_svh, down_suh, seg_expert, row_slot, seg_count, max_segments, hidden,
                            logical_hidden, seg_rows, xhat);
}

cudaError_t launch_finish_and_reduce_padded(const float* raw, const __half* down_svh, const uint32_t* selected,
                                            const uint32_t* slot_row, int experts, const void* scores, int score_dtype,
                                            int64_t rows, int top_k, int out, int max_segments, int seg_rows, void* y, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const unsigned grid = grid_for(rows * (out / 128));
    return launch_dependent(score_dtype == kF32 ? finish_and_reduce_padded_kernel<true> : finish_and_reduce_padded_kernel<false>, dim3(grid),
                            dim3(kWarpsPerBlock * 32), 0, stream, raw, down_svh, selected, slot_row, experts, scores, rows, top_k, out,
                            max_segments, seg_rows, y);
}

}  // namespace b200exl3
