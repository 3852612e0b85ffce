// Expert parallelism for the grouped-expert SwiGLU block: every rank owns a contiguous range of experts (its own
// gate|up and down banks) and holds the token rows and the routes (the router is replicated).  One call does:
//   1. plan     -- the (token, choice) slots whose expert lives here, compacted in slot order;
//   2. dispatch -- the routed input rotation of exactly those slots (rows gathered by token index);
//   3. the two expert-mapped products and the SwiGLU glue on the local slots only;
//   4. combine  -- every owner rotates and scales its slots' down products and publishes them into EVERY rank's inbox
//                  over peer memory; every rank then adds, for each of its rows, the top-k slot results in slot order.
// Steps 1-2 and 4 are the dispatch and combine halves of the all-to-all: a slot's data crosses NVLink once per
// receiving rank, as 8-byte {two fp16 values, sequence number} words written with single 64-bit stores, so arrival
// is detected on the data itself (no fence, no flag, no collective launch); every wait is bounded.
//
// Reference behaviour kept bit for bit: native/src/moe.rs:184-236 (routed input rotation), 586-609 (finish_and_reduce:
// half(raw) -> H128 -> * down_svh[expert] -> * score, summed over the choices in order in the scores' type).  The
// reference runs all experts on one device; the partition is this build's.
#include "hadamard.cuh"
#include "kernels.h"

namespace b200exl3 {

namespace {

constexpr int kEpWarps = 8;

__device__ __forceinline__ void ep_store_word(unsigned long long* p, uint32_t value, uint32_t seq) {
    const unsigned long long w = (static_cast<unsigned long long>(seq) << 32) | value;
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ep_load_word(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// One CTA: local_slot[i] = i-th slot (ascending) whose expert is in [first, first + count); local_expert[i] = its
// expert relative to `first`.  Ballot + popcount keep the order deterministic.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const uint32_t* __restrict__ selected, int64_t slots, int first, int count, int* __restrict__ local_count,
               uint32_t* __restrict__ local_slot, uint32_t* __restrict__ local_expert) {
    __shared__ int s_warp[32];
    __shared__ int s_base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int64_t s0 = 0; s0 < slots; s0 += 1024) {
        const int64_t s = s0 + threadIdx.x;
        const uint32_t e = s < slots ? selected[s] : 0xffffffffu;
        const bool mine = s < slots && e >= static_cast<uint32_t>(first) && e < static_cast<uint32_t>(first + count);
        const unsigned int votes = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) s_warp[warp] = __popc(votes);
        __syncthreads();
        int before = s_base;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        if (mine) {
            const int at = before + __popc(votes & ((1u << lane) - 1u));
            local_slot[at] = static_cast<uint32_t>(s);
            local_expert[at] = e - static_cast<uint32_t>(first);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 32; ++w) total += s_warp[w];
            s_base += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *local_count = s_base;
}

// xhat[(i * 2 + p), :] = H128(half(half(x[token of local slot i]) * gu_suh[local expert, p])) for i < *local_count
__global__ void __launch_bounds__(kEpWarps * 32)
ep_dispatch_kernel(const void* __restrict__ x, int x_dtype, const __half* __restrict__ gu_suh, const int* __restrict__ local_count,
                   const uint32_t* __restrict__ local_slot, const uint32_t* __restrict__ local_expert, int top_k, int in,
                   int64_t max_slots, __half* __restrict__ xhat) {
    const int lane = threadIdx.x & 31;
    const int blocks = in >> 7;
    const int64_t total = static_cast<int64_t>(min(static_cast<int64_t>(*local_count), max_slots)) * 2 * blocks;
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kEpWarps) {
        const int64_t ip = unit / blocks;
        const int col = static_cast<int>(unit - ip * blocks) * 128 + lane * 4;
        const int64_t i = ip >> 1;
        const int p = static_cast<int>(ip & 1);
        const int64_t token = local_slot[i] / top_k;
        const __half* sc = gu_suh + (static_cast<int64_t>(local_expert[i]) * 2 + p) * in + col;
        __align__(8) __half h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(load_as_half(x, x_dtype, token * in + col + j), sc[j]);
        warp_hadamard128_f16(h, lane);
        *reinterpret_cast<uint2*>(xhat + ip * in + col) = *reinterpret_cast<uint2*>(h);
    }
}

// Owner side of the combine: slot result = half(H128(half(raw)) * down_svh[local expert]) as fp16, published to every
// rank's inbox [parity][slot][out / 2] as {two values, sequence} words.
__global__ void __launch_bounds__(kEpWarps * 32)
ep_publish_kernel(const float* __restrict__ raw, const __half* __restrict__ down_svh, const int* __restrict__ local_count,
                  const uint32_t* __restrict__ local_slot, const uint32_t* __restrict__ local_expert, int out, int64_t max_slots,
                  EpPeers ep) {
    const int lane = threadIdx.x & 31;
    const int blocks = out >> 7;
    const int64_t total = static_cast<int64_t>(min(static_cast<int64_t>(*local_count), max_slots)) * blocks;
    const size_t parity_words = static_cast<size_t>(ep.max_slots) * (out >> 1);
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kEpWarps) {
        const int64_t i = unit / blocks;
        const int col = static_cast<int>(unit - i * blocks) * 128 + lane * 4;
        const float4 r = *reinterpret_cast<const float4*>(raw + i * out + col);
        __half h[4] = {__float2half_rn(r.x), __float2half_rn(r.y), __float2half_rn(r.z), __float2half_rn(r.w)};
        warp_hadamard128_f16(h, lane);
        const __half* sv = down_svh + static_cast<int64_t>(local_expert[i]) * out + col;
        __align__(8) __half v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __hmul_rn(h[j], sv[j]);
        const uint32_t slot = local_slot[i];
        const uint32_t seq = ep.done[slot] + 1u;                 // every rank counts every slot of every call
        const size_t at = (seq & 1u) * parity_words + static_cast<size_t>(slot) * (out >> 1) + (col >> 1);
        const uint32_t* bits = reinterpret_cast<const uint32_t*>(v);
#pragma unroll 1
        for (int r2 = 0; r2 < ep.world; ++r2) {
            ep_store_word(ep.inbox[r2] + at, bits[0], seq);
            ep_store_word(ep.inbox[r2] + at + 1, bits[1], seq);
        }
    }
}

// Receiver side: y[row] = sum over the row's choices, in order, of slot result * score (fp16 or fp32 scores), once the
// slot results of this call have arrived from their owners.
template <bool F32>
__global__ void __launch_bounds__(kEpWarps * 32)
ep_combine_kernel(const void* __restrict__ scores, int64_t rows, int top_k, int out, void* __restrict__ y, EpPeers ep) {
    const int lane = threadIdx.x & 31;
    const int blocks = out >> 7;
    const int64_t total = rows * blocks;
    const size_t parity_words = static_cast<size_t>(ep.max_slots) * (out >> 1);
    const unsigned long long* inbox = ep.inbox[ep.rank];
    for (int64_t unit = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); unit < total;
         unit += static_cast<int64_t>(gridDim.x) * kEpWarps) {
        const int64_t row = unit / blocks;
        const int block = static_cast<int>(unit - row * blocks);
        const int col = block * 128 + lane * 4;
        float acc32[4] = {0.f, 0.f, 0.f, 0.f};
        __half acc16[4];
        bool lost = false;
        for (int t = 0; t < top_k; ++t) {
            const int64_t slot = row * top_k + t;
            const uint32_t seq = ep.done[slot] + 1u;
            const unsigned long long* src = inbox + (seq & 1u) * parity_words + static_cast<size_t>(slot) * (out >> 1) + (col >> 1);
            unsigned long long w0 = 0, w1 = 0;
            unsigned long long t0 = 0;
#pragma unroll 1
            for (int i = 0;; ++i) {
                w0 = ep_load_word(src);
                w1 = ep_load_word(src + 1);
                if (static_cast<uint32_t>(w0 >> 32) == seq && static_cast<uint32_t>(w1 >> 32) == seq) break;
                if ((i & 255) == 255) {
                    if (t0 == 0) t0 = global_ns();
                    if (*reinterpret_cast<volatile unsigned int*>(ep.error) != 0 || global_ns() - t0 > ep.wait_ns) { lost = true; break; }
                }
            }
            const uint32_t pair[2] = {static_cast<uint32_t>(w0), static_cast<uint32_t>(w1)};
            const __half* v = reinterpret_cast<const __half*>(pair);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (F32) {
                    const float p = __fmul_rn(__half2float(v[j]), reinterpret_cast<const float*>(scores)[slot]);
                    acc32[j] = t == 0 ? p : __fadd_rn(acc32[j], p);
                } else {
                    const __half p = __hmul_rn(v[j], reinterpret_cast<const __half*>(scores)[slot]);
                    acc16[j] = t == 0 ? p : __hadd_rn(acc16[j], p);
                }
            }
        }
        if (__any_sync(0xffffffffu, lost) && lane == 0) atomicExch(ep.error, 7u);
        if (F32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + row * out + col) = make_float4(acc32[0], acc32[1], acc32[2], acc32[3]);
        else *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(y) + row * out + col) = *reinterpret_cast<uint2*>(acc16);
        // (the slots' use counts advance in a kernel of their own: every 128-block of a row reads them here)
    }
}

__global__ void ep_count_kernel(unsigned int* done, int64_t slots) {
    const int64_t s = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (s < slots) done[s] += 1u;
}

unsigned ep_grid(int64_t units) {
    const int64_t blocks = (units + kEpWarps - 1) / kEpWarps;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

cudaError_t launch_ep_plan(const uint32_t* selected, int64_t slots, int first, int count, int* local_count, uint32_t* local_slot,
                           uint32_t* local_expert, cudaStream_t stream) {
    ep_plan_kernel<<<1, 1024, 0, stream>>>(selected, slots, first, count, local_count, local_slot, local_expert);
    return cudaGetLastError();
}

cudaError_t launch_ep_dispatch(const void* x, int x_dtype, const __half* gu_suh, const int* local_count, const uint32_t* local_slot,
                               const uint32_t* local_expert, int top_k, int in, int64_t max_slots, __half* xhat, cudaStream_t stream) {
    ep_dispatch_kernel<<<ep_grid(max_slots * 2 * (in / 128)), kEpWarps * 32, 0, stream>>>(x, x_dtype, gu_suh, local_count, local_slot,
                                                                                         local_expert, top_k, in, max_slots, xhat);
    return cudaGetLastError();
}

cudaError_t launch_ep_publish(const float* raw, const __half* down_svh, const int* local_count, const uint32_t* local_slot,
                              const uint32_t* local_expert, int out, int64_t max_slots, const EpPeers& ep, cudaStream_t stream) {
    ep_publish_kernel<<<ep_grid(max_slots * (out / 128)), kEpWarps * 32, 0, stream>>>(raw, down_svh, local_count, local_slot, local_expert,
                                                                                     out, max_slots, ep);
    return cudaGetLastError();
}

cudaError_t launch_ep_combine(const void* scores, int score_dtype, int64_t rows, int top_k, int out, void* y, const EpPeers& ep,
                              cudaStream_t stream) {
    const unsigned grid = ep_grid(rows * (out / 128));
    if (score_dtype == kF32) ep_combine_kernel<true><<<grid, kEpWarps * 32, 0, stream>>>(scores, rows, top_k, out, y, ep);
    else ep_combine_kernel<false><<<grid, kEpWarps * 32, 0, stream>>>(scores, rows, top_k, out, y, ep);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int64_t slots = rows * top_k;
    ep_count_kernel<<<static_cast<unsigned>((slots + 255) / 256), 256, 0, stream>>>(ep.done, slots);
    return cudaGetLastError();
}

}  // namespace b200exl3
