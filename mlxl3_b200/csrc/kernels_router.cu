// MoE router: fp16 gate product, row softmax and stable top-k (reference behaviour: native/src/router.rs:28-120,
// native/shaders/router_topk.h:1-34, call site native/src/qwen35.rs:196-242).
//
// Contract kept bit for bit: experts are ordered by value with both zeros equal and NaN above every number, ties
// go to the higher expert index, the k winners are written in ascending order (best last), and with `normalize`
// the scores are divided by their sum, added slot by slot from slot 0 in the values' own type.
//
// Design: ONE WARP PER TOKEN ROW, several rows per CTA, no shared memory and no block barrier.  A lane keeps the
// 64-bit sort keys of experts lane, lane+32, ... in registers; the winners are peeled off one per round, each
// round a per-lane maximum below the previous winner followed by a five-step shuffle maximum.  Round r's winner
// is output slot k-1-r.  The softmax in front (fp32, as MLX's precise softmax) runs in the same registers, so
// logits -> probabilities -> routes is one pass over a row that is read once.
#include "kernels.h"

namespace b200exl3 {

namespace {

constexpr int kRouterWarps = 4;        // token rows per CTA

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
__device__ __forceinline__ float add_t(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ __half add_t(__half a, __half b) { return __hadd_rn(a, b); }
__device__ __forceinline__ float div_t(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ __half div_t(__half a, __half b) { return __float2half_rn(__fdiv_rn(__half2float(a), __half2float(b))); }

// order-preserving image of a float: -x < -0 == +0 < +x < NaN
__device__ __forceinline__ uint32_t order_bits(float v) {
    if (isnan(v)) return 0xffffffffu;
    const uint32_t b = v == 0.0f ? 0u : __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, v, d);
        v = o > v ? o : v;
    }
    return v;
}

// NJ = experts per lane (experts <= 32 * NJ).  SOFTMAX: the values are logits; route on their softmax.
template <typename T, int NJ, bool SOFTMAX>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_kernel(const T* __restrict__ values, int64_t rows, int experts, int k, int normalize, uint32_t* __restrict__ indices,
              T* __restrict__ scores, T* __restrict__ probabilities) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRouterWarps + (threadIdx.x >> 5);
    if (row >= rows) return;                                      // whole warps leave together
    const T* in = values + row * experts;
    T held[NJ];                                                    // the value that is ranked and reported
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        held[j] = e < experts ? in[e] : from_float<T>(0.0f);
    }
    if constexpr (SOFTMAX) {
        // fp32 softmax of the row, rounded to the values' type: exp(x - max) * (1 / sum)
        float top = -INFINITY;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j < experts) top = fmaxf(top, to_float(held[j]));
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, d));
        float ex[NJ], sum = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            ex[j] = lane + 32 * j < experts ? expf(to_float(held[j]) - top) : 0.0f;
            sum += ex[j];
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        const float inv = 1.0f / sum;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            held[j] = from_float<T>(ex[j] * inv);
            if (probabilities != nullptr && lane + 32 * j < experts) probabilities[row * experts + lane + 32 * j] = held[j];
        }
    }
    unsigned long long key[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        const int e = lane + 32 * j;
        // experts beyond the row get key 0, below every real key (a real key has a non-zero order image or index)
        key[j] = e < experts ? (static_cast<unsigned long long>(order_bits(to_float(held[j]))) << 32) | static_cast<unsigned>(e) + 1ull
                             : 0ull;
    }
    // keys carry index + 1 so that expert 0 with the smallest value still beats the padding key 0
    unsigned long long bound = ~0ull;
    uint32_t* out_i = indices + row * k;
    T* out_s = scores + row * k;
    for (int r = 0; r < k; ++r) {
        unsigned long long best = 0;
        T best_v = from_float<T>(0.0f);
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (key[j] < bound && key[j] > best) { best = key[j]; best_v = held[j]; }
        const unsigned long long winner = warp_max_u64(best);
        if (best == winner) {                                      // keys are unique: exactly one lane
            out_i[k - 1 - r] = static_cast<uint32_t>(winner & 0xffffffffull) - 1u;
            out_s[k - 1 - r] = best_v;
        }
        bound = winner;
    }
    if (!normalize) return;
    __syncwarp();                                                  // the winners' stores, before any lane reads them back
    T sum = from_float<T>(0.0f);
    for (int i = 0; i < k; ++i) sum = add_t(out_s[i], sum);        // every lane: the same sequential sum
    T mine[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j)
        if (lane + 32 * j < k) mine[j] = out_s[lane + 32 * j];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < NJ; ++j)
        if (lane + 32 * j < k) out_s[lane + 32 * j] = div_t(mine[j], sum);
}

template <typename T, bool SOFTMAX>
cudaError_t launch_router(const T* values, int64_t rows, int experts, int k, bool normalize, uint32_t* indices, T* scores,
                          T* probabilities, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>((rows + kRouterWarps - 1) / kRouterWarps);
    const int per_lane = (experts + 31) / 32;
#define B200_ROUTER_CASE(NJ)                                                                                             \
    if (per_lane <= NJ) {                                                                                                \
        router_kernel<T, NJ, SOFTMAX><<<grid, kRouterWarps * 32, 0, stream>>>(values, rows, experts, k, normalize, indices, \
                                                                               scores, probabilities);                   \
        return cudaGetLastError();                                                                                       \
    }
    B200_ROUTER_CASE(1)
    B200_ROUTER_CASE(2)
    B200_ROUTER_CASE(4)
    B200_ROUTER_CASE(8)
    B200_ROUTER_CASE(16)
    B200_ROUTER_CASE(32)
#undef B200_ROUTER_CASE
    return cudaErrorInvalidValue;
}

// logits[row, e] = half(sum_i float(x[row, i]) * float(w[e, i])): one warp owns one expert for up to eight token
// rows at a time, so a weight row is read once per eight tokens; fp32 accumulation, lanes combined by shuffles.
constexpr int kGateRows = 8;
__global__ void __launch_bounds__(128)
router_gate_kernel(const void* __restrict__ x, int x_dtype, const __half* __restrict__ w, int64_t rows, int in, int experts,
                   __half* __restrict__ logits) {
    const int lane = threadIdx.x & 31;
    const int expert = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (expert >= experts) return;
    const int64_t row0 = static_cast<int64_t>(blockIdx.y) * kGateRows;
    const int n = rows - row0 < kGateRows ? static_cast<int>(rows - row0) : kGateRows;
    float acc[kGateRows] = {};
    const __half* wr = w + static_cast<int64_t>(expert) * in;
    for (int i = lane * 2; i < in; i += 64) {
        const float2 wv = __half22float2(*reinterpret_cast<const __half2*>(wr + i));
#pragma unroll
        for (int r = 0; r < kGateRows; ++r)
            if (r < n) {
                const int64_t at = (row0 + r) * in + i;
                acc[r] = fmaf(__half2float(load_as_half(x, x_dtype, at)), wv.x, acc[r]);
                acc[r] = fmaf(__half2float(load_as_half(x, x_dtype, at + 1)), wv.y, acc[r]);
            }
    }
#pragma unroll
    for (int r = 0; r < kGateRows; ++r) {
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], d);
        if (lane == 0 && r < n) logits[(row0 + r) * experts + expert] = __float2half_rn(acc[r]);
    }
}

}  // namespace

cudaError_t launch_router_topk(const void* values, int dtype, int64_t rows, int experts, int k, bool normalize, bool softmax,
                               uint32_t* indices, void* scores, void* probabilities, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    if (dtype == kF32) {
        auto v = static_cast<const float*>(values);
        auto s = static_cast<float*>(scores);
        auto p = static_cast<float*>(probabilities);
        return softmax ? launch_router<float, true>(v, rows, experts, k, normalize, indices, s, p, stream)
                       : launch_router<float, false>(v, rows, experts, k, normalize, indices, s, p, stream);
    }
    auto v = static_cast<const __half*>(values);
    auto s = static_cast<__half*>(scores);
    auto p = static_cast<__half*>(probabilities);
    return softmax ? launch_router<__half, true>(v, rows, experts, k, normalize, indices, s, p, stream)
                   : launch_router<__half, false>(v, rows, experts, k, normalize, indices, s, p, stream);
}

cudaError_t launch_router_gate(const void* x, int x_dtype, const __half* w, int64_t rows, int in, int experts, __half* logits,
                               cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    const dim3 grid(static_cast<unsigned>((experts + 3) / 4), static_cast<unsigned>((rows + kGateRows - 1) / kGateRows));
    router_gate_kernel<<<grid, 128, 0, stream>>>(x, x_dtype, w, rows, in, experts, logits);
    return cudaGetLastError();
}

}  // namespace b200exl3
