// Stable top-k of router values, one CTA per token row (reference: native/shaders/router_topk.h:1-34,
// native/src/router.rs:28-120).  Thread t holds expert t's value; its key is the value mapped to an
// order-preserving unsigned integer (zeros of both signs compare equal, NaN ranks above everything) with the
// expert index in the low bits, so ties go to the higher index.  An expert with `above` larger keys lands in
// output slot k-1-above: the outputs are ascending, the best expert last.  Scores are the selected values,
// optionally divided by their sum; the sum runs over the slots in order in the values' own type.
#include "kernels.h"

namespace b200exl3 {

namespace {

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

template <typename T>
__global__ void __launch_bounds__(1024)
router_topk_kernel(const T* __restrict__ values, int experts, int k, int normalize, uint32_t* __restrict__ indices,
                   T* __restrict__ scores) {
    extern __shared__ unsigned long long s_keys[];                 // [experts] keys, then [k] selected values
    float* selected = reinterpret_cast<float*>(s_keys + experts);
    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x;
    unsigned long long key = 0;
    float value = 0.0f;
    if (tid < experts) {
        value = to_float(values[row * experts + tid]);
        const uint32_t bits = value == 0.0f ? 0u : __float_as_uint(value);
        const uint32_t monotonic = isnan(value) ? 0xffffffffu
                                                : bits ^ (static_cast<uint32_t>(static_cast<int32_t>(bits) >> 31) | 0x80000000u);
        key = (static_cast<unsigned long long>(monotonic) << 32) | static_cast<unsigned long long>(tid);
        s_keys[tid] = key;
    }
    __syncthreads();
    if (tid < experts) {
        int above = 0;
        for (int i = 0; i < experts; ++i) above += s_keys[i] > key;
        if (above < k) {
            const int slot = k - 1 - above;
            indices[row * k + slot] = static_cast<uint32_t>(tid);
            selected[slot] = value;
        }
    }
    __syncthreads();
    if (tid == 0) {
        T sum = from_float<T>(0.0f);
        if (normalize)
            for (int i = 0; i < k; ++i) sum = add_t(from_float<T>(selected[i]), sum);
        for (int i = 0; i < k; ++i) {
            const T score = from_float<T>(selected[i]);
            scores[row * k + i] = normalize ? div_t(score, sum) : score;
        }
    }
}

}  // namespace

cudaError_t launch_router_topk(const void* values, int dtype, int64_t rows, int experts, int k, bool normalize,
                               uint32_t* indices, void* scores, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    const int threads = (experts + 31) / 32 * 32;
    const size_t smem = static_cast<size_t>(experts) * sizeof(unsigned long long) + static_cast<size_t>(k) * sizeof(float);
    if (dtype == kF32)
        router_topk_kernel<float><<<static_cast<unsigned>(rows), threads, smem, stream>>>(
            static_cast<const float*>(values), experts, k, normalize, indices, static_cast<float*>(scores));
    else
        router_topk_kernel<__half><<<static_cast<unsigned>(rows), threads, smem, stream>>>(
            static_cast<const __half*>(values), experts, k, normalize, indices, static_cast<__half*>(scores));
    return cudaGetLastError();
}

}  // namespace b200exl3
