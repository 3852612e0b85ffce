// Shared device/host helpers for the EXL3 kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200exl3 {

// dtype codes of the reference's FFI (native/src/array.rs:21-36)
constexpr int kU16 = 2;
constexpr int kU32 = 3;
constexpr int kF16 = 9;
constexpr int kF32 = 10;
constexpr int kBF16 = 12;

constexpr int kDefaultSmCount = 148;   // B200; sm_count() asks the device

// Word offset of row `tk` (16 inputs) of 128-column block `cblock` in the quad layout [tiles_n/8, tiles_k, 2, 8K, 4]:
// a row is 64K words, the rows of a block follow one another.
__host__ __device__ __forceinline__ int64_t quad_row_offset(int tk, int cblock, int tiles_k, int k) {
    return (static_cast<int64_t>(cblock) * tiles_k + tk) * (64 * k);
}

__host__ __device__ inline bool dtype_is_float(int code) { return code == kF16 || code == kF32 || code == kBF16; }
__host__ __device__ inline size_t dtype_size(int code) { return code == kF32 ? 4 : 2; }

// 2^-3.5 exactly as the reference spells it (native/shaders/exl3.metal:213)
__device__ __forceinline__ float had_scale() { return __uint_as_float(0x3db504f3u); }

__device__ __forceinline__ __half load_as_half(const void* p, int dtype, int64_t i) {
    if (dtype == kF16) return reinterpret_cast<const __half*>(p)[i];
    if (dtype == kF32) return __float2half_rn(reinterpret_cast<const float*>(p)[i]);
    return __float2half_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]));
}

// y.astype(x.dtype) then + bias, as native/src/linear.rs:990-996 orders it.
__device__ __forceinline__ void store_from_half(void* p, int dtype, int64_t i, __half v, const __half* bias, int col) {
    if (dtype == kF16) {
        reinterpret_cast<__half*>(p)[i] = bias ? __hadd_rn(v, bias[col]) : v;
    } else if (dtype == kF32) {
        float f = __half2float(v);
        reinterpret_cast<float*>(p)[i] = bias ? __fadd_rn(f, __half2float(bias[col])) : f;
    } else {
        __nv_bfloat16 b = __float2bfloat16_rn(__half2float(v));
        if (bias) b = __float2bfloat16_rn(__fadd_rn(__bfloat162float(b), __half2float(bias[col])));
        reinterpret_cast<__nv_bfloat16*>(p)[i] = b;
    }
}

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t mask, uint32_t flip) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(mask), "r"(flip));  // (a & mask) ^ flip
    return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier + bulk (TMA) copies ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking probe of a barrier phase (the answer takes a few hundred cycles: issue it well before it is needed).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll already blocks for a while in hardware) so a
// lost copy can never hang the GPU; the caller records the failure and carries on.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = 1 << 20) {
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// contiguous global -> shared copy by the TMA unit; dst, src and bytes are multiples of 16
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// cudaFuncSetAttribute is per device: remembers, per kernel instantiation, the devices it was done on.
struct PerDeviceOnce {
    bool done[64] = {};
    bool needed() const {
        int device = 0;
        return cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64 || !done[device];
    }
    void mark() {
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64) done[device] = true;
    }
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Programmatic dependent launch: let the next kernel in the stream start its preamble, and wait for
// the previous kernel's memory to be visible.  Both are no-ops for a plain launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace b200exl3
