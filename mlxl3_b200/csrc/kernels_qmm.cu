// Tensor-core product for many activation rows (prefill, verify batches): decode trellis tiles into
// shared memory and feed tcgen05.mma with the accumulator in tensor memory.
//
// Reference behaviour replaced: native/shaders/_qmm_tensor_shared_kernel.metal (decode a weight tile
// once, share it across row groups, matrix-unit product with fp32 accumulation) driven by
// native/src/linear.rs:1874-2081.  Output here: fp32 partial products partials[split, row, n], which
// the output-rotation kernel sums and rotates (the reference stores the raw product and finishes it
// in native/src/linear.rs:1940-1963).
//
// Mapping.  The product is computed transposed, D[out, token] = W^T[out, in] . Xhat^T[in, token]:
//  * one CTA owns 128 output columns (the 128 lanes of tensor memory), up to 256 tokens (256 fp32
//    columns of tensor memory) and a contiguous range of 64-input stages (split-K across CTAs);
//  * A operand = decoded weights, [128 out, 64 in] fp16, K-major with the 128-byte swizzle.  Four
//    decoder warps each own one 16-input tile row of the stage: a warp streams its packed row with
//    TMA bulk copies into its own ring, decodes the eight tiles bit-exactly in registers (the lane's
//    eight weights are two 4-byte pairs for rows g and g+8 of the A tile) and stores them with the
//    swizzle applied (conflict-free);
//  * B operand = rotated activations, [256 token, 64 in] fp16, K-major, loaded by one TMA tensor copy
//    per stage with the 128-byte swizzle (rows past the batch are zero-filled by the copy);
//  * one thread issues four tcgen05.mma (M=128, N=256, K=16) per stage and commits the stage back to
//    the producers; after the last stage the decoder warps read the accumulator with tcgen05.ld and
//    store the partial products.
// Every wait on an mbarrier is bounded; a wait that gives up sets the status word and the kernel still
// releases its tensor memory.
#include <cuda.h>

#include <algorithm>

#include "kernels.h"
#include "tile_decode.cuh"

namespace b200exl3 {

namespace {

constexpr int kStages = 4;            // A/B stages in flight
constexpr int kRawDepth = 3;          // packed rows in flight per decoder warp
constexpr int kTokTile = 256;         // tokens per CTA = MMA N
constexpr int kDecoders = 4;          // decoder warps (= 16-input tile rows per stage)
constexpr int kThreads = 32 * (kDecoders + 2);
constexpr uint32_t kAStageBytes = 128 * 128;           // 128 rows x 64 fp16
constexpr uint32_t kBStageBytes = kTokTile * 128;      // 256 rows x 64 fp16

struct QmmArgs {
    const uint32_t* wq;        // quad layout
    float* partials;           // [splits, rows, out]
    unsigned int* error;
    int in, out, rows, tiles_n, splits, stages_total;   // stages_total = in / 64
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
    // K-major operand, 128-byte swizzle: 8-row groups 1024 bytes apart, descriptor version 1
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_byte_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;                 // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                 // version
    d |= static_cast<uint64_t>(2) << 61;                 // SWIZZLE_128B
    return d;
}

constexpr uint32_t kInstrDesc = (1u << 4)                      // D = fp32
                                | (0u << 7) | (0u << 10)       // A, B = fp16
                                | (0u << 15) | (0u << 16)      // both K-major
                                | ((kTokTile >> 3) << 17)      // N
                                | ((128u >> 4) << 24);         // M

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_dst)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t taddr, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Wait that gives up after about a quarter of a second, or at once when another role of the CTA has
// already given up, so that a lost copy or a miscounted barrier ends the kernel instead of hanging it.
__device__ __forceinline__ bool qmm_wait(uint64_t* bar, uint32_t parity, volatile int* cta_failed) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (int i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 0 && (*cta_failed || global_ns() - t0 > 250000000ull)) { *cta_failed = 1; return false; }
    }
}

template <int K, int CB>
__global__ void __launch_bounds__(kThreads, 1)
qmm_kernel(const __grid_constant__ CUtensorMap xmap, const QmmArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kRowWords = 64 * K;                        // one 8-tile row of packed words
    constexpr uint32_t kRowBytes = kRowWords * 4;
    __shared__ __align__(8) uint64_t full_a[kStages], full_b[kStages], empty[kStages], accum_bar;
    __shared__ __align__(8) uint64_t raw_bar[kDecoders][kRawDepth];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int col_blocks = p.out >> 7;
    const int cblock = blockIdx.x % col_blocks;
    const int split = blockIdx.x / col_blocks;
    const int tok0 = blockIdx.y * kTokTile;
    const int st0 = static_cast<int>(static_cast<int64_t>(p.stages_total) * split / p.splits);
    const int st1 = static_cast<int>(static_cast<int64_t>(p.stages_total) * (split + 1) / p.splits);
    const int nst = st1 - st0;

    // shared memory: A stages | B stages | raw rings; the swizzled stages need 1024-byte alignment
    unsigned char* a_base = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned char* b_base = a_base + kStages * kAStageBytes;
    uint32_t* raw_base = reinterpret_cast<uint32_t*>(b_base + kStages * kBStageBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_a[s], kDecoders); mbar_init(&full_b[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&accum_bar, 1);
        for (int w = 0; w < kDecoders; ++w)
            for (int d = 0; d < kRawDepth; ++d) mbar_init(&raw_bar[w][d], 1);
        s_failed = 0;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kDecoders + 1) tmem_alloc(&tmem_base_slot, kTokTile);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;

    if (warp < kDecoders) {
        // ================= decoder warps: packed row -> 16 x 128 slice of the A stage =================
        const LaneGeom<K> geom(lane);
        uint32_t* ring = raw_base + static_cast<size_t>(warp) * kRawDepth * kRowWords;
        const size_t row_stride = static_cast<size_t>(p.tiles_n) * (32 * K);
        // this warp's rows: input tile 4*stage + warp, for stage = st0 .. st1-1
        const char* next_src = reinterpret_cast<const char*>(
            p.wq + (static_cast<int64_t>(4 * st0 + warp) * p.tiles_n + cblock * 8) * (8 * K));
        if (lane == 0)
            for (int d = 0; d < kRawDepth; ++d)
                if (d < nst) {
                    mbar_expect_tx(&raw_bar[warp][d], kRowBytes);
                    bulk_copy_g2s(ring + d * kRowWords, next_src + static_cast<size_t>(d) * 4 * row_stride, kRowBytes, &raw_bar[warp][d]);
                }
        next_src += static_cast<size_t>(kRawDepth) * 4 * row_stride;
        int rslot = 0;
        uint32_t rparity = 0;
        for (int it = 0; it < nst; ++it) {
            const int s = it % kStages;
            const uint32_t par = (it / kStages) & 1u;
            // the MMAs that read this stage are done, and this warp's packed row has landed
            const bool ready = qmm_wait(&empty[s], par ^ 1u, &s_failed) && qmm_wait(&raw_bar[warp][rslot], rparity, &s_failed);
            if (!__all_sync(0xffffffffu, ready)) break;
            unsigned char* a_stage = a_base + s * kAStageBytes;
            const uint32_t* row_words = ring + rslot * kRowWords;
#pragma unroll
            for (int quad = 0; quad < 2; ++quad) {
                const uint4* qw = reinterpret_cast<const uint4*>(row_words + quad * (32 * K));
                const uint4 W2 = qw[geom.i2];
                const uint4 W1 = qw[geom.i1];
                uint4 W0 = make_uint4(0, 0, 0, 0);
                if constexpr (K >= 5) W0 = qw[geom.i0];
                const uint32_t w2[4] = {W2.x, W2.y, W2.z, W2.w}, w1[4] = {W1.x, W1.y, W1.z, W1.w},
                               w0[4] = {W0.x, W0.y, W0.z, W0.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t a0, a1, a2, a3;
                    lane_weights_exact<K, CB>(w2[j], w1[j], w0[j], geom.slack, a0, a1, a2, a3);
                    // rows (= output columns) 16t+g and 16t+g+8 of the A tile; 16-byte chunks 2w and 2w+1 of
                    // the row, XORed with the row index modulo 8 (the 128-byte swizzle); 4q bytes into the chunk
                    const int t = quad * 4 + j;
                    unsigned char* r0 = a_stage + (16 * t + g) * 128 + 4 * q;
                    const int c0 = ((2 * warp) ^ g) << 4, c1 = ((2 * warp + 1) ^ g) << 4;
                    *reinterpret_cast<uint32_t*>(r0 + c0) = a0;
                    *reinterpret_cast<uint32_t*>(r0 + 8 * 128 + c0) = a1;
                    *reinterpret_cast<uint32_t*>(r0 + c1) = a2;
                    *reinterpret_cast<uint32_t*>(r0 + 8 * 128 + c1) = a3;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA unit
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&full_a[s]);
                if (it + kRawDepth < nst) {
                    mbar_expect_tx(&raw_bar[warp][rslot], kRowBytes);
                    bulk_copy_g2s(ring + rslot * kRowWords, next_src, kRowBytes, &raw_bar[warp][rslot]);
                }
            }
            next_src += 4 * row_stride;
            if (++rslot == kRawDepth) { rslot = 0; rparity ^= 1u; }
        }
    } else if (warp == kDecoders) {
        // ================= activation producer: one tensor copy per stage =================
        if (lane == 0) {
            for (int it = 0; it < nst; ++it) {
                const int s = it % kStages;
                const uint32_t par = (it / kStages) & 1u;
                if (!qmm_wait(&empty[s], par ^ 1u, &s_failed)) break;
                mbar_expect_tx(&full_b[s], kBStageBytes);
                tma_load_2d(b_base + s * kBStageBytes, &xmap, (st0 + it) * 64, tok0, &full_b[s]);
            }
        }
    } else {
        // ================= MMA issuer =================
        if (lane == 0) {
            for (int it = 0; it < nst; ++it) {
                const int s = it % kStages;
                const uint32_t par = (it / kStages) & 1u;
                if (!qmm_wait(&full_a[s], par, &s_failed)) break;
                if (!qmm_wait(&full_b[s], par, &s_failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(a_base + s * kAStageBytes), b_addr = smem_addr(b_base + s * kBStageBytes);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)                          // 4 x 16 inputs = one 64-input stage
                    umma_f16(tmem, umma_desc(a_addr + kk * 32), umma_desc(b_addr + kk * 32), kInstrDesc, (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&empty[s]);                                 // stage free once these MMAs have read it
            }
            umma_commit(&accum_bar);                                    // accumulator complete
        }
    }

    // ================= epilogue: accumulator -> fp32 partial products =================
    if (warp < kDecoders) {
        if (nst > 0) {
            qmm_wait(&accum_bar, 0, &s_failed);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const int col = cblock * 128 + warp * 32 + lane;                // this thread's output column = its TMEM lane
        float* dst = p.partials + (static_cast<int64_t>(split) * p.rows) * p.out + col;
        for (int c = 0; c < kTokTile; c += 32) {
            if (tok0 + c >= p.rows) break;
            uint32_t r[32];
            if (nst > 0) tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + c, r);
            else
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int tok = tok0 + c + i;
                if (tok < p.rows) dst[static_cast<int64_t>(tok) * p.out] = __uint_as_float(r[i]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_failed) {
        // copies that were still in flight when a wait gave up must land before the CTA's shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    if (warp == kDecoders + 1) tmem_dealloc(tmem, kTokTile);
    if (threadIdx.x == 0 && s_failed) atomicExch(p.error, 3u);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeFn>(ptr);
    }
    return fn;
}

template <int K, int CB>
cudaError_t qmm_launch_one(const CUtensorMap& map, const QmmArgs& p, dim3 grid, size_t smem, cudaStream_t stream) {
    auto kernel = qmm_kernel<K, CB>;
    static bool attribute_set = false;
    if (!attribute_set) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attribute_set = true;
    }
    kernel<<<grid, kThreads, smem, stream>>>(map, p);
    return cudaGetLastError();
}

template <int K>
cudaError_t qmm_launch_k(int cb, const CUtensorMap& map, const QmmArgs& p, dim3 grid, size_t smem, cudaStream_t stream) {
    if (cb == 0) return qmm_launch_one<K, 0>(map, p, grid, smem, stream);
    if (cb == 1) return qmm_launch_one<K, 1>(map, p, grid, smem, stream);
    return qmm_launch_one<K, 2>(map, p, grid, smem, stream);
}

}  // namespace

static int g_qmm_waves = 1;
void qmm_set_tuning(int waves) { if (waves > 0) g_qmm_waves = waves; }

QmmPlan plan_qmm(int in, int out, int64_t rows) {
    QmmPlan plan{};
    const int col_blocks = out / 128;
    plan.token_tiles = static_cast<int>((rows + kTokTile - 1) / kTokTile);
    const int stages_total = in / 64;
    const int64_t base = static_cast<int64_t>(col_blocks) * plan.token_tiles;
    // split the input range so that the CTAs fill the 148 SMs g_qmm_waves times (one CTA per SM: the
    // stages take most of the shared memory); every split keeps at least 8 stages
    int splits = static_cast<int>((static_cast<int64_t>(kSmCount) * g_qmm_waves + base / 2) / base);
    splits = std::max(1, std::min(splits, std::max(1, stages_total / 8)));
    plan.splits = splits;
    return plan;
}

size_t qmm_partial_bytes(const QmmPlan& plan, int out, int64_t rows) {
    return (static_cast<size_t>(plan.splits) * rows * out * sizeof(float) + 255) / 256 * 256;
}

cudaError_t launch_qmm(const uint32_t* wq, int in, int out, int k, int cb, const __half* xhat, int64_t rows,
                       const QmmPlan& plan, float* partials, unsigned int* error, cudaStream_t stream) {
    if (in % 128 || out % 128 || rows <= 0) return cudaErrorInvalidValue;
    EncodeFn encode = encode_fn();
    if (!encode) return cudaErrorNotSupported;
    // rotated activations [rows, in] fp16 as a 2-D tensor: boxes of 64 inputs x 256 tokens, 128-byte swizzle
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in) * sizeof(__half)};
    const cuuint32_t box[2] = {64, kTokTile};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xhat), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    QmmArgs p{};
    p.wq = wq; p.partials = partials; p.error = error;
    p.in = in; p.out = out; p.rows = static_cast<int>(rows); p.tiles_n = out / 16;
    p.splits = plan.splits; p.stages_total = in / 64;
    const dim3 grid(static_cast<unsigned>((out / 128) * plan.splits), static_cast<unsigned>(plan.token_tiles));
    const size_t smem = kStages * (kAStageBytes + kBStageBytes) + static_cast<size_t>(kDecoders) * kRawDepth * 64 * 8 * 4 + 1024;
    switch (k) {
        case 1: return qmm_launch_k<1>(cb, map, p, grid, smem, stream);
        case 2: return qmm_launch_k<2>(cb, map, p, grid, smem, stream);
        case 3: return qmm_launch_k<3>(cb, map, p, grid, smem, stream);
        case 4: return qmm_launch_k<4>(cb, map, p, grid, smem, stream);
        case 5: return qmm_launch_k<5>(cb, map, p, grid, smem, stream);
        case 6: return qmm_launch_k<6>(cb, map, p, grid, smem, stream);
        case 7: return qmm_launch_k<7>(cb, map, p, grid, smem, stream);
        case 8: return qmm_launch_k<8>(cb, map, p, grid, smem, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200exl3
