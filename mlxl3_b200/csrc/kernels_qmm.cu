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
//  * one CTA owns 128 output columns (the 128 lanes of tensor memory), up to 512 tokens (all 512 fp32
//    columns of tensor memory, as two halves of 256) and a contiguous range of 64-input stages
//    (split-K across CTAs), so a batch of up to 512 rows decodes every weight exactly once;
//  * A operand = decoded weights, [128 out, 64 in] fp16, K-major with the 128-byte swizzle.  One thread streams the
//    packed stages (4 tile rows x 8 tiles, contiguous in the quad layout) with bulk copies into a ring; eight
//    decoder warps each own four tiles (one interleaved quad) of one 16-input tile row of the stage, decode them
//    bit-exactly in registers (the lane's eight weights are two 4-byte pairs for rows g and g+8 of the A tile) and
//    store them with the swizzle applied;
//  * B operand = rotated activations, [256 token, 64 in] fp16 per half, K-major, loaded by one TMA
//    tensor copy per half and stage with the 128-byte swizzle (rows past the batch are zero-filled);
//    the B ring is decoupled from the A ring;
//  * one thread issues four tcgen05.mma (M=128, N=256, K=16) per half and stage and one commit per stage, which
//    frees the A stage and the B slots; in the large shape a watcher warp tests the barriers for it (one lane per
//    barrier, one instruction) and publishes a count; after the last stage the decoder warps read the accumulator
//    with tcgen05.ld and either store partial products or rotate and store the outputs.
// Every wait on an mbarrier is bounded in time; a wait that gives up sets the status word and the
// kernel still releases its tensor memory.
#include <cuda.h>

#include <algorithm>
#include <atomic>

#include "kernels.h"
#include "hadamard.cuh"
#include "tile_decode.cuh"

namespace b200exl3 {

namespace {

constexpr int kStages = 3;            // decoded A stages in flight
// packed stages (4 tile rows x 8 tiles = 1024*K bytes) in flight: a 16 KiB ring, at most 8 slots
constexpr int raw_depth(int k) { return 16 / k > 8 ? 8 : 16 / k; }
constexpr int kRawDepthMax = 8;
constexpr uint32_t kRawBytes = 16 * 1024;
constexpr int kGroupWarps = 8;        // decoder warps of a group: (tile row of the stage, quad of the 8-tile row)
// Warp roles.  The single-thread roles take the lowest warp numbers: the scheduler favours older warps, and a
// producer starved by spinning decoder warps stalls the whole pipeline.
constexpr int kMmaWarp = 0, kActWarp = 1, kWeightWarp = 2, kWatchWarp = 3, kFirstDecoder = 4;
constexpr uint32_t kAStageBytes = 128 * 128;           // 128 rows x 64 fp16

// Two shapes of the same kernel.  Large (more than 64 rows): a CTA holds up to 512 tokens (two accumulator
// halves of 256), sixteen decoder warps in two groups on alternate stages, one CTA per SM.  Small (up to 64
// rows): 64 tokens per CTA, eight decoder warps, under half of the shared memory and registers, so two CTAs
// share an SM and twice as many warps decode -- these batches are bound by the decode, not by the MMAs.
template <bool SMALL>
struct QmmShape {
    static constexpr int kTokHalf = SMALL ? 64 : 256;          // tokens per accumulator half = MMA N
    static constexpr int kMaxHalves = SMALL ? 1 : 2;
    static constexpr int kTokTile = kTokHalf * kMaxHalves;     // tokens per CTA
    static constexpr int kDecoderGroups = SMALL ? 1 : 2;       // groups of eight decoder warps that take alternate stages
    static constexpr int kDecoders = kDecoderGroups * kGroupWarps;
    static constexpr int kThreads = 32 * (kFirstDecoder + kDecoders);
    static constexpr int kMinBlocks = SMALL ? 2 : 1;
    static constexpr int kBSlots = SMALL ? 4 : 5;              // activation half-stages in flight
    static constexpr uint32_t kBSlotBytes = kTokHalf * 128;    // kTokHalf rows x 64 fp16
    static constexpr uint32_t kInstrDesc = (1u << 4)                      // D = fp32
                                           | (0u << 7) | (0u << 10)       // A, B = fp16
                                           | (0u << 15) | (0u << 16)      // both K-major
                                           | ((kTokHalf >> 3) << 17)      // N
                                           | ((128u >> 4) << 24);         // M
    static constexpr size_t kSmemBytes = kStages * kAStageBytes + kBSlots * kBSlotBytes + kRawBytes + 1024;
};

struct QmmArgs {
    const uint32_t* wq;        // quad layout
    float* partials;           // [splits, rows, out]
    unsigned int* error;
    int in, out, rows, tiles_n, splits, stages_total;   // stages_total = in / 64
    unsigned long long* trace;   // optional [CTA, 8] nanosecond stamps of the phases
    const __half* svh;           // fused output rotation (y != nullptr; one input split): [out]
    const __half* bias;          // [out] or nullptr
    void* y;                     // [rows, out] in y_dtype, or nullptr: store fp32 partial products
    int y_dtype;
    // Expert-mapped mode (map_expert != nullptr; small shape, one split, fp32 products): the `out` axis is virtual,
    // [segments, map_proj, map_blocks * 128]; segment s holds 64 padded rows that all use expert map_expert[s], whose
    // columns start at column block map_proj_index * map_stride_blocks + expert * map_blocks of the bank.
    const uint32_t* map_expert;
    const int* map_count;      // segments in use; the CTAs of later segments return at once
    int map_blocks, map_proj, map_stride_blocks, map_experts;
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
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool qmm_wait(uint64_t* bar, uint32_t parity, volatile int* cta_failed) {
    // non-blocking tests: a suspended try_wait was seen to resume long after the phase completed.
    // Reading the global timer costs about 0.2 us, so the clock only starts after many plain polls.
    for (int i = 0; i < 4096; ++i)
        if (mbar_test_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (int i = 1;; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((i & 255) == 0 && (*cta_failed || global_ns() - t0 > 250000000ull)) { *cta_failed = 1; return false; }
    }
}
__device__ __forceinline__ uint32_t ld_acquire_shared(const uint32_t* ptr) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr(ptr)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_shared(uint32_t* ptr, uint32_t v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_addr(ptr)), "r"(v) : "memory");
}
// Bounded wait of one thread until the watcher's count has passed `it` (a shared-memory load answers in tens of
// cycles, a barrier test in a few hundred).
__device__ __forceinline__ bool qmm_wait_count(const uint32_t* count, int it, volatile int* cta_failed) {
    for (int i = 0; i < 16384; ++i)
        if (ld_acquire_shared(count) > static_cast<uint32_t>(it)) return true;
    const unsigned long long t0 = global_ns();
    for (int i = 1;; ++i) {
        if (ld_acquire_shared(count) > static_cast<uint32_t>(it)) return true;
        if ((i & 255) == 0 && (*cta_failed || global_ns() - t0 > 250000000ull)) { *cta_failed = 1; return false; }
    }
}
// The same wait for a whole warp: one lane polls (32 lanes polling one barrier flood the shared-memory
// pipe that the copies, the stores and the MMA issue also need), then every lane observes the completed
// phase itself, which makes the data the barrier guards visible to it.
__device__ __forceinline__ bool qmm_wait_warp(uint64_t* bar, uint32_t parity, volatile int* cta_failed, int lane) {
    int ok = 1;
    if (lane == 0) ok = qmm_wait(bar, parity, cta_failed);
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    return mbar_test_wait(bar, parity) || qmm_wait(bar, parity, cta_failed);
}

template <int K, int CB, bool SMALL>
__global__ void __launch_bounds__(QmmShape<SMALL>::kThreads, QmmShape<SMALL>::kMinBlocks)
qmm_kernel(const __grid_constant__ CUtensorMap xmap, const QmmArgs p) {
    using S = QmmShape<SMALL>;
    // Dependent launch: this kernel may be scheduled under the tail of the kernel before it (the input rotation, the
    // glue of the expert block).  The packed weights are nobody's output, so the barriers, the tensor memory and the
    // first weight copies do not wait; what that kernel wrote -- the rotated rows, the segment table -- is read only
    // after griddepcontrol.wait (expert-mapped mode: at once, the table is read first; otherwise by the activation
    // producer before its first copy), and nothing is stored to global memory before it either (the decoders wait
    // before the epilogue).
    pdl_launch_dependents();
    if (p.map_expert != nullptr) pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kQuadWords = 32 * K;                       // four interleaved tiles
    constexpr int kRawStageWords = 8 * kQuadWords;           // 4 tile rows x 2 quads
    constexpr uint32_t kRawStageBytes = kRawStageWords * 4;
    constexpr int kRawDepth = raw_depth(K);
    __shared__ __align__(8) uint64_t full_a[kStages], done[kStages], full_b[S::kBSlots], accum_bar;
    __shared__ __align__(8) uint64_t raw_full[kRawDepthMax], raw_empty[kRawDepthMax];
    __shared__ uint32_t tmem_base_slot;
    __shared__ uint32_t s_mma_ready;      // written by the watcher warp: product stages whose operands are in place
    __shared__ volatile int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    unsigned long long* tr = p.trace ? p.trace + (blockIdx.y * gridDim.x + blockIdx.x) * 8 : nullptr;
    if (tr && threadIdx.x == 0) tr[0] = global_ns();
    const int col_blocks = p.out >> 7;
    const int cblock = blockIdx.x % col_blocks;
    const int split = blockIdx.x / col_blocks;
    const int tok0 = blockIdx.y * S::kTokTile;
    int wblock = cblock;            // column block of the weight array
    int brow0 = tok0;               // first row of the activation tile
    if (p.map_expert != nullptr) {
        const int sp = cblock / p.map_blocks, j = cblock - sp * p.map_blocks;
        const int seg = sp / p.map_proj, proj = sp - seg * p.map_proj;
        if (seg >= *p.map_count) return;                          // uniform for the CTA; nothing is allocated yet
        const int expert = static_cast<int>(min(p.map_expert[seg], static_cast<uint32_t>(p.map_experts - 1)));
        wblock = proj * p.map_stride_blocks + expert * p.map_blocks + j;
        brow0 = sp * S::kTokTile;
    }
    const int halves = (S::kMaxHalves == 2 && p.rows - tok0 > S::kTokHalf) ? 2 : 1;      // accumulator halves this CTA fills
    const uint32_t tmem_cols = halves * S::kTokHalf;
    const int st0 = static_cast<int>(static_cast<int64_t>(p.stages_total) * split / p.splits);
    const int st1 = static_cast<int>(static_cast<int64_t>(p.stages_total) * (split + 1) / p.splits);
    const int nst = st1 - st0;

    // shared memory: A stages | B slots | raw rings; the swizzled operands need 1024-byte alignment
    unsigned char* a_base = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned char* b_base = a_base + kStages * kAStageBytes;
    uint32_t* raw_base = reinterpret_cast<uint32_t*>(b_base + S::kBSlots * S::kBSlotBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_a[s], kGroupWarps); mbar_init(&done[s], 1); }
        for (int s = 0; s < S::kBSlots; ++s) mbar_init(&full_b[s], 1);
        mbar_init(&accum_bar, 1);
        for (int d = 0; d < kRawDepth; ++d) { mbar_init(&raw_full[d], 1); mbar_init(&raw_empty[d], kGroupWarps); }
        s_failed = 0;
        s_mma_ready = 0;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(&tmem_base_slot, tmem_cols);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_slot;
    if (tr && threadIdx.x == 0) tr[1] = global_ns();

    const int dec = warp - kFirstDecoder;                        // decoder index, negative for the other roles
    if (dec >= 0) {
        // ================= decoder warps: packed quad -> 16 inputs x 64 outputs of the A stage =================
        // Two groups of eight warps take alternate stages, so that one group's barrier round trips and
        // proxy fence overlap the other group's arithmetic.  Within a group: (tile row of the stage, quad).
        const int group = dec >> 3, trow = dec & 3, quad = (dec >> 2) & 1;
        const LaneGeom<K> geom(lane);
        // this warp's quad of a packed stage: input tile 4*stage + trow, output tiles 8*cblock + 4*quad .. +3
        const uint32_t* my_quad = raw_base + (trow * 2 + quad) * kQuadWords;
        // A barrier test takes a few hundred cycles to answer, so the tests for the warp's next stage are
        // issued before the current stage is decoded and their answer is only looked at afterwards.
        // Large shape: lane 0 tests the packed words and lane 1 the A stage in ONE instruction, so the warp stalls
        // once, not twice (the warp barrier below orders the other lanes' reads after the two observations).  With two
        // small CTAs per SM that was measured slower than every lane testing both.
        auto stage_ready = [&](int it) -> bool {
            if constexpr (SMALL) {
                return mbar_test_wait(&raw_full[it % kRawDepth], (it / kRawDepth) & 1u) &
                       mbar_test_wait(&done[it % kStages], ((it / kStages) & 1u) ^ 1u);
            } else {
                uint64_t* bar = lane == 0 ? &raw_full[it % kRawDepth] : &done[it % kStages];
                const uint32_t par = lane == 0 ? (it / kRawDepth) & 1u : ((it / kStages) & 1u) ^ 1u;
                bool ok = true;
                if (lane < 2) ok = mbar_test_wait(bar, par);
                return ok;
            }
        };
        bool ready = group < nst && stage_ready(group);
        for (int it = group; it < nst; it += S::kDecoderGroups) {
            const int s = it % kStages, rslot = it % kRawDepth;
            if (!__all_sync(0xffffffffu, ready)) {
                // the packed stage has landed, and the MMAs that read this A stage last time are done
                ready = qmm_wait(&raw_full[rslot], (it / kRawDepth) & 1u, &s_failed) &&
                        qmm_wait(&done[s], ((it / kStages) & 1u) ^ 1u, &s_failed);
                if (!__all_sync(0xffffffffu, ready)) break;
            }
            if constexpr (!SMALL) __syncwarp();
            unsigned char* a_stage = a_base + s * kAStageBytes;
            const uint4* qw = reinterpret_cast<const uint4*>(my_quad + rslot * kRawStageWords);
            const uint4 W2 = qw[geom.i2];
            const uint4 W1 = qw[geom.i1];
            uint4 W0 = make_uint4(0, 0, 0, 0);
            if constexpr (K >= 5) W0 = qw[geom.i0];
            const uint32_t w2[4] = {W2.x, W2.y, W2.z, W2.w}, w1[4] = {W1.x, W1.y, W1.z, W1.w},
                           w0[4] = {W0.x, W0.y, W0.z, W0.w};
            ready = it + S::kDecoderGroups < nst && stage_ready(it + S::kDecoderGroups);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a0, a1, a2, a3;
                lane_weights_exact<K, CB>(w2[j], w1[j], w0[j], geom.slack, a0, a1, a2, a3);
                // rows (= output columns) 16t+g and 16t+g+8 of the A tile; 16-byte chunks 2*trow and 2*trow+1 of
                // the row, XORed with the row index modulo 8 (the 128-byte swizzle); 4q bytes into the chunk
                const int t = quad * 4 + j;
                unsigned char* r0 = a_stage + (16 * t + g) * 128 + 4 * q;
                const int c0 = ((2 * trow) ^ g) << 4, c1 = ((2 * trow + 1) ^ g) << 4;
                *reinterpret_cast<uint32_t*>(r0 + c0) = a0;
                *reinterpret_cast<uint32_t*>(r0 + 8 * 128 + c0) = a1;
                *reinterpret_cast<uint32_t*>(r0 + c1) = a2;
                *reinterpret_cast<uint32_t*>(r0 + 8 * 128 + c1) = a3;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA unit
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&raw_empty[rslot]);                         // the packed words were consumed: slot free for this warp
                mbar_arrive(&full_a[s]);
            }
        }
        if (tr && threadIdx.x == 32 * kFirstDecoder) tr[2] = global_ns();
    } else if (warp == kActWarp) {
        // ================= activation producer: one tensor copy per half and stage =================
        if (lane < halves) {
            // Lane h copies half h: the two halves' barrier tests (a few hundred cycles each) run side by side.
            // A slot is free once the MMAs of the stage that used it last are done.
            const int h = lane;
            pdl_wait();
            for (int it = 0; it < nst && !s_failed; ++it) {
                const int u = it * halves + h, slot = u % S::kBSlots;
                const int before = u - S::kBSlots;                       // the use of this slot one lap earlier
                if (before >= 0) {
                    const int st = before / halves;
                    if (!qmm_wait(&done[st % kStages], (st / kStages) & 1u, &s_failed)) break;
                }
                mbar_expect_tx(&full_b[slot], S::kBSlotBytes);
                tma_load_2d(b_base + slot * S::kBSlotBytes, &xmap, (st0 + it) * 64, brow0 + h * S::kTokHalf, &full_b[slot]);
            }
            if (tr && lane == 0) tr[7] = global_ns();
        }
    } else if (warp == kWeightWarp) {
        // ================= weight producer: one bulk copy (4 tile rows x 8 tiles, contiguous) per stage =================
        if (lane == 0) {
            int slot = 0;
            uint32_t par = 0;
            for (int it = 0; it < nst && !s_failed; ++it) {
                if (!qmm_wait(&raw_empty[slot], par ^ 1u, &s_failed)) break;
                mbar_expect_tx(&raw_full[slot], kRawStageBytes);
                bulk_copy_g2s(raw_base + slot * kRawStageWords, p.wq + quad_row_offset(4 * (st0 + it), wblock, p.in / 16, K), kRawStageBytes,
                              &raw_full[slot]);
                if (++slot == kRawDepth) { slot = 0; par ^= 1u; }
            }
        }
    } else if (!SMALL && warp == kWatchWarp) {
        // ================= watcher: all barriers of the next product stage in ONE test instruction =================
        // A barrier test answers after a few hundred cycles and the thread that reads the answer stalls that long.
        // Up to three tests in a row per stage (A stage, one or two activation slots) cost the issuing thread more
        // time than issuing the stage's products: it, not the tensor pipe, set the pace.  Here lane 0 looks at the A
        // stage and lanes 1, 2 at the activation slots, one instruction tests them all, and the count of stages whose
        // operands are in place is published in shared memory, where the issuing thread reads it in tens of cycles.
        // (Large shape only: with two small CTAs per SM the decoders set the pace and a second polling warp costs more
        // than it saves -- measured.)
        const uint32_t mask = halves == 2 ? 7u : 3u;
        int idle = 0;
        unsigned long long t0 = 0;
        for (int it = 0; it < nst;) {
            uint64_t* bar = nullptr;
            uint32_t par = 0;
            if (lane == 0) {
                bar = &full_a[it % kStages]; par = (it / kStages) & 1u;
            } else if (lane <= halves) {
                const int u = it * halves + lane - 1;
                bar = &full_b[u % S::kBSlots]; par = (u / S::kBSlots) & 1u;
            }
            bool ok = false;
            if (bar != nullptr) ok = mbar_test_wait(bar, par);
            if ((__ballot_sync(0xffffffffu, ok) & mask) == mask) {
                ++it;
                idle = 0;
                if (lane == 0) st_release_shared(&s_mma_ready, static_cast<uint32_t>(it));
                continue;
            }
            if ((++idle & 1023) == 0) {                                   // bounded like every other wait of the kernel
                int give_up = 0;
                if (lane == 0) {
                    if (idle == 1024) t0 = global_ns();
                    give_up = s_failed || global_ns() - t0 > 250000000ull;
                    if (give_up) s_failed = 1;
                }
                if (__shfl_sync(0xffffffffu, give_up, 0)) break;
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer =================
        if (lane == 0) {
            // small shape: the thread tests the barriers itself, all tests of the next stage right after the commit
            auto stage_ready = [&](int it) -> bool {
                return mbar_test_wait(&full_a[it % kStages], (it / kStages) & 1u) &
                       mbar_test_wait(&full_b[it % S::kBSlots], (it / S::kBSlots) & 1u);
            };
            bool ready = SMALL && nst > 0 && stage_ready(0);
            for (int it = 0; it < nst && !s_failed; ++it) {
                const int s = it % kStages;
                if constexpr (SMALL) {
                    if (!ready && (!qmm_wait(&full_a[s], (it / kStages) & 1u, &s_failed) ||
                                   !qmm_wait(&full_b[it % S::kBSlots], (it / S::kBSlots) & 1u, &s_failed)))
                        break;
                } else if (!qmm_wait_count(&s_mma_ready, it, &s_failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_addr(a_base + s * kAStageBytes);
                for (int h = 0; h < halves; ++h) {
                    const uint32_t b_addr = smem_addr(b_base + ((it * halves + h) % S::kBSlots) * S::kBSlotBytes);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)                      // 4 x 16 inputs = one 64-input stage
                        umma_f16(tmem + h * S::kTokHalf, umma_desc(a_addr + kk * 32), umma_desc(b_addr + kk * 32), S::kInstrDesc,
                                 (it > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&done[s]);                                  // A stage and B slots free once these MMAs have read them
                if constexpr (SMALL) ready = it + 1 < nst && stage_ready(it + 1);
            }
            umma_commit(&accum_bar);                                    // accumulator complete
            if (tr) tr[3] = global_ns();
        }
    }

    // ================= epilogue: accumulator -> fp32 partial products =================
    if (dec >= 0) {
        pdl_wait();                                                     // returns at once: the kernel before ended long ago
        if (nst > 0) {
            qmm_wait_warp(&accum_bar, 0, &s_failed, lane);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        if (tr && threadIdx.x == 32 * kFirstDecoder) tr[4] = global_ns();
        // a warp may read the 32 lanes 32*(warp%4)..; the warps of a lane quarter share the token columns
        const int lq = warp & 3, cpart = dec >> 2;
        const int col = cblock * 128 + lq * 32 + lane;                  // this thread's output column = its TMEM lane
        float* dst = p.partials + (static_cast<int64_t>(split) * p.rows) * p.out + col;
        const int c_span = static_cast<int>(tmem_cols) / (S::kDecoders / 4);
        const int c_begin = cpart * c_span, c_end = c_begin + c_span;
        if (p.y == nullptr) {
            for (int c = c_begin; c < c_end; c += 32) {
                if (tok0 + c >= p.rows) break;
                uint32_t r[32];
                if (nst > 0) tmem_ld32(tmem + (static_cast<uint32_t>(lq * 32) << 16) + c, r);
                else
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int tok = tok0 + c + i;
                    if (tok < p.rows) dst[static_cast<int64_t>(tok) * p.out] = __uint_as_float(r[i]);
                }
            }
        } else {
            // Output rotation fused (one input split only): the four warps that share a range of token
            // columns transpose 32 tokens x 128 outputs through shared memory (the operand rings are free
            // once the accumulator is complete), then every warp rotates eight token rows:
            // half(sum) -> H128 -> * svh (+ bias), stored in the caller's dtype.
            __half* stage_base = reinterpret_cast<__half*>(b_base) + cpart * (2 * 32 * 128);
            const __half* sv = p.svh + cblock * 128 + lane * 4;
            const __half* bias = p.bias ? p.bias + cblock * 128 : nullptr;
            int buf = 0;
            for (int c = c_begin; c < c_end; c += 32) {
                if (tok0 + c >= p.rows) break;
                uint32_t r[32];
                tmem_ld32(tmem + (static_cast<uint32_t>(lq * 32) << 16) + c, r);
                __half* stage = stage_base + buf * (32 * 128);
#pragma unroll
                for (int i = 0; i < 32; ++i) stage[i * 128 + lq * 32 + lane] = __float2half_rn(__uint_as_float(r[i]));
                asm volatile("bar.sync %0, %1;" ::"r"(1 + cpart), "r"(128) : "memory");
#pragma unroll 2
                for (int j = 0; j < 8; ++j) {                            // two rows' shuffle chains in flight
                    const int t = lq * 8 + j, tok = tok0 + c + t;
                    if (tok >= p.rows) break;
                    __align__(8) __half h[4];
                    *reinterpret_cast<uint2*>(h) = *reinterpret_cast<const uint2*>(stage + t * 128 + lane * 4);
                    warp_hadamard128_f16(h, lane);
                    if (p.y_dtype == kF16) {                            // one 8-byte store per lane
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            h[e] = __hmul_rn(h[e], sv[e]);
                            if (bias) h[e] = __hadd_rn(h[e], bias[lane * 4 + e]);
                        }
                        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.y) + static_cast<int64_t>(tok) * p.out + cblock * 128 +
                                                  lane * 4) = *reinterpret_cast<const uint2*>(h);
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            store_from_half(p.y, p.y_dtype, static_cast<int64_t>(tok) * p.out + cblock * 128 + lane * 4 + e,
                                            __hmul_rn(h[e], sv[e]), bias, lane * 4 + e);
                    }
                }
                buf ^= 1;
            }
        }
    }
    if (tr && threadIdx.x == 32 * kFirstDecoder) tr[5] = global_ns();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tr && threadIdx.x == 0) tr[6] = global_ns();
    if (s_failed) {
        // copies that were still in flight when a wait gave up must land before the CTA's shared memory is released
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    if (warp == kMmaWarp) tmem_dealloc(tmem, tmem_cols);
    if (threadIdx.x == 0 && s_failed) {
        pdl_wait();
        atomicExch(p.error, 3u);
    }
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

template <int K, int CB, bool SMALL>
cudaError_t qmm_launch_shape(const CUtensorMap& map, const QmmArgs& p, dim3 grid, cudaStream_t stream) {
    using S = QmmShape<SMALL>;
    constexpr size_t smem = S::kSmemBytes;
    auto kernel = qmm_kernel<K, CB, SMALL>;
    static PerDeviceOnce attribute;                         // once per kernel and device
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        attribute.mark();
    }
    return launch_dependent(kernel, grid, dim3(S::kThreads), smem, stream, map, p);
}

template <int K, int CB>
cudaError_t qmm_launch_one(const CUtensorMap& map, const QmmArgs& p, dim3 grid, bool small, cudaStream_t stream) {
    return small ? qmm_launch_shape<K, CB, true>(map, p, grid, stream) : qmm_launch_shape<K, CB, false>(map, p, grid, stream);
}

template <int K>
cudaError_t qmm_launch_k(int cb, const CUtensorMap& map, const QmmArgs& p, dim3 grid, bool small, cudaStream_t stream) {
    if (cb == 0) return qmm_launch_one<K, 0>(map, p, grid, small, stream);
    if (cb == 1) return qmm_launch_one<K, 1>(map, p, grid, small, stream);
    return qmm_launch_one<K, 2>(map, p, grid, small, stream);
}

}  // namespace

std::atomic<unsigned long long*> g_qmm_trace{nullptr};
static std::atomic<int> g_qmm_splits{0};                              // 0 = chosen by the cost model below
void qmm_set_tuning(int splits) { g_qmm_splits = splits > 0 ? splits : 0; }

constexpr int64_t kQmmSmallMaxRows = 64;     // one token tile: a second one would decode every weight twice

QmmPlan plan_qmm(int in, int out, int64_t rows) {
    QmmPlan plan{};
    plan.small = rows <= kQmmSmallMaxRows;
    const int col_blocks = out / 128;
    const int tile = plan.small ? QmmShape<true>::kTokTile : QmmShape<false>::kTokTile;
    plan.token_tiles = static_cast<int>((rows + tile - 1) / tile);
    const int stages_total = in / 64;
    const int64_t base = static_cast<int64_t>(col_blocks) * plan.token_tiles;
    const int max_splits = std::max(1, stages_total / 8);     // every split keeps at least 8 stages
    if (const int forced = g_qmm_splits.load()) { plan.splits = std::min(forced, max_splits); return plan; }
    // CTAs that run at once: one per SM for the large shape (the operand rings take most of the shared memory),
    // two for the small one.  Estimated time of a choice: waves x (stages per CTA + fixed prologue/epilogue) + the
    // fp32 partials that several splits write and the separate output rotation reads back.
    const int64_t slots = static_cast<int64_t>(sm_count()) * (plan.small ? 2 : 1);
    const double stage_us = plan.small ? 0.55 : (rows > 256 ? 0.6 : 0.35), fixed_us = 4.0;
    const double partial_us = static_cast<double>(rows) * out * 8.0 / 8.0e6;
    double best = 0;
    for (int s = 1; s <= max_splits; ++s) {
        const int64_t waves = (base * s + slots - 1) / slots;
        // with one split the output rotation runs in the epilogue; more splits write fp32 partials and add a launch
        const double t = waves * (((stages_total + s - 1) / s) * stage_us + fixed_us) + (s > 1 ? s * partial_us + 5.0 : 0.0);
        if (s == 1 || t < best) { best = t; plan.splits = s; }
    }
    return plan;
}

size_t qmm_partial_bytes(const QmmPlan& plan, int out, int64_t rows) {
    return (static_cast<size_t>(plan.splits) * rows * out * sizeof(float) + 255) / 256 * 256;
}

cudaError_t launch_qmm(const uint32_t* wq, int in, int out, int k, int cb, const __half* xhat, int64_t rows,
                       const QmmPlan& plan, float* partials, unsigned int* error, const __half* svh, const __half* bias,
                       void* y, int y_dtype, cudaStream_t stream, int ld_tiles, int col_tile0) {
    if (in % 128 || out % 128 || rows <= 0 || col_tile0 % 8) return cudaErrorInvalidValue;
    if (ld_tiles <= 0) ld_tiles = out / 16;
    // a member of a group: its column blocks follow those of the members before it
    (void)ld_tiles;
    wq += quad_row_offset(0, col_tile0 / 8, in / 16, k);
    if (y != nullptr && plan.splits != 1) return cudaErrorInvalidValue;     // the fused rotation needs the complete sum
    EncodeFn encode = encode_fn();
    if (!encode) return cudaErrorNotSupported;
    // rotated activations [rows, in] fp16 as a 2-D tensor: boxes of 64 inputs x 256 tokens, 128-byte swizzle
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in) * sizeof(__half)};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(plan.small ? QmmShape<true>::kTokHalf : QmmShape<false>::kTokHalf)};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xhat), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    // packed weights: the four tile rows of a stage are contiguous in the quad layout, so the weight producer issues plain
    // bulk copies and needs no tensor map
    QmmArgs p{};
    p.wq = wq; p.partials = partials; p.error = error;
    p.svh = svh; p.bias = bias; p.y = y; p.y_dtype = y_dtype;
    p.in = in; p.out = out; p.rows = static_cast<int>(rows); p.tiles_n = out / 16;
    p.splits = plan.splits; p.stages_total = in / 64; p.trace = g_qmm_trace.load();
    const dim3 grid(static_cast<unsigned>((out / 128) * plan.splits), static_cast<unsigned>(plan.token_tiles));
    switch (k) {
        case 1: return qmm_launch_k<1>(cb, map, p, grid, plan.small, stream);
        case 2: return qmm_launch_k<2>(cb, map, p, grid, plan.small, stream);
        case 3: return qmm_launch_k<3>(cb, map, p, grid, plan.small, stream);
        case 4: return qmm_launch_k<4>(cb, map, p, grid, plan.small, stream);
        case 5: return qmm_launch_k<5>(cb, map, p, grid, plan.small, stream);
        case 6: return qmm_launch_k<6>(cb, map, p, grid, plan.small, stream);
        case 7: return qmm_launch_k<7>(cb, map, p, grid, plan.small, stream);
        case 8: return qmm_launch_k<8>(cb, map, p, grid, plan.small, stream);
        default: return cudaErrorInvalidValue;
    }
}


cudaError_t launch_qmm_mapped(const uint32_t* wq, int in, int width, int bank_tiles_n, int k, int cb, const __half* xhat,
                              int max_segments, int proj, int stride_blocks, int experts, const uint32_t* seg_expert,
                              const int* seg_count, float* products, unsigned int* error, cudaStream_t stream) {
    using S = QmmShape<true>;
    if (in % 128 || width % 128 || max_segments <= 0 || proj <= 0) return cudaErrorInvalidValue;
    EncodeFn encode = encode_fn();
    if (!encode) return cudaErrorNotSupported;
    const int64_t rows = static_cast<int64_t>(max_segments) * proj * S::kTokTile;   // padded activation rows
    const int out = max_segments * proj * width;                                   // virtual output width
    CUtensorMap map;
    const cuuint32_t elem[2] = {1, 1};
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in) * sizeof(__half)};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(S::kTokHalf)};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(xhat), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    QmmArgs p{};
    p.wq = wq; p.partials = products; p.error = error;
    p.in = in; p.out = out; p.rows = S::kTokTile; p.tiles_n = bank_tiles_n;
    p.splits = 1; p.stages_total = in / 64; p.trace = nullptr;
    p.map_expert = seg_expert; p.map_count = seg_count;
    p.map_blocks = width / 128; p.map_proj = proj; p.map_stride_blocks = stride_blocks; p.map_experts = experts;
    const dim3 grid(static_cast<unsigned>(out / 128), 1);
    switch (k) {
        case 1: return qmm_launch_k<1>(cb, map, p, grid, true, stream);
        case 2: return qmm_launch_k<2>(cb, map, p, grid, true, stream);
        case 3: return qmm_launch_k<3>(cb, map, p, grid, true, stream);
        case 4: return qmm_launch_k<4>(cb, map, p, grid, true, stream);
        case 5: return qmm_launch_k<5>(cb, map, p, grid, true, stream);
        case 6: return qmm_launch_k<6>(cb, map, p, grid, true, stream);
        case 7: return qmm_launch_k<7>(cb, map, p, grid, true, stream);
        case 8: return qmm_launch_k<8>(cb, map, p, grid, true, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200exl3
