// A whole decode step of EXL3 linear layers in ONE persistent launch.
//
// Reference behaviour replaced: a decode step of the reference is a recorded sequence of per-layer dispatches
// (replay object, native/ffi/mlx_bridge.cpp:150-175); its own measurements name the dispatch count, not the bytes,
// as what a step costs (the input-rotation note at native/src/linear.rs:855-861 and the fused prologue kernels exist
// for that reason).  Here the sequence itself is one kernel: a table of layers in device memory, walked by a grid
// of one wave of CTAs that stays resident for the whole step.
//
// What stays from the per-layer kernel (kernels_qmv_impl.cuh): the warp-level stream-K partition of every layer,
// the per-warp TMA ring, the register decode and the mma.sync product, the reduction of a column block inside the
// CTA and across CTAs in a fixed order, the output rotation by the warp that holds the complete sum.
// What changes:
//  * the weight stream never stops at a layer boundary: a warp's ring is refilled from a cursor that runs through
//    its rows of ALL layers, so while a layer's last blocks are being reduced and the next layer's activations are
//    not ready yet, that next layer's packed words are already on their way into shared memory (weights depend on
//    nothing);
//  * the layer boundary is a counter, not a kernel boundary: the warp that stores a finished column block adds one
//    to the layer's count with a release; a warp that needs the next layer's activations waits until the count of
//    the layer before it is complete (one warp per CTA polls global memory with acquire loads, the others watch a
//    shared-memory word), bounded in time -- when a wait gives up the status word is set and everybody carries on,
//    so a lost signal ends the kernel instead of hanging the GPU;
//  * CTAs that share a column block meet through one acq_rel atomic instead of two fences and an atomic.
// The counters are zero when the kernel starts and the last CTA to leave sets them back to zero.
#pragma once

#include "kernels_qmv_impl.cuh"

namespace b200exl3 {

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int atom_acq_rel_gpu_add(unsigned int* p, unsigned int v) {
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ int ld_acquire_cta_shared(const int* p) {
    int v;
    asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_addr(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_cta_shared(int* p, int v) {
    asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_addr(p)), "r"(v) : "memory");
}

// this warp's units [w0, w1) of a layer with T units shared by `warps` warps (warps beyond that have none)
struct StackRange {
    int w0, w1;
};
__device__ __forceinline__ int stack_unit_begin(int T, int warps, int wid, bool narrow) {
    if (wid >= warps) return T;
    return narrow ? static_cast<int>(static_cast<unsigned int>(T) * static_cast<unsigned int>(wid) / static_cast<unsigned int>(warps))
                  : static_cast<int>(static_cast<unsigned long long>(T) * wid / warps);
}

// Where a warp's weight stream stands: the row (8 tiles of one 128-column block and 16 inputs) that is copied next.
// The sequence is: for every layer, for every column block the warp has units in, the block's rows in order -- the
// order in which the warp consumes them.
template <int K>
struct StackCursor {
    int op, cblock, tk, tk_last, w1, UB;
    const char* src;
    size_t stride;
    bool valid;

    __device__ __forceinline__ void segment(const StackOp& o, int w0) {
        const int u0 = max(w0, cblock * UB) - cblock * UB;
        const int u1 = min(w1, (cblock + 1) * UB) - cblock * UB;
        tk = u0 >> 3;
        tk_last = (u1 - 1) >> 3;
        stride = static_cast<size_t>(o.tiles_n) * (32 * K);
        src = reinterpret_cast<const char*>(o.wq + (static_cast<int64_t>(tk) * o.tiles_n + cblock * 8) * (8 * K));
    }
    // first layer at or after `first` in which the warp has work
    __device__ __forceinline__ void seek(const StackOp* ops, int n_ops, int first, int wid) {
        valid = false;
        for (op = first; op < n_ops; ++op) {
            const StackOp& o = ops[op];
            UB = o.tiles_k * 8;
            const int T = UB * o.col_blocks;
            const int w0 = stack_unit_begin(T, o.warps, wid, o.narrow != 0);
            w1 = stack_unit_begin(T, o.warps, wid + 1, o.narrow != 0);
            if (w1 > w0) {
                cblock = w0 / UB;
                segment(o, w0);
                valid = true;
                return;
            }
        }
    }
    __device__ __forceinline__ void next(const StackOp* ops, int n_ops, int wid) {
        if (tk < tk_last) {
            ++tk;
            src += stride;
        } else if ((cblock + 1) * UB < w1) {
            ++cblock;
            segment(ops[op], cblock * UB);          // a later block of the range starts at its first unit
        } else {
            seek(ops, n_ops, op + 1, wid);
        }
    }
};

// Makes sure every layer before `op` is complete before this warp reads activations.  One warp of the CTA polls
// the previous layer's count in global memory; the others wait for the shared word it sets.
__device__ __forceinline__ void stack_wait(const StackArgs& a, int op, int* s_ready, unsigned int* s_poller, int lane) {
    if (op > 0 && lane == 0 && ld_acquire_cta_shared(s_ready) < op) {
        const unsigned int target = static_cast<unsigned int>(a.ops[op - 1].col_blocks);
        const unsigned int* count = a.op_done + (op - 1);
        unsigned long long t0 = 0;
#pragma unroll 1
        for (int i = 0;; ++i) {
            if (ld_acquire_cta_shared(s_ready) >= op) break;
            if (atomicCAS(s_poller, 0u, 1u) == 0u) {
                if (ld_acquire_cta_shared(s_ready) < op) {
                    bool ok = false;
#pragma unroll 1
                    for (int j = 0;; ++j) {
                        if (ld_acquire_gpu(count) >= target) { ok = true; break; }
                        if ((j & 31) == 31) {
                            if (t0 == 0) t0 = global_ns();
                            if (*reinterpret_cast<volatile unsigned int*>(a.error) != 0 || global_ns() - t0 > a.wait_ns) break;
                        }
                        __nanosleep(32);
                    }
                    if (!ok) atomicCAS(a.error, 0u, 5u);
                    st_release_cta_shared(s_ready, op);
                }
                atomicExch(s_poller, 0u);
                break;
            }
            __nanosleep(64);
            if ((i & 255) == 255) {                       // the poller is bounded; this bounds a waiter on its own as well
                if (t0 == 0) t0 = global_ns();
                if (global_ns() - t0 > 2 * a.wait_ns) { atomicCAS(a.error, 0u, 5u); break; }
            }
        }
    }
    __syncwarp();
}

// Activations of input 128-blocks [kb0, kb0 + nblk) of every row, rotated into the warp's shared memory.  As
// qmv_rotate_chunk, but the activations are read from L2 (another SM wrote them a moment ago).
__device__ __forceinline__ void stack_rotate_chunk(const void* x, int x_dtype, const __half* suh, int in, int rows, int kb0,
                                                   int nblk, __half* xs, int lane) {
    constexpr int kXsHalves = kQmvXBlocks * 128;
    const int total = rows * nblk;
    auto fetch = [&](int unit, uint2& sv, __half (&xv)[4]) {
        const int row = unit / nblk, blk = unit - row * nblk;
        const int col = (kb0 + blk) * 128 + lane * 4;
        sv = *reinterpret_cast<const uint2*>(suh + col);
        const int64_t at = static_cast<int64_t>(row) * in + col;
        if (x_dtype == kF16) {
            const uint2 v = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(x) + at));
            *reinterpret_cast<uint2*>(xv) = v;
        } else if (x_dtype == kF32) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + at));
            xv[0] = __float2half_rn(v.x); xv[1] = __float2half_rn(v.y); xv[2] = __float2half_rn(v.z); xv[3] = __float2half_rn(v.w);
        } else {
            const uint2 v = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + at));
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) xv[j] = __float2half_rn(__bfloat162float(b[j]));
        }
    };
    uint2 sv_next;
    __align__(8) __half xv_next[4];
    fetch(0, sv_next, xv_next);
#pragma unroll 1
    for (int unit = 0; unit < total; ++unit) {
        const uint2 sv = sv_next;
        __align__(8) __half h[4];
        const __half* sc = reinterpret_cast<const __half*>(&sv);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(xv_next[j], sc[j]);
        if (unit + 1 < total) fetch(unit + 1, sv_next, xv_next);
        warp_hadamard128_f16(h, lane);
        const int row = unit / nblk, blk = unit - row * nblk;
        *reinterpret_cast<uint2*>(xs + row * kXsHalves + blk * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
    }
    __syncwarp();
}

__device__ __forceinline__ int stack_group_of(const StackOp& o, int cblock) {
    int grp = 0;
#pragma unroll 1
    while (grp + 1 < o.groups && cblock * 128 >= o.gcol0[grp + 1]) ++grp;
    return grp;
}

// The last warp of a CTA to stage its tile of column block `cblock`: adds the CTA's staged tiles in warp order,
// meets the other CTAs of the block in global memory (the last one adds the pieces in piece order), and whoever
// holds the complete sum exchanges it with the other ranks (row shard), rotates, stores, and counts the block as done.
__device__ __forceinline__ void stack_finish_block(const StackArgs& a, const StackOp& o, int op, int cblock, unsigned int warp_mask,
                                                   unsigned int second_mask, int pieces, int piece, const unsigned char* smem_base,
                                                   int lane) {
    const int rows = a.rows;
    const int tile_floats = rows * 128;
    float* partials = a.partials[op & 1];
    unsigned int* counters = a.counters[op & 1];
    const float* piece_base = partials + static_cast<int64_t>(cblock) * o.max_pieces * tile_floats;
    float* piece_dst = partials + (static_cast<int64_t>(cblock) * o.max_pieces + piece) * tile_floats;
    const int stage_floats = rows * kQmvRedStride;
#pragma unroll 1
    for (int pass = 0; pass < (pieces > 1 ? 2 : 1); ++pass) {
        if (pass == 1) {
            __syncwarp();                                       // every lane's piece stores, before lane 0's release
            unsigned int prev = 0;
            if (lane == 0) prev = atom_acq_rel_gpu_add(counters + cblock, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev != static_cast<unsigned int>(pieces - 1)) return;       // not the last CTA of this block
            if (lane == 0) counters[cblock] = 0;                // ready for the next layer that uses this slot
        }
        const bool complete = pass == 1 || pieces == 1;
#pragma unroll 1
        for (int row = 0; row < rows; ++row) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (pass == 0) {
                bool any = false;
#pragma unroll 1
                for (int w = 0; w < kQmvWarps; ++w) {
                    if (!((warp_mask >> w) & 1u)) continue;
                    const float4 t4 = *reinterpret_cast<const float4*>(
                        reinterpret_cast<const float*>(smem_base + static_cast<size_t>(w) * a.warp_smem + a.stage_offset) +
                        ((second_mask >> w) & 1u) * stage_floats + row * kQmvRedStride + lane * 4);
                    if (!any) { v = t4; any = true; }
                    else { v.x = __fadd_rn(v.x, t4.x); v.y = __fadd_rn(v.y, t4.y); v.z = __fadd_rn(v.z, t4.z); v.w = __fadd_rn(v.w, t4.w); }
                }
            } else {
                const float* src = piece_base + row * 128 + lane * 4;
                v = __ldcg(reinterpret_cast<const float4*>(src));
#pragma unroll 1
                for (int s0 = 1; s0 < pieces; s0 += 4) {
                    float4 part[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (s0 + j < pieces) part[j] = __ldcg(reinterpret_cast<const float4*>(src + (s0 + j) * tile_floats));
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (s0 + j < pieces) {
                            v.x = __fadd_rn(v.x, part[j].x); v.y = __fadd_rn(v.y, part[j].y);
                            v.z = __fadd_rn(v.z, part[j].z); v.w = __fadd_rn(v.w, part[j].w);
                        }
                }
            }
            if (!complete) {
                __stcg(reinterpret_cast<float4*>(piece_dst + row * 128 + lane * 4), v);
                continue;
            }
            const int col = cblock * 128 + lane * 4;
            if (o.tp_unit0 >= 0) v = tp_exchange_unit(a.tp, o.tp_unit0 + row * o.col_blocks + cblock, v, lane);
            __half h[4] = {__float2half_rn(v.x), __float2half_rn(v.y), __float2half_rn(v.z), __float2half_rn(v.w)};
            warp_hadamard128_f16(h, lane);
            __align__(8) __half sv[4];
            *reinterpret_cast<uint2*>(sv) = *reinterpret_cast<const uint2*>(o.svh + col);
            const int grp = stack_group_of(o, cblock);
            const int gcol = col - o.gcol0[grp];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                store_from_half(o.gy[grp], a.y_dtype, static_cast<int64_t>(row) * o.gout[grp] + gcol + j, __hmul_rn(h[j], sv[j]),
                                o.bias ? o.bias + (col - gcol) : nullptr, gcol + j);
        }
    }
    // the block's outputs are stored: count it (release: the stores of every lane come before the count)
    __syncwarp();
    if (lane == 0) red_release_gpu_add(a.op_done + op, 1u);
}

template <int K, int CB, int MODE>
__global__ void __launch_bounds__(kQmvWarps * 32, 2)
stack_kernel(const StackArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = kQmvWarps;
    constexpr int DEPTH = stack_depth(K);
    constexpr int kRowWords = 64 * K;
    constexpr uint32_t kRowBytes = kRowWords * 4;
    constexpr int kXsHalves = kQmvXBlocks * 128;
    constexpr int NB = 1;
    __shared__ __align__(8) uint64_t s_bar[WARPS][DEPTH];
    __shared__ unsigned int s_arrived[WARPS + 2];
    __shared__ int s_ready;
    __shared__ unsigned int s_poller;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int rows = a.rows;
    const int wid = static_cast<int>(blockIdx.x) * WARPS + warp;

    unsigned char* mine = smem_raw + static_cast<size_t>(warp) * a.warp_smem;
    uint32_t* ring = reinterpret_cast<uint32_t*>(mine);
    __half* xs = reinterpret_cast<__half*>(mine + a.xs_offset);
    const int stage_floats = rows * kQmvRedStride;
    uint64_t* bars = s_bar[warp];
    const LaneGeom<K> geom(lane);
    const bool tracing = a.trace != nullptr && threadIdx.x == 0;
    if (tracing) a.trace[blockIdx.x * 4 + 0] = global_ns();

    if (threadIdx.x < WARPS + 2) s_arrived[threadIdx.x] = 0;
    if (threadIdx.x == 0) { s_ready = 0; s_poller = 0; }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) mbar_init(bars + i, 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ---- start the weight stream: the first DEPTH rows of this warp, whatever layers they belong to ----------
    StackCursor<K> cur;
    cur.seek(a.ops, a.n_ops, 0, wid);
#pragma unroll 1
    for (int i = 0; i < DEPTH && cur.valid; ++i) {
        if (lane == 0) {
            mbar_expect_tx(bars + i, kRowBytes);
            bulk_copy_g2s(ring + i * kRowWords, cur.src, kRowBytes, bars + i);
        }
        cur.next(a.ops, a.n_ops, wid);
    }
    pdl_wait();                                   // the step's inputs come from whatever ran before in the stream

    int slot = 0;
    uint32_t parity = 0;
    bool copy_lost = false;

#pragma unroll 1
    for (int op = 0; op < a.n_ops; ++op) {
        const StackOp& o = a.ops[op];
        const int UB = o.tiles_k * 8;
        const int T = UB * o.col_blocks;
        const bool narrow = o.narrow != 0;
        const int w0 = stack_unit_begin(T, o.warps, wid, narrow);
        const int w1 = stack_unit_begin(T, o.warps, wid + 1, narrow);
        if (w1 <= w0) continue;
        if (w1 - w0 > UB) {                                     // the planner guarantees this; never run past two blocks
            if (lane == 0) atomicCAS(a.error, 0u, 2u);
            break;
        }
        bool waited = false;
#pragma unroll 1
        for (int cblock = w0 / UB; cblock * UB < w1; ++cblock) {
            const int u0 = max(w0, cblock * UB) - cblock * UB;
            const int u1 = min(w1, (cblock + 1) * UB) - cblock * UB;
            float* stage = reinterpret_cast<float*>(mine + a.stage_offset) + (cblock - w0 / UB) * stage_floats;
            const int grp = stack_group_of(o, cblock);
            {
                const int tk_first = u0 >> 3, tk_last = (u1 - 1) >> 3;
                const int lo_first = u0 & 7, hi_last = ((u1 - 1) & 7) + 1;
                float acc[8][NB][4];
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[t][0][i] = 0.0f;

#pragma unroll 1
                for (int tk0 = tk_first; tk0 <= tk_last;) {
                    const int kb0 = tk0 >> 3;
                    const int tk_end = min(tk_last + 1, (kb0 + kQmvXBlocks) * 8);
                    const int nrows = tk_end - tk0;
                    if (!waited) {
                        stack_wait(a, op, &s_ready, &s_poller, lane);
                        waited = true;
                    }
                    stack_rotate_chunk(o.x, a.x_dtype, o.suh + static_cast<int64_t>(grp) * o.in, o.in, rows, kb0,
                                       ((tk_end - 1) >> 3) - kb0 + 1, xs, lane);
                    const uint32_t* xfrag =
                        reinterpret_cast<const uint32_t*>(xs + min(g, rows - 1) * kXsHalves + (tk0 * 16 - kb0 * 128)) + q;
#pragma unroll 1
                    for (int r = 0; r < nrows; ++r) {
                        const int tk = tk0 + r;
                        uint32_t bx[NB][4];
                        uint32_t p0 = xfrag[r * 8], p1 = xfrag[r * 8 + 4];
                        if (g >= rows) { p0 = 0; p1 = 0; }
                        if constexpr (MODE == 0) {
                            bx[0][0] = prmt(p0, p0, 0x1010); bx[0][1] = prmt(p0, p0, 0x3232);
                            bx[0][2] = prmt(p1, p1, 0x1010); bx[0][3] = prmt(p1, p1, 0x3232);
                        } else {
                            bx[0][0] = p0; bx[0][1] = p1; bx[0][2] = 0; bx[0][3] = 0;
                        }
                        if (!mbar_wait(bars + slot, parity)) copy_lost = true;
                        const uint32_t* row_words = ring + slot * kRowWords;
                        const int lo = tk == tk_first ? lo_first : 0, hi = tk == tk_last ? hi_last : 8;
                        if (lo == 0 && hi == 8) qmv_row<K, CB, NB, MODE, true>(row_words, geom, 0, 8, bx, acc);
                        else qmv_row<K, CB, NB, MODE, false>(row_words, geom, lo, hi, bx, acc);
                        __syncwarp();                           // every lane has read the slot
                        if (cur.valid) {
                            if (lane == 0) {
                                mbar_expect_tx(bars + slot, kRowBytes);
                                bulk_copy_g2s(ring + slot * kRowWords, cur.src, kRowBytes, bars + slot);
                            }
                            cur.next(a.ops, a.n_ops, wid);
                        }
                        if (++slot == DEPTH) { slot = 0; parity ^= 1u; }
                    }
                    tk0 = tk_end;
                }
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                        if (row < rows) stage[row * kQmvRedStride + col] = acc[t][0][i];
                    }
            }

            // ---- the last warp of the CTA to arrive at this block adds the CTA's tiles and carries the block on ----
            // unit ranges of the CTA's warps: lane w holds the begin of warp w (lane 8: the end of warp 7)
            const int my_b = lane <= WARPS ? stack_unit_begin(T, o.warps, static_cast<int>(blockIdx.x) * WARPS + lane, narrow) : 0;
            const int next_b = __shfl_down_sync(0xffffffffu, my_b, 1);
            const bool has = lane < WARPS && min(next_b, (cblock + 1) * UB) > max(my_b, cblock * UB);
            const unsigned int mask = __ballot_sync(0xffffffffu, has);
            const unsigned int second = __ballot_sync(0xffffffffu, has && my_b / UB != cblock);
            const int cta0 = __shfl_sync(0xffffffffu, my_b, 0);
            unsigned int prev = 0;
            if (lane == 0) {
                __threadfence_block();                          // the staged tile before the arrival
                prev = atomicAdd(&s_arrived[cblock - cta0 / UB], 1u);
            }
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev + 1 == static_cast<unsigned int>(__popc(mask))) {
                __threadfence_block();
                if (lane == 0) s_arrived[cblock - cta0 / UB] = 0;         // the next layer's arrivals start from zero
                const int Wop = o.warps;
                const int i_first = narrow ? static_cast<int>(((static_cast<unsigned int>(cblock * UB + 1) * Wop - 1u) / T) / WARPS)
                                           : static_cast<int>((((static_cast<int64_t>(cblock) * UB + 1) * Wop - 1) / T) / WARPS);
                const int i_last = narrow ? static_cast<int>(((static_cast<unsigned int>((cblock + 1) * UB) * Wop - 1u) / T) / WARPS)
                                          : static_cast<int>(((static_cast<int64_t>(cblock + 1) * UB * Wop - 1) / T) / WARPS);
                stack_finish_block(a, o, op, cblock, mask, second, i_last - i_first + 1, static_cast<int>(blockIdx.x) - i_first,
                                   smem_raw, lane);
            }
        }
    }
    if (copy_lost && lane == 0) atomicCAS(a.error, 0u, 1u);
    if (tracing) a.trace[blockIdx.x * 4 + 1] = global_ns();

    // ---- the last CTA to leave puts the step's counters back to zero ----------------------------------------
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int left = atomicAdd(a.exit_count, 1u);
        if (left == gridDim.x - 1) {
            for (int i = 0; i < a.n_ops; ++i) a.op_done[i] = 0;
            *a.exit_count = 0;
            __threadfence();
        }
    }
}

template <int K, int CB, int MODE>
cudaError_t stack_launch_one(const StackArgs& a, const StackPlan& plan, cudaStream_t stream) {
    auto kernel = stack_kernel<K, CB, MODE>;
    static PerDeviceOnce attribute;
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQmvMaxSmemBytes);
        if (e != cudaSuccess) return e;
        attribute.mark();
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
    cfg.blockDim = dim3(kQmvWarps * 32);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;              // every CTA resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = plan.cooperative ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

template <int K>
cudaError_t stack_launch_k(const StackArgs& a, int cb, bool exact, const StackPlan& plan, cudaStream_t stream) {
    if (cb == 2) return stack_launch_one<K, 2, 1>(a, plan, stream);
    if (cb == 0) return exact ? stack_launch_one<K, 0, 1>(a, plan, stream) : stack_launch_one<K, 0, 0>(a, plan, stream);
    return exact ? stack_launch_one<K, 1, 1>(a, plan, stream) : stack_launch_one<K, 1, 0>(a, plan, stream);
}

}  // namespace b200exl3
