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
//  * CTAs that share a column block meet without any fence: partial sums travel as 8-byte {value, tag} words (the
//    tag names the launch and the layer), which the block's first CTA polls and adds in piece order;
//  * one CTA of 12 warps per SM (three per scheduler, up to 170 registers each): warps of one age advance evenly,
//    a column block is shared by fewer CTAs, and the decode loop gets the registers it wants.
// The layer counts are zero when the kernel starts and the last CTA to leave sets them back to zero and advances the
// launch number the tags are made of.
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

// an 8-byte word {value, tag}: written and read as one 64-bit scalar access, so value and tag are seen together
__device__ __forceinline__ void st_flagged(unsigned long long* p, uint32_t value, uint32_t tag) {
    const unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | value;
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_flagged(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// This warp's units [w0, w1) of a layer with T units (tiles, column-block-major) shared by `warps` warps (warps beyond
// that have none).  The layer is dealt out in whole rows of 8 tiles: a warp never shares a row with another warp, so
// no row is copied twice and no row is decoded tile by tile with a test per tile (with tile-exact shares every warp
// touched one row more than it owned tiles for, and the layer waited for the warps with two partial rows).
// `mode` bit 0: the products fit 32 bits; bit 1: every column block is dealt to a whole number of warps (block c gets
// warps [c W / C, (c + 1) W / C), which share its rows evenly), so no warp's range runs from one block into the next.
// The planner picks that whenever it does not raise the largest share: a warp that crosses a block boundary stages and
// arrives twice and rotates activations twice, and was measured to finish 1-2.4 us after the others of its layer.
__device__ __forceinline__ int stack_unit_begin(int T, int warps, int wid, int mode, int col_blocks) {
    if (wid >= warps) return T;
    const unsigned int rows = static_cast<unsigned int>(T) >> 3;
    if (mode & 2) {
        const unsigned int C = static_cast<unsigned int>(col_blocks), W = static_cast<unsigned int>(warps), w = static_cast<unsigned int>(wid);
        const unsigned int c = ((w + 1u) * C - 1u) / W;                        // the block of this warp
        const unsigned int first = c * W / C, count = (c + 1u) * W / C - first;
        const unsigned int rb = rows / C;
        return 8 * static_cast<int>(c * rb + rb * (w - first) / count);
    }
    return 8 * ((mode & 1) ? static_cast<int>(rows * static_cast<unsigned int>(wid) / static_cast<unsigned int>(warps))
                           : static_cast<int>(static_cast<unsigned long long>(rows) * wid / warps));
}

// Where a warp's weight stream stands: the chunk (up to R consecutive rows of one 128-column block; a row is 8 tiles
// and 16 inputs) that is copied next.  The sequence is: for every layer, for every column block the warp has units in,
// the block's rows in order -- the order in which the warp consumes them.  The rows of a block are contiguous in
// memory, so a chunk is ONE bulk copy; chunks are counted from the first row of the warp's range in the block, which
// is how the consumer finds their boundaries again.
template <int K, int R>
struct StackCursor {
    int op, cblock, tk, tk_last, w1, UB;
    const char* src;
    bool valid;

    __device__ __forceinline__ int rows() const { return min(R, tk_last - tk + 1); }
    __device__ __forceinline__ void segment(const StackOpLite& o, int w0) {
        const int u0 = max(w0, cblock * UB) - cblock * UB;
        const int u1 = min(w1, (cblock + 1) * UB) - cblock * UB;
        tk = u0 >> 3;
        tk_last = (u1 - 1) >> 3;
        src = reinterpret_cast<const char*>(o.wq + quad_row_offset(tk, cblock, o.tiles_k, K));
    }
    // first layer at or after `first` in which the warp has work
    __device__ __forceinline__ void seek(const StackOpLite* ops, int n_ops, int first, int wid) {
        valid = false;
#pragma unroll 1
        for (op = first; op < n_ops; ++op) {
            const StackOpLite& o = ops[op];
            UB = o.tiles_k * 8;
            const int T = UB * o.col_blocks;
            const int w0 = stack_unit_begin(T, o.warps, wid, o.narrow, o.col_blocks);
            w1 = stack_unit_begin(T, o.warps, wid + 1, o.narrow, o.col_blocks);
            if (w1 > w0) {
                cblock = w0 / UB;
                segment(o, w0);
                valid = true;
                return;
            }
        }
    }
    __device__ __forceinline__ void next(const StackOpLite* ops, int n_ops, int wid) {
        if (tk + R <= tk_last) {
            tk += R;
            src += R * (256 * K);
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
__device__ __forceinline__ void stack_wait(const StackArgs& a, int op, int prev_blocks, int* s_ready, unsigned int* s_poller, int lane) {
    if (op > 0 && lane == 0 && ld_acquire_cta_shared(s_ready) < op) {
        const unsigned int target = static_cast<unsigned int>(prev_blocks);
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

// Input scales of 128-blocks [kb0, kb0 + nblk) for this lane's four columns of each block.  They do not depend on
// the previous layer, so they are fetched before the layer-boundary wait.
__device__ __forceinline__ void stack_fetch_scales(const __half* suh, int kb0, int nblk, int lane, uint2 (&sv)[kQmvXBlocks]) {
#pragma unroll
    for (int b = 0; b < kQmvXBlocks; ++b)
        if (b < nblk) sv[b] = __ldg(reinterpret_cast<const uint2*>(suh + (kb0 + b) * 128 + lane * 4));
}

// Activations of input 128-blocks [kb0, kb0 + nblk) of every row, rotated into the warp's shared memory:
// xs[row][blk][128] = H128(half(half(x) * suh)).  The activations are read from L2 (another SM wrote them a moment
// ago), and all loads of a row are issued before the first butterfly, so a row costs one memory round trip.
__device__ __forceinline__ void stack_rotate_chunk(const void* x, int x_dtype, const uint2 (&sv)[kQmvXBlocks], int in, int rows,
                                                   int kb0, int nblk, int kXsHalves, __half* xs, int lane) {
#pragma unroll 1
    for (int row = 0; row < rows; ++row) {
        const int64_t at = static_cast<int64_t>(row) * in + kb0 * 128 + lane * 4;
        uint2 raw[kQmvXBlocks];
        if (x_dtype == kF32) {
#pragma unroll
            for (int b = 0; b < kQmvXBlocks; ++b)
                if (b < nblk) {
                    const float4 wide = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + at + b * 128));
                    const __half2 lo = __floats2half2_rn(wide.x, wide.y), hi = __floats2half2_rn(wide.z, wide.w);
                    raw[b] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                }
        } else {
#pragma unroll
            for (int b = 0; b < kQmvXBlocks; ++b)
                if (b < nblk) raw[b] = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + at + b * 128));
            if (x_dtype == kBF16) {
#pragma unroll
                for (int b = 0; b < kQmvXBlocks; ++b)
                    if (b < nblk) {
                        const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&raw[b]);
                        const __half2 lo = __floats2half2_rn(__bfloat162float(v[0]), __bfloat162float(v[1]));
                        const __half2 hi = __floats2half2_rn(__bfloat162float(v[2]), __bfloat162float(v[3]));
                        raw[b] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                    }
            }
        }
#pragma unroll
        for (int b = 0; b < kQmvXBlocks; ++b)
            if (b < nblk) {
                __align__(8) __half h[4];
                const __half* xv = reinterpret_cast<const __half*>(&raw[b]);
                const __half* sc = reinterpret_cast<const __half*>(&sv[b]);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __hmul_rn(xv[j], sc[j]);
                warp_hadamard128_f16(h, lane);
                *reinterpret_cast<uint2*>(xs + row * kXsHalves + b * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
            }
    }
    __syncwarp();
}

// The same rotation with an operator fused in front of the input scales (fp16 steps; the arithmetic of the per-layer
// kernel's prologues, statement by statement): kind 3 = RMSNorm of the input row from the sums of squares per 128-block
// that the layer before left (the row's 1 / rms is added up by every warp from those 32-112 floats, in a fixed order);
// kind 2 = SwiGLU, x = gate rows and aux = up rows.  All loads of a row go out before the first use.
__device__ __forceinline__ void stack_rotate_chunk_fused(const StackOp& f, const uint2 (&sv)[kQmvXBlocks], int rows, int kb0, int nblk,
                                                         int kXsHalves, __half* xs, int lane) {
    const __half* x = reinterpret_cast<const __half*>(f.x);
    constexpr int kBatch = 3;                                  // blocks whose loads are in flight together (registers)
#pragma unroll 1
    for (int row = 0; row < rows; ++row) {
        float inv = 0.0f;
        if (f.prologue == 3) {
            float acc = 0.0f;
            for (int b = lane; b < (f.in >> 7); b += 32) acc += __ldcg(f.pro_sumsq + row * (f.in >> 7) + b);
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
            inv = rsqrtf(acc / static_cast<float>(f.in) + f.pro_eps);
        }
#pragma unroll
        for (int b0 = 0; b0 < kQmvXBlocks; b0 += kBatch) {
            if (b0 >= nblk) break;
            const int64_t at = static_cast<int64_t>(row) * f.in + (kb0 + b0) * 128 + lane * 4;
            uint2 raw[kBatch], aux[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b)
                if (b0 + b < nblk) {
                    raw[b] = __ldcg(reinterpret_cast<const uint2*>(x + at + b * 128));
                    aux[b] = f.prologue == 3 ? __ldg(reinterpret_cast<const uint2*>(f.pro_weight + (kb0 + b0 + b) * 128 + lane * 4))
                                             : __ldcg(reinterpret_cast<const uint2*>(f.pro_aux + at + b * 128));
                }
#pragma unroll
            for (int b = 0; b < kBatch; ++b)
                if (b0 + b < nblk) {
                    const __half2* xh = reinterpret_cast<const __half2*>(&raw[b]);
                    const __half2* ah = reinterpret_cast<const __half2*>(&aux[b]);
                    __half2 v[2];
                    if (f.prologue == 3) {
                        const float2 f0 = __half22float2(xh[0]), f1 = __half22float2(xh[1]);
                        v[0] = __hmul2_rn(ah[0], __floats2half2_rn(f0.x * inv, f0.y * inv));
                        v[1] = __hmul2_rn(ah[1], __floats2half2_rn(f1.x * inv, f1.y * inv));
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const float2 g = __half22float2(xh[j]);
                            const __half2 sg = __floats2half2_rn(1.0f / (1.0f + expf(-g.x)), 1.0f / (1.0f + expf(-g.y)));
                            v[j] = __hmul2_rn(__hmul2_rn(xh[j], sg), ah[j]);
                        }
                    }
                    const __half2* sh = reinterpret_cast<const __half2*>(&sv[b0 + b]);
                    __align__(8) __half h[4];
                    *reinterpret_cast<__half2*>(h) = __hmul2_rn(v[0], sh[0]);
                    *reinterpret_cast<__half2*>(h + 2) = __hmul2_rn(v[1], sh[1]);
                    warp_hadamard128_f16(h, lane);
                    *reinterpret_cast<uint2*>(xs + row * kXsHalves + (b0 + b) * 128 + lane * 4) = *reinterpret_cast<uint2*>(h);
                }
        }
    }
    __syncwarp();
}

__device__ __forceinline__ int stack_group_of(const StackOp& o, int cblock) {
    int grp = 0;
#pragma unroll 1
    while (grp + 1 < o.groups && cblock * 128 >= o.gcol0[grp + 1]) ++grp;
    return grp;
}

// The last warp of a CTA to stage its tile of column block `cblock`: adds the CTA's staged tiles in warp order and
// meets the other CTAs of the block in global memory: every CTA but the block's first publishes its sum as tagged
// words, the first CTA collects them and adds them in piece order.  The warp that holds the complete sum exchanges
// it with the other ranks (row shard), rotates, stores, and counts the block as done.  Everything the last steps need
// from memory (output scales, bias, the output pointer of a grouped layer) is requested at the start, so that the
// chain of memory round trips is: pieces out, pieces in, result out.
template <bool FUSED>
__device__ __forceinline__ void stack_finish_block(const StackArgs& a, const StackOpLite& o, int op, int cblock,
                                                   unsigned int warp_mask, unsigned int second_mask, int pieces, int piece,
                                                   uint32_t tag, const unsigned char* smem_base, int lane) {
    const int rows = a.rows;
    const int tile_floats = rows * 128;
    const int stage_floats = rows * kQmvRedStride;
    const int col = cblock * 128 + lane * 4;
    unsigned long long* stamp = a.trace != nullptr && lane == 0 ? a.trace + (static_cast<size_t>(op) * gridDim.x + blockIdx.x) * kStackTraceSlots : nullptr;
    if (stamp) stamp[4] = global_ns();
    // requested now, used at the very end
    const uint2 sv2 = __ldg(reinterpret_cast<const uint2*>(o.svh + col));
    uint2 bias2 = make_uint2(0u, 0u);
    if (o.bias != nullptr) bias2 = __ldg(reinterpret_cast<const uint2*>(o.bias + col));
    void* y = o.y0;
    int gout = o.gout0, gcol = col;
    if (o.groups > 1) {
        const StackOp& full = a.ops[op];
        const int grp = stack_group_of(full, cblock);
        y = full.gy[grp];
        gout = full.gout[grp];
        gcol = col - full.gcol0[grp];
    }
    float4 v[kStackMaxRows];
#pragma unroll
    for (int row = 0; row < kStackMaxRows; ++row) {
        v[row] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < rows) {
            bool any = false;
#pragma unroll 1
            for (int w = 0; w < kStackWarps; ++w) {
                if (!((warp_mask >> w) & 1u)) continue;
                const float4 t4 = *reinterpret_cast<const float4*>(
                    reinterpret_cast<const float*>(smem_base + static_cast<size_t>(w) * a.warp_smem + a.stage_offset) +
                    ((second_mask >> w) & 1u) * stage_floats + row * kQmvRedStride + lane * 4);
                if (!any) { v[row] = t4; any = true; }
                else {
                    v[row].x = __fadd_rn(v[row].x, t4.x); v[row].y = __fadd_rn(v[row].y, t4.y);
                    v[row].z = __fadd_rn(v[row].z, t4.z); v[row].w = __fadd_rn(v[row].w, t4.w);
                }
            }
        }
    }
    if (pieces > 1) {
        // CTAs that share the block meet without a fence or an atomic: every partial sum travels in an 8-byte word
        // together with this layer's tag (one store publishes it), and the block's first CTA polls the others' words.
        unsigned long long* words = a.piece_words[op & 1] + (static_cast<int64_t>(cblock) * o.max_pieces + piece) * tile_floats + lane;
        if (piece != 0) {
#pragma unroll
            for (int row = 0; row < kStackMaxRows; ++row)
                if (row < rows) {
                    const float f[4] = {v[row].x, v[row].y, v[row].z, v[row].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) st_flagged(words + row * 128 + j * 32, __float_as_uint(f[j]), tag);   // word j of all lanes: one coalesced store
                }
            if (stamp) stamp[5] = global_ns();
            return;
        }
        if (stamp) stamp[5] = global_ns();
        unsigned long long t0 = 0;
        bool lost = false;
        constexpr int kBatch = 4;                                // pieces polled together: one memory round trip per batch
#pragma unroll 1
        for (int row = 0; row < rows; ++row) {
#pragma unroll 1
            for (int p0 = 1; p0 < pieces; p0 += kBatch) {
                const unsigned long long* src = words + static_cast<int64_t>(p0) * tile_floats + row * 128;
                unsigned long long w[kBatch][4];
#pragma unroll 1
                for (int i = 0;; ++i) {
                    bool ok = true;
#pragma unroll
                    for (int b = 0; b < kBatch; ++b)
                        if (p0 + b < pieces) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) w[b][j] = ld_flagged(src + static_cast<int64_t>(b) * tile_floats + j * 32);
                        }
#pragma unroll
                    for (int b = 0; b < kBatch; ++b)
                        if (p0 + b < pieces) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) ok = ok && static_cast<uint32_t>(w[b][j] >> 32) == tag;
                        }
                    if (__all_sync(0xffffffffu, ok)) break;
                    if ((i & 63) == 63) {
                        if (t0 == 0) t0 = global_ns();
                        if (*reinterpret_cast<volatile unsigned int*>(a.error) != 0 || global_ns() - t0 > a.wait_ns) { lost = true; break; }
                    }
                }
#pragma unroll
                for (int b = 0; b < kBatch; ++b)
                    if (p0 + b < pieces) {
                        const float4 part = make_float4(__uint_as_float(static_cast<uint32_t>(w[b][0])), __uint_as_float(static_cast<uint32_t>(w[b][1])),
                                                        __uint_as_float(static_cast<uint32_t>(w[b][2])), __uint_as_float(static_cast<uint32_t>(w[b][3])));
#pragma unroll
                        for (int r = 0; r < kStackMaxRows; ++r)
                            if (r == row) {
                                v[r].x = __fadd_rn(v[r].x, part.x); v[r].y = __fadd_rn(v[r].y, part.y);
                                v[r].z = __fadd_rn(v[r].z, part.z); v[r].w = __fadd_rn(v[r].w, part.w);
                            }
                    }
            }
        }
        if (lost && lane == 0) atomicCAS(a.error, 0u, 6u);
    }
    if (stamp) stamp[6] = global_ns();
    const __half* sv = reinterpret_cast<const __half*>(&sv2);
    const __half* bias = o.bias != nullptr ? reinterpret_cast<const __half*>(&bias2) : nullptr;
#pragma unroll
    for (int row = 0; row < kStackMaxRows; ++row)
        if (row < rows) {
            float4 s = v[row];
            if (o.tp_unit0 >= 0) s = tp_exchange_unit(a.tp, o.tp_unit0 + row * o.col_blocks + cblock, s, lane);
            __half h[4] = {__float2half_rn(s.x), __float2half_rn(s.y), __float2half_rn(s.z), __float2half_rn(s.w)};
            warp_hadamard128_f16(h, lane);
            if (a.y_dtype == kF16) {                            // one 8-byte store per lane
                __align__(8) __half out[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    out[j] = __hmul_rn(h[j], sv[j]);
                    if (bias) out[j] = __hadd_rn(out[j], bias[j]);
                }
                if (FUSED && o.epilogue == 1) {
                    // residual add and the block's sum of squares for the next RMSNorm (fixed shuffle order)
                    const StackOp& f = a.ops[op];
                    const int64_t at = static_cast<int64_t>(row) * f.out + col;
                    const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(f.epi_residual + at));
                    const __half* rh = reinterpret_cast<const __half*>(&rv);
                    float sq = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        out[j] = __hadd_rn(rh[j], out[j]);
                        const float v1 = __half2float(out[j]);
                        sq = fmaf(v1, v1, sq);
                    }
                    *reinterpret_cast<uint2*>(f.epi_sum + at) = *reinterpret_cast<const uint2*>(out);
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
                    if (lane == 0) f.epi_sumsq[row * (f.out >> 7) + cblock] = sq;
                    continue;
                }
                if (FUSED && o.epilogue == 2) {
                    // [q | k | v] with 128-wide heads: this block is one head.  Rotary embedding of q and k heads (pairs
                    // (i, i + 64): lane L holds columns 4L..4L+3, its partner is lane L ^ 16); keys and values go straight
                    // into row `pos` of the caches.
                    const StackOp& f = a.ops[op];
                    const int grp = stack_group_of(f, cblock);
                    int pos = __ldg(f.epi_pos);
                    pos = pos < 0 ? 0 : (pos >= f.epi_max_ctx ? f.epi_max_ctx - 1 : pos);
                    if (grp < 2) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float mine = __half2float(out[j]);
                            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                            const int i = (lane & 15) * 4 + j;
                            const float inv_freq = exp2f(-f.epi_log2_theta * static_cast<float>(2 * i) / 128.0f);
                            float sn, cs;
                            sincosf(static_cast<float>(pos) * inv_freq, &sn, &cs);
                            const float a0 = lane < 16 ? mine : other, b0 = lane < 16 ? other : mine;
                            out[j] = __float2half_rn(lane < 16 ? a0 * cs - b0 * sn : a0 * sn + b0 * cs);
                        }
                    }
                    __half* dst = grp == 0 ? reinterpret_cast<__half*>(f.gy[0]) + gcol
                                           : (grp == 1 ? f.epi_k_cache : f.epi_v_cache) +
                                                 (static_cast<int64_t>(gcol >> 7) * f.epi_max_ctx + pos) * 128 + lane * 4;
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(out);
                    continue;
                }
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(y) + static_cast<int64_t>(row) * gout + gcol) =
                    *reinterpret_cast<const uint2*>(out);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    store_from_half(y, a.y_dtype, static_cast<int64_t>(row) * gout + gcol + j, __hmul_rn(h[j], sv[j]), bias, j);
            }
        }
    // the block's outputs are stored: count it (release: the stores of every lane come before the count)
    __syncwarp();
    if (lane == 0) red_release_gpu_add(a.op_done + op, 1u);
    if (stamp) stamp[7] = global_ns();
}

// B fragments of one row of 16 inputs from the lane's two activation words: split-halves mode multiplies every
// activation by both halves of a weight, so each activation appears twice.
template <int MODE>
__device__ __forceinline__ void stack_fragment(uint32_t p0, uint32_t p1, uint32_t (&bx)[4]) {
    if constexpr (MODE == 0) {
        bx[0] = prmt(p0, p0, 0x1010); bx[1] = prmt(p0, p0, 0x3232);
        bx[2] = prmt(p1, p1, 0x1010); bx[3] = prmt(p1, p1, 0x3232);
    } else {
        bx[0] = p0; bx[1] = p1; bx[2] = 0; bx[3] = 0;
    }
}

// FUSED: the step contains layers with a fused prologue or epilogue.  A kernel of its own, so that the plain step keeps
// its registers (with that code compiled in, the plain step spilled and ran 11 % slower).
template <int K, int CB, int MODE, bool FUSED>
__global__ void __launch_bounds__(kStackWarps * 32, kStackCtasPerSm)
stack_kernel(const StackArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int WARPS = kStackWarps;
    constexpr int R = stack_chunk_rows(K);                    // rows per bulk copy
    constexpr int SLOTS = kStackSlots;                         // chunks in flight per warp
    constexpr int kRowWords = 64 * K;
    constexpr uint32_t kRowBytes = kRowWords * 4;
    const int kXsHalves = a.x_blocks * 128;
    constexpr int NB = 1;
    __shared__ __align__(8) uint64_t s_bar[WARPS][SLOTS];
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
    // the fields of every layer that the stream cursor and the main loop need, staged once
    StackOpLite* lite = reinterpret_cast<StackOpLite*>(smem_raw + a.table_offset);
    for (int i = threadIdx.x; i < a.n_ops; i += blockDim.x) {
        const StackOp& o = a.ops[i];
        StackOpLite l;
        l.wq = o.wq; l.x = o.x; l.suh = o.suh;
        l.tiles_k = o.tiles_k; l.tiles_n = o.tiles_n; l.col_blocks = o.col_blocks; l.warps = o.warps; l.narrow = o.narrow;
        l.in = o.in; l.groups = o.groups; l.max_pieces = o.max_pieces; l.tp_unit0 = o.tp_unit0; l.gout0 = o.gout[0];
        l.svh = o.svh; l.bias = o.bias; l.y0 = o.gy[0];
        l.prologue = o.prologue; l.epilogue = o.epilogue;
        lite[i] = l;
    }
    if (threadIdx.x < WARPS + 2) s_arrived[threadIdx.x] = 0;
    if (threadIdx.x == 0) { s_ready = 0; s_poller = 0; }
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < SLOTS; ++i) mbar_init(bars + i, 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ---- start the weight stream: the first chunks of this warp, whatever layers they belong to ---------------
    StackCursor<K, R> cur;
    cur.seek(lite, a.n_ops, 0, wid);
    auto refill = [&](int s) {                    // the next chunk of the stream into chunk slot s
        if (lane == 0) {
            const uint32_t bytes = static_cast<uint32_t>(cur.rows()) * kRowBytes;
            mbar_expect_tx(bars + s, bytes);
            bulk_copy_g2s(ring + s * (R * kRowWords), cur.src, bytes, bars + s);
        }
        cur.next(lite, a.n_ops, wid);
    };
#pragma unroll 1
    for (int i = 0; i < SLOTS && cur.valid; ++i) refill(i);
    pdl_wait();                                   // the step's inputs come from whatever ran before in the stream
    // tags of this launch: the launch number (advanced by the last CTA to leave) and the layer
    const uint32_t tag_base = *reinterpret_cast<volatile unsigned int*>(a.launch) * 4096u;

    int slot = 0;
    uint32_t parity = 0;
    bool copy_lost = false;
    bool ready = false;                           // the barrier of the chunk consumed next has already been seen complete

#pragma unroll 1
    for (int op = 0; op < a.n_ops; ++op) {
        const StackOpLite& o = lite[op];
        const int UB = o.tiles_k * 8;
        const int T = UB * o.col_blocks;
        const bool narrow = (o.narrow & 1) != 0;
        const bool tracing = a.trace != nullptr && threadIdx.x == 0;
        unsigned long long* stamp = a.trace == nullptr ? nullptr : a.trace + (static_cast<size_t>(op) * gridDim.x + blockIdx.x) * kStackTraceSlots;
        const int w0 = stack_unit_begin(T, o.warps, wid, o.narrow, o.col_blocks);
        const int w1 = stack_unit_begin(T, o.warps, wid + 1, o.narrow, o.col_blocks);
        if (w1 <= w0) continue;
        if (w1 - w0 > UB) {                                     // the planner guarantees this; never run past two blocks
            if (lane == 0) atomicCAS(a.error, 0u, 2u);
            break;
        }
        bool waited = false;
        // unit ranges of the CTA's warps: lane w holds the begin of warp w (lane WARPS: the end of the last warp)
        const int my_b = lane <= WARPS ? stack_unit_begin(T, o.warps, static_cast<int>(blockIdx.x) * WARPS + lane, o.narrow, o.col_blocks) : 0;
        const int next_b = __shfl_down_sync(0xffffffffu, my_b, 1);
        const int cta0 = __shfl_sync(0xffffffffu, my_b, 0);
        const uint32_t tag = tag_base + static_cast<uint32_t>(op) + 1u;
        auto arrive = [&](int cblock) {
            const bool has = lane < WARPS && min(next_b, (cblock + 1) * UB) > max(my_b, cblock * UB);
            const unsigned int mask = __ballot_sync(0xffffffffu, has);
            const unsigned int second = __ballot_sync(0xffffffffu, has && my_b / UB != cblock);
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
                // first and last CTA with rows of this block: the inverse of stack_unit_begin, in rows (RB per block, RT in all)
                const int RB = UB >> 3, RT = T >> 3;
                int i_first, i_last;
                if (o.narrow & 2) {
                    i_first = static_cast<int>(static_cast<unsigned int>(cblock) * Wop / o.col_blocks) / WARPS;
                    i_last = (static_cast<int>(static_cast<unsigned int>(cblock + 1) * Wop / o.col_blocks) - 1) / WARPS;
                } else if (narrow) {
                    i_first = static_cast<int>(((static_cast<unsigned int>(cblock * RB + 1) * Wop - 1u) / RT) / WARPS);
                    i_last = static_cast<int>(((static_cast<unsigned int>((cblock + 1) * RB) * Wop - 1u) / RT) / WARPS);
                } else {
                    i_first = static_cast<int>((((static_cast<int64_t>(cblock) * RB + 1) * Wop - 1) / RT) / WARPS);
                    i_last = static_cast<int>(((static_cast<int64_t>(cblock + 1) * RB * Wop - 1) / RT) / WARPS);
                }
                stack_finish_block<FUSED>(a, o, op, cblock, mask, second, i_last - i_first + 1, static_cast<int>(blockIdx.x) - i_first, tag,
                                   smem_raw, lane);
            }
            if (tracing) stamp[3] = global_ns();
        };
#pragma unroll 1
        for (int cblock = w0 / UB; cblock * UB < w1; ++cblock) {
            const int u0 = max(w0, cblock * UB) - cblock * UB;
            const int u1 = min(w1, (cblock + 1) * UB) - cblock * UB;
            float* stage = reinterpret_cast<float*>(mine + a.stage_offset) + (cblock - w0 / UB) * stage_floats;
            const int grp = o.groups > 1 ? stack_group_of(a.ops[op], cblock) : 0;
            {
                const int tk_first = u0 >> 3, tk_last = (u1 - 1) >> 3;      // u0 and u1 are multiples of 8: whole rows
                float acc[8][NB][4];
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[t][0][i] = 0.0f;

#pragma unroll 1
                for (int tk0 = tk_first; tk0 <= tk_last;) {
                    const int kb0 = tk0 >> 3;
                    const int tk_end = min(tk_last + 1, (kb0 + a.x_blocks) * 8);
                    const int nrows = tk_end - tk0;
                    const bool first_chunk = !waited;
                    const int nblk = ((tk_end - 1) >> 3) - kb0 + 1;
                    uint2 sv[kQmvXBlocks];
                    stack_fetch_scales(o.suh + static_cast<int64_t>(grp) * o.in, kb0, nblk, lane, sv);
                    if (!waited) {
                        stack_wait(a, op, lite[op > 0 ? op - 1 : 0].col_blocks, &s_ready, &s_poller, lane);
                        waited = true;
                        if (tracing) stamp[0] = global_ns();
                    }
                    if (FUSED && o.prologue != 0) stack_rotate_chunk_fused(a.ops[op], sv, rows, kb0, nblk, kXsHalves, xs, lane);
                    else stack_rotate_chunk(o.x, a.x_dtype, sv, o.in, rows, kb0, nblk, kXsHalves, xs, lane);
                    if (tracing && first_chunk) stamp[1] = global_ns();
                    const uint32_t* xfrag =
                        reinterpret_cast<const uint32_t*>(xs + min(g, rows - 1) * kXsHalves + (tk0 * 16 - kb0 * 128)) + q;
                    // The rows of this stretch are walked run by run: a run is the part of one stream chunk that lies inside
                    // the stretch.  Everything that happens once per chunk (barrier, probe of the next chunk, hand-back of the
                    // slot) is outside the row loop, whose body tests nothing per tile.  The activation fragment of the
                    // next row is loaded while a row is decoded.  Lanes whose
                    // activation row does not exist (g >= rows) multiply whatever the last row holds: column n of the
                    // product depends on column n of the activations only, and those columns are never stored.
                    uint32_t p0 = xfrag[0], p1 = xfrag[4];
                    xfrag += 8;
#pragma unroll 1
                    for (int r = 0; r < nrows;) {
                        const int tk = tk0 + r;
                        const int ri = (tk - tk_first) & (R - 1);               // row inside its chunk
                        const int run = min(R - ri, nrows - r);                 // whole rows only: a warp's range starts and ends on a row
                        if (ri == 0) {
                            if (!ready && !copy_lost && !mbar_wait(bars + slot, parity)) copy_lost = true;   // after a lost copy: no more waits
                            const int nslot = slot + 1 == SLOTS ? 0 : slot + 1;
                            ready = mbar_test_wait(bars + nslot, slot + 1 == SLOTS ? parity ^ 1u : parity);
                        }
                        const uint32_t* row_words = ring + (slot * R + ri) * kRowWords;
#pragma unroll 1
                        for (int j = 0; j < run; ++j) {
                            uint32_t bx[NB][4];
                            stack_fragment<MODE>(p0, p1, bx[0]);
                            p0 = xfrag[0]; p1 = xfrag[4];                       // one row past the stretch at most: inside the warp's buffer
                            xfrag += 8;
                            qmv_row<K, CB, NB, MODE, true>(row_words, geom, 0, 8, bx, acc);
                            row_words += kRowWords;
                        }
                        r += run;
                        if (ri + run == R || tk0 + r > tk_last) {               // the chunk is consumed: its slot takes the next one
                            __syncwarp();                                       // every lane has read the slot
                            if (cur.valid) refill(slot);
                            if (++slot == SLOTS) { slot = 0; parity ^= 1u; }
                        }
                    }
                    tk0 = tk_end;
                }
                if (tracing) stamp[2] = global_ns();
                if (a.trace != nullptr && lane == 0) stamp[8 + warp] = global_ns();          // every warp: its tiles are done
#pragma unroll
                for (int t = 0; t < 8; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = 2 * q + (i & 1), col = t * 16 + g + ((i & 2) ? 8 : 0);
                        if (row < rows) stage[row * kQmvRedStride + col] = acc[t][0][i];
                    }
            }
            // the last warp of the CTA to arrive at this block adds the CTA's tiles and carries the block on (measured:
            // doing this only after all of the warp's tiles of the layer makes the step 4 % slower, not faster)
            arrive(cblock);
        }
    }
    if (copy_lost && lane == 0) atomicCAS(a.error, 0u, 1u);
    // ---- the last CTA to leave puts the step's counters back to zero ----------------------------------------
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int left = atomicAdd(a.exit_count, 1u);
        if (left == gridDim.x - 1) {
            for (int i = 0; i < a.n_ops; ++i) a.op_done[i] = 0;
            *a.exit_count = 0;
            *a.launch = *a.launch + 1u;
            __threadfence();
        }
    }
}

template <int K, int CB, int MODE, bool FUSED>
cudaError_t stack_launch_one(const StackArgs& a, const StackPlan& plan, cudaStream_t stream) {
    auto kernel = stack_kernel<K, CB, MODE, FUSED>;
    static PerDeviceOnce attribute;
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kStackMaxSmemBytes);
        if (e != cudaSuccess) return e;
        attribute.mark();
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
    cfg.blockDim = dim3(kStackWarps * 32);
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
    if (a.fused) {
        if (cb == 2) return stack_launch_one<K, 2, 1, true>(a, plan, stream);
        if (cb == 0) return exact ? stack_launch_one<K, 0, 1, true>(a, plan, stream) : stack_launch_one<K, 0, 0, true>(a, plan, stream);
        return exact ? stack_launch_one<K, 1, 1, true>(a, plan, stream) : stack_launch_one<K, 1, 0, true>(a, plan, stream);
    }
    if (cb == 2) return stack_launch_one<K, 2, 1, false>(a, plan, stream);
    if (cb == 0) return exact ? stack_launch_one<K, 0, 1, false>(a, plan, stream) : stack_launch_one<K, 0, 0, false>(a, plan, stream);
    return exact ? stack_launch_one<K, 1, 1, false>(a, plan, stream) : stack_launch_one<K, 1, 0, false>(a, plan, stream);
}

}  // namespace b200exl3
