// Internal launcher declarations shared by the kernel translation units and the C ABI layer.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tp_exchange.cuh"

namespace b200exl3 {

// Multiprocessors of the current device, asked once per device (148 when no device answers, so that the launch
// planners can be exercised on a machine without a GPU).
int sm_count();

// True when kernels are launched with programmatic stream serialization (option "pdl"): a kernel may then start while
// its predecessor in the stream is still running, and must execute griddepcontrol.wait before it touches memory.
bool pdl_enabled();

// Launch of a small dependent kernel: with "pdl" on, the kernel is allowed to start early (its first statements are
// pdl_launch_dependents(); pdl_wait();), which hides its launch latency behind the predecessor's tail.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- codec (kernels_codec.cu) ---------------------------------------------------------------------
cudaError_t launch_unpack_states(const uint16_t* packed, int64_t tiles, int k, int cb, uint16_t* states, __half* values,
                                 cudaStream_t stream);
cudaError_t launch_codebook(const uint16_t* states, int64_t n, int cb, __half* values, cudaStream_t stream);
cudaError_t launch_reconstruct(const uint16_t* trellis, int tiles_k, int tiles_n, int k, int cb, __half* w,
                               cudaStream_t stream);

// ---- rotations (kernels_rotate.cu) ----------------------------------------------------------------
// xhat[r, :] = H128(half(half(x[r, :]) * suh[(r % scale_rows), :])); scale_rows is 1 or rows.
cudaError_t launch_prepare(const void* x, int x_dtype, const __half* suh, int64_t scale_rows, int64_t rows, int in,
                           __half* xhat, cudaStream_t stream, const __half* glu_up = nullptr);
// y = half(H128(half(sum_s partials[s, r, :]))) * svh (+ bias), written in y_dtype.
cudaError_t launch_finish(const float* partials, int splits, int64_t split_stride, const __half* svh,
                          int64_t scale_rows, const __half* bias, int64_t rows, int out, int y_dtype, void* y,
                          cudaStream_t stream);

// ---- fused linear layer (kernels_qmv*.cu) ----------------------------------------------------------
constexpr int kQmvWarps = 8;         // warps per CTA (measured: 12 warps in one CTA per SM is no faster for the per-layer kernel)
constexpr int kQmvRedStride = 132;   // floats per reduced row: 128 + 4 keeps the fragment stores conflict-free
constexpr int kQmvMaxGroups = 8;     // projections fused in one launch (q/k/v, gate/up)
constexpr int kQmvMaxRows = 16;      // activation rows one launch can take
constexpr int kQmvMaxSmemBytes = 200 * 1024;
constexpr int kQmvXBlocks = 6;       // 128-blocks of rotated activations a warp keeps per row
constexpr int kQmvFusedRows = 2;     // up to this many rows the kernel rotates the activations itself

// The weight stream of a warp: chunks of consecutive rows of a column block (a row is 8 tiles; one bulk copy per chunk),
// a few chunks in flight: 8 rows for 1-2 bits, 6 for 3-4 bits, 4 above (4 to 8 KB per warp)
__host__ __device__ constexpr int qmv_chunk_rows(int k) { return k <= 2 ? 4 : 2; }
__host__ __device__ constexpr int qmv_slots(int k) { return (k == 3 || k == 4) ? 3 : 2; }

struct QmvArgs {
    const uint32_t* wq;        // quad layout [tiles_n/8, tiles_k, 2, 8K, 4] words
    const void* x;             // [rows, in] activations in x_dtype (used when xhat == nullptr)
    const __half* suh;         // [groups, in]
    const __half* xhat;        // [groups, rows, in] already rotated activations, or nullptr
    float* partials;           // [out/128, max_pieces, rows, 128] scratch for column blocks shared by several CTAs
    unsigned int* counters;    // [out/128] arrival counters, zero on entry and on exit
    unsigned int* error;       // set to 1 if a weight copy never arrived (bounded wait gave up)
    unsigned long long* trace; // optional [grid, 8] nanosecond stamps of the phases of each CTA, or nullptr
    const __half* svh;         // [out]   (output rotation; used when y != nullptr)
    const __half* bias;        // [out] or nullptr
    float* yhat;               // [rows, out] summed fp32 product (raw output) when not nullptr; else:
    void* gy[kQmvMaxGroups];   // per group: [rows, gout[g]] rotated output in y_dtype
    int gcol0[kQmvMaxGroups];  // per group: first column in the concatenated output space
    int gout[kQmvMaxGroups];   // per group: output width
    int groups;                // 1 for a plain layer
    int64_t xhat_group_stride; // halves between the rotated activations of consecutive groups
    int x_dtype, y_dtype;
    int in, out, rows, tiles_k, tiles_n, max_pieces;
    int warp_smem;             // bytes of shared memory per warp
    int xs_offset;             // offset of the rotated activations inside a warp's shared memory
    int stage_offset;          // offset of the staged result tiles inside a warp's shared memory
    int pdl_early;             // 1: let the next kernel start as soon as this one has started its copies
    // Expert-mapped mode (map_selected != nullptr; rows == 1, raw output): the `out` axis is virtual,
    // [slots, map_proj, map_blocks * 128]; slot s reads the columns of expert map_selected[s] in the bank
    // (column block map_proj_index * map_stride_blocks + expert * map_blocks + j; tiles_n is the bank's width)
    // and multiplies them with its own rotated activations xhat[s * map_proj + projection, :].
    const uint32_t* map_selected;
    const int* map_count;      // optional: number of slots in use; the blocks of later slots are skipped
    int map_blocks, map_proj, map_stride_blocks, map_experts;
    int map_top_k;             // with xhat == nullptr: slot s reads row s / map_top_k of x and rotates it with suh[expert, projection]
    // Fused prologue (fp16 rows, the kernel rotates the rows itself): 0 none; 1 RMSNorm of x (+ residual `pro_aux`) with
    // weight `pro_weight`, the sum stored to `pro_sum` (a buffer other than x) by the warps of the first column block;
    // 2 SwiGLU: the input is swiglu(x, pro_aux).
    // 3 RMSNorm of x whose per-128-block sums of squares `pro_sumsq` [rows, in / 128] were left by the layer before.
    int prologue;
    const __half* pro_aux;
    const __half* pro_weight;
    __half* pro_sum;
    const float* pro_sumsq;
    float pro_eps;
    // Fused epilogue (plain fp16 layer): 1 = the output is added to the residual rows `epi_residual` [rows, out]; the sum
    // goes to `epi_sum` (may be the residual buffer itself: a column block is read and written by one warp only) and the
    // sum of its squares over each 128-block to `epi_sumsq` [rows, out / 128] for the next layer's RMSNorm.
    const int* epi_pos;        // epilogue 2 (a [q | k | v] group, one row): position of the token ...
    float epi_log2_theta;      // ... log2 of the rotary base ...
    int epi_max_ctx;           // ... rows per head of the caches ...
    __half* epi_k_cache;       // ... [k heads, max_ctx, 128]: rotated keys go to row *epi_pos
    __half* epi_v_cache;       // ... values are copied there
    // expert-mapped down product of a small batch (one row per slot) with the glue around it in the same launch:
    // prologue 4 = the SwiGLU glue (native/src/moe.rs:438-533) from the raw gate/up products of the launch before,
    const float* pro_ygu;      // [slots * 2, in] raw gate and up products (in = the experts' width)
    const __half* pro_gu_svh;  // [experts, 2, in] output scales of gate and up; suh = [experts, in] input scales of down
    int pro_logical;           // columns at and past this one are padding: their activation is zero
    // epilogue 3 = finish_and_reduce (moe.rs:586-609): every slot's block is rotated, scaled by svh[expert] and its score
    // and parked in yhat; the last slot of a token to arrive adds the token's top_k blocks in slot order into gy[0]
    const void* epi_scores;    // [slots] routing weights, fp16 or fp32 (the output has their type)
    int epi_score_f32;
    int epi_counter0;          // first of the (token, block) arrival counters inside `counters`
    int epilogue;
    const __half* epi_residual;
    __half* epi_sum;
    float* epi_sumsq;
    // Tensor-parallel row shard (tp.world > 0; rotated output): the complete sum of a column block is
    // exchanged with the other ranks (unit = (tp_row0 + row) * out/128 + block) before the output rotation.
    TpPeers tp;
    int tp_row0;
};

struct QmvPlan {
    int grid;            // CTAs of 8 warps: every warp gets the same number of tiles (+-1)
    int max_pieces;      // upper bound on the CTAs that share one 128-column block
    int col_blocks;      // out / 128
    int warp_smem;       // bytes of shared memory per warp
    int xs_offset;       // offset of the rotated activations inside a warp's shared memory
    int stage_offset;    // offset of the staged result tiles inside a warp's shared memory
    bool fused_rotation; // the kernel rotates the activations itself (rows <= kQmvFusedRows)
    size_t smem_bytes;   // dynamic shared memory per CTA
    bool pdl;            // launch with programmatic stream serialization (overlap with the previous kernel's tail)
    bool pdl_early;      // trigger the dependent launch before the main loop instead of after it
};
QmvPlan plan_qmv(int in, int out, int k, int64_t rows);
// Scratch a launch needs: counters first (zero-initialised once by the owner), then the partial sums.
size_t qmv_partial_bytes(const QmvPlan& plan, int out, int64_t rows);
// exact: decode the reference's fp16 weight bit for bit before multiplying (codebooks 0/1 default to
// feeding the two fp16 halves of a weight as two products, which differs by fp16 rounding of the weight).
cudaError_t launch_qmv(QmvArgs args, int k, int cb, bool exact, const QmvPlan& plan, cudaStream_t stream);
void qmv_set_tuning(int ctas_per_sm, int force_grid, int pdl);
void qmv_set_trace(unsigned long long* device_buffer);

// ---- a whole decode step in one persistent launch (kernels_stack*.cu) ------------------------------------------
// The kernel streams weights in chunks of consecutive rows of a column block (one bulk copy each; a row is 8 tiles)
// and keeps three chunks per warp in flight (9 to 12 KB), so that the stream does not run dry while a layer boundary
// is crossed.  Measured: chunk and ring geometry hardly matter (1 row x 8 slots to 8 rows x 2 slots: within 3 %);
// what a chunk buys is that the barrier wait, the probe and the refill leave the row loop.
__host__ __device__ constexpr int stack_chunk_rows(int k) { return k <= 4 ? 4 : 2; }
constexpr int kStackSlots = 3;                  // chunks in flight per warp
#ifndef B200_STACK_WARPS
#define B200_STACK_WARPS 12
#endif
constexpr int kStackWarps = B200_STACK_WARPS;   // warps per CTA, one CTA per SM.  Measured on one decoder layer: 12 warps (3 per scheduler, up to 170 registers each) 88 us, 16 warps (128 registers) 100 us, 8 warps 98 us, 10 and 14 (uneven over the four schedulers) 103-106 us
constexpr int kStackCtasPerSm = 1;
constexpr int kStackMaxRows = 2;
constexpr int kStackTraceSlots = 8 + kStackWarps;   // stamps per (layer, CTA) in the optional trace buffer
constexpr int kStackMaxSmemBytes = 224 * 1024;   // dynamic shared memory the kernel may ask for (227 KB per CTA less the static part)     // activation rows of a step (batch-1 decode and small speculative batches)

struct StackOp {               // one layer of the step; lives in device memory
    const uint32_t* wq;        // quad layout
    const void* x;             // [rows, in] activations (x_dtype of the stack)
    const __half* suh;         // [groups, in]
    const __half* svh;         // [out]
    const __half* bias;        // [out] or nullptr
    void* gy[kQmvMaxGroups];   // per group: [rows, gout[g]] output
    int gcol0[kQmvMaxGroups];
    int gout[kQmvMaxGroups];
    int groups;
    int in, out, tiles_k, tiles_n, col_blocks;
    int warps;                 // warps of the grid that share this layer's tiles (a multiple of the CTA's warps)
    int narrow;                // bit 0: (tiles + 1) * warps fits 32 bits; bit 1: whole warps per column block (see stack_unit_begin)
    int max_pieces;            // bound on the CTAs that share one column block
    int tp_unit0;              // >= 0: row shard of a tensor-parallel layer, first exchange unit; -1: none
    // operators fused around the layer (fp16 steps; the arithmetic of the per-layer kernel's prologues and epilogues)
    int prologue;              // 0 none, 2 SwiGLU (x = gate rows, pro_aux = up rows), 3 RMSNorm from block sums of squares
    int epilogue;              // 0 none, 1 residual add + block sums of squares, 2 rotary embedding + cache append ([q|k|v])
    const __half* pro_aux;
    const __half* pro_weight;  // [in] norm weight
    const float* pro_sumsq;    // [rows, in / 128]
    float pro_eps;
    const __half* epi_residual;// [rows, out]
    __half* epi_sum;           // [rows, out] (may be epi_residual)
    float* epi_sumsq;          // [rows, out / 128]
    const int* epi_pos;
    float epi_log2_theta;
    int epi_max_ctx;
    __half* epi_k_cache;
    __half* epi_v_cache;
};

// What every warp needs at a layer boundary, staged in shared memory at kernel start so that the weight cursor
// and the main loop never wait for a table read from global memory.
struct StackOpLite {
    const uint32_t* wq;
    const void* x;
    const __half* suh;
    const __half* svh;
    const __half* bias;
    void* y0;                  // output of a plain layer (grouped layers read their outputs from the full table)
    int tiles_k, tiles_n, col_blocks, warps, narrow, in, groups, max_pieces, tp_unit0, gout0;
    int prologue, epilogue;    // the rest of a fused layer's description is read from the full table
};
constexpr int kStackMaxOps = 256;    // layers per launch: the staged table takes 88 bytes per layer

struct StackArgs {
    const StackOp* ops;
    int n_ops, rows, x_dtype, y_dtype;
    unsigned int* op_done;     // [n_ops] finished column blocks per layer: zero at launch, zero again at exit
    unsigned int* exit_count;  // CTAs that have left
    unsigned int* error;       // status word: 1 lost copy, 2 plan violated, 5 a layer-boundary wait gave up, 6 a partial sum never arrived
    unsigned long long* piece_words[2];   // by layer parity: [col_blocks, max_pieces, rows, 128] {partial sum, tag} words
    unsigned int* launch;      // number of completed launches (the tags of a launch are made of it)
    int warp_smem, xs_offset, stage_offset;
    int x_blocks;              // 128-blocks of rotated activations a warp keeps per row (the chunk length of its walk)
    unsigned long long wait_ns;
    unsigned long long* trace; // optional [n_ops, grid, kStackTraceSlots] stamps; warp 0: boundary passed, rotated, main loop done, block carried on; the warp that
                               // carries a block on: start, after the atomic, pieces added, stored and counted; then every warp: its tiles done
    int table_offset;          // offset of the staged layer table in dynamic shared memory
    int fused;                 // 1: some layer of the step has a fused prologue or epilogue (a kernel of its own)
    TpPeers tp;
};

struct StackPlan {
    int grid;
    size_t smem_bytes;
    int warp_smem, xs_offset, stage_offset, table_offset, x_blocks;
    bool cooperative;
};
// grid and shared memory of a step with `rows` activation rows at K bits
StackPlan plan_stack(int k, int rows, int n_ops);
// fills the partition fields of one layer (warps, narrow, max_pieces); false if the layer cannot be part of a step
bool plan_stack_op(const StackPlan& plan, StackOp& op);
cudaError_t launch_stack(const StackArgs& args, int k, int cb, bool exact, const StackPlan& plan, cudaStream_t stream);

// ---- grouped experts (kernels_moe.cu) ------------------------------------------------------------------
// SwiGLU glue between the expert projections (native/src/moe.rs:438-533, SiLU): raw gate/up sums
// ygu[slot * 2 + {0,1}, :] -> rotated input of the down projection xhat[slot, :]
// `count` (optional, device): only slots below *count are computed
cudaError_t launch_glu_down_input(const float* ygu, const __half* gu_svh, const __half* down_suh, const uint32_t* selected,
                                  int experts, int64_t slots, int hidden, int logical_hidden, __half* xhat,
                                  cudaStream_t stream, const int* count = nullptr);
// y[row, :] = sum over the row's top_k slots of rotate(half(raw[slot, :])) * svh[selected[slot], :] * score
// (native/src/moe.rs:586-609); scores and y are fp16 or fp32 (score_dtype)
cudaError_t launch_finish_and_reduce(const float* raw, const __half* down_svh, const uint32_t* selected, int experts,
                                     const void* scores, int score_dtype, int64_t rows, int top_k, int out, void* y,
                                     cudaStream_t stream);

// ---- expert parallelism (kernels_ep.cu) -------------------------------------------------------------------------------
struct EpPeers {
    unsigned long long* inbox[kTpMaxWorld];   // every rank's inbox [2, max_slots, out / 2] of {two fp16 values, sequence} words
    unsigned int* done;                       // [max_slots] calls that used each slot index (identical on all ranks)
    unsigned int* error;                      // status word: 7 = a slot result never arrived
    int rank, world, max_slots;
    unsigned long long wait_ns;
};
cudaError_t launch_ep_plan(const uint32_t* selected, int64_t slots, int first, int count, int* local_count, uint32_t* local_slot,
                           uint32_t* local_expert, cudaStream_t stream);
cudaError_t launch_ep_dispatch(const void* x, int x_dtype, const __half* gu_suh, const int* local_count, const uint32_t* local_slot,
                               const uint32_t* local_expert, int top_k, int in, int64_t max_slots, __half* xhat, cudaStream_t stream);
cudaError_t launch_ep_publish(const float* raw, const __half* down_svh, const int* local_count, const uint32_t* local_slot,
                              const uint32_t* local_expert, int out, int64_t max_slots, const EpPeers& ep, cudaStream_t stream);
cudaError_t launch_ep_combine(const void* scores, int score_dtype, int64_t rows, int top_k, int out, void* y, const EpPeers& ep,
                              cudaStream_t stream);

// ---- row-parallel sum over peer memory + output rotation (kernels_tp.cu) -----------------------------------
struct TpArgs {
    const float* yhat;               // [rows, out] this rank's fp32 partial product
    TpPeers peers;
    const __half* svh;               // [out]
    const __half* bias;              // [out] or nullptr
    void* y;                         // [rows, out] in y_dtype
    int rows, out, y_dtype;
};
cudaError_t launch_tp_finish(const TpArgs& args, cudaStream_t stream);

// Expert-sorted form for many slots (native/src/moe.rs:66-182 route_plan, 1001-1085): slots are grouped by expert
// into segments of up to R rows (seg_rows), so that an expert's columns are decoded once per R rows that use them.
// R = kMoeSegRows = 8 is one block of rows of the fused kernel, whose one-block form runs two CTAs per SM and decodes
// almost twice as fast per tile as the two-block form that 16 rows would need; R = kQmmSegRows = 64 is the token tile
// of the small tensor-core shape, for batches that give most experts many rows.
//   seg_count[0]        number of segments
//   seg_expert[s]       expert of segment s
//   row_slot[R s + r]   slot in row r of segment s, or 0xffffffff for a padding row
//   slot_row[slot]      padded row R s + r that holds the slot
// max_segments bounds the arrays (min(experts, slots) + slots / R always suffices).
constexpr int kMoeSegRows = 8;
cudaError_t launch_route_plan(const uint32_t* selected, int64_t slots, int experts, int max_segments, int seg_rows, int* seg_count,
                              uint32_t* seg_expert, uint32_t* row_slot, uint32_t* slot_row, cudaStream_t stream);
// padded-row forms of the three glue kernels; activations and products are laid out per segment:
// xhat[(s * proj + p) * R + r, :], products y[r, (s * proj + p) * width + col] with row stride max_segments * proj * width
cudaError_t launch_routed_prepare_padded(const void* x, int x_dtype, const __half* suh, const uint32_t* seg_expert,
                                         const uint32_t* slot_row, int64_t slots, int top_k, int proj, int max_segments,
                                         int seg_rows, int in, __half* xhat, cudaStream_t stream);
cudaError_t launch_glu_down_input_padded(const float* ygu, const __half* gu_svh, const __half* down_suh,
                                         const uint32_t* seg_expert, const uint32_t* row_slot, const int* seg_count,
                                         int experts, int max_segments, int seg_rows, int hidden, int logical_hidden, __half* xhat,
                                         cudaStream_t stream);
cudaError_t launch_finish_and_reduce_padded(const float* raw, const __half* down_svh, const uint32_t* selected,
                                            const uint32_t* slot_row, int experts, const void* scores, int score_dtype,
                                            int64_t rows, int top_k, int out, int max_segments, int seg_rows, void* y, cudaStream_t stream);

// ---- router (kernels_router.cu) --------------------------------------------------------------------------
// stable top-k per row with index tie-break; values and scores fp16 or fp32; experts <= 1024.  With `softmax` the
// values are logits and the routes are taken on their row softmax (fp32 arithmetic, rounded to the values' type),
// which is also stored to `probabilities` when that is not nullptr.
cudaError_t launch_router_topk(const void* values, int dtype, int64_t rows, int experts, int k, bool normalize, bool softmax,
                               uint32_t* indices, void* scores, void* probabilities, cudaStream_t stream);
// logits [rows, experts] fp16 = x [rows, in] times the fp16 router weights w [experts, in], fp32 accumulation
cudaError_t launch_router_gate(const void* x, int x_dtype, const __half* w, int64_t rows, int in, int experts, __half* logits,
                               cudaStream_t stream);

// ---- decoder-block glue, fp16, batch-1 decode (kernels_decoder.cu) -------------------------------------------------
cudaError_t launch_embed(const __half* table, const int* token, int64_t rows, int64_t vocab, int hidden, __half* out, cudaStream_t stream);
// s = half(x + residual) (residual and the stored sum are optional); y = weight * half(s * rsqrt(mean(s^2) + eps))
cudaError_t launch_rms_norm(const __half* x, const __half* residual, const __half* weight, int64_t rows, int n, float eps, __half* sum,
                            __half* y, cudaStream_t stream);
cudaError_t launch_swiglu(const __half* gate, const __half* up, int64_t n, __half* out, cudaStream_t stream);
// rotates q in place, writes the rotated k and v into row *pos of their heads' caches [kv_heads, max_ctx, dim]
cudaError_t launch_rope_append(__half* q, const __half* k, const __half* v, int heads, int kv_heads, int dim, const int* pos, float theta,
                               int max_ctx, __half* k_cache, __half* v_cache, cudaStream_t stream);
int attention_splits(int kv_heads, int heads);
size_t attention_workspace_bytes(int heads, int kv_heads);
// one query row against keys 0..*pos of the cache; dim must be 128
cudaError_t launch_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache, int heads, int kv_heads, int dim,
                                    const int* pos, int max_ctx, float scale, __half* out, void* workspace, cudaStream_t stream);
int head_candidates();
// logits (optional) and the arg-max (value, index + index_offset) of x [hidden] times w [vocab, hidden]^T
cudaError_t launch_head_argmax(const __half* x, const __half* w, int64_t vocab, int hidden, int64_t index_offset, __half* logits,
                               float* cand_value, long long* cand_index, float* out_value, long long* out_index, cudaStream_t stream);

// ---- tensor-core product for many rows (kernels_qmm.cu) ---------------------------------------------------
struct QmmPlan {
    int splits;        // CTAs that share one (128 columns x token tile) output tile along the input axis
    int token_tiles;   // ceil(rows / 512), or ceil(rows / 64) for the small shape
    bool small;        // up to 64 rows: 64 tokens per CTA, two CTAs per SM
};
QmmPlan plan_qmm(int in, int out, int64_t rows);
size_t qmm_partial_bytes(const QmmPlan& plan, int out, int64_t rows);
// partials[s, r, n] (fp32) = sum over the inputs of split s of xhat[r, :] (fp16, rotated) x W[:, n]; with one
// split and y != nullptr the output rotation (half -> H128 -> * svh, + bias) is applied in the kernel's epilogue
// and y[r, n] is stored in y_dtype instead.
// A member of a group (projections concatenated on the output axis) is addressed by ld_tiles (tiles per row of the
// whole weight array; 0 = out / 16) and col_tile0 (the member's first tile column, a multiple of 8).
cudaError_t launch_qmm(const uint32_t* wq, int in, int out, int k, int cb, const __half* xhat, int64_t rows,
                       const QmmPlan& plan, float* partials, unsigned int* error, const __half* svh, const __half* bias,
                       void* y, int y_dtype, cudaStream_t stream, int ld_tiles = 0, int col_tile0 = 0);
// Expert-mapped form of the small shape: segment s = 64 padded rows xhat[(s * proj + p) * 64 + r, :] that all use expert
// seg_expert[s]; products[r, (s * proj + p) * width + col] (fp32, row stride max_segments * proj * width).
constexpr int kQmmSegRows = 64;
cudaError_t launch_qmm_mapped(const uint32_t* wq, int in, int width, int bank_tiles_n, int k, int cb, const __half* xhat,
                              int max_segments, int proj, int stride_blocks, int experts, const uint32_t* seg_expert,
                              const int* seg_count, float* products, unsigned int* error, cudaStream_t stream);
void qmm_set_tuning(int splits);   // force the number of input splits (0 = automatic)

// ---- weight layout (kernels_codec.cu) -----------------------------------------------------------------
// checkpoint layout [tiles_k, tiles_n, 8K] words -> quad layout [tiles_n/8, tiles_k, 2, 8K, 4]: the stream words of four
// neighbouring tiles interleaved word by word (a quad), two quads = one row of a 128-column block (256K bytes), and
// the rows of a column block one after the other, so any run of a block's rows is one contiguous copy
cudaError_t launch_repack_quads(const uint32_t* trellis, int tiles_k, int tiles_n, int k, uint32_t* wq, cudaStream_t stream);
// inner matrix from the quad layout, bit-exact
cudaError_t launch_reconstruct_quads(const uint32_t* wq, int tiles_k, int tiles_n, int k, int cb, __half* w,
                                     cudaStream_t stream);

}  // namespace b200exl3
