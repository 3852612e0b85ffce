/*
 * b200exl3 -- C ABI of the B200 (sm_100a) implementation of the EXL3 quantized-linear path.
 *
 * Conventions (they mirror the reference's FFI, native/ffi/mlx_bridge.cpp:49-66 and
 * native/src/array.rs:319-369):
 *   - every function returns 0 on success and -1 on error; it never throws or aborts;
 *   - after an error, b200exl3_last_error() returns a NUL-terminated message that stays valid
 *     until the next call of this library on the same thread;
 *   - objects are opaque handles created by *_create and released by *_free;
 *   - dtype codes are the reference's (native/src/array.rs:21-36): 2 = u16, 3 = u32, 9 = f16,
 *     10 = f32, 12 = bf16.
 * Differences forced by CUDA: tensors are caller-owned DEVICE pointers with explicit shapes
 * (the reference passes opaque lazy MLX arrays), every launch takes a cudaStream_t (passed as
 * void*), and forward calls allocate nothing: scratch memory is a caller-provided workspace whose
 * first B200EXL3_WORKSPACE_HEADER_BYTES bytes were zeroed once.  All device pointers must be
 * 16-byte aligned.  Handles are immutable after creation, so one handle may be used from several
 * threads and streams at once, each with its own workspace; calls that share a workspace must be
 * ordered on one stream.
 */
#ifndef B200EXL3_H
#define B200EXL3_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200EXL3_U16 2
#define B200EXL3_U32 3
#define B200EXL3_F16 9
#define B200EXL3_F32 10
#define B200EXL3_BF16 12

/* flags of b200exl3_linear_create */
#define B200EXL3_EXACT_WEIGHTS 2u  /* multiply with the bit-exact fp16 weight instead of its two fp16 halves */

/* A workspace starts with this many bytes of arrival counters.  They must be zero before the first
 * call that uses the workspace (b200exl3_memset); every call leaves them zero again. */
#define B200EXL3_WORKSPACE_HEADER_BYTES 16384

typedef struct b200exl3_linear b200exl3_linear;
typedef struct b200exl3_group b200exl3_group;
typedef void* b200exl3_stream;     /* cudaStream_t */

/* ---- runtime (replaces mlxl3_mlx_init / mlxl3_mlx_error, native/ffi/mlx_bridge.cpp:176, 222-232) ---- */

/* Selects `device` for the calling thread and checks that it is an sm_100 part.  Idempotent. */
int b200exl3_init(int device);
const char* b200exl3_last_error(void);
/* major*10000 + minor*100 + patch */
int b200exl3_version(void);
/* Process-wide knobs: "qmv_ctas_per_sm" (CTAs per SM the grids are sized for), "qmv_force_grid"
 * (CTAs per launch, 0 = heuristic), "pdl" (1 or 2 = launch layer kernels with programmatic stream serialization, so the
 * weight prefetch of a layer overlaps the tail of the previous kernel in the stream; 1 releases the
 * next kernel after the main loop, 2 as soon as the first copies are in flight), "qmv_trace_buffer"
 * (device address of a uint64 [grid, 8] array that receives nanosecond stamps of each CTA's phases:
 * start, activations visible, rotated, main loop done, warps joined, reduced, finished; 0 = off), "qmm" (0 = batches
 * of more than 8 rows also go through the small-batch kernel (16 rows per launch) instead of the tensor-core product; default 1),
 * "qmm_splits" (input splits of the tensor-core product, 0 = chosen by a cost model; set it before asking for
 * workspace sizes), "moe_sorted" (0 = the expert block runs one row per slot for any batch instead of grouping
 * slots by expert for larger batches; set it before asking for workspace sizes), "moe_fused" (1 = a small batch of the
 * expert block runs its SwiGLU glue and its weighted reduction as the prologue and the epilogue of the down product, two
 * launches instead of four; same bits either way, measured no faster; default 0), "qmm_trace_buffer" (device address of a uint64 [CTAs, 8] array that receives nanosecond
 * stamps of the tensor-core kernel's phases: start, set up, decoders done, MMAs issued, accumulator ready,
 * epilogue done, end, activation copies issued; 0 = off), "tp_wait_ms" (how long a rank waits for the other ranks'
 * words inside a tensor- or expert-parallel kernel before it gives up with status 4; default 4000), "stack_wait_ms"
 * (the same bound for every wait inside the decode-step kernel: status 5 = a layer never completed, 6 = a piece of
 * a column block never arrived; default 2000), "stack_trace_buffer" (device address of a uint64
 * [layers, CTAs, 20] array that receives nanosecond stamps of the decode-step kernel: boundary passed, activations
 * rotated, last tile, block staged, finish begun, pieces out, pieces in, block stored, then one stamp per warp when
 * its tiles of the layer were done; 0 = off).  Options are atomics: they may be set from any thread, and a launch
 * reads each of them once. */
int b200exl3_set_option(const char* name, int64_t value);

/* The launch policy as data, for tests and reports (replaces the Kani proofs beside exl3_projection_splits and
 * qmv_batch_layout, native/src/contracts.rs:1995-2012, 1051-1069, by values an exhaustive test can check; needs no GPU:
 * without one the planners assume 148 multiprocessors).  kind "qmv": {CTAs, bound on CTAs sharing a column block,
 * column blocks, warps per CTA, shared memory per CTA, kernel rotates the rows itself}; "qmm": {input splits, token
 * tiles, small shape, 64-input stages}; "stack": {CTAs, bound on CTAs per block, column blocks, warps per CTA, shared
 * memory, warps that share the layer, 32-bit partition arithmetic, layer accepted}. */
int b200exl3_plan_query(const char* kind, int in, int out, int k, int64_t rows, int64_t* out_values, int capacity);

/* Plain device-memory plumbing for hosts that have no CUDA binding of their own (replaces
 * mlxl3_array_from_bytes, mlxl3_array_copy_bytes, mlxl3_array_free and mlxl3_synchronize,
 * native/ffi/mlx_bridge.cpp:337, 610, 233, 192).  Streams are created non-blocking. */
int b200exl3_malloc(size_t bytes, void** out_device_ptr);
int b200exl3_free(void* device_ptr);
int b200exl3_host_alloc(size_t bytes, void** out_pinned_ptr);
int b200exl3_host_free(void* pinned_ptr);
int b200exl3_memcpy_h2d(void* dst_device, const void* src_host, size_t bytes, b200exl3_stream stream);
int b200exl3_memcpy_d2h(void* dst_host, const void* src_device, size_t bytes, b200exl3_stream stream);
int b200exl3_memset(void* dst_device, int value, size_t bytes, b200exl3_stream stream);
int b200exl3_stream_create(b200exl3_stream* out);
int b200exl3_stream_destroy(b200exl3_stream stream);
int b200exl3_stream_sync(b200exl3_stream stream);
int b200exl3_event_create(void** out_event);
int b200exl3_event_destroy(void* event);
int b200exl3_event_record(void* event, b200exl3_stream stream);
/* Waits for `stop`, then returns the device time between the two events in milliseconds. */
int b200exl3_event_elapsed_ms(void* start, void* stop, float* out_ms);

/* Graph replay (replaces mlxl3_replay_capture / mlxl3_replay_apply / mlxl3_replay_free,
 * native/ffi/mlx_bridge.cpp:150-175).  Every launch issued on `stream` between begin and end is
 * recorded instead of run; the returned graph replays them with one launch.  Forward calls allocate
 * nothing, so whole decode steps can be recorded; run each distinct call once before recording. */
int b200exl3_graph_begin(b200exl3_stream stream);
int b200exl3_graph_end(b200exl3_stream stream, void** out_graph);
int b200exl3_graph_launch(void* graph, b200exl3_stream stream);
int b200exl3_graph_free(void* graph);

/* ---- codec (replaces exl3_decode / exl3_codebook of native/shaders/exl3.metal:102-114 and
 *      codec::unpack / decode_codeword / reconstruct_inner of native/src/codec.rs:52-71, 102-124, 159-190) ---- */

/* packed [tiles, 16k] u16 -> states [tiles, 256] u16 (kernel order) and/or fp16 values [tiles, 256];
 * either output may be NULL. */
int b200exl3_unpack_states(const uint16_t* d_packed, int64_t tiles, int k, int codebook, uint16_t* d_states,
                           uint16_t* d_values_f16, b200exl3_stream stream);
/* states [n] u16 -> fp16 weights [n]; d_states == NULL enumerates the states 0..n-1. */
int b200exl3_codebook(const uint16_t* d_states, int64_t n, int codebook, uint16_t* d_values_f16,
                      b200exl3_stream stream);
/* trellis [in/16, out/16, 16k] u16 -> inner matrix W [in, out] fp16 row-major, bit-exact with
 * codec::reconstruct_inner.  in and out are multiples of 16. */
int b200exl3_reconstruct(const uint16_t* d_trellis, int in, int out, int k, int codebook, uint16_t* d_w_f16,
                         b200exl3_stream stream);

/* ---- rotations (replace the MLX chains of native/src/linear.rs:855-861 and 978-996, the fused
 *      glue_prologue / glue_epilogue of native/src/linear.rs:1452-1600, mlxl3_flash_prepare128 of
 *      native/ffi/mlx_bridge.cpp:237 and exl3_prepare128 / flash_finish128 of
 *      native/shaders/exl3.metal:204-235) ---- */

/* xhat[r, :] = H128(half(half(x[r, :]) * suh)) as fp16.  d_suh_f16 holds [in] (scale_rows == 1) or
 * [rows, in] (scale_rows == rows).  Bit-exact with MLX's fp16 hadamard_transform. */
int b200exl3_prepare(const void* d_x, int x_dtype, const uint16_t* d_suh_f16, int64_t scale_rows, int64_t rows, int in,
                     uint16_t* d_xhat_f16, b200exl3_stream stream);
/* y[r, :] = half(H128(half(sum_s partials[s, r, :]))) * svh (+ bias) written as y_dtype.
 * partials is fp32 [splits, rows, out]; d_bias_f16 may be NULL. */
int b200exl3_finish(const float* d_partials, int splits, const uint16_t* d_svh_f16, int64_t scale_rows,
                    const uint16_t* d_bias_f16, int64_t rows, int out, int y_dtype, void* d_y, b200exl3_stream stream);

/* ---- Exl3Linear (replaces native/src/linear.rs:424-1236) ---- */

/* Same validation as Exl3Linear::new (native/src/linear.rs:577-639): k in 1..8, codebook in 0..2
 * (0 default, 1 MCG, 2 MUL1), in and out positive multiples of 128, trellis [in/16, out/16, 16k]
 * 16-bit integers.  suh [in], svh [out] and the optional bias [out] are given in `scale_dtype`
 * (f16, bf16 or f32) and converted once to fp16, as the reference does at load.  The trellis is
 * re-laid into library-owned memory (four neighbouring tiles interleaved word by word, same size;
 * this replaces the loader's tile-layout preparation), so none of the caller's buffers is referenced
 * after the call returns. */
int b200exl3_linear_create(const uint16_t* d_trellis, const void* d_suh, const void* d_svh, const void* d_bias_or_null,
                           int scale_dtype, int in, int out, int k, int codebook, uint32_t flags,
                           b200exl3_linear** out_handle);
void b200exl3_linear_free(b200exl3_linear* handle);
int b200exl3_linear_input_dims(const b200exl3_linear* handle);    /* Exl3Linear::input_dims  */
int b200exl3_linear_output_dims(const b200exl3_linear* handle);   /* Exl3Linear::output_dims */
int b200exl3_linear_workspace_bytes(const b200exl3_linear* handle, int64_t rows, size_t* out_bytes);
/* Waits for the device and reads the status word of a workspace: 0 = every kernel that used it ran to
 * completion, 1 = a bounded device-side wait gave up (the results of that call are invalid).  The
 * kernels never spin without a limit, so a lost copy shows up here instead of as a hung GPU. */
int b200exl3_workspace_status(const void* d_workspace, int* out_status);
/* Exl3Linear::forward (native/src/linear.rs:731-997): x [rows, in] in x_dtype -> y [rows, out] in
 * the same dtype.  rows >= 1.  The workspace must hold b200exl3_linear_workspace_bytes(rows). */
int b200exl3_linear_forward(const b200exl3_linear* handle, const void* d_x, int x_dtype, int64_t rows, void* d_y,
                            void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);
/* Allocation-free variant of b200exl3_linear_forward.  It has no counterpart in the reference.
 * Meant for hosts that cannot give the library a workspace -- code running inside another runtime's
 * memory pool, latency-critical loops that must stay away from the allocator, bindings that only
 * ever see input and output pointers: the scratch memory is a fixed 4 MiB array inside the library's
 * device image (held by every GPU that loads the library, until the process exits), and the call
 * itself allocates and frees nothing.  x and y are as in b200exl3_linear_forward.
 *   - A call whose scratch need (b200exl3_linear_workspace_bytes) exceeds 4 MiB is rejected with an
 *     error; decode-sized calls (a few rows) of any layer of the supported models fit.
 *   - The first call on each device looks up the array's device address; make that first call
 *     outside any stream capture.
 *   - All calls share the one array: every call clears the counters at its head on `stream` first,
 *     so calls must not overlap on the GPU (same stream, or otherwise ordered) -- two calls running
 *     at the same time would race on the scratch. */
int b200exl3_linear_forward_static(const b200exl3_linear* handle, const void* d_x, int x_dtype, int64_t rows, void* d_y,
                                   b200exl3_stream stream);
/* Status word of the static scratch on the current device (the counterpart of b200exl3_workspace_status for
 * b200exl3_linear_forward_static; no counterpart in the reference): 0, or the code of the bounded wait that gave up
 * during some earlier static call.  The word is sticky; a non-zero `clear` resets it after reading.  Synchronises
 * with the device, so call it after the stream of the static calls has drained. */
int b200exl3_static_status(int* out_status, int clear);
/* The middle of forward alone: fp32 yhat [rows, out] = xhat [rows, in] (fp16, already rotated) times
 * the inner matrix -- what the reference's QMV/QMM kernels return before the output rotation. */
int b200exl3_linear_forward_raw(const b200exl3_linear* handle, const uint16_t* d_xhat_f16, int64_t rows, float* d_yhat,
                                void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);
/* Row-parallel tensor parallelism.  The reference sums split-K partials in fp32 before the output
 * rotation (native/src/linear.rs:978-982); a layer whose input rows are sharded over GPUs is the same
 * thing with the partials on different devices.  forward_partial = input rotation + product, giving
 * this shard's fp32 yhat [rows, out]; the caller all-reduces yhat and then calls linear_finish, which
 * applies the output rotation, svh and bias of the handle. */
int b200exl3_linear_forward_partial(const b200exl3_linear* handle, const void* d_x, int x_dtype, int64_t rows,
                                    float* d_yhat, void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);
int b200exl3_linear_finish(const b200exl3_linear* handle, const float* d_yhat, int64_t rows, int y_dtype, void* d_y,
                           b200exl3_stream stream);
/* Inner matrix W [in, out] fp16 of this layer (the bit-exact deliverable). */
int b200exl3_linear_decode(const b200exl3_linear* handle, uint16_t* d_w_f16, b200exl3_stream stream);

/* ---- Exl3Group (replaces native/src/linear.rs:2285-2814 and native/shaders/_qmv_mapped_tile_kernel.metal
 *      in its identity-map use): projections that read the same input (q/k/v, gate/up), each with its
 *      own suh, run as ONE launch ---- */

/* Same rule as Exl3Group::compatible (native/src/linear.rs:2303-2311): at least two members with equal
 * input width, K and codebook (K = 7 is accepted too; the reference excludes it for an Apple-specific
 * reason).  Weights and scales are copied (concatenated along the output axis, native/src/linear.rs:
 * 2313-2375), so the members may be freed afterwards.  At most 8 members. */
int b200exl3_group_create(const b200exl3_linear* const* members, int count, b200exl3_group** out_handle);
void b200exl3_group_free(b200exl3_group* handle);
int b200exl3_group_count(const b200exl3_group* handle);
int b200exl3_group_workspace_bytes(const b200exl3_group* handle, int64_t rows, size_t* out_bytes);
/* Exl3Group::forward (native/src/linear.rs:2377-2814): x [rows, in] -> count outputs, d_ys[g] is
 * [rows, out_g] in x's dtype. */
int b200exl3_group_forward(const b200exl3_group* handle, const void* d_x, int x_dtype, int64_t rows, void* const* d_ys,
                           void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);

/* ---- Exl3SwitchGlu: grouped SwiGLU experts ---------------------------------------------------------------
 * Replaces Exl3SwitchGlu::{new, forward} (native/src/moe.rs:808-971; SiLU activation) and, under it,
 * routed_inputs (moe.rs:184-236), expert_mapped / prepared_expert_raw (native/src/linear.rs:2817-2885),
 * glu_down_input (moe.rs:438-533) and finish_and_reduce (moe.rs:586-609).
 *
 * Banks, in the checkpoint tile layout: gu_trellis [in/16, experts*2*hidden/16, 16K] holds the gate columns of
 * all experts followed by the up columns of all experts (expert e, projection p starts at tile column
 * p*experts*hidden/16 + e*hidden/16); down_trellis [hidden/16, experts*in/16, 16K].  Scales: gu_suh
 * [experts, 2, in], gu_svh [experts, 2, hidden], down_suh [experts, hidden], down_svh [experts, in], all in
 * scale_dtype.  Requirements as in the reference: in and hidden multiples of 128, 1 <= top_k <= experts, K != 7.
 * The banks are re-laid into library-owned memory. */
typedef struct b200exl3_moe b200exl3_moe;
int b200exl3_moe_create(const uint16_t* d_gu_trellis, const void* d_gu_suh, const void* d_gu_svh,
                        const uint16_t* d_down_trellis, const void* d_down_suh, const void* d_down_svh, int scale_dtype,
                        int experts, int in, int hidden, int top_k, int k, int codebook, uint32_t flags,
                        b200exl3_moe** out);
void b200exl3_moe_free(b200exl3_moe* handle);
int b200exl3_moe_workspace_bytes(const b200exl3_moe* handle, int64_t rows, size_t* out_bytes);
/* x [rows, in] in x_dtype; selected [rows, top_k] expert ids (u32; ids past the bank are clamped to the last
 * expert instead of reading out of bounds); scores [rows, top_k] routing weights in score_dtype (fp16 = 9 or
 * fp32 = 10); y [rows, in] in score_dtype (the reference's result dtype: fp16 products promoted by the scores).
 * Small batches run one activation row per (token, choice) slot against the slot's expert's columns.  From 33
 * slots and two slots per expert on, the slots are grouped by expert on the device (the reference's route_plan, native/src/moe.rs:66-182) into
 * segments of 8 rows (fused kernel) or, from 12 slots per expert on, of 64 rows (tensor cores), so that an expert's
 * columns are decoded once per segment; rows are
 * processed in passes of at most 16384 slots.  No host synchronisation either way.
 * The workspace follows the rules of the linear layer's workspace. */
int b200exl3_moe_forward(const b200exl3_moe* handle, const void* d_x, int x_dtype, int64_t rows,
                         const uint32_t* d_selected, const void* d_scores, int score_dtype, void* d_y,
                         void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);

/* ---- layers with a fused prologue (fp16; 1 to 8 rows, the SwiGLU prologue alone any number of rows) --------------
 * The reference fuses the operators around a projection into its prologue kernels where dispatch count matters
 * (flash_up_finish_swiglu_prepare and its neighbours, native/shaders/exl3.metal:240-291).  Here the layer kernel's own
 * input rotation takes the operator in front of it:
 *   kind 1  RMSNorm: s = half(x + aux) (aux = residual rows or NULL), input = weight * half(s * rsqrt(mean(s^2) + eps));
 *           s is also stored to d_sum when that is not NULL (it must not be x: other warps still read x);
 *   kind 2  SwiGLU: input = half(half(x * half(sigmoid(x))) * aux), x = gate rows, aux = up rows.  With more than 8
 *           rows (prefill: the tensor-core product) it is applied by the input-rotation kernel, so a dense MLP block
 *           is [gate | up] -> down with no kernel between them.
 * Same arithmetic as b200exl3_rms_norm / b200exl3_swiglu followed by the plain forward; the row sum of the norm is added
 * in another order, so the last fp32 bit of 1/rms may differ from the stand-alone kernel's.  Kind 1 makes every warp
 * add up the whole row; the cheaper pairing is the residual EPILOGUE of the layer before (which already holds each
 * output block in registers) with a kind-3 prologue. */
typedef struct {
    int kind;
    const uint16_t* d_aux;
    const uint16_t* d_weight;
    uint16_t* d_sum;
    float eps;
    /* kind 3: RMSNorm of x whose sums of squares per 128-block, [rows, in / 128] fp32, were left in d_sumsq by the
     * residual epilogue of the layer before (d_weight and eps as for kind 1; no residual, nothing stored) */
    const float* d_sumsq;
    /* epilogue (plain layers only; 0 = none): 1 = the layer's output is added to the residual rows d_residual [rows,
     * out], the sum is stored to d_residual_out (may be d_residual itself) instead of d_y, and the sum of its squares
     * over every 128-block to d_sumsq_out [rows, out / 128] -- what the next layer's kind-3 prologue reads */
    int epilogue;
    const uint16_t* d_residual;
    uint16_t* d_residual_out;
    float* d_sumsq_out;
    /* epilogue 2 (a group of exactly three members [q | k | v] with 128-wide heads, one row): rotary embedding and
     * cache append in the kernel that produces q, k and v -- q heads are rotated by the angle of position *d_pos
     * (pairs (i, i + 64), frequency theta^(-2i/128), as b200exl3_rope_append does) and stored to the group's first
     * output, k heads are rotated into row *d_pos of d_k_cache [k heads, max_ctx, 128], v heads are copied into
     * d_v_cache; the group's second and third output pointers are not written */
    const int32_t* d_pos;
    float theta;
    int max_ctx;
    uint16_t* d_k_cache;
    uint16_t* d_v_cache;
} b200exl3_prologue;
typedef struct b200exl3_tp b200exl3_tp;
int b200exl3_linear_forward_fused(const b200exl3_linear* handle, const b200exl3_prologue* prologue, b200exl3_tp* tp_or_null,
                                  const void* d_x_f16, int64_t rows, void* d_y_f16, void* d_workspace, size_t workspace_bytes,
                                  b200exl3_stream stream);
int b200exl3_group_forward_fused(const b200exl3_group* handle, const b200exl3_prologue* prologue, const void* d_x_f16, int64_t rows,
                                 void* const* d_ys_f16, void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);

/* ---- a decode step as ONE launch -------------------------------------------------------------------------------
 * Replaces the reference's recorded decode step (mlxl3_replay_capture / mlxl3_replay_apply,
 * native/ffi/mlx_bridge.cpp:150-175): `count` (1..256) layers (Exl3Linear or Exl3Group), each with its input and output
 * pointers, become one object, and b200exl3_stack_forward runs them all, in order, in a single persistent kernel:
 * the result is what the per-layer forward calls issued in that order on one stream would give (same kernels'
 * arithmetic, same summation order), but the weight stream does not stop at layer boundaries and a boundary costs
 * a counter instead of a launch.  Layer i+1 may read anything layer i wrote.
 *   - all layers share bit width, codebook and weight mode; 1..2 activation rows in `x_dtype`; outputs in x_dtype;
 *   - pointers are fixed at creation (as a recorded graph fixes them); the object owns its scratch memory, so
 *     forward allocates nothing and can itself be recorded into a graph;
 *   - a layer with `tp` set is a row shard: its column-block sums are exchanged with the other ranks inside the
 *     kernel (all such layers of a step use the same context, all ranks run the same step);
 *   - every wait inside the kernel is bounded (option "stack_wait_ms", default 2000): b200exl3_stack_status reads
 *     0, or 1 (a weight copy never arrived), 2 (partition violated), 5 (a layer boundary was never reached);
 *     after a non-zero status call b200exl3_stack_reset before the next forward;
 *   - one forward at a time per object (calls on one stream, or otherwise ordered). */
typedef struct b200exl3_stack b200exl3_stack;
typedef struct {
    const b200exl3_linear* linear;   /* exactly one of linear and group */
    const b200exl3_group* group;
    const void* d_x;                 /* [rows, in] */
    void* d_y[8];                    /* one [rows, out] pointer per member (a plain layer uses d_y[0]) */
    b200exl3_tp* tp;                 /* NULL, or the exchange context of a row-parallel layer */
    /* NULL, or the operators fused around the layer as in b200exl3_linear_forward_fused / b200exl3_group_forward_fused
     * (fp16 steps): prologue kind 2 (SwiGLU) or 3 (RMSNorm from the block sums the layer before left), epilogue 1
     * (residual add + block sums; plain layers) or 2 (rotary embedding + cache append; a [q | k | v] group, one row).
     * Kind 1 is not taken: it needs the whole input row before the first block.  With these a decoder block's
     * o, [gate | up], down and the next block's [q | k | v] are one step. */
    const b200exl3_prologue* fused;
} b200exl3_stack_op;
int b200exl3_stack_create(const b200exl3_stack_op* ops, int count, int x_dtype, int64_t rows, b200exl3_stack** out);
void b200exl3_stack_free(b200exl3_stack* handle);
int b200exl3_stack_forward(b200exl3_stack* handle, b200exl3_stream stream);
int b200exl3_stack_status(const b200exl3_stack* handle, int* out_status);
int b200exl3_stack_reset(b200exl3_stack* handle);
/* CTAs of the persistent grid and dynamic shared memory per CTA (for reports). */
int b200exl3_stack_geometry(const b200exl3_stack* handle, int* out_grid, size_t* out_smem_bytes);

/* expert_mapped (native/src/linear.rs:2817-2851) as a stand-alone operator: row r = slot * projections + p of x [rows,
 * in] against the columns of expert selected[slot] of projection p in a bank trellis [in/16, source_tiles, 16k]
 * (checkpoint layout; projection p starts projection_stride_tiles tiles in, expert e another e * out/16).  The input is
 * rotated with its own row of d_suh [rows, in] unless input_pretransformed; the result is the raw fp32 product [rows,
 * out] (return_raw) or its output rotation scaled by the row's d_svh [rows, out], in x_dtype.  A tool-level call: it
 * re-lays the bank, allocates its temporaries and waits for the stream.  K = 7 is refused as in the reference. */
int b200exl3_expert_mapped(const void* d_x, int x_dtype, const uint16_t* d_trellis, int64_t source_tiles, const uint16_t* d_suh_f16,
                           const uint16_t* d_svh_f16, const uint32_t* d_selected, int64_t slots, int in, int out, int projections,
                           int64_t projection_stride_tiles, int k, int codebook, int input_pretransformed, int return_raw,
                           void* d_out, b200exl3_stream stream);
/* moe::swiglu_down_input (native/src/moe.rs:438-533): raw gate/up products [slots * 2, hidden] fp32 -> the rotated
 * input of the down projection [slots, hidden] fp16; gu_svh [experts, 2, hidden], down_suh [experts, hidden]. */
int b200exl3_swiglu_down_input(const float* d_gate_up_raw, const uint16_t* d_gu_svh_f16, const uint16_t* d_down_suh_f16,
                               const uint32_t* d_selected, int experts, int64_t slots, int hidden, uint16_t* d_xhat_f16,
                               b200exl3_stream stream);
/* moe::finish_and_reduce (native/src/moe.rs:586-609): y[row] = sum over the row's top_k slots, in order, of
 * half(H128(half(raw[slot]))) * svh[selected[slot]] * score[slot]; scores and y fp16 or fp32. */
int b200exl3_finish_and_reduce(const float* d_raw, const uint16_t* d_svh_f16, const uint32_t* d_selected, int experts,
                               const void* d_scores, int score_dtype, int64_t rows, int top_k, int out, void* d_y,
                               b200exl3_stream stream);

/* ---- expert parallelism for Exl3SwitchGlu -----------------------------------------------------------------------
 * No counterpart in the reference (it runs every expert on one device, native/src/moe.rs:905-971); the arithmetic of
 * a slot and of the final sum is the reference's (moe.rs:184-236 routed rotation, 586-609 finish_and_reduce), only
 * where a slot is computed changes.  Rank r owns experts [first_expert, first_expert + E_local): its b200exl3_moe
 * handle is created from that range's banks.  Every rank passes the same token rows, routes (GLOBAL expert ids) and
 * scores and receives the same output.  One call = plan (local slots, in slot order) -> dispatch (routed rotation of
 * those slots) -> local expert products and SwiGLU glue -> combine: owners publish their slots' rotated, scaled fp16
 * results into every rank's inbox over peer memory as {two values, sequence number} words, and every rank adds its
 * rows' top-k slot results in slot order.  No library collective, no separate exchange launch beyond these kernels.
 * Set-up mirrors the tensor-parallel context: every rank allocates an inbox of b200exl3_ep_buffer_bytes with
 * b200exl3_ipc_alloc, the host exchanges the 64-byte handles, opens the peers' inboxes with b200exl3_tp_open and passes
 * all `world` pointers (its own at index rank) to b200exl3_ep_create.  max_slots bounds rows * top_k of one pass (a
 * call with more rows runs in passes of b200exl3_moe's chunk).  Waits are bounded by the "tp_wait_ms" option; a wait
 * that gives up sets status 7 (b200exl3_ep_status). */
typedef struct b200exl3_ep b200exl3_ep;
int b200exl3_ipc_alloc(size_t bytes, void** out_buffer, unsigned char* out_handle64);
int b200exl3_ep_buffer_bytes(int max_slots, int out, size_t* out_bytes);
int b200exl3_ep_create(int rank, int world, int max_slots, int out, void* const* buffers, b200exl3_ep** out_handle);
void b200exl3_ep_free(b200exl3_ep* handle);
int b200exl3_ep_status(const b200exl3_ep* handle, int* out_status);
int b200exl3_moe_ep_workspace_bytes(const b200exl3_moe* local_experts, int64_t rows, size_t* out_bytes);
int b200exl3_moe_forward_ep(const b200exl3_moe* local_experts, b200exl3_ep* ep, int first_expert, const void* d_x, int x_dtype,
                            int64_t rows, const uint32_t* d_selected, const void* d_scores, int score_dtype, void* d_y,
                            void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);

/* ---- decoder-block glue: fp16, one token per call (batch-1 decode) ----------------------------------------------
 * The operators a decoder block runs between its quantized projections (call order: native/src/lfm2.rs:704-793), as
 * the reference reaches them through MLX (native/src/array.rs:1517-1519 rope, 1662-1664 rms_norm, 1741-1743 swiglu,
 * 1766-1777 sdpa; native/ffi/mlx_bridge.cpp:678, 743, 745-750, 846-849).  All tensors are fp16 device arrays;
 * positions and token ids live in device memory so that a recorded step can be replayed while they advance. */

/* out[r, :] = table[tokens[r], :]  (ids are clamped to the table) */
int b200exl3_embed(const uint16_t* d_table_f16, const int32_t* d_tokens, int64_t rows, int64_t vocab, int hidden,
                   uint16_t* d_out_f16, b200exl3_stream stream);
/* s = half(x + residual) (d_residual may be NULL; s is stored to d_sum when that is not NULL; d_sum may alias either
 * input); y = weight * half(s * rsqrt(mean(s^2) + eps)), fp32 inside, as fast::rms_norm.  n <= 49152. */
int b200exl3_rms_norm(const uint16_t* d_x_f16, const uint16_t* d_residual_f16, const uint16_t* d_weight_f16, int64_t rows,
                      int n, float eps, uint16_t* d_sum_f16, uint16_t* d_y_f16, b200exl3_stream stream);
/* out = half(half(gate * half(sigmoid(gate))) * up) */
int b200exl3_swiglu(const uint16_t* d_gate_f16, const uint16_t* d_up_f16, int64_t n, uint16_t* d_out_f16, b200exl3_stream stream);
/* Rotary embedding of the new token's heads at position *d_pos (pairs (i, i + head_dim/2), base theta): q [heads,
 * head_dim] is rotated in place; the rotated k and v [kv_heads, head_dim] are written to row *d_pos of the caches
 * [kv_heads, max_ctx, head_dim]. */
int b200exl3_rope_append(uint16_t* d_q_f16, const uint16_t* d_k_f16, const uint16_t* d_v_f16, int heads, int kv_heads,
                         int head_dim, const int32_t* d_pos, float theta, int max_ctx, uint16_t* d_k_cache_f16,
                         uint16_t* d_v_cache_f16, b200exl3_stream stream);
/* softmax(q k^T * scale) v for one query row per head against keys 0..*d_pos of the caches (grouped-query: heads /
 * kv_heads query heads share a key head), fp32 inside, split over the context and merged in split order by the last
 * CTA to arrive: one launch; head_dim must be 128.  The workspace starts with arrival counters: clear it
 * once before the first call (b200exl3_memset); every call leaves them zero.  Calls that overlap on the
 * GPU need workspaces of their own. */
int b200exl3_attention_workspace_bytes(int heads, int kv_heads, size_t* out_bytes);
int b200exl3_attention_decode(const uint16_t* d_q_f16, const uint16_t* d_k_cache_f16, const uint16_t* d_v_cache_f16, int heads,
                              int kv_heads, int head_dim, const int32_t* d_pos, int max_ctx, float scale, uint16_t* d_out_f16,
                              void* d_workspace, size_t workspace_bytes, b200exl3_stream stream);
/* fp16 vocabulary head: logits [vocab] = half(x [hidden] . weight [vocab, hidden]) (stored when d_logits is not NULL)
 * and their arg-max (first index on ties) as (*d_best_value, *d_best_index + index_offset); a vocabulary shard passes
 * its first row as index_offset. */
int b200exl3_head_workspace_bytes(size_t* out_bytes);
int b200exl3_head_argmax(const uint16_t* d_x_f16, const uint16_t* d_weight_f16, int64_t vocab, int hidden, int64_t index_offset,
                         uint16_t* d_logits_f16, float* d_best_value, int64_t* d_best_index, void* d_workspace,
                         size_t workspace_bytes, b200exl3_stream stream);

/* ---- router: stable top-k ----------------------------------------------------------------------------------
 * Replaces router::topk / routes (native/src/router.rs:28-120, native/shaders/router_topk.h:1-34): values
 * [rows, experts] (fp16 = 9 or fp32 = 10, experts <= 1024) -> indices [rows, top_k] (u32) and scores
 * [rows, top_k] in the values' dtype.  Per row the top_k largest values in ascending order (the best last); equal
 * values go to the higher expert index, +0 and -0 compare equal, NaN ranks above every number.  With `normalize`
 * the scores are divided by their sum, added in slot order in the values' own type.  The outputs feed
 * b200exl3_moe_forward directly, on the device. */
int b200exl3_router_topk(const void* d_values, int dtype, int64_t rows, int experts, int top_k, int normalize,
                         uint32_t* d_indices, void* d_scores, b200exl3_stream stream);
/* The same on logits: routes are taken on the row softmax of d_logits, computed in fp32 and rounded to `dtype` as
 * the reference's softmax_precise() does (native/src/qwen35.rs:214, 240: topk(&logits.softmax_precise(), k, true));
 * d_probabilities [rows, experts] receives the softmax when it is not NULL.  One pass: a warp per token row. */
int b200exl3_router_softmax_topk(const void* d_logits, int dtype, int64_t rows, int experts, int top_k, int normalize,
                                 uint32_t* d_indices, void* d_scores, void* d_probabilities, b200exl3_stream stream);
/* Router gate product (the plain fp16 linear in front of the router, `self.gate.forward(x)`, native/src/qwen35.rs:207-213,
 * 240): logits [rows, experts] fp16 = x [rows, in] times weight [experts, in] fp16, fp32 accumulation. */
int b200exl3_router_gate(const void* d_x, int x_dtype, const uint16_t* d_weight_f16, int64_t rows, int in, int experts,
                         uint16_t* d_logits_f16, b200exl3_stream stream);

/* ---- tensor parallelism over peer memory (one process per GPU of one node) -----------------------------------
 * No counterpart in the reference (single GPU).  Column-parallel shards need nothing from here.  A row-parallel
 * shard computes its fp32 partial product with b200exl3_linear_forward_partial; b200exl3_linear_finish_tp then
 * replaces "all-reduce + b200exl3_linear_finish" by one kernel: every rank stores its partial sums into all
 * ranks' exchange buffers over NVLink as 8-byte {value, sequence number} words (no fence, no flag), polls its
 * own buffer (bounded, about four seconds) until the other ranks' words of this call have arrived, adds them in
 * rank order in fp32 (the reference's split-K sum, native/src/linear.rs:978-982; every rank gets the same bits)
 * and applies the output rotation.  It is a plain kernel launch: it can be recorded into a graph.
 *
 * Set-up: every rank calls b200exl3_tp_alloc (buffer + 64-byte IPC handle), the host exchanges the handles by
 * its own means, opens the other ranks' buffers with b200exl3_tp_open, and passes all `world` buffers (its own
 * at index `rank`) to b200exl3_tp_create.  max_units bounds rows * out / 128 of any layer finished through the
 * context.  All ranks must issue the same sequence of b200exl3_linear_finish_tp calls.  A rank polls for its
 * peers' sums for at most four seconds (option "tp_wait_ms": 1..60000); a wait that gives up sets the
 * context's status to 4 (b200exl3_tp_status) instead of hanging, the kernel returns with what it has, and
 * later waits of that context give up after a few hundred polls.  The ranks' use counts may then disagree:
 * once every rank has stopped launching, each calls b200exl3_tp_reset (own inbox, use counts and status back
 * to zero; synchronises the device) before the context is used again, or the contexts are rebuilt. */
int b200exl3_tp_buffer_bytes(int world, int max_units, size_t* out_bytes);
int b200exl3_tp_alloc(int world, int max_units, void** out_buffer, unsigned char* out_handle64);
int b200exl3_tp_open(const unsigned char* handle64, void** out_peer_buffer);
int b200exl3_tp_close(void* peer_buffer);
int b200exl3_tp_create(int rank, int world, int max_units, void* const* buffers, b200exl3_tp** out);
void b200exl3_tp_free(b200exl3_tp* handle);
int b200exl3_tp_status(const b200exl3_tp* handle, int* out_status);
int b200exl3_tp_reset(b200exl3_tp* handle);
/* The whole row-parallel layer in one launch: input rotation of this rank's input slice, product, exchange of
 * the partial sums with the other ranks inside the kernel's final reduction, output rotation.  Same result as
 * b200exl3_linear_forward_partial followed by b200exl3_linear_finish_tp.  Up to 8 rows this is one launch; from 9 rows
 * on the product runs on the tensor cores with a single input split and the exchange kernel follows it. */
int b200exl3_linear_forward_tp(const b200exl3_linear* handle, b200exl3_tp* tp, const void* d_x, int x_dtype,
                               int64_t rows, void* d_y, void* d_workspace, size_t workspace_bytes,
                               b200exl3_stream stream);
int b200exl3_linear_finish_tp(const b200exl3_linear* handle, b200exl3_tp* tp, const float* d_yhat, int64_t rows,
                              int y_dtype, void* d_y, b200exl3_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200EXL3_H */
