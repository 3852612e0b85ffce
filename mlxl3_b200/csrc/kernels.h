// Internal launcher declarations shared by the kernel translation units and the C ABI layer.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200exl3 {

// ---- codec (kernels_codec.cu) ---------------------------------------------------------------------
cudaError_t launch_unpack_states(const uint16_t* packed, int64_t tiles, int k, int cb, uint16_t* states, __half* values,
                                 cudaStream_t stream);
cudaError_t launch_codebook(const uint16_t* states, int64_t n, int cb, __half* values, cudaStream_t stream);
cudaError_t launch_reconstruct(const uint16_t* trellis, int tiles_k, int tiles_n, int k, int cb, __half* w,
                               cudaStream_t stream);

// ---- rotations (kernels_rotate.cu) ----------------------------------------------------------------
// xhat[r, :] = H128(half(half(x[r, :]) * suh[(r % scale_rows), :])); scale_rows is 1 or rows.
cudaError_t launch_prepare(const void* x, int x_dtype, const __half* suh, int64_t scale_rows, int64_t rows, int in,
                           __half* xhat, cudaStream_t stream);
// y = half(H128(half(sum_s partials[s, r, :]))) * svh (+ bias), written in y_dtype.
cudaError_t launch_finish(const float* partials, int splits, int64_t split_stride, const __half* svh,
                          int64_t scale_rows, const __half* bias, int64_t rows, int out, int y_dtype, void* y,
                          cudaStream_t stream);

// ---- fused product (kernels_qmv.cu) ---------------------------------------------------------------
struct QmvPlan {
    int splits;          // split-K factor: partial sums per output element
    int warps;           // warps per CTA
    int col_blocks;      // out / 128
    size_t smem_bytes;   // dynamic shared memory per CTA
};
QmvPlan plan_qmv(int in, int out, int k, int64_t rows);
// partials[s, r, n] (fp32, r < rows <= 32) = sum over split s of xhat[r, :] . W[:, n]
// exact: decode the reference's fp16 weight bit for bit before multiplying (codebooks 0/1 default to
// feeding the two fp16 halves of a weight as two products, which differs by fp16 rounding of the weight).
cudaError_t launch_qmv(const uint16_t* trellis, int in, int out, int k, int cb, const __half* xhat, int64_t rows,
                       bool exact, const QmvPlan& plan, float* partials, cudaStream_t stream);
void qmv_set_tuning(int ctas_per_sm, int force_splits);

}  // namespace b200exl3
