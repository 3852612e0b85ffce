// Decoder-block glue around the quantized projections, for batch-1 decode in fp16: embedding row, RMSNorm (with the
// residual add folded in), RoPE + KV-cache append, grouped-query decode attention over an fp16 cache, SwiGLU, and
// the fp16 vocabulary head with its arg-max.
//
// Reference behaviour (the call order of a decoder block: native/src/lfm2.rs:704-793; the array operators it calls:
// native/src/array.rs:1517-1519 rope, 1662-1664 rms_norm, 1741-1743 swiglu, 1766-1777 sdpa, which the bridge maps to
// MLX's fast::rope (non-traditional: pairs (i, i + dims/2)), fast::rms_norm, a compiled x * sigmoid(x) * up and
// fast::scaled_dot_product_attention, native/ffi/mlx_bridge.cpp:678, 743, 745-750, 846-849).  MLX is a third-party
// dependency that is not part of the reference tree: its published arithmetic is restated here (fp32 inside every
// operator, one rounding to fp16 at each operator's output; rms_norm rounds the normalised value before it
// multiplies by the weight), and no stored reference output pins the last bit.
//
// All of these are bound by HBM bandwidth or by launch latency; none is a contraction worth tensor cores.
#include "hadamard.cuh"
#include "kernels.h"

#include <algorithm>
#include <climits>

namespace b200exl3 {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// ---- embedding row ----------------------------------------------------------------------------------------
__global__ void embed_kernel(const __half* __restrict__ table, const int* __restrict__ token, int64_t vocab, int hidden,
                             __half* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    int64_t id = token[blockIdx.x];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + id * hidden);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<int64_t>(blockIdx.x) * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// ---- RMSNorm, optionally after a residual add ---------------------------------------------------------------
// s = half(x + residual) (stored to `sum` when given); y = weight * half(s * rsqrt(mean(s^2) + eps)).  One CTA per row.
constexpr int kNormThreads = 256;
__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ residual, const __half* __restrict__ weight, int n,
                float eps, __half* __restrict__ sum, __half* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __half s_row[];                    // the (summed) row, kept for the second pass
    __shared__ float s_part[kNormThreads / 32];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * n;
    float acc = 0.0f;
    for (int i = threadIdx.x * 2; i < n; i += kNormThreads * 2) {
        __half2 v = *reinterpret_cast<const __half2*>(x + base + i);
        if (residual != nullptr) v = __hadd2_rn(v, *reinterpret_cast<const __half2*>(residual + base + i));
        *reinterpret_cast<__half2*>(s_row + i) = v;
        if (sum != nullptr) *reinterpret_cast<__half2*>(sum + base + i) = v;
        const float2 f = __half22float2(v);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += s_part[w];
    const float inv = rsqrtf(total / static_cast<float>(n) + eps);
    for (int i = threadIdx.x * 2; i < n; i += kNormThreads * 2) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(s_row + i));
        const __half2 normed = __floats2half2_rn(f.x * inv, f.y * inv);
        *reinterpret_cast<__half2*>(y + base + i) = __hmul2_rn(*reinterpret_cast<const __half2*>(weight + i), normed);
    }
}

// ---- SwiGLU --------------------------------------------------------------------------------------------------
// out = half(half(x * half(sigmoid(x))) * up): the three fp16 operators of the reference's compiled expression.
__global__ void swiglu_kernel(const __half* __restrict__ gate, const __half* __restrict__ up, int64_t n, __half* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const __half2 g = *reinterpret_cast<const __half2*>(gate + i);
    const float2 f = __half22float2(g);
    const __half2 s = __floats2half2_rn(1.0f / (1.0f + expf(-f.x)), 1.0f / (1.0f + expf(-f.y)));
    *reinterpret_cast<__half2*>(out + i) = __hmul2_rn(__hmul2_rn(g, s), *reinterpret_cast<const __half2*>(up + i));
}

// ---- RoPE and KV-cache append -----------------------------------------------------------------------------------
// One warp per head (query heads first, then key heads, then value heads).  Rotation of the pairs (i, i + dim/2) by the
// angle pos * theta^(-2i/dim), computed in fp32 and rounded once.  Queries are rotated in place; keys are rotated into
// the cache row `pos` of their head; values are copied there.
__global__ void rope_append_kernel(__half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v, int heads,
                                   int kv_heads, int dim, const int* __restrict__ pos_ptr, float log2_theta, int max_ctx,
                                   __half* __restrict__ k_cache, __half* __restrict__ v_cache) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (head >= heads + 2 * kv_heads) return;
    int pos = *pos_ptr;
    pos = pos < 0 ? 0 : (pos >= max_ctx ? max_ctx - 1 : pos);
    const int half_dim = dim / 2;
    if (head >= heads + kv_heads) {                       // value head: copy
        const int h = head - heads - kv_heads;
        const __half* src = v + h * dim;
        __half* dst = v_cache + (static_cast<int64_t>(h) * max_ctx + pos) * dim;
        for (int i = lane * 2; i < dim; i += 64) *reinterpret_cast<__half2*>(dst + i) = *reinterpret_cast<const __half2*>(src + i);
        return;
    }
    const bool is_q = head < heads;
    const __half* src = is_q ? q + head * dim : k + (head - heads) * dim;
    __half* dst = is_q ? q + head * dim : k_cache + (static_cast<int64_t>(head - heads) * max_ctx + pos) * dim;
    for (int i = lane; i < half_dim; i += 32) {
        const float inv_freq = exp2f(-log2_theta * static_cast<float>(2 * i) / static_cast<float>(dim));
        float sn, cs;
        sincosf(static_cast<float>(pos) * inv_freq, &sn, &cs);
        const float a = __half2float(src[i]), b = __half2float(src[i + half_dim]);
        const __half ra = __float2half_rn(a * cs - b * sn), rb = __float2half_rn(a * sn + b * cs);
        dst[i] = ra;
        dst[i + half_dim] = rb;
    }
}

}  // namespace

// ---- grouped-query decode attention (one new token against the cache), split over the context ----------------------
// CTA (split s, key head h, pass p): up to four query heads that share key head h against keys [chunk s).  A lane is
// (key slot kg = lane / 8, slice j = lane % 8): a warp instruction loads four whole 256-byte cache rows, fully
// coalesced, and lane (kg, j) holds 16 of the 128 dimensions of key kg.  Scores are reduced over the 8 slices with
// three shuffles for all four keys at once; the softmax is the online form in fp32; the partial result of a CTA is
// (max, sum, unnormalised output) per query head.  The CTAs of a (key head, pass) count their arrivals; the last one
// merges the splits in split order and normalises, so the result does not depend on who was last and the whole
// attention is one launch.  The counters live in the caller's workspace: zero before the first use, zero after every call.
namespace {

constexpr int kAttnDim = 128;
constexpr int kAttnWarps = 4;
constexpr int kAttnHeadsPerPass = 4;

__global__ void __launch_bounds__(kAttnWarps * 32)
attention_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
                    int heads, int kv_heads, const int* __restrict__ pos_ptr, int max_ctx, float scale_log2e,
                    float* __restrict__ part_acc, float2* __restrict__ part_ml, unsigned int* __restrict__ arrived,
                    __half* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int GQ = kAttnHeadsPerPass;
    __shared__ float s_acc[kAttnWarps][GQ][kAttnDim];
    __shared__ float s_m[kAttnWarps][GQ], s_l[kAttnWarps][GQ];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, kg = lane >> 3, j = lane & 7;
    const int group = heads / kv_heads, passes = (group + GQ - 1) / GQ;
    const int split = blockIdx.x, splits = gridDim.x;
    const int kvh = blockIdx.y / passes, pass = blockIdx.y - kvh * passes;
    const int head0 = kvh * group + pass * GQ;
    const int nheads = min(GQ, group - pass * GQ);
    int nkeys = *pos_ptr + 1;
    nkeys = nkeys < 1 ? 1 : (nkeys > max_ctx ? max_ctx : nkeys);
    const int chunk = (nkeys + splits - 1) / splits;
    const int key0 = split * chunk, key1 = min(nkeys, key0 + chunk);

    float qv[GQ][16];
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
        const __half* src = q + static_cast<int64_t>(head0 + min(h, nheads - 1)) * kAttnDim + j * 16;
        const uint4 a = *reinterpret_cast<const uint4*>(src), b = *reinterpret_cast<const uint4*>(src + 8);
        const __half2* ha = reinterpret_cast<const __half2*>(&a);
        const __half2* hb = reinterpret_cast<const __half2*>(&b);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __half22float2(ha[i]), fb = __half22float2(hb[i]);
            qv[h][2 * i] = fa.x * scale_log2e; qv[h][2 * i + 1] = fa.y * scale_log2e;
            qv[h][8 + 2 * i] = fb.x * scale_log2e; qv[h][8 + 2 * i + 1] = fb.y * scale_log2e;
        }
    }
    float m[GQ], l[GQ], acc[GQ][16];
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
        for (int d = 0; d < 16; ++d) acc[h][d] = 0.0f;
    }
    const __half* kbase = k_cache + static_cast<int64_t>(kvh) * max_ctx * kAttnDim + j * 16;
    const __half* vbase = v_cache + static_cast<int64_t>(kvh) * max_ctx * kAttnDim + j * 16;
    // the rows of the NEXT round are requested before this round's arithmetic: a chunk is three or four rounds, and a
    // round that waits for its own loads costs a trip to memory each time
    uint4 nka, nkb, nva, nvb;
    auto request = [&](int first) {
        const int key = first + kg;
        const int64_t at = static_cast<int64_t>(key < key1 ? key : key1 - 1) * kAttnDim;
        nka = __ldcs(reinterpret_cast<const uint4*>(kbase + at)); nkb = __ldcs(reinterpret_cast<const uint4*>(kbase + at + 8));
        nva = __ldcs(reinterpret_cast<const uint4*>(vbase + at)); nvb = __ldcs(reinterpret_cast<const uint4*>(vbase + at + 8));
    };
    if (key0 + warp * 4 < key1) request(key0 + warp * 4);
#pragma unroll 1
    for (int first = key0 + warp * 4; first < key1; first += kAttnWarps * 4) {
        const int key = first + kg;
        const bool valid = key < key1;
        const uint4 ka = nka, kb = nkb, va = nva, vb = nvb;
        if (first + kAttnWarps * 4 < key1) request(first + kAttnWarps * 4);
        float kf[16], vf[16];
        {
            const __half2* h0 = reinterpret_cast<const __half2*>(&ka);
            const __half2* h1 = reinterpret_cast<const __half2*>(&kb);
            const __half2* g0 = reinterpret_cast<const __half2*>(&va);
            const __half2* g1 = reinterpret_cast<const __half2*>(&vb);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 f = __half22float2(h0[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y;
                f = __half22float2(h1[i]); kf[8 + 2 * i] = f.x; kf[8 + 2 * i + 1] = f.y;
                f = __half22float2(g0[i]); vf[2 * i] = f.x; vf[2 * i + 1] = f.y;
                f = __half22float2(g1[i]); vf[8 + 2 * i] = f.x; vf[8 + 2 * i + 1] = f.y;
            }
        }
#pragma unroll
        for (int h = 0; h < GQ; ++h) {
            float s = 0.0f;
#pragma unroll
            for (int d = 0; d < 16; ++d) s = fmaf(qv[h][d], kf[d], s);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (valid) {                                        // scores are in log2 units: exp2 throughout
                const float m_new = fmaxf(m[h], s);
                const float corr = exp2f(m[h] - m_new), p = exp2f(s - m_new);
                m[h] = m_new;
                l[h] = fmaf(l[h], corr, p);
#pragma unroll
                for (int d = 0; d < 16; ++d) acc[h][d] = fmaf(acc[h][d], corr, p * vf[d]);
            }
        }
    }
    // ---- merge the four key slots of the warp (lanes that hold the same slice), then the warps, in a fixed order ----
#pragma unroll
    for (int h = 0; h < GQ; ++h) {
#pragma unroll
        for (int step = 8; step <= 16; step <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m[h], step), l_o = __shfl_xor_sync(0xffffffffu, l[h], step);
            const float m_new = fmaxf(m[h], m_o);
            const float c_self = m[h] == -INFINITY ? 0.0f : exp2f(m[h] - m_new), c_o = m_o == -INFINITY ? 0.0f : exp2f(m_o - m_new);
            l[h] = l[h] * c_self + l_o * c_o;
#pragma unroll
            for (int d = 0; d < 16; ++d) {
                const float a_o = __shfl_xor_sync(0xffffffffu, acc[h][d], step);
                acc[h][d] = acc[h][d] * c_self + a_o * c_o;
            }
            m[h] = m_new;
        }
        if (kg == 0) {
#pragma unroll
            for (int d = 0; d < 16; ++d) s_acc[warp][h][j * 16 + d] = acc[h][d];
            if (j == 0) { s_m[warp][h] = m[h]; s_l[warp][h] = l[h]; }
        }
    }
    __syncthreads();
    // thread t owns dimension t of every head of the pass
    const int d = threadIdx.x;
    for (int h = 0; h < nheads; ++h) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_m[w][h]);
        float ll = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float c = s_m[w][h] == -INFINITY ? 0.0f : exp2f(s_m[w][h] - mm);
            ll = fmaf(s_l[w][h], c, ll);
            o = fmaf(s_acc[w][h][d], c, o);
        }
        const int64_t slot = static_cast<int64_t>(head0 + h) * splits + split;
        part_acc[slot * kAttnDim + d] = o;
        if (d == 0) part_ml[slot] = make_float2(mm, ll);
    }
    // ---- the last CTA of this (key head, pass) merges the splits: thread d owns dimension d --------------------------
    __shared__ bool s_last;
    __threadfence();                                            // this CTA's partials before its arrival
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int before = atomicAdd(arrived + blockIdx.y, 1u);
        s_last = before + 1 == static_cast<unsigned int>(splits);
        if (s_last) arrived[blockIdx.y] = 0;                    // the next call starts from zero
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // warp h merges query head h: lane i weighs splits i and i + 32 (at most 64 splits), then every lane adds its four
    // dimensions over the splits in split order, sixteen loads in flight
    if (warp < nheads) {
        const int64_t base = static_cast<int64_t>(head0 + warp) * splits;
        const float2 ml0 = lane < splits ? __ldcg(&part_ml[base + lane]) : make_float2(-INFINITY, 0.0f);
        const float2 ml1 = lane + 32 < splits ? __ldcg(&part_ml[base + lane + 32]) : make_float2(-INFINITY, 0.0f);
        float mm = fmaxf(ml0.x, ml1.x);
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, step));
        const float c0 = ml0.x == -INFINITY ? 0.0f : exp2f(ml0.x - mm), c1 = ml1.x == -INFINITY ? 0.0f : exp2f(ml1.x - mm);
        float ll = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* acc_base = part_acc + base * kAttnDim + lane * 4;
#pragma unroll 1
        for (int s0 = 0; s0 < splits; s0 += 16) {
            float4 part[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (s0 + i < splits) part[i] = __ldcg(reinterpret_cast<const float4*>(acc_base + static_cast<int64_t>(s0 + i) * kAttnDim));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int sp = s0 + i;                                              // uniform over the warp
                const float c = __shfl_sync(0xffffffffu, sp < 32 ? c0 : c1, sp & 31);
                const float l_s = __shfl_sync(0xffffffffu, sp < 32 ? ml0.y : ml1.y, sp & 31);
                if (sp < splits) {
                    ll = fmaf(l_s, c, ll);
                    o.x = fmaf(part[i].x, c, o.x); o.y = fmaf(part[i].y, c, o.y);
                    o.z = fmaf(part[i].z, c, o.z); o.w = fmaf(part[i].w, c, o.w);
                }
            }
        }
        const float inv = 1.0f / ll;
        const __half2 lo = __floats2half2_rn(o.x * inv, o.y * inv), hi = __floats2half2_rn(o.z * inv, o.w * inv);
        *reinterpret_cast<uint2*>(out + static_cast<int64_t>(head0 + warp) * kAttnDim + lane * 4) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

}  // namespace

// ---- fp16 vocabulary head and arg-max -------------------------------------------------------------------------------
// logits[v] = half(sum_i float(x[i]) * float(W[v, i])).  One warp per vocabulary row at a time (a row is read once, 16
// bytes per lane and step, fully coalesced); the activation row sits in shared memory.  Every warp keeps the best
// (logit, index) of its rows -- the first index wins a tie, as an arg-max over the fp16 logits does -- and the CTA writes
// one candidate; a second one-CTA kernel picks among the candidates.
namespace {

constexpr int kHeadWarps = 8;

__device__ __forceinline__ bool better(float v, int64_t i, float bv, int64_t bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(kHeadWarps * 32)
head_kernel(const __half* __restrict__ x, const __half* __restrict__ w, int64_t vocab, int hidden, int64_t index_offset,
            __half* __restrict__ logits, float* __restrict__ cand_value, long long* __restrict__ cand_index) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) __half s_x[];
    __shared__ float s_v[kHeadWarps];
    __shared__ long long s_i[kHeadWarps];
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) reinterpret_cast<uint4*>(s_x)[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float best_v = -INFINITY;
    int64_t best_i = INT64_MAX;
    // Two rows per round and eight loads per lane in flight: the kernel streams 1 GB, so what counts is how many bytes
    // each warp keeps on their way.  Every row's sum is still added in the same order (lane-strided, then the warp sum).
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kHeadWarps;
    const int steps = hidden / 8;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * kHeadWarps + warp; row < vocab; row += 2 * stride) {
        const bool two = row + stride < vocab;
        const uint4* wr0 = reinterpret_cast<const uint4*>(w + row * hidden);
        const uint4* wr1 = reinterpret_cast<const uint4*>(w + (two ? row + stride : row) * hidden);
        float acc0 = 0.0f, acc1 = 0.0f;
        int i = lane;
        for (; i + 96 < steps; i += 128) {
            uint4 wa[4], wb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { wa[u] = __ldcs(wr0 + i + 32 * u); wb[u] = __ldcs(wr1 + i + 32 * u); }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint4 xv = reinterpret_cast<const uint4*>(s_x)[i + 32 * u];
                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
                const __half2* ah = reinterpret_cast<const __half2*>(&wa[u]);
                const __half2* bh = reinterpret_cast<const __half2*>(&wb[u]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 b = __half22float2(xh[j]), a0 = __half22float2(ah[j]), a1 = __half22float2(bh[j]);
                    acc0 = fmaf(a0.x, b.x, acc0); acc0 = fmaf(a0.y, b.y, acc0);
                    acc1 = fmaf(a1.x, b.x, acc1); acc1 = fmaf(a1.y, b.y, acc1);
                }
            }
        }
        for (; i < steps; i += 32) {
            const uint4 va = __ldcs(wr0 + i), vb = __ldcs(wr1 + i);
            const uint4 xv = reinterpret_cast<const uint4*>(s_x)[i];
            const __half2* xh = reinterpret_cast<const __half2*>(&xv);
            const __half2* ah = reinterpret_cast<const __half2*>(&va);
            const __half2* bh = reinterpret_cast<const __half2*>(&vb);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 b = __half22float2(xh[j]), a0 = __half22float2(ah[j]), a1 = __half22float2(bh[j]);
                acc0 = fmaf(a0.x, b.x, acc0); acc0 = fmaf(a0.y, b.y, acc0);
                acc1 = fmaf(a1.x, b.x, acc1); acc1 = fmaf(a1.y, b.y, acc1);
            }
        }
        acc0 = warp_sum(acc0);
        acc1 = warp_sum(acc1);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r == 1 && !two) break;
            const int64_t at = row + r * stride;
            const __half rounded = __float2half_rn(r == 0 ? acc0 : acc1);
            if (lane == 0 && logits != nullptr) logits[at] = rounded;
            const float v = __half2float(rounded);
            if (better(v, at + index_offset, best_v, best_i)) { best_v = v; best_i = at + index_offset; }
        }
    }
    if (lane == 0) { s_v[warp] = best_v; s_i[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int wv = 1; wv < kHeadWarps; ++wv)
            if (better(s_v[wv], s_i[wv], best_v, best_i)) { best_v = s_v[wv]; best_i = s_i[wv]; }
        cand_value[blockIdx.x] = best_v;
        cand_index[blockIdx.x] = best_i;
    }
}

__global__ void __launch_bounds__(256)
argmax_candidates_kernel(const float* __restrict__ cand_value, const long long* __restrict__ cand_index, int n,
                         float* __restrict__ out_value, long long* __restrict__ out_index) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float s_v[8];
    __shared__ long long s_i[8];
    float best_v = -INFINITY;
    int64_t best_i = INT64_MAX;
    for (int i = threadIdx.x; i < n; i += 256)
        if (better(cand_value[i], cand_index[i], best_v, best_i)) { best_v = cand_value[i]; best_i = cand_index[i]; }
    // "better" is a total order on (value, index) pairs, so the reduction tree gives the same winner as a serial scan
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, d);
        const long long oi = __shfl_xor_sync(0xffffffffu, static_cast<long long>(best_i), d);
        if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best_v; s_i[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i)
            if (better(s_v[i], s_i[i], best_v, best_i)) { best_v = s_v[i]; best_i = s_i[i]; }
        *out_value = best_v;
        *out_index = best_i;
    }
}

}  // namespace

// ---- launchers -----------------------------------------------------------------------------------------------------

cudaError_t launch_embed(const __half* table, const int* token, int64_t rows, int64_t vocab, int hidden, __half* out, cudaStream_t stream) {
    return launch_dependent(embed_kernel, dim3(static_cast<unsigned>(rows)), dim3(128), 0, stream, table, token, vocab, hidden, out);
}

cudaError_t launch_rms_norm(const __half* x, const __half* residual, const __half* weight, int64_t rows, int n, float eps, __half* sum,
                            __half* y, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(n) * sizeof(__half);
    if (smem > 96 * 1024) return cudaErrorInvalidValue;
    static PerDeviceOnce attribute;
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(rms_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        attribute.mark();
    }
    return launch_dependent(rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), smem, stream, x, residual, weight, n, eps, sum, y);
}

cudaError_t launch_swiglu(const __half* gate, const __half* up, int64_t n, __half* out, cudaStream_t stream) {
    const int64_t threads = (n + 1) / 2;
    return launch_dependent(swiglu_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, stream, gate, up, n, out);
}

cudaError_t launch_rope_append(__half* q, const __half* k, const __half* v, int heads, int kv_heads, int dim, const int* pos, float theta,
                               int max_ctx, __half* k_cache, __half* v_cache, cudaStream_t stream) {
    const int total = heads + 2 * kv_heads;
    return launch_dependent(rope_append_kernel, dim3((total + 3) / 4), dim3(128), 0, stream, q, k, v, heads, kv_heads, dim, pos, log2f(theta), max_ctx,
                            k_cache, v_cache);
}

int attention_splits(int kv_heads, int heads) {
    const int passes = (heads / kv_heads + kAttnHeadsPerPass - 1) / kAttnHeadsPerPass;
    const int per_split = kv_heads * passes;
    return std::max(1, std::min(64, (2 * sm_count() + per_split - 1) / per_split));
}

size_t attention_workspace_bytes(int heads, int kv_heads) {
    const size_t splits = static_cast<size_t>(attention_splits(kv_heads, heads));
    const size_t passes = (heads / kv_heads + kAttnHeadsPerPass - 1) / kAttnHeadsPerPass;
    // [arrival counters, one per (key head, pass): zero before the first use | partial outputs | partial (max, sum)]
    return 256 * ((kv_heads * passes * sizeof(unsigned int) + 255) / 256) + heads * splits * (kAttnDim * sizeof(float) + sizeof(float2));
}

cudaError_t launch_attention_decode(const __half* q, const __half* k_cache, const __half* v_cache, int heads, int kv_heads, int dim,
                                    const int* pos, int max_ctx, float scale, __half* out, void* workspace, cudaStream_t stream) {
    if (dim != kAttnDim || kv_heads <= 0 || heads % kv_heads) return cudaErrorInvalidValue;
    const int splits = attention_splits(kv_heads, heads);
    const int passes = (heads / kv_heads + kAttnHeadsPerPass - 1) / kAttnHeadsPerPass;
    unsigned int* arrived = static_cast<unsigned int*>(workspace);
    float* part_acc = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256 * ((kv_heads * passes * sizeof(unsigned int) + 255) / 256));
    float2* part_ml = reinterpret_cast<float2*>(part_acc + static_cast<size_t>(heads) * splits * kAttnDim);
    return launch_dependent(attention_decode_kernel, dim3(splits, kv_heads * passes), dim3(kAttnWarps * 32), 0, stream, q, k_cache, v_cache,
                            heads, kv_heads, pos, max_ctx, scale * 1.4426950408889634f, part_acc, part_ml, arrived, out);
}

int head_candidates() { return 4 * sm_count(); }

cudaError_t launch_head_argmax(const __half* x, const __half* w, int64_t vocab, int hidden, int64_t index_offset, __half* logits,
                               float* cand_value, long long* cand_index, float* out_value, long long* out_index, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(hidden) * sizeof(__half);
    if (smem > 96 * 1024 || hidden % 8) return cudaErrorInvalidValue;
    static PerDeviceOnce attribute;
    if (attribute.needed()) {
        cudaError_t e = cudaFuncSetAttribute(head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return e;
        attribute.mark();
    }
    const int grid = head_candidates();
    cudaError_t e = launch_dependent(head_kernel, dim3(grid), dim3(kHeadWarps * 32), smem, stream, x, w, vocab, hidden, index_offset, logits,
                                     cand_value, cand_index);
    if (e != cudaSuccess) return e;
    return launch_dependent(argmax_candidates_kernel, dim3(1), dim3(256), 0, stream, cand_value, cand_index, grid, out_value, out_index);
}

}  // namespace b200exl3
