/*
 * CPU oracle for the EXL3 quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's CPU/GPU arithmetic for
 * the EXL3 quantized linear layer.  It exists to check the CUDA kernels and to
 * give a timed CPU baseline; nothing in the shipped library links or calls it.
 *
 * Parity status: PINNED.  The codec functions reproduce bit-for-bit the
 * reference's 21 pack/unpack/decode fixtures (tests/fixtures/native-quantizer)
 * and its 4 real-checkpoint tile sets (docs/native-coverage/baselines/exl3);
 * the Hadamard-128 reproduces the 17 SHA-256 known answers in
 * docs/native-coverage/h128/physical.json.  The accumulation order inside the
 * matrix product is not pinned by any stored reference output, so layer outputs
 * are compared with a stated tolerance, not bit-for-bit.
 *
 * Reference locations restated here (paths inside the reference project):
 *   native/src/codec.rs:34-50     pack_source / unpack_window / packed_pair
 *   native/src/codec.rs:52-71     decode_codeword (three procedural codebooks)
 *   native/src/codec.rs:73-124    pack / unpack
 *   native/src/codec.rs:126-156   permutation / permutation_inverse
 *   native/src/codec.rs:159-190   reconstruct_inner
 *   native/shaders/exl3.metal:156-170, native/src/linear.rs:1383-1427
 *                                 Hadamard-128 with two fp16 rounding points
 *   native/src/linear.rs:855-861  input rotation chain
 *   native/shaders/_qmv_tile_kernel.metal:183-221  fp32 fma of float(half)*float(half)
 *   native/src/linear.rs:978-996  split sum, output rotation, bias
 *   native/src/moe.rs:27-53, 192-236, 438-533, 586-609   MoE glue numerics
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXL3O_F16 9
#define EXL3O_F32 10
#define EXL3O_BF16 12

/* ------------------------------------------------------------------ fp16 -- */

static float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* double -> fp16, round to nearest even, one rounding. */
static uint16_t d2h(double d) {
    uint64_t bits;
    memcpy(&bits, &d, 8);
    uint16_t sign = (uint16_t)((bits >> 48) & 0x8000u);
    int64_t exp = (int64_t)((bits >> 52) & 0x7ff);
    uint64_t man = bits & 0xfffffffffffffull;
    if (exp == 0x7ff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp == 0 && man == 0) return sign;
    int64_t e = exp - 1023;              /* unbiased */
    uint64_t full = man | (1ull << 52);  /* 53-bit significand, value = full * 2^(e-52) */
    if (exp == 0) return sign;           /* double subnormals are far below half range */
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    int shift;                           /* bits to drop from the 53-bit significand */
    int64_t he;
    if (e >= -14) { shift = 42; he = e + 15; } else { shift = (int)(42 + (-14 - e)); he = 0; }
    if (shift > 63) return sign;
    uint64_t kept = full >> shift;
    uint64_t rem = full & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (kept & 1))) ++kept;
    uint32_t out;
    if (he == 0) {
        out = (uint32_t)kept;            /* subnormal; may carry into exponent 1 */
    } else {
        out = (uint32_t)(((uint64_t)(he - 1) << 10) + kept); /* kept has the hidden bit */
    }
    if (out >= 0x7c00u) out = 0x7c00u;
    return (uint16_t)(sign | out);
}

static uint16_t f2h(float f) { return d2h((double)f); }

static float bf2f(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t f2bf(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x40u);
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7fffu + lsb;
    return (uint16_t)(bits >> 16);
}

/* fp16 multiply with one rounding: the 22-bit product is exact in fp32. */
static uint16_t hmul(uint16_t a, uint16_t b) { return f2h(h2f(a) * h2f(b)); }

uint16_t exl3o_f32_to_f16(float f) { return f2h(f); }
float exl3o_f16_to_f32(uint16_t h) { return h2f(h); }

/* ------------------------------------------------------------- codebooks -- */

/* native/src/codec.rs:52-71 */
uint16_t exl3o_decode_codeword(uint16_t state, int cb) {
    uint32_t x = state;
    uint32_t bits;
    if (cb == 2) {
        bits = x * 0x83dcd12du;
        uint32_t sum = 0x6400u + (bits & 255u) + ((bits >> 8) & 255u) + ((bits >> 16) & 255u) + (bits >> 24);
        double h = (double)h2f((uint16_t)sum);
        double inv = (double)h2f(0x1eee);
        double bias = (double)h2f(0xc931);
        return d2h(h * inv + bias);      /* exact in double, then one fp16 rounding */
    }
    bits = cb == 0 ? x * 89226354u + 64248484u : x * 0xcbac1fedu;
    bits = 0x3b603b60u ^ (bits & 0x8fff8fffu);
    /* both halves lie in [2^-3, 2): the fp32 sum is exact, so this is one fp16 rounding */
    return f2h(h2f((uint16_t)bits) + h2f((uint16_t)(bits >> 16)));
}

void exl3o_codebook_table(int cb, uint16_t* out) {
    for (uint32_t s = 0; s < 65536u; ++s) out[s] = exl3o_decode_codeword((uint16_t)s, cb);
}

/* ------------------------------------------------------------ pack/unpack -- */

static int valid_k(int k) { return k >= 1 && k <= 8; }

/* native/src/codec.rs:73-100 */
int exl3o_pack(const uint16_t* states, size_t nstates, int k, uint16_t* packed) {
    if (!valid_k(k) || nstates % 256) return -1;
    size_t tiles = nstates / 256;
    for (size_t t = 0; t < tiles; ++t) {
        const uint16_t* tile = states + t * 256;
        uint16_t* out = packed + t * 16 * (size_t)k;
        for (int logical = 0; logical < 16 * k; ++logical) {
            uint16_t word = 0;
            for (int bit = 0; bit < 16; ++bit) {
                int span = logical / k;
                int stream_bit = (logical % k) * 16 + bit;
                int index = span * 16 + stream_bit / k;
                int shift = k - 1 - stream_bit % k;
                word = (uint16_t)((word << 1) | ((tile[index] >> shift) & 1u));
            }
            out[logical ^ 1] = word;
        }
    }
    return 0;
}

static uint32_t tile_word(const uint16_t* tile, int k, int i) {
    int p = 2 * (i % (8 * k));
    return (uint32_t)tile[p] | ((uint32_t)tile[p + 1] << 16);
}

/* native/src/codec.rs:40-46, 112-122 */
static uint16_t tile_state(const uint16_t* tile, int k, int t) {
    int b0 = t * k + k + 256 * k - 16;
    int b1 = b0 + 16;
    int i0 = b0 / 32;
    int i1 = (b1 - 1) / 32;
    int shift = (i1 + 1) * 32 - b1;
    uint64_t merged = ((uint64_t)tile_word(tile, k, i0) << 32) | tile_word(tile, k, i1);
    return (uint16_t)(merged >> shift);
}

int exl3o_unpack(const uint16_t* packed, size_t npacked, int k, uint16_t* states) {
    if (!valid_k(k) || npacked % (16 * (size_t)k)) return -1;
    size_t tiles = npacked / (16 * (size_t)k);
    for (size_t t = 0; t < tiles; ++t)
        for (int s = 0; s < 256; ++s) states[t * 256 + s] = tile_state(packed + t * 16 * (size_t)k, k, s);
    return 0;
}

/* native/src/codec.rs:126-138: kernel-order index -> row*16+col inside the tile */
void exl3o_permutation(int32_t* out) {
    for (int lane = 0; lane < 32; ++lane) {
        int r = (lane % 4) * 2, c = lane / 4;
        const int rows[4] = {r, r + 1, r + 8, r + 9};
        for (int cg = 0; cg < 2; ++cg)
            for (int ri = 0; ri < 4; ++ri) out[lane * 8 + cg * 4 + ri] = rows[ri] * 16 + c + 8 * cg;
    }
}

void exl3o_permutation_inverse(int32_t* out) {
    int32_t perm[256];
    exl3o_permutation(perm);
    for (int i = 0; i < 256; ++i) out[perm[i]] = i;
}

/* --------------------------------------------------------- thread helper -- */

typedef void (*range_fn)(void* ctx, int64_t begin, int64_t end);
typedef struct { range_fn fn; void* ctx; int64_t begin, end; } job_t;
static void* job_main(void* p) { job_t* j = (job_t*)p; j->fn(j->ctx, j->begin, j->end); return NULL; }

static void parallel_for(int64_t n, int threads, range_fn fn, void* ctx) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if ((int64_t)threads > n) threads = (int)(n > 0 ? n : 1);
    if (threads == 1) { fn(ctx, 0, n); return; }
    pthread_t tid[256];
    job_t jobs[256];
    int started[256];
    for (int i = 0; i < threads; ++i) {
        jobs[i].fn = fn; jobs[i].ctx = ctx;
        jobs[i].begin = n * i / threads; jobs[i].end = n * (i + 1) / threads;
        started[i] = pthread_create(&tid[i], NULL, job_main, &jobs[i]) == 0;
        if (!started[i]) job_main(&jobs[i]);
    }
    for (int i = 0; i < threads; ++i) if (started[i]) pthread_join(tid[i], NULL);
}

/* ------------------------------------------------------ reconstruct_inner -- */

typedef struct {
    const uint16_t* packed; int k, cb, rows, cols; uint16_t* out; const uint16_t* table; const int32_t* perm;
} recon_t;

static void recon_range(void* p, int64_t begin, int64_t end) {
    recon_t* c = (recon_t*)p;
    int tn_count = c->cols / 16;
    for (int64_t tile = begin; tile < end; ++tile) {
        int row = (int)(tile / tn_count) * 16, col = (int)(tile % tn_count) * 16;
        const uint16_t* src = c->packed + tile * 16 * (int64_t)c->k;
        for (int t = 0; t < 256; ++t) {
            int pos = c->perm[t];
            c->out[(int64_t)(row + pos / 16) * c->cols + col + pos % 16] = c->table[tile_state(src, c->k, t)];
        }
    }
}

/* native/src/codec.rs:159-190: packed [rows/16, cols/16, 16k] -> fp16 W[rows, cols] row-major */
int exl3o_reconstruct_inner(const uint16_t* packed, int k, int cb, int rows, int cols, uint16_t* out, int threads) {
    if (!valid_k(k) || cb < 0 || cb > 2 || rows <= 0 || cols <= 0 || rows % 16 || cols % 16) return -1;
    uint16_t* table = (uint16_t*)malloc(65536 * 2);
    if (!table) return -2;
    exl3o_codebook_table(cb, table);
    int32_t perm[256];
    exl3o_permutation(perm);
    recon_t c = {packed, k, cb, rows, cols, out, table, perm};
    parallel_for((int64_t)(rows / 16) * (cols / 16), threads, recon_range, &c);
    free(table);
    return 0;
}

/* ------------------------------------------------------------ Hadamard 128 -- */

/* 128 fp32 values in place.  Butterflies at strides 1..64 in fp32; values are
 * rounded to fp16 after the stride-8 stage when round_mid is set and after the
 * stride-64 stage when round_end is set (native/shaders/exl3.metal:156-170;
 * the MoE glue of native/src/moe.rs:27-53 clears both for SiLU models). */
static void had128_raw(float* v, int round_mid, int round_end) {
    for (int stride = 1; stride <= 64; stride <<= 1) {
        for (int base = 0; base < 128; base += 2 * stride)
            for (int i = base; i < base + stride; ++i) {
                float a = v[i], b = v[i + stride];
                v[i] = a + b;
                v[i + stride] = a - b;
            }
        if ((stride == 8 && round_mid) || (stride == 64 && round_end))
            for (int i = 0; i < 128; ++i) v[i] = h2f(f2h(v[i]));
    }
}

static float had_scale(void) {
    uint32_t bits = 0x3db504f3u;         /* 2^-3.5 as the reference spells it */
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* fp16 in -> fp16 out, the transform MLX applies to fp16 data, scale included. */
void exl3o_hadamard128(const uint16_t* in, uint16_t* out, size_t nblocks) {
    float v[128];
    float s = had_scale();
    for (size_t b = 0; b < nblocks; ++b) {
        for (int i = 0; i < 128; ++i) v[i] = h2f(in[b * 128 + i]);
        had128_raw(v, 1, 1);
        for (int i = 0; i < 128; ++i) out[b * 128 + i] = f2h(v[i] * s);
    }
}

static uint16_t load_as_f16(const void* x, int dtype, int64_t i) {
    if (dtype == EXL3O_F16) return ((const uint16_t*)x)[i];
    if (dtype == EXL3O_F32) return f2h(((const float*)x)[i]);
    return f2h(bf2f(((const uint16_t*)x)[i]));
}

/* native/src/linear.rs:855-861: xhat = H128(half(half(x) * suh)), per row.
 * scale_rows is 1 (one suh for every row) or `rows` (one per row, the MoE case). */
int exl3o_prepare(const void* x, int x_dtype, const uint16_t* suh, int64_t scale_rows, int64_t rows, int in, uint16_t* xhat) {
    if (in <= 0 || in % 128 || rows < 0 || (scale_rows != 1 && scale_rows != rows)) return -1;
    if (x_dtype != EXL3O_F16 && x_dtype != EXL3O_F32 && x_dtype != EXL3O_BF16) return -1;
    uint16_t p[128];
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* s = suh + (scale_rows == 1 ? 0 : r * in);
        for (int b = 0; b < in / 128; ++b) {
            for (int i = 0; i < 128; ++i) p[i] = hmul(load_as_f16(x, x_dtype, r * in + b * 128 + i), s[b * 128 + i]);
            exl3o_hadamard128(p, xhat + r * in + b * 128, 1);
        }
    }
    return 0;
}

static void store_out(void* y, int dtype, int64_t i, uint16_t h, const uint16_t* bias, int col) {
    /* linear.rs:990-996: y.astype(x.dtype) then + bias (fp16 bias) */
    if (dtype == EXL3O_F16) {
        ((uint16_t*)y)[i] = bias ? d2h((double)h2f(h) + (double)h2f(bias[col])) : h;
    } else if (dtype == EXL3O_F32) {
        ((float*)y)[i] = bias ? h2f(h) + h2f(bias[col]) : h2f(h);
    } else {
        uint16_t v = f2bf(h2f(h));
        ((uint16_t*)y)[i] = bias ? f2bf(bf2f(v) + h2f(bias[col])) : v;
    }
}

/* native/src/linear.rs:978-996: yhat fp32 [rows, out] (splits already summed)
 * -> half -> H128 -> * svh -> x dtype -> + bias. */
int exl3o_finish(const float* yhat, const uint16_t* svh, int64_t scale_rows, const uint16_t* bias,
                 int64_t rows, int out, int y_dtype, void* y) {
    if (out <= 0 || out % 128 || rows < 0 || (scale_rows != 1 && scale_rows != rows)) return -1;
    uint16_t p[128], q[128];
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* s = svh + (scale_rows == 1 ? 0 : r * out);
        for (int b = 0; b < out / 128; ++b) {
            for (int i = 0; i < 128; ++i) p[i] = f2h(yhat[r * out + b * 128 + i]);
            exl3o_hadamard128(p, q, 1);
            for (int i = 0; i < 128; ++i)
                store_out(y, y_dtype, r * out + b * 128 + i, hmul(q[i], s[b * 128 + i]), bias, b * 128 + i);
        }
    }
    return 0;
}

/* ------------------------------------------------------- fused decode+dot -- */

typedef struct {
    const uint16_t* packed; int k, in, out; int64_t rows; const uint16_t* xhat; float* yhat;
    const float* table; const int32_t* perm; int tk_begin, tk_end; int f64acc;
} dot_t;

/* One output tile column per unit: acc[row][col] += float(xhat[k]) * float(W16[k, col]) in fp32
 * (native/shaders/_qmv_tile_kernel.metal:196-221), k ascending. */
static void dot_range(void* p, int64_t begin, int64_t end) {
    dot_t* c = (dot_t*)p;
    int tn_count = c->out / 16;
    float w[256];
    float* xf = (float*)malloc(sizeof(float) * 16 * (size_t)(c->rows > 0 ? c->rows : 1));
    for (int64_t tn = begin; tn < end; ++tn) {
        float* accf = (float*)calloc((size_t)c->rows * 16, sizeof(float));
        double* accd = c->f64acc ? (double*)calloc((size_t)c->rows * 16, sizeof(double)) : NULL;
        for (int tk = c->tk_begin; tk < c->tk_end; ++tk) {
            const uint16_t* src = c->packed + ((int64_t)tk * tn_count + tn) * 16 * c->k;
            for (int t = 0; t < 256; ++t) w[c->perm[t]] = c->table[tile_state(src, c->k, t)];
            for (int64_t r = 0; r < c->rows; ++r) {
                for (int i = 0; i < 16; ++i) xf[i] = h2f(c->xhat[r * c->in + tk * 16 + i]);
                if (accd) {
                    for (int i = 0; i < 16; ++i)
                        for (int j = 0; j < 16; ++j) accd[r * 16 + j] += (double)xf[i] * (double)w[i * 16 + j];
                } else {
                    for (int i = 0; i < 16; ++i)
                        for (int j = 0; j < 16; ++j) accf[r * 16 + j] = fmaf(xf[i], w[i * 16 + j], accf[r * 16 + j]);
                }
            }
        }
        for (int64_t r = 0; r < c->rows; ++r)
            for (int j = 0; j < 16; ++j)
                c->yhat[r * c->out + tn * 16 + j] = accd ? (float)accd[r * 16 + j] : accf[r * 16 + j];
        free(accf);
        free(accd);
    }
    free(xf);
}

/* yhat[rows, out] fp32 = xhat[rows, in] (fp16) x W (decoded on the fly) over input tiles [tk_begin, tk_end). */
int exl3o_matmul_raw(const uint16_t* packed, int k, int cb, int in, int out, const uint16_t* xhat, int64_t rows,
                     int tk_begin, int tk_end, int f64acc, float* yhat, int threads) {
    if (!valid_k(k) || cb < 0 || cb > 2 || in <= 0 || out <= 0 || in % 16 || out % 16 || rows < 0) return -1;
    if (tk_begin < 0 || tk_end > in / 16 || tk_begin > tk_end) return -1;
    uint16_t* t16 = (uint16_t*)malloc(65536 * 2);
    float* table = (float*)malloc(65536 * 4);
    if (!t16 || !table) { free(t16); free(table); return -2; }
    exl3o_codebook_table(cb, t16);
    for (int i = 0; i < 65536; ++i) table[i] = h2f(t16[i]);
    free(t16);
    int32_t perm[256];
    exl3o_permutation(perm);
    dot_t c = {packed, k, in, out, rows, xhat, yhat, table, perm, tk_begin, tk_end, f64acc};
    parallel_for(out / 16, threads, dot_range, &c);
    free(table);
    return 0;
}

/* Exl3Linear::forward (native/src/linear.rs:731-997): x [rows, in] -> y [rows, out], y in x's dtype. */
int exl3o_linear_forward(const uint16_t* packed, int k, int cb, int in, int out, const uint16_t* suh,
                         const uint16_t* svh, const uint16_t* bias, const void* x, int x_dtype, int64_t rows,
                         void* y, int threads) {
    if (in % 128 || out % 128 || rows <= 0) return -1;
    uint16_t* xhat = (uint16_t*)malloc((size_t)rows * in * 2);
    float* yhat = (float*)malloc((size_t)rows * out * 4);
    int rc = -2;
    if (xhat && yhat) {
        rc = exl3o_prepare(x, x_dtype, suh, 1, rows, in, xhat);
        if (!rc) rc = exl3o_matmul_raw(packed, k, cb, in, out, xhat, rows, 0, in / 16, 0, yhat, threads);
        if (!rc) rc = exl3o_finish(yhat, svh, 1, bias, rows, out, x_dtype, y);
    }
    free(xhat);
    free(yhat);
    return rc;
}

/* ---------------------------------------------------------------- MoE glue -- */

static float silu(float v) { return v / (1.0f + expf(-v)); }

/* native/src/moe.rs:438-533 (SiLU models): raw fp32 gate/up sums [routes, h] ->
 * down-projection input xhat [routes, h] fp16.
 *   g = float(half(raw)); H128 with no intermediate rounding; * 2^-3.5 in fp32;
 *   gate_v = half(g * svh_gate), up_v likewise; act = half(silu_f32(gate_v) * up_v);
 *   a = half(act * down_suh); H128 again without rounding; out = half(. * 2^-3.5). */
int exl3o_glu_down_input(const float* gate_raw, const float* up_raw, const uint16_t* svh_gate,
                         const uint16_t* svh_up, const uint16_t* down_suh, int64_t routes, int h, uint16_t* out) {
    if (h <= 0 || h % 128 || routes < 0) return -1;
    float g[128], u[128], a[128];
    float s = had_scale();
    for (int64_t r = 0; r < routes; ++r)
        for (int b = 0; b < h / 128; ++b) {
            int64_t o = r * h + b * 128;
            for (int i = 0; i < 128; ++i) { g[i] = h2f(f2h(gate_raw[o + i])); u[i] = h2f(f2h(up_raw[o + i])); }
            had128_raw(g, 0, 0);
            had128_raw(u, 0, 0);
            for (int i = 0; i < 128; ++i) {
                float gv = h2f(f2h(g[i] * s * h2f(svh_gate[o + i])));
                float uv = h2f(f2h(u[i] * s * h2f(svh_up[o + i])));
                float act = h2f(f2h(silu(gv) * uv));
                a[i] = h2f(f2h(act * h2f(down_suh[o + i])));
            }
            had128_raw(a, 0, 0);
            for (int i = 0; i < 128; ++i) out[o + i] = f2h(a[i] * s);
        }
    return 0;
}

/* native/src/moe.rs:586-609: per-route y = half(H128(half(raw))) * svh) * score, summed over top_k in fp16. */
int exl3o_finish_and_reduce(const float* down_raw, const uint16_t* down_svh, const uint16_t* scores,
                            int64_t rows, int top_k, int out, uint16_t* y) {
    if (out <= 0 || out % 128 || rows < 0 || top_k <= 0) return -1;
    uint16_t p[128], q[128];
    for (int64_t r = 0; r < rows; ++r)
        for (int b = 0; b < out / 128; ++b) {
            float acc[128];
            for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
            for (int t = 0; t < top_k; ++t) {
                int64_t route = r * top_k + t;
                for (int i = 0; i < 128; ++i) p[i] = f2h(down_raw[route * out + b * 128 + i]);
                exl3o_hadamard128(p, q, 1);
                for (int i = 0; i < 128; ++i) {
                    uint16_t v = hmul(hmul(q[i], down_svh[route * out + b * 128 + i]), scores[route]);
                    acc[i] = t == 0 ? h2f(v) : h2f(f2h(acc[i] + h2f(v)));
                }
            }
            for (int i = 0; i < 128; ++i) y[r * out + b * 128 + i] = f2h(acc[i]);
        }
    return 0;
}
