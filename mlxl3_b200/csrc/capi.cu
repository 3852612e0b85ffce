// C ABI of the library: argument validation, handle ownership, workspace carving and kernel dispatch.
// Error convention of the reference's FFI (native/ffi/mlx_bridge.cpp:49-66): int status plus a
// thread-local message; nothing throws across the boundary.
#include "../../include/b200exl3.h"

#include <cstdarg>
#include <cstdio>
#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include <atomic>
namespace b200exl3 { extern std::atomic<unsigned long long*> g_qmm_trace; }

using namespace b200exl3;

namespace {

thread_local std::string g_error;

int fail(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return -1;
}

int check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    return fail("%s: %s", what, cudaGetErrorString(e));
}

#define B200_TRY(expr, what)                      \
    do {                                          \
        if (check((expr), (what)) != 0) return -1; \
    } while (0)

cudaStream_t as_stream(b200exl3_stream s) { return static_cast<cudaStream_t>(s); }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__global__ void to_half_kernel(const void* src, int dtype, int64_t n, __half* dst) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = load_as_half(src, dtype, i);
}

int valid_format(int k, int cb) {
    if (k < 1 || k > 8) return fail("K must be in 1..=8, got %d", k);
    if (cb < 0 || cb > 2) return fail("invalid EXL3 codebook %d", cb);
    return 0;
}

std::atomic<bool> g_moe_sorted{true};                    // "moe_sorted" option: 0 keeps one row per slot for any batch
std::atomic<bool> g_moe_fused{false};                    // "moe_fused" option: 1 folds the glue of a small batch into the down product (measured: no faster)
std::atomic<bool> g_qmm_enabled{true};                   // "qmm" option: 0 sends every batch through the fused kernel
std::atomic<long long> g_tp_wait_ms{4000};
std::atomic<long long> g_stack_wait_ms{2000};            // "stack_wait_ms" option: bound of a layer-boundary wait inside a step
std::atomic<unsigned long long*> g_stack_trace{nullptr}; // "stack_trace_buffer" option               // "tp_wait_ms" option: how long a rank polls for its peers' sums
constexpr int kMaxBatchRows = kQmvMaxRows;              // rows handled by one launch of the fused kernel
constexpr size_t kCounterBytes = B200EXL3_WORKSPACE_HEADER_BYTES;   // arrival counters at the head of a workspace

}  // namespace

// One launchable layer: a plain Exl3Linear (groups == 1) or several projections that share their
// input, concatenated along the output axis (Exl3Group).
struct LayerCore {
    int in, out, k, cb;
    uint32_t flags;
    uint32_t* wq;       // weights in the quad layout [out/128, in/16, 2, 8K, 4], owned
    __half* suh;        // [groups, in]
    __half* svh;        // [out]
    __half* bias;       // [out] or nullptr
    int groups;
    int gcol0[kQmvMaxGroups], gout[kQmvMaxGroups];
};

struct b200exl3_linear { LayerCore c; };
struct b200exl3_group { LayerCore c; };

// Peer-memory context of one tensor-parallel rank: every rank's exchange buffer ([flags | inbox]) mapped into
// this process, and this rank's per-unit use counts.
struct b200exl3_tp {
    int rank, world, max_units;
    void* buffers[kTpMaxWorld];
    unsigned int* done;      // [max_units] + one status word
};

// Grouped experts of a SwiGLU block: two banks in the quad layout (gate columns of all experts, then up
// columns of all experts; down columns of all experts) and the per-expert scales.
struct b200exl3_moe {
    int experts, in, hidden, top_k, k, cb;
    uint32_t flags;
    uint32_t* gu_wq;     // [in/16, experts*2*hidden/16] tiles
    uint32_t* down_wq;   // [hidden/16, experts*in/16] tiles
    __half* gu_suh;      // [experts, 2, in]
    __half* gu_svh;      // [experts, 2, hidden]
    __half* down_suh;    // [experts, hidden]
    __half* down_svh;    // [experts, in]
};

static void core_free(LayerCore& c) {
    cudaFree(c.suh);
    cudaFree(c.svh);
    cudaFree(c.bias);
    cudaFree(c.wq);
}

extern "C" {

const char* b200exl3_last_error(void) { return g_error.c_str(); }

int b200exl3_version(void) { return 100; }

int b200exl3_init(int device) {
    int count = 0;
    B200_TRY(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (device < 0 || device >= count) return fail("device %d out of range (%d visible)", device, count);
    B200_TRY(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop{};
    B200_TRY(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major != 10) return fail("device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
    return 0;
}

int b200exl3_set_option(const char* name, int64_t value) {
    static std::atomic<int> ctas{0}, grid{0}, pdl{0};
    if (!name) return fail("option name is NULL");
    if (!strcmp(name, "qmv_ctas_per_sm")) ctas = static_cast<int>(value);
    else if (!strcmp(name, "qmv_force_grid")) grid = static_cast<int>(value);
    else if (!strcmp(name, "pdl")) pdl = static_cast<int>(value);
    else if (!strcmp(name, "qmm")) { g_qmm_enabled = value != 0; return 0; }
    else if (!strcmp(name, "stack_wait_ms")) {
        if (value < 1 || value > 60000) return fail("stack_wait_ms must be between 1 and 60000");
        g_stack_wait_ms = value;
        return 0;
    }
    else if (!strcmp(name, "stack_trace_buffer")) { g_stack_trace = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(value)); return 0; }
    else if (!strcmp(name, "tp_wait_ms")) {
        if (value < 1 || value > 60000) return fail("tp_wait_ms must be between 1 and 60000");
        g_tp_wait_ms = value;
        return 0;
    }
    else if (!strcmp(name, "qmm_trace_buffer")) { b200exl3::g_qmm_trace = reinterpret_cast<unsigned long long*>(value); return 0; }
    else if (!strcmp(name, "moe_sorted")) { g_moe_sorted = value != 0; return 0; }
    else if (!strcmp(name, "moe_fused")) { g_moe_fused = value != 0; return 0; }
    else if (!strcmp(name, "qmm_splits")) { qmm_set_tuning(static_cast<int>(value)); return 0; }
    else if (!strcmp(name, "qmv_trace_buffer")) {
        qmv_set_trace(reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(value)));
        return 0;
    }
    else return fail("unknown option %s", name);
    qmv_set_tuning(ctas, grid, pdl);
    return 0;
}

/* ---- launch policy, as data (host arithmetic only: needs no GPU) --------------------------------------------------- */

int b200exl3_plan_query(const char* kind, int in, int out, int k, int64_t rows, int64_t* out_values, int capacity) {
    if (!kind || !out_values || capacity < 8) return fail("plan query needs room for 8 values");
    if (in <= 0 || out <= 0 || in % 128 || out % 128 || k < 1 || k > 8 || rows <= 0) return fail("invalid plan query");
    for (int i = 0; i < 8; ++i) out_values[i] = 0;
    if (!strcmp(kind, "qmv")) {
        const QmvPlan p = plan_qmv(in, out, k, rows);
        out_values[0] = p.grid; out_values[1] = p.max_pieces; out_values[2] = p.col_blocks; out_values[3] = kQmvWarps;
        out_values[4] = static_cast<int64_t>(p.smem_bytes); out_values[5] = p.fused_rotation ? 1 : 0;
        return 0;
    }
    if (!strcmp(kind, "qmm")) {
        const QmmPlan p = plan_qmm(in, out, rows);
        out_values[0] = p.splits; out_values[1] = p.token_tiles; out_values[2] = p.small ? 1 : 0; out_values[3] = in / 64;
        return 0;
    }
    if (!strcmp(kind, "stack")) {
        const StackPlan p = plan_stack(k, static_cast<int>(std::min<int64_t>(rows, kStackMaxRows)), 1);
        StackOp op{};
        op.in = in; op.out = out;
        const bool ok = plan_stack_op(p, op);
        out_values[0] = p.grid; out_values[1] = ok ? op.max_pieces : 0; out_values[2] = ok ? op.col_blocks : 0; out_values[3] = kStackWarps;
        out_values[4] = static_cast<int64_t>(p.smem_bytes); out_values[5] = ok ? op.warps : 0; out_values[6] = ok ? op.narrow : 0;
        out_values[7] = ok ? 1 : 0;
        return 0;
    }
    return fail("unknown plan kind %s", kind);
}

/* ---- memory / stream plumbing ---------------------------------------------------------------- */

int b200exl3_malloc(size_t bytes, void** out) {
    if (!out) return fail("out pointer is NULL");
    *out = nullptr;
    if (bytes == 0) return 0;
    return check(cudaMalloc(out, bytes), "cudaMalloc");
}
int b200exl3_free(void* p) { return p ? check(cudaFree(p), "cudaFree") : 0; }
int b200exl3_host_alloc(size_t bytes, void** out) {
    if (!out) return fail("out pointer is NULL");
    *out = nullptr;
    if (bytes == 0) return 0;
    return check(cudaMallocHost(out, bytes), "cudaMallocHost");
}
int b200exl3_host_free(void* p) { return p ? check(cudaFreeHost(p), "cudaFreeHost") : 0; }
int b200exl3_memcpy_h2d(void* dst, const void* src, size_t bytes, b200exl3_stream s) {
    if (bytes == 0) return 0;
    return check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(s)), "cudaMemcpyAsync(h2d)");
}
int b200exl3_memcpy_d2h(void* dst, const void* src, size_t bytes, b200exl3_stream s) {
    if (bytes == 0) return 0;
    return check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(s)), "cudaMemcpyAsync(d2h)");
}
int b200exl3_memset(void* dst, int value, size_t bytes, b200exl3_stream s) {
    if (bytes == 0) return 0;
    return check(cudaMemsetAsync(dst, value, bytes, as_stream(s)), "cudaMemsetAsync");
}
int b200exl3_stream_create(b200exl3_stream* out) {
    if (!out) return fail("out pointer is NULL");
    cudaStream_t s;
    B200_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    *out = s;
    return 0;
}
int b200exl3_stream_destroy(b200exl3_stream s) { return s ? check(cudaStreamDestroy(as_stream(s)), "cudaStreamDestroy") : 0; }
int b200exl3_stream_sync(b200exl3_stream s) { return check(cudaStreamSynchronize(as_stream(s)), "cudaStreamSynchronize"); }
int b200exl3_event_create(void** out) {
    if (!out) return fail("out pointer is NULL");
    cudaEvent_t e;
    B200_TRY(cudaEventCreate(&e), "cudaEventCreate");
    *out = e;
    return 0;
}
int b200exl3_event_destroy(void* e) { return e ? check(cudaEventDestroy(static_cast<cudaEvent_t>(e)), "cudaEventDestroy") : 0; }
int b200exl3_event_record(void* e, b200exl3_stream s) {
    return check(cudaEventRecord(static_cast<cudaEvent_t>(e), as_stream(s)), "cudaEventRecord");
}
int b200exl3_event_elapsed_ms(void* start, void* stop, float* out_ms) {
    if (!out_ms) return fail("out pointer is NULL");
    B200_TRY(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)), "cudaEventSynchronize");
    return check(cudaEventElapsedTime(out_ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)),
                 "cudaEventElapsedTime");
}

/* ---- graph replay ------------------------------------------------------------------------------ */

int b200exl3_graph_begin(b200exl3_stream s) {
    return check(cudaStreamBeginCapture(as_stream(s), cudaStreamCaptureModeRelaxed), "cudaStreamBeginCapture");
}
int b200exl3_graph_end(b200exl3_stream s, void** out_graph) {
    if (!out_graph) return fail("out pointer is NULL");
    *out_graph = nullptr;
    cudaGraph_t graph = nullptr;
    B200_TRY(cudaStreamEndCapture(as_stream(s), &graph), "cudaStreamEndCapture");
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (check(e, "cudaGraphInstantiate")) return -1;
    *out_graph = exec;
    return 0;
}
int b200exl3_graph_launch(void* graph, b200exl3_stream s) {
    if (!graph) return fail("NULL graph");
    return check(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph), as_stream(s)), "cudaGraphLaunch");
}
int b200exl3_graph_free(void* graph) {
    return graph ? check(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph)), "cudaGraphExecDestroy") : 0;
}

/* ---- codec ------------------------------------------------------------------------------------- */

int b200exl3_unpack_states(const uint16_t* d_packed, int64_t tiles, int k, int cb, uint16_t* d_states,
                           uint16_t* d_values, b200exl3_stream s) {
    if (valid_format(k, cb)) return -1;
    if (tiles < 0) return fail("packed length is not a whole tile");
    if (tiles > 0 && (!d_packed || (!d_states && !d_values))) return fail("NULL buffer");
    return check(launch_unpack_states(d_packed, tiles, k, cb, d_states, reinterpret_cast<__half*>(d_values), as_stream(s)),
                 "unpack_states");
}

int b200exl3_codebook(const uint16_t* d_states, int64_t n, int cb, uint16_t* d_values, b200exl3_stream s) {
    if (valid_format(1, cb)) return -1;
    if (n < 0 || (n > 0 && !d_values)) return fail("invalid codebook request");
    return check(launch_codebook(d_states, n, cb, reinterpret_cast<__half*>(d_values), as_stream(s)), "codebook");
}

int b200exl3_reconstruct(const uint16_t* d_trellis, int in, int out, int k, int cb, uint16_t* d_w, b200exl3_stream s) {
    if (valid_format(k, cb)) return -1;
    if (in <= 0 || out <= 0 || in % 16 || out % 16) return fail("dimensions must be positive multiples of 16");
    if (!d_trellis || !d_w) return fail("NULL buffer");
    if (!aligned16(d_trellis) || !aligned16(d_w)) return fail("device pointers must be 16-byte aligned");
    return check(launch_reconstruct(d_trellis, in / 16, out / 16, k, cb, reinterpret_cast<__half*>(d_w), as_stream(s)),
                 "reconstruct");
}

/* ---- rotations ------------------------------------------------------------------------------- */

int b200exl3_prepare(const void* d_x, int x_dtype, const uint16_t* d_suh, int64_t scale_rows, int64_t rows, int in,
                     uint16_t* d_xhat, b200exl3_stream s) {
    if (in <= 0 || in % 128) return fail("expected complete 128-aligned rows");
    if (rows < 0) return fail("negative row count");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (scale_rows != 1 && scale_rows != rows) return fail("scales must have one row or one per input row");
    if (rows == 0) return 0;
    if (!d_x || !d_suh || !d_xhat) return fail("NULL buffer");
    if (!aligned16(d_xhat)) return fail("device pointers must be 16-byte aligned");
    return check(launch_prepare(d_x, x_dtype, reinterpret_cast<const __half*>(d_suh), scale_rows, rows, in,
                                reinterpret_cast<__half*>(d_xhat), as_stream(s)), "prepare");
}

int b200exl3_finish(const float* d_partials, int splits, const uint16_t* d_svh, int64_t scale_rows,
                    const uint16_t* d_bias, int64_t rows, int out, int y_dtype, void* d_y, b200exl3_stream s) {
    if (out <= 0 || out % 128) return fail("expected complete 128-aligned rows");
    if (rows < 0 || splits < 1) return fail("invalid finish request");
    if (!dtype_is_float(y_dtype)) return fail("unsupported output dtype %d", y_dtype);
    if (scale_rows != 1 && scale_rows != rows) return fail("scales must have one row or one per input row");
    if (rows == 0) return 0;
    if (!d_partials || !d_svh || !d_y) return fail("NULL buffer");
    if (!aligned16(d_partials)) return fail("device pointers must be 16-byte aligned");
    return check(launch_finish(d_partials, splits, rows * out, reinterpret_cast<const __half*>(d_svh), scale_rows,
                               reinterpret_cast<const __half*>(d_bias), rows, out, y_dtype, d_y, as_stream(s)), "finish");
}

/* ---- Exl3Linear ------------------------------------------------------------------------------ */

int b200exl3_linear_create(const uint16_t* d_trellis, const void* d_suh, const void* d_svh, const void* d_bias,
                           int scale_dtype, int in, int out, int k, int cb, uint32_t flags, b200exl3_linear** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (valid_format(k, cb)) return -1;
    if (in <= 0 || out <= 0) return fail("invalid trellis shape");
    if (in % 128 || out % 128) return fail("public EXL3 projections require 128-aligned dimensions");
    if (!d_trellis) return fail("invalid trellis shape");
    if (!d_suh || !d_svh) return fail("EXL3 scales have wrong dimensions");
    if (!dtype_is_float(scale_dtype)) return fail("unsupported scale dtype %d", scale_dtype);
    if (!aligned16(d_trellis)) return fail("device pointers must be 16-byte aligned");
    if (out / 128 >= static_cast<int>(kCounterBytes / sizeof(unsigned int))) return fail("output dimension %d is too large", out);
    b200exl3_linear* handle = new (std::nothrow) b200exl3_linear{};
    if (!handle) return fail("out of host memory");
    LayerCore* h = &handle->c;
    h->in = in; h->out = out; h->k = k; h->cb = cb; h->flags = flags;
    h->groups = 1; h->gcol0[0] = 0; h->gout[0] = out;
    auto convert = [&](const void* src, int n, __half** dst) -> int {
        B200_TRY(cudaMalloc(dst, static_cast<size_t>(n) * sizeof(__half)), "cudaMalloc(scales)");
        to_half_kernel<<<(n + 255) / 256, 256>>>(src, scale_dtype, n, *dst);
        return check(cudaGetLastError(), "convert scales");
    };
    int rc = convert(d_suh, in, &h->suh);
    if (!rc) rc = convert(d_svh, out, &h->svh);
    if (!rc && d_bias) rc = convert(d_bias, out, &h->bias);
    if (!rc) {
        size_t bytes = static_cast<size_t>(in / 16) * (out / 16) * 16 * k * sizeof(uint16_t);
        rc = check(cudaMalloc(&h->wq, bytes), "cudaMalloc(weights)");
        if (!rc) rc = check(launch_repack_quads(reinterpret_cast<const uint32_t*>(d_trellis), in / 16, out / 16, k, h->wq, 0),
                            "repack weights");
    }
    if (!rc) rc = check(cudaDeviceSynchronize(), "linear_create");
    if (rc) {
        b200exl3_linear_free(handle);
        return -1;
    }
    *out_handle = handle;
    return 0;
}

void b200exl3_linear_free(b200exl3_linear* h) {
    if (!h) return;
    core_free(h->c);
    delete h;
}

int b200exl3_linear_input_dims(const b200exl3_linear* h) { return h ? h->c.in : fail("NULL handle"); }
int b200exl3_linear_output_dims(const b200exl3_linear* h) { return h ? h->c.out : fail("NULL handle"); }

static size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// workspace = [counters + status | partial tiles | rotated activations (only when the kernel does not rotate)]
static size_t xhat_bytes(const LayerCore& c, int64_t rows) {
    return rows > kQmvFusedRows ? round256(static_cast<size_t>(c.groups) * rows * c.in * sizeof(__half)) : 0;
}

// From this many rows on, a plain layer's forward runs the tensor-core product (rotate all rows, tcgen05 product,
// output rotation) instead of the fused kernel: its small shape (two CTAs per SM) takes 43 us for 9..64 rows of a
// 4096 -> 14336 layer where the fused kernel's two-block form takes 61 us for 9..16 rows.
constexpr int64_t kQmmMinRows = 9;

static int core_workspace_bytes(const LayerCore& c, int64_t rows, size_t* out_bytes) {
    if (!out_bytes) return fail("NULL argument");
    if (rows <= 0) return fail("EXL3 linear input cannot be empty");
    QmvPlan plan = plan_qmv(c.in, c.out, c.k, rows);
    size_t bytes = kCounterBytes + qmv_partial_bytes(plan, c.out, rows) + xhat_bytes(c, rows);
    if (rows >= kQmmMinRows) {
        // tensor-core path: one rotated copy of the rows at a time (per member of a group) and the member's partials
        for (int g = 0; g < c.groups; ++g) {
            const QmmPlan qp = plan_qmm(c.in, c.gout[g], rows);
            bytes = std::max(bytes, kCounterBytes + round256(static_cast<size_t>(rows) * c.in * sizeof(__half)) +
                                        qmm_partial_bytes(qp, c.gout[g], rows));
        }
    }
    *out_bytes = bytes;
    return 0;
}

int b200exl3_linear_workspace_bytes(const b200exl3_linear* h, int64_t rows, size_t* out_bytes) {
    if (!h) return fail("NULL argument");
    return core_workspace_bytes(h->c, rows, out_bytes);
}

// One fused launch per batch of up to kMaxBatchRows rows.  Exactly one of d_x / d_xhat is given;
// ys (one pointer per group) selects the rotated output, otherwise the summed fp32 product goes to d_yhat.
static TpPeers tp_peers(const b200exl3_tp* tp);

static int forward_common(const LayerCore& c, const void* d_x, int x_dtype, const uint16_t* d_xhat, int64_t rows,
                          void* const* ys, float* d_yhat, void* ws, size_t ws_bytes, cudaStream_t stream,
                          const b200exl3_tp* tp = nullptr, const b200exl3_prologue* pro = nullptr) {
    if (rows <= 0) return fail("EXL3 linear input cannot be empty");
    size_t need = 0;
    if (core_workspace_bytes(c, rows, &need)) return -1;
    if (!ws || ws_bytes < need) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, need);
    if (!aligned16(ws)) return fail("device pointers must be 16-byte aligned");
    char* base = static_cast<char*>(ws);
    const bool exact = (c.flags & B200EXL3_EXACT_WEIGHTS) != 0;
    const size_t x_size = dtype_size(x_dtype);
    const __half* xhat = reinterpret_cast<const __half*>(d_xhat);
    // more rows than the fused kernel rotates itself: the input rotation is a kernel of its own, and the SwiGLU
    // prologue (the only one taken with that many rows) is applied there
    const __half* glu_up = nullptr;
    if (pro && pro->kind == 2 && rows > kQmvFusedRows) {
        glu_up = reinterpret_cast<const __half*>(pro->d_aux);
        pro = nullptr;
    }
    if (rows >= kQmmMinRows && ys && !d_xhat && g_qmm_enabled) {
        // many rows: input rotation -> tensor-core product (fp32 partials per input split) -> output rotation.
        // A group runs member by member (each member has its own input scales, so its own rotated rows); a row shard
        // of a tensor-parallel layer keeps one split, and the sum over ranks and the rotation follow as one kernel.
        __half* buf = reinterpret_cast<__half*>(base + kCounterBytes);
        float* partials = reinterpret_cast<float*>(base + kCounterBytes + round256(static_cast<size_t>(rows) * c.in * sizeof(__half)));
        unsigned int* status = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
        for (int g = 0; g < c.groups; ++g) {
            QmmPlan qp = plan_qmm(c.in, c.gout[g], rows);
            const __half* svh = c.svh + c.gcol0[g];
            const __half* bias = c.bias ? c.bias + c.gcol0[g] : nullptr;
            const int ld = c.out / 16, col0 = c.gcol0[g] / 16;
            B200_TRY(launch_prepare(d_x, x_dtype, c.suh + static_cast<size_t>(g) * c.in, 1, rows, c.in, buf, stream, glu_up), "prepare");
            if (tp) {
                qp.splits = 1;
                B200_TRY(launch_qmm(c.wq, c.in, c.gout[g], c.k, c.cb, buf, rows, qp, partials, status, nullptr, nullptr, nullptr, 0, stream, ld, col0),
                         "tensor-core product kernel");
                TpArgs a{};
                a.yhat = partials; a.peers = tp_peers(tp); a.svh = svh; a.bias = bias; a.y = ys[g];
                a.rows = static_cast<int>(rows); a.out = c.gout[g]; a.y_dtype = x_dtype;
                B200_TRY(launch_tp_finish(a, stream), "tensor-parallel finish kernel");
            } else if (qp.splits == 1) {
                // one CTA holds the whole input range of its columns: the output rotation runs in its epilogue
                B200_TRY(launch_qmm(c.wq, c.in, c.gout[g], c.k, c.cb, buf, rows, qp, partials, status, svh, bias, ys[g], x_dtype, stream, ld, col0),
                         "tensor-core product kernel");
            } else {
                B200_TRY(launch_qmm(c.wq, c.in, c.gout[g], c.k, c.cb, buf, rows, qp, partials, status, nullptr, nullptr, nullptr, 0, stream, ld, col0),
                         "tensor-core product kernel");
                B200_TRY(launch_finish(partials, qp.splits, rows * c.gout[g], svh, 1, bias, rows, c.gout[g], x_dtype, ys[g], stream), "finish");
            }
        }
        return 0;
    }
    if (!xhat && rows > kQmvFusedRows) {
        // more than two rows: rotate all of them once per group, the product kernel reads the rotated rows
        const QmvPlan first = plan_qmv(c.in, c.out, c.k, rows);
        __half* buf = reinterpret_cast<__half*>(base + kCounterBytes + qmv_partial_bytes(first, c.out, rows));
        for (int g = 0; g < c.groups; ++g)
            B200_TRY(launch_prepare(d_x, x_dtype, c.suh + static_cast<size_t>(g) * c.in, 1, rows, c.in,
                                    buf + static_cast<size_t>(g) * rows * c.in, stream, glu_up), "prepare");
        xhat = buf;
    }
    for (int64_t r0 = 0; r0 < rows; r0 += kMaxBatchRows) {
        const int64_t n = rows - r0 < kMaxBatchRows ? rows - r0 : kMaxBatchRows;
        const QmvPlan plan = plan_qmv(c.in, c.out, c.k, n);
        QmvArgs a{};
        a.wq = c.wq;
        a.x = !xhat ? static_cast<const char*>(d_x) + static_cast<size_t>(r0) * c.in * x_size : nullptr;
        a.suh = c.suh;
        a.xhat = xhat ? xhat + r0 * c.in : nullptr;
        a.xhat_group_stride = rows * c.in;
        a.counters = reinterpret_cast<unsigned int*>(base);
        a.error = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
        a.partials = reinterpret_cast<float*>(base + kCounterBytes);
        a.svh = c.svh;
        a.bias = c.bias;
        a.yhat = d_yhat ? d_yhat + r0 * c.out : nullptr;
        a.groups = c.groups;
        for (int g = 0; g < c.groups; ++g) {
            a.gcol0[g] = c.gcol0[g];
            a.gout[g] = c.gout[g];
            a.gy[g] = ys ? static_cast<char*>(ys[g]) + static_cast<size_t>(r0) * c.gout[g] * x_size : nullptr;
        }
        a.x_dtype = x_dtype;
        a.y_dtype = x_dtype;
        a.in = c.in; a.out = c.out; a.rows = static_cast<int>(n);
        if (tp) { a.tp = tp_peers(tp); a.tp_row0 = static_cast<int>(r0); }
        if (pro && pro->kind != 0) {
            a.prologue = pro->kind;
            a.pro_aux = reinterpret_cast<const __half*>(pro->d_aux);
            a.pro_weight = reinterpret_cast<const __half*>(pro->d_weight);
            a.pro_sum = reinterpret_cast<__half*>(pro->d_sum);
            a.pro_eps = pro->eps;
            a.pro_sumsq = pro->d_sumsq;
        }
        if (pro && pro->epilogue == 2) {
            a.epilogue = 2;
            a.epi_pos = pro->d_pos;
            a.epi_log2_theta = log2f(pro->theta);
            a.epi_max_ctx = pro->max_ctx;
            a.epi_k_cache = reinterpret_cast<__half*>(pro->d_k_cache);
            a.epi_v_cache = reinterpret_cast<__half*>(pro->d_v_cache);
        }
        if (pro && pro->epilogue == 1) {
            a.epilogue = 1;
            a.epi_residual = reinterpret_cast<const __half*>(pro->d_residual);
            a.epi_sum = reinterpret_cast<__half*>(pro->d_residual_out);
            a.epi_sumsq = pro->d_sumsq_out;
        }
        B200_TRY(launch_qmv(a, c.k, c.cb, exact, plan, stream), "fused linear kernel");
    }
    return 0;
}

int b200exl3_workspace_status(const void* ws, int* out_status) {
    if (!ws || !out_status) return fail("NULL argument");
    unsigned int flag = 0;
    B200_TRY(cudaMemcpy(&flag, static_cast<const char*>(ws) + kCounterBytes - sizeof(unsigned int), sizeof flag,
                        cudaMemcpyDeviceToHost), "read workspace status");
    *out_status = static_cast<int>(flag);
    return 0;
}

int b200exl3_linear_forward(const b200exl3_linear* h, const void* d_x, int x_dtype, int64_t rows, void* d_y, void* ws,
                            size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_y) return fail("NULL buffer");
    void* ys[1] = {d_y};
    return forward_common(h->c, d_x, x_dtype, nullptr, rows, ys, nullptr, ws, ws_bytes, as_stream(s));
}

int b200exl3_linear_forward_raw(const b200exl3_linear* h, const uint16_t* d_xhat, int64_t rows, float* d_yhat, void* ws,
                                size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!d_xhat || !d_yhat) return fail("NULL buffer");
    if (!aligned16(d_xhat)) return fail("device pointers must be 16-byte aligned");
    return forward_common(h->c, nullptr, kF16, d_xhat, rows, nullptr, d_yhat, ws, ws_bytes, as_stream(s));
}

int b200exl3_linear_forward_partial(const b200exl3_linear* h, const void* d_x, int x_dtype, int64_t rows, float* d_yhat,
                                    void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_yhat) return fail("NULL buffer");
    return forward_common(h->c, d_x, x_dtype, nullptr, rows, nullptr, d_yhat, ws, ws_bytes, as_stream(s));
}

int b200exl3_linear_finish(const b200exl3_linear* h, const float* d_yhat, int64_t rows, int y_dtype, void* d_y,
                           b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (rows <= 0) return fail("EXL3 linear input cannot be empty");
    if (!dtype_is_float(y_dtype)) return fail("unsupported output dtype %d", y_dtype);
    if (!d_yhat || !d_y) return fail("NULL buffer");
    if (!aligned16(d_yhat)) return fail("device pointers must be 16-byte aligned");
    return check(launch_finish(d_yhat, 1, rows * h->c.out, h->c.svh, 1, h->c.bias, rows, h->c.out, y_dtype, d_y, as_stream(s)),
                 "finish");
}

int b200exl3_linear_decode(const b200exl3_linear* h, uint16_t* d_w, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!d_w || !aligned16(d_w)) return fail("device pointers must be 16-byte aligned");
    return check(launch_reconstruct_quads(h->c.wq, h->c.in / 16, h->c.out / 16, h->c.k, h->c.cb, reinterpret_cast<__half*>(d_w),
                                          as_stream(s)), "reconstruct");
}

static int check_prologue(const b200exl3_prologue* pro, const void* d_x, int64_t rows) {
    if (!pro) return fail("NULL argument");
    // any number of rows for the SwiGLU prologue alone (with many rows it is applied by the input-rotation kernel)
    const bool glu_only = pro->kind == 2 && pro->epilogue == 0;
    if (rows < 1 || (rows > kQmvFusedRows && !glu_only))
        return fail("a fused prologue takes 1 to %d rows (the SwiGLU prologue alone: any number), got %lld", kQmvFusedRows, static_cast<long long>(rows));
    if (pro->kind < 0 || pro->kind > 3) return fail("unknown prologue kind %d", pro->kind);
    if ((pro->kind == 1 || pro->kind == 3) && (!pro->d_weight || !(pro->eps >= 0.0f)))
        return fail("the RMSNorm prologue needs a weight and a non-negative epsilon");
    if (pro->kind == 3 && !pro->d_sumsq) return fail("the RMSNorm prologue of kind 3 needs the block sums of squares");
    if (pro->epilogue < 0 || pro->epilogue > 2) return fail("unknown epilogue kind %d", pro->epilogue);
    if (pro->epilogue == 2) {
        if (rows != 1) return fail("the rotary epilogue takes one row");
        if (!pro->d_pos || !pro->d_k_cache || !pro->d_v_cache || pro->max_ctx <= 0 || !(pro->theta > 1.0f))
            return fail("the rotary epilogue needs a position, both caches, their length and a base above 1");
        if (!aligned16(pro->d_k_cache) || !aligned16(pro->d_v_cache)) return fail("device pointers must be 16-byte aligned");
    }
    if (pro->epilogue == 1 && (!pro->d_residual || !pro->d_residual_out || !pro->d_sumsq_out)) return fail("the residual epilogue needs its three buffers");
    if (!aligned16(pro->d_residual) || !aligned16(pro->d_residual_out)) return fail("device pointers must be 16-byte aligned");
    if (pro->kind == 1 && pro->d_sum == d_x) return fail("the RMSNorm prologue cannot store the sum over its own input");
    if (pro->kind == 2 && !pro->d_aux) return fail("the SwiGLU prologue needs the up rows");
    if (!aligned16(pro->d_aux) || !aligned16(pro->d_weight) || !aligned16(pro->d_sum)) return fail("device pointers must be 16-byte aligned");
    return 0;
}

int b200exl3_linear_forward_fused(const b200exl3_linear* h, const b200exl3_prologue* pro, b200exl3_tp* tp, const void* d_x, int64_t rows,
                                  void* d_y, void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!d_x || (!d_y && !(pro && pro->epilogue == 1))) return fail("NULL buffer");
    if (check_prologue(pro, d_x, rows)) return -1;
    if (pro->epilogue == 2) return fail("the rotary epilogue belongs to a [q | k | v] group");
    if (tp && rows * (h->c.out / 128) > tp->max_units) return fail("units exceed the exchange buffers' %d", tp->max_units);
    void* ys[1] = {d_y};
    return forward_common(h->c, d_x, kF16, nullptr, rows, ys, nullptr, ws, ws_bytes, as_stream(s), tp, pro);
}

/* ---- allocation-free forward ------------------------------------------------------------------- */

// Scratch for b200exl3_linear_forward_static.  Some hosts cannot hand the library a workspace: a
// plugin that runs inside somebody else's memory pool, a real-time loop that must not touch the
// allocator, a caller that only ever receives input and output pointers.  For them the scratch lives
// in the library's own device image: every GPU that loads the library holds these bytes until the
// process exits.  The name below is the host-side handle of the array, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (looked up on first use).
int static_scratch(void** out) {
    int device = 0;
    B200_TRY(cudaGetDevice(&device), "cudaGetDevice");
    if (device < 0 || device >= kMaxDevices) return fail("device %d is beyond the %d devices supported", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[device]) {
        void* ptr = nullptr;
        B200_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
        if (!ptr) return fail("the static scratch array has no device address");
        g_static_ptr[device] = ptr;
    }
    *out = g_static_ptr[device];
    return 0;
}
}  // namespace

int b200exl3_linear_forward_static(const b200exl3_linear* h, const void* d_x, int x_dtype, int64_t rows, void* d_y,
                                   b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_y) return fail("NULL buffer");
    size_t need = 0;
    if (core_workspace_bytes(h->c, rows, &need)) return -1;
    if (need > kStaticScratchBytes)
        return fail("this call needs %zu bytes of scratch but the allocation-free entry point owns %zu; "
                    "use b200exl3_linear_forward with a caller workspace", need, kStaticScratchBytes);
    void* scratch = nullptr;
    if (static_scratch(&scratch)) return -1;
    // The array keeps whatever the previous call left; the arrival counters at its head must start at
    // zero, the partial sums behind them are overwritten before they are read.  The status word (the
    // last word of the header) is left alone, so a failure stays visible to b200exl3_static_status
    // until that call clears it, as it does in a caller's workspace.
    B200_TRY(cudaMemsetAsync(scratch, 0, kCounterBytes - sizeof(unsigned int), as_stream(s)), "clear static scratch");
    void* ys[1] = {d_y};
    return forward_common(h->c, d_x, x_dtype, nullptr, rows, ys, nullptr, scratch, kStaticScratchBytes, as_stream(s));
}

int b200exl3_static_status(int* out_status, int clear) {
    if (!out_status) return fail("NULL argument");
    void* scratch = nullptr;
    if (static_scratch(&scratch)) return -1;
    unsigned int* word = reinterpret_cast<unsigned int*>(static_cast<char*>(scratch) + kCounterBytes - sizeof(unsigned int));
    unsigned int flag = 0;
    B200_TRY(cudaMemcpy(&flag, word, sizeof flag, cudaMemcpyDeviceToHost), "read static scratch status");
    if (clear && flag) B200_TRY(cudaMemset(word, 0, sizeof flag), "clear static scratch status");
    *out_status = static_cast<int>(flag);
    return 0;
}

/* ---- Exl3Group --------------------------------------------------------------------------------- */

int b200exl3_group_create(const b200exl3_linear* const* members, int count, b200exl3_group** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (!members || count < 2 || count > kQmvMaxGroups) return fail("incompatible grouped projections");
    for (int g = 0; g < count; ++g) {
        if (!members[g]) return fail("incompatible grouped projections");
        const LayerCore& m = members[g]->c;
        const LayerCore& f = members[0]->c;
        if (m.groups != 1 || m.in != f.in || m.k != f.k || m.cb != f.cb || (m.flags != f.flags))
            return fail("incompatible grouped projections");
    }
    b200exl3_group* handle = new (std::nothrow) b200exl3_group{};
    if (!handle) return fail("out of host memory");
    LayerCore* c = &handle->c;
    const LayerCore& f = members[0]->c;
    c->in = f.in; c->k = f.k; c->cb = f.cb; c->flags = f.flags; c->groups = count;
    int64_t total = 0;
    bool any_bias = false;
    for (int g = 0; g < count; ++g) {
        c->gcol0[g] = static_cast<int>(total);
        c->gout[g] = members[g]->c.out;
        total += members[g]->c.out;
        any_bias = any_bias || members[g]->c.bias != nullptr;
    }
    int rc = 0;
    if (total / 128 >= static_cast<int64_t>(kCounterBytes / sizeof(unsigned int))) rc = fail("group width overflow");
    c->out = static_cast<int>(total);
    const size_t row_bytes = static_cast<size_t>(c->out / 16) * 32 * c->k;       // one input-tile row of all column blocks
    if (!rc) rc = check(cudaMalloc(&c->wq, row_bytes * (c->in / 16)), "cudaMalloc(weights)");
    if (!rc) rc = check(cudaMalloc(&c->suh, static_cast<size_t>(count) * c->in * sizeof(__half)), "cudaMalloc(scales)");
    if (!rc) rc = check(cudaMalloc(&c->svh, static_cast<size_t>(c->out) * sizeof(__half)), "cudaMalloc(scales)");
    if (!rc && any_bias) {
        rc = check(cudaMalloc(&c->bias, static_cast<size_t>(c->out) * sizeof(__half)), "cudaMalloc(bias)");
        if (!rc) rc = check(cudaMemset(c->bias, 0, static_cast<size_t>(c->out) * sizeof(__half)), "clear bias");
    }
    for (int g = 0; g < count && !rc; ++g) {
        const LayerCore& m = members[g]->c;
        // concatenate along the output axis: the layout is column-block-major, so a member's blocks go behind the
        // previous members' blocks as one contiguous copy
        rc = check(cudaMemcpy(c->wq + quad_row_offset(0, c->gcol0[g] / 128, c->in / 16, c->k), m.wq,
                              static_cast<size_t>(m.out / 16) * 32 * m.k * (m.in / 16), cudaMemcpyDeviceToDevice), "concatenate weights");
        if (!rc) rc = check(cudaMemcpy(c->suh + static_cast<size_t>(g) * c->in, m.suh, static_cast<size_t>(c->in) * sizeof(__half),
                                       cudaMemcpyDeviceToDevice), "copy scales");
        if (!rc) rc = check(cudaMemcpy(c->svh + c->gcol0[g], m.svh, static_cast<size_t>(m.out) * sizeof(__half),
                                       cudaMemcpyDeviceToDevice), "copy scales");
        if (!rc && m.bias) rc = check(cudaMemcpy(c->bias + c->gcol0[g], m.bias, static_cast<size_t>(m.out) * sizeof(__half),
                                                 cudaMemcpyDeviceToDevice), "copy bias");
    }
    if (!rc) rc = check(cudaDeviceSynchronize(), "group_create");
    if (rc) {
        b200exl3_group_free(handle);
        return -1;
    }
    *out_handle = handle;
    return 0;
}

void b200exl3_group_free(b200exl3_group* h) {
    if (!h) return;
    core_free(h->c);
    delete h;
}

int b200exl3_group_count(const b200exl3_group* h) { return h ? h->c.groups : fail("NULL handle"); }

int b200exl3_group_workspace_bytes(const b200exl3_group* h, int64_t rows, size_t* out_bytes) {
    if (!h) return fail("NULL argument");
    return core_workspace_bytes(h->c, rows, out_bytes);
}

int b200exl3_group_forward(const b200exl3_group* h, const void* d_x, int x_dtype, int64_t rows, void* const* d_ys, void* ws,
                           size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_ys) return fail("NULL buffer");
    for (int g = 0; g < h->c.groups; ++g)
        if (!d_ys[g]) return fail("NULL buffer");
    return forward_common(h->c, d_x, x_dtype, nullptr, rows, d_ys, nullptr, ws, ws_bytes, as_stream(s));
}

int b200exl3_group_forward_fused(const b200exl3_group* h, const b200exl3_prologue* pro, const void* d_x, int64_t rows, void* const* d_ys,
                                 void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (!d_x || !d_ys) return fail("NULL buffer");
    if (check_prologue(pro, d_x, rows)) return -1;
    for (int g = 0; g < h->c.groups; ++g)
        if (!d_ys[g] && !(pro->epilogue == 2 && g > 0)) return fail("NULL buffer");       // the rotary epilogue writes k and v to the caches
    if (pro->epilogue == 1) return fail("the residual epilogue belongs to plain layers");
    if (pro->epilogue == 2) {
        const LayerCore& c = h->c;
        if (c.groups != 3 || c.gout[1] != c.gout[2] || c.gout[0] % 128 || c.gout[1] % 128)
            return fail("the rotary epilogue needs a group of three members [q | k | v] with 128-wide heads and as many k as v heads");
    }
    return forward_common(h->c, d_x, kF16, nullptr, rows, d_ys, nullptr, ws, ws_bytes, as_stream(s), nullptr, pro);
}

/* ---- a decode step as one persistent launch ----------------------------------------------------------------- */

struct b200exl3_stack {
    int n_ops, k, cb;
    bool exact;
    StackPlan plan;
    StackOp* d_ops;
    char* scratch;
    size_t sync_bytes, scratch_bytes;
    StackArgs args;
};

int b200exl3_stack_create(const b200exl3_stack_op* ops, int count, int x_dtype, int64_t rows, b200exl3_stack** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (!ops || count <= 0 || count > kStackMaxOps) return fail("a step needs between 1 and %d layers", kStackMaxOps);
    if (rows <= 0 || rows > kStackMaxRows) return fail("a step takes 1 to %d activation rows, got %lld", kStackMaxRows, static_cast<long long>(rows));
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    const LayerCore* first = nullptr;
    const b200exl3_tp* tp = nullptr;
    std::vector<StackOp> table(static_cast<size_t>(count));
    for (int i = 0; i < count; ++i) {
        const b200exl3_stack_op& src = ops[i];
        if ((src.linear != nullptr) == (src.group != nullptr)) return fail("layer %d: give exactly one of linear and group", i);
        const LayerCore& c = src.linear ? src.linear->c : src.group->c;
        if (!first) first = &c;
        if (c.k != first->k || c.cb != first->cb || ((c.flags ^ first->flags) & B200EXL3_EXACT_WEIGHTS))
            return fail("layer %d: every layer of a step must share bit width, codebook and weight mode", i);
        if (!src.d_x || !aligned16(src.d_x)) return fail("layer %d: input pointer is NULL or not 16-byte aligned", i);
        for (int g = 0; g < c.groups; ++g) {
            // the residual epilogue stores through its own pointer, the rotary one writes k and v into the caches
            const bool unused = src.fused && ((src.fused->epilogue == 1) || (src.fused->epilogue == 2 && g > 0));
            if ((!src.d_y[g] && !unused) || !aligned16(src.d_y[g])) return fail("layer %d: output pointer %d is NULL or not 16-byte aligned", i, g);
        }
        if (src.tp) {
            if (c.groups != 1) return fail("layer %d: a grouped layer cannot be a row shard", i);
            if (tp && tp != src.tp) return fail("layer %d: a step uses one exchange context", i);
            tp = src.tp;
            if (rows * (c.out / 128) > src.tp->max_units)
                return fail("layer %d: %lld units exceed the exchange buffers' %d", i, static_cast<long long>(rows * (c.out / 128)), src.tp->max_units);
        }
        StackOp& o = table[static_cast<size_t>(i)];
        o = StackOp{};
        o.wq = c.wq; o.x = src.d_x; o.suh = c.suh; o.svh = c.svh; o.bias = c.bias;
        o.groups = c.groups; o.in = c.in; o.out = c.out;
        for (int g = 0; g < c.groups; ++g) { o.gy[g] = src.d_y[g]; o.gcol0[g] = c.gcol0[g]; o.gout[g] = c.gout[g]; }
        o.tp_unit0 = src.tp ? 0 : -1;
        if (src.fused && (src.fused->kind != 0 || src.fused->epilogue != 0)) {
            const b200exl3_prologue* f = src.fused;
            if (x_dtype != kF16) return fail("layer %d: fused operators need an fp16 step", i);
            if (check_prologue(f, src.d_x, rows)) return -1;
            if (f->kind == 1) return fail("layer %d: a step takes the RMSNorm prologue from block sums (kind 3), not kind 1", i);
            if (f->epilogue == 1 && c.groups != 1) return fail("layer %d: the residual epilogue belongs to plain layers", i);
            if (f->epilogue == 2 && (c.groups != 3 || c.gout[1] != c.gout[2] || c.gout[0] % 128 || c.gout[1] % 128))
                return fail("layer %d: the rotary epilogue needs a group of three members [q | k | v] with 128-wide heads", i);
            o.prologue = f->kind; o.epilogue = f->epilogue;
            o.pro_aux = reinterpret_cast<const __half*>(f->d_aux);
            o.pro_weight = reinterpret_cast<const __half*>(f->d_weight);
            o.pro_sumsq = f->d_sumsq; o.pro_eps = f->eps;
            o.epi_residual = reinterpret_cast<const __half*>(f->d_residual);
            o.epi_sum = reinterpret_cast<__half*>(f->d_residual_out);
            o.epi_sumsq = f->d_sumsq_out;
            if (f->epilogue == 2) {
                o.epi_pos = f->d_pos; o.epi_log2_theta = log2f(f->theta); o.epi_max_ctx = f->max_ctx;
                o.epi_k_cache = reinterpret_cast<__half*>(f->d_k_cache);
                o.epi_v_cache = reinterpret_cast<__half*>(f->d_v_cache);
            }
        }
    }
    b200exl3_stack* h = new (std::nothrow) b200exl3_stack{};
    if (!h) return fail("out of host memory");
    h->n_ops = count; h->k = first->k; h->cb = first->cb; h->exact = (first->flags & B200EXL3_EXACT_WEIGHTS) != 0;
    h->plan = plan_stack(h->k, static_cast<int>(rows), count);
    size_t max_words = 0;
    for (int i = 0; i < count; ++i) {
        StackOp& o = table[static_cast<size_t>(i)];
        if (!plan_stack_op(h->plan, o)) {
            delete h;
            return fail("layer %d (%d -> %d) cannot be part of a step", i, o.in, o.out);
        }
        max_words = std::max(max_words, static_cast<size_t>(o.col_blocks) * o.max_pieces * rows * 128 * sizeof(unsigned long long));
    }
    // [finished blocks per layer | CTAs that left | status | launch number] then the tagged partial sums, by layer parity
    h->sync_bytes = round256((static_cast<size_t>(count) + 3) * sizeof(unsigned int));
    max_words = round256(max_words);
    h->scratch_bytes = h->sync_bytes + 2 * max_words;
    int rc = check(cudaMalloc(&h->d_ops, table.size() * sizeof(StackOp)), "cudaMalloc(step table)");
    if (!rc) rc = check(cudaMalloc(&h->scratch, h->scratch_bytes), "cudaMalloc(step scratch)");
    if (!rc) rc = check(cudaMemcpy(h->d_ops, table.data(), table.size() * sizeof(StackOp), cudaMemcpyHostToDevice), "copy step table");
    if (!rc) rc = check(cudaMemset(h->scratch, 0, h->scratch_bytes), "clear step scratch");
    if (!rc) rc = check(cudaDeviceSynchronize(), "stack_create");
    if (rc) {
        b200exl3_stack_free(h);
        return -1;
    }
    StackArgs& a = h->args;
    a = StackArgs{};
    a.ops = h->d_ops; a.n_ops = count; a.rows = static_cast<int>(rows); a.x_dtype = x_dtype; a.y_dtype = x_dtype;
    a.op_done = reinterpret_cast<unsigned int*>(h->scratch);
    a.exit_count = a.op_done + count;
    a.error = a.op_done + count + 1;
    a.launch = a.op_done + count + 2;
    a.piece_words[0] = reinterpret_cast<unsigned long long*>(h->scratch + h->sync_bytes);
    a.piece_words[1] = reinterpret_cast<unsigned long long*>(h->scratch + h->sync_bytes + max_words);
    a.warp_smem = h->plan.warp_smem; a.xs_offset = h->plan.xs_offset; a.stage_offset = h->plan.stage_offset;
    a.table_offset = h->plan.table_offset; a.x_blocks = h->plan.x_blocks;
    for (const StackOp& o : table) a.fused |= (o.prologue != 0 || o.epilogue != 0) ? 1 : 0;
    a.wait_ns = static_cast<unsigned long long>(g_stack_wait_ms.load()) * 1000000ull;
    if (tp) a.tp = tp_peers(tp);
    *out_handle = h;
    return 0;
}

void b200exl3_stack_free(b200exl3_stack* h) {
    if (!h) return;
    cudaFree(h->d_ops);
    cudaFree(h->scratch);
    delete h;
}

int b200exl3_stack_forward(b200exl3_stack* h, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    h->args.trace = g_stack_trace.load();
    return check(launch_stack(h->args, h->k, h->cb, h->exact, h->plan, as_stream(s)), "decode-step kernel");
}

int b200exl3_stack_status(const b200exl3_stack* h, int* out_status) {
    if (!h || !out_status) return fail("NULL argument");
    unsigned int flag = 0;
    B200_TRY(cudaMemcpy(&flag, h->args.error, sizeof flag, cudaMemcpyDeviceToHost), "read step status");
    *out_status = static_cast<int>(flag);
    return 0;
}

int b200exl3_stack_reset(b200exl3_stack* h) {
    if (!h) return fail("NULL handle");
    B200_TRY(cudaDeviceSynchronize(), "stack_reset");
    B200_TRY(cudaMemset(h->scratch, 0, h->scratch_bytes), "clear step scratch");
    return check(cudaDeviceSynchronize(), "stack_reset");
}

int b200exl3_stack_geometry(const b200exl3_stack* h, int* out_grid, size_t* out_smem_bytes) {
    if (!h) return fail("NULL handle");
    if (out_grid) *out_grid = h->plan.grid;
    if (out_smem_bytes) *out_smem_bytes = h->plan.smem_bytes;
    return 0;
}

/* ---- Exl3SwitchGlu ----------------------------------------------------------------------------- */

// Slots (token, choice) handled per pass: bounds the scratch and keeps the virtual column blocks of one
// launch below the arrival-counter capacity.
constexpr int64_t kMoeChunkSlots = 256;

static int64_t moe_blocks_per_slot(int in, int hidden) { return std::max(2 * hidden / 128, in / 128); }
static int64_t moe_chunk_rows(const b200exl3_moe* h) {
    const int64_t counters = static_cast<int64_t>(kCounterBytes / sizeof(unsigned int)) - 2;
    const int64_t slots = std::min(kMoeChunkSlots, counters / moe_blocks_per_slot(h->in, h->hidden));
    return std::max<int64_t>(1, slots / h->top_k);
}

struct MoeLayout {
    size_t xgu, ygu, xdown, ydown, partials, total;
    QmvPlan gu_plan, down_plan;
};

static MoeLayout moe_layout(const b200exl3_moe* h, int64_t rows) {
    MoeLayout l{};
    const int64_t slots = std::min(rows, moe_chunk_rows(h)) * h->top_k;
    l.gu_plan = plan_qmv(h->in, static_cast<int>(slots * 2 * h->hidden), h->k, 1);
    l.down_plan = plan_qmv(h->hidden, static_cast<int>(slots * h->in), h->k, 1);
    size_t at = kCounterBytes;
    l.xgu = at; at += round256(static_cast<size_t>(slots) * 2 * h->in * sizeof(__half));
    l.ygu = at; at += round256(static_cast<size_t>(slots) * 2 * h->hidden * sizeof(float));
    l.xdown = at; at += round256(static_cast<size_t>(slots) * h->hidden * sizeof(__half));
    l.ydown = at; at += round256(static_cast<size_t>(slots) * h->in * sizeof(float));
    l.partials = at;
    at += std::max(qmv_partial_bytes(l.gu_plan, static_cast<int>(slots * 2 * h->hidden), 1),
                   qmv_partial_bytes(l.down_plan, static_cast<int>(slots * h->in), 1));
    l.total = at;
    return l;
}

// Expert-sorted form, used from this many slots on: slots are grouped by expert into segments of kMoeSegRows rows,
// so an expert's columns are decoded once per segment instead of once per slot.
constexpr int64_t kMoeSortedMinSlots = 33;

static int64_t moe_max_segments(const b200exl3_moe* h, int64_t slots, int seg_rows) {
    return std::min<int64_t>(h->experts, slots) + slots / seg_rows;   // one partly filled segment per expert at most
}
// Segments of 8 rows run in the fused kernel; once most experts see many rows, segments of 64 rows run on the tensor cores.
constexpr int64_t kMoeTensorSlotsPerExpert = 12;
static int moe_seg_rows(const b200exl3_moe* h, int64_t rows) {
    return g_qmm_enabled && rows * h->top_k >= kMoeTensorSlotsPerExpert * h->experts ? kQmmSegRows : kMoeSegRows;
}
// rows per pass (bounds the scratch); the passes of a call get equal shares
constexpr int64_t kMoeSortedPassSlots = 16384;
static int64_t moe_sorted_chunk_rows(const b200exl3_moe* h, int64_t rows) {
    const int64_t cap = std::max<int64_t>(1, kMoeSortedPassSlots / h->top_k);
    const int64_t passes = (rows + cap - 1) / cap;
    return (rows + passes - 1) / passes;
}

struct MoeSortedLayout {
    size_t counters, counter_bytes, seg_count, seg_expert, row_slot, slot_row, xgu, ygu, xdown, ydown, partials, total;
    int max_segments, seg_rows;
    QmvPlan gu_plan, down_plan;
};

static MoeSortedLayout moe_sorted_layout(const b200exl3_moe* h, int64_t rows) {
    MoeSortedLayout l{};
    const int64_t slots = moe_sorted_chunk_rows(h, rows) * h->top_k;
    const int seg_rows = moe_seg_rows(h, rows);
    const int64_t segs = moe_max_segments(h, slots, seg_rows);
    l.max_segments = static_cast<int>(segs);
    l.seg_rows = seg_rows;
    l.gu_plan = plan_qmv(h->in, static_cast<int>(segs * 2 * h->hidden), h->k, kMoeSegRows);
    l.down_plan = plan_qmv(h->hidden, static_cast<int>(segs * h->in), h->k, kMoeSegRows);
    size_t at = kCounterBytes;
    // arrival counters of its own (one per virtual column block; the header's 16 KiB would cap a pass at 4093 blocks),
    // cleared at the start of every call
    l.counter_bytes = round256((static_cast<size_t>(segs) * moe_blocks_per_slot(h->in, h->hidden) + 2) * sizeof(unsigned int));
    l.counters = at; at += l.counter_bytes;
    l.seg_count = at; at += 256;
    l.seg_expert = at; at += round256(static_cast<size_t>(segs) * sizeof(uint32_t));
    l.row_slot = at; at += round256(static_cast<size_t>(segs) * seg_rows * sizeof(uint32_t));
    l.slot_row = at; at += round256(static_cast<size_t>(slots) * sizeof(uint32_t));
    l.xgu = at; at += round256(static_cast<size_t>(segs) * 2 * seg_rows * h->in * sizeof(__half));
    l.ygu = at; at += round256(static_cast<size_t>(segs) * 2 * seg_rows * h->hidden * sizeof(float));
    l.xdown = at; at += round256(static_cast<size_t>(segs) * seg_rows * h->hidden * sizeof(__half));
    l.ydown = at; at += round256(static_cast<size_t>(segs) * seg_rows * h->in * sizeof(float));
    l.partials = at;
    if (seg_rows == kMoeSegRows)
        at += std::max(qmv_partial_bytes(l.gu_plan, static_cast<int>(segs * 2 * h->hidden), kMoeSegRows),
                       qmv_partial_bytes(l.down_plan, static_cast<int>(segs * h->in), kMoeSegRows));
    l.total = at;
    return l;
}

static bool moe_sorted(const b200exl3_moe* h, int64_t rows) {
    // worth it once experts see several rows each: below two slots per expert one row per slot is faster
    if (!g_moe_sorted || rows * h->top_k < std::max<int64_t>(kMoeSortedMinSlots, 2 * static_cast<int64_t>(h->experts))) return false;
    // the route plan keeps 2 * experts + 1 counters and one 16-bit expert id per slot of a pass in 48 KiB of shared
    // memory; shapes beyond that keep one row per slot
    const size_t plan_smem = (2 * static_cast<size_t>(h->experts) + 1) * sizeof(int) +
                             static_cast<size_t>(moe_sorted_chunk_rows(h, rows)) * h->top_k * sizeof(unsigned short);
    return plan_smem <= 48 * 1024 && h->experts <= 65535;
}

int b200exl3_moe_create(const uint16_t* d_gu_trellis, const void* d_gu_suh, const void* d_gu_svh,
                        const uint16_t* d_down_trellis, const void* d_down_suh, const void* d_down_svh, int scale_dtype,
                        int experts, int in, int hidden, int top_k, int k, int cb, uint32_t flags, b200exl3_moe** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (valid_format(k, cb)) return -1;
    if (experts <= 0 || top_k <= 0 || top_k > experts || in <= 0 || hidden <= 0 || in % 128 || hidden % 128 || k == 7 ||
        static_cast<int64_t>(experts) * 2 * hidden > INT32_MAX || static_cast<int64_t>(experts) * in > INT32_MAX)
        return fail("invalid or overflowing SwitchGLU dimensions");
    if (top_k * moe_blocks_per_slot(in, hidden) > static_cast<int64_t>(kCounterBytes / sizeof(unsigned int)) - 2)
        return fail("invalid or overflowing SwitchGLU dimensions");
    if (!d_gu_trellis || !d_down_trellis || !d_gu_suh || !d_gu_svh || !d_down_suh || !d_down_svh)
        return fail("SwitchGLU trellis/scales disagree");
    if (!dtype_is_float(scale_dtype)) return fail("unsupported scale dtype %d", scale_dtype);
    if (!aligned16(d_gu_trellis) || !aligned16(d_down_trellis)) return fail("device pointers must be 16-byte aligned");
    b200exl3_moe* h = new (std::nothrow) b200exl3_moe{};
    if (!h) return fail("out of host memory");
    h->experts = experts; h->in = in; h->hidden = hidden; h->top_k = top_k; h->k = k; h->cb = cb; h->flags = flags;
    auto convert = [&](const void* src, int64_t n, __half** dst) -> int {
        B200_TRY(cudaMalloc(dst, static_cast<size_t>(n) * sizeof(__half)), "cudaMalloc(scales)");
        to_half_kernel<<<static_cast<unsigned>((n + 255) / 256), 256>>>(src, scale_dtype, n, *dst);
        return check(cudaGetLastError(), "convert scales");
    };
    auto repack = [&](const uint16_t* src, int tiles_k, int64_t tiles_n, uint32_t** dst) -> int {
        const size_t bytes = static_cast<size_t>(tiles_k) * tiles_n * 16 * k * sizeof(uint16_t);
        B200_TRY(cudaMalloc(dst, bytes), "cudaMalloc(weights)");
        return check(launch_repack_quads(reinterpret_cast<const uint32_t*>(src), tiles_k, static_cast<int>(tiles_n), k, *dst, 0),
                     "repack weights");
    };
    int rc = convert(d_gu_suh, static_cast<int64_t>(experts) * 2 * in, &h->gu_suh);
    if (!rc) rc = convert(d_gu_svh, static_cast<int64_t>(experts) * 2 * hidden, &h->gu_svh);
    if (!rc) rc = convert(d_down_suh, static_cast<int64_t>(experts) * hidden, &h->down_suh);
    if (!rc) rc = convert(d_down_svh, static_cast<int64_t>(experts) * in, &h->down_svh);
    if (!rc) rc = repack(d_gu_trellis, in / 16, static_cast<int64_t>(experts) * 2 * hidden / 16, &h->gu_wq);
    if (!rc) rc = repack(d_down_trellis, hidden / 16, static_cast<int64_t>(experts) * in / 16, &h->down_wq);
    if (!rc) rc = check(cudaDeviceSynchronize(), "moe_create");
    if (rc) {
        b200exl3_moe_free(h);
        return -1;
    }
    *out_handle = h;
    return 0;
}

void b200exl3_moe_free(b200exl3_moe* h) {
    if (!h) return;
    cudaFree(h->gu_wq); cudaFree(h->down_wq);
    cudaFree(h->gu_suh); cudaFree(h->gu_svh); cudaFree(h->down_suh); cudaFree(h->down_svh);
    delete h;
}

int b200exl3_moe_workspace_bytes(const b200exl3_moe* h, int64_t rows, size_t* out_bytes) {
    if (!h || !out_bytes) return fail("NULL argument");
    if (rows <= 0) return fail("invalid SwitchGLU input/routes");
    *out_bytes = moe_sorted(h, rows) ? moe_sorted_layout(h, rows).total : moe_layout(h, rows).total;
    return 0;
}

// Two launches instead of four for a small batch (one row per slot): the down product takes the SwiGLU glue as its
// prologue and finish_and_reduce as its epilogue.  The (token, block) arrival counters of the epilogue sit behind the
// column-block counters in the workspace header; batches whose counters do not fit take the four-launch form.
// Measured on 128 experts, top-8, 2048 <-> 768, 3 bits, one token: 39.5 us against 39.1 us for the four launches with
// dependent launch on (42.1 against 40.2 without): the launch gaps were already hidden, and every warp of the down
// product now redoes the glue of its own input blocks.  Same bits either way; off unless the option asks for it.
static bool moe_fused_fits(const b200exl3_moe* h, int64_t rows) {
    const int64_t blocks = h->in / 128;
    return g_moe_fused.load() != 0 && (rows * h->top_k + rows) * blocks + 1 <= static_cast<int64_t>(kCounterBytes / sizeof(unsigned int)) - 1;
}

int b200exl3_moe_forward(const b200exl3_moe* h, const void* d_x, int x_dtype, int64_t rows, const uint32_t* d_selected,
                         const void* d_scores, int score_dtype, void* d_y, void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (!h) return fail("NULL handle");
    if (rows <= 0) return fail("invalid SwitchGLU input/routes");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (score_dtype != kF16 && score_dtype != kF32) return fail("unsupported score dtype %d", score_dtype);
    if (!d_x || !d_selected || !d_scores || !d_y) return fail("NULL buffer");
    if (!aligned16(ws) || !aligned16(d_y)) return fail("device pointers must be 16-byte aligned");
    cudaStream_t stream = as_stream(s);
    char* base = static_cast<char*>(ws);
    const bool exact = (h->flags & B200EXL3_EXACT_WEIGHTS) != 0;
    const size_t x_size = dtype_size(x_dtype), score_size = dtype_size(score_dtype);
    if (moe_sorted(h, rows)) {
        const MoeSortedLayout l = moe_sorted_layout(h, rows);
        if (!ws || ws_bytes < l.total) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, l.total);
        int* seg_count = reinterpret_cast<int*>(base + l.seg_count);
        uint32_t* seg_expert = reinterpret_cast<uint32_t*>(base + l.seg_expert);
        uint32_t* row_slot = reinterpret_cast<uint32_t*>(base + l.row_slot);
        uint32_t* slot_row = reinterpret_cast<uint32_t*>(base + l.slot_row);
        __half* xgu = reinterpret_cast<__half*>(base + l.xgu);
        float* ygu = reinterpret_cast<float*>(base + l.ygu);
        __half* xdown = reinterpret_cast<__half*>(base + l.xdown);
        float* ydown = reinterpret_cast<float*>(base + l.ydown);
        const int segs = l.max_segments, seg_rows = l.seg_rows;
        const int64_t chunk = moe_sorted_chunk_rows(h, rows);
        B200_TRY(cudaMemsetAsync(base + l.counters, 0, l.counter_bytes, stream), "clear arrival counters");
        for (int64_t r0 = 0; r0 < rows; r0 += chunk) {
            const int64_t n = std::min(chunk, rows - r0), slots = n * h->top_k;
            const uint32_t* sel = d_selected + r0 * h->top_k;
            // kMoeSegRows rows per segment against the columns of the segment's expert; segments past the count are skipped
            auto mapped = [&](const uint32_t* wq, const __half* xhat, int in, int width, int proj, int stride_blocks, float* yhat,
                              const QmvPlan& plan) {
                const int out = segs * proj * width;
                QmvArgs a{};
                a.wq = wq; a.xhat = xhat; a.xhat_group_stride = static_cast<int64_t>(kMoeSegRows) * in;
                a.counters = reinterpret_cast<unsigned int*>(base + l.counters);
                a.error = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
                a.partials = reinterpret_cast<float*>(base + l.partials);
                a.yhat = yhat;
                a.groups = 1; a.gcol0[0] = 0; a.gout[0] = out;
                a.x_dtype = kF16; a.y_dtype = kF16;
                a.in = in; a.out = out; a.rows = kMoeSegRows;
                a.tiles_n = h->experts * proj * width / 16;
                a.map_selected = seg_expert; a.map_count = seg_count;
                a.map_blocks = width / 128; a.map_proj = proj; a.map_stride_blocks = stride_blocks; a.map_experts = h->experts;
                return launch_qmv(a, h->k, h->cb, exact, plan, stream);
            };
            // the same on the tensor cores: 64 rows per segment, one CTA per (segment, projection, 128 columns)
            auto mapped_tensor = [&](const uint32_t* wq, const __half* xhat, int in, int width, int proj, int stride_blocks, float* yhat) {
                return launch_qmm_mapped(wq, in, width, h->experts * proj * width / 16, h->k, h->cb, xhat, segs, proj, stride_blocks,
                                         h->experts, seg_expert, seg_count, yhat,
                                         reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int)), stream);
            };
            const bool tensor = seg_rows == kQmmSegRows;
            B200_TRY(launch_route_plan(sel, slots, h->experts, segs, seg_rows, seg_count, seg_expert, row_slot, slot_row, stream), "route plan");
            B200_TRY(launch_routed_prepare_padded(static_cast<const char*>(d_x) + static_cast<size_t>(r0) * h->in * x_size, x_dtype,
                                                  h->gu_suh, seg_expert, slot_row, slots, h->top_k, 2, segs, seg_rows, h->in, xgu,
                                                  stream), "routed prepare");
            B200_TRY(tensor ? mapped_tensor(h->gu_wq, xgu, h->in, h->hidden, 2, h->experts * (h->hidden / 128), ygu)
                            : mapped(h->gu_wq, xgu, h->in, h->hidden, 2, h->experts * (h->hidden / 128), ygu, l.gu_plan),
                     "expert gate/up kernel");
            B200_TRY(launch_glu_down_input_padded(ygu, h->gu_svh, h->down_suh, seg_expert, row_slot, seg_count, h->experts, segs,
                                                  seg_rows, h->hidden, h->hidden, xdown, stream), "SwiGLU glue");
            B200_TRY(tensor ? mapped_tensor(h->down_wq, xdown, h->hidden, h->in, 1, 0, ydown)
                            : mapped(h->down_wq, xdown, h->hidden, h->in, 1, 0, ydown, l.down_plan),
                     "expert down kernel");
            B200_TRY(launch_finish_and_reduce_padded(ydown, h->down_svh, sel, slot_row, h->experts,
                                                     static_cast<const char*>(d_scores) + static_cast<size_t>(r0) * h->top_k * score_size,
                                                     score_dtype, n, h->top_k, h->in, segs, seg_rows,
                                                     static_cast<char*>(d_y) + static_cast<size_t>(r0) * h->in * score_size, stream),
                     "expert reduction");
        }
        return 0;
    }
    const MoeLayout l = moe_layout(h, rows);
    if (!ws || ws_bytes < l.total) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, l.total);
    __half* xgu = reinterpret_cast<__half*>(base + l.xgu);
    float* ygu = reinterpret_cast<float*>(base + l.ygu);
    __half* xdown = reinterpret_cast<__half*>(base + l.xdown);
    float* ydown = reinterpret_cast<float*>(base + l.ydown);
    const int64_t chunk = moe_chunk_rows(h);
    for (int64_t r0 = 0; r0 < rows; r0 += chunk) {
        const int64_t n = std::min(chunk, rows - r0), slots = n * h->top_k;
        const uint32_t* sel = d_selected + r0 * h->top_k;
        // every slot is one activation row against the columns of its own expert
        auto mapped = [&](const uint32_t* wq, const __half* xhat, int in, int width, int proj, int stride_blocks, float* yhat) {
            const int out = static_cast<int>(slots * proj * width);
            QmvArgs a{};
            a.wq = wq; a.xhat = xhat; a.xhat_group_stride = in;
            if (!xhat) {                                      // fused routed rotation
                a.x = static_cast<const char*>(d_x) + static_cast<size_t>(r0) * h->in * x_size;
                a.suh = h->gu_suh;
                a.map_top_k = h->top_k;
            }
            a.counters = reinterpret_cast<unsigned int*>(base);
            a.error = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
            a.partials = reinterpret_cast<float*>(base + l.partials);
            a.yhat = yhat;
            a.groups = 1; a.gcol0[0] = 0; a.gout[0] = out;
            a.x_dtype = xhat ? kF16 : x_dtype; a.y_dtype = kF16;
            a.in = in; a.out = out; a.rows = 1;
            a.tiles_n = h->experts * proj * width / 16;
            a.map_selected = sel; a.map_blocks = width / 128; a.map_proj = proj; a.map_stride_blocks = stride_blocks;
            a.map_experts = h->experts;
            return launch_qmv(a, h->k, h->cb, exact, plan_qmv(in, out, h->k, 1), stream);
        };
        // gate/up: the kernel rotates each slot's token row itself, with the input scales of the slot's expert
        B200_TRY(mapped(h->gu_wq, nullptr, h->in, h->hidden, 2, h->experts * (h->hidden / 128), ygu), "expert gate/up kernel");
        if (moe_fused_fits(h, n)) {
            const int out = static_cast<int>(slots * h->in);
            QmvArgs a{};
            a.wq = h->down_wq; a.xhat = nullptr; a.xhat_group_stride = h->hidden;
            a.x = ygu;                                        // read through the prologue only
            a.suh = h->down_suh;
            a.prologue = 4; a.pro_ygu = ygu; a.pro_gu_svh = h->gu_svh; a.pro_logical = h->hidden;
            a.map_top_k = h->top_k;
            a.counters = reinterpret_cast<unsigned int*>(base);
            a.error = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
            a.partials = reinterpret_cast<float*>(base + l.partials);
            a.yhat = ydown;
            a.epilogue = 3; a.svh = h->down_svh;
            a.epi_scores = static_cast<const char*>(d_scores) + static_cast<size_t>(r0) * h->top_k * score_size;
            a.epi_score_f32 = score_dtype == kF32 ? 1 : 0;
            a.epi_counter0 = static_cast<int>(slots * (h->in / 128));
            a.groups = 1; a.gcol0[0] = 0; a.gout[0] = out;
            a.gy[0] = static_cast<char*>(d_y) + static_cast<size_t>(r0) * h->in * score_size;
            a.x_dtype = kF16; a.y_dtype = kF16;
            a.in = h->hidden; a.out = out; a.rows = 1;
            a.tiles_n = h->experts * h->in / 16;
            a.map_selected = sel; a.map_blocks = h->in / 128; a.map_proj = 1; a.map_stride_blocks = 0; a.map_experts = h->experts;
            B200_TRY(launch_qmv(a, h->k, h->cb, exact, plan_qmv(h->hidden, out, h->k, 1), stream), "expert down kernel");
            continue;
        }
        B200_TRY(launch_glu_down_input(ygu, h->gu_svh, h->down_suh, sel, h->experts, slots, h->hidden, h->hidden, xdown, stream),
                 "SwiGLU glue");
        B200_TRY(mapped(h->down_wq, xdown, h->hidden, h->in, 1, 0, ydown), "expert down kernel");
        B200_TRY(launch_finish_and_reduce(ydown, h->down_svh, sel, h->experts,
                                          static_cast<const char*>(d_scores) + static_cast<size_t>(r0) * h->top_k * score_size,
                                          score_dtype, n, h->top_k, h->in,
                                          static_cast<char*>(d_y) + static_cast<size_t>(r0) * h->in * score_size, stream),
                 "expert reduction");
    }
    return 0;
}



/* ---- expert_mapped and the two glue operators of the expert block, as stand-alone entry points ------------------------ */

int b200exl3_expert_mapped(const void* d_x, int x_dtype, const uint16_t* d_trellis, int64_t source_tiles, const uint16_t* d_suh,
                           const uint16_t* d_svh, const uint32_t* d_selected, int64_t slots, int in, int out, int projections,
                           int64_t projection_stride_tiles, int k, int cb, int input_pretransformed, int return_raw, void* d_out,
                           b200exl3_stream s) {
    if (valid_format(k, cb)) return -1;
    if (k == 7) return fail("K = 7 is not supported by the expert-mapped product");
    if (slots <= 0 || projections <= 0 || in <= 0 || out <= 0 || in % 128 || out % 128 || source_tiles <= 0 || source_tiles % 8 ||
        projection_stride_tiles < 0 || projection_stride_tiles % 8)
        return fail("invalid expert-mapped dimensions");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_trellis || !d_selected || !d_out || (!input_pretransformed && !d_suh) || (!return_raw && !d_svh)) return fail("NULL buffer");
    if (input_pretransformed && x_dtype != kF16) return fail("pretransformed expert input must be fp16");
    const int width_tiles = out / 16;
    const int64_t experts = projection_stride_tiles > 0 ? projection_stride_tiles / width_tiles : source_tiles / width_tiles;
    if (experts <= 0 || (projections - 1) * projection_stride_tiles + experts * width_tiles > source_tiles)
        return fail("expert bank is smaller than the routes' layout");
    cudaStream_t stream = as_stream(s);
    const int64_t rows = slots * projections;
    const int blocks_per_slot = projections * (out / 128);
    const int64_t pass_slots = std::max<int64_t>(1, (static_cast<int64_t>(kCounterBytes / sizeof(unsigned int)) - 2) / blocks_per_slot);
    // temporaries of a tool-level call: the bank in the quad layout, rotated rows, raw products, scratch
    uint32_t* wq = nullptr;
    __half* xhat = nullptr;
    float* raw = nullptr;
    char* ws = nullptr;
    const size_t bank_bytes = static_cast<size_t>(in / 16) * source_tiles * 16 * k * sizeof(uint16_t);
    const QmvPlan plan = plan_qmv(in, static_cast<int>(std::min(pass_slots, slots) * projections * out), k, 1);
    const size_t ws_bytes = kCounterBytes + qmv_partial_bytes(plan, static_cast<int>(std::min(pass_slots, slots) * projections * out), 1);
    int rc = check(cudaMalloc(&wq, bank_bytes), "cudaMalloc(bank)");
    if (!rc) rc = check(cudaMalloc(&xhat, static_cast<size_t>(rows) * in * sizeof(__half)), "cudaMalloc(rows)");
    if (!rc && !return_raw) rc = check(cudaMalloc(&raw, static_cast<size_t>(rows) * out * sizeof(float)), "cudaMalloc(products)");
    if (!rc) rc = check(cudaMalloc(&ws, ws_bytes), "cudaMalloc(scratch)");
    if (!rc) rc = check(cudaMemsetAsync(ws, 0, kCounterBytes, stream), "clear scratch");
    if (!rc) rc = check(launch_repack_quads(reinterpret_cast<const uint32_t*>(d_trellis), in / 16, static_cast<int>(source_tiles), k, wq, stream),
                        "repack weights");
    if (!rc) {
        if (input_pretransformed) rc = check(cudaMemcpyAsync(xhat, d_x, static_cast<size_t>(rows) * in * sizeof(__half), cudaMemcpyDeviceToDevice, stream), "copy rows");
        else rc = check(launch_prepare(d_x, x_dtype, reinterpret_cast<const __half*>(d_suh), rows, rows, in, xhat, stream), "prepare");
    }
    float* products = return_raw ? static_cast<float*>(d_out) : raw;
    for (int64_t s0 = 0; s0 < slots && !rc; s0 += pass_slots) {
        const int64_t n = std::min(pass_slots, slots - s0);
        const int vout = static_cast<int>(n * projections * out);
        QmvArgs a{};
        a.wq = wq; a.xhat = xhat + s0 * projections * in; a.xhat_group_stride = in;
        a.counters = reinterpret_cast<unsigned int*>(ws);
        a.error = reinterpret_cast<unsigned int*>(ws + kCounterBytes - sizeof(unsigned int));
        a.partials = reinterpret_cast<float*>(ws + kCounterBytes);
        a.yhat = products + s0 * projections * out;
        a.groups = 1; a.gcol0[0] = 0; a.gout[0] = vout;
        a.x_dtype = kF16; a.y_dtype = kF16;
        a.in = in; a.out = vout; a.rows = 1;
        a.tiles_n = static_cast<int>(source_tiles);
        a.map_selected = d_selected + s0; a.map_blocks = out / 128; a.map_proj = projections;
        a.map_stride_blocks = static_cast<int>(projection_stride_tiles / 8); a.map_experts = static_cast<int>(experts);
        rc = check(launch_qmv(a, k, cb, true, plan_qmv(in, vout, k, 1), stream), "expert-mapped kernel");
    }
    if (!rc && !return_raw)
        rc = check(launch_finish(raw, 1, rows * out, reinterpret_cast<const __half*>(d_svh), rows, nullptr, rows, out, x_dtype, d_out, stream), "finish");
    if (!rc) rc = check(cudaStreamSynchronize(stream), "expert_mapped");
    cudaFree(wq); cudaFree(xhat); cudaFree(raw); cudaFree(ws);
    return rc;
}

int b200exl3_swiglu_down_input(const float* d_gate_up_raw, const uint16_t* d_gu_svh, const uint16_t* d_down_suh, const uint32_t* d_selected,
                               int experts, int64_t slots, int hidden, uint16_t* d_xhat, b200exl3_stream s) {
    if (experts <= 0 || slots <= 0 || hidden <= 0 || hidden % 128) return fail("invalid SwiGLU glue dimensions");
    if (!d_gate_up_raw || !d_gu_svh || !d_down_suh || !d_selected || !d_xhat) return fail("NULL buffer");
    if (!aligned16(d_gate_up_raw) || !aligned16(d_xhat)) return fail("device pointers must be 16-byte aligned");
    return check(launch_glu_down_input(d_gate_up_raw, reinterpret_cast<const __half*>(d_gu_svh), reinterpret_cast<const __half*>(d_down_suh),
                                       d_selected, experts, slots, hidden, hidden, reinterpret_cast<__half*>(d_xhat), as_stream(s)), "SwiGLU glue");
}

int b200exl3_finish_and_reduce(const float* d_raw, const uint16_t* d_svh, const uint32_t* d_selected, int experts, const void* d_scores,
                               int score_dtype, int64_t rows, int top_k, int out, void* d_y, b200exl3_stream s) {
    if (experts <= 0 || rows <= 0 || top_k <= 0 || out <= 0 || out % 128) return fail("invalid expert reduction dimensions");
    if (score_dtype != kF16 && score_dtype != kF32) return fail("unsupported score dtype %d", score_dtype);
    if (!d_raw || !d_svh || !d_selected || !d_scores || !d_y) return fail("NULL buffer");
    if (!aligned16(d_raw) || !aligned16(d_y)) return fail("device pointers must be 16-byte aligned");
    return check(launch_finish_and_reduce(d_raw, reinterpret_cast<const __half*>(d_svh), d_selected, experts, d_scores, score_dtype, rows, top_k,
                                          out, d_y, as_stream(s)), "expert reduction");
}

/* ---- router ------------------------------------------------------------------------------------------------ */

static int router_check(int64_t rows, int experts, int top_k, int dtype) {
    if (rows <= 0 || experts <= 0 || experts > 1024) return fail("native router accepts positive rows and at most 1024 experts");
    if (top_k <= 0 || top_k > experts) return fail("invalid router top-k");
    if (dtype != kF16 && dtype != kF32) return fail("native router expects FP16 or FP32 values");
    if (rows * static_cast<int64_t>(top_k) > INT32_MAX || rows * static_cast<int64_t>(experts) > INT32_MAX) return fail("router index overflow");
    return 0;
}

int b200exl3_router_topk(const void* d_values, int dtype, int64_t rows, int experts, int top_k, int normalize,
                         uint32_t* d_indices, void* d_scores, b200exl3_stream s) {
    if (router_check(rows, experts, top_k, dtype)) return -1;
    if (!d_values || !d_indices || !d_scores) return fail("NULL buffer");
    return check(launch_router_topk(d_values, dtype, rows, experts, top_k, normalize != 0, false, d_indices, d_scores, nullptr,
                                    as_stream(s)), "router kernel");
}

int b200exl3_router_softmax_topk(const void* d_logits, int dtype, int64_t rows, int experts, int top_k, int normalize,
                                 uint32_t* d_indices, void* d_scores, void* d_probabilities, b200exl3_stream s) {
    if (router_check(rows, experts, top_k, dtype)) return -1;
    if (!d_logits || !d_indices || !d_scores) return fail("NULL buffer");
    return check(launch_router_topk(d_logits, dtype, rows, experts, top_k, normalize != 0, true, d_indices, d_scores,
                                    d_probabilities, as_stream(s)), "router kernel");
}

int b200exl3_router_gate(const void* d_x, int x_dtype, const uint16_t* d_weight_f16, int64_t rows, int in, int experts,
                         uint16_t* d_logits_f16, b200exl3_stream s) {
    if (rows <= 0 || rows > 8 * 65535ll || in <= 0 || in % 2 || experts <= 0) return fail("invalid router gate dimensions");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_weight_f16 || !d_logits_f16) return fail("NULL buffer");
    return check(launch_router_gate(d_x, x_dtype, reinterpret_cast<const __half*>(d_weight_f16), rows, in, experts,
                                    reinterpret_cast<__half*>(d_logits_f16), as_stream(s)), "router gate kernel");
}

/* ---- expert parallelism ---------------------------------------------------------------------------------------------- */

struct b200exl3_ep {
    int rank, world, max_slots, out;
    void* buffers[kTpMaxWorld];
    unsigned int* done;          // [max_slots] use counts + one status word
};

int b200exl3_ep_buffer_bytes(int max_slots, int out, size_t* out_bytes) {
    if (!out_bytes) return fail("NULL argument");
    if (max_slots < 1 || out <= 0 || out % 128) return fail("invalid expert-parallel geometry");
    *out_bytes = static_cast<size_t>(2) * max_slots * (out / 2) * sizeof(unsigned long long);
    return 0;
}

int b200exl3_ipc_alloc(size_t bytes, void** out_buffer, unsigned char* out_handle64) {
    if (!out_buffer || !out_handle64 || bytes == 0) return fail("NULL argument");
    *out_buffer = nullptr;
    void* p = nullptr;
    B200_TRY(cudaMalloc(&p, bytes), "cudaMalloc(exchange buffer)");
    cudaIpcMemHandle_t handle;
    if (check(cudaMemset(p, 0, bytes), "clear exchange buffer") || check(cudaDeviceSynchronize(), "clear exchange buffer") ||
        check(cudaIpcGetMemHandle(&handle, p), "cudaIpcGetMemHandle")) {
        cudaFree(p);
        return -1;
    }
    memcpy(out_handle64, &handle, sizeof handle);
    *out_buffer = p;
    return 0;
}

int b200exl3_ep_create(int rank, int world, int max_slots, int out, void* const* buffers, b200exl3_ep** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world || max_slots < 1 || out <= 0 || out % 128)
        return fail("invalid expert-parallel geometry");
    if (!buffers) return fail("NULL argument");
    for (int r = 0; r < world; ++r)
        if (!buffers[r] || !aligned16(buffers[r])) return fail("exchange buffer of rank %d is NULL or misaligned", r);
    b200exl3_ep* h = new (std::nothrow) b200exl3_ep{};
    if (!h) return fail("out of host memory");
    h->rank = rank; h->world = world; h->max_slots = max_slots; h->out = out;
    for (int r = 0; r < world; ++r) h->buffers[r] = buffers[r];
    const size_t bytes = (static_cast<size_t>(max_slots) + 1) * sizeof(unsigned int);
    if (check(cudaMalloc(&h->done, bytes), "cudaMalloc(use counts)") || check(cudaMemset(h->done, 0, bytes), "clear use counts") ||
        check(cudaDeviceSynchronize(), "ep_create")) {
        cudaFree(h->done);
        delete h;
        return -1;
    }
    *out_handle = h;
    return 0;
}

void b200exl3_ep_free(b200exl3_ep* h) {
    if (!h) return;
    cudaFree(h->done);
    delete h;
}

int b200exl3_ep_status(const b200exl3_ep* h, int* out_status) {
    if (!h || !out_status) return fail("NULL argument");
    unsigned int flag = 0;
    B200_TRY(cudaMemcpy(&flag, h->done + h->max_slots, sizeof flag, cudaMemcpyDeviceToHost), "read status");
    *out_status = static_cast<int>(flag);
    return 0;
}

struct MoeEpLayout {
    size_t local_count, local_slot, local_expert, xgu, ygu, xdown, ydown, partials, total;
    QmvPlan gu_plan, down_plan;
};

static MoeEpLayout moe_ep_layout(const b200exl3_moe* h, int64_t slots) {
    MoeEpLayout l{};
    l.gu_plan = plan_qmv(h->in, static_cast<int>(slots * 2 * h->hidden), h->k, 1);
    l.down_plan = plan_qmv(h->hidden, static_cast<int>(slots * h->in), h->k, 1);
    size_t at = kCounterBytes;
    l.local_count = at; at += 256;
    l.local_slot = at; at += round256(static_cast<size_t>(slots) * sizeof(uint32_t));
    l.local_expert = at; at += round256(static_cast<size_t>(slots) * sizeof(uint32_t));
    l.xgu = at; at += round256(static_cast<size_t>(slots) * 2 * h->in * sizeof(__half));
    l.ygu = at; at += round256(static_cast<size_t>(slots) * 2 * h->hidden * sizeof(float));
    l.xdown = at; at += round256(static_cast<size_t>(slots) * h->hidden * sizeof(__half));
    l.ydown = at; at += round256(static_cast<size_t>(slots) * h->in * sizeof(float));
    l.partials = at;
    at += std::max(qmv_partial_bytes(l.gu_plan, static_cast<int>(slots * 2 * h->hidden), 1),
                   qmv_partial_bytes(l.down_plan, static_cast<int>(slots * h->in), 1));
    l.total = at;
    return l;
}

int b200exl3_moe_ep_workspace_bytes(const b200exl3_moe* h, int64_t rows, size_t* out_bytes) {
    if (!h || !out_bytes) return fail("NULL argument");
    if (rows <= 0) return fail("invalid SwitchGLU input/routes");
    *out_bytes = moe_ep_layout(h, std::min(rows, moe_chunk_rows(h)) * h->top_k).total;
    return 0;
}

int b200exl3_moe_forward_ep(const b200exl3_moe* h, b200exl3_ep* ep, int first_expert, const void* d_x, int x_dtype, int64_t rows,
                            const uint32_t* d_selected, const void* d_scores, int score_dtype, void* d_y, void* ws, size_t ws_bytes,
                            b200exl3_stream s) {
    if (!h || !ep) return fail("NULL handle");
    if (rows <= 0) return fail("invalid SwitchGLU input/routes");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (score_dtype != kF16 && score_dtype != kF32) return fail("unsupported score dtype %d", score_dtype);
    if (!d_x || !d_selected || !d_scores || !d_y) return fail("NULL buffer");
    if (!aligned16(ws) || !aligned16(d_y)) return fail("device pointers must be 16-byte aligned");
    if (first_expert < 0) return fail("invalid first expert");
    if (ep->out != h->in) return fail("the exchange buffers were made for rows of %d values, the block produces %d", ep->out, h->in);
    const int64_t chunk = moe_chunk_rows(h);
    if (std::min(rows, chunk) * h->top_k > ep->max_slots)
        return fail("%lld slots exceed the exchange buffers' %d", static_cast<long long>(std::min(rows, chunk) * h->top_k), ep->max_slots);
    const MoeEpLayout l = moe_ep_layout(h, std::min(rows, chunk) * h->top_k);
    if (!ws || ws_bytes < l.total) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, l.total);
    cudaStream_t stream = as_stream(s);
    char* base = static_cast<char*>(ws);
    const bool exact = (h->flags & B200EXL3_EXACT_WEIGHTS) != 0;
    const size_t x_size = dtype_size(x_dtype), score_size = dtype_size(score_dtype);
    int* local_count = reinterpret_cast<int*>(base + l.local_count);
    uint32_t* local_slot = reinterpret_cast<uint32_t*>(base + l.local_slot);
    uint32_t* local_expert = reinterpret_cast<uint32_t*>(base + l.local_expert);
    __half* xgu = reinterpret_cast<__half*>(base + l.xgu);
    float* ygu = reinterpret_cast<float*>(base + l.ygu);
    __half* xdown = reinterpret_cast<__half*>(base + l.xdown);
    float* ydown = reinterpret_cast<float*>(base + l.ydown);
    EpPeers peers{};
    for (int r = 0; r < ep->world; ++r) peers.inbox[r] = static_cast<unsigned long long*>(ep->buffers[r]);
    peers.done = ep->done; peers.error = ep->done + ep->max_slots;
    peers.rank = ep->rank; peers.world = ep->world; peers.max_slots = ep->max_slots;
    peers.wait_ns = static_cast<unsigned long long>(g_tp_wait_ms.load()) * 1000000ull;
    for (int64_t r0 = 0; r0 < rows; r0 += chunk) {
        const int64_t n = std::min(chunk, rows - r0), slots = n * h->top_k;
        const uint32_t* sel = d_selected + r0 * h->top_k;
        // one activation row per local slot against the columns of its (local) expert; slots past the count are skipped
        auto mapped = [&](const uint32_t* wq, const __half* xhat, int in, int width, int proj, int stride_blocks, float* yhat) {
            const int out = static_cast<int>(slots * proj * width);
            QmvArgs a{};
            a.wq = wq; a.xhat = xhat; a.xhat_group_stride = in;
            a.counters = reinterpret_cast<unsigned int*>(base);
            a.error = reinterpret_cast<unsigned int*>(base + kCounterBytes - sizeof(unsigned int));
            a.partials = reinterpret_cast<float*>(base + l.partials);
            a.yhat = yhat;
            a.groups = 1; a.gcol0[0] = 0; a.gout[0] = out;
            a.x_dtype = kF16; a.y_dtype = kF16;
            a.in = in; a.out = out; a.rows = 1;
            a.tiles_n = h->experts * proj * width / 16;
            a.map_selected = local_expert; a.map_count = local_count;
            a.map_blocks = width / 128; a.map_proj = proj; a.map_stride_blocks = stride_blocks; a.map_experts = h->experts;
            return launch_qmv(a, h->k, h->cb, exact, plan_qmv(in, out, h->k, 1), stream);
        };
        B200_TRY(launch_ep_plan(sel, slots, first_expert, h->experts, local_count, local_slot, local_expert, stream), "expert plan");
        B200_TRY(launch_ep_dispatch(static_cast<const char*>(d_x) + static_cast<size_t>(r0) * h->in * x_size, x_dtype, h->gu_suh, local_count,
                                    local_slot, local_expert, h->top_k, h->in, slots, xgu, stream), "expert dispatch");
        B200_TRY(mapped(h->gu_wq, xgu, h->in, h->hidden, 2, h->experts * (h->hidden / 128), ygu), "expert gate/up kernel");
        B200_TRY(launch_glu_down_input(ygu, h->gu_svh, h->down_suh, local_expert, h->experts, slots, h->hidden, h->hidden, xdown, stream,
                                       local_count), "SwiGLU glue");
        B200_TRY(mapped(h->down_wq, xdown, h->hidden, h->in, 1, 0, ydown), "expert down kernel");
        B200_TRY(launch_ep_publish(ydown, h->down_svh, local_count, local_slot, local_expert, h->in, slots, peers, stream), "expert publish");
        B200_TRY(launch_ep_combine(static_cast<const char*>(d_scores) + static_cast<size_t>(r0) * h->top_k * score_size, score_dtype, n,
                                   h->top_k, h->in, static_cast<char*>(d_y) + static_cast<size_t>(r0) * h->in * score_size, peers, stream),
                 "expert combine");
    }
    return 0;
}

/* ---- decoder-block glue (fp16, batch-1 decode) ----------------------------------------------------------------- */

int b200exl3_embed(const uint16_t* d_table, const int32_t* d_tokens, int64_t rows, int64_t vocab, int hidden, uint16_t* d_out,
                   b200exl3_stream s) {
    if (rows <= 0 || rows > INT32_MAX || vocab <= 0 || hidden <= 0 || hidden % 8) return fail("invalid embedding dimensions");
    if (!d_table || !d_tokens || !d_out) return fail("NULL buffer");
    if (!aligned16(d_table) || !aligned16(d_out)) return fail("device pointers must be 16-byte aligned");
    return check(launch_embed(reinterpret_cast<const __half*>(d_table), d_tokens, rows, vocab, hidden, reinterpret_cast<__half*>(d_out),
                              as_stream(s)), "embedding kernel");
}

int b200exl3_rms_norm(const uint16_t* d_x, const uint16_t* d_residual, const uint16_t* d_weight, int64_t rows, int n, float eps,
                      uint16_t* d_sum, uint16_t* d_y, b200exl3_stream s) {
    if (rows <= 0 || rows > INT32_MAX || n <= 0 || n % 2 || n > 48 * 1024) return fail("invalid RMSNorm dimensions");
    if (!(eps >= 0.0f)) return fail("invalid RMSNorm epsilon");
    if (!d_x || !d_weight || !d_y) return fail("NULL buffer");
    return check(launch_rms_norm(reinterpret_cast<const __half*>(d_x), reinterpret_cast<const __half*>(d_residual),
                                 reinterpret_cast<const __half*>(d_weight), rows, n, eps, reinterpret_cast<__half*>(d_sum),
                                 reinterpret_cast<__half*>(d_y), as_stream(s)), "RMSNorm kernel");
}

int b200exl3_swiglu(const uint16_t* d_gate, const uint16_t* d_up, int64_t n, uint16_t* d_out, b200exl3_stream s) {
    if (n <= 0 || n % 2) return fail("invalid SwiGLU length");
    if (!d_gate || !d_up || !d_out) return fail("NULL buffer");
    return check(launch_swiglu(reinterpret_cast<const __half*>(d_gate), reinterpret_cast<const __half*>(d_up), n,
                               reinterpret_cast<__half*>(d_out), as_stream(s)), "SwiGLU kernel");
}

static int attention_shape(int heads, int kv_heads, int head_dim, int max_ctx) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || max_ctx <= 0) return fail("invalid attention head counts");
    if (head_dim != 128) return fail("decode attention is built for a head dimension of 128, got %d", head_dim);
    return 0;
}

int b200exl3_rope_append(uint16_t* d_q, const uint16_t* d_k, const uint16_t* d_v, int heads, int kv_heads, int head_dim,
                         const int32_t* d_pos, float theta, int max_ctx, uint16_t* d_k_cache, uint16_t* d_v_cache, b200exl3_stream s) {
    if (attention_shape(heads, kv_heads, head_dim, max_ctx)) return -1;
    if (!(theta > 1.0f)) return fail("invalid RoPE base");
    if (!d_q || !d_k || !d_v || !d_pos || !d_k_cache || !d_v_cache) return fail("NULL buffer");
    return check(launch_rope_append(reinterpret_cast<__half*>(d_q), reinterpret_cast<const __half*>(d_k), reinterpret_cast<const __half*>(d_v),
                                    heads, kv_heads, head_dim, d_pos, theta, max_ctx, reinterpret_cast<__half*>(d_k_cache),
                                    reinterpret_cast<__half*>(d_v_cache), as_stream(s)), "RoPE kernel");
}

int b200exl3_attention_workspace_bytes(int heads, int kv_heads, size_t* out_bytes) {
    if (!out_bytes) return fail("NULL argument");
    if (attention_shape(heads, kv_heads, 128, 1)) return -1;
    *out_bytes = round256(attention_workspace_bytes(heads, kv_heads));
    return 0;
}

int b200exl3_attention_decode(const uint16_t* d_q, const uint16_t* d_k_cache, const uint16_t* d_v_cache, int heads, int kv_heads,
                              int head_dim, const int32_t* d_pos, int max_ctx, float scale, uint16_t* d_out, void* ws, size_t ws_bytes,
                              b200exl3_stream s) {
    if (attention_shape(heads, kv_heads, head_dim, max_ctx)) return -1;
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out) return fail("NULL buffer");
    if (!aligned16(d_q) || !aligned16(d_k_cache) || !aligned16(d_v_cache) || !aligned16(ws)) return fail("device pointers must be 16-byte aligned");
    const size_t need = round256(attention_workspace_bytes(heads, kv_heads));
    if (!ws || ws_bytes < need) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, need);
    return check(launch_attention_decode(reinterpret_cast<const __half*>(d_q), reinterpret_cast<const __half*>(d_k_cache),
                                         reinterpret_cast<const __half*>(d_v_cache), heads, kv_heads, head_dim, d_pos, max_ctx, scale,
                                         reinterpret_cast<__half*>(d_out), ws, as_stream(s)), "attention kernel");
}

int b200exl3_head_workspace_bytes(size_t* out_bytes) {
    if (!out_bytes) return fail("NULL argument");
    *out_bytes = round256(static_cast<size_t>(head_candidates()) * (sizeof(float) + sizeof(long long)));
    return 0;
}

int b200exl3_head_argmax(const uint16_t* d_x, const uint16_t* d_weight, int64_t vocab, int hidden, int64_t index_offset,
                         uint16_t* d_logits, float* d_best_value, int64_t* d_best_index, void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (vocab <= 0 || hidden <= 0 || hidden % 8 || hidden > 48 * 1024) return fail("invalid head dimensions");
    if (!d_x || !d_weight || !d_best_value || !d_best_index) return fail("NULL buffer");
    if (!aligned16(d_x) || !aligned16(d_weight) || !aligned16(ws)) return fail("device pointers must be 16-byte aligned");
    size_t need = 0;
    b200exl3_head_workspace_bytes(&need);
    if (!ws || ws_bytes < need) return fail("workspace too small: %zu bytes given, %zu needed", ws_bytes, need);
    const int n = head_candidates();
    long long* cand_index = static_cast<long long*>(ws);
    float* cand_value = reinterpret_cast<float*>(cand_index + n);
    return check(launch_head_argmax(reinterpret_cast<const __half*>(d_x), reinterpret_cast<const __half*>(d_weight), vocab, hidden,
                                    index_offset, reinterpret_cast<__half*>(d_logits), cand_value, cand_index, d_best_value,
                                    reinterpret_cast<long long*>(d_best_index), as_stream(s)), "head kernel");
}

/* ---- tensor parallelism over peer memory ------------------------------------------------------------ */

int b200exl3_tp_buffer_bytes(int world, int max_units, size_t* out_bytes) {
    if (!out_bytes) return fail("NULL argument");
    if (world < 1 || world > kTpMaxWorld || max_units < 1) return fail("invalid tensor-parallel geometry");
    // inbox [2 slots, world sources, max_units, 128 words of {value, sequence number}]
    *out_bytes = static_cast<size_t>(2) * world * max_units * kTpUnitWords * sizeof(uint2);
    return 0;
}

int b200exl3_tp_alloc(int world, int max_units, void** out_buffer, unsigned char* out_handle64) {
    if (!out_buffer || !out_handle64) return fail("NULL argument");
    *out_buffer = nullptr;
    size_t bytes = 0;
    if (b200exl3_tp_buffer_bytes(world, max_units, &bytes)) return -1;
    void* p = nullptr;
    B200_TRY(cudaMalloc(&p, bytes), "cudaMalloc(exchange buffer)");
    cudaIpcMemHandle_t handle;
    if (check(cudaMemset(p, 0, bytes), "clear exchange buffer") || check(cudaDeviceSynchronize(), "clear exchange buffer") ||
        check(cudaIpcGetMemHandle(&handle, p), "cudaIpcGetMemHandle")) {
        cudaFree(p);
        return -1;
    }
    static_assert(sizeof(handle) == 64, "IPC handle size");
    memcpy(out_handle64, &handle, sizeof handle);
    *out_buffer = p;
    return 0;
}

int b200exl3_tp_open(const unsigned char* handle64, void** out_peer) {
    if (!handle64 || !out_peer) return fail("NULL argument");
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle64, sizeof handle);
    return check(cudaIpcOpenMemHandle(out_peer, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int b200exl3_tp_close(void* peer) { return peer ? check(cudaIpcCloseMemHandle(peer), "cudaIpcCloseMemHandle") : 0; }

int b200exl3_tp_create(int rank, int world, int max_units, void* const* buffers, b200exl3_tp** out_handle) {
    if (!out_handle) return fail("out pointer is NULL");
    *out_handle = nullptr;
    if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world || max_units < 1)
        return fail("invalid tensor-parallel geometry");
    if (!buffers) return fail("NULL argument");
    for (int r = 0; r < world; ++r)
        if (!buffers[r] || !aligned16(buffers[r])) return fail("exchange buffer of rank %d is NULL or misaligned", r);
    b200exl3_tp* h = new (std::nothrow) b200exl3_tp{};
    if (!h) return fail("out of host memory");
    h->rank = rank; h->world = world; h->max_units = max_units;
    for (int r = 0; r < world; ++r) h->buffers[r] = buffers[r];
    const size_t bytes = (static_cast<size_t>(max_units) + 1) * sizeof(unsigned int);
    if (check(cudaMalloc(&h->done, bytes), "cudaMalloc(use counts)") || check(cudaMemset(h->done, 0, bytes), "clear use counts") ||
        check(cudaDeviceSynchronize(), "tp_create")) {
        cudaFree(h->done);
        delete h;
        return -1;
    }
    *out_handle = h;
    return 0;
}

void b200exl3_tp_free(b200exl3_tp* h) {
    if (!h) return;
    cudaFree(h->done);
    delete h;
}

int b200exl3_tp_status(const b200exl3_tp* h, int* out_status) {
    if (!h || !out_status) return fail("NULL argument");
    unsigned int flag = 0;
    B200_TRY(cudaMemcpy(&flag, h->done + h->max_units, sizeof flag, cudaMemcpyDeviceToHost), "read status");
    *out_status = static_cast<int>(flag);
    return 0;
}

int b200exl3_tp_reset(b200exl3_tp* h) {
    if (!h) return fail("NULL handle");
    B200_TRY(cudaDeviceSynchronize(), "tp_reset");
    size_t bytes = 0;
    if (b200exl3_tp_buffer_bytes(h->world, h->max_units, &bytes)) return -1;
    B200_TRY(cudaMemset(h->buffers[h->rank], 0, bytes), "clear exchange buffer");
    B200_TRY(cudaMemset(h->done, 0, (static_cast<size_t>(h->max_units) + 1) * sizeof(unsigned int)), "clear use counts");
    return check(cudaDeviceSynchronize(), "tp_reset");
}

int b200exl3_linear_forward_tp(const b200exl3_linear* h, b200exl3_tp* tp, const void* d_x, int x_dtype, int64_t rows, void* d_y,
                              void* ws, size_t ws_bytes, b200exl3_stream s) {
    if (!h || !tp) return fail("NULL handle");
    if (!dtype_is_float(x_dtype)) return fail("unsupported input dtype %d", x_dtype);
    if (!d_x || !d_y) return fail("NULL buffer");
    if (rows > 0 && rows * (h->c.out / 128) > tp->max_units)
        return fail("%lld units exceed the exchange buffers' %d", static_cast<long long>(rows * (h->c.out / 128)), tp->max_units);
    void* ys[1] = {d_y};
    return forward_common(h->c, d_x, x_dtype, nullptr, rows, ys, nullptr, ws, ws_bytes, as_stream(s), tp);
}

int b200exl3_linear_finish_tp(const b200exl3_linear* h, b200exl3_tp* tp, const float* d_yhat, int64_t rows, int y_dtype,
                              void* d_y, b200exl3_stream s) {
    if (!h || !tp) return fail("NULL handle");
    if (rows <= 0) return fail("EXL3 linear input cannot be empty");
    if (!dtype_is_float(y_dtype)) return fail("unsupported output dtype %d", y_dtype);
    if (!d_yhat || !d_y) return fail("NULL buffer");
    if (!aligned16(d_yhat)) return fail("device pointers must be 16-byte aligned");
    const int64_t units = rows * (h->c.out / 128);
    if (units > tp->max_units) return fail("%lld units exceed the exchange buffers' %d", static_cast<long long>(units), tp->max_units);
    TpArgs a{};
    a.yhat = d_yhat;
    a.peers = tp_peers(tp);
    a.svh = h->c.svh; a.bias = h->c.bias; a.y = d_y;
    a.rows = static_cast<int>(rows); a.out = h->c.out; a.y_dtype = y_dtype;
    return check(launch_tp_finish(a, as_stream(s)), "tensor-parallel finish kernel");
}


}  // extern "C"

static TpPeers tp_peers(const b200exl3_tp* tp) {
    TpPeers t{};
    for (int r = 0; r < tp->world; ++r) t.inbox[r] = static_cast<uint2*>(tp->buffers[r]);
    t.done = tp->done;
    t.error = tp->done + tp->max_units;
    t.rank = tp->rank; t.world = tp->world; t.max_units = tp->max_units;
    t.wait_ns = static_cast<unsigned long long>(g_tp_wait_ms.load()) * 1000000ull;
    return t;
}
