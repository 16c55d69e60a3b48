// Host side of the backend: the C++ mirror of the reference's MetalBackend for the
// matmul path (src/backend/metal/mod.rs:163-176 state, :185 new, :445-494 upload/alloc,
// :496-687 matmul dispatch, :979-1002 readback/sync, :264-272 GPU-time accounting), and
// the extern "C" surface declared in include/llmrs_cuda.h.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <functional>
#include <string>
#include <vector>

#include "../../include/llmrs_cuda.h"
#include "gguf.h"
#include "kernels.h"

using namespace llmrs;

namespace {
thread_local std::string g_create_error;
}

// One device, one stream, event-based GPU time: the state MetalBackend keeps in
// its device/queue/command-buffer fields.
struct llmrs_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
    bool span_open = false;      // work enqueued since the last synchronisation point
    double gpu_secs = 0.0;
    uint64_t launches = 0;
    int sm_count = 0;
    int gemv_max_m = 4;              // M <= this: exact decode kernel (1e-4 class); above: tensor-core GEMM
    bool cost_rule = true;           // up to 64 tokens the decode kernel also runs where it is the cheaper one;
                                     // an explicit LLMRS_GEMV_MAX_M makes the boundary hard
    bool exact = true;               // up to 64 tokens the tensor-core path runs the exact-integer-operand kernel
                                     // (gemm_exact.cu); LLMRS_TC_EXACT=0: the older two-term kernel of gemm_tc.cu
    bool two_term = true;            // tensor-core GEMM up to 64 tokens carries hi + lo f16 terms (1e-4 class);
                                     // LLMRS_TC_TWO_TERM=0: one term (2e-3 class, about half the time)
    void *scratch = nullptr;         // f16 copy of the activations for the tensor-core path
    size_t scratch_bytes = 0;
    // Several weights multiplied with one input inside one call (q/k/v, gate/up) share the conversion of
    // the activations the small-batch tensor-core kernel needs: acts_share is set for the length of
    // such a call, acts_x/K/M/dtype say what the matmul scratch holds.
    bool acts_share = false, acts_have = false;
    const void *acts_x = nullptr;
    uint32_t acts_K = 0, acts_M = 0, acts_dtype = 0;
    bool pdl = true;                 // decode kernels overlap their prologue with the previous kernel's tail (LLMRS_NO_PDL=1: off)
    int gemm_split = -1;             // LLMRS_GEMM_SPLIT at creation: 0 never, 1 always, otherwise the estimate decides
    const llmrs_buf *residual = nullptr;   // set by matmul_add around its call of matmul
    void *norm_tmp = nullptr;              // normalised activations where the norm is not fused into the matmul
    size_t norm_tmp_bytes = 0;
    const float *norm_w = nullptr;         // set by the rms_norm_matmul calls around theirs
    float norm_eps = 0.0f;
    const float *conv_norm_w = nullptr;    // likewise, above four tokens: the norm rides in the small-batch kernel's conversion
    float conv_norm_eps = 0.0f;
    float *att_ws = nullptr;         // partial results of attention over split sequences
    size_t att_ws_bytes = 0;
    uint32_t *argmax_out = nullptr;  // device word argmax writes its result to
    uint32_t *tokens = nullptr;      // device copy of embed's token ids
    // GGUF uploads: two pinned host pieces, two device pieces (raw Q6_K before its re-layout), one event each
    uint8_t *stage_host[2] = {nullptr, nullptr};
    uint8_t *stage_dev[2] = {nullptr, nullptr};
    cudaEvent_t stage_done[2] = {nullptr, nullptr};
    size_t upload_piece = 32u << 20;  // LLMRS_UPLOAD_PIECE_MB (1..1024)
    int upload_readers = 8;           // LLMRS_UPLOAD_READERS (1..64)
    size_t tokens_cap = 0;
    void *split_ws = nullptr;        // workspace of the tensor-core path's split of the last wave (zero between launches)
    uint32_t *dev_error = nullptr;   // device word: first KernelError reported by a kernel; next word: CTA counter
    uint32_t mbar_polls = DEFAULT_MBAR_POLLS;      // LLMRS_WAIT_POLLS at creation shortens both limits (tests of the
    uint32_t gather_polls = DEFAULT_GATHER_POLLS;  // give-up path); see ErrSink
    // Internal buffers that were outgrown.  They are kept until the context is destroyed, because a CUDA
    // graph captured earlier has their addresses baked in and may still be replayed.
    std::vector<void *> retired;
    // LLMRS_PERF=1: one event pair per operation, a table per kernel at every sync (metal/mod.rs:323-400).
    bool perf = false;
    double peak_gbs = 8000.0, peak_tflops = 2250.0;   // LLMRS_PEAK_HBM_GBS / LLMRS_PEAK_TFLOPS override the nominal figures
    struct PerfOp { std::string name; double bytes, flops; cudaEvent_t a, b; };
    std::vector<PerfOp> perf_ops;
    std::vector<cudaEvent_t> perf_free;
    std::string perf_last;           // the table of the last sync
    std::string error;

    ErrSink sink() const { return ErrSink(dev_error, mbar_polls, gather_polls); }

    int fail(int code, const char *fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        error = buf;
        return code;
    }
    int cuda_fail(cudaError_t e, const char *what) {
        return fail(LLMRS_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    // After a synchronisation point: did a kernel abandon one of its bounded waits?
    int check_kernel_error(const char *what) {
        uint32_t code = 0;
        cudaError_t e = cudaMemcpy(&code, dev_error, sizeof code, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return cuda_fail(e, what);
        if (code == 0) return LLMRS_OK;
        cudaMemset(dev_error, 0, 2 * sizeof code);
        if (split_ws) cudaMemset(split_ws, 0, gemm_split_counter_bytes());     // an abandoned launch may have left counters behind
        if (code == 7) return fail(LLMRS_ERR_ARG, "%s: embed was given a token id beyond the table", what);
        return fail(LLMRS_ERR_KERNEL, "%s: a kernel gave up a bounded wait (code %u); results are incomplete", what, code);
    }
    // Grows one of the context's internal buffers.  Never while the stream is being captured (an
    // allocation cannot be part of a graph); the outgrown buffer is parked in `retired`, not freed, so
    // that graphs captured while it was current stay valid.  Sizes at least double, which bounds what
    // the parked buffers can add up to.
    cudaError_t grow(void **buf, size_t *have, size_t need) {
        if (need <= *have) return cudaSuccess;
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &st);
        if (st != cudaStreamCaptureStatusNone) return cudaErrorStreamCaptureUnsupported;
        const size_t want = std::max(need, 2 * *have);
        void *fresh = nullptr;
        acts_have = false;                               // whatever the old buffer held stays behind
        cudaError_t e = cudaMalloc(&fresh, want);
        if (e != cudaSuccess && want > need) {
            (void)cudaGetLastError();
            e = cudaMalloc(&fresh, need);
            if (e == cudaSuccess) { if (*buf) retired.push_back(*buf); *buf = fresh; *have = need; return e; }
        }
        if (e != cudaSuccess) return e;
        if (*buf) {
            try { retired.push_back(*buf); } catch (...) { cudaFree(fresh); return cudaErrorMemoryAllocation; }
        }
        *buf = fresh;
        *have = want;
        return cudaSuccess;
    }
    cudaError_t reserve_scratch(size_t bytes) { return grow(&scratch, &scratch_bytes, bytes); }
    // Called before enqueueing: opens the timed span the way the reference opens a
    // command buffer lazily on the first dispatch (metal/mod.rs:287-319).
    cudaError_t begin_work() {
        if (span_open) return cudaSuccess;
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &st);
        if (st != cudaStreamCaptureStatusNone) return cudaSuccess;   // no events inside a graph capture
        cudaError_t e = cudaEventRecord(ev_begin, stream);
        if (e == cudaSuccess) span_open = true;
        return e;
    }
    // Synchronisation point: closes the span and adds its device time (metal/mod.rs:264-272).
    cudaError_t finish_work() {
        if (span_open) {
            cudaError_t e = cudaEventRecord(ev_end, stream);
            if (e != cudaSuccess) return e;
            e = cudaEventSynchronize(ev_end);
            if (e != cudaSuccess) return e;
            float ms = 0.f;
            e = cudaEventElapsedTime(&ms, ev_begin, ev_end);
            if (e != cudaSuccess) return e;
            gpu_secs += (double)ms * 1e-3;
            span_open = false;
            return cudaSuccess;
        }
        return cudaStreamSynchronize(stream);
    }
};

namespace {

size_t dense_elem_bytes(uint32_t dtype) {
    return dtype == LLMRS_F32 ? 4 : dtype == LLMRS_BF16 ? 2 : 0;
}

// Bytes of the tensor as stored in a GGUF file (DType::storage_size, src/tensor/mod.rs:89-93).
bool storage_size(uint32_t dtype, uint64_t n_elems, size_t *out) {
    if (dtype == LLMRS_Q4K || dtype == LLMRS_Q6K) {
        if (n_elems % QK_K) return false;
        *out = (size_t)(n_elems / QK_K) * (dtype == LLMRS_Q4K ? Q4K_BLOCK_BYTES : Q6K_BLOCK_BYTES);
        return true;
    }
    if (dtype == LLMRS_Q8_0 || dtype == LLMRS_Q4_0) {
        if (n_elems % 32) return false;
        *out = (size_t)(n_elems / 32) * (dtype == LLMRS_Q8_0 ? 34 : 18);
        return true;
    }
    size_t eb = dtype == LLMRS_I32 ? 4 : dtype == LLMRS_F16 ? 2 : dense_elem_bytes(dtype);
    if (!eb) return false;
    *out = (size_t)n_elems * eb;
    return true;
}

bool is_kquant(uint32_t dtype) { return dtype == LLMRS_Q4K || dtype == LLMRS_Q6K; }
bool is_block32(uint32_t dtype) { return dtype == LLMRS_Q8_0 || dtype == LLMRS_Q4_0; }
// Weight types beside the K-quants that matmul takes: dense F32 / F16 / BF16 and Q8_0 / Q4_0.
bool is_other_weight(uint32_t dtype) {
    return dtype == LLMRS_F32 || dtype == LLMRS_F16 || dtype == LLMRS_BF16 || is_block32(dtype);
}
uint32_t weight_layout(uint32_t dtype) {
    return dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : is_block32(dtype) ? LLMRS_LAYOUT_BLOCK32_PLANES : LLMRS_LAYOUT_RAW;
}

bool shape_dims(const uint64_t *shape, int ndims, uint32_t *d0, uint32_t *d1) {
    if (!shape || ndims < 1 || ndims > 2) return false;
    if (shape[0] == 0 || shape[0] > 0x7FFFFFFFull) return false;
    if (ndims == 2 && (shape[1] == 0 || shape[1] > 0x7FFFFFFFull)) return false;
    *d0 = (uint32_t)shape[0];
    *d1 = ndims > 1 ? (uint32_t)shape[1] : 0;   // 1-D buffers carry dim1 = 0 (metal/mod.rs:460,493)
    return true;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// LLMRS_PERF=1: brackets one operation with an event pair.  The reference's LLM_PERF does the same with
// GPU timestamps per dispatch and prints a per-kernel table with bytes/s and flop/s against the
// machine's speed of light (metal/mod.rs:150-153,323-400,996-1002).  Nothing is recorded while the
// stream is being captured.  `bytes` and `flops` are the algorithmic figures of the call.
struct PerfScope {
    llmrs_ctx *ctx;
    cudaEvent_t a = nullptr, b = nullptr;
    const char *name;
    double bytes, flops;
    PerfScope(llmrs_ctx *c, const char *n, double by, double fl) : ctx(c), name(n), bytes(by), flops(fl) {
        if (!ctx->perf) return;
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(ctx->stream, &st);
        if (st != cudaStreamCaptureStatusNone) return;
        for (cudaEvent_t *ev : {&a, &b}) {
            if (!ctx->perf_free.empty()) { *ev = ctx->perf_free.back(); ctx->perf_free.pop_back(); }
            else if (cudaEventCreate(ev) != cudaSuccess) { *ev = nullptr; }
        }
        if (!a || !b || cudaEventRecord(a, ctx->stream) != cudaSuccess) {
            if (a) ctx->perf_free.push_back(a);
            if (b) ctx->perf_free.push_back(b);
            a = b = nullptr;
        }
    }
    ~PerfScope() {
        if (!a) return;
        cudaEventRecord(b, ctx->stream);
        try { ctx->perf_ops.push_back({name, bytes, flops, a, b}); } catch (...) { cudaEventDestroy(a); cudaEventDestroy(b); }
    }
};

const char *dtype_name(uint32_t dt) {
    switch (dt) {
        case LLMRS_F32: return "f32";
        case LLMRS_Q4K: return "q4_k";
        case LLMRS_Q6K: return "q6_k";
        case LLMRS_BF16: return "bf16";
        case LLMRS_F16: return "f16";
        case LLMRS_Q8_0: return "q8_0";
        case LLMRS_Q4_0: return "q4_0";
        case LLMRS_I32: return "i32";
        default: return "?";
    }
}

// Algorithmic bytes of a matmul: the weight as stored on disk, the activations in, the results out.
double matmul_bytes(const llmrs_buf *w, const llmrs_buf *in, const llmrs_buf *out) {
    size_t wb = 0;
    storage_size(w->dtype, (uint64_t)w->dim0 * (w->dim1 ? w->dim1 : 1), &wb);
    return (double)wb + (double)in->dim0 * (in->dim1 ? in->dim1 : 1) * dense_elem_bytes(in->dtype) +
           (double)out->dim0 * (out->dim1 ? out->dim1 : 1) * dense_elem_bytes(out->dtype);
}
double matmul_flops(const llmrs_buf *w, const llmrs_buf *in) {
    return 2.0 * w->dim0 * (w->dim1 ? w->dim1 : 1) * (in->dim1 ? in->dim1 : 1);
}

// After a synchronisation point: the operations recorded since the last one, one line per kind, in
// first-use order; printed to stderr and kept for llmrs_cuda_perf_table.
void perf_flush(llmrs_ctx *ctx) {
    if (ctx->perf_ops.empty()) return;
    struct Row { std::string name; int calls; double ms, bytes, flops; };
    std::vector<Row> rows;
    for (auto &op : ctx->perf_ops) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, op.a, op.b) != cudaSuccess) { (void)cudaGetLastError(); ms = 0.f; }
        ctx->perf_free.push_back(op.a);
        ctx->perf_free.push_back(op.b);
        auto it = std::find_if(rows.begin(), rows.end(), [&](const Row &r) { return r.name == op.name; });
        if (it == rows.end()) rows.push_back({op.name, 1, ms, op.bytes, op.flops});
        else { it->calls++; it->ms += ms; it->bytes += op.bytes; it->flops += op.flops; }
    }
    ctx->perf_ops.clear();
    double total = 0.0;
    for (auto &r : rows) total += r.ms;
    char line[256];
    std::string t;
    snprintf(line, sizeof line, "%-34s %6s %10s %6s %9s %6s %9s %6s\n", "kernel", "calls", "us", "share", "GB/s", "of pk",
             "TFLOP/s", "of pk");
    t += line;
    for (auto &r : rows) {
        const double secs = r.ms * 1e-3, gbs = secs > 0 ? r.bytes / secs * 1e-9 : 0.0, tf = secs > 0 ? r.flops / secs * 1e-12 : 0.0;
        snprintf(line, sizeof line, "%-34s %6d %10.1f %5.1f%% %9.1f %5.1f%% %9.2f %5.1f%%\n", r.name.c_str(), r.calls, r.ms * 1e3,
                 total > 0 ? 100.0 * r.ms / total : 0.0, gbs, 100.0 * gbs / ctx->peak_gbs, tf, 100.0 * tf / ctx->peak_tflops);
        t += line;
    }
    snprintf(line, sizeof line, "(peaks: %.0f GB/s, %.0f TFLOP/s; times are per operation, events around each)\n", ctx->peak_gbs,
             ctx->peak_tflops);
    t += line;
    fputs(t.c_str(), stderr);
    ctx->perf_last = t;
}

}  // namespace

extern "C" {

int llmrs_cuda_create(int device, void *stream, llmrs_ctx **out) {
    if (!out) { g_create_error = "llmrs_cuda_create: out is null"; return LLMRS_ERR_ARG; }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        g_create_error = std::string("no CUDA device: ") + cudaGetErrorString(e);
        return LLMRS_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) { g_create_error = "device ordinal out of range"; return LLMRS_ERR_ARG; }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { g_create_error = cudaGetErrorString(e); return LLMRS_ERR_CUDA; }
    if (prop.major != 10) {
        char buf[160];
        snprintf(buf, sizeof buf, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                 prop.major, prop.minor);
        g_create_error = buf;
        return LLMRS_ERR_NO_DEVICE;
    }
    llmrs_ctx *ctx = new (std::nothrow) llmrs_ctx();
    if (!ctx) { g_create_error = "out of host memory"; return LLMRS_ERR_ARG; }
    ctx->device = device;
    DeviceGuard guard(device);
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { g_create_error = cudaGetErrorString(e); delete ctx; return LLMRS_ERR_CUDA; }
        ctx->own_stream = true;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (const char *env = getenv("LLMRS_GEMV_MAX_M")) {
        int v = atoi(env);
        if (v >= 0) { ctx->gemv_max_m = v; ctx->cost_rule = false; }
    }
    if (const char *env = getenv("LLMRS_NO_PDL")) ctx->pdl = atoi(env) == 0;
    if (const char *env = getenv("LLMRS_TC_TWO_TERM")) ctx->two_term = atoi(env) != 0;
    if (const char *env = getenv("LLMRS_TC_EXACT")) ctx->exact = atoi(env) != 0;
    if (const char *env = getenv("LLMRS_UPLOAD_PIECE_MB")) {
        const int v = atoi(env);
        if (v >= 1 && v <= 1024) ctx->upload_piece = (size_t)v << 20;
    }
    if (const char *env = getenv("LLMRS_UPLOAD_READERS")) {
        const int v = atoi(env);
        if (v >= 1 && v <= 64) ctx->upload_readers = v;
    }
    if (const char *env = getenv("LLMRS_GEMM_SPLIT")) ctx->gemm_split = atoi(env) ? 1 : 0;
    if (const char *env = getenv("LLMRS_WAIT_POLLS")) {
        const long v = atol(env);
        if (v >= 16 && v <= (1L << 30)) ctx->mbar_polls = ctx->gather_polls = (uint32_t)v;
    }
    if (const char *env = getenv("LLMRS_PERF")) ctx->perf = atoi(env) != 0;
    if (const char *env = getenv("LLMRS_PEAK_HBM_GBS")) { const double v = atof(env); if (v > 0) ctx->peak_gbs = v; }
    if (const char *env = getenv("LLMRS_PEAK_TFLOPS")) { const double v = atof(env); if (v > 0) ctx->peak_tflops = v; }
    e = cudaEventCreate(&ctx->ev_begin);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_end);
    if (e == cudaSuccess) e = cudaMalloc((void **)&ctx->dev_error, 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_error, 0, 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc((void **)&ctx->argmax_out, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->split_ws, gemm_split_workspace_bytes(ctx->sm_count));
    if (e == cudaSuccess) e = cudaMemset(ctx->split_ws, 0, gemm_split_counter_bytes());
    if (e != cudaSuccess) {
        g_create_error = cudaGetErrorString(e);
        llmrs_cuda_destroy(ctx);
        return LLMRS_ERR_CUDA;
    }
    *out = ctx;
    return LLMRS_OK;
}

int llmrs_cuda_destroy(llmrs_ctx *ctx) {
    if (!ctx) return LLMRS_OK;
    DeviceGuard guard(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->ev_begin) cudaEventDestroy(ctx->ev_begin);
    if (ctx->ev_end) cudaEventDestroy(ctx->ev_end);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->dev_error) cudaFree(ctx->dev_error);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->split_ws) cudaFree(ctx->split_ws);
    if (ctx->tokens) cudaFree(ctx->tokens);
    if (ctx->argmax_out) cudaFree(ctx->argmax_out);
    if (ctx->att_ws) cudaFree(ctx->att_ws);
    if (ctx->norm_tmp) cudaFree(ctx->norm_tmp);
    for (void *old : ctx->retired) cudaFree(old);
    for (auto &op : ctx->perf_ops) { cudaEventDestroy(op.a); cudaEventDestroy(op.b); }
    for (cudaEvent_t ev : ctx->perf_free) cudaEventDestroy(ev);
    for (int i = 0; i < 2; i++) {
        if (ctx->stage_host[i]) cudaFreeHost(ctx->stage_host[i]);
        if (ctx->stage_dev[i]) cudaFree(ctx->stage_dev[i]);
        if (ctx->stage_done[i]) cudaEventDestroy(ctx->stage_done[i]);
    }
    delete ctx;
    return LLMRS_OK;
}

const char *llmrs_cuda_last_error(llmrs_ctx *ctx) {
    return ctx ? ctx->error.c_str() : g_create_error.c_str();
}

int llmrs_cuda_alloc(llmrs_ctx *ctx, uint32_t dtype, const uint64_t *shape, int ndims, llmrs_buf *out) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out) return ctx->fail(LLMRS_ERR_ARG, "alloc: out is null");
    uint32_t d0, d1;
    if (!shape_dims(shape, ndims, &d0, &d1)) return ctx->fail(LLMRS_ERR_SHAPE, "alloc: bad shape");
    size_t eb = dtype == LLMRS_I32 ? 4 : dense_elem_bytes(dtype);
    if (!eb) return ctx->fail(LLMRS_ERR_DTYPE, "alloc: dtype %u is not F32/BF16/I32", dtype);
    size_t nbytes = (size_t)d0 * (d1 ? d1 : 1) * eb;
    DeviceGuard guard(ctx->device);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, nbytes);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "alloc: cudaMalloc");
    *out = llmrs_buf{p, nbytes, dtype, d0, d1, LLMRS_LAYOUT_RAW, 1u, (uint32_t)ctx->device};
    return LLMRS_OK;
}

int llmrs_cuda_wrap(llmrs_ctx *ctx, void *dptr, uint32_t dtype, const uint64_t *shape, int ndims, llmrs_buf *out) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !dptr) return ctx->fail(LLMRS_ERR_ARG, "wrap: null pointer");
    uint32_t d0, d1;
    if (!shape_dims(shape, ndims, &d0, &d1)) return ctx->fail(LLMRS_ERR_SHAPE, "wrap: bad shape");
    size_t eb = dtype == LLMRS_I32 ? 4 : dense_elem_bytes(dtype);
    if (!eb) return ctx->fail(LLMRS_ERR_DTYPE, "wrap: dtype %u is not F32/BF16/I32", dtype);
    if ((uintptr_t)dptr % 16) return ctx->fail(LLMRS_ERR_ARG, "wrap: pointer must be 16-byte aligned");
    *out = llmrs_buf{dptr, (size_t)d0 * (d1 ? d1 : 1) * eb, dtype, d0, d1, LLMRS_LAYOUT_RAW, 0u,
                     (uint32_t)ctx->device};
    return LLMRS_OK;
}

int llmrs_cuda_free(llmrs_ctx *ctx, llmrs_buf *buf) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!buf) return LLMRS_OK;
    if (buf->owned && buf->dptr) {
        if (buf->device != (uint32_t)ctx->device) return ctx->fail(LLMRS_ERR_ARG, "free: buffer of another device");
        DeviceGuard guard(ctx->device);
        cudaError_t e = cudaStreamSynchronize(ctx->stream);   // nothing in flight may still read it
        if (e == cudaSuccess) e = cudaFree(buf->dptr);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "free");
    }
    memset(buf, 0, sizeof *buf);
    return LLMRS_OK;
}

int llmrs_cuda_upload_tensor(llmrs_ctx *ctx, uint32_t dtype, const uint64_t *shape, int ndims,
                             const void *host, size_t nbytes, llmrs_buf *out) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !host) return ctx->fail(LLMRS_ERR_ARG, "upload_tensor: null pointer");
    uint32_t d0, d1;
    if (!shape_dims(shape, ndims, &d0, &d1)) return ctx->fail(LLMRS_ERR_SHAPE, "upload_tensor: bad shape");
    const uint64_t n_elems = (uint64_t)d0 * (d1 ? d1 : 1);
    size_t want = 0;
    const bool quant = dtype == LLMRS_Q4K || dtype == LLMRS_Q6K;
    if (quant && d0 % QK_K)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_tensor: in_features %u is not a multiple of 256", d0);
    if (is_block32(dtype) && d0 % 32)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_tensor: in_features %u is not a multiple of 32", d0);
    if (!storage_size(dtype, n_elems, &want))
        return ctx->fail(LLMRS_ERR_DTYPE, "upload_tensor: dtype %u is not supported (F32, F16, BF16, I32, Q4_0, Q8_0, Q4_K, Q6_K)", dtype);
    if (want != nbytes)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_tensor: %zu bytes given, shape needs %zu", nbytes, want);
    DeviceGuard guard(ctx->device);
    const int K = (int)d0, N = (int)(d1 ? d1 : 1);
    const size_t dev_bytes = quant ? weight_device_bytes((int)dtype, K, N) : is_block32(dtype) ? block32_device_bytes((int)dtype, K, N) : nbytes;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, dev_bytes);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "upload_tensor: cudaMalloc");
    const uint32_t layout = weight_layout(dtype);
    if (layout != LLMRS_LAYOUT_RAW) {
        // Re-layout on the device: raw bytes into a staging buffer, one kernel, staging freed.
        void *stage = nullptr;
        e = cudaMalloc(&stage, nbytes);
        if (e == cudaSuccess) e = cudaMemcpyAsync(stage, host, nbytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) {
            if (dtype == LLMRS_Q6K) e = launch_q6k_repack((const uint8_t *)stage, (uint8_t *)p, K, N, ctx->stream);
            else e = launch_block32_repack((int)dtype, (const uint8_t *)stage, (uint8_t *)p,
                                           (uint8_t *)p + (size_t)N * block32_quant_stride((int)dtype, K), K, N, ctx->stream);
            ctx->launches++;
        }
        cudaError_t e2 = cudaStreamSynchronize(ctx->stream);
        if (stage) cudaFree(stage);
        if (e == cudaSuccess) e = e2;
    } else {
        e = cudaMemcpyAsync(p, host, nbytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);   // host memory is not retained
    }
    if (e != cudaSuccess) {
        cudaFree(p);
        return ctx->cuda_fail(e, "upload_tensor: copy");
    }
    *out = llmrs_buf{p, dev_bytes, dtype, d0, d1, layout, 1u, (uint32_t)ctx->device};
    return LLMRS_OK;
}

// Piece size of a streamed upload (default 32 MiB): large enough that eight readers each get the 4 MiB
// requests the reference issues (src/gguf/mod.rs:311-312) and that a copy runs at the link's rate, small
// enough that two pinned pieces cost little host memory.

int llmrs_cuda_upload_gguf_tensor(llmrs_ctx *ctx, const llmrs_gguf *gf, const char *name, llmrs_buf *out) {
    return llmrs_cuda_upload_gguf_tensor_rows(ctx, gf, name, 0, UINT64_MAX, out);
}

int llmrs_cuda_upload_gguf_tensor_rows(llmrs_ctx *ctx, const llmrs_gguf *gf, const char *name, uint64_t first_row,
                                       uint64_t n_rows, llmrs_buf *out) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!gf || !name || !out) return ctx->fail(LLMRS_ERR_ARG, "upload_gguf_tensor: null pointer");
    const llmrs::GgufFile *g = reinterpret_cast<const llmrs::GgufFile *>(gf);
    const llmrs::GgufTensor *t = g->find_tensor(name);
    if (!t) return ctx->fail(LLMRS_ERR_NOT_FOUND, "tensor not found: %s", name);
    int ndims = (int)t->n_dims;
    while (ndims > 2 && t->shape[ndims - 1] == 1) ndims--;          // [K, N, 1, 1] is the 2-D tensor [K, N]
    uint32_t d0, d1;
    if (!shape_dims(t->shape, ndims, &d0, &d1))
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s has a shape this backend does not hold (1-D or 2-D)", name);
    const uint32_t dtype = t->dtype;
    const bool quant = dtype == LLMRS_Q4K || dtype == LLMRS_Q6K;
    if (quant && d0 % QK_K)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s: in_features %u is not a multiple of 256", name, d0);
    if (is_block32(dtype) && d0 % 32)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s: in_features %u is not a multiple of 32", name, d0);
    size_t whole = 0;
    if (!storage_size(dtype, (uint64_t)d0 * (d1 ? d1 : 1), &whole))
        return ctx->fail(LLMRS_ERR_DTYPE, "upload_gguf_tensor: %s: dtype %u is not supported (F32, F16, BF16, I32, Q4_0, Q8_0, Q4_K, Q6_K)", name, dtype);
    if (whole != t->nbytes) return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s: directory and shape disagree on the size", name);
    // a slice of the rows: rows [first_row, first_row + n_rows) of the outer dimension
    const uint64_t all_rows = d1 ? d1 : 1;
    if (n_rows == UINT64_MAX && first_row == 0) n_rows = all_rows;
    if (n_rows == 0 || first_row >= all_rows || n_rows > all_rows - first_row)
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s: rows [%llu, +%llu) of %llu", name, (unsigned long long)first_row,
                         (unsigned long long)n_rows, (unsigned long long)all_rows);
    if (n_rows != all_rows && !d1) return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s is 1-D: it has no rows to slice", name);
    const size_t src_row_bytes = whole / (size_t)all_rows;
    const size_t want = src_row_bytes * (size_t)n_rows;
    if (d1) d1 = (uint32_t)n_rows;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        if (!ctx->stage_host[i]) e = cudaHostAlloc((void **)&ctx->stage_host[i], ctx->upload_piece, cudaHostAllocDefault);
        if (e == cudaSuccess && !ctx->stage_done[i]) e = cudaEventCreateWithFlags(&ctx->stage_done[i], cudaEventDisableTiming);
        if (e == cudaSuccess && weight_layout(dtype) != LLMRS_LAYOUT_RAW && !ctx->stage_dev[i]) e = cudaMalloc((void **)&ctx->stage_dev[i], ctx->upload_piece);
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "upload_gguf_tensor: staging buffers");
    const int K = (int)d0, N = (int)(d1 ? d1 : 1);
    const size_t dev_bytes = quant ? weight_device_bytes((int)dtype, K, N) : is_block32(dtype) ? block32_device_bytes((int)dtype, K, N) : want;
    uint8_t *p = nullptr;
    e = cudaMalloc((void **)&p, dev_bytes);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "upload_gguf_tensor: cudaMalloc");
    // pieces of whole rows, so that the Q6_K re-layout can run piece by piece
    const size_t row_bytes = want / (size_t)N;
    if (row_bytes > ctx->upload_piece) {
        cudaFree(p);
        return ctx->fail(LLMRS_ERR_SHAPE, "upload_gguf_tensor: %s: one row is %zu bytes, more than a staging piece", name, row_bytes);
    }
    const size_t rows_per_piece = ctx->upload_piece / row_bytes;
    const uint64_t file_pos = g->data_offset + t->offset + first_row * src_row_bytes;
    bool io_ok = true;
    int piece = 0;
    for (size_t row = 0; row < (size_t)N && e == cudaSuccess && io_ok; row += rows_per_piece, piece++) {
        const int sb = piece & 1;
        const size_t rows = std::min(rows_per_piece, (size_t)N - row), bytes = rows * row_bytes;
        if (piece >= 2) e = cudaEventSynchronize(ctx->stage_done[sb]);      // the copy out of this piece, two pieces ago
        if (e != cudaSuccess) break;
        io_ok = llmrs::gguf_pread_parallel(g->fd, ctx->stage_host[sb], file_pos + row * row_bytes, bytes, ctx->upload_readers);
        if (!io_ok) break;
        if (weight_layout(dtype) != LLMRS_LAYOUT_RAW) {
            e = cudaMemcpyAsync(ctx->stage_dev[sb], ctx->stage_host[sb], bytes, cudaMemcpyHostToDevice, ctx->stream);
            if (e == cudaSuccess) {
                if (dtype == LLMRS_Q6K)
                    e = launch_q6k_repack(ctx->stage_dev[sb], p + row * q6k_row_stride(K), K, (int)rows, ctx->stream);
                else
                    e = launch_block32_repack((int)dtype, ctx->stage_dev[sb], p + row * block32_quant_stride((int)dtype, K),
                                              p + (size_t)N * block32_quant_stride((int)dtype, K) + row * block32_scale_stride(K), K,
                                              (int)rows, ctx->stream);
                ctx->launches++;
            }
        } else {
            e = cudaMemcpyAsync(p + row * row_bytes, ctx->stage_host[sb], bytes, cudaMemcpyHostToDevice, ctx->stream);
        }
        if (e == cudaSuccess) e = cudaEventRecord(ctx->stage_done[sb], ctx->stream);
    }
    const cudaError_t e2 = cudaStreamSynchronize(ctx->stream);    // also on failure: nothing may still read the pieces
    if (e == cudaSuccess) e = e2;
    if (!io_ok || e != cudaSuccess) {
        cudaFree(p);
        if (!io_ok) return ctx->fail(LLMRS_ERR_IO, "IO error: reading tensor %s", name);
        return ctx->cuda_fail(e, "upload_gguf_tensor: copy");
    }
    *out = llmrs_buf{p, dev_bytes, dtype, d0, d1, weight_layout(dtype), 1u, (uint32_t)ctx->device};
    return LLMRS_OK;
}

int llmrs_cuda_write(llmrs_ctx *ctx, llmrs_buf *dst, const void *host, size_t nbytes) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!dst || !dst->dptr || !host) return ctx->fail(LLMRS_ERR_ARG, "write: null pointer");
    if (!dense_elem_bytes(dst->dtype)) return ctx->fail(LLMRS_ERR_DTYPE, "write: only F32/BF16 buffers");
    if (nbytes > dst->nbytes) return ctx->fail(LLMRS_ERR_SHAPE, "write: %zu bytes into a %llu-byte buffer", nbytes,
                                               (unsigned long long)dst->nbytes);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e == cudaSuccess) e = cudaMemcpyAsync(dst->dptr, host, nbytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "write");
    return LLMRS_OK;
}

// The tensor-core path: which kernel serves M tokens, how much scratch it needs, and its launch.
static bool uses_exact_kernel(const llmrs_ctx *ctx, uint32_t M) {
    return ctx->two_term && ctx->exact && M <= (uint32_t)GEMM_EXACT_MAX_TOKENS;
}
static size_t tc_scratch_bytes(const llmrs_ctx *ctx, uint32_t K, uint32_t M) {
    return uses_exact_kernel(ctx, M) ? gemm_exact_scratch_bytes((int)K, (int)M) : gemm_scratch_bytes((int)K, (int)M);
}
// For the length of one call that multiplies several weights with the same input.
struct ActsShareScope {
    llmrs_ctx *ctx;
    explicit ActsShareScope(llmrs_ctx *c) : ctx(c) { ctx->acts_share = true; ctx->acts_have = false; }
    ~ActsShareScope() { ctx->acts_share = false; ctx->acts_have = false; }
};
static cudaError_t tc_matmul(llmrs_ctx *ctx, uint32_t wdtype, const void *w, const void *x, uint32_t x_dtype, void *out,
                             uint32_t out_dtype, uint32_t K, uint32_t N, uint32_t M, const GemmGather *gather = nullptr) {
    if (uses_exact_kernel(ctx, M)) {
        int acts_mode = EXACT_ACTS_CONVERT;
        if (ctx->acts_share) {
            const bool same = ctx->acts_have && ctx->acts_x == x && ctx->acts_K == K && ctx->acts_M == M && ctx->acts_dtype == x_dtype;
            acts_mode = same ? EXACT_ACTS_REUSE : EXACT_ACTS_CONVERT_ALL;
            ctx->acts_have = true; ctx->acts_x = x; ctx->acts_K = K; ctx->acts_M = M; ctx->acts_dtype = x_dtype;
        }
        return launch_gemm_exact((int)wdtype, (const uint8_t *)w, x, (int)x_dtype, out, (int)out_dtype, (int)K, (int)N, (int)M,
                                 ctx->scratch, ctx->split_ws, ctx->gemm_split, ctx->sink(), ctx->stream, &ctx->launches, gather,
                                 ctx->pdl, ctx->sm_count, acts_mode, ctx->conv_norm_w, ctx->conv_norm_eps);
    }
    ctx->acts_have = false;                              // the other kernel writes its own conversion into the scratch
    return launch_gemm((int)wdtype, (const uint8_t *)w, x, (int)x_dtype, out, (int)out_dtype, (int)K, (int)N, (int)M,
                       ctx->scratch, ctx->split_ws, ctx->gemm_split, ctx->sink(), ctx->stream, &ctx->launches, gather,
                       ctx->two_term, ctx->pdl);
}

// Several K-quant weights of one format against one input on the small-batch tensor-core kernel, one launch.
// The caller has checked shapes and devices; false: not eligible, use single calls.
static bool tc_matmul_multi_ok(const llmrs_ctx *ctx, int n, const llmrs_buf *const *ws, const llmrs_buf *const *outs, uint32_t M) {
    if (n < 2 || n > 3 || !uses_exact_kernel(ctx, M)) return false;
    for (int i = 0; i < n; i++) {
        if (ws[i]->dtype != ws[0]->dtype || ws[i]->dim0 != ws[0]->dim0 || outs[i]->dtype != outs[0]->dtype) return false;
        if (ws[i]->dtype != LLMRS_Q4K && ws[i]->dtype != LLMRS_Q6K) return false;
        if (ws[i]->layout != (ws[i]->dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : LLMRS_LAYOUT_RAW)) return false;
    }
    return true;
}
static cudaError_t tc_matmul_multi(llmrs_ctx *ctx, int n, const llmrs_buf *const *ws, void *const *outs, uint32_t out_dtype,
                                   const void *x, uint32_t x_dtype, uint32_t K, uint32_t M) {
    const uint8_t *wp[3];
    int ns[3];
    for (int i = 0; i < n; i++) {
        wp[i] = (const uint8_t *)ws[i]->dptr;
        ns[i] = (int)(ws[i]->dim1 ? ws[i]->dim1 : 1);
    }
    ctx->acts_have = false;
    return launch_gemm_exact_multi((int)ws[0]->dtype, n, wp, ns, outs, x, (int)x_dtype, (int)out_dtype, (int)K, (int)M,
                                   ctx->scratch, ctx->split_ws, ctx->gemm_split, ctx->sink(), ctx->stream, &ctx->launches,
                                   ctx->pdl, ctx->sm_count, ctx->conv_norm_w, ctx->conv_norm_eps);
}

// Between the decode kernel's token limit and 64 tokens both kernels meet the decode tolerance, so
// the cheaper one runs.  The decode kernel streams the weights once per pass of up to four tokens
// (fewer where the staged activations of four do not fit): about 2 us + 0.15 us per MB and token,
// at least 4.4 us + 0.3 us per token a pass.  The small-batch tensor-core kernel streams the weights once behind a floor
// (activation conversion, pipeline fill, the exchange of tiles cut along K): 8.3 us + 0.3 us/MB up to 16
// tokens, rising to 11.2 us + 0.5 us/MB at 64 (fitted on a B200 to 4096x1024 .. 4096x128256 weights,
// calls replayed from a CUDA graph).  The older kernels it replaces (LLMRS_TC_EXACT=0): two-term
// max(47 us, 0.61 us/MB), or 27 us + 0.6 us/MB where its tiles are cut along K; one-term max(25 us, 0.31 us/MB).
static bool decode_kernel_cheaper(const llmrs_ctx *ctx, const llmrs_buf *weight, uint32_t M, uint32_t K) {
    if (M > (uint32_t)GEMM_TWO_TERM_MAX_TOKENS || K > gemv_max_k()) return false;
    const int per_pass = std::min(4, gemv_single_launch_max_tokens((int)weight->dtype, (int)K));
    if (per_pass <= 0) return false;
    const double mb = (double)weight->nbytes * 1e-6;
    // two-term: weights of up to half a wave of tiles and K >= 4096 are cut along K over all SMs
    const bool cut = ctx->split_ws && ctx->gemm_split != 0 && K >= 4096 && (weight->dim1 + 127) / 128 <= (uint32_t)ctx->sm_count / 2;
    const double over16 = M > 16 ? (double)(M - 16) : 0.0;
    const double per_mb = weight->dtype == LLMRS_Q6K ? 0.26 : 0.3;
    const double tc = !ctx->two_term ? std::max(25.0, 0.31 * mb)
                      : ctx->exact   ? (8.3 + 0.06 * over16) + (per_mb + 0.0042 * over16) * mb
                      : cut          ? 27.0 + 0.6 * mb
                                     : std::max(47.0, 0.61 * mb);
    double decode = 0.0;
    for (uint32_t done = 0; done < M; done += (uint32_t)per_pass) {
        const double t = (double)std::min<uint32_t>((uint32_t)per_pass, M - done);
        decode += std::max(4.4 + 0.3 * t, 2.0 + 0.15 * mb * t);
    }
    return decode < tc;
}

// The kernel llmrs_cuda_matmul picks for M tokens of this weight: the decode kernel or the tensor cores.
// One token is always the decode kernel's.  With the estimate on (the default), two tokens and more go
// to whichever the estimate makes cheaper, as long as the tensor-core kernel in use meets the decode
// tolerance (the small-batch kernel does; the one-term kernel takes over only above gemv_max_m tokens).
// LLMRS_GEMV_MAX_M fixes the border instead: the decode kernel up to that many tokens.
static bool matmul_uses_decode_kernel(const llmrs_ctx *ctx, const llmrs_buf *weight, uint32_t M, uint32_t K) {
    if (M <= 1) return true;
    if (!ctx->cost_rule) return (int)M <= ctx->gemv_max_m;
    if ((int)M <= ctx->gemv_max_m && !(ctx->two_term && ctx->exact)) return true;
    return decode_kernel_cheaper(ctx, weight, M, K);
}

// matmul for the weight types beside the K-quants (metal/mod.rs:503-518, 542-562, 634-686): dense F32 / F16 /
// BF16 and Q8_0 / Q4_0.  Up to 8 tokens the streaming kernel; dense weights from 9 tokens on run on the tensor
// cores; the block formats take the streaming kernel in passes of 8 tokens (the reference runs one matvec per
// position for them).
static int matmul_other(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input) {
    const uint32_t K = weight->dim0, N = weight->dim1 ? weight->dim1 : 1, M = input->dim1 ? input->dim1 : 1;
    if (weight->layout != weight_layout(weight->dtype))
        return ctx->fail(LLMRS_ERR_ARG, "matmul: weight was not created by upload_tensor (layout %u)", weight->layout);
    if (!dense_elem_bytes(input->dtype) || !dense_elem_bytes(out->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul: activations must be F32 or BF16 (got %u -> %u)", input->dtype, out->dtype);
    if (!dense_gemv_shape_ok((int)weight->dtype, (int)K))
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: in_features %u: a multiple of %d is needed for this weight type", K,
                         is_block32(weight->dtype) ? 32 : weight->dtype == LLMRS_F32 ? 4 : 8);
    if (input->dim0 != K)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: input has %u features, weight expects %u", input->dim0, K);
    if (out->dim0 != N || (out->dim1 ? out->dim1 : 1) != M)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: output is [%u, %u], expected [%u, %u]", out->dim0, out->dim1, N, M);
    if (weight->device != (uint32_t)ctx->device || input->device != (uint32_t)ctx->device || out->device != (uint32_t)ctx->device)
        return ctx->fail(LLMRS_ERR_ARG, "matmul: buffers belong to another device");
    if ((reinterpret_cast<uintptr_t>(input->dptr) & 15) || (reinterpret_cast<uintptr_t>(weight->dptr) & 15))
        return ctx->fail(LLMRS_ERR_ARG, "matmul: buffers must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    const bool tensor_cores = M > 8 && !is_block32(weight->dtype) && dense_gemm_shape_ok((int)weight->dtype, (int)K);
    cudaError_t e = cudaSuccess;
    if (tensor_cores) {
        ctx->acts_have = false;                          // this kernel's conversion overwrites the shared scratch
        e = ctx->reserve_scratch(dense_gemm_scratch_bytes((int)weight->dtype, (int)K, (int)M));
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: scratch (grow it with one call outside graph capture)");
    }
    e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: event");
    char perf_name[48];
    if (ctx->perf) snprintf(perf_name, sizeof perf_name, "matmul %s %s", dtype_name(weight->dtype), tensor_cores ? "tensor cores" : "streaming kernel");
    PerfScope perf(ctx, perf_name, matmul_bytes(weight, input, out), matmul_flops(weight, input));
    if (tensor_cores)
        e = launch_dense_gemm((int)weight->dtype, (const uint8_t *)weight->dptr, input->dptr, (int)input->dtype, out->dptr,
                              (int)out->dtype, (int)K, (int)N, (int)M, ctx->scratch, ctx->sm_count, ctx->sink(), ctx->stream,
                              &ctx->launches);
    else
        e = launch_dense_gemv((int)weight->dtype, (const uint8_t *)weight->dptr, input->dptr, (int)input->dtype, out->dptr,
                              (int)out->dtype, (int)K, (int)N, (int)M, ctx->sm_count, ctx->pdl, ctx->stream, &ctx->launches);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: launch");
    return LLMRS_OK;
}

int llmrs_cuda_matmul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !weight || !input || !out->dptr || !weight->dptr || !input->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "matmul: null buffer");
    // K = weight.dim0, N = weight.dim1, M = max(input.dim1, 1)  (metal/mod.rs:497-499)
    const uint32_t K = weight->dim0, N = weight->dim1 ? weight->dim1 : 1, M = input->dim1 ? input->dim1 : 1;
    if (is_other_weight(weight->dtype)) return matmul_other(ctx, out, weight, input);
    if (weight->dtype != LLMRS_Q4K && weight->dtype != LLMRS_Q6K)
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul: weight dtype %u is not supported (F32, F16, BF16, Q4_0, Q8_0, Q4_K, Q6_K)", weight->dtype);
    const uint32_t want_layout = weight->dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : LLMRS_LAYOUT_RAW;
    if (weight->layout != want_layout)
        return ctx->fail(LLMRS_ERR_ARG, "matmul: weight was not created by upload_tensor (layout %u)", weight->layout);
    if (!dense_elem_bytes(input->dtype) || !dense_elem_bytes(out->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul: activations must be F32 or BF16 (got %u -> %u)", input->dtype,
                         out->dtype);
    if (K % QK_K) return ctx->fail(LLMRS_ERR_SHAPE, "matmul: in_features %u is not a multiple of 256", K);
    // a caller that folded a norm or a residual into this call has already chosen the decode kernel
    const bool decode = !ctx->conv_norm_w && (ctx->norm_w || ctx->residual || matmul_uses_decode_kernel(ctx, weight, M, K));
    if (decode && K > gemv_max_k())
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: in_features %u exceeds the supported maximum %zu", K, gemv_max_k());
    if (input->dim0 != K)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: input has %u features, weight expects %u", input->dim0, K);
    const uint32_t out_m = out->dim1 ? out->dim1 : 1;
    if (out->dim0 != N || out_m != M)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul: output is [%u, %u], expected [%u, %u]", out->dim0, out_m, N, M);
    if (weight->device != (uint32_t)ctx->device || input->device != (uint32_t)ctx->device ||
        out->device != (uint32_t)ctx->device)
        return ctx->fail(LLMRS_ERR_ARG, "matmul: buffers belong to another device");
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: event");
    char perf_name[48];
    if (ctx->perf)
        snprintf(perf_name, sizeof perf_name, "matmul %s %s", dtype_name(weight->dtype),
                 decode ? "decode kernel" : uses_exact_kernel(ctx, M) ? "tensor cores, exact" :
                 (M <= (uint32_t)GEMM_TWO_TERM_MAX_TOKENS && ctx->two_term) ? "tensor cores, two-term" : "tensor cores");
    PerfScope perf(ctx, perf_name, matmul_bytes(weight, input, out), matmul_flops(weight, input));
    if (decode) {
        e = launch_gemv((int)weight->dtype, (const uint8_t *)weight->dptr, input->dptr, (int)input->dtype, out->dptr,
                        (int)out->dtype, (int)K, (int)N, (int)M, ctx->sm_count, ctx->pdl, ctx->sink(), ctx->stream,
                        &ctx->launches, ctx->residual ? ctx->residual->dptr : nullptr,
                        ctx->residual ? (int)ctx->residual->dtype : DT_F32, ctx->norm_w, ctx->norm_eps);
    } else {
        // The reference switches to its tiled GEMM kernels by seq_len too (metal/mod.rs:542-633).
        e = ctx->reserve_scratch(tc_scratch_bytes(ctx, K, M));
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: scratch (grow it with one call outside graph capture)");
        e = tc_matmul(ctx, weight->dtype, weight->dptr, input->dptr, input->dtype, out->dptr, out->dtype, K, N, M);
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul: launch");
    return LLMRS_OK;
}

static size_t buf_elems(const llmrs_buf *b) { return (size_t)b->dim0 * (b->dim1 ? b->dim1 : 1); }

static int elementwise(llmrs_ctx *ctx, const char *name, int op, llmrs_buf *out, const llmrs_buf *a, const llmrs_buf *b) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !a || !out->dptr || !a->dptr || (op && (!b || !b->dptr))) return ctx->fail(LLMRS_ERR_ARG, "%s: null buffer", name);
    if (!dense_elem_bytes(out->dtype) || !dense_elem_bytes(a->dtype) || (op && !dense_elem_bytes(b->dtype)))
        return ctx->fail(LLMRS_ERR_DTYPE, "%s: buffers must be F32 or BF16", name);
    const size_t n = buf_elems(out);
    if (buf_elems(a) != n || (op && buf_elems(b) != n)) return ctx->fail(LLMRS_ERR_SHAPE, "%s: buffers differ in size", name);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, name, (double)n * (dense_elem_bytes(a->dtype) + (op ? dense_elem_bytes(b->dtype) : 0) + dense_elem_bytes(out->dtype)),
                   (double)n);
    if (e == cudaSuccess)
        e = launch_elementwise(op, a->dptr, (int)a->dtype, op ? b->dptr : nullptr, op ? (int)b->dtype : DT_F32, out->dptr,
                               (int)out->dtype, n, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, name);
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_silu(llmrs_ctx *ctx, llmrs_buf *x) { return elementwise(ctx, "silu", 0, x, x, nullptr); }
int llmrs_cuda_mul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *a, const llmrs_buf *b) {
    return elementwise(ctx, "mul", 1, out, a, b);
}
int llmrs_cuda_add(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *a, const llmrs_buf *b) {
    return elementwise(ctx, "add", 2, out, a, b);
}

int llmrs_cuda_rms_norm(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *input, const llmrs_buf *weight, float eps) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !input || !weight || !out->dptr || !input->dptr || !weight->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "rms_norm: null buffer");
    if (!dense_elem_bytes(out->dtype) || !dense_elem_bytes(input->dtype) || weight->dtype != LLMRS_F32)
        return ctx->fail(LLMRS_ERR_DTYPE, "rms_norm: activations F32 or BF16, weight F32");
    const uint32_t dim = input->dim0, rows = input->dim1 ? input->dim1 : 1;
    if (weight->dim0 != dim || out->dim0 != dim || (out->dim1 ? out->dim1 : 1) != rows)
        return ctx->fail(LLMRS_ERR_SHAPE, "rms_norm: input [%u, %u], weight [%u], output [%u, %u]", dim, rows, weight->dim0,
                         out->dim0, out->dim1);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "rms_norm", (double)dim * rows * (dense_elem_bytes(input->dtype) + dense_elem_bytes(out->dtype)) + 4.0 * dim,
                   3.0 * dim * rows);
    if (e == cudaSuccess)
        e = launch_rms_norm(input->dptr, (int)input->dtype, (const float *)weight->dptr, out->dptr, (int)out->dtype,
                            (int)dim, (int)rows, eps, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_argmax(llmrs_ctx *ctx, const llmrs_buf *logits, uint32_t *index) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!logits || !logits->dptr || !index) return ctx->fail(LLMRS_ERR_ARG, "argmax: null pointer");
    if (!dense_elem_bytes(logits->dtype)) return ctx->fail(LLMRS_ERR_DTYPE, "argmax: logits must be F32 or BF16");
    const size_t n = buf_elems(logits);
    if (n == 0 || n > 0xFFFFFFFFull) return ctx->fail(LLMRS_ERR_SHAPE, "argmax: %zu values", n);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    {
        PerfScope perf(ctx, "argmax", (double)n * dense_elem_bytes(logits->dtype), 0.0);
        if (e == cudaSuccess) e = launch_argmax(logits->dptr, (int)logits->dtype, (uint32_t)n, ctx->argmax_out, ctx->stream);
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "argmax");
    ctx->launches++;
    int rc = llmrs_cuda_sync(ctx);                       // the trait returns the index: the call completes the stream
    if (rc != LLMRS_OK) return rc;
    e = cudaMemcpy(index, ctx->argmax_out, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "argmax: read");
    return LLMRS_OK;
}

int llmrs_cuda_rms_norm_heads(llmrs_ctx *ctx, llmrs_buf *x, const llmrs_buf *weight, float eps) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!x || !weight || !x->dptr || !weight->dptr) return ctx->fail(LLMRS_ERR_ARG, "rms_norm_heads: null buffer");
    if (!dense_elem_bytes(x->dtype) || weight->dtype != LLMRS_F32)
        return ctx->fail(LLMRS_ERR_DTYPE, "rms_norm_heads: activations F32 or BF16, weight F32");
    const size_t dim = buf_elems(weight), n = buf_elems(x);
    if (dim == 0 || n % dim) return ctx->fail(LLMRS_ERR_SHAPE, "rms_norm_heads: %zu values are not chunks of %zu", n, dim);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "rms_norm_heads", 2.0 * n * dense_elem_bytes(x->dtype), 3.0 * n);
    if (e == cudaSuccess)
        e = launch_rms_norm(x->dptr, (int)x->dtype, (const float *)weight->dptr, x->dptr, (int)x->dtype, (int)dim,
                            (int)(n / dim), eps, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_heads");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_rope(llmrs_ctx *ctx, llmrs_buf *q, llmrs_buf *k, const llmrs_buf *positions, uint32_t head_dim,
                    float rope_theta, uint32_t split_half) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!q || !k || !positions || !q->dptr || !k->dptr || !positions->dptr) return ctx->fail(LLMRS_ERR_ARG, "rope: null buffer");
    if (!dense_elem_bytes(q->dtype) || !dense_elem_bytes(k->dtype) || positions->dtype != LLMRS_I32)
        return ctx->fail(LLMRS_ERR_DTYPE, "rope: q and k F32 or BF16, positions I32");
    const uint32_t seq = q->dim1 ? q->dim1 : 1;
    if (head_dim == 0 || head_dim % 2 || q->dim0 % head_dim || k->dim0 % head_dim || (k->dim1 ? k->dim1 : 1) != seq ||
        buf_elems(positions) < seq)
        return ctx->fail(LLMRS_ERR_SHAPE, "rope: q [%u, %u], k [%u, %u], head_dim %u, %zu positions", q->dim0, q->dim1,
                         k->dim0, k->dim1, head_dim, buf_elems(positions));
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "rope", 2.0 * (buf_elems(q) * dense_elem_bytes(q->dtype) + buf_elems(k) * dense_elem_bytes(k->dtype)), 0.0);
    if (e == cudaSuccess)
        e = launch_rope(q->dptr, (int)q->dtype, (int)q->dim0, k->dptr, (int)k->dtype, (int)k->dim0,
                        (const uint32_t *)positions->dptr, (int)head_dim, rope_theta, (int)seq, split_half != 0,
                        ctx->stream, ctx->pdl);
    ctx->launches++;
    if (e != cudaSuccess) return ctx->cuda_fail(e, "rope");
    return LLMRS_OK;
}

int llmrs_cuda_rope_scatter_kv(llmrs_ctx *ctx, llmrs_buf *q, llmrs_buf *k, const llmrs_buf *v, const llmrs_buf *positions,
                               uint32_t head_dim, float rope_theta, uint32_t split_half, llmrs_buf *k_pool,
                               llmrs_buf *v_pool, const llmrs_buf *slot_mapping) {
    if (!ctx) return LLMRS_ERR_ARG;
    const llmrs_buf *all[7] = {q, k, v, positions, k_pool, v_pool, slot_mapping};
    for (const llmrs_buf *b : all)
        if (!b || !b->dptr) return ctx->fail(LLMRS_ERR_ARG, "rope_scatter_kv: null buffer");
    if (!dense_elem_bytes(q->dtype) || k->dtype != q->dtype || v->dtype != q->dtype || k_pool->dtype != q->dtype ||
        v_pool->dtype != q->dtype || positions->dtype != LLMRS_I32 || slot_mapping->dtype != LLMRS_I32)
        return ctx->fail(LLMRS_ERR_DTYPE, "rope_scatter_kv: q, k, v and the pools of one type (F32 or BF16), indices I32");
    const uint32_t seq = q->dim1 ? q->dim1 : 1;
    if (head_dim == 0 || head_dim % 2 || q->dim0 % head_dim || k->dim0 % head_dim || v->dim0 != k->dim0 ||
        (k->dim1 ? k->dim1 : 1) != seq || (v->dim1 ? v->dim1 : 1) != seq || buf_elems(positions) < seq ||
        buf_elems(slot_mapping) < seq || buf_elems(k_pool) % k->dim0 || buf_elems(v_pool) % k->dim0)
        return ctx->fail(LLMRS_ERR_SHAPE, "rope_scatter_kv: q [%u, %u], k [%u, %u], v [%u, %u], head_dim %u", q->dim0, q->dim1,
                         k->dim0, k->dim1, v->dim0, v->dim1, head_dim);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "rope_scatter_kv", dense_elem_bytes(q->dtype) * (2.0 * buf_elems(q) + 3.0 * buf_elems(k) + 2.0 * buf_elems(v)), 0.0);
    if (e == cudaSuccess)
        e = launch_rope_scatter(q->dptr, (int)q->dim0, k->dptr, v->dptr, (int)k->dim0, (int)q->dtype,
                                (const uint32_t *)positions->dptr, (const uint32_t *)slot_mapping->dptr, k_pool->dptr,
                                v_pool->dptr, (int)head_dim, rope_theta, (int)seq, split_half != 0, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "rope_scatter_kv");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_scatter_kv(llmrs_ctx *ctx, llmrs_buf *pool, const llmrs_buf *src, const llmrs_buf *slot_mapping,
                          uint32_t kv_dim, uint32_t num_tokens) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!pool || !src || !slot_mapping || !pool->dptr || !src->dptr || !slot_mapping->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "scatter_kv: null buffer");
    if (!dense_elem_bytes(pool->dtype) || pool->dtype != src->dtype || slot_mapping->dtype != LLMRS_I32)
        return ctx->fail(LLMRS_ERR_DTYPE, "scatter_kv: pool and src of one type (F32 or BF16), slot_mapping I32");
    if ((size_t)kv_dim * num_tokens > buf_elems(src) || buf_elems(slot_mapping) < num_tokens || kv_dim == 0 ||
        buf_elems(pool) % kv_dim)
        return ctx->fail(LLMRS_ERR_SHAPE, "scatter_kv: %u tokens of %u values from %zu, %zu slots", num_tokens, kv_dim,
                         buf_elems(src), buf_elems(slot_mapping));
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "scatter_kv", 2.0 * kv_dim * num_tokens * dense_elem_bytes(src->dtype), 0.0);
    if (e == cudaSuccess)
        e = launch_move_rows(pool->dptr, src->dptr, (const uint32_t *)slot_mapping->dptr, 1,
                             (size_t)kv_dim * dense_elem_bytes(src->dtype), (int)num_tokens, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "scatter_kv");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_gather(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *src, const llmrs_buf *indices,
                      uint32_t num_indices) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !src || !indices || !out->dptr || !src->dptr || !indices->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "gather: null buffer");
    if (!dense_elem_bytes(out->dtype) || out->dtype != src->dtype || indices->dtype != LLMRS_I32)
        return ctx->fail(LLMRS_ERR_DTYPE, "gather: out and src of one type (F32 or BF16), indices I32");
    const uint32_t dim = src->dim0;
    if (out->dim0 != dim || (size_t)dim * num_indices > buf_elems(out) || buf_elems(indices) < num_indices)
        return ctx->fail(LLMRS_ERR_SHAPE, "gather: %u columns of %u values into [%u, %u]", num_indices, dim, out->dim0, out->dim1);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    PerfScope perf(ctx, "gather", 2.0 * dim * num_indices * dense_elem_bytes(src->dtype), 0.0);
    if (e == cudaSuccess)
        e = launch_move_rows(out->dptr, src->dptr, (const uint32_t *)indices->dptr, 0,
                             (size_t)dim * dense_elem_bytes(src->dtype), (int)num_indices, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "gather");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_attention(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *q, const llmrs_buf *k_pool,
                         const llmrs_buf *v_pool, const llmrs_buf *block_table, const llmrs_buf *query_starts,
                         const llmrs_buf *seq_lens, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                         uint32_t block_size, uint32_t max_blocks_per_seq) {
    if (!ctx) return LLMRS_ERR_ARG;
    const llmrs_buf *all[7] = {out, q, k_pool, v_pool, block_table, query_starts, seq_lens};
    for (const llmrs_buf *b : all)
        if (!b || !b->dptr) return ctx->fail(LLMRS_ERR_ARG, "attention: null buffer");
    if (!dense_elem_bytes(q->dtype) || out->dtype != q->dtype || k_pool->dtype != q->dtype || v_pool->dtype != q->dtype)
        return ctx->fail(LLMRS_ERR_DTYPE, "attention: q, out and the pools of one type (F32 or BF16)");
    if (block_table->dtype != LLMRS_I32 || query_starts->dtype != LLMRS_I32 || seq_lens->dtype != LLMRS_I32)
        return ctx->fail(LLMRS_ERR_DTYPE, "attention: block_table, query_starts and seq_lens are I32");
    if (n_heads == 0 || n_kv_heads == 0 || n_heads % n_kv_heads || head_dim == 0 || head_dim % 32 || head_dim > 256 ||
        block_size == 0 || max_blocks_per_seq == 0)
        return ctx->fail(LLMRS_ERR_SHAPE, "attention: %u heads, %u kv heads, head_dim %u, pages of %u", n_heads, n_kv_heads,
                         head_dim, block_size);
    const size_t row = (size_t)n_heads * head_dim;
    const size_t total_q = buf_elems(q) / row, num_req = buf_elems(seq_lens);
    if (buf_elems(q) % row || buf_elems(out) != buf_elems(q) || buf_elems(query_starts) < num_req + 1 ||
        buf_elems(block_table) < num_req * max_blocks_per_seq)
        return ctx->fail(LLMRS_ERR_SHAPE, "attention: q of %zu values, %zu requests, %zu query_starts, %zu page entries",
                         buf_elems(q), num_req, buf_elems(query_starts), buf_elems(block_table));
    DeviceGuard guard(ctx->device);
    cudaError_t e;
    PerfScope perf(ctx, "attention", 2.0 * buf_elems(q) * dense_elem_bytes(q->dtype), 0.0);   // bytes: q and out only (the KV read depends on the lengths, which live on the device)
    if (attention_gqa_supported((int)q->dtype, (int)n_heads, (int)n_kv_heads, (int)head_dim)) {
        // The request lengths live on the device; the host knows the totals.  As many query tokens as requests:
        // a decode batch, split-sequence kernel.  One request: a prefill, tensor-core kernel.  Otherwise the batch
        // may mix the two: the tensor-core kernel takes the requests with several query tokens, the split-sequence
        // kernel, its grid over requests, those with one.
        const bool decode_only = total_q == num_req, prefill_only = num_req == 1 && total_q > 1;
        const int split_tokens = (int)num_req;            // single-token requests at most
        const int splits = prefill_only ? 1 : attention_splits(split_tokens, (int)n_kv_heads, (int)(block_size * max_blocks_per_seq), ctx->sm_count);
        // the workspace is indexed by query token
        const size_t need = attention_workspace_bytes((int)total_q, (int)n_heads, (int)head_dim, splits);
        if (need > ctx->att_ws_bytes) {              // grows outside stream capture only, like the scratch
            e = ctx->grow((void **)&ctx->att_ws, &ctx->att_ws_bytes, need);
            if (e == cudaErrorStreamCaptureUnsupported)
                return ctx->fail(LLMRS_ERR_CUDA, "attention: workspace must grow (make one call outside graph capture)");
            if (e != cudaSuccess) return ctx->cuda_fail(e, "attention: workspace");
        }
        e = ctx->begin_work();
        if (e == cudaSuccess && !decode_only) {
            e = launch_attention_prefill(q->dptr, k_pool->dptr, v_pool->dptr, out->dptr, (const uint32_t *)block_table->dptr,
                                         (const uint32_t *)query_starts->dptr, (const uint32_t *)seq_lens->dptr, (int)total_q,
                                         (int)num_req, (int)n_heads, (int)n_kv_heads, (int)head_dim, (int)block_size,
                                         (int)max_blocks_per_seq, !prefill_only, ctx->stream, ctx->pdl);
            ctx->launches++;
        }
        if (e == cudaSuccess && !prefill_only) {
            e = launch_attention_gqa(q->dptr, k_pool->dptr, v_pool->dptr, out->dptr, ctx->att_ws,
                                     (const uint32_t *)block_table->dptr, (const uint32_t *)query_starts->dptr,
                                     (const uint32_t *)seq_lens->dptr, (int)total_q, (int)num_req, (int)n_heads,
                                     (int)n_kv_heads, (int)head_dim, (int)block_size, (int)max_blocks_per_seq, splits,
                                     !decode_only, ctx->stream, ctx->pdl);
            ctx->launches += splits > 1 ? 2 : 1;
        }
        if (e != cudaSuccess) return ctx->cuda_fail(e, "attention");
        return LLMRS_OK;
    }
    e = ctx->begin_work();
    if (e == cudaSuccess)
        e = launch_attention(q->dptr, k_pool->dptr, v_pool->dptr, out->dptr, (int)q->dtype,
                             (const uint32_t *)block_table->dptr, (const uint32_t *)query_starts->dptr,
                             (const uint32_t *)seq_lens->dptr, (int)total_q, (int)num_req, (int)n_heads, (int)n_kv_heads,
                             (int)head_dim, (int)block_size, (int)max_blocks_per_seq, ctx->stream, ctx->pdl);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "attention");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_matmul_add(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input,
                          const llmrs_buf *residual) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!residual || !residual->dptr || !out) return ctx->fail(LLMRS_ERR_ARG, "matmul_add: null buffer");
    if (!dense_elem_bytes(residual->dtype)) return ctx->fail(LLMRS_ERR_DTYPE, "matmul_add: residual must be F32 or BF16");
    if (residual->dim0 != out->dim0 || (residual->dim1 ? residual->dim1 : 1) != (out->dim1 ? out->dim1 : 1))
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_add: residual is [%u, %u], output [%u, %u]", residual->dim0, residual->dim1,
                         out->dim0, out->dim1);
    const uint32_t M = input && input->dim1 ? input->dim1 : 1;
    const bool quant = weight && (weight->dtype == LLMRS_Q4K || weight->dtype == LLMRS_Q6K);
    const bool decode = input && quant && matmul_uses_decode_kernel(ctx, weight, M, weight->dim0);
    if (!decode) {                                   // tensor-core path: the matmul, then the add as its own kernel
        const uint8_t *r0 = (const uint8_t *)residual->dptr, *o0 = (const uint8_t *)out->dptr;
        const bool overlap = r0 < o0 + out->nbytes && o0 < r0 + residual->nbytes;
        if (!overlap || !input || !weight || !out->dptr) {
            int rc = llmrs_cuda_matmul(ctx, out, weight, input);
            return rc != LLMRS_OK ? rc : llmrs_cuda_add(ctx, out, out, residual);
        }
        if (!quant) {                                // another weight type: the product goes to a buffer of its own first
            const size_t need = (size_t)out->dim0 * (out->dim1 ? out->dim1 : 1) * sizeof(float);
            DeviceGuard guard(ctx->device);
            cudaError_t e = ctx->grow(&ctx->norm_tmp, &ctx->norm_tmp_bytes, need);
            if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_add: temporary (grow it with one call outside graph capture)");
            llmrs_buf tmp = *out;
            tmp.dptr = ctx->norm_tmp;
            tmp.nbytes = need;
            tmp.dtype = LLMRS_F32;
            tmp.owned = 0;
            int rc = llmrs_cuda_matmul(ctx, &tmp, weight, input);
            return rc != LLMRS_OK ? rc : llmrs_cuda_add(ctx, out, &tmp, residual);
        }
        // The residual IS the output (x = x + matmul(w, h), the usual call): the product goes to float32
        // scratch behind the GEMM's own scratch first, because the GEMM would overwrite the residual.
        const uint32_t K = weight->dim0, N = weight->dim1 ? weight->dim1 : 1;
        const size_t gemm_bytes = (tc_scratch_bytes(ctx, K, M) + 255) / 256 * 256;
        DeviceGuard guard(ctx->device);
        cudaError_t e = ctx->reserve_scratch(gemm_bytes + (size_t)M * N * sizeof(float));
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_add: scratch (grow it with one call outside graph capture)");
        llmrs_buf tmp = *out;
        tmp.dptr = (uint8_t *)ctx->scratch + gemm_bytes;
        tmp.nbytes = (size_t)M * N * sizeof(float);
        tmp.dtype = LLMRS_F32;
        tmp.owned = 0;
        int rc = llmrs_cuda_matmul(ctx, &tmp, weight, input);
        return rc != LLMRS_OK ? rc : llmrs_cuda_add(ctx, out, &tmp, residual);
    }
    ctx->residual = residual;                        // picked up by llmrs_cuda_matmul's decode branch
    int rc = llmrs_cuda_matmul(ctx, out, weight, input);
    ctx->residual = nullptr;
    return rc;
}

// rms_norm fused into the staging of the decode kernel where that kernel serves the call in one launch;
// otherwise rms_norm into a temporary, then the plain call.
static int with_norm(llmrs_ctx *ctx, const char *name, const llmrs_buf *input, const llmrs_buf *norm_weight, float eps,
                     bool fused_ok, bool conv_ok, const std::function<int(const llmrs_buf *)> &call) {
    if (!norm_weight || !norm_weight->dptr || !input || !input->dptr) return ctx->fail(LLMRS_ERR_ARG, "%s: null buffer", name);
    if (norm_weight->dtype != LLMRS_F32 || norm_weight->dim0 != input->dim0)
        return ctx->fail(LLMRS_ERR_SHAPE, "%s: norm weight must be F32 [%u]", name, input->dim0);
    if (fused_ok) {
        ctx->norm_w = (const float *)norm_weight->dptr;
        ctx->norm_eps = eps;
        int rc = call(input);
        ctx->norm_w = nullptr;
        return rc;
    }
    // Above the decode kernel's token limit, where the small-batch tensor-core kernel will run: the norm is folded
    // into that kernel's conversion of the activations (one kernel less, no rounding of the normalised values).
    const uint32_t M_in = input->dim1 ? input->dim1 : 1;
    if (conv_ok && (int)M_in > ctx->gemv_max_m && uses_exact_kernel(ctx, M_in) && dense_elem_bytes(input->dtype)) {
        ctx->conv_norm_w = (const float *)norm_weight->dptr;
        ctx->conv_norm_eps = eps;
        int rc = call(input);
        ctx->conv_norm_w = nullptr;
        return rc;
    }
    // the normalised activations go to a buffer of the context (grown outside stream capture only)
    const size_t need = (size_t)input->dim0 * (input->dim1 ? input->dim1 : 1) * dense_elem_bytes(input->dtype);
    if (!need) return ctx->fail(LLMRS_ERR_DTYPE, "%s: activations must be F32 or BF16", name);
    if (need > ctx->norm_tmp_bytes) {
        DeviceGuard guard(ctx->device);
        cudaError_t e = ctx->grow(&ctx->norm_tmp, &ctx->norm_tmp_bytes, need);
        if (e == cudaErrorStreamCaptureUnsupported)
            return ctx->fail(LLMRS_ERR_CUDA, "%s: temporary must grow (make one call outside graph capture)", name);
        if (e != cudaSuccess) return ctx->cuda_fail(e, name);
    }
    llmrs_buf tmp = *input;
    tmp.dptr = ctx->norm_tmp;
    tmp.nbytes = need;
    tmp.owned = 0;
    int rc = llmrs_cuda_rms_norm(ctx, &tmp, input, norm_weight, eps);
    return rc == LLMRS_OK ? call(&tmp) : rc;
}

int llmrs_cuda_rms_norm_matmul(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight, const llmrs_buf *input,
                               const llmrs_buf *norm_weight, float eps) {
    if (!ctx) return LLMRS_ERR_ARG;
    const uint32_t M = input && input->dim1 ? input->dim1 : 1;
    const bool fused = weight && input && (int)M <= ctx->gemv_max_m &&
                       (int)M <= gemv_single_launch_max_tokens((int)weight->dtype, (int)weight->dim0);
    const bool kquant = weight && (weight->dtype == LLMRS_Q4K || weight->dtype == LLMRS_Q6K);
    return with_norm(ctx, "rms_norm_matmul", input, norm_weight, eps, fused, kquant,
                     [&](const llmrs_buf *x) { return llmrs_cuda_matmul(ctx, out, weight, x); });
}

int llmrs_cuda_rms_norm_matmul_qkv(llmrs_ctx *ctx, llmrs_buf *out_q, llmrs_buf *out_k, llmrs_buf *out_v,
                                   const llmrs_buf *wq, const llmrs_buf *wk, const llmrs_buf *wv, const llmrs_buf *input,
                                   const llmrs_buf *norm_weight, float eps) {
    if (!ctx) return LLMRS_ERR_ARG;
    llmrs_buf *outs[3] = {out_q, out_k, out_v};
    const llmrs_buf *ws[3] = {wq, wk, wv};
    for (int i = 0; i < 3; i++)
        if (!outs[i] || !ws[i] || !outs[i]->dptr || !ws[i]->dptr) return ctx->fail(LLMRS_ERR_ARG, "rms_norm_matmul_qkv: null buffer");
    if (!input || !input->dptr || !norm_weight || !norm_weight->dptr) return ctx->fail(LLMRS_ERR_ARG, "rms_norm_matmul_qkv: null buffer");
    const uint32_t K = input->dim0, M = input->dim1 ? input->dim1 : 1;
    // One launch serves weights of one format whose call the decode kernel would take in one pass; anything
    // else (more tokens, odd shapes, an argument error to report) goes through the single calls.
    bool one_pass = (int)M <= ctx->gemv_max_m && M <= 4 && dense_elem_bytes(input->dtype) && norm_weight->dtype == LLMRS_F32 &&
                    norm_weight->dim0 == K && K % QK_K == 0 && K <= gemv_max_k() && input->device == (uint32_t)ctx->device;
    for (int i = 0; i < 3 && one_pass; i++) {
        const llmrs_buf *w = ws[i], *o = outs[i];
        const uint32_t want_layout = w->dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : LLMRS_LAYOUT_RAW;
        const uint32_t n = w->dim1 ? w->dim1 : 1;
        one_pass = (w->dtype == LLMRS_Q4K || w->dtype == LLMRS_Q6K) && w->layout == want_layout && w->dim0 == K &&
                   (int)M <= gemv_single_launch_max_tokens((int)w->dtype, (int)K) && o->dtype == outs[0]->dtype &&
                   dense_elem_bytes(o->dtype) && o->dim0 == n && (o->dim1 ? o->dim1 : 1) == M &&
                   w->device == (uint32_t)ctx->device && o->device == (uint32_t)ctx->device;
    }
    if (!one_pass) {
        bool all_kquant = true;
        for (int i = 0; i < 3; i++) all_kquant = all_kquant && (ws[i]->dtype == LLMRS_Q4K || ws[i]->dtype == LLMRS_Q6K);
        if ((int)M > ctx->gemv_max_m)                    // above the decode kernel's limit: the norm once, in front (or in the conversion)
            return with_norm(ctx, "rms_norm_matmul_qkv", input, norm_weight, eps, false, all_kquant, [&](const llmrs_buf *x) {
                // one launch over the three weights where they share a format; else three calls, one conversion
                bool shapes_ok = true;
                for (int i = 0; i < 3; i++) {
                    const uint32_t n = ws[i]->dim1 ? ws[i]->dim1 : 1;
                    shapes_ok = shapes_ok && ws[i]->dim0 == K && K % QK_K == 0 && outs[i]->dim0 == n &&
                                (outs[i]->dim1 ? outs[i]->dim1 : 1) == M && dense_elem_bytes(outs[i]->dtype) &&
                                dense_elem_bytes(x->dtype) && ws[i]->device == (uint32_t)ctx->device &&
                                outs[i]->device == (uint32_t)ctx->device &&
                                !(reinterpret_cast<uintptr_t>(ws[i]->dptr) & 15);
                }
                if (shapes_ok && tc_matmul_multi_ok(ctx, 3, ws, outs, M)) {
                    DeviceGuard guard(ctx->device);
                    cudaError_t e = ctx->reserve_scratch(tc_scratch_bytes(ctx, K, M));
                    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_matmul_qkv: scratch (grow it with one call outside graph capture)");
                    e = ctx->begin_work();
                    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_matmul_qkv: event");
                    PerfScope perf(ctx, "matmul q/k/v, one launch", matmul_bytes(wq, x, out_q) + matmul_bytes(wk, x, out_k) + matmul_bytes(wv, x, out_v),
                                   matmul_flops(wq, x) + matmul_flops(wk, x) + matmul_flops(wv, x));
                    void *op[3] = {out_q->dptr, out_k->dptr, out_v->dptr};
                    e = tc_matmul_multi(ctx, 3, ws, op, outs[0]->dtype, x->dptr, x->dtype, K, M);
                    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_matmul_qkv: launch");
                    return (int)LLMRS_OK;
                }
                ActsShareScope share(ctx);
                int rc = LLMRS_OK;
                for (int i = 0; i < 3 && rc == LLMRS_OK; i++) rc = llmrs_cuda_matmul(ctx, outs[i], ws[i], x);
                return rc;
            });
        int rc = LLMRS_OK;
        for (int i = 0; i < 3 && rc == LLMRS_OK; i++) rc = llmrs_cuda_rms_norm_matmul(ctx, outs[i], ws[i], input, norm_weight, eps);
        return rc;
    }
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_matmul_qkv: event");
    PerfScope perf(ctx, "rms_norm_matmul_qkv", matmul_bytes(wq, input, out_q) + matmul_bytes(wk, input, out_k) + matmul_bytes(wv, input, out_v) -
                   2.0 * K * M * dense_elem_bytes(input->dtype), matmul_flops(wq, input) + matmul_flops(wk, input) + matmul_flops(wv, input));
    for (uint32_t dt : {(uint32_t)LLMRS_Q4K, (uint32_t)LLMRS_Q6K}) {
        const uint8_t *gw[3];
        void *go[3];
        int gn[3], n = 0;
        for (int i = 0; i < 3; i++)
            if (ws[i]->dtype == dt) {
                gw[n] = (const uint8_t *)ws[i]->dptr;
                go[n] = outs[i]->dptr;
                gn[n++] = (int)(ws[i]->dim1 ? ws[i]->dim1 : 1);
            }
        if (n == 0) continue;
        if (n == 1)
            e = launch_gemv((int)dt, gw[0], input->dptr, (int)input->dtype, go[0], (int)outs[0]->dtype, (int)K, gn[0], (int)M,
                            ctx->sm_count, ctx->pdl, ctx->sink(), ctx->stream, &ctx->launches, nullptr, DT_F32,
                            (const float *)norm_weight->dptr, eps);
        else
            e = launch_gemv_multi((int)dt, n, gw, gn, go, input->dptr, (int)input->dtype, (int)outs[0]->dtype, (int)K, (int)M,
                                  ctx->sm_count, ctx->pdl, ctx->sink(), ctx->stream, &ctx->launches,
                                  (const float *)norm_weight->dptr, eps);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "rms_norm_matmul_qkv: launch");
    }
    return LLMRS_OK;
}

int llmrs_cuda_rms_norm_matmul_gate_up(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *w_gate, const llmrs_buf *w_up,
                                       const llmrs_buf *input, const llmrs_buf *norm_weight, float eps) {
    if (!ctx) return LLMRS_ERR_ARG;
    const uint32_t M = input && input->dim1 ? input->dim1 : 1;
    const bool fused = w_gate && input && (int)M <= ctx->gemv_max_m &&
                       gemv_gate_up_fits((int)w_gate->dtype, (int)w_gate->dim0, (int)M);
    return with_norm(ctx, "rms_norm_matmul_gate_up", input, norm_weight, eps, fused, true,
                     [&](const llmrs_buf *x) { return llmrs_cuda_matmul_gate_up(ctx, out, w_gate, w_up, x); });
}

int llmrs_cuda_matmul_gate_up(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *w_gate, const llmrs_buf *w_up,
                              const llmrs_buf *input) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !w_gate || !w_up || !input || !out->dptr || !w_gate->dptr || !w_up->dptr || !input->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_gate_up: null buffer");
    const uint32_t K = w_gate->dim0, N = w_gate->dim1 ? w_gate->dim1 : 1, M = input->dim1 ? input->dim1 : 1;
    if (w_gate->dtype != LLMRS_Q4K && w_gate->dtype != LLMRS_Q6K)
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_gate_up: weight dtype %u is not Q4_K/Q6_K", w_gate->dtype);
    if (w_up->dtype != w_gate->dtype || w_up->dim0 != K || (w_up->dim1 ? w_up->dim1 : 1) != N)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: gate and up weights differ in type or shape");
    const uint32_t want_layout = w_gate->dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : LLMRS_LAYOUT_RAW;
    if (w_gate->layout != want_layout || w_up->layout != want_layout)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_gate_up: weights were not created by upload_tensor");
    if (!dense_elem_bytes(input->dtype) || !dense_elem_bytes(out->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_gate_up: activations must be F32 or BF16");
    if (K % QK_K) return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: in_features %u is not a multiple of 256", K);
    if (input->dim0 != K)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: input has %u features, weights expect %u", input->dim0, K);
    if (out->dim0 != N || (out->dim1 ? out->dim1 : 1) != M)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: output is [%u, %u], expected [%u, %u]", out->dim0, out->dim1, N, M);
    if (w_gate->device != (uint32_t)ctx->device || w_up->device != (uint32_t)ctx->device ||
        input->device != (uint32_t)ctx->device || out->device != (uint32_t)ctx->device)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_gate_up: buffers belong to another device");
    const bool decode = (int)M <= ctx->gemv_max_m;
    if (decode && K > gemv_max_k())
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: in_features %u exceeds the supported maximum %zu", K, gemv_max_k());
    DeviceGuard guard(ctx->device);
    cudaError_t e;
    PerfScope perf(ctx, w_gate->dtype == LLMRS_Q4K ? "matmul_gate_up q4_k" : "matmul_gate_up q6_k",
                   2.0 * matmul_bytes(w_gate, input, out) - (double)K * M * dense_elem_bytes(input->dtype) - (double)N * M * dense_elem_bytes(out->dtype),
                   2.0 * matmul_flops(w_gate, input));
    if (decode && gemv_gate_up_fits((int)w_gate->dtype, (int)K, (int)M)) {
        e = ctx->begin_work();
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_gate_up: event");
        e = launch_gemv_gate_up((int)w_gate->dtype, (const uint8_t *)w_gate->dptr, (const uint8_t *)w_up->dptr,
                                input->dptr, (int)input->dtype, out->dptr, (int)out->dtype, (int)K, (int)N, (int)M,
                                ctx->sm_count, ctx->pdl, ctx->sink(), ctx->stream, &ctx->launches, ctx->norm_w,
                                ctx->norm_eps);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_gate_up: launch");
        return LLMRS_OK;
    }
    if (ctx->norm_w) return ctx->fail(LLMRS_ERR_SHAPE, "matmul_gate_up: the fused norm needs the one-launch path");
    // Two matmuls into float32 scratch behind the GEMM's own scratch, then the element-wise tail.
    const size_t gemm_bytes = decode ? 0 : (tc_scratch_bytes(ctx, K, M) + 255) / 256 * 256;
    const size_t half = ((size_t)M * N * sizeof(float) + 255) / 256 * 256;
    e = ctx->reserve_scratch(gemm_bytes + 2 * half);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_gate_up: scratch (grow it with one call outside graph capture)");
    float *g = (float *)((uint8_t *)ctx->scratch + gemm_bytes), *u = (float *)((uint8_t *)g + half);
    e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_gate_up: event");
    const llmrs_buf *ws[2] = {w_gate, w_up};
    float *dst[2] = {g, u};
    ActsShareScope share(ctx);
    llmrs_buf gbuf = *out, ubuf = *out;              // float32 stand-ins for the eligibility check
    gbuf.dtype = ubuf.dtype = LLMRS_F32;
    const llmrs_buf *tmp_outs[2] = {&gbuf, &ubuf};
    if (!decode && tc_matmul_multi_ok(ctx, 2, ws, tmp_outs, M)) {
        void *op[2] = {g, u};
        e = tc_matmul_multi(ctx, 2, ws, op, LLMRS_F32, input->dptr, input->dtype, K, M);
    } else
    for (int i = 0; i < 2 && e == cudaSuccess; i++) {
        if (decode)
            e = launch_gemv((int)ws[i]->dtype, (const uint8_t *)ws[i]->dptr, input->dptr, (int)input->dtype, dst[i],
                            DT_F32, (int)K, (int)N, (int)M, ctx->sm_count, ctx->pdl, ctx->sink(), ctx->stream,
                            &ctx->launches);
        else
            e = tc_matmul(ctx, ws[i]->dtype, ws[i]->dptr, input->dptr, input->dtype, dst[i], LLMRS_F32, K, N, M);
    }
    if (e == cudaSuccess) {
        e = launch_silu_mul(g, u, out->dptr, (int)out->dtype, (size_t)M * N, ctx->stream);
        ctx->launches++;
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_gate_up: launch");
    return LLMRS_OK;
}

int llmrs_cuda_embed(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *table, const uint32_t *tokens,
                     uint32_t n_tokens) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !table || !out->dptr || !table->dptr || (!tokens && n_tokens))
        return ctx->fail(LLMRS_ERR_ARG, "embed: null pointer");
    const bool dense_table = table->dtype == LLMRS_F32 || table->dtype == LLMRS_F16 || table->dtype == LLMRS_BF16;
    if (!dense_table && table->dtype != LLMRS_Q4K && table->dtype != LLMRS_Q6K)      // the reference's list: metal/mod.rs:852-859
        return ctx->fail(LLMRS_ERR_DTYPE, "embed: table dtype %u is not F32/F16/BF16/Q4_K/Q6_K", table->dtype);
    if (table->dtype == LLMRS_Q6K && table->layout != LLMRS_LAYOUT_Q6K_SLICES)
        return ctx->fail(LLMRS_ERR_ARG, "embed: table was not created by upload_tensor");
    if (!dense_elem_bytes(out->dtype)) return ctx->fail(LLMRS_ERR_DTYPE, "embed: output must be F32 or BF16");
    const uint32_t K = table->dim0, vocab = table->dim1 ? table->dim1 : 1;
    if (!dense_table && K % QK_K) return ctx->fail(LLMRS_ERR_SHAPE, "embed: dim %u is not a multiple of 256", K);
    if (out->dim0 != K || (out->dim1 ? out->dim1 : 1) != (n_tokens ? n_tokens : 1))
        return ctx->fail(LLMRS_ERR_SHAPE, "embed: output is [%u, %u], expected [%u, %u]", out->dim0, out->dim1, K, n_tokens);
    if (n_tokens > 65535) return ctx->fail(LLMRS_ERR_SHAPE, "embed: %u tokens in one call (at most 65535)", n_tokens);
    if (!dense_table && (reinterpret_cast<uintptr_t>(out->dptr) & 15)) return ctx->fail(LLMRS_ERR_ARG, "embed: output must be 16-byte aligned");
    if (table->device != (uint32_t)ctx->device || out->device != (uint32_t)ctx->device)
        return ctx->fail(LLMRS_ERR_ARG, "embed: buffers belong to another device");
    if (n_tokens == 0) return LLMRS_OK;
    for (uint32_t i = 0; i < n_tokens; i++)
        if (tokens[i] >= vocab)
            return ctx->fail(LLMRS_ERR_ARG, "embed: token %u is %u, the table has %u rows", i, tokens[i], vocab);
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaSuccess;
    if (n_tokens > ctx->tokens_cap) {            // grows outside stream capture only, like the scratch
        size_t have = ctx->tokens_cap * sizeof(uint32_t);
        e = ctx->grow((void **)&ctx->tokens, &have, (size_t)(n_tokens < 256 ? 256 : n_tokens) * sizeof(uint32_t));
        if (e == cudaErrorStreamCaptureUnsupported)
            return ctx->fail(LLMRS_ERR_CUDA, "embed: token buffer must grow (make one call outside graph capture)");
        if (e != cudaSuccess) return ctx->cuda_fail(e, "embed: token buffer");
        ctx->tokens_cap = have / sizeof(uint32_t);
    }
    e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "embed: event");
    size_t table_row_bytes = 0;
    storage_size(table->dtype, K, &table_row_bytes);
    PerfScope perf(ctx, "embed", (double)n_tokens * ((double)table_row_bytes + (double)K * dense_elem_bytes(out->dtype)), 0.0);
    e = cudaMemcpyAsync(ctx->tokens, tokens, (size_t)n_tokens * sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess && dense_table)
        e = launch_dense_embed((int)table->dtype, (const uint8_t *)table->dptr, (int)K, vocab, ctx->tokens, (int)n_tokens, out->dptr,
                               (int)out->dtype, ctx->dev_error, ctx->stream, false);
    else if (e == cudaSuccess)
        e = launch_embed((int)table->dtype, (const uint8_t *)table->dptr, (int)K, vocab, ctx->tokens, (int)n_tokens,
                         out->dptr, (int)out->dtype, ctx->dev_error, ctx->stream);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "embed: launch");
    ctx->launches++;
    return LLMRS_OK;
}

int llmrs_cuda_matmul_static_scratch(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight,
                                     const llmrs_buf *input) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !weight || !input || !out->dptr || !weight->dptr || !input->dptr)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_static_scratch: null buffer");
    const uint32_t K = weight->dim0, N = weight->dim1 ? weight->dim1 : 1, M = input->dim1 ? input->dim1 : 1;
    if (weight->dtype != LLMRS_Q4K && weight->dtype != LLMRS_Q6K)
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_static_scratch: weight dtype %u is not Q4_K/Q6_K", weight->dtype);
    const uint32_t want_layout = weight->dtype == LLMRS_Q6K ? LLMRS_LAYOUT_Q6K_SLICES : LLMRS_LAYOUT_RAW;
    if (weight->layout != want_layout)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_static_scratch: weight was not created by upload_tensor");
    if (!dense_elem_bytes(input->dtype) || !dense_elem_bytes(out->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_static_scratch: activations must be F32 or BF16");
    if (K % QK_K) return ctx->fail(LLMRS_ERR_SHAPE, "matmul_static_scratch: in_features %u is not a multiple of 256", K);
    if (input->dim0 != K)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_static_scratch: input has %u features, weight expects %u",
                         input->dim0, K);
    const uint32_t out_m = out->dim1 ? out->dim1 : 1;
    if (out->dim0 != N || out_m != M)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_static_scratch: output is [%u, %u], expected [%u, %u]", out->dim0,
                         out_m, N, M);
    if (weight->device != (uint32_t)ctx->device || input->device != (uint32_t)ctx->device ||
        out->device != (uint32_t)ctx->device)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_static_scratch: buffers belong to another device");
    const size_t need = tc_scratch_bytes(ctx, K, M), have = gemm_static_scratch_capacity();
    if (need > have)
        return ctx->fail(LLMRS_ERR_SHAPE,
                         "matmul_static_scratch: %u tokens x %u features need %zu bytes of scratch, the built-in "
                         "array holds %zu; use llmrs_cuda_matmul or fewer tokens per call",
                         M, K, need, have);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_static_scratch: event");
    PerfScope perf(ctx, "matmul_static_scratch", matmul_bytes(weight, input, out), matmul_flops(weight, input));
    e = launch_gemm_static_scratch((int)weight->dtype, (const uint8_t *)weight->dptr, input->dptr, (int)input->dtype,
                                   out->dptr, (int)out->dtype, (int)K, (int)N, (int)M, ctx->device, ctx->sink(),
                                   ctx->stream, &ctx->launches, ctx->two_term, uses_exact_kernel(ctx, M));
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_static_scratch: launch");
    return LLMRS_OK;
}

int llmrs_cuda_matmul_allgather(llmrs_ctx *ctx, llmrs_buf *out, const llmrs_buf *weight_shard,
                                const llmrs_buf *input, uint32_t rank, uint32_t world, void *const *peer_mailbox,
                                uint32_t *step_word) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!out || !weight_shard || !input || !out->dptr || !weight_shard->dptr || !input->dptr || !peer_mailbox ||
        !step_word)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_allgather: null pointer");
    const uint32_t K = weight_shard->dim0, N = weight_shard->dim1 ? weight_shard->dim1 : 1;
    const uint32_t M = input->dim1 ? input->dim1 : 1;
    if (weight_shard->dtype != LLMRS_Q4K && weight_shard->dtype != LLMRS_Q6K)
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_allgather: weight dtype %u is not Q4_K/Q6_K", weight_shard->dtype);
    if (weight_shard->dtype == LLMRS_Q6K && weight_shard->layout != LLMRS_LAYOUT_Q6K_SLICES)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_allgather: weight was not created by upload_tensor");
    if (!dense_elem_bytes(input->dtype) || !dense_elem_bytes(out->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "matmul_allgather: activations must be F32 or BF16");
    if (world < 1 || world > 8 || rank >= world)
        return ctx->fail(LLMRS_ERR_ARG, "matmul_allgather: rank %u of %u (at most 8 ranks)", rank, world);
    if (input->dim0 != K || K % QK_K || K > gemv_max_k())
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_allgather: input has %u features, weight expects %u", input->dim0, K);
    if ((uint64_t)N * world != out->dim0 || (out->dim1 ? out->dim1 : 1) != M)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_allgather: output is [%u, %u], expected [%u ranks x %u rows, %u]",
                         out->dim0, out->dim1, world, N, M);
    // up to gemv_max_m tokens, where one launch of the decode kernel holds them: exact kernel;
    // otherwise the tensor-core kernel, whose epilogue runs the same mailbox exchange
    const bool decode = (int)M <= ctx->gemv_max_m && (int)M <= gemv_single_launch_max_tokens((int)weight_shard->dtype, (int)K);
    if (!decode && M > LLMRS_ALLGATHER_MAX_TOKENS)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_allgather: %u tokens; the fused exchange serves at most %d "
                                          "(use matmul + a collective above that)", M, LLMRS_ALLGATHER_MAX_TOKENS);
    if (!decode && N % 8)
        return ctx->fail(LLMRS_ERR_SHAPE, "matmul_allgather: %u rows per rank; the tensor-core path needs a multiple of 8", N);
    for (uint32_t d = 0; d < world; d++)
        if (!peer_mailbox[d]) return ctx->fail(LLMRS_ERR_ARG, "matmul_allgather: null mailbox pointer");
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_allgather: event");
    PerfScope perf(ctx, "matmul_allgather", matmul_bytes(weight_shard, input, out), matmul_flops(weight_shard, input));
    if (decode) {
        e = launch_gemv_allgather((int)weight_shard->dtype, (const uint8_t *)weight_shard->dptr, input->dptr,
                                  (int)input->dtype, out->dptr, (int)out->dtype, (int)K, (int)N, (int)M, (int)rank,
                                  (int)world, peer_mailbox, ctx->dev_error + 1, step_word, ctx->sm_count, ctx->pdl,
                                  ctx->sink(), ctx->stream, &ctx->launches);
    } else {
        e = ctx->reserve_scratch(tc_scratch_bytes(ctx, K, M));
        if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_allgather: scratch (grow it with one call outside graph capture)");
        const GemmGather gg{(int)world, (int)rank, peer_mailbox, ctx->dev_error + 1, step_word};
        e = tc_matmul(ctx, weight_shard->dtype, weight_shard->dptr, input->dptr, input->dtype, out->dptr, out->dtype, K, N, M, &gg);
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "matmul_allgather: launch");
    return LLMRS_OK;
}

size_t llmrs_cuda_allgather_mailbox_bytes(uint32_t n_total, uint32_t tokens) {
    return gemv_allgather_mailbox_bytes((int)n_total, (int)tokens);
}

int llmrs_cuda_matmul_allgather_max_tokens(uint32_t weight_dtype, uint32_t in_features) {
    if ((weight_dtype != LLMRS_Q4K && weight_dtype != LLMRS_Q6K) || in_features == 0 || in_features % QK_K) return 0;
    return LLMRS_ALLGATHER_MAX_TOKENS;
}

int llmrs_cuda_dequantize(llmrs_ctx *ctx, const llmrs_buf *weight, float *dev_out) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!weight || !weight->dptr || !dev_out) return ctx->fail(LLMRS_ERR_ARG, "dequantize: null pointer");
    if (!is_kquant(weight->dtype) && !is_other_weight(weight->dtype))
        return ctx->fail(LLMRS_ERR_DTYPE, "dequantize: weight dtype %u is not supported", weight->dtype);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->begin_work();
    if (e == cudaSuccess && is_other_weight(weight->dtype)) {
        e = launch_dense_dequant((int)weight->dtype, (const uint8_t *)weight->dptr, (int)weight->dim0,
                                 (int)(weight->dim1 ? weight->dim1 : 1), dev_out, ctx->stream);
        ctx->launches++;
    } else if (e == cudaSuccess) {
        e = launch_dequant((int)weight->dtype, (const uint8_t *)weight->dptr, (int)weight->dim0,
                           (int)(weight->dim1 ? weight->dim1 : 1), dev_out, ctx->stream);
        ctx->launches++;
    }
    if (e != cudaSuccess) return ctx->cuda_fail(e, "dequantize");
    return LLMRS_OK;
}

int llmrs_cuda_sync(llmrs_ctx *ctx) {
    if (!ctx) return LLMRS_ERR_ARG;
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->finish_work();
    if (e != cudaSuccess) return ctx->cuda_fail(e, "sync");
    if (ctx->perf) {
        try { perf_flush(ctx); } catch (...) { ctx->perf_ops.clear(); }
    }
    return ctx->check_kernel_error("sync");
}

int llmrs_cuda_read_f32(llmrs_ctx *ctx, const llmrs_buf *buf, float *host, size_t n) {
    if (!ctx) return LLMRS_ERR_ARG;
    if (!buf || !buf->dptr || !host) return ctx->fail(LLMRS_ERR_ARG, "read_f32: null pointer");
    const size_t eb = dense_elem_bytes(buf->dtype);
    if (!eb) return ctx->fail(LLMRS_ERR_DTYPE, "read_f32: only F32/BF16 buffers");
    if (n * eb > buf->nbytes) return ctx->fail(LLMRS_ERR_SHAPE, "read_f32: %zu elements exceed the buffer", n);
    DeviceGuard guard(ctx->device);
    cudaError_t e = ctx->finish_work();           // readback forces completion (metal/mod.rs:980)
    if (e != cudaSuccess) return ctx->cuda_fail(e, "read_f32: sync");
    if (int rc = ctx->check_kernel_error("read_f32")) return rc;
    if (buf->dtype == LLMRS_F32) {
        e = cudaMemcpy(host, buf->dptr, n * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return ctx->cuda_fail(e, "read_f32: copy");
        return LLMRS_OK;
    }
    std::vector<uint16_t> tmp;
    try { tmp.resize(n); } catch (...) { return ctx->fail(LLMRS_ERR_ARG, "read_f32: out of host memory"); }
    e = cudaMemcpy(tmp.data(), buf->dptr, n * 2, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return ctx->cuda_fail(e, "read_f32: copy");
    for (size_t i = 0; i < n; i++) {              // bf16 -> f32 widening is exact (metal/mod.rs:985-990)
        uint32_t u = (uint32_t)tmp[i] << 16;
        memcpy(&host[i], &u, 4);
    }
    return LLMRS_OK;
}

int llmrs_cuda_gpu_secs_total(llmrs_ctx *ctx, double *secs) {
    if (!ctx || !secs) return LLMRS_ERR_ARG;
    *secs = ctx->gpu_secs;
    return LLMRS_OK;
}

int llmrs_cuda_reset_gpu_secs(llmrs_ctx *ctx) {
    if (!ctx) return LLMRS_ERR_ARG;
    ctx->gpu_secs = 0.0;
    return LLMRS_OK;
}

size_t llmrs_cuda_perf_table(llmrs_ctx *ctx, char *buf, size_t cap) {
    if (!ctx) return 0;
    const size_t n = ctx->perf_last.size();
    if (buf && cap) {
        const size_t k = n < cap - 1 ? n : cap - 1;
        memcpy(buf, ctx->perf_last.data(), k);
        buf[k] = 0;
    }
    return n;
}

int llmrs_cuda_launch_count(llmrs_ctx *ctx, uint64_t *count) {
    if (!ctx || !count) return LLMRS_ERR_ARG;
    *count = ctx->launches;
    return LLMRS_OK;
}

}  // extern "C"
