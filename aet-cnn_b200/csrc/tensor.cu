// Context (device, stream, scratch arena, status word, per-kernel profiling) and tensor
// containers with their host taps.  The host side of every tap speaks the reference's layout
// (FP32 NCHW, dnn/NData.h:14-68); device storage is NHWC padded to 4 channels, so a tap is one
// copy plus one transposing kernel.  Replaces MtcsMem / MtcsStream call sites
// (mtcs/MtcsTool.c:22-30, mtcs/MtcsIOData.c:15-52) and DataFactory.create*Data.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.h"

static thread_local char g_error[512] = "";

void aet_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char *aet_last_error(void) { return g_error; }
extern "C" const char *aet_version(void) { return "aet-cnn-b200 0.1 (sm_100a)"; }

namespace {

// NCHW (dense, c channels) <-> NHWC (cp channels); pad channels are written as zero.
__global__ void nchw_to_nhwc_kernel(const float *__restrict__ src, float *__restrict__ dst, int n, int c, int h, int w,
                                    int cp) {
    pdl_enter();
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n * h * w * cp;
    if (e >= total) return;
    const int ch = (int)(e % cp);
    size_t p = e / cp;
    const int x = (int)(p % w); p /= w;
    const int y = (int)(p % h);
    const int b = (int)(p / h);
    dst[e] = ch < c ? src[(((size_t)b * c + ch) * h + y) * w + x] : 0.f;
}
__global__ void nhwc_to_nchw_kernel(const float *__restrict__ src, float *__restrict__ dst, int n, int c, int h, int w,
                                    int cp) {
    pdl_enter();
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n * c * h * w;
    if (e >= total) return;
    const int x = (int)(e % w);
    size_t p = e / w;
    const int y = (int)(p % h); p /= h;
    const int ch = (int)(p % c);
    const int b = (int)(p / c);
    dst[e] = src[(((size_t)b * h + y) * w + x) * cp + ch];
}

}  // namespace

// ---------------------------------------------------------------------------- profiling
void prof_begin(aet_context *ctx, const char *name, double bytes, double flops, const char *variant) {
    if (ctx->event_next + 2 > ctx->event_pool.size()) {
        for (int i = 0; i < 256; ++i) {
            cudaEvent_t e;
            if (cudaEventCreate(&e) != cudaSuccess) return;
            ctx->event_pool.push_back(e);
        }
    }
    ProfileRecord r;
    r.span_slot = -1;
    if (ctx->span_dev && ctx->records.size() < (size_t)kMaxSpanSlots) {
        r.span_slot = (int)ctx->records.size();
        ctx->span_ptr = ctx->span_dev + 2 * (size_t)r.span_slot;
    }
    if (variant && *variant) snprintf(r.name, sizeof(r.name), "%s.%s", name, variant);
    else snprintf(r.name, sizeof(r.name), "%s", name);
    r.tag = ctx->prof_tag; r.bytes = bytes; r.flops = flops;
    r.e0 = ctx->event_pool[ctx->event_next++];
    r.e1 = ctx->event_pool[ctx->event_next++];
    cudaEventRecord(r.e0, ctx->stream);
    ctx->records.push_back(r);
}
void prof_end(aet_context *ctx) {
    if (!ctx->records.empty()) cudaEventRecord(ctx->records.back().e1, ctx->stream);
}

int ctx_smem_attr_impl(aet_context *ctx, const void *func, int bytes) {
    for (const void *f : ctx->smem_attr_done)
        if (f == func) return AET_OK;
    AET_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    ctx->smem_attr_done.push_back(func);
    return AET_OK;
}

namespace {
struct OptionDesc {
    const char *name, *env;
    int def;
    int env_value;   // value taken when the variable is set; -1: the variable's integer value
};
const OptionDesc kOptions[OPT_COUNT] = {
    {"rows", "AET_NO_ROWS", 1, 0},
    {"rows_fprop", "AET_ROWS_F", 0, 1},
    {"rows_dgrad", "AET_NO_ROWS_D", 1, 0},
    {"smerge", "AET_NO_SMERGE", 1, 0},
    {"ksplit", "AET_NO_KSPLIT", 1, 0},
    {"mt2", "AET_NO_MT2", 1, 0},
    {"rows_multi", "AET_ROWS_MULTI", 0, 1},
    {"par_epilogue", "AET_NO_PAR_EPILOGUE", 1, 0},
    {"fc_alias", "AET_NO_FC_ALIAS", 1, 0},
    {"epilogue_stats", "AET_NO_EPILOGUE_STATS", 1, 0},
    {"thin", "AET_NO_THIN", 1, 0},
    {"overlap_wgrad", "AET_NO_OVERLAP", 1, 0},
    {"wgrad_splits", "AET_WGRAD_SPLITS", 0, -1},
    {"bn_tile", "AET_BN", 0, -1},
    {"fuse", "AET_NO_FUSE", 1, 0},
    {"linear_head", "AET_NO_LINEAR_HEAD", 1, 0},
    {"xchg_cap_floats", "AET_XCHG_CAP_FLOATS", 0, -1},
    {"nccl_max_ctas", "AET_NCCL_MAX_CTAS", 0, -1},
    {"dual_acc", "AET_DUAL_ACC", 0, 1},
    {"rotate", "AET_NO_ROTATE", 1, 0},
    {"stem", "AET_NO_STEM", 1, 0},
    {"comm_stamps", "AET_COMM_STAMPS", 0, 1},
    {"merge_tail", "AET_NO_MERGE_TAIL", 1, 0},
    {"ragged", "AET_NO_RAGGED", 1, 0},
    {"pair", "AET_PAIR", 0, 1},
    {"s2d", "AET_NO_S2D", 1, 0},
    {"fd_split", "AET_NO_FD_SPLIT", 1, 0},
};
}  // namespace

extern "C" int aet_context_set_option(aet_context *ctx, const char *name, int value) {
    if (!ctx || !name) { aet_set_error("aet_context_set_option: null argument"); return AET_E_INVALID; }
    if (strcmp(name, "gather_only") == 0) { ctx->conv_path = value ? 1 : 0; return AET_OK; }
    for (int i = 0; i < OPT_COUNT; ++i)
        if (strcmp(kOptions[i].name, name) == 0) { ctx->opt[i] = value; return AET_OK; }
    aet_set_error("aet_context_set_option: unknown option '%s'", name);
    return AET_E_INVALID;
}
extern "C" int aet_context_get_option(const aet_context *ctx, const char *name, int *value) {
    if (!ctx || !name || !value) { aet_set_error("aet_context_get_option: null argument"); return AET_E_INVALID; }
    if (strcmp(name, "gather_only") == 0) { *value = ctx->conv_path; return AET_OK; }
    for (int i = 0; i < OPT_COUNT; ++i)
        if (strcmp(kOptions[i].name, name) == 0) { *value = ctx->opt[i]; return AET_OK; }
    aet_set_error("aet_context_get_option: unknown option '%s'", name);
    return AET_E_INVALID;
}

int ctx_scratch(aet_context *ctx, size_t bytes, float **out) {
    float *&buf = ctx->on_side ? ctx->scratch_side : ctx->scratch;
    size_t &have = ctx->on_side ? ctx->scratch_side_bytes : ctx->scratch_bytes;
    if (bytes > have) {
        if (ctx->capturing) {
            aet_set_error("scratch arena too small during graph capture (%zu > %zu)", bytes, have);
            return AET_E_NOMEM;
        }
        AET_CUDA(cudaStreamSynchronize(ctx->stream));
        if (buf) cudaFree(buf);
        buf = nullptr;
        have = 0;
        size_t want = round_up_sz(bytes + bytes / 4, 1 << 20);
        AET_CUDA(cudaMalloc(&buf, want));
        have = want;
    }
    *out = buf;
    return AET_OK;
}

int side_begin(aet_context *ctx) {
    if (!ctx->side_stream) {
        AET_CUDA(cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
        AET_CUDA(cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming));
        AET_CUDA(cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming));
    }
    AET_CUDA(cudaEventRecord(ctx->ev_fork, ctx->stream));
    AET_CUDA(cudaStreamWaitEvent(ctx->side_stream, ctx->ev_fork, 0));
    ctx->main_stream_saved = ctx->stream;
    ctx->stream = ctx->side_stream;
    ctx->on_side = true;
    ctx->side_pending = true;
    pdl_skip_next();   // the kernel after a cross-stream wait is launched plainly
    return AET_OK;
}

void side_end(aet_context *ctx) {
    if (!ctx->on_side) return;
    ctx->stream = ctx->main_stream_saved;
    ctx->on_side = false;
}

int side_join(aet_context *ctx) {
    side_end(ctx);
    if (!ctx->side_pending) return AET_OK;
    AET_CUDA(cudaEventRecord(ctx->ev_join, ctx->side_stream));
    AET_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_join, 0));
    ctx->side_pending = false;
    pdl_skip_next();
    return AET_OK;
}

int ctx_staging(aet_context *ctx, size_t bytes) {
    if (bytes > ctx->staging_bytes) {
        if (ctx->capturing) {
            aet_set_error("staging buffer too small during graph capture");
            return AET_E_NOMEM;
        }
        AET_CUDA(cudaStreamSynchronize(ctx->stream));
        if (ctx->staging) cudaFree(ctx->staging);
        if (ctx->pinned) cudaFreeHost(ctx->pinned);
        ctx->staging = nullptr; ctx->pinned = nullptr; ctx->staging_bytes = 0; ctx->pinned_bytes = 0;
        size_t want = round_up_sz(bytes, 1 << 20);
        AET_CUDA(cudaMalloc(&ctx->staging, want));
        AET_CUDA(cudaMallocHost(&ctx->pinned, want));
        ctx->staging_bytes = want;
        ctx->pinned_bytes = want;
    }
    return AET_OK;
}

// ---------------------------------------------------------------------------- context
extern "C" aet_context *aet_context_create(int device) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        aet_set_error("no CUDA device available (%s); this library has no CPU path", cudaGetErrorString(e));
        return nullptr;
    }
    if (device < 0 || device >= count) {
        aet_set_error("device %d out of range (0..%d)", device, count - 1);
        return nullptr;
    }
    if (cudaSetDevice(device) != cudaSuccess) {
        aet_set_error("cudaSetDevice(%d) failed", device);
        return nullptr;
    }
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, device);
    if (prop.major != 10) {
        aet_set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return nullptr;
    }
    aet_context *ctx = new aet_context();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        aet_set_error("cudaStreamCreate failed");
        delete ctx;
        return nullptr;
    }
    ctx->owns_stream = true;
    if (cudaMalloc(&ctx->status_dev, sizeof(int)) != cudaSuccess || cudaMemset(ctx->status_dev, 0, sizeof(int)) != cudaSuccess) {
        aet_set_error("status word allocation failed");
        delete ctx;
        return nullptr;
    }
    // the environment only supplies initial values, here and nowhere else
    for (int i = 0; i < OPT_COUNT; ++i) {
        ctx->opt[i] = kOptions[i].def;
        const char *e = getenv(kOptions[i].env);
        if (e && *e) ctx->opt[i] = kOptions[i].env_value >= 0 ? kOptions[i].env_value : atoi(e);
    }
    const char *path = getenv("AET_CONV_PATH");
    if (path && strcmp(path, "gather") == 0) ctx->conv_path = 1;
    return ctx;
}

extern "C" void aet_context_destroy(aet_context *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
    if (ctx->staging) cudaFree(ctx->staging);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->side_stream) {
        cudaStreamSynchronize(ctx->side_stream);
        cudaStreamDestroy(ctx->side_stream);
        cudaEventDestroy(ctx->ev_fork);
        cudaEventDestroy(ctx->ev_join);
    }
    if (ctx->scratch_side) cudaFree(ctx->scratch_side);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->span_dev) cudaFree(ctx->span_dev);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

extern "C" int aet_context_set_stream(aet_context *ctx, void *cuda_stream) {
    if (!ctx) { aet_set_error("null context"); return AET_E_INVALID; }
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    if (cuda_stream) {
        ctx->stream = static_cast<cudaStream_t>(cuda_stream);
        ctx->owns_stream = false;
    } else {
        AET_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        ctx->owns_stream = true;
    }
    return AET_OK;
}
extern "C" void *aet_context_stream(aet_context *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" int aet_context_set_parity(aet_context *ctx, aet_parity_mode mode) {
    if (!ctx || (mode != AET_PARITY_CPU && mode != AET_PARITY_MTCS)) { aet_set_error("bad parity mode"); return AET_E_INVALID; }
    ctx->parity = mode;
    return AET_OK;
}
extern "C" int aet_context_set_math(aet_context *ctx, aet_math_mode mode) {
    if (!ctx || (mode != AET_MATH_TF32 && mode != AET_MATH_3XTF32)) { aet_set_error("bad math mode"); return AET_E_INVALID; }
    ctx->math = mode;
    return AET_OK;
}
extern "C" int aet_context_synchronize(aet_context *ctx) {
    ctx_enter(ctx);
    if (!ctx) { aet_set_error("null context"); return AET_E_INVALID; }
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    return AET_OK;
}
extern "C" int aet_context_check(aet_context *ctx) {
    ctx_enter(ctx);
    if (!ctx) { aet_set_error("null context"); return AET_E_INVALID; }
    int st = 0;
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    AET_CUDA(cudaMemcpy(&st, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(ctx->status_dev, 0, sizeof(int));
        if (st & AET_STATUS_TIMEOUT) {
            aet_set_error("a bounded device-side wait expired (status %d)", st);
            return AET_E_TIMEOUT;
        }
        aet_set_error("non-finite values were found in weights or gradients and replaced as the reference's update does (status %d)", st);
        return AET_E_NAN;
    }
    return AET_OK;
}

extern "C" int aet_context_set_wait_limit(aet_context *ctx, unsigned long long nanoseconds) {
    if (!ctx || nanoseconds == 0) { aet_set_error("aet_context_set_wait_limit: bad argument"); return AET_E_INVALID; }
    AET_CUDA(cudaSetDevice(ctx->device));
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    AET_TRY(conv_set_wait_limit(nanoseconds));
    return elementwise_set_wait_limit(nanoseconds);
}

extern "C" int aet_context_wait_probe(aet_context *ctx) {
    ctx_enter(ctx);
    if (!ctx) { aet_set_error("null context"); return AET_E_INVALID; }
    return conv_wait_probe(ctx);
}

extern "C" int aet_context_profile(aet_context *ctx, int enable) {
    ctx_enter(ctx);
    if (!ctx) { aet_set_error("null context"); return AET_E_INVALID; }
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->profiling = enable != 0;
    ctx->records.clear();
    ctx->event_next = 0;
    ctx->span_ptr = nullptr;
    if (enable) {
        if (!ctx->span_dev) AET_CUDA(cudaMalloc(&ctx->span_dev, (size_t)kMaxSpanSlots * 2 * sizeof(unsigned long long)));
        std::vector<unsigned long long> init((size_t)kMaxSpanSlots * 2);
        for (int i = 0; i < kMaxSpanSlots; ++i) { init[2 * i] = ~0ull; init[2 * i + 1] = 0ull; }
        AET_CUDA(cudaMemcpy(ctx->span_dev, init.data(), init.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
    }
    return AET_OK;
}

extern "C" int aet_context_profile_read(aet_context *ctx, aet_kernel_time *table, int capacity, int *count) {
    ctx_enter(ctx);
    if (!ctx || !table || !count) { aet_set_error("null argument"); return AET_E_INVALID; }
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    std::vector<unsigned long long> spans;
    if (ctx->span_dev) {
        spans.resize((size_t)kMaxSpanSlots * 2);
        AET_CUDA(cudaMemcpy(spans.data(), ctx->span_dev, spans.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    }
    int n = 0;
    for (const ProfileRecord &r : ctx->records) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) continue;
        double span_ms = 0.0;
        if (r.span_slot >= 0 && !spans.empty()) {
            const unsigned long long t0 = spans[2 * (size_t)r.span_slot], t1 = spans[2 * (size_t)r.span_slot + 1];
            if (t0 != ~0ull && t1 > t0) span_ms = (double)(t1 - t0) * 1e-6;
        }
        char label[sizeof(table[0].name)];
        if (r.tag >= 0) snprintf(label, sizeof(label), "%s#%d", r.name, r.tag);   // kernels of a network carry their layer
        else snprintf(label, sizeof(label), "%s", r.name);
        int k = 0;
        for (; k < n; ++k)
            if (strcmp(table[k].name, label) == 0 && table[k].algo_bytes == r.bytes && table[k].algo_flops == r.flops) break;
        if (k == n) {
            if (n == capacity) continue;
            memset(&table[n], 0, sizeof(table[n]));
            strncpy(table[n].name, label, sizeof(table[n].name) - 1);
            table[n].algo_bytes = r.bytes;
            table[n].algo_flops = r.flops;
            ++n;
        }
        table[k].launches += 1;
        table[k].total_ms += ms;
        table[k].span_ms += span_ms;
    }
    *count = n;
    return AET_OK;
}

extern "C" long aet_context_launch_count(const aet_context *ctx) { return ctx ? ctx->launches : 0; }

// ---------------------------------------------------------------------------- layout taps
int tensor_upload_nchw(aet_context *ctx, float *dev_nhwc, const float *host, int n, int c, int h, int w, int cp,
                       bool async_pinned) {
    const size_t dense = (size_t)n * c * h * w;
    if (dense == 0) return AET_OK;
    AET_TRY(ctx_staging(ctx, dense * sizeof(float)));
    if (async_pinned) {
        // the pinned mirror is reused every step: wait for the previous upload to have left it
        AET_CUDA(cudaStreamSynchronize(ctx->stream));
        memcpy(ctx->pinned, host, dense * sizeof(float));
        AET_CUDA(cudaMemcpyAsync(ctx->staging, ctx->pinned, dense * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    } else {
        AET_CUDA(cudaMemcpyAsync(ctx->staging, host, dense * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    }
    const size_t total = (size_t)n * h * w * cp;
    ctx->launches++;
    launch_k(ctx->stream, (unsigned)((total + 255) / 256), 256, 0, nchw_to_nhwc_kernel, ctx->staging, dev_nhwc, n, c, h, w, cp);
    AET_TRY(aet_check_launch("nchw_to_nhwc"));
    if (!async_pinned) AET_CUDA(cudaStreamSynchronize(ctx->stream));
    return AET_OK;
}

// Transposes a dense NCHW image already resident in device memory into the NHWC tensor.
int tensor_upload_staged(aet_context *ctx, float *dev_nhwc, const float *dev_nchw, int n, int c, int h, int w, int cp,
                         cudaStream_t stream) {
    const size_t total = (size_t)n * h * w * cp;
    if (stream) pdl_skip_next();   // behind a copy on another stream: a plain launch
    else ctx->launches++;
    launch_k(stream ? stream : ctx->stream, (unsigned)((total + 255) / 256), 256, 0, nchw_to_nhwc_kernel, dev_nchw, dev_nhwc, n, c, h, w, cp);
    return aet_check_launch("nchw_to_nhwc");
}

int tensor_download_nchw(aet_context *ctx, const float *dev_nhwc, float *host, int n, int c, int h, int w, int cp) {
    const size_t dense = (size_t)n * c * h * w;
    if (dense == 0) return AET_OK;
    AET_TRY(ctx_staging(ctx, dense * sizeof(float)));
    ctx->launches++;
    launch_k(ctx->stream, (unsigned)((dense + 255) / 256), 256, 0, nhwc_to_nchw_kernel, dev_nhwc, ctx->staging, n, c, h, w, cp);
    AET_TRY(aet_check_launch("nhwc_to_nchw"));
    AET_CUDA(cudaMemcpyAsync(host, ctx->staging, dense * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    return AET_OK;
}

int tensor_download_nchw_int(aet_context *ctx, const int *dev_nhwc, int *host, int n, int c, int h, int w, int cp) {
    // the transposing kernel only moves 32-bit words
    return tensor_download_nchw(ctx, reinterpret_cast<const float *>(dev_nhwc), reinterpret_cast<float *>(host), n, c, h, w, cp);
}

int vector_upload(aet_context *ctx, float *dev, const float *host, size_t count) {
    AET_CUDA(cudaMemcpyAsync(dev, host, count * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    return AET_OK;
}
int vector_download(aet_context *ctx, const float *dev, float *host, size_t count) {
    AET_CUDA(cudaMemcpyAsync(host, dev, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AET_CUDA(cudaStreamSynchronize(ctx->stream));
    return AET_OK;
}

// ---------------------------------------------------------------------------- tensors
extern "C" aet_tensor *aet_tensor_create(aet_context *ctx, int batch, int c, int h, int w) {
    ctx_enter(ctx);
    if (!ctx || batch <= 0 || c <= 0 || h <= 0 || w <= 0) {
        aet_set_error("aet_tensor_create: bad shape %d x %d x %d x %d", batch, c, h, w);
        return nullptr;
    }
    aet_tensor *t = new aet_tensor();
    t->ctx = ctx; t->n = batch; t->c = c; t->h = h; t->w = w; t->cp = round_up(c, 4);
    if (cudaMalloc(&t->d, t->elems() * sizeof(float)) != cudaSuccess ||
        cudaMemsetAsync(t->d, 0, t->elems() * sizeof(float), ctx->stream) != cudaSuccess) {
        aet_set_error("aet_tensor_create: device allocation of %zu bytes failed", t->elems() * sizeof(float));
        cudaGetLastError();
        delete t;
        return nullptr;
    }
    return t;
}
extern "C" void aet_tensor_destroy(aet_tensor *t) {
    ctx_enter(t ? t->ctx : nullptr);
    if (!t) return;
    if (t->owns && t->d) {
        cudaStreamSynchronize(t->ctx->stream);
        cudaFree(t->d);
    }
    delete t;
}
extern "C" int aet_tensor_shape(const aet_tensor *t, int *batch, int *c, int *h, int *w) {
    if (!t) { aet_set_error("null tensor"); return AET_E_INVALID; }
    if (batch) *batch = t->n;
    if (c) *c = t->c;
    if (h) *h = t->h;
    if (w) *w = t->w;
    return AET_OK;
}
extern "C" size_t aet_tensor_count(const aet_tensor *t) { return t ? t->count() : 0; }
extern "C" int aet_tensor_write(aet_tensor *t, const float *host_nchw) {
    ctx_enter(t ? t->ctx : nullptr);
    if (!t || !host_nchw) { aet_set_error("aet_tensor_write: null argument"); return AET_E_INVALID; }
    return tensor_upload_nchw(t->ctx, t->d, host_nchw, t->n, t->c, t->h, t->w, t->cp, false);
}
extern "C" int aet_tensor_read(const aet_tensor *t, float *host_nchw) {
    ctx_enter(t ? t->ctx : nullptr);
    if (!t || !host_nchw) { aet_set_error("aet_tensor_read: null argument"); return AET_E_INVALID; }
    return tensor_download_nchw(t->ctx, t->d, host_nchw, t->n, t->c, t->h, t->w, t->cp);
}
extern "C" int aet_tensor_zero(aet_tensor *t) {
    ctx_enter(t ? t->ctx : nullptr);
    if (!t) { aet_set_error("null tensor"); return AET_E_INVALID; }
    AET_CUDA(cudaMemsetAsync(t->d, 0, t->elems() * sizeof(float), t->ctx->stream));
    return AET_OK;
}
