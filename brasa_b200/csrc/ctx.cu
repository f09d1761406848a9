// Device runtime: context, buffers, commands (the CUDA counterpart of crates/metal/src/runtime.rs).
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>

#include "brasa_internal.h"

int32_t brasa_fail(brasa_ctx *ctx, int32_t code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    return code;
}

int32_t brasa_check_cuda(brasa_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return BRASA_OK;
    int32_t code = e == cudaErrorMemoryAllocation ? BRASA_ENOMEM : BRASA_ECUDA;
    return brasa_fail(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

// The attribute belongs to a (device, kernel) pair of the process, and setting it replaces the earlier value. Two
// contexts on one device share it, so what has been granted is remembered per process and only ever raised: a context
// that asks for less than another one got never takes the larger grant away.
int32_t brasa_smem_optin(brasa_ctx *ctx, const void *fn, size_t bytes) {
    static std::mutex mu;
    static std::map<std::pair<int, const void *>, size_t> granted;
    std::lock_guard<std::mutex> lock(mu);
    size_t &have = granted[std::make_pair(ctx->device, fn)];
    if (have >= bytes) return BRASA_OK;
    BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
    BRASA_CUDA(ctx, cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    have = bytes;
    return BRASA_OK;
}

extern "C" {

int32_t brasa_ctx_create(int32_t device, brasa_ctx **out) {
    if (!out) return BRASA_EINVAL;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return BRASA_ECUDA;
    if (cudaSetDevice(device) != cudaSuccess) return BRASA_ECUDA;
    brasa_ctx *ctx = new brasa_ctx();
    ctx->device = device;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return BRASA_ECUDA;
    }
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, device);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaMalloc(&ctx->status, 256) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return BRASA_ENOMEM;
    }
    cudaMemset(ctx->status, 0, 256);
    const char *env = getenv("BRASA_PDL");
    if (env && env[0] == '0') ctx->pdl = false;
#ifdef BRASA_TRACE_BUILD
    env = getenv("BRASA_TRACE");
    if (env && env[0] == '1' && cudaMalloc(&ctx->gemv_trace, 65536) == cudaSuccess) cudaMemset(ctx->gemv_trace, 0, 65536);
#endif
    env = getenv("BRASA_GRAPH");
    if (env && env[0] == '0') ctx->graphs = false;
    env = getenv("BRASA_TOKEN_KERNEL");
    if (env && env[0] == '0') ctx->token_kernel = false;
    *out = ctx;
    return BRASA_OK;
}

void brasa_ctx_destroy(brasa_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (brasa_buf *b : ctx->bufs) {
        cudaFree(b->ptr);
        delete b;
    }
    cudaFree(ctx->gemv_partials);
    cudaFree(ctx->gemv_counters);
    cudaFree(ctx->argmax_scratch);
    cudaFree(ctx->gemm_part);
    cudaFree(ctx->kv_expand);
    cudaFree(ctx->gemm_counters);
    cudaFree(ctx->sample_scratch);
    cudaFree(ctx->gemv_trace);
    cudaFree(ctx->status);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *brasa_last_error(brasa_ctx *ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
int32_t brasa_ctx_device(brasa_ctx *ctx) { return ctx ? ctx->device : -1; }
void *brasa_ctx_stream(brasa_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int32_t brasa_ctx_mem_info(brasa_ctx *ctx, uint64_t *free_bytes, uint64_t *total_bytes) {
    if (!ctx) return BRASA_EINVAL;
    size_t f = 0, t = 0;
    BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
    BRASA_CUDA(ctx, cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return BRASA_OK;
}

uint64_t brasa_ctx_launch_count(brasa_ctx *ctx) { return ctx ? ctx->launches : 0; }

#ifdef BRASA_TRACE_BUILD
int32_t brasa_debug_gemv_trace(brasa_ctx *ctx, uint64_t out[16]) {
    if (!ctx || !out) return BRASA_EINVAL;
    BRASA_REQUIRE(ctx, ctx->gemv_trace, "tracing is off: create the context with BRASA_TRACE=1");
    BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    BRASA_CUDA(ctx, cudaMemcpy(out, ctx->gemv_trace, 128, cudaMemcpyDeviceToHost));
    return BRASA_OK;
}

int32_t brasa_debug_trace_read(brasa_ctx *ctx, uint64_t *out, uint32_t n) {
    if (!ctx || !out) return BRASA_EINVAL;
    BRASA_REQUIRE(ctx, ctx->gemv_trace && n <= 8192, "tracing is off (create the context with BRASA_TRACE=1) or more than 8192 words asked");
    BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    BRASA_CUDA(ctx, cudaMemcpy(out, ctx->gemv_trace, (size_t)n * 8, cudaMemcpyDeviceToHost));
    return BRASA_OK;
}

#endif

int32_t brasa_ctx_sync(brasa_ctx *ctx) {
    if (!ctx) return BRASA_EINVAL;
    BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    uint32_t st = 0;
    BRASA_CUDA(ctx, cudaMemcpy(&st, ctx->status, 4, cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(ctx->status, 0, 4);
        ++ctx->timeouts;
        if (ctx->gemm_counters) cudaMemset(ctx->gemm_counters, 0, GEMM_TC_COUNTERS * 4);  // a kernel that gave up may have left arrivals behind
        return brasa_fail(ctx, BRASA_ETIMEOUT, "a bounded device-side wait ran out (status %u)", st);
    }
    return BRASA_OK;
}

int32_t brasa_buf_alloc(brasa_ctx *ctx, uint64_t bytes, brasa_buf **out) {
    if (!ctx || !out) return BRASA_EINVAL;
    *out = nullptr;
    BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
    void *p = nullptr;
    uint64_t n = std::max<uint64_t>(bytes, 16);
    cudaError_t e = cudaMalloc(&p, n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return brasa_fail(ctx, BRASA_ENOMEM, "cudaMalloc(%llu bytes): %s", (unsigned long long)n, cudaGetErrorString(e));
    }
    e = cudaMemsetAsync(p, 0, n, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return brasa_check_cuda(ctx, e, "cudaMemsetAsync");
    }
    brasa_buf *b = new brasa_buf{ctx, p, bytes};
    ctx->bufs.push_back(b);
    *out = b;
    return BRASA_OK;
}

int32_t brasa_buf_free(brasa_buf *buf) {
    if (!buf) return BRASA_EINVAL;
    brasa_ctx *ctx = buf->ctx;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    auto it = std::find(ctx->bufs.begin(), ctx->bufs.end(), buf);
    if (it != ctx->bufs.end()) ctx->bufs.erase(it);
    cudaFree(buf->ptr);
    delete buf;
    return BRASA_OK;
}

int32_t brasa_buf_upload(brasa_buf *buf, uint64_t offset, const void *src, uint64_t n) {
    if (!buf || (!src && n)) return BRASA_EINVAL;
    brasa_ctx *ctx = buf->ctx;
    BRASA_REQUIRE(ctx, offset <= buf->bytes && n <= buf->bytes - offset, "upload of %llu bytes at %llu exceeds the buffer (%llu)",
                  (unsigned long long)n, (unsigned long long)offset, (unsigned long long)buf->bytes);
    if (n == 0) return BRASA_OK;
    BRASA_CUDA(ctx, cudaMemcpyAsync((uint8_t *)buf->ptr + offset, src, n, cudaMemcpyHostToDevice, ctx->stream));
    BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BRASA_OK;
}

int32_t brasa_buf_download(brasa_buf *buf, uint64_t offset, void *dst, uint64_t n) {
    if (!buf || (!dst && n)) return BRASA_EINVAL;
    brasa_ctx *ctx = buf->ctx;
    BRASA_REQUIRE(ctx, offset <= buf->bytes && n <= buf->bytes - offset, "download of %llu bytes at %llu exceeds the buffer (%llu)",
                  (unsigned long long)n, (unsigned long long)offset, (unsigned long long)buf->bytes);
    if (n == 0) return BRASA_OK;
    BRASA_CUDA(ctx, cudaMemcpyAsync(dst, (uint8_t *)buf->ptr + offset, n, cudaMemcpyDeviceToHost, ctx->stream));
    BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BRASA_OK;
}

int32_t brasa_buf_fill(brasa_buf *buf, uint64_t offset, int32_t byte, uint64_t n) {
    if (!buf) return BRASA_EINVAL;
    brasa_ctx *ctx = buf->ctx;
    BRASA_REQUIRE(ctx, offset <= buf->bytes && n <= buf->bytes - offset, "fill exceeds the buffer");
    if (n == 0) return BRASA_OK;
    BRASA_CUDA(ctx, cudaMemsetAsync((uint8_t *)buf->ptr + offset, byte, n, ctx->stream));
    return BRASA_OK;
}

uint64_t brasa_buf_bytes(brasa_buf *buf) { return buf ? buf->bytes : 0; }
void *brasa_buf_ptr(brasa_buf *buf) { return buf ? buf->ptr : nullptr; }

int32_t brasa_cmd_begin(brasa_ctx *ctx, brasa_cmd **out) {
    if (!ctx || !out) return BRASA_EINVAL;
    *out = nullptr;
    BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
    brasa_cmd *c = new brasa_cmd{ctx, nullptr, nullptr, false};
    if (cudaEventCreate(&c->start) != cudaSuccess || cudaEventCreate(&c->end) != cudaSuccess) {
        delete c;
        return brasa_fail(ctx, BRASA_ECUDA, "cudaEventCreate failed");
    }
    cudaEventRecord(c->start, ctx->stream);
    *out = c;
    return BRASA_OK;
}

int32_t brasa_cmd_commit(brasa_cmd *cmd) {
    if (!cmd) return BRASA_EINVAL;
    if (!cmd->committed) {
        BRASA_CUDA(cmd->ctx, cudaEventRecord(cmd->end, cmd->ctx->stream));
        cmd->committed = true;
    }
    return BRASA_OK;
}

int32_t brasa_cmd_wait(brasa_cmd *cmd, double *gpu_seconds) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    int32_t rc = brasa_cmd_commit(cmd);
    if (rc == BRASA_OK) rc = brasa_check_cuda(ctx, cudaEventSynchronize(cmd->end), "cudaEventSynchronize");
    if (rc == BRASA_OK) {
        float ms = 0;
        cudaEventElapsedTime(&ms, cmd->start, cmd->end);
        if (gpu_seconds) *gpu_seconds = ms * 1e-3;
        uint32_t st = 0;
        cudaMemcpy(&st, ctx->status, 4, cudaMemcpyDeviceToHost);
        if (st != 0) {
            cudaMemset(ctx->status, 0, 4);
            ++ctx->timeouts;
            if (ctx->gemm_counters) cudaMemset(ctx->gemm_counters, 0, GEMM_TC_COUNTERS * 4);
            rc = brasa_fail(ctx, BRASA_ETIMEOUT, "a bounded device-side wait ran out (status %u)", st);
        }
    }
    cudaEventDestroy(cmd->start);
    cudaEventDestroy(cmd->end);
    delete cmd;
    return rc;
}

// ---- CUDA graphs: record the kernels enqueued between begin and end, replay them with one launch ----

int32_t brasa_graph_capture_begin(brasa_ctx *ctx) {
    if (!ctx) return BRASA_EINVAL;
    BRASA_REQUIRE(ctx, !ctx->capturing, "a capture is already open on this context");
    BRASA_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->capture_launches = 0;
    return BRASA_OK;
}

int32_t brasa_graph_capture_end(brasa_ctx *ctx, brasa_graph **out) {
    if (!ctx || !out) return BRASA_EINVAL;
    *out = nullptr;
    BRASA_REQUIRE(ctx, ctx->capturing, "no capture is open on this context");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    BRASA_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    BRASA_CUDA(ctx, e);
    *out = new brasa_graph{ctx, exec, ctx->capture_launches};
    return BRASA_OK;
}

int32_t brasa_graph_launch(brasa_cmd *cmd, brasa_graph *graph) {
    if (!cmd || !graph || graph->ctx != cmd->ctx) return BRASA_EINVAL;
    BRASA_CUDA(cmd->ctx, cudaGraphLaunch(graph->exec, cmd->ctx->stream));
    cmd->ctx->launches += graph->kernels;
    return BRASA_OK;
}

void brasa_graph_free(brasa_graph *graph) {
    if (!graph) return;
    cudaGraphExecDestroy(graph->exec);
    delete graph;
}

// ---- helpers ------------------------------------------------------------------------------------

uint64_t brasa_decode_partials_len(uint32_t hq, uint32_t lk) {
    return (uint64_t)hq * ((lk + BRASA_DECODE_CHUNK - 1) / BRASA_DECODE_CHUNK) * 130;
}
uint32_t brasa_norm_partials(uint32_t n) { return (n + BRASA_NORM_PREP_TG - 1) / BRASA_NORM_PREP_TG; }
int32_t brasa_gqa_supported(uint32_t hq, uint32_t hkv) {
    if (hkv == 0 || hq % hkv != 0) return 0;
    uint32_t g = hq / hkv;
    return g == 1 || g == 2 || g == 4 || g == 8;
}
uint64_t brasa_kv_bytes(int32_t kv, uint64_t n) {
    switch (kv) {
    case BRASA_KV_F32: return n * 4;
    case BRASA_KV_F16: return n * 2;
    case BRASA_KV_Q8_0: return n / BRASA_KV_Q8_DIM * BRASA_KV_Q8_ROW;
    default: return 0;
    }
}
uint64_t brasa_qtype_nbytes(int32_t q, uint64_t n) {
    switch (q) {
    case BRASA_Q4_0: return n / 32 * 18;
    case BRASA_Q8_0: return n / 32 * 34;
    case BRASA_Q6_0: return n / 32 * 26;
    default: return 0;
    }
}
int32_t brasa_rope_table(double theta, uint32_t dim, uint32_t max_pos, float *cos_out, float *sin_out) {
    if (!cos_out || !sin_out || dim == 0 || dim % 2) return BRASA_EINVAL;
    uint32_t half = dim / 2;
    std::vector<double> inv(half);
    for (uint32_t i = 0; i < half; ++i) inv[i] = 1.0 / pow(theta, (double)(2 * i) / (double)dim);
    for (uint32_t p = 0; p < max_pos; ++p)
        for (uint32_t i = 0; i < half; ++i) {
            double a = (double)p * inv[i];
            cos_out[(size_t)p * half + i] = (float)cos(a);
            sin_out[(size_t)p * half + i] = (float)sin(a);
        }
    return BRASA_OK;
}

}  // extern "C"

int32_t brasa_post_launch(brasa_cmd *cmd, const char *name) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return brasa_fail(cmd->ctx, BRASA_ECUDA, "launch of %s: %s", name, cudaGetErrorString(e));
    if (cmd->ctx->capturing) cmd->ctx->capture_launches += 1;
    else cmd->ctx->launches += 1;
    return BRASA_OK;
}

int32_t brasa_gemv_scratch(brasa_ctx *ctx, size_t partial_floats, size_t counters) {
    if (partial_floats > ctx->gemv_partials_floats) {
        BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->gemv_partials);
        ctx->gemv_partials = nullptr;
        ctx->gemv_partials_floats = 0;
        BRASA_CUDA(ctx, cudaMalloc(&ctx->gemv_partials, partial_floats * sizeof(float)));
        ctx->gemv_partials_floats = partial_floats;
    }
    if (counters > ctx->gemv_counters_n) {
        BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->gemv_counters);
    cudaFree(ctx->argmax_scratch);
    cudaFree(ctx->gemm_part);
    cudaFree(ctx->kv_expand);
    cudaFree(ctx->gemm_counters);
    cudaFree(ctx->sample_scratch);
    cudaFree(ctx->gemv_trace);
        ctx->gemv_counters = nullptr;
        ctx->gemv_counters_n = 0;
        BRASA_CUDA(ctx, cudaMalloc(&ctx->gemv_counters, counters * sizeof(uint32_t)));
        BRASA_CUDA(ctx, cudaMemset(ctx->gemv_counters, 0, counters * sizeof(uint32_t)));
        ctx->gemv_counters_n = counters;
    }
    return BRASA_OK;
}
