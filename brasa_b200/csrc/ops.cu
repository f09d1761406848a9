// Element-wise, normalisation, RoPE, embedding and KV-store kernels
// (crates/kernels/src/lib.rs:391-658, 976-1050 and the MSL files they dispatch).
#include "brasa_internal.h"

namespace {

__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

__global__ void add_kernel(const float *a, const float *b, float *out, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

template <bool HALF_OUT>
__global__ void swiglu_kernel(const float *g, const float *u, void *out, uint64_t n) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = silu_mul(g[i], u[i]);
    if (HALF_OUT) reinterpret_cast<__half *>(out)[i] = __float2half_rn(v);
    else reinterpret_cast<float *>(out)[i] = v;
}

__device__ float block_reduce_sum(float v, float *red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];
    __syncthreads();
    return t;
}
__device__ float block_reduce_max(float v, float *red) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; ++i) t = fmaxf(t, red[i]);
    __syncthreads();
    return t;
}

// out = x * (1 / sqrt(mean(x^2) + eps)) * w, one block per row
template <bool HALF_OUT>
__global__ void rms_norm_kernel(const float *x, const float *w, void *out, uint32_t n, float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (launched as a programmatic dependent: see brasa_launch_dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float red[32];
    const float *xr = x + (size_t)blockIdx.x * n;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
    ss = block_reduce_sum(ss, red);
    float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i] * scale * w[i];
        if (HALF_OUT) reinterpret_cast<__half *>(out)[(size_t)blockIdx.x * n + i] = __float2half_rn(v);
        else reinterpret_cast<float *>(out)[(size_t)blockIdx.x * n + i] = v;
    }
}

// The same with one warp per row and the row held in registers (n a multiple of 128, at most 128 * RMS_MAX_CHUNKS):
// one pass over x with 16-byte loads, no shared memory, two rows per block. Used for many rows (prefill, batch steps).
constexpr int RMS_MAX_CHUNKS = 20;
template <bool HALF_OUT>
__global__ void __launch_bounds__(64) rms_norm_rows_kernel(const float *x, const float *w, void *out, uint32_t rows, uint32_t n, float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (launched as a programmatic dependent: see brasa_launch_dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t row = blockIdx.x * 2 + (threadIdx.x >> 5), lane = threadIdx.x & 31, chunks = n / 128;
    if (row >= rows) return;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * n);
    float4 v[RMS_MAX_CHUNKS];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < RMS_MAX_CHUNKS; ++c) {
        if (c < (int)chunks) {
            v[c] = xr[c * 32 + lane];
            ss += (v[c].x * v[c].x + v[c].y * v[c].y) + (v[c].z * v[c].z + v[c].w * v[c].w);
        }
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    const float4 *wr = reinterpret_cast<const float4 *>(w);
#pragma unroll
    for (int c = 0; c < RMS_MAX_CHUNKS; ++c) {
        if (c < (int)chunks) {
            const float4 ww = wr[c * 32 + lane];
            const float a = v[c].x * scale * ww.x, b = v[c].y * scale * ww.y, cc = v[c].z * scale * ww.z, d = v[c].w * scale * ww.w;
            if (HALF_OUT) {
                const __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(cc, d);
                reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(out) + (size_t)row * n)[c * 32 + lane] =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
            } else {
                reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)row * n)[c * 32 + lane] = make_float4(a, b, cc, d);
            }
        }
    }
}

// One block of 128 threads per row, the row in registers (n a multiple of 512, at most 512 * RMS_BLOCK_CHUNKS): one pass with
// 16-byte loads and one block barrier. For few rows (a decode step of a batch), where the row count cannot hide latency.
constexpr int RMS_BLOCK_CHUNKS = 10;
template <bool HALF_OUT>
__global__ void __launch_bounds__(128) rms_norm_block_kernel(const float *x, const float *w, void *out, uint32_t n, float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (launched as a programmatic dependent: see brasa_launch_dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float red[4];
    const uint32_t t = threadIdx.x, chunks = n / 512;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)blockIdx.x * n);
    float4 v[RMS_BLOCK_CHUNKS];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < RMS_BLOCK_CHUNKS; ++c) {
        if (c < (int)chunks) {
            v[c] = xr[c * 128 + t];
            ss += (v[c].x * v[c].x + v[c].y * v[c].y) + (v[c].z * v[c].z + v[c].w * v[c].w);
        }
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((t & 31) == 0) red[t >> 5] = ss;
    __syncthreads();
    ss = (red[0] + red[1]) + (red[2] + red[3]);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    const float4 *wr = reinterpret_cast<const float4 *>(w);
#pragma unroll
    for (int c = 0; c < RMS_BLOCK_CHUNKS; ++c) {
        if (c < (int)chunks) {
            const float4 ww = wr[c * 128 + t];
            const float a = v[c].x * scale * ww.x, b = v[c].y * scale * ww.y, cc = v[c].z * scale * ww.z, d = v[c].w * scale * ww.w;
            if (HALF_OUT) {
                const __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(cc, d);
                reinterpret_cast<uint2 *>(reinterpret_cast<__half *>(out) + (size_t)blockIdx.x * n)[c * 128 + t] =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
            } else {
                reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + (size_t)blockIdx.x * n)[c * 128 + t] = make_float4(a, b, cc, d);
            }
        }
    }
}

__global__ void softmax_kernel(const float *x, float *out, uint32_t n) {
    __shared__ float red[32];
    const float *xr = x + (size_t)blockIdx.x * n;
    float m = -INFINITY;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, xr[i]);
    m = block_reduce_max(m, red);
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s += expf(xr[i] - m);
    s = block_reduce_sum(s, red);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = expf(xr[i] - m) / s;
}

// x: [tokens, heads, dim]; pairs (i, i + dim/2); grid over tokens*heads*dim/2
__global__ void rope_kernel(float *x, const float *cos_t, const float *sin_t, uint32_t tokens, uint32_t heads, uint32_t dim, uint32_t pos0) {
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t half = dim / 2;
    if (idx >= (uint64_t)tokens * heads * half) return;
    uint32_t i = idx % half;
    uint64_t th = idx / half;
    uint32_t t = (uint32_t)(th / heads);
    float *v = x + th * dim;
    float c = cos_t[(size_t)(pos0 + t) * half + i], s = sin_t[(size_t)(pos0 + t) * half + i];
    float a = v[i], b = v[i + half];
    v[i] = a * c - b * s;
    v[i + half] = b * c + a * s;
}

// Embedding gather: one thread per element. Handles q6_0 / q8_0 in the file layout and q6_0 tiled.
template <int QT, bool TILED>
__global__ void embed_kernel(const uint8_t *table, const uint32_t *ids, float *out, uint32_t h, uint32_t tokens, uint32_t vocab) {
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)tokens * h) return;
    uint32_t t = (uint32_t)(idx / h), col = (uint32_t)(idx % h);
    uint32_t r = ids[t];
    if (r >= vocab) { out[idx] = 0.0f; return; }
    uint32_t nb = h / 32, b = col / 32, j = col % 32;
    float d;
    int q;
    if (!TILED) {
        constexpr int BB = QT == BRASA_Q6_0 ? 26 : 34;
        const uint8_t *p = table + ((size_t)r * nb + b) * BB;
        d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(p)));
        if (QT == BRASA_Q8_0) q = (int8_t)p[2 + j];
        else {
            int ql = p[2 + (j & 15)];
            int lo = j < 16 ? (ql & 15) : (ql >> 4);
            int hi = (p[18 + (j & 7)] >> (2 * (j >> 3))) & 3;
            q = (lo | (hi << 4)) - 32;
        }
    } else {
        const uint8_t *row = table + (size_t)r * tiled_row_bytes(BRASA_Q6_0, h);
        const uint8_t *codes = row + b * 16;
        const uint32_t *hw = reinterpret_cast<const uint32_t *>(row + tiled_hi_off(h) + b * 8);
        d = __half2float(*reinterpret_cast<const __half *>(row + tiled_scale_off(BRASA_Q6_0, h) + b * 2));
        int byte = codes[j & 15];
        int lo = j < 16 ? (byte & 15) : (byte >> 4);
        // element j lives in code word w = (j & 15) / 4 as nibble k = 2 * (j & 3) + (j >= 16)
        int w = (j & 15) >> 2, k = 2 * (j & 3) + (j >> 4);
        int hi = (hw[w >> 1] >> q6_hi_bitpos(w & 1, k)) & 3;
        q = (lo | (hi << 4)) - 32;
    }
    out[idx] = d * (float)q;
}

// x += h (optional); xw = x*w; ss[block] = sum of x^2 over this block's 256 elements
__global__ void add_norm_prep_kernel(float *x, const float *h, const float *w, float *xw, float *ss, uint32_t n, int add) {
    __shared__ float red[8];
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    float v = 0.0f;
    if (i < n) {
        v = x[i];
        if (add) { v += h[i]; x[i] = v; }
        xw[i] = v * w[i];
    }
    float s = block_reduce_sum(v * v, red);
    if (threadIdx.x == 0) ss[blockIdx.x] = s;
}

__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Writes the value of element (lane + 32 j) of cache row `row` in the cache's type. For Q8 the 32
// lanes with the same j are one quantisation block (crates/quant/src/qtype.rs:89-111).
template <int KV>
__device__ __forceinline__ void store_elem(uint8_t *cache, size_t row, float v, int lane, int j) {
    if (KV == BRASA_KV_Q8_0) {
        float amax = warp_max(fabsf(v));
        __half dh = __float2half_rn(__fdiv_rn(amax, 127.0f));
        float d = __half2float(dh);
        float q = d == 0.0f ? 0.0f : fminf(fmaxf(rintf(__fdiv_rn(v, d)), -127.0f), 127.0f);
        uint8_t *r = cache + row * BRASA_KV_Q8_ROW;
        reinterpret_cast<int8_t *>(r)[lane + 32 * j] = (int8_t)q;
        if (lane == 0) reinterpret_cast<__half *>(r + 128)[j] = dh;
    } else if (KV == BRASA_KV_F16) {
        reinterpret_cast<__half *>(cache)[row * 128 + lane + 32 * j] = __float2half_rn(v);
    } else {
        reinterpret_cast<float *>(cache)[row * 128 + lane + 32 * j] = v;
    }
}

// One warp per row of 128: rows of a token are hq query heads, then hkv key heads, then hkv value heads.
template <int KV>
__global__ void qk_norm_rope_store_kernel(float *q, float *k, const float *v, const float *q_norm, const float *k_norm, const float *cos_t,
                                          const float *sin_t, uint8_t *kc, uint8_t *vc, uint32_t hq, uint32_t hkv, uint32_t pos0, float eps,
                                          uint32_t rows) {
    uint32_t gr = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (gr >= rows) return;
    uint32_t per_tok = hq + 2 * hkv, t = gr / per_tok, r = gr % per_tok;
    if (r >= hq + hkv) {
        size_t vh = (size_t)t * hkv + (r - hq - hkv);
        for (int j = 0; j < 4; ++j) store_elem<KV>(vc, vh, v[vh * 128 + lane + 32 * j], lane, j);
        return;
    }
    bool is_q = r < hq;
    size_t idx = is_q ? (size_t)t * hq + r : (size_t)t * hkv + (r - hq);
    float *x = (is_q ? q : k) + idx * 128;
    const float *w = is_q ? q_norm : k_norm;
    float xv[4], ss = 0.0f;
    for (int j = 0; j < 4; ++j) {
        xv[j] = x[lane + 32 * j];
        ss += xv[j] * xv[j];
    }
    ss = warp_sum(ss);
    float scale = 1.0f / sqrtf(ss / 128.0f + eps);
    float y[4];
    for (int j = 0; j < 4; ++j) y[j] = xv[j] * scale * w[lane + 32 * j];
    uint32_t pos = pos0 + t;
    for (int j = 0; j < 2; ++j) {
        int i = lane + 32 * j;
        float c = cos_t[(size_t)pos * 64 + i], s = sin_t[(size_t)pos * 64 + i];
        float a = y[j], b = y[j + 2];
        y[j] = a * c - b * s;
        y[j + 2] = b * c + a * s;
    }
    for (int j = 0; j < 4; ++j) {
        x[lane + 32 * j] = y[j];
        if (!is_q) store_elem<KV>(kc, idx, y[j], lane, j);
    }
}

// store_kv: f32 copy, f16 RNE, or Q8 rows (one warp per 32-value block)
__global__ void store_kv_plain_kernel(const float *src, void *dst, uint64_t n, int half_out) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (half_out) reinterpret_cast<__half *>(dst)[i] = __float2half_rn(src[i]);
    else reinterpret_cast<float *>(dst)[i] = src[i];
}
__global__ void store_kv_q8_kernel(const float *src, uint8_t *dst, uint64_t nblocks) {
    uint64_t blk = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    uint64_t row = blk / 4;
    int j = (int)(blk % 4);
    float v = src[blk * 32 + lane];
    float amax = warp_max(fabsf(v));
    __half dh = __float2half_rn(__fdiv_rn(amax, 127.0f));
    float d = __half2float(dh);
    float q = d == 0.0f ? 0.0f : fminf(fmaxf(rintf(__fdiv_rn(v, d)), -127.0f), 127.0f);
    uint8_t *r = dst + row * BRASA_KV_Q8_ROW;
    reinterpret_cast<int8_t *>(r)[32 * j + lane] = (int8_t)q;
    if (lane == 0) reinterpret_cast<__half *>(r + 128)[j] = dh;
}

inline unsigned blocks_for(uint64_t n, unsigned per) { return (unsigned)((n + per - 1) / per); }

}  // namespace

extern "C" {

int32_t brasa_k_add(brasa_cmd *cmd, brasa_arg a, brasa_arg b, brasa_arg out, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(a, n * 4) && arg_fits(b, n * 4) && arg_fits(out, n * 4), "add: buffers shorter than n");
    if (n == 0) return BRASA_OK;
    add_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>((const float *)arg_ptr(a), (const float *)arg_ptr(b), (float *)arg_ptr(out), n);
    return brasa_post_launch(cmd, "add");
}

int32_t brasa_k_swiglu(brasa_cmd *cmd, brasa_arg gate, brasa_arg up, brasa_arg out, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(gate, n * 4) && arg_fits(up, n * 4) && arg_fits(out, n * 4), "swiglu: buffers shorter than n");
    if (n == 0) return BRASA_OK;
    swiglu_kernel<false><<<blocks_for(n, 256), 256, 0, ctx->stream>>>((const float *)arg_ptr(gate), (const float *)arg_ptr(up), arg_ptr(out), n);
    return brasa_post_launch(cmd, "swiglu");
}

int32_t brasa_k_swiglu_f16(brasa_cmd *cmd, brasa_arg gate, brasa_arg up, brasa_arg out, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(gate, n * 4) && arg_fits(up, n * 4) && arg_fits(out, n * 2), "swiglu_f16: buffers shorter than n");
    if (n == 0) return BRASA_OK;
    swiglu_kernel<true><<<blocks_for(n, 256), 256, 0, ctx->stream>>>((const float *)arg_ptr(gate), (const float *)arg_ptr(up), arg_ptr(out), n);
    return brasa_post_launch(cmd, "swiglu_f16");
}

static int32_t rms_norm_common(brasa_cmd *cmd, brasa_arg x, brasa_arg w, brasa_arg out, uint32_t rows, uint32_t n, float eps, bool half_out) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    uint64_t tot = (uint64_t)rows * n;
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(x, tot * 4) && arg_fits(w, (uint64_t)n * 4) && arg_fits(out, tot * (half_out ? 2 : 4)), "rms_norm: buffers too small");
    if (rows == 0) return BRASA_OK;
    if (rows >= 256 && n % 128 == 0 && n <= 128 * RMS_MAX_CHUNKS && x.offset % 16 == 0 && w.offset % 16 == 0 && out.offset % 16 == 0) {
        const unsigned blocks = (rows + 1) / 2;
        if (half_out) BRASA_CUDA(ctx, brasa_launch_dependent(ctx, rms_norm_rows_kernel<true>, dim3(blocks), dim3(64), 0, (const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), rows, n, eps));
        else BRASA_CUDA(ctx, brasa_launch_dependent(ctx, rms_norm_rows_kernel<false>, dim3(blocks), dim3(64), 0, (const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), rows, n, eps));
        return brasa_post_launch(cmd, "rms_norm");
    }
    if (rows >= 2 && n % 512 == 0 && n <= 512 * RMS_BLOCK_CHUNKS && x.offset % 16 == 0 && w.offset % 16 == 0 && out.offset % 16 == 0) {
        if (half_out) BRASA_CUDA(ctx, brasa_launch_dependent(ctx, rms_norm_block_kernel<true>, dim3(rows), dim3(128), 0, (const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), n, eps));
        else BRASA_CUDA(ctx, brasa_launch_dependent(ctx, rms_norm_block_kernel<false>, dim3(rows), dim3(128), 0, (const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), n, eps));
        return brasa_post_launch(cmd, "rms_norm");
    }
    unsigned threads = n >= 1024 ? 256 : (n >= 256 ? 128 : 32);
    if (half_out) rms_norm_kernel<true><<<rows, threads, 0, ctx->stream>>>((const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), n, eps);
    else rms_norm_kernel<false><<<rows, threads, 0, ctx->stream>>>((const float *)arg_ptr(x), (const float *)arg_ptr(w), arg_ptr(out), n, eps);
    return brasa_post_launch(cmd, "rms_norm");
}
int32_t brasa_k_rms_norm(brasa_cmd *cmd, brasa_arg x, brasa_arg w, brasa_arg out, uint32_t rows, uint32_t n, float eps) {
    return rms_norm_common(cmd, x, w, out, rows, n, eps, false);
}
int32_t brasa_k_rms_norm_f16(brasa_cmd *cmd, brasa_arg x, brasa_arg w, brasa_arg out, uint32_t rows, uint32_t n, float eps) {
    return rms_norm_common(cmd, x, w, out, rows, n, eps, true);
}

int32_t brasa_k_softmax(brasa_cmd *cmd, brasa_arg x, brasa_arg out, uint32_t rows, uint32_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(x, (uint64_t)rows * n * 4) && arg_fits(out, (uint64_t)rows * n * 4), "softmax: buffers too small");
    if (rows == 0) return BRASA_OK;
    softmax_kernel<<<rows, 256, 0, ctx->stream>>>((const float *)arg_ptr(x), (float *)arg_ptr(out), n);
    return brasa_post_launch(cmd, "softmax");
}

int32_t brasa_k_rope_neox(brasa_cmd *cmd, brasa_arg x, brasa_arg cos_t, brasa_arg sin_t, uint32_t table_dim, uint32_t table_max_pos,
                          uint32_t tokens, uint32_t heads, uint32_t dim, uint32_t pos0) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, dim == table_dim && dim % 2 == 0, "rope: table dimension");
    BRASA_REQUIRE(ctx, (uint64_t)pos0 + tokens <= table_max_pos, "rope: position outside the table");
    uint64_t tb = (uint64_t)table_max_pos * (dim / 2) * 4;
    BRASA_REQUIRE(ctx, arg_fits(cos_t, tb) && arg_fits(sin_t, tb) && arg_fits(x, (uint64_t)tokens * heads * dim * 4), "rope: buffers too small");
    uint64_t n = (uint64_t)tokens * heads * (dim / 2);
    if (n == 0) return BRASA_OK;
    rope_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>((float *)arg_ptr(x), (const float *)arg_ptr(cos_t), (const float *)arg_ptr(sin_t), tokens,
                                                            heads, dim, pos0);
    return brasa_post_launch(cmd, "rope_neox");
}

int32_t brasa_k_embed(brasa_cmd *cmd, brasa_qmatrix table, brasa_arg ids, brasa_arg out, uint32_t tokens) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, table.qtype == BRASA_Q8_0 || table.qtype == BRASA_Q6_0, "embedding table must be q8_0 or q6_0");
    BRASA_REQUIRE(ctx, table.cols % 32 == 0 && qm_fits(table), "embed: bad table");
    BRASA_REQUIRE(ctx, arg_fits(ids, (uint64_t)tokens * 4) && arg_fits(out, (uint64_t)tokens * table.cols * 4), "embed: ids or out too small");
    if (tokens == 0) return BRASA_OK;
    uint64_t n = (uint64_t)tokens * table.cols;
    const uint8_t *tp = arg_ptr(table.data);
    const uint32_t *ip = (const uint32_t *)arg_ptr(ids);
    float *op = (float *)arg_ptr(out);
    unsigned g = blocks_for(n, 256);
    if (table.layout == BRASA_LAYOUT_TILED) {
        BRASA_REQUIRE(ctx, table.qtype == BRASA_Q6_0 && tiled_ok(table.qtype, table.rows, table.cols), "embed: tiled tables are q6_0");
        embed_kernel<BRASA_Q6_0, true><<<g, 256, 0, ctx->stream>>>(tp, ip, op, table.cols, tokens, table.rows);
    } else if (table.qtype == BRASA_Q6_0) {
        embed_kernel<BRASA_Q6_0, false><<<g, 256, 0, ctx->stream>>>(tp, ip, op, table.cols, tokens, table.rows);
    } else {
        embed_kernel<BRASA_Q8_0, false><<<g, 256, 0, ctx->stream>>>(tp, ip, op, table.cols, tokens, table.rows);
    }
    return brasa_post_launch(cmd, "embed");
}

int32_t brasa_k_add_norm_prep(brasa_cmd *cmd, brasa_arg x, brasa_arg h, brasa_arg w, brasa_arg xw, brasa_arg ss, uint32_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    uint32_t np = brasa_norm_partials(n);
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(x, (uint64_t)n * 4) && arg_fits(w, (uint64_t)n * 4) && arg_fits(xw, (uint64_t)n * 4) && arg_fits(ss, (uint64_t)np * 4),
                  "add_norm_prep: buffers too small");
    if (h.buf) BRASA_REQUIRE(ctx, arg_fits(h, (uint64_t)n * 4), "add_norm_prep: h too small");
    add_norm_prep_kernel<<<np, BRASA_NORM_PREP_TG, 0, ctx->stream>>>((float *)arg_ptr(x), (const float *)arg_ptr(h), (const float *)arg_ptr(w),
                                                                    (float *)arg_ptr(xw), (float *)arg_ptr(ss), n, h.buf ? 1 : 0);
    return brasa_post_launch(cmd, "add_norm_prep");
}

int32_t brasa_k_qk_norm_rope_store(brasa_cmd *cmd, int32_t kv, const brasa_arg qkv[3], const brasa_arg norms[2], float eps, brasa_arg cos_t,
                                   brasa_arg sin_t, uint32_t table_dim, uint32_t table_max_pos, const brasa_arg dst[2], brasa_attn_shape sh) {
    if (!cmd || !qkv || !norms || !dst) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, sh.dim == 128, "qk_norm_rope_store needs head_dim 128");
    BRASA_REQUIRE(ctx, table_dim == sh.dim, "RoPE table dimension");
    BRASA_REQUIRE(ctx, (uint64_t)sh.pos0 + sh.tokens <= table_max_pos, "position outside the RoPE table");
    BRASA_REQUIRE(ctx, kv >= BRASA_KV_F32 && kv <= BRASA_KV_Q8_0, "unknown KV type %d", kv);
    uint64_t tq = (uint64_t)sh.tokens * sh.hq * 128, tk = (uint64_t)sh.tokens * sh.hkv * 128;
    uint64_t tb = (uint64_t)table_max_pos * 64 * 4;
    BRASA_REQUIRE(ctx, arg_fits(qkv[0], tq * 4) && arg_fits(qkv[1], tk * 4) && arg_fits(qkv[2], tk * 4), "qk_norm_rope_store: q, k or v too small");
    BRASA_REQUIRE(ctx, arg_fits(norms[0], 512) && arg_fits(norms[1], 512) && arg_fits(cos_t, tb) && arg_fits(sin_t, tb), "qk_norm_rope_store: norm or table too small");
    BRASA_REQUIRE(ctx, arg_fits(dst[0], brasa_kv_bytes(kv, tk)) && arg_fits(dst[1], brasa_kv_bytes(kv, tk)), "qk_norm_rope_store: cache too small");
    uint32_t rows = sh.tokens * (sh.hq + 2 * sh.hkv);
    if (rows == 0) return BRASA_OK;
    unsigned grid = (rows + 3) / 4;
#define LAUNCH_QK(KVT)                                                                                                                      \
    qk_norm_rope_store_kernel<KVT><<<grid, 128, 0, ctx->stream>>>((float *)arg_ptr(qkv[0]), (float *)arg_ptr(qkv[1]), (const float *)arg_ptr(qkv[2]), \
                                                                  (const float *)arg_ptr(norms[0]), (const float *)arg_ptr(norms[1]),               \
                                                                  (const float *)arg_ptr(cos_t), (const float *)arg_ptr(sin_t), arg_ptr(dst[0]),    \
                                                                  arg_ptr(dst[1]), sh.hq, sh.hkv, sh.pos0, eps, rows)
    if (kv == BRASA_KV_F32) LAUNCH_QK(BRASA_KV_F32);
    else if (kv == BRASA_KV_F16) LAUNCH_QK(BRASA_KV_F16);
    else LAUNCH_QK(BRASA_KV_Q8_0);
#undef LAUNCH_QK
    return brasa_post_launch(cmd, "qk_norm_rope_store");
}

int32_t brasa_k_store_kv(brasa_cmd *cmd, int32_t kv, brasa_arg src, brasa_arg dst, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, kv >= BRASA_KV_F32 && kv <= BRASA_KV_Q8_0, "unknown KV type %d", kv);
    if (kv == BRASA_KV_Q8_0) BRASA_REQUIRE(ctx, n % BRASA_KV_Q8_DIM == 0, "KV Q8: rows of 128 values");
    BRASA_REQUIRE(ctx, arg_fits(src, n * 4) && arg_fits(dst, brasa_kv_bytes(kv, n)), "store_kv: buffers too small");
    if (n == 0) return BRASA_OK;
    if (kv == BRASA_KV_Q8_0) store_kv_q8_kernel<<<blocks_for(n / 32, 8), 256, 0, ctx->stream>>>((const float *)arg_ptr(src), arg_ptr(dst), n / 32);
    else store_kv_plain_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>((const float *)arg_ptr(src), arg_ptr(dst), n, kv == BRASA_KV_F16);
    return brasa_post_launch(cmd, "store_kv");
}

}  // extern "C"
