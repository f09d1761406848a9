// Weight formats on the device: file <-> tiled layout, quantisers, dequantiser, seeded random init.
//
// The `.brasa` block formats follow crates/quant/src/qtype.rs:5-29 and the quantisers
// crates/quant/src/convert.rs:70-151 (IEEE division, round-half-even, f16 scale with
// round-to-nearest-even); every kernel here is bit-exact against that specification.
#include <type_traits>

#include "brasa_internal.h"

namespace {

__device__ __forceinline__ uint16_t ld16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ void st16(uint8_t *p, uint16_t v) { *reinterpret_cast<uint16_t *>(p) = v; }

// One thread per 32-weight block.
template <int QT, bool TO_TILED>
__global__ void repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint32_t rows, uint32_t nb) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)rows * nb) return;
    uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
    constexpr int BB = QT == BRASA_Q4_0 ? 18 : 26;
    const uint32_t cols = nb * 32;
    uint8_t *fp = (uint8_t *)(TO_TILED ? src : dst) + i * BB;                                   // file-layout block
    uint8_t *row = (uint8_t *)(TO_TILED ? dst : src) + (size_t)r * tiled_row_bytes(QT, cols);   // tiled row
    uint8_t *codes = row + b * 16;
    uint8_t *scale = row + tiled_scale_off(QT, cols) + b * 2;
    if (TO_TILED) {
        st16(scale, ld16(fp));
        for (int j = 0; j < 8; ++j) st16(codes + 2 * j, ld16(fp + 2 + 2 * j));
    } else {
        st16(fp, ld16(scale));
        for (int j = 0; j < 8; ++j) st16(fp + 2 + 2 * j, ld16(codes + 2 * j));
    }
    if (QT == BRASA_Q6_0) {
        uint32_t *hi = reinterpret_cast<uint32_t *>(row + tiled_hi_off(cols) + b * 8);  // two words
        if (TO_TILED) {
            uint32_t h[2] = {0, 0};
            for (int w = 0; w < 4; ++w)
                for (int k = 0; k < 8; ++k) {
                    int e = 4 * w + (k >> 1) + 16 * (k & 1);
                    uint32_t two = (fp[18 + (e & 7)] >> (2 * (e >> 3))) & 3u;
                    h[w >> 1] |= two << q6_hi_bitpos(w & 1, k);
                }
            hi[0] = h[0];
            hi[1] = h[1];
        } else {
            uint32_t h[2] = {hi[0], hi[1]};
            uint8_t qh[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int w = 0; w < 4; ++w)
                for (int k = 0; k < 8; ++k) {
                    int e = 4 * w + (k >> 1) + 16 * (k & 1);
                    uint32_t two = (h[w >> 1] >> q6_hi_bitpos(w & 1, k)) & 3u;
                    qh[e & 7] |= (uint8_t)(two << (2 * (e >> 3)));
                }
            for (int j = 0; j < 8; ++j) fp[18 + j] = qh[j];
        }
    }
}

// One thread per block; bit-exact with quant_q4_0 / quant_q6_0 / quant_q8_0.
template <int QT>
__global__ void quantize_kernel(const float *__restrict__ w, uint8_t *__restrict__ out, uint64_t nblocks) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblocks) return;
    const float4 *v4 = reinterpret_cast<const float4 *>(w + i * 32);
    float v[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float4 t = v4[j];
        v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
    float best = fabsf(v[0]), m = v[0];
#pragma unroll
    for (int j = 1; j < 32; ++j) {
        float a = fabsf(v[j]);
        if (a > best) { best = a; m = v[j]; }  // first index of the largest magnitude, sign kept
    }
    constexpr int BB = QT == BRASA_Q4_0 ? 18 : (QT == BRASA_Q6_0 ? 26 : 34);
    uint8_t *p = out + i * BB;
    if (QT == BRASA_Q8_0) {
        __half dh = __float2half_rn(__fdiv_rn(best, 127.0f));
        float d = __half2float(dh);
        st16(p, __half_as_ushort(dh));
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float q = d == 0.0f ? 0.0f : fminf(fmaxf(rintf(__fdiv_rn(v[j], d)), -127.0f), 127.0f);
            p[2 + j] = (uint8_t)(int8_t)q;
        }
        return;
    }
    constexpr float BIAS = QT == BRASA_Q4_0 ? 8.0f : 32.0f;
    constexpr float QMAX = QT == BRASA_Q4_0 ? 15.0f : 63.0f;
    __half dh = __float2half_rn(__fdiv_rn(m, -BIAS));
    float d = __half2float(dh);
    uint8_t q[32];
#pragma unroll
    for (int j = 0; j < 32; ++j)
        q[j] = d != 0.0f ? (uint8_t)fminf(fmaxf(rintf(__fdiv_rn(v[j], d)) + BIAS, 0.0f), QMAX) : (uint8_t)BIAS;
    st16(p, __half_as_ushort(dh));
#pragma unroll
    for (int j = 0; j < 16; ++j) p[2 + j] = (uint8_t)((q[j] & 15) | ((q[j + 16] & 15) << 4));
    if (QT == BRASA_Q6_0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            p[18 + j] = (uint8_t)((q[j] >> 4) | ((q[j + 8] >> 4) << 2) | ((q[j + 16] >> 4) << 4) | ((q[j + 24] >> 4) << 6));
    }
}

template <int QT>
__global__ void dequantize_kernel(const uint8_t *__restrict__ data, float *__restrict__ out, uint64_t nblocks) {
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblocks) return;
    constexpr int BB = QT == BRASA_Q4_0 ? 18 : (QT == BRASA_Q6_0 ? 26 : 34);
    const uint8_t *p = data + i * BB;
    float d = __half2float(__ushort_as_half(ld16(p)));
    float *o = out + i * 32;
    for (int j = 0; j < 32; ++j) {
        int q;
        if (QT == BRASA_Q4_0) q = (j < 16 ? (p[2 + j] & 15) : (p[2 + j - 16] >> 4)) - 8;
        else if (QT == BRASA_Q8_0) q = (int8_t)p[2 + j];
        else {
            int ql = p[2 + (j & 15)];
            int lo = j < 16 ? (ql & 15) : (ql >> 4);
            int hi = (p[18 + (j & 7)] >> (2 * (j >> 3))) & 3;
            q = (lo | (hi << 4)) - 32;
        }
        o[j] = d * (float)q;
    }
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// Two normals per counter value (Box-Muller over a splitmix64 hash of seed and index).
__global__ void randn_kernel(float *__restrict__ out, uint64_t n, uint64_t seed, uint64_t offset, float std) {
    uint64_t pair = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t i = pair * 2;
    if (i >= n) return;
    uint64_t h = mix64(mix64(seed) ^ (offset + pair));
    float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    float u2 = (float)(uint32_t)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    float r = sqrtf(-2.0f * logf(u1)) * std;
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    out[i] = r * c;
    if (i + 1 < n) out[i + 1] = r * s;
}

template <typename F>
int32_t launch_by_qtype(brasa_cmd *cmd, int32_t qtype, F &&f) {
    switch (qtype) {
    case BRASA_Q4_0: f(std::integral_constant<int, BRASA_Q4_0>()); break;
    case BRASA_Q6_0: f(std::integral_constant<int, BRASA_Q6_0>()); break;
    case BRASA_Q8_0: f(std::integral_constant<int, BRASA_Q8_0>()); break;
    default: return brasa_fail(cmd->ctx, BRASA_EINVAL, "unknown weight type %d", qtype);
    }
    return BRASA_OK;
}

int32_t repack_common(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst, uint32_t rows, uint32_t cols, bool to_tiled) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, tiled_ok(qtype, rows, cols), "the tiled layout needs q4_0 or q6_0 and cols %% 256 == 0 (got %u x %u)", rows, cols);
    uint64_t bytes = brasa_qtype_nbytes(qtype, (uint64_t)rows * cols);
    BRASA_REQUIRE(ctx, arg_fits(src, bytes) && arg_fits(dst, bytes), "repack: buffers smaller than the matrix");
    BRASA_REQUIRE(ctx, arg_ptr(src) != arg_ptr(dst), "repack cannot run in place");
    BRASA_REQUIRE(ctx, (src.offset % 16 == 0) && (dst.offset % 16 == 0), "repack: offsets must be 16-byte aligned");
    uint32_t nb = cols / 32;
    uint64_t n = (uint64_t)rows * nb;
    unsigned grid = (unsigned)((n + 255) / 256);
    if (qtype == BRASA_Q4_0) {
        if (to_tiled) repack_kernel<BRASA_Q4_0, true><<<grid, 256, 0, ctx->stream>>>(arg_ptr(src), arg_ptr(dst), rows, nb);
        else repack_kernel<BRASA_Q4_0, false><<<grid, 256, 0, ctx->stream>>>(arg_ptr(src), arg_ptr(dst), rows, nb);
    } else {
        if (to_tiled) repack_kernel<BRASA_Q6_0, true><<<grid, 256, 0, ctx->stream>>>(arg_ptr(src), arg_ptr(dst), rows, nb);
        else repack_kernel<BRASA_Q6_0, false><<<grid, 256, 0, ctx->stream>>>(arg_ptr(src), arg_ptr(dst), rows, nb);
    }
    return brasa_post_launch(cmd, "repack");
}

}  // namespace

extern "C" {

int32_t brasa_k_repack(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst, uint32_t rows, uint32_t cols) {
    return repack_common(cmd, qtype, src, dst, rows, cols, true);
}
int32_t brasa_k_unpack(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst, uint32_t rows, uint32_t cols) {
    return repack_common(cmd, qtype, src, dst, rows, cols, false);
}

int32_t brasa_k_quantize(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n % 32 == 0, "quantize: n %% 32 != 0");
    BRASA_REQUIRE(ctx, arg_fits(src, n * 4) && arg_fits(dst, brasa_qtype_nbytes(qtype, n)), "quantize: buffers too small");
    BRASA_REQUIRE(ctx, src.offset % 16 == 0 && dst.offset % 2 == 0, "quantize: misaligned offsets");
    if (n == 0) return BRASA_OK;
    uint64_t nb = n / 32;
    unsigned grid = (unsigned)((nb + 127) / 128);
    BRASA_TRY(launch_by_qtype(cmd, qtype, [&](auto qt) {
        quantize_kernel<decltype(qt)::value><<<grid, 128, 0, ctx->stream>>>((const float *)arg_ptr(src), arg_ptr(dst), nb);
    }));
    return brasa_post_launch(cmd, "quantize");
}

int32_t brasa_k_dequantize(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst, uint64_t n) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n % 32 == 0, "dequantize: n %% 32 != 0");
    BRASA_REQUIRE(ctx, arg_fits(dst, n * 4) && arg_fits(src, brasa_qtype_nbytes(qtype, n)), "dequantize: buffers too small");
    BRASA_REQUIRE(ctx, src.offset % 2 == 0 && dst.offset % 4 == 0, "dequantize: misaligned offsets");
    if (n == 0) return BRASA_OK;
    uint64_t nb = n / 32;
    unsigned grid = (unsigned)((nb + 127) / 128);
    BRASA_TRY(launch_by_qtype(cmd, qtype, [&](auto qt) {
        dequantize_kernel<decltype(qt)::value><<<grid, 128, 0, ctx->stream>>>(arg_ptr(src), (float *)arg_ptr(dst), nb);
    }));
    return brasa_post_launch(cmd, "dequantize");
}

int32_t brasa_k_randn(brasa_cmd *cmd, brasa_arg dst, uint64_t n, uint64_t seed, uint64_t stream_offset, float std) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(dst, n * 4) && dst.offset % 4 == 0, "randn: buffer too small or misaligned");
    if (n == 0) return BRASA_OK;
    uint64_t pairs = (n + 1) / 2;
    randn_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, ctx->stream>>>((float *)arg_ptr(dst), n, seed, stream_offset, std);
    return brasa_post_launch(cmd, "randn");
}

}  // extern "C"
