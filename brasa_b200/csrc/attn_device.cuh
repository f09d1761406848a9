// Device-side pieces shared by the fused decode attention kernel and the whole-token decode kernel: KV tile rows in
// the cache's own type, the new row's rounding and store, per-head RMSNorm + NeoX RoPE of a row held by a warp.
#pragma once
#include "brasa_internal.h"

namespace brasa_dev {

template <int KV> struct KvRow;
template <> struct KvRow<BRASA_KV_F32> { static constexpr int BYTES = 512, STRIDE = 528; };
template <> struct KvRow<BRASA_KV_F16> { static constexpr int BYTES = 256, STRIDE = 272; };
template <> struct KvRow<BRASA_KV_Q8_0> { static constexpr int BYTES = 136, STRIDE = 144; };

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// element d of a tile row in the cache's type
template <int KV>
__device__ __forceinline__ float tile_at(const uint8_t *row, int d) {
    if (KV == BRASA_KV_F32) return reinterpret_cast<const float *>(row)[d];
    if (KV == BRASA_KV_F16) return __half2float(reinterpret_cast<const __half *>(row)[d]);
    return __half2float(reinterpret_cast<const __half *>(row + 128)[d >> 5]) * (float)reinterpret_cast<const int8_t *>(row)[d];
}

// elements d and d + 1 (d even)
template <int KV>
__device__ __forceinline__ float2 tile_at2(const uint8_t *row, int d) {
    if (KV == BRASA_KV_F32) return *reinterpret_cast<const float2 *>(row + d * 4);
    if (KV == BRASA_KV_F16) return __half22float2(*reinterpret_cast<const __half2 *>(row + d * 2));
    const char2 q = *reinterpret_cast<const char2 *>(row + d);
    const float sc = __half2float(reinterpret_cast<const __half *>(row + 128)[d >> 5]);
    return make_float2(sc * (float)q.x, sc * (float)q.y);
}

// 8 consecutive elements starting at d (d % 8 == 0)
template <int KV>
__device__ __forceinline__ void tile_load8(const uint8_t *row, int d, float out[8]) {
    if (KV == BRASA_KV_F32) {
        float4 a = reinterpret_cast<const float4 *>(row)[d / 4], b = reinterpret_cast<const float4 *>(row)[d / 4 + 1];
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else if (KV == BRASA_KV_F16) {
        uint4 v = reinterpret_cast<const uint4 *>(row)[d / 8];
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
        for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            out[2 * j] = f.x; out[2 * j + 1] = f.y;
        }
    } else {
        uint2 v = reinterpret_cast<const uint2 *>(row)[d / 8];
        float sc = __half2float(reinterpret_cast<const __half *>(row + 128)[d >> 5]);
        const int8_t *c = reinterpret_cast<const int8_t *>(&v);
        for (int j = 0; j < 8; ++j) out[j] = sc * (float)c[j];
    }
}

// The warp holds one row of 128 values (lane + 32 j). Writes it, rounded to the cache type, to both the
// cache row in global memory and the tile row in shared memory.
template <int KV>
__device__ __forceinline__ void put_row(uint8_t *grow, uint8_t *srow, const float y[4], int lane) {
    for (int j = 0; j < 4; ++j) {
        if (KV == BRASA_KV_Q8_0) {
            float amax = fabsf(y[j]);
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            __half dh = __float2half_rn(__fdiv_rn(amax, 127.0f));
            float d = __half2float(dh);
            int8_t q = (int8_t)(d == 0.0f ? 0.0f : fminf(fmaxf(rintf(__fdiv_rn(y[j], d)), -127.0f), 127.0f));
            reinterpret_cast<int8_t *>(grow)[lane + 32 * j] = q;
            reinterpret_cast<int8_t *>(srow)[lane + 32 * j] = q;
            if (lane == 0) {
                reinterpret_cast<__half *>(grow + 128)[j] = dh;
                reinterpret_cast<__half *>(srow + 128)[j] = dh;
            }
        } else if (KV == BRASA_KV_F16) {
            __half h = __float2half_rn(y[j]);
            reinterpret_cast<__half *>(grow)[lane + 32 * j] = h;
            reinterpret_cast<__half *>(srow)[lane + 32 * j] = h;
        } else {
            reinterpret_cast<float *>(grow)[lane + 32 * j] = y[j];
            reinterpret_cast<float *>(srow)[lane + 32 * j] = y[j];
        }
    }
}

// per-head RMSNorm then NeoX RoPE of one row held by a warp (qkv.metal semantics)
__device__ __forceinline__ void norm_rope_row(const float *x, const float *w, const float *cos_t, const float *sin_t, uint32_t pos, float eps,
                                              int lane, float y[4]) {
    float xv[4], ss = 0.0f;
    for (int j = 0; j < 4; ++j) {
        xv[j] = x[lane + 32 * j];
        ss += xv[j] * xv[j];
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float scale = 1.0f / sqrtf(ss / 128.0f + eps);
    for (int j = 0; j < 4; ++j) y[j] = xv[j] * scale * w[lane + 32 * j];
    for (int j = 0; j < 2; ++j) {
        int i = lane + 32 * j;
        float c = cos_t[(size_t)pos * 64 + i], s = sin_t[(size_t)pos * 64 + i];
        float a = y[j], b = y[j + 2];
        y[j] = a * c - b * s;
        y[j + 2] = b * c + a * s;
    }
}

// The same for a row the warp already holds in registers (xv[j] = element lane + 32 j).
__device__ __forceinline__ void norm_rope_vals(const float xv[4], const float *w, const float *cos_t, const float *sin_t, uint32_t pos, float eps,
                                               int lane, float y[4]) {
    float ss = 0.0f;
    for (int j = 0; j < 4; ++j) ss += xv[j] * xv[j];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float scale = 1.0f / sqrtf(ss / 128.0f + eps);
    for (int j = 0; j < 4; ++j) y[j] = xv[j] * scale * w[lane + 32 * j];
    for (int j = 0; j < 2; ++j) {
        int i = lane + 32 * j;
        float c = cos_t[(size_t)pos * 64 + i], s = sin_t[(size_t)pos * 64 + i];
        float a = y[j], b = y[j + 2];
        y[j] = a * c - b * s;
        y[j + 2] = b * c + a * s;
    }
}


// The same with the norm weight and the table entries already in registers (wv[j] = w[lane + 32 j], cs[j] / sn[j] =
// cos / sin of pair lane + 32 j): what does not depend on the row can then be fetched before the row arrives.
__device__ __forceinline__ void norm_rope_regs(const float xv[4], const float wv[4], const float cs[2], const float sn[2], float eps, float y[4]) {
    float ss = 0.0f;
    for (int j = 0; j < 4; ++j) ss += xv[j] * xv[j];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float scale = 1.0f / sqrtf(ss / 128.0f + eps);
    for (int j = 0; j < 4; ++j) y[j] = xv[j] * scale * wv[j];
    for (int j = 0; j < 2; ++j) {
        float a = y[j], b = y[j + 2];
        y[j] = a * cs[j] - b * sn[j];
        y[j + 2] = b * cs[j] + a * sn[j];
    }
}

}  // namespace brasa_dev
