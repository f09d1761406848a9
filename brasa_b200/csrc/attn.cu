// Attention: split-K GQA decode attention (one query token over f32 / f16 / Q8 KV) and the causal
// prefill attention. crates/kernels/src/lib.rs:1056-1248; decode_attention.metal, flash_attention.metal.
//
// KV cache rows are [position][kv head][128] in the cache's type; a Q8 row is 128 int8 codes followed
// by four f16 scales (136 bytes, crates/quant/src/qtype.rs:81-111).
#include <stdlib.h>

#include "brasa_internal.h"
#include "attn_device.cuh"

using namespace brasa_dev;

int32_t brasa_flash_tc_launch(brasa_cmd *cmd, int32_t kv, const float *q, const uint8_t *kc, const uint8_t *vc, __half *o, brasa_attn_shape sh);

namespace {

constexpr int D = 128;
constexpr int TS = D + 4;  // padded row of the shared f32 tile

// Loads rows [key0, key0+nkeys) of one kv head into ts[key][d] as f32.
template <int KV>
__device__ __forceinline__ void load_tile(const uint8_t *cache, float *ts, uint32_t key0, uint32_t nkeys, uint32_t hkv, uint32_t kh) {
    if (KV == BRASA_KV_F32) {
        for (uint32_t i = threadIdx.x; i < nkeys * (D / 4); i += blockDim.x) {
            uint32_t key = i / (D / 4), v4 = i % (D / 4);
            float4 v = reinterpret_cast<const float4 *>(cache + ((size_t)(key0 + key) * hkv + kh) * D * 4)[v4];
            float *o = ts + key * TS + v4 * 4;
            o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
        }
    } else if (KV == BRASA_KV_F16) {
        for (uint32_t i = threadIdx.x; i < nkeys * (D / 8); i += blockDim.x) {
            uint32_t key = i / (D / 8), v8 = i % (D / 8);
            uint4 v = reinterpret_cast<const uint4 *>(cache + ((size_t)(key0 + key) * hkv + kh) * D * 2)[v8];
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
            float *o = ts + key * TS + v8 * 8;
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h[j]);
                o[2 * j] = f.x; o[2 * j + 1] = f.y;
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < nkeys * (D / 8); i += blockDim.x) {
            uint32_t key = i / (D / 8), v8 = i % (D / 8);
            const uint8_t *row = cache + ((size_t)(key0 + key) * hkv + kh) * BRASA_KV_Q8_ROW;
            uint2 v = reinterpret_cast<const uint2 *>(row)[v8];
            float d = __half2float(reinterpret_cast<const __half *>(row + 128)[v8 / 4]);
            const int8_t *c = reinterpret_cast<const int8_t *>(&v);
            float *o = ts + key * TS + v8 * 8;
            for (int j = 0; j < 8; ++j) o[j] = d * (float)c[j];
        }
    }
}

// One block per (128-key chunk, kv head): all G query heads of the group share the K and V reads.
// partial layout per (head, chunk): m, l, acc[128]  (crates/kernels/src/lib.rs:1335).
template <int KV>
__global__ void __launch_bounds__(128) decode_partial_kernel(const float *q, const uint8_t *kc, const uint8_t *vc, float *partials, uint32_t hq,
                                                             uint32_t hkv, uint32_t lk, float scale) {
    extern __shared__ __align__(16) float sm[];
    float *ts = sm;                    // [128][TS]
    float *qs = ts + 128 * TS;         // [G][128]
    float *ps = qs + 8 * D;            // [G][128] scores, then probabilities
    float *red = ps + 8 * 128;         // [8]
    const uint32_t chunk = blockIdx.x, kh = blockIdx.y, G = hq / hkv, chunks = gridDim.x;
    const uint32_t key0 = chunk * 128, nkeys = min(128u, lk - key0);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (uint32_t i = t; i < G * D; i += 128) qs[i] = q[(size_t)kh * G * D + i];
    load_tile<KV>(kc, ts, key0, nkeys, hkv, kh);
    __syncthreads();
    for (uint32_t g = 0; g < G; ++g) {
        float s = -INFINITY;
        if ((uint32_t)t < nkeys) {
            const float4 *kr = reinterpret_cast<const float4 *>(ts + t * TS);
            const float4 *qr = reinterpret_cast<const float4 *>(qs + g * D);
            float a = 0.0f;
#pragma unroll 8
            for (int i = 0; i < D / 4; ++i) {
                float4 kk = kr[i], qq = qr[i];
                a = fmaf(qq.x, kk.x, a); a = fmaf(qq.y, kk.y, a); a = fmaf(qq.z, kk.z, a); a = fmaf(qq.w, kk.w, a);
            }
            s = a * scale;
        }
        ps[g * 128 + t] = s;
    }
    __syncthreads();
    load_tile<KV>(vc, ts, key0, nkeys, hkv, kh);  // K is no longer needed
    for (uint32_t g = 0; g < G; ++g) {
        float s = ps[g * 128 + t];
        float m = s;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        float p = (uint32_t)t < nkeys ? expf(s - m) : 0.0f;
        ps[g * 128 + t] = p;
        float l = p;
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        __syncthreads();
        if (lane == 0) red[4 + warp] = l;
        __syncthreads();
        if (t == 0) {
            float *out = partials + ((size_t)(kh * G + g) * chunks + chunk) * 130;
            out[0] = m;
            out[1] = (red[4] + red[5]) + (red[6] + red[7]);
        }
    }
    __syncthreads();
    for (uint32_t g = 0; g < G; ++g) {
        float acc = 0.0f;
        const float *pg = ps + g * 128;
        for (uint32_t j = 0; j < nkeys; ++j) acc = fmaf(pg[j], ts[j * TS + t], acc);
        partials[((size_t)(kh * G + g) * chunks + chunk) * 130 + 2 + t] = acc;
    }
}

__global__ void __launch_bounds__(128) decode_reduce_kernel(const float *partials, float *o, uint32_t chunks) {
    const uint32_t h = blockIdx.x, t = threadIdx.x;
    const float *p = partials + (size_t)h * chunks * 130;
    float M = -INFINITY;
    for (uint32_t c = 0; c < chunks; ++c) M = fmaxf(M, p[c * 130]);
    float L = 0.0f, acc = 0.0f;
    for (uint32_t c = 0; c < chunks; ++c) {
        float w = expf(p[c * 130] - M);
        L = fmaf(p[c * 130 + 1], w, L);
        acc = fmaf(p[c * 130 + 2 + t], w, acc);
    }
    o[(size_t)h * D + t] = acc / L;
}

// Scratch for brasa_k_decode_attention_static: the chunk partials live in this array instead of a
// caller-provided buffer. Sized for 64 query heads and 8192 keys (64 chunks of 128): 64 * 64 * 130 floats.
constexpr uint32_t STATIC_MAX_HQ = 64, STATIC_MAX_KEYS = 8192;
constexpr size_t STATIC_PARTIAL_FLOATS = (size_t)STATIC_MAX_HQ * (STATIC_MAX_KEYS / 128) * 130;
static __device__ __align__(256) float g_decode_partials[STATIC_PARTIAL_FLOATS];

// Causal prefill attention, f32 arithmetic throughout. One block = 64 queries of one query head;
// keys in tiles of 32. HALF_IO: Q*scale is rounded to f16 and the output is written as f16, like the
// reference's PrefillPrecision::F16 (flash_attention.metal:213,320); otherwise Q stays f32, the
// score is (q.k)*scale and the output is f32.
template <int KV, bool HALF_IO>
__global__ void __launch_bounds__(256) prefill_attn_kernel(const float *q, const uint8_t *kc, const uint8_t *vc, void *o, uint32_t tokens,
                                                           uint32_t hq, uint32_t hkv, uint32_t pos0, float scale) {
    extern __shared__ __align__(16) float sm[];
    constexpr int QB = 64, KB = 32;
    float *qs = sm;                 // [64][TS]
    float *ks = qs + QB * TS;       // [32][TS]
    float *vs = ks + KB * TS;       // [32][TS]
    float *ss = vs + KB * TS;       // [64][33]
    float *mrow = ss + QB * 33;     // [64] running max
    float *lrow = mrow + QB;        // [64] running sum
    float *crow = lrow + QB;        // [64] correction of this tile
    // longest query blocks first (they see the most keys)
    const uint32_t qblocks = gridDim.x, qb = qblocks - 1 - blockIdx.x, h = blockIdx.y, kh = h / (hq / hkv);
    const uint32_t q0 = qb * QB, nq = min((uint32_t)QB, tokens - q0);
    const int t = threadIdx.x, ty = t >> 4, tx = t & 15;  // ty: 4 queries, tx: 2 keys / 8 dims
    for (uint32_t i = t; i < QB * D; i += 256) {
        uint32_t r = i / D, d = i % D;
        float v = r < nq ? q[((size_t)(q0 + r) * hq + h) * D + d] : 0.0f;
        if (HALF_IO) v = __half2float(__float2half_rn(v * scale));
        qs[r * TS + d] = v;
    }
    if (t < QB) { mrow[t] = -INFINITY; lrow[t] = 0.0f; }
    float oacc[4][8];
    for (int a = 0; a < 4; ++a)
        for (int b = 0; b < 8; ++b) oacc[a][b] = 0.0f;
    const uint32_t last_key = pos0 + q0 + nq - 1;  // inclusive
    __syncthreads();
    for (uint32_t k0 = 0; k0 <= last_key; k0 += KB) {
        uint32_t nk = min((uint32_t)KB, last_key + 1 - k0);
        load_tile<KV>(kc, ks, k0, nk, hkv, kh);
        load_tile<KV>(vc, vs, k0, nk, hkv, kh);
        __syncthreads();
        float s[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};
        for (int d = 0; d < D; d += 4) {
            float4 k0v = *reinterpret_cast<const float4 *>(ks + (2 * tx) * TS + d);
            float4 k1v = *reinterpret_cast<const float4 *>(ks + (2 * tx + 1) * TS + d);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float4 qv = *reinterpret_cast<const float4 *>(qs + (4 * ty + a) * TS + d);
                s[a][0] = fmaf(qv.x, k0v.x, s[a][0]); s[a][0] = fmaf(qv.y, k0v.y, s[a][0]);
                s[a][0] = fmaf(qv.z, k0v.z, s[a][0]); s[a][0] = fmaf(qv.w, k0v.w, s[a][0]);
                s[a][1] = fmaf(qv.x, k1v.x, s[a][1]); s[a][1] = fmaf(qv.y, k1v.y, s[a][1]);
                s[a][1] = fmaf(qv.z, k1v.z, s[a][1]); s[a][1] = fmaf(qv.w, k1v.w, s[a][1]);
            }
        }
        for (int a = 0; a < 4; ++a)
            for (int b = 0; b < 2; ++b) {
                uint32_t key = k0 + 2 * tx + b, qi = 4 * ty + a;
                bool ok = (2u * tx + b) < nk && qi < nq && key <= pos0 + q0 + qi;
                float v = HALF_IO ? s[a][b] : s[a][b] * scale;
                ss[qi * 33 + 2 * tx + b] = ok ? v : -INFINITY;
            }
        __syncthreads();
        if (t < QB) {
            float m_old = mrow[t], m = m_old;
            for (int j = 0; j < KB; ++j) m = fmaxf(m, ss[t * 33 + j]);
            float l = 0.0f;
            for (int j = 0; j < KB; ++j) {
                float p = m == -INFINITY ? 0.0f : expf(ss[t * 33 + j] - m);
                ss[t * 33 + j] = p;
                l += p;
            }
            float c = m_old == -INFINITY ? 0.0f : expf(m_old - m);
            crow[t] = c;
            lrow[t] = lrow[t] * c + l;
            mrow[t] = m;
        }
        __syncthreads();
        for (int a = 0; a < 4; ++a) {
            float c = crow[4 * ty + a];
            for (int b = 0; b < 8; ++b) oacc[a][b] *= c;
        }
        for (uint32_t j = 0; j < nk; ++j) {
            float4 v0 = *reinterpret_cast<const float4 *>(vs + j * TS + 8 * tx);
            float4 v1 = *reinterpret_cast<const float4 *>(vs + j * TS + 8 * tx + 4);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float p = ss[(4 * ty + a) * 33 + j];
                oacc[a][0] = fmaf(p, v0.x, oacc[a][0]); oacc[a][1] = fmaf(p, v0.y, oacc[a][1]);
                oacc[a][2] = fmaf(p, v0.z, oacc[a][2]); oacc[a][3] = fmaf(p, v0.w, oacc[a][3]);
                oacc[a][4] = fmaf(p, v1.x, oacc[a][4]); oacc[a][5] = fmaf(p, v1.y, oacc[a][5]);
                oacc[a][6] = fmaf(p, v1.z, oacc[a][6]); oacc[a][7] = fmaf(p, v1.w, oacc[a][7]);
            }
        }
        __syncthreads();
    }
    for (int a = 0; a < 4; ++a) {
        uint32_t qi = 4 * ty + a;
        if (qi >= nq) continue;
        float inv = 1.0f / lrow[qi];
        size_t base = ((size_t)(q0 + qi) * hq + h) * D + 8 * tx;
        for (int b = 0; b < 8; ++b) {
            float v = oacc[a][b] * inv;
            if (HALF_IO) reinterpret_cast<__half *>(o)[base + b] = __float2half_rn(v);
            else reinterpret_cast<float *>(o)[base + b] = v;
        }
    }
}

// ---- fused decode attention: QK-norm + RoPE + KV store + split-K attention + merge, one kernel ----
// The position comes from device memory, so the same launch (recorded in a CUDA graph) serves every
// step. Grid: (ceil(ctx / 128), kv heads); blocks whose chunk lies past the position return at once.
// K and V tiles stay in the cache's own type in shared memory and are fetched with cp.async before the
// kernel waits for q, k and v of this token (older rows never change). The block that owns the newest
// position normalises, rotates, rounds and stores the new K and V rows and uses the rounded values.
// The last block of a kv head to finish merges the chunk partials (arrival counter, no spinning).
struct FusedAttnParams {
    const float *q, *k_new, *v_new, *q_norm, *k_norm, *cos_t, *sin_t;
    uint8_t *kc, *vc;      // this layer's cache, position 0
    float *partials;       // [hq][gridDim.x][130]
    uint32_t *counters;    // [hkv], zero between launches
    float *o;              // [hq][128]
    const uint32_t *pos;   // device scalar: position of this token
    uint32_t hq, hkv;
    float eps, scale;
};

template <int KV>
__global__ void __launch_bounds__(128) attn_decode_fused_kernel(FusedAttnParams p) {
    constexpr int RB = KvRow<KV>::BYTES, RS = KvRow<KV>::STRIDE;
    extern __shared__ __align__(16) uint8_t smraw[];
    uint8_t *kt = smraw, *vt = smraw + 128 * RS;
    float *qs = reinterpret_cast<float *>(vt + 128 * RS);  // [G][128]
    float *ps = qs + 8 * 128;                               // [G][128]
    float *red = ps + 8 * 128;                              // [16]
    __shared__ bool last_block;
    const uint32_t pos = *p.pos, lk = pos + 1, nchunks = (lk + 127) / 128;
    const uint32_t chunk = blockIdx.x, kh = blockIdx.y, G = p.hq / p.hkv, max_chunks = gridDim.x;
    if (chunk >= nchunks) return;
    const uint32_t key0 = chunk * 128, nkeys = min(128u, lk - key0);
    const bool has_new = chunk == nchunks - 1;
    const uint32_t nold = has_new ? nkeys - 1 : nkeys;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // older rows never change: fetch them before this token's q, k, v exist
    {
        constexpr int VEC = KV == BRASA_KV_Q8_0 ? 8 : 16, PER_ROW = RB / VEC;
        for (uint32_t i = t; i < nold * PER_ROW; i += 128) {
            uint32_t r = i / PER_ROW, v = i % PER_ROW;
            size_t goff = ((size_t)(key0 + r) * p.hkv + kh) * RB + (size_t)v * VEC;
            if (KV == BRASA_KV_Q8_0) { cp_async8(kt + r * RS + v * VEC, p.kc + goff); cp_async8(vt + r * RS + v * VEC, p.vc + goff); }
            else { cp_async16(kt + r * RS + v * VEC, p.kc + goff); cp_async16(vt + r * RS + v * VEC, p.vc + goff); }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // q heads of this group: norm + rope into shared memory (warps take heads round robin)
    for (uint32_t g = warp; g < G; g += 4) {
        float y[4];
        norm_rope_row(p.q + (size_t)(kh * G + g) * 128, p.q_norm, p.cos_t, p.sin_t, pos, p.eps, lane, y);
        for (int j = 0; j < 4; ++j) qs[g * 128 + lane + 32 * j] = y[j];
    }
    if (has_new) {
        size_t grow = ((size_t)pos * p.hkv + kh) * RB;
        if (warp == 3) {
            float y[4];
            norm_rope_row(p.k_new + (size_t)kh * 128, p.k_norm, p.cos_t, p.sin_t, pos, p.eps, lane, y);
            put_row<KV>(p.kc + grow, kt + (nkeys - 1) * RS, y, lane);
        } else if (warp == 2) {
            float y[4];
            for (int j = 0; j < 4; ++j) y[j] = p.v_new[(size_t)kh * 128 + lane + 32 * j];
            put_row<KV>(p.vc + grow, vt + (nkeys - 1) * RS, y, lane);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // scores: one key per thread, all heads of the group
    {
        float s[8];
        for (int g = 0; g < 8; ++g) s[g] = 0.0f;
        if ((uint32_t)t < nkeys) {
            const uint8_t *row = kt + t * RS;
            for (int d = 0; d < 128; d += 8) {
                float kv8[8];
                tile_load8<KV>(row, d, kv8);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if ((uint32_t)g >= G) break;
                    const float4 qa = *reinterpret_cast<const float4 *>(qs + g * 128 + d), qb = *reinterpret_cast<const float4 *>(qs + g * 128 + d + 4);
                    float a = s[g];
                    a = fmaf(qa.x, kv8[0], a); a = fmaf(qa.y, kv8[1], a); a = fmaf(qa.z, kv8[2], a); a = fmaf(qa.w, kv8[3], a);
                    a = fmaf(qb.x, kv8[4], a); a = fmaf(qb.y, kv8[5], a); a = fmaf(qb.z, kv8[6], a); a = fmaf(qb.w, kv8[7], a);
                    s[g] = a;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 8; ++g)
            if ((uint32_t)g < G) ps[g * 128 + t] = (uint32_t)t < nkeys ? s[g] * p.scale : -INFINITY;
    }
    __syncthreads();
    // partial softmax per head: warp w reduces heads w, w + 4
    for (uint32_t g = warp; g < G; g += 4) {
        float v0 = ps[g * 128 + lane], v1 = ps[g * 128 + lane + 32], v2 = ps[g * 128 + lane + 64], v3 = ps[g * 128 + lane + 96];
        float m = fmaxf(fmaxf(v0, v1), fmaxf(v2, v3));
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        v0 = expf(v0 - m); v1 = expf(v1 - m); v2 = expf(v2 - m); v3 = expf(v3 - m);
        ps[g * 128 + lane] = v0; ps[g * 128 + lane + 32] = v1; ps[g * 128 + lane + 64] = v2; ps[g * 128 + lane + 96] = v3;
        float l = (v0 + v1) + (v2 + v3);
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) { red[g] = m; red[8 + g] = l; }
    }
    __syncthreads();
    // P V: one output dimension per thread
    float acc[8];
    for (int g = 0; g < 8; ++g) acc[g] = 0.0f;
    for (uint32_t j = 0; j < nkeys; ++j) {
        float vv = tile_at<KV>(vt + j * RS, t);
#pragma unroll
        for (int g = 0; g < 8; ++g)
            if ((uint32_t)g < G) acc[g] = fmaf(ps[g * 128 + j], vv, acc[g]);
    }
    if (nchunks == 1) {  // nothing to merge
#pragma unroll
        for (int g = 0; g < 8; ++g)
            if ((uint32_t)g < G) p.o[(size_t)(kh * G + g) * 128 + t] = acc[g] / red[8 + g];
        return;
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        if ((uint32_t)g >= G) break;
        float *out = p.partials + ((size_t)(kh * G + g) * max_chunks + chunk) * 130;
        __stcg(out + 2 + t, acc[g]);
        if (t == 0) { __stcg(out, red[g]); __stcg(out + 1, red[8 + g]); }
    }
    __threadfence();
    __syncthreads();
    if (t == 0) last_block = atomicAdd(&p.counters[kh], 1u) == nchunks - 1;
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    if (t == 0) p.counters[kh] = 0;
    // merge: every thread reads the chunks' maxima and sums straight from the partials (broadcast loads that stay in
    // L2), so nothing is staged per chunk and the context length is not bounded by shared memory. Two sweeps: the
    // head's maximum first, then weights and accumulators in chunk order, eight chunks in flight at a time.
    for (uint32_t g = 0; g < G; ++g) {
        const float *ph = p.partials + (size_t)(kh * G + g) * max_chunks * 130;
        float M = -INFINITY;
        for (uint32_t c0 = 0; c0 < nchunks; c0 += 8) {
            float mm[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mm[j] = c0 + j < nchunks ? __ldcg(ph + (size_t)(c0 + j) * 130) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) M = fmaxf(M, mm[j]);
        }
        float L = 0.0f, a = 0.0f;
        for (uint32_t c0 = 0; c0 < nchunks; c0 += 8) {
            float mm[8], ll[8], v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool in = c0 + j < nchunks;
                const float *pc = ph + (size_t)(c0 + j) * 130;
                mm[j] = in ? __ldcg(pc) : -INFINITY;
                ll[j] = in ? __ldcg(pc + 1) : 0.0f;
                v[j] = in ? __ldcg(pc + 2 + t) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (c0 + j < nchunks) {
                    float w = expf(mm[j] - M);
                    L = fmaf(ll[j], w, L);
                    a = fmaf(v[j], w, a);
                }
            }
        }
        p.o[(size_t)(kh * G + g) * 128 + t] = a / L;
    }
}

int32_t check_decode(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len, brasa_arg o,
                     const brasa_attn_shape &sh) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, sh.tokens == 1, "decode_attention is for one token");
    BRASA_REQUIRE(ctx, sh.dim == 128, "decode_attention needs head_dim 128");
    BRASA_REQUIRE(ctx, sh.hkv > 0 && sh.hq % sh.hkv == 0 && sh.hq / sh.hkv <= 8, "decode_attention: GQA group must divide and be <= 8");
    BRASA_REQUIRE(ctx, sh.kv >= BRASA_KV_F32 && sh.kv <= BRASA_KV_Q8_0, "unknown KV type %d", sh.kv);
    BRASA_REQUIRE(ctx, sh.pos0 != 0xffffffffu, "decode_attention: position out of range");
    uint32_t lk = sh.pos0 + 1;
    BRASA_REQUIRE(ctx, partials_len >= brasa_decode_partials_len(sh.hq, lk) && arg_fits(partials, partials_len * 4), "decode scratch too small");
    uint64_t kvb = brasa_kv_bytes(sh.kv, (uint64_t)lk * sh.hkv * 128);
    BRASA_REQUIRE(ctx, arg_fits(q, (uint64_t)sh.hq * 512) && arg_fits(o, (uint64_t)sh.hq * 512) && arg_fits(k, kvb) && arg_fits(v, kvb),
                  "decode_attention: q, o or cache too small");
    BRASA_REQUIRE(ctx, k.offset % 16 == 0 && v.offset % 16 == 0 || sh.kv == BRASA_KV_Q8_0, "decode_attention: misaligned cache");
    return BRASA_OK;
}

int32_t decode_common(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len, brasa_arg o,
                      brasa_attn_shape sh) {
    BRASA_TRY(check_decode(cmd, q, k, v, partials, partials_len, o, sh));
    brasa_ctx *ctx = cmd->ctx;
    uint32_t lk = sh.pos0 + 1, chunks = (lk + 127) / 128;
    float scale = 1.0f / sqrtf((float)sh.dim);
    size_t smem = (128 * TS + 8 * D + 8 * 128 + 16) * sizeof(float);
    dim3 grid(chunks, sh.hkv);
    const float *qp = (const float *)arg_ptr(q);
    float *pp = (float *)arg_ptr(partials);
#define LAUNCH_DEC(KVT)                                                                                                   \
    do {                                                                                                                  \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_kernel<KVT>, smem)); \
        decode_partial_kernel<KVT><<<grid, 128, smem, ctx->stream>>>(qp, arg_ptr(k), arg_ptr(v), pp, sh.hq, sh.hkv, lk, scale); \
    } while (0)
    if (sh.kv == BRASA_KV_F32) LAUNCH_DEC(BRASA_KV_F32);
    else if (sh.kv == BRASA_KV_F16) LAUNCH_DEC(BRASA_KV_F16);
    else LAUNCH_DEC(BRASA_KV_Q8_0);
#undef LAUNCH_DEC
    BRASA_TRY(brasa_post_launch(cmd, "decode_partial"));
    decode_reduce_kernel<<<sh.hq, 128, 0, ctx->stream>>>(pp, (float *)arg_ptr(o), chunks);
    return brasa_post_launch(cmd, "decode_reduce");
}

}  // namespace

// Used by the model's decode graph. Launched with programmatic dependent launch so that the KV tile
// fetch overlaps the GEMV that produces q, k and v.
int32_t brasa_attn_decode_fused_launch(brasa_cmd *cmd, int32_t kv, const float *q, const float *k_new, const float *v_new, const float *q_norm,
                                       const float *k_norm, const float *cos_t, const float *sin_t, uint8_t *kc, uint8_t *vc, float *partials,
                                       uint32_t *counters, float *o, const uint32_t *pos, uint32_t hq, uint32_t hkv, uint32_t ctx_len, float eps) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, hkv > 0 && hq % hkv == 0 && hq / hkv <= 8, "fused decode attention: GQA group must divide and be <= 8");
    FusedAttnParams p{q, k_new, v_new, q_norm, k_norm, cos_t, sin_t, kc, vc, partials, counters, o, pos, hq, hkv, eps, 1.0f / sqrtf(128.0f)};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((ctx_len + 127) / 128, hkv);
    cfg.blockDim = dim3(128);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define LAUNCH_FUSED(KVT)                                                                                                          \
    do {                                                                                                                           \
        size_t smem = 2 * 128 * KvRow<KVT>::STRIDE + (8 * 128 * 2 + 16) * sizeof(float);                                           \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)attn_decode_fused_kernel<KVT>, smem)); \
        cfg.dynamicSmemBytes = smem;                                                                                               \
        BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, attn_decode_fused_kernel<KVT>, p));                                               \
    } while (0)
    if (kv == BRASA_KV_F32) LAUNCH_FUSED(BRASA_KV_F32);
    else if (kv == BRASA_KV_F16) LAUNCH_FUSED(BRASA_KV_F16);
    else LAUNCH_FUSED(BRASA_KV_Q8_0);
#undef LAUNCH_FUSED
    return brasa_post_launch(cmd, "attn_decode_fused");
}

extern "C" {

int32_t brasa_k_decode_attention(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len, brasa_arg o,
                                 brasa_attn_shape shape) {
    if (!cmd) return BRASA_EINVAL;
    return decode_common(cmd, q, k, v, partials, partials_len, o, shape);
}

int32_t brasa_k_decode_attention_lanes(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len,
                                       brasa_arg o, brasa_attn_shape shape) {
    if (!cmd) return BRASA_EINVAL;
    BRASA_REQUIRE(cmd->ctx, brasa_gqa_supported(shape.hq, shape.hkv), "decode_attention_lanes: GQA group not in {1, 2, 4, 8}");
    return decode_common(cmd, q, k, v, partials, partials_len, o, shape);
}

int32_t brasa_k_flash_attention_with(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o, brasa_attn_shape sh, int32_t precision) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, sh.dim == 128, "flash_attention needs head_dim 128");
    BRASA_REQUIRE(ctx, sh.hkv > 0 && sh.hq % sh.hkv == 0, "hq must be a multiple of hkv");
    BRASA_REQUIRE(ctx, sh.kv >= BRASA_KV_F32 && sh.kv <= BRASA_KV_Q8_0, "unknown KV type %d", sh.kv);
    BRASA_REQUIRE(ctx, precision == BRASA_PREFILL_F16 || precision == BRASA_PREFILL_F32, "unknown precision %d", precision);
    if (sh.tokens == 0) return BRASA_OK;
    uint64_t lk = (uint64_t)sh.pos0 + sh.tokens;
    uint64_t kvb = brasa_kv_bytes(sh.kv, lk * sh.hkv * 128);
    uint64_t qn = (uint64_t)sh.tokens * sh.hq * 128;
    bool half_io = precision == BRASA_PREFILL_F16;
    BRASA_REQUIRE(ctx, arg_fits(q, qn * 4) && arg_fits(o, qn * (half_io ? 2 : 4)) && arg_fits(k, kvb) && arg_fits(v, kvb), "flash_attention: buffers too small");
    // the F16 precision runs on the tensor cores (BRASA_FLASH_TC=0 keeps the f32 kernel below)
    static const bool tc_on = [] { const char *e = getenv("BRASA_FLASH_TC"); return !(e && e[0] == '0'); }();
    if (half_io && tc_on && k.offset % 16 == 0 && v.offset % 16 == 0 && q.offset % 16 == 0 && o.offset % 16 == 0)
        return brasa_flash_tc_launch(cmd, sh.kv, (const float *)arg_ptr(q), arg_ptr(k), arg_ptr(v), (__half *)arg_ptr(o), sh);
    float scale = 1.0f / sqrtf((float)sh.dim);
    size_t smem = ((64 + 32 + 32) * TS + 64 * 33 + 3 * 64) * sizeof(float);
    dim3 grid((sh.tokens + 63) / 64, sh.hq);
#define LAUNCH_FA(KVT, H)                                                                                                    \
    do {                                                                                                                     \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)prefill_attn_kernel<KVT, H>, smem)); \
        prefill_attn_kernel<KVT, H><<<grid, 256, smem, ctx->stream>>>((const float *)arg_ptr(q), arg_ptr(k), arg_ptr(v), arg_ptr(o), sh.tokens, \
                                                                      sh.hq, sh.hkv, sh.pos0, scale);                      \
    } while (0)
    if (half_io) {
        if (sh.kv == BRASA_KV_F32) LAUNCH_FA(BRASA_KV_F32, true);
        else if (sh.kv == BRASA_KV_F16) LAUNCH_FA(BRASA_KV_F16, true);
        else LAUNCH_FA(BRASA_KV_Q8_0, true);
    } else {
        if (sh.kv == BRASA_KV_F32) LAUNCH_FA(BRASA_KV_F32, false);
        else if (sh.kv == BRASA_KV_F16) LAUNCH_FA(BRASA_KV_F16, false);
        else LAUNCH_FA(BRASA_KV_Q8_0, false);
    }
#undef LAUNCH_FA
    return brasa_post_launch(cmd, "prefill_attention");
}

int32_t brasa_k_flash_attention(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o_f16, brasa_attn_shape shape) {
    return brasa_k_flash_attention_with(cmd, q, k, v, o_f16, shape, BRASA_PREFILL_F16);
}

int32_t brasa_k_decode_attention_static(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o, brasa_attn_shape shape) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, shape.hq <= STATIC_MAX_HQ && (uint64_t)shape.pos0 + 1 <= STATIC_MAX_KEYS,
                  "decode_attention_static holds scratch for at most %u query heads and %u keys (got %u heads, %llu keys); use "
                  "brasa_k_decode_attention with a caller-allocated scratch buffer for larger shapes",
                  STATIC_MAX_HQ, STATIC_MAX_KEYS, shape.hq, (unsigned long long)shape.pos0 + 1);
    // In host code the array's name stands for the symbol, not for device memory: each device has its own
    // copy, whose address is looked up once per device with that device current.
    static float *scratch_of_device[64] = {};
    BRASA_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "device index %d out of range", ctx->device);
    if (!scratch_of_device[ctx->device]) {
        BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
        float *ptr = nullptr;
        BRASA_CUDA(ctx, cudaGetSymbolAddress((void **)&ptr, g_decode_partials));
        scratch_of_device[ctx->device] = ptr;
    }
    float *partials = scratch_of_device[ctx->device];
    // same checks and launches as brasa_k_decode_attention, minus the scratch argument
    BRASA_REQUIRE(ctx, shape.tokens == 1, "decode_attention is for one token");
    BRASA_REQUIRE(ctx, shape.dim == 128, "decode_attention needs head_dim 128");
    BRASA_REQUIRE(ctx, shape.hkv > 0 && shape.hq % shape.hkv == 0 && shape.hq / shape.hkv <= 8, "decode_attention: GQA group must divide and be <= 8");
    BRASA_REQUIRE(ctx, shape.kv >= BRASA_KV_F32 && shape.kv <= BRASA_KV_Q8_0, "unknown KV type %d", shape.kv);
    const uint32_t lk = shape.pos0 + 1, chunks = (lk + 127) / 128;
    const uint64_t kvb = brasa_kv_bytes(shape.kv, (uint64_t)lk * shape.hkv * 128);
    BRASA_REQUIRE(ctx, arg_fits(q, (uint64_t)shape.hq * 512) && arg_fits(o, (uint64_t)shape.hq * 512) && arg_fits(k, kvb) && arg_fits(v, kvb),
                  "decode_attention_static: q, o or cache too small");
    BRASA_REQUIRE(ctx, shape.kv == BRASA_KV_Q8_0 || (k.offset % 16 == 0 && v.offset % 16 == 0), "decode_attention_static: misaligned cache");
    const float scale = 1.0f / sqrtf((float)shape.dim);
    const size_t smem = (128 * TS + 8 * D + 8 * 128 + 16) * sizeof(float);
    dim3 grid(chunks, shape.hkv);
    const float *qp = (const float *)arg_ptr(q);
#define LAUNCH_STATIC(KVT)                                                                                                 \
    do {                                                                                                                   \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_kernel<KVT>, smem)); \
        decode_partial_kernel<KVT><<<grid, 128, smem, ctx->stream>>>(qp, arg_ptr(k), arg_ptr(v), partials, shape.hq, shape.hkv, lk, scale); \
    } while (0)
    if (shape.kv == BRASA_KV_F32) LAUNCH_STATIC(BRASA_KV_F32);
    else if (shape.kv == BRASA_KV_F16) LAUNCH_STATIC(BRASA_KV_F16);
    else LAUNCH_STATIC(BRASA_KV_Q8_0);
#undef LAUNCH_STATIC
    BRASA_TRY(brasa_post_launch(cmd, "decode_partial"));
    decode_reduce_kernel<<<shape.hq, 128, 0, ctx->stream>>>(partials, (float *)arg_ptr(o), chunks);
    return brasa_post_launch(cmd, "decode_reduce");
}

}  // extern "C"

