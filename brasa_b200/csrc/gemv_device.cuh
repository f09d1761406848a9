// Device-side pieces shared by the GEMV kernel and the whole-token decode kernel: mbarrier and bulk-copy wrappers,
// the fixed-point form of the input vector and the exact integer dot product of a half block (see gemv.cu).
#pragma once
#include "brasa_internal.h"

namespace brasa_dev {

constexpr uint32_t WAIT_LIMIT = 1u << 20;  // try_wait rounds before a wait gives up

__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. False when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    int r;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {  // unsigned codes x signed bytes
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// The lane's x values of one half block in fixed point with P byte planes: quad j (4 values) x plane d (the top plane
// signed, the others unsigned), the sum of the 16 integers, and the power-of-two step. The 16 values share the step
// 2^(e - 20) (P = 3) or 2^(e - 14) (P = 2), e the exponent of the largest magnitude among them, and the integer dot
// products are exact.
//   P = 3: 22 bits below the group's largest value per element, the accuracy class of an f32 dot product (the
//          stand-alone GEMV entry points, and every decode path of a model with an f32 cache);
//   P = 2: 15 bits, an order of magnitude inside the 1e-5 * sum |w x| the reference allows its own f32 GEMV
//          (crates/kernels/src/lib.rs:13) and one third fewer integer operations: the whole-token kernel of models
//          whose cache is f16 or q8_0, where the reference's own logits bound is 1e-3 / 2e-2
//          (crates/models/tests/forward.rs:40-55).
template <int P>
struct XFixed {
    uint32_t d[4][P];
    int total;
    float step;
};
// 16-byte chunks of a record in shared memory: 4 P plane words, the total, the step
template <int P>
struct XRec {
    static constexpr uint32_t CHUNKS = P == 3 ? 4 : 3;
};

// Record hbi from shared memory. P = 3: 64-byte records, chunk c of record h stored at chunk c ^ ((h >> 1) & 3)
// (conflict-free for consecutive h). P = 2: 48-byte records; every quarter warp covers all 32 banks once, no swizzle.
template <int P>
__device__ __forceinline__ XFixed<P> x_fixed_load(const uint4 *xf, uint32_t hbi) {
    XFixed<P> x;
    if (P == 3) {
        const uint32_t sw = (hbi >> 1) & 3;
        const uint4 c0 = xf[hbi * 4 + (0 ^ sw)], c1 = xf[hbi * 4 + (1 ^ sw)], c2 = xf[hbi * 4 + (2 ^ sw)], c3 = xf[hbi * 4 + (3 ^ sw)];
        const uint32_t w[12] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int d = 0; d < P; ++d) x.d[j][d] = w[P * j + d];
        x.total = (int)c3.x;
        x.step = __uint_as_float(c3.y);
    } else {
        const uint4 c0 = xf[hbi * 3], c1 = xf[hbi * 3 + 1], c2 = xf[hbi * 3 + 2];
        const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int d = 0; d < P; ++d) x.d[j][d] = w[P * j + d];
        x.total = (int)c2.x;
        x.step = __uint_as_float(c2.y);
    }
    return x;
}

// sum over the 16 weights of a half block of (code - bias) * X, as an integer.
// Quads: 0 = low nibbles of word x, 1 = high nibbles of word x, 2 and 3 likewise for word y.
template <int QT, int P>
__device__ __forceinline__ int half_block_idot(uint2 codes, uint32_t hb, const XFixed<P> &x) {
    uint32_t a[4];
    a[0] = codes.x & 0x0F0F0F0Fu;
    a[1] = (codes.x >> 4) & 0x0F0F0F0Fu;
    a[2] = codes.y & 0x0F0F0F0Fu;
    a[3] = (codes.y >> 4) & 0x0F0F0F0Fu;
    if (QT == BRASA_Q6_0) {  // the two high bits of each code, stored so a shift puts them at bits 4-5 of its byte
        a[0] = lop_and_or(hb, 0x30303030u, a[0]);
        a[1] = lop_and_or(hb >> 2, 0x30303030u, a[1]);
        a[2] = lop_and_or(hb << 2, 0x30303030u, a[2]);
        a[3] = lop_and_or(hb << 4, 0x30303030u, a[3]);
    }
    constexpr int BIAS = QT == BRASA_Q4_0 ? 8 : 32;
    int s[P];
    s[0] = -BIAS * x.total;
#pragma unroll
    for (int d = 1; d < P; ++d) s[d] = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int d = 0; d < P; ++d) s[d] = d == P - 1 ? dp4a_us(a[j], x.d[j][d], s[d]) : dp4a_uu(a[j], x.d[j][d], s[d]);
    }
    int r = s[0];
#pragma unroll
    for (int d = 1; d < P; ++d) r += s[d] << (8 * d);
    return r;
}

// Dot products of two rows of a slot with the lane's share of x (row_b == row_a when there is only one).
// After folding across lanes, lane 0 holds the sum of row a and lane 8 the sum of row b. The body is kept
// small on purpose: a fully unrolled four-row version ran out of instruction cache.
template <int QT, int N, int P>
__device__ __forceinline__ float row_pair_dot(const uint8_t *row_a, const uint8_t *row_b, const XFixed<P> (&xr)[N], uint32_t slice, uint32_t nhb,
                                              uint32_t hi_off, uint32_t sc_off, int lane, int nact = N) {
    float acc_a = 0.0f, acc_b = 0.0f;
    // straight-line code: lanes past the end of the row read the last half block and have step 0
#pragma unroll
    for (int it = 0; it < N; ++it) {
        if (it < nact) {  // nact < N: a narrower input in a kernel built for N (uniform across the block)
            const uint32_t hbi = min((slice * nact + it) * 32 + lane, nhb - 1);
            uint2 ca = *reinterpret_cast<const uint2 *>(row_a + hbi * 8);
            uint2 cb = *reinterpret_cast<const uint2 *>(row_b + hbi * 8);
            uint32_t ha = 0, hb = 0;
            if (QT == BRASA_Q6_0) {
                ha = *reinterpret_cast<const uint32_t *>(row_a + hi_off + hbi * 4);
                hb = *reinterpret_cast<const uint32_t *>(row_b + hi_off + hbi * 4);
            }
            float da = __half2float(*reinterpret_cast<const __half *>(row_a + sc_off + (hbi >> 1) * 2));
            float db = __half2float(*reinterpret_cast<const __half *>(row_b + sc_off + (hbi >> 1) * 2));
            int sa = half_block_idot<QT, P>(ca, ha, xr[it]);
            int sb = half_block_idot<QT, P>(cb, hb, xr[it]);
            acc_a = fmaf(da * xr[it].step, (float)sa, acc_a);
            acc_b = fmaf(db * xr[it].step, (float)sb, acc_b);
        }
    }
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 16);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 16);
    const bool hi3 = lane & 8;
    float z = hi3 ? acc_b : acc_a, z_send = hi3 ? acc_a : acc_b;
    z += __shfl_xor_sync(0xffffffffu, z_send, 8);
    z += __shfl_xor_sync(0xffffffffu, z, 4);
    z += __shfl_xor_sync(0xffffffffu, z, 2);
    z += __shfl_xor_sync(0xffffffffu, z, 1);
    return z;
}

// One row only (the last row of an odd count): every lane ends up with the sum.
template <int QT, int N, int P>
__device__ __forceinline__ float row_single_dot(const uint8_t *row_a, const XFixed<P> (&xr)[N], uint32_t slice, uint32_t nhb, uint32_t hi_off,
                                                uint32_t sc_off, int lane, int nact = N) {
    float acc_a = 0.0f;
#pragma unroll
    for (int it = 0; it < N; ++it) {
        if (it < nact) {
            const uint32_t hbi = min((slice * nact + it) * 32 + lane, nhb - 1);
            uint2 ca = *reinterpret_cast<const uint2 *>(row_a + hbi * 8);
            uint32_t ha = 0;
            if (QT == BRASA_Q6_0) ha = *reinterpret_cast<const uint32_t *>(row_a + hi_off + hbi * 4);
            float da = __half2float(*reinterpret_cast<const __half *>(row_a + sc_off + (hbi >> 1) * 2));
            int sa = half_block_idot<QT, P>(ca, ha, xr[it]);
            acc_a = fmaf(da * xr[it].step, (float)sa, acc_a);
        }
    }
    for (int o = 16; o > 0; o >>= 1) acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o);
    return acc_a;
}

// ---- the same dot products with every address worked out beforehand ----
// The rows of a ring slot lie in shared memory and a lane's half blocks are 32 apart, so for all iterations but the
// last one the loads are [row + lane offset + constant]; the last iteration, whose lanes may lie past the end of the
// row, uses offsets clamped once per operation. The bias term -BIAS * sum(X) is folded into the record when it is
// loaded (XFixed::total then holds it) and starts the first accumulator.
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

// Lane offsets inside a row: first half block (codes, scale, q6_0 high bits) and the clamped ones of the last iteration.
struct RowLaneOffsets {
    uint32_t c, s, h, lc, ls, lh;
};
template <int QT, int N>
__device__ __forceinline__ RowLaneOffsets row_lane_offsets(uint32_t cols, uint32_t slice, int lane) {
    const uint32_t nhb = cols / 16, first = slice * N * 32 + lane, last = min(first + (N - 1) * 32, nhb - 1);
    RowLaneOffsets o;
    o.c = first * 8;
    o.s = tiled_scale_off(QT, cols) + (first >> 1) * 2;
    o.h = tiled_hi_off(cols) + first * 4;
    o.lc = last * 8;
    o.ls = tiled_scale_off(QT, cols) + (last >> 1) * 2;
    o.lh = tiled_hi_off(cols) + last * 4;
    return o;
}

template <int QT, int P>
__device__ __forceinline__ int half_block_idot_pre(uint2 codes, uint32_t hb, const XFixed<P> &x) {  // x.total = -BIAS * sum(X)
    uint32_t a[4];
    a[0] = codes.x & 0x0F0F0F0Fu;
    a[1] = (codes.x >> 4) & 0x0F0F0F0Fu;
    a[2] = codes.y & 0x0F0F0F0Fu;
    a[3] = (codes.y >> 4) & 0x0F0F0F0Fu;
    if (QT == BRASA_Q6_0) {
        a[0] = lop_and_or(hb, 0x30303030u, a[0]);
        a[1] = lop_and_or(hb >> 2, 0x30303030u, a[1]);
        a[2] = lop_and_or(hb << 2, 0x30303030u, a[2]);
        a[3] = lop_and_or(hb << 4, 0x30303030u, a[3]);
    }
    int s[P];
    s[0] = x.total;
#pragma unroll
    for (int d = 1; d < P; ++d) s[d] = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int d = 0; d < P; ++d) s[d] = d == P - 1 ? dp4a_us(a[j], x.d[j][d], s[d]) : dp4a_uu(a[j], x.d[j][d], s[d]);
    }
    int r = s[0];
#pragma unroll
    for (int d = 1; d < P; ++d) r += s[d] << (8 * d);
    return r;
}

// Two rows at shared addresses ra, rb. After folding across lanes, lane 0 holds the sum of row a and lane 8 that of row b.
template <int QT, int N, int P>
__device__ __forceinline__ float row_pair_dot_at(uint32_t ra, uint32_t rb, const RowLaneOffsets &o, const XFixed<P> (&xr)[N], int lane) {
    float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll
    for (int it = 0; it < N; ++it) {
        const bool last = it == N - 1;
        const uint32_t oc = last ? o.lc : o.c + it * 256, os = last ? o.ls : o.s + it * 32, oh = last ? o.lh : o.h + it * 128;
        const uint2 ca = lds_u64(ra + oc), cb = lds_u64(rb + oc);
        uint32_t ha = 0, hb = 0;
        if (QT == BRASA_Q6_0) {
            ha = lds_u32(ra + oh);
            hb = lds_u32(rb + oh);
        }
        const float da = lds_f16(ra + os), db = lds_f16(rb + os);
        const int sa = half_block_idot_pre<QT, P>(ca, ha, xr[it]);
        const int sb = half_block_idot_pre<QT, P>(cb, hb, xr[it]);
        acc_a = fmaf(da * xr[it].step, (float)sa, acc_a);
        acc_b = fmaf(db * xr[it].step, (float)sb, acc_b);
    }
    acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 16);
    acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 16);
    const bool hi3 = lane & 8;
    float z = hi3 ? acc_b : acc_a, z_send = hi3 ? acc_a : acc_b;
    z += __shfl_xor_sync(0xffffffffu, z_send, 8);
    z += __shfl_xor_sync(0xffffffffu, z, 4);
    z += __shfl_xor_sync(0xffffffffu, z, 2);
    z += __shfl_xor_sync(0xffffffffu, z, 1);
    return z;
}

template <int QT, int N, int P>
__device__ __forceinline__ float row_single_dot_at(uint32_t ra, const RowLaneOffsets &o, const XFixed<P> (&xr)[N]) {
    float acc_a = 0.0f;
#pragma unroll
    for (int it = 0; it < N; ++it) {
        const bool last = it == N - 1;
        const uint32_t oc = last ? o.lc : o.c + it * 256, os = last ? o.ls : o.s + it * 32, oh = last ? o.lh : o.h + it * 128;
        const uint2 ca = lds_u64(ra + oc);
        uint32_t ha = 0;
        if (QT == BRASA_Q6_0) ha = lds_u32(ra + oh);
        const float da = lds_f16(ra + os);
        const int sa = half_block_idot_pre<QT, P>(ca, ha, xr[it]);
        acc_a = fmaf(da * xr[it].step, (float)sa, acc_a);
    }
    for (int o2 = 16; o2 > 0; o2 >>= 1) acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o2);
    return acc_a;
}

// x to fixed point with P byte planes: one half block (16 values, as the four quads that meet the low / high nibbles
// of code word 0 and of code word 1) becomes a record in xf: 4 P byte-plane words, the sum of the integers, the step.
template <int P>
__device__ __forceinline__ void x_half_block_to_fixed(uint4 *xf, uint32_t hbi, float4 q0, float4 q1, float4 q2, float4 q3) {
    constexpr uint32_t BITS = P == 3 ? 22 : 16;  // |x| / step stays below 2^(BITS - 1): 21 (P = 3) or 15 (P = 2)
    float v[4][4] = {{q0.x, q0.y, q0.z, q0.w}, {q1.x, q1.y, q1.z, q1.w}, {q2.x, q2.y, q2.z, q2.w}, {q3.x, q3.y, q3.z, q3.w}};
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(v[j][e]));
    // step = 2^(exponent(amax) - (BITS - 2)); zero (or denormal) groups get step 0
    uint32_t ebits = __float_as_uint(amax) & 0x7F800000u;
    bool live = ebits > ((BITS - 1) << 23) && ebits < 0x7F800000u;
    // infinities and NaNs are not representable: their group's step carries them into the result
    float step = live ? __uint_as_float(ebits - ((BITS - 2) << 23)) : (ebits == 0x7F800000u ? amax : 0.0f);
    float inv = live ? __uint_as_float((254u << 23) - (ebits - ((BITS - 2) << 23))) : 0.0f;  // 1 / step, exact
    int total = 0;
    uint32_t rec[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int X[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            X[e] = __float2int_rn(v[j][e] * inv);
            if (P == 2) X[e] = min(X[e], 32767);  // a value that rounds up to 2^15 stays inside the signed top byte
            total += X[e];
        }
        // byte planes of the four integers: byte k of every X gathered into one word
        uint32_t lo01 = __byte_perm(X[0], X[1], 0x5140), lo23 = __byte_perm(X[2], X[3], 0x5140);
        rec[P * j + 0] = __byte_perm(lo01, lo23, 0x5410);
        rec[P * j + 1] = __byte_perm(lo01, lo23, 0x7632);
        if (P == 3) {
            uint32_t hi01 = __byte_perm(X[0], X[1], 0x7362), hi23 = __byte_perm(X[2], X[3], 0x7362);
            rec[P * j + 2] = __byte_perm(hi01, hi23, 0x5410);
        }
    }
    rec[4 * P] = (uint32_t)total;
    rec[4 * P + 1] = __float_as_uint(step);
    rec[4 * P + 2] = rec[4 * P + 3] = 0;
    if (P == 3) {
        const uint32_t sw = (hbi >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 4; ++c) xf[hbi * 4 + (c ^ sw)] = make_uint4(rec[4 * c], rec[4 * c + 1], rec[4 * c + 2], rec[4 * c + 3]);
    } else {
#pragma unroll
        for (int c = 0; c < 3; ++c) xf[hbi * 3 + c] = make_uint4(rec[4 * c], rec[4 * c + 1], rec[4 * c + 2], rec[4 * c + 3]);
    }
}

}  // namespace brasa_dev
