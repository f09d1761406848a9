// Decode GEMVs: y = W x for quantised W (q4_0 / q6_0 in the tiled layout), one token.
//
// The reference's GEMV family (crates/kernels/src/lib.rs:633-838 and the MSL bodies it dispatches)
// is HBM-bound: every weight byte is read once per token. On B200 the matrices are small next to
// the machine (o_proj is 40 KB per SM), so the kernel is built around three things:
//   * weights move HBM -> shared memory with bulk async copies (cp.async.bulk + mbarrier), issued
//     by one thread before the kernel waits for its input vector (programmatic dependent launch),
//     so the stream of weight bytes does not stop at kernel boundaries;
//   * work is cut into 4.6 KB micro-tiles (64 rows x 128 columns) spread evenly over all SMs
//     (split-K); the warp that completes a 64-row group sums its partials in a fixed order, so the
//     result is deterministic, and applies the epilogue (RMSNorm scale, SwiGLU);
//   * one lane owns one row (two per warp pass): x is read from shared memory as a warp-wide
//     broadcast, codes as conflict-free 128-bit loads, no cross-lane reduction is needed.
// Dequantisation is fused and exact: a 4-bit (6-bit) code is OR-ed into the mantissa of 2^23, the
// constant is subtracted (packed f32x2 add), and the product with the pre-scaled x is accumulated
// in f32 (packed f32x2 fma): (q - 8) * 16^k * (x * 16^-k).
#include <type_traits>

#include "brasa_internal.h"

namespace {

constexpr int CONSUMER_WARPS = 8;
constexpr int GEMV_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // try_wait rounds before a wait gives up

enum { EPI_SCALE = 0, EPI_SWIGLU = 1 };

struct GemvParams {
    const uint8_t *w[3];
    float *y[3];
    uint32_t mt_count[3];  // micro-tiles per matrix
    uint32_t nmat;
    uint32_t cols, nkc;    // nkc = cols / 128 micro-tile columns
    uint32_t total_mt;
    uint32_t nslot;        // ring slots in shared memory
    int epilogue;
    // input vector: either `x` alone (already multiplied by the norm weight, reference form, with
    // optional partial sums ss[nss] of x^2), or x (+ h) with norm weight for the fused form
    const float *x, *h, *normw, *ss;
    float *x_out;          // fused form: block 0 writes x + h here
    uint32_t nss;
    int scaled;            // multiply outputs by 1/sqrt(mean(x^2) + eps)
    float eps;
    float *partials;
    uint32_t *counters;
    uint32_t *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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

typedef unsigned long long f2;  // two packed floats
__device__ __forceinline__ f2 pack2(float a, float b) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ f2 pack2u(uint32_t a, uint32_t b) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
    f2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
    f2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float sum2(f2 a) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a));
    return lo + hi;
}
__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

constexpr uint32_t MAGIC = 0x4B000000u;  // 2^23 as float bits: the code becomes the low mantissa

// Adds the dot products of one 8-code word `a` (and, for q6_0, the aligned high-bit words) with
// the 8 pre-scaled x values {x01, x23, x45, x67} to acc.
template <int QT>
__device__ __forceinline__ f2 word_dot(uint32_t a, uint32_t hb, f2 x01, f2 x23, f2 x45, f2 x67, f2 c01, f2 c23, f2 acc) {
    uint32_t ah = a >> 16;
    uint32_t f0, f1, f2_, f3, f4, f5, f6, f7;
    f0 = lop_and_or(a, 0x000Fu, MAGIC);
    f1 = lop_and_or(a, 0x00F0u, MAGIC);
    f2_ = lop_and_or(a, 0x0F00u, MAGIC);
    f3 = lop_and_or(a, 0xF000u, MAGIC);
    f4 = lop_and_or(ah, 0x000Fu, MAGIC);
    f5 = lop_and_or(ah, 0x00F0u, MAGIC);
    f6 = lop_and_or(ah, 0x0F00u, MAGIC);
    f7 = lop_and_or(ah, 0xF000u, MAGIC);
    if (QT == BRASA_Q6_0) {
        uint32_t hh = hb >> 2;
        f0 = lop_and_or(hb, 0x00030u, f0);
        f1 = lop_and_or(hb, 0x00300u, f1);
        f2_ = lop_and_or(hb, 0x03000u, f2_);
        f3 = lop_and_or(hb, 0x30000u, f3);
        f4 = lop_and_or(hh, 0x00030u, f4);
        f5 = lop_and_or(hh, 0x00300u, f5);
        f6 = lop_and_or(hh, 0x03000u, f6);
        f7 = lop_and_or(hh, 0x30000u, f7);
    }
    acc = fma2(add2(pack2u(f0, f1), c01), x01, acc);
    acc = fma2(add2(pack2u(f2_, f3), c23), x23, acc);
    acc = fma2(add2(pack2u(f4, f5), c01), x45, acc);
    acc = fma2(add2(pack2u(f6, f7), c23), x67, acc);
    return acc;
}

// One micro-tile (64 rows x 4 blocks) against xs (this column chunk's 128 pre-scaled values).
// Lane owns rows `lane` and `lane + 32`.
template <int QT>
__device__ __forceinline__ void microtile_dot(const uint8_t *tile, const float *xs, int lane, float &out0, float &out1) {
    constexpr int NSLOT = MT_BLOCKS * MT_ROWS;
    constexpr float BIAS = QT == BRASA_Q4_0 ? 8.0f : 32.0f;
    const f2 c01 = pack2(-(8388608.0f + BIAS), -(8388608.0f + BIAS * 16.0f));
    const f2 c23 = pack2(-(8388608.0f + BIAS * 256.0f), -(8388608.0f + BIAS * 4096.0f));
    const uint4 *codes = reinterpret_cast<const uint4 *>(tile);
    const uint2 *hi = reinterpret_cast<const uint2 *>(tile + NSLOT * 16);
    const __half *sc = reinterpret_cast<const __half *>(tile + NSLOT * (QT == BRASA_Q4_0 ? 16 : 24));
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int blk = 0; blk < MT_BLOCKS; ++blk) {
        int s0 = blk * MT_ROWS + lane, s1 = s0 + 32;
        uint4 p0 = codes[s0], p1 = codes[s1];
        float d0 = __half2float(sc[s0]), d1 = __half2float(sc[s1]);
        uint2 h0 = make_uint2(0, 0), h1 = make_uint2(0, 0);
        if (QT == BRASA_Q6_0) { h0 = hi[s0]; h1 = hi[s1]; }
        const ulonglong2 *xv = reinterpret_cast<const ulonglong2 *>(xs + blk * 32);
        f2 acc0 = 0ull, acc1 = 0ull;
        uint32_t w0[4] = {p0.x, p0.y, p0.z, p0.w}, w1[4] = {p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            ulonglong2 xa = xv[2 * w], xb = xv[2 * w + 1];  // warp-wide broadcast
            uint32_t hb0 = (w & 2) ? h0.y : h0.x, hb1 = (w & 2) ? h1.y : h1.x;
            if (QT == BRASA_Q6_0 && (w & 1)) {
                hb0 = __funnelshift_r(hb0, hb0, 16);
                hb1 = __funnelshift_r(hb1, hb1, 16);
            }
            acc0 = word_dot<QT>(w0[w], hb0, xa.x, xa.y, xb.x, xb.y, c01, c23, acc0);
            acc1 = word_dot<QT>(w1[w], hb1, xa.x, xa.y, xb.x, xb.y, c01, c23, acc1);
        }
        a0 = fmaf(d0, sum2(acc0), a0);
        a1 = fmaf(d1, sum2(acc1), a1);
    }
    out0 = a0;
    out1 = a1;
}

template <int QT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_tiled_kernel(GemvParams p) {
    constexpr int MTB = QT == BRASA_Q4_0 ? MT_BYTES_Q4 : MT_BYTES_Q6;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: ring [nslot][MTB] | xs [cols] floats | barriers | red
    uint8_t *ring = smem;
    float *xs = reinterpret_cast<float *>(smem + (size_t)p.nslot * MTB);
    uint64_t *full = reinterpret_cast<uint64_t *>(xs + p.cols);
    uint64_t *empty = full + p.nslot;
    float *red = reinterpret_cast<float *>(empty + p.nslot);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t G = gridDim.x, b = blockIdx.x;
    const uint32_t m0 = (uint32_t)((uint64_t)p.total_mt * b / G), m1 = (uint32_t)((uint64_t)p.total_mt * (b + 1) / G);
    const uint32_t items = m1 - m0;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.nslot; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel of the stream start its own weight prefetch.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    auto tile_src = [&](uint32_t m) -> const uint8_t * {
        uint32_t mi = 0;
        while (mi + 1 < p.nmat && m >= p.mt_count[mi]) { m -= p.mt_count[mi]; ++mi; }
        return p.w[mi] + (size_t)m * MTB;
    };

    uint32_t issued = 0;
    if (warp == CONSUMER_WARPS && lane == 0) {
        // weights are immutable: the first ring-full of copies starts before the input is ready
        uint32_t first = items < p.nslot ? items : p.nslot;
        for (; issued < first; ++issued) {
            mbar_expect_tx(&full[issued], MTB);
            bulk_g2s(ring + (size_t)issued * MTB, tile_src(m0 + issued), MTB, &full[issued]);
        }
    }
    // Everything below depends on the previous kernel's output.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == CONSUMER_WARPS) {
        if (lane == 0) {
            bool ok = true;
            for (; issued < items && ok; ++issued) {
                uint32_t s = issued % p.nslot, round = issued / p.nslot;
                ok = mbar_wait(&empty[s], (round - 1) & 1);
                if (!ok) break;
                mbar_expect_tx(&full[s], MTB);
                bulk_g2s(ring + (size_t)s * MTB, tile_src(m0 + issued), MTB, &full[s]);
            }
            if (!ok) atomicExch(p.status, 1u);
        }
        // the producer warp takes no part in the block-wide sums below: consumers use named barrier 1
        return;
    }

    // ---- stage x: permuted and pre-scaled so that each code meets its x in mantissa position ----
    const int ct = threadIdx.x, CT = CONSUMER_WARPS * 32;
    float ssq = 0.0f;
    for (uint32_t j = ct; j < p.cols; j += CT) {
        float v = p.x[j];
        if (p.h) v += p.h[j];
        if (p.x_out && b == 0) p.x_out[j] = v;
        ssq += v * v;
        if (p.normw) v *= p.normw[j];
        uint32_t blk = j >> 5, e = j & 31;
        uint32_t k = 2 * (e & 3) + (e >> 4), w = (e & 15) >> 2;
        float sc = (k & 3) == 0 ? 1.0f : ((k & 3) == 1 ? 0.0625f : ((k & 3) == 2 ? 0.00390625f : 0.000244140625f));
        xs[blk * 32 + w * 8 + k] = v * sc;
    }
    float scale = 1.0f;
    if (p.scaled) {
        float tot;
        if (p.ss) {  // reference form: fixed-order sum of add_norm_prep's partials
            tot = 0.0f;
            for (uint32_t i = 0; i < p.nss; ++i) tot += p.ss[i];
        } else {
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) red[warp] = ssq;
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            tot = 0.0f;
            for (int i = 0; i < CONSUMER_WARPS; ++i) tot += red[i];
        }
        scale = 1.0f / sqrtf(tot / (float)p.cols + p.eps);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");

    // ---- consume micro-tiles ----
    const uint32_t contributors = p.nkc * (p.epilogue == EPI_SWIGLU ? 2u : 1u);
    for (uint32_t i = warp; i < items; i += CONSUMER_WARPS) {
        uint32_t s = i % p.nslot, round = i / p.nslot;
        if (!mbar_wait(&full[s], round & 1)) {
            if (lane == 0) atomicExch(p.status, 2u);
            return;
        }
        uint32_t m = m0 + i;          // logical micro-tile
        uint32_t rt = m / p.nkc, c = m % p.nkc;  // 64-row group (over all matrices) and column chunk
        float v0, v1;
        microtile_dot<QT>(ring + (size_t)s * MTB, xs + c * 128, lane, v0, v1);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        float *part = p.partials + (size_t)m * MT_ROWS;
        __stcg(part + lane, v0);
        __stcg(part + lane + 32, v1);
        __threadfence();
        __syncwarp();
        // which counter: SwiGLU pairs the gate and up groups of the same rows
        uint32_t rt_gate = 0, ci = rt;
        if (p.epilogue == EPI_SWIGLU) {
            uint32_t per = p.mt_count[0] / p.nkc;
            rt_gate = rt % per;
            ci = rt_gate;
        }
        uint32_t old = 0;
        if (lane == 0) old = atomicAdd(&p.counters[ci], 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != contributors - 1) continue;
        // last to arrive for this row group: fixed-order sum of all column chunks, epilogue, store
        __threadfence();
        if (lane == 0) p.counters[ci] = 0;
        if (p.epilogue == EPI_SWIGLU) {
            uint32_t per = p.mt_count[0] / p.nkc;
            const float *pg = p.partials + (size_t)rt_gate * p.nkc * MT_ROWS;
            const float *pu = p.partials + (size_t)(per + rt_gate) * p.nkc * MT_ROWS;
            float g0 = 0, g1 = 0, u0 = 0, u1 = 0;
            for (uint32_t cc = 0; cc < p.nkc; ++cc) {
                g0 += __ldcg(pg + cc * MT_ROWS + lane);
                g1 += __ldcg(pg + cc * MT_ROWS + lane + 32);
                u0 += __ldcg(pu + cc * MT_ROWS + lane);
                u1 += __ldcg(pu + cc * MT_ROWS + lane + 32);
            }
            g0 *= scale; g1 *= scale; u0 *= scale; u1 *= scale;
            float *y = p.y[0] + (size_t)rt_gate * MT_ROWS;
            y[lane] = (g0 / (1.0f + expf(-g0))) * u0;
            y[lane + 32] = (g1 / (1.0f + expf(-g1))) * u1;
        } else {
            const float *pp = p.partials + (size_t)rt * p.nkc * MT_ROWS;
            float t0 = 0, t1 = 0;
            for (uint32_t cc = 0; cc < p.nkc; ++cc) {
                t0 += __ldcg(pp + cc * MT_ROWS + lane);
                t1 += __ldcg(pp + cc * MT_ROWS + lane + 32);
            }
            uint32_t mi = 0, r = rt;
            while (mi + 1 < p.nmat && r >= p.mt_count[mi] / p.nkc) { r -= p.mt_count[mi] / p.nkc; ++mi; }
            float *y = p.y[mi] + (size_t)r * MT_ROWS;
            y[lane] = t0 * scale;
            y[lane + 32] = t1 * scale;
        }
    }
}

// ---- file-layout fallback: one warp per row, any shape (cols % 32 == 0) ----------------------
template <int QT>
__global__ void gemv_file_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, uint32_t rows,
                                 uint32_t cols, const float *ss, uint32_t nss, float eps, int scaled) {
    constexpr int BB = QT == BRASA_Q4_0 ? 18 : (QT == BRASA_Q6_0 ? 26 : 34);
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), t = blockIdx.y, lane = threadIdx.x & 31;
    if (row >= rows) return;
    uint32_t nb = cols / 32;
    const uint8_t *wr = w + (size_t)row * nb * BB;
    const float *xt = x + (size_t)t * cols;
    float acc = 0.0f;
    for (uint32_t bi = lane; bi < nb; bi += 32) {
        const uint8_t *p = wr + (size_t)bi * BB;
        float d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(p)));
        const float *xb = xt + bi * 32;
        float s = 0.0f;
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
            s = fmaf((float)q, xb[j], s);
        }
        acc = fmaf(d, s, acc);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        float scale = 1.0f;
        if (scaled) {
            float tot = 0.0f;
            for (uint32_t i = 0; i < nss; ++i) tot += ss[i];
            scale = 1.0f / sqrtf(tot / (float)cols + eps);
        }
        y[(size_t)t * rows + row] = acc * scale;
    }
}

__global__ void swiglu_inplace_kernel(float *g, const float *u, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float a = g[i];
        g[i] = (a / (1.0f + expf(-a))) * u[i];
    }
}

}  // namespace

// Shared by the model's fused decode path (model.cu) and the reference-shaped entry points below.
int32_t brasa_gemv_launch(brasa_cmd *cmd, int qtype, uint32_t nmat, const brasa_qmatrix *w, float *const *y, const float *x,
                          const float *h, const float *normw, float *x_out, const float *ss, uint32_t nss, int scaled, float eps,
                          int epilogue) {
    brasa_ctx *ctx = cmd->ctx;
    GemvParams p{};
    p.nmat = nmat;
    p.cols = w[0].cols;
    p.nkc = p.cols / (32 * MT_BLOCKS);
    uint32_t total = 0, groups = 0;
    for (uint32_t i = 0; i < nmat; ++i) {
        BRASA_REQUIRE(ctx, w[i].layout == BRASA_LAYOUT_TILED && w[i].qtype == qtype && w[i].cols == p.cols && tiled_ok(qtype, w[i].rows, w[i].cols),
                      "gemv: matrix %u is not a tiled %s matrix of %u columns", i, qtype == BRASA_Q4_0 ? "q4_0" : "q6_0", p.cols);
        BRASA_REQUIRE(ctx, qm_fits(w[i]) && w[i].data.offset % 16 == 0, "gemv: matrix %u exceeds its buffer or is misaligned", i);
        p.w[i] = arg_ptr(w[i].data);
        p.y[i] = y[i];
        p.mt_count[i] = (w[i].rows / MT_ROWS) * p.nkc;
        total += p.mt_count[i];
        groups += w[i].rows / MT_ROWS;
    }
    if (epilogue == EPI_SWIGLU) BRASA_REQUIRE(ctx, nmat == 2 && w[0].rows == w[1].rows, "gemv swiglu: gate and up must have the same rows");
    p.total_mt = total;
    p.epilogue = epilogue;
    p.x = x; p.h = h; p.normw = normw; p.x_out = x_out; p.ss = ss; p.nss = nss;
    p.scaled = scaled; p.eps = eps;
    BRASA_TRY(brasa_gemv_scratch(ctx, (size_t)total * MT_ROWS, groups));
    p.partials = ctx->gemv_partials;
    p.counters = ctx->gemv_counters;
    p.status = ctx->status;

    const int mtb = mt_bytes(qtype);
    uint32_t grid = std::min<uint32_t>((uint32_t)ctx->sm_count, total);
    uint32_t per_block = (total + grid - 1) / grid;
    size_t fixed = (size_t)p.cols * 4 + 256;
    size_t budget = ctx->smem_optin - fixed - 2048;
    uint32_t nslot = (uint32_t)std::min<size_t>(per_block, budget / (mtb + 16));
    BRASA_REQUIRE(ctx, nslot >= 1, "gemv: %u columns do not fit shared memory", p.cols);
    p.nslot = nslot;
    size_t smem = (size_t)nslot * mtb + fixed + (size_t)nslot * 16;

    auto kern = qtype == BRASA_Q4_0 ? gemv_tiled_kernel<BRASA_Q4_0> : gemv_tiled_kernel<BRASA_Q6_0>;
    bool &attr_done = ctx->gemv_attr_done[qtype == BRASA_Q4_0 ? 0 : 1];
    if (!attr_done) {
        BRASA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return BRASA_OK;
}

namespace {

int32_t gemv_file(brasa_cmd *cmd, const brasa_qmatrix &w, const float *x, float *y, uint32_t tokens, const float *ss, uint32_t nss,
                  float eps, int scaled) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, w.cols % 32 == 0 && qm_fits(w), "gemv: bad file-layout matrix");
    dim3 grid((w.rows + 3) / 4, tokens);
    switch (w.qtype) {
    case BRASA_Q4_0: gemv_file_kernel<BRASA_Q4_0><<<grid, 128, 0, ctx->stream>>>(arg_ptr(w.data), x, y, w.rows, w.cols, ss, nss, eps, scaled); break;
    case BRASA_Q6_0: gemv_file_kernel<BRASA_Q6_0><<<grid, 128, 0, ctx->stream>>>(arg_ptr(w.data), x, y, w.rows, w.cols, ss, nss, eps, scaled); break;
    case BRASA_Q8_0: gemv_file_kernel<BRASA_Q8_0><<<grid, 128, 0, ctx->stream>>>(arg_ptr(w.data), x, y, w.rows, w.cols, ss, nss, eps, scaled); break;
    default: return brasa_fail(ctx, BRASA_EINVAL, "gemv: unknown weight type %d", w.qtype);
    }
    return brasa_post_launch(cmd, "gemv_file");
}

// y = W x (optionally scaled) for one matrix in either layout, `tokens` input rows.
int32_t gemv_any(brasa_cmd *cmd, const brasa_qmatrix &w, brasa_arg x, brasa_arg y, uint32_t tokens, brasa_arg ss, float eps, int scaled) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, tokens >= 1, "gemv: no tokens");
    BRASA_REQUIRE(ctx, arg_fits(x, (uint64_t)tokens * w.cols * 4) && arg_fits(y, (uint64_t)tokens * w.rows * 4), "gemv: x or y too small");
    BRASA_REQUIRE(ctx, x.offset % 16 == 0 && y.offset % 4 == 0, "gemv: misaligned x or y");
    uint32_t nss = brasa_norm_partials(w.cols);
    if (scaled) BRASA_REQUIRE(ctx, arg_fits(ss, (uint64_t)nss * 4), "gemv_scaled: ss too small");
    const float *ssp = scaled ? (const float *)arg_ptr(ss) : nullptr;
    if (w.layout == BRASA_LAYOUT_TILED) {
        for (uint32_t t = 0; t < tokens; ++t) {
            float *yt = (float *)arg_ptr(y) + (size_t)t * w.rows;
            BRASA_TRY(brasa_gemv_launch(cmd, w.qtype, 1, &w, &yt, (const float *)arg_ptr(x) + (size_t)t * w.cols, nullptr, nullptr, nullptr, ssp,
                                        nss, scaled, eps, EPI_SCALE));
        }
        return BRASA_OK;
    }
    return gemv_file(cmd, w, (const float *)arg_ptr(x), (float *)arg_ptr(y), tokens, ssp, nss, eps, scaled);
}

}  // namespace

extern "C" {

int32_t brasa_k_gemv(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens) {
    if (!cmd) return BRASA_EINVAL;
    return gemv_any(cmd, w, x, y, tokens, brasa_arg{nullptr, 0}, 0.0f, 0);
}

int32_t brasa_k_gemv_simple(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, w.layout == BRASA_LAYOUT_FILE, "gemv_simple reads the file layout");
    BRASA_REQUIRE(ctx, tokens >= 1 && arg_fits(x, (uint64_t)tokens * w.cols * 4) && arg_fits(y, (uint64_t)tokens * w.rows * 4), "gemv_simple: x or y too small");
    return gemv_file(cmd, w, (const float *)arg_ptr(x), (float *)arg_ptr(y), tokens, nullptr, 0, 0.0f, 0);
}

int32_t brasa_k_gemv_scaled(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg xw, brasa_arg ss, float eps, brasa_arg y) {
    if (!cmd) return BRASA_EINVAL;
    BRASA_REQUIRE(cmd->ctx, w.rows % 8 == 0, "gemv_scaled: rows %% 8");
    BRASA_REQUIRE(cmd->ctx, w.qtype == BRASA_Q4_0 || w.qtype == BRASA_Q6_0, "gemv_scaled: q4_0 or q6_0");
    return gemv_any(cmd, w, xw, y, 1, ss, eps, 1);
}

int32_t brasa_k_gemv_scaled3(brasa_cmd *cmd, const brasa_qmatrix w[3], brasa_arg xw, brasa_arg ss, float eps, const brasa_arg y[3]) {
    if (!cmd || !w || !y) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    bool tiled = true;
    for (int i = 0; i < 3; ++i) {
        BRASA_REQUIRE(ctx, w[i].qtype == BRASA_Q4_0, "gemv_scaled3: q4_0");
        BRASA_REQUIRE(ctx, w[i].cols == w[0].cols, "gemv_scaled3: same input");
        BRASA_REQUIRE(ctx, w[i].rows % 8 == 0, "gemv_scaled3: rows %% 8");
        BRASA_REQUIRE(ctx, arg_fits(y[i], (uint64_t)w[i].rows * 4), "gemv_scaled3: y too small");
        tiled = tiled && w[i].layout == BRASA_LAYOUT_TILED;
    }
    if (!tiled) {
        for (int i = 0; i < 3; ++i) BRASA_TRY(gemv_any(cmd, w[i], xw, y[i], 1, ss, eps, 1));
        return BRASA_OK;
    }
    uint32_t nss = brasa_norm_partials(w[0].cols);
    BRASA_REQUIRE(ctx, arg_fits(xw, (uint64_t)w[0].cols * 4) && arg_fits(ss, (uint64_t)nss * 4), "gemv_scaled3: xw or ss too small");
    float *ys[3] = {(float *)arg_ptr(y[0]), (float *)arg_ptr(y[1]), (float *)arg_ptr(y[2])};
    return brasa_gemv_launch(cmd, BRASA_Q4_0, 3, w, ys, (const float *)arg_ptr(xw), nullptr, nullptr, nullptr, (const float *)arg_ptr(ss), nss, 1,
                             eps, EPI_SCALE);
}

int32_t brasa_k_gemv_scaled_swiglu(brasa_cmd *cmd, brasa_qmatrix gate, brasa_qmatrix up, brasa_arg xw, brasa_arg ss, float eps, brasa_arg y) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, gate.qtype == BRASA_Q4_0 && up.qtype == BRASA_Q4_0, "gemv_scaled_swiglu: q4_0");
    BRASA_REQUIRE(ctx, gate.rows == up.rows && gate.cols == up.cols && gate.rows % 8 == 0, "gemv_scaled_swiglu: gate and up shapes");
    uint32_t nss = brasa_norm_partials(gate.cols);
    BRASA_REQUIRE(ctx, arg_fits(xw, (uint64_t)gate.cols * 4) && arg_fits(ss, (uint64_t)nss * 4) && arg_fits(y, (uint64_t)gate.rows * 4),
                  "gemv_scaled_swiglu: buffers too small");
    if (gate.layout == BRASA_LAYOUT_TILED && up.layout == BRASA_LAYOUT_TILED) {
        brasa_qmatrix w[2] = {gate, up};
        float *ys[2] = {(float *)arg_ptr(y), nullptr};
        return brasa_gemv_launch(cmd, BRASA_Q4_0, 2, w, ys, (const float *)arg_ptr(xw), nullptr, nullptr, nullptr, (const float *)arg_ptr(ss), nss,
                                 1, eps, EPI_SWIGLU);
    }
    // file layout: gate into y, up into the split-K scratch, then SwiGLU in place
    BRASA_TRY(brasa_gemv_scratch(ctx, gate.rows, 1));
    BRASA_TRY(gemv_file(cmd, gate, (const float *)arg_ptr(xw), (float *)arg_ptr(y), 1, (const float *)arg_ptr(ss), nss, eps, 1));
    BRASA_TRY(gemv_file(cmd, up, (const float *)arg_ptr(xw), ctx->gemv_partials, 1, (const float *)arg_ptr(ss), nss, eps, 1));
    swiglu_inplace_kernel<<<(gate.rows + 255) / 256, 256, 0, ctx->stream>>>((float *)arg_ptr(y), ctx->gemv_partials, gate.rows);
    return brasa_post_launch(cmd, "swiglu_inplace");
}

}  // extern "C"
