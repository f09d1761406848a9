// Decode GEMVs: y = W x for quantised W (q4_0 / q6_0 in the row-planar tiled layout), one token.
//
// The reference's GEMV family (crates/kernels/src/lib.rs:633-838 and the MSL bodies it dispatches)
// is HBM-bound: every weight byte is read once per token. On B200 the matrices are small next to the
// machine (o_proj is 40 KB per SM) and each GEMV depends on the previous one, so the kernel is built
// to keep the weight stream flowing and the per-kernel latency short:
//   * every block owns whole output rows, rows / grid of them (balanced to one row), so no partial
//     result ever crosses blocks: no atomics, no second pass, the epilogue (RMSNorm scale, SwiGLU,
//     residual add) runs where the row was computed;
//   * the block's rows are one contiguous byte range; it moves HBM -> shared memory with bulk async
//     copies (cp.async.bulk + mbarrier) issued before the kernel waits for its input vector
//     (programmatic dependent launch): the weight stream does not stop at kernel boundaries;
//   * a warp computes (row, column slice) dot products, two rows at a time. Each lane owns the same
//     16-column half blocks of every row, so its share of x stays in registers for the whole kernel;
//     the 32 partial sums are combined with warp shuffles.
// Dequantisation is fused and the integer part of the arithmetic is exact. The packed f32x2
// instructions of sm_100 issue at a fraction of the scalar rate and a scalar float path needs three
// instructions per weight, so the dot product runs on the integer pipe instead: the lane's x values are
// converted once per kernel to 22-bit fixed point relative to the largest of each 16-value group and
// split into three byte planes; a code word becomes two registers of four byte-wide codes with two
// logic instructions, and dp4a accumulates codes x bytes exactly in int32:
//     sum_j (q_j - bias) X_j = S0 + 256 S1 + 65536 S2 - bias * sum_j X_j
// One int-to-float conversion and one multiply by (block scale x group scale) per 16 weights follow.
#include <type_traits>

#include "brasa_internal.h"

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 20;  // try_wait rounds before a wait gives up
constexpr int MAX_WARPS = 10;              // consumer warps per block (a multiple of the slice count)
constexpr int PRODUCER_LANES = 1;

enum { EPI_SCALE = 0, EPI_SWIGLU = 1, EPI_RESID = 2 };

struct GemvParams {
    const uint8_t *w[3];
    float *y[3];
    uint32_t rows[3];
    uint32_t nmat;
    uint32_t cols;
    uint32_t slices;       // column slices per row (S); consumer warps are a multiple of it
    uint32_t warps;        // consumer warps
    uint32_t rows_per_slot;  // 2 * warps / slices
    uint32_t nslot;        // ring slots in shared memory
    uint32_t max_items;    // partial sums kept in shared memory per block
    int epilogue;
    // input vector: x (optionally + h) times normw when given; ss: partial sums of x^2 computed by
    // add_norm_prep (reference form), else the block computes the sum itself
    const float *x, *h, *normw, *ss;
    float *x_out;          // when h is given: block 0 writes x + h here
    const float *resid;    // EPI_RESID: y = resid + W x
    uint32_t nss;
    int scaled;            // multiply outputs by 1/sqrt(mean(x^2) + eps)
    float eps;
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

// The lane's x values of one half block in fixed point: quad j (4 values) x byte plane d, the sum of
// the 16 integers, and the power-of-two step.
struct XFixed {
    uint32_t d[4][3];
    int total;
    float step;
};

// sum over the 16 weights of a half block of (code - bias) * X, as an integer.
// Quads: 0 = low nibbles of word x, 1 = high nibbles of word x, 2 and 3 likewise for word y.
template <int QT>
__device__ __forceinline__ int half_block_idot(uint2 codes, uint32_t hb, const XFixed &x) {
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
    int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        s0 = dp4a_uu(a[j], x.d[j][0], s0);
        s1 = dp4a_uu(a[j], x.d[j][1], s1);
        s2 = dp4a_us(a[j], x.d[j][2], s2);
    }
    constexpr int BIAS = QT == BRASA_Q4_0 ? 8 : 32;
    return s0 + 256 * s1 + 65536 * s2 - BIAS * x.total;
}

// N = half blocks per lane and slice (the lane's x registers hold 16 N values).
template <int QT, int N>
__global__ void __launch_bounds__((MAX_WARPS + 1) * 32, 1) gemv_rows_kernel(GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t row_bytes = tiled_row_bytes(QT, p.cols);
    const uint32_t slot_bytes = p.rows_per_slot * row_bytes;
    // layout: ring [nslot][slot_bytes] | xs [cols] | nws [cols] (norm weight, when given) | xf [14][cols/16] | part [max_items]
    //         | full, empty [nslot] | xbar, wbar | red
    uint8_t *ring = smem;
    float *xs = reinterpret_cast<float *>(smem + (size_t)p.nslot * slot_bytes);
    float *nws = xs + p.cols;
    uint32_t *xf = reinterpret_cast<uint32_t *>(nws + (p.normw ? p.cols : 0));  // fixed-point x: [14][cols / 16] words
    float *part = reinterpret_cast<float *>(xf + 14 * (p.cols / 16));
    uint64_t *full = reinterpret_cast<uint64_t *>(part + ((p.max_items + 1) & ~1u));
    uint64_t *empty = full + p.nslot;
    uint64_t *xbar = empty + p.nslot, *wbar = xbar + 1;
    float *red = reinterpret_cast<float *>(wbar + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t W = p.warps, S = p.slices, RPS = p.rows_per_slot;
    const uint32_t G = gridDim.x, b = blockIdx.x;
    // logical rows: matrices one after another (SwiGLU: the rows of gate; up follows the same range)
    const uint32_t nseg = p.epilogue == EPI_SWIGLU ? 2 : p.nmat;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < (p.epilogue == EPI_SWIGLU ? 1u : p.nmat); ++i) total_rows += p.rows[i];
    const uint32_t r0 = (uint32_t)((uint64_t)total_rows * b / G), r1 = (uint32_t)((uint64_t)total_rows * (b + 1) / G);
    // per segment: first row inside its matrix and row count
    // per segment: first row inside its matrix, row count, first slot, rows of the segments before it.
    // Only constant indices below, so the arrays stay in registers.
    uint32_t seg_first[3] = {0, 0, 0}, seg_rows[3] = {0, 0, 0}, seg_slot0[3] = {0, 0, 0}, seg_before[3] = {0, 0, 0};
    {
        uint32_t base = 0, slot = 0, before = 0;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            if ((uint32_t)i < nseg) {
                if (p.epilogue == EPI_SWIGLU) { seg_first[i] = r0; seg_rows[i] = r1 - r0; }
                else {
                    uint32_t lo = max(r0, base), hi = min(r1, base + p.rows[i]);
                    seg_first[i] = lo > base ? lo - base : 0;
                    seg_rows[i] = hi > lo ? hi - lo : 0;
                    base += p.rows[i];
                }
            }
            seg_slot0[i] = slot;
            seg_before[i] = before;
            slot += (seg_rows[i] + RPS - 1) / RPS;
            before += seg_rows[i];
        }
    }
    const uint32_t total_slots = seg_slot0[2] + (seg_rows[2] + RPS - 1) / RPS;
    auto seg_of = [&](uint32_t k) -> uint32_t { return (uint32_t)(nseg > 1 && k >= seg_slot0[1]) + (uint32_t)(nseg > 2 && k >= seg_slot0[2]); };
#define SEG_PICK(arr, i) ((i) == 0 ? arr[0] : ((i) == 1 ? arr[1] : arr[2]))

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.nslot; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        mbar_init(xbar, 1);
        mbar_init(wbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](uint32_t k) {  // slot k of this block -> ring[k % nslot]
        const uint32_t i = seg_of(k);
        uint32_t first = (k - SEG_PICK(seg_slot0, i)) * RPS, n = min(RPS, SEG_PICK(seg_rows, i) - first);
        const uint8_t *src = p.w[i] + (size_t)(SEG_PICK(seg_first, i) + first) * row_bytes;
        uint32_t s = k % p.nslot;
        mbar_expect_tx(&full[s], n * row_bytes);
        bulk_g2s(ring + (size_t)s * slot_bytes, src, n * row_bytes, &full[s]);
    };

    if (warp == (int)W) {  // producer warp: lanes 0..3 issue alternating slots
        if (lane < PRODUCER_LANES) {
            // weights are immutable: the first ring-full of copies starts before the input is ready
            uint32_t k = lane;
            if (lane == 0 && p.normw) {  // the norm weight is a weight too
                mbar_expect_tx(wbar, p.cols * 4);
                bulk_g2s(nws, p.normw, p.cols * 4, wbar);
            }
            for (; k < total_slots && k < p.nslot; k += PRODUCER_LANES) issue(k);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (lane == 0 && !p.h) {  // the input vector: one bulk copy once the previous kernel is done
                mbar_expect_tx(xbar, p.cols * 4);
                bulk_g2s(xs, p.x, p.cols * 4, xbar);
            }
            for (; k < total_slots; k += PRODUCER_LANES) {
                if (!mbar_wait(&empty[k % p.nslot], (k / p.nslot - 1) & 1)) {
                    atomicExch(p.status, 1u);
                    break;
                }
                issue(k);
            }
        }
        return;
    }
    // Everything below depends on the previous kernel's output. Once that kernel is complete the next one
    // of the stream may start its own weight prefetch: at most two kernels of the chain overlap, so a
    // kernel's early reads (weights, older KV rows) never race with a producer further back.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- x in shared memory (bulk copy; with h: x + h through registers), sum of squares ----
    const uint32_t CT = W * 32;
    bool ok_in = true;
    if (p.h) {
        for (uint32_t j = threadIdx.x; j < p.cols; j += CT) {
            float v = p.x[j] + p.h[j];
            if (p.x_out && b == 0) p.x_out[j] = v;
            xs[j] = v;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
    } else {
        ok_in = mbar_wait(xbar, 0);
    }
    if (p.normw) ok_in = mbar_wait(wbar, 0) && ok_in;
    if (!ok_in && lane == 0) atomicExch(p.status, 3u);
    float scale = 1.0f;
    if (p.scaled) {
        float tot = 0.0f;
        if (p.ss) {  // reference form: fixed-order sum of add_norm_prep's partials
            for (uint32_t i = 0; i < p.nss; ++i) tot += p.ss[i];
        } else {
            float ssq = 0.0f;
            for (uint32_t j = threadIdx.x; j < p.cols; j += CT) ssq = fmaf(xs[j], xs[j], ssq);
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) red[warp] = ssq;
            asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
            for (uint32_t i = 0; i < W; ++i) tot += red[i];
        }
        scale = 1.0f / sqrtf(tot / (float)p.cols + p.eps);
    }

    // ---- x to fixed point, once per block: thread t converts half block t (t + CT, ...) into shared memory ----
    const uint32_t slice = warp % S, row_in_slot = warp / S;
    const uint32_t nhb = p.cols / 16;
    for (uint32_t hbi = threadIdx.x; hbi < nhb; hbi += CT) {
        const uint32_t blk = hbi >> 1, half = hbi & 1;
        float v[4][4];  // quad j: values that meet low/high nibbles of word x (j = 0, 1) and word y (j = 2, 3)
#pragma unroll
        for (int ww = 0; ww < 2; ++ww) {
            const uint32_t e0 = blk * 32 + 8 * half + 4 * ww;
            float4 lo = *reinterpret_cast<const float4 *>(xs + e0), hi = *reinterpret_cast<const float4 *>(xs + e0 + 16);
            if (p.normw) {
                float4 wl = *reinterpret_cast<const float4 *>(nws + e0), wh = *reinterpret_cast<const float4 *>(nws + e0 + 16);
                lo.x *= wl.x; lo.y *= wl.y; lo.z *= wl.z; lo.w *= wl.w;
                hi.x *= wh.x; hi.y *= wh.y; hi.z *= wh.z; hi.w *= wh.w;
            }
            v[2 * ww][0] = lo.x; v[2 * ww][1] = lo.y; v[2 * ww][2] = lo.z; v[2 * ww][3] = lo.w;
            v[2 * ww + 1][0] = hi.x; v[2 * ww + 1][1] = hi.y; v[2 * ww + 1][2] = hi.z; v[2 * ww + 1][3] = hi.w;
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(v[j][e]));
        // step = 2^(exponent(amax) - 20): every |x| / step is below 2^21; zero (or denormal) groups get step 0
        uint32_t ebits = __float_as_uint(amax) & 0x7F800000u;
        bool live = ebits > (21u << 23) && ebits < 0x7F800000u;
        // infinities and NaNs are not representable: their group's step carries them into the result
        float step = live ? __uint_as_float(ebits - (20u << 23)) : (ebits == 0x7F800000u ? amax : 0.0f);
        float inv = live ? __uint_as_float((254u << 23) - (ebits - (20u << 23))) : 0.0f;  // 1 / step, exact
        int total = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int X[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                X[e] = __float2int_rn(v[j][e] * inv);
                total += X[e];
            }
            // byte planes of the four integers: byte k of every X gathered into one word
            uint32_t lo01 = __byte_perm(X[0], X[1], 0x5140), lo23 = __byte_perm(X[2], X[3], 0x5140);  // b0 b0' b1 b1'
            uint32_t hi01 = __byte_perm(X[0], X[1], 0x7362), hi23 = __byte_perm(X[2], X[3], 0x7362);  // b2 b2' b3 b3'
            xf[(3 * j + 0) * nhb + hbi] = __byte_perm(lo01, lo23, 0x5410);
            xf[(3 * j + 1) * nhb + hbi] = __byte_perm(lo01, lo23, 0x7632);
            xf[(3 * j + 2) * nhb + hbi] = __byte_perm(hi01, hi23, 0x5410);
        }
        xf[12 * nhb + hbi] = (uint32_t)total;
        xf[13 * nhb + hbi] = __float_as_uint(step);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
    // ---- the lane's share: the same half blocks of every row ----
    XFixed xr[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        uint32_t hbi = (slice * N + i) * 32 + lane;
        bool ok = hbi < nhb;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int d = 0; d < 3; ++d) xr[i].d[j][d] = ok ? xf[(3 * j + d) * nhb + hbi] : 0u;
        xr[i].total = ok ? (int)xf[12 * nhb + hbi] : 0;
        xr[i].step = ok ? __uint_as_float(xf[13 * nhb + hbi]) : 0.0f;
    }
    const uint32_t hi_off = tiled_hi_off(p.cols), sc_off = tiled_scale_off(QT, p.cols);

    // ---- consume slots: warp = (row pair in slot, slice); two rows at a time for instruction-level parallelism ----
    for (uint32_t k = 0; k < total_slots; ++k) {
        uint32_t s = k % p.nslot;
        if (!mbar_wait(&full[s], (k / p.nslot) & 1)) {
            // give up on the remaining slots but still meet the other warps at the barrier below
            if (lane == 0) atomicExch(p.status, 2u);
            break;
        }
        const uint32_t i = seg_of(k);
        uint32_t first = (k - SEG_PICK(seg_slot0, i)) * RPS, n = min(RPS, SEG_PICK(seg_rows, i) - first);
        const uint32_t ra = row_in_slot * 2;
        if (ra < n) {
            const bool two = ra + 1 < n;
            const uint8_t *row_a = ring + (size_t)s * slot_bytes + (size_t)ra * row_bytes;
            const uint8_t *row_b = two ? row_a + row_bytes : row_a;
            float acc_a = 0.0f, acc_b = 0.0f;
            // straight-line code: lanes past the end of the row read the last half block and multiply by step 0
#pragma unroll
            for (int it = 0; it < N; ++it) {
                const uint32_t hbi = min((slice * N + it) * 32 + lane, nhb - 1);
                uint2 ca = *reinterpret_cast<const uint2 *>(row_a + hbi * 8);
                uint2 cb = *reinterpret_cast<const uint2 *>(row_b + hbi * 8);
                uint32_t ha = 0, hb = 0;
                if (QT == BRASA_Q6_0) {
                    ha = *reinterpret_cast<const uint32_t *>(row_a + hi_off + hbi * 4);
                    hb = *reinterpret_cast<const uint32_t *>(row_b + hi_off + hbi * 4);
                }
                float da = __half2float(*reinterpret_cast<const __half *>(row_a + sc_off + (hbi >> 1) * 2));
                float db = __half2float(*reinterpret_cast<const __half *>(row_b + sc_off + (hbi >> 1) * 2));
                int sa = half_block_idot<QT>(ca, ha, xr[it]);
                int sb = half_block_idot<QT>(cb, hb, xr[it]);
                acc_a = fmaf(da * xr[it].step, (float)sa, acc_a);
                acc_b = fmaf(db * xr[it].step, (float)sb, acc_b);
            }
            for (int o = 16; o > 0; o >>= 1) {
                acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o);
                acc_b += __shfl_xor_sync(0xffffffffu, acc_b, o);
            }
            // partial index: rows of all segments in order, slices innermost
            const uint32_t rows_before = SEG_PICK(seg_before, i);
            if (lane == 0) {
                part[(rows_before + first + ra) * S + slice] = acc_a;
                if (two) part[(rows_before + first + ra + 1) * S + slice] = acc_b;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");

    // ---- epilogue: one thread per output row of this block ----
    if (p.epilogue == EPI_SWIGLU) {
        uint32_t nr = r1 - r0;
        for (uint32_t j = threadIdx.x; j < nr; j += CT) {
            float g = 0.0f, u = 0.0f;
            for (uint32_t sl = 0; sl < S; ++sl) { g += part[j * S + sl]; u += part[(nr + j) * S + sl]; }
            g *= scale; u *= scale;
            p.y[0][r0 + j] = (g / (1.0f + expf(-g))) * u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 3; ++i) {
            for (uint32_t j = threadIdx.x; j < seg_rows[i]; j += CT) {
                float v = 0.0f;
                for (uint32_t sl = 0; sl < S; ++sl) v += part[(seg_before[i] + j) * S + sl];
                uint32_t r = seg_first[i] + j;
                v *= scale;
                if (p.epilogue == EPI_RESID) v += p.resid[r];
                p.y[i][r] = v;
            }
        }
    }
#undef SEG_PICK
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
// epilogue: 0 scale, 1 SwiGLU (w[0] = gate, w[1] = up, y[0]), 2 residual (y = resid + W x).
int32_t brasa_gemv_launch(brasa_cmd *cmd, int qtype, uint32_t nmat, const brasa_qmatrix *w, float *const *y, const float *x,
                          const float *h, const float *normw, float *x_out, const float *ss, uint32_t nss, int scaled, float eps,
                          int epilogue, const float *resid) {
    brasa_ctx *ctx = cmd->ctx;
    GemvParams p{};
    p.nmat = nmat;
    p.cols = w[0].cols;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < nmat; ++i) {
        BRASA_REQUIRE(ctx, w[i].layout == BRASA_LAYOUT_TILED && w[i].qtype == qtype && w[i].cols == p.cols && tiled_ok(qtype, w[i].rows, w[i].cols),
                      "gemv: matrix %u is not a tiled %s matrix of %u columns", i, qtype == BRASA_Q4_0 ? "q4_0" : "q6_0", p.cols);
        BRASA_REQUIRE(ctx, qm_fits(w[i]) && w[i].data.offset % 16 == 0, "gemv: matrix %u exceeds its buffer or is misaligned", i);
        p.w[i] = arg_ptr(w[i].data);
        p.y[i] = y[i];
        p.rows[i] = w[i].rows;
        total_rows += w[i].rows;
    }
    if (epilogue == EPI_SWIGLU) {
        BRASA_REQUIRE(ctx, nmat == 2 && w[0].rows == w[1].rows, "gemv swiglu: gate and up must have the same rows");
        total_rows = w[0].rows;
    }
    if (epilogue == EPI_RESID) BRASA_REQUIRE(ctx, nmat == 1 && resid, "gemv residual: one matrix and a residual vector");
    p.epilogue = epilogue;
    p.x = x; p.h = h; p.normw = normw; p.x_out = x_out; p.ss = ss; p.nss = nss; p.resid = resid;
    p.scaled = scaled; p.eps = eps;
    p.status = ctx->status;

    // slices and half blocks per lane: the smallest slice count that keeps a lane's x within 5 half blocks
    const uint32_t nhb = p.cols / 16;
    uint32_t S = 1, N = 0;
    for (;; ++S) {
        N = (nhb + 32 * S - 1) / (32 * S);
        if (N <= 5) break;
    }
    BRASA_REQUIRE(ctx, S <= MAX_WARPS, "gemv: %u columns need more column slices than the kernel has warps", p.cols);
    uint32_t warps = 8 % S == 0 ? 8 : (MAX_WARPS / S) * S;
    p.slices = S;
    p.warps = warps;
    p.rows_per_slot = 2 * warps / S;  // every warp takes two rows of a slot

    const uint32_t row_bytes = tiled_row_bytes(qtype, p.cols);
    const uint32_t slot_bytes = p.rows_per_slot * row_bytes;
    uint32_t grid = std::min<uint32_t>((uint32_t)ctx->sm_count, total_rows);
    uint32_t rows_per_block = (total_rows + grid - 1) / grid;
    p.max_items = (rows_per_block + 1) * S * (epilogue == EPI_SWIGLU ? 2 : 1) + S * nmat;
    size_t fixed = (size_t)p.cols * 4 * (normw ? 2 : 1) + (size_t)(p.cols / 16) * 56 + (size_t)((p.max_items + 1) & ~1u) * 4 + 160;
    BRASA_REQUIRE(ctx, fixed + slot_bytes + 64 <= ctx->smem_optin, "gemv: %u columns do not fit shared memory", p.cols);
    uint32_t segs = epilogue == EPI_SWIGLU ? 2 : nmat;
    uint32_t need_slots = (rows_per_block + 1 + p.rows_per_slot - 1) / p.rows_per_slot * (epilogue == EPI_SWIGLU ? 2 : 1) + segs;
    size_t budget = ctx->smem_optin - fixed - 1024;
    uint32_t nslot = (uint32_t)std::min<size_t>(need_slots, budget / (slot_bytes + 16));
    BRASA_REQUIRE(ctx, nslot >= 1, "gemv: no room for a ring slot");
    p.nslot = nslot;
    size_t smem = (size_t)nslot * slot_bytes + fixed + (size_t)nslot * 16;

    void (*kern)(GemvParams) = nullptr;
#define PICK(QT)                                                 \
    switch (N) {                                                 \
    case 1: kern = gemv_rows_kernel<QT, 1>; break;               \
    case 2: kern = gemv_rows_kernel<QT, 2>; break;               \
    case 3: kern = gemv_rows_kernel<QT, 3>; break;               \
    case 4: kern = gemv_rows_kernel<QT, 4>; break;               \
    default: kern = gemv_rows_kernel<QT, 5>; break;              \
    }
    if (qtype == BRASA_Q4_0) { PICK(BRASA_Q4_0) } else { PICK(BRASA_Q6_0) }
#undef PICK
    bool &attr_done = ctx->gemv_attr_done[(qtype == BRASA_Q4_0 ? 0 : 5) + (N - 1)];
    if (!attr_done) {
        BRASA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin));
        attr_done = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((warps + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    return brasa_post_launch(cmd, "gemv_rows");
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
                                        nss, scaled, eps, EPI_SCALE, nullptr));
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
                             eps, EPI_SCALE, nullptr);
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
                                 1, eps, EPI_SWIGLU, nullptr);
    }
    // file layout: gate into y, up into scratch, then SwiGLU in place
    BRASA_TRY(brasa_gemv_scratch(ctx, gate.rows, 1));
    BRASA_TRY(gemv_file(cmd, gate, (const float *)arg_ptr(xw), (float *)arg_ptr(y), 1, (const float *)arg_ptr(ss), nss, eps, 1));
    BRASA_TRY(gemv_file(cmd, up, (const float *)arg_ptr(xw), ctx->gemv_partials, 1, (const float *)arg_ptr(ss), nss, eps, 1));
    swiglu_inplace_kernel<<<(gate.rows + 255) / 256, 256, 0, ctx->stream>>>((float *)arg_ptr(y), ctx->gemv_partials, gate.rows);
    return brasa_post_launch(cmd, "swiglu_inplace");
}

}  // extern "C"
