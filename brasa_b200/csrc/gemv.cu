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
#include "gemv_device.cuh"

using namespace brasa_dev;

namespace {

constexpr int GEMV_WARPS = 16;              // consumer warps per block; column slices per row divide it

enum { EPI_SCALE = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_PUSH = 3 };

struct GemvParams {
    const uint8_t *w[3];
    float *y[3];
    uint32_t rows[3];
    uint32_t nmat;
    uint32_t total_rows;   // logical rows the grid shares out (SwiGLU: the rows of gate)
    uint32_t cols;
    uint32_t slices;       // column slices per row (S); consumer warps are a multiple of it
    uint32_t warps;        // consumer warps
    uint32_t rows_per_slot;  // rows of one ring slot: the rows half of the warps take per iteration
    uint32_t nslot;        // ring slots in shared memory
    uint32_t max_items;    // partial sums kept in shared memory per block
    int epilogue;
    // input vector: x (optionally + h) times normw when given; ss: partial sums of x^2 computed by
    // add_norm_prep (reference form), else the block computes the sum itself
    const float *x, *h, *normw, *ss;
    float *x_out;          // when h is given: block 0 writes x + h here
    const float *resid;    // EPI_RESID: y = resid + W x
    // EPI_PUSH (tensor parallel): W x is this rank's share of a sum over ranks; every output goes, tagged with the
    // exchange number, into slot [this rank] of every rank's exchange buffer instead of a local vector
    brasa_tp_push_target push;
    uint32_t nss;
    int scaled;            // multiply outputs by 1/sqrt(mean(x^2) + eps)
    float eps;
    uint32_t *status;
    unsigned long long *trace;  // optional: block 0 records the time of each phase (debugging aid)
    // weights of the GEMV that follows in the token loop: this block asks L2 for the rows the same block
    // index will own there, so that kernel's bulk copies find them on chip
    const uint8_t *pf_w[3];
    uint32_t pf_rows[3];
    uint32_t pf_nmat, pf_total_rows, pf_row_bytes, pf_swiglu;
};

#ifdef BRASA_TRACE_BUILD
#define TRACE(i) do { if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) p.trace[i] = gtime(); } while (0)
#else
#define TRACE(i) do { } while (0)
#endif
// N = half blocks per lane and slice (the lane's x registers hold 14 N words).
constexpr int R = 2;         // rows a warp works on at a time
constexpr int GEMV_PLANES = 3;  // byte planes of the fixed-point input: the f32 accuracy class (gemv_device.cuh)
constexpr int MAX_CONV = 3;  // half blocks of x a thread converts with all its loads in flight

template <int QT, int N>
__global__ void __maxnreg__(128) gemv_rows_kernel(GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t row_bytes = tiled_row_bytes(QT, p.cols);
    const uint32_t slot_bytes = p.rows_per_slot * row_bytes;
    const uint32_t nhb = p.cols / 16;
    // layout: ring [nslot][slot_bytes] | xf [nhb] records of 16 words | part [max_items] | full, empty [nslot] | red
    uint8_t *ring = smem;
    uint4 *xf = reinterpret_cast<uint4 *>(smem + (size_t)p.nslot * slot_bytes);
    float *part = reinterpret_cast<float *>(xf + XRec<GEMV_PLANES>::CHUNKS * nhb);
    uint64_t *full = reinterpret_cast<uint64_t *>(part + ((p.max_items + 1) & ~1u));
    uint64_t *empty = full + p.nslot;
    float *red = reinterpret_cast<float *>(empty + p.nslot);

    TRACE(0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t W = p.warps, S = p.slices, RPS = p.rows_per_slot;
    const uint32_t Wp = W / S;                                     // warps side by side on different rows
    const uint32_t split = (Wp & 1) ? 1u : 2u;                     // slots consumed per iteration of the block
    const uint32_t G = gridDim.x, b = blockIdx.x;
    // logical rows: matrices one after another (SwiGLU: the rows of gate; up follows the same range)
    const uint32_t nseg = p.epilogue == EPI_SWIGLU ? 2 : p.nmat;
    const uint32_t r0 = p.total_rows * b / G, r1 = p.total_rows * (b + 1) / G;
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

    uint32_t *done = reinterpret_cast<uint32_t *>(empty);  // per slot: warps that have finished with it
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.nslot; ++s) {
            mbar_init(&full[s], 1);
            done[s] = 0;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Slot k of this block -> ring[k % nslot]. There is no producer warp: thread 0 starts the first ring-full of
    // copies, and the warp that is last to finish with a slot starts the copy that reuses it.
    auto issue = [&](uint32_t k) {
        const uint32_t i = seg_of(k);
        uint32_t first = (k - SEG_PICK(seg_slot0, i)) * RPS, n = min(RPS, SEG_PICK(seg_rows, i) - first);
        const uint8_t *src = p.w[i] + (size_t)(SEG_PICK(seg_first, i) + first) * row_bytes;
        uint32_t s = k % p.nslot;
        mbar_expect_tx(&full[s], n * row_bytes);
        bulk_g2s(ring + (size_t)s * slot_bytes, src, n * row_bytes, &full[s]);
    };
    if (threadIdx.x == 0) {
        // weights are immutable: these copies start before the input is ready
        for (uint32_t k = 0; k < total_slots && k < p.nslot; ++k) issue(k);
        if (p.pf_total_rows) {  // ask L2 for the rows this block index owns in the next GEMV of the chain
            const uint32_t q0 = p.pf_total_rows * b / G, q1 = p.pf_total_rows * (b + 1) / G;
            uint32_t base = 0;
            for (uint32_t i = 0; i < p.pf_nmat; ++i) {
                uint32_t lo = p.pf_swiglu ? q0 : max(q0, base), hi = p.pf_swiglu ? q1 : min(q1, base + p.pf_rows[i]);
                if (hi > lo) {
                    const uint8_t *ptr = p.pf_w[i] + (size_t)(lo - (p.pf_swiglu ? 0 : base)) * p.pf_row_bytes;
                    size_t bytes = (size_t)(hi - lo) * p.pf_row_bytes;
                    for (size_t off = 0; off < bytes; off += 32768) {
                        uint32_t n = (uint32_t)min((size_t)32768, bytes - off);
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr + off), "r"(n) : "memory");
                    }
                }
                base += p.pf_rows[i];
            }
        }
    }

    // ---- before the input exists: the norm weights of the half blocks this thread will convert ----
    const uint32_t CT = W * 32;
    float4 nw0[4];  // of this thread's first half block; wider inputs fetch the rest later
    if (p.normw && threadIdx.x < nhb) {
        const float4 *w4 = reinterpret_cast<const float4 *>(p.normw + (threadIdx.x >> 1) * 32 + 8 * (threadIdx.x & 1));
        nw0[0] = w4[0]; nw0[1] = w4[4]; nw0[2] = w4[1]; nw0[3] = w4[5];
    }
    // Everything below depends on the previous kernel's output. Once that kernel is complete the next one
    // of the stream may start its own weight prefetch: at most two kernels of the chain overlap, so a
    // kernel's early reads (weights, older KV rows) never race with a producer further back.
    TRACE(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    TRACE(2);

    // ---- x to 22-bit fixed point, once per block: thread t converts half blocks t, t + CT, ... into records ----
    // quad j of a half block: the values that meet the low / high nibbles of code word 0 (j = 0, 1) and 1 (j = 2, 3)
    float ssq = 0.0f;
    auto convert = [&](uint32_t hbi, float4 q0, float4 q1, float4 q2, float4 q3) { x_half_block_to_fixed<GEMV_PLANES>(xf, hbi, q0, q1, q2, q3); };
    {
        float4 xq[MAX_CONV][4];
#pragma unroll
        for (int c = 0; c < MAX_CONV; ++c) {
            const uint32_t hbi = threadIdx.x + c * CT;
            if (hbi < nhb) {
                const uint32_t e0 = (hbi >> 1) * 32 + 8 * (hbi & 1);
                const float4 *x4 = reinterpret_cast<const float4 *>(p.x + e0);
                xq[c][0] = x4[0]; xq[c][1] = x4[4]; xq[c][2] = x4[1]; xq[c][3] = x4[5];
                if (p.h) {
                    const float4 *h4 = reinterpret_cast<const float4 *>(p.h + e0);
                    const float4 hv[4] = {h4[0], h4[4], h4[1], h4[5]};
#pragma unroll
                    for (int j = 0; j < 4; ++j) { xq[c][j].x += hv[j].x; xq[c][j].y += hv[j].y; xq[c][j].z += hv[j].z; xq[c][j].w += hv[j].w; }
                    if (p.x_out && b == 0) {
                        float4 *o4 = reinterpret_cast<float4 *>(p.x_out + e0);
                        o4[0] = xq[c][0]; o4[4] = xq[c][1]; o4[1] = xq[c][2]; o4[5] = xq[c][3];
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < MAX_CONV; ++c) {
            const uint32_t hbi = threadIdx.x + c * CT;
            if (hbi < nhb) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float4 &q = xq[c][j];
                    ssq = fmaf(q.x, q.x, ssq); ssq = fmaf(q.y, q.y, ssq); ssq = fmaf(q.z, q.z, ssq); ssq = fmaf(q.w, q.w, ssq);
                    if (p.normw) {
                        const int off[4] = {0, 16, 4, 20};
                        float4 wv = c == 0 ? nw0[j] : *reinterpret_cast<const float4 *>(p.normw + (hbi >> 1) * 32 + 8 * (hbi & 1) + off[j]);
                        q.x *= wv.x; q.y *= wv.y; q.z *= wv.z; q.w *= wv.w;
                    }
                }
                convert(hbi, xq[c][0], xq[c][1], xq[c][2], xq[c][3]);
            }
        }
        // very wide inputs: the rest one at a time
        for (uint32_t hbi = threadIdx.x + MAX_CONV * CT; hbi < nhb; hbi += CT) {
            const uint32_t e0 = (hbi >> 1) * 32 + 8 * (hbi & 1);
            float4 q[4];
            const int off[4] = {0, 16, 4, 20};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                q[j] = *reinterpret_cast<const float4 *>(p.x + e0 + off[j]);
                if (p.h) {
                    float4 hv = *reinterpret_cast<const float4 *>(p.h + e0 + off[j]);
                    q[j].x += hv.x; q[j].y += hv.y; q[j].z += hv.z; q[j].w += hv.w;
                    if (p.x_out && b == 0) *reinterpret_cast<float4 *>(p.x_out + e0 + off[j]) = q[j];
                }
                ssq = fmaf(q[j].x, q[j].x, ssq); ssq = fmaf(q[j].y, q[j].y, ssq); ssq = fmaf(q[j].z, q[j].z, ssq); ssq = fmaf(q[j].w, q[j].w, ssq);
                if (p.normw) {
                    float4 wv = *reinterpret_cast<const float4 *>(p.normw + e0 + off[j]);
                    q[j].x *= wv.x; q[j].y *= wv.y; q[j].z *= wv.z; q[j].w *= wv.w;
                }
            }
            convert(hbi, q[0], q[1], q[2], q[3]);
        }
    }
    // the residual this thread will add in the epilogue (one output row per thread)
    float resid = 0.0f;
    if (p.epilogue == EPI_RESID && threadIdx.x < seg_rows[0]) resid = p.resid[seg_first[0] + threadIdx.x];
    TRACE(3);
    for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (lane == 0) red[warp] = ssq;
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
    float scale = 1.0f;
    if (p.scaled) {
        float tot = 0.0f;
        if (p.ss) {  // reference form: fixed-order sum of add_norm_prep's partials
            for (uint32_t i = 0; i < p.nss; ++i) tot += p.ss[i];
        } else {
            for (uint32_t i = 0; i < W; ++i) tot += red[i];
        }
        scale = 1.0f / sqrtf(tot / (float)p.cols + p.eps);
    }
    TRACE(4);
    // ---- the lane's share: the same half blocks of every row ----
    const uint32_t slice = warp % S, rw = warp / S;
    XFixed<GEMV_PLANES> xr[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t want = (slice * N + i) * 32 + lane;
        const uint32_t hbi = min(want, nhb - 1);
        xr[i] = x_fixed_load<GEMV_PLANES>(xf, hbi);
        if (want >= nhb) xr[i].step = 0.0f;  // lanes past the end of the row contribute nothing
    }
    const uint32_t hi_off = tiled_hi_off(p.cols), sc_off = tiled_scale_off(QT, p.cols);
    // When every lane's half blocks before its last iteration lie inside the row (all the model shapes), the loads use
    // addresses worked out once (row_pair_dot_at); the bias term then rides in the record's total.
    const bool fast = N < 2 || (S * N - 2) * 32 + 31 < nhb;
    const RowLaneOffsets lo = row_lane_offsets<QT, N>(p.cols, slice, lane);
    if (fast) {
#pragma unroll
        for (int i = 0; i < N; ++i) xr[i].total *= -(QT == BRASA_Q4_0 ? 8 : 32);
    }
    const uint32_t ring32 = smem_u32(ring);
    TRACE(5);

    // ---- consume: per iteration the block covers Wp * R rows of a segment; a warp takes R rows of one slot ----
    const uint32_t half_w = Wp / split;                     // row-warps per slot
    const uint32_t my_sub = split == 2 ? rw / half_w : 0;   // which of the iteration's slots
#pragma unroll
    for (int sgi = 0; sgi < 3; ++sgi) {
        const uint32_t nslots_seg = (seg_rows[sgi] + RPS - 1) / RPS;
        // Slots go to the two halves of the warps by the parity of their index in the block's whole list, and a reused
        // ring has an even number of slots: a ring slot is then always consumed by the same warps, which wait for every
        // one of its uses (a warp that skipped a use could mistake the previous phase for the one it waits for).
        for (uint32_t ks = split == 2 ? ((my_sub + seg_slot0[sgi]) & 1u) : 0u; ks < nslots_seg; ks += split) {
            const uint32_t k = seg_slot0[sgi] + ks, s = k % p.nslot;
            if (!mbar_wait(&full[s], (k / p.nslot) & 1)) {
                // give up on the remaining slots but still meet the other warps at the barrier below
                if (lane == 0) atomicExch(p.status, 2u);
                break;
            }
            if (k == 0) TRACE(6);
            // the slot's rows are shared out evenly among the warps that consume it (a last, partial slot
            // gives each warp fewer than R rows instead of leaving most warps idle)
            const uint32_t n_slot = min(RPS, seg_rows[sgi] - ks * RPS);
            const uint32_t q = (n_slot + half_w - 1) / half_w, in_slot = (rw % half_w) * q;
            const uint32_t nv = in_slot < n_slot ? min(q, n_slot - in_slot) : 0u;
            if (nv > 0) {
                const uint8_t *row0 = ring + (size_t)s * slot_bytes + (size_t)in_slot * row_bytes;
#pragma unroll 1
                for (uint32_t r = 0; r < nv; r += 2) {
                    const bool two = r + 1 < nv;
                    const uint8_t *row_a = row0 + (size_t)r * row_bytes, *row_b = two ? row_a + row_bytes : row_a;
                    float z;
                    if (fast) {
                        const uint32_t ra = ring32 + s * slot_bytes + (in_slot + r) * row_bytes;
                        z = row_pair_dot_at<QT, N, GEMV_PLANES>(ra, two ? ra + row_bytes : ra, lo, xr, lane);
                    } else {
                        z = row_pair_dot<QT, N>(row_a, row_b, xr, slice, nhb, hi_off, sc_off, lane);
                    }
                    // lane 0 holds row r, lane 8 row r + 1
                    if ((lane & 23) == 0 && (lane == 0 || two))
                        part[(seg_before[sgi] + ks * RPS + in_slot + r + (lane >> 3)) * S + slice] = z;
                }
            }
            __syncwarp();
            if (lane == 0 && k + p.nslot < total_slots) {
                __threadfence_block();
                if (atomicAdd(&done[s], 1u) == W / split - 1) {
                    done[s] = 0;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue(k + p.nslot);
                }
            }
        }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(CT) : "memory");
    TRACE(7);

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
                if (p.epilogue == EPI_RESID) v += (i == 0 && j == threadIdx.x) ? resid : p.resid[r];
                if (p.epilogue == EPI_PUSH) {
                    const uint32_t e = *reinterpret_cast<const volatile uint32_t *>(p.push.state);
                    const unsigned long long word = (unsigned long long)__float_as_uint(v) | ((unsigned long long)(e + 1) << 32);
                    const uint64_t at = (uint64_t)(e & 1) * p.push.world * p.push.max_elems + (uint64_t)p.push.rank * p.push.max_elems + r;
                    for (uint32_t q = 0; q < p.push.world; ++q)
                        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p.push.peer[q] + at), "l"(word) : "memory");
                } else {
                    p.y[i][r] = v;
                }
            }
        }
    }
    TRACE(8);
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

// Tells the next brasa_gemv_launch on this context which matrices the GEMV after it will read, so that it can
// ask L2 for them while it runs (tiled matrices sharing one column count; swiglu: gate and up row for row).
void brasa_gemv_hint_next(brasa_ctx *ctx, uint32_t nmat, const brasa_qmatrix *w, bool swiglu) {
    auto &n = ctx->gemv_next;
    n = {};
    if (nmat == 0 || nmat > 3) return;
    uint32_t total = 0;
    for (uint32_t i = 0; i < nmat; ++i) {
        if (w[i].layout != BRASA_LAYOUT_TILED) return;
        n.w[i] = arg_ptr(w[i].data);
        n.rows[i] = w[i].rows;
        total += w[i].rows;
    }
    n.nmat = nmat;
    n.swiglu = swiglu ? 1 : 0;
    n.row_bytes = tiled_row_bytes(w[0].qtype, w[0].cols);
    n.total_rows = swiglu ? w[0].rows : total;
}

// Shared by the model's fused decode path (model.cu) and the reference-shaped entry points below.
// epilogue: 0 scale, 1 SwiGLU (w[0] = gate, w[1] = up, y[0]), 2 residual (y = resid + W x).
int32_t brasa_gemv_launch(brasa_cmd *cmd, int qtype, uint32_t nmat, const brasa_qmatrix *w, float *const *y, const float *x,
                          const float *h, const float *normw, float *x_out, const float *ss, uint32_t nss, int scaled, float eps,
                          int epilogue, const float *resid, const brasa_tp_push_target *push) {
    brasa_ctx *ctx = cmd->ctx;
    GemvParams p{};
    if (epilogue == EPI_PUSH) {
        BRASA_REQUIRE(ctx, push && nmat == 1 && push->world >= 1 && w[0].rows <= push->max_elems, "gemv push: one matrix whose rows fit the exchange buffer");
        p.push = *push;
    }
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
    p.trace = ctx->gemv_trace;
    if (ctx->gemv_next.total_rows) {
        for (int i = 0; i < 3; ++i) { p.pf_w[i] = ctx->gemv_next.w[i]; p.pf_rows[i] = ctx->gemv_next.rows[i]; }
        p.pf_nmat = ctx->gemv_next.nmat; p.pf_total_rows = ctx->gemv_next.total_rows;
        p.pf_row_bytes = ctx->gemv_next.row_bytes; p.pf_swiglu = ctx->gemv_next.swiglu;
        ctx->gemv_next.total_rows = 0;
    }

    // column slices per row: the smallest power of two that keeps a lane's share of x within 5 half blocks
    const uint32_t nhb = p.cols / 16;
    uint32_t S = 1, N = (nhb + 31) / 32;
    while (N > 5 && S < GEMV_WARPS) {
        S *= 2;
        N = (nhb + 32 * S - 1) / (32 * S);
    }
    BRASA_REQUIRE(ctx, N <= 5, "gemv: %u columns are more than this kernel takes (%u)", p.cols, 5 * 32 * 16 * GEMV_WARPS);
    const uint32_t warps = GEMV_WARPS, Wp = warps / S;
    p.slices = S;
    p.warps = warps;
    p.total_rows = total_rows;
    p.rows_per_slot = (Wp & 1) ? Wp * R : Wp * R / 2;

    const uint32_t row_bytes = tiled_row_bytes(qtype, p.cols);
    const uint32_t slot_bytes = p.rows_per_slot * row_bytes;
    uint32_t grid = std::min<uint32_t>((uint32_t)ctx->sm_count, total_rows);
    uint32_t rows_per_block = (total_rows + grid - 1) / grid;
    uint32_t segs = epilogue == EPI_SWIGLU ? 2 : nmat;
    p.max_items = (rows_per_block + 1) * S * (epilogue == EPI_SWIGLU ? 2 : 1) + S * nmat;
    size_t fixed = (size_t)nhb * 16 * XRec<GEMV_PLANES>::CHUNKS + (size_t)((p.max_items + 1) & ~1u) * 4 + 160;
    uint32_t need_slots = (rows_per_block + 1 + p.rows_per_slot - 1) / p.rows_per_slot * (epilogue == EPI_SWIGLU ? 2 : 1) + segs;
    // When the block's whole share of rows fits next to a second block (100 KB each), stay under that: the
    // next kernel's block can then start on the same SM and prefetch its weights meanwhile. A larger share
    // takes the whole shared memory instead: a deep ring matters more than the overlap there.
    const size_t cap = 100 * 1024;
    size_t budget = fixed + (size_t)need_slots * (slot_bytes + 16) <= cap ? cap - fixed : ctx->smem_optin - fixed - 1024;
    BRASA_REQUIRE(ctx, fixed + slot_bytes + 1024 <= ctx->smem_optin, "gemv: %u columns do not fit shared memory", p.cols);
    uint32_t nslot = (uint32_t)std::min<size_t>(need_slots, budget / (slot_bytes + 16));
    if (nslot < need_slots && nslot > 1) nslot &= ~1u;  // reused ring: even, see the slot loop of the kernel
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
    BRASA_TRY(brasa_smem_optin(ctx, (const void *)kern, ctx->smem_optin));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(warps * 32);
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
                                        nss, scaled, eps, EPI_SCALE, nullptr, nullptr));
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
                             eps, EPI_SCALE, nullptr, nullptr);
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
                                 1, eps, EPI_SWIGLU, nullptr, nullptr);
    }
    // file layout: gate into y, up into scratch, then SwiGLU in place
    BRASA_TRY(brasa_gemv_scratch(ctx, gate.rows, 1));
    BRASA_TRY(gemv_file(cmd, gate, (const float *)arg_ptr(xw), (float *)arg_ptr(y), 1, (const float *)arg_ptr(ss), nss, eps, 1));
    BRASA_TRY(gemv_file(cmd, up, (const float *)arg_ptr(xw), ctx->gemv_partials, 1, (const float *)arg_ptr(ss), nss, eps, 1));
    swiglu_inplace_kernel<<<(gate.rows + 255) / 256, 256, 0, ctx->stream>>>((float *)arg_ptr(y), ctx->gemv_partials, gate.rows);
    return brasa_post_launch(cmd, "swiglu_inplace");
}

}  // extern "C"
