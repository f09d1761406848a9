// One decode token as ONE persistent kernel (the token loop of crates/models/src/qwen3.rs:551-831 for a single
// token, plus the greedy choice of crates/runtime/src/sampler.rs:148-170).
//
// A token is a chain of about 180 small dependent operations (per layer: QKV GEMV, attention, o_proj GEMV, gate/up
// GEMV, down GEMV). Launched as separate kernels each link costs about 10 us on B200 although its bytes need 1-4 us,
// so the chain runs here inside one cooperative launch, one block per SM:
//   * Weights never wait. Every block owns the same share of rows of every matrix, known when the model is loaded,
//     so its weight traffic is a fixed list of byte ranges (slots). They stream through a shared-memory ring with
//     bulk async copies; the warp that is last to finish with a slot starts the copy that reuses it, across
//     operation boundaries. HBM keeps working while the blocks exchange activations.
//   * Activations cross blocks without barriers. Every operation has its own output vector in L2, twice (launches
//     alternate between the two copies). A word holds either the float or the bit pattern VS_EMPTY, a NaN no
//     arithmetic produces; a consumer polls the words it needs until none is empty. A 4-byte store is indivisible, so
//     no fence, flag or grid barrier is needed, and one round trip to L2 both synchronises and delivers the data.
//     The thread that writes a word of this launch's copy also empties the same word of the other copy, which the
//     launch before wrote and read and the next launch will fill: the end of the kernel orders that store before
//     every load of the next launch, so inside one launch a word changes exactly once, from empty to its value.
//     (Attention partials, the argmax candidates and the words that cross GPUs are 8-byte {float, epoch} words,
//     valid when they carry the epoch of the producing operation of this launch.)
//   * Every poll and every mbarrier wait is bounded. A wait that runs out sets the context's status word and a
//     block-wide flag after which the block stops waiting and runs to its end; the host reports BRASA_ETIMEOUT.
// GEMV arithmetic, x conversion and epilogues are those of gemv.cu (same rounding); attention works on 64-key
// chunks (32 for an f32 cache) shared out over the blocks and is merged per head by the blocks at the far end of
// the grid.
#include <stdlib.h>

#include <memory>

#include "attn_device.cuh"
#include "decode_token.h"
#include "gemv_device.cuh"

using namespace brasa_dev;

namespace {

constexpr int TK_WARPS = 16, TK_THREADS = TK_WARPS * 32;
constexpr uint32_t SLOT_CAP = 24 * 1024;   // bytes of one ring slot
constexpr uint32_t POLL_LIMIT = 1u << 20;  // polls of an activation word before the wait gives up
constexpr int R = 2;                       // rows a warp works on at a time
constexpr int NMAX = 5;                    // half blocks of x a lane keeps per column slice
constexpr uint32_t EPOCH_SPAN = 1024;      // epochs of one launch; operations + 2 must stay below it
constexpr uint32_t VS_EMPTY = 0xffffffffu;  // an activation word nobody has written in this launch

enum { OP_GEMV = 0, OP_ATTN = 1 };
enum { IN_LL = 0, IN_EMBED = 1 };
enum { EPI_SCALE = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_LOGITS = 3 };

struct SlotDesc {
    const uint8_t *src;
    uint32_t bytes;
    uint32_t pad;
};

struct TokOp {
    uint32_t type, qtype, cols, nmat;
    uint32_t rows[3], total_rows;
    uint32_t epilogue, scaled, log2S, nact;
    uint32_t in_kind, in_op, save_resid, next_cols;  // next_cols: length of next_normw
    float eps;
    uint32_t xchg;  // tensor parallel: 1 + index of this residual add among the token's exchanges (0: no exchange)
    uint32_t fast;  // every lane's half blocks before its last iteration lie inside the row (see gemv_rows)
    uint32_t pad1[1];
    const uint8_t *w[3];
    const float *normw;
    const uint32_t *in;  // first copy; the second one lies TokParams::par_words further
    uint32_t *out;
    const float *q_norm, *k_norm;
    uint8_t *kc, *vc;
    const float *next_normw;  // norm weight of the operation after this one (null: none): staged in shared memory meanwhile
    uint64_t pad2;
};
constexpr uint32_t OP_WORDS = sizeof(TokOp) / 4;
constexpr uint32_t OPS_WORDS = OP_WORDS + 4;  // in shared memory the block's row counts follow the operation
static_assert(sizeof(TokOp) % 16 == 0, "TokOp is copied as words");

struct TokParams {
    const TokOp *ops;
    uint32_t nops;
    const SlotDesc *slots;
    const uint32_t *slot_begin;  // [grid + 1]
    const uint4 *block_ops;      // [nops][grid]: first output row, rows of segments 0 | 1 << 16, rows of segment 2, -
    uint32_t nslot, xf_bytes, part_floats, resid_floats, sdesc_n, nw_floats;
    uint32_t par_words;  // words of one copy of the activation vectors
    uint32_t *state, *ids, *next_id, *out_ids;
    uint32_t out_cap;
    const uint8_t *embed;
    uint32_t vocab, hidden, heads, kv_heads, max_chunks;
    const float *cos_t, *sin_t;
    float *logits;
    unsigned long long *cand;      // [grid][2]: best logit, its index
    unsigned long long *partials;  // [heads][max_chunks][130]
    float attn_scale;
    uint32_t *status;
    unsigned long long *trace;  // optional: block 0 stamps the phases of 16 operations from trace_op on (debugging aid)
    uint32_t trace_op;
    // tensor parallel (tp_world > 1): every rank's exchange area as seen from here, see brasa_tp_token_area
    uint32_t tp_world, tp_rank, tp_row0, tp_poll_limit;
    unsigned long long tp_stride;
    unsigned long long *tp_peer[BRASA_TP_MAX_RANKS];
};

struct Best {
    float v;
    uint32_t i;
};
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

__device__ __forceinline__ void ll_store(unsigned long long *p, uint32_t bits, uint32_t epoch) {
    unsigned long long w = ((unsigned long long)epoch << 32) | bits;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// An activation word of this launch's copy, and the same word of the other copy emptied for the next launch.
__device__ __forceinline__ void vs_store(uint32_t *cur, uint32_t *alt, uint32_t bits) {
    if (bits == VS_EMPTY) bits = 0x7fffffffu;  // this one NaN pattern means "empty": another NaN takes its place
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(cur), "r"(bits) : "memory");
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(alt), "r"(VS_EMPTY) : "memory");
}
__device__ __forceinline__ uint32_t vs_load(const uint32_t *p) {
    uint32_t w;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ uint4 vs_load4(const uint32_t *p) {  // four words, each indivisible on its own
    uint4 w;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(p) : "memory");
    return w;
}

// Words that cross GPUs (a peer's store into this rank's exchange area over NVLink): system scope.
__device__ __forceinline__ void xg_store(unsigned long long *p, uint32_t bits, uint32_t epoch) {
    unsigned long long w = ((unsigned long long)epoch << 32) | bits;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long xg_load(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// Rows of block b: logical rows [r0, r1) of `total` (matrices one after another; SwiGLU: the rows of gate, up follows
// the same range), cut into per-matrix segments.
BRASA_HD inline void block_rows(uint32_t total, uint32_t nmat, const uint32_t rows[3], bool swiglu, uint32_t b, uint32_t G, uint32_t &r0,
                                uint32_t &r1, uint32_t first[3], uint32_t nrows[3]) {
    r0 = (uint32_t)((uint64_t)total * b / G);
    r1 = (uint32_t)((uint64_t)total * (b + 1) / G);
    uint32_t base = 0;
    const uint32_t nseg = swiglu ? 2 : nmat;
    for (int i = 0; i < 3; ++i) {
        first[i] = 0;
        nrows[i] = 0;
        if ((uint32_t)i < nseg) {
            if (swiglu) {
                first[i] = r0;
                nrows[i] = r1 - r0;
            } else {
                uint32_t lo = r0 > base ? r0 : base, hi = r1 < base + rows[i] ? r1 : base + rows[i];
                first[i] = lo > base ? lo - base : 0;
                nrows[i] = hi > lo ? hi - lo : 0;
                base += rows[i];
            }
        }
    }
}

// 16 values of row `row` of a tiled q6_0 table as the four quads of half block hbi (embed_kernel's arithmetic).
__device__ __forceinline__ void embed_half_block(const uint8_t *table, uint32_t row, uint32_t cols, uint32_t hbi, float4 q[4]) {
    const uint8_t *r = table + (size_t)row * tiled_row_bytes(BRASA_Q6_0, cols);
    const uint2 codes = *reinterpret_cast<const uint2 *>(r + hbi * 8);
    const uint32_t hb = *reinterpret_cast<const uint32_t *>(r + tiled_hi_off(cols) + hbi * 4);
    const float d = __half2float(*reinterpret_cast<const __half *>(r + tiled_scale_off(BRASA_Q6_0, cols) + (hbi >> 1) * 2));
    uint32_t a[4];
    a[0] = lop_and_or(hb, 0x30303030u, codes.x & 0x0F0F0F0Fu);
    a[1] = lop_and_or(hb >> 2, 0x30303030u, (codes.x >> 4) & 0x0F0F0F0Fu);
    a[2] = lop_and_or(hb << 2, 0x30303030u, codes.y & 0x0F0F0F0Fu);
    a[3] = lop_and_or(hb << 4, 0x30303030u, (codes.y >> 4) & 0x0F0F0F0Fu);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        q[j].x = d * (float)((int)(a[j] & 255u) - 32);
        q[j].y = d * (float)((int)((a[j] >> 8) & 255u) - 32);
        q[j].z = d * (float)((int)((a[j] >> 16) & 255u) - 32);
        q[j].w = d * (float)((int)(a[j] >> 24) - 32);
    }
}

#ifdef BRASA_TRACE_BUILD
#define TRACEB(i) do { if (c.trace && threadIdx.x == 0 && c.oi >= c.trace_op && c.oi < c.trace_op + 5) c.trace[512 + ((c.oi - c.trace_op) * 160 + c.b) * 4 + (i)] = gtime(); } while (0)
#define TRACE(i) do { if (c.trace && c.b == 0 && threadIdx.x == 0 && c.oi >= c.trace_op && c.oi < c.trace_op + 16) c.trace[16 + (c.oi - c.trace_op) * 16 + (i)] = (unsigned long long)clock64(); } while (0)
#else
#define TRACE(i) do { } while (0)
#define TRACEB(i) do { } while (0)
#endif

// What the phases of an operation share. The phase functions are inlined: with 227 KB of shared memory in use the
// L1 cache is a few KB, so a stack frame (calls, spills) costs a trip to L2 per access.
struct TokCtx {
    uint8_t *ring, *xfb;
    float *part, *resid, *red, *nwbuf;
    uint4 *sdesc;
    uint64_t *full;
    uint32_t *done;
    volatile uint32_t *s_abort;
    const uint4 *myslots;
    uint32_t *status;
    unsigned long long *trace;
    uint32_t trace_op, my_slots, nslot, G, b, pos, seq, token, h0, hn;
    uint32_t par_cur, par_alt;  // word offsets of this launch's copy of the activation vectors and of the other one
    uint32_t oi;  // current operation (trace builds)
};

// This warp's place in the block's slot list: next list index, its ring slot, that use's phase parity.
struct WarpRing {
    uint32_t kk, rs, rph;
};

// A wait ran out: remember it, stop waiting in this block.
__device__ __forceinline__ void give_up(const TokCtx &c, uint32_t code) {
    atomicExch(c.status, code);
    *c.s_abort = 1;
}

// Four activation words at once: all loads in flight together, so a wait costs one round trip to L2 when the data is there.
__device__ __forceinline__ void ll_wait4(const TokCtx &c, const unsigned long long *p0, const unsigned long long *p1, const unsigned long long *p2,
                                         const unsigned long long *p3, uint32_t epoch, uint32_t out[4]) {
    for (uint32_t it = 0;; ++it) {
        const unsigned long long w0 = ll_load(p0), w1 = ll_load(p1), w2 = ll_load(p2), w3 = ll_load(p3);
        out[0] = (uint32_t)w0; out[1] = (uint32_t)w1; out[2] = (uint32_t)w2; out[3] = (uint32_t)w3;
        const bool ok = (uint32_t)(w0 >> 32) == epoch && (uint32_t)(w1 >> 32) == epoch && (uint32_t)(w2 >> 32) == epoch && (uint32_t)(w3 >> 32) == epoch;
        if (ok || *c.s_abort) break;
        if (it >= POLL_LIMIT) {
            give_up(c, 3);
            break;
        }
    }
}

// Four activation words of a vector (attention's q, k, v rows).
__device__ __forceinline__ void vs_wait4(const TokCtx &c, const uint32_t *p0, const uint32_t *p1, const uint32_t *p2, const uint32_t *p3, uint32_t out[4]) {
    for (uint32_t it = 0;; ++it) {
        out[0] = vs_load(p0); out[1] = vs_load(p1); out[2] = vs_load(p2); out[3] = vs_load(p3);
        const bool ok = out[0] != VS_EMPTY && out[1] != VS_EMPTY && out[2] != VS_EMPTY && out[3] != VS_EMPTY;
        if (ok || *c.s_abort) break;
        if (it >= POLL_LIMIT) {
            give_up(c, 3);
            break;
        }
    }
}

// Bounded wait for a ring slot's bytes. The block's abort flag is looked at only while the wait has to spin, so a slot
// that is already there costs one try. False when the limit ran out.
__device__ __forceinline__ bool slot_wait(const TokCtx &c, uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
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
        if ((it & 15) == 15 && *c.s_abort) return true;  // the block has given up: nobody waits any more
    }
    return false;
}

// a slot descriptor {address lo, address hi, bytes, -} -> ring[s]
__device__ __forceinline__ void issue_slot(const TokCtx &c, uint4 d, uint32_t s) {
    const uint8_t *src = reinterpret_cast<const uint8_t *>(((unsigned long long)d.y << 32) | d.x);
    mbar_expect_tx(&c.full[s], d.z);
    bulk_g2s(c.ring + (size_t)s * SLOT_CAP, src, d.z, &c.full[s]);
}

// ---- GEMV, phase 1: wait for the input, fold the norm weight, convert to fixed point. A thread takes one quad of four
// values at a time (quads t, t + 512, ..), so that the whole block polls at once; the four lanes of a half block share
// its largest magnitude and its integer sum by shuffles and each writes its own words of the record (the record
// x_half_block_to_fixed builds, same arithmetic). Returns the thread's share of sum x^2. (Asking for all of a thread's
// quads at once measured 5 % slower over the token than one quad after the other: polls and weights share the L2.)

// element index of quad qi: the quads of a half block start at +0, +16, +4, +20
__device__ __forceinline__ uint32_t quad_elem(uint32_t qi) {
    const uint32_t hbi = qi >> 2, j = qi & 3;
    return (hbi >> 1) * 32 + 8 * (hbi & 1) + 16 * (j & 1) + 2 * (j & 2);
}

template <int P>
__device__ __forceinline__ void quad_to_fixed(const TokCtx &c, const TokOp &op, uint32_t *xw, uint32_t qi, float4 v, float &ssq) {
    constexpr uint32_t BITS = P == 3 ? 22 : 16;
    const uint32_t hbi = qi >> 2, j = qi & 3, e = quad_elem(qi);
    ssq = fmaf(v.x, v.x, ssq); ssq = fmaf(v.y, v.y, ssq); ssq = fmaf(v.z, v.z, ssq); ssq = fmaf(v.w, v.w, ssq);
    if (op.save_resid) {  // this vector is the residual a later epilogue adds: keep this block's rows
        const uint32_t r = e - c.h0;  // wraps for rows before h0
        if (r + 0 < c.hn) c.resid[r + 0] = v.x;
        if (r + 1 < c.hn) c.resid[r + 1] = v.y;
        if (r + 2 < c.hn) c.resid[r + 2] = v.z;
        if (r + 3 < c.hn) c.resid[r + 3] = v.w;
    }
    if (op.normw) {
        const float4 nw = *reinterpret_cast<const float4 *>(c.nwbuf + e);
        v.x *= nw.x; v.y *= nw.y; v.z *= nw.z; v.w *= nw.w;
    }
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // step = 2^(exponent(amax) - (BITS - 2)); zero (or denormal) groups get step 0; infinities travel in the step
    const uint32_t ebits = __float_as_uint(amax) & 0x7F800000u;
    const bool live = ebits > ((BITS - 1) << 23) && ebits < 0x7F800000u;
    const float step = live ? __uint_as_float(ebits - ((BITS - 2) << 23)) : (ebits == 0x7F800000u ? amax : 0.0f);
    const float inv = live ? __uint_as_float((254u << 23) - (ebits - ((BITS - 2) << 23))) : 0.0f;  // 1 / step, exact
    int X[4] = {__float2int_rn(v.x * inv), __float2int_rn(v.y * inv), __float2int_rn(v.z * inv), __float2int_rn(v.w * inv)};
    if (P == 2) {  // a value that rounds up to 2^15 stays inside the signed top byte
#pragma unroll
        for (int k = 0; k < 4; ++k) X[k] = min(X[k], 32767);
    }
    int total = X[0] + X[1] + X[2] + X[3];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    // byte planes of the four integers: byte k of every X gathered into one word
    const uint32_t lo01 = __byte_perm(X[0], X[1], 0x5140), lo23 = __byte_perm(X[2], X[3], 0x5140);
    const uint32_t w0 = __byte_perm(lo01, lo23, 0x5410), w1 = __byte_perm(lo01, lo23, 0x7632);
    if (P == 3) {
        const uint32_t hi01 = __byte_perm(X[0], X[1], 0x7362), hi23 = __byte_perm(X[2], X[3], 0x7362);
        const uint32_t w2 = __byte_perm(hi01, hi23, 0x5410);
        const uint32_t sw = (hbi >> 1) & 3;  // record words 3j .. 3j + 2; 16-byte chunk n of a record lies at n ^ sw
        const uint32_t i0 = 3 * j, i1 = 3 * j + 1, i2 = 3 * j + 2;
        xw[(hbi * 4 + ((i0 >> 2) ^ sw)) * 4 + (i0 & 3)] = w0;
        xw[(hbi * 4 + ((i1 >> 2) ^ sw)) * 4 + (i1 & 3)] = w1;
        xw[(hbi * 4 + ((i2 >> 2) ^ sw)) * 4 + (i2 & 3)] = w2;
        if (j == 0) *reinterpret_cast<uint4 *>(xw + (hbi * 4 + (3 ^ sw)) * 4) = make_uint4((uint32_t)total, __float_as_uint(step), 0, 0);
    } else {
        *reinterpret_cast<uint2 *>(xw + hbi * 12 + 2 * j) = make_uint2(w0, w1);
        if (j == 0) *reinterpret_cast<uint4 *>(xw + hbi * 12 + 8) = make_uint4((uint32_t)total, __float_as_uint(step), 0, 0);
    }
}

template <int P>
__device__ __forceinline__ float gemv_input(const TokCtx &c, const TokOp &op, const uint8_t *embed, uint32_t vocab) {
    const int tid = threadIdx.x;
    const uint32_t cols = op.cols, nq = cols / 4;  // a multiple of 64: a warp is inside or outside as a whole
    uint32_t *xw = reinterpret_cast<uint32_t *>(c.xfb);
    const uint32_t *in = op.in + c.par_cur;
    float ssq = 0.0f;
    if (op.in_kind == IN_EMBED) {
#pragma unroll 1
        for (uint32_t qi = tid; qi < nq; qi += TK_THREADS) {
            const uint32_t j = qi & 3;
            float4 q[4];
            if (c.token < vocab) embed_half_block(embed, c.token, cols, qi >> 2, q);
            else q[0] = q[1] = q[2] = q[3] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            quad_to_fixed<P>(c, op, xw, qi, j == 0 ? q[0] : (j == 1 ? q[1] : (j == 2 ? q[2] : q[3])), ssq);
        }
        return ssq;
    }
#pragma unroll 1
    for (uint32_t qi = tid; qi < nq; qi += 2 * TK_THREADS) {  // two quads of the thread in flight: half the round trips
        const uint32_t qj = qi + TK_THREADS;
        const bool two = qj < nq;
        uint4 w0, w1 = make_uint4(0, 0, 0, 0);
        for (uint32_t it = 0;; ++it) {
            w0 = vs_load4(in + quad_elem(qi));
            if (two) w1 = vs_load4(in + quad_elem(qj));
            const bool ok = w0.x != VS_EMPTY && w0.y != VS_EMPTY && w0.z != VS_EMPTY && w0.w != VS_EMPTY &&
                            w1.x != VS_EMPTY && w1.y != VS_EMPTY && w1.z != VS_EMPTY && w1.w != VS_EMPTY;
            if (ok || *c.s_abort) break;
            if (it >= POLL_LIMIT) {
                give_up(c, 3);
                break;
            }
        }
        TRACE(2);
        quad_to_fixed<P>(c, op, xw, qi, make_float4(__uint_as_float(w0.x), __uint_as_float(w0.y), __uint_as_float(w0.z), __uint_as_float(w0.w)), ssq);
        if (two) quad_to_fixed<P>(c, op, xw, qj, make_float4(__uint_as_float(w1.x), __uint_as_float(w1.y), __uint_as_float(w1.z), __uint_as_float(w1.w)), ssq);
    }
    return ssq;
}

// ---- GEMV, phase 2: the rows. A slot holds up to RPS rows of one segment; its eight warps (half_w rows x S slices)
// share them; a lane keeps the same half blocks of x for every row.
// NACT > 0: the operation's half blocks per lane are known when the kernel is built and every lane's half blocks but those
// of the last iteration lie inside the row (TokOp::fast): loads at addresses worked out once (row_pair_dot_at).
// NACT = 0: any shape the kernel takes, addresses worked out per half block.
template <int QT, int P, int NACT>
__device__ __forceinline__ WarpRing gemv_rows(const TokCtx &c, const TokOp &op, const uint32_t *bo, uint32_t gslot, const WarpRing wr) {
    constexpr int NX = NACT > 0 ? NACT : NMAX;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cols = op.cols, nhb = cols / 16, lS = op.log2S, S = 1u << lS, nact = op.nact;
    const uint32_t lRPS = 4 - lS, RPS = 1u << lRPS, lhw = lRPS - 1, half_w = 1u << lhw;  // rows per slot = warps side by side
    const uint32_t row_bytes = tiled_row_bytes(QT, cols);
    const uint32_t rows0 = bo[1] & 0xffffu, rows1 = bo[1] >> 16, rows2 = bo[2];
    const uint32_t sl0 = (rows0 + RPS - 1) >> lRPS, sl1 = sl0 + ((rows1 + RPS - 1) >> lRPS), total_slots = sl1 + ((rows2 + RPS - 1) >> lRPS);
    const uint4 *xf = reinterpret_cast<const uint4 *>(c.xfb);
    const uint32_t slice = warp & (S - 1), rwl = (warp >> lS) & (half_w - 1);
    XFixed<P> xr[NX];
#pragma unroll
    for (int i = 0; i < NX; ++i) {
        const uint32_t want = (slice * nact + i) * 32 + lane;
        const uint32_t hbi = min(want, nhb - 1);
        xr[i] = x_fixed_load<P>(xf, hbi);
        if (want >= nhb || (uint32_t)i >= nact) xr[i].step = 0.0f;  // lanes past the end of the row, unused registers
        if (NACT > 0) xr[i].total *= -(QT == BRASA_Q4_0 ? 8 : 32);  // the bias term of half_block_idot_pre
    }
    const uint32_t hi_off = tiled_hi_off(cols), sc_off = tiled_scale_off(QT, cols);
    RowLaneOffsets lo{};
    if (NACT > 0) lo = row_lane_offsets<QT, NX>(cols, slice, lane);
    const uint32_t ring32 = smem_u32(c.ring);
    uint32_t kk = wr.kk, rs = wr.rs, rph = wr.rph;
    bool first_slot = true;
    TRACE(5);
#pragma unroll 1
    for (uint32_t j = kk - gslot; j < total_slots; j += 2) {
        const uint32_t sgi = (j >= sl0) + (j >= sl1);
        const uint32_t ks = j - (sgi == 0 ? 0u : (sgi == 1 ? sl0 : sl1));
        const uint32_t sg_rows = sgi == 0 ? rows0 : (sgi == 1 ? rows1 : rows2), sg_before = sgi == 0 ? 0u : (sgi == 1 ? rows0 : rows0 + rows1);
#ifdef BRASA_TRACE_BUILD
        const long long tw0 = clock64();
#endif
        if (!slot_wait(c, &c.full[rs], rph) && lane == 0) give_up(c, 2);
#ifdef BRASA_TRACE_BUILD
        if (c.trace && c.b == 0 && (threadIdx.x == 0 || threadIdx.x == 256) && c.oi >= c.trace_op && c.oi < c.trace_op + 16) {
            const uint32_t rnd = (j - (kk - gslot - (kk - gslot) % 2)) ;  // unused
            (void)rnd;
            const uint32_t round = (j >> 1) & 7;
            c.trace[4096 + ((c.oi - c.trace_op) * 2 + (threadIdx.x >> 8)) * 16 + round * 2] = (unsigned long long)(clock64() - tw0);
            c.trace[4096 + ((c.oi - c.trace_op) * 2 + (threadIdx.x >> 8)) * 16 + round * 2 + 1] = (unsigned long long)tw0;
        }
#endif
        if (first_slot) {
            TRACE(6);
            first_slot = false;
        }
        const uint32_t n_slot = min(RPS, sg_rows - (ks << lRPS));
        const uint32_t qn = (n_slot + half_w - 1) >> lhw, in_slot = rwl * qn;
        const uint32_t nv = in_slot < n_slot ? min(qn, n_slot - in_slot) : 0u;
        const uint8_t *row0 = c.ring + (size_t)rs * SLOT_CAP + (size_t)in_slot * row_bytes;
        const uint32_t row0_32 = ring32 + rs * SLOT_CAP + in_slot * row_bytes;
        uint32_t r = 0;
#pragma unroll 1
        for (; r + 1 < nv; r += 2) {
            float z;
            if (NACT > 0) {
                z = row_pair_dot_at<QT, NX, P>(row0_32 + r * row_bytes, row0_32 + (r + 1) * row_bytes, lo, xr, lane);
            } else {
                const uint8_t *row_a = row0 + (size_t)r * row_bytes;
                z = row_pair_dot<QT, NX>(row_a, row_a + row_bytes, xr, slice, nhb, hi_off, sc_off, lane, (int)nact);
            }
            if ((lane & 23) == 0) c.part[((sg_before + (ks << lRPS) + in_slot + r + (lane >> 3)) << lS) + slice] = z;
        }
        if (r < nv) {  // an odd row on its own: half the work of a pair (short last slots are shared out one row per warp)
            float z;
            if (NACT > 0) z = row_single_dot_at<QT, NX, P>(row0_32 + r * row_bytes, lo, xr);
            else z = row_single_dot<QT, NX>(row0 + (size_t)r * row_bytes, xr, slice, nhb, hi_off, sc_off, lane, (int)nact);
            if (lane == 0) c.part[((sg_before + (ks << lRPS) + in_slot + r) << lS) + slice] = z;
        }
        __syncwarp();
        if (lane == 0 && kk + c.nslot < c.my_slots) {
            // (the warp's reads of the slot are complete: their values went into the sums stored above)
            if (atomicAdd(&c.done[rs], 1u) == TK_WARPS / 2 - 1) {  // last of the eight: the slot is free, refill it
                c.done[rs] = 0;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_slot(c, c.sdesc[j], rs);
            }
        }
        kk += 2;
        rs += 2;
        if (rs >= c.nslot) {
            rs -= c.nslot;
            rph ^= 1;
        }
    }
    return WarpRing{kk, rs, rph};
}

// ---- GEMV, phase 3: one thread per output row of this block; the result goes out as activation words.
__device__ __forceinline__ void gemv_epilogue(const TokCtx &c, const TokOp &op, const uint32_t *bo, float scale, uint32_t epoch, float *logits,
                                           unsigned long long *cand, const TokParams &p) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t lS = op.log2S, S = 1u << lS;
    const bool swiglu = op.epilogue == EPI_SWIGLU;
    const uint32_t r0 = bo[0], rows0 = bo[1] & 0xffffu, rows1 = bo[1] >> 16, rows2 = bo[2];
    const uint32_t nr = swiglu ? rows0 : rows0 + rows1 + rows2;  // segments follow one another in part[] and in the output
    const float *part = c.part;
    Best bst{-INFINITY, 0xffffffffu};
#ifdef BRASA_TRACE_BUILD
    {
        TRACE(13);
        volatile float dummy = *reinterpret_cast<volatile float *>(c.part);
        if (dummy == 1.2345e-33f) c.part[0] = 0.0f;
        TRACE(14);
        volatile uint32_t d2 = *reinterpret_cast<volatile uint32_t *>(&c.red[40]);
        if (d2 == 0x12345678u) c.part[0] = 0.0f;
        TRACE(15);
    }
#endif
#pragma unroll 1
    for (uint32_t j = tid; j < nr; j += TK_THREADS) {
        float v = 0.0f;
#pragma unroll 1
        for (uint32_t sl = 0; sl < S; ++sl) v += part[(j << lS) + sl];
        v *= scale;
        if (swiglu) {
            float u = 0.0f;
#pragma unroll 1
            for (uint32_t sl = 0; sl < S; ++sl) u += part[((nr + j) << lS) + sl];
            u *= scale;
            v = (v / (1.0f + expf(-v))) * u;
        }
        if (op.epilogue == EPI_RESID && op.xchg) {
            // Tensor parallel: v is this rank's share of the sum over the split columns. It goes into slot [this rank] of
            // every rank's exchange area (parity of the exchange: a slot is rewritten two exchanges later, when its
            // reader has long passed); the owner of the row on every rank then adds the slots in rank order, so all
            // ranks hold the same bits.
            const size_t base = (size_t)((op.xchg - 1) & 1) * p.tp_world * p.tp_stride + r0 + j;
            for (uint32_t q = 0; q < p.tp_world; ++q) xg_store(p.tp_peer[q] + base + (size_t)p.tp_rank * p.tp_stride, __float_as_uint(v), epoch);
            // all ranks' slots are asked for together and only the missing ones again: one round trip once they are there
            const unsigned long long *mine = p.tp_peer[p.tp_rank] + base;
            unsigned long long w[BRASA_TP_MAX_RANKS];
#pragma unroll
            for (int q = 0; q < BRASA_TP_MAX_RANKS; ++q) w[q] = 0;  // epoch 0 is never a launch's
            for (uint32_t it = 0;; ++it) {
                bool ok = true;
#pragma unroll
                for (int q = 0; q < BRASA_TP_MAX_RANKS; ++q) {
                    if ((uint32_t)q < p.tp_world && (uint32_t)(w[q] >> 32) != epoch) {
                        w[q] = xg_load(mine + (size_t)q * p.tp_stride);
                        ok = ok && (uint32_t)(w[q] >> 32) == epoch;
                    }
                }
                if (ok || *c.s_abort) break;
                if (it >= p.tp_poll_limit) {
                    give_up(c, 6);
                    break;
                }
            }
            float sum = __uint_as_float((uint32_t)w[0]);
#pragma unroll
            for (int q = 1; q < BRASA_TP_MAX_RANKS; ++q)
                if ((uint32_t)q < p.tp_world) sum += __uint_as_float((uint32_t)w[q]);
            v = sum;
        }
        if (op.epilogue == EPI_RESID) v += c.resid[j];
        if (op.epilogue == EPI_LOGITS) {
            logits[r0 + j] = v;
            if (v > bst.v) bst = Best{v, r0 + j};
        } else {
            TRACE(9);
            vs_store(op.out + c.par_cur + r0 + j, op.out + c.par_alt + r0 + j, __float_as_uint(v));
            TRACE(10);
        }
    }
    if (op.epilogue == EPI_LOGITS) {  // this block's best logit for the greedy choice
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, bst.v, o), __shfl_xor_sync(0xffffffffu, bst.i, o)};
            bst = better(bst, other);
        }
        if (lane == 0) { c.red[16 + warp] = bst.v; c.red[32 + warp] = __uint_as_float(bst.i); }
        __syncthreads();
        if (tid == 0) {
#pragma unroll 1
            for (int w = 1; w < TK_WARPS; ++w) bst = better(bst, Best{c.red[16 + w], __float_as_uint(c.red[32 + w])});
            ll_store(cand + 2 * c.b, __float_as_uint(bst.v), epoch);
            ll_store(cand + 2 * c.b + 1, bst.i, epoch);
        }
    }
}

// ---- attention of this token over the cache, new row included ----
template <int KV>
__device__ __forceinline__ void attention_op(const TokCtx &c, const TokOp &op, uint32_t oi, uint32_t epoch, uint32_t heads,
                                          uint32_t kv_heads, uint32_t max_chunks, const float *cos_t, const float *sin_t,
                                          unsigned long long *partials, float attn_scale) {
    constexpr int RB = KvRow<KV>::BYTES, RS = KvRow<KV>::STRIDE;
    constexpr uint32_t C = KV == BRASA_KV_F32 ? 32 : 64;  // keys per work item
    constexpr int KPW = C / TK_WARPS, LPK = 32 / KPW, DPL = 128 / LPK;  // keys per warp, lanes per key, dims per lane
    // q in shared memory: 16-float segments 20 floats apart, so the lanes of a key (one segment or half segment each)
    // read conflict-free
    constexpr int QS_SEG = 20, QS_HEAD = 8 * QS_SEG;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t Gq = heads / kv_heads, pos = c.pos;
    const uint32_t lk = pos + 1, nchunks = (lk + C - 1) / C;
    uint8_t *kt = c.xfb, *vt = c.xfb + C * RS;
    float *qs = reinterpret_cast<float *>(vt + C * RS);  // [8][QS_HEAD]
    float *ps = qs + 8 * QS_HEAD;                        // [8][C]
    float *red = c.red;
    // A work item is (kv head, group of consecutive chunks). While the chunks are few there is one chunk per group;
    // a long cache has more chunks than the grid has blocks per kv head, and a block then walks its group's chunks with
    // a running maximum and sum, so that a head is merged from a dozen partial results instead of hundreds.
    const uint32_t groups_max = max(1u, c.G / kv_heads);
    const uint32_t cpg = (nchunks + groups_max - 1) / groups_max, ngroups = (nchunks + cpg - 1) / cpg;
    const uint32_t nitems = kv_heads * ngroups;
#pragma unroll 1
    for (uint32_t item = c.b; item < nitems; item += c.G) {
        const uint32_t kh = item / ngroups, gi = item - kh * ngroups;
        const uint32_t ch_lo = gi * cpg, ch_hi = min(nchunks, ch_lo + cpg);
        float run[8][2];  // this thread's share (its key class) of an output element pair of every head
#pragma unroll
        for (int g = 0; g < 8; ++g) run[g][0] = run[g][1] = 0.0f;
        if (tid < 8) { red[16 + tid] = -INFINITY; red[24 + tid] = 0.0f; }  // running maximum and sum per head
        // The cached rows of chunk ch2 into a tile, one copy group per tile. K of the next chunk is asked for as soon as the
        // scores of this one are out, V as soon as P V is done, so a block that walks several chunks (a long cache) waits
        // for neither; groups complete in the order K(ch), V(ch), K(ch + 1), .., and every wait below leaves one pending.
        auto load_tile = [&](uint8_t *tile, const uint8_t *cache, uint32_t ch2) {
            if (ch2 < ch_hi) {
                constexpr int VEC = KV == BRASA_KV_Q8_0 ? 8 : 16, PER_ROW = RB / VEC;
                const uint32_t k0 = ch2 * C, nk = min(C, lk - k0), n = ch2 == nchunks - 1 ? nk - 1 : nk;  // the new row is not in the cache yet
#pragma unroll 1
                for (uint32_t i = tid; i < n * PER_ROW; i += TK_THREADS) {
                    const uint32_t r = i / PER_ROW, v = i % PER_ROW;
                    const size_t goff = ((size_t)(k0 + r) * kv_heads + kh) * RB + (size_t)v * VEC;
                    if (KV == BRASA_KV_Q8_0) cp_async8(tile + r * RS + v * VEC, cache + goff);
                    else cp_async16(tile + r * RS + v * VEC, cache + goff);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        load_tile(kt, op.kc, ch_lo);
        load_tile(vt, op.vc, ch_lo);
#pragma unroll 1
        for (uint32_t ch = ch_lo; ch < ch_hi; ++ch) {
        const uint32_t key0 = ch * C, nkeys = min(C, lk - key0);
        const bool has_new = ch == nchunks - 1;
        if ((uint32_t)warp < Gq + 2 && (((uint32_t)warp < Gq && ch == ch_lo) || ((uint32_t)warp >= Gq && has_new))) {
            // warps 0 .. Gq-1: a query head (once per item); warp Gq: the new key row; warp Gq + 1: the new value row
            const uint32_t g = warp;
            const uint32_t *src = op.in + c.par_cur + (g < Gq ? (size_t)(kh * Gq + g) * 128 : (size_t)(heads + (g - Gq) * kv_heads + kh) * 128);
            float xv[4], y[4], wv[4], cs[2], sn[2];
            {   // what does not depend on this token's q, k, v first: norm weight, cos and sin of this position
                const float *nw = g < Gq ? op.q_norm : op.k_norm;
                for (int j = 0; j < 4; ++j) wv[j] = nw[lane + 32 * j];
                for (int j = 0; j < 2; ++j) {
                    cs[j] = cos_t[(size_t)pos * 64 + lane + 32 * j];
                    sn[j] = sin_t[(size_t)pos * 64 + lane + 32 * j];
                }
                uint32_t raw[4];
                vs_wait4(c, src + lane, src + lane + 32, src + lane + 64, src + lane + 96, raw);
                for (int j = 0; j < 4; ++j) xv[j] = __uint_as_float(raw[j]);
            }
            if (g <= Gq) norm_rope_regs(xv, wv, cs, sn, op.eps, y);
            if (g < Gq) {
                for (int j = 0; j < 4; ++j) qs[g * QS_HEAD + ((lane + 32 * j) >> 4) * QS_SEG + ((lane + 32 * j) & 15)] = y[j];
            } else {
                const size_t grow = ((size_t)pos * kv_heads + kh) * RB;
                if (g == Gq) put_row<KV>(op.kc + grow, kt + (nkeys - 1) * RS, y, lane);
                else put_row<KV>(op.vc + grow, vt + (nkeys - 1) * RS, xv, lane);
            }
        }
        TRACE(1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // K of this chunk
        __syncthreads();
        TRACE(2);
        {   // scores: KPW keys per warp, LPK lanes share a key
            const uint32_t key = warp * KPW + lane / LPK;
            const int d0 = (lane % LPK) * DPL;
            float kv[DPL];
            const uint8_t *row = kt + min(key, nkeys - 1) * RS;
#pragma unroll
            for (int d = 0; d < DPL; d += 8) tile_load8<KV>(row, d0 + d, kv + d);
#pragma unroll 1
            for (uint32_t g0 = 0; g0 < Gq; g0 += 4) {  // four heads side by side: four independent chains (qs has eight head slots)
                float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int d = 0; d < DPL; d += 4) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) {
                        const float4 qa = *reinterpret_cast<const float4 *>(qs + (g0 + gg) * QS_HEAD + (d0 >> 4) * QS_SEG + ((d0 + d) & 15));
                        a[gg] = fmaf(qa.x, kv[d], a[gg]); a[gg] = fmaf(qa.y, kv[d + 1], a[gg]);
                        a[gg] = fmaf(qa.z, kv[d + 2], a[gg]); a[gg] = fmaf(qa.w, kv[d + 3], a[gg]);
                    }
                }
                for (int o = LPK / 2; o > 0; o >>= 1) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg) a[gg] += __shfl_xor_sync(0xffffffffu, a[gg], o);
                }
                if (lane % LPK == 0) {
#pragma unroll
                    for (int gg = 0; gg < 4; ++gg)
                        if (g0 + gg < Gq) ps[key * 8 + g0 + gg] = key < nkeys ? a[gg] * attn_scale : -INFINITY;
                }
            }
        }
        __syncthreads();
        load_tile(kt, op.kc, ch + 1);
        TRACE(3);
        if ((uint32_t)warp < Gq) {  // softmax numerators of this chunk against the running maximum, head = warp; ps is [key][8 heads]
            const uint32_t g = warp;
            float v0 = ps[lane * 8 + g], v1 = C == 64 ? ps[(lane + 32) * 8 + g] : -INFINITY;
            float m = fmaxf(v0, v1);
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float m_old = red[16 + g], m_new = fmaxf(m_old, m);
            v0 = expf(v0 - m_new);
            v1 = C == 64 ? expf(v1 - m_new) : 0.0f;
            ps[lane * 8 + g] = v0;
            if (C == 64) ps[(lane + 32) * 8 + g] = v1;
            float l = v0 + v1;
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            if (lane == 0) {
                const float keep = m_old == -INFINITY ? 0.0f : expf(m_old - m_new);  // what the earlier chunks still weigh
                red[32 + g] = keep;
                red[24 + g] = red[24 + g] * keep + l;
                red[16 + g] = m_new;
            }
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // V of this chunk (K of the next one may still be on its way)
        __syncthreads();
        TRACE(4);
        {   // P V. Warp w owns output elements 8w .. 8w + 7 of every head; its lanes are 4 element pairs x 8 key classes
            // (keys ks, ks + 8, ..): a value pair is read once for all heads, the key's probabilities come as one
            // broadcast vector, and no two lanes of a load share a bank. The key classes meet at the end of the item.
            const float *pt = ps;
            const int d = warp * 8 + 2 * (lane & 3);
            float acc[8][2];
#pragma unroll
            for (int g = 0; g < 8; ++g) acc[g][0] = acc[g][1] = 0.0f;
#pragma unroll 2
            for (uint32_t j = lane >> 2; j < nkeys; j += 8) {
                const float2 v = tile_at2<KV>(vt + j * RS, d);
                const float4 p0 = *reinterpret_cast<const float4 *>(pt + j * 8);
                acc[0][0] = fmaf(p0.x, v.x, acc[0][0]); acc[0][1] = fmaf(p0.x, v.y, acc[0][1]);
                acc[1][0] = fmaf(p0.y, v.x, acc[1][0]); acc[1][1] = fmaf(p0.y, v.y, acc[1][1]);
                acc[2][0] = fmaf(p0.z, v.x, acc[2][0]); acc[2][1] = fmaf(p0.z, v.y, acc[2][1]);
                acc[3][0] = fmaf(p0.w, v.x, acc[3][0]); acc[3][1] = fmaf(p0.w, v.y, acc[3][1]);
                if (Gq > 4) {
                    const float4 p1 = *reinterpret_cast<const float4 *>(pt + j * 8 + 4);
                    acc[4][0] = fmaf(p1.x, v.x, acc[4][0]); acc[4][1] = fmaf(p1.x, v.y, acc[4][1]);
                    acc[5][0] = fmaf(p1.y, v.x, acc[5][0]); acc[5][1] = fmaf(p1.y, v.y, acc[5][1]);
                    acc[6][0] = fmaf(p1.z, v.x, acc[6][0]); acc[6][1] = fmaf(p1.z, v.y, acc[6][1]);
                    acc[7][0] = fmaf(p1.w, v.x, acc[7][0]); acc[7][1] = fmaf(p1.w, v.y, acc[7][1]);
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if ((uint32_t)g < Gq) {  // heads past Gq multiplied whatever lay in their column: never used
                    const float keep = red[32 + g];
                    run[g][0] = run[g][0] * keep + acc[g][0];
                    run[g][1] = run[g][1] * keep + acc[g][1];
                }
            }
        }
        __syncthreads();
        load_tile(vt, op.vc, ch + 1);
        }  // chunks of the group
        {   // the key classes of an output element meet (lanes 4 apart), lanes 0-3 of the warp send the element pair out
            const uint32_t d = warp * 8 + 2 * (lane & 3);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                if ((uint32_t)g < Gq) {
                    float r0 = run[g][0], r1 = run[g][1];
                    for (int o = 4; o < 32; o <<= 1) {
                        r0 += __shfl_xor_sync(0xffffffffu, r0, o);
                        r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                    }
                    if (lane < 4) {
                        const uint32_t head = kh * Gq + g;
                        if (ngroups == 1) {
                            const float l = red[24 + g];
                            uint32_t *o0 = op.out + (size_t)head * 128 + d;
                            vs_store(o0 + c.par_cur, o0 + c.par_alt, __float_as_uint(r0 / l));
                            vs_store(o0 + c.par_cur + 1, o0 + c.par_alt + 1, __float_as_uint(r1 / l));
                        } else {
                            unsigned long long *pp = partials + ((size_t)head * max_chunks + gi) * 130;
                            ll_store(pp + 2 + d, __float_as_uint(r0), epoch);
                            ll_store(pp + 3 + d, __float_as_uint(r1), epoch);
                            if (d == 0) { ll_store(pp, __float_as_uint(red[16 + g]), epoch); ll_store(pp + 1, __float_as_uint(red[24 + g]), epoch); }
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    TRACE(5);
    if (ngroups > 1) {
        // merge the groups of a head; heads go to the blocks at the far end of the grid (the work items start at block 0)
#pragma unroll 1
        for (uint32_t head = c.G - 1 - c.b; head < heads; head += c.G) {
            const unsigned long long *pp = partials + (size_t)head * max_chunks * 130;
            // thread (d, cg) merges the chunks cg, cg + 4, .. of output element d on its own (running maximum), four
            // chunks per round trip with m, l and the accumulator in flight together; the four classes meet below
            const uint32_t d = tid & 127, cg = tid >> 7;
            float M = -INFINITY, L = 0.0f, a = 0.0f;
#pragma unroll 1
            for (uint32_t ch = cg; ch < ngroups; ch += 16) {
                uint32_t cc[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) cc[j] = min(ch + 4 * j, ngroups - 1);
                unsigned long long w[12];
                for (uint32_t it = 0;; ++it) {
                    uint32_t bad = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const unsigned long long *q = pp + (size_t)cc[j] * 130;
                        w[3 * j] = ll_load(q);
                        w[3 * j + 1] = ll_load(q + 1);
                        w[3 * j + 2] = ll_load(q + 2 + d);
                    }
#pragma unroll
                    for (int j = 0; j < 12; ++j) bad |= (uint32_t)(w[j] >> 32) ^ epoch;
                    if (bad == 0 || *c.s_abort) break;
                    if (it >= POLL_LIMIT) {
                        give_up(c, 3);
                        break;
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (ch + 4 * j < ngroups) {
                        const float mc = __uint_as_float((uint32_t)w[3 * j]), lc = __uint_as_float((uint32_t)w[3 * j + 1]);
                        const float ac = __uint_as_float((uint32_t)w[3 * j + 2]);
                        const float Mn = fmaxf(M, mc), so = expf(M - Mn), sn = expf(mc - Mn);  // M = -inf at first: so = 0
                        L = L * so + lc * sn;
                        a = a * so + ac * sn;
                        M = Mn;
                    }
                }
            }
            // classes with no chunk keep M = -inf, L = a = 0
            qs[cg * 128 + d] = a;
            if (d == 0) { qs[512 + cg] = L; qs[516 + cg] = M; }
            __syncthreads();
            if (tid < 128) {
                const float Mt = fmaxf(fmaxf(qs[516], qs[517]), fmaxf(qs[518], qs[519]));
                float A = 0.0f, Lt = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float wj = qs[516 + j] == -INFINITY ? 0.0f : expf(qs[516 + j] - Mt);
                    A = fmaf(qs[j * 128 + d], wj, A);
                    Lt = fmaf(qs[512 + j], wj, Lt);
                }
                vs_store(op.out + c.par_cur + (size_t)head * 128 + d, op.out + c.par_alt + (size_t)head * 128 + d, __float_as_uint(A / Lt));
            }
            __syncthreads();
        }
    }
}

template <int KV>
__global__ void __maxnreg__(128) decode_token_kernel(TokParams p) {
    // byte planes of the fixed-point input of the GEMVs (gemv_device.cuh): an f32 cache keeps the f32 accuracy class of
    // the kernel-per-operation path; f16 and q8_0 caches, whose own rounding is orders of magnitude larger, take two
    constexpr int PLANES = KV == BRASA_KV_F32 ? 3 : 2;
    extern __shared__ __align__(128) uint8_t smem[];
    TokCtx c;
    c.ring = smem;
    c.xfb = c.ring + (size_t)p.nslot * SLOT_CAP;
    c.part = reinterpret_cast<float *>(c.xfb + p.xf_bytes);
    c.resid = c.part + p.part_floats;
    c.nwbuf = c.resid + p.resid_floats;                              // norm weight of the current operation
    c.sdesc = reinterpret_cast<uint4 *>(c.nwbuf + p.nw_floats);      // descriptors of the slots this operation refills
    c.full = reinterpret_cast<uint64_t *>(c.sdesc + p.sdesc_n);
    c.done = reinterpret_cast<uint32_t *>(c.full + p.nslot);
    c.red = reinterpret_cast<float *>(c.done + p.nslot);             // [48]
    uint32_t *ops_s = reinterpret_cast<uint32_t *>(c.red + 48);      // [2][OPS_WORDS]: operation, then this block's rows
    c.s_abort = ops_s + 2 * OPS_WORDS;
    c.status = p.status;
    c.trace = p.trace;
    c.trace_op = p.trace_op;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t G = gridDim.x, b = blockIdx.x;
    c.G = G;
    c.b = b;
    c.pos = p.state[0];
    c.seq = p.state[2];
    c.par_cur = (c.seq & 1) * p.par_words;
    c.par_alt = p.par_words - c.par_cur;
    c.token = p.ids[0];
    c.nslot = p.nslot;
    const uint32_t slot_lo = p.slot_begin[b];
    c.my_slots = p.slot_begin[b + 1] - slot_lo;
    c.myslots = reinterpret_cast<const uint4 *>(p.slots + slot_lo);
    c.h0 = p.hidden * b / G;  // this block's rows of a hidden-size vector
    c.hn = p.hidden * (b + 1) / G - c.h0;

    // operation oi and this block's row counts for it -> ops_s[oi & 1]
    // (by the last threads of the block: the first ones are the busiest in the input phase)
    auto fetch_op = [&](uint32_t oi) {
        const int t = TK_THREADS - 1 - tid;
        if (t < (int)OP_WORDS) ops_s[(oi & 1) * OPS_WORDS + t] = reinterpret_cast<const uint32_t *>(p.ops + oi)[t];
        else if (t < (int)OPS_WORDS) ops_s[(oi & 1) * OPS_WORDS + t] = reinterpret_cast<const uint32_t *>(p.block_ops + (size_t)oi * G + b)[t - OP_WORDS];
    };
    if (tid == 0) {
        for (uint32_t s = 0; s < p.nslot; ++s) {
            mbar_init(&c.full[s], 1);
            c.done[s] = 0;
        }
        *c.s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fetch_op(0);
    __syncthreads();
    {   // the first operation's norm weight (later ones are staged one operation ahead)
        const TokOp &op0 = *reinterpret_cast<const TokOp *>(ops_s);
        if (op0.normw)
            for (uint32_t i = tid; i < op0.cols / 4; i += TK_THREADS) cp_async16(c.nwbuf + 4 * i, op0.normw + 4 * i);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }
    if (tid == 0) {
        uint32_t k = 0;
        for (; k < c.my_slots && k < p.nslot; ++k) issue_slot(c, c.myslots[k], k);
    }

    // This warp's slots are the list entries kk = sub, sub + 2, ..: warps 0-7 take the even ones, warps 8-15 the odd
    // ones, and with an even ring a ring slot always serves the same eight warps, which all wait for every use of it.
    WarpRing wr{(uint32_t)warp >> 3, (uint32_t)warp >> 3, 0u};
    uint32_t gslot = 0;  // list index of the current operation's first slot

#pragma unroll 1
    for (uint32_t oi = 0; oi < p.nops; ++oi) {
        const TokOp &op = *reinterpret_cast<const TokOp *>(ops_s + (oi & 1) * OPS_WORDS);
        const uint32_t *bo = ops_s + (oi & 1) * OPS_WORDS + OP_WORDS;  // r0, rows of segments 0 and 1 (16 bits each), rows of segment 2
        if (oi + 1 < p.nops) fetch_op(oi + 1);
        const uint32_t epoch = c.seq * EPOCH_SPAN + oi + 1;

        c.oi = oi;
        TRACE(0);
        TRACEB(0);
        if (op.next_normw) {  // the next operation's norm weight, copied while this one runs (the idle end of the block first)
            for (uint32_t i = TK_THREADS - 1 - tid; i < op.next_cols / 4; i += TK_THREADS) cp_async16(c.nwbuf + 4 * i, op.next_normw + 4 * i);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        if (op.type == OP_GEMV) {
            const uint32_t lRPS = 4 - op.log2S, RPS = 1u << lRPS;
            const uint32_t total_slots = (((bo[1] & 0xffffu) + RPS - 1) >> lRPS) + (((bo[1] >> 16) + RPS - 1) >> lRPS) + ((bo[2] + RPS - 1) >> lRPS);
            // the descriptors this operation's refills and L2 requests will need, fetched by the threads that poll least
            for (uint32_t i = TK_THREADS - 1 - tid; i < total_slots; i += TK_THREADS) {
                const uint32_t k = gslot + p.nslot + i;
                c.sdesc[i] = k < c.my_slots ? c.myslots[k] : make_uint4(0, 0, 0, 0);
            }
            TRACE(1);
            float ssq = gemv_input<PLANES>(c, op, p.embed, p.vocab);
            TRACE(3);
            TRACEB(1);
            for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) c.red[warp] = ssq;
            __syncthreads();
            TRACE(4);
            if (warp == TK_WARPS - 1) {  // 1 / rms of the whole input from the warps' sums, parked for the epilogue
                float tot = c.red[lane & (TK_WARPS - 1)];
                for (int o = TK_WARPS / 2; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
                if (lane == 0) c.red[47] = op.scaled ? 1.0f / sqrtf(tot / (float)op.cols + op.eps) : 1.0f;
            }
            if (op.qtype == BRASA_Q4_0) {
                if (op.fast && op.nact == 5) wr = gemv_rows<BRASA_Q4_0, PLANES, 5>(c, op, bo, gslot, wr);
                else if (op.fast && op.nact == 4) wr = gemv_rows<BRASA_Q4_0, PLANES, 4>(c, op, bo, gslot, wr);
                else wr = gemv_rows<BRASA_Q4_0, PLANES, 0>(c, op, bo, gslot, wr);
            } else {
                if (op.fast && op.nact == 5) wr = gemv_rows<BRASA_Q6_0, PLANES, 5>(c, op, bo, gslot, wr);
                else wr = gemv_rows<BRASA_Q6_0, PLANES, 0>(c, op, bo, gslot, wr);
            }
            TRACE(7);
            TRACEB(2);
            gslot += total_slots;
            __syncthreads();
            TRACE(8);
            gemv_epilogue(c, op, bo, c.red[47], epoch, p.logits, p.cand, p);
        } else {
            attention_op<KV>(c, op, oi, epoch, p.heads, p.kv_heads, p.max_chunks, p.cos_t, p.sin_t, p.partials, p.attn_scale);
        }
        TRACE(11);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        TRACE(12);
        TRACEB(3);
    }

    // ---- greedy choice and the step's bookkeeping: block 0 gathers every block's best logit ----
    if (b == 0) {
        const uint32_t epoch = c.seq * EPOCH_SPAN + p.nops;  // of the lm_head, the last operation
        Best bst{-INFINITY, 0xffffffffu};
#pragma unroll 1
        for (uint32_t i = tid; i < G; i += TK_THREADS) {
            uint32_t raw[4];
            ll_wait4(c, p.cand + 2 * i, p.cand + 2 * i + 1, p.cand + 2 * i, p.cand + 2 * i + 1, epoch, raw);
            bst = better(bst, Best{__uint_as_float(raw[0]), raw[1]});
        }
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, bst.v, o), __shfl_xor_sync(0xffffffffu, bst.i, o)};
            bst = better(bst, other);
        }
        if (lane == 0) { c.red[16 + warp] = bst.v; c.red[32 + warp] = __uint_as_float(bst.i); }
        __syncthreads();
        if (tid == 0) {
#pragma unroll 1
            for (int w = 1; w < TK_WARPS; ++w) bst = better(bst, Best{c.red[16 + w], __float_as_uint(c.red[32 + w])});
            if (p.tp_world > 1) {
                // this rank's best (logit, vocabulary row) to every rank, then the best of all: largest logit, lowest row
                // among equals (NaN never wins: it never became a candidate)
                const size_t abase = 2 * (size_t)p.tp_world * p.tp_stride + (size_t)(c.seq & 1) * p.tp_world * 2;
                const uint32_t mine = bst.i == 0xffffffffu ? 0xffffffffu : bst.i + p.tp_row0;
                for (uint32_t q = 0; q < p.tp_world; ++q) {
                    xg_store(p.tp_peer[q] + abase + 2 * p.tp_rank, __float_as_uint(bst.v), epoch);
                    xg_store(p.tp_peer[q] + abase + 2 * p.tp_rank + 1, mine, epoch);
                }
                Best all{-INFINITY, 0xffffffffu};
                for (uint32_t q = 0; q < p.tp_world; ++q) {
                    const unsigned long long *src = p.tp_peer[p.tp_rank] + abase + 2 * q;
                    unsigned long long w0 = 0, w1 = 0;
                    for (uint32_t it = 0;; ++it) {
                        w0 = xg_load(src);
                        w1 = xg_load(src + 1);
                        if (((uint32_t)(w0 >> 32) == epoch && (uint32_t)(w1 >> 32) == epoch) || *c.s_abort) break;
                        if (it >= p.tp_poll_limit) {
                            give_up(c, 6);
                            break;
                        }
                    }
                    if ((uint32_t)(w0 >> 32) == epoch && (uint32_t)(w1 >> 32) == epoch)
                        all = better(all, Best{__uint_as_float((uint32_t)w0), (uint32_t)w1});
                }
                bst = all;
            }
            const uint32_t tok = (bst.v == -INFINITY || bst.i == 0xffffffffu) ? 0u : bst.i;
            *p.next_id = tok;
            p.ids[0] = tok;
            const uint32_t n = p.state[1];
            if (n < p.out_cap) p.out_ids[n] = tok;
            p.state[1] = n + 1;
            p.state[0] = c.pos + 1;
            p.state[2] = c.seq + 1;
        }
    }
}

uint32_t attn_chunk(int32_t kv) { return kv == BRASA_KV_F32 ? 32u : 64u; }
uint32_t attn_row_stride(int32_t kv) { return kv == BRASA_KV_F32 ? 528u : (kv == BRASA_KV_F16 ? 272u : 144u); }

// Column slices and active half blocks per lane for a GEMV of this width; false when the kernel does not take it.
bool gemv_shape(int qtype, uint32_t cols, uint32_t *S_out, uint32_t *nact_out) {
    if (cols == 0 || cols % 256 != 0) return false;
    const uint32_t nhb = cols / 16, row_bytes = tiled_row_bytes(qtype, cols);
    for (uint32_t S = 1; S <= 8; S *= 2) {
        uint32_t N = (nhb + 32 * S - 1) / (32 * S);
        uint32_t RPS = TK_WARPS / S * R / 2;
        if (N <= NMAX && (uint64_t)RPS * row_bytes <= SLOT_CAP) {
            *S_out = S;
            *nact_out = N;
            return true;
        }
    }
    return false;
}

}  // namespace

struct brasa_token_program {
    brasa_ctx *ctx = nullptr;
    TokParams params{};
    size_t smem = 0;
    int32_t kv = 0;
    uint32_t grid = 0;
    std::vector<void *> device;  // allocations owned by the program
    void *vectors = nullptr;     // both copies of the activation vectors
    size_t vector_bytes = 0;
    uint32_t timeouts_seen = 0;  // the context's count of abandoned waits when the vectors were last known clean
};

bool brasa_token_program_supported(brasa_ctx *ctx, const brasa_token_model &m) {
    if (m.head_dim != 128 || m.kv_heads == 0 || m.heads % m.kv_heads != 0 || m.heads / m.kv_heads > 8) return false;
    if (m.layers.empty() || m.layers.size() * 5 + 3 >= EPOCH_SPAN) return false;
    if (m.embed.layout != BRASA_LAYOUT_TILED || m.embed.qtype != BRASA_Q6_0 || m.embed.cols != m.hidden) return false;
    if (m.head.layout != BRASA_LAYOUT_TILED || (m.head.qtype != BRASA_Q4_0 && m.head.qtype != BRASA_Q6_0)) return false;
    uint32_t S, n;
    if (!gemv_shape(m.head.qtype, m.hidden, &S, &n) || !gemv_shape(BRASA_Q4_0, m.hidden, &S, &n) ||
        !gemv_shape(BRASA_Q4_0, m.heads * 128, &S, &n) || !gemv_shape(BRASA_Q4_0, m.ffn, &S, &n))
        return false;
    for (const brasa_token_layer &l : m.layers)
        for (const brasa_qmatrix *w : {&l.wq, &l.wk, &l.wv, &l.wo, &l.gate, &l.up, &l.down})
            if (w->layout != BRASA_LAYOUT_TILED || w->qtype != BRASA_Q4_0) return false;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device) != cudaSuccess || !coop) return false;
    return true;
}

void brasa_token_program_free(brasa_token_program *p) {
    if (!p) return;
    for (void *d : p->device) cudaFree(d);
    delete p;
}

int32_t brasa_token_program_create(brasa_ctx *ctx, const brasa_token_model &m, brasa_token_program **out) {
    BRASA_REQUIRE(ctx, out && brasa_token_program_supported(ctx, m), "token program: model shape not supported");
    std::unique_ptr<brasa_token_program, void (*)(brasa_token_program *)> prog(new brasa_token_program, brasa_token_program_free);
    prog->ctx = ctx;
    prog->kv = m.kv;
    const uint32_t G = (uint32_t)ctx->sm_count;
    prog->grid = G;
    const uint32_t H = m.hidden, QD = m.heads * 128, KD = m.kv_heads * 128, F = m.ffn;
    const uint32_t C = attn_chunk(m.kv), max_chunks = (m.cache_positions + C - 1) / C;

    auto dev_alloc = [&](size_t bytes, void **ptr) -> int32_t {
        BRASA_CUDA(ctx, cudaMalloc(ptr, bytes));
        prog->device.push_back(*ptr);
        return brasa_check_cuda(ctx, cudaMemset(*ptr, 0, bytes), "cudaMemset");
    };
    // attention partials and argmax candidates as {value, epoch} words
    unsigned long long *partials, *cand;
    const size_t ll_words = (size_t)m.heads * max_chunks * 130 + 2 * G;
    void *ll_base;
    BRASA_TRY(dev_alloc(ll_words * 8, &ll_base));
    partials = (unsigned long long *)ll_base;
    cand = partials + (size_t)m.heads * max_chunks * 130;
    // every operation's output vector: two copies of par_words 4-byte words, all empty at first
    const size_t per_layer = (size_t)(QD + 2 * KD) + QD + H + F + H;
    const size_t par_words = (per_layer * m.layers.size() + 31) / 32 * 32;
    BRASA_REQUIRE(ctx, par_words < (1u << 31), "token program: activation vectors too large");
    void *vs_base;
    BRASA_TRY(dev_alloc(par_words * 8, &vs_base));
    BRASA_CUDA(ctx, cudaMemset(vs_base, 0xff, par_words * 8));
    prog->vectors = vs_base;
    prog->vector_bytes = par_words * 8;
    prog->timeouts_seen = ctx->timeouts;
    uint32_t *vs_next = (uint32_t *)vs_base;
    auto vec_alloc = [&](size_t n) { uint32_t *r = vs_next; vs_next += n; return r; };

    // ---- the operations ----
    std::vector<TokOp> ops;
    auto gemv_op = [&](uint32_t nmat, const brasa_qmatrix *w, uint32_t epilogue, bool scaled, const float *normw, int in_op, bool save_resid) {
        TokOp o{};
        o.type = OP_GEMV;
        o.qtype = (uint32_t)w[0].qtype;
        o.cols = w[0].cols;
        o.nmat = nmat;
        o.total_rows = 0;
        for (uint32_t i = 0; i < nmat; ++i) {
            o.rows[i] = w[i].rows;
            o.w[i] = arg_ptr(w[i].data);
            o.total_rows += w[i].rows;
        }
        if (epilogue == EPI_SWIGLU) o.total_rows = w[0].rows;
        o.epilogue = epilogue;
        o.scaled = scaled ? 1 : 0;
        uint32_t S = 1;
        gemv_shape(w[0].qtype, o.cols, &S, &o.nact);
        for (o.log2S = 0; (1u << o.log2S) < S; ++o.log2S) {}
        o.fast = o.nact >= 2 ? ((S * o.nact - 2) * 32 + 31 < o.cols / 16) : 1;
        o.in_kind = in_op < 0 ? IN_EMBED : IN_LL;
        o.in_op = in_op < 0 ? 0 : (uint32_t)in_op;
        o.save_resid = save_resid ? 1 : 0;
        o.eps = m.eps;
        o.normw = normw;
        o.in = in_op < 0 ? nullptr : ops[in_op].out;
        o.out = epilogue == EPI_LOGITS ? nullptr : vec_alloc(o.total_rows);
        ops.push_back(o);
        return (int)ops.size() - 1;
    };
    int x_op = -1;  // operation that produced the current residual stream (-1: the embedding row)
    const bool tp_on = m.tp.world > 1;
    BRASA_REQUIRE(ctx, !tp_on || (m.tp.world <= BRASA_TP_MAX_RANKS && m.tp.rank < m.tp.world && m.tp.stride >= H),
                  "token program: the exchange area is smaller than the hidden size");
    uint32_t nxchg = 0;
    for (const brasa_token_layer &l : m.layers) {
        brasa_qmatrix wqkv[3] = {l.wq, l.wk, l.wv};
        BRASA_REQUIRE(ctx, l.wq.rows == QD && l.wk.rows == KD && l.wv.rows == KD && l.wq.cols == H && l.wo.rows == H && l.wo.cols == QD &&
                               l.gate.rows == F && l.up.rows == F && l.gate.cols == H && l.down.rows == H && l.down.cols == F,
                      "token program: unexpected matrix shape");
        int qkv_op = gemv_op(3, wqkv, EPI_SCALE, true, l.attn_norm, x_op, true);
        TokOp a{};
        a.type = OP_ATTN;
        a.in_op = (uint32_t)qkv_op;
        a.eps = m.eps;
        a.in = ops[qkv_op].out;
        a.out = vec_alloc(QD);
        a.q_norm = l.q_norm;
        a.k_norm = l.k_norm;
        a.kc = l.kc;
        a.vc = l.vc;
        ops.push_back(a);
        int attn_op = (int)ops.size() - 1;
        int o_op = gemv_op(1, &l.wo, EPI_RESID, false, nullptr, attn_op, false);
        if (tp_on) ops[o_op].xchg = ++nxchg;
        brasa_qmatrix wgu[2] = {l.gate, l.up};
        int gu_op = gemv_op(2, wgu, EPI_SWIGLU, true, l.ffn_norm, o_op, true);
        x_op = gemv_op(1, &l.down, EPI_RESID, false, nullptr, gu_op, false);
        if (tp_on) ops[x_op].xchg = ++nxchg;
    }
    BRASA_REQUIRE(ctx, (tp_on ? m.head.rows + m.head_row0 <= m.vocab : m.head.rows == m.vocab) && m.head.cols == H, "token program: unexpected lm_head shape");
    gemv_op(1, &m.head, EPI_LOGITS, true, m.final_norm, x_op, false);
    BRASA_REQUIRE(ctx, (size_t)(vs_next - (uint32_t *)vs_base) <= par_words, "token program: activation vectors overran their area");
    BRASA_REQUIRE(ctx, ops.size() + 2 < EPOCH_SPAN, "token program: too many operations");
    uint32_t nw_floats = 0;
    for (size_t i = 0; i < ops.size(); ++i) {
        if (ops[i].normw) nw_floats = std::max(nw_floats, ops[i].cols);
        if (i + 1 < ops.size() && ops[i + 1].normw) {
            BRASA_REQUIRE(ctx, !ops[i].normw, "token program: two operations in a row with a norm weight");
            ops[i].next_normw = ops[i + 1].normw;
            ops[i].next_cols = ops[i + 1].cols;
        }
    }

    // ---- every block's slot list, in the order the kernel consumes it, and its rows of every operation ----
    std::vector<SlotDesc> slots;
    std::vector<uint32_t> slot_begin(G + 1, 0);
    std::vector<uint4> block_ops(ops.size() * G, make_uint4(0, 0, 0, 0));
    uint32_t part_floats = 0, max_cols = 0, max_op_slots = 0;
    for (uint32_t b = 0; b < G; ++b) {
        slot_begin[b] = (uint32_t)slots.size();
        for (size_t oi = 0; oi < ops.size(); ++oi) {
            const TokOp &o = ops[oi];
            if (o.type != OP_GEMV) continue;
            const bool swiglu = o.epilogue == EPI_SWIGLU;
            uint32_t r0, r1, first[3], nrows[3];
            block_rows(o.total_rows, o.nmat, o.rows, swiglu, b, G, r0, r1, first, nrows);
            BRASA_REQUIRE(ctx, nrows[0] < 65536 && nrows[1] < 65536, "token program: too many rows per block");
            block_ops[oi * G + b] = make_uint4(r0, nrows[0] | (nrows[1] << 16), nrows[2], 0);
            const uint32_t S = 1u << o.log2S, RPS = TK_WARPS / S * R / 2, row_bytes = tiled_row_bytes((int)o.qtype, o.cols);
            uint32_t items = 0, op_slots = 0;
            for (int i = 0; i < 3; ++i) {
                for (uint32_t f = 0; f < nrows[i]; f += RPS) {
                    uint32_t n = std::min(RPS, nrows[i] - f);
                    slots.push_back(SlotDesc{o.w[i] + (size_t)(first[i] + f) * row_bytes, n * row_bytes, 0});
                    ++op_slots;
                }
                items += nrows[i];
            }
            part_floats = std::max(part_floats, items * S);
            max_cols = std::max(max_cols, o.cols);
            max_op_slots = std::max(max_op_slots, op_slots);
        }
    }
    slot_begin[G] = (uint32_t)slots.size();

    TokParams &p = prog->params;
    void *d_ops, *d_slots, *d_begin, *d_bops;
    BRASA_TRY(dev_alloc(block_ops.size() * sizeof(uint4), &d_bops));
    BRASA_CUDA(ctx, cudaMemcpy(d_bops, block_ops.data(), block_ops.size() * sizeof(uint4), cudaMemcpyHostToDevice));
    BRASA_TRY(dev_alloc(ops.size() * sizeof(TokOp), &d_ops));
    BRASA_TRY(dev_alloc(std::max<size_t>(slots.size(), 1) * sizeof(SlotDesc), &d_slots));
    BRASA_TRY(dev_alloc(slot_begin.size() * 4, &d_begin));
    BRASA_CUDA(ctx, cudaMemcpy(d_ops, ops.data(), ops.size() * sizeof(TokOp), cudaMemcpyHostToDevice));
    BRASA_CUDA(ctx, cudaMemcpy(d_slots, slots.data(), slots.size() * sizeof(SlotDesc), cudaMemcpyHostToDevice));
    BRASA_CUDA(ctx, cudaMemcpy(d_begin, slot_begin.data(), slot_begin.size() * 4, cudaMemcpyHostToDevice));
    p.ops = (const TokOp *)d_ops;
    p.nops = (uint32_t)ops.size();
    p.slots = (const SlotDesc *)d_slots;
    p.slot_begin = (const uint32_t *)d_begin;
    p.block_ops = (const uint4 *)d_bops;

    // ---- shared memory ----
    const size_t attn_bytes = (size_t)2 * C * attn_row_stride(m.kv) + (8 * 160 + 8 * C + 2 * max_chunks) * 4;
    p.xf_bytes = (uint32_t)((std::max<size_t>((size_t)max_cols / 16 * 16 * (m.kv == BRASA_KV_F32 ? XRec<3>::CHUNKS : XRec<2>::CHUNKS), attn_bytes) + 127) / 128 * 128);
    p.part_floats = (part_floats + 3) & ~3u;
    p.resid_floats = ((H + G - 1) / G + 4) & ~3u;
    p.sdesc_n = max_op_slots;
    p.nw_floats = (nw_floats + 3) & ~3u;
    const size_t fixed = p.xf_bytes + (size_t)(p.part_floats + p.resid_floats + p.nw_floats) * 4 + (size_t)p.sdesc_n * 16 + 48 * 4 + 2 * OPS_WORDS * 4 + 16;
    BRASA_REQUIRE(ctx, fixed + 2 * (SLOT_CAP + 12) + 1024 <= ctx->smem_optin, "token program: the model's vectors do not fit shared memory");
    uint32_t nslot = (uint32_t)((ctx->smem_optin - 1024 - fixed) / (SLOT_CAP + 12));
    nslot &= ~1u;  // even: a ring slot always serves the same half of the warps
    p.nslot = nslot;
    prog->smem = (size_t)nslot * (SLOT_CAP + 12) + fixed;

    p.state = m.state;
    p.ids = m.ids;
    p.next_id = m.next_id;
    p.out_ids = m.out_ids;
    p.out_cap = m.out_cap;
    p.embed = arg_ptr(m.embed.data);
    p.vocab = m.vocab;
    p.hidden = H;
    p.heads = m.heads;
    p.kv_heads = m.kv_heads;
    p.max_chunks = max_chunks;
    p.cos_t = m.cos_t;
    p.sin_t = m.sin_t;
    p.logits = m.logits;
    p.cand = cand;
    p.par_words = (uint32_t)par_words;
    p.partials = partials;
    p.attn_scale = 1.0f / sqrtf(128.0f);
    p.status = ctx->status;
    p.tp_world = tp_on ? m.tp.world : 1;
    p.tp_rank = tp_on ? m.tp.rank : 0;
    p.tp_row0 = m.head_row0;
    p.tp_stride = m.tp.stride;
    p.tp_poll_limit = m.tp.poll_limit ? m.tp.poll_limit : POLL_LIMIT;
    for (uint32_t r = 0; r < BRASA_TP_MAX_RANKS; ++r) p.tp_peer[r] = tp_on && r < m.tp.world ? m.tp.peer[r] : nullptr;
    p.trace = ctx->gemv_trace;
    {
        const char *env = getenv("BRASA_TRACE_OP");
        p.trace_op = env ? (uint32_t)atoi(env) : 5;
    }

#define SET_ATTR(KVT) BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_token_kernel<KVT>, prog->smem))
    if (m.kv == BRASA_KV_F32) SET_ATTR(BRASA_KV_F32);
    else if (m.kv == BRASA_KV_F16) SET_ATTR(BRASA_KV_F16);
    else SET_ATTR(BRASA_KV_Q8_0);
#undef SET_ATTR
    int per_sm = 0;
    const void *fn = m.kv == BRASA_KV_F32 ? (const void *)decode_token_kernel<BRASA_KV_F32>
                     : m.kv == BRASA_KV_F16 ? (const void *)decode_token_kernel<BRASA_KV_F16> : (const void *)decode_token_kernel<BRASA_KV_Q8_0>;
    BRASA_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, TK_THREADS, prog->smem));
    BRASA_REQUIRE(ctx, per_sm >= 1, "token program: the kernel does not fit an SM");
    *out = prog.release();
    return BRASA_OK;
}

int32_t brasa_token_program_launch(brasa_cmd *cmd, brasa_token_program *prog) {
    brasa_ctx *ctx = cmd->ctx;
    if (prog->timeouts_seen != ctx->timeouts) {
        // a launch that gave up may have left words of either copy unwritten or not emptied: start from all empty
        BRASA_CUDA(ctx, cudaMemsetAsync(prog->vectors, 0xff, prog->vector_bytes, ctx->stream));
        prog->timeouts_seen = ctx->timeouts;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(prog->grid);
    cfg.blockDim = dim3(TK_THREADS);
    cfg.dynamicSmemBytes = prog->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every block resident at once: blocks wait for one another's outputs
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (prog->kv == BRASA_KV_F32) BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, decode_token_kernel<BRASA_KV_F32>, prog->params));
    else if (prog->kv == BRASA_KV_F16) BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, decode_token_kernel<BRASA_KV_F16>, prog->params));
    else BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, decode_token_kernel<BRASA_KV_Q8_0>, prog->params));
    return brasa_post_launch(cmd, "decode_token");
}
