// Batched decode over a paged KV pool: many independent sequences of one model decoded together, one token each per
// step (the serving case the reference handles one process at a time: crates/daemon/src/engine.rs:1-3 keeps a single
// model thread, crates/runtime/src/session.rs:230-237 reuses one cached prefix).
//
// KV lives in pages of 16 positions, [layer][page][16][kv head][128] in the model's cache type; a sequence is a list
// of pages. A prefix shared by every sequence is computed once and its pages are attached to each sequence, the
// reference's prefix reuse generalised from one cached sequence to many. Prefill keeps using the model's contiguous
// cache (the prefix stays resident there at positions [0, P), a sequence's own tokens are prefilled after it) and the
// new rows are then copied into that sequence's pages, so the prefill kernels need no page tables. A decode step runs
// the layer sequence of qwen3.rs:763-831 for `n` tokens at once: projections as GEMMs (f16 inputs above 8 sequences,
// like a prefill chunk), QK-norm + RoPE + page store with one position per sequence, paged split-K attention, and the
// batched sampler with one PCG32 stream per sequence.
#include <memory>
#include <unordered_map>

#include "attn_device.cuh"
#include "model_internal.h"

using namespace brasa_dev;

int32_t brasa_sample_batched_launch(brasa_cmd *cmd, const float *logits, uint32_t n, uint32_t count, float temperature, uint32_t top_k, float top_p,
                                    unsigned long long *rng, float *scratch, uint32_t *out);

namespace {

constexpr uint32_t PAGE = 16;
constexpr int D = 128, TS = D + 4;

struct Paged {
    const uint8_t *pool;     // this layer's pages
    const int32_t *table;    // [seq][max_pages]
    uint32_t max_pages, hkv;
};

template <int KV>
__device__ __forceinline__ const uint8_t *paged_row(const Paged &p, uint32_t seq, uint32_t key, uint32_t kh) {
    const int32_t page = p.table[(size_t)seq * p.max_pages + key / PAGE];
    return p.pool + (((size_t)page * PAGE + key % PAGE) * p.hkv + kh) * KvRow<KV>::BYTES;
}

// rows [key0, key0 + nkeys) of one kv head of one sequence -> ts[key][d] as f32
template <int KV>
__device__ __forceinline__ void load_tile_paged(const Paged &p, uint32_t seq, float *ts, uint32_t key0, uint32_t nkeys, uint32_t kh) {
    for (uint32_t i = threadIdx.x; i < nkeys * (D / 8); i += blockDim.x) {
        const uint32_t key = i / (D / 8), v8 = i % (D / 8);
        float v[8];
        tile_load8<KV>(paged_row<KV>(p, seq, key0 + key, kh), (int)(v8 * 8), v);
        float *o = ts + key * TS + v8 * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[j];
    }
}

// One block per (128-key chunk, kv head, sequence); partial layout per (sequence, head, chunk): m, l, acc[128]
// (the layout of crates/kernels/src/lib.rs:1335 with a sequence dimension in front).
template <int KV>
__global__ void __launch_bounds__(128) decode_partial_paged_kernel(const float *q, Paged kp, Paged vp, const uint32_t *lens, float *partials, uint32_t hq,
                                                                   uint32_t max_chunks, float scale) {
    extern __shared__ __align__(16) float sm[];
    float *ts = sm, *qs = ts + 128 * TS, *ps = qs + 8 * D, *red = ps + 8 * 128;
    const uint32_t chunk = blockIdx.x, kh = blockIdx.y, seq = blockIdx.z, hkv = kp.hkv, G = hq / hkv;
    const uint32_t lk = lens[seq] + 1;  // the new token's row is already in its page
    if (chunk * 128 >= lk) return;
    const uint32_t key0 = chunk * 128, nkeys = min(128u, lk - key0);
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (uint32_t i = t; i < G * D; i += 128) qs[i] = q[((size_t)seq * hq + kh * G) * D + i];
    load_tile_paged<KV>(kp, seq, ts, key0, nkeys, kh);
    __syncthreads();
    for (uint32_t g = 0; g < G; ++g) {
        float s = -INFINITY;
        if ((uint32_t)t < nkeys) {
            const float4 *kr = reinterpret_cast<const float4 *>(ts + t * TS), *qr = reinterpret_cast<const float4 *>(qs + g * D);
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
    load_tile_paged<KV>(vp, seq, ts, key0, nkeys, kh);  // K is no longer needed
    for (uint32_t g = 0; g < G; ++g) {
        float s = ps[g * 128 + t], m = s;
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
            float *out = partials + (((size_t)seq * hq + kh * G + g) * max_chunks + chunk) * 130;
            out[0] = m;
            out[1] = (red[4] + red[5]) + (red[6] + red[7]);
        }
    }
    __syncthreads();
    for (uint32_t g = 0; g < G; ++g) {
        float acc = 0.0f;
        const float *pg = ps + g * 128;
        for (uint32_t j = 0; j < nkeys; ++j) acc = fmaf(pg[j], ts[j * TS + t], acc);
        partials[(((size_t)seq * hq + kh * G + g) * max_chunks + chunk) * 130 + 2 + t] = acc;
    }
}


// ---- the same partial for an f16 pool on the tensor cores ----------------------------------------------------------
// With many sequences the step reads gigabytes of KV and the scalar kernel above is bound by its FMA and shared-memory
// traffic, not by HBM. Here a block (4 warps) takes the same (128-key chunk, kv head, sequence): K and V rows arrive
// with cp.async as raw f16 (rows of 256 bytes, 16-byte pieces XOR-swizzled by the row), warp w owns keys [32 w, 32 w + 32):
//   S = Q K^T with mma.sync m16n8k16 (rows = the GQA group's heads, padded to 16; Q enters as two f16 terms hi + lo, so the
//   scores keep f32 accuracy: K is f16 in the cache, nothing else is rounded), block-wide row maximum and sum through
//   shared memory, P = exp(S - m) again as hi + lo f16 terms, O = P V with V fragments from ldmatrix.trans, and the four
//   warps' O added in shared memory. Output: the partial layout of the kernel above, so the reduction is shared.
__device__ __forceinline__ void cp_async16_zfill(void *dst, const void *src, bool valid) {
    const uint32_t bytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// two floats -> packed f16 pair (hi) and the pair of what the rounding dropped (lo)
__device__ __forceinline__ void split_h2(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - back.x, y - back.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}
// byte offset of the 16-byte piece `c` of row `r` in a [128 rows][256 bytes] tile
__device__ __forceinline__ uint32_t piece(uint32_t r, uint32_t c) { return r * 256u + ((c ^ (r & 7u)) << 4); }

constexpr uint32_t MMA_TILE = 128 * 256;  // one K or V tile
constexpr int PAGED_MMA_TILES = 2;       // groups of 16 / G sequences a shared-prefix block serves with one pair of tiles
constexpr size_t MMA_SMEM = 2 * MMA_TILE + (2 * 4 * 16 + 16) * sizeof(float);  // three blocks per SM

__device__ __forceinline__ void mma_f16_full(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MULTI = false: the 16 MMA rows hold the G heads of ONE sequence's group (rows >= G are zero); grid z = sequence, chunk =
// first_chunk + grid x. MULTI = true: chunks that lie wholly inside the prefix every sequence shares: the rows hold the
// groups of 16 / G consecutive sequences (row = local sequence * G + head in group), so the shared K and V tiles are
// fetched and multiplied once per 16 / G sequences; grid z = sequence group; the pages are those of the group's first
// sequence (the prefix pages are the same for all).
template <bool MULTI>
__global__ void __launch_bounds__(128) decode_partial_paged_mma_kernel(const float *q, Paged kp, Paged vp, const uint32_t *lens, float *partials,
                                                                       uint32_t hq, uint32_t max_chunks, float scale, uint32_t first_chunk, uint32_t nseq,
                                                                       uint32_t late_wait) {
    // Launched as a programmatic dependent. late_wait: the kernel before this one is the shared-prefix form of the same step,
    // which has itself waited for the step's K/V rows and whose output this one does not read: the two run side by side,
    // and this one waits for the other only at its end, so that whoever waits for this kernel has waited for both.
    if (!late_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int RH = MULTI ? 2 : 1;  // row halves in use: rows g (and g + 8)
    // MULTI: a block serves PAGED_MMA_TILES groups of 16 / G sequences with the same K and V tiles: all their scores first (K is
    // then done with), then group by group softmax, P V and the four warps' sum in shared memory over the K tile.
    constexpr int RT = MULTI ? PAGED_MMA_TILES : 1;
    extern __shared__ __align__(128) uint8_t smem_b[];
    uint8_t *kt = smem_b, *vt = smem_b + MMA_TILE;
    float *osum = reinterpret_cast<float *>(kt);  // [4 warps][16 rows][128], over the K tile once every warp is done with it
    float *wmax = reinterpret_cast<float *>(smem_b + 2 * MMA_TILE), *wsum = wmax + 4 * 16;  // [4 warps][16 rows] each
    const uint32_t chunk = first_chunk + blockIdx.x, kh = blockIdx.y, hkv = kp.hkv, G = hq / hkv;
    const uint32_t spb = MULTI ? 16 / G : 1, seq00 = blockIdx.z * spb * RT;
    const uint32_t lk = MULTI ? (chunk + 1) * 128 : lens[seq00] + 1;
    if (chunk * 128 >= lk) {
        if (late_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }
    const uint32_t key0 = chunk * 128, nkeys = min(128u, lk - key0);
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5, g = lane >> 2, tq = lane & 3;
    // ---- K then V: 128 rows x 16 pieces each; rows past the end are zero-filled. The chunk's eight page numbers are read
    // first, all at once: a look-up in front of every copy (which the copies' ordering keeps in program order) held a block
    // for thirty-two L2 round trips before its first product ----
    int32_t pg[8];
    {
        const int32_t *trow = kp.table + (size_t)seq00 * kp.max_pages + key0 / PAGE;
#pragma unroll
        for (int j = 0; j < 8; ++j) pg[j] = (uint32_t)(j * PAGE) < nkeys ? trow[j] : trow[0];
    }
    const uint32_t r_lo = t >> 4, pc = t & 15;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const uint32_t r = 8 * k + r_lo;
        const bool ok = r < nkeys;
        const size_t row = ((size_t)(ok ? pg[k >> 1] : pg[0]) * PAGE + (ok ? (r & (PAGE - 1)) : 0u)) * hkv + kh;
        cp_async16_zfill(kt + piece(r, pc), kp.pool + row * KvRow<BRASA_KV_F16>::BYTES + 16 * pc, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const uint32_t r = 8 * k + r_lo;
        const bool ok = r < nkeys;
        const size_t row = ((size_t)(ok ? pg[k >> 1] : pg[0]) * PAGE + (ok ? (r & (PAGE - 1)) : 0u)) * hkv + kh;
        cp_async16_zfill(vt + piece(r, pc), vp.pool + row * KvRow<BRASA_KV_F16>::BYTES + 16 * pc, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    // ---- S[row g (c0, c1) and g + 8 (c2, c3)][keys 32 warp + 8 j + 2 tq, +1], j = 0..3, for every group of sequences ----
    float sc[RT][4][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const uint32_t seq0 = seq00 + rt * spb;
        const uint32_t nrows = seq0 < nseq ? min(spb, nseq - seq0) * G : 0u;  // rows of the MMA that carry a (sequence, head)
        // Q fragments of rows g and g + 8: for k-step ks, a0/a1 = dims 16 ks + 2 tq, +1; a2/a3 = those + 8
        uint32_t qh0[RH][8], qh2[RH][8], ql0[RH][8], ql2[RH][8];
#pragma unroll
        for (int rh = 0; rh < RH; ++rh) {
            const uint32_t r = g + 8 * rh;
            const bool live = r < nrows;
            const float *qrow = q + ((size_t)(seq0 + (live ? r / G : 0)) * hq + kh * G + (live ? r % G : 0)) * D;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                float2 a = make_float2(0.0f, 0.0f), b = a;
                if (live) {
                    a = *reinterpret_cast<const float2 *>(qrow + 16 * ks + 2 * tq);
                    b = *reinterpret_cast<const float2 *>(qrow + 16 * ks + 2 * tq + 8);
                }
                split_h2(a.x, a.y, qh0[rh][ks], ql0[rh][ks]);
                split_h2(b.x, b.y, qh2[rh][ks], ql2[rh][ks]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) sc[rt][j][0] = sc[rt][j][1] = sc[rt][j][2] = sc[rt][j][3] = 0.0f;
        // ldmatrix.x4: lanes 0-7 address rows of tile 0, 8-15 tile 1, 16-23 tile 2, 24-31 tile 3;
        // tiles = (dims 16 ks .. +7), (dims 16 ks + 8 ..), (dims 16 (ks + 1) ..), (dims 16 (ks + 1) + 8 ..) of 8 keys
        const uint32_t lrow = lane & 7, ltile = lane >> 3;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t krow = 32 * warp + 8 * j + lrow;
#pragma unroll
            for (int ks = 0; ks < 8; ks += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + piece(krow, 2 * ks + ltile));
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t h1 = MULTI ? qh0[RH - 1][ks + u] : 0u, h3 = MULTI ? qh2[RH - 1][ks + u] : 0u;
                    const uint32_t l1 = MULTI ? ql0[RH - 1][ks + u] : 0u, l3 = MULTI ? ql2[RH - 1][ks + u] : 0u;
                    mma_f16_full(sc[rt][j], qh0[0][ks + u], h1, qh2[0][ks + u], h3, b[2 * u], b[2 * u + 1]);
                    mma_f16_full(sc[rt][j], ql0[0][ks + u], l1, ql2[0][ks + u], l3, b[2 * u], b[2 * u + 1]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // V (waited for here once; the barriers below publish it)
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const uint32_t seq0 = seq00 + rt * spb;
        const uint32_t nrows = seq0 < nseq ? min(spb, nseq - seq0) * G : 0u;
        if (nrows == 0) break;  // (the same for the whole block)
        // ---- scale, mask, row maxima over the block ----
        float mx[RH], m[RH], l[RH];
#pragma unroll
        for (int rh = 0; rh < RH; ++rh) {
            mx[rh] = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t key = 32 * warp + 8 * j + 2 * tq + e;
                    const float v = key < nkeys ? sc[rt][j][2 * rh + e] * scale : -INFINITY;
                    sc[rt][j][2 * rh + e] = v;
                    mx[rh] = fmaxf(mx[rh], v);
                }
            }
            mx[rh] = fmaxf(mx[rh], __shfl_xor_sync(0xffffffffu, mx[rh], 1));
            mx[rh] = fmaxf(mx[rh], __shfl_xor_sync(0xffffffffu, mx[rh], 2));
            if (tq == 0) wmax[warp * 16 + g + 8 * rh] = mx[rh];
        }
        __syncthreads();  // (also: every warp is done with the K tile, whose place osum takes)
        uint32_t ph[RH][4], pl[RH][4];  // P of n-tile j as packed pairs: A fragment a0/a1 (j even) or a2/a3 (j odd) of k-step j / 2
#pragma unroll
        for (int rh = 0; rh < RH; ++rh) {
            const uint32_t r = g + 8 * rh;
            m[rh] = fmaxf(fmaxf(wmax[r], wmax[16 + r]), fmaxf(wmax[32 + r], wmax[48 + r]));
            l[rh] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float s0 = sc[rt][j][2 * rh], s1 = sc[rt][j][2 * rh + 1];
                const float p0 = s0 == -INFINITY ? 0.0f : expf(s0 - m[rh]), p1 = s1 == -INFINITY ? 0.0f : expf(s1 - m[rh]);
                l[rh] += p0 + p1;
                split_h2(p0, p1, ph[rh][j], pl[rh][j]);
            }
            l[rh] += __shfl_xor_sync(0xffffffffu, l[rh], 1);
            l[rh] += __shfl_xor_sync(0xffffffffu, l[rh], 2);
            if (tq == 0) wsum[warp * 16 + r] = l[rh];
        }
        __syncthreads();
        // ---- O[row][dims 8 n + 2 tq, +1] += P[16 x 32 keys] V[32 keys x 128 dims] ----
        float oc[16][4];
#pragma unroll
        for (int n = 0; n < 16; ++n) oc[n][0] = oc[n][1] = oc[n][2] = oc[n][3] = 0.0f;
        {
            // ldmatrix.x4.trans over V rows (keys): tiles = (keys 0-7, dims 8 n ..), (keys 8-15, dims 8 n ..),
            // (keys 0-7, dims 8 (n + 1) ..), (keys 8-15, dims 8 (n + 1) ..) -> b0, b1 of n-tile n and of n-tile n + 1
            const uint32_t lrow = lane & 7, ltile = lane >> 3;
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                const uint32_t vrow = 32 * warp + 16 * kk + 8 * (ltile & 1) + lrow;
                const uint32_t h1 = MULTI ? ph[RH - 1][2 * kk] : 0u, h3 = MULTI ? ph[RH - 1][2 * kk + 1] : 0u;
                const uint32_t l1 = MULTI ? pl[RH - 1][2 * kk] : 0u, l3 = MULTI ? pl[RH - 1][2 * kk + 1] : 0u;
#pragma unroll
                for (int n = 0; n < 16; n += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vt + piece(vrow, n + (ltile >> 1)));
                    mma_f16_full(oc[n], ph[0][2 * kk], h1, ph[0][2 * kk + 1], h3, b[0], b[1]);
                    mma_f16_full(oc[n], pl[0][2 * kk], l1, pl[0][2 * kk + 1], l3, b[0], b[1]);
                    mma_f16_full(oc[n + 1], ph[0][2 * kk], h1, ph[0][2 * kk + 1], h3, b[2], b[3]);
                    mma_f16_full(oc[n + 1], pl[0][2 * kk], l1, pl[0][2 * kk + 1], l3, b[2], b[3]);
                }
            }
        }
#pragma unroll
        for (int rh = 0; rh < RH; ++rh) {
            const uint32_t r = g + 8 * rh;
            if (r < nrows) {
#pragma unroll
                for (int n = 0; n < 16; ++n)
                    *reinterpret_cast<float2 *>(osum + (warp * 16 + r) * D + 8 * n + 2 * tq) = make_float2(oc[n][2 * rh], oc[n][2 * rh + 1]);
            }
        }
        __syncthreads();
        for (uint32_t r = 0; r < nrows; ++r) {
            const uint32_t seq = seq0 + r / G, h = kh * G + r % G;
            float *out = partials + (((size_t)seq * hq + h) * max_chunks + chunk) * 130;
            out[2 + t] = (osum[(0 * 16 + r) * D + t] + osum[(1 * 16 + r) * D + t]) + (osum[(2 * 16 + r) * D + t] + osum[(3 * 16 + r) * D + t]);
            if (t == 0) {
                out[0] = fmaxf(fmaxf(wmax[r], wmax[16 + r]), fmaxf(wmax[32 + r], wmax[48 + r]));
                out[1] = (wsum[r] + wsum[16 + r]) + (wsum[32 + r] + wsum[48 + r]);
            }
        }
        if (RT > 1) __syncthreads();  // the next group of sequences reuses wmax, wsum and osum
    }
    if (late_wait) asm volatile("griddepcontrol.wait;" ::: "memory");
}

// grid (head, sequence); output f32 or f16 (the input type of the o_proj GEMM)
template <bool HALF_OUT>
__global__ void __launch_bounds__(128) decode_reduce_paged_kernel(const float *partials, const uint32_t *lens, void *o, uint32_t hq, uint32_t max_chunks) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (launched as a programmatic dependent: see brasa_launch_dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t h = blockIdx.x, seq = blockIdx.y, t = threadIdx.x;
    const uint32_t chunks = (lens[seq] + 1 + 127) / 128;
    const float *p = partials + ((size_t)seq * hq + h) * max_chunks * 130;
    float M = -INFINITY;  // (a lane per chunk: one round trip for all the maxima, whatever the number of chunks)
    for (uint32_t c = t & 31; c < chunks; c += 32) M = fmaxf(M, p[c * 130]);
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.0f, acc = 0.0f;
#pragma unroll 8
    for (uint32_t c = 0; c < chunks; ++c) {  // (unrolled: the chunks' loads are independent, only the sums are a chain)
        float w = expf(p[c * 130] - M);
        L = fmaf(p[c * 130 + 1], w, L);
        acc = fmaf(p[c * 130 + 2 + t], w, acc);
    }
    const size_t idx = ((size_t)seq * hq + h) * D + t;
    if (HALF_OUT) reinterpret_cast<__half *>(o)[idx] = __float2half_rn(acc / L);
    else reinterpret_cast<float *>(o)[idx] = acc / L;
}

// Per-head RMSNorm + RoPE of q and k (in place) and the page store of k and v, one token per sequence at that
// sequence's own position (its current length). One warp per row.
template <int KV>
__global__ void __launch_bounds__(128) qk_norm_rope_store_paged_kernel(float *q, float *k, const float *v, const float *q_norm, const float *k_norm,
                                                                       const float *cos_t, const float *sin_t, uint8_t *kpool, uint8_t *vpool,
                                                                       const int32_t *table, uint32_t max_pages, const uint32_t *lens, uint32_t hq,
                                                                       uint32_t hkv, float eps, uint32_t rows) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // (launched as a programmatic dependent: see brasa_launch_dependent)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ __align__(16) uint8_t scratch[4][528];
    const uint32_t gr = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (gr >= rows) return;
    const uint32_t per_tok = hq + 2 * hkv, t = gr / per_tok, r = gr % per_tok, pos = lens[t];
    const size_t slot = (size_t)table[(size_t)t * max_pages + pos / PAGE] * PAGE + pos % PAGE;
    if (r >= hq + hkv) {
        const uint32_t kh = r - hq - hkv;
        float y[4];
        for (int j = 0; j < 4; ++j) y[j] = v[((size_t)t * hkv + kh) * 128 + lane + 32 * j];
        put_row<KV>(vpool + (slot * hkv + kh) * KvRow<KV>::BYTES, scratch[warp], y, lane);
        return;
    }
    const bool is_q = r < hq;
    float *x = is_q ? q + ((size_t)t * hq + r) * 128 : k + ((size_t)t * hkv + (r - hq)) * 128;
    float y[4];
    norm_rope_row(x, is_q ? q_norm : k_norm, cos_t, sin_t, pos, eps, lane, y);
    for (int j = 0; j < 4; ++j) x[lane + 32 * j] = y[j];
    if (!is_q) put_row<KV>(kpool + (slot * hkv + (r - hq)) * KvRow<KV>::BYTES, scratch[warp], y, lane);
}

// Rows [p0, p0 + n) of every layer of the contiguous cache -> the pages of one sequence (16-byte units).
__global__ void pages_from_cache_kernel(const uint8_t *cache, uint8_t *pool, const int32_t *table_row, uint32_t p0, uint32_t n, uint32_t row_bytes,
                                        size_t cache_layer_bytes, size_t pool_layer_bytes) {
    const uint32_t layer = blockIdx.y, units = row_bytes / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n * units; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t pos = p0 + (uint32_t)(i / units), u = (uint32_t)(i % units);
        const uint4 val = *reinterpret_cast<const uint4 *>(cache + layer * cache_layer_bytes + (size_t)pos * row_bytes + (size_t)u * 16);
        const size_t slot = (size_t)table_row[pos / PAGE] * PAGE + pos % PAGE;
        *reinterpret_cast<uint4 *>(pool + layer * pool_layer_bytes + slot * row_bytes + (size_t)u * 16) = val;
    }
}

// The inverse: pages of one sequence -> rows [p0, p0 + n) of every layer of the contiguous cache (a sequence admitted
// behind pages another sequence computed needs their rows where the prefill kernels read them).
__global__ void cache_from_pages_kernel(uint8_t *cache, const uint8_t *pool, const int32_t *table_row, uint32_t p0, uint32_t n, uint32_t row_bytes,
                                        size_t cache_layer_bytes, size_t pool_layer_bytes) {
    const uint32_t layer = blockIdx.y, units = row_bytes / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n * units; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t pos = p0 + (uint32_t)(i / units), u = (uint32_t)(i % units);
        const size_t slot = (size_t)table_row[pos / PAGE] * PAGE + pos % PAGE;
        const uint4 val = *reinterpret_cast<const uint4 *>(pool + layer * pool_layer_bytes + slot * row_bytes + (size_t)u * 16);
        *reinterpret_cast<uint4 *>(cache + layer * cache_layer_bytes + (size_t)pos * row_bytes + (size_t)u * 16) = val;
    }
}

__global__ void gather_ids_kernel(uint32_t *dst, const uint32_t *src, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[i];
}
__global__ void bump_lens_kernel(uint32_t *lens, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lens[i] += 1;
}

}  // namespace

struct brasa_batch {
    brasa_model *m = nullptr;
    brasa_ctx *ctx = nullptr;
    uint32_t max_seqs = 0, num_pages = 0, max_pages = 0;  // max_pages: per sequence
    uint32_t nseq = 0, next_page = 0, prefix_len = 0;
    size_t row_bytes = 0, pool_layer_bytes = 0, cache_layer_bytes = 0;
    uint64_t max_chunks = 0;
    brasa_buf *kpool = nullptr, *vpool = nullptr, *table = nullptr, *lens = nullptr, *ids = nullptr, *rng = nullptr, *logits = nullptr,
              *partials = nullptr, *scratch = nullptr, *out = nullptr;
    brasa_buf *tp_pad = nullptr, *tp_full = nullptr;  // tensor parallel: full-width logits of tp_rows sequences (this rank's share, all ranks')
    uint32_t tp_rows = 0;
    std::vector<int32_t> h_table;  // host mirror [max_seqs][max_pages]
    std::vector<uint32_t> h_lens;
    std::vector<brasa_buf *> owned;
    // The prefix cache: every full page of prompt tokens ever computed, found again by what it holds. A page's key
    // chains the key of the page before it with its own 16 token ids, so a key names the whole token sequence up to
    // and including the page (a radix tree over pages, stored as a hash map of its nodes).
    struct CachedPage {
        int32_t page;
        uint64_t parent;
        uint32_t ids[PAGE];
    };
    std::unordered_map<uint64_t, CachedPage> cached;
    std::vector<uint64_t> resident;     // key of the page whose rows the contiguous cache holds at page index i (0: none)
    std::vector<uint32_t> prefix_ids;   // the declared prefix (brasa_batch_set_prefix)
    uint32_t common_pages = 0;          // leading pages every sequence of the batch shares
    uint64_t hit_tokens = 0, prefilled_tokens = 0;
};

namespace {

constexpr uint64_t CHAIN_ROOT = 0x9E3779B97F4A7C15ull;

// Key of a page given the key of the page before it (CHAIN_ROOT for the first) and its 16 token ids. Never 0.
uint64_t chain_key(uint64_t parent, const uint32_t *ids) {
    uint64_t h = parent;
    for (uint32_t i = 0; i < PAGE; ++i) {
        h ^= (uint64_t)ids[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
        h *= 0xBF58476D1CE4E5B9ull;
        h ^= h >> 29;
    }
    return h ? h : 1;
}

int32_t balloc(brasa_batch *b, uint64_t bytes, brasa_buf **out) {
    BRASA_TRY(brasa_buf_alloc(b->ctx, bytes, out));
    b->owned.push_back(*out);
    return BRASA_OK;
}

int32_t upload_table_row(brasa_batch *b, uint32_t seq) {
    return brasa_buf_upload(b->table, (uint64_t)seq * b->max_pages * 4, b->h_table.data() + (size_t)seq * b->max_pages, (uint64_t)b->max_pages * 4);
}

// copies positions [p0, p0 + n) of the model's contiguous cache into the pages of sequence `seq`
int32_t copy_rows_to_pages(brasa_batch *b, brasa_cmd *cmd, uint32_t seq, uint32_t p0, uint32_t n) {
    if (n == 0) return BRASA_OK;
    brasa_model *m = b->m;
    dim3 grid(std::min<uint32_t>(1024, (uint32_t)(((size_t)n * (b->row_bytes / 16) + 255) / 256)), m->cfg.layers);
    const int32_t *row = (const int32_t *)b->table->ptr + (size_t)seq * b->max_pages;
    pages_from_cache_kernel<<<grid, 256, 0, b->ctx->stream>>>((const uint8_t *)m->kc->ptr, (uint8_t *)b->kpool->ptr, row, p0, n, (uint32_t)b->row_bytes,
                                                              b->cache_layer_bytes, b->pool_layer_bytes);
    BRASA_TRY(brasa_post_launch(cmd, "pages_from_cache"));
    pages_from_cache_kernel<<<grid, 256, 0, b->ctx->stream>>>((const uint8_t *)m->vc->ptr, (uint8_t *)b->vpool->ptr, row, p0, n, (uint32_t)b->row_bytes,
                                                              b->cache_layer_bytes, b->pool_layer_bytes);
    return brasa_post_launch(cmd, "pages_from_cache");
}

// copies the pages of sequence `seq` that hold positions [p0, p0 + n) into the model's contiguous cache
int32_t copy_pages_to_rows(brasa_batch *b, brasa_cmd *cmd, uint32_t seq, uint32_t p0, uint32_t n) {
    if (n == 0) return BRASA_OK;
    brasa_model *m = b->m;
    dim3 grid(std::min<uint32_t>(1024, (uint32_t)(((size_t)n * (b->row_bytes / 16) + 255) / 256)), m->cfg.layers);
    const int32_t *row = (const int32_t *)b->table->ptr + (size_t)seq * b->max_pages;
    cache_from_pages_kernel<<<grid, 256, 0, b->ctx->stream>>>((uint8_t *)m->kc->ptr, (const uint8_t *)b->kpool->ptr, row, p0, n, (uint32_t)b->row_bytes,
                                                              b->cache_layer_bytes, b->pool_layer_bytes);
    BRASA_TRY(brasa_post_launch(cmd, "cache_from_pages"));
    cache_from_pages_kernel<<<grid, 256, 0, b->ctx->stream>>>((uint8_t *)m->vc->ptr, (const uint8_t *)b->vpool->ptr, row, p0, n, (uint32_t)b->row_bytes,
                                                              b->cache_layer_bytes, b->pool_layer_bytes);
    return brasa_post_launch(cmd, "cache_from_pages");
}

// prefill of `n` tokens at positions [pos0, pos0 + n) through the model's contiguous cache, in chunks of max_tokens;
// the logits of the last token stay in the model's logits buffer
int32_t prefill_contiguous(brasa_batch *b, const uint32_t *ids, uint32_t n, uint32_t pos0) {
    brasa_model *m = b->m;
    for (uint32_t off = 0; off < n; off += m->limits.max_tokens) {
        const uint32_t c = std::min(m->limits.max_tokens, n - off);
        BRASA_TRY(brasa_model_forward(m, ids + off, c, pos0 + off, 1, nullptr, nullptr));
    }
    return BRASA_OK;
}

// x += h: the plain add, or for a tensor-parallel shard the sum over ranks of every rank's h
int32_t batch_residual_add(brasa_model *m, brasa_cmd *cmd, uint64_t n) {
    if (m->tp) return brasa_k_tp_allreduce_add(cmd, m->tp, A(m->h), A(m->x), A(m->x), n);
    return brasa_k_add(cmd, A(m->x), A(m->h), A(m->x), n);
}

// full[r][v] = shard[r][v - row0] for this rank's rows of the vocabulary, 0 elsewhere
__global__ void spread_shard_kernel(const float *shard, float *full, uint32_t n, uint32_t rows, uint32_t row0, uint32_t vocab) {
    const uint64_t tot = (uint64_t)n * vocab;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < tot; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / vocab), v = (uint32_t)(i - (uint64_t)r * vocab);
        full[i] = (v >= row0 && v < row0 + rows) ? shard[(size_t)r * rows + (v - row0)] : 0.0f;
    }
}

// Next token of `count` rows of logits (row stride = this rank's lm_head rows). A tensor-parallel shard holds only its
// rows of the vocabulary: a greedy choice exchanges each row's best (value, index) pair between the ranks, a sampled one the rows.
int32_t choose_tokens(brasa_batch *b, brasa_cmd *cmd, brasa_buf *logits, uint32_t count, brasa_sampling_params params, unsigned long long *rng,
                      float *scratch, brasa_buf *out, uint64_t out_index) {
    brasa_model *m = b->m;
    const uint32_t rows = m->cfg.head_rows;
    if (!m->tp || (params.temperature > 0.0f && rows == m->cfg.vocab))  // (a one-rank group holds the whole vocabulary)
        return brasa_sample_batched_launch(cmd, F(logits), rows, count, params.temperature, params.top_k, params.top_p, rng, scratch,
                                           (uint32_t *)out->ptr + out_index);
    if (params.temperature <= 0.0f) {
        for (uint32_t r = 0; r < count; ++r)
            BRASA_TRY(brasa_k_tp_argmax(cmd, m->tp, A(logits, (uint64_t)r * rows * 4), rows, m->cfg.head_row0, A(out, (out_index + r) * 4)));
        return BRASA_OK;
    }
    // Sampling needs every row's logits over the whole vocabulary on every rank. Each rank lays its rows of the vocabulary
    // into a zeroed full-width copy and the copies are added across the ranks (x + 0 is exact, so the sum is the
    // concatenation, bit for bit the same on every rank); then every rank runs the same sampler on the same numbers with
    // the same PCG32 streams and draws the same tokens. As many sequences per exchange as it can carry.
    const uint32_t vocab = m->cfg.vocab;
    const uint64_t cap = brasa_tp_max_elems(m->tp);
    BRASA_REQUIRE(b->ctx, b->tp_pad && b->tp_full && vocab % 2 == 0 && cap >= vocab, "batch: the tensor-parallel exchange is too small for one row of logits (%u values)", vocab);
    const uint32_t per = (uint32_t)std::min<uint64_t>(b->tp_rows, cap / vocab);
    for (uint32_t r0 = 0; r0 < count; r0 += per) {
        const uint32_t n = std::min(per, count - r0);
        const uint64_t tot = (uint64_t)n * vocab;
        spread_shard_kernel<<<(unsigned)std::min<uint64_t>((tot + 255) / 256, 4096), 256, 0, b->ctx->stream>>>(
            F(logits) + (size_t)r0 * rows, F(b->tp_pad), n, rows, m->cfg.head_row0, vocab);
        BRASA_TRY(brasa_post_launch(cmd, "spread_shard"));
        BRASA_TRY(brasa_k_tp_allreduce_add(cmd, m->tp, A(b->tp_pad), brasa_arg{nullptr, 0}, A(b->tp_full), tot));
        BRASA_TRY(brasa_sample_batched_launch(cmd, F(b->tp_full), vocab, n, params.temperature, params.top_k, params.top_p, rng + 2 * (size_t)r0,
                                              scratch + (size_t)r0 * 2 * vocab, (uint32_t *)out->ptr + out_index + r0));
    }
    return BRASA_OK;
}

// One decode step for the first n sequences: ids[n] -> logits[n][vocab]. Uses the model's workspace (n <= max_tokens).
int32_t encode_step(brasa_batch *b, brasa_cmd *cmd, uint32_t n) {
    brasa_model *m = b->m;
    brasa_ctx *ctx = b->ctx;
    const brasa_config &c = m->cfg;
    const uint32_t H = c.hidden;
    const bool half_io = n > GEMV_MAX_TOKENS && m->prefill_precision == BRASA_PREFILL_F16;
    const int32_t prec = half_io ? BRASA_PREFILL_F16 : BRASA_PREFILL_F32;
    auto mm = [&](const Matrix &w, brasa_arg x, brasa_arg y) -> int32_t {
        if (n <= GEMV_MAX_TOKENS) return brasa_k_gemv(cmd, w.q, x, y, n);
        return brasa_k_gemm_with(cmd, w.q, x, y, n, prec);
    };
    BRASA_TRY(brasa_k_embed(cmd, m->embed.q, A(b->ids), A(m->x), n));
    const uint32_t rows = n * (c.heads + 2 * c.kv_heads);
    const float scale = 1.0f / sqrtf(128.0f);
    const size_t smem = (128 * TS + 8 * D + 8 * 128 + 16) * sizeof(float);
    for (uint32_t li = 0; li < c.layers; ++li) {
        Layer &l = m->layers[li];
        brasa_arg xin;
        if (half_io) {
            // (after the first layer the norm was formed behind the down projection of the layer before: see below)
            if (li == 0 || m->tp) BRASA_TRY(brasa_k_rms_norm_f16(cmd, A(m->x), A(l.attn_norm), A(m->xh), n, H, c.eps));
            xin = A(m->xh);
        } else {
            BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x), A(l.attn_norm), A(m->norm_out), n, H, c.eps));
            xin = A(m->norm_out);
        }
        if (n > GEMV_MAX_TOKENS) {
            brasa_qmatrix wqkv[3] = {l.wq.q, l.wk.q, l.wv.q};
            brasa_arg yqkv[3] = {A(m->q), A(m->k_new), A(m->v_new)};
            BRASA_TRY(brasa_k_gemm_multi(cmd, wqkv, 3, xin, yqkv, n, prec));
        } else {
            BRASA_TRY(mm(l.wq, xin, A(m->q)));
            BRASA_TRY(mm(l.wk, xin, A(m->k_new)));
            BRASA_TRY(mm(l.wv, xin, A(m->v_new)));
        }
        uint8_t *kl = (uint8_t *)b->kpool->ptr + li * b->pool_layer_bytes, *vl = (uint8_t *)b->vpool->ptr + li * b->pool_layer_bytes;
        const int32_t *table = (const int32_t *)b->table->ptr;
        const uint32_t *lens = (const uint32_t *)b->lens->ptr;
        Paged kp{kl, table, b->max_pages, c.kv_heads}, vp{vl, table, b->max_pages, c.kv_heads};
        dim3 agrid((uint32_t)b->max_chunks, c.kv_heads, n), rgrid(c.heads, n);
        void *attn_out = half_io ? m->xh->ptr : m->attn->ptr;
#define LAUNCH_BATCH(KVT)                                                                                                                        \
    do {                                                                                                                                         \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_kernel<KVT>, smem)); \
        qk_norm_rope_store_paged_kernel<KVT><<<(rows + 3) / 4, 128, 0, ctx->stream>>>(F(m->q), F(m->k_new), F(m->v_new), F(l.q_norm), F(l.k_norm),   \
                                                                                     F(m->rope_cos), F(m->rope_sin), kl, vl, table, b->max_pages,  \
                                                                                     lens, c.heads, c.kv_heads, c.eps, rows);                     \
        BRASA_TRY(brasa_post_launch(cmd, "qk_norm_rope_store_paged"));                                                                           \
        decode_partial_paged_kernel<KVT><<<agrid, 128, smem, ctx->stream>>>(F(m->q), kp, vp, lens, F(b->partials), c.heads, (uint32_t)b->max_chunks, \
                                                                           scale);                                                               \
        BRASA_TRY(brasa_post_launch(cmd, "decode_partial_paged"));                                                                               \
    } while (0)
        if (m->limits.kv == BRASA_KV_F32) LAUNCH_BATCH(BRASA_KV_F32);
        else if (m->limits.kv == BRASA_KV_F16) {
                BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_mma_kernel<false>, MMA_SMEM));
                BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_mma_kernel<true>, MMA_SMEM));
            // the step's kernels are programmatic dependents of one another: each sets itself up while the one before it ends
            BRASA_CUDA(ctx, brasa_launch_dependent(ctx, qk_norm_rope_store_paged_kernel<BRASA_KV_F16>, dim3((rows + 3) / 4), dim3(128), 0, F(m->q), F(m->k_new),
                                                   F(m->v_new), F(l.q_norm), F(l.k_norm), F(m->rope_cos), F(m->rope_sin), kl, vl, table, b->max_pages, lens,
                                                   c.heads, c.kv_heads, c.eps, rows));
            BRASA_TRY(brasa_post_launch(cmd, "qk_norm_rope_store_paged"));
            // chunks wholly inside the shared prefix: one block serves 16 / G sequences; the rest per sequence
            const uint32_t G = c.heads / c.kv_heads;
            const uint32_t shared_chunks = (n > 1 && 16 % G == 0 && G < 16) ? b->common_pages * PAGE / 128 : 0;
            if (shared_chunks) {
                const uint32_t spb = 16 / G;
                BRASA_CUDA(ctx, brasa_launch_dependent(ctx, decode_partial_paged_mma_kernel<true>,
                                                       dim3(shared_chunks, c.kv_heads, (n + spb * PAGED_MMA_TILES - 1) / (spb * PAGED_MMA_TILES)), dim3(128), MMA_SMEM,
                                                       F(m->q), kp, vp, lens, F(b->partials), c.heads, (uint32_t)b->max_chunks, scale, 0u, n, 0u));
                BRASA_TRY(brasa_post_launch(cmd, "decode_partial_paged_mma_shared"));
            }
            if ((uint32_t)b->max_chunks > shared_chunks) {
                // (behind the shared-prefix form it runs beside it and waits for it at its end)
                BRASA_CUDA(ctx, brasa_launch_dependent(ctx, decode_partial_paged_mma_kernel<false>, dim3((uint32_t)b->max_chunks - shared_chunks, c.kv_heads, n),
                                                       dim3(128), MMA_SMEM, F(m->q), kp, vp, lens, F(b->partials), c.heads, (uint32_t)b->max_chunks, scale,
                                                       shared_chunks, n, shared_chunks ? 1u : 0u));
                BRASA_TRY(brasa_post_launch(cmd, "decode_partial_paged_mma"));
            }
        } else if (m->limits.kv == BRASA_KV_F16) LAUNCH_BATCH(BRASA_KV_F16);
        else LAUNCH_BATCH(BRASA_KV_Q8_0);
#undef LAUNCH_BATCH
        if (half_io) BRASA_CUDA(ctx, brasa_launch_dependent(ctx, decode_reduce_paged_kernel<true>, rgrid, dim3(128), 0, F(b->partials), lens, attn_out, c.heads, (uint32_t)b->max_chunks));
        else BRASA_CUDA(ctx, brasa_launch_dependent(ctx, decode_reduce_paged_kernel<false>, rgrid, dim3(128), 0, F(b->partials), lens, attn_out, c.heads, (uint32_t)b->max_chunks));
        BRASA_TRY(brasa_post_launch(cmd, "decode_reduce_paged"));
        // x += Wo attn and the norm of the feed-forward block: one call (one GEMM and one kernel behind it when the few-token
        // kernel takes the product)
        if (half_io && !m->tp) BRASA_TRY(brasa_k_gemm_add_rms_norm_f16(cmd, l.wo.q, A(m->xh), A(m->x), A(m->h), A(l.ffn_norm), A(m->xh), n, c.eps));
        else {
            BRASA_TRY(mm(l.wo, half_io ? A(m->xh) : A(m->attn), A(m->h)));
            BRASA_TRY(batch_residual_add(m, cmd, (uint64_t)n * H));
        }
        brasa_arg act;
        if (half_io) {
            if (m->tp) BRASA_TRY(brasa_k_rms_norm_f16(cmd, A(m->x), A(l.ffn_norm), A(m->xh), n, H, c.eps));
            act = brasa_gemm_swiglu_fuses(l.gate.q, l.up.q, n) ? A(m->up) : A(m->xh);
            BRASA_TRY(brasa_k_gemm_swiglu(cmd, l.gate.q, l.up.q, A(m->xh), A(m->gate), A(m->up), act, n));
        } else {
            BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x), A(l.ffn_norm), A(m->norm_out), n, H, c.eps));
            BRASA_TRY(mm(l.gate, A(m->norm_out), A(m->gate)));
            BRASA_TRY(mm(l.up, A(m->norm_out), A(m->up)));
            BRASA_TRY(brasa_k_swiglu(cmd, A(m->gate), A(m->up), A(m->gate), (uint64_t)n * c.ffn));
            act = A(m->gate);
        }
        // x += Wdown act and the norm that opens the next layer (the final norm after the last one)
        if (half_io && !m->tp)
            BRASA_TRY(brasa_k_gemm_add_rms_norm_f16(cmd, l.down.q, act, A(m->x), A(m->h), li + 1 < c.layers ? A(m->layers[li + 1].attn_norm) : A(m->final_norm),
                                                  A(m->xh), n, c.eps));
        else {
            BRASA_TRY(mm(l.down, act, A(m->h)));
            BRASA_TRY(batch_residual_add(m, cmd, (uint64_t)n * H));
        }
    }
    if (half_io) {
        if (m->tp) BRASA_TRY(brasa_k_rms_norm_f16(cmd, A(m->x), A(m->final_norm), A(m->xh), n, H, c.eps));
        return brasa_k_gemm_with(cmd, m->head.q, A(m->xh), A(b->logits), n, BRASA_PREFILL_F16);
    }
    BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x), A(m->final_norm), A(m->norm_out), n, H, c.eps));
    return brasa_k_gemv(cmd, m->head.q, A(m->norm_out), A(b->logits), n);
}

}  // namespace

extern "C" {

static int32_t check_paged(brasa_ctx *ctx, const brasa_paged_kv &pg, uint32_t hq, uint32_t hkv) {
    BRASA_REQUIRE(ctx, pg.kv >= BRASA_KV_F32 && pg.kv <= BRASA_KV_Q8_0, "paged kv: unknown KV type %d", pg.kv);
    BRASA_REQUIRE(ctx, hkv > 0 && hq % hkv == 0 && hq / hkv <= 8, "paged kv: GQA group must divide and be <= 8");
    BRASA_REQUIRE(ctx, pg.seqs >= 1 && pg.max_pages >= 1 && pg.num_pages >= 1, "paged kv: empty batch or pool");
    const uint64_t pool_bytes = brasa_kv_bytes(pg.kv, (uint64_t)pg.num_pages * PAGE * hkv * 128);
    BRASA_REQUIRE(ctx, arg_fits(pg.kpool, pool_bytes) && arg_fits(pg.vpool, pool_bytes), "paged kv: the pools are smaller than num_pages pages");
    BRASA_REQUIRE(ctx, arg_fits(pg.table, (uint64_t)pg.seqs * pg.max_pages * 4) && arg_fits(pg.lens, (uint64_t)pg.seqs * 4), "paged kv: table or lens too small");
    BRASA_REQUIRE(ctx, pg.kpool.offset % 16 == 0 && pg.vpool.offset % 16 == 0 && pg.table.offset % 4 == 0 && pg.lens.offset % 4 == 0, "paged kv: misaligned");
    return BRASA_OK;
}

int32_t brasa_k_qk_norm_rope_store_paged(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg q_norm, brasa_arg k_norm, brasa_arg rope_cos,
                                         brasa_arg rope_sin, float eps, brasa_paged_kv pg, uint32_t hq, uint32_t hkv) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_TRY(check_paged(ctx, pg, hq, hkv));
    BRASA_REQUIRE(ctx, arg_fits(q, (uint64_t)pg.seqs * hq * 512) && arg_fits(k, (uint64_t)pg.seqs * hkv * 512) && arg_fits(v, (uint64_t)pg.seqs * hkv * 512),
                  "qk_norm_rope_store_paged: q, k or v too small");
    BRASA_REQUIRE(ctx, arg_fits(q_norm, 512) && arg_fits(k_norm, 512), "qk_norm_rope_store_paged: norm weights too small");
    // the tables must cover every position a sequence of max_pages pages can reach
    const uint64_t table_floats = (uint64_t)pg.max_pages * PAGE * 64;
    BRASA_REQUIRE(ctx, arg_fits(rope_cos, table_floats * 4) && arg_fits(rope_sin, table_floats * 4), "qk_norm_rope_store_paged: RoPE tables shorter than max_pages pages");
    const uint32_t rows = pg.seqs * (hq + 2 * hkv);
    float *qp = (float *)arg_ptr(q), *kp = (float *)arg_ptr(k);
    const float *vp = (const float *)arg_ptr(v), *qn = (const float *)arg_ptr(q_norm), *kn = (const float *)arg_ptr(k_norm),
                *cs = (const float *)arg_ptr(rope_cos), *sn = (const float *)arg_ptr(rope_sin);
    const int32_t *table = (const int32_t *)arg_ptr(pg.table);
    const uint32_t *lens = (const uint32_t *)arg_ptr(pg.lens);
#define STORE_PAGED(KVT)                                                                                                                      \
    qk_norm_rope_store_paged_kernel<KVT><<<(rows + 3) / 4, 128, 0, ctx->stream>>>(qp, kp, vp, qn, kn, cs, sn, arg_ptr(pg.kpool), arg_ptr(pg.vpool), table, \
                                                                                 pg.max_pages, lens, hq, hkv, eps, rows)
    if (pg.kv == BRASA_KV_F32) STORE_PAGED(BRASA_KV_F32);
    else if (pg.kv == BRASA_KV_F16) STORE_PAGED(BRASA_KV_F16);
    else STORE_PAGED(BRASA_KV_Q8_0);
#undef STORE_PAGED
    return brasa_post_launch(cmd, "qk_norm_rope_store_paged");
}

int32_t brasa_k_decode_attention_paged(brasa_cmd *cmd, brasa_arg q, brasa_paged_kv pg, brasa_arg partials, uint64_t partials_len, brasa_arg o, uint32_t hq,
                                       uint32_t hkv) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_TRY(check_paged(ctx, pg, hq, hkv));
    const uint32_t max_chunks = (uint32_t)(((uint64_t)pg.max_pages * PAGE + 127) / 128);
    const uint64_t need = (uint64_t)pg.seqs * hq * max_chunks * 130;
    BRASA_REQUIRE(ctx, partials_len >= need && arg_fits(partials, partials_len * 4), "decode_attention_paged: scratch of %llu floats needed",
                  (unsigned long long)need);
    BRASA_REQUIRE(ctx, arg_fits(q, (uint64_t)pg.seqs * hq * 512) && arg_fits(o, (uint64_t)pg.seqs * hq * 512), "decode_attention_paged: q or o too small");
    const float scale = 1.0f / sqrtf(128.0f);
    const int32_t *table = (const int32_t *)arg_ptr(pg.table);
    const uint32_t *lens = (const uint32_t *)arg_ptr(pg.lens);
    Paged kp{arg_ptr(pg.kpool), table, pg.max_pages, hkv}, vp{arg_ptr(pg.vpool), table, pg.max_pages, hkv};
    const float *qp = (const float *)arg_ptr(q);
    float *pp = (float *)arg_ptr(partials);
    dim3 agrid(max_chunks, hkv, pg.seqs), rgrid(hq, pg.seqs);
    if (pg.kv == BRASA_KV_F16) {  // tensor-core partials (one block per chunk, kv head and sequence)
        BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_mma_kernel<false>, MMA_SMEM));
        decode_partial_paged_mma_kernel<false><<<agrid, 128, MMA_SMEM, ctx->stream>>>(qp, kp, vp, lens, pp, hq, max_chunks, scale, 0, pg.seqs, 0);
    } else {
        const size_t smem = (128 * TS + 8 * D + 8 * 128 + 16) * sizeof(float);
        if (pg.kv == BRASA_KV_F32) {
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_kernel<BRASA_KV_F32>, smem));
            decode_partial_paged_kernel<BRASA_KV_F32><<<agrid, 128, smem, ctx->stream>>>(qp, kp, vp, lens, pp, hq, max_chunks, scale);
        } else {
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)decode_partial_paged_kernel<BRASA_KV_Q8_0>, smem));
            decode_partial_paged_kernel<BRASA_KV_Q8_0><<<agrid, 128, smem, ctx->stream>>>(qp, kp, vp, lens, pp, hq, max_chunks, scale);
        }
    }
    BRASA_TRY(brasa_post_launch(cmd, "decode_partial_paged"));
    decode_reduce_paged_kernel<false><<<rgrid, 128, 0, ctx->stream>>>(pp, lens, arg_ptr(o), hq, max_chunks);
    return brasa_post_launch(cmd, "decode_reduce_paged");
}

// The buffers of brasa_batch_create, one term each, at the allocation granularity of the planner.
int32_t brasa_plan_batch(const brasa_model_shape *m, const brasa_batch_shape *s, brasa_batch_plan *out) {
    if (!m || !s || !out) return BRASA_EINVAL;
    if (s->kv < BRASA_KV_F32 || s->kv > BRASA_KV_Q8_0 || s->max_seqs == 0 || s->max_positions < PAGE) return BRASA_EINVAL;
    auto g = [](uint64_t n) { return brasa_plan_buffer_bytes(n); };
    const uint64_t max_pages = ((uint64_t)s->max_positions + PAGE - 1) / PAGE, max_chunks = (max_pages * PAGE + 127) / 128;
    const uint64_t row_bytes = brasa_kv_bytes(s->kv, (uint64_t)m->kv_heads * 128);
    out->kv_pages = 2 * g((uint64_t)m->layers * s->num_pages * PAGE * row_bytes);
    out->tables = g((uint64_t)s->max_seqs * max_pages * 4) + 3 * g((uint64_t)s->max_seqs * 4) + g((uint64_t)s->max_seqs * 16);
    out->logits = g((uint64_t)s->max_seqs * s->head_rows * 4);
    out->attention_partials = g((uint64_t)s->max_seqs * m->heads * max_chunks * 130 * 4);
    out->sampler = g((uint64_t)s->max_seqs * 2 * m->vocab * 4);
    // a tensor-parallel shard (fewer lm_head rows than the vocabulary) samples over logits gathered from all ranks
    if (s->head_rows < m->vocab) out->sampler += 2 * g((uint64_t)s->max_seqs * m->vocab * 4);
    out->total = out->kv_pages + out->tables + out->logits + out->attention_partials + out->sampler;
    return BRASA_OK;
}

int32_t brasa_plan_batch_max_seqs(brasa_ctx *ctx, const brasa_model_shape *m, int32_t kv, uint32_t head_rows, uint32_t shared_prefix,
                                  uint32_t positions_per_seq, uint32_t max_seqs_cap, uint64_t budget, uint32_t *max_seqs_out,
                                  uint32_t *num_pages_out, brasa_batch_plan *plan_out) {
    if (!m || !max_seqs_out) return BRASA_EINVAL;
    BRASA_REQUIRE(ctx, shared_prefix % PAGE == 0 && positions_per_seq > shared_prefix && max_seqs_cap >= 1,
                  "plan_batch: the shared prefix must fill whole pages and lie inside a sequence's positions");
    if (budget == 0) {
        if (!ctx) return BRASA_EINVAL;
        uint64_t free_b = 0, total_b = 0;
        BRASA_TRY(brasa_ctx_mem_info(ctx, &free_b, &total_b));
        budget = free_b > (512ull << 20) ? free_b - (512ull << 20) : 0;
    }
    const uint32_t max_pages = (positions_per_seq + PAGE - 1) / PAGE, own = max_pages - shared_prefix / PAGE;
    auto plan_of = [&](uint32_t n, brasa_batch_plan *p, uint32_t *pages) {
        const uint64_t np = (uint64_t)shared_prefix / PAGE + (uint64_t)n * own;
        *pages = (uint32_t)std::min<uint64_t>(np, UINT32_MAX);
        const brasa_batch_shape s{n, *pages, positions_per_seq, head_rows, kv};
        return brasa_plan_batch(m, &s, p);
    };
    uint32_t lo = 0, hi = max_seqs_cap;  // the plan grows with the number of sequences
    while (lo < hi) {
        const uint32_t mid = lo + (hi - lo + 1) / 2;
        brasa_batch_plan p;
        uint32_t pages;
        BRASA_TRY(plan_of(mid, &p, &pages));
        if (p.total <= budget) lo = mid;
        else hi = mid - 1;
    }
    *max_seqs_out = lo;
    if (lo == 0) return brasa_fail(ctx, BRASA_EBUDGET, "plan_batch: not even one sequence of %u positions fits %.2f GiB", positions_per_seq, budget / 1073741824.0);
    brasa_batch_plan p;
    uint32_t pages;
    BRASA_TRY(plan_of(lo, &p, &pages));
    if (plan_out) *plan_out = p;
    if (num_pages_out) *num_pages_out = pages;
    return BRASA_OK;
}

int32_t brasa_batch_allocated(brasa_batch *b, uint64_t *bytes) {
    if (!b || !bytes) return BRASA_EINVAL;
    uint64_t sum = 0;
    for (brasa_buf *x : b->owned) sum += brasa_plan_buffer_bytes(x->bytes);
    *bytes = sum;
    return BRASA_OK;
}

void brasa_batch_free(brasa_batch *b) {
    if (!b) return;
    for (brasa_buf *x : b->owned) brasa_buf_free(x);
    delete b;
}

int32_t brasa_batch_create(brasa_model *m, uint32_t max_seqs, uint32_t num_pages, uint32_t max_positions, brasa_batch **out) {
    if (!m || !out) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_REQUIRE(ctx, max_seqs >= 1 && max_seqs <= m->limits.max_tokens, "batch: 1 to max_tokens (%u) sequences", m->limits.max_tokens);
    BRASA_REQUIRE(ctx, m->cfg.head_dim == 128 && m->cfg.heads % m->cfg.kv_heads == 0 && m->cfg.heads / m->cfg.kv_heads <= 8,
                  "batch: head_dim 128 and a GQA group of at most 8");
    BRASA_REQUIRE(ctx, max_positions >= PAGE && max_positions <= m->limits.ctx, "batch: max_positions within the model's context");
    BRASA_REQUIRE(ctx, m->tp || m->cfg.head_rows == m->cfg.vocab, "batch: a tensor-parallel shard needs its exchange attached first (brasa_model_set_tp)");
    std::unique_ptr<brasa_batch, void (*)(brasa_batch *)> b(new brasa_batch, brasa_batch_free);
    b->m = m;
    b->ctx = ctx;
    b->max_seqs = max_seqs;
    b->num_pages = num_pages;
    b->max_pages = (max_positions + PAGE - 1) / PAGE;
    const uint64_t kvd = (uint64_t)m->cfg.kv_heads * 128;
    b->row_bytes = brasa_kv_bytes(m->limits.kv, kvd);
    b->pool_layer_bytes = (size_t)num_pages * PAGE * b->row_bytes;
    b->cache_layer_bytes = (size_t)m->cap * b->row_bytes;
    b->max_chunks = ((uint64_t)b->max_pages * PAGE + 127) / 128;
    // the plan first: a batch that cannot fit is refused before anything is allocated
    const brasa_model_shape shape{0, m->cfg.layers, m->cfg.hidden, m->cfg.heads, m->cfg.kv_heads, m->cfg.head_dim, m->cfg.ffn, m->cfg.vocab};
    const brasa_batch_shape bshape{max_seqs, num_pages, max_positions, m->cfg.head_rows, m->limits.kv};
    brasa_batch_plan plan;
    BRASA_TRY(brasa_plan_batch(&shape, &bshape, &plan));
    uint64_t free_b = 0, total_b = 0;
    BRASA_TRY(brasa_ctx_mem_info(ctx, &free_b, &total_b));
    if (plan.total + (512ull << 20) > free_b)
        return brasa_fail(ctx, BRASA_EBUDGET, "batch: %u sequences over %u pages need %.2f GiB (KV pages %.2f) and the device has %.2f GiB free",
                          max_seqs, num_pages, plan.total / 1073741824.0, plan.kv_pages / 1073741824.0, free_b / 1073741824.0);
    BRASA_TRY(balloc(b.get(), (uint64_t)m->cfg.layers * b->pool_layer_bytes, &b->kpool));
    BRASA_TRY(balloc(b.get(), (uint64_t)m->cfg.layers * b->pool_layer_bytes, &b->vpool));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * b->max_pages * 4, &b->table));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * 4, &b->lens));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * 4, &b->ids));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * 4, &b->out));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * 16, &b->rng));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * m->cfg.head_rows * 4, &b->logits));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * m->cfg.heads * b->max_chunks * 130 * 4, &b->partials));
    BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * 2 * m->cfg.vocab * 4, &b->scratch));
    if (m->cfg.head_rows < m->cfg.vocab) {
        BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * m->cfg.vocab * 4, &b->tp_pad));
        BRASA_TRY(balloc(b.get(), (uint64_t)max_seqs * m->cfg.vocab * 4, &b->tp_full));
        b->tp_rows = max_seqs;
    }
    b->h_table.assign((size_t)max_seqs * b->max_pages, 0);
    b->h_lens.assign(max_seqs, 0);
    b->resident.assign(b->max_pages, 0);
    *out = b.release();
    return BRASA_OK;
}

// The prefix every sequence starts with: computed once, kept in the model's contiguous cache at [0, n) and in pages that
// the prefix cache hands to every sequence that starts with these tokens.
int32_t brasa_batch_set_prefix(brasa_batch *b, const uint32_t *ids, uint32_t n) {
    if (!b || (!ids && n)) return BRASA_EINVAL;
    brasa_ctx *ctx = b->ctx;
    BRASA_REQUIRE(ctx, b->nseq == 0 && b->next_page == 0, "batch: the prefix comes before the sequences");
    BRASA_REQUIRE(ctx, n % PAGE == 0, "batch: the shared prefix must fill whole pages of %u positions", PAGE);
    BRASA_REQUIRE(ctx, n / PAGE <= b->max_pages && n / PAGE <= b->num_pages, "batch: prefix longer than the page budget");
    b->prefix_len = n;
    b->prefix_ids.assign(ids, ids + n);
    if (n == 0) return BRASA_OK;
    BRASA_TRY(prefill_contiguous(b, ids, n, 0));
    b->prefilled_tokens += n;
    // pages 0 .. n/16 - 1, listed in row 0 of the table for the copy, and entered into the prefix cache
    uint64_t key = CHAIN_ROOT;
    for (uint32_t i = 0; i < n / PAGE; ++i) {
        b->h_table[i] = (int32_t)i;
        brasa_batch::CachedPage cp{(int32_t)i, key, {}};
        memcpy(cp.ids, ids + (size_t)i * PAGE, sizeof cp.ids);
        key = chain_key(key, ids + (size_t)i * PAGE);
        b->cached.emplace(key, cp);
        b->resident[i] = key;
    }
    b->next_page = n / PAGE;
    BRASA_TRY(upload_table_row(b, 0));
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = copy_rows_to_pages(b, cmd, 0, 0, n);
    int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
    BRASA_TRY(rc);
    return rc2;
}

// A new sequence: the declared prefix followed by its own n tokens (n >= 1). Every leading full page of that token
// sequence that some earlier sequence (or the declared prefix) already computed is attached instead of recomputed
// (crates/runtime/src/session.rs:230-237 for many sequences: the longest cached prefix is reused and at least the last
// prompt token is always recomputed); the rest is prefilled and its full pages join the cache. Its first generated
// token is drawn from the logits of its last prompt token with its own PCG32 stream (params.seed + sequence index).
int32_t brasa_batch_add_sequence(brasa_batch *b, const uint32_t *ids, uint32_t n, brasa_sampling_params params, uint32_t *seq_out) {
    if (!b || !ids) return BRASA_EINVAL;
    brasa_ctx *ctx = b->ctx;
    brasa_model *m = b->m;
    BRASA_REQUIRE(ctx, b->nseq < b->max_seqs, "batch: all %u sequence slots are in use", b->max_seqs);
    BRASA_REQUIRE(ctx, n >= 1 && (uint64_t)b->prefix_len + n < (uint64_t)b->max_pages * PAGE, "batch: sequence longer than max_positions");
    const uint32_t seq = b->nseq, total = b->prefix_len + n;
    std::vector<uint32_t> full(b->prefix_ids);
    full.insert(full.end(), ids, ids + n);
    // walk the cache: page h of this sequence is a hit when its key is known and names these very tokens
    int32_t *row = b->h_table.data() + (size_t)seq * b->max_pages;
    std::vector<uint64_t> keys;
    uint64_t key = CHAIN_ROOT;
    uint32_t hit = 0;
    const uint32_t max_hit = (total - 1) / PAGE;  // the last prompt token is computed here, whatever the cache holds
    while (hit < max_hit) {
        const uint64_t k = chain_key(key, full.data() + (size_t)hit * PAGE);
        auto it = b->cached.find(k);
        if (it == b->cached.end() || it->second.parent != key || memcmp(it->second.ids, full.data() + (size_t)hit * PAGE, sizeof it->second.ids) != 0) break;
        row[hit] = it->second.page;
        keys.push_back(k);
        key = k;
        ++hit;
    }
    const uint32_t matched = hit * PAGE, own = b->max_pages - hit;
    BRASA_REQUIRE(ctx, b->next_page + own <= b->num_pages, "batch: out of KV pages (%u of %u in use)", b->next_page, b->num_pages);
    for (uint32_t i = 0; i < own; ++i) row[hit + i] = (int32_t)(b->next_page + i);
    b->next_page += own;
    BRASA_TRY(upload_table_row(b, seq));
    // the prefill kernels read earlier positions from the contiguous cache: bring in the hit pages it does not hold
    {
        brasa_cmd *cmd;
        BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
        int32_t rc = BRASA_OK;
        for (uint32_t i = 0; i < hit && rc == BRASA_OK;) {
            if (b->resident[i] == keys[i]) {
                ++i;
                continue;
            }
            uint32_t j = i;
            while (j < hit && b->resident[j] != keys[j]) ++j;
            rc = copy_pages_to_rows(b, cmd, seq, i * PAGE, (j - i) * PAGE);
            for (uint32_t q = i; q < j; ++q) b->resident[q] = keys[q];
            i = j;
        }
        int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
        BRASA_TRY(rc);
        BRASA_TRY(rc2);
    }
    BRASA_TRY(prefill_contiguous(b, full.data() + matched, total - matched, matched));
    b->hit_tokens += matched;
    b->prefilled_tokens += total - matched;
    // the full pages computed just now join the cache; what lies behind them in the contiguous cache is not a page
    const uint32_t full_pages = total / PAGE;
    for (uint32_t i = hit; i < b->max_pages; ++i) {
        if (i < full_pages) {
            brasa_batch::CachedPage cp{row[i], key, {}};
            memcpy(cp.ids, full.data() + (size_t)i * PAGE, sizeof cp.ids);
            key = chain_key(key, full.data() + (size_t)i * PAGE);
            b->cached.emplace(key, cp);  // an equal key already there (the page at max_hit of an identical prompt) keeps its page
            b->resident[i] = key;
        } else {
            b->resident[i] = 0;
        }
    }
    // leading pages shared by every sequence of the batch: their keys are read once per group of sequences by the
    // attention kernel
    if (seq == 0) {
        b->common_pages = full_pages;
    } else {
        const int32_t *row0 = b->h_table.data();
        uint32_t c = 0;
        while (c < b->common_pages && c < hit && row[c] == row0[c]) ++c;
        b->common_pages = c;
    }
    uint64_t st[2];
    brasa_pcg32_seed(params.seed + seq, st);
    BRASA_TRY(brasa_buf_upload(b->rng, (uint64_t)seq * 16, st, 16));
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = copy_rows_to_pages(b, cmd, seq, matched, total - matched);
    if (rc == BRASA_OK)
        rc = choose_tokens(b, cmd, m->logits, 1, params, (unsigned long long *)b->rng->ptr + 2 * seq, F(b->scratch) + (size_t)seq * 2 * m->cfg.vocab,
                           b->ids, seq);
    int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
    BRASA_TRY(rc);
    BRASA_TRY(rc2);
    b->h_lens[seq] = total;
    BRASA_TRY(brasa_buf_upload(b->lens, (uint64_t)seq * 4, &total, 4));
    b->nseq = seq + 1;
    if (seq_out) *seq_out = seq;
    return BRASA_OK;
}

// `steps` tokens for every sequence, on the device: step s feeds each sequence its previous token, samples the next.
// out_ids[seq * (steps + 1) + s]: s = 0 is the token drawn at add time, then the steps' tokens.
int32_t brasa_batch_decode(brasa_batch *b, uint32_t steps, brasa_sampling_params params, uint32_t *out_ids, double *gpu_seconds) {
    if (!b) return BRASA_EINVAL;
    brasa_ctx *ctx = b->ctx;
    brasa_model *m = b->m;
    const uint32_t n = b->nseq;
    BRASA_REQUIRE(ctx, n >= 1, "batch: no sequences");
    for (uint32_t s = 0; s < n; ++s)
        BRASA_REQUIRE(ctx, (uint64_t)b->h_lens[s] + steps <= (uint64_t)b->max_pages * PAGE, "batch: sequence %u would pass max_positions", s);
    std::vector<uint32_t> tok(n);
    if (out_ids) {
        BRASA_TRY(brasa_buf_download(b->ids, 0, tok.data(), (uint64_t)n * 4));
        for (uint32_t s = 0; s < n; ++s) out_ids[(size_t)s * (steps + 1)] = tok[s];
    }
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = BRASA_OK;
    std::vector<uint32_t> all((size_t)n * steps);
    brasa_buf *hist = nullptr;
    rc = brasa_buf_alloc(ctx, std::max<uint64_t>(4, (uint64_t)n * steps * 4), &hist);
    for (uint32_t s = 0; s < steps && rc == BRASA_OK; ++s) {
        rc = encode_step(b, cmd, n);
        if (rc != BRASA_OK) break;
        rc = choose_tokens(b, cmd, b->logits, n, params, (unsigned long long *)b->rng->ptr, F(b->scratch), b->out, 0);
        if (rc != BRASA_OK) break;
        gather_ids_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((uint32_t *)b->ids->ptr, (const uint32_t *)b->out->ptr, n);
        rc = brasa_post_launch(cmd, "next_ids");
        if (rc != BRASA_OK) break;
        gather_ids_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((uint32_t *)hist->ptr + (size_t)s * n, (const uint32_t *)b->out->ptr, n);
        rc = brasa_post_launch(cmd, "history");
        if (rc != BRASA_OK) break;
        bump_lens_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>((uint32_t *)b->lens->ptr, n);
        rc = brasa_post_launch(cmd, "advance_lengths");
    }
    int32_t rc2 = brasa_cmd_wait(cmd, gpu_seconds);
    if (rc == BRASA_OK) rc = rc2;
    if (rc == BRASA_OK && out_ids && steps) {
        rc = brasa_buf_download(hist, 0, all.data(), (uint64_t)n * steps * 4);
        for (uint32_t s = 0; s < steps; ++s)
            for (uint32_t q = 0; q < n; ++q) out_ids[(size_t)q * (steps + 1) + 1 + s] = all[(size_t)s * n + q];
    }
    if (hist) brasa_buf_free(hist);
    if (rc == BRASA_OK)
        for (uint32_t s = 0; s < n; ++s) b->h_lens[s] += steps;
    return rc;
}

// Logits of every sequence's next token for its current input token, without sampling or advancing (tests).
int32_t brasa_batch_peek_logits(brasa_batch *b, float *logits) {
    if (!b || !logits) return BRASA_EINVAL;
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(b->ctx, &cmd));
    int32_t rc = encode_step(b, cmd, b->nseq);
    int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
    BRASA_TRY(rc);
    BRASA_TRY(rc2);
    return brasa_buf_download(b->logits, 0, logits, (uint64_t)b->nseq * b->m->cfg.head_rows * 4);
}

uint32_t brasa_batch_sequences(brasa_batch *b) { return b ? b->nseq : 0; }
uint32_t brasa_batch_pages_in_use(brasa_batch *b) { return b ? b->next_page : 0; }

int32_t brasa_batch_prefix_cache_stats(brasa_batch *b, uint64_t *hit_tokens, uint64_t *prefilled_tokens, uint32_t *cached_pages, uint32_t *common_pages) {
    if (!b) return BRASA_EINVAL;
    if (hit_tokens) *hit_tokens = b->hit_tokens;
    if (prefilled_tokens) *prefilled_tokens = b->prefilled_tokens;
    if (cached_pages) *cached_pages = (uint32_t)b->cached.size();
    if (common_pages) *common_pages = b->common_pages;
    return BRASA_OK;
}

}  // extern "C"
