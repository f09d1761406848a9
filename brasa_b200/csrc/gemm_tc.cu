// Prefill GEMM on the 5th-generation tensor cores: Y[t, :] = W X[t, :] for many tokens, W q4_0 in the tiled layout,
// X f16, f32 accumulation (crates/kernels/src/lib.rs:842-970 and matmul_tiled.metal:35-53: each dequantised weight
// is rounded to f16 as f16(f32(d) * (q - 8)) before it meets the f16 activation).
//
// One CTA computes a [MT x 128 tokens] x [128 weight rows] block of Y with tcgen05.mma (M = 128 tokens, N = 128
// rows, K = 16 per instruction), accumulating in tensor memory (MT x 128 columns of 128 lanes), K in stages of 64:
//   * warp 0, one lane: TMA. The X tile of a stage (MT boxes of 128 tokens x 64 halves) arrives by
//     cp.async.bulk.tensor with the 128-byte swizzle; tokens past the end read as zeros.
//   * warps 4-11: weights. Each thread owns one quantisation block (32 columns) of one weight row per stage: it reads
//     16 code bytes and the scale, turns nibbles into f16 with exact arithmetic (0x6400 | q is the half 1024 + q; minus 1032;
//     times d in f16 rounds the exact product once, as the reference's f32 product does) and writes the row in the
//     same swizzled K-major form the TMA produces. The tensor core reads both operands from shared memory.
//   * warp 1, one lane: tcgen05.mma for the stage, then tcgen05.commit to hand the stage back.
//   * after the last stage warps 4-11 read the accumulators (tcgen05.ld, one token per lane) and store Y.
// Up to three matrices that share X (q, k, v) go into one launch: the grid's x index walks their 128-row tiles.
// Every wait is bounded: a wait that runs out raises the context's status word and a CTA-wide flag, every role
// leaves its loop, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <cmath>

#include "brasa_internal.h"
#include "gemv_device.cuh"

using namespace brasa_dev;

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr uint32_t A_TILE = BM * BK * 2, B_TILE = BN * BK * 2;  // 16 KB each
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ __half2 u2h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
// two nibbles (already in the low 4 bits of each half lane) -> f16(d * (q - 8)) for both
__device__ __forceinline__ uint32_t deq2(uint32_t lanes, __half2 bias, __half2 d2, uint32_t mask = 0x000F000Fu) {
    return h22u(__hmul2(__hsub2(u2h2((lanes & mask) | 0x64006400u), bias), d2));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

struct GemmTcParams {
    const uint8_t *w[3];   // up to three matrices that share the input (q, k, v)
    float *y[3];
    uint32_t rows[3];
    uint32_t tile_end[3];  // 128-row tiles of matrices 0..i, cumulative
    uint32_t cols, tokens, stages;
    uint32_t *status;
    __half *glu;          // when set: w[0] = gate, w[1] = up, a CTA holds 128 rows of each and writes f16(silu(gate) * up) here
    const float *resid;   // when set (one matrix only): Y = resid + W X, the residual add of the layer (resid may be Y itself)
    uint32_t ksplit;      // grid.z CTAs share one output tile, each over its own range of K stages
    float *part;          // ksplit > 1: [z][tile][MT x 128 tokens][BNT rows] partial tiles
    uint32_t *counters;   // ksplit > 1: arrivals per output tile (zero between launches)
};

// One tensor map per weight matrix: the tiled matrix as bytes [rows][row_bytes], box = 32 bytes x the CTA's rows. The
// same box fetches a stage's codes (two blocks of 16 bytes per row) and, from the scale area behind the codes, the
// 16 scales of 8 consecutive stages.
struct WeightMaps {
    CUtensorMap m[3];
};
constexpr uint32_t RAW_TILE = BN * 32;  // codes of one stage for 128 rows; as many bytes again for the scales

// RAW: the stage's weight bytes come through TMA into shared memory and the conversion reads them there (few tokens:
// weight traffic decides, and per-thread 16-byte loads from 128 different rows keep too few bytes in flight); otherwise
// every conversion thread loads its codes straight from global memory one stage of its group ahead (many tokens: the
// ring is only two stages deep and a weight tile that waits for a free slot before it even leaves L2 would stall it).
// QT: q4_0, or q6_0 (the tied lm_head of a batch step; direct loads only): the codes' two high bits come from the row's
// high-bit words, laid out so that one shift per quad of codes puts them at bits 4-5 of the bytes (see brasa_internal.h).
template <int MT, int G, int NB, bool RAW, int QT = BRASA_Q4_0>
__global__ void __launch_bounds__(384, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ WeightMaps wmaps,
                                                         GemmTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the dynamic shared memory base is only 16-byte aligned by contract: round up to the swizzle atom
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t BNT = BN * NB;  // weight rows of this CTA: one MMA covers them all (N = 128 or 256)
    const uint32_t stage_bytes = MT * A_TILE + NB * B_TILE + (RAW ? NB * 2 * RAW_TILE : 0);  // X tiles, converted W, raw codes, raw scales
    __shared__ uint64_t full_x[8], full_w[8], empty[8], acc_full;
    __shared__ uint32_t tmem_base_s, abort_s, last_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // which matrix and which BNT rows of it
    const bool glu = NB == 2 && p.glu != nullptr;  // gate and up side by side: weight rows [0, 128) of the CTA are gate's, [128, 256) up's
    const uint32_t mi = glu ? 0u : (blockIdx.x >= p.tile_end[0]) + (blockIdx.x >= p.tile_end[1]);
    const uint32_t n0 = glu ? blockIdx.x * BN : (blockIdx.x - (mi == 0 ? 0u : (mi == 1 ? p.tile_end[0] : p.tile_end[1]))) * BNT,
                   tok0 = blockIdx.y * (MT * BM);
    const uint8_t *wmat = mi == 0 ? p.w[0] : (mi == 1 ? p.w[1] : p.w[2]);
    float *ymat = mi == 0 ? p.y[0] : (mi == 1 ? p.y[1] : p.y[2]);
    const uint32_t yrows = mi == 0 ? p.rows[0] : (mi == 1 ? p.rows[1] : p.rows[2]);
    const uint32_t NS = p.stages;
    // this CTA's K stages: [kbeg, kbeg + nk) of the cols / BK stages of the product
    const uint32_t nk_all = p.cols / BK, kbeg = (uint32_t)((uint64_t)blockIdx.z * nk_all / p.ksplit),
                   nk = (uint32_t)((uint64_t)(blockIdx.z + 1) * nk_all / p.ksplit) - kbeg;

    if (tid == 0) {
        for (uint32_t s = 0; s < NS; ++s) {
            mbar_init(&full_x[s], 1);
            mbar_init(&full_w[s], 8 / G);  // one arrival per warp of the group that converts the stage
            mbar_init(&empty[s], 1);
        }
        mbar_init(&acc_full, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory for the accumulators: MT x BNT columns
        uint32_t ncols = MT * BNT;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // Launched as a programmatic dependent: everything above ran while the kernel before this one was still finishing, and
    // so do the copies of the first stages' weights (weights never change); that kernel's results (X, the residual, the
    // split-K workspace) are read only after the wait.
    auto issue_weights = [&](uint32_t k) {  // raw codes and scales of stage k (RAW only); the stage's byte count is announced here
        const uint32_t s = k % NS;
        uint8_t *raw = smem + (size_t)s * stage_bytes + MT * A_TILE + NB * B_TILE;
        mbar_expect_tx(&full_x[s], MT * A_TILE + NB * 2 * RAW_TILE);
        const CUtensorMap *wm = &wmaps.m[mi];
        const uint32_t kk = kbeg + k, sc_x = tiled_scale_off(BRASA_Q4_0, p.cols) + 32 * (kk >> 3);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(raw)),
                     "l"(wm), "r"((int)(kk * 32)), "r"((int)n0), "r"(smem_u32(&full_x[s]))
                     : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         smem_u32(raw + NB * RAW_TILE)),
                     "l"(wm), "r"((int)sc_x), "r"((int)n0), "r"(smem_u32(&full_x[s]))
                     : "memory");
    };
    const uint32_t early = RAW ? min(NS, nk) : 0u;  // stages whose weights are asked for before the wait
    if (RAW && tid == 0) {
        for (uint32_t k = 0; k < early; ++k) issue_weights(k);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    volatile uint32_t *abort_flag = &abort_s;

    // bounded wait shared by every role; false when it gave up (or another role did)
    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
        for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
            if (mbar_try(bar, parity)) return true;
            if (*abort_flag) return false;
        }
        atomicExch(p.status, 4u);
        *abort_flag = 1;
        return false;
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t issued = 0;
            for (uint32_t k = 0; k < nk; ++k) {
                const uint32_t s = k % NS;
                if (k >= NS && !wait(&empty[s], ((k / NS) - 1) & 1)) break;
                uint8_t *dst = smem + (size_t)s * stage_bytes;
                if (RAW) {
                    if (k >= early) issue_weights(k);  // (announces the stage's bytes; the first stages' went out before the wait)
                } else {
                    mbar_expect_tx(&full_x[s], MT * A_TILE);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                                     smem_u32(dst + mt * A_TILE)),
                                 "l"(&tmap_x), "r"((int)((kbeg + k) * BK)), "r"((int)(tok0 + mt * BM)), "r"(smem_u32(&full_x[s]))
                                 : "memory");
                }
                issued = k + 1;
            }
            if (*abort_flag) {  // leaving early: let the copies already in flight land before the CTA exits
                // (the first stages' weights went out before the loop: a stage whose X never followed cannot complete its
                // barrier, and the bounded spin below is then simply the time its weight copies are given to land)
                const uint32_t last = max(issued, early);
                for (uint32_t k = last > NS ? last - NS : 0; k < last; ++k)
                    for (uint32_t it = 0; it < TC_WAIT_LIMIT && !mbar_try(&full_x[k % NS], (k / NS) & 1); ++it) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D f32, A and B f16, both K-major, N = BNT, M = 128
            const uint32_t idesc = (1u << 4) | ((uint32_t)(BNT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (uint32_t k = 0; k < nk && ok; ++k) {
                const uint32_t s = k % NS, ph = (k / NS) & 1;
                ok = wait(&full_x[s], ph) && wait(&full_w[s], ph);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = smem_u32(smem + (size_t)s * stage_bytes), b0 = a0 + MT * A_TILE;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks) {
                        const uint64_t da = smem_desc(a0 + mt * A_TILE + ks * 32), db = smem_desc(b0 + ks * 32);
                        const uint32_t acc = (k > 0 || ks > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                            ::"r"(tmem_base + mt * BNT), "l"(da), "l"(db), "r"(idesc), "r"(acc)
                            : "memory");
                    }
                }
                // the stage is free once these MMAs have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
            }
            if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&acc_full)) : "memory");
        }
    } else if (warp >= 4) {
        // ---- weights. The eight warps form G groups that take the stages in turn (group g: stages g, g + G, ..), so
        // G stages are being converted at once: the fence that makes a stage's writes visible to the tensor core costs
        // far more than the conversion itself and must overlap with the next stages' work. A thread of a group owns G
        // units of its stage, a unit being one quantisation block (32 columns) of one weight row. ----
        constexpr uint32_t GT = 256 / G;  // threads of a group
        const uint32_t dt = tid - 128, grp = dt / GT, gt = dt % GT;
        constexpr int UN = G * NB;  // units of a thread per stage
        const uint32_t row_bytes = tiled_row_bytes(QT, p.cols), sc_off = tiled_scale_off(QT, p.cols), hi_off = tiled_hi_off(p.cols);
        uint32_t soff[UN], roff[UN];
        const uint8_t *wp[UN];
        const uint8_t *sp[UN];
        const uint8_t *hp[UN];  // q6_0: the unit's two high-bit words (8 bytes per block behind the row's codes)
#pragma unroll
        for (int i = 0; i < UN; ++i) {
            const uint32_t u = gt + i * GT, wr = u & (BNT - 1), blk = u / BNT;
            soff[i] = (wr >> 3) * 1024 + (wr & 7) * 128 + (blk << 16) + ((wr & 7) << 20);  // row offset | block | row & 7
            roff[i] = wr * 32 + blk * 16;                                                   // the unit's codes in the raw tile
            const uint8_t *wbase = (glu && wr >= BN) ? p.w[1] : wmat;
            const uint32_t grow = glu ? n0 + (wr & (BN - 1)) : n0 + wr;
            wp[i] = wbase + (size_t)grow * row_bytes + blk * 16 + (size_t)kbeg * 32;
            sp[i] = wbase + (size_t)grow * row_bytes + sc_off + blk * 2 + (size_t)kbeg * 4;
            hp[i] = wbase + (size_t)grow * row_bytes + hi_off + blk * 8 + (size_t)kbeg * 16;
        }
        uint4 cwq[UN];
        uint2 hwq[UN];
        unsigned short scq[UN];
        if (!RAW) {
            const uint32_t kj = min(grp, nk - 1);
#pragma unroll
            for (int i = 0; i < UN; ++i) {
                cwq[i] = *reinterpret_cast<const uint4 *>(wp[i] + (size_t)kj * 32);
                scq[i] = *reinterpret_cast<const unsigned short *>(sp[i] + (size_t)kj * 4);
                if (QT == BRASA_Q6_0) hwq[i] = *reinterpret_cast<const uint2 *>(hp[i] + (size_t)kj * 16);
            }
        }
        bool ok = true;
        for (uint32_t k = grp; k < nk && ok; k += G) {
            const uint32_t s = k % NS;
            uint4 cw[UN];
            uint2 hw[UN];
            unsigned short sc[UN];
            if (RAW) {
                // A parity wait cannot tell a phase from the one two before it. The copies of stage k - NS (same slot) may land
                // after those of a later stage this group has already converted, and a wait for "stage k has landed" entered
                // before that would then return at once. So first the slot's previous use must be over (its MMAs complete: that
                // wait is never two phases behind because a group's previous stage is less than NS stages back), then the landing.
                if (k >= NS) ok = wait(&empty[s], ((k / NS) - 1) & 1);
                ok = ok && wait(&full_x[s], (k / NS) & 1);
                if (!ok) break;
                const uint8_t *raw = smem + (size_t)s * stage_bytes + MT * A_TILE + NB * B_TILE;
                const uint8_t *rsc = raw + NB * RAW_TILE + ((kbeg + k) & 7) * 4;
#pragma unroll
                for (int i = 0; i < UN; ++i) {
                    cw[i] = *reinterpret_cast<const uint4 *>(raw + roff[i]);
                    sc[i] = *reinterpret_cast<const unsigned short *>(rsc + (roff[i] & ~31u) + ((roff[i] & 16u) >> 3));  // row * 32 + block * 2
                }
            } else {
                const uint32_t kn = min(k + G, nk - 1);  // this group's next stage: in flight during this one
#pragma unroll
                for (int i = 0; i < UN; ++i) {
                    cw[i] = cwq[i];
                    sc[i] = scq[i];
                    cwq[i] = *reinterpret_cast<const uint4 *>(wp[i] + (size_t)kn * 32);
                    scq[i] = *reinterpret_cast<const unsigned short *>(sp[i] + (size_t)kn * 4);
                    if (QT == BRASA_Q6_0) {
                        hw[i] = hwq[i];
                        hwq[i] = *reinterpret_cast<const uint2 *>(hp[i] + (size_t)kn * 16);
                    }
                }
                if (k >= NS) ok = wait(&empty[s], ((k / NS) - 1) & 1);
                if (!ok) break;
            }
            uint8_t *btile = smem + (size_t)s * stage_bytes + MT * A_TILE;
#pragma unroll
            for (int i = 0; i < UN; ++i) {
                const uint32_t r8 = soff[i] >> 20, blk = (soff[i] >> 16) & 1;
                uint8_t *brow = btile + (soff[i] & 0xffffu);
                const __half2 d2 = __half2half2(__ushort_as_half(sc[i]));
                const __half2 bias = __half2half2(__ushort_as_half((unsigned short)(QT == BRASA_Q6_0 ? 0x6420 : 0x6408)));  // 1024 + 32 or + 8
                constexpr uint32_t cmask = QT == BRASA_Q6_0 ? 0x003F003Fu : 0x000F000Fu;
                const uint32_t words[4] = {cw[i].x, cw[i].y, cw[i].z, cw[i].w};
                // elements 0..15 are the low nibbles of bytes 0..15, elements 16..31 the high nibbles
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t wv = words[j] & 0x0F0F0F0Fu, wh = (words[j] >> 4) & 0x0F0F0F0Fu;
                    if (QT == BRASA_Q6_0) {  // bits 4-5 of every code: one shift of the pair's high-bit word per quad of codes
                        const uint32_t h = j < 2 ? hw[i].x : hw[i].y;
                        wv |= ((j & 1) ? (h << 2) : h) & 0x30303030u;
                        wh |= ((j & 1) ? (h << 4) : (h >> 2)) & 0x30303030u;
                    }
                    const uint32_t p01 = __byte_perm(wv, 0, 0x4140), p23 = __byte_perm(wv, 0, 0x4342);  // bytes (0, 1) and (2, 3) into half lanes
                    const uint32_t q01 = __byte_perm(wh, 0, 0x4140), q23 = __byte_perm(wh, 0, 0x4342);
                    lo[2 * j] = deq2(p01, bias, d2, cmask);
                    lo[2 * j + 1] = deq2(p23, bias, d2, cmask);
                    hi[2 * j] = deq2(q01, bias, d2, cmask);
                    hi[2 * j + 1] = deq2(q23, bias, d2, cmask);
                }
                // four 16-byte chunks of the row: columns 8c .. 8c + 7 of this block at chunk (4 blk + c) ^ (row & 7)
                *reinterpret_cast<uint4 *>(brow + (((4 * blk + 0) ^ r8) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(brow + (((4 * blk + 1) ^ r8) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                *reinterpret_cast<uint4 *>(brow + (((4 * blk + 2) ^ r8) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(brow + (((4 * blk + 3) ^ r8) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these writes are read by the tensor core's proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_w[s]);
        }
        // ---- epilogue: lane = token inside a 128-token tile, columns = weight rows ----
        ok = ok && wait(&acc_full, 0);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below need the whole warp
        // with split K the tile goes to this CTA's partial buffer and the last CTA of the tile to arrive adds them up
        const uint32_t tile_elems = MT * BM * BNT, tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        float *ptile = p.ksplit > 1 ? p.part + ((size_t)blockIdx.z * gridDim.x * gridDim.y + tile_id) * tile_elems : nullptr;
        if (ok && glu) {
            // silu(gate) * up, rounded to f16: columns [0, 128) of a token tile's accumulator are gate's, [128, 256) up's.
            // As below, 32 tokens x 32 results are turned around in shared memory: four lanes then store one token's 64 bytes.
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t q = warp & 3;
            const int c_begin = ((warp - 4) >> 2) * (BN / 2);
            uint32_t *tb = reinterpret_cast<uint32_t *>(smem) + (warp - 4) * (32 * 17);  // [32 tokens][16 words + 1]
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll 1
                for (int c = c_begin; c < c_begin + BN / 2; c += 32) {
                    __syncwarp();  // the previous round's reads of tb are done
#pragma unroll 1
                    for (int sub = 0; sub < 2; ++sub) {
                        uint32_t g[16], u[16];
                        const uint32_t taddr = tmem_base + ((q * 32u) << 16) + mt * BNT + c + 16 * sub;
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                            : "=r"(g[0]), "=r"(g[1]), "=r"(g[2]), "=r"(g[3]), "=r"(g[4]), "=r"(g[5]), "=r"(g[6]), "=r"(g[7]), "=r"(g[8]), "=r"(g[9]),
                              "=r"(g[10]), "=r"(g[11]), "=r"(g[12]), "=r"(g[13]), "=r"(g[14]), "=r"(g[15])
                            : "r"(taddr)
                            : "memory");
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                            : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]),
                              "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                            : "r"(taddr + BN)
                            : "memory");
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const float g0 = __uint_as_float(g[i]), g1 = __uint_as_float(g[i + 1]);
                            const float v0 = (g0 / (1.0f + expf(-g0))) * __uint_as_float(u[i]), v1 = (g1 / (1.0f + expf(-g1))) * __uint_as_float(u[i + 1]);
                            const __half2 hh = __floats2half2_rn(v0, v1);
                            tb[lane * 17 + 8 * sub + (i >> 1)] = *reinterpret_cast<const uint32_t *>(&hh);
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t f = lane + 32 * r, trow = f >> 2, q4 = f & 3;  // token of the warp's 32, group of eight results
                        const uint32_t token = tok0 + mt * BM + q * 32 + trow;
                        if (token < p.tokens) {
                            const uint32_t *src = tb + trow * 17 + 4 * q4;
                            *reinterpret_cast<uint4 *>(p.glu + (size_t)token * yrows + n0 + c + 8 * q4) = make_uint4(src[0], src[1], src[2], src[3]);
                        }
                    }
                }
            }
        } else if (ok) {
            // A lane of tensor memory is a token, so a thread holds one token's values and a warp's store would touch 32
            // rows of Y at once (32 cache lines per instruction). Each warp therefore turns 32 tokens x 32 columns around in
            // a private piece of shared memory (the stage ring is idle by now: every MMA has completed) and stores with eight
            // lanes per token: four full 128-byte lines per instruction. The residual is read the same way.
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t q = warp & 3;           // the lane quarter of tensor memory this warp may read
            const int c_begin = ((warp - 4) >> 2) * (BNT / 2);  // two warps per quarter: half of the columns each
            float *tb = reinterpret_cast<float *>(smem) + (warp - 4) * (32 * 33);  // [32 tokens][32 columns + 1]
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll 1
                for (int c = c_begin; c < c_begin + (int)BNT / 2; c += 32) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem_base + ((q * 32u) << 16) + mt * BNT + c;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    __syncwarp();  // the previous round's reads of tb are done
#pragma unroll
                    for (int i = 0; i < 32; ++i) tb[lane * 33 + i] = __uint_as_float(v[i]);
                    __syncwarp();
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const uint32_t f = lane + 32 * r, trow = f >> 3, c4 = f & 7;  // token of the warp's 32, group of four columns
                        const uint32_t tl = mt * BM + q * 32 + trow, token = tok0 + tl;
                        if (token < p.tokens) {
                            const float *src = tb + trow * 33 + 4 * c4;
                            float4 o = make_float4(src[0], src[1], src[2], src[3]);
                            if (ptile) {
                                *reinterpret_cast<float4 *>(ptile + (size_t)tl * BNT + c + 4 * c4) = o;
                            } else {
                                const size_t at = (size_t)token * yrows + n0 + c + 4 * c4;
                                if (p.resid) {
                                    const float4 rr = *reinterpret_cast<const float4 *>(p.resid + at);
                                    o = make_float4(rr.x + o.x, rr.y + o.y, rr.z + o.z, rr.w + o.w);
                                }
                                *reinterpret_cast<float4 *>(ymat + at) = o;
                            }
                        }
                    }
                }
            }
        }
        if (p.ksplit > 1) {
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps
            if (tid == 128) last_s = (*abort_flag == 0 && atomicAdd(&p.counters[tile_id], 1u) == p.ksplit - 1) ? 1u : 0u;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (last_s) {
                __threadfence();
                const float *p0 = p.part + (size_t)tile_id * tile_elems;
                const size_t zstride = (size_t)gridDim.x * gridDim.y * tile_elems;
                // rows of the tile past the last token were never written: stop there
                const uint32_t live = min((uint32_t)(MT * BM), p.tokens > tok0 ? p.tokens - tok0 : 0u) * (BNT / 4);
#pragma unroll 1
                for (uint32_t i0 = tid - 128; i0 < live; i0 += 4 * 256) {
                    float4 a[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t i = i0 + u * 256;
                        a[u] = i < live ? __ldcg(reinterpret_cast<const float4 *>(p0) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    for (uint32_t z = 1; z < p.ksplit; ++z) {  // always in the order of the K ranges, whoever arrives last
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t i = i0 + u * 256;
                            if (i < live) {
                                const float4 b = __ldcg(reinterpret_cast<const float4 *>(p0 + z * zstride) + i);
                                a[u].x += b.x; a[u].y += b.y; a[u].z += b.z; a[u].w += b.w;
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t i = i0 + u * 256;
                        if (i < live) {
                            const size_t at = (size_t)(tok0 + (i * 4) / BNT) * yrows + n0 + (i * 4) % BNT;
                            if (p.resid) {
                                const float4 r = *reinterpret_cast<const float4 *>(p.resid + at);
                                a[u] = make_float4(r.x + a[u].x, r.y + a[u].y, r.z + a[u].z, r.w + a[u].w);
                            }
                            *reinterpret_cast<float4 *>(ymat + at) = a[u];
                        }
                    }
                }
                if (tid == 128) p.counters[tile_id] = 0;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ncols = MT * BNT;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return (EncodeTiledFn)f;
    }();
    return fn;
}

}  // namespace

// True when the tensor-core kernel takes this product (the caller falls back to the warp-MMA kernel otherwise).
bool brasa_gemm_tc_supported(const brasa_qmatrix &w, uint32_t tokens) {
    return (w.qtype == BRASA_Q4_0 || w.qtype == BRASA_Q6_0) && w.layout == BRASA_LAYOUT_TILED && w.rows % BN == 0 && w.cols % BK == 0 && w.cols >= BK && tokens > 0 &&
           encode_tiled() != nullptr;
}

// Y_i = W_i X for 1 to 3 matrices that share X (f16, [tokens][cols]); every W_i must pass brasa_gemm_tc_supported.
// resid (optional, one matrix): Y = resid + W X (same shape as Y; may be Y itself).
// glu (optional, two matrices gate and up of equal shape, rows a multiple of 128): out = f16(silu(W_gate X) * (W_up X)), [tokens][rows];
// ys is not written then.
int32_t brasa_gemm_tc_launch(brasa_cmd *cmd, uint32_t count, const brasa_qmatrix *ws, const __half *x, float *const *ys, uint32_t tokens,
                             const float *resid, __half *glu) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, count >= 1 && count <= 3, "gemm: 1 to 3 matrices");
    BRASA_REQUIRE(ctx, !glu || (count == 2 && ws[0].rows == ws[1].rows && !resid && (reinterpret_cast<uintptr_t>(glu) & 15) == 0),
                  "gemm: the fused SwiGLU takes gate and up of equal shape");
    BRASA_REQUIRE(ctx, !resid || (count == 1 && (reinterpret_cast<uintptr_t>(resid) & 15) == 0), "gemm: a residual goes with one matrix and must be 16-byte aligned");
    GemmTcParams p{};
    p.resid = resid;
    p.glu = glu;
    bool rows256 = true;
    uint32_t tiles128 = 0;
    for (uint32_t i = 0; i < count; ++i) {
        BRASA_REQUIRE(ctx, brasa_gemm_tc_supported(ws[i], tokens) && ws[i].cols == ws[0].cols, "gemm: shape not taken by the tensor-core kernel");
        BRASA_REQUIRE(ctx, glu || (reinterpret_cast<uintptr_t>(ys[i]) & 15) == 0, "gemm: misaligned y");
        rows256 = rows256 && ws[i].rows % 256 == 0;
        tiles128 += ws[i].rows / BN;
    }
    // Shape of a CTA: MT token tiles of 128 x NB weight tiles of 128 rows (MT x NB x 128 accumulator columns <= 512).
    // Every CTA reads its token tiles' X once per launch, so X crosses L2 -> SM (weight tiles / NB) times: the
    // estimate is the larger of that traffic at about 4.5 TB/s and waves x stages x cycles per stage of one CTA.
    // When the output tiles are too few for the SMs (few tokens: a decode step of a batch; narrow matrices), the K
    // stages of a tile are shared by `ksplit` CTAs (grid z) that each write a partial tile; the last to arrive adds
    // them in K order. A split keeps at least 8 stages.
    const uint32_t ntile = (tokens + BM - 1) / BM, nkst = ws[0].cols / BK;
    uint32_t mt = 1, nb = 1, ksplit = 1;
    double best = 1e30;
    for (uint32_t b = 1; b <= (rows256 ? 2u : 1u); ++b) {
        for (uint32_t c = 1; c * b <= 4 && c <= std::max(1u, ntile); c *= 2) {
            const uint32_t ctas = (tiles128 / b) * ((ntile + c - 1) / c);
            uint32_t ks = 1;
            if (c * b <= 2 && ctas * 2 <= (uint32_t)ctx->sm_count && ctas <= GEMM_TC_COUNTERS)
                ks = std::max(1u, std::min((uint32_t)ctx->sm_count / ctas, nkst / 8));
            const double waves = std::ceil((double)ctas * ks / ctx->sm_count);
            const double pipe = waves * ((nkst + ks - 1) / ks) * (300.0 * c * b + 400.0) + (ks > 1 ? 4000.0 + 3000.0 * ks * c * b : 0.0);  // + the last CTA's sum over ks partial tiles
            const double xbytes = (double)ctas * c * BM * ws[0].cols * 2.0;
            const double cost = std::max(pipe, xbytes * 1.965e9 / 4.5e12);
            if (cost < best * 0.999 || (cost < best * 1.001 && c * b > mt * nb)) {
                best = cost;
                mt = c;
                nb = b;
                ksplit = ks;
            }
        }
    }
    const bool q6 = ws[0].qtype == BRASA_Q6_0;
    for (uint32_t i = 0; i < count; ++i) BRASA_REQUIRE(ctx, (ws[i].qtype == BRASA_Q6_0) == q6, "gemm: q4_0 and q6_0 matrices cannot share a launch");
    BRASA_REQUIRE(ctx, !q6 || (count == 1 && !glu), "gemm: a q6_0 matrix goes alone");
    if (q6) {  // one token tile, 128 rows, direct loads: the shape the q6_0 conversion is built for
        mt = 1;
        nb = 1;
    }
    if (glu) {  // 128 rows of gate and the same 128 rows of up per CTA: the 256-row shape, one or two token tiles
        nb = 2;
        mt = ntile >= 2 ? 2 : 1;
        ksplit = 1;
    }
    uint32_t ncta_n = 0;
    for (uint32_t i = 0; i < 3; ++i) {
        if (i < count) {
            p.w[i] = arg_ptr(ws[i].data);
            p.y[i] = ys ? ys[i] : nullptr;
            p.rows[i] = ws[i].rows;
            ncta_n += ws[i].rows / (BN * nb);
        }
        p.tile_end[i] = ncta_n;
    }
    if (glu) ncta_n = ws[0].rows / BN;
    const brasa_qmatrix &w = ws[0];
    BRASA_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x) & 15) == 0, "gemm: misaligned x");
    // X as a 2-D tensor [tokens][cols] of f16; a box is 64 columns x 128 tokens, 128-byte swizzle, zeros past the end
    CUtensorMap tmap;
    cuuint64_t dims[2] = {w.cols, tokens}, strides[1] = {(cuuint64_t)w.cols * 2};
    cuuint32_t box[2] = {BK, BM}, estr[2] = {1, 1};
    CUresult cr = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return brasa_fail(ctx, BRASA_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)cr);

    // the weight matrices as byte tensors [rows][row_bytes]: box = 32 bytes x this CTA's rows, no swizzle
    const bool raw = mt == 1 && nb == 1 && !q6;  // weight bytes through TMA when one token tile per CTA leaves the weights as the main traffic
    WeightMaps wmaps;
    memset(&wmaps, 0, sizeof wmaps);
    for (uint32_t i = 0; raw && i < 3; ++i) {
        const brasa_qmatrix &wi = ws[i < count ? i : 0];
        const uint32_t rb = tiled_row_bytes(BRASA_Q4_0, wi.cols);
        cuuint64_t wdims[2] = {rb, wi.rows}, wstrides[1] = {rb};
        cuuint32_t wbox[2] = {32, BN * nb}, westr[2] = {1, 1};
        BRASA_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(arg_ptr(wi.data)) & 15) == 0, "gemm: misaligned weights");
        CUresult wr = encode_tiled()(&wmaps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, arg_ptr(wi.data), wdims, wstrides, wbox, westr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (wr != CUDA_SUCCESS) return brasa_fail(ctx, BRASA_ECUDA, "cuTensorMapEncodeTiled failed for the weights (%d)", (int)wr);
    }
    const uint32_t stage_bytes = mt * A_TILE + nb * B_TILE + (raw ? nb * 2 * RAW_TILE : 0);
    uint32_t stages = (uint32_t)std::min<size_t>(8, (ctx->smem_optin - 4096) / stage_bytes);
    stages = std::min<uint32_t>(stages, std::max<uint32_t>(2, (w.cols / BK + ksplit - 1) / ksplit));
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    p.cols = w.cols;
    p.tokens = tokens;
    p.stages = stages;
    p.status = ctx->status;
    p.ksplit = ksplit;
    dim3 grid(ncta_n, (ntile + mt - 1) / mt, ksplit);
    if (ksplit > 1) {
        const size_t need = (size_t)ksplit * grid.x * grid.y * mt * BM * nb * BN * sizeof(float);
        if (ctx->gemm_part_bytes < need) {
            BRASA_REQUIRE(ctx, !ctx->capturing, "gemm: the split-K workspace cannot grow while a graph is recorded");
            BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            if (ctx->gemm_part) cudaFree(ctx->gemm_part);
            ctx->gemm_part = nullptr;
            ctx->gemm_part_bytes = 0;
            BRASA_CUDA(ctx, cudaMalloc((void **)&ctx->gemm_part, need));
            ctx->gemm_part_bytes = need;
        }
        if (!ctx->gemm_counters) {
            BRASA_REQUIRE(ctx, !ctx->capturing, "gemm: the split-K counters cannot be created while a graph is recorded");
            BRASA_CUDA(ctx, cudaMalloc((void **)&ctx->gemm_counters, GEMM_TC_COUNTERS * 4));
            BRASA_CUDA(ctx, cudaMemset(ctx->gemm_counters, 0, GEMM_TC_COUNTERS * 4));
        }
        p.part = ctx->gemm_part;
        p.counters = ctx->gemm_counters;
    }
    // programmatic dependent launch: the kernel's set-up overlaps the end of the kernel before it (see griddepcontrol.wait)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(384);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define LAUNCH_TC(MTV, GV, NBV, RAWV)                                                                                                        \
    do {                                                                                                                         \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)gemm_tc_kernel<MTV, GV, NBV, RAWV>, ctx->smem_optin - 2048)); \
        BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_kernel<MTV, GV, NBV, RAWV>, tmap, wmaps, p));                                                  \
    } while (0)
    // conversion groups: as many stages in flight as the ring holds, at most four
    if (q6) {
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)gemm_tc_kernel<1, 4, 1, false, BRASA_Q6_0>, ctx->smem_optin - 2048));
        BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_kernel<1, 4, 1, false, BRASA_Q6_0>, tmap, wmaps, p));
    } else if (nb == 1 && mt == 1) LAUNCH_TC(1, 4, 1, true);
    else if (nb == 1 && mt == 2) LAUNCH_TC(2, 4, 1, false);
    else if (nb == 1) LAUNCH_TC(4, 2, 1, false);
    else if (mt == 1) LAUNCH_TC(1, 2, 2, false);
    else LAUNCH_TC(2, 2, 2, false);
#undef LAUNCH_TC
    return brasa_post_launch(cmd, "gemm_tc");
}
