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
// the same test without the suspension try_wait may make: what a role does first when the phase is most likely over
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// true in one lane of the (converged) warp: the form under which the compiler keeps the issuing code on the uniform path
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
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

// ---- few tokens (a decode step of a batch, a short prompt): the weights are the M operand, the tokens N ----------------
// With at most 64 tokens a step is nothing but the weight stream, and what decides its rate is how many weight bytes an
// SM keeps in flight and how cheaply they reach the tensor core. So the kernel is persistent and:
//   * raw weights travel in chunks of four K stages: one box of 128 rows x 128 code bytes (whole cache lines, 128-byte
//     swizzle so that the conversion's 16-byte reads of eight rows fall on eight bank groups) and one of 128 rows x 16
//     scale bytes, into a ring of `raw_slots` chunks (warp 0, one lane) that runs ahead of everything else;
//   * tcgen05.mma takes the weights as A (M = 128 rows) out of TENSOR memory and X as B (N = 64 tokens) out of shared
//     memory. A lane of tensor memory is a weight row, so a conversion thread (warps 4-11: warp & 3 picks the 32 rows,
//     the other bit the quantisation block of the stage) turns the 32 codes of its row into 16 registers of f16 pairs
//     and stores them with one tcgen05.st: no write of a 16 KB tile to shared memory, no proxy fence. Three chunks
//     of A (four stages of 32 columns each) and the accumulator (64 columns) live in tensor memory;
//   * everything behind the raw ring moves a chunk at a time (one wait per role and chunk, one commit): a role's loop is
//     one lane's chain of dependent instructions, and a stage of 4.6 KB of weights must not cost it hundreds of cycles;
//   * the ring in shared memory behind the raw one holds only X (64 tokens x 64 halves per stage by TMA: warp 2, one lane);
//   * the accumulator's lanes are weight rows: the epilogue's stores are 128-byte lines of Y, no turn through shared memory.
// Work is cut evenly: the launch's (row tile, K stage) pairs, in that order, are split into gridDim.x equal runs. A run
// that covers a tile's whole K range stores Y; any other writes a partial tile, and a second small kernel, launched as
// this one's dependent, adds each shared tile's partial tiles in K order and the residual (every SM takes part; one block
// doing it as the last to arrive took longer than the products themselves).
constexpr uint32_t SK_TT = 64, SK_X_TILE = SK_TT * BK * 2;  // 8 KB of X per stage
constexpr uint32_t SK_NCS = 3, SK_X_CHUNK = 4 * SK_X_TILE;  // ring of three chunks (four stages each): 32 KB of X per slot
constexpr uint32_t SK_ACOL = 128, SK_TMEM = 512;  // A in tensor memory: 128 columns per chunk slot from column 128; accumulator at column 0
constexpr uint32_t SK_CODES = BN * 128, SK_RAW = SK_CODES + BN * 16;                     // 16 KB of codes + 2 KB of scales per four stages

struct SkinnyMaps {
    CUtensorMap codes[3], scales[3];
};

struct SkinnyParams {
    float *y[3];
    uint32_t rows[3];
    uint32_t tile_end[3];  // 128-row tiles of matrices 0..i, cumulative
    uint32_t cols, tokens, raw_slots;
    uint32_t units;      // row tiles x K stages of the launch
    uint32_t max_parts;  // most blocks that share one tile
    uint32_t *status;
    const float *resid;
    float *part;         // [tile][max_parts][64 tokens][128 rows]: what the blocks that share a tile leave for the kernel below
    __half *glu;         // when set (two matrices, gate then up): every tile goes to `part` and the kernel below writes f16(silu(gate) * up) here
    uint32_t defer;      // every tile goes to `part`: the kernel that follows forms Y (and more) from the partial tiles
    unsigned long long *trace;  // a developer's build only: phase time stamps
};

#ifdef BRASA_TRACE_BUILD
#define SKT(idx) do { if (p.trace && blockIdx.x == 0) p.trace[idx] = (unsigned long long)clock64(); } while (0)
#define SKG(j) do { if (p.trace) p.trace[512 + blockIdx.x * 4 + (j)] = gtime(); } while (0)
#else
#define SKT(idx) do { } while (0)
#define SKG(j) do { } while (0)
#endif

// The block whose run holds unit u when `units` units are cut into `blocks` runs [b units / blocks, (b + 1) units / blocks).
// (units x blocks stays below 2^32: the launcher sees to it, and the kernels divide 32-bit numbers)
BRASA_HD static inline uint32_t skinny_owner(uint32_t u, uint32_t units, uint32_t blocks) {
    uint32_t c = u * blocks / units;
    while ((c + 1) * units / blocks <= u) ++c;
    while (c * units / blocks > u) --c;
    return c;
}

__global__ void __launch_bounds__(384, 1) gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ SkinnyMaps maps,
                                                                SkinnyParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_x[SK_NCS], full_a[SK_NCS], empty[SK_NCS], raw_full[8], raw_empty[8], acc_full, acc_empty;
    __shared__ uint32_t tmem_base_s, abort_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t RC = p.raw_slots, nkst = p.cols / BK, cpt = (nkst + 3) / 4, P = gridDim.x;
    const uint32_t u_beg = blockIdx.x * p.units / P, u_end = (blockIdx.x + 1) * p.units / P;  // (units x blocks < 2^32)
    const uint32_t nu = u_end - u_beg;  // this block's run of (tile, K stage) units
    auto chunk_of = [&](uint32_t u) { return (u / nkst) * cpt + ((u % nkst) >> 2); };
    const uint32_t g0 = nu ? chunk_of(u_beg) : 0u, nc = nu ? chunk_of(u_end - 1) - g0 + 1 : 0u;  // its chunks
    const uint32_t k_beg = nu ? u_beg % nkst : 0u;
    uint8_t *raw_base = smem + (size_t)SK_NCS * SK_X_CHUNK;
    auto tile_matrix = [&](uint32_t t) { return (uint32_t)(t >= p.tile_end[0]) + (uint32_t)(t >= p.tile_end[1]); };
    auto tile_row0 = [&](uint32_t t, uint32_t mi) { return (t - (mi == 0 ? 0u : (mi == 1 ? p.tile_end[0] : p.tile_end[1]))) * BN; };
    // Every role walks the run chunk by chunk with the same three numbers: k, the chunk's first stage in its tile; n, how
    // many of the chunk's stages belong to the run (the run may begin or end inside a chunk; a tile's end ends one); left,
    // the stages of the run not yet handed out. No division per chunk: a role's loop is mostly one lane's dependent chain.
    auto chunk_len = [&](uint32_t k, uint32_t left) { return min(min(4u - (k & 3u), nkst - k), left); };

    if (tid == 0) {
        SKT(400);
        SKG(0);
        for (uint32_t s = 0; s < SK_NCS; ++s) {
            mbar_init(&full_x[s], 1);
            mbar_init(&full_a[s], 8);  // one arrival per conversion warp
            mbar_init(&empty[s], 1);
        }
        for (uint32_t s = 0; s < 8; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], 8);  // one arrival per conversion warp
        }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, 8);  // one arrival per epilogue warp
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        uint32_t ncols = SK_TMEM;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    auto issue_chunk = [&](uint32_t ci) {  // codes and scales of the run's chunk ci
        const uint32_t gch = g0 + ci, t = gch / cpt, kc = gch % cpt, mi = tile_matrix(t), n0 = tile_row0(t, mi), r = ci % RC;
        uint8_t *dst = raw_base + (size_t)r * SK_RAW;
        mbar_expect_tx(&raw_full[r], SK_RAW);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                     "l"(&maps.codes[mi]), "r"((int)(kc * 128)), "r"((int)n0), "r"(smem_u32(&raw_full[r]))
                     : "memory");
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                         smem_u32(dst + SK_CODES)),
                     "l"(&maps.scales[mi]), "r"((int)(tiled_scale_off(BRASA_Q4_0, p.cols) + kc * 16)), "r"((int)n0), "r"(smem_u32(&raw_full[r]))
                     : "memory");
    };
    // Launched as a programmatic dependent: the set-up above and the first chunks of weights (weights never change) overlap
    // the end of the kernel before this one; what that kernel wrote (X, the residual, the workspace) is read after the wait.
    const uint32_t early = min(RC, nc);
    if (tid == 0) {
        for (uint32_t ci = 0; ci < early; ++ci) issue_chunk(ci);
    }
    if (tid == 0) SKT(401);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        SKT(402);
        SKG(1);
    }
    const uint32_t tmem_base = tmem_base_s;
    volatile uint32_t *abort_flag = &abort_s;
    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {  // bounded; false when it gave up (or another role did)
        if (mbar_test(bar, parity)) return true;
        for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
            if (mbar_try(bar, parity)) return true;
            if (*abort_flag) return false;
        }
        atomicExch(p.status, 4u);
        *abort_flag = 1;
        return false;
    };

    if (warp == 0) {
        if (lane == 0) {  // ---- raw weight chunks ----
            uint32_t issued = early;
            for (uint32_t ci = early; ci < nc; ++ci) {
                if (!wait(&raw_empty[ci % RC], ((ci / RC) - 1) & 1)) break;  // (ci >= RC here: the first RC chunks went out above)
                issue_chunk(ci);
                issued = ci + 1;
            }
            if (*abort_flag) {  // leaving early: let the copies in flight land before the block exits
                for (uint32_t ci = issued > RC ? issued - RC : 0; ci < issued; ++ci)
                    for (uint32_t it = 0; it < TC_WAIT_LIMIT && !mbar_try(&raw_full[ci % RC], (ci / RC) & 1); ++it) {}
            }
        }
    } else if (warp == 2) {
        if (lane == 0) {  // ---- X tiles: the chunk's stages, 64 tokens x 64 halves each, on one barrier ----
            uint32_t issued = 0, k = k_beg, left = nu, cs = 0, ph = 0;
            for (uint32_t c = 0; c < nc; ++c) {
                const uint32_t n = chunk_len(k, left);
                if (c >= SK_NCS && !wait(&empty[cs], ph ^ 1)) break;
                if (c < 48) SKT(16 + c * 8 + 0);
                mbar_expect_tx(&full_x[cs], n * SK_X_TILE);
                for (uint32_t j = 0; j < n; ++j) {
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                                     smem_u32(smem + (size_t)cs * SK_X_CHUNK + (size_t)((k + j) & 3) * SK_X_TILE)),
                                 "l"(&tmap_x), "r"((int)((k + j) * BK)), "r"(0), "r"(smem_u32(&full_x[cs]))
                                 : "memory");
                }
                issued = c + 1;
                left -= n;
                k = k + n == nkst ? 0 : k + n;
                cs = cs + 1 == SK_NCS ? 0 : cs + 1;
                ph ^= (cs == 0);
            }
            if (*abort_flag) {
                for (uint32_t c = issued > SK_NCS ? issued - SK_NCS : 0; c < issued; ++c)
                    for (uint32_t w = 0; w < TC_WAIT_LIMIT && !mbar_try(&full_x[c % SK_NCS], (c / SK_NCS) & 1); ++w) {}
            }
        }
    } else if (warp == 1) {
        // ---- tensor core. The whole warp walks the chunks and waits; one lane issues. A chunk costs the issuing lane two
        // waits, up to sixteen products (operand addresses are constants of the unrolled slots) and one commit. ----
        // instruction descriptor: D f32, A and B f16, both K-major, M = 128 weight rows, N = 64 tokens
        const uint32_t idesc = (1u << 4) | ((uint32_t)(SK_TT >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
        const uint64_t db_slot0 = smem_desc(smem_u32(smem));
        uint32_t seg = 0, k = k_beg, left = nu, ph = 0;  // seg: runs of one tile finished so far
        bool first = true, ok = true;
        for (uint32_t c0 = 0; c0 < nc && ok; c0 += SK_NCS, ph ^= 1) {
#pragma unroll
            for (uint32_t cs = 0; cs < SK_NCS; ++cs) {
                if (c0 + cs >= nc) break;
                const uint32_t n = chunk_len(k, left), kq0 = k & 3;
                const bool last = k + n == nkst || n == left;
                if (first && seg > 0) ok = wait(&acc_empty, (seg - 1) & 1);  // the epilogue has read the tile before this one
                ok = ok && wait(&full_x[cs], ph) && wait(&full_a[cs], ph);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (elect_one()) {
                    if (c0 + cs < 48) SKT(16 + (c0 + cs) * 8 + 2);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        if (j >= kq0 && j < kq0 + n) {
                            const uint64_t db = db_slot0 + (uint64_t)((cs * SK_X_CHUNK + j * SK_X_TILE) >> 4);
                            const uint32_t a0 = tmem_base + SK_ACOL + 128 * cs + 32 * j;
#pragma unroll
                            for (int ks = 0; ks < BK / 16; ++ks) {  // A: 16 halves of K = 8 columns of tensor memory; B: 32 bytes further along K
                                const uint32_t acc = (!first || j > kq0 || ks > 0) ? 1u : 0u;
                                asm volatile(
                                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                    "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                                    ::"r"(tmem_base), "r"(a0 + ks * 8), "l"(db + (uint64_t)(ks * 2)), "r"(idesc), "r"(acc)
                                    : "memory");
                            }
                        }
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[cs])) : "memory");
                    if (last) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&acc_full)) : "memory");
                    if (c0 + cs < 48) SKT(16 + (c0 + cs) * 8 + 3);
                }
                __syncwarp();
                seg += last;
                first = last;
                left -= n;
                k = k + n == nkst ? 0 : k + n;
            }
        }
    } else if (warp >= 4) {
        // ---- weights, then each finished tile's epilogue. Every chunk is converted by all eight warps: a thread owns one
        // quantisation block (32 columns) of one weight row, the row its lane of tensor memory stands for, in each stage. ----
        const uint32_t q = warp & 3, th = (warp - 4) >> 2;  // lane quarter of tensor memory (weight rows 32 q ..); block of the stage, half of the tokens
        const uint32_t wr = 32 * q + lane, r8 = wr & 7;
        const uint32_t coff = wr * 128, soff = SK_CODES + wr * 16 + th * 2;  // the row's codes and its scale in a raw chunk
        const uint32_t a_lane = tmem_base + ((q * 32u) << 16) + SK_ACOL + 16 * th;
        bool ok = true;
        uint32_t seg = 0, left = nu, k = k_beg, c = 0, cs = 0, ph = 0, rslot = 0, rph = 0;  // (slots and phases are carried along)
        uint32_t t = nu ? u_beg / nkst : 0u;
        while (left > 0) {
            const uint32_t k0 = k;  // this tile's run: stages [k0, k0 + seg_len)
            const uint32_t seg_len = min(nkst - k0, left);
            uint32_t seg_left = seg_len;
            while (seg_left > 0 && ok) {
                // the stages of one raw chunk together: their loads, conversions and stores overlap, one wait covers the stores
                const uint32_t n = chunk_len(k, seg_left), kq0 = k & 3;
                if (tid == 128 && c < 48) SKT(16 + c * 8 + 4);
                // (a slot is refilled only after every warp has arrived for its previous use: no parity wait can be a whole phase behind)
                ok = wait(&raw_full[rslot], rph);
                if (c >= SK_NCS) ok = ok && wait(&empty[cs], ph ^ 1);
                if (tid == 128 && c < 48) SKT(16 + c * 8 + 6);
                ok = __all_sync(0xffffffffu, ok);  // the tensor-memory stores need the whole warp
                if (!ok) break;
                const uint8_t *raw = raw_base + (size_t)rslot * SK_RAW;
                const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6408));  // 1024 + 8
                uint4 cws[4];  // (all the loads first: a tensor-memory store orders what follows it behind it)
                unsigned short scs[4];
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    cws[j] = *reinterpret_cast<const uint4 *>(raw + coff + (((2 * j + th) ^ r8) << 4));
                    scs[j] = *reinterpret_cast<const unsigned short *>(raw + soff + j * 4);
                }
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    if (j >= kq0 && j < kq0 + n) {
                        const uint4 cw = cws[j];
                        const __half2 d2 = __half2half2(__ushort_as_half(scs[j]));
                        const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
                        uint32_t e[16];  // pairs of consecutive columns: elements 0..15 are the low nibbles of bytes 0..15, 16..31 the high nibbles
#pragma unroll
                        for (int w4 = 0; w4 < 4; ++w4) {
                            const uint32_t wv = words[w4] & 0x0F0F0F0Fu, wh = (words[w4] >> 4) & 0x0F0F0F0Fu;
                            // one byte permutation puts two codes under the 0x64 bytes of two halves: 1024 + q each
                            e[2 * w4] = h22u(__hmul2(__hsub2(u2h2(__byte_perm(wv, 0x64646464u, 0x4140)), bias), d2));
                            e[2 * w4 + 1] = h22u(__hmul2(__hsub2(u2h2(__byte_perm(wv, 0x64646464u, 0x4342)), bias), d2));
                            e[8 + 2 * w4] = h22u(__hmul2(__hsub2(u2h2(__byte_perm(wh, 0x64646464u, 0x4140)), bias), d2));
                            e[8 + 2 * w4 + 1] = h22u(__hmul2(__hsub2(u2h2(__byte_perm(wh, 0x64646464u, 0x4342)), bias), d2));
                        }
                        asm volatile(
                            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(
                                a_lane + 128 * cs + 32 * j),
                            "r"(e[0]), "r"(e[1]), "r"(e[2]), "r"(e[3]), "r"(e[4]), "r"(e[5]), "r"(e[6]), "r"(e[7]), "r"(e[8]), "r"(e[9]), "r"(e[10]),
                            "r"(e[11]), "r"(e[12]), "r"(e[13]), "r"(e[14]), "r"(e[15])
                            : "memory");
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full_a[cs]);
                    mbar_arrive(&raw_empty[rslot]);  // this warp has read what it needs of the chunk
                }
                if (tid == 128 && c < 48) SKT(16 + c * 8 + 7);
                seg_left -= n;
                k += n;
                ++c;
                cs = cs + 1 == SK_NCS ? 0 : cs + 1;
                ph ^= (cs == 0);
                rslot = rslot + 1 == RC ? 0 : rslot + 1;
                rph ^= (rslot == 0);
            }
            // ---- this tile's run is converted: read its accumulator (lane = weight row, column = token) ----
            const uint32_t mi = tile_matrix(t), n0 = tile_row0(t, mi), yrows = mi == 0 ? p.rows[0] : (mi == 1 ? p.rows[1] : p.rows[2]);
            float *ymat = mi == 0 ? p.y[0] : (mi == 1 ? p.y[1] : p.y[2]);
            const bool whole = k0 == 0 && seg_len == nkst && !p.defer;  // otherwise other blocks hold the rest of this tile's K range (or gate meets up below)
            if (tid == 128 && seg < 4) SKT(410 + seg * 8 + 0);
            if (tid == 128 && seg == 0) SKG(2);
            ok = ok && wait(&acc_full, seg & 1);
            ok = __all_sync(0xffffffffu, ok);  // the tensor-memory load needs the whole warp
            if (tid == 128 && seg < 4) SKT(410 + seg * 8 + 1);
            uint32_t v[32];
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + 32 * th;
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
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty);  // the next tile's products may overwrite the accumulator
                const uint32_t row = 32 * q + lane;
                if (whole) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t token = 32 * th + i;
                        if (token < p.tokens) {
                            const size_t at = (size_t)token * yrows + n0 + row;
                            float o = __uint_as_float(v[i]);
                            if (p.resid) o = p.resid[at] + o;
                            ymat[at] = o;
                        }
                    }
                } else {
                    const uint32_t z = k0 == 0 ? 0u : blockIdx.x - skinny_owner(t * nkst, p.units, P);  // (a tile begun here is this block's from its first stage)
                    float *ptile = p.part + ((size_t)t * p.max_parts + z) * (SK_TT * BN);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t token = 32 * th + i;
                        if (token < p.tokens) ptile[token * BN + row] = __uint_as_float(v[i]);
                    }
                }
            }
            if (tid == 128 && seg < 4) SKT(410 + seg * 8 + 2);
            left -= seg_len;
            ++seg;
            ++t;  // (a run goes on only into the next tile, from its first stage)
            k = 0;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        SKT(403);
        SKG(3);
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ncols = SK_TMEM;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
    }
}

// Y = resid + the partial tiles in K order, for every tile that more than one block of the kernel above worked on.
// Launched as its dependent: its blocks sit beside the GEMM's and start the moment the last partial tile is out, and
// every SM takes part (one float4 of Y per thread, all of its partial tiles' loads in flight at once).
__device__ __forceinline__ float4 skinny_tile_sum(const SkinnyParams &p, uint32_t t, uint32_t parts, uint32_t i) {
    const float *p0 = p.part + (size_t)t * p.max_parts * (SK_TT * BN);
    float4 a = __ldcg(reinterpret_cast<const float4 *>(p0) + i);
    for (uint32_t z0 = 1; z0 < parts; z0 += 8) {  // always in the order of the K ranges
        float4 b[8];
#pragma unroll
        for (int dz = 0; dz < 8; ++dz)
            b[dz] = z0 + dz < parts ? __ldcg(reinterpret_cast<const float4 *>(p0 + (size_t)(z0 + dz) * (SK_TT * BN)) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int dz = 0; dz < 8; ++dz) {
            if (z0 + dz < parts) {
                a.x += b[dz].x; a.y += b[dz].y; a.z += b[dz].z; a.w += b[dz].w;
            }
        }
    }
    return a;
}

__global__ void __launch_bounds__(256) gemm_tc_skinny_sum_kernel(SkinnyParams p, uint32_t blocks) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t t = blockIdx.x, nkst = p.cols / BK;
    const uint32_t parts = skinny_owner(t * nkst + nkst - 1, p.units, blocks) - skinny_owner(t * nkst, p.units, blocks) + 1;
    const uint32_t live = min(SK_TT, p.tokens) * (BN / 4);  // float4s of the tile that hold tokens
    if (p.glu) {  // tile t of gate and tile t of up: out = f16(silu(gate) * up), four rows of a token per thread
        const uint32_t tu = t + p.tile_end[0];
        const uint32_t parts_u = skinny_owner(tu * nkst + nkst - 1, p.units, blocks) - skinny_owner(tu * nkst, p.units, blocks) + 1;
        for (uint32_t i = blockIdx.y * 256 + threadIdx.x; i < live; i += gridDim.y * 256) {
            const float4 g = skinny_tile_sum(p, t, parts, i), u = skinny_tile_sum(p, tu, parts_u, i);
            const __half2 lo = __floats2half2_rn((g.x / (1.0f + expf(-g.x))) * u.x, (g.y / (1.0f + expf(-g.y))) * u.y);
            const __half2 hi = __floats2half2_rn((g.z / (1.0f + expf(-g.z))) * u.z, (g.w / (1.0f + expf(-g.w))) * u.w);
            const size_t at = (size_t)(i / (BN / 4)) * p.rows[0] + t * BN + (i % (BN / 4)) * 4;
            *reinterpret_cast<uint2 *>(p.glu + at) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
        }
        return;
    }
    if (parts == 1) return;  // one block held the tile's whole K range and stored Y itself
    const uint32_t mi = (uint32_t)(t >= p.tile_end[0]) + (uint32_t)(t >= p.tile_end[1]);
    const uint32_t n0 = (t - (mi == 0 ? 0u : (mi == 1 ? p.tile_end[0] : p.tile_end[1]))) * BN, yrows = mi == 0 ? p.rows[0] : (mi == 1 ? p.rows[1] : p.rows[2]);
    float *ymat = mi == 0 ? p.y[0] : (mi == 1 ? p.y[1] : p.y[2]);
    for (uint32_t i = blockIdx.y * 256 + threadIdx.x; i < live; i += gridDim.y * 256) {
        float4 a = skinny_tile_sum(p, t, parts, i);
        const size_t at = (size_t)(i / (BN / 4)) * yrows + n0 + (i % (BN / 4)) * 4;
        if (p.resid) {
            const float4 r = *reinterpret_cast<const float4 *>(p.resid + at);
            a = make_float4(r.x + a.x, r.y + a.y, r.z + a.z, r.w + a.w);
        }
        *reinterpret_cast<float4 *>(ymat + at) = a;
    }
}

// The residual add and the RMS norm that follows it in one pass over the partial tiles: block = token; acc = acc + W X
// (stored), out = f16(norm(acc) * w). The sums are formed by 512 threads (many loads in flight) and left in shared
// memory; the norm then runs with the thread layout, the order of additions and the rounding of rms_norm_block_kernel,
// so that the result has the bits of the two kernels run one after the other.
constexpr int SK_NORM_CHUNKS = 10;  // rows of up to 512 x 10 values
__global__ void __launch_bounds__(512) gemm_tc_skinny_sum_norm_kernel(SkinnyParams p, uint32_t blocks, const float *w, __half *out, float eps) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float4 row[128 * SK_NORM_CHUNKS];
    __shared__ uint32_t parts_s[4 * SK_NORM_CHUNKS];
    __shared__ float red[4];
    const uint32_t token = blockIdx.x, t = threadIdx.x, n = p.rows[0], nkst = p.cols / BK, tiles = n / BN;
    if (t < tiles) parts_s[t] = skinny_owner(t * nkst + nkst - 1, p.units, blocks) - skinny_owner(t * nkst, p.units, blocks) + 1;
    __syncthreads();
    float *acc = p.y[0] + (size_t)token * n;
    for (uint32_t f = t; f < n / 4; f += 512) {  // float4 f of the row: tile f / 32, place token x 32 + f % 32 in it
        float4 a = skinny_tile_sum(p, f / (BN / 4), parts_s[f / (BN / 4)], token * (BN / 4) + f % (BN / 4));
        const float4 r = reinterpret_cast<const float4 *>(acc)[f];
        a = make_float4(r.x + a.x, r.y + a.y, r.z + a.z, r.w + a.w);
        reinterpret_cast<float4 *>(acc)[f] = a;
        row[f] = a;
    }
    __syncthreads();
    if (t >= 128) return;
    const uint32_t chunks = n / 512;
    float4 v[SK_NORM_CHUNKS];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < SK_NORM_CHUNKS; ++c) {
        if (c < (int)chunks) {
            v[c] = row[c * 128 + t];
            ss += (v[c].x * v[c].x + v[c].y * v[c].y) + (v[c].z * v[c].z + v[c].w * v[c].w);
        }
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((t & 31) == 0) red[t >> 5] = ss;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    ss = (red[0] + red[1]) + (red[2] + red[3]);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    const float4 *wr = reinterpret_cast<const float4 *>(w);
#pragma unroll
    for (int c = 0; c < SK_NORM_CHUNKS; ++c) {
        if (c < (int)chunks) {
            const float4 ww = wr[c * 128 + t];
            const float a = v[c].x * scale * ww.x, b = v[c].y * scale * ww.y, cc = v[c].z * scale * ww.z, d = v[c].w * scale * ww.w;
            const __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(cc, d);
            reinterpret_cast<uint2 *>(out + (size_t)token * n)[c * 128 + t] = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
        }
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

// The few-token form: see gemm_tc_skinny_kernel. Every matrix is q4_0, tiled, rows a multiple of 128, rows of whole 16 bytes.
// (brasa_gemm_few_tokens_plan, below the namespace, is the one place that decides the cut.)
int32_t launch_skinny(brasa_cmd *cmd, uint32_t count, const brasa_qmatrix *ws, const __half *x, float *const *ys, uint32_t tokens, const float *resid,
                      __half *glu, const float *norm_w = nullptr, __half *norm_out = nullptr, float eps = 0.0f) {
    brasa_ctx *ctx = cmd->ctx;
    SkinnyParams p{};
    SkinnyMaps maps;
    memset(&maps, 0, sizeof maps);
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < 3; ++i) {
        if (i < count) {
            p.y[i] = ys ? ys[i] : nullptr;
            p.rows[i] = ws[i].rows;
            tiles += ws[i].rows / BN;
        }
        p.tile_end[i] = tiles;
    }
    const uint32_t cols = ws[0].cols, nkst = cols / BK, units = tiles * nkst;
    uint32_t blocks = 0, max_parts = 0;
    uint64_t scratch = 0;
    BRASA_REQUIRE(ctx, brasa_gemm_few_tokens_plan((uint32_t)ctx->sm_count, tiles, nkst, &blocks, &max_parts, &scratch) == BRASA_OK, "gemm: shape outside the few-token kernel");
    BRASA_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x) & 15) == 0, "gemm: misaligned x");
    CUtensorMap tmap;
    {
        cuuint64_t dims[2] = {cols, tokens}, strides[1] = {(cuuint64_t)cols * 2};
        cuuint32_t box[2] = {BK, SK_TT}, estr[2] = {1, 1};
        CUresult cr = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) return brasa_fail(ctx, BRASA_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
    }
    const uint32_t rb = tiled_row_bytes(BRASA_Q4_0, cols);
    for (uint32_t i = 0; i < 3; ++i) {
        const brasa_qmatrix &wi = ws[i < count ? i : 0];
        BRASA_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(arg_ptr(wi.data)) & 15) == 0, "gemm: misaligned weights");
        cuuint64_t wdims[2] = {rb, wi.rows}, wstrides[1] = {rb};
        cuuint32_t cbox[2] = {128, BN}, sbox[2] = {16, BN}, westr[2] = {1, 1};
        CUresult wr = encode_tiled()(&maps.codes[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, arg_ptr(wi.data), wdims, wstrides, cbox, westr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (wr == CUDA_SUCCESS)
            wr = encode_tiled()(&maps.scales[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, arg_ptr(wi.data), wdims, wstrides, sbox, westr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (wr != CUDA_SUCCESS) return brasa_fail(ctx, BRASA_ECUDA, "cuTensorMapEncodeTiled failed for the weights (%d)", (int)wr);
    }
    p.cols = cols;
    p.tokens = tokens;
    p.raw_slots = 7;
    p.units = units;
    p.max_parts = max_parts;
    p.status = ctx->status;
    p.resid = resid;
    p.glu = glu;
    p.defer = (glu || norm_out) ? 1u : 0u;
#ifdef BRASA_TRACE_BUILD
    p.trace = (unsigned long long *)ctx->gemv_trace;
#endif
    if (max_parts > 1 || p.defer) {
        const size_t need = (size_t)scratch;
        if (ctx->gemm_part_bytes < need) {
            BRASA_REQUIRE(ctx, !ctx->capturing, "gemm: the split-K workspace cannot grow while a graph is recorded");
            BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            if (ctx->gemm_part) cudaFree(ctx->gemm_part);
            ctx->gemm_part = nullptr;
            ctx->gemm_part_bytes = 0;
            BRASA_CUDA(ctx, cudaMalloc((void **)&ctx->gemm_part, need));
            ctx->gemm_part_bytes = need;
        }
        p.part = ctx->gemm_part;
    }
    const size_t smem = (size_t)SK_NCS * SK_X_CHUNK + (size_t)p.raw_slots * SK_RAW + 1024;
    BRASA_TRY(brasa_smem_optin(ctx, (const void *)gemm_tc_skinny_kernel, ctx->smem_optin - 2048));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(384);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    BRASA_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_tc_skinny_kernel, tmap, maps, p));
    BRASA_TRY(brasa_post_launch(cmd, "gemm_tc_skinny"));
    if (norm_out) {  // one matrix, Y = the residual stream itself: sum, residual add and the norm behind it
        BRASA_CUDA(ctx, brasa_launch_dependent(ctx, gemm_tc_skinny_sum_norm_kernel, dim3(tokens), dim3(512), 0, p, blocks, norm_w, norm_out, eps));
        return brasa_post_launch(cmd, "gemm_tc_skinny_sum_norm");
    }
    if (max_parts == 1 && !glu) return BRASA_OK;
    BRASA_CUDA(ctx, brasa_launch_dependent(ctx, gemm_tc_skinny_sum_kernel, dim3(glu ? tiles / 2 : tiles, 8), dim3(256), 0, p, blocks));
    return brasa_post_launch(cmd, "gemm_tc_skinny_sum");
}

}  // namespace

// How a product of up to 64 tokens is cut over the SMs (include/brasa_cuda.h): the (tile, stage) units in order, `blocks`
// equal runs, run b = units [b units / blocks, (b + 1) units / blocks).
extern "C" int32_t brasa_gemm_few_tokens_plan(uint32_t sm_count, uint32_t tiles, uint32_t stages, uint32_t *blocks, uint32_t *max_parts,
                                              uint64_t *scratch_bytes) {
    if (!blocks || !max_parts || !scratch_bytes || sm_count == 0 || tiles == 0 || stages == 0) return BRASA_EINVAL;
    if ((uint64_t)tiles * stages * ((uint64_t)sm_count + 1) >= (1ull << 32)) return BRASA_EINVAL;  // the kernels divide 32-bit numbers
    const uint32_t units = tiles * stages;
    const uint32_t nb = std::min<uint32_t>(sm_count, std::max(1u, units / 4));  // a run keeps at least four stages
    uint32_t mp = 1;
    for (uint32_t t = 0; t < tiles; ++t) mp = std::max(mp, skinny_owner(t * stages + stages - 1, units, nb) - skinny_owner(t * stages, units, nb) + 1);
    *blocks = nb;
    *max_parts = mp;
    *scratch_bytes = (uint64_t)tiles * mp * SK_TT * BN * sizeof(float);
    return BRASA_OK;
}

extern "C" uint32_t brasa_gemm_few_tokens_owner(uint32_t units, uint32_t blocks, uint32_t unit) {
    if (units == 0 || blocks == 0 || blocks > units || unit >= units || (uint64_t)units * ((uint64_t)blocks + 1) >= (1ull << 32)) return UINT32_MAX;
    return skinny_owner(unit, units, blocks);
}

// True when the tensor-core kernel takes this product (the caller falls back to the warp-MMA kernel otherwise).
bool brasa_gemm_tc_supported(const brasa_qmatrix &w, uint32_t tokens) {
    return (w.qtype == BRASA_Q4_0 || w.qtype == BRASA_Q6_0) && w.layout == BRASA_LAYOUT_TILED && w.rows % BN == 0 && w.cols % BK == 0 && w.cols >= BK && tokens > 0 &&
           encode_tiled() != nullptr;
}

// True when brasa_gemm_tc_launch takes these matrices with the few-token kernel (whose fused SwiGLU may write over X: its
// output is stored by a kernel that starts after every product has been formed).
bool brasa_gemm_tc_few_tokens(brasa_ctx *ctx, const brasa_qmatrix *ws, uint32_t count, uint32_t tokens) {
    if (tokens == 0 || tokens > SK_TT || count < 1 || count > 3) return false;
    uint64_t tiles = 0;
    for (uint32_t i = 0; i < count; ++i) {
        if (!brasa_gemm_tc_supported(ws[i], tokens) || ws[i].qtype != BRASA_Q4_0 || ws[i].cols != ws[0].cols) return false;
        tiles += ws[i].rows / BN;
    }
    return tiled_row_bytes(BRASA_Q4_0, ws[0].cols) % 16 == 0 && tiles * (ws[0].cols / BK) * (uint64_t)(ctx->sm_count + 1) < (1ull << 32);
}

// acc = acc + W X and out = f16(rms_norm(acc) * norm_w) for at most 64 tokens (brasa_gemm_tc_few_tokens holds for w, its rows
// are a multiple of 512 up to 5120, pointers 16-byte aligned): the few-token kernel, then one kernel for sum, add and norm.
int32_t brasa_gemm_tc_add_norm(brasa_cmd *cmd, const brasa_qmatrix &w, const __half *x, float *acc, const float *norm_w, __half *out, uint32_t tokens,
                               float eps) {
    float *ys[1] = {acc};
    return launch_skinny(cmd, 1, &w, x, ys, tokens, acc, nullptr, norm_w, out, eps);
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
    // at most 64 tokens of q4_0 matrices: the persistent form whose accumulator rows are weight rows
    bool few = tokens <= SK_TT && tiled_row_bytes(BRASA_Q4_0, ws[0].cols) % 16 == 0 &&
               (uint64_t)tiles128 * (ws[0].cols / BK) * (uint64_t)(ctx->sm_count + 1) < (1ull << 32);
    for (uint32_t i = 0; i < count; ++i) few = few && ws[i].qtype == BRASA_Q4_0;
    if (few) return launch_skinny(cmd, count, ws, x, ys, tokens, resid, glu);
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
