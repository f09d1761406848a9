// Causal GQA prefill attention on the 5th-generation tensor cores (crates/kernels/src/lib.rs:1185-1248,
// flash_attention.metal:184-323), for the F16 prefill precision: Q * scale is rounded to f16,
// S, P and O are f32, the output is f16.
//
// One CTA = 128 queries of one query head. Per 128-key tile, S = Q K^T is 8 tcgen05.mma (M = 128 queries, N = 128
// keys, K = 16 dims each) into tensor memory; the softmax threads (one per query row) read their row with
// tcgen05.ld (two threads per row, 64 columns each). Softmax is done in two sweeps over the keys instead of rescaling O: the first sweep only finds each
// row's maximum m and sum l, the second recomputes S (tensor-core work is cheap next to everything else here),
// forms P = exp(S - m) and accumulates O += P V in tensor memory. The reference keeps P in f32; a tensor core takes
// f16 operands, so P goes in as two f16 terms (P = hi + lo, error 2^-22) and O += hi V + lo V.
// K, V and Q tiles are written to shared memory in the 128-byte-swizzle layout tcgen05 reads: K and Q as K-major
// operands (row = key / query, 128 dims in two 64-wide blocks), V with the same bytes as an MN-major B operand
// (N = dim is contiguous), P as a K-major A operand (row = query, K = key).
// Every wait is bounded; a wait that runs out raises the context's status word and the CTA leaves.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "attn_device.cuh"
#include "brasa_internal.h"
#include "gemv_device.cuh"

using namespace brasa_dev;

namespace {

constexpr uint32_t FA_WAIT_LIMIT = 1u << 22;
constexpr uint32_t TILE_BYTES = 128 * 128 * 2;  // one 128 x 128 f16 tile: two [128][64] blocks of 16 KB

__device__ __forceinline__ bool fa_mbar_try(uint64_t *bar, uint32_t parity) {
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

// byte offset of the 16-byte chunk holding columns [8c, 8c + 8) of row r in a swizzled 128 x 128 f16 tile
__device__ __forceinline__ uint32_t tile_chunk(uint32_t r, uint32_t c) {
    return (c >> 6) * 16384 + (r >> 3) * 1024 + (r & 7) * 128 + ((((c >> 3) & 7) ^ (r & 7)) << 4);
}

// K-major operand (rows 128 bytes wide, 8-row groups 1024 bytes apart), 128-byte swizzle
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: 64 contiguous N elements per row of 128 bytes, 8 K-rows per 1024-byte group (stride along K),
// the next 64 N elements 16384 bytes further (leading offset)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, "
        "%21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// p0, p1 in [0, 1] -> packed f16 pair `hi` (each value cut to 11 significant bits in f32 first, so the f16 rounding is
// exact down to the subnormals) and the packed pair `lo` of what the cut dropped: hi + lo = p to 2^-22.
__device__ __forceinline__ void split_pair(float p0, float p1, uint32_t &hi, uint32_t &lo) {
    const float h0 = __uint_as_float((__float_as_uint(p0) + 0x1000u) & 0xFFFFE000u), h1 = __uint_as_float((__float_as_uint(p1) + 0x1000u) & 0xFFFFE000u);
    const __half2 hh = __floats2half2_rn(h0, h1), ll = __floats2half2_rn(p0 - h0, p1 - h1);
    hi = *reinterpret_cast<const uint32_t *>(&hh);
    lo = *reinterpret_cast<const uint32_t *>(&ll);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t v[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, "
        "%21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
          "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
          "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

struct FlashTcParams {
    const float *q;        // [tokens][hq][128] after QK-norm and RoPE
    const uint8_t *kc, *vc;  // cache rows [position][hkv][128] in the cache's type, from position 0
    __half *o;             // [tokens][hq][128]
    uint32_t tokens, hq, hkv, pos0;
    float scale;
    uint32_t *status;
};

template <int KV>
__global__ void __launch_bounds__(256, 1) flash_tc_kernel(FlashTcParams p) {
    // an f16 cache enters the tensor core as it is; q8_0 and f32 rows are written as two f16 tiles (value = hi + lo,
    // exact for q8_0, 2^-22 for f32) and every product with K or V becomes two
    constexpr bool SPLIT = KV != BRASA_KV_F16;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *qt = smem, *kt = smem + TILE_BYTES, *vt = smem + 2 * TILE_BYTES, *ph = smem + 3 * TILE_BYTES, *pl = smem + 4 * TILE_BYTES;
    uint8_t *kl = smem + 5 * TILE_BYTES, *vl = smem + 6 * TILE_BYTES;  // SPLIT: low terms of K and V; else their second buffers
    __shared__ uint64_t bar_s2[2], bar_o;  // S lives in two tensor-memory buffers when K is double-buffered (f16 caches)
    __shared__ uint32_t tmem_base_s, abort_s;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // longest query tiles first (they see the most keys)
    const uint32_t qtile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, kh = h / (p.hq / p.hkv);
    const uint32_t q0 = qtile * 128, nq = min(128u, p.tokens - q0);
    const uint32_t last_key = p.pos0 + q0 + nq - 1, lk = p.pos0 + p.tokens;  // inclusive; keys in the cache
    const uint32_t nkt = last_key / 128 + 1;

    if (tid == 0) {
        mbar_init(&bar_s2[0], 1);
        mbar_init(&bar_s2[1], 1);
        mbar_init(&bar_o, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: S in columns [0, 128) and [128, 256), O in [256, 384)
        uint32_t ncols = 512;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q tile: scale, round to f16, swizzled K-major; rows past the last query are zeros
    for (uint32_t i = tid; i < 128 * 16; i += 256) {
        const uint32_t r = i >> 4, c8 = (i & 15) * 8;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (r < nq) {
            const float4 *src = reinterpret_cast<const float4 *>(p.q + ((size_t)(q0 + r) * p.hq + h) * 128 + c8);
            const float4 a = src[0], b = src[1];
            __half2 h0 = __floats2half2_rn(a.x * p.scale, a.y * p.scale), h1 = __floats2half2_rn(a.z * p.scale, a.w * p.scale);
            __half2 h2 = __floats2half2_rn(b.x * p.scale, b.y * p.scale), h3 = __floats2half2_rn(b.z * p.scale, b.w * p.scale);
            out = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1), *reinterpret_cast<uint32_t *>(&h2),
                             *reinterpret_cast<uint32_t *>(&h3));
        }
        *reinterpret_cast<uint4 *>(qt + tile_chunk(r, c8)) = out;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 256;
    uint64_t &bar_s = bar_s2[0];
    volatile uint32_t *abort_flag = &abort_s;

    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
        for (uint32_t it = 0; it < FA_WAIT_LIMIT; ++it) {
            if (fa_mbar_try(bar, parity)) return true;
            if (*abort_flag) return false;
        }
        atomicExch(p.status, 5u);
        *abort_flag = 1;
        return false;
    };
    // rows [j * 128, j * 128 + 128) of one kv head's cache -> a swizzled tile; rows past the cache are zeros
    auto load_tile = [&](const uint8_t *cache, uint8_t *tile, uint8_t *tile_lo, uint32_t j) {
        for (uint32_t i = tid; i < 128 * 16; i += 256) {
            const uint32_t r = i >> 4, c8 = (i & 15) * 8, key = j * 128 + r;
            const uint32_t off = tile_chunk(r, c8);
            if (!SPLIT) {
                if (key < lk) cp_async16(tile + off, cache + ((size_t)key * p.hkv + kh) * 256 + c8 * 2);
                else *reinterpret_cast<uint4 *>(tile + off) = make_uint4(0, 0, 0, 0);
            } else {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.0f;
                if (key < lk) tile_load8<KV>(cache + ((size_t)key * p.hkv + kh) * KvRow<KV>::BYTES, (int)c8, v);
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const __half2 hh = __floats2half2_rn(v[e], v[e + 1]);
                    const float2 hf = __half22float2(hh);
                    const __half2 ll = __floats2half2_rn(v[e] - hf.x, v[e + 1] - hf.y);
                    hi[e >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                    lo[e >> 1] = *reinterpret_cast<const uint32_t *>(&ll);
                }
                *reinterpret_cast<uint4 *>(tile + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(tile_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
    };
    // instruction descriptors: D f32, A and B f16, M = N = 128; V is an MN-major B operand
    const uint32_t idesc_s = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t idesc_o = idesc_s | (1u << 16);
    // An f16 cache leaves room for two K and two V buffers: the next tile's rows travel while this tile is worked on.
    constexpr bool PIPE = !SPLIT;
    auto KB = [&](uint32_t j) { return (PIPE && (j & 1)) ? kl : kt; };
    auto VB = [&](uint32_t j) { return (PIPE && (j & 1)) ? vl : vt; };
    auto issue_s = [&](const uint8_t *kb, uint32_t sbuf = 0) {  // S[sbuf] = Q K^T
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
            umma(tmem_s + 128 * sbuf, desc_kmajor(smem_u32(qt) + off), desc_kmajor(smem_u32(kb) + off), idesc_s, ks > 0);
            if (SPLIT) umma(tmem_s + 128 * sbuf, desc_kmajor(smem_u32(qt) + off), desc_kmajor(smem_u32(kl) + off), idesc_s, 1u);
        }
        umma_commit(&bar_s2[sbuf]);
    };

    // softmax: two threads per query row (warp w: rows 32 (w & 3) .. + 31, columns 64 (w >> 2) .. + 63)
    const uint32_t row = (warp & 3) * 32 + lane, chalf = (warp >> 2) * 64;
    const uint32_t qpos = p.pos0 + q0 + row;
    const uint32_t trow = ((warp & 3) * 32u) << 16;         // lane field of a tensor-memory address
    constexpr float LOG2E = 1.4426950408889634f;
    float m = -INFINITY, l = 0.0f;
    uint32_t ph_s = 0, ph_o = 0;
    bool ok = true;

    // ---- sweep 1: row maxima and sums ----
    uint32_t phs0 = 0, phs1 = 0;  // phases of the two S barriers
    if constexpr (PIPE) {
        // S of tile j + 1 is issued into the other tensor-memory buffer before tile j's scores are read, so the tensor
        // core works while the rows are scanned; the K tile after that travels meanwhile.
        load_tile(p.kc, KB(0), kl, 0);
        if (nkt > 1) load_tile(p.kc, KB(1), kl, 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(KB(0), 0);
        }
        for (uint32_t j = 0; j < nkt; ++j) {
            if (j > 0) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");  // K of tile j + 1
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            ok = __syncthreads_and(ok);  // tile j - 1's scores have been read by everyone: its S buffer may be overwritten
            if (!ok) break;
            if (tid == 0 && j + 1 < nkt) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(KB(j + 1), (j + 1) & 1);
            }
            ok = wait(&bar_s2[j & 1], (j & 1) ? phs1 : phs0);
            if (j & 1) phs1 ^= 1;
            else phs0 ^= 1;
            ok = __all_sync(0xffffffffu, ok);
            if (ok && j + 2 < nkt) {  // S of tile j is complete: its K buffer is free
                load_tile(p.kc, KB(j + 2), kl, j + 2);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (uint32_t c = chalf; c < chalf + 64; c += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_s + 128 * (j & 1) + trow + c, v);
                float cm = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const uint32_t key = j * 128 + c + i;
                    const float sv = key <= qpos ? __uint_as_float(v[i]) : -INFINITY;
                    v[i] = __float_as_uint(sv);
                    cm = fmaxf(cm, sv);
                }
                m = fmaxf(m, cm);
            }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        ok = __syncthreads_and(ok);
    } else {
        if (PIPE) {
            load_tile(p.kc, KB(0), kl, 0);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (uint32_t j = 0; j < nkt && ok; ++j) {
            if (!PIPE) {
                load_tile(p.kc, kt, kl, j);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(KB(j));
            }
            if (PIPE && j + 1 < nkt) {  // the other K buffer was last read by S of tile j - 1, which this thread has seen finish
                load_tile(p.kc, KB(j + 1), kl, j + 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            ok = wait(&bar_s, ph_s);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    #pragma unroll 1
                for (uint32_t c = chalf; c < chalf + 64; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_s + trow + c, v);
                    float cm = -INFINITY;
    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t key = j * 128 + c + i;
                        const float sv = key <= qpos ? __uint_as_float(v[i]) : -INFINITY;
                        v[i] = __float_as_uint(sv);
                        cm = fmaxf(cm, sv);
                    }
                    m = fmaxf(m, cm);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            ph_s ^= 1;
            ok = __syncthreads_and(ok);  // S has been read: the K tile and S may be overwritten
        }
    }
    // the two halves of a row agree on its maximum (the P tiles are free until the second sweep writes them); the sum
    // of the row is gathered in the second sweep from the very probabilities that go into P V
    {
        float *stat = reinterpret_cast<float *>(ph);  // [2][128] maxima
        stat[(warp >> 2) * 128 + row] = m;
        __syncthreads();
        m = fmaxf(stat[row], stat[128 + row]);
        __syncthreads();
    }

    // ---- sweep 2: P = exp(S - m), O += P V ----
    if constexpr (PIPE) {
        // Tensor-core order: .. P V of tile j - 1, S of tile j + 1, P V of tile j ..: S of the next tile is computed while
        // this tile's probabilities are formed (in registers; they are stored once P V of the previous tile has let go of the
        // P tiles), and P V of this tile runs while the next tile's probabilities are formed.
        if (ok) {
            load_tile(p.kc, KB(0), kl, 0);
            load_tile(p.vc, VB(0), vl, 0);
            if (nkt > 1) load_tile(p.kc, KB(1), kl, 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        ok = __syncthreads_and(ok);
        if (ok && tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(KB(0), 0);
        }
        for (uint32_t j = 0; j < nkt && ok; ++j) {
            if (j > 0) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");  // K of tile j + 1 and V of tile j
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            ok = __syncthreads_and(ok);
            if (!ok) break;
            if (tid == 0 && j + 1 < nkt) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(KB(j + 1), (j + 1) & 1);
            }
            ok = wait(&bar_s2[j & 1], (j & 1) ? phs1 : phs0);
            if (j & 1) phs1 ^= 1;
            else phs0 ^= 1;
            ok = __all_sync(0xffffffffu, ok);
            if (ok && j + 2 < nkt) {
                load_tile(p.kc, KB(j + 2), kl, j + 2);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            uint32_t hi[2][16], lo[2][16];
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const uint32_t c = chalf + 32 * cc;
                    uint32_t v[32];
                    tmem_ld32(tmem_s + 128 * (j & 1) + trow + c, v);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const uint32_t key = j * 128 + c + i;
                        const float p0 = key <= qpos ? exp2f((__uint_as_float(v[i]) - m) * LOG2E) : 0.0f;
                        const float p1 = key + 1 <= qpos ? exp2f((__uint_as_float(v[i + 1]) - m) * LOG2E) : 0.0f;
                        l += p0 + p1;
                        split_pair(p0, p1, hi[cc][i >> 1], lo[cc][i >> 1]);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            if (ok && j > 0) {  // the P tiles and the other V buffer are free once P V of tile j - 1 has finished
                ok = wait(&bar_o, ph_o);
                ph_o ^= 1;
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // four 16-byte chunks of 8 keys
                        const uint32_t off = tile_chunk(row, chalf + 32 * cc + 8 * g);
                        *reinterpret_cast<uint4 *>(ph + off) = make_uint4(hi[cc][4 * g], hi[cc][4 * g + 1], hi[cc][4 * g + 2], hi[cc][4 * g + 3]);
                        *reinterpret_cast<uint4 *>(pl + off) = make_uint4(lo[cc][4 * g], lo[cc][4 * g + 1], lo[cc][4 * g + 2], lo[cc][4 * g + 3]);
                    }
                }
                if (j + 1 < nkt) {
                    load_tile(p.vc, VB(j + 1), vl, j + 1);
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            ok = __syncthreads_and(ok);
            if (!ok) break;
            if (tid == 0) {  // O += P_hi V + P_lo V over the tile's 128 keys, 16 per instruction
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t aoff = (ks >> 2) * 16384 + (ks & 3) * 32;  // K-major P: 16 keys = 32 bytes along the row
                    const uint32_t boff = ks * 2048;                          // MN-major V: 16 keys = two 8-key groups
                    umma(tmem_o, desc_kmajor(smem_u32(ph) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                    umma(tmem_o, desc_kmajor(smem_u32(pl) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, 1u);
                }
                umma_commit(&bar_o);
            }
        }
    } else {
        if (PIPE && ok) {
            load_tile(p.kc, KB(0), kl, 0);
            load_tile(p.vc, VB(0), vl, 0);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (uint32_t j = 0; j < nkt && ok; ++j) {
            if (!PIPE) {
                if (j > 0) {  // the previous tile's P V must have finished reading V and P
                    ok = wait(&bar_o, ph_o);
                    ph_o ^= 1;
                }
                load_tile(p.kc, kt, kl, j);
                load_tile(p.vc, vt, vl, j);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            ok = __syncthreads_and(ok);
            if (!ok) break;
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(KB(j));
            }
            if (PIPE && j + 1 < nkt) {
                load_tile(p.kc, KB(j + 1), kl, j + 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            bool ok_o = true;
            if (PIPE && j > 0) {  // P and the other V buffer are free once the previous tile's P V has finished
                ok_o = wait(&bar_o, ph_o);
                ph_o ^= 1;
            }
            if (PIPE && j + 1 < nkt) {
                load_tile(p.vc, VB(j + 1), vl, j + 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            ok = wait(&bar_s, ph_s) && ok_o;
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    #pragma unroll 1
                for (uint32_t c = chalf; c < chalf + 64; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_s + trow + c, v);
                    uint32_t hi[16], lo[16];
    #pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const uint32_t key = j * 128 + c + i;
                        const float p0 = key <= qpos ? exp2f((__uint_as_float(v[i]) - m) * LOG2E) : 0.0f;
                        const float p1 = key + 1 <= qpos ? exp2f((__uint_as_float(v[i + 1]) - m) * LOG2E) : 0.0f;
                        l += p0 + p1;
                        split_pair(p0, p1, hi[i >> 1], lo[i >> 1]);
                    }
    #pragma unroll
                    for (int g = 0; g < 4; ++g) {  // four 16-byte chunks of 8 keys
                        const uint32_t off = tile_chunk(row, c + 8 * g);
                        *reinterpret_cast<uint4 *>(ph + off) = make_uint4(hi[4 * g], hi[4 * g + 1], hi[4 * g + 2], hi[4 * g + 3]);
                        *reinterpret_cast<uint4 *>(pl + off) = make_uint4(lo[4 * g], lo[4 * g + 1], lo[4 * g + 2], lo[4 * g + 3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            ph_s ^= 1;
            ok = __syncthreads_and(ok);
            if (!ok) break;
            if (tid == 0) {  // O += P_hi V + P_lo V over the tile's 128 keys, 16 per instruction
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    #pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t aoff = (ks >> 2) * 16384 + (ks & 3) * 32;  // K-major P: 16 keys = 32 bytes along the row
                    const uint32_t boff = ks * 2048;                          // MN-major V: 16 keys = two 8-key groups
                    umma(tmem_o, desc_kmajor(smem_u32(ph) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                    umma(tmem_o, desc_kmajor(smem_u32(pl) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, 1u);
                    if (SPLIT) umma(tmem_o, desc_kmajor(smem_u32(ph) + aoff), desc_mnmajor(smem_u32(vl) + boff), idesc_o, 1u);  // lo x lo is below 2^-22
                }
                umma_commit(&bar_o);
            }
        }
    }
    // ---- output: O / l, rounded to f16 ----
    if (ok) {
        ok = wait(&bar_o, ph_o);
        ok = __all_sync(0xffffffffu, ok);
    }
    ok = __syncthreads_and(ok);  // the last P V has finished: the P tiles are free
    if (ok) {
        float *stat = reinterpret_cast<float *>(ph);  // [2][128] row sums of the two column halves
        stat[(warp >> 2) * 128 + row] = l;
        __syncthreads();
        l = stat[row] + stat[128 + row];
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = 1.0f / l;
#pragma unroll 1
        for (uint32_t c = chalf; c < chalf + 64; c += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_o + trow + c, v);
            if (row < nq) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const __half2 hh = __floats2half2_rn(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                }
                uint4 *dst = reinterpret_cast<uint4 *>(p.o + ((size_t)(q0 + row) * p.hq + h) * 128 + c);
#pragma unroll
                for (int g = 0; g < 4; ++g) dst[g] = make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ncols = 512;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(ncols) : "memory");
    }
}


// ---- f16 caches: K and V tiles by TMA, two S buffers, two K and two V buffers -------------------------------------
// The kernel above spends most of its instructions on moving tiles with per-thread copies and on a softmax written
// for clarity. For an f16 cache the tiles are exactly what the tensor core reads, so one thread fetches them with
// cp.async.bulk.tensor (the cache as a tensor [position][kv head][128], two boxes of 64 dims with the 128-byte swizzle;
// positions past the end read as zeros) and nobody else touches them. The softmax threads only read S from tensor
// memory and write P: tiles wholly below the diagonal skip the causal test, exp2 is one instruction on a fused
// multiply-add, and the row sum is taken from the very probabilities that enter P V.
// Order on the tensor core: .. P V (j - 1), S (j + 1), P V (j) ..: S of the next tile is computed while this tile's
// probabilities are formed, P V of this tile while the next tile's are.
struct FlashF16Maps {
    CUtensorMap k, v, klo, vlo;  // klo, vlo: the low f16 terms of a cache that was expanded from q8_0 (SPLITKV)
};

// A q8_0 cache for this kernel: every value d * q (f16 scale, 8-bit code) is written as two f16 terms hi + lo, which is
// exact, into f16 arrays shaped like an f16 cache; the kernel then adds the products with the low terms.
__global__ void __launch_bounds__(256) kv_q8_expand_kernel(const uint8_t *cache, __half *hi, __half *lo, uint64_t rows) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 8 values
    if (i >= rows * 16) return;
    const uint64_t r = i >> 4;
    const int c8 = (int)(i & 15) * 8;
    float v[8];
    tile_load8<BRASA_KV_Q8_0>(cache + r * KvRow<BRASA_KV_Q8_0>::BYTES, c8, v);
    uint32_t h[4], l[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const __half2 hh = __floats2half2_rn(v[e], v[e + 1]);
        const float2 hf = __half22float2(hh);
        const __half2 ll = __floats2half2_rn(v[e] - hf.x, v[e + 1] - hf.y);
        h[e >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
        l[e >> 1] = *reinterpret_cast<const uint32_t *>(&ll);
    }
    *reinterpret_cast<uint4 *>(hi + r * 128 + c8) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4 *>(lo + r * 128 + c8) = make_uint4(l[0], l[1], l[2], l[3]);
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool MASK>
__device__ __forceinline__ void max_chunk(uint32_t taddr, uint32_t key0, uint32_t qpos, float &m) {
    uint32_t v[32];
    tmem_ld32(taddr, v);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float sv = __uint_as_float(v[i]);
        if (MASK && key0 + i > qpos) sv = -INFINITY;
        m = fmaxf(m, sv);
    }
}

// 32 scores -> probabilities exp2(s * log2 e - m * log2 e) as packed hi and lo f16 pairs; their sum is added to l
template <bool MASK>
__device__ __forceinline__ void prob_chunk(uint32_t taddr, uint32_t key0, uint32_t qpos, float mneg, float &l, uint32_t hi[16], uint32_t lo[16]) {
    constexpr float LOG2E = 1.4426950408889634f;
    uint32_t v[32];
    tmem_ld32(taddr, v);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), LOG2E, mneg)), p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), LOG2E, mneg));
        if (MASK) {
            if (key0 + i > qpos) p0 = 0.0f;
            if (key0 + i + 1 > qpos) p1 = 0.0f;
        }
        l += p0 + p1;
        split_pair(p0, p1, hi[i >> 1], lo[i >> 1]);
    }
}

// SPLITKV: K and V come as hi + lo tiles (one buffer each instead of two), S = Q K_hi + Q K_lo and
// O += P_hi V_hi + P_lo V_hi + P_hi V_lo (lo x lo is below 2^-22).
// One sweep over the keys. Each row keeps a reference value m_ref for its exponentials; a tile whose largest
// score exceeds m_ref by more than ONEPASS_SLACK (or the first tile) moves the reference to that score, and the row of O
// accumulated so far and the row sum are multiplied by exp(old - new) in tensor memory before the tile's P V is issued.
// With the slack such moves are rare after the first tile, probabilities stay below e^slack = 256 (well inside f16), and
// no separate sweep has to look for the row maxima first (that would be a second Q K^T per tile).
constexpr float ONEPASS_SLACK = 5.545177444f;  // 8 ln 2
constexpr int FLASH_SW = 8;

// SW = 8 softmax warps: 2 threads per query row, 64 score columns each; warp SW is the issuing warp.
template <bool SPLITKV>
__global__ void __launch_bounds__(32 * (FLASH_SW + 1), 1) flash_tc_f16_kernel(const __grid_constant__ FlashF16Maps maps, FlashTcParams p) {
    constexpr int SW = FLASH_SW;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *qt = smem, *ph = smem + 5 * TILE_BYTES, *pl = smem + 6 * TILE_BYTES;
    // tiles 1-4: K and V, two buffers each; with SPLITKV: K hi, K lo, V hi, V lo, one buffer each
    auto KI = [&](uint32_t j) { return SPLITKV ? 0u : (j & 1); };  // which K (V) buffer and barrier tile j uses
    auto KB = [&](uint32_t j) { return smem + (1 + KI(j)) * TILE_BYTES; };
    auto VB = [&](uint32_t j) { return smem + (3 + KI(j)) * TILE_BYTES; };
    uint8_t *klo = smem + 2 * TILE_BYTES, *vlo = smem + 4 * TILE_BYTES;
    __shared__ uint64_t bar_s[2], bar_k[2], bar_v[2], bar_o;
    __shared__ uint32_t tmem_base_s, abort_s;
    __shared__ __half pair_max[4][128];  // a tile's largest score of each column group, by row (f16: a reference value
                                         // need not be the exact maximum, only the same for every thread of the row)
    constexpr int NG = SW / 4, CPT = 128 / NG, NCH = CPT / 32;  // column groups, columns per thread, 32-column chunks per thread

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t qtile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, kh = h / (p.hq / p.hkv);  // longest query tiles first
    const uint32_t q0 = qtile * 128, nq = min(128u, p.tokens - q0);
    const uint32_t last_key = p.pos0 + q0 + nq - 1;
    const uint32_t nkt = last_key / 128 + 1;
    const uint32_t nfree = (p.pos0 + q0 + 1) / 128;  // tiles [0, nfree) lie wholly at or below every row's own position

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_s[i], 1);
            mbar_init(&bar_k[i], 1);
            mbar_init(&bar_v[i], 1);
        }
        mbar_init(&bar_o, 1);
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // tensor memory: S in columns [0, 128) and [128, 256), O in [256, 384)
        uint32_t ncols = 512;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Q tile: scale, round to f16, swizzled K-major; rows past the last query are zeros
    for (uint32_t i = tid; i < 128 * 16; i += 32 * (SW + 1)) {
        const uint32_t r = i >> 4, c8 = (i & 15) * 8;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (r < nq) {
            const float4 *src = reinterpret_cast<const float4 *>(p.q + ((size_t)(q0 + r) * p.hq + h) * 128 + c8);
            const float4 a = src[0], b = src[1];
            __half2 h0 = __floats2half2_rn(a.x * p.scale, a.y * p.scale), h1 = __floats2half2_rn(a.z * p.scale, a.w * p.scale);
            __half2 h2 = __floats2half2_rn(b.x * p.scale, b.y * p.scale), h3 = __floats2half2_rn(b.z * p.scale, b.w * p.scale);
            out = make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1), *reinterpret_cast<uint32_t *>(&h2),
                             *reinterpret_cast<uint32_t *>(&h3));
        }
        *reinterpret_cast<uint4 *>(qt + tile_chunk(r, c8)) = out;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 256;
    volatile uint32_t *abort_flag = &abort_s;

    auto wait = [&](uint64_t *bar, uint32_t parity) -> bool {
        for (uint32_t it = 0; it < FA_WAIT_LIMIT; ++it) {
            if (fa_mbar_try(bar, parity)) return true;
            if (*abort_flag) return false;
        }
        atomicExch(p.status, 5u);
        *abort_flag = 1;
        return false;
    };
    uint32_t inflight = 0;  // issuing thread: bit b = a K copy into buffer b, bit 2 + b = a V copy, not yet waited for
    // one thread: rows [128 j, 128 j + 128) of this kv head -> a tile (two boxes of 64 dims), completion on `bar`
    auto fetch1 = [&](const CUtensorMap *map, uint8_t *dst, uint64_t *bar, uint32_t j) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                             smem_u32(dst + half * 16384)),
                         "l"(map), "r"(half * 64), "r"((int)kh), "r"((int)(j * 128)), "r"(smem_u32(bar))
                         : "memory");
    };
    auto fetch_k = [&](uint32_t j) {
        mbar_expect_tx(&bar_k[KI(j)], (SPLITKV ? 2 : 1) * TILE_BYTES);
        fetch1(&maps.k, KB(j), &bar_k[KI(j)], j);
        if (SPLITKV) fetch1(&maps.klo, klo, &bar_k[KI(j)], j);
        inflight |= 1u << KI(j);
    };
    auto fetch_v = [&](uint32_t j) {
        mbar_expect_tx(&bar_v[KI(j)], (SPLITKV ? 2 : 1) * TILE_BYTES);
        fetch1(&maps.v, VB(j), &bar_v[KI(j)], j);
        if (SPLITKV) fetch1(&maps.vlo, vlo, &bar_v[KI(j)], j);
        inflight |= 4u << KI(j);
    };
    const uint32_t idesc_s = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t idesc_o = idesc_s | (1u << 16);  // V is an MN-major B operand
    auto issue_s = [&](const uint8_t *kb, uint32_t sbuf) {  // S[sbuf] = Q K^T
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
            umma(tmem_s + 128 * sbuf, desc_kmajor(smem_u32(qt) + off), desc_kmajor(smem_u32(kb) + off), idesc_s, ks > 0);
            if (SPLITKV) umma(tmem_s + 128 * sbuf, desc_kmajor(smem_u32(qt) + off), desc_kmajor(smem_u32(klo) + off), idesc_s, 1u);
        }
        umma_commit(&bar_s[sbuf]);
    };

    // Warps 0-7 are the softmax: two threads per query row (warp w: rows 32 (w & 3) .. + 31, columns 64 (w >> 2) .. + 63).
    // Warp 8, one lane, fetches tiles and issues the tensor-core work, so that no softmax warp carries that serial
    // chain; the two sides meet at one block-wide barrier per tile.
    const bool issuer = tid == 32 * SW, softmax = tid < 32 * SW;
    const uint32_t row = (warp & 3) * 32 + lane, cgrp = (warp >> 2) % NG, chalf = cgrp * CPT;
    const uint32_t qpos = p.pos0 + q0 + row;
    const uint32_t trow = ((warp & 3) * 32u) << 16;  // lane field of a tensor-memory address
    float m = -INFINITY, l = 0.0f;
    uint32_t phs0 = 0, phs1 = 0, ph_o = 0;           // phases every thread follows
    uint32_t pk0 = 0, pk1 = 0, pv0 = 0, pv1 = 0;     // phases of the tile barriers (thread 0)
    bool ok = true;
    auto wait_k = [&](uint32_t j) -> bool {
        const uint32_t b = KI(j);
        const bool r = wait(&bar_k[b], b ? pk1 : pk0);
        if (b) pk1 ^= 1;
        else pk0 ^= 1;
        if (r) inflight &= ~(1u << b);
        return r;
    };
    auto wait_v = [&](uint32_t j) -> bool {
        const uint32_t b = KI(j);
        const bool r = wait(&bar_v[b], b ? pv1 : pv0);
        if (b) pv1 ^= 1;
        else pv0 ^= 1;
        if (r) inflight &= ~(4u << b);
        return r;
    };
    auto wait_s = [&](uint32_t j) -> bool {
        bool r = wait(&bar_s[j & 1], (j & 1) ? phs1 : phs0);
        if (j & 1) phs1 ^= 1;
        else phs0 ^= 1;
        return __all_sync(0xffffffffu, r);
    };

    float mneg = -m * 1.4426950408889634f;  // m is still -inf here and moves with the tiles

    // ---- the sweep over the key tiles: P = exp(S - m_ref), O += P V ----
    if (ok && issuer) {
        fetch_k(0);
        fetch_v(0);
        if (!SPLITKV && nkt > 1) fetch_k(1);
        if (wait_k(0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(KB(0), 0);
        }
    }
    for (uint32_t j = 0; j < nkt && ok; ++j) {
        if (!SPLITKV && issuer && j + 1 < nkt && wait_k(j + 1)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(KB(j + 1), (j + 1) & 1);
        }
        ok = wait_s(j);
        uint32_t hi[NCH][16], lo[NCH][16];
        if (ok) {
            if (issuer && !SPLITKV && j + 2 < nkt) fetch_k(j + 2);
            if (issuer && SPLITKV && j + 1 < nkt) fetch_k(j + 1);
            float rescale = 1.0f;
            bool move = false;
            if (softmax) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t ts = tmem_s + 128 * (j & 1) + trow + chalf;
                {
                    // this tile's largest score of the row: own 64 columns, then the other half's through shared memory
                    float tmax = -INFINITY;
#pragma unroll
                    for (int cc = 0; cc < NCH; ++cc) {
                        if (j < nfree) max_chunk<false>(ts + 32 * cc, 0, 0, tmax);
                        else max_chunk<true>(ts + 32 * cc, j * 128 + chalf + 32 * cc, qpos, tmax);
                    }
                    pair_max[cgrp][row] = __float2half_rn(tmax);
                    asm volatile("bar.sync %0, %1;" ::"r"(1 + (warp & 3)), "r"(32 * NG) : "memory");  // the warps that share these rows
                    tmax = -INFINITY;
#pragma unroll
                    for (int g = 0; g < NG; ++g) tmax = fmaxf(tmax, __half2float(pair_max[g][row]));
                    if (tmax > m + ONEPASS_SLACK || (m == -INFINITY && tmax != -INFINITY)) {
                        move = m != -INFINITY;
                        rescale = move ? ex2_approx((m - tmax) * 1.4426950408889634f) : 1.0f;
                        l *= rescale;
                        m = tmax;
                        mneg = -m * 1.4426950408889634f;
                    }
                }
#pragma unroll
                for (int cc = 0; cc < NCH; ++cc) {
                    if (j < nfree) prob_chunk<false>(ts + 32 * cc, 0, 0, mneg, l, hi[cc], lo[cc]);
                    else prob_chunk<true>(ts + 32 * cc, j * 128 + chalf + 32 * cc, qpos, mneg, l, hi[cc], lo[cc]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            if (j > 0) {  // the P tiles and the other V buffer are free once P V of tile j - 1 has finished
                ok = wait(&bar_o, ph_o);
                ph_o ^= 1;
                ok = __all_sync(0xffffffffu, ok);
            }
            if (softmax && ok && __any_sync(0xffffffffu, move)) {
                // a row's reference moved: what O holds for it was accumulated against the old one (P V of tile j - 1 is
                // complete, P V of tile j not yet issued); each half of the pair scales its own 64 dims
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (uint32_t c = chalf; c < chalf + CPT; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_o + trow + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * rescale);
                    tmem_st32(tmem_o + trow + c, v);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        if (ok) {
            if (issuer) {
                if (!SPLITKV && j + 1 < nkt) fetch_v(j + 1);
                if (SPLITKV) {  // one V buffer, free now that P V of tile j - 1 is done; then S of the next tile
                    if (j > 0) fetch_v(j);
                    if (j + 1 < nkt && wait_k(j + 1)) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        issue_s(KB(j + 1), (j + 1) & 1);
                    }
                }
            }
            if (softmax) {
#pragma unroll
                for (int cc = 0; cc < NCH; ++cc) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // four 16-byte chunks of 8 keys
                        const uint32_t off = tile_chunk(row, chalf + 32 * cc + 8 * g);
                        *reinterpret_cast<uint4 *>(ph + off) = make_uint4(hi[cc][4 * g], hi[cc][4 * g + 1], hi[cc][4 * g + 2], hi[cc][4 * g + 3]);
                        *reinterpret_cast<uint4 *>(pl + off) = make_uint4(lo[cc][4 * g], lo[cc][4 * g + 1], lo[cc][4 * g + 2], lo[cc][4 * g + 3]);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
        }
        ok = __syncthreads_and(ok);  // P of tile j is complete; every read of S of tile j is done
        if (!ok) break;
        if (issuer) {  // O += P_hi V + P_lo V over the tile's 128 keys, 16 per instruction
            if (wait_v(j)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t aoff = (ks >> 2) * 16384 + (ks & 3) * 32;  // K-major P: 16 keys = 32 bytes along the row
                    const uint32_t boff = ks * 2048;                          // MN-major V: 16 keys = two 8-key groups
                    umma(tmem_o, desc_kmajor(smem_u32(ph) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                    umma(tmem_o, desc_kmajor(smem_u32(pl) + aoff), desc_mnmajor(smem_u32(VB(j)) + boff), idesc_o, 1u);
                    if (SPLITKV) umma(tmem_o, desc_kmajor(smem_u32(ph) + aoff), desc_mnmajor(smem_u32(vlo) + boff), idesc_o, 1u);
                }
                umma_commit(&bar_o);
            }
        }
    }
    // ---- output: O / l, rounded to f16 ----
    if (ok) {
        ok = wait(&bar_o, ph_o);
        ok = __all_sync(0xffffffffu, ok);
    }
    ok = __syncthreads_and(ok);  // the last P V has finished: the P tiles are free
    if (ok) {
        float *stat = reinterpret_cast<float *>(ph);  // [2][128] row sums of the two column halves
        if (softmax) stat[cgrp * 128 + row] = l;
        __syncthreads();
        l = stat[row];
#pragma unroll
        for (int g = 1; g < NG; ++g) l += stat[g * 128 + row];
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = 1.0f / l;
#pragma unroll 1
        for (uint32_t c = chalf; softmax && c < chalf + CPT; c += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_o + trow + c, v);
            if (row < nq) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const __half2 hh = __floats2half2_rn(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                    packed[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                }
                uint4 *dst = reinterpret_cast<uint4 *>(p.o + ((size_t)(q0 + row) * p.hq + h) * 128 + c);
#pragma unroll
                for (int g = 0; g < 4; ++g) dst[g] = make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
            }
        }
    } else if (issuer) {
        // leaving early: let the tile copies already in flight land before the CTA's shared memory is handed on
        for (int b = 0; b < 2; ++b) {
            if (inflight & (1u << b))
                for (uint32_t it = 0; it < FA_WAIT_LIMIT && !fa_mbar_try(&bar_k[b], b ? pk1 : pk0); ++it) {}
            if (inflight & (4u << b))
                for (uint32_t it = 0; it < FA_WAIT_LIMIT && !fa_mbar_try(&bar_v[b], b ? pv1 : pv0); ++it) {}
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t ncols = 512;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(ncols) : "memory");
    }
}

}  // namespace

// F16 prefill precision over a cache of type kv; q, k, v, o as for brasa_k_flash_attention_with (already validated there).
namespace {
typedef CUresult (*FlashEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
FlashEncodeFn flash_encode() {
    static FlashEncodeFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return (FlashEncodeFn)f;
    }();
    return fn;
}
}  // namespace

int32_t brasa_flash_tc_launch(brasa_cmd *cmd, int32_t kv, const float *q, const uint8_t *kc, const uint8_t *vc, __half *o, brasa_attn_shape sh) {
    brasa_ctx *ctx = cmd->ctx;
    FlashTcParams p{q, kc, vc, o, sh.tokens, sh.hq, sh.hkv, sh.pos0, 1.0f / sqrtf(128.0f), ctx->status};
    dim3 grid((sh.tokens + 127) / 128, sh.hq);
    if ((kv == BRASA_KV_F16 || kv == BRASA_KV_Q8_0) && flash_encode() &&
        ((reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc)) & 15) == 0) {
        const bool split = kv == BRASA_KV_Q8_0;
        const uint64_t npos = (uint64_t)sh.pos0 + sh.tokens, rows = npos * sh.hkv;
        const uint8_t *kh = kc, *vh = vc, *kl = nullptr, *vl = nullptr;
        if (split) {  // q8_0: the rows seen by this call as f16 hi + lo arrays (exact), rebuilt on every call
            const size_t one = rows * 256, need = 4 * one;
            if (ctx->kv_expand_bytes < need) {
                BRASA_REQUIRE(ctx, !ctx->capturing, "flash attention: the q8_0 expansion buffer cannot grow while a graph is recorded");
                BRASA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
                if (ctx->kv_expand) cudaFree(ctx->kv_expand);
                ctx->kv_expand = nullptr;
                ctx->kv_expand_bytes = 0;
                const size_t grow = need + need / 4;  // a prompt fed in chunks asks for a little more every call
                BRASA_CUDA(ctx, cudaMalloc((void **)&ctx->kv_expand, grow));
                ctx->kv_expand_bytes = grow;
            }
            uint8_t *base = ctx->kv_expand;
            const uint32_t blocks = (uint32_t)((rows * 16 + 255) / 256);
            kv_q8_expand_kernel<<<blocks, 256, 0, ctx->stream>>>(kc, (__half *)base, (__half *)(base + one), rows);
            BRASA_TRY(brasa_post_launch(cmd, "kv_q8_expand"));
            kv_q8_expand_kernel<<<blocks, 256, 0, ctx->stream>>>(vc, (__half *)(base + 2 * one), (__half *)(base + 3 * one), rows);
            BRASA_TRY(brasa_post_launch(cmd, "kv_q8_expand"));
            kh = base; kl = base + one; vh = base + 2 * one; vl = base + 3 * one;
        }
        // the caches as tensors [position][kv head][128] of f16, positions [0, pos0 + tokens); a box is 128 positions x 64 dims
        FlashF16Maps maps;
        memset(&maps, 0, sizeof maps);
        const cuuint64_t dims[3] = {128, sh.hkv, npos}, strides[2] = {256, (cuuint64_t)sh.hkv * 256};
        const cuuint32_t box[3] = {64, 1, 128}, estr[3] = {1, 1, 1};
        auto enc = [&](CUtensorMap *m, const uint8_t *ptr) {
            return flash_encode()(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<uint8_t *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        };
        CUresult r1 = enc(&maps.k, kh), r2 = enc(&maps.v, vh), r3 = split ? enc(&maps.klo, kl) : CUDA_SUCCESS, r4 = split ? enc(&maps.vlo, vl) : CUDA_SUCCESS;
        if (r1 != CUDA_SUCCESS || r2 != CUDA_SUCCESS || r3 != CUDA_SUCCESS || r4 != CUDA_SUCCESS)
            return brasa_fail(ctx, BRASA_ECUDA, "cuTensorMapEncodeTiled failed for the KV cache (%d, %d, %d, %d)", (int)r1, (int)r2, (int)r3, (int)r4);
        const size_t smem = 7 * TILE_BYTES + 1024;
        if (split) {
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)flash_tc_f16_kernel<true>, smem));
            flash_tc_f16_kernel<true><<<grid, 32 * (FLASH_SW + 1), smem, ctx->stream>>>(maps, p);
        } else {
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)flash_tc_f16_kernel<false>, smem));
            flash_tc_f16_kernel<false><<<grid, 32 * (FLASH_SW + 1), smem, ctx->stream>>>(maps, p);
        }
        return brasa_post_launch(cmd, "flash_tc_f16");
    }
#define LAUNCH_FTC(KVT, TILES)                                                                                              \
    do {                                                                                                                   \
        const size_t smem = (TILES) * TILE_BYTES + 1024;                                                                   \
            BRASA_TRY(brasa_smem_optin(ctx, (const void *)flash_tc_kernel<KVT>, smem)); \
        flash_tc_kernel<KVT><<<grid, 256, smem, ctx->stream>>>(p);                                                         \
    } while (0)
    if (kv == BRASA_KV_F16) LAUNCH_FTC(BRASA_KV_F16, 7);
    else if (kv == BRASA_KV_F32) LAUNCH_FTC(BRASA_KV_F32, 7);
    else LAUNCH_FTC(BRASA_KV_Q8_0, 7);
#undef LAUNCH_FTC
    return brasa_post_launch(cmd, "flash_tc");
}
