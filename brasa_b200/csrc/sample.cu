// On-device token choice (crates/runtime/src/sampler.rs:148-170): greedy argmax.
#include "brasa_internal.h"

namespace {

struct Best {
    float v;
    uint32_t i;
};
// larger value wins; equal values keep the smaller index (first maximum)
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

__device__ Best block_best(Best b, Best *sh) {
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) sh[warp] = b;
    __syncthreads();
    if (warp == 0) {
        b = lane < (int)(blockDim.x >> 5) ? sh[lane] : Best{-INFINITY, 0xffffffffu};
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
            b = better(b, other);
        }
    }
    return b;  // valid in warp 0
}

// NaN never compares greater, so it never wins; an all -inf (or empty) input yields index 0.
__global__ void __launch_bounds__(256) argmax_kernel(const float *v, uint32_t n, uint32_t *out, Best *partial, uint32_t *counter) {
    __shared__ Best sh[8];
    __shared__ bool last;
    Best b{-INFINITY, 0xffffffffu};
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float x = v[i];
        if (x > b.v) b = Best{x, i};
    }
    b = block_best(b, sh);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = b;
        __threadfence();
        last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    Best f{-INFINITY, 0xffffffffu};
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += blockDim.x) {
        Best pb;
        pb.v = __ldcg(&partial[i].v);
        pb.i = __ldcg(&partial[i].i);
        f = better(f, pb);
    }
    f = block_best(f, sh);
    if (threadIdx.x == 0) {
        *out = (f.v == -INFINITY || f.i == 0xffffffffu) ? 0u : f.i;
        *counter = 0;
    }
}

// End of a decode step: the chosen token becomes the next input, is appended to the output list, and
// the position advances. One thread.
__global__ void advance_kernel(uint32_t *ids, const uint32_t *next, uint32_t *out_ids, uint32_t *out_count, uint32_t out_cap, uint32_t *pos) {
    uint32_t tok = *next;
    ids[0] = tok;
    uint32_t n = *out_count;
    if (n < out_cap) out_ids[n] = tok;
    *out_count = n + 1;
    *pos += 1;
}


// ---- temperature / top-k / top-p sampling on the device (crates/runtime/src/sampler.rs:60-146) ----------------
// The reference sorts the candidates (descending logit, f32 total order), turns them into weights
// exp((l - max) / T), keeps the shortest prefix whose normalised mass reaches top_p and walks that prefix with one
// PCG32 draw. Here nothing is sorted: a prefix of the sorted order is the set {key >= t} for a threshold t, its mass
// is a block-wide sum, and the three prefixes the algorithm needs (the top_k-th candidate, the top_p cut, the drawn
// token) are found by bisection over the 32-bit order key, then over the token id among candidates with equal logits
// (equal logits keep ascending id, as the host sampler does). Sums are tree sums where the reference adds in sorted
// order, so a draw that lands within rounding of a boundary may pick the neighbouring token.
struct Prefix {
    uint32_t t;   // candidates with key > t are in
    uint32_t id;  // candidates with key == t are in when their id <= id
};

__device__ __forceinline__ uint32_t order_key(float f) {  // larger key = earlier in the descending total order
    int32_t b = __float_as_int(f);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return (uint32_t)b ^ 0x80000000u;
}
__device__ __forceinline__ bool in_prefix(uint32_t key, uint32_t id, Prefix p) { return key > p.t || (key == p.t && id <= p.id); }

__device__ float block_sum(float v, float *sh) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();  // sh may still be read from the previous call
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = sh[threadIdx.x & 31];  // 1024 threads: 32 warp sums
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// Sum of g over {i in `inside`: key_i > t or (key_i == t and id <= id_max)}; g = 1 counts.
template <bool COUNT>
__device__ float mass(const float *logits, const float *w, uint32_t n, Prefix inside, Prefix q, float *sh) {
    float a = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t k = order_key(logits[i]);
        if (in_prefix(k, i, inside) && in_prefix(k, i, q)) a += COUNT ? 1.0f : w[i];
    }
    return block_sum(a, sh);
}

// The shortest prefix of the sorted order (inside `inside`) whose mass reaches `bound`; `inside` itself when none does.
template <bool COUNT>
__device__ Prefix shortest_prefix(const float *logits, const float *w, uint32_t n, Prefix inside, float bound, float *sh) {
    if (!(mass<COUNT>(logits, w, n, inside, Prefix{0u, 0xffffffffu}, sh) >= bound)) return inside;
    // largest key t with mass{key >= t} >= bound
    uint32_t lo = 0, hi = 0xffffffffu;
    while (lo < hi) {
        const uint32_t mid = lo + (hi - lo) / 2 + 1;
        if (mass<COUNT>(logits, w, n, inside, Prefix{mid, 0xffffffffu}, sh) >= bound) lo = mid;
        else hi = mid - 1;
    }
    const uint32_t t = lo;
    // among the candidates with that key, the smallest id bound that still reaches it
    uint32_t a = 0, b = n - 1;
    while (a < b) {
        const uint32_t mid = a + (b - a) / 2;
        if (mass<COUNT>(logits, w, n, inside, Prefix{t, mid}, sh) >= bound) b = mid;
        else a = mid + 1;
    }
    return Prefix{t, a};
}

__global__ void __launch_bounds__(1024) sample_kernel(const float *logits, uint32_t n, float temperature, uint32_t top_k, float top_p,
                                                      unsigned long long *rng, float *w, uint32_t *out, uint32_t *ids0, uint32_t *out_ids,
                                                      const uint32_t *out_count) {
    __shared__ float sh[32];
    __shared__ uint32_t shk[32];
    const uint32_t tid = threadIdx.x;
    // one block per sequence: its logits row, its weights, its PCG32 state, its output word
    logits += (size_t)blockIdx.x * n;
    w += (size_t)blockIdx.x * 2 * n;
    rng += 2 * blockIdx.x;
    out += blockIdx.x;
    // largest key: the maximum logit in the total order
    uint32_t kmax = 0;
    for (uint32_t i = tid; i < n; i += blockDim.x) kmax = max(kmax, order_key(logits[i]));
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    if ((tid & 31) == 0) shk[tid >> 5] = kmax;
    __syncthreads();
    kmax = shk[tid & 31];
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    int32_t mb = (int32_t)(kmax ^ 0x80000000u);
    mb ^= (int32_t)(((uint32_t)(mb >> 31)) >> 1);
    const float mx = __int_as_float(mb);

    Prefix kept{0u, 0xffffffffu};  // everything
    if (top_k > 0 && top_k < n) kept = shortest_prefix<true>(logits, nullptr, n, kept, (float)top_k, sh);
    // weights of the kept candidates, their sum, and the normalised weights for the top-p cut
    float a = 0.0f;
    for (uint32_t i = tid; i < n; i += blockDim.x) {
        const float v = in_prefix(order_key(logits[i]), i, kept) ? expf((logits[i] - mx) / temperature) : 0.0f;
        w[i] = v;
        a += v;
    }
    const float sum = block_sum(a, sh);
    if (top_p < 1.0f) {
        for (uint32_t i = tid; i < n; i += blockDim.x) w[n + i] = w[i] / sum;
        __syncthreads();
        kept = shortest_prefix<false>(logits, w + n, n, kept, top_p, sh);
    }
    const float total = mass<false>(logits, w, n, kept, Prefix{0u, 0xffffffffu}, sh);
    // one PCG32 draw (every thread computes the same value; thread 0 stores the new state)
    const unsigned long long old = rng[0], inc = rng[1];
    uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27), rot = (uint32_t)(old >> 59);
    const uint32_t u = (x >> rot) | (x << ((32 - rot) & 31));
    const float r = (float)(u >> 8) / 16777216.0f * total;
    // (a draw of exactly 0 picks the first candidate, as the reference's walk does)
    Prefix pick = shortest_prefix<false>(logits, w, n, kept, fmaxf(r, 1.17549435e-38f), sh);  // first prefix whose weight reaches r; the kept set's end otherwise
    // the chosen token is the last element of that prefix: the smallest key in it, largest id among equals
    uint32_t best_k = 0xffffffffu, best_i = 0;
    for (uint32_t i = tid; i < n; i += blockDim.x) {
        const uint32_t k = order_key(logits[i]);
        if (in_prefix(k, i, kept) && in_prefix(k, i, pick) && (k < best_k || (k == best_k && i > best_i))) {
            best_k = k;
            best_i = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const uint32_t ok = __shfl_xor_sync(0xffffffffu, best_k, o), oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ok < best_k || (ok == best_k && oi > best_i)) { best_k = ok; best_i = oi; }
    }
    __syncthreads();
    if ((tid & 31) == 0) { shk[tid >> 5] = best_k; sh[tid >> 5] = __uint_as_float(best_i); }
    __syncthreads();
    if (tid == 0) {
        for (int wi = 1; wi < 32; ++wi) {
            const uint32_t ok = shk[wi], oi = __float_as_uint(sh[wi]);
            if (ok < best_k || (ok == best_k && oi > best_i)) { best_k = ok; best_i = oi; }
        }
        rng[0] = old * 6364136223846793005ULL + inc;
        *out = best_i;
        if (ids0) *ids0 = best_i;
        if (out_ids && out_count && *out_count > 0) out_ids[*out_count - 1] = best_i;
    }
}


// ---- the same sampler for many rows at once, every row spread over several blocks --------------------------------
// One block per row walks the vocabulary some hundred times (a bisection step is a pass); with 64 rows that costs
// milliseconds per decode step. Here a row is shared by up to 16 blocks and each search is a radix select: four
// passes of 8 key bits, each building a 256-bin histogram of the candidates' mass under the prefix chosen so far;
// the last block of a row to arrive picks the bin in which the running mass reaches the bound. Masses are 64-bit
// fixed point (weight x 2^40, truncated), so sums do not depend on the order of the additions and a row's choice is
// reproducible whatever the grid; candidates with equal logits have equal weights, so the cut inside a group of
// equals is a count, resolved by rows_tie_kernel in ascending id order as the host sampler does.
// A row's scratch: RowState, then 8 histograms (2 searches x 4 digits) of 256 x u64.
constexpr int ROWS_THREADS = 256, ROWS_WARPS = ROWS_THREADS / 32, ROWS_MAX_BLOCKS = 16;
constexpr float ROWS_FIX = 1099511627776.0f;  // 2^40

struct RowState {
    unsigned long long total, bound[2], above[2], m[2], wt[2];
    uint32_t kmax, pref[2], t[2], id_cut, arrive[8];
};
constexpr size_t ROWS_STATE_BYTES = 256, ROWS_SCRATCH_BYTES = ROWS_STATE_BYTES + 8 * 256 * 8;
static_assert(sizeof(RowState) <= ROWS_STATE_BYTES, "row state");

__device__ __forceinline__ float key_value(uint32_t k) {  // inverse of order_key
    int32_t b = (int32_t)(k ^ 0x80000000u);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return __int_as_float(b);
}
__device__ __forceinline__ unsigned long long fixed_weight(float l, float mx, float temperature) {
    return __float2ull_rz(expf((l - mx) / temperature) * ROWS_FIX);
}

__global__ void __launch_bounds__(ROWS_THREADS) rows_max_kernel(const float *logits, uint32_t n, uint8_t *scratch) {
    RowState *st = reinterpret_cast<RowState *>(scratch + (size_t)blockIdx.y * ROWS_SCRATCH_BYTES);
    const float *row = logits + (size_t)blockIdx.y * n;
    uint32_t kmax = 0;
    for (uint32_t i = blockIdx.x * ROWS_THREADS + threadIdx.x; i < n; i += gridDim.x * ROWS_THREADS) kmax = max(kmax, order_key(row[i]));
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    if ((threadIdx.x & 31) == 0) atomicMax(&st->kmax, kmax);
}

// phase 0: the top-p cut over the whole row; phase 1: the drawn token inside the cut. digit 3 (top byte) first.
__global__ void __launch_bounds__(ROWS_THREADS) rows_hist_kernel(const float *logits, uint32_t n, uint8_t *scratch, float temperature, float top_p,
                                                                 int phase, int digit) {
    __shared__ unsigned long long wh[ROWS_WARPS][256];
    __shared__ unsigned long long wtot[ROWS_WARPS];
    __shared__ bool last;
    RowState *st = reinterpret_cast<RowState *>(scratch + (size_t)blockIdx.y * ROWS_SCRATCH_BYTES);
    unsigned long long *hist = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(st) + ROWS_STATE_BYTES) + (phase * 4 + 3 - digit) * 256;
    const float *row = logits + (size_t)blockIdx.y * n;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (uint32_t i = tid; i < ROWS_WARPS * 256; i += ROWS_THREADS) (&wh[0][0])[i] = 0;
    __syncthreads();
    const float mx = key_value(st->kmax);
    const uint32_t shift = 8u * digit, pref = st->pref[phase];
    const Prefix cut = phase ? Prefix{st->t[0], st->id_cut} : Prefix{0u, 0xffffffffu};
    for (uint32_t i = blockIdx.x * ROWS_THREADS + tid; i < n; i += gridDim.x * ROWS_THREADS) {
        const float l = row[i];
        const uint32_t k = order_key(l);
        if (digit < 3 && (k >> (shift + 8)) != (pref >> (shift + 8))) continue;
        if (phase && !in_prefix(k, i, cut)) continue;
        const unsigned long long w = fixed_weight(l, mx, temperature);
        if (w) atomicAdd(&wh[warp][(k >> shift) & 255u], w);
    }
    __syncthreads();
    {
        unsigned long long s = 0;
        for (int w = 0; w < ROWS_WARPS; ++w) s += wh[w][tid];
        if (s) atomicAdd(&hist[tid], s);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) last = atomicAdd(&st->arrive[phase * 4 + 3 - digit], 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // ---- the row's histogram is complete: pick the bin where the mass, summed from the top, reaches the bound ----
    const unsigned long long h = __ldcg(&hist[tid]);
    unsigned long long v = h;  // inclusive suffix sum over bins >= tid
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_down_sync(0xffffffffu, v, o);
        if (lane + o < 32) v += up;
    }
    if (lane == 0) wtot[warp] = v;
    __syncthreads();
    for (int w = warp + 1; w < ROWS_WARPS; ++w) v += wtot[w];
    unsigned long long bound, above;
    if (phase == 0 && digit == 3) {
        unsigned long long total = 0;
        for (int w = 0; w < ROWS_WARPS; ++w) total += wtot[w];
        const double b = ceil((double)total * (double)top_p);
        bound = b >= (double)total ? total : (unsigned long long)b;
        if (bound < 1) bound = 1;
        above = 0;
        if (tid == 0) {
            st->total = total;
            st->bound[0] = bound;
        }
    } else {
        bound = st->bound[phase];
        above = st->above[phase];
    }
    const unsigned long long mine = above + v;                       // mass of the bins >= tid under this prefix
    const unsigned long long next = __shfl_down_sync(0xffffffffu, mine, 1);
    __syncthreads();
    wtot[warp] = 0;  // reuse: first value of the following warp
    __syncthreads();
    if (lane == 0 && warp > 0) wtot[warp - 1] = mine;
    __syncthreads();
    const unsigned long long higher = tid == 255 ? above : (lane == 31 ? wtot[warp] : next);  // mass of the bins > tid
    if (mine >= bound && higher < bound) {
        const uint32_t chosen = pref | ((uint32_t)tid << shift);
        st->pref[phase] = chosen;
        st->above[phase] = higher;
        if (digit == 0) {
            const unsigned long long wt = fixed_weight(key_value(chosen), mx, temperature);
            st->t[phase] = chosen;
            st->wt[phase] = wt;
            st->m[phase] = wt ? (bound - higher + wt - 1) / wt : 1;  // how many of the equal candidates the prefix takes
        }
    }
}

// The m-th candidate, in ascending id order, among those whose key equals the search's threshold: the last member of
// the prefix. phase 0: it closes the top-p cut, then the row's PCG32 draw sets the bound of the second search;
// phase 1: it is the sampled token.
__global__ void __launch_bounds__(1024) rows_tie_kernel(const float *logits, uint32_t n, uint8_t *scratch, int phase, unsigned long long *rng,
                                                        uint32_t *out) {
    __shared__ uint32_t wsum[32];
    RowState *st = reinterpret_cast<RowState *>(scratch + (size_t)blockIdx.x * ROWS_SCRATCH_BYTES);
    const float *row = logits + (size_t)blockIdx.x * n;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t = st->t[phase];
    const unsigned long long m = st->m[phase];
    const Prefix cut = phase ? Prefix{st->t[0], st->id_cut} : Prefix{0u, 0xffffffffu};
    const uint32_t seg = (n + 1023) / 1024, lo = min(n, tid * seg), hi = min(n, lo + seg);
    uint32_t cnt = 0;
    for (uint32_t i = lo; i < hi; ++i) cnt += (order_key(row[i]) == t && in_prefix(t, i, cut)) ? 1u : 0u;
    uint32_t incl = cnt;
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t dn = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)lane >= o) incl += dn;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    uint32_t before = incl - cnt, all = 0;
    for (uint32_t w = 0; w < 32; ++w) {
        if (w < warp) before += wsum[w];
        all += wsum[w];
    }
    if (all == 0) {  // nothing carries the threshold key (a row of NaN): token 0, and a second search that selects nothing
        if (tid == 0) {
            if (phase == 0) st->bound[1] = 1;
            else out[blockIdx.x] = 0;
        }
        return;
    }
    const unsigned long long mm = m < 1 ? 1 : (m > all ? all : m);
    if (!(before < mm && mm <= (unsigned long long)before + cnt)) return;
    uint32_t left = (uint32_t)(mm - before), id = lo;
    for (uint32_t i = lo; i < hi; ++i)
        if (order_key(row[i]) == t && in_prefix(t, i, cut) && --left == 0) {
            id = i;
            break;
        }
    if (phase == 0) {
        st->id_cut = id;
        const unsigned long long kept = st->above[0] + mm * st->wt[0];
        unsigned long long *state = rng + 2 * blockIdx.x;
        const unsigned long long old = state[0], inc = state[1];
        const uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27), rot = (uint32_t)(old >> 59);
        const uint32_t u24 = ((x >> rot) | (x << ((32 - rot) & 31))) >> 8;
        state[0] = old * 6364136223846793005ULL + inc;
        // the walk stops at the first candidate whose running mass reaches u24 / 2^24 of the kept mass (at least 1 unit:
        // a draw of 0 takes the first candidate)
        const unsigned long long hi64 = __umul64hi(kept, (unsigned long long)u24), lo64 = kept * (unsigned long long)u24;
        unsigned long long b = (hi64 << 40) | (lo64 >> 24);
        if (lo64 & 0xffffffull) b += 1;
        st->bound[1] = b < 1 ? 1 : b;
        st->above[1] = 0;
        st->pref[1] = 0;
    } else {
        out[blockIdx.x] = id;
    }
}

// greedy choice per row: first index of the maximum, NaN ignored, 0 when every logit is -inf
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *logits, uint32_t n, uint32_t *out) {
    __shared__ Best sh[32];
    const float *v = logits + (size_t)blockIdx.x * n;
    Best b{-INFINITY, 0xffffffffu};
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float x = v[i];
        if (x > b.v) b = Best{x, i};
    }
    b = block_best(b, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = (b.v == -INFINITY || b.i == 0xffffffffu) ? 0u : b.i;
}

}  // namespace

// Sampler::sample for `count` rows of n logits at once: row r uses the PCG32 state at rng + 2 r and scratch of 2 n floats
// at scratch + 2 n r; out[r] receives its token.
int32_t brasa_sample_batched_launch(brasa_cmd *cmd, const float *logits, uint32_t n, uint32_t count, float temperature, uint32_t top_k, float top_p,
                                    unsigned long long *rng, float *scratch, uint32_t *out) {
    brasa_ctx *ctx = cmd->ctx;
    if (count == 0) return BRASA_OK;
    if (temperature <= 0.0f) {
        argmax_rows_kernel<<<count, 1024, 0, ctx->stream>>>(logits, n, out);
        return brasa_post_launch(cmd, "argmax_rows");
    }
    BRASA_REQUIRE(ctx, top_p > 0.0f, "sample_top_p: top_p must be positive");
    if (count > 1 && (top_k == 0 || top_k >= n) && (size_t)n * 8 >= ROWS_SCRATCH_BYTES) {
        // many rows: every row over several blocks (a row's scratch of 2 n floats holds its state and histograms)
        uint8_t *sc = reinterpret_cast<uint8_t *>(scratch);
        BRASA_CUDA(ctx, cudaMemsetAsync(sc, 0, (size_t)count * ROWS_SCRATCH_BYTES, ctx->stream));
        const dim3 grid(std::min<uint32_t>(ROWS_MAX_BLOCKS, (n + 4095) / 4096), count);
        rows_max_kernel<<<grid, ROWS_THREADS, 0, ctx->stream>>>(logits, n, sc);
        BRASA_TRY(brasa_post_launch(cmd, "sample_rows_max"));
        for (int phase = 0; phase < 2; ++phase) {
            for (int digit = 3; digit >= 0; --digit) {
                rows_hist_kernel<<<grid, ROWS_THREADS, 0, ctx->stream>>>(logits, n, sc, temperature, top_p, phase, digit);
                BRASA_TRY(brasa_post_launch(cmd, "sample_rows_hist"));
            }
            rows_tie_kernel<<<count, 1024, 0, ctx->stream>>>(logits, n, sc, phase, rng, out);
            BRASA_TRY(brasa_post_launch(cmd, "sample_rows_tie"));
        }
        return BRASA_OK;
    }
    sample_kernel<<<count, 1024, 0, ctx->stream>>>(logits, n, temperature, top_k, top_p, rng, scratch, out, nullptr, nullptr, nullptr);
    return brasa_post_launch(cmd, "sample_top_p");
}

int32_t brasa_advance_launch(brasa_cmd *cmd, uint32_t *ids, const uint32_t *next, uint32_t *out_ids, uint32_t *out_count, uint32_t out_cap,
                             uint32_t *pos) {
    advance_kernel<<<1, 1, 0, cmd->ctx->stream>>>(ids, next, out_ids, out_count, out_cap, pos);
    return brasa_post_launch(cmd, "advance");
}

int32_t brasa_argmax_launch(brasa_cmd *cmd, const float *logits, uint32_t n, uint32_t *out) {
    brasa_ctx *ctx = cmd->ctx;
    // scratch: 256 partials (8 bytes each) after the counter, inside the context's status block
    if (!ctx->argmax_scratch) {
        BRASA_CUDA(ctx, cudaMalloc(&ctx->argmax_scratch, 4096));
        BRASA_CUDA(ctx, cudaMemset(ctx->argmax_scratch, 0, 4096));
    }
    uint32_t grid = n == 0 ? 1 : std::min<uint32_t>(256, (n + 1023) / 1024);
    uint32_t *counter = (uint32_t *)ctx->argmax_scratch;
    Best *partial = (Best *)((uint8_t *)ctx->argmax_scratch + 64);
    argmax_kernel<<<grid, 256, 0, ctx->stream>>>(logits, n, out, partial, counter);
    return brasa_post_launch(cmd, "argmax");
}

extern "C" {

int32_t brasa_k_argmax(brasa_cmd *cmd, brasa_arg logits, uint32_t n, brasa_arg out_u32) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(logits, (uint64_t)n * 4) && arg_fits(out_u32, 4), "argmax: buffers too small");
    return brasa_argmax_launch(cmd, (const float *)arg_ptr(logits), n, (uint32_t *)arg_ptr(out_u32));
}


int32_t brasa_k_sample_top_p(brasa_cmd *cmd, brasa_arg logits, uint32_t n, float temperature, uint32_t top_k, float top_p, brasa_arg rng_state,
                             brasa_arg out_u32) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(logits, (uint64_t)n * 4) && arg_fits(out_u32, 4) && arg_fits(rng_state, 16) && rng_state.offset % 8 == 0,
                  "sample_top_p: buffers too small or misaligned");
    if (temperature <= 0.0f) return brasa_argmax_launch(cmd, (const float *)arg_ptr(logits), n, (uint32_t *)arg_ptr(out_u32));
    BRASA_REQUIRE(ctx, top_p > 0.0f, "sample_top_p: top_p must be positive");
    if (ctx->sample_scratch_n < 2 * (size_t)n) {  // weights and normalised weights
        if (ctx->sample_scratch) cudaFree(ctx->sample_scratch);
        ctx->sample_scratch = nullptr;
        ctx->sample_scratch_n = 0;
        BRASA_CUDA(ctx, cudaMalloc(&ctx->sample_scratch, 2 * (size_t)n * 4));
        ctx->sample_scratch_n = 2 * (size_t)n;
    }
    sample_kernel<<<1, 1024, 0, ctx->stream>>>((const float *)arg_ptr(logits), n, temperature, top_k, top_p, (unsigned long long *)arg_ptr(rng_state),
                                               ctx->sample_scratch, (uint32_t *)arg_ptr(out_u32), nullptr, nullptr, nullptr);
    return brasa_post_launch(cmd, "sample_top_p");
}

int32_t brasa_k_sample_rows(brasa_cmd *cmd, brasa_arg logits, uint32_t n, uint32_t count, float temperature, uint32_t top_k, float top_p,
                            brasa_arg rng_states, brasa_arg scratch, brasa_arg out_u32) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(logits, (uint64_t)count * n * 4) && arg_fits(out_u32, (uint64_t)count * 4) &&
                           arg_fits(rng_states, (uint64_t)count * 16) && arg_fits(scratch, (uint64_t)count * n * 8),
                  "sample_rows: buffers too small");
    BRASA_REQUIRE(ctx, rng_states.offset % 8 == 0 && scratch.offset % 8 == 0, "sample_rows: misaligned");
    return brasa_sample_batched_launch(cmd, (const float *)arg_ptr(logits), n, count, temperature, top_k, top_p,
                                       (unsigned long long *)arg_ptr(rng_states), (float *)arg_ptr(scratch), (uint32_t *)arg_ptr(out_u32));
}

void brasa_pcg32_seed(uint64_t seed, uint64_t state_inc[2]) {
    // Pcg32::new of the reference (sampler.rs:13-20): the state after seeding, and the increment
    uint64_t state = 0, inc = (0xda3e39cb94b95bdbULL << 1) | 1;
    state = state * 6364136223846793005ULL + inc;
    state += seed;
    state = state * 6364136223846793005ULL + inc;
    state_inc[0] = state;
    state_inc[1] = inc;
}

}  // extern "C"
