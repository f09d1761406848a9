// Tensor-parallel exchange between the ranks of one node: a one-shot push all-reduce over peer memory.
//
// The reference runs on one device; a model too large or too slow for one GPU is split Megatron-style (q/k/v and
// gate/up by rows, o_proj and down_proj by columns), which leaves one sum over ranks after o_proj and one after
// down_proj in every layer (the two residual adds of qwen3.rs:763-831), plus one (max, index) exchange after the
// vocabulary-sharded lm_head.
//
// Every rank owns one exchange buffer of 8-byte words {f32 value, u32 tag}: [2 parities][world][max_elems]. In an
// exchange a rank WRITES its values into slot [parity][its rank] of every rank's buffer (its own included) and then
// READS all slots of its OWN buffer, waiting word by word until the tag equals the exchange's number: the flag
// travels inside the data word (an aligned 8-byte store is not torn), so there is no separate barrier, no fence and
// nobody polls remote memory. Sums run in rank order on every rank, so all ranks hold bit-identical results and the
// replicated residual stream never diverges. Two parities are enough: a rank can start exchange e + 2 only after it
// finished e + 1, which needs every peer's e + 1 values, which a peer sends only after it finished reading e.
// All waits are bounded; a wait that runs out raises the context's status word and the kernel finishes with whatever
// it has (the host then reports BRASA_ETIMEOUT).
#include <algorithm>

#include "brasa_internal.h"

int32_t brasa_argmax_launch(brasa_cmd *cmd, const float *logits, uint32_t n, uint32_t *out);
int32_t brasa_tp_allreduce_add_launch(brasa_cmd *cmd, brasa_tp *tp, const float *src, const float *resid, float *out, uint64_t n, int phases);

struct brasa_tp {
    brasa_ctx *ctx = nullptr;
    uint32_t rank = 0, world = 1;
    uint64_t max_elems = 0;
    uint64_t *local = nullptr;                 // this rank's exchange buffer
    uint64_t *peer[BRASA_TP_MAX_RANKS] = {};   // every rank's buffer as seen from here; peer[rank] == local
    bool ipc_opened[BRASA_TP_MAX_RANKS] = {};
    uint32_t *state = nullptr;                 // device: [0] exchanges done so far, [1] arrival counter, [2] local argmax index
    bool connected = false;
    uint32_t poll_limit = 1u << 22;            // loads of one exchange word before a wait gives up (brasa_tp_set_poll_limit)
    uint64_t token_stride = 0;                 // words per rank slot of the whole-token kernel's own exchange area
    bool shares_device = false;                // another rank of the group lives on this rank's device (tests)
};

namespace {

enum { TP_PUSH = 1, TP_GATHER = 2 };

struct TpParams {
    uint64_t *peer[BRASA_TP_MAX_RANKS];
    uint32_t rank, world;
    uint64_t max_elems;
    uint32_t *state, *status;
    uint32_t poll_limit;
};

__device__ __forceinline__ void st_words(uint64_t *p, uint64_t a, uint64_t b) {
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_words(const uint64_t *p, uint64_t &a, uint64_t &b) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ uint64_t word(float v, uint32_t tag) { return (uint64_t)__float_as_uint(v) | ((uint64_t)tag << 32); }

// Waits for the two words at p to carry `tag`. dead: a wait of this thread already ran out (do not wait again).
__device__ __forceinline__ void wait_words(const uint64_t *p, uint32_t tag, uint64_t &a, uint64_t &b, bool &dead, uint32_t *status, uint32_t limit) {
    for (uint32_t it = 0;; ++it) {
        ld_words(p, a, b);
        if (((uint32_t)(a >> 32) == tag && (uint32_t)(b >> 32) == tag) || dead) return;
        if (it >= limit) {
            atomicExch(status, 6u);
            dead = true;
            return;
        }
    }
}

// The last block of an exchange's gather phase advances the exchange counter for the next kernel on the stream.
__device__ __forceinline__ void finish_exchange(const TpParams &p, uint32_t e) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) {
            p.state[1] = 0;
            *reinterpret_cast<volatile uint32_t *>(&p.state[0]) = e + 1;
        }
    }
}

// out[i] = resid[i] + (src_0[i] + src_1[i] + ..) over ranks, n even. phases: TP_PUSH | TP_GATHER in the product path.
__global__ void __launch_bounds__(256) tp_allreduce_add_kernel(TpParams p, const float *src, const float *resid, float *out, uint64_t n, int phases) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&p.state[0]), tag = e + 1;
    const uint64_t base = (uint64_t)(e & 1) * p.world * p.max_elems;
    const uint64_t n2 = n / 2, stride = (uint64_t)gridDim.x * blockDim.x, first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (phases & TP_PUSH) {
        for (uint64_t i = first; i < n2; i += stride) {
            const float2 v = reinterpret_cast<const float2 *>(src)[i];
            const uint64_t a = word(v.x, tag), b = word(v.y, tag);
            for (uint32_t r = 0; r < p.world; ++r) st_words(p.peer[r] + base + (uint64_t)p.rank * p.max_elems + 2 * i, a, b);
        }
    }
    if (phases & TP_GATHER) {
        bool dead = false;
        const uint64_t *mine = p.peer[p.rank] + base;
        for (uint64_t i = first; i < n2; i += stride) {
            // every rank's pair is asked for together and only the missing ones again: one round trip once they are there
            uint64_t wa[BRASA_TP_MAX_RANKS], wb[BRASA_TP_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < BRASA_TP_MAX_RANKS; ++r) wa[r] = wb[r] = 0;  // tag 0 is never an exchange's
            for (uint32_t it = 0; !dead; ++it) {
                bool ok = true;
#pragma unroll
                for (int r = 0; r < BRASA_TP_MAX_RANKS; ++r) {
                    if ((uint32_t)r < p.world && !((uint32_t)(wa[r] >> 32) == tag && (uint32_t)(wb[r] >> 32) == tag)) {
                        ld_words(mine + (uint64_t)r * p.max_elems + 2 * i, wa[r], wb[r]);
                        ok = ok && (uint32_t)(wa[r] >> 32) == tag && (uint32_t)(wb[r] >> 32) == tag;
                    }
                }
                if (ok) break;
                if (it >= p.poll_limit) {
                    atomicExch(p.status, 6u);
                    dead = true;
                }
            }
            float sx = __uint_as_float((uint32_t)wa[0]), sy = __uint_as_float((uint32_t)wb[0]);
#pragma unroll
            for (int r = 1; r < BRASA_TP_MAX_RANKS; ++r) {
                if ((uint32_t)r < p.world) {
                    sx += __uint_as_float((uint32_t)wa[r]);
                    sy += __uint_as_float((uint32_t)wb[r]);
                }
            }
            float2 o = make_float2(sx, sy);
            if (resid) {
                const float2 x = reinterpret_cast<const float2 *>(resid)[i];
                o = make_float2(x.x + sx, x.y + sy);
            }
            reinterpret_cast<float2 *>(out)[i] = o;
        }
        finish_exchange(p, e);
    }
}

// One warp. Every rank contributes (logits[local index], local index + row0); the winner is the largest value, the
// lowest index among equals, NaN never (sampler.rs:150-170 argmax over the whole vocabulary).
__global__ void __launch_bounds__(32) tp_argmax_kernel(TpParams p, const float *logits, uint32_t row0, uint32_t *out, int phases) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&p.state[0]), tag = e + 1, lane = threadIdx.x;
    const uint64_t base = (uint64_t)(e & 1) * p.world * p.max_elems;
    if ((phases & TP_PUSH) && lane < p.world) {
        const uint32_t idx = p.state[2];
        st_words(p.peer[lane] + base + (uint64_t)p.rank * p.max_elems, word(logits[idx], tag), word(__uint_as_float(idx + row0), tag));
    }
    if (phases & TP_GATHER) {
        float v = -INFINITY;
        uint32_t id = 0xffffffffu;
        if (lane < p.world) {
            uint64_t a, b;
            bool dead = false;
            wait_words(p.peer[p.rank] + base + (uint64_t)lane * p.max_elems, tag, a, b, dead, p.status, p.poll_limit);
            const float got = __uint_as_float((uint32_t)a);
            if (!dead) {
                id = (uint32_t)b;
                v = got == got ? got : -INFINITY;
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, id, o);
            if (ov > v || (ov == v && oi < id)) {
                v = ov;
                id = oi;
            }
        }
        // nothing valid arrived (every wait ran out): token 0, as the argmax of sampler.rs:150-170 gives when no logit
        // exceeds -inf
        if (lane == 0) *out = id == 0xffffffffu ? 0u : id;
        finish_exchange(p, e);
    }
}

TpParams params_of(brasa_tp *tp) {
    TpParams p{};
    for (uint32_t r = 0; r < tp->world; ++r) p.peer[r] = tp->peer[r];
    p.rank = tp->rank;
    p.world = tp->world;
    p.max_elems = tp->max_elems;
    p.state = tp->state;
    p.status = tp->ctx->status;
    p.poll_limit = tp->poll_limit;
    return p;
}

// The exchange buffer: [2 parities][world][max_elems] words for the kernels of this file, followed by the area the
// whole-token decode kernel uses on its own (its words carry that kernel's epochs, which must never meet the exchange
// numbers used here): [2][world][token_stride] partial sums and [2][world][2] (best logit, index) pairs. One
// allocation, so one IPC handle opens all of it.
uint64_t main_words(const brasa_tp *tp) { return 2ull * tp->world * tp->max_elems; }
uint64_t buffer_bytes(const brasa_tp *tp) { return (main_words(tp) + 2ull * tp->world * tp->token_stride + 4ull * tp->world) * 8; }

}  // namespace

bool brasa_tp_token_area_get(brasa_tp *tp, brasa_tp_token_area *out) {
    // Ranks that share a device cannot run kernels that wait for one another (nothing makes two launches on one GPU
    // run at the same time): such a group keeps the exchange kernels of this file, queued send-before-receive.
    if (!tp || !out || !tp->connected || tp->shares_device) return false;
    out->world = tp->world;
    out->rank = tp->rank;
    out->stride = tp->token_stride;
    out->poll_limit = tp->poll_limit;
    for (uint32_t r = 0; r < tp->world; ++r) out->peer[r] = reinterpret_cast<unsigned long long *>(tp->peer[r] + main_words(tp));
    return true;
}

bool brasa_tp_push_target_get(brasa_tp *tp, brasa_tp_push_target *out) {
    if (!tp || !out || !tp->connected) return false;
    for (uint32_t r = 0; r < BRASA_TP_MAX_RANKS; ++r) out->peer[r] = r < tp->world ? reinterpret_cast<unsigned long long *>(tp->peer[r]) : nullptr;
    out->world = tp->world;
    out->rank = tp->rank;
    out->max_elems = tp->max_elems;
    out->state = tp->state;
    return true;
}

// y = W x of a column-split matrix (o_proj, down_proj) summed over the ranks, plus the residual: the GEMV's epilogue
// writes its rows straight into every rank's exchange slot (no local vector, no separate send pass), and the receive
// half of the exchange adds the slots in rank order. phases as in brasa_tp_allreduce_add_launch.
int32_t brasa_tp_gemv_allreduce_launch(brasa_cmd *cmd, brasa_tp *tp, const brasa_qmatrix &w, const float *x, const float *resid, float *out, int phases) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, tp->connected, "tp: the ranks are not connected yet");
    BRASA_REQUIRE(ctx, w.rows % 2 == 0 && w.rows <= tp->max_elems, "tp gemv: %u rows (even, at most %llu)", w.rows, (unsigned long long)tp->max_elems);
    if (phases & TP_PUSH) {
        brasa_tp_push_target target;
        brasa_tp_push_target_get(tp, &target);
        float *none[1] = {nullptr};
        BRASA_TRY(brasa_gemv_launch(cmd, w.qtype, 1, &w, none, x, nullptr, nullptr, nullptr, nullptr, 0, 0, 0.0f, 3, nullptr, &target));
    }
    if (phases & TP_GATHER) BRASA_TRY(brasa_tp_allreduce_add_launch(cmd, tp, nullptr, resid, out, w.rows, TP_GATHER));
    return BRASA_OK;
}

uint64_t brasa_tp_max_elems(const brasa_tp *tp) { return tp ? tp->max_elems : 0; }

int32_t brasa_tp_allreduce_add_launch(brasa_cmd *cmd, brasa_tp *tp, const float *src, const float *resid, float *out, uint64_t n, int phases) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, tp->connected, "tp: the ranks are not connected yet");
    BRASA_REQUIRE(ctx, n % 2 == 0 && n <= tp->max_elems, "tp all-reduce: %llu values (even, at most %llu)", (unsigned long long)n,
                  (unsigned long long)tp->max_elems);
    if (n == 0) return BRASA_OK;
    const uint32_t grid = (uint32_t)std::min<uint64_t>((n / 2 + 255) / 256, (uint64_t)ctx->sm_count * 4);
    tp_allreduce_add_kernel<<<grid, 256, 0, ctx->stream>>>(params_of(tp), src, resid, out, n, phases);
    return brasa_post_launch(cmd, "tp_allreduce_add");
}

int32_t brasa_tp_argmax_launch(brasa_cmd *cmd, brasa_tp *tp, const float *logits, uint32_t n, uint32_t row0, uint32_t *out, int phases) {
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, tp->connected && tp->max_elems >= 2, "tp: the ranks are not connected yet");
    if (phases & TP_PUSH) BRASA_TRY(brasa_argmax_launch(cmd, logits, n, tp->state + 2));
    tp_argmax_kernel<<<1, 32, 0, ctx->stream>>>(params_of(tp), logits, row0, out, phases);
    return brasa_post_launch(cmd, "tp_argmax");
}

extern "C" {

int32_t brasa_tp_create(brasa_ctx *ctx, uint32_t rank, uint32_t world, uint64_t max_elems, brasa_tp **out) {
    if (!ctx || !out) return BRASA_EINVAL;
    *out = nullptr;
    BRASA_REQUIRE(ctx, world >= 1 && world <= BRASA_TP_MAX_RANKS && rank < world, "tp: rank %u of %u", rank, world);
    BRASA_REQUIRE(ctx, max_elems >= 2 && max_elems % 2 == 0, "tp: the exchange size must be even and at least 2");
    brasa_tp *tp = new brasa_tp();
    tp->ctx = ctx;
    tp->rank = rank;
    tp->world = world;
    tp->max_elems = max_elems;
    tp->token_stride = std::min<uint64_t>(max_elems, 16384);
    int32_t rc = [&]() -> int32_t {
        BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
        BRASA_CUDA(ctx, cudaMalloc((void **)&tp->local, buffer_bytes(tp)));
        BRASA_CUDA(ctx, cudaMemset(tp->local, 0, buffer_bytes(tp)));  // tag 0 is never waited for
        BRASA_CUDA(ctx, cudaMalloc((void **)&tp->state, 64));
        BRASA_CUDA(ctx, cudaMemset(tp->state, 0, 64));
        BRASA_CUDA(ctx, cudaDeviceSynchronize());
        return BRASA_OK;
    }();
    if (rc != BRASA_OK) {
        brasa_tp_free(tp);
        return rc;
    }
    tp->peer[rank] = tp->local;
    tp->connected = world == 1;
    *out = tp;
    return BRASA_OK;
}

void brasa_tp_free(brasa_tp *tp) {
    if (!tp) return;
    cudaSetDevice(tp->ctx->device);
    cudaDeviceSynchronize();
    for (uint32_t r = 0; r < tp->world; ++r)
        if (tp->ipc_opened[r]) cudaIpcCloseMemHandle(tp->peer[r]);
    cudaFree(tp->local);
    cudaFree(tp->state);
    delete tp;
}

int32_t brasa_tp_set_poll_limit(brasa_tp *tp, uint32_t polls) {
    if (!tp) return BRASA_EINVAL;
    BRASA_REQUIRE(tp->ctx, polls >= 1, "tp: the poll limit must be at least 1");
    tp->poll_limit = polls;
    return BRASA_OK;
}

uint32_t brasa_tp_rank(const brasa_tp *tp) { return tp ? tp->rank : 0; }
uint32_t brasa_tp_world(const brasa_tp *tp) { return tp ? tp->world : 0; }

int32_t brasa_tp_handle(brasa_tp *tp, uint8_t *handle) {
    if (!tp || !handle) return BRASA_EINVAL;
    static_assert(sizeof(cudaIpcMemHandle_t) == BRASA_TP_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    BRASA_CUDA(tp->ctx, cudaIpcGetMemHandle(&h, tp->local));
    memcpy(handle, &h, sizeof h);
    return BRASA_OK;
}

// handles: world x BRASA_TP_HANDLE_BYTES, entry r from rank r's brasa_tp_handle (the entry of this rank is ignored).
// The caller synchronises the ranks around this call (every buffer exists before, nobody exchanges until all returned).
int32_t brasa_tp_connect(brasa_tp *tp, const uint8_t *handles) {
    if (!tp || !handles) return BRASA_EINVAL;
    brasa_ctx *ctx = tp->ctx;
    BRASA_REQUIRE(ctx, !tp->connected || tp->world == 1, "tp: already connected");
    BRASA_CUDA(ctx, cudaSetDevice(ctx->device));
    for (uint32_t r = 0; r < tp->world; ++r) {
        if (r == tp->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * BRASA_TP_HANDLE_BYTES, sizeof h);
        void *p = nullptr;
        BRASA_CUDA(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        tp->peer[r] = (uint64_t *)p;
        tp->ipc_opened[r] = true;
    }
    tp->connected = true;
    return BRASA_OK;
}

// Ranks that live in one process (one context per device, or several ranks on one device in tests): plain pointers,
// with peer access enabled between different devices.
int32_t brasa_tp_connect_same_process(brasa_tp *const *tps, uint32_t n) {
    if (!tps || n == 0) return BRASA_EINVAL;
    brasa_ctx *ctx = tps[0]->ctx;
    for (uint32_t i = 0; i < n; ++i)
        BRASA_REQUIRE(ctx, tps[i] && tps[i]->world == n && tps[i]->rank == i && tps[i]->max_elems == tps[0]->max_elems, "tp: rank list does not match");
    for (uint32_t i = 0; i < n; ++i) {
        for (uint32_t r = 0; r < n; ++r) {
            if (r == i) continue;
            if (tps[i]->ctx->device != tps[r]->ctx->device) {
                BRASA_CUDA(ctx, cudaSetDevice(tps[i]->ctx->device));
                cudaError_t e = cudaDeviceEnablePeerAccess(tps[r]->ctx->device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else BRASA_CUDA(ctx, e);
            } else {
                tps[i]->shares_device = true;
            }
            tps[i]->peer[r] = tps[r]->local;
        }
        tps[i]->connected = true;
    }
    return BRASA_OK;
}

int32_t brasa_k_tp_allreduce_add(brasa_cmd *cmd, brasa_tp *tp, brasa_arg partial, brasa_arg resid, brasa_arg out, uint64_t n) {
    if (!cmd || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, ctx == tp->ctx, "tp: command of another context");
    BRASA_REQUIRE(ctx, arg_fits(partial, n * 4) && arg_fits(out, n * 4) && (!resid.buf || arg_fits(resid, n * 4)), "tp all-reduce: buffers too small");
    BRASA_REQUIRE(ctx, partial.offset % 8 == 0 && out.offset % 8 == 0 && resid.offset % 8 == 0, "tp all-reduce: misaligned");
    return brasa_tp_allreduce_add_launch(cmd, tp, (const float *)arg_ptr(partial), resid.buf ? (const float *)arg_ptr(resid) : nullptr,
                                         (float *)arg_ptr(out), n, TP_PUSH | TP_GATHER);
}

int32_t brasa_k_tp_argmax(brasa_cmd *cmd, brasa_tp *tp, brasa_arg logits, uint32_t n, uint32_t row0, brasa_arg out_u32) {
    if (!cmd || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, ctx == tp->ctx, "tp: command of another context");
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(logits, (uint64_t)n * 4) && arg_fits(out_u32, 4), "tp argmax: buffers too small");
    return brasa_tp_argmax_launch(cmd, tp, (const float *)arg_ptr(logits), n, row0, (uint32_t *)arg_ptr(out_u32), TP_PUSH | TP_GATHER);
}

static int32_t gemv_allreduce_checked(brasa_cmd *cmd, brasa_tp *tp, brasa_qmatrix w, brasa_arg x, brasa_arg resid, brasa_arg out, int phases) {
    if (!cmd || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, ctx == tp->ctx, "tp: command of another context");
    BRASA_REQUIRE(ctx, w.layout == BRASA_LAYOUT_TILED && (w.qtype == BRASA_Q4_0 || w.qtype == BRASA_Q6_0), "tp gemv: a tiled q4_0 or q6_0 matrix");
    BRASA_REQUIRE(ctx, arg_fits(x, (uint64_t)w.cols * 4) && arg_fits(out, (uint64_t)w.rows * 4) && (!resid.buf || arg_fits(resid, (uint64_t)w.rows * 4)),
                  "tp gemv: buffers too small");
    BRASA_REQUIRE(ctx, x.offset % 16 == 0 && out.offset % 8 == 0 && resid.offset % 8 == 0, "tp gemv: misaligned");
    return brasa_tp_gemv_allreduce_launch(cmd, tp, w, (const float *)arg_ptr(x), resid.buf ? (const float *)arg_ptr(resid) : nullptr, (float *)arg_ptr(out),
                                          phases);
}

int32_t brasa_k_gemv_allreduce(brasa_cmd *cmd, brasa_tp *tp, brasa_qmatrix w, brasa_arg x, brasa_arg resid, brasa_arg out) {
    return gemv_allreduce_checked(cmd, tp, w, x, resid, out, TP_PUSH | TP_GATHER);
}

int32_t brasa_k_gemv_allreduce_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_qmatrix w, brasa_arg x, brasa_arg resid, brasa_arg out, int32_t gather) {
    return gemv_allreduce_checked(cmd, tp, w, x, resid, out, gather ? TP_GATHER : TP_PUSH);
}

// The two halves of an exchange as separate launches, for ranks that share one device: a kernel that waits for a
// peer's values must not be queued before the kernel that sends them, so all ranks push first and gather afterwards.
int32_t brasa_k_tp_allreduce_add_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_arg partial, brasa_arg resid, brasa_arg out, uint64_t n, int32_t gather) {
    if (!cmd || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, arg_fits(partial, n * 4) && arg_fits(out, n * 4) && (!resid.buf || arg_fits(resid, n * 4)), "tp all-reduce: buffers too small");
    return brasa_tp_allreduce_add_launch(cmd, tp, (const float *)arg_ptr(partial), resid.buf ? (const float *)arg_ptr(resid) : nullptr,
                                         (float *)arg_ptr(out), n, gather ? TP_GATHER : TP_PUSH);
}

int32_t brasa_k_tp_argmax_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_arg logits, uint32_t n, uint32_t row0, brasa_arg out_u32, int32_t gather) {
    if (!cmd || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, n > 0 && arg_fits(logits, (uint64_t)n * 4) && arg_fits(out_u32, 4), "tp argmax: buffers too small");
    return brasa_tp_argmax_launch(cmd, tp, (const float *)arg_ptr(logits), n, row0, (uint32_t *)arg_ptr(out_u32), gather ? TP_GATHER : TP_PUSH);
}

}  // extern "C"
