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

}  // namespace

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

}  // extern "C"
