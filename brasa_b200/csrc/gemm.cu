// Prefill GEMM: Y[t, :] = W X[t, :] for `tokens` rows of X (crates/kernels/src/lib.rs:842-970,
// matmul_tiled.metal). Precision F16 is the hot path: X is f16, each dequantised weight is rounded to
// f16 as f16(f32(d) * (q - bias)) and products are accumulated in f32 (matmul_tiled.metal:35-53).
// Precision F32 keeps both in f32.
//
// This file holds the warp-MMA version (mma.sync m16n8k16), valid for every shape, and the exact f32 version; tiled q4_0
// matrices whose rows are a multiple of 128 go to the tcgen05 kernel of gemm_tc.cu (BRASA_GEMM_TC=0 keeps them here).
#include <stdlib.h>

#include "brasa_internal.h"

bool brasa_gemm_tc_supported(const brasa_qmatrix &w, uint32_t tokens);
bool brasa_gemm_tc_few_tokens(brasa_ctx *ctx, const brasa_qmatrix *ws, uint32_t count, uint32_t tokens);
int32_t brasa_gemm_tc_add_norm(brasa_cmd *cmd, const brasa_qmatrix &w, const __half *x, float *acc, const float *norm_w, __half *out, uint32_t tokens,
                               float eps);
int32_t brasa_gemm_tc_launch(brasa_cmd *cmd, uint32_t count, const brasa_qmatrix *ws, const __half *x, float *const *ys, uint32_t tokens,
                             const float *resid, __half *glu);

namespace {

// Code (bias removed) and scale of element (r, c) for both layouts and all weight types.
struct WView {
    const uint8_t *p;
    int qtype, layout;
    uint32_t rows, cols;
};

// Dequantises block (r, b) into 32 floats d * (q - bias), element order 0..31.
__device__ __forceinline__ void dequant_block(const WView &w, uint32_t r, uint32_t b, float *out) {
    uint32_t nb = w.cols / 32;
    const uint8_t *codes, *hi = nullptr;
    float d;
    if (w.layout == BRASA_LAYOUT_FILE) {
        int bb = w.qtype == BRASA_Q4_0 ? 18 : (w.qtype == BRASA_Q6_0 ? 26 : 34);
        const uint8_t *p = w.p + ((size_t)r * nb + b) * bb;
        d = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(p)));
        codes = p + 2;
        if (w.qtype == BRASA_Q8_0) {
            for (int j = 0; j < 32; ++j) out[j] = d * (float)(int8_t)codes[j];
            return;
        }
        if (w.qtype == BRASA_Q6_0) {
            for (int j = 0; j < 32; ++j) {
                int ql = codes[j & 15];
                int lo = j < 16 ? (ql & 15) : (ql >> 4);
                int h2 = (p[18 + (j & 7)] >> (2 * (j >> 3))) & 3;
                out[j] = d * (float)((lo | (h2 << 4)) - 32);
            }
            return;
        }
    } else {
        const uint8_t *row = w.p + (size_t)r * tiled_row_bytes(w.qtype, w.cols);
        codes = row + b * 16;
        d = __half2float(*reinterpret_cast<const __half *>(row + tiled_scale_off(w.qtype, w.cols) + b * 2));
        if (w.qtype == BRASA_Q6_0) {
            const uint32_t *hw = reinterpret_cast<const uint32_t *>(row + tiled_hi_off(w.cols) + b * 8);
            for (int j = 0; j < 32; ++j) {
                int byte = codes[j & 15];
                int lo = j < 16 ? (byte & 15) : (byte >> 4);
                int ww = (j & 15) >> 2, k = 2 * (j & 3) + (j >> 4);
                int h2 = (int)((hw[ww >> 1] >> q6_hi_bitpos(ww & 1, k)) & 3u);   // signed before the bias is removed
                out[j] = d * (float)((lo | (h2 << 4)) - 32);
            }
            return;
        }
        (void)hi;
    }
    // q4_0, either layout: 16 code bytes at `codes` (16-byte aligned only in the tiled layout)
    for (int j = 0; j < 16; ++j) {
        int byte = codes[j];
        out[j] = d * (float)((byte & 15) - 8);
        out[j + 16] = d * (float)((byte >> 4) - 8);
    }
}

constexpr int TM = 64;   // tokens per block
constexpr int TN = 64;   // weight rows per block
constexpr int TK = 32;   // one quantisation block per step
constexpr int LDH = TK + 8;

__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// F16 inputs, f32 accumulate. Block: 4 warps; warp w owns tokens [16w, 16w+16) x all 64 rows.
__global__ void __launch_bounds__(128) gemm_f16_kernel(WView w, const __half *x, float *y, uint32_t tokens) {
    __shared__ __align__(16) __half xs[TM * LDH];
    __shared__ __align__(16) __half ws[TN * LDH];
    const uint32_t row0 = blockIdx.x * TN, tok0 = blockIdx.y * TM;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
    float acc[8][4];
    for (int i = 0; i < 8; ++i)
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    const uint32_t nb = w.cols / 32;
    for (uint32_t b = 0; b < nb; ++b) {
        // X tile: 64 tokens x 32 halves = 64 x 4 uint4
        for (int i = t; i < TM * 4; i += 128) {
            uint32_t r = i >> 2, v = i & 3;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (tok0 + r < tokens) val = reinterpret_cast<const uint4 *>(x + (size_t)(tok0 + r) * w.cols + b * 32)[v];
            *reinterpret_cast<uint4 *>(&xs[r * LDH + v * 8]) = val;
        }
        // W tile: 64 rows x 1 block, dequantised and rounded to f16
        if (t < TN) {
            float f[32];
            if (row0 + t < w.rows) dequant_block(w, row0 + t, b, f);
            else
                for (int j = 0; j < 32; ++j) f[j] = 0.0f;
            for (int j = 0; j < 32; j += 2) *reinterpret_cast<__half2 *>(&ws[t * LDH + j]) = __floats2half2_rn(f[j], f[j + 1]);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t a[4];
            const __half *xa = xs + (16 * warp + g) * LDH + ks * 16 + 2 * tq;
            a[0] = *reinterpret_cast<const uint32_t *>(xa);
            a[1] = *reinterpret_cast<const uint32_t *>(xa + 8 * LDH);
            a[2] = *reinterpret_cast<const uint32_t *>(xa + 8);
            a[3] = *reinterpret_cast<const uint32_t *>(xa + 8 * LDH + 8);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t bb[2];
                const __half *wb = ws + (8 * nt + g) * LDH + ks * 16 + 2 * tq;
                bb[0] = *reinterpret_cast<const uint32_t *>(wb);
                bb[1] = *reinterpret_cast<const uint32_t *>(wb + 8);
                mma16816(acc[nt], a, bb);
            }
        }
        __syncthreads();
    }
    for (int nt = 0; nt < 8; ++nt) {
        uint32_t col = row0 + 8 * nt + 2 * tq;
        uint32_t r0 = tok0 + 16 * warp + g, r1 = r0 + 8;
        if (col < w.rows) {
            if (r0 < tokens) { y[(size_t)r0 * w.rows + col] = acc[nt][0]; if (col + 1 < w.rows) y[(size_t)r0 * w.rows + col + 1] = acc[nt][1]; }
            if (r1 < tokens) { y[(size_t)r1 * w.rows + col] = acc[nt][2]; if (col + 1 < w.rows) y[(size_t)r1 * w.rows + col + 1] = acc[nt][3]; }
        }
    }
}

// F32 inputs and weights, f32 FMA. Block 16x16 threads, each 4 tokens x 4 rows.
__global__ void __launch_bounds__(256) gemm_f32_kernel(WView w, const float *x, float *y, uint32_t tokens) {
    __shared__ float xs[TM][TK + 1];
    __shared__ float ws[TN][TK + 1];
    const uint32_t row0 = blockIdx.x * TN, tok0 = blockIdx.y * TM;
    const int t = threadIdx.x, ty = t >> 4, tx = t & 15;
    float acc[4][4] = {};
    const uint32_t nb = w.cols / 32;
    for (uint32_t b = 0; b < nb; ++b) {
        for (int i = t; i < TM * TK; i += 256) {
            uint32_t r = i / TK, c = i % TK;
            xs[r][c] = tok0 + r < tokens ? x[(size_t)(tok0 + r) * w.cols + b * 32 + c] : 0.0f;
        }
        if (t < TN) {
            float f[32];
            if (row0 + t < w.rows) dequant_block(w, row0 + t, b, f);
            else
                for (int j = 0; j < 32; ++j) f[j] = 0.0f;
            for (int j = 0; j < 32; ++j) ws[t][j] = f[j];
        }
        __syncthreads();
        for (int k = 0; k < TK; ++k) {
            float xv[4], wv[4];
            for (int i = 0; i < 4; ++i) { xv[i] = xs[4 * ty + i][k]; wv[i] = ws[4 * tx + i][k]; }
            for (int i = 0; i < 4; ++i)
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) {
            uint32_t r = tok0 + 4 * ty + i, c = row0 + 4 * tx + j;
            if (r < tokens && c < w.rows) y[(size_t)r * w.rows + c] = acc[i][j];
        }
}

bool tc_enabled() {
    static const bool on = [] { const char *e = getenv("BRASA_GEMM_TC"); return !(e && e[0] == '0'); }();
    return on;
}

}  // namespace

// True when brasa_k_gemm_swiglu runs as one tensor-core launch for these matrices and token count (given an output that
// does not overlap the input). The model then hands it a separate output buffer.
bool brasa_gemm_swiglu_fuses(const brasa_qmatrix &wg, const brasa_qmatrix &wu, uint32_t tokens) {
    return tc_enabled() && tokens >= 128 && wg.rows == wu.rows && wg.cols == wu.cols && wg.qtype == BRASA_Q4_0 && wu.qtype == BRASA_Q4_0 &&
           qm_fits(wg) && qm_fits(wu) && brasa_gemm_tc_supported(wg, tokens) && brasa_gemm_tc_supported(wu, tokens);
}

extern "C" {

int32_t brasa_k_gemm_with(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens, int32_t precision) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    BRASA_REQUIRE(ctx, precision == BRASA_PREFILL_F16 || precision == BRASA_PREFILL_F32, "unknown precision %d", precision);
    BRASA_REQUIRE(ctx, w.qtype >= BRASA_Q4_0 && w.qtype <= BRASA_Q6_0 && w.cols % 32 == 0 && qm_fits(w), "gemm: bad matrix");
    if (w.layout == BRASA_LAYOUT_TILED) BRASA_REQUIRE(ctx, tiled_ok(w.qtype, w.rows, w.cols), "gemm: shape not valid for the tiled layout");
    bool half_in = precision == BRASA_PREFILL_F16;
    BRASA_REQUIRE(ctx, arg_fits(x, (uint64_t)tokens * w.cols * (half_in ? 2 : 4)) && arg_fits(y, (uint64_t)tokens * w.rows * 4), "gemm: x or y too small");
    BRASA_REQUIRE(ctx, x.offset % 16 == 0 && y.offset % 8 == 0, "gemm: misaligned x or y");
    if (tokens == 0) return BRASA_OK;
    if (half_in && tc_enabled() && tokens > 8 && brasa_gemm_tc_supported(w, tokens)) {
        float *yp = (float *)arg_ptr(y);
        return brasa_gemm_tc_launch(cmd, 1, &w, (const __half *)arg_ptr(x), &yp, tokens, nullptr, nullptr);
    }
    WView v{arg_ptr(w.data), w.qtype, w.layout, w.rows, w.cols};
    dim3 grid((w.rows + TN - 1) / TN, (tokens + TM - 1) / TM);
    if (half_in) gemm_f16_kernel<<<grid, 128, 0, ctx->stream>>>(v, (const __half *)arg_ptr(x), (float *)arg_ptr(y), tokens);
    else gemm_f32_kernel<<<grid, 256, 0, ctx->stream>>>(v, (const float *)arg_ptr(x), (float *)arg_ptr(y), tokens);
    return brasa_post_launch(cmd, "gemm");
}

// acc += W X for f16 inputs (the residual add of a layer folded into the GEMM's epilogue when the tensor-core kernel
// takes the product; otherwise the product goes to `scratch` and is added by the element-wise kernel).
int32_t brasa_k_gemm_add(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg acc, brasa_arg scratch, uint32_t tokens) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    const uint64_t n = (uint64_t)tokens * w.rows;
    BRASA_REQUIRE(ctx, arg_fits(acc, n * 4) && arg_fits(scratch, n * 4), "gemm_add: acc or scratch too small");
    if (tokens == 0) return BRASA_OK;
    if (tc_enabled() && tokens > 8 && w.qtype >= BRASA_Q4_0 && w.qtype <= BRASA_Q6_0 && qm_fits(w) && brasa_gemm_tc_supported(w, tokens) &&
        arg_fits(x_f16, (uint64_t)tokens * w.cols * 2) && x_f16.offset % 16 == 0 && acc.offset % 16 == 0) {
        float *yp = (float *)arg_ptr(acc);
        return brasa_gemm_tc_launch(cmd, 1, &w, (const __half *)arg_ptr(x_f16), &yp, tokens, yp, nullptr);
    }
    BRASA_TRY(brasa_k_gemm_with(cmd, w, x_f16, scratch, tokens, BRASA_PREFILL_F16));
    return brasa_k_add(cmd, acc, scratch, acc, n);
}

// acc += W x, then out = f16(rms_norm(acc) * norm_w): the residual add of a layer and the norm that opens the next block.
// One GEMM and one kernel behind it when the few-token tensor-core kernel takes the product; otherwise the two calls.
int32_t brasa_k_gemm_add_rms_norm_f16(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg acc, brasa_arg scratch, brasa_arg norm_w, brasa_arg out_f16,
                                    uint32_t tokens, float eps) {
    if (!cmd) return BRASA_EINVAL;
    brasa_ctx *ctx = cmd->ctx;
    const uint64_t n = (uint64_t)tokens * w.rows;
    if (tc_enabled() && tokens >= 2 && tokens > 8 && qm_fits(w) && brasa_gemm_tc_few_tokens(ctx, &w, 1, tokens) && w.rows % 512 == 0 && w.rows <= 5120 &&
        arg_fits(x_f16, (uint64_t)tokens * w.cols * 2) && arg_fits(acc, n * 4) && arg_fits(out_f16, n * 2) && arg_fits(norm_w, (uint64_t)w.rows * 4) &&
        x_f16.offset % 16 == 0 && acc.offset % 16 == 0 && out_f16.offset % 16 == 0 && norm_w.offset % 16 == 0)
        return brasa_gemm_tc_add_norm(cmd, w, (const __half *)arg_ptr(x_f16), (float *)arg_ptr(acc), (const float *)arg_ptr(norm_w),
                                      (__half *)arg_ptr(out_f16), tokens, eps);
    BRASA_TRY(brasa_k_gemm_add(cmd, w, x_f16, acc, scratch, tokens));
    return brasa_k_rms_norm_f16(cmd, acc, norm_w, out_f16, tokens, w.rows, eps);
}

int32_t brasa_k_gemm(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg y, uint32_t tokens) {
    return brasa_k_gemm_with(cmd, w, x_f16, y, tokens, BRASA_PREFILL_F16);
}

int32_t brasa_k_gemm_multi(brasa_cmd *cmd, const brasa_qmatrix *ws, uint32_t count, brasa_arg x, const brasa_arg *ys, uint32_t tokens,
                           int32_t precision) {
    if (!cmd || !ws || !ys) return BRASA_EINVAL;
    BRASA_REQUIRE(cmd->ctx, count >= 1 && count <= 3, "gemm_multi: 1 to 3 matrices");
    // one tensor-core launch for all of them when every matrix qualifies
    bool all_tc = precision == BRASA_PREFILL_F16 && tc_enabled() && tokens > 8;
    for (uint32_t i = 0; i < count && all_tc; ++i)
        all_tc = brasa_gemm_tc_supported(ws[i], tokens) && (count == 1 || ws[i].qtype == BRASA_Q4_0) && ws[i].cols == ws[0].cols && qm_fits(ws[i]) &&
                 arg_fits(x, (uint64_t)tokens * ws[i].cols * 2) && arg_fits(ys[i], (uint64_t)tokens * ws[i].rows * 4) && ys[i].offset % 16 == 0;
    if (all_tc && x.offset % 16 == 0) {
        float *yp[3] = {nullptr, nullptr, nullptr};
        for (uint32_t i = 0; i < count; ++i) yp[i] = (float *)arg_ptr(ys[i]);
        return brasa_gemm_tc_launch(cmd, count, ws, (const __half *)arg_ptr(x), yp, tokens, nullptr, nullptr);
    }
    for (uint32_t i = 0; i < count; ++i) {
        BRASA_REQUIRE(cmd->ctx, ws[i].cols == ws[0].cols, "gemm_multi: matrices must share the input");
        BRASA_TRY(brasa_k_gemm_with(cmd, ws[i], x, ys[i], tokens, precision));
    }
    return BRASA_OK;
}

int32_t brasa_k_gemm_swiglu(brasa_cmd *cmd, brasa_qmatrix wg, brasa_qmatrix wu, brasa_arg x_f16, brasa_arg gate, brasa_arg up, brasa_arg out_f16,
                            uint32_t tokens) {
    if (!cmd) return BRASA_EINVAL;
    BRASA_REQUIRE(cmd->ctx, wg.rows == wu.rows && wg.cols == wu.cols, "gemm_swiglu: gate and up shapes");
    // many tokens: one tensor-core launch whose epilogue forms silu(gate) * up (gate and up are then not written). The
    // output must not share memory with the input: other CTAs still read X while the first results are stored.
    const bool apart = x_f16.buf != out_f16.buf || x_f16.offset + (uint64_t)tokens * wg.cols * 2 <= out_f16.offset ||
                       out_f16.offset + (uint64_t)tokens * wg.rows * 2 <= x_f16.offset;
    if (apart && brasa_gemm_swiglu_fuses(wg, wu, tokens) && arg_fits(x_f16, (uint64_t)tokens * wg.cols * 2) &&
        arg_fits(out_f16, (uint64_t)tokens * wg.rows * 2) && x_f16.offset % 16 == 0 && out_f16.offset % 16 == 0) {
        const brasa_qmatrix ws[2] = {wg, wu};
        return brasa_gemm_tc_launch(cmd, 2, ws, (const __half *)arg_ptr(x_f16), nullptr, tokens, nullptr, (__half *)arg_ptr(out_f16));
    }
    // (few tokens: gate and up in one launch when the tensor-core kernel takes both, so that its runs cover all the SMs)
    const brasa_qmatrix both[2] = {wg, wu};
    if (tc_enabled() && tokens > 8 && qm_fits(wg) && qm_fits(wu) && brasa_gemm_tc_few_tokens(cmd->ctx, both, 2, tokens) &&
        arg_fits(x_f16, (uint64_t)tokens * wg.cols * 2) && arg_fits(out_f16, (uint64_t)tokens * wg.rows * 2) && x_f16.offset % 16 == 0 &&
        out_f16.offset % 16 == 0)  // its SwiGLU is formed by the kernel that adds up the blocks' partial tiles (the output may be X itself)
        return brasa_gemm_tc_launch(cmd, 2, both, (const __half *)arg_ptr(x_f16), nullptr, tokens, nullptr, (__half *)arg_ptr(out_f16));
    const brasa_arg outs[2] = {gate, up};
    BRASA_TRY(brasa_k_gemm_multi(cmd, both, 2, x_f16, outs, tokens, BRASA_PREFILL_F16));
    return brasa_k_swiglu_f16(cmd, gate, up, out_f16, (uint64_t)tokens * wg.rows);
}

}  // extern "C"
