// Qwen3 dense model and generation session on the device
// (crates/models/src/qwen3.rs, crates/runtime/src/session.rs).
//
// Per layer (T tokens from position pos0):
//   h = RMSNorm(x); q, k, v = W h; q, k = per-head RMSNorm then RoPE; K, V -> cache;
//   o = attention(q, K, V); x += Wo o; h = RMSNorm(x); x += Wdown (silu(Wgate h) * Wup h)
// Activations are f32. With more than GEMV_MAX_TOKENS tokens the projections run as GEMMs whose
// inputs are f16 (PrefillPrecision::F16) and attention takes Q*scale in f16; with fewer they run as
// GEMVs on f32 inputs. One token takes the fused decode path: RMSNorm folded into the GEMVs, the
// residual adds folded into the next GEMV's input stage.
#include <string.h>
#include <unistd.h>

#include <chrono>
#include <thread>

#include "brasa_internal.h"
#include "decode_token.h"
#include "host_util.h"
#include "model_internal.h"

int32_t brasa_argmax_launch(brasa_cmd *cmd, const float *logits, uint32_t n, uint32_t *out);
void brasa_gemv_hint_next(brasa_ctx *ctx, uint32_t nmat, const brasa_qmatrix *w, bool swiglu);
int32_t brasa_advance_launch(brasa_cmd *cmd, uint32_t *ids, const uint32_t *next, uint32_t *out_ids, uint32_t *out_count, uint32_t out_cap,
                             uint32_t *pos);
int32_t brasa_attn_decode_fused_launch(brasa_cmd *cmd, int32_t kv, const float *q, const float *k_new, const float *v_new, const float *q_norm,
                                       const float *k_norm, const float *cos_t, const float *sin_t, uint8_t *kc, uint8_t *vc, float *partials,
                                       uint32_t *counters, float *o, const uint32_t *pos, uint32_t hq, uint32_t hkv, uint32_t ctx_len, float eps);

namespace {

int32_t cfg_from_json(brasa_ctx *ctx, const brasa::Json &c, brasa_config *out, std::string &err) {
    auto u = [&](const char *k, uint32_t *v) {
        const brasa::Json *j = c.get(k);
        if (!j || j->kind != brasa::Json::Num) {
            err = std::string("config.json: missing ") + k;
            return false;
        }
        *v = (uint32_t)j->inum;
        return true;
    };
    const brasa::Json *mt = c.get("model_type");
    if (!mt || mt->kind != brasa::Json::Str || mt->str != "qwen3") {
        err = "model_type is not qwen3";
        return false;
    }
    const brasa::Json *tie = c.get("tie_word_embeddings");
    out->tied = (tie && tie->kind == brasa::Json::Bool && tie->b) ? 1 : 0;
    if (!u("hidden_size", &out->hidden) || !u("num_hidden_layers", &out->layers) || !u("num_attention_heads", &out->heads) ||
        !u("num_key_value_heads", &out->kv_heads) || !u("head_dim", &out->head_dim) || !u("intermediate_size", &out->ffn) ||
        !u("vocab_size", &out->vocab) || !u("max_position_embeddings", &out->max_position))
        return false;
    const brasa::Json *e = c.get("rms_norm_eps"), *th = c.get("rope_theta");
    out->eps = e && e->kind == brasa::Json::Num ? (float)e->num : 1e-6f;
    out->rope_theta = th && th->kind == brasa::Json::Num ? th->num : 1e6;
    // a tensor-parallel shard names the vocabulary row its lm_head starts at; the row count comes from the tensor
    const brasa::Json *off = c.get("tp_vocab_offset");
    out->head_rows = out->vocab;
    out->head_row0 = off && off->kind == brasa::Json::Num ? (uint32_t)off->inum : 0;
    (void)ctx;
    return true;
}

}  // namespace

// File bytes -> device through two pinned buffers (crates/quant/src/brasa_file.rs:64-131 hands out slices of a mapped
// file; a GPU cannot read those, and a copy straight from pageable memory is staged by the driver one small buffer at a
// time, after a page fault per 4 KiB of the mapping). Here several host threads pread the file into a pinned chunk (no
// page of the mapping is touched) while the previous chunk travels by DMA, and nothing waits for the device except the
// reuse of a chunk: tensors follow one another on the stream.
struct brasa_model_detail::Stager {
    static constexpr size_t CHUNK = 32u << 20;
    static constexpr int THREADS = 4;
    brasa_ctx *ctx = nullptr;
    uint8_t *pin[2] = {nullptr, nullptr};
    cudaEvent_t idle[2] = {nullptr, nullptr};
    int next = 0;
    uint64_t bytes = 0;

    int32_t init(brasa_ctx *c) {
        ctx = c;
        for (int i = 0; i < 2; ++i) {
            BRASA_CUDA(ctx, cudaMallocHost((void **)&pin[i], CHUNK));
            BRASA_CUDA(ctx, cudaEventCreateWithFlags(&idle[i], cudaEventDisableTiming));
        }
        return BRASA_OK;
    }
    ~Stager() {
        for (int i = 0; i < 2; ++i) {
            if (idle[i]) {
                cudaEventSynchronize(idle[i]);
                cudaEventDestroy(idle[i]);
            }
            if (pin[i]) cudaFreeHost(pin[i]);
        }
    }
    // n bytes of the file at offset file_off (also mapped at src) -> dst (device), asynchronously on the context's stream
    int32_t upload(void *dst, int fd, uint64_t file_off, const uint8_t *src, size_t n) {
        bool failed = false;
        auto fetch = [&failed, fd, file_off, src](uint8_t *to, size_t at, size_t len) {
            size_t done = 0;
            while (fd >= 0 && done < len) {
                const ssize_t r = pread(fd, to + done, len - done, (off_t)(file_off + at + done));
                if (r <= 0) break;
                done += (size_t)r;
            }
            if (done < len) {
                if (src) memcpy(to + done, src + at + done, len - done);
                else failed = true;
            }
        };
        for (size_t off = 0; off < n; off += CHUNK) {
            const size_t len = std::min(CHUNK, n - off);
            const int i = next;
            next ^= 1;
            BRASA_CUDA(ctx, cudaEventSynchronize(idle[i]));  // the copy that last used this chunk has left it
            if (len >= (4u << 20)) {
                std::thread workers[THREADS];
                const size_t piece = (len / THREADS + 4095) & ~(size_t)4095;
                for (int t = 0; t < THREADS; ++t) {
                    const size_t b = std::min(len, piece * t), e = std::min(len, piece * (t + 1));
                    workers[t] = std::thread([=, &fetch] { if (e > b) fetch(pin[i] + b, off + b, e - b); });
                }
                for (auto &w : workers) w.join();
            } else {
                fetch(pin[i], off, len);
            }
            if (failed) return brasa_fail(ctx, BRASA_EIO, "reading the model file failed");
            BRASA_CUDA(ctx, cudaMemcpyAsync((uint8_t *)dst + off, pin[i], len, cudaMemcpyHostToDevice, ctx->stream));
            BRASA_CUDA(ctx, cudaEventRecord(idle[i], ctx->stream));
        }
        bytes += n;
        return BRASA_OK;
    }
};

namespace {

int32_t alloc_buf(brasa_model *m, uint64_t bytes, brasa_buf **out, uint64_t *account) {
    BRASA_TRY(brasa_buf_alloc(m->ctx, bytes, out));
    m->owned.push_back(*out);
    if (account) *account += brasa_plan_buffer_bytes(bytes);
    return BRASA_OK;
}

int32_t load_f32(brasa_model *m, const brasa::BrasaFile &f, const std::string &name, uint64_t n, brasa_buf **out) {
    brasa_ctx *ctx = m->ctx;
    const brasa::TensorInfo *t = f.tensor(name);
    if (!t) return brasa_fail(ctx, BRASA_EIO, "missing tensor %s", name.c_str());
    if (t->dtype != "f32" || t->numel() != n) return brasa_fail(ctx, BRASA_EIO, "%s: expected %llu f32 values", name.c_str(), (unsigned long long)n);
    BRASA_TRY(alloc_buf(m, t->nbytes, out, &m->alloc.weights));
    return m->stager->upload((*out)->ptr, f.fd(), t->offset, f.data(*t), t->nbytes);
}

// Uploads a quantised matrix and regroups it into the tiled layout when its shape allows.
int32_t load_matrix(brasa_model *m, brasa_cmd *load_cmd, const brasa::BrasaFile &f, const std::string &name, uint32_t rows, uint32_t cols, brasa_buf *staging,
                    Matrix *out) {
    brasa_ctx *ctx = m->ctx;
    const brasa::TensorInfo *t = f.tensor(name);
    if (!t) return brasa_fail(ctx, BRASA_EIO, "missing tensor %s", name.c_str());
    int qt = brasa::dtype_qtype(t->dtype);
    if (qt < 0) return brasa_fail(ctx, BRASA_EIO, "%s: expected a quantised tensor", name.c_str());
    if (t->shape.size() != 2 || t->shape[0] != rows || t->shape[1] != cols)
        return brasa_fail(ctx, BRASA_EIO, "%s: unexpected shape", name.c_str());
    BRASA_TRY(alloc_buf(m, t->nbytes, &out->buf, &m->alloc.weights));
    out->q.data = A(out->buf);
    out->q.qtype = qt;
    out->q.rows = rows;
    out->q.cols = cols;
    if (tiled_ok(qt, rows, cols)) {
        if (brasa_buf_bytes(staging) < t->nbytes) return brasa_fail(ctx, BRASA_EINVAL, "staging buffer too small for %s", name.c_str());
        // the file's bytes into the device staging buffer, regrouped from there; the next tensor's upload follows the
        // regrouping on the same stream, so the host never waits here
        BRASA_TRY(m->stager->upload(staging->ptr, f.fd(), t->offset, f.data(*t), t->nbytes));
        BRASA_TRY(brasa_k_repack(load_cmd, qt, A(staging), A(out->buf), rows, cols));
        out->q.layout = BRASA_LAYOUT_TILED;
    } else {
        BRASA_TRY(m->stager->upload(out->buf->ptr, f.fd(), t->offset, f.data(*t), t->nbytes));
        out->q.layout = BRASA_LAYOUT_FILE;
    }
    return BRASA_OK;
}

struct KvView {
    brasa_arg k, v;
};
// K and V of layer li from position pos.
KvView kv_at(brasa_model *m, uint32_t li, uint32_t pos) {
    uint64_t kvd = (uint64_t)m->cfg.kv_heads * m->cfg.head_dim;
    uint64_t off = brasa_kv_bytes(m->limits.kv, ((uint64_t)li * m->cap + pos) * kvd);
    return KvView{A(m->kc, off), A(m->vc, off)};
}

int32_t matmul(brasa_model *m, brasa_cmd *cmd, const Matrix &w, brasa_arg x, brasa_arg y, uint32_t tokens, bool x_is_half) {
    if (tokens <= GEMV_MAX_TOKENS) return brasa_k_gemv(cmd, w.q, x, y, tokens);
    return brasa_k_gemm_with(cmd, w.q, x, y, tokens, x_is_half ? BRASA_PREFILL_F16 : BRASA_PREFILL_F32);
}

int32_t precision_for(brasa_model *m, uint32_t tokens) { return tokens <= GEMV_MAX_TOKENS ? BRASA_PREFILL_F32 : m->prefill_precision; }

// x += h for n values: the plain add on one device, the sum over ranks of every rank's h for a tensor-parallel shard.
int32_t residual_add(brasa_model *m, brasa_cmd *cmd, uint64_t n) {
    if (m->tp) return brasa_k_tp_allreduce_add(cmd, m->tp, A(m->h), A(m->x), A(m->x), n);
    return brasa_k_add(cmd, A(m->x), A(m->h), A(m->x), n);
}

// Layer li for `tokens` > 1 tokens from pos0 (also used for a single token by run_layers when asked
// for the unfused order). Input and output in ws.x.
int32_t encode_layer_prefill(brasa_model *m, brasa_cmd *cmd, uint32_t li, uint32_t tokens, uint32_t pos0) {
    const brasa_config &c = m->cfg;
    Layer &l = m->layers[li];
    const bool half_io = precision_for(m, tokens) == BRASA_PREFILL_F16;
    const uint32_t H = c.hidden;
    brasa_arg xin;
    if (half_io) {
        BRASA_TRY(brasa_k_rms_norm_f16(cmd, A(m->x), A(l.attn_norm), A(m->xh), tokens, H, c.eps));
        xin = A(m->xh);
    } else {
        BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x), A(l.attn_norm), A(m->norm_out), tokens, H, c.eps));
        xin = A(m->norm_out);
    }
    if (tokens > GEMV_MAX_TOKENS) {  // one launch for q, k and v where the kernels allow it
        brasa_qmatrix wqkv[3] = {l.wq.q, l.wk.q, l.wv.q};
        brasa_arg yqkv[3] = {A(m->q), A(m->k_new), A(m->v_new)};
        BRASA_TRY(brasa_k_gemm_multi(cmd, wqkv, 3, xin, yqkv, tokens, half_io ? BRASA_PREFILL_F16 : BRASA_PREFILL_F32));
    } else {
        BRASA_TRY(matmul(m, cmd, l.wq, xin, A(m->q), tokens, half_io));
        BRASA_TRY(matmul(m, cmd, l.wk, xin, A(m->k_new), tokens, half_io));
        BRASA_TRY(matmul(m, cmd, l.wv, xin, A(m->v_new), tokens, half_io));
    }
    brasa_attn_shape sh{tokens, c.heads, c.kv_heads, c.head_dim, pos0, m->limits.kv};
    KvView dst = kv_at(m, li, pos0), all = kv_at(m, li, 0);
    brasa_arg qkv[3] = {A(m->q), A(m->k_new), A(m->v_new)}, norms[2] = {A(l.q_norm), A(l.k_norm)}, dsts[2] = {dst.k, dst.v};
    BRASA_TRY(brasa_k_qk_norm_rope_store(cmd, m->limits.kv, qkv, norms, c.eps, A(m->rope_cos), A(m->rope_sin), c.head_dim, m->limits.ctx, dsts, sh));
    brasa_arg attn = half_io ? A(m->xh) : A(m->attn);
    if (tokens == 1) {
        BRASA_TRY(brasa_k_decode_attention(cmd, A(m->q), all.k, all.v, A(m->partials), m->partials_len, A(m->attn), sh));
    } else {
        BRASA_TRY(brasa_k_flash_attention_with(cmd, A(m->q), all.k, all.v, attn, sh, half_io ? BRASA_PREFILL_F16 : BRASA_PREFILL_F32));
    }
    if (half_io && !m->tp) BRASA_TRY(brasa_k_gemm_add(cmd, l.wo.q, attn, A(m->x), A(m->h), tokens));  // x += Wo attn in the GEMM's epilogue
    else {
        BRASA_TRY(matmul(m, cmd, l.wo, attn, A(m->h), tokens, half_io));
        BRASA_TRY(residual_add(m, cmd, (uint64_t)tokens * H));
    }
    brasa_arg act;
    if (half_io) {
        BRASA_TRY(brasa_k_rms_norm_f16(cmd, A(m->x), A(l.ffn_norm), A(m->xh), tokens, H, c.eps));
        // one fused launch writes the f16 activations while X is still being read: they go to the (then unused) up buffer
        act = brasa_gemm_swiglu_fuses(l.gate.q, l.up.q, tokens) ? A(m->up) : A(m->xh);
        BRASA_TRY(brasa_k_gemm_swiglu(cmd, l.gate.q, l.up.q, A(m->xh), A(m->gate), A(m->up), act, tokens));
    } else {
        BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x), A(l.ffn_norm), A(m->norm_out), tokens, H, c.eps));
        BRASA_TRY(matmul(m, cmd, l.gate, A(m->norm_out), A(m->gate), tokens, false));
        BRASA_TRY(matmul(m, cmd, l.up, A(m->norm_out), A(m->up), tokens, false));
        BRASA_TRY(brasa_k_swiglu(cmd, A(m->gate), A(m->up), A(m->gate), (uint64_t)tokens * c.ffn));
        act = A(m->gate);
    }
    if (half_io && !m->tp) return brasa_k_gemm_add(cmd, l.down.q, act, A(m->x), A(m->h), tokens);
    BRASA_TRY(matmul(m, cmd, l.down, act, A(m->h), tokens, half_io));
    return residual_add(m, cmd, (uint64_t)tokens * H);
}

bool decode_fused_ok(brasa_model *m) {
    for (Layer &l : m->layers)
        for (const Matrix *w : {&l.wq, &l.wk, &l.wv, &l.wo, &l.gate, &l.up, &l.down})
            if (w->q.layout != BRASA_LAYOUT_TILED || w->q.qtype != BRASA_Q4_0) return false;
    return m->head.q.layout == BRASA_LAYOUT_TILED && (m->head.q.qtype == BRASA_Q4_0 || m->head.q.qtype == BRASA_Q6_0) &&
           m->cfg.heads / m->cfg.kv_heads <= 8;
}

// One token through layers [layer_begin, layer_end), fused decode order, in place on ws.x:
//   q, k, v = W (RMSNorm(x));  attention;  x += Wo attn;  act = silu(Wg n) * (Wu n), n = RMSNorm(x);  x += Wd act
// RMSNorm is folded into the GEMV that consumes it and the residual adds into the GEMV that produces
// the addend. with_head adds the final norm and the lm_head GEMV into ws.logits. The position is read by
// the attention kernel from dev_state[0], so the same sequence of launches serves every step.
int32_t encode_decode_token(brasa_model *m, brasa_cmd *cmd, uint32_t layer_begin, uint32_t layer_end, bool with_head) {
    const brasa_config &c = m->cfg;
    enum { SCALE = 0, SWIGLU = 1, RESID = 2 };  // epilogues of brasa_gemv_launch
    float *x = F(m->x);
    for (uint32_t li = layer_begin; li < layer_end; ++li) {
        Layer &l = m->layers[li];
        {
            brasa_qmatrix w[3] = {l.wq.q, l.wk.q, l.wv.q};
            float *y[3] = {F(m->q), F(m->k_new), F(m->v_new)};
            brasa_gemv_hint_next(m->ctx, 1, &l.wo.q, false);
            BRASA_TRY(brasa_gemv_launch(cmd, BRASA_Q4_0, 3, w, y, x, nullptr, F(l.attn_norm), nullptr, nullptr, 0, 1, c.eps, SCALE, nullptr));
        }
        KvView all = kv_at(m, li, 0);
        uint32_t *st = (uint32_t *)m->dev_state->ptr;
        BRASA_TRY(brasa_attn_decode_fused_launch(cmd, m->limits.kv, F(m->q), F(m->k_new), F(m->v_new), F(l.q_norm), F(l.k_norm), F(m->rope_cos),
                                                 F(m->rope_sin), arg_ptr(all.k), arg_ptr(all.v), F(m->partials), st + 4, F(m->attn), st,
                                                 c.heads, c.kv_heads, m->limits.ctx, c.eps));
        {
            float *y[1] = {x};
            brasa_qmatrix nxt[2] = {l.gate.q, l.up.q};
            brasa_gemv_hint_next(m->ctx, 2, nxt, true);
            if (m->tp) {  // this rank's part of Wo attn, then the sum over ranks lands in x
                BRASA_TRY(brasa_tp_gemv_allreduce_launch(cmd, m->tp, l.wo.q, F(m->attn), x, x, 3));
            } else
            BRASA_TRY(brasa_gemv_launch(cmd, BRASA_Q4_0, 1, &l.wo.q, y, F(m->attn), nullptr, nullptr, nullptr, nullptr, 0, 0, 0.0f, RESID, x));
        }
        {
            brasa_qmatrix w[2] = {l.gate.q, l.up.q};
            float *y[2] = {F(m->gate), nullptr};
            brasa_gemv_hint_next(m->ctx, 1, &l.down.q, false);
            BRASA_TRY(brasa_gemv_launch(cmd, BRASA_Q4_0, 2, w, y, x, nullptr, F(l.ffn_norm), nullptr, nullptr, 0, 1, c.eps, SWIGLU, nullptr));
        }
        {
            float *y[1] = {x};
            if (li + 1 < layer_end) {
                Layer &nl = m->layers[li + 1];
                brasa_qmatrix nxt[3] = {nl.wq.q, nl.wk.q, nl.wv.q};
                brasa_gemv_hint_next(m->ctx, 3, nxt, false);
            } else if (with_head) {
                brasa_gemv_hint_next(m->ctx, 1, &m->head.q, false);
            }
            if (m->tp) {
                BRASA_TRY(brasa_tp_gemv_allreduce_launch(cmd, m->tp, l.down.q, F(m->gate), x, x, 3));
            } else
            BRASA_TRY(brasa_gemv_launch(cmd, BRASA_Q4_0, 1, &l.down.q, y, F(m->gate), nullptr, nullptr, nullptr, nullptr, 0, 0, 0.0f, RESID, x));
        }
    }
    if (with_head) {
        float *y[1] = {F(m->logits)};
        BRASA_TRY(brasa_gemv_launch(cmd, m->head.q.qtype, 1, &m->head.q, y, x, nullptr, F(m->final_norm), nullptr, nullptr, 0, 1, c.eps, SCALE, nullptr));
    }
    return BRASA_OK;
}

int32_t check_tokens(brasa_model *m, uint32_t tokens, uint32_t pos0) {
    if (tokens == 0 || tokens > m->limits.max_tokens)
        return brasa_fail(m->ctx, BRASA_EINVAL, "%u tokens per forward; the maximum is %u", tokens, m->limits.max_tokens);
    if ((uint64_t)pos0 + tokens > m->limits.ctx)
        return brasa_fail(m->ctx, BRASA_EINVAL, "position %llu outside the context (%u)", (unsigned long long)pos0 + tokens, m->limits.ctx);
    return BRASA_OK;
}

// One full decode step for the token in ws.ids[0] at position pos0: embed, layers, lm_head, argmax into
// next_id, then "advance" (next_id -> ids[0] and the output list, position + 1). The first call runs the
// kernels directly and records them; later calls replay the CUDA graph.
int32_t decode_step_kernels(brasa_model *m, brasa_cmd *cmd) {
    uint32_t *st = (uint32_t *)m->dev_state->ptr;
    BRASA_TRY(brasa_k_embed(cmd, m->embed.q, A(m->ids), A(m->x), 1));
    BRASA_TRY(encode_decode_token(m, cmd, 0, m->cfg.layers, true));
    if (m->tp) BRASA_TRY(brasa_k_tp_argmax(cmd, m->tp, A(m->logits), m->cfg.head_rows, m->cfg.head_row0, A(m->next_id)));
    else BRASA_TRY(brasa_argmax_launch(cmd, F(m->logits), m->cfg.head_rows, (uint32_t *)m->next_id->ptr));
    return brasa_advance_launch(cmd, (uint32_t *)m->ids->ptr, (const uint32_t *)m->next_id->ptr, (uint32_t *)m->out_ids->ptr, st + 1,
                                m->limits.ctx, st);
}

int32_t set_position(brasa_model *m, uint32_t pos0) {
    return brasa_check_cuda(m->ctx, cudaMemcpyAsync(m->dev_state->ptr, &pos0, 4, cudaMemcpyHostToDevice, m->ctx->stream), "position upload");
}

// Describes the model to the whole-token kernel and builds its program, once. Leaves token_prog null when the
// shapes do not fit or BRASA_TOKEN_KERNEL=0 asks for the kernel-per-operation path.
int32_t make_token_program(brasa_model *m) {
    m->token_prog_tried = true;
    brasa_tp_token_area area{};
    if (m->tp) {
        if (!brasa_tp_token_area_get(m->tp, &area)) return BRASA_OK;  // not connected yet: the kernel-per-operation path
    } else if (m->cfg.head_rows != m->cfg.vocab) {
        return BRASA_OK;  // a shard without its exchange cannot choose a token
    }
    if (!m->ctx->token_kernel) return BRASA_OK;
    const brasa_config &c = m->cfg;
    brasa_token_model d{};
    d.hidden = c.hidden; d.heads = c.heads; d.kv_heads = c.kv_heads; d.head_dim = c.head_dim; d.ffn = c.ffn; d.vocab = c.vocab;
    d.cache_positions = m->cap;
    d.kv = m->limits.kv;
    d.eps = c.eps;
    for (uint32_t li = 0; li < c.layers; ++li) {
        Layer &l = m->layers[li];
        KvView all = kv_at(m, li, 0);
        d.layers.push_back(brasa_token_layer{l.wq.q, l.wk.q, l.wv.q, l.wo.q, l.gate.q, l.up.q, l.down.q, F(l.attn_norm), F(l.q_norm), F(l.k_norm),
                                             F(l.ffn_norm), arg_ptr(all.k), arg_ptr(all.v)});
    }
    d.embed = m->embed.q;
    d.head = m->head.q;
    d.final_norm = F(m->final_norm);
    d.cos_t = F(m->rope_cos);
    d.sin_t = F(m->rope_sin);
    d.state = (uint32_t *)m->dev_state->ptr;
    d.ids = (uint32_t *)m->ids->ptr;
    d.next_id = (uint32_t *)m->next_id->ptr;
    d.out_ids = (uint32_t *)m->out_ids->ptr;
    d.out_cap = m->limits.ctx;
    d.logits = F(m->logits);
    d.head_row0 = m->cfg.head_row0;
    d.tp = area;
    if (!brasa_token_program_supported(m->ctx, d)) return BRASA_OK;
    return brasa_token_program_create(m->ctx, d, &m->token_prog);
}

// pos0 == UINT32_MAX keeps the position the device already holds (device-resident loop).
int32_t decode_step(brasa_model *m, brasa_cmd *cmd, uint32_t pos0) {
    if (pos0 != UINT32_MAX) BRASA_TRY(set_position(m, pos0));
    if (!m->token_prog_tried) BRASA_TRY(make_token_program(m));
    if (m->token_prog) return brasa_token_program_launch(cmd, m->token_prog);
    if (m->decode_graph) return brasa_graph_launch(cmd, m->decode_graph);
    BRASA_TRY(decode_step_kernels(m, cmd));
    if (m->ctx->graphs && !m->ctx->capturing) {
        // everything lazily created (scratch, function attributes) exists now: record the same sequence
        BRASA_TRY(brasa_graph_capture_begin(m->ctx));
        int32_t rc = decode_step_kernels(m, cmd);
        brasa_graph *g = nullptr;
        int32_t rc2 = brasa_graph_capture_end(m->ctx, &g);
        BRASA_TRY(rc);
        BRASA_TRY(rc2);
        m->decode_graph = g;
    }
    return BRASA_OK;
}

// Enqueues a whole forward for ids already in ws.ids; logits of the last logit_rows positions end
// up in ws.logits.
int32_t encode_forward(brasa_model *m, brasa_cmd *cmd, uint32_t tokens, uint32_t pos0, uint32_t logit_rows) {
    const brasa_config &c = m->cfg;
    if (tokens == 1 && decode_fused_ok(m)) return decode_step(m, cmd, pos0);
    BRASA_TRY(brasa_k_embed(cmd, m->embed.q, A(m->ids), A(m->x), tokens));
    for (uint32_t li = 0; li < c.layers; ++li) BRASA_TRY(encode_layer_prefill(m, cmd, li, tokens, pos0));
    uint32_t first = tokens - logit_rows;
    BRASA_TRY(brasa_k_rms_norm(cmd, A(m->x, (uint64_t)first * c.hidden * 4), A(m->final_norm), A(m->norm_out), logit_rows, c.hidden, c.eps));
    return brasa_k_gemv(cmd, m->head.q, A(m->norm_out), A(m->logits), logit_rows);
}

}  // namespace

extern "C" {

int32_t brasa_model_shape_from_file(const char *path, brasa_model_shape *shape, brasa_config *cfg, char *err, uint64_t err_len) {
    std::string e;
    auto f = brasa::BrasaFile::open(path ? path : "", e);
    brasa_config c{};
    if (f && f->family() != "qwen3") { e = "family " + f->family() + " is not supported"; f.reset(); }
    if (f && !cfg_from_json(nullptr, f->config(), &c, e)) f.reset();
    if (!f) {
        if (err && err_len) snprintf(err, (size_t)err_len, "%s", e.c_str());
        return BRASA_EIO;
    }
    if (shape) {
        uint64_t wb = 0;
        for (auto &t : f->tensors()) wb += brasa_plan_buffer_bytes(t.nbytes);
        *shape = brasa_model_shape{wb, c.layers, c.hidden, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab};
    }
    if (cfg) *cfg = c;
    if (err && err_len) err[0] = 0;
    return BRASA_OK;
}

void brasa_model_free(brasa_model *m) {
    if (!m) return;
    if (m->decode_graph) brasa_graph_free(m->decode_graph);
    brasa_token_program_free(m->token_prog);
    for (brasa_buf *b : m->owned) brasa_buf_free(b);
    if (m->pinned_id) cudaFreeHost(m->pinned_id);
    delete m;
}

int32_t brasa_model_load(brasa_ctx *ctx, const char *path, brasa_limits limits, brasa_model **out) {
    if (!ctx || !path || !out) return BRASA_EINVAL;
    *out = nullptr;
    std::string e;
    auto f = brasa::BrasaFile::open(path, e);
    if (!f) return brasa_fail(ctx, BRASA_EIO, "%s", e.c_str());
    if (f->family() != "qwen3") return brasa_fail(ctx, BRASA_EIO, "family %s is not supported", f->family().c_str());
    brasa_config c{};
    if (!cfg_from_json(ctx, f->config(), &c, e)) return brasa_fail(ctx, BRASA_EIO, "%s", e.c_str());
    BRASA_REQUIRE(ctx, limits.ctx <= c.max_position, "context %u larger than the model's maximum (%u)", limits.ctx, c.max_position);
    BRASA_REQUIRE(ctx, limits.ctx > 0 && limits.max_tokens > 0 && limits.max_logit_rows > 0, "limits must be positive");
    BRASA_REQUIRE(ctx, limits.kv >= BRASA_KV_F32 && limits.kv <= BRASA_KV_Q8_0, "unknown KV type %d", limits.kv);
    BRASA_REQUIRE(ctx, c.head_dim == 128, "the kernels need head_dim 128 (got %u)", c.head_dim);
    BRASA_REQUIRE(ctx, c.kv_heads > 0 && c.heads % c.kv_heads == 0, "heads must be a multiple of kv heads");
    if (!c.tied && !f->tensor("lm_head.weight")) return brasa_fail(ctx, BRASA_EIO, "untied model without lm_head.weight");

    brasa_model *m = new brasa_model();
    m->ctx = ctx;
    m->cfg = c;
    m->limits = limits;
    int32_t rc = [&]() -> int32_t {
        const uint32_t H = c.hidden, qd = c.heads * c.head_dim, kvd = c.kv_heads * c.head_dim, ffn = c.ffn;
        uint64_t biggest = 0;
        for (auto &t : f->tensors()) biggest = std::max<uint64_t>(biggest, t.nbytes);
        brasa_buf *staging = nullptr;
        BRASA_TRY(brasa_buf_alloc(ctx, biggest, &staging));
        const auto t_load = std::chrono::steady_clock::now();
        Stager stager;
        BRASA_TRY(stager.init(ctx));
        m->stager = &stager;
        brasa_cmd *load_cmd = nullptr;
        BRASA_TRY(brasa_cmd_begin(ctx, &load_cmd));
        struct CmdGuard {  // the command is waited for and freed on every way out
            brasa_cmd *&c;
            brasa_model *m;
            ~CmdGuard() {
                if (c) brasa_cmd_wait(c, nullptr);
                m->stager = nullptr;
            }
        } guard{load_cmd, m};
        m->layers.resize(c.layers);
        for (uint32_t i = 0; i < c.layers; ++i) {
            auto n = [&](const char *s) { return "model.layers." + std::to_string(i) + "." + s; };
            Layer &l = m->layers[i];
            BRASA_TRY(load_f32(m, *f, n("input_layernorm.weight"), H, &l.attn_norm));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("self_attn.q_proj.weight"), qd, H, staging, &l.wq));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("self_attn.k_proj.weight"), kvd, H, staging, &l.wk));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("self_attn.v_proj.weight"), kvd, H, staging, &l.wv));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("self_attn.o_proj.weight"), H, qd, staging, &l.wo));
            BRASA_TRY(load_f32(m, *f, n("self_attn.q_norm.weight"), c.head_dim, &l.q_norm));
            BRASA_TRY(load_f32(m, *f, n("self_attn.k_norm.weight"), c.head_dim, &l.k_norm));
            BRASA_TRY(load_f32(m, *f, n("post_attention_layernorm.weight"), H, &l.ffn_norm));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("mlp.gate_proj.weight"), ffn, H, staging, &l.gate));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("mlp.up_proj.weight"), ffn, H, staging, &l.up));
            BRASA_TRY(load_matrix(m, load_cmd, *f, n("mlp.down_proj.weight"), H, ffn, staging, &l.down));
        }
        BRASA_TRY(load_matrix(m, load_cmd, *f, "model.embed_tokens.weight", c.vocab, H, staging, &m->embed));
        if (m->embed.q.qtype != BRASA_Q8_0 && m->embed.q.qtype != BRASA_Q6_0)
            return brasa_fail(ctx, BRASA_EIO, "the embedding table must be q8_0 or q6_0");
        if (c.tied) m->head = m->embed;
        else {
            const brasa::TensorInfo *ht = f->tensor("lm_head.weight");
            if (ht->shape.size() != 2 || ht->shape[0] == 0 || ht->shape[0] > c.vocab || m->cfg.head_row0 + ht->shape[0] > c.vocab)
                return brasa_fail(ctx, BRASA_EIO, "lm_head.weight: unexpected shape");
            m->cfg.head_rows = (uint32_t)ht->shape[0];
            BRASA_TRY(load_matrix(m, load_cmd, *f, "lm_head.weight", m->cfg.head_rows, H, staging, &m->head));
        }
        BRASA_TRY(load_f32(m, *f, "model.norm.weight", H, &m->final_norm));
        {
            brasa_cmd *c2 = load_cmd;
            load_cmd = nullptr;
            BRASA_TRY(brasa_cmd_wait(c2, nullptr));  // every tensor is on the device and regrouped
        }
        m->load_bytes = stager.bytes;
        m->load_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count();
        m->stager = nullptr;
        // staging is not part of the steady-state footprint
        m->owned.erase(std::remove(m->owned.begin(), m->owned.end(), staging), m->owned.end());
        BRASA_TRY(brasa_buf_free(staging));

        uint64_t *ws = &m->alloc.workspace;
        std::vector<float> cs((size_t)limits.ctx * c.head_dim / 2), sn(cs.size());
        BRASA_TRY(brasa_rope_table(c.rope_theta, c.head_dim, limits.ctx, cs.data(), sn.data()));
        BRASA_TRY(alloc_buf(m, cs.size() * 4, &m->rope_cos, ws));
        BRASA_TRY(alloc_buf(m, sn.size() * 4, &m->rope_sin, ws));
        BRASA_TRY(brasa_buf_upload(m->rope_cos, 0, cs.data(), cs.size() * 4));
        BRASA_TRY(brasa_buf_upload(m->rope_sin, 0, sn.data(), sn.size() * 4));

        const uint64_t t = limits.max_tokens;
        m->cap = (limits.ctx + BRASA_KV_ALIGN - 1) / BRASA_KV_ALIGN * BRASA_KV_ALIGN;
        uint64_t kv_elems = (uint64_t)c.layers * m->cap * kvd;
        BRASA_TRY(alloc_buf(m, brasa_kv_bytes(limits.kv, kv_elems), &m->kc, &m->alloc.kv));
        BRASA_TRY(alloc_buf(m, brasa_kv_bytes(limits.kv, kv_elems), &m->vc, &m->alloc.kv));
        BRASA_TRY(alloc_buf(m, t * H * 4, &m->x, ws));
        BRASA_TRY(alloc_buf(m, t * H * 4, &m->h, ws));
        BRASA_TRY(alloc_buf(m, t * H * 4, &m->norm_out, ws));
        BRASA_TRY(alloc_buf(m, t * qd * 4, &m->q, ws));
        BRASA_TRY(alloc_buf(m, t * qd * 4, &m->attn, ws));
        BRASA_TRY(alloc_buf(m, t * kvd * 4, &m->k_new, ws));
        BRASA_TRY(alloc_buf(m, t * kvd * 4, &m->v_new, ws));
        BRASA_TRY(alloc_buf(m, t * ffn * 4, &m->gate, ws));
        BRASA_TRY(alloc_buf(m, t * ffn * 4, &m->up, ws));
        BRASA_TRY(alloc_buf(m, 2 * t * std::max<uint64_t>(ffn, std::max<uint64_t>(qd, H)), &m->xh, ws));
        BRASA_TRY(alloc_buf(m, t * 4, &m->ids, ws));
        BRASA_TRY(alloc_buf(m, (uint64_t)brasa_norm_partials(H) * 4, &m->ss, ws));
        m->partials_len = brasa_decode_partials_len(c.heads, limits.ctx);
        BRASA_TRY(alloc_buf(m, m->partials_len * 4, &m->partials, ws));
        BRASA_TRY(alloc_buf(m, (uint64_t)limits.max_logit_rows * m->cfg.head_rows * 4, &m->logits, ws));
        BRASA_TRY(alloc_buf(m, 64, &m->next_id, nullptr));
        BRASA_TRY(alloc_buf(m, (uint64_t)limits.ctx * 4, &m->out_ids, nullptr));
        BRASA_TRY(alloc_buf(m, 256, &m->dev_state, nullptr));
        BRASA_CUDA(ctx, cudaHostAlloc((void **)&m->pinned_id, 64, cudaHostAllocDefault));
        return brasa_ctx_sync(ctx);
    }();
    if (rc != BRASA_OK) {
        std::string keep = ctx->last_error;
        brasa_model_free(m);
        ctx->last_error = keep;
        return rc;
    }
    *out = m;
    return BRASA_OK;
}

int32_t brasa_model_set_tp(brasa_model *m, brasa_tp *tp) {
    if (!m || !tp) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_REQUIRE(ctx, !m->decode_graph && !m->token_prog, "set_tp: attach the exchange before the first decode step");
    BRASA_REQUIRE(ctx, m->cfg.hidden % 2 == 0, "set_tp: odd hidden size");
    BRASA_REQUIRE(ctx, m->cfg.head_row0 == 0 || brasa_tp_world(tp) > 1, "set_tp: a shard with a vocabulary offset needs its peers");
    m->tp = tp;
    return BRASA_OK;
}

int32_t brasa_model_config(brasa_model *m, brasa_config *out) {
    if (!m || !out) return BRASA_EINVAL;
    *out = m->cfg;
    return BRASA_OK;
}
int32_t brasa_model_limits(brasa_model *m, brasa_limits *out) {
    if (!m || !out) return BRASA_EINVAL;
    *out = m->limits;
    return BRASA_OK;
}
int32_t brasa_model_allocated(brasa_model *m, brasa_allocated *out) {
    if (!m || !out) return BRASA_EINVAL;
    *out = m->alloc;
    return BRASA_OK;
}
int32_t brasa_model_load_stats(brasa_model *m, double *seconds, uint64_t *bytes) {
    if (!m) return BRASA_EINVAL;
    if (seconds) *seconds = m->load_seconds;
    if (bytes) *bytes = m->load_bytes;
    return BRASA_OK;
}
int32_t brasa_model_set_prefill_precision(brasa_model *m, int32_t precision) {
    if (!m) return BRASA_EINVAL;
    BRASA_REQUIRE(m->ctx, precision == BRASA_PREFILL_F16 || precision == BRASA_PREFILL_F32, "unknown precision %d", precision);
    m->prefill_precision = precision;
    return BRASA_OK;
}

int32_t brasa_model_forward(brasa_model *m, const uint32_t *ids, uint32_t tokens, uint32_t pos0, uint32_t logit_rows, float *logits,
                            double *gpu_seconds) {
    if (!m || !ids) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_TRY(check_tokens(m, tokens, pos0));
    BRASA_REQUIRE(ctx, logit_rows >= 1 && logit_rows <= std::min(tokens, m->limits.max_logit_rows), "logit_rows %u is not valid", logit_rows);
    for (uint32_t i = 0; i < tokens; ++i) BRASA_REQUIRE(ctx, ids[i] < m->cfg.vocab, "token id %u outside the vocabulary", ids[i]);
    BRASA_CUDA(ctx, cudaMemcpyAsync(m->ids->ptr, ids, (size_t)tokens * 4, cudaMemcpyHostToDevice, ctx->stream));
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = encode_forward(m, cmd, tokens, pos0, logit_rows);
    int32_t rc2 = brasa_cmd_wait(cmd, gpu_seconds);
    BRASA_TRY(rc);
    BRASA_TRY(rc2);
    if (logits) BRASA_TRY(brasa_buf_download(m->logits, 0, logits, (uint64_t)logit_rows * m->cfg.head_rows * 4));
    return BRASA_OK;
}

int32_t brasa_model_run_layers(brasa_model *m, float *x, uint32_t tokens, uint32_t pos0, uint32_t layer_begin, uint32_t layer_end) {
    if (!m || !x) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_TRY(check_tokens(m, tokens, pos0));
    BRASA_REQUIRE(ctx, layer_begin <= layer_end && layer_end <= m->cfg.layers, "layer range");
    uint64_t n = (uint64_t)tokens * m->cfg.hidden * 4;
    BRASA_TRY(brasa_buf_upload(m->x, 0, x, n));
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = BRASA_OK;
    if (tokens == 1 && decode_fused_ok(m)) {
        rc = set_position(m, pos0);
        if (rc == BRASA_OK) rc = encode_decode_token(m, cmd, layer_begin, layer_end, false);
    }
    else
        for (uint32_t li = layer_begin; li < layer_end && rc == BRASA_OK; ++li) rc = encode_layer_prefill(m, cmd, li, tokens, pos0);
    int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
    BRASA_TRY(rc);
    BRASA_TRY(rc2);
    return brasa_buf_download(m->x, 0, x, n);
}

int32_t brasa_model_decode_greedy(brasa_model *m, uint32_t first, uint32_t pos0, uint32_t steps, uint32_t *out_ids, double *gpu_seconds) {
    if (!m || !out_ids) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_REQUIRE(ctx, steps >= 1 && (uint64_t)pos0 + steps <= m->limits.ctx, "decode range outside the context");
    BRASA_REQUIRE(ctx, first < m->cfg.vocab, "token id %u outside the vocabulary", first);
    BRASA_REQUIRE(ctx, decode_fused_ok(m), "the device-resident loop needs tiled q4_0 layers");
    BRASA_TRY(brasa_buf_upload(m->ids, 0, &first, 4));
    uint32_t st[2] = {pos0, 0};  // position, output count
    BRASA_TRY(brasa_buf_upload(m->dev_state, 0, st, 8));
    brasa_cmd *cmd;
    BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
    int32_t rc = BRASA_OK;
    for (uint32_t s = 0; s < steps && rc == BRASA_OK; ++s) rc = decode_step(m, cmd, UINT32_MAX);
    int32_t rc2 = brasa_cmd_wait(cmd, gpu_seconds);
    BRASA_TRY(rc);
    BRASA_TRY(rc2);
    return brasa_buf_download(m->out_ids, 0, out_ids, (uint64_t)steps * 4);
}

int32_t brasa_model_read_kv(brasa_model *m, uint32_t layer, int32_t which_v, uint32_t pos_begin, uint32_t pos_end, void *dst, uint64_t dst_bytes) {
    if (!m || !dst) return BRASA_EINVAL;
    brasa_ctx *ctx = m->ctx;
    BRASA_REQUIRE(ctx, layer < m->cfg.layers && pos_begin <= pos_end && pos_end <= m->limits.ctx, "read_kv: range");
    uint64_t kvd = (uint64_t)m->cfg.kv_heads * m->cfg.head_dim;
    uint64_t off = brasa_kv_bytes(m->limits.kv, ((uint64_t)layer * m->cap + pos_begin) * kvd);
    uint64_t n = brasa_kv_bytes(m->limits.kv, (uint64_t)(pos_end - pos_begin) * kvd);
    BRASA_REQUIRE(ctx, dst_bytes >= n, "read_kv: destination too small");
    return brasa_buf_download(which_v ? m->vc : m->kc, off, dst, n);
}

}  // extern "C"

// ---- session ------------------------------------------------------------------------------------

struct brasa_session {
    brasa_ctx *ctx = nullptr;
    brasa_model *model = nullptr;
    std::vector<uint32_t> cached;  // tokens whose K and V are in the cache
    std::vector<uint32_t> stop_ids;
    bool ignore_stop = false;
    std::vector<float> logits;
};

extern "C" {

int32_t brasa_session_create(brasa_ctx *ctx, const char *path, brasa_limits limits, uint64_t budget_bytes, brasa_session **out) {
    if (!ctx || !path || !out) return BRASA_EINVAL;
    *out = nullptr;
    brasa_model_shape shape;
    brasa_config cfg;
    char err[512];
    if (brasa_model_shape_from_file(path, &shape, &cfg, err, sizeof err) != BRASA_OK) return brasa_fail(ctx, BRASA_EIO, "%s", err);
    brasa_session_shape ss{limits.ctx, limits.max_tokens, limits.max_logit_rows, limits.kv};
    // the plan is checked before anything is loaded: a rejection allocates nothing
    BRASA_TRY(brasa_plan_check(ctx, &shape, &ss, budget_bytes, nullptr, nullptr));
    BRASA_REQUIRE(ctx, cfg.head_row0 == 0, "a tensor-parallel shard cannot run as a session");
    brasa_model *m = nullptr;
    BRASA_TRY(brasa_model_load(ctx, path, limits, &m));
    if (m->cfg.head_rows != m->cfg.vocab) {
        brasa_model_free(m);
        return brasa_fail(ctx, BRASA_EINVAL, "a tensor-parallel shard cannot run as a session");
    }
    brasa_session *s = new brasa_session();
    s->ctx = ctx;
    s->model = m;
    s->logits.resize(cfg.vocab);
    *out = s;
    return BRASA_OK;
}

void brasa_session_free(brasa_session *s) {
    if (!s) return;
    brasa_model_free(s->model);
    delete s;
}

brasa_model *brasa_session_model(brasa_session *s) { return s ? s->model : nullptr; }

int32_t brasa_session_reset(brasa_session *s) {
    if (!s) return BRASA_EINVAL;
    s->cached.clear();
    return BRASA_OK;
}

int32_t brasa_session_set_stop_ids(brasa_session *s, const uint32_t *ids, uint32_t n, int32_t ignore_stop) {
    if (!s || (!ids && n)) return BRASA_EINVAL;
    s->stop_ids.assign(ids, ids + n);
    s->ignore_stop = ignore_stop != 0;
    return BRASA_OK;
}

int32_t brasa_session_generate(brasa_session *s, const uint32_t *prompt, uint32_t prompt_len, uint32_t max_new, brasa_sampling_params params,
                               brasa_token_cb on_token, void *user, uint32_t *out_ids, brasa_gen_stats *stats) {
    if (!s || !prompt) return BRASA_EINVAL;
    brasa_ctx *ctx = s->ctx;
    brasa_model *m = s->model;
    const brasa_limits lim = m->limits;
    using clk = std::chrono::steady_clock;
    auto ms_since = [](clk::time_point t0) { return std::chrono::duration<double, std::milli>(clk::now() - t0).count(); };
    BRASA_REQUIRE(ctx, prompt_len > 0, "empty prompt");
    BRASA_REQUIRE(ctx, prompt_len < lim.ctx, "the prompt has %u tokens and the context is %u", prompt_len, lim.ctx);
    // longest common prefix with what the cache holds; the last prompt token is always recomputed
    uint32_t common = 0;
    while (common < s->cached.size() && common < prompt_len && s->cached[common] == prompt[common]) ++common;
    common = std::min(common, prompt_len - 1);
    s->cached.resize(common);

    const bool greedy = params.temperature <= 0.0f;
    // Greedy with nothing to mask keeps the logits on the device: the token is chosen there and only
    // its id crosses to the host.
    const bool masked = s->ignore_stop && !s->stop_ids.empty();
    const bool device_pick = greedy && !masked;
    // Sampling with nothing to mask also stays on the device (brasa_k_sample_top_p, same PCG32 stream as the host
    // sampler); the host sampler remains for the masked case.
    const bool device_sample = !greedy && !masked && params.top_p > 0.0f;
    brasa::Sampler sampler(params.temperature, params.top_k, params.top_p, params.seed, m->cfg.vocab);
    const brasa_arg rng_arg = A(m->dev_state, 128);
    if (device_sample) {
        uint64_t st[2];
        brasa_pcg32_seed(params.seed, st);
        BRASA_TRY(brasa_buf_upload(m->dev_state, 128, st, 16));
    }
    const bool host_logits = !device_pick && !device_sample;

    auto t0 = clk::now();
    for (uint32_t off = common; off < prompt_len; off += lim.max_tokens) {
        uint32_t n = std::min(lim.max_tokens, prompt_len - off);
        bool last = off + n == prompt_len;
        BRASA_TRY(brasa_model_forward(m, prompt + off, n, (uint32_t)s->cached.size(), 1, (last && host_logits) ? s->logits.data() : nullptr, nullptr));
        s->cached.insert(s->cached.end(), prompt + off, prompt + off + n);
    }
    double prefill_ms = ms_since(t0);

    uint32_t generated = 0;
    double ttft_ms = 0.0;
    int32_t stop = 1;  // MaxTokens
    auto t1 = clk::now();
    // Greedy with the fused decode path: the device keeps the position and feeds the chosen token back
    // itself; per token the host launches one graph and reads one id (pinned memory), nothing else.
    const bool resident = device_pick && decode_fused_ok(m);
    bool primed = false;  // device position and input token are set up
    // Resident decode keeps the device one step ahead of the host: the step that consumes token t + 1 (which the device
    // feeds itself) is queued before the host waits for the id of token t + 1, so the GPU never idles while the host
    // checks stop ids and calls back. A step queued ahead of a token that then ends the generation is harmless: the
    // position is set again at the next call and the row it wrote lies behind the cached tokens.
    // The id of a step is read back on a stream of its own (from the step's own place in the device's list of chosen
    // tokens), so that the copy does not sit between two steps on the compute stream.
    struct StepEvents {
        cudaEvent_t ev[2] = {nullptr, nullptr}, done[2] = {nullptr, nullptr};
        cudaStream_t copy = nullptr;
        ~StepEvents() {
            if (copy) {
                cudaStreamSynchronize(copy);
                cudaStreamDestroy(copy);
            }
            for (cudaEvent_t e : ev)
                if (e) cudaEventDestroy(e);
            for (cudaEvent_t e : done)
                if (e) cudaEventDestroy(e);
        }
    } sev;
    uint32_t steps_launched = 0;  // resident steps queued so far; step i consumes the i-th token of this call and yields the next
    auto launch_step = [&]() -> int32_t {
        brasa_cmd step{ctx, nullptr, nullptr, false};
        BRASA_TRY(decode_step(m, &step, UINT32_MAX));
        const uint32_t slot = steps_launched & 1;
        BRASA_CUDA(ctx, cudaEventRecord(sev.done[slot], ctx->stream));
        BRASA_CUDA(ctx, cudaStreamWaitEvent(sev.copy, sev.done[slot], 0));
        BRASA_CUDA(ctx, cudaMemcpyAsync(m->pinned_id + slot, (const uint32_t *)m->out_ids->ptr + steps_launched, 4, cudaMemcpyDeviceToHost, sev.copy));
        BRASA_CUDA(ctx, cudaEventRecord(sev.ev[slot], sev.copy));
        ++steps_launched;
        return BRASA_OK;
    };
    if (resident) {
        for (int i = 0; i < 2; ++i) {
            BRASA_CUDA(ctx, cudaEventCreateWithFlags(&sev.ev[i], cudaEventDisableTiming));
            BRASA_CUDA(ctx, cudaEventCreateWithFlags(&sev.done[i], cudaEventDisableTiming));
        }
        BRASA_CUDA(ctx, cudaStreamCreateWithFlags(&sev.copy, cudaStreamNonBlocking));
    }
    while (generated < max_new) {
        uint32_t next;
        if (device_pick && !(resident && primed)) {
            brasa_cmd *cmd;
            BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
            int32_t rc = brasa_argmax_launch(cmd, (const float *)m->logits->ptr, m->cfg.vocab, (uint32_t *)m->next_id->ptr);
            if (rc == BRASA_OK)
                rc = brasa_check_cuda(ctx, cudaMemcpyAsync(m->pinned_id, m->next_id->ptr, 4, cudaMemcpyDeviceToHost, ctx->stream), "token read");
            int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
            BRASA_TRY(rc);
            BRASA_TRY(rc2);
            next = *m->pinned_id;
        } else if (device_pick) {
            const uint32_t slot = (generated - 1) & 1;  // the step that consumed the token before this one
            BRASA_CUDA(ctx, cudaEventSynchronize(sev.ev[slot]));
            next = m->pinned_id[slot];
        } else if (device_sample) {
            brasa_cmd *cmd;
            BRASA_TRY(brasa_cmd_begin(ctx, &cmd));
            int32_t rc = brasa_k_sample_top_p(cmd, A(m->logits), m->cfg.vocab, params.temperature, params.top_k, params.top_p, rng_arg, A(m->next_id));
            if (rc == BRASA_OK)
                rc = brasa_check_cuda(ctx, cudaMemcpyAsync(m->pinned_id, m->next_id->ptr, 4, cudaMemcpyDeviceToHost, ctx->stream), "token read");
            int32_t rc2 = brasa_cmd_wait(cmd, nullptr);
            BRASA_TRY(rc);
            BRASA_TRY(rc2);
            next = *m->pinned_id;
        } else {
            if (s->ignore_stop)
                for (uint32_t id : s->stop_ids)
                    if (id < s->logits.size()) s->logits[id] = -INFINITY;
            next = sampler.sample(s->logits.data(), s->logits.size());
        }
        if (generated == 0) ttft_ms = ms_since(t0);
        if (out_ids) out_ids[generated] = next;
        ++generated;
        if (std::find(s->stop_ids.begin(), s->stop_ids.end(), next) != s->stop_ids.end()) {
            stop = 0;
            break;
        }
        if (on_token && !on_token(user, next)) {
            stop = 3;
            break;
        }
        if (s->cached.size() >= lim.ctx) {
            stop = 2;
            break;
        }
        if (resident) {
            if (!primed) {
                uint32_t st[2] = {(uint32_t)s->cached.size(), 0};
                BRASA_CUDA(ctx, cudaMemcpyAsync(m->ids->ptr, &next, 4, cudaMemcpyHostToDevice, ctx->stream));
                BRASA_CUDA(ctx, cudaMemcpyAsync(m->dev_state->ptr, st, 8, cudaMemcpyHostToDevice, ctx->stream));
                primed = true;
            }
            while (steps_launched < generated) BRASA_TRY(launch_step());  // this token's step (its cache row, the next id)
            // one step ahead, if the next token can still be followed by another one
            if (steps_launched == generated && generated < max_new && s->cached.size() + 2 <= lim.ctx) BRASA_TRY(launch_step());
        } else {
            BRASA_TRY(brasa_model_forward(m, &next, 1, (uint32_t)s->cached.size(), 1, host_logits ? s->logits.data() : nullptr, nullptr));
        }
        s->cached.push_back(next);
    }
    BRASA_TRY(brasa_ctx_sync(ctx));  // surfaces a device-side wait that gave up during the loop
    if (stats) {
        stats->prompt_tokens = prompt_len;
        stats->reused_tokens = common;
        stats->generated = generated;
        stats->stop = stop;
        stats->prefill_ms = prefill_ms;
        stats->ttft_ms = ttft_ms;
        stats->decode_ms = ms_since(t1) - (ttft_ms - prefill_ms);
    }
    return BRASA_OK;
}

}  // extern "C"
