// The model's device state, shared by model.cu (single-sequence path) and batch.cu (batched serving path).
#pragma once
#include <vector>

#include "brasa_internal.h"
#include "decode_token.h"

bool brasa_gemm_swiglu_fuses(const brasa_qmatrix &wg, const brasa_qmatrix &wu, uint32_t tokens);

namespace brasa_model_detail {

constexpr uint32_t GEMV_MAX_TOKENS = 8;  // qwen3.rs:276

struct Matrix {
    brasa_buf *buf = nullptr;
    brasa_qmatrix q{};
};

struct Layer {
    brasa_buf *attn_norm, *q_norm, *k_norm, *ffn_norm;
    Matrix wq, wk, wv, wo, gate, up, down;
};

inline brasa_arg A(brasa_buf *b, uint64_t off = 0) { return brasa_arg{b, off}; }
inline float *F(brasa_buf *b, uint64_t off_floats = 0) { return (float *)b->ptr + off_floats; }

struct Stager;

}  // namespace brasa_model_detail

using namespace brasa_model_detail;

struct brasa_model {
    brasa_ctx *ctx = nullptr;
    brasa_tp *tp = nullptr;  // set for a tensor-parallel shard: residual adds are sums over ranks (not owned)
    brasa_config cfg{};
    brasa_limits limits{};
    int32_t prefill_precision = BRASA_PREFILL_F16;
    Matrix embed, head;  // head aliases embed when tied
    brasa_buf *final_norm = nullptr;
    std::vector<Layer> layers;
    brasa_buf *rope_cos = nullptr, *rope_sin = nullptr;
    brasa_buf *kc = nullptr, *vc = nullptr;  // [layers, cap, kv_heads, head_dim] in the cache type
    uint32_t cap = 0;
    // workspace
    brasa_buf *x = nullptr, *h = nullptr, *q = nullptr, *k_new = nullptr, *v_new = nullptr, *attn = nullptr, *xh = nullptr,
              *gate = nullptr, *up = nullptr, *ids = nullptr, *norm_out = nullptr, *ss = nullptr, *partials = nullptr, *logits = nullptr,
              *next_id = nullptr, *out_ids = nullptr, *dev_state = nullptr;  // dev_state: u32 pos, out_count, attention counters
    brasa_graph *decode_graph = nullptr;  // one decode step: embed .. lm_head, argmax, advance
    brasa_token_program *token_prog = nullptr;  // the same step as one persistent kernel, when the shapes allow
    bool token_prog_tried = false;
    uint64_t partials_len = 0;
    brasa_allocated alloc{};
    std::vector<brasa_buf *> owned;
    uint32_t *pinned_id = nullptr;  // pinned host word for the per-step token read
    struct Stager *stager = nullptr;  // pinned staging of the file's bytes while the model loads (null afterwards)
    double load_seconds = 0.0;        // wall time of brasa_model_load, file bytes read included
    uint64_t load_bytes = 0;          // tensor bytes that went to the device
};

