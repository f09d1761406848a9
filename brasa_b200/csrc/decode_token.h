// Host interface of the whole-token decode kernel (decode_token.cu): the model describes its weights, cache and
// state once; the program built from that description is launched once per token.
#pragma once
#include <vector>

#include "brasa_internal.h"

struct brasa_token_layer {
    brasa_qmatrix wq, wk, wv, wo, gate, up, down;  // tiled q4_0
    const float *attn_norm, *q_norm, *k_norm, *ffn_norm;
    uint8_t *kc, *vc;  // this layer's cache rows from position 0: [position][kv head][128] in the cache type
};

struct brasa_token_model {
    uint32_t hidden, heads, kv_heads, head_dim, ffn, vocab;
    uint32_t cache_positions;  // rows the cache holds
    int32_t kv;                // BRASA_KV_*
    float eps;
    std::vector<brasa_token_layer> layers;
    brasa_qmatrix embed, head;  // tiled q6_0 table; tiled q4_0 / q6_0 lm_head
    const float *final_norm, *cos_t, *sin_t;
    uint32_t *state;    // [0] position of this token, [1] tokens written to out_ids, [2] launch sequence number
    uint32_t *ids;      // [0] token to run; receives the chosen token
    uint32_t *next_id;  // the chosen token
    uint32_t *out_ids;
    uint32_t out_cap;
    float *logits;      // [rows of the lm_head]
    // Tensor parallelism: this rank's shard (q/k/v, gate/up and the lm_head split by rows, o_proj and down_proj by
    // columns). world == 1: no exchange. Otherwise the two residual adds of a layer sum the ranks' partial vectors and
    // the greedy choice runs over every rank's lm_head rows, both through the peers' exchange areas.
    uint32_t head_row0 = 0;  // vocabulary row of this rank's first lm_head row
    brasa_tp_token_area tp{};  // tp.world <= 1: single rank
};

struct brasa_token_program;

// True when the model's shapes fit the kernel (otherwise the caller keeps the kernel-per-operation path).
bool brasa_token_program_supported(brasa_ctx *ctx, const brasa_token_model &m);
int32_t brasa_token_program_create(brasa_ctx *ctx, const brasa_token_model &m, brasa_token_program **out);
void brasa_token_program_free(brasa_token_program *p);
// One token: embed, every layer, lm_head, argmax, and the step's bookkeeping (chosen token to ids[0], next_id and
// out_ids; position and output count advance).
int32_t brasa_token_program_launch(brasa_cmd *cmd, brasa_token_program *p);
