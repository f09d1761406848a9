/*
 * brasa_cuda.h — C ABI of libbrasa_cuda.so: the CUDA (sm_100a) device layer and kernel set for the
 * Qwen3 token loop. It stands where the reference's Metal device layer and kernel dispatch stand:
 *
 *   crates/metal/src/runtime.rs:134-425   Context, Buffer<T>, Arg, Command, Pending, GpuTiming
 *   crates/kernels/src/lib.rs:391-1404    Kernels::* (one entry point per method, same order of
 *                                         arguments), AttnShape, KvType, WeightType, helpers
 *   crates/models/src/qwen3.rs:345-831    Qwen3::{load, forward, run_layers, allocated}
 *   crates/runtime/src/session.rs:210-295 Session::generate (prefix reuse, prefill chunks, decode)
 *   crates/runtime/src/sampler.rs:46-170  Sampler, Pcg32, argmax
 *   crates/memory/src/planner.rs:57-95    plan / workspace_bytes / kv_bytes
 *   crates/quant/src/brasa_file.rs:64-131 BrasaFile::{open, verify}
 *
 * Conventions: every function returns 0 on success or a negative BRASA_E* code; the message of the
 * last failure on a context is read with brasa_last_error(). Nothing here aborts or traps:
 * precondition violations (the reference's assert!) return BRASA_EINVAL. Functions on one context
 * are not re-entrant; distinct contexts (distinct GPUs) are independent. Plain pointers and sizes
 * only. Kernels are enqueued on the context's stream and run in submission order, like dispatches
 * on one Metal command queue.
 */
#ifndef BRASA_CUDA_H
#define BRASA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BRASA_OK 0
#define BRASA_EINVAL (-1)   /* bad argument / shape precondition */
#define BRASA_ENOMEM (-2)   /* device allocation failed */
#define BRASA_ECUDA (-3)    /* CUDA runtime error (message has the detail) */
#define BRASA_ETIMEOUT (-4) /* a bounded device-side wait ran out */
#define BRASA_EIO (-5)      /* file errors: open, truncated, checksum */
#define BRASA_EBUDGET (-6)  /* memory plan does not fit the budget */

/* crates/kernels/src/lib.rs:85-90 (discriminants in declaration order) */
enum brasa_weight_type { BRASA_Q4_0 = 0, BRASA_Q8_0 = 1, BRASA_Q6_0 = 2 };
/* crates/kernels/src/lib.rs:93-101 */
enum brasa_kv_type { BRASA_KV_F32 = 0, BRASA_KV_F16 = 1, BRASA_KV_Q8_0 = 2 };
/* crates/kernels/src/lib.rs:1308-1314 */
enum brasa_prefill_precision { BRASA_PREFILL_F16 = 0, BRASA_PREFILL_F32 = 1 };
/* Byte layout of a quantised matrix in device memory.
 * FILE  = the `.brasa` layout (crates/quant/src/qtype.rs:5-29): row-major blocks, scale then codes.
 * TILED = the device layout produced by brasa_k_repack: same bytes, regrouped into micro-tiles of
 *         64 rows x 128 columns in which codes, high-bit words and scales are separate, 16-byte
 *         aligned planes (q4_0 and q6_0; rows % 64 == 0 and cols % 128 == 0). */
enum brasa_layout { BRASA_LAYOUT_FILE = 0, BRASA_LAYOUT_TILED = 1 };

typedef struct brasa_ctx brasa_ctx; /* crates/metal/src/runtime.rs:134 Context */
typedef struct brasa_buf brasa_buf; /* crates/metal/src/runtime.rs:44  Buffer<T> (untyped bytes) */
typedef struct brasa_cmd brasa_cmd; /* crates/metal/src/runtime.rs:306 Command / Pending */

/* crates/metal/src/runtime.rs:255-295 Arg::buf / Arg::buf_at: a buffer and a byte offset. */
typedef struct brasa_arg {
    brasa_buf *buf;
    uint64_t offset;
} brasa_arg;

/* crates/kernels/src/lib.rs:146-152 QMatrix, plus the device layout of `data`. */
typedef struct brasa_qmatrix {
    brasa_arg data;
    int32_t qtype;  /* brasa_weight_type */
    int32_t layout; /* brasa_layout */
    uint32_t rows, cols;
} brasa_qmatrix;

/* crates/kernels/src/lib.rs:1354-1364 AttnShape */
typedef struct brasa_attn_shape {
    uint32_t tokens, hq, hkv, dim, pos0;
    int32_t kv; /* brasa_kv_type */
} brasa_attn_shape;

/* ---- context, buffers, commands (crates/metal/src/runtime.rs) ------------------------------- */

int32_t brasa_ctx_create(int32_t device, brasa_ctx **out);            /* Context::new :158 */
void brasa_ctx_destroy(brasa_ctx *ctx);                               /* frees stragglers */
const char *brasa_last_error(brasa_ctx *ctx);
int32_t brasa_ctx_device(brasa_ctx *ctx);
int32_t brasa_ctx_mem_info(brasa_ctx *ctx, uint64_t *free_bytes, uint64_t *total_bytes);
int32_t brasa_ctx_sync(brasa_ctx *ctx);
/* Kernels enqueued on this context so far; a graph replay counts every kernel it holds. */
uint64_t brasa_ctx_launch_count(brasa_ctx *ctx);
/* cudaStream_t of the context, for callers that order their own work (NCCL, torch) against it. */
void *brasa_ctx_stream(brasa_ctx *ctx);

int32_t brasa_buf_alloc(brasa_ctx *ctx, uint64_t bytes, brasa_buf **out); /* zero-filled, :177 */
int32_t brasa_buf_free(brasa_buf *buf);
int32_t brasa_buf_upload(brasa_buf *buf, uint64_t offset, const void *src, uint64_t n);   /* buffer_from / as_mut_slice */
int32_t brasa_buf_download(brasa_buf *buf, uint64_t offset, void *dst, uint64_t n);      /* as_slice */
int32_t brasa_buf_fill(brasa_buf *buf, uint64_t offset, int32_t byte, uint64_t n);
uint64_t brasa_buf_bytes(brasa_buf *buf);
void *brasa_buf_ptr(brasa_buf *buf); /* device address */

int32_t brasa_cmd_begin(brasa_ctx *ctx, brasa_cmd **out);     /* Context::command :237 */
int32_t brasa_cmd_commit(brasa_cmd *cmd);                     /* Command::commit :379 */
int32_t brasa_cmd_wait(brasa_cmd *cmd, double *gpu_seconds);  /* Pending::wait -> GpuTiming :411; frees cmd */

/* CUDA graphs. No counterpart call in the reference, whose two command buffers per forward play this
 * role (crates/models/src/qwen3.rs:781-797): kernels enqueued on the context between begin and end are
 * recorded instead of run, and brasa_graph_launch replays them in one submission. Nothing that
 * allocates or synchronises may be called while a capture is open. */
typedef struct brasa_graph brasa_graph;
int32_t brasa_graph_capture_begin(brasa_ctx *ctx);
int32_t brasa_graph_capture_end(brasa_ctx *ctx, brasa_graph **out);
int32_t brasa_graph_launch(brasa_cmd *cmd, brasa_graph *graph);
void brasa_graph_free(brasa_graph *graph);

/* ---- helpers (crates/kernels/src/lib.rs:1316-1404) ------------------------------------------ */

#define BRASA_DECODE_CHUNK 128 /* DECODE_CHUNK :1332 */
#define BRASA_KV_ALIGN 64      /* KV_ALIGN :1351 */
#define BRASA_NORM_PREP_TG 256 /* NORM_PREP_TG :1343 */
#define BRASA_KV_Q8_DIM 128    /* crates/quant/src/qtype.rs:81 */
#define BRASA_KV_Q8_ROW 136    /* crates/quant/src/qtype.rs:83 */

uint64_t brasa_decode_partials_len(uint32_t hq, uint32_t lk);  /* floats; :1335 */
uint32_t brasa_norm_partials(uint32_t n);                      /* :1346 */
int32_t brasa_gqa_supported(uint32_t hq, uint32_t hkv);        /* :1319 */
uint64_t brasa_kv_bytes(int32_t kv, uint64_t n_elems);         /* KvType::bytes :113 */
uint64_t brasa_qtype_nbytes(int32_t qtype, uint64_t n_elems);  /* QType::nbytes qtype.rs:22 */
/* cos/sin(p * theta^(-2i/dim)), double precision, stored as float [max_pos, dim/2]; :1389 */
int32_t brasa_rope_table(double theta, uint32_t dim, uint32_t max_pos, float *cos_out, float *sin_out);

/* ---- weight layout and converter kernels (crates/quant/src/convert.rs:70-151) --------------- */

/* FILE -> TILED and back; exact inverses, same byte count. rows % 64 == 0 and cols % 128 == 0;
 * src and dst must not overlap. */
int32_t brasa_k_repack(brasa_cmd *cmd, int32_t qtype, brasa_arg src_file, brasa_arg dst_tiled, uint32_t rows, uint32_t cols);
int32_t brasa_k_unpack(brasa_cmd *cmd, int32_t qtype, brasa_arg src_tiled, brasa_arg dst_file, uint32_t rows, uint32_t cols);
/* f32 -> q4_0 / q6_0 / q8_0 blocks in FILE layout, bit-identical to quant_q4_0/q6_0/q8_0. */
int32_t brasa_k_quantize(brasa_cmd *cmd, int32_t qtype, brasa_arg src_f32, brasa_arg dst, uint64_t n);
/* FILE-layout blocks -> f32, bit-identical to crates/quant/src/qtype.rs:141 dequantize. */
int32_t brasa_k_dequantize(brasa_cmd *cmd, int32_t qtype, brasa_arg src, brasa_arg dst_f32, uint64_t n);
/* Seeded N(0, std) floats (counter-based generator; same values for the same seed and offset on
 * every GPU): the synthetic random-init weights of the benchmark configurations. */
int32_t brasa_k_randn(brasa_cmd *cmd, brasa_arg dst_f32, uint64_t n, uint64_t seed, uint64_t stream_offset, float std);

/* ---- kernels: one per Kernels method (crates/kernels/src/lib.rs) ---------------------------- */

int32_t brasa_k_add(brasa_cmd *cmd, brasa_arg a, brasa_arg b, brasa_arg out, uint64_t n);                     /* :391 */
int32_t brasa_k_swiglu(brasa_cmd *cmd, brasa_arg gate, brasa_arg up, brasa_arg out, uint64_t n);              /* :409 */
int32_t brasa_k_swiglu_f16(brasa_cmd *cmd, brasa_arg gate, brasa_arg up, brasa_arg out_f16, uint64_t n);      /* :433 */
int32_t brasa_k_rms_norm(brasa_cmd *cmd, brasa_arg x, brasa_arg w, brasa_arg out, uint32_t rows, uint32_t n, float eps);     /* :531 */
int32_t brasa_k_rms_norm_f16(brasa_cmd *cmd, brasa_arg x, brasa_arg w, brasa_arg out_f16, uint32_t rows, uint32_t n, float eps); /* :511 */
int32_t brasa_k_softmax(brasa_cmd *cmd, brasa_arg x, brasa_arg out, uint32_t rows, uint32_t n);               /* :550 */
int32_t brasa_k_rope_neox(brasa_cmd *cmd, brasa_arg x, brasa_arg cos_t, brasa_arg sin_t, uint32_t table_dim, uint32_t table_max_pos,
                          uint32_t tokens, uint32_t heads, uint32_t dim, uint32_t pos0);                      /* :569 */
int32_t brasa_k_embed(brasa_cmd *cmd, brasa_qmatrix table, brasa_arg ids_u32, brasa_arg out, uint32_t tokens); /* :600 */
/* x += h (when h.buf != NULL); xw = x*w; ss[i] = sum of x^2 over elements [256 i, 256 i + 256) :633 */
int32_t brasa_k_add_norm_prep(brasa_cmd *cmd, brasa_arg x, brasa_arg h, brasa_arg w, brasa_arg xw, brasa_arg ss, uint32_t n);
/* y = (W xw) / sqrt(sum(ss)/cols + eps) :663 */
int32_t brasa_k_gemv_scaled(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg xw, brasa_arg ss, float eps, brasa_arg y);
int32_t brasa_k_gemv_scaled3(brasa_cmd *cmd, const brasa_qmatrix w[3], brasa_arg xw, brasa_arg ss, float eps, const brasa_arg y[3]); /* :698 */
int32_t brasa_k_gemv_scaled_swiglu(brasa_cmd *cmd, brasa_qmatrix gate, brasa_qmatrix up, brasa_arg xw, brasa_arg ss, float eps, brasa_arg y); /* :746 */
int32_t brasa_k_gemv(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens);            /* :781 */
int32_t brasa_k_gemv_simple(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens);     /* :813 */
/* y[t, :] = W x[t, :]; precision F16: x is f16 and dequantised weights are rounded to f16 :856 */
int32_t brasa_k_gemm_with(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x, brasa_arg y, uint32_t tokens, int32_t precision);
int32_t brasa_k_gemm(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg y, uint32_t tokens);
/* acc += W x for f16 inputs: the layer's residual add folded into the GEMM (scratch: tokens x rows f32, used when the
 * product takes the generic kernel). New: the reference adds with a separate `add` dispatch (qwen3.rs:810-826). */
int32_t brasa_k_gemm_add(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg acc, brasa_arg scratch, uint32_t tokens);        /* :842 */
/* How a product of 9 to 64 tokens with tiled q4_0 matrices is cut over the SMs (no counterpart in the reference: its Metal
 * GEMM takes one threadgroup per output tile, matmul_tiled.metal:35-53). The (128-row tile, 64-column stage) pairs of the
 * launch's matrices, in that order, are `tiles x stages` units; block b of `blocks` takes units [b units / blocks,
 * (b + 1) units / blocks). A tile shared by several blocks is summed from their partial tiles in K order by a second kernel;
 * `max_parts` is the most blocks that share a tile and `scratch_bytes` what the library keeps for the partial tiles (inside
 * the planners' overhead allowance). BRASA_EINVAL for an empty shape or one whose unit count does not fit 32-bit arithmetic. */
int32_t brasa_gemm_few_tokens_plan(uint32_t sm_count, uint32_t tiles, uint32_t stages, uint32_t *blocks, uint32_t *max_parts, uint64_t *scratch_bytes);
/* the block whose run holds `unit` (UINT32_MAX for arguments outside a plan) */
uint32_t brasa_gemm_few_tokens_owner(uint32_t units, uint32_t blocks, uint32_t unit);
/* acc += W x, then out_f16 = f16(rms_norm(acc) * norm_w): a layer's residual add and the norm that opens the next block
 * (qwen3.rs:810-826 then :700-712 as one call). One GEMM and one kernel behind it for up to 64 tokens; otherwise the two calls. */
int32_t brasa_k_gemm_add_rms_norm_f16(brasa_cmd *cmd, brasa_qmatrix w, brasa_arg x_f16, brasa_arg acc, brasa_arg scratch, brasa_arg norm_w,
                                      brasa_arg out_f16, uint32_t tokens, float eps);
int32_t brasa_k_gemm_multi(brasa_cmd *cmd, const brasa_qmatrix *ws, uint32_t count, brasa_arg x, const brasa_arg *ys, uint32_t tokens, int32_t precision); /* :872 */
/* out_f16[t, :] = f16(silu(Wg x) * (Wu x)); gate/up scratch [tokens, rows] f32 may be used :455 */
int32_t brasa_k_gemm_swiglu(brasa_cmd *cmd, brasa_qmatrix wg, brasa_qmatrix wu, brasa_arg x_f16, brasa_arg gate, brasa_arg up, brasa_arg out_f16, uint32_t tokens);
/* per-head RMSNorm of q and k, RoPE of q and k, K and V written to the cache at pos0 :976 */
int32_t brasa_k_qk_norm_rope_store(brasa_cmd *cmd, int32_t kv, const brasa_arg qkv[3], const brasa_arg norms[2], float eps,
                                   brasa_arg cos_t, brasa_arg sin_t, uint32_t table_dim, uint32_t table_max_pos,
                                   const brasa_arg dst[2], brasa_attn_shape shape);
int32_t brasa_k_store_kv(brasa_cmd *cmd, int32_t kv, brasa_arg src, brasa_arg dst, uint64_t n);              /* :1029 */
/* one query token at pos0 against keys 0..pos0; partials >= brasa_decode_partials_len floats :1056,:1110 */
int32_t brasa_k_decode_attention(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len, brasa_arg o, brasa_attn_shape shape);
int32_t brasa_k_decode_attention_lanes(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg partials, uint64_t partials_len, brasa_arg o, brasa_attn_shape shape);
/* Decode attention for callers that cannot allocate device memory. It has no counterpart in the reference,
 * whose caller always hands the kernel a preallocated `partials` buffer (crates/models/src/qwen3.rs:400).
 * Who needs it: code running where cudaMalloc is forbidden or unaffordable, such as a host thread that is
 * inside a stream capture, a plugin that was given a fixed memory budget by its host process, or a
 * latency-critical loop that must never enter the allocator. Same arithmetic and same result as
 * brasa_k_decode_attention; the per-chunk partial results go to an array that is part of the library image
 * instead (2.1 MB, present on every GPU that loads the library until the process exits).
 * Limits: at most 64 query heads and 8192 keys (pos0 + 1 <= 8192); larger shapes are refused with
 * BRASA_EINVAL and a message that names the limit. The first call on each device looks up the array's
 * device address (a CUDA runtime query, no allocation); make that first call before any stream capture
 * begins. Every call uses the same array and nothing in it has to be cleared, since each call overwrites
 * what it later reads; for the same reason two calls must not overlap on the GPU (two streams or two
 * contexts of one process): they would read each other's partials. */
int32_t brasa_k_decode_attention_static(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o, brasa_attn_shape shape);
/* causal GQA attention for a chunk; precision F16: Q*scale rounded to f16, o in f16 :1185 */
int32_t brasa_k_flash_attention_with(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o, brasa_attn_shape shape, int32_t precision);
int32_t brasa_k_flash_attention(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg o_f16, brasa_attn_shape shape); /* :1169 */

/* ---- sampling on the device (crates/runtime/src/sampler.rs) --------------------------------- */

/* first index of the maximum, NaN ignored, 0 when nothing exceeds -inf (:148-170); out: one u32 */
int32_t brasa_k_argmax(brasa_cmd *cmd, brasa_arg logits, uint32_t n, brasa_arg out_u32);
/* Sampler::sample on the device (crates/runtime/src/sampler.rs:60-146): temperature, top-k (0 = off) and top-p over
 * n logits, one PCG32 draw from the 16-byte state {u64 state, u64 increment} in rng_state (advanced in place; fill it
 * with brasa_pcg32_seed). temperature <= 0 is the greedy argmax. The chosen token id goes to out_u32. */
int32_t brasa_k_sample_top_p(brasa_cmd *cmd, brasa_arg logits, uint32_t n, float temperature, uint32_t top_k, float top_p, brasa_arg rng_state,
                             brasa_arg out_u32);
/* The same for `count` rows of n logits, row r with its own state at rng_states + 16 r and its token in out_u32[r];
 * scratch: count x n x 8 bytes. With top-k off and two or more rows every row is spread over several blocks (radix
 * select over 64-bit fixed-point masses: a row's token does not depend on how many rows share the launch). */
int32_t brasa_k_sample_rows(brasa_cmd *cmd, brasa_arg logits, uint32_t n, uint32_t count, float temperature, uint32_t top_k, float top_p,
                            brasa_arg rng_states, brasa_arg scratch, brasa_arg out_u32);
/* Pcg32::new(seed) (sampler.rs:13-20) as the two words brasa_k_sample_top_p keeps on the device. */
void brasa_pcg32_seed(uint64_t seed, uint64_t state_inc[2]);

/* ---- memory planner (crates/memory/src/planner.rs) ------------------------------------------ */

typedef struct brasa_model_shape { /* planner.rs:23-35 ModelShape (tensor bytes summed by the caller) */
    uint64_t weight_bytes;
    uint32_t layers, hidden, heads, kv_heads, head_dim, ffn, vocab;
} brasa_model_shape;
typedef struct brasa_session_shape { /* planner.rs:37-47 SessionShape */
    uint32_t ctx, max_tokens, max_logit_rows;
    int32_t kv; /* brasa_kv_type */
} brasa_session_shape;
typedef struct brasa_memory_plan { /* planner.rs:49-55 MemoryPlan */
    uint64_t weights, kv, workspace, overhead, total;
} brasa_memory_plan;
uint64_t brasa_plan_buffer_bytes(uint64_t n); /* device allocation granularity; planner.rs:57 */
int32_t brasa_plan(const brasa_model_shape *m, const brasa_session_shape *s, brasa_memory_plan *out); /* :83 */
/* 0 when the plan fits budget_bytes (0 = device free memory minus a reserve); else BRASA_EBUDGET
 * and *max_ctx_out = the largest context that fits (0 if none) :237-313 */
int32_t brasa_plan_check(brasa_ctx *ctx, const brasa_model_shape *m, const brasa_session_shape *s, uint64_t budget_bytes,
                         brasa_memory_plan *out, uint32_t *max_ctx_out);

/* ---- model and session (crates/models/src/qwen3.rs, crates/runtime/src/session.rs) ---------- */

typedef struct brasa_model brasa_model;     /* Qwen3 */
typedef struct brasa_session brasa_session; /* Session */

typedef struct brasa_limits { /* qwen3.rs:175-185 Limits */
    uint32_t ctx, max_tokens, max_logit_rows;
    int32_t kv; /* brasa_kv_type */
} brasa_limits;

typedef struct brasa_config { /* qwen3.rs:28-41 Config */
    uint32_t hidden, layers, heads, kv_heads, head_dim, ffn, vocab, max_position;
    float eps;
    double rope_theta;
    int32_t tied; /* 1: lm_head is the embedding table (the reference supports only this) */
    uint32_t head_rows, head_row0; /* rows of the lm_head held here and the vocabulary row of the first (vocab, 0 unless sharded) */
} brasa_config;

typedef struct brasa_allocated { /* qwen3.rs:430 Allocated */
    uint64_t weights, kv, workspace;
} brasa_allocated;

/* BrasaFile::open + verify over a path: structure checks always, sha256 when verify != 0. */
int32_t brasa_file_check(const char *path, int32_t verify, char *err, uint64_t err_len);
int32_t brasa_model_shape_from_file(const char *path, brasa_model_shape *shape, brasa_config *cfg, char *err, uint64_t err_len); /* qwen3.rs:79 */

int32_t brasa_model_load(brasa_ctx *ctx, const char *path, brasa_limits limits, brasa_model **out); /* Qwen3::load :345 */
void brasa_model_free(brasa_model *m);
int32_t brasa_model_config(brasa_model *m, brasa_config *out);
int32_t brasa_model_limits(brasa_model *m, brasa_limits *out);
int32_t brasa_model_allocated(brasa_model *m, brasa_allocated *out);
/* How the weights came in: wall seconds from the first tensor to the last one regrouped on the device (the file is read
 * through two pinned staging buffers while the previous chunk travels by DMA), and the tensor bytes moved. */
int32_t brasa_model_load_stats(brasa_model *m, double *seconds, uint64_t *bytes);
int32_t brasa_model_set_prefill_precision(brasa_model *m, int32_t precision); /* qwen3.rs:310 */
/* Qwen3::forward :763. ids: host u32[tokens]; logits: host f32[logit_rows * vocab] (may be NULL to
 * leave them on the device); gpu_seconds: device time of the call (may be NULL). */
int32_t brasa_model_forward(brasa_model *m, const uint32_t *ids, uint32_t tokens, uint32_t pos0, uint32_t logit_rows, float *logits, double *gpu_seconds);
/* Qwen3::run_layers :743. x: host f32[tokens*hidden], replaced by the output. */
int32_t brasa_model_run_layers(brasa_model *m, float *x, uint32_t tokens, uint32_t pos0, uint32_t layer_begin, uint32_t layer_end);
/* Device-resident decode: feeds the token chosen on the device back as the next input for `steps`
 * greedy steps starting from `first` at position pos0, without host round trips; out_ids: host
 * u32[steps] read once at the end. Used for the HBM-resident throughput figure. */
int32_t brasa_model_decode_greedy(brasa_model *m, uint32_t first, uint32_t pos0, uint32_t steps, uint32_t *out_ids, double *gpu_seconds);
/* Copies K or V cache rows [pos_begin, pos_end) of a layer to the host in the cache's own bytes. */
int32_t brasa_model_read_kv(brasa_model *m, uint32_t layer, int32_t which_v, uint32_t pos_begin, uint32_t pos_end, void *dst, uint64_t dst_bytes);

typedef struct brasa_sampling_params { /* sampler.rs:5-13 SamplingParams */
    float temperature; /* 0 = greedy */
    uint32_t top_k;    /* 0 = no limit */
    float top_p;       /* 1.0 = no limit */
    uint64_t seed;
} brasa_sampling_params;

typedef struct brasa_gen_stats { /* session.rs:29-53 GenStats */
    uint32_t prompt_tokens, reused_tokens, generated;
    int32_t stop; /* 0 Stop, 1 MaxTokens, 2 ContextFull, 3 Cancelled */
    double prefill_ms, ttft_ms, decode_ms;
} brasa_gen_stats;

/* return 0 to cancel (the reference's on_text returning false) */
typedef int32_t (*brasa_token_cb)(void *user, uint32_t token);

int32_t brasa_session_create(brasa_ctx *ctx, const char *path, brasa_limits limits, uint64_t budget_bytes, brasa_session **out); /* load_with_budget :150 */
void brasa_session_free(brasa_session *s);
brasa_model *brasa_session_model(brasa_session *s);
int32_t brasa_session_reset(brasa_session *s); /* :182 */
int32_t brasa_session_set_stop_ids(brasa_session *s, const uint32_t *ids, uint32_t n, int32_t ignore_stop);
/* Session::generate :210. prompt: host ids; out_ids: host u32[max_new]. */
int32_t brasa_session_generate(brasa_session *s, const uint32_t *prompt, uint32_t prompt_len, uint32_t max_new,
                               brasa_sampling_params params, brasa_token_cb on_token, void *user,
                               uint32_t *out_ids, brasa_gen_stats *stats);

/* ---- batched decode over a paged KV pool (serving: many independent sequences of one model) -------------------
 * No counterpart in the reference, which serves one sequence per process (crates/daemon/src/engine.rs:1-3) and
 * reuses one cached prefix (crates/runtime/src/session.rs:230-237); this is that prefix reuse for many sequences.
 * KV pages hold BRASA_KV_PAGE positions in the model's cache type. */
#define BRASA_KV_PAGE 16
typedef struct brasa_batch brasa_batch;
/* up to max_seqs sequences (<= the model's max_tokens) of at most max_positions positions each, num_pages pages in all */
int32_t brasa_batch_create(brasa_model *m, uint32_t max_seqs, uint32_t num_pages, uint32_t max_positions, brasa_batch **out);
void brasa_batch_free(brasa_batch *b);
/* a prefix declared up front (a multiple of BRASA_KV_PAGE tokens, possibly 0): prefilled once; every sequence added later
 * starts with it */
int32_t brasa_batch_set_prefix(brasa_batch *b, const uint32_t *ids, uint32_t n);
/* a sequence = the declared prefix + its own n >= 1 tokens. Prefix cache (crates/runtime/src/session.rs:230-237 for many
 * sequences): every full page of prompt tokens ever computed in this batch is kept under a key that chains the 16 token
 * ids of the page with the key of the page before it; the leading pages of a new sequence that are found there are
 * attached instead of recomputed (at least its last prompt token is always computed), whoever computed them, and the
 * output never depends on what was reused. The rest is prefilled and its full pages join the cache. Draws the
 * sequence's first token (PCG32 seed = params.seed + index). */
int32_t brasa_batch_add_sequence(brasa_batch *b, const uint32_t *ids, uint32_t n, brasa_sampling_params params, uint32_t *seq_out);
/* prompt tokens served from the prefix cache / computed so far, pages the cache knows, leading pages all sequences share */
int32_t brasa_batch_prefix_cache_stats(brasa_batch *b, uint64_t *hit_tokens, uint64_t *prefilled_tokens, uint32_t *cached_pages,
                                       uint32_t *common_pages);
/* `steps` tokens for every sequence; out_ids[seq * (steps + 1) + s], s = 0 being the token drawn when the sequence was added */
int32_t brasa_batch_decode(brasa_batch *b, uint32_t steps, brasa_sampling_params params, uint32_t *out_ids, double *gpu_seconds);
/* logits [sequences][vocab] of the next token of every sequence, without sampling or advancing */
int32_t brasa_batch_peek_logits(brasa_batch *b, float *logits);
/* Kernel-level paged-KV operators, for a caller that keeps its own layer loop (crates/models/src/qwen3.rs on top of
 * brasa_k_*) and its own page tables. One layer's pages: [page][BRASA_KV_PAGE positions][hkv][128] in the cache type;
 * table: i32 [seqs][max_pages] page numbers (< num_pages) of every sequence in position order; lens: u32 [seqs], the
 * positions a sequence already holds = the position of its new token. All of it lives in device buffers. */
typedef struct brasa_paged_kv {
    brasa_arg kpool, vpool, table, lens;
    uint32_t seqs, max_pages, num_pages;
    int32_t kv; /* brasa_kv_type */
} brasa_paged_kv;
/* crates/kernels/src/lib.rs:976-1025 qk_norm_rope_store for one new token per sequence: q f32[seqs][hq][128] and
 * k f32[seqs][hkv][128] are normalised and rotated in place at position lens[seq], K and V (v f32[seqs][hkv][128]) are
 * rounded to the cache type and stored into the sequence's page of that position */
int32_t brasa_k_qk_norm_rope_store_paged(brasa_cmd *cmd, brasa_arg q, brasa_arg k, brasa_arg v, brasa_arg q_norm, brasa_arg k_norm,
                                         brasa_arg rope_cos, brasa_arg rope_sin, float eps, brasa_paged_kv paged, uint32_t hq, uint32_t hkv);
/* lib.rs:1110-1164 decode_attention_lanes over page tables: every sequence's new token attends to its lens[seq] + 1
 * positions. partials: f32 scratch of at least brasa_decode_partials_len(hq, max_pages * BRASA_KV_PAGE) * seqs;
 * o f32[seqs][hq][128] */
int32_t brasa_k_decode_attention_paged(brasa_cmd *cmd, brasa_arg q, brasa_paged_kv paged, brasa_arg partials, uint64_t partials_len, brasa_arg o,
                                       uint32_t hq, uint32_t hkv);

/* Memory of a batch before it is created (crates/memory/src/planner.rs:57-95 for the paged pool): the same sums
 * brasa_batch_create allocates, buffer by buffer. head_rows: the model's lm_head rows (its vocabulary unless it is a
 * tensor-parallel shard). */
typedef struct brasa_batch_shape {
    uint32_t max_seqs, num_pages, max_positions, head_rows;
    int32_t kv; /* brasa_kv_type */
} brasa_batch_shape;
typedef struct brasa_batch_plan {
    uint64_t kv_pages, tables, logits, attention_partials, sampler, total;
} brasa_batch_plan;
int32_t brasa_plan_batch(const brasa_model_shape *m, const brasa_batch_shape *s, brasa_batch_plan *out);
/* The largest batch that fits (planner.rs:237-281 max_context, for sequences instead of positions): every sequence may
 * reach positions_per_seq positions, the first shared_prefix of them (a multiple of BRASA_KV_PAGE) held once for all.
 * budget_bytes 0: the free memory of ctx's device minus a 512 MiB reserve. Returns BRASA_EBUDGET when not even one
 * sequence fits. *plan_out (optional): the plan of that batch; *num_pages_out: the pages it needs. */
int32_t brasa_plan_batch_max_seqs(brasa_ctx *ctx, const brasa_model_shape *m, int32_t kv, uint32_t head_rows, uint32_t shared_prefix,
                                  uint32_t positions_per_seq, uint32_t max_seqs_cap, uint64_t budget_bytes, uint32_t *max_seqs_out,
                                  uint32_t *num_pages_out, brasa_batch_plan *plan_out);
/* bytes brasa_batch_create allocated for this batch: equals the total of brasa_plan_batch for its shape */
int32_t brasa_batch_allocated(brasa_batch *b, uint64_t *bytes);
uint32_t brasa_batch_sequences(brasa_batch *b);
uint32_t brasa_batch_pages_in_use(brasa_batch *b);

/* ---- tensor parallelism inside one node (large models split over GPUs) ---------------------------------------
 * No counterpart in the reference (one device). A model shard is an ordinary `.brasa` file whose config carries this
 * rank's share of the heads, KV heads and FFN rows (q/k/v and gate/up split by rows, o_proj and down_proj by columns,
 * an untied lm_head by vocabulary rows, `tp_vocab_offset` = its first row); the two residual adds of every layer
 * (qwen3.rs:763-831) become a sum over ranks, done by a one-shot push exchange through peer memory. One process per
 * GPU: each rank creates its exchange buffer, the 64-byte handles travel over the job's own channel, every rank
 * connects, and the ranks then make the same calls in the same order. */
#define BRASA_TP_MAX_RANKS 8
#define BRASA_TP_HANDLE_BYTES 64
typedef struct brasa_tp brasa_tp;
/* max_elems: the largest number of f32 values one exchange carries (max_tokens x hidden; even) */
int32_t brasa_tp_create(brasa_ctx *ctx, uint32_t rank, uint32_t world, uint64_t max_elems, brasa_tp **out);
void brasa_tp_free(brasa_tp *tp);
uint32_t brasa_tp_rank(const brasa_tp *tp);
uint32_t brasa_tp_world(const brasa_tp *tp);
int32_t brasa_tp_handle(brasa_tp *tp, uint8_t *handle /* BRASA_TP_HANDLE_BYTES */);
int32_t brasa_tp_connect(brasa_tp *tp, const uint8_t *handles /* world x BRASA_TP_HANDLE_BYTES, by rank */);
int32_t brasa_tp_connect_same_process(brasa_tp *const *tps, uint32_t n); /* ranks of one process: plain pointers */
/* How many times a receive re-reads one exchange word before it gives up (default 2^22, seconds of waiting). A rank
 * whose peer stopped calling then finishes its kernel with what it has, the next brasa_cmd_wait / brasa_ctx_sync on its
 * context returns BRASA_ETIMEOUT, and the context stays usable. */
int32_t brasa_tp_set_poll_limit(brasa_tp *tp, uint32_t polls);
/* out = resid + sum over ranks of partial (resid.buf NULL: out = the sum); n even; identical bits on every rank */
int32_t brasa_k_tp_allreduce_add(brasa_cmd *cmd, brasa_tp *tp, brasa_arg partial, brasa_arg resid, brasa_arg out, uint64_t n);
/* out = resid + sum over ranks of (w x): the GEMV of a column-split o_proj / down_proj (crates/kernels/src/lib.rs:781-810
 * gemv, matmul.metal:243) fused with the exchange: the GEMV's epilogue stores this rank's rows straight into every rank's
 * exchange slot over peer memory (plain stores: no TMA, no multicast), the receive half adds the slots in rank order.
 * w: tiled q4_0 / q6_0, rows even and <= max_elems; x f32[cols]; resid.buf NULL: out = the sum. */
int32_t brasa_k_gemv_allreduce(brasa_cmd *cmd, brasa_tp *tp, brasa_qmatrix w, brasa_arg x, brasa_arg resid, brasa_arg out);
/* its send (gather = 0: the GEMV) and receive (gather = 1) halves, for ranks that share one device */
int32_t brasa_k_gemv_allreduce_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_qmatrix w, brasa_arg x, brasa_arg resid, brasa_arg out, int32_t gather);
/* argmax over the concatenation of every rank's logits[n] (this rank's rows start at row0): out_u32 = global index */
int32_t brasa_k_tp_argmax(brasa_cmd *cmd, brasa_tp *tp, brasa_arg logits, uint32_t n, uint32_t row0, brasa_arg out_u32);
/* the send (gather = 0) and receive (gather = 1) halves as separate launches, for ranks that share one device:
 * queue every rank's send before any rank's receive */
int32_t brasa_k_tp_allreduce_add_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_arg partial, brasa_arg resid, brasa_arg out, uint64_t n, int32_t gather);
int32_t brasa_k_tp_argmax_phase(brasa_cmd *cmd, brasa_tp *tp, brasa_arg logits, uint32_t n, uint32_t row0, brasa_arg out_u32, int32_t gather);
/* attaches the exchange to a model shard (before its first forward): residual adds become all-reduces, the greedy
 * token of brasa_model_decode_greedy is chosen over all ranks' lm_head rows; brasa_model_forward returns this rank's
 * rows of the logits (brasa_config.head_rows of them, starting at vocabulary row head_row0) */
int32_t brasa_model_set_tp(brasa_model *m, brasa_tp *tp);

#ifdef __cplusplus
}
#endif
#endif /* BRASA_CUDA_H */
