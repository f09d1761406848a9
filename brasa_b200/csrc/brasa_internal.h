// Internal declarations shared by the .cu files of libbrasa_cuda.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/brasa_cuda.h"

constexpr uint32_t GEMM_TC_COUNTERS = 8192;

struct brasa_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string last_error;
    std::vector<brasa_buf *> bufs;  // live buffers, freed with the context
    int sm_count = 0;
    size_t smem_optin = 0;
    // scratch shared by the split-K GEMV kernels (partials + arrival counters + status word)
    float *gemv_partials = nullptr;
    size_t gemv_partials_floats = 0;
    uint32_t *gemv_counters = nullptr;
    size_t gemv_counters_n = 0;
    uint32_t *status = nullptr;  // device status word: non-zero after a bounded wait gave up
    uint32_t timeouts = 0;       // waits that gave up so far (kernels with state across launches compare it to what they last saw)
    bool pdl = true;             // programmatic dependent launch between decode kernels
    bool capturing = false;      // a stream capture is open (brasa_graph_capture_begin)
    unsigned long long *gemv_trace = nullptr;  // device buffer of phase timestamps when BRASA_TRACE=1
    struct {
        const uint8_t *w[3];
        uint32_t rows[3];
        uint32_t nmat, total_rows, row_bytes, swiglu;
    } gemv_next = {};  // see brasa_gemv_hint_next
    bool graphs = true;          // replay the decode step as a CUDA graph (BRASA_GRAPH=0 turns it off)
    bool token_kernel = true;    // run a decode token as one persistent kernel (BRASA_TOKEN_KERNEL=0 turns it off)
    uint64_t launches = 0;       // kernels enqueued on this context (graph replays count their nodes)
    uint64_t capture_launches = 0;
    float *sample_scratch = nullptr;  // weights of the device sampler (2 x vocabulary)
    size_t sample_scratch_n = 0;
    void *argmax_scratch = nullptr;  // arrival counter + per-block partial maxima
    uint8_t *kv_expand = nullptr;    // f16 hi/lo expansion of a q8_0 KV cache for the tensor-core prefill attention (K hi, K lo, V hi, V lo)
    size_t kv_expand_bytes = 0;
    float *gemm_part = nullptr;      // partial output tiles of the split-K tensor-core GEMM
    size_t gemm_part_bytes = 0;
    uint32_t *gemm_counters = nullptr;  // arrivals per output tile of that GEMM (GEMM_TC_COUNTERS words, zero between launches)
};

// Launches `kernel` as a programmatic dependent of the kernel before it on the context's stream: it may start while that
// kernel is still running and must execute griddepcontrol.wait before it touches anything that kernel produces (and the
// kernels before that one are complete by then only if every kernel of the chain waits before it lets its own dependent
// start). With BRASA_PDL=0 it is an ordinary launch.
template <typename... KArgs, typename... Args>
inline cudaError_t brasa_launch_dependent(brasa_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Makes at least `bytes` of dynamic shared memory available to kernel `fn` on the context's device (the grant is
// per device and kernel, shared by every context of the process on that device, and never lowered; cheap afterwards).
int32_t brasa_smem_optin(brasa_ctx *ctx, const void *fn, size_t bytes);

// The part of a tensor-parallel exchange buffer that belongs to the whole-token decode kernel, as seen from this rank:
// peer[r] points at rank r's area, laid out [2 parities][world][stride] words {f32, epoch} (partial sums of a residual
// add, slot = sending rank) followed by [2][world][2] words (best logit, its index).
struct brasa_tp;
// values one exchange of this group can carry
uint64_t brasa_tp_max_elems(const brasa_tp *tp);
struct brasa_tp_token_area {
    uint32_t world, rank;
    uint64_t stride;
    uint32_t poll_limit;
    unsigned long long *peer[BRASA_TP_MAX_RANKS];
};
bool brasa_tp_token_area_get(brasa_tp *tp, brasa_tp_token_area *out);

// Where a kernel of this rank writes its share of an all-reduce: slot [rank] of every rank's exchange buffer
// ([2 parities][world][max_elems] words {f32, exchange number}); state[0] counts the exchanges done so far.
struct brasa_tp_push_target {
    unsigned long long *peer[BRASA_TP_MAX_RANKS];
    uint32_t world, rank;
    uint64_t max_elems;
    const uint32_t *state;
};
bool brasa_tp_push_target_get(brasa_tp *tp, brasa_tp_push_target *out);

// The row-owning GEMV over tiled q4_0 / q6_0 matrices (gemv.cu). epilogue: 0 y = scale * W x, 1 SwiGLU (w[0] = gate,
// w[1] = up, y[0]), 2 y = resid + W x, 3 W x pushed into the tensor-parallel exchange buffers named by `push`.
int32_t brasa_tp_gemv_allreduce_launch(brasa_cmd *cmd, brasa_tp *tp, const brasa_qmatrix &w, const float *x, const float *resid, float *out, int phases);
int32_t brasa_gemv_launch(brasa_cmd *cmd, int qtype, uint32_t nmat, const brasa_qmatrix *w, float *const *y, const float *x, const float *h,
                          const float *normw, float *x_out, const float *ss, uint32_t nss, int scaled, float eps, int epilogue, const float *resid,
                          const brasa_tp_push_target *push = nullptr);

// Phase time stamps of the GEMV and whole-token kernels exist only in builds with -DBRASA_TRACE_BUILD (a
// developer's build; the shipped library carries neither the stamps nor these entry points).
#ifdef BRASA_TRACE_BUILD
extern "C" int32_t brasa_debug_gemv_trace(brasa_ctx *ctx, uint64_t out[16]);
extern "C" int32_t brasa_debug_trace_read(brasa_ctx *ctx, uint64_t *out, uint32_t n);
#endif

struct brasa_buf {
    brasa_ctx *ctx;
    void *ptr;
    uint64_t bytes;
};

struct brasa_graph {
    brasa_ctx *ctx;
    cudaGraphExec_t exec;
    uint64_t kernels;  // kernel nodes recorded
};

struct brasa_cmd {
    brasa_ctx *ctx;
    cudaEvent_t start, end;
    bool committed;
};

int32_t brasa_fail(brasa_ctx *ctx, int32_t code, const char *fmt, ...);
int32_t brasa_check_cuda(brasa_ctx *ctx, cudaError_t e, const char *what);

#define BRASA_TRY(expr)                    \
    do {                                   \
        int32_t _rc = (expr);              \
        if (_rc != BRASA_OK) return _rc;   \
    } while (0)
#define BRASA_CUDA(ctx, expr) BRASA_TRY(brasa_check_cuda((ctx), (expr), #expr))
#define BRASA_REQUIRE(ctx, cond, ...)                                   \
    do {                                                                \
        if (!(cond)) return brasa_fail((ctx), BRASA_EINVAL, __VA_ARGS__); \
    } while (0)

// Device pointer of an argument, or nullptr when the argument has no buffer.
static inline uint8_t *arg_ptr(const brasa_arg &a) {
    return a.buf ? static_cast<uint8_t *>(a.buf->ptr) + a.offset : nullptr;
}
// True when [offset, offset + n) lies inside the buffer.
static inline bool arg_fits(const brasa_arg &a, uint64_t n) {
    return a.buf && a.offset <= a.buf->bytes && n <= a.buf->bytes - a.offset;
}
static inline bool qm_fits(const brasa_qmatrix &m) {
    return arg_fits(m.data, brasa_qtype_nbytes(m.qtype, (uint64_t)m.rows * m.cols));
}

int32_t brasa_post_launch(brasa_cmd *cmd, const char *name);
// Makes sure the context's split-K scratch holds at least this many floats / counters.
int32_t brasa_gemv_scratch(brasa_ctx *ctx, size_t partial_floats, size_t counters);

// ---- tiled (row-planar) weight layout ----------------------------------------------------------
// Each row keeps its own bytes, regrouped into planes so that every access is an aligned vector:
//     q4_0: codes [nb][16 bytes] | scales [nb] f16
//     q6_0: codes [nb][16 bytes] | high-bit words [nb][2] u32 | scales [nb] f16
// nb = cols / 32 blocks per row; total bytes equal the file layout's (18 or 26 per block). The code
// bytes of a block are unchanged (byte j = element j in the low nibble, element j + 16 in the high
// nibble). A q6_0 high-bit word serves the two code words of one half block (16 codes). After
// `word & 0x0F0F0F0F` or `(word >> 4) & 0x0F0F0F0F` a register holds four codes, one per byte; the
// 2-bit field of the code in byte b of quad {word 0 low nibbles, word 0 high nibbles, word 1 low, word 1
// high} sits in byte b of the high-bit word at bit 4, 6, 2 or 0, so a shift by 0, >>2, <<2 or <<4 puts
// all four fields of a quad at bits 4-5 of their bytes.
// Row strides stay 16-byte multiples because cols % 256 == 0 is required.
#if defined(__CUDACC__)
#define BRASA_HD __host__ __device__
#else
#define BRASA_HD
#endif
BRASA_HD static inline uint32_t tiled_row_bytes(int qtype, uint32_t cols) { return cols / 32 * (qtype == BRASA_Q4_0 ? 18u : 26u); }
BRASA_HD static inline uint32_t tiled_hi_off(uint32_t cols) { return cols / 32 * 16u; }
BRASA_HD static inline uint32_t tiled_scale_off(int qtype, uint32_t cols) { return cols / 32 * (qtype == BRASA_Q4_0 ? 16u : 24u); }
// word_in_pair: code word 0 or 1 of the half block; k: nibble 0..7 inside that word
BRASA_HD static inline int q6_hi_bitpos(int word_in_pair, int k) {
    int quad = 2 * word_in_pair + (k & 1), byte = k >> 1;
    int field = quad == 0 ? 4 : (quad == 1 ? 6 : (quad == 2 ? 2 : 0));
    return 8 * byte + field;
}
static inline bool tiled_ok(int qtype, uint32_t rows, uint32_t cols) {
    return (qtype == BRASA_Q4_0 || qtype == BRASA_Q6_0) && rows > 0 && cols > 0 && cols % 256 == 0;
}
