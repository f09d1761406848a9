// Internal declarations shared by the .cu files of libbrasa_cuda.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/brasa_cuda.h"

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
    bool pdl = true;             // programmatic dependent launch between decode kernels
    void *argmax_scratch = nullptr;  // arrival counter + per-block partial maxima
    bool gemv_attr_done[2] = {false, false};  // opt-in shared memory size set on this device
};

struct brasa_buf {
    brasa_ctx *ctx;
    void *ptr;
    uint64_t bytes;
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

// ---- tiled weight layout --------------------------------------------------------------------
// A matrix [rows, cols] is cut into micro-tiles of 64 rows x 4 blocks (128 columns), stored one
// after another with the column index fastest. Inside a micro-tile, for q4_0:
//     codes  [4 blocks][64 rows][16 bytes]   the block's 16 code bytes, unchanged
//     scales [4 blocks][64 rows] f16
// q6_0 adds the high-bit plane:  ql [4][64][16], qh [4][64][8], scales [4][64] f16.
// Total bytes equal the file layout's (18 or 26 bytes per 32 weights).
constexpr int MT_ROWS = 64;
constexpr int MT_BLOCKS = 4;
constexpr int MT_BYTES_Q4 = MT_BLOCKS * MT_ROWS * 18;  // 4608
constexpr int MT_BYTES_Q6 = MT_BLOCKS * MT_ROWS * 26;  // 6656
static inline int mt_bytes(int qtype) { return qtype == BRASA_Q4_0 ? MT_BYTES_Q4 : MT_BYTES_Q6; }
static inline bool tiled_ok(int qtype, uint32_t rows, uint32_t cols) {
    return (qtype == BRASA_Q4_0 || qtype == BRASA_Q6_0) && rows % MT_ROWS == 0 && cols % (32 * MT_BLOCKS) == 0;
}
