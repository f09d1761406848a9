// Host-side helpers: JSON, SHA-256, `.brasa` reader, CPU sampler, memory planner.
#include "host_util.h"

#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>

#include "brasa_internal.h"

namespace brasa {

// ---- JSON ------------------------------------------------------------------------------------
namespace {
struct Parser {
    const char *p, *end;
    std::string err;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
    }
    bool fail(const char *m) {
        if (err.empty()) err = m;
        return false;
    }
    static void utf8(std::string &s, uint32_t c) {
        if (c < 0x80) s += (char)c;
        else if (c < 0x800) { s += (char)(0xC0 | (c >> 6)); s += (char)(0x80 | (c & 63)); }
        else if (c < 0x10000) { s += (char)(0xE0 | (c >> 12)); s += (char)(0x80 | ((c >> 6) & 63)); s += (char)(0x80 | (c & 63)); }
        else { s += (char)(0xF0 | (c >> 18)); s += (char)(0x80 | ((c >> 12) & 63)); s += (char)(0x80 | ((c >> 6) & 63)); s += (char)(0x80 | (c & 63)); }
    }
    bool hex4(uint32_t &v) {
        if (end - p < 4) return fail("bad \\u escape");
        v = 0;
        for (int i = 0; i < 4; ++i) {
            char c = *p++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else return fail("bad \\u escape");
        }
        return true;
    }
    bool string(std::string &s) {
        if (p >= end || *p != '"') return fail("expected string");
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) return fail("bad escape");
                char c = *p++;
                switch (c) {
                case 'n': s += '\n'; break;
                case 't': s += '\t'; break;
                case 'r': s += '\r'; break;
                case 'b': s += '\b'; break;
                case 'f': s += '\f'; break;
                case 'u': {
                    uint32_t v;
                    if (!hex4(v)) return false;
                    if (v >= 0xD800 && v < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        uint32_t lo;
                        if (!hex4(lo)) return false;
                        v = 0x10000 + ((v - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(s, v);
                    break;
                }
                default: s += c;
                }
            } else {
                s += *p++;
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool value(Json &j, int depth) {
        if (depth > 64) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end");
        char c = *p;
        if (c == '{') {
            j.kind = Json::Obj;
            ++p;
            ws();
            if (p < end && *p == '}') { ++p; return true; }
            for (;;) {
                ws();
                std::string k;
                if (!string(k)) return false;
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                ++p;
                j.obj.emplace_back(std::move(k), Json());
                if (!value(j.obj.back().second, depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            j.kind = Json::Arr;
            ++p;
            ws();
            if (p < end && *p == ']') { ++p; return true; }
            for (;;) {
                j.arr.emplace_back();
                if (!value(j.arr.back(), depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') {
            j.kind = Json::Str;
            return string(j.str);
        }
        if (end - p >= 4 && !strncmp(p, "true", 4)) { j.kind = Json::Bool; j.b = true; p += 4; return true; }
        if (end - p >= 5 && !strncmp(p, "false", 5)) { j.kind = Json::Bool; j.b = false; p += 5; return true; }
        if (end - p >= 4 && !strncmp(p, "null", 4)) { j.kind = Json::Null; p += 4; return true; }
        const char *s = p;
        bool isint = true;
        if (p < end && (*p == '-' || *p == '+')) ++p;
        while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
            if (*p == '.' || *p == 'e' || *p == 'E') isint = false;
            ++p;
        }
        if (p == s) return fail("unexpected character");
        std::string t(s, p);
        j.kind = Json::Num;
        j.num = strtod(t.c_str(), nullptr);
        j.is_int = isint;
        if (isint) j.inum = strtoll(t.c_str(), nullptr, 10);
        return true;
    }
};
}  // namespace

const Json *Json::get(const std::string &key) const {
    if (kind != Obj) return nullptr;
    for (auto &kv : obj)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

bool json_parse(const char *text, size_t len, Json &out, std::string &err) {
    Parser ps{text, text + len, ""};
    if (!ps.value(out, 0)) { err = ps.err; return false; }
    ps.ws();
    if (ps.p != ps.end) { err = "trailing characters"; return false; }
    return true;
}

// ---- SHA-256 (FIPS 180-4) ----------------------------------------------------------------------
namespace {
const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be,
    0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa,
    0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85,
    0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3,
    0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f,
    0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
void sha_block(uint32_t h[8], const uint8_t *p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
        uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
        uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
        w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
        uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K256[i] + w[i];
        uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
        hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
}  // namespace

std::string sha256_hex(const uint8_t *data, size_t len) {
    uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    size_t full = len / 64;
    for (size_t i = 0; i < full; ++i) sha_block(h, data + 64 * i);
    uint8_t tail[128] = {0};
    size_t rem = len - full * 64;
    if (rem) memcpy(tail, data + full * 64, rem);
    tail[rem] = 0x80;
    size_t tl = rem + 9 <= 64 ? 64 : 128;
    uint64_t bits = (uint64_t)len * 8;
    for (int i = 0; i < 8; ++i) tail[tl - 1 - i] = (uint8_t)(bits >> (8 * i));
    sha_block(h, tail);
    if (tl == 128) sha_block(h, tail + 64);
    static const char *hex = "0123456789abcdef";
    std::string out(64, '0');
    for (int i = 0; i < 8; ++i)
        for (int j = 0; j < 4; ++j) {
            uint8_t byte = (uint8_t)(h[i] >> (24 - 8 * j));
            out[8 * i + 2 * j] = hex[byte >> 4];
            out[8 * i + 2 * j + 1] = hex[byte & 15];
        }
    return out;
}

// ---- `.brasa` ----------------------------------------------------------------------------------
int dtype_qtype(const std::string &d) {
    if (d == "q4_0") return BRASA_Q4_0;
    if (d == "q8_0") return BRASA_Q8_0;
    if (d == "q6_0") return BRASA_Q6_0;
    return -1;
}
uint64_t dtype_nbytes(const std::string &d, uint64_t n) {
    if (d == "f32") return n * 4;
    int q = dtype_qtype(d);
    return q < 0 ? 0 : brasa_qtype_nbytes(q, n);
}

BrasaFile::~BrasaFile() {
    if (map_) munmap((void *)map_, size_);
    if (fd_ >= 0) close(fd_);
}

std::unique_ptr<BrasaFile> BrasaFile::open(const std::string &path, std::string &err) {
    auto bad = [&](const std::string &m) {
        err = path + ": " + m;
        return std::unique_ptr<BrasaFile>();
    };
    std::unique_ptr<BrasaFile> f(new BrasaFile());
    f->fd_ = ::open(path.c_str(), O_RDONLY);
    if (f->fd_ < 0) return bad("cannot open");
    struct stat st;
    if (fstat(f->fd_, &st) != 0) return bad("cannot stat");
    f->size_ = (size_t)st.st_size;
    if (f->size_ < 16) return bad("not a .brasa file");
    void *m = mmap(nullptr, f->size_, PROT_READ, MAP_PRIVATE, f->fd_, 0);
    if (m == MAP_FAILED) return bad("mmap failed");
    f->map_ = (const uint8_t *)m;
    const uint8_t *b = f->map_;
    if (memcmp(b, "BRSA", 4) != 0) return bad("not a .brasa file");
    uint32_t version;
    uint64_t jlen;
    memcpy(&version, b + 4, 4);
    memcpy(&jlen, b + 8, 8);
    if (version != 1) return bad("unsupported version " + std::to_string(version));
    if (jlen > f->size_ - 16) return bad("truncated header");
    std::string jerr;
    if (!json_parse((const char *)b + 16, (size_t)jlen, f->meta_, jerr)) return bad("header: " + jerr);
    const Json &meta = f->meta_;
    const Json *fmt = meta.get("format"), *ver = meta.get("version"), *model = meta.get("model"), *page = meta.get("page"),
               *tensors = meta.get("tensors"), *dsha = meta.get("data_sha256");
    if (!fmt || fmt->kind != Json::Str || fmt->str != "brasa" || !ver || ver->kind != Json::Num || ver->inum != 1) return bad("inconsistent header");
    if (!model || !page || page->kind != Json::Num || page->inum <= 0 || !tensors || tensors->kind != Json::Arr || !dsha || dsha->kind != Json::Str)
        return bad("header: missing fields");
    const Json *fam = model->get("family"), *cfg = model->get("config");
    if (!fam || fam->kind != Json::Str || !cfg || cfg->kind != Json::Obj) return bad("header: missing model fields");
    f->family_ = fam->str;
    f->config_ = cfg;
    f->page_ = (uint64_t)page->inum;
    f->data_sha256_ = dsha->str;
    for (const Json &t : tensors->arr) {
        TensorInfo ti;
        const Json *n = t.get("name"), *d = t.get("dtype"), *s = t.get("shape"), *o = t.get("offset"), *nb = t.get("nbytes"), *sh = t.get("sha256");
        if (!n || n->kind != Json::Str || !d || d->kind != Json::Str || !s || s->kind != Json::Arr || !o || o->kind != Json::Num || !nb ||
            nb->kind != Json::Num || !sh || sh->kind != Json::Str)
            return bad("header: bad tensor entry");
        ti.name = n->str;
        ti.dtype = d->str;
        ti.sha256 = sh->str;
        for (const Json &e : s->arr) ti.shape.push_back((uint64_t)e.inum);
        ti.offset = (uint64_t)o->inum;
        ti.nbytes = (uint64_t)nb->inum;
        if (ti.dtype != "f32" && dtype_qtype(ti.dtype) < 0) return bad(ti.name + ": unknown dtype " + ti.dtype);
        if (ti.offset % f->page_ != 0) return bad(ti.name + " is not page aligned");
        if (ti.dtype != "f32" && (ti.shape.empty() || ti.shape.back() % 32 != 0)) return bad(ti.name + ": last dimension is not a multiple of 32");
        if (dtype_nbytes(ti.dtype, ti.numel()) != ti.nbytes) return bad(ti.name + ": inconsistent size");
        if (ti.offset > f->size_ || ti.nbytes > f->size_ - ti.offset) return bad(ti.name + ": outside the file");
        f->tensors_.push_back(std::move(ti));
    }
    return f;
}

const TensorInfo *BrasaFile::tensor(const std::string &name) const {
    for (auto &t : tensors_)
        if (t.name == name) return &t;
    return nullptr;
}

bool BrasaFile::verify(std::string &err) const {
    std::string all;
    all.reserve(64 * tensors_.size());
    for (auto &t : tensors_) {
        std::string h = sha256_hex(data(t), t.nbytes);
        if (h != t.sha256) {
            err = t.name + ": sha256 mismatch";
            return false;
        }
        all += h;
    }
    if (sha256_hex((const uint8_t *)all.data(), all.size()) != data_sha256_) {
        err = "data_sha256 mismatch";
        return false;
    }
    return true;
}

// ---- sampler -----------------------------------------------------------------------------------
Pcg32::Pcg32(uint64_t seed) {
    state = 0;
    inc = (0xda3e39cb94b95bdbULL << 1) | 1;
    next_u32();
    state += seed;
    next_u32();
}
uint32_t Pcg32::next_u32() {
    uint64_t old = state;
    state = old * 6364136223846793005ULL + inc;
    uint32_t x = (uint32_t)(((old >> 18) ^ old) >> 27);
    uint32_t rot = (uint32_t)(old >> 59);
    return (x >> rot) | (x << ((32 - rot) & 31));
}
float Pcg32::next_f32() { return (float)(next_u32() >> 8) / 16777216.0f; }

uint32_t argmax_host(const float *v, size_t n) {
    float m = -INFINITY;
    for (size_t i = 0; i < n; ++i)
        if (v[i] > m) m = v[i];
    if (m == -INFINITY) return 0;
    for (size_t i = 0; i < n; ++i)
        if (v[i] == m) return (uint32_t)i;
    return 0;
}

Sampler::Sampler(float temperature, uint32_t top_k, float top_p, uint64_t seed, size_t vocab)
    : temperature_(temperature), top_p_(top_p), top_k_(top_k), rng_(seed) {
    cand_.reserve(vocab);
}

static inline int32_t total_key(float f) {
    int32_t b;
    memcpy(&b, &f, 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}

uint32_t Sampler::sample(const float *logits, size_t n) {
    if (temperature_ <= 0.0f) return argmax_host(logits, n);
    cand_.clear();
    for (size_t i = 0; i < n; ++i) cand_.emplace_back((uint32_t)i, logits[i]);
    // descending by logit in f32 total order; equal logits keep ascending token id
    auto by_logit = [](const std::pair<uint32_t, float> &a, const std::pair<uint32_t, float> &b) {
        int32_t ka = total_key(a.second), kb = total_key(b.second);
        return ka != kb ? ka > kb : a.first < b.first;
    };
    if (top_k_ > 0 && top_k_ < cand_.size()) {
        std::nth_element(cand_.begin(), cand_.begin() + (top_k_ - 1), cand_.end(), by_logit);
        cand_.resize(top_k_);
    }
    std::sort(cand_.begin(), cand_.end(), by_logit);
    float mx = cand_[0].second, sum = 0.0f;
    for (auto &c : cand_) {
        c.second = expf((c.second - mx) / temperature_);
        sum += c.second;
    }
    size_t keep = cand_.size();
    if (top_p_ < 1.0f) {
        float acc = 0.0f;
        for (size_t i = 0; i < cand_.size(); ++i) {
            acc += cand_[i].second / sum;
            if (acc >= top_p_) { keep = i + 1; break; }
        }
    }
    float total = 0.0f;
    for (size_t i = 0; i < keep; ++i) total += cand_[i].second;
    float r = rng_.next_f32() * total;
    for (size_t i = 0; i < keep; ++i) {
        r -= cand_[i].second;
        if (r <= 0.0f) return cand_[i].first;
    }
    return cand_[keep - 1].first;
}

}  // namespace brasa

// ---- memory planner (crates/memory/src/planner.rs:57-95, retargeted) -------------------------------
// Device allocations come in 2 MiB granules for large buffers and 512-byte granules for small ones;
// the plan charges every buffer the next multiple of 512 bytes (what cudaMalloc hands out inside a
// granule) and one 2 MiB granule of slack per large class.
extern "C" {

uint64_t brasa_plan_buffer_bytes(uint64_t n) {
    const uint64_t g = 512;
    if (n == 0) n = 1;
    return (n + g - 1) / g * g;
}

static uint64_t workspace_bytes(const brasa_model_shape *m, const brasa_session_shape *s) {
    auto f = [](uint64_t n) { return brasa_plan_buffer_bytes(4 * n); };
    uint64_t t = s->max_tokens, h = m->hidden, qd = (uint64_t)m->heads * m->head_dim, kvd = (uint64_t)m->kv_heads * m->head_dim, ffn = m->ffn;
    uint64_t widest = std::max(ffn, std::max(qd, h));
    return 3 * f(t * h)                                 // x, h, norm_out
           + 2 * f(t * qd)                              // q, attn
           + 2 * f(t * kvd)                             // k_new, v_new
           + 2 * f(t * ffn)                             // gate, up
           + brasa_plan_buffer_bytes(2 * t * widest)    // xh: f16 input of the prefill GEMMs
           + f(t)                                       // ids
           + f(brasa_norm_partials(m->hidden))          // partial sums of RMSNorm in decode
           + f(brasa_decode_partials_len(m->heads, s->ctx))  // decode attention partials
           + f((uint64_t)s->max_logit_rows * m->vocab)  // logits
           + 2 * f((uint64_t)s->ctx * m->head_dim / 2); // RoPE cos and sin tables
}

static uint64_t kv_cache_bytes(const brasa_model_shape *m, const brasa_session_shape *s) {
    uint64_t cap = ((uint64_t)s->ctx + BRASA_KV_ALIGN - 1) / BRASA_KV_ALIGN * BRASA_KV_ALIGN;
    uint64_t elems = (uint64_t)m->layers * cap * m->kv_heads * m->head_dim;
    return 2 * brasa_plan_buffer_bytes(brasa_kv_bytes(s->kv, elems));
}

int32_t brasa_plan(const brasa_model_shape *m, const brasa_session_shape *s, brasa_memory_plan *out) {
    if (!m || !s || !out) return BRASA_EINVAL;
    if (s->kv < BRASA_KV_F32 || s->kv > BRASA_KV_Q8_0) return BRASA_EINVAL;
    out->weights = m->weight_bytes;
    out->kv = kv_cache_bytes(m, s);
    out->workspace = workspace_bytes(m, s);
    out->overhead = 256ull << 20;  // CUDA context, kernel images and split-K scratch
    out->total = out->weights + out->kv + out->workspace + out->overhead;
    return BRASA_OK;
}

int32_t brasa_plan_check(brasa_ctx *ctx, const brasa_model_shape *m, const brasa_session_shape *s, uint64_t budget, brasa_memory_plan *out,
                         uint32_t *max_ctx_out) {
    if (!m || !s) return BRASA_EINVAL;
    brasa_memory_plan plan;
    BRASA_TRY(brasa_plan(m, s, &plan));
    if (out) *out = plan;
    if (budget == 0) {
        if (!ctx) return BRASA_EINVAL;
        uint64_t free_b = 0, total_b = 0;
        BRASA_TRY(brasa_ctx_mem_info(ctx, &free_b, &total_b));
        uint64_t reserve = 512ull << 20;
        budget = free_b > reserve ? free_b - reserve : 0;
        budget += plan.overhead;  // the context is already paid for inside `free`
    }
    if (max_ctx_out) *max_ctx_out = s->ctx;
    if (plan.total <= budget) return BRASA_OK;
    // largest context that fits: the plan grows monotonically with ctx
    uint32_t lo = 0, hi = s->ctx;
    while (lo < hi) {
        uint32_t mid = lo + (hi - lo + 1) / 2;
        brasa_session_shape t = *s;
        t.ctx = mid;
        if (t.max_tokens > mid) t.max_tokens = mid;
        brasa_memory_plan p;
        brasa_plan(m, &t, &p);
        if (p.total <= budget) lo = mid;
        else hi = mid - 1;
    }
    if (max_ctx_out) *max_ctx_out = lo;
    return brasa_fail(ctx, BRASA_EBUDGET, "the model needs %.2f GiB (weights %.2f, KV %.2f, workspace %.2f, overhead %.2f) and the budget is %.2f GiB; the largest context that fits is %u",
                      plan.total / 1073741824.0, plan.weights / 1073741824.0, plan.kv / 1073741824.0, plan.workspace / 1073741824.0,
                      plan.overhead / 1073741824.0, budget / 1073741824.0, lo);
}

int32_t brasa_file_check(const char *path, int32_t verify, char *err, uint64_t err_len) {
    std::string e;
    auto f = brasa::BrasaFile::open(path ? path : "", e);
    if (f && verify && !f->verify(e)) f.reset();
    if (!f) {
        if (err && err_len) snprintf(err, (size_t)err_len, "%s", e.c_str());
        return BRASA_EIO;
    }
    if (err && err_len) err[0] = 0;
    return BRASA_OK;
}

}  // extern "C"
