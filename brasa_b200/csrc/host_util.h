// Host-side pieces shared by the model and session code: a small JSON reader, SHA-256, the `.brasa`
// container reader, and the CPU sampler.
#pragma once
#include <stdint.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace brasa {

// ---- JSON (only what a `.brasa` header needs: objects, arrays, strings, numbers, literals) ------
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    bool is_int = false;
    int64_t inum = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json *get(const std::string &key) const;
    bool has(const std::string &key) const { return get(key) != nullptr; }
};
// Parses `text`; on failure returns false and sets err.
bool json_parse(const char *text, size_t len, Json &out, std::string &err);

// ---- SHA-256 ---------------------------------------------------------------------------------
std::string sha256_hex(const uint8_t *data, size_t len);

// ---- `.brasa` file (crates/quant/src/brasa_file.rs) --------------------------------------------
struct TensorInfo {
    std::string name, dtype, sha256;
    std::vector<uint64_t> shape;
    uint64_t offset = 0, nbytes = 0;
    uint64_t numel() const {
        uint64_t n = 1;
        for (uint64_t s : shape) n *= s;
        return n;
    }
};

class BrasaFile {
  public:
    ~BrasaFile();
    // Opens and validates structure: magic, version, bounds, page alignment, tensor sizes.
    static std::unique_ptr<BrasaFile> open(const std::string &path, std::string &err);
    // Checks every tensor's sha256 and data_sha256.
    bool verify(std::string &err) const;
    const std::vector<TensorInfo> &tensors() const { return tensors_; }
    const TensorInfo *tensor(const std::string &name) const;
    const uint8_t *data(const TensorInfo &t) const { return map_ + t.offset; }
    int fd() const { return fd_; }  // for readers that fetch tensor bytes with pread instead of touching the mapping
    const Json &config() const { return *config_; }
    const std::string &family() const { return family_; }

  private:
    const uint8_t *map_ = nullptr;
    size_t size_ = 0;
    int fd_ = -1;
    Json meta_;
    const Json *config_ = nullptr;
    std::string family_, data_sha256_;
    uint64_t page_ = 0;
    std::vector<TensorInfo> tensors_;
};

int dtype_qtype(const std::string &dtype);  // "q4_0" -> BRASA_Q4_0 ...; -1 for f32 / unknown
uint64_t dtype_nbytes(const std::string &dtype, uint64_t numel);

// ---- CPU sampler (crates/runtime/src/sampler.rs) -----------------------------------------------
struct Pcg32 {
    uint64_t state = 0, inc = 0;
    explicit Pcg32(uint64_t seed = 0);
    uint32_t next_u32();
    float next_f32();
};
uint32_t argmax_host(const float *v, size_t n);
class Sampler {
  public:
    Sampler(float temperature, uint32_t top_k, float top_p, uint64_t seed, size_t vocab);
    uint32_t sample(const float *logits, size_t n);
    bool greedy() const { return temperature_ <= 0.0f; }

  private:
    float temperature_, top_p_;
    uint32_t top_k_;
    Pcg32 rng_;
    std::vector<std::pair<uint32_t, float>> cand_;
};

}  // namespace brasa
