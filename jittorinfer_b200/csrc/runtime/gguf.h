// GGUF v2/v3 reader over a read-only memory mapping.
//
// Counterpart of the reference's gguf_init_from_file + llama_model_loader metadata side
// (ggml/src/gguf.cpp; src/llama-model-loader.cpp:488-541, 113-303) and llama_mmap (src/llama-mmap.cpp:144-404):
// header / KV / tensor table are parsed once, tensor data stays in the mapping and is handed out as pointers, so a
// tensor-parallel rank touches only the bytes of its own shard.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace jib {

enum GgufType : uint32_t { GT_U8 = 0, GT_I8, GT_U16, GT_I16, GT_U32, GT_I32, GT_F32, GT_BOOL, GT_STR, GT_ARR, GT_U64, GT_I64, GT_F64 };

struct GgufValue {
    uint32_t type = GT_U32;          // GgufType; for arrays the element type is in arr_type
    uint32_t arr_type = GT_U32;
    uint64_t u = 0;                  // integer / bool payload
    double f = 0.0;                  // float payload
    std::string s;                   // string payload
    uint64_t arr_n = 0;
    const uint8_t * arr_data = nullptr;          // numeric arrays: points into the mapping
    std::vector<std::string> arr_s;              // string arrays

    bool is_int() const { return type != GT_F32 && type != GT_F64 && type != GT_STR && type != GT_ARR; }
    double as_f64() const { return (type == GT_F32 || type == GT_F64) ? f : (double) (int64_t) u; }
    int64_t as_i64() const {
        if (type != GT_F32 && type != GT_F64) return (int64_t) u;
        return f >= -9.2e18 && f <= 9.2e18 ? (int64_t) f : 0;          // NaN and out-of-range values have no integer reading
    }
};

struct GgufTensor {
    std::string name;
    std::vector<uint64_t> ne;        // ggml order: ne[0] is the contiguous axis
    uint32_t type = 0;               // ggml_type
    uint64_t offset = 0;             // relative to the data section
    uint64_t nbytes = 0;
};

class GgufFile {
  public:
    GgufFile() = default;
    ~GgufFile();
    GgufFile(const GgufFile &) = delete;
    GgufFile & operator=(const GgufFile &) = delete;

    // Returns an empty string on success, else the reason.
    std::string open(const std::string & path, bool populate = false);
    void close();

    uint32_t version() const { return version_; }
    uint32_t alignment() const { return alignment_; }
    const std::map<std::string, GgufValue> & kv() const { return kv_; }
    const GgufValue * find(const std::string & key) const;
    const std::vector<GgufTensor> & tensors() const { return tensors_; }
    const GgufTensor * tensor(const std::string & name) const;
    const uint8_t * tensor_data(const GgufTensor & t) const { return base_ + data_offset_ + t.offset; }
    uint64_t file_size() const { return size_; }

    static uint64_t type_block(uint32_t ggml_type);     // elements per block (0 = unknown type)
    static uint64_t type_block_bytes(uint32_t ggml_type);

  private:
    int fd_ = -1;
    const uint8_t * base_ = nullptr;
    uint64_t size_ = 0, data_offset_ = 0;
    uint32_t version_ = 0, alignment_ = 32;
    std::map<std::string, GgufValue> kv_;
    std::vector<GgufTensor> tensors_;
    std::map<std::string, size_t> tensor_index_;
};

}  // namespace jib
