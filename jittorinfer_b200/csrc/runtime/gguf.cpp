#include "gguf.h"

#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace jib {

namespace {

struct Cursor {
    const uint8_t * p;
    const uint8_t * end;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (p + sizeof(T) > end) { ok = false; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > (uint64_t) (end - p)) { ok = false; return ""; }
        std::string s((const char *) p, n);
        p += n;
        return s;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
        case GT_U8: case GT_I8: case GT_BOOL: return 1;
        case GT_U16: case GT_I16: return 2;
        case GT_U32: case GT_I32: case GT_F32: return 4;
        case GT_U64: case GT_I64: case GT_F64: return 8;
        default: return 0;
    }
}

bool read_scalar(Cursor & c, uint32_t t, GgufValue & v) {
    switch (t) {
        case GT_U8: v.u = c.get<uint8_t>(); break;
        case GT_I8: v.u = (uint64_t) (int64_t) c.get<int8_t>(); break;
        case GT_U16: v.u = c.get<uint16_t>(); break;
        case GT_I16: v.u = (uint64_t) (int64_t) c.get<int16_t>(); break;
        case GT_U32: v.u = c.get<uint32_t>(); break;
        case GT_I32: v.u = (uint64_t) (int64_t) c.get<int32_t>(); break;
        case GT_U64: v.u = c.get<uint64_t>(); break;
        case GT_I64: v.u = (uint64_t) c.get<int64_t>(); break;
        case GT_BOOL: v.u = c.get<uint8_t>() != 0; break;
        case GT_F32: v.f = c.get<float>(); break;
        case GT_F64: v.f = c.get<double>(); break;
        default: return false;
    }
    return c.ok;
}

}  // namespace

uint64_t GgufFile::type_block(uint32_t t) {
    switch (t) {
        case 0: case 1: case 30: case 24: case 25: case 26: case 27: case 28: return 1;      // F32 F16 BF16 I8 I16 I32 I64 F64
        case 2: case 3: case 6: case 7: case 8: case 9: return 32;                            // Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q8_1
        case 10: case 11: case 12: case 13: case 14: case 15: return 256;                     // Q2_K Q3_K Q4_K Q5_K Q6_K Q8_K
        default: return 0;
    }
}
uint64_t GgufFile::type_block_bytes(uint32_t t) {
    switch (t) {
        case 0: return 4; case 1: return 2; case 30: return 2; case 24: return 1; case 25: return 2; case 26: return 4;
        case 27: return 8; case 28: return 8;
        case 2: return 18; case 3: return 20; case 6: return 22; case 7: return 24; case 8: return 34; case 9: return 36;
        case 10: return 84; case 11: return 110; case 12: return 144; case 13: return 176; case 14: return 210; case 15: return 292;
        default: return 0;
    }
}

GgufFile::~GgufFile() { close(); }

void GgufFile::close() {
    if (base_ != nullptr) munmap((void *) base_, size_);
    if (fd_ >= 0) ::close(fd_);
    base_ = nullptr;
    fd_ = -1;
    kv_.clear();
    tensors_.clear();
    tensor_index_.clear();
}

std::string GgufFile::open(const std::string & path, bool populate) {
    close();
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) return "cannot open " + path;
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 24) { close(); return "file too small to be GGUF"; }
    size_ = (uint64_t) st.st_size;
    int flags = MAP_PRIVATE;
#ifdef MAP_POPULATE
    if (populate) flags |= MAP_POPULATE;
#endif
    void * m = mmap(nullptr, size_, PROT_READ, flags, fd_, 0);
    if (m == MAP_FAILED) { close(); return "mmap failed"; }
    base_ = (const uint8_t *) m;
    Cursor c{base_, base_ + size_};
    if (memcmp(c.p, "GGUF", 4) != 0) { close(); return "not a GGUF file (bad magic)"; }
    c.p += 4;
    version_ = c.get<uint32_t>();
    if (version_ < 2 || version_ > 3) { close(); return "unsupported GGUF version " + std::to_string(version_); }
    const uint64_t n_tensors = c.get<uint64_t>();
    const uint64_t n_kv = c.get<uint64_t>();
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        const std::string key = c.str();
        GgufValue v;
        v.type = c.get<uint32_t>();
        if (v.type == GT_STR) {
            v.s = c.str();
        } else if (v.type == GT_ARR) {
            v.arr_type = c.get<uint32_t>();
            v.arr_n = c.get<uint64_t>();
            if (v.arr_type == GT_STR) {
                if (v.arr_n > (uint64_t) (c.end - c.p) / 8) { c.ok = false; break; }      // every string has an 8-byte length
                v.arr_s.reserve(v.arr_n);
                for (uint64_t k = 0; k < v.arr_n && c.ok; ++k) v.arr_s.push_back(c.str());
            } else {
                const size_t es = scalar_size(v.arr_type);
                if (es == 0 || v.arr_n > (uint64_t) (c.end - c.p) / es) { c.ok = false; break; }
                v.arr_data = c.p;
                c.p += v.arr_n * es;
            }
        } else if (!read_scalar(c, v.type, v)) {
            c.ok = false;
        }
        kv_[key] = std::move(v);
    }
    if (!c.ok) { close(); return "corrupt GGUF metadata"; }
    if (const GgufValue * a = find("general.alignment")) alignment_ = (uint32_t) a->as_i64();
    if (alignment_ == 0 || (alignment_ & (alignment_ - 1))) { close(); return "bad general.alignment"; }
    if (n_tensors > (uint64_t) (c.end - c.p) / 24) { close(); return "corrupt GGUF tensor table"; }      // name length + dims + type + offset
    tensors_.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        GgufTensor t;
        t.name = c.str();
        const uint32_t nd = c.get<uint32_t>();
        if (nd > 8) { c.ok = false; break; }
        uint64_t n = 1;
        for (uint32_t d = 0; d < nd; ++d) {
            t.ne.push_back(c.get<uint64_t>());
            if (t.ne.back() != 0 && n > UINT64_MAX / 64 / t.ne.back()) { c.ok = false; break; }      // element count (x block bytes) must not wrap
            n *= t.ne.back();
        }
        if (!c.ok) break;
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        const uint64_t blk = type_block(t.type);
        if (blk == 0 || n % blk) { close(); return "tensor " + t.name + ": unsupported ggml type " + std::to_string(t.type); }
        t.nbytes = n / blk * type_block_bytes(t.type);
        tensor_index_[t.name] = tensors_.size();
        tensors_.push_back(std::move(t));
    }
    if (!c.ok) { close(); return "corrupt GGUF tensor table"; }
    const uint64_t pos = (uint64_t) (c.p - base_);
    data_offset_ = (pos + alignment_ - 1) / alignment_ * alignment_;
    for (const GgufTensor & t : tensors_)
        if (data_offset_ > size_ || t.offset > size_ - data_offset_ || t.nbytes > size_ - data_offset_ - t.offset) {
            const std::string name = t.name;
            close();
            return "tensor " + name + " runs past the end of the file";
        }
    return "";
}

const GgufValue * GgufFile::find(const std::string & key) const {
    auto it = kv_.find(key);
    return it == kv_.end() ? nullptr : &it->second;
}

const GgufTensor * GgufFile::tensor(const std::string & name) const {
    auto it = tensor_index_.find(name);
    return it == tensor_index_.end() ? nullptr : &tensors_[it->second];
}

}  // namespace jib
