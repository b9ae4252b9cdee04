#pragma once
// GGUF reader, format versions 2 and 3 on a little-endian host. The file is treated as hostile: every read is bounds-checked, every count capped, any
// inconsistency comes back as a Status. Behaviour (limits, error codes, what is accepted) follows the reference's reader, src/format/gguf.h:1-100 and
// src/format/gguf.cpp:179-317; the tests compare the two on the same bytes.
//   DataLoss: truncated / corrupt / inconsistent     Unsupported: version or tensor type not handled     ResourceExhausted: a limit exceeded
//   NotFound / InvalidArgument / OutOfRange: the typed getters
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <string_view>
#include <vector>

#include "dtype.h"
#include "status.h"

namespace dooms {

struct GgufLimits {
    uint64_t max_kv = uint64_t(1) << 20;
    uint64_t max_tensors = uint64_t(1) << 20;
    uint64_t max_name_bytes = 256;
    uint64_t max_string_bytes = uint64_t(64) << 20;
    uint64_t max_array_elements = uint64_t(1) << 22;
    uint64_t max_alignment = uint64_t(1) << 24;
};

enum class GgufValueType : int32_t { U8 = 0, I8, U16, I16, U32, I32, F32, Bool, String, Array, U64, I64, F64 };
const char * gguf_value_type_name(GgufValueType t);

struct GgufValue {
    GgufValueType type = GgufValueType::U8;
    GgufValueType element_type = GgufValueType::U8;   // arrays
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0;
    std::string s;
    std::vector<GgufValue> items;
};

constexpr int kGgufMaxDims = 4;

struct GgufTensorInfo {
    std::string name;
    DType dtype = DType::F32;
    int rank = 0;
    int64_t shape[kGgufMaxDims] = {0, 0, 0, 0};   // row-major, outermost first (the file lists the fastest dimension first)
    uint64_t offset = 0;                          // from the start of the file
    uint64_t nbytes = 0;
    int64_t numel() const { int64_t n = 1; for (int d = 0; d < rank; d++) n *= shape[d]; return n; }
};

// A read-only mapping of a whole file.
class MappedFile {
public:
    static Result<std::shared_ptr<const MappedFile>> open(const std::string & path);
    ~MappedFile();
    MappedFile(const MappedFile &) = delete;
    MappedFile & operator=(const MappedFile &) = delete;
    const uint8_t * data() const { return data_; }
    size_t size() const { return size_; }
private:
    MappedFile(const uint8_t * d, size_t n) : data_(d), size_(n) {}
    const uint8_t * data_;
    size_t size_;
};

class GgufParser;

class GgufFile {
public:
    static Result<GgufFile> parse(const uint8_t * data, size_t size, const GgufLimits & limits = GgufLimits());   // data must outlive the object
    static Result<GgufFile> open(const std::string & path, const GgufLimits & limits = GgufLimits());             // owns the mapping

    uint32_t version() const { return version_; }
    uint64_t alignment() const { return alignment_; }
    const std::map<std::string, GgufValue> & metadata() const { return kv_; }
    Result<std::string> get_string(std::string_view key) const;
    Result<uint64_t> get_uint(std::string_view key) const;
    Result<int64_t> get_int(std::string_view key) const;
    Result<double> get_float(std::string_view key) const;
    Result<bool> get_bool(std::string_view key) const;
    const std::vector<GgufTensorInfo> & tensors() const { return tensors_; }
    Result<const GgufTensorInfo *> find_tensor(std::string_view name) const;
    const uint8_t * tensor_data(const GgufTensorInfo & info) const { return data_ + info.offset; }

private:
    friend class GgufParser;
    const GgufValue * lookup(std::string_view key) const;
    const uint8_t * data_ = nullptr;
    size_t size_ = 0;
    std::shared_ptr<const MappedFile> mapping_;
    uint32_t version_ = 0;
    uint64_t alignment_ = 0;
    std::map<std::string, GgufValue> kv_;
    std::vector<GgufTensorInfo> tensors_;
    std::map<std::string, size_t, std::less<>> index_;
};

}  // namespace dooms
