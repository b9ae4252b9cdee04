#include "gguf.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <limits>

namespace dooms {

static_assert(__BYTE_ORDER__ == __ORDER_LITTLE_ENDIAN__, "little-endian hosts only");

// ---- file mapping (the reference's src/format/mapped_file.cpp:14-32: NotFound / DataLoss / InvalidArgument / ResourceExhausted) ----
Result<std::shared_ptr<const MappedFile>> MappedFile::open(const std::string & path) {
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) return not_found("cannot open '" + path + "': " + std::strerror(errno));
    struct stat st;
    if (::fstat(fd, &st) != 0) { const int e = errno; ::close(fd); return data_loss("cannot stat '" + path + "': " + std::strerror(e)); }
    if (!S_ISREG(st.st_mode)) { ::close(fd); return invalid_argument("'" + path + "' is not a regular file"); }
    if (st.st_size <= 0) { ::close(fd); return data_loss("'" + path + "' is empty"); }
    void * p = ::mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    const int e = errno;
    ::close(fd);
    if (p == MAP_FAILED) return resource_exhausted("cannot map '" + path + "': " + std::strerror(e));
    return std::shared_ptr<const MappedFile>(new MappedFile(static_cast<const uint8_t *>(p), static_cast<size_t>(st.st_size)));
}
MappedFile::~MappedFile() { if (data_) ::munmap(const_cast<uint8_t *>(data_), size_); }

namespace {

// ggml_type ids of the tensor types the decoder can hold (ggml.h enum ggml_type; the reference's src/format/gguf.cpp:22-23).
bool ggml_type_to_dtype(int32_t id, DType * out) {
    switch (id) {
        case 0: *out = DType::F32; return true;
        case 1: *out = DType::F16; return true;
        case 2: *out = DType::Q4_0; return true;
        case 6: *out = DType::Q5_0; return true;
        case 8: *out = DType::Q8_0; return true;
        case 12: *out = DType::Q4_K; return true;
        case 14: *out = DType::Q6_K; return true;
        case 26: *out = DType::I32; return true;
        case 30: *out = DType::BF16; return true;
    }
    return false;
}

// Byte width of the fixed-size value types; 0 for string / array.
int scalar_width(GgufValueType t) {
    switch (t) {
        case GgufValueType::U8: case GgufValueType::I8: case GgufValueType::Bool: return 1;
        case GgufValueType::U16: case GgufValueType::I16: return 2;
        case GgufValueType::U32: case GgufValueType::I32: case GgufValueType::F32: return 4;
        case GgufValueType::U64: case GgufValueType::I64: case GgufValueType::F64: return 8;
        default: return 0;
    }
}
bool is_signed_int(GgufValueType t) { return t == GgufValueType::I8 || t == GgufValueType::I16 || t == GgufValueType::I32 || t == GgufValueType::I64; }
bool is_unsigned_int(GgufValueType t) { return t == GgufValueType::U8 || t == GgufValueType::U16 || t == GgufValueType::U32 || t == GgufValueType::U64; }

// A bounds-checked forward reader over the file's bytes.
struct Reader {
    const uint8_t * base;
    uint64_t size, at = 0;
    uint64_t left() const { return size - at; }
    Status short_read(const char * what, uint64_t need) const {
        return data_loss("file truncated at offset " + std::to_string(at) + " while reading " + what + " (needs " + std::to_string(need) + " bytes, " +
                         std::to_string(left()) + " left)");
    }
    Status bytes(void * out, uint64_t n, const char * what) {
        if (left() < n) return short_read(what, n);
        std::memcpy(out, base + at, static_cast<size_t>(n));
        at += n;
        return Status();
    }
    template <class T> Status get(T * out, const char * what) { return bytes(out, sizeof(T), what); }
    Status string(std::string * out, const char * what, uint64_t cap) {
        uint64_t n = 0;
        DOOMS_RETURN_IF_ERROR(get(&n, what));
        if (n > cap) {
            return resource_exhausted(std::string(what) + ": string of " + std::to_string(n) + " bytes at offset " + std::to_string(at) + " exceeds the limit of " +
                                      std::to_string(cap));
        }
        if (left() < n) return short_read(what, n);
        out->assign(reinterpret_cast<const char *>(base + at), static_cast<size_t>(n));
        at += n;
        return Status();
    }
};

Status read_plain(Reader & r, GgufValueType t, GgufValue * v, const GgufLimits & lim, const char * what) {
    v->type = t;
    if (t == GgufValueType::String) return r.string(&v->s, what, lim.max_string_bytes);
    const int w = scalar_width(t);
    if (w == 0) return internal_error("read_plain on an array");
    uint8_t raw[8] = {0};
    DOOMS_RETURN_IF_ERROR(r.bytes(raw, static_cast<uint64_t>(w), what));
    if (t == GgufValueType::F32) { float f; std::memcpy(&f, raw, 4); v->f = f; }
    else if (t == GgufValueType::F64) { std::memcpy(&v->f, raw, 8); }
    else if (is_signed_int(t)) {
        int64_t x = 0;
        std::memcpy(&x, raw, static_cast<size_t>(w));
        const int shift = 64 - 8 * w;
        v->i = static_cast<int64_t>(static_cast<uint64_t>(x) << shift) >> shift;   // sign-extend
    } else {
        std::memcpy(&v->u, raw, static_cast<size_t>(w));
        if (t == GgufValueType::Bool && v->u > 1) return data_loss(std::string(what) + ": bool value " + std::to_string(v->u) + " is not 0 or 1");
    }
    return Status();
}

Status value_type_of(int32_t id, const std::string & what, GgufValueType * out) {
    if (id < 0 || id > static_cast<int32_t>(GgufValueType::F64)) return unsupported(what + ": unknown value type " + std::to_string(id));
    *out = static_cast<GgufValueType>(id);
    return Status();
}

Status read_kv_value(Reader & r, GgufValue * v, const GgufLimits & lim, const std::string & key) {
    const std::string what = "value of '" + key + "'";
    int32_t id = 0;
    DOOMS_RETURN_IF_ERROR(r.get(&id, what.c_str()));
    GgufValueType t;
    DOOMS_RETURN_IF_ERROR(value_type_of(id, what, &t));
    if (t != GgufValueType::Array) return read_plain(r, t, v, lim, what.c_str());
    v->type = GgufValueType::Array;
    int32_t elem_id = 0;
    uint64_t count = 0;
    DOOMS_RETURN_IF_ERROR(r.get(&elem_id, what.c_str()));
    DOOMS_RETURN_IF_ERROR(r.get(&count, what.c_str()));
    GgufValueType et;
    DOOMS_RETURN_IF_ERROR(value_type_of(elem_id, what, &et));
    if (et == GgufValueType::Array) return unsupported(what + ": nested arrays are not supported");
    v->element_type = et;
    if (count > lim.max_array_elements) {
        return resource_exhausted(what + ": array of " + std::to_string(count) + " elements exceeds the limit of " + std::to_string(lim.max_array_elements));
    }
    if (count > r.left()) return data_loss(what + ": array claims " + std::to_string(count) + " elements but only " + std::to_string(r.left()) + " bytes remain");
    v->items.resize(static_cast<size_t>(count));
    for (GgufValue & item : v->items) DOOMS_RETURN_IF_ERROR(read_plain(r, et, &item, lim, what.c_str()));
    return Status();
}

}  // namespace

const char * gguf_value_type_name(GgufValueType t) {
    static const char * names[] = {"u8", "i8", "u16", "i16", "u32", "i32", "f32", "bool", "string", "array", "u64", "i64", "f64"};
    const int32_t i = static_cast<int32_t>(t);
    return (i >= 0 && i <= 12) ? names[i] : "unknown";
}

Result<GgufFile> GgufFile::parse(const uint8_t * data, size_t size, const GgufLimits & lim) {
    if (!data || size == 0) return invalid_argument("no data to parse");
    Reader r{data, size};
    char magic[4];
    DOOMS_RETURN_IF_ERROR(r.get(&magic, "magic"));
    if (std::memcmp(magic, "GGUF", 4) != 0) return data_loss("not a GGUF file (bad magic)");
    GgufFile f;
    f.data_ = data;
    f.size_ = size;
    DOOMS_RETURN_IF_ERROR(r.get(&f.version_, "version"));
    if (f.version_ < 2 || f.version_ > 3) {
        std::string msg = "GGUF version " + std::to_string(f.version_) + " is not supported (supported: 2 to 3)";
        if ((f.version_ & 0xFFFF) == 0) msg += "; the file may have been written on a machine with different endianness";
        return unsupported(msg);
    }
    uint64_t n_tensors = 0, n_kv = 0;
    DOOMS_RETURN_IF_ERROR(r.get(&n_tensors, "tensor count"));
    DOOMS_RETURN_IF_ERROR(r.get(&n_kv, "metadata count"));
    if (n_tensors > lim.max_tensors) return resource_exhausted("tensor count " + std::to_string(n_tensors) + " exceeds the limit of " + std::to_string(lim.max_tensors));
    if (n_kv > lim.max_kv) return resource_exhausted("metadata count " + std::to_string(n_kv) + " exceeds the limit of " + std::to_string(lim.max_kv));

    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key;
        DOOMS_RETURN_IF_ERROR(r.string(&key, "metadata key", lim.max_name_bytes));
        if (key.empty()) return data_loss("metadata entry " + std::to_string(k) + " has an empty key");
        GgufValue v;
        DOOMS_RETURN_IF_ERROR(read_kv_value(r, &v, lim, key));
        if (!f.kv_.emplace(key, std::move(v)).second) return data_loss("duplicate metadata key '" + key + "'");
    }

    f.alignment_ = 32;
    if (const GgufValue * al = f.lookup("general.alignment")) {
        if (al->type != GgufValueType::U32) return data_loss(std::string("general.alignment must be a u32, got ") + gguf_value_type_name(al->type));
        f.alignment_ = al->u;
        if (f.alignment_ == 0 || (f.alignment_ & (f.alignment_ - 1)) != 0 || f.alignment_ > lim.max_alignment) {
            return data_loss("general.alignment = " + std::to_string(f.alignment_) + " must be a power of two no larger than " + std::to_string(lim.max_alignment));
        }
    }

    f.tensors_.reserve(static_cast<size_t>(std::min<uint64_t>(n_tensors, r.left())));
    for (uint64_t t = 0; t < n_tensors; t++) {
        GgufTensorInfo info;
        DOOMS_RETURN_IF_ERROR(r.string(&info.name, "tensor name", lim.max_name_bytes));
        if (info.name.empty()) return data_loss("tensor " + std::to_string(t) + " has an empty name");
        if (f.index_.count(info.name)) return data_loss("duplicate tensor name '" + info.name + "'");
        uint32_t n_dims = 0;
        DOOMS_RETURN_IF_ERROR(r.get(&n_dims, "tensor rank"));
        if (n_dims > static_cast<uint32_t>(kGgufMaxDims)) {
            return data_loss("tensor '" + info.name + "' has " + std::to_string(n_dims) + " dimensions; the maximum is " + std::to_string(kGgufMaxDims));
        }
        info.rank = static_cast<int>(n_dims);
        int64_t numel = 1;
        for (uint32_t d = 0; d < n_dims; d++) {
            int64_t dim = 0;
            DOOMS_RETURN_IF_ERROR(r.get(&dim, "tensor dimension"));
            if (dim < 1) return data_loss("tensor '" + info.name + "' dimension " + std::to_string(d) + " is " + std::to_string(dim) + "; dimensions must be >= 1");
            if (numel > std::numeric_limits<int64_t>::max() / dim) return data_loss("tensor '" + info.name + "': the element count overflows");
            numel *= dim;
            info.shape[n_dims - 1 - d] = dim;
        }
        int32_t type_id = 0;
        DOOMS_RETURN_IF_ERROR(r.get(&type_id, "tensor type"));
        if (!ggml_type_to_dtype(type_id, &info.dtype)) {
            return unsupported("tensor '" + info.name + "' has ggml type " + std::to_string(type_id) + ", which this reader does not support");
        }
        const int64_t block = dtype_block_elems(info.dtype);
        const int64_t row = info.rank > 0 ? info.shape[info.rank - 1] : 1;
        if (row % block != 0) {
            return data_loss("tensor '" + info.name + "' has rows of " + std::to_string(row) + " elements, not a multiple of the " + dtype_name(info.dtype) +
                             " block of " + std::to_string(block));
        }
        const uint64_t blocks = static_cast<uint64_t>(numel / block), bb = static_cast<uint64_t>(dtype_block_bytes(info.dtype));
        if (blocks > std::numeric_limits<uint64_t>::max() / bb) return data_loss("tensor '" + info.name + "' byte size overflows");
        info.nbytes = blocks * bb;
        DOOMS_RETURN_IF_ERROR(r.get(&info.offset, "tensor data offset"));   // relative to the data section until the checks below pass
        f.index_.emplace(info.name, f.tensors_.size());
        f.tensors_.push_back(std::move(info));
    }
    if (f.tensors_.empty()) return f;

    const uint64_t data_start = (r.at + (f.alignment_ - 1)) & ~(f.alignment_ - 1);
    if (data_start > size) return data_loss("file ends at " + std::to_string(size) + " before the data section at " + std::to_string(data_start));
    const uint64_t data_size = size - data_start;
    for (const GgufTensorInfo & t : f.tensors_) {
        if (t.offset % f.alignment_ != 0) {
            return data_loss("tensor '" + t.name + "' offset " + std::to_string(t.offset) + " is not a multiple of the alignment " + std::to_string(f.alignment_));
        }
        if (t.offset > data_size || t.nbytes > data_size - t.offset) {
            return data_loss("tensor '" + t.name + "' (" + std::to_string(t.nbytes) + " bytes at data offset " + std::to_string(t.offset) +
                             ") extends past the end of the file (data section is " + std::to_string(data_size) + " bytes)");
        }
    }
    std::vector<const GgufTensorInfo *> by_offset;
    for (const GgufTensorInfo & t : f.tensors_) by_offset.push_back(&t);
    std::sort(by_offset.begin(), by_offset.end(), [](const GgufTensorInfo * a, const GgufTensorInfo * b) { return a->offset < b->offset; });
    for (size_t i = 1; i < by_offset.size(); i++) {
        if (by_offset[i - 1]->offset + by_offset[i - 1]->nbytes > by_offset[i]->offset) {
            return data_loss("tensors '" + by_offset[i - 1]->name + "' and '" + by_offset[i]->name + "' overlap in the data section");
        }
    }
    for (GgufTensorInfo & t : f.tensors_) t.offset += data_start;
    return f;
}

Result<GgufFile> GgufFile::open(const std::string & path, const GgufLimits & lim) {
    auto mapped = MappedFile::open(path);
    if (!mapped.is_ok()) return mapped.status();
    auto parsed = parse(mapped.value()->data(), mapped.value()->size(), lim);
    if (!parsed.is_ok()) return Status(parsed.status().code(), path + ": " + parsed.status().message());
    GgufFile f = std::move(parsed).value();
    f.mapping_ = mapped.value();
    return f;
}

const GgufValue * GgufFile::lookup(std::string_view key) const {
    auto it = kv_.find(std::string(key));
    return it == kv_.end() ? nullptr : &it->second;
}

namespace {
Status missing(std::string_view key) { return not_found("no metadata key '" + std::string(key) + "'"); }
Status mistyped(std::string_view key, GgufValueType got, const char * want) {
    return invalid_argument("metadata '" + std::string(key) + "' has type " + gguf_value_type_name(got) + ", expected " + want);
}
}  // namespace

Result<std::string> GgufFile::get_string(std::string_view key) const {
    const GgufValue * v = lookup(key);
    if (!v) return missing(key);
    if (v->type != GgufValueType::String) return mistyped(key, v->type, "string");
    return v->s;
}
Result<uint64_t> GgufFile::get_uint(std::string_view key) const {
    const GgufValue * v = lookup(key);
    if (!v) return missing(key);
    if (is_unsigned_int(v->type)) return v->u;
    if (!is_signed_int(v->type)) return mistyped(key, v->type, "an integer");
    if (v->i < 0) return out_of_range("metadata '" + std::string(key) + "' is " + std::to_string(v->i) + ", expected >= 0");
    return static_cast<uint64_t>(v->i);
}
Result<int64_t> GgufFile::get_int(std::string_view key) const {
    const GgufValue * v = lookup(key);
    if (!v) return missing(key);
    if (is_signed_int(v->type)) return v->i;
    if (!is_unsigned_int(v->type)) return mistyped(key, v->type, "an integer");
    if (v->u > static_cast<uint64_t>(std::numeric_limits<int64_t>::max())) {
        return out_of_range("metadata '" + std::string(key) + "' is " + std::to_string(v->u) + ", which does not fit in int64");
    }
    return static_cast<int64_t>(v->u);
}
Result<double> GgufFile::get_float(std::string_view key) const {
    const GgufValue * v = lookup(key);
    if (!v) return missing(key);
    if (v->type != GgufValueType::F32 && v->type != GgufValueType::F64) return mistyped(key, v->type, "a float");
    return v->f;
}
Result<bool> GgufFile::get_bool(std::string_view key) const {
    const GgufValue * v = lookup(key);
    if (!v) return missing(key);
    if (v->type != GgufValueType::Bool) return mistyped(key, v->type, "bool");
    return v->u != 0;
}
Result<const GgufTensorInfo *> GgufFile::find_tensor(std::string_view name) const {
    auto it = index_.find(name);
    if (it == index_.end()) return not_found("no tensor named '" + std::string(name) + "'");
    return &tensors_[it->second];
}

}  // namespace dooms
