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

// The file's sections in the order they are laid out: header, metadata, tensor directory, then (after padding to the alignment) the tensor data. One
// method per section; each leaves what it read in the GgufFile under construction and returns the first inconsistency it meets. What is refused, with which
// code and in which order is the reference reader's behaviour (src/format/gguf.cpp:179-317); the differential tests feed both readers the same bytes.
class GgufParser {
public:
    GgufParser(const uint8_t * data, size_t size, const GgufLimits & limits, GgufFile * out) : in_{data, size}, limits_(limits), out_(*out) {}

    Status run() {
        DOOMS_RETURN_IF_ERROR(header());
        for (uint64_t i = 0; i < kv_count_; i++) DOOMS_RETURN_IF_ERROR(metadata_entry(i));
        DOOMS_RETURN_IF_ERROR(alignment());
        out_.tensors_.reserve(static_cast<size_t>(std::min<uint64_t>(tensor_count_, in_.left())));      // a hostile count cannot reserve more than the file holds
        for (uint64_t i = 0; i < tensor_count_; i++) DOOMS_RETURN_IF_ERROR(directory_entry(i));
        return out_.tensors_.empty() ? Status() : place_data();
    }

private:
    // "GGUF", version, tensor count, metadata count.
    Status header() {
        uint8_t magic[4];
        DOOMS_RETURN_IF_ERROR(in_.bytes(magic, 4, "the magic"));
        if (magic[0] != 'G' || magic[1] != 'G' || magic[2] != 'U' || magic[3] != 'F') return data_loss("the first four bytes are not 'GGUF'");
        DOOMS_RETURN_IF_ERROR(in_.get(&out_.version_, "the format version"));
        if (out_.version_ != 2 && out_.version_ != 3) {
            // a big-endian writer's 2 or 3 reads as a multiple of 65536 here
            const bool swapped = (out_.version_ & 0xFFFFu) == 0;
            return unsupported("format version " + std::to_string(out_.version_) + "; this reader handles versions 2 and 3" +
                               (swapped ? " (the low half is zero: a file written with the other byte order?)" : ""));
        }
        DOOMS_RETURN_IF_ERROR(in_.get(&tensor_count_, "the tensor count"));
        DOOMS_RETURN_IF_ERROR(in_.get(&kv_count_, "the metadata count"));
        if (tensor_count_ > limits_.max_tensors) return over_limit("tensors", tensor_count_, limits_.max_tensors);
        if (kv_count_ > limits_.max_kv) return over_limit("metadata entries", kv_count_, limits_.max_kv);
        return Status();
    }

    Status metadata_entry(uint64_t i) {
        std::string key;
        DOOMS_RETURN_IF_ERROR(in_.string(&key, "metadata key", limits_.max_name_bytes));
        if (key.empty()) return data_loss("metadata entry #" + std::to_string(i) + ": empty key");
        GgufValue value;
        DOOMS_RETURN_IF_ERROR(read_kv_value(in_, &value, limits_, key));
        const bool fresh = out_.kv_.emplace(key, std::move(value)).second;
        return fresh ? Status() : data_loss("metadata key '" + key + "' occurs twice");
    }

    // general.alignment (u32, a power of two) positions the data section and every tensor in it; 32 when absent.
    Status alignment() {
        out_.alignment_ = 32;
        const auto it = out_.kv_.find("general.alignment");
        if (it == out_.kv_.end()) return Status();
        const GgufValue & v = it->second;
        if (v.type != GgufValueType::U32) return data_loss(std::string("general.alignment is stored as ") + gguf_value_type_name(v.type) + "; the format wants u32");
        const uint64_t a = v.u;
        out_.alignment_ = a;
        const bool power_of_two = a != 0 && (a & (a - 1)) == 0;
        if (!power_of_two || a > limits_.max_alignment) {
            return data_loss("general.alignment " + std::to_string(a) + " is not a power of two up to " + std::to_string(limits_.max_alignment));
        }
        return Status();
    }

    // name, rank, dimensions (fastest first in the file, outermost first in memory here), ggml type, offset within the data section.
    Status directory_entry(uint64_t i) {
        GgufTensorInfo t;
        DOOMS_RETURN_IF_ERROR(in_.string(&t.name, "tensor name", limits_.max_name_bytes));
        if (t.name.empty()) return data_loss("tensor #" + std::to_string(i) + ": empty name");
        if (out_.index_.find(t.name) != out_.index_.end()) return data_loss("tensor name '" + t.name + "' occurs twice");
        const std::string who = "tensor '" + t.name + "'";
        uint32_t rank = 0;
        DOOMS_RETURN_IF_ERROR(in_.get(&rank, "tensor rank"));
        if (rank > static_cast<uint32_t>(kGgufMaxDims)) return data_loss(who + ": rank " + std::to_string(rank) + " is above the format's " + std::to_string(kGgufMaxDims));
        t.rank = static_cast<int>(rank);
        int64_t elements = 1;
        for (uint32_t d = 0; d < rank; d++) {
            int64_t extent = 0;
            DOOMS_RETURN_IF_ERROR(in_.get(&extent, "tensor dimension"));
            if (extent < 1) return data_loss(who + ": extent " + std::to_string(extent) + " in dimension " + std::to_string(d) + " (must be positive)");
            if (elements > std::numeric_limits<int64_t>::max() / extent) return data_loss(who + ": more elements than 63 bits count");
            elements *= extent;
            t.shape[rank - 1 - d] = extent;
        }
        int32_t ggml_type = 0;
        DOOMS_RETURN_IF_ERROR(in_.get(&ggml_type, "tensor type"));
        if (!ggml_type_to_dtype(ggml_type, &t.dtype)) return unsupported(who + ": ggml type id " + std::to_string(ggml_type) + " is none of the types this backend holds");
        // rows are whole quantization blocks
        const int64_t per_block = dtype_block_elems(t.dtype), row = rank > 0 ? t.shape[rank - 1] : 1;
        if (row % per_block != 0) {
            return data_loss(who + ": a row of " + std::to_string(row) + " elements cannot be cut into " + dtype_name(t.dtype) + " blocks of " + std::to_string(per_block));
        }
        const uint64_t n_blocks = static_cast<uint64_t>(elements / per_block), block_bytes = static_cast<uint64_t>(dtype_block_bytes(t.dtype));
        if (n_blocks > std::numeric_limits<uint64_t>::max() / block_bytes) return data_loss(who + ": its size in bytes does not fit 64 bits");
        t.nbytes = n_blocks * block_bytes;
        DOOMS_RETURN_IF_ERROR(in_.get(&t.offset, "tensor data offset"));      // still relative to the data section; place_data() makes it absolute
        out_.index_.emplace(t.name, out_.tensors_.size());
        out_.tensors_.push_back(std::move(t));
        return Status();
    }

    // The data section starts at the next multiple of the alignment after the directory. Every tensor must start on the alignment, lie inside the file and
    // share no byte with another.
    Status place_data() {
        const uint64_t a = out_.alignment_, file_size = in_.size;
        const uint64_t section = (in_.at + a - 1) / a * a;
        if (section > file_size) return data_loss("the tensor data would start at byte " + std::to_string(section) + ", the file has " + std::to_string(file_size));
        const uint64_t room = file_size - section;
        for (const GgufTensorInfo & t : out_.tensors_) {
            if (t.offset % a != 0) return data_loss("tensor '" + t.name + "': data offset " + std::to_string(t.offset) + " is off the " + std::to_string(a) + "-byte alignment");
            if (t.offset > room || t.nbytes > room - t.offset) {
                return data_loss("tensor '" + t.name + "': bytes " + std::to_string(t.offset) + " .. " + std::to_string(t.offset) + " + " + std::to_string(t.nbytes) +
                                 " of a data section that holds " + std::to_string(room));
            }
        }
        std::vector<size_t> order(out_.tensors_.size());
        for (size_t i = 0; i < order.size(); i++) order[i] = i;
        std::sort(order.begin(), order.end(), [&](size_t x, size_t y) { return out_.tensors_[x].offset < out_.tensors_[y].offset; });
        for (size_t i = 0; i + 1 < order.size(); i++) {
            const GgufTensorInfo & lo = out_.tensors_[order[i]], & hi = out_.tensors_[order[i + 1]];
            if (lo.offset + lo.nbytes > hi.offset) return data_loss("tensor '" + lo.name + "' runs into tensor '" + hi.name + "'");
        }
        for (GgufTensorInfo & t : out_.tensors_) t.offset += section;
        return Status();
    }

    static Status over_limit(const char * what, uint64_t n, uint64_t cap) {
        return resource_exhausted("the header announces " + std::to_string(n) + " " + what + "; this reader accepts up to " + std::to_string(cap));
    }

    Reader in_;
    const GgufLimits & limits_;
    GgufFile & out_;
    uint64_t tensor_count_ = 0, kv_count_ = 0;
};

Result<GgufFile> GgufFile::parse(const uint8_t * data, size_t size, const GgufLimits & limits) {
    if (data == nullptr || size == 0) return invalid_argument("GgufFile::parse was given no bytes");
    GgufFile file;
    file.data_ = data;
    file.size_ = size;
    DOOMS_RETURN_IF_ERROR(GgufParser(data, size, limits, &file).run());
    return file;
}

Result<GgufFile> GgufFile::open(const std::string & path, const GgufLimits & limits) {
    auto mapping = MappedFile::open(path);
    if (!mapping.is_ok()) return mapping.status();
    std::shared_ptr<const MappedFile> bytes = mapping.value();
    auto file = parse(bytes->data(), bytes->size(), limits);
    if (!file.is_ok()) return Status(file.status().code(), "'" + path + "': " + file.status().message());
    file.value().mapping_ = std::move(bytes);      // the parsed view points into the mapping: they travel together
    return file;
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
