// TEST INFRASTRUCTURE - not part of the product.
//
// A C entry point around the reference's own GGUF reader, dtype tables and host argmax, compiled from the reference's sources where they lie (see
// oracle/Makefile, target `ref`). The tests use it as a differential check of the new reader: the same bytes must give the same tensors, metadata and
// error codes. Nothing of the reference is copied into this repository; this file only calls its public interface
// (src/format/gguf.h:63-100, src/core/dtype.h:15-27, src/core/argmax.h:15, src/core/status.h:13-23).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <sstream>
#include <string>

#include "core/argmax.h"
#include "core/dtype.h"
#include "core/status.h"
#include "format/gguf.h"

using namespace dooms;

namespace {
// The C ABI's numbering of the status codes (include/dooms/dooms_c.h:23-32, src/api/c_api.cpp:36-47).
int c_code(Code c) {
    switch (c) {
        case Code::Ok: return 0;
        case Code::InvalidArgument: case Code::OutOfRange: return 1;
        case Code::NotFound: return 2;
        case Code::DataLoss: return 3;
        case Code::Unsupported: return 4;
        case Code::ResourceExhausted: return 5;
        case Code::IoError: return 6;
        case Code::Internal: return 7;
    }
    return 7;
}
void json_string(std::ostringstream & o, const std::string & s) {
    o << '"';
    for (unsigned char ch : s) {
        if (ch == '"' || ch == '\\') o << '\\' << ch;
        else if (ch < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", ch); o << b; }
        else o << ch;
    }
    o << '"';
}
void json_value(std::ostringstream & o, const GgufValue & v) {
    switch (v.type) {
        case GgufValueType::String: json_string(o, v.s); break;
        case GgufValueType::F32: case GgufValueType::F64: { char b[64]; std::snprintf(b, sizeof b, "%.17g", v.f); o << b; break; }
        case GgufValueType::I8: case GgufValueType::I16: case GgufValueType::I32: case GgufValueType::I64: o << v.i; break;
        case GgufValueType::Array: {
            o << '[';
            for (size_t i = 0; i < v.items.size(); i++) { if (i) o << ','; json_value(o, v.items[i]); }
            o << ']';
            break;
        }
        default: o << v.u; break;
    }
}
std::string dump(const GgufFile & f) {
    std::ostringstream o;
    o << "{\"version\":" << f.version() << ",\"alignment\":" << f.alignment() << ",\"kv\":{";
    bool first = true;
    for (const auto & kv : f.metadata()) {
        if (!first) o << ',';
        first = false;
        json_string(o, kv.first);
        o << ":{\"type\":\"" << gguf_value_type_name(kv.second.type) << "\",\"value\":";
        json_value(o, kv.second);
        o << '}';
    }
    o << "},\"tensors\":[";
    first = true;
    for (const GgufTensorInfo & t : f.tensors()) {
        if (!first) o << ',';
        first = false;
        o << "{\"name\":";
        json_string(o, t.name);
        o << ",\"dtype\":\"" << dtype_name(t.dtype) << "\",\"shape\":[";
        for (int i = 0; i < t.shape.rank(); i++) { if (i) o << ','; o << t.shape.dim(i); }
        o << "],\"offset\":" << t.offset << ",\"nbytes\":" << t.nbytes << '}';
    }
    o << "]}";
    return o.str();
}
int finish(const Result<GgufFile> & r, char * out, size_t cap) {
    const std::string text = r.is_ok() ? dump(r.value()) : r.status().message();
    if (out && cap) { std::strncpy(out, text.c_str(), cap - 1); out[cap - 1] = 0; }
    return r.is_ok() ? 0 : c_code(r.status().code());
}
}  // namespace

extern "C" {
// Parses `size` bytes; on success writes a JSON description into out, else the error message. Returns the status code (C ABI numbering).
__attribute__((visibility("default"))) int ref_gguf_parse(const uint8_t * data, size_t size, char * out, size_t cap) { return finish(GgufFile::parse(data, size), out, cap); }
__attribute__((visibility("default"))) int ref_gguf_open(const char * path, char * out, size_t cap) { return finish(GgufFile::open(path), out, cap); }
__attribute__((visibility("default"))) int64_t ref_argmax_f32(const float * v, size_t n) { return static_cast<int64_t>(argmax_f32(v, n)); }
// dtype by the reference's name ("q4_0", "q6_k", ...): block elements and bytes; 0 for an unknown name.
__attribute__((visibility("default"))) int64_t ref_block_elems(const char * name) { auto t = dtype_from_name(name); return t.is_ok() ? dtype_block_elems(t.value()) : 0; }
__attribute__((visibility("default"))) int64_t ref_block_bytes(const char * name) { auto t = dtype_from_name(name); return t.is_ok() ? dtype_block_bytes(t.value()) : 0; }
}
