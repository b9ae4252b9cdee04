#pragma once
// Status / Result: how every fallible host operation reports errors; no exception crosses a module boundary. Same codes and helper names as the reference's
// src/core/status.h:13-72, so that code written against either reads the same. The numeric values of Code are internal; the C ABI maps them (c_api.cpp).
#include <optional>
#include <string>
#include <utility>

namespace dooms {

enum class Code { Ok = 0, InvalidArgument, OutOfRange, NotFound, Unsupported, DataLoss, ResourceExhausted, IoError, Internal };

inline const char * code_name(Code c) {
    switch (c) {
        case Code::Ok: return "Ok";
        case Code::InvalidArgument: return "InvalidArgument";
        case Code::OutOfRange: return "OutOfRange";
        case Code::NotFound: return "NotFound";
        case Code::Unsupported: return "Unsupported";
        case Code::DataLoss: return "DataLoss";
        case Code::ResourceExhausted: return "ResourceExhausted";
        case Code::IoError: return "IoError";
        case Code::Internal: return "Internal";
    }
    return "Unknown";
}

class Status {
public:
    Status() = default;
    Status(Code code, std::string message) : code_(code), message_(code == Code::Ok ? std::string() : std::move(message)) {}
    bool is_ok() const { return code_ == Code::Ok; }
    Code code() const { return code_; }
    const std::string & message() const { return message_; }
    std::string to_string() const { return is_ok() ? "Ok" : std::string(code_name(code_)) + ": " + message_; }
private:
    Code code_ = Code::Ok;
    std::string message_;
};

inline Status invalid_argument(std::string m) { return Status(Code::InvalidArgument, std::move(m)); }
inline Status out_of_range(std::string m) { return Status(Code::OutOfRange, std::move(m)); }
inline Status not_found(std::string m) { return Status(Code::NotFound, std::move(m)); }
inline Status unsupported(std::string m) { return Status(Code::Unsupported, std::move(m)); }
inline Status data_loss(std::string m) { return Status(Code::DataLoss, std::move(m)); }
inline Status resource_exhausted(std::string m) { return Status(Code::ResourceExhausted, std::move(m)); }
inline Status io_error(std::string m) { return Status(Code::IoError, std::move(m)); }
inline Status internal_error(std::string m) { return Status(Code::Internal, std::move(m)); }

// A value or a non-Ok Status. value() on an error is a programming error (checked by the callers with is_ok()).
template <class T>
class Result {
public:
    Result(T value) : value_(std::move(value)) {}
    Result(Status status) : status_(std::move(status)) {}
    bool is_ok() const { return value_.has_value(); }
    const Status & status() const { return status_; }
    T & value() & { return *value_; }
    const T & value() const & { return *value_; }
    T && value() && { return std::move(*value_); }
private:
    std::optional<T> value_;
    Status status_;
};

}  // namespace dooms

#define DOOMS_RETURN_IF_ERROR(expr)                   \
    do {                                              \
        ::dooms::Status _dooms_st = (expr);           \
        if (!_dooms_st.is_ok()) return _dooms_st;     \
    } while (0)
