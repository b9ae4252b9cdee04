#pragma once
// Element types and ggml block tables (the reference's src/core/dtype.h:15-27 and src/core/dtype.cpp:19-52). The enum values equal dooms_dtype in
// include/dooms_cuda.h.
#include <cstdint>
#include <string>

#include "status.h"

namespace dooms {

enum class DType : int32_t { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, Q4_0 = 4, Q5_0 = 5, Q8_0 = 6, Q4_K = 7, Q6_K = 8 };

struct DTypeInfo { const char * name; int64_t block_bytes; int64_t block_elems; };

// q4_0 {f16 d; u8 qs[16]}, q5_0 {f16 d; u8 qh[4]; u8 qs[16]}, q8_0 {f16 d; i8 qs[32]}, q4_K {f16 d, dmin; u8 scales[12]; u8 qs[128]},
// q6_K {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}.
inline const DTypeInfo * dtype_info(int32_t t) {
    static const DTypeInfo table[] = {{"f32", 4, 1}, {"f16", 2, 1}, {"bf16", 2, 1}, {"i32", 4, 1}, {"q4_0", 18, 32},
                                      {"q5_0", 22, 32}, {"q8_0", 34, 32}, {"q4_k", 144, 256}, {"q6_k", 210, 256}};
    return (t >= 0 && t <= 8) ? &table[t] : nullptr;
}
inline bool dtype_valid(int32_t t) { return dtype_info(t) != nullptr; }
inline int64_t dtype_block_elems(DType t) { return dtype_info(static_cast<int32_t>(t))->block_elems; }
inline int64_t dtype_block_bytes(DType t) { return dtype_info(static_cast<int32_t>(t))->block_bytes; }
inline bool dtype_is_quantized(DType t) { return dtype_block_elems(t) > 1; }
inline const char * dtype_name(DType t) { return dtype_info(static_cast<int32_t>(t))->name; }
// Bytes of n elements: InvalidArgument when n is not a whole number of blocks.
inline Result<uint64_t> dtype_bytes(DType t, int64_t n) {
    const DTypeInfo & i = *dtype_info(static_cast<int32_t>(t));
    if (n < 0 || n % i.block_elems != 0) {
        return invalid_argument(std::to_string(n) + " elements are not a whole number of " + i.name + " blocks of " + std::to_string(i.block_elems));
    }
    return static_cast<uint64_t>(n / i.block_elems) * static_cast<uint64_t>(i.block_bytes);
}

}  // namespace dooms
