#pragma once
// ggml block formats read in place on the device. Layouts: q4_0 {f16 d; u8 qs[16]} 18 B / 32; q5_0 {f16 d; u8 qh[4]; u8 qs[16]} 22 B / 32;
// q8_0 {f16 d; i8 qs[32]} 34 B / 32; q4_K {f16 d, dmin; u8 scales[12]; u8 qs[128]} 144 B / 256; q6_K {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}
// 210 B / 256. Blocks are only 2-byte aligned in general (rows follow each other unpadded), so the scalar accessors read bytes and halves.
//
// elem<DT>() gives the value of one element bit for bit as the reference's Q::elem (src/backend/metal/llama_kernels.h:1014-1018, 1046-1050, 1076-1079,
// 1108-1115, 1147-1154): every product and difference is rounded on its own (__fmul_rn / __fsub_rn keep the compiler from fusing them).
// unit_dot<DT>() is the dot product of one 32-element unit of a row with the input, with the formats' offsets folded out of the per-element work as the
// reference's Q::dot does (llama_kernels.h:1036-1040, 1066-1071, 1092-1097, 1130-1138, 1176-1187).
#include <cuda_fp16.h>
#include <cstdint>

namespace dooms {
namespace dev {

enum : int { kF32 = 0, kF16 = 1, kBF16 = 2, kI32 = 3, kQ4_0 = 4, kQ5_0 = 5, kQ8_0 = 6, kQ4_K = 7, kQ6_K = 8 };

template <int DT> struct BlockInfo;
template <> struct BlockInfo<kF16> { static constexpr int elems = 32, bytes = 64; };   // 32 halves treated as one unit
template <> struct BlockInfo<kQ4_0> { static constexpr int elems = 32, bytes = 18; };
template <> struct BlockInfo<kQ5_0> { static constexpr int elems = 32, bytes = 22; };
template <> struct BlockInfo<kQ8_0> { static constexpr int elems = 32, bytes = 34; };
template <> struct BlockInfo<kQ4_K> { static constexpr int elems = 256, bytes = 144; };
template <> struct BlockInfo<kQ6_K> { static constexpr int elems = 256, bytes = 210; };

__host__ __device__ inline int64_t row_bytes_of(int dt, int64_t cols) {
    switch (dt) {
        case kF32: case kI32: return cols * 4;
        case kF16: case kBF16: return cols * 2;
        case kQ4_0: return cols / 32 * 18;
        case kQ5_0: return cols / 32 * 22;
        case kQ8_0: return cols / 32 * 34;
        case kQ4_K: return cols / 256 * 144;
        case kQ6_K: return cols / 256 * 210;
    }
    return 0;
}

__device__ __forceinline__ float ld_half(const uint8_t * p) { return __half2float(*reinterpret_cast<const __half *>(p)); }
__device__ __forceinline__ uint32_t ld_u16(const uint8_t * p) { return *reinterpret_cast<const uint16_t *>(p); }
// Four bytes at a 2-byte aligned address.
__device__ __forceinline__ uint32_t ld_u32_b2(const uint8_t * p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }

// ggml's get_scale_min_k4: the 6-bit scale and min of sub-block j of a q4_K block (q = the block's 12 scale bytes).
__device__ __forceinline__ void scale_min_k4(uint32_t j, const uint8_t * q, float & d, float & m) {
    if (j < 4) { d = float(q[j] & 63u); m = float(q[j + 4] & 63u); }
    else { d = float((q[j + 4] & 15u) | ((q[j - 4] >> 6) << 4)); m = float((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

template <int DT> __device__ __forceinline__ float elem(const uint8_t * row, uint32_t i);

template <> __device__ __forceinline__ float elem<kF32>(const uint8_t * row, uint32_t i) { return reinterpret_cast<const float *>(row)[i]; }
template <> __device__ __forceinline__ float elem<kF16>(const uint8_t * row, uint32_t i) { return ld_half(row + 2 * size_t(i)); }
template <> __device__ __forceinline__ float elem<kQ4_0>(const uint8_t * row, uint32_t i) {
    const uint8_t * b = row + size_t(i / 32) * 18;
    const uint32_t j = i % 32, q = b[2 + (j & 15)];
    return __fmul_rn(ld_half(b), float(j < 16 ? (q & 15u) : (q >> 4)) - 8.f);
}
template <> __device__ __forceinline__ float elem<kQ5_0>(const uint8_t * row, uint32_t i) {
    const uint8_t * b = row + size_t(i / 32) * 22;
    const uint32_t j = i % 32, q = b[6 + (j & 15)], low = j < 16 ? (q & 15u) : (q >> 4);
    const uint32_t qh = ld_u32_b2(b + 2);
    return __fmul_rn(ld_half(b), float(low | (((qh >> j) & 1u) << 4)) - 16.f);
}
template <> __device__ __forceinline__ float elem<kQ8_0>(const uint8_t * row, uint32_t i) {
    const uint8_t * b = row + size_t(i / 32) * 34;
    return __fmul_rn(ld_half(b), float(reinterpret_cast<const int8_t *>(b)[2 + i % 32]));
}
template <> __device__ __forceinline__ float elem<kQ4_K>(const uint8_t * row, uint32_t i) {
    const uint8_t * b = row + size_t(i / 256) * 144;
    const uint32_t j = i % 256, c = j / 32, l = j % 32;
    float sc, m;
    scale_min_k4(c, b + 4, sc, m);
    const uint32_t q = b[16 + 32 * (c / 2) + l];
    const float v = __fmul_rn(__fmul_rn(ld_half(b), sc), float((c & 1u) ? (q >> 4) : (q & 15u)));
    return __fsub_rn(v, __fmul_rn(ld_half(b + 2), m));
}
template <> __device__ __forceinline__ float elem<kQ6_K>(const uint8_t * row, uint32_t i) {
    const uint8_t * b = row + size_t(i / 256) * 210;
    const uint32_t j = i % 256, h = j / 128, k = (j % 128) / 32, l = j % 32;
    const uint32_t qlb = b[64 * h + (k & 1u) * 32 + l], low = k < 2 ? (qlb & 15u) : (qlb >> 4);
    const uint32_t hb = (b[128 + 32 * h + l] >> (2 * k)) & 3u;
    const float sc = float(reinterpret_cast<const int8_t *>(b + 192)[8 * h + l / 16 + 2 * k]);
    return __fmul_rn(__fmul_rn(ld_half(b + 208), sc), float(int(low | (hb << 4)) - 32));
}

// ---- unit dots: 32 consecutive elements of a row (unit u = elements 32u .. 32u+31) times x[32u ..], x read through the accessor X (x(k) = input k). ----

__device__ __forceinline__ float nib_lo(uint32_t w, int i) { return float((w >> (8 * i)) & 15u); }
__device__ __forceinline__ float nib_hi(uint32_t w, int i) { return float((w >> (8 * i + 4)) & 15u); }

template <int DT> struct UnitDot;

template <> struct UnitDot<kF16> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const __half2 * w = reinterpret_cast<const __half2 *>(row + size_t(u) * 64);
        float acc = 0.f;
        #pragma unroll
        for (int i = 0; i < 16; i++) { const float2 v = __half22float2(w[i]); acc += v.x * x(32 * u + 2 * i) + v.y * x(32 * u + 2 * i + 1); }
        return acc;
    }
};
template <> struct UnitDot<kQ4_0> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const uint8_t * b = row + size_t(u) * 18;
        float acc = 0.f, sx = 0.f;
        #pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t q = ld_u32_b2(b + 2 + 4 * w);
            #pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x0 = x(32 * u + 4 * w + i), x1 = x(32 * u + 16 + 4 * w + i);
                acc += nib_lo(q, i) * x0 + nib_hi(q, i) * x1;
                sx += x0 + x1;
            }
        }
        return ld_half(b) * (acc - 8.f * sx);
    }
};
template <> struct UnitDot<kQ5_0> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const uint8_t * b = row + size_t(u) * 22;
        const uint32_t qh = ld_u32_b2(b + 2);
        float acc = 0.f, sx = 0.f;
        #pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t q = ld_u32_b2(b + 6 + 4 * w);
            #pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = 4 * w + i;
                const float x0 = x(32 * u + j), x1 = x(32 * u + 16 + j);
                const float q0 = float(((q >> (8 * i)) & 15u) | (((qh >> j) & 1u) << 4)), q1 = float(((q >> (8 * i + 4)) & 15u) | (((qh >> (j + 16)) & 1u) << 4));
                acc += q0 * x0 + q1 * x1;
                sx += x0 + x1;
            }
        }
        return ld_half(b) * (acc - 16.f * sx);
    }
};
template <> struct UnitDot<kQ8_0> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const uint8_t * b = row + size_t(u) * 34;
        float acc = 0.f;
        #pragma unroll
        for (int w = 0; w < 8; w++) {
            const uint32_t q = ld_u32_b2(b + 2 + 4 * w);
            #pragma unroll
            for (int i = 0; i < 4; i++) acc += float(int8_t((q >> (8 * i)) & 0xFFu)) * x(32 * u + 4 * w + i);
        }
        return ld_half(b) * acc;
    }
};
template <> struct UnitDot<kQ4_K> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const uint8_t * b = row + size_t(u / 8) * 144;
        const uint32_t c = u % 8, shift = (c & 1u) * 4;
        float sc, m;
        scale_min_k4(c, b + 4, sc, m);
        const uint32_t * qs = reinterpret_cast<const uint32_t *>(b + 16 + 32 * (c / 2));   // 144-byte blocks in a 16-byte aligned row: 4-byte aligned
        float acc = 0.f, sx = 0.f;
        #pragma unroll
        for (int w = 0; w < 8; w++) {
            const uint32_t q = (qs[w] >> shift) & 0x0F0F0F0Fu;
            #pragma unroll
            for (int i = 0; i < 4; i++) { const float xv = x(32 * u + 4 * w + i); acc += float((q >> (8 * i)) & 0xFFu) * xv; sx += xv; }
        }
        return ld_half(b) * sc * acc - ld_half(b + 2) * m * sx;
    }
};
template <> struct UnitDot<kQ6_K> {
    template <class X> static __device__ __forceinline__ float dot(const uint8_t * row, uint32_t u, const X & x) {
        const uint8_t * b = row + size_t(u / 8) * 210;
        const uint32_t c = u % 8, h = c / 4, k = c % 4;           // elements 128h + 32k + l
        const uint8_t * ql = b + 64 * h + (k & 1u) * 32;
        const uint8_t * qh = b + 128 + 32 * h;
        const int8_t * scp = reinterpret_cast<const int8_t *>(b + 192) + 8 * h + 2 * k;
        float acc0 = 0.f, acc1 = 0.f, sx0 = 0.f, sx1 = 0.f;
        #pragma unroll
        for (int l = 0; l < 16; l += 2) {
            const uint32_t lo = ld_u16(ql + l), hi = ld_u16(qh + l), lo2 = ld_u16(ql + 16 + l), hi2 = ld_u16(qh + 16 + l);
            #pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t a = (((k < 2 ? lo : lo >> 4) >> (8 * i)) & 15u) | ((((hi >> (8 * i)) >> (2 * k)) & 3u) << 4);
                const uint32_t c2 = (((k < 2 ? lo2 : lo2 >> 4) >> (8 * i)) & 15u) | ((((hi2 >> (8 * i)) >> (2 * k)) & 3u) << 4);
                const float x0 = x(32 * u + l + i), x1 = x(32 * u + 16 + l + i);
                acc0 += float(a) * x0; sx0 += x0;
                acc1 += float(c2) * x1; sx1 += x1;
            }
        }
        return ld_half(b + 208) * (float(scp[0]) * (acc0 - 32.f * sx0) + float(scp[1]) * (acc1 - 32.f * sx1));
    }
};

}  // namespace dev
}  // namespace dooms
