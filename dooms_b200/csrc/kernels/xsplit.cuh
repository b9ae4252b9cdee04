#pragma once
// The input-vector format of the staged q4_0 GEMV (gemv_q4_0.cu): per 32-element block a power-of-two scale s and, for every element, the fixed-point
// value X = rint(x / s * 2^26) cut into four balanced base-128 digits (int8). Layout of xq for a vector of nb blocks: nb x 128 digit bytes
// ([digit 0..3][32 bytes], a lane t of an MMA fragment finding its 8 bytes of a digit contiguous at 8 t), then nb x 2 floats (the factors that turn the
// integer sums of the lower and the upper digit pair back into values).
#include <cstdint>

namespace dooms {
namespace dev {

// One warp, one block: lane holds element `lane` of block blk.
__device__ __forceinline__ void split_block(float v, int lane, int blk, int nb, uint8_t * xq) {
    float amax = fabsf(v);
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    uint32_t eb = (__float_as_uint(amax) >> 23) & 0xFFu;       // biased exponent of the largest magnitude
    eb = max(eb, 30u);                                         // blocks below 2^-97 are treated as that small: their digits come out zero
    eb = min(eb, 250u);
    const float inv = __uint_as_float((279u - eb) << 23);      // 2^26 / s with s = 2^(eb - 126) > amax
    int X = __float2int_rn(v * inv);
    int l[4];
    #pragma unroll
    for (int i = 0; i < 3; i++) { l[i] = ((X + 64) & 127) - 64; X = (X - l[i]) >> 7; }
    l[3] = X;
    const int pos = ((lane & 15) >> 2) * 8 + (lane >> 4) * 4 + (lane & 3);
    uint8_t * dst = xq + size_t(blk) * 128;
    #pragma unroll
    for (int i = 0; i < 4; i++) dst[i * 32 + pos] = uint8_t(int8_t(l[i]));
    if (lane == 0) {
        float * sx = reinterpret_cast<float *>(xq + size_t(nb) * 128) + blk * 2;
        sx[0] = __uint_as_float((eb - 29u) << 23);             // s * 2^-26 / 16: the weights carry a factor 16
        sx[1] = __uint_as_float((eb - 15u) << 23);             // the same for the upper digit pair (x 2^14)
    }
}

}  // namespace dev
}  // namespace dooms
