// Causal flash attention for a prefill chunk with grouped-query heads: out[t][h] = softmax(q[t][h] . K[0 .. p0 + t]^T / sqrt(d)) V, queries at absolute
// positions p0 + t over the f16 KV cache. One block of 8 warps per (128 queries, head); keys and values stream through shared memory 128 positions at a time
// (cp.async, double buffered); S = Q K^T and O += P V run on the tensor cores (mma.sync m16n8k16, f16 operands, f32 accumulators) with the running
// max / sum of the online softmax in registers. Q, K, V and P are rounded to f16, scores and the output accumulate in f32, as in the reference's
// attention_prefill<64 / 128> (src/backend/metal/llama_kernels.h:640-769), which this replaces. head_dim 64 or 128; other sizes take the CUDA-core kernel.
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kQ = 128, kK = 128, kWarps = 8;      // 16 queries per warp; tiles of 128 keys measured 6 % faster than 64 (half as many barriers per key)

__device__ __forceinline__ void cp16(uint32_t dst, const void * src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) { const __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<const uint32_t *>(&h); }

template <int D>
__global__ void __launch_bounds__(kWarps * 32) k_attention_flash(const float * qkv, const __half * kc, const __half * vc, float * out, __half * out16,
                                                                const DevState * st, int M, AttnShape p) {
    constexpr int LD = D + 8;                       // row stride in halves: 16 bytes of padding keep ldmatrix rows on different banks
    extern __shared__ __align__(16) uint8_t smem[];
    __half * Qs = reinterpret_cast<__half *>(smem);                    // [kQ][LD]
    __half * KVs = Qs + kQ * LD;                                       // [2 stages][K | V][kK][LD]
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    // the last query tiles see the most keys: they go first, so that the short ones fill the tail
    const int h = blockIdx.x, t0 = int(gridDim.y - 1 - blockIdx.y) * kQ, p0 = st->pos;
    const int kvh = h / (p.n_head / p.n_head_kv);
    const int last_key = p0 + min(t0 + kQ, M) - 1;
    const int ntiles = last_key / kK + 1;
    const __half * kbase = kc + kvh * D, * vbase = vc + kvh * D;

    auto load_tile = [&](int tile, int stage) {
        __half * Ks = KVs + stage * 2 * kK * LD, * Vs = Ks + kK * LD;
        for (int i = threadIdx.x; i < kK * D / 8; i += kWarps * 32) {
            const int r = i / (D / 8), c = (i % (D / 8)) * 8, j = tile * kK + r;
            if (j <= last_key) {
                cp16(smem_u32(Ks + r * LD + c), kbase + int64_t(j) * p.kv_stride + c);
                cp16(smem_u32(Vs + r * LD + c), vbase + int64_t(j) * p.kv_stride + c);
            } else {      // past the last visible key: zeros, so that no stale cache bytes reach a product
                *reinterpret_cast<uint4 *>(Ks + r * LD + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(Vs + r * LD + c) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_tile(0, 0);
    cp_commit();
    // the query tile, rounded to f16 (rows past the chunk are zero)
    for (int i = threadIdx.x; i < kQ * D / 4; i += kWarps * 32) {
        const int r = i / (D / 4), c = (i % (D / 4)) * 4, tq = t0 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tq < M) v = *reinterpret_cast<const float4 *>(qkv + int64_t(tq) * p.qkv_stride + h * D + c);
        *reinterpret_cast<uint2 *>(Qs + r * LD + c) = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
    }
    __syncthreads();
    uint32_t qa[D / 16][4];      // this warp's 16 queries as A fragments
    {
        const int i = lane / 8, row = warp * 16 + 8 * (i & 1) + lane % 8;
        #pragma unroll
        for (int k = 0; k < D / 16; k++) ldsm4(smem_u32(Qs + row * LD + k * 16 + 8 * (i >> 1)), qa[k][0], qa[k][1], qa[k][2], qa[k][3]);
    }
    float o[D / 8][4];
    #pragma unroll
    for (int n = 0; n < D / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    const float scale = rsqrtf(float(D)) * 1.44269504f;      // scores in units of log2 e
    const int qpos0 = p0 + t0 + warp * 16 + g, qpos1 = qpos0 + 8;

    for (int tile = 0; tile < ntiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < ntiles) load_tile(tile + 1, stage ^ 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const __half * Ks = KVs + stage * 2 * kK * LD, * Vs = Ks + kK * LD;
        const int j0 = tile * kK;
        if (j0 <= p0 + t0 + warp * 16 + 15) {      // warp-uniform: some key of this tile is visible to some query of the warp
            float s[kK / 8][4];
            #pragma unroll
            for (int n = 0; n < kK / 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
            {
                const int i = lane / 8;
                #pragma unroll
                for (int k2 = 0; k2 < D / 32; k2++) {
                    #pragma unroll
                    for (int n = 0; n < kK / 8; n++) {
                        uint32_t b0, b1, b2, b3;      // keys n*8.., d (k2*32 + 8 i ..): two k16 steps
                        ldsm4(smem_u32(Ks + (n * 8 + lane % 8) * LD + k2 * 32 + 8 * i), b0, b1, b2, b3);
                        mma_f16(s[n], qa[2 * k2][0], qa[2 * k2][1], qa[2 * k2][2], qa[2 * k2][3], b0, b1);
                        mma_f16(s[n], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], qa[2 * k2 + 1][2], qa[2 * k2 + 1][3], b2, b3);
                    }
                }
            }
            // scale, causal mask, running max
            float mx0 = m0, mx1 = m1;
            #pragma unroll
            for (int n = 0; n < kK / 8; n++) {
                const int j = j0 + n * 8 + 2 * t;
                s[n][0] = j <= qpos0 ? s[n][0] * scale : -CUDART_INF_F;
                s[n][1] = j + 1 <= qpos0 ? s[n][1] * scale : -CUDART_INF_F;
                s[n][2] = j <= qpos1 ? s[n][2] * scale : -CUDART_INF_F;
                s[n][3] = j + 1 <= qpos1 ? s[n][3] * scale : -CUDART_INF_F;
                mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // key 0 is visible to every query, so after the first tile the maxima are finite; a row whose keys are all masked in a later tile keeps its maximum
            const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);
            m0 = mx0; m1 = mx1;
            float sum0 = 0.f, sum1 = 0.f;
            uint32_t pa[kK / 16][4];      // P as A fragments of the second product
            #pragma unroll
            for (int n = 0; n < kK / 8; n++) {
                const float e0 = exp2f(s[n][0] - mx0), e1 = exp2f(s[n][1] - mx0), e2 = exp2f(s[n][2] - mx1), e3 = exp2f(s[n][3] - mx1);
                sum0 += e0 + e1;
                sum1 += e2 + e3;
                pa[n / 2][(n & 1) * 2] = pack_h2(e0, e1);
                pa[n / 2][(n & 1) * 2 + 1] = pack_h2(e2, e3);
            }
            sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
            sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
            l0 = l0 * c0 + sum0;
            l1 = l1 * c1 + sum1;
            #pragma unroll
            for (int n = 0; n < D / 8; n++) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
            // O += P V
            {
                const int i = lane / 8;
                #pragma unroll
                for (int kk = 0; kk < kK / 16; kk++) {
                    #pragma unroll
                    for (int n2 = 0; n2 < D / 16; n2++) {
                        uint32_t b0, b1, b2, b3;      // keys kk*16 + 8 (i & 1) .., dims n2*16 + 8 (i >> 1) ..
                        ldsm4_t(smem_u32(Vs + (kk * 16 + 8 * (i & 1) + lane % 8) * LD + n2 * 16 + 8 * (i >> 1)), b0, b1, b2, b3);
                        mma_f16(o[2 * n2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                        mma_f16(o[2 * n2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                    }
                }
            }
        }
        __syncthreads();      // every warp is done with this stage before the next iteration refills it
    }
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
    const int ta = t0 + warp * 16 + g, tb = ta + 8;
    #pragma unroll
    for (int n = 0; n < D / 8; n++) {
        const int col = h * D + n * 8 + 2 * t;
        if (ta < M) {
            const float x = o[n][0] * inv0, y = o[n][1] * inv0;
            if (out) *reinterpret_cast<float2 *>(out + int64_t(ta) * p.out_stride + col) = make_float2(x, y);
            if (out16) *reinterpret_cast<uint32_t *>(out16 + int64_t(ta) * p.out_stride + col) = pack_h2(x, y);
        }
        if (tb < M) {
            const float x = o[n][2] * inv1, y = o[n][3] * inv1;
            if (out) *reinterpret_cast<float2 *>(out + int64_t(tb) * p.out_stride + col) = make_float2(x, y);
            if (out16) *reinterpret_cast<uint32_t *>(out16 + int64_t(tb) * p.out_stride + col) = pack_h2(x, y);
        }
    }
}

template <int D>
cudaError_t launch_d(const float * qkv, const void * kc, const void * vc, float * out, void * out16, const DevState * st, int M, const AttnShape & s,
                     cudaStream_t stream) {
    const size_t smem = size_t(kQ + 4 * kK) * (D + 8) * 2;
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_attention_flash<D>, int(smem), configured); e != cudaSuccess) return e;
    const dim3 grid(s.n_head, (M + kQ - 1) / kQ);
    k_attention_flash<D><<<grid, kWarps * 32, smem, stream>>>(qkv, static_cast<const __half *>(kc), static_cast<const __half *>(vc), out,
                                                              static_cast<__half *>(out16), st, M, s);
    return cudaGetLastError();
}

}  // namespace

bool attention_flash_supported(const AttnShape & s) {
    return (s.head_dim == 64 || s.head_dim == 128) && s.kv_stride % 8 == 0 && s.qkv_stride % 4 == 0 && s.out_stride % 2 == 0;
}

cudaError_t launch_attention_flash(const float * qkv, const void * kc, const void * vc, float * out, void * out16, const DevState * st, int M, const AttnShape & s,
                                   cudaStream_t stream) {
    if (!attention_flash_supported(s)) return cudaErrorInvalidValue;
    return s.head_dim == 64 ? launch_d<64>(qkv, kc, vc, out, out16, st, M, s, stream) : launch_d<128>(qkv, kc, vc, out, out16, st, M, s, stream);
}

}  // namespace cuda
}  // namespace dooms
