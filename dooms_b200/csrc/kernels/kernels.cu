// The decoder's general kernels: every weight format, every shape the decoder accepts. The specialised fast paths (staged decode GEMV, tensor-core
// prefill GEMM, flash attention) live in their own files and are chosen by the host when a shape qualifies; these are what runs otherwise.
#include "kernels.h"

#include <cuda_fp16.h>
#include <math_constants.h>

#include "quant.cuh"
#include "launch.cuh"
#include "xsplit.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Calls f.template operator()<DT>() for the matrix type dt; false for a type the kernels do not take.
template <class F>
bool dispatch_mat(int dt, F && f) {
    switch (dt) {
        case kF16: f.template operator()<kF16>(); return true;
        case kQ4_0: f.template operator()<kQ4_0>(); return true;
        case kQ5_0: f.template operator()<kQ5_0>(); return true;
        case kQ8_0: f.template operator()<kQ8_0>(); return true;
        case kQ4_K: f.template operator()<kQ4_K>(); return true;
        case kQ6_K: f.template operator()<kQ6_K>(); return true;
    }
    return false;
}

struct GlobalX {
    const float * x;
    __device__ __forceinline__ float operator()(uint32_t k) const { return __ldg(x + k); }
};

// ---------------------------------------------------------------- state

__global__ void k_set_state(DevState * st, int32_t pos, int32_t tok_in, int32_t tok_out) {
    pdl_trigger();
    pdl_wait();
    st->pos = pos;
    st->tok_in = tok_in;
    st->tok_out = tok_out;
}

// ---------------------------------------------------------------- embedding lookup

template <int DT>
__global__ void k_embed(const uint8_t * table, const int32_t * ids, const int32_t * index, float * x, int E) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= E) return;
    const int64_t tok = ids[(index ? *index : 0) + row];
    x[int64_t(row) * E + i] = elem<DT>(table + tok * row_bytes_of(DT, E), uint32_t(i));
}

// ---------------------------------------------------------------- RMS norm

// One block of 1024 threads per row. Every thread loads its elements (and their gains) up front, so the loads are in flight together instead of one round
// trip to L2 per loop iteration; rows wider than kNormMaxPerThread x 1024 take the looping path. Element i belongs to thread (i / 32) % 32 * 32 + i % 32
// of pass i / 1024: a warp holds whole 32-element blocks, which is what the split for the staged q4_0 GEMV needs.
// xq (optional, one row only, E a multiple of 32): the normalized row also split for that kernel (xsplit.cuh).
// Many rows (a prefill chunk, a batched step) take blocks of 256 threads with up to 16 elements each: eight blocks share an SM and cover each other's
// round trips, where 1024-thread blocks ran in waves of two per SM (22 us for 2048 rows of 4096 floats; the bytes alone are 8 us).
template <int kNormThreads, int kNormMaxPerThread>
__global__ void __launch_bounds__(kNormThreads) k_rms_norm(const float * x, const float * gamma, float * out, __half * out16, uint8_t * xq, int E, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[kNormThreads / 32];
    const float * xr = x + int64_t(blockIdx.x) * E;
    const int64_t obase = int64_t(blockIdx.x) * E;
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    float ss = 0.f;
    if (E <= kNormThreads * kNormMaxPerThread) {
        float v[kNormMaxPerThread], g[kNormMaxPerThread];
        #pragma unroll
        for (int k = 0; k < kNormMaxPerThread; k++) {
            const int i = k * kNormThreads + threadIdx.x;
            v[k] = i < E ? xr[i] : 0.f;
            g[k] = i < E ? gamma[i] : 0.f;
        }
        #pragma unroll
        for (int k = 0; k < kNormMaxPerThread; k++) ss += v[k] * v[k];
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float total = 0.f;
        #pragma unroll
        for (int w = 0; w < kNormThreads / 32; w++) total += red[w];
        const float inv = rsqrtf(total / float(E) + eps);
        #pragma unroll
        for (int k = 0; k < kNormMaxPerThread; k++) {
            const int i = k * kNormThreads + threadIdx.x;
            if (i - lane >= E) break;      // warp-uniform: the whole 32-element block is past the row
            const float r = v[k] * inv * g[k];
            if (i < E) {
                if (out) out[obase + i] = r;
                if (out16) out16[obase + i] = __float2half_rn(r);
            }
            if (xq) split_block(r, lane, i / 32, E / 32, xq);
        }
        return;
    }
    for (int i = threadIdx.x; i < E; i += kNormThreads) { const float t = xr[i]; ss += t * t; }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < kNormThreads / 32; w++) total += red[w];
    const float inv = rsqrtf(total / float(E) + eps);
    for (int i0 = warp * 32; i0 < E; i0 += kNormThreads) {
        const int i = i0 + lane;
        const float r = i < E ? xr[i] * inv * gamma[i] : 0.f;
        if (i < E) {
            if (out) out[obase + i] = r;
            if (out16) out16[obase + i] = __float2half_rn(r);
        }
        if (xq) split_block(r, lane, i / 32, E / 32, xq);
    }
}

// ---------------------------------------------------------------- one-token projections (general path: one warp per row, 32-element units over the lanes)

constexpr int kMvWarps = 4;

template <int DT>
__global__ void __launch_bounds__(kMvWarps * 32) k_matvec(const uint8_t * W, const float * x, float * y, const float * bias, int64_t rows, int cols, uint32_t flags) {
    if (!(flags & kFlagLateDependents)) pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int64_t r = int64_t(blockIdx.x) * kMvWarps + warp;
    if (r >= rows) return;
    const uint8_t * row = W + r * row_bytes_of(DT, cols);
    const GlobalX X{x};
    float acc = 0.f;
    for (uint32_t u = lane; u < uint32_t(cols) / 32; u += 32) acc += UnitDot<DT>::dot(row, u, X);
    acc = warp_sum(acc);
    if (lane == 0) {
        if (flags & kFlagBias) acc += bias[r];
        y[r] = (flags & kFlagAccumulate) ? accumulate_base(y[r], flags) + acc : acc;
    }
}

template <int DT>
__global__ void __launch_bounds__(kMvWarps * 32) k_gate_up(const uint8_t * Wg, const uint8_t * Wu, const float * x, float * h, int64_t rows, int cols) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int64_t r = int64_t(blockIdx.x) * kMvWarps + warp;
    if (r >= rows) return;
    const int64_t RB = row_bytes_of(DT, cols);
    const GlobalX X{x};
    float g = 0.f, u = 0.f;
    for (uint32_t i = lane; i < uint32_t(cols) / 32; i += 32) { g += UnitDot<DT>::dot(Wg + r * RB, i, X); u += UnitDot<DT>::dot(Wu + r * RB, i, X); }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) h[r] = g / (1.f + expf(-g)) * u;
}

// ---------------------------------------------------------------- multi-token projections on CUDA cores (any shape; f32 operands)

constexpr int kTileM = 64, kTileN = 64, kTileK = 32;

template <int DT, bool GATE>
__global__ void __launch_bounds__(256) k_matmul_tile(const uint8_t * W, const uint8_t * W2, const float * X, int64_t x_stride, float * Y, int64_t y_stride,
                                                     const float * bias, int M, int64_t N, int K, uint32_t flags) {
    __shared__ float Xs[kTileK][kTileM + 1];
    __shared__ float Ws[kTileK][kTileN + 1];
    __shared__ float W2s[GATE ? kTileK : 1][kTileN + 1];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // tx: weight rows (n), ty: tokens (m)
    const int64_t n0 = int64_t(blockIdx.x) * kTileN;
    const int m0 = blockIdx.y * kTileM;
    const int64_t RB = row_bytes_of(DT, K);
    float acc[4][4] = {}, acc2[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kTileK) {
        for (int idx = threadIdx.x; idx < kTileM * kTileK; idx += 256) {
            const int m = idx / kTileK, k = idx % kTileK;
            Xs[k][m] = (m0 + m < M && k0 + k < K) ? X[int64_t(m0 + m) * x_stride + k0 + k] : 0.f;
        }
        for (int idx = threadIdx.x; idx < kTileN * kTileK; idx += 256) {
            const int n = idx / kTileK, k = idx % kTileK;
            const bool ok = n0 + n < N && k0 + k < K;
            Ws[k][n] = ok ? elem<DT>(W + (n0 + n) * RB, uint32_t(k0 + k)) : 0.f;
            if (GATE) W2s[k][n] = ok ? elem<DT>(W2 + (n0 + n) * RB, uint32_t(k0 + k)) : 0.f;
        }
        __syncthreads();
        #pragma unroll 8
        for (int k = 0; k < kTileK; k++) {
            float a[4], b[4], b2[4];
            #pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = Xs[k][ty * 4 + i]; b[i] = Ws[k][tx * 4 + i]; if (GATE) b2[i] = W2s[k][tx * 4 + i]; }
            #pragma unroll
            for (int i = 0; i < 4; i++) {
                #pragma unroll
                for (int j = 0; j < 4; j++) { acc[i][j] += a[i] * b[j]; if (GATE) acc2[i][j] += a[i] * b2[j]; }
            }
        }
        __syncthreads();
    }
    #pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATE) v = v / (1.f + expf(-v)) * acc2[i][j];
            else if (flags & kFlagBias) v += bias[n];
            float * y = Y + int64_t(m) * y_stride + n;
            *y = (flags & kFlagAccumulate) ? *y + v : v;
        }
    }
}

// ---------------------------------------------------------------- dequantization to f32

template <int DT>
__global__ void k_dequantize(const uint8_t * blocks, float * out, int64_t rows, int cols) {
    const int64_t RB = row_bytes_of(DT, cols);
    const int64_t total = rows * cols;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / cols;
        out[i] = elem<DT>(blocks + r * RB, uint32_t(i - r * cols));
    }
}

__global__ void k_add(float * x, const float * y, int64_t n) {
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) x[i] += y[i];
}

// ---------------------------------------------------------------- rotary embedding + cache write

// cs[i] = (cos, sin)(st->pos * inv_freq[i]) for the head_dim / 2 rotary pairs, in double precision, rounded to f32: what every head of every layer of one
// decode step rotates by, computed once per step instead of in every attention launch.
__global__ void k_rope_table(const DevState * st, const double * inv_freq, float2 * cs, int pairs, unsigned * zero) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0 && zero) { zero[0] = 0u; zero[32] = 0u; }      // the fused step's barrier words
    if (i >= pairs) return;
    double sd, cd;
    sincos(double(st->pos) * inv_freq[i], &sd, &cd);
    cs[i] = make_float2(float(cd), float(sd));
}

// grid (M), head_dim / 2 x (up to 4) threads: a thread owns rotary pair i and every fourth slot; slots are query heads (rotated in place), key heads
// (rotated into the cache), value heads (copied). The angle pos * inv_freq[i] and its sine / cosine are computed once per thread in double precision, so that
// positions in the thousands keep their low bits (rotate_pair, llama_kernels.h:513-518).
__global__ void k_rope_store(float * qkv, __half * kc, __half * vc, const DevState * st, const double * inv_freq, AttnShape p) {
    pdl_trigger();
    pdl_wait();
    const int hd = p.head_dim, t = blockIdx.x, i = threadIdx.x % (hd / 2), lanes = blockDim.x / (hd / 2);
    const int pos = st->pos + t;
    const int e0 = p.neox ? i : 2 * i, e1 = p.neox ? i + hd / 2 : 2 * i + 1;
    float * row = qkv + int64_t(t) * p.qkv_stride;
    double sd, cd;
    sincos(double(pos) * inv_freq[i], &sd, &cd);
    const float c = float(cd), s = float(sd);
    for (int slot = threadIdx.x / (hd / 2); slot < p.n_head + 2 * p.n_head_kv; slot += lanes) {
        if (slot < p.n_head + p.n_head_kv) {
            float * x = row + slot * hd;
            const float a = x[e0], b = x[e1];
            const float r0 = a * c - b * s, r1 = a * s + b * c;
            if (slot < p.n_head) { x[e0] = r0; x[e1] = r1; }
            else {
                __half * dst = kc + int64_t(pos) * p.kv_stride + (slot - p.n_head) * hd;
                dst[e0] = __float2half_rn(r0);
                dst[e1] = __float2half_rn(r1);
            }
        } else {
            const int kvh = slot - p.n_head - p.n_head_kv;
            const float * x = row + (p.n_head + p.n_head_kv + kvh) * hd;
            __half * dst = vc + int64_t(pos) * p.kv_stride + kvh * hd;
            dst[e0] = __float2half_rn(x[e0]);
            dst[e1] = __float2half_rn(x[e1]);
        }
    }
}

// ---------------------------------------------------------------- attention on CUDA cores (any head_dim that is a power of two in [4, 256])

constexpr int kAttnWarps = 4;
constexpr int kMaxDimsPerLane = 8;   // head_dim <= 256

// One block per (head, split, query row): the block's warps share the split's key range, each with its own running softmax, merged in shared memory.
// part entry: (max, sum, values[head_dim]) unnormalised; direct: splits == 1, the normalised result goes straight to out.
__global__ void __launch_bounds__(kAttnWarps * 32) k_attention(const float * q, const __half * kc, const __half * vc, float * out, __half * out16, float * part,
                                                               const DevState * st, int n_keys_fixed, int splits, int direct, AttnShape p) {
    pdl_trigger();
    pdl_wait();
    __shared__ float qs[256];
    __shared__ float wm[kAttnWarps], wl[kAttnWarps];
    __shared__ float wo[kAttnWarps][256];
    const int h = blockIdx.x, sidx = blockIdx.y, t = blockIdx.z, hd = p.head_dim;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int n_keys = n_keys_fixed > 0 ? n_keys_fixed : st->pos + t + 1;
    const int chunk = (n_keys + splits - 1) / splits;
    const int j_begin = sidx * chunk, j_end = min(n_keys, j_begin + chunk);
    const int kvh = h / (p.n_head / p.n_head_kv);
    const float scale = rsqrtf(float(hd));
    for (int i = threadIdx.x; i < hd; i += blockDim.x) qs[i] = q[int64_t(t) * p.qkv_stride + h * hd + i] * scale;
    __syncthreads();
    float m_run = -CUDART_INF_F, l_run = 0.f;
    float o[kMaxDimsPerLane];
    #pragma unroll
    for (int d = 0; d < kMaxDimsPerLane; d++) o[d] = 0.f;
    for (int j0 = j_begin + warp * 32; j0 < j_end; j0 += kAttnWarps * 32) {
        const int j = j0 + lane;
        float sc = -CUDART_INF_F;
        if (j < j_end) {
            const __half2 * k2 = reinterpret_cast<const __half2 *>(kc + int64_t(j) * p.kv_stride + kvh * hd);
            float a = 0.f;
            for (int d = 0; d < hd / 2; d++) { const float2 kv = __half22float2(k2[d]); a += qs[2 * d] * kv.x + qs[2 * d + 1] * kv.y; }
            sc = a;
        }
        const float m_new = fmaxf(m_run, warp_max(sc));
        const float corr = expf(m_run - m_new);          // m_run = -inf on the first group: exp(-inf) = 0 and l, o are 0 anyway
        const float pj = j < j_end ? expf(sc - m_new) : 0.f;
        l_run = l_run * corr + warp_sum(pj);
        m_run = m_new;
        #pragma unroll
        for (int d = 0; d < kMaxDimsPerLane; d++) o[d] *= corr;
        const int cnt = min(32, j_end - j0);
        for (int jj = 0; jj < cnt; jj++) {
            const float pb = __shfl_sync(0xffffffffu, pj, jj);
            const __half * v = vc + int64_t(j0 + jj) * p.kv_stride + kvh * hd;
            #pragma unroll
            for (int d = 0; d < kMaxDimsPerLane; d++) { const int e = lane + 32 * d; if (e < hd) o[d] += pb * __half2float(v[e]); }
        }
    }
    if (lane == 0) { wm[warp] = m_run; wl[warp] = l_run; }
    #pragma unroll
    for (int d = 0; d < kMaxDimsPerLane; d++) { const int e = lane + 32 * d; if (e < hd) wo[warp][e] = o[d]; }
    __syncthreads();
    float mx = wm[0];
    for (int w = 1; w < kAttnWarps; w++) mx = fmaxf(mx, wm[w]);
    float total = 0.f;
    float wgt[kAttnWarps];
    for (int w = 0; w < kAttnWarps; w++) { wgt[w] = wl[w] > 0.f ? expf(wm[w] - mx) : 0.f; total += wl[w] * wgt[w]; }
    float * dst = direct ? out + int64_t(t) * p.out_stride + h * hd : part + ((int64_t(t) * p.n_head + h) * splits + sidx) * (2 + hd) + 2;
    for (int e = threadIdx.x; e < hd; e += blockDim.x) {
        float a = 0.f;
        for (int w = 0; w < kAttnWarps; w++) a += wo[w][e] * wgt[w];
        dst[e] = direct ? a / total : a;
        if (direct && out16) out16[int64_t(t) * p.out_stride + h * hd + e] = __float2half_rn(a / total);
    }
    if (!direct && threadIdx.x == 0) { dst[-2] = mx; dst[-1] = total; }
}

// out[t][h] = merge of the splits' partial results (attention_combine, llama_kernels.h:914-929). grid (n_head, M), head_dim threads.
__global__ void k_attention_combine(const float * part, float * out, uint8_t * xq, int splits, AttnShape p) {
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x, t = blockIdx.y, hd = p.head_dim, i = threadIdx.x;
    const float * base = part + (int64_t(t) * p.n_head + h) * splits * (2 + hd);
    float mx = -CUDART_INF_F;
    for (int s = 0; s < splits; s++) if (base[s * (2 + hd) + 1] > 0.f) mx = fmaxf(mx, base[s * (2 + hd)]);
    float total = 0.f, acc = 0.f;
    for (int s = 0; s < splits; s++) {
        const float * ps = base + s * (2 + hd);
        if (!(ps[1] > 0.f)) continue;   // an empty split
        const float w = expf(ps[0] - mx);
        total += ps[1] * w;
        acc += ps[2 + i] * w;
    }
    const float r = acc / total;
    out[int64_t(t) * p.out_stride + h * hd + i] = r;
    // the row as the staged q4_0 GEMV wants it (head_dim a multiple of 32: a warp holds whole 32-element blocks)
    if (xq) split_block(r, i % 32, (h * hd + i) / 32, p.n_head * hd / 32, xq);
}

// ---------------------------------------------------------------- argmax

struct Best { float v; int32_t i; };   // i < 0: nothing yet
__device__ __forceinline__ bool better(float av, int32_t ai, float bv, int32_t bi) {
    // a beats b: a is a number and (b is empty, or a is larger, or equal with the lower index)
    if (ai < 0 || av != av) return false;
    return bi < 0 || av > bv || (av == bv && ai < bi);
}
__device__ __forceinline__ Best warp_best(Best b) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int32_t oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        if (better(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
    }
    return b;
}
__device__ __forceinline__ Best block_best(Best b) {
    __shared__ float sv[32];
    __shared__ int32_t si[32];
    b = warp_best(b);
    if (threadIdx.x % 32 == 0) { sv[threadIdx.x / 32] = b.v; si[threadIdx.x / 32] = b.i; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = (blockDim.x + 31) / 32;
        Best c{threadIdx.x < nw ? sv[threadIdx.x] : 0.f, threadIdx.x < nw ? si[threadIdx.x] : -1};
        b = warp_best(c);
    }
    return b;   // valid in warp 0
}

constexpr int kArgmaxThreads = 256, kArgmaxPerBlock = 4096;

__global__ void __launch_bounds__(kArgmaxThreads) k_argmax_part(const float * logits, int64_t n, Best * part) {
    pdl_trigger();
    pdl_wait();
    const int64_t begin = int64_t(blockIdx.x) * kArgmaxPerBlock, end = min(n, begin + kArgmaxPerBlock);
    Best b{0.f, -1};
    for (int64_t i = begin + threadIdx.x; i < end; i += kArgmaxThreads) {
        const float v = logits[i];
        if (better(v, int32_t(i), b.v, b.i)) { b.v = v; b.i = int32_t(i); }
    }
    b = block_best(b);
    if (threadIdx.x == 0) part[blockIdx.x] = b;
}

__global__ void __launch_bounds__(kArgmaxThreads) k_argmax_final(const Best * part, int nparts, int32_t * tokens, int32_t * host_tokens, DevState * st,
                                                                 int32_t * plain_out, int advance) {
    pdl_trigger();
    pdl_wait();
    Best b{0.f, -1};
    for (int i = threadIdx.x; i < nparts; i += kArgmaxThreads) if (better(part[i].v, part[i].i, b.v, b.i)) b = part[i];
    b = block_best(b);
    if (threadIdx.x == 0) {
        const int32_t tok = b.i < 0 ? 0 : b.i;   // all NaN: 0
        if (plain_out) { *plain_out = tok; return; }
        const int32_t o = st->tok_out;
        tokens[o] = tok;
        if (host_tokens) host_tokens[o] = tok;
        if (advance) { st->pos += 1; st->tok_in += 1; st->tok_out = o + 1; }
    }
}

// Tensor parallelism, two stages: every rank reduces its own slice of the vocabulary to one (value, global index) pair (k_argmax_part, then this kernel
// with `offset` = the slice's first row); the pairs of all ranks are gathered (8 bytes per rank instead of the logits) and k_argmax_pairs picks among them
// by the same rule, lowest global index on ties, so that every rank writes the same token.
__global__ void __launch_bounds__(kArgmaxThreads) k_argmax_pair(const Best * part, int nparts, int32_t offset, Best * pair) {
    Best b{0.f, -1};
    for (int i = threadIdx.x; i < nparts; i += kArgmaxThreads) if (better(part[i].v, part[i].i, b.v, b.i)) b = part[i];
    b = block_best(b);
    if (threadIdx.x == 0) *pair = Best{b.v, b.i < 0 ? -1 : b.i + offset};
}
__global__ void k_argmax_pairs(const Best * pairs, int n, int32_t * tokens, int32_t * host_tokens, DevState * st, int advance) {
    Best b{0.f, -1};
    for (int r = 0; r < n; r++) if (better(pairs[r].v, pairs[r].i, b.v, b.i)) b = pairs[r];
    const int32_t tok = b.i < 0 ? 0 : b.i;
    const int32_t o = st->tok_out;
    tokens[o] = tok;
    if (host_tokens) host_tokens[o] = tok;
    if (advance) { st->pos += 1; st->tok_in += 1; st->tok_out = o + 1; }
}

// The same reduction for every row of a batched decode step: grid (blocks per row, rows), then one block per row.
__global__ void __launch_bounds__(kArgmaxThreads) k_argmax_rows_part(const float * logits, int64_t n, int64_t stride, const int32_t * slot, Best * part) {
    const int row = blockIdx.y;
    if (slot[row] < 0) return;
    const float * v0 = logits + int64_t(row) * stride;
    const int64_t begin = int64_t(blockIdx.x) * kArgmaxPerBlock, end = min(n, begin + kArgmaxPerBlock);
    Best b{0.f, -1};
    for (int64_t i = begin + threadIdx.x; i < end; i += kArgmaxThreads) {
        const float v = v0[i];
        if (better(v, int32_t(i), b.v, b.i)) { b.v = v; b.i = int32_t(i); }
    }
    b = block_best(b);
    if (threadIdx.x == 0) part[int64_t(row) * gridDim.x + blockIdx.x] = b;
}

__global__ void __launch_bounds__(kArgmaxThreads) k_argmax_rows_final(const Best * part, int nparts, const int32_t * slot, int32_t * pos, int32_t * tok, int32_t * out,
                                                                      int32_t * step) {
    const int row = blockIdx.x, rows = gridDim.x;
    const int32_t at = *step;      // read by every block before the last block to finish bumps it: the bump happens in a kernel of its own, below
    if (slot[row] < 0) {
        if (threadIdx.x == 0) out[int64_t(at) * rows + row] = -1;
        return;
    }
    const Best * mine = part + int64_t(row) * nparts;
    Best b{0.f, -1};
    for (int i = threadIdx.x; i < nparts; i += kArgmaxThreads) if (better(mine[i].v, mine[i].i, b.v, b.i)) b = mine[i];
    b = block_best(b);
    if (threadIdx.x == 0) {
        const int32_t t = b.i < 0 ? 0 : b.i;
        tok[row] = t;
        pos[row] += 1;
        out[int64_t(at) * rows + row] = t;
    }
}

__global__ void k_bump(int32_t * counter) { *counter += 1; }

}  // namespace

// ---------------------------------------------------------------- launchers

cudaError_t launch_set_state(DevState * st, int32_t pos, int32_t tok_in, int32_t tok_out, cudaStream_t stream) {
    return launch_pdl(k_set_state, dim3(1), dim3(1), 0, stream, st, pos, tok_in, tok_out);
}

cudaError_t launch_embed(int dt, const void * table, const int32_t * ids, const int32_t * index, float * x, int rows, int E, cudaStream_t stream) {
    const dim3 grid((E + 255) / 256, rows);
    cudaError_t e = cudaSuccess;
    const bool ok = dispatch_mat(dt, [&]<int DT>() { e = launch_pdl(k_embed<DT>, grid, dim3(256), 0, stream, static_cast<const uint8_t *>(table), ids, index, x, E); });
    return ok ? e : cudaErrorInvalidValue;
}

cudaError_t launch_rms_norm(const float * x, const float * gamma, float * out, void * out16, void * xq, int rows, int E, float eps, cudaStream_t stream) {
    if (xq && (rows != 1 || E % 32 != 0)) return cudaErrorInvalidValue;
    if (rows >= 64 && E <= 256 * 16) {
        return launch_pdl(k_rms_norm<256, 16>, dim3(rows), dim3(256), 0, stream, x, gamma, out, static_cast<__half *>(out16), static_cast<uint8_t *>(xq), E, eps);
    }
    return launch_pdl(k_rms_norm<1024, 8>, dim3(rows), dim3(1024), 0, stream, x, gamma, out, static_cast<__half *>(out16), static_cast<uint8_t *>(xq), E, eps);
}

cudaError_t launch_matvec(int dt, const void * W, const float * x, float * y, const float * bias, int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream) {
    if (gemv_blocks_supported(dt, W, x, rows, cols)) return launch_gemv_blocks(dt, W, nullptr, x, nullptr, 0.f, y, bias, rows, cols, flags, stream);
    const unsigned grid = unsigned((rows + kMvWarps - 1) / kMvWarps);
    cudaError_t e = cudaSuccess;
    const bool ok = dispatch_mat(dt, [&]<int DT>() {
        e = launch_pdl(k_matvec<DT>, dim3(grid), dim3(kMvWarps * 32), 0, stream, static_cast<const uint8_t *>(W), x, y, bias, rows, int(cols), flags);
    });
    return ok ? e : cudaErrorInvalidValue;
}

cudaError_t launch_gate_up(int dt, const void * Wg, const void * Wu, const float * x, float * h, int64_t rows, int64_t cols, cudaStream_t stream) {
    if (gemv_blocks_supported(dt, Wg, x, rows, cols) && gemv_blocks_supported(dt, Wu, x, rows, cols)) {
        return launch_gemv_blocks(dt, Wg, Wu, x, nullptr, 0.f, h, nullptr, rows, cols, 0u, stream);
    }
    const unsigned grid = unsigned((rows + kMvWarps - 1) / kMvWarps);
    cudaError_t e = cudaSuccess;
    const bool ok = dispatch_mat(dt, [&]<int DT>() {
        e = launch_pdl(k_gate_up<DT>, dim3(grid), dim3(kMvWarps * 32), 0, stream, static_cast<const uint8_t *>(Wg), static_cast<const uint8_t *>(Wu), x, h, rows, int(cols));
    });
    return ok ? e : cudaErrorInvalidValue;
}

cudaError_t launch_matmul_tile(int dt, const void * W, const void * W2, const float * X, int64_t x_stride, float * Y, int64_t y_stride, const float * bias,
                               int M, int64_t N, int64_t K, uint32_t flags, cudaStream_t stream) {
    const dim3 grid(unsigned((N + kTileN - 1) / kTileN), unsigned((M + kTileM - 1) / kTileM));
    const uint8_t * w = static_cast<const uint8_t *>(W), * w2 = static_cast<const uint8_t *>(W2);
    const bool ok = dispatch_mat(dt, [&]<int DT>() {
        if (W2) k_matmul_tile<DT, true><<<grid, 256, 0, stream>>>(w, w2, X, x_stride, Y, y_stride, bias, M, N, int(K), flags);
        else k_matmul_tile<DT, false><<<grid, 256, 0, stream>>>(w, w2, X, x_stride, Y, y_stride, bias, M, N, int(K), flags);
    });
    return ok ? cudaGetLastError() : cudaErrorInvalidValue;
}

cudaError_t launch_dequantize(int dt, const void * blocks, int64_t rows, int64_t cols, float * out, cudaStream_t stream) {
    const int64_t total = rows * cols;
    const unsigned grid = unsigned(std::min<int64_t>((total + 255) / 256, sm_count() * 16));
    const bool ok = dispatch_mat(dt, [&]<int DT>() { k_dequantize<DT><<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(blocks), out, rows, int(cols)); });
    return ok ? cudaGetLastError() : cudaErrorInvalidValue;
}

__global__ void __launch_bounds__(256) k_add_shares(float * x, const float * shares, int k_splits, int64_t n, int64_t split_stride) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        float v = x[i];
        for (int s = 0; s < k_splits; s++) v += __ldcg(shares + s * split_stride + i);
        x[i] = v;
    }
}
cudaError_t launch_add_shares(float * x, const float * shares, int k_splits, int64_t n, int64_t split_stride, cudaStream_t stream) {
    if (!x || !shares || k_splits < 1 || n < 1) return cudaErrorInvalidValue;
    return launch_pdl(k_add_shares, dim3(unsigned(std::min<int64_t>((n + 255) / 256, sm_count() * 8))), dim3(256), 0, stream, x, shares, k_splits, n, split_stride);
}

cudaError_t launch_add(float * x, const float * y, int64_t n, cudaStream_t stream) {
    k_add<<<unsigned(std::min<int64_t>((n + 255) / 256, sm_count() * 8)), 256, 0, stream>>>(x, y, n);
    return cudaGetLastError();
}

cudaError_t launch_rope_table(const DevState * st, const double * inv_freq, void * cs, int head_dim, cudaStream_t stream, unsigned * zero) {
    const int pairs = head_dim / 2;
    k_rope_table<<<(pairs + 127) / 128, 128, 0, stream>>>(st, inv_freq, static_cast<float2 *>(cs), pairs, zero);
    return cudaGetLastError();
}

cudaError_t launch_rope_store(float * qkv, void * kc, void * vc, const DevState * st, const double * inv_freq, int M, const AttnShape & s, cudaStream_t stream) {
    const int pairs = s.head_dim / 2;
    const int lanes = std::max(1, std::min(4, 256 / pairs));
    return launch_pdl(k_rope_store, dim3(M), dim3(pairs * lanes), 0, stream, qkv, static_cast<__half *>(kc), static_cast<__half *>(vc), st, inv_freq, s);
}

int attention_splits(int n_head, int n_ctx) {
    // enough blocks to fill the SMs a few times over, ranges of at least 64 positions once the context is long
    const int want = std::max(1, (sm_count() * 2 + n_head - 1) / n_head);
    return std::max(1, std::min(want, (n_ctx + 63) / 64));
}

cudaError_t launch_attention_decode(const float * q, const void * kc, const void * vc, float * out, float * part, void * xq, const DevState * st,
                                    int n_keys_fixed, int splits, const AttnShape & s, cudaStream_t stream) {
    if (xq && (splits == 1 || s.head_dim % 32 != 0)) return cudaErrorInvalidValue;
    const dim3 grid(s.n_head, splits, 1);
    cudaError_t e = launch_pdl(k_attention, grid, dim3(kAttnWarps * 32), 0, stream, q, static_cast<const __half *>(kc), static_cast<const __half *>(vc), out,
                               static_cast<__half *>(nullptr), part, st, n_keys_fixed, splits, splits == 1 ? 1 : 0, s);
    if (e != cudaSuccess || splits == 1) return e;
    return launch_pdl(k_attention_combine, dim3(s.n_head, 1), dim3(s.head_dim), 0, stream, static_cast<const float *>(part), out, static_cast<uint8_t *>(xq), splits, s);
}

cudaError_t launch_attention_combine(const float * part, float * out, void * xq, int splits, const AttnShape & s, cudaStream_t stream) {
    if (xq && s.head_dim % 32 != 0) return cudaErrorInvalidValue;
    return launch_pdl(k_attention_combine, dim3(s.n_head, 1), dim3(s.head_dim), 0, stream, part, out, static_cast<uint8_t *>(xq), splits, s);
}

cudaError_t launch_attention_prefill(const float * qkv, const void * kc, const void * vc, float * out, void * out16, const DevState * st, int M,
                                     const AttnShape & s, cudaStream_t stream) {
    const dim3 grid(s.n_head, 1, M);
    return launch_pdl(k_attention, grid, dim3(kAttnWarps * 32), 0, stream, qkv, static_cast<const __half *>(kc), static_cast<const __half *>(vc), out,
                      static_cast<__half *>(out16), static_cast<float *>(nullptr), st, 0, 1, 1, s);
}

int argmax_blocks(int64_t n) { return int((n + kArgmaxPerBlock - 1) / kArgmaxPerBlock); }

cudaError_t launch_argmax(const float * logits, int64_t n, int32_t * tokens, int32_t * host_tokens, DevState * st, void * part, int advance, cudaStream_t stream) {
    const int blocks = argmax_blocks(n);
    const cudaError_t e = launch_pdl(k_argmax_part, dim3(blocks), dim3(kArgmaxThreads), 0, stream, logits, n, static_cast<Best *>(part));
    if (e != cudaSuccess) return e;
    return launch_pdl(k_argmax_final, dim3(1), dim3(kArgmaxThreads), 0, stream, static_cast<const Best *>(part), blocks, tokens, host_tokens, st,
                      static_cast<int32_t *>(nullptr), advance);
}

cudaError_t launch_argmax_rows(const float * logits, int64_t n, int64_t stride, const BatchRows & rows, int n_rows, int32_t * out, int32_t * step, void * part,
                               cudaStream_t stream) {
    const int blocks = argmax_blocks(n);
    k_argmax_rows_part<<<dim3(blocks, n_rows), kArgmaxThreads, 0, stream>>>(logits, n, stride, rows.slot, static_cast<Best *>(part));
    k_argmax_rows_final<<<n_rows, kArgmaxThreads, 0, stream>>>(static_cast<const Best *>(part), blocks, rows.slot, rows.pos, rows.tok, out, step);
    k_bump<<<1, 1, 0, stream>>>(step);
    return cudaGetLastError();
}

cudaError_t launch_argmax_local_pair(const float * logits, int64_t n, int32_t offset, void * pair, void * part, cudaStream_t stream) {
    const int blocks = argmax_blocks(std::max<int64_t>(n, 1));
    if (n > 0) k_argmax_part<<<blocks, kArgmaxThreads, 0, stream>>>(logits, n, static_cast<Best *>(part));
    k_argmax_pair<<<1, kArgmaxThreads, 0, stream>>>(static_cast<const Best *>(part), n > 0 ? blocks : 0, offset, static_cast<Best *>(pair));
    return cudaGetLastError();
}

cudaError_t launch_argmax_pairs(const void * pairs, int n, int32_t * tokens, int32_t * host_tokens, DevState * st, int advance, cudaStream_t stream) {
    k_argmax_pairs<<<1, 1, 0, stream>>>(static_cast<const Best *>(pairs), n, tokens, host_tokens, st, advance);
    return cudaGetLastError();
}

cudaError_t launch_argmax_plain(const float * logits, int64_t n, int32_t * out, void * part, cudaStream_t stream) {
    const int blocks = argmax_blocks(n);
    const cudaError_t e = launch_pdl(k_argmax_part, dim3(blocks), dim3(kArgmaxThreads), 0, stream, logits, n, static_cast<Best *>(part));
    if (e != cudaSuccess) return e;
    return launch_pdl(k_argmax_final, dim3(1), dim3(kArgmaxThreads), 0, stream, static_cast<const Best *>(part), blocks, static_cast<int32_t *>(nullptr),
                      static_cast<int32_t *>(nullptr), static_cast<DevState *>(nullptr), out, 0);
}

}  // namespace cuda
}  // namespace dooms
