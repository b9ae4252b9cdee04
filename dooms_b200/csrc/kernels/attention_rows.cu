// Decode attention of a batched step on the tensor cores: one new position for each of many sequences ("rows"), every row over its own KV-cache slot at
// its own length. Replaces, for such a step, rope_store + attention_split + attention_combine (src/backend/metal/llama_kernels.h:521-545, 860-929), which
// the reference runs once per sequence.
//
// A step over 256 sequences of a few thousand positions reads gigabytes of keys and values and nothing twice, so the kernel has to stream; on CUDA cores
// the two dot products per key cost ~4 fused multiply-adds per byte and bound the step. Here the G query heads that share a key/value head are the rows
// of an m16n8k16 MMA (G <= 16, the rest of the 16 rows zero): S = Q K^T and O += P V as in the prefill kernel (attention_flash.cu), f16 operands, f32
// accumulators, online softmax in registers.
//
// Grid (key/value head, range, row); a range is a fixed number of cache positions, so a row has ceil(n_keys / range) blocks with work and the others
// leave at once. The 4 warps of a block take the range's tiles of TK keys in turn, each warp streaming its own tiles through its own two stages of shared
// memory (16-byte asynchronous copies, commit / wait groups: no barrier inside the loop) with its own running maximum / sum / output; the warps' results
// are merged through shared memory, a row with one range is written out directly, otherwise the range's (max, sum, output) goes to `part` and the last
// block of the (row, key/value head) to arrive (an atomic counter, reset by that block) merges the ranges.
// The block whose range holds the row's new position first rotates the new key, writes key and value into the f16 cache, and only then loads its tiles.
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kWarps = 4, kThreads = kWarps * 32;

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

struct RowsParams {
    const float * qkv;            // [row][qkv_stride]: q heads, k heads, v heads of the row's new position, not yet rotated
    __half * kc, * vc;            // this layer's caches, slot 0
    float * part;                 // [row][splits][n_head][2 + D]: (max in units of log2 e, sum, unnormalized output) of a range
    int * counters;               // [row][n_head_kv], zero between launches
    float * out;                  // [row][out_stride]
    __half * out16;               // optional [row][n_head * D]
    const double * inv_freq;
    const int32_t * slot, * pos;
    int64_t slot_elems;
    int splits, range;            // ranges per row and positions per range (a multiple of the tile)
    AttnShape s;
};

// Keys per tile: 32 for head_dim 64, 16 for 128, so that a block's 4 x 2 stages stay under 76 KB and three blocks share an SM.
template <int D> constexpr int tile_keys() { return D == 64 ? 32 : 16; }
template <int D> constexpr size_t rows_smem_bytes() {
    return size_t(16) * (D + 8) * 2 + size_t(D / 2) * 8 + 16 + size_t(kWarps) * 2 * 2 * tile_keys<D>() * (D + 8) * 2;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 3) k_attention_rows_tc(const RowsParams p) {
    constexpr int TK = tile_keys<D>();
    constexpr int LD = D + 8;                      // halves between rows in shared memory: 16 bytes of padding keep the 8 rows of an ldmatrix on different banks
    constexpr int STAGE = 2 * TK * LD;             // halves: keys, then values
    extern __shared__ __align__(16) uint8_t smem[];
    __half * Qs = reinterpret_cast<__half *>(smem);                                   // [16][LD]
    float2 * cs = reinterpret_cast<float2 *>(smem + 16 * LD * 2);                     // [D / 2] (cos, sin) of the row's position
    int * flag = reinterpret_cast<int *>(smem + 16 * LD * 2 + (D / 2) * 8);
    __half * stages = reinterpret_cast<__half *>(smem + 16 * LD * 2 + (D / 2) * 8 + 16);   // [warp][2][K | V][TK][LD]

    pdl_trigger();
    pdl_wait();
    const int kvh = blockIdx.x, split = blockIdx.y, row = blockIdx.z;
    const int slot = p.slot[row];
    if (slot < 0) return;                          // an idle row
    const int pos = p.pos[row], n_keys = pos + 1;
    const int active = (n_keys + p.range - 1) / p.range;
    if (split >= active) return;
    const int j_begin = split * p.range, j_end = min(n_keys, j_begin + p.range);
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane >> 2, t = lane & 3;
    const int G = p.s.n_head / p.s.n_head_kv;
    const float * qkv = p.qkv + int64_t(row) * p.s.qkv_stride;
    __half * kc = p.kc + int64_t(slot) * p.slot_elems + kvh * D, * vc = p.vc + int64_t(slot) * p.slot_elems + kvh * D;

    if (tid < D / 2) {
        double sd, cd;
        sincos(double(pos) * p.inv_freq[tid], &sd, &cd);
        cs[tid] = make_float2(float(cd), float(sd));
    }
    __syncthreads();
    if (pos >= j_begin && pos < j_end) {
        // the new position's own key (rotated) and value go into the cache before this block reads its tiles from there
        for (int d = tid; d < D / 2; d += kThreads) {
            const int e0 = p.s.neox ? d : 2 * d, e1 = p.s.neox ? d + D / 2 : 2 * d + 1;
            const float * x = qkv + (p.s.n_head + kvh) * D;
            const float a = __ldcg(x + e0), b = __ldcg(x + e1);
            const float2 r = cs[d];
            kc[int64_t(pos) * p.s.kv_stride + e0] = __float2half_rn(a * r.x - b * r.y);
            kc[int64_t(pos) * p.s.kv_stride + e1] = __float2half_rn(a * r.y + b * r.x);
        }
        for (int e = tid; e < D; e += kThreads) {
            vc[int64_t(pos) * p.s.kv_stride + e] = __float2half_rn(__ldcg(qkv + (p.s.n_head + p.s.n_head_kv + kvh) * D + e));
        }
        __threadfence_block();
    }
    // the group's queries, rotated and rounded to f16 (rows past the group are zero)
    for (int i = tid; i < 16 * D / 2; i += kThreads) {
        const int hq = i / (D / 2), d = i % (D / 2);
        const int e0 = p.s.neox ? d : 2 * d, e1 = p.s.neox ? d + D / 2 : 2 * d + 1;
        float r0 = 0.f, r1 = 0.f;
        if (hq < G) {
            const float * x = qkv + (kvh * G + hq) * D;
            const float a = __ldcg(x + e0), b = __ldcg(x + e1);
            const float2 r = cs[d];
            r0 = a * r.x - b * r.y;
            r1 = a * r.y + b * r.x;
        }
        Qs[hq * LD + e0] = __float2half_rn(r0);
        Qs[hq * LD + e1] = __float2half_rn(r1);
    }
    __syncthreads();      // the queries are in place; the new key and value are visible to this block's copies

    const int ntiles = (j_end - j_begin + TK - 1) / TK;          // of the block; warp w takes tiles w, w + kWarps, ...
    const int mine = warp < ntiles ? (ntiles - warp - 1) / kWarps + 1 : 0;
    __half * my = stages + warp * 2 * STAGE;
    auto load_tile = [&](int i) {
        const int j0 = j_begin + (warp + i * kWarps) * TK;
        __half * Ks = my + (i & 1) * STAGE, * Vs = Ks + TK * LD;
        #pragma unroll
        for (int it = 0; it < TK * D / 8 / 32; it++) {
            const int idx = lane + it * 32, r = idx / (D / 8), c = (idx % (D / 8)) * 8;
            if (j0 + r < j_end) {
                cp16(smem_u32(Ks + r * LD + c), kc + int64_t(j0 + r) * p.s.kv_stride + c);
                cp16(smem_u32(Vs + r * LD + c), vc + int64_t(j0 + r) * p.s.kv_stride + c);
            } else {      // past the range: zeros, so that nothing stale reaches a product
                *reinterpret_cast<uint4 *>(Ks + r * LD + c) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(Vs + r * LD + c) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (mine > 0) load_tile(0);
    cp_commit();

    uint32_t qa[D / 16][4];
    {
        const int i = lane / 8, r = 8 * (i & 1) + lane % 8;
        #pragma unroll
        for (int k = 0; k < D / 16; k++) ldsm4(smem_u32(Qs + r * LD + k * 16 + 8 * (i >> 1)), qa[k][0], qa[k][1], qa[k][2], qa[k][3]);
    }
    float o[D / 8][4];
    #pragma unroll
    for (int n = 0; n < D / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    const float scale = rsqrtf(float(D)) * 1.44269504f;      // scores in units of log2 e

    for (int i = 0; i < mine; i++) {
        if (i + 1 < mine) load_tile(i + 1);
        cp_commit();
        cp_wait<1>();
        __syncwarp();
        const __half * Ks = my + (i & 1) * STAGE, * Vs = Ks + TK * LD;
        const int j0 = j_begin + (warp + i * kWarps) * TK;
        float s[TK / 8][4];
        #pragma unroll
        for (int n = 0; n < TK / 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        {
            const int q4 = lane / 8;
            #pragma unroll
            for (int k2 = 0; k2 < D / 32; k2++) {
                #pragma unroll
                for (int n = 0; n < TK / 8; n++) {
                    uint32_t b0, b1, b2, b3;      // keys 8 n .., dims 32 k2 + 8 q4 ..: two k16 steps
                    ldsm4(smem_u32(Ks + (n * 8 + lane % 8) * LD + k2 * 32 + 8 * q4), b0, b1, b2, b3);
                    mma_f16(s[n], qa[2 * k2][0], qa[2 * k2][1], qa[2 * k2][2], qa[2 * k2][3], b0, b1);
                    mma_f16(s[n], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], qa[2 * k2 + 1][2], qa[2 * k2 + 1][3], b2, b3);
                }
            }
        }
        float mx0 = m0, mx1 = m1;
        #pragma unroll
        for (int n = 0; n < TK / 8; n++) {
            const int j = j0 + n * 8 + 2 * t;
            s[n][0] = j < j_end ? s[n][0] * scale : -CUDART_INF_F;
            s[n][1] = j + 1 < j_end ? s[n][1] * scale : -CUDART_INF_F;
            s[n][2] = j < j_end ? s[n][2] * scale : -CUDART_INF_F;
            s[n][3] = j + 1 < j_end ? s[n][3] * scale : -CUDART_INF_F;
            mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
            mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // a tile of this warp always holds at least one key of the range, so the maxima are finite from the first tile on
        const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);
        m0 = mx0; m1 = mx1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pa[TK / 16][4];
        #pragma unroll
        for (int n = 0; n < TK / 8; n++) {
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
        {
            const int q4 = lane / 8;
            #pragma unroll
            for (int kk = 0; kk < TK / 16; kk++) {
                #pragma unroll
                for (int n2 = 0; n2 < D / 16; n2++) {
                    uint32_t b0, b1, b2, b3;      // keys 16 kk + 8 (q4 & 1) .., dims 16 n2 + 8 (q4 >> 1) ..
                    ldsm4_t(smem_u32(Vs + (kk * 16 + 8 * (q4 & 1) + lane % 8) * LD + n2 * 16 + 8 * (q4 >> 1)), b0, b1, b2, b3);
                    mma_f16(o[2 * n2], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    mma_f16(o[2 * n2 + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncwarp();      // every lane is done with this stage before the next iteration's copies refill it
    }
    cp_wait<0>();
    __syncwarp();

    // the warps' results side by side in shared memory (each warp over its own stages): [warp][16 heads][2 + D]
    float * mine_out = reinterpret_cast<float *>(my);
    constexpr int RS = 2 + D;
    if (t == 0) {
        mine_out[g * RS] = m0; mine_out[g * RS + 1] = l0;
        mine_out[(g + 8) * RS] = m1; mine_out[(g + 8) * RS + 1] = l1;
    }
    #pragma unroll
    for (int n = 0; n < D / 8; n++) {
        *reinterpret_cast<float2 *>(mine_out + g * RS + 2 + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2 *>(mine_out + (g + 8) * RS + 2 + n * 8 + 2 * t) = make_float2(o[n][2], o[n][3]);
    }
    __syncthreads();
    const size_t warp_floats = size_t(2 * STAGE) / 2;      // a warp's stages, counted in floats
    const float * all = reinterpret_cast<const float *>(stages);
    float * part = p.part + (int64_t(row) * p.splits + split) * p.s.n_head * RS;
    float * out = p.out + int64_t(row) * p.s.out_stride;
    __half * out16 = p.out16 ? p.out16 + int64_t(row) * p.s.n_head * D : nullptr;
    for (int idx = tid; idx < G * D; idx += kThreads) {
        const int hq = idx / D, d = idx % D, head = kvh * G + hq;
        float M = -CUDART_INF_F;
        #pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, all[w * warp_floats + hq * RS]);
        float L = 0.f, O = 0.f;
        #pragma unroll
        for (int w = 0; w < kWarps; w++) {
            const float mw = all[w * warp_floats + hq * RS];
            const float f = mw == -CUDART_INF_F ? 0.f : exp2f(mw - M);
            L += all[w * warp_floats + hq * RS + 1] * f;
            O += all[w * warp_floats + hq * RS + 2 + d] * f;
        }
        if (active == 1) {
            const float v = O / L;
            out[head * D + d] = v;
            if (out16) out16[head * D + d] = __float2half_rn(v);
        } else {
            if (d == 0) { part[head * RS] = M; part[head * RS + 1] = L; }
            part[head * RS + 2 + d] = O;
        }
    }
    if (active == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int * counter = p.counters + row * p.s.n_head_kv + kvh;
        const int last = atomicAdd(counter, 1) == active - 1;
        if (last) *counter = 0;      // nobody adds to it again in this launch
        *flag = last;
    }
    __syncthreads();
    if (!*flag) return;
    __threadfence();
    const float * rp = p.part + int64_t(row) * p.splits * p.s.n_head * RS;
    for (int idx = tid; idx < G * D; idx += kThreads) {
        const int hq = idx / D, d = idx % D, head = kvh * G + hq;
        float M = -CUDART_INF_F;
        for (int sp = 0; sp < active; sp++) M = fmaxf(M, __ldcg(rp + (int64_t(sp) * p.s.n_head + head) * RS));
        float L = 0.f, O = 0.f;
        for (int sp = 0; sp < active; sp++) {
            const float * e = rp + (int64_t(sp) * p.s.n_head + head) * RS;
            const float f = exp2f(__ldcg(e) - M);
            L += __ldcg(e + 1) * f;
            O += __ldcg(e + 2 + d) * f;
        }
        const float v = O / L;
        out[head * D + d] = v;
        if (out16) out16[head * D + d] = __float2half_rn(v);
    }
}

template <int D>
cudaError_t launch_rows(const RowsParams & p, int n_rows, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_attention_rows_tc<D>, int(rows_smem_bytes<D>()), configured); e != cudaSuccess) return e;
    return launch_pdl(k_attention_rows_tc<D>, dim3(unsigned(p.s.n_head_kv), unsigned(p.splits), unsigned(n_rows)), dim3(kThreads), rows_smem_bytes<D>(), stream, p);
}

}  // namespace

bool attention_rows_tc_supported(const AttnShape & s) {
    const int G = s.n_head_kv > 0 ? s.n_head / s.n_head_kv : 0;
    return (s.head_dim == 64 || s.head_dim == 128) && G >= 1 && G <= 16 && s.n_head % s.n_head_kv == 0 && s.kv_stride % 8 == 0;
}

cudaError_t launch_attention_rows_tc(const float * qkv, void * kc, void * vc, float * part, const double * inv_freq, int splits, int n_ctx, const AttnShape & s,
                                     int * counters, float * out, void * out16, const BatchRows & rows, int n_rows, cudaStream_t stream) {
    if (!attention_rows_tc_supported(s) || !inv_freq || !counters || !out || !part || n_rows < 1 || splits < 1 || n_ctx < 1) return cudaErrorInvalidValue;
    const int tile = s.head_dim == 64 ? 32 : 16;
    const int range = ((n_ctx + splits - 1) / splits + tile - 1) / tile * tile;      // splits x range covers the context
    const RowsParams p{qkv, static_cast<__half *>(kc), static_cast<__half *>(vc), part, counters, out, static_cast<__half *>(out16), inv_freq, rows.slot, rows.pos,
                       rows.slot_elems, splits, range, s};
    return s.head_dim == 64 ? launch_rows<64>(p, n_rows, stream) : launch_rows<128>(p, n_rows, stream);
}

}  // namespace cuda
}  // namespace dooms
