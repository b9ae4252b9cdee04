#pragma once
// The body of the grouped-query decode attention kernel (attention_decode.cu holds the description and the launchers), as a device function so that the
// kernel of its own and the fused decode step (decode_step.cu) run the same code.
#include <cuda_fp16.h>
#include <math_constants.h>

#include "kernels.h"
#include "ptx.cuh"
#include "xsplit.cuh"

namespace dooms {
namespace cuda {
namespace attn_decode {

using namespace dooms::dev;

constexpr int kThreads = 256;
constexpr int kTileKeys = 64;
constexpr int kStages = 4;      // two pairs of tiles: the block's 8 warps work on one pair while the next is on its way

struct AttnDecodeParams {
    const float * qkv;        // the new token's row: query heads, then key heads, then value heads
    __half * kc;
    __half * vc;
    float * part;             // [n_head][splits][2 + head_dim]
    const DevState * st;
    const double * inv_freq;  // head_dim / 2 rotary frequencies; nullptr: q is used as it is and nothing is written to the cache
    int n_keys_fixed, splits;
    AttnShape s;
    // With counters (one zeroed int per key/value head, left zeroed): the block that finishes a key/value head's last range merges the ranges of its
    // query heads itself (attention_combine, llama_kernels.h:914-929) into out, and into xq the row split for the staged q4_0 GEMV when xq is given.
    int * counters;
    float * out;
    uint8_t * xq;
    const float2 * rope_cs;   // optional: (cos, sin) of the head_dim / 2 rotary angles at st->pos, computed once per decode step
    // One step over several sequences (grid z = row of the step): row r reads its position from b_pos[r] and works on the cache of slot b_slot[r] (a
    // negative slot: the row is idle and its blocks leave at once). qkv, part, counters, out and out16 are then indexed by row.
    const int32_t * b_slot;
    const int32_t * b_pos;
    int b_rows;
    int64_t slot_elems;       // f16 elements between the caches of consecutive slots
    int64_t part_row_floats;  // floats of `part` per row
    __half * out16;           // optional: the merged rows as f16 as well ([row][n_head * head_dim]), the tensor-core GEMM's operand
    int l2_hint;              // single-row decode: before waiting for the projection in front of it, a block asks for its range of the caches to be brought to L2
};

__device__ __forceinline__ void cp16(uint32_t dst, const void * src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8, f32) += A(16x16, f16, row) B(16x8, f16, col) with rows 8..15 of A zero: only a0 (row g, k 2t..) and a2 (row g, k 2t+8..) are given, and of
// the result only c0, c1 (row g, columns 2t, 2t+1) mean anything.
__device__ __forceinline__ void mma_f16_top(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
// x as the sum of two f16 numbers (the second one the rounding error of the first): products with an f16 operand, accumulated in f32 by the tensor
// core, then carry x to about 22 bits instead of 11.
__device__ __forceinline__ void split_h2(float x, float y, uint32_t & hi, uint32_t & lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - back.x, y - back.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// The work of one block of kThreads threads: key/value head `kvh`, range `split` of `n_splits`, row `row` of a batched step (0 otherwise), with `smem`
// (attention_decode_smem_bytes<D, GP>(), 128-byte aligned) as its staging memory. WHOLE = true: the calling block has exactly kThreads threads and its
// barriers are __syncthreads(); false: the first kThreads threads of a larger block run this while the others do not, so the barriers are the named
// barrier 1 over kThreads threads. Inputs written earlier in the same launch (the fused decode step calls this right after a grid-wide barrier) are read
// with loads that bypass L1.
// D: head_dim (64 or 128). GP: query heads per key/value head, rounded up to 1, 2, 4 or 8.
template <bool WHOLE>
__device__ __forceinline__ void attn_bar() {
    if constexpr (WHOLE) __syncthreads();
    else asm volatile("bar.sync 1, 256;" ::: "memory");
}
// The scores and the weighted sums run on the tensor cores (mma.sync m16n8k16): the G <= 8 query heads of the key/value head are the first rows of the
// A operand, the cached keys / values the B operand straight from the staged f16 rows (ldmatrix). The query and the probabilities go in as pairs of f16
// numbers (value and rounding error, two MMAs), so the products are as exact as the f32 arithmetic they replace: one position per call keeps the
// reference's token-by-token tolerance (tests/unit/test_metal_llama_decoder.cpp:335). The 8 warps take 16 keys each of a pair of 64-key tiles with their
// own running maximum / sum / output and are merged through shared memory at the end of the range.
template <int D, int GP>
constexpr size_t attention_decode_smem_bytes() { return size_t(16) * (D + 8) * 2 + size_t(kStages) * kTileKeys * 2 * (D * 2 + 16); }

template <int D, int GP, bool WHOLE>
__device__ __forceinline__ void attention_decode_body(const AttnDecodeParams & pp, const int kvh, const int split, const int n_splits, const int row, uint8_t * smem) {
    constexpr int LD = D + 8;                           // halves between staged rows: 16 bytes of padding keep the 8 rows of an ldmatrix on different banks
    constexpr int KP = LD * 2, VP = LD * 2;             // the same in bytes
    constexpr int STAGE = kTileKeys * (KP + VP);
    constexpr int OUT_IT = (GP * D / 2 + kThreads - 1) / kThreads;   // (head, dim pair) outputs per thread
    constexpr int MERGE_IT = (GP * D + kThreads - 1) / kThreads;     // single outputs per thread in the merge
    constexpr int RS = 2 + D;                                          // floats per head in the warps' results
    static_assert(GP <= 8 && size_t(8) * 8 * RS * 4 <= size_t(kStages) * STAGE, "the warps' results are laid over the stages");
    __half * Qh = reinterpret_cast<__half *>(smem);                    // [8 heads: values][LD], then [8 heads: rounding errors][LD]
    uint8_t * stages = smem + 16 * LD * 2;
    const uint32_t stages_u = smem_u32(stages);

    // the row's view of the arguments
    AttnDecodeParams p = pp;
    int row_pos = 0;
    if (pp.b_slot) {
        const int slot = pp.b_slot[row];
        if (slot < 0) return;
        row_pos = pp.b_pos[row];
        p.kc = pp.kc + int64_t(slot) * pp.slot_elems;
        p.vc = pp.vc + int64_t(slot) * pp.slot_elems;
        p.qkv = pp.qkv + int64_t(row) * pp.s.qkv_stride;
        p.part = pp.part + int64_t(row) * pp.part_row_floats;
        p.counters = pp.counters + row * pp.s.n_head_kv;
        p.out = pp.out + int64_t(row) * pp.s.out_stride;
        if (pp.out16) p.out16 = pp.out16 + int64_t(row) * pp.s.n_head * D;
    }
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane >> 2, t = lane & 3;
    const int G = p.s.n_head / p.s.n_head_kv;
    const bool fuse = p.inv_freq != nullptr;
    const int pos = !fuse ? 0 : pp.b_slot ? row_pos : p.st->pos;
    const int n_keys = p.n_keys_fixed > 0 ? p.n_keys_fixed : pos + 1;
    // ranges of whole tiles, the same for every head: at least one tile per range, so short contexts leave the later ranges empty
    const int tiles_total = (n_keys + kTileKeys - 1) / kTileKeys;
    const int tiles_per = (tiles_total + p.splits - 1) / p.splits;
    const int j_begin = min(n_keys, split * tiles_per * kTileKeys), j_end = min(n_keys, j_begin + tiles_per * kTileKeys);
    const int ntiles = (j_end - j_begin + kTileKeys - 1) / kTileKeys;

    auto fetch = [&](int tile) {
        const int j0 = j_begin + tile * kTileKeys, cnt = min(kTileKeys, j_end - j0);
        const uint32_t base = stages_u + uint32_t(tile % kStages) * STAGE;
        constexpr int PIECES = D * 2 / 16;      // 16-byte pieces per row
        for (int i = tid; i < kTileKeys * PIECES; i += kThreads) {
            const int r = i / PIECES, c = i % PIECES;
            if (r < cnt) {
                cp16(base + r * KP + c * 16, p.kc + int64_t(j0 + r) * p.s.kv_stride + kvh * D + c * 8);
                cp16(base + kTileKeys * KP + r * VP + c * 16, p.vc + int64_t(j0 + r) * p.s.kv_stride + kvh * D + c * 8);
            } else {      // past the range: zeros (a probability of 0 times old bytes that happen to read as NaN would not be 0)
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + r * KP + c * 16), "r"(0u) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(base + kTileKeys * KP + r * VP + c * 16), "r"(0u) : "memory");
            }
        }
    };
    #pragma unroll
    for (int i = 0; i < kStages; i++) {
        if (i < ntiles) fetch(i);
        cp_commit();
    }

    // the group's queries, rotated (when asked), each as an f16 value and the f16 rounding error of that value
    for (int i = tid; i < 8 * D / 2; i += kThreads) {
        const int hq = i / (D / 2), d = i % (D / 2);
        const int e0 = p.s.neox ? d : 2 * d, e1 = p.s.neox ? d + D / 2 : 2 * d + 1;
        float r0 = 0.f, r1 = 0.f;
        if (hq < G) {
            const float * x = p.qkv + (kvh * G + hq) * D;
            r0 = __ldcg(x + e0);
            r1 = __ldcg(x + e1);
            if (fuse) {
                float c, s;
                if (p.rope_cs) { const float2 cs = p.rope_cs[d]; c = cs.x; s = cs.y; }
                else { double sd, cd; sincos(double(pos) * p.inv_freq[d], &sd, &cd); c = float(cd); s = float(sd); }
                const float a = r0, b = r1;
                r0 = a * c - b * s;
                r1 = a * s + b * c;
            }
        }
        const __half h0 = __float2half_rn(r0), h1 = __float2half_rn(r1);
        Qh[hq * LD + e0] = h0;
        Qh[hq * LD + e1] = h1;
        Qh[(8 + hq) * LD + e0] = __float2half_rn(r0 - __half2float(h0));
        Qh[(8 + hq) * LD + e1] = __float2half_rn(r1 - __half2float(h1));
    }

    // this warp's share of every pair of tiles: 16 keys of the pair's first (warps 0-3) or second (warps 4-7) tile
    const int pair_tile = warp >> 2, wk = (warp & 3) * 16;
    const float scale = rsqrtf(float(D));
    uint32_t qh[D / 16][2], ql[D / 16][2];      // A fragments of the queries: rows g of the values and of the rounding errors
    float o[D / 8][4];
    #pragma unroll
    for (int n = 0; n < D / 8; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m_w = -CUDART_INF_F, l_w = 0.f;        // of head g, over this warp's keys (the four lanes of a quad hold the same)

    for (int t2 = 0; t2 < ntiles; t2 += 2) {
        cp_wait<kStages - 2>();                   // this pair has landed (this thread's pieces) ...
        attn_bar<WHOLE>();                        // ... and everybody's; the queries are in place
        bool patched = false;
        #pragma unroll
        for (int k = 0; k < 2; k++) {
            const int tile = t2 + k, j0 = j_begin + tile * kTileKeys, cnt = min(kTileKeys, j_end - j0);
            if (tile < ntiles && fuse && pos >= j0 && pos < j0 + cnt) {
                // the new token's own key and value: into the cache and over the (stale) row that was just copied from it
                uint8_t * ks = stages + (tile % kStages) * STAGE, * vs = ks + kTileKeys * KP;
                const int r = pos - j0;
                if (tid < D / 2) {
                    const int d = tid;
                    const int e0 = p.s.neox ? d : 2 * d, e1 = p.s.neox ? d + D / 2 : 2 * d + 1;
                    const float * x = p.qkv + (p.s.n_head + kvh) * D;
                    float c, s;
                    if (p.rope_cs) { const float2 cs = p.rope_cs[d]; c = cs.x; s = cs.y; }
                    else { double sd, cd; sincos(double(pos) * p.inv_freq[d], &sd, &cd); c = float(cd); s = float(sd); }
                    const float a = __ldcg(x + e0), b = __ldcg(x + e1);
                    const __half h0 = __float2half_rn(a * c - b * s), h1 = __float2half_rn(a * s + b * c);
                    __half * dst = p.kc + int64_t(pos) * p.s.kv_stride + kvh * D;
                    __half * srow = reinterpret_cast<__half *>(ks + r * KP);
                    dst[e0] = h0; dst[e1] = h1;
                    srow[e0] = h0; srow[e1] = h1;
                } else if (tid >= 64 && tid < 64 + D) {
                    const int e = tid - 64;
                    const __half hv = __float2half_rn(__ldcg(p.qkv + (p.s.n_head + p.s.n_head_kv + kvh) * D + e));
                    p.vc[int64_t(pos) * p.s.kv_stride + kvh * D + e] = hv;
                    reinterpret_cast<__half *>(vs + r * VP)[e] = hv;
                }
                patched = true;
            }
        }
        if (patched) attn_bar<WHOLE>();           // (the same for every thread of the block)
        if (t2 == 0) {
            const int mi = lane >> 3, r = lane & 7;
            #pragma unroll
            for (int k2 = 0; k2 < D / 32; k2++) {
                ldsm4(smem_u32(Qh + r * LD + k2 * 32 + mi * 8), qh[2 * k2][0], qh[2 * k2][1], qh[2 * k2 + 1][0], qh[2 * k2 + 1][1]);
                ldsm4(smem_u32(Qh + (8 + r) * LD + k2 * 32 + mi * 8), ql[2 * k2][0], ql[2 * k2][1], ql[2 * k2 + 1][0], ql[2 * k2 + 1][1]);
            }
        }
        const int tile = t2 + pair_tile;
        const int cnt = tile < ntiles ? min(kTileKeys, j_end - (j_begin + tile * kTileKeys)) : 0;
        if (wk < cnt) {
            const __half * Ks = reinterpret_cast<const __half *>(stages + (tile % kStages) * STAGE), * Vs = Ks + kTileKeys * LD;
            const int mi = lane >> 3;
            float s[2][4];
            #pragma unroll
            for (int n = 0; n < 2; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
            #pragma unroll
            for (int k2 = 0; k2 < D / 32; k2++) {
                #pragma unroll
                for (int n = 0; n < 2; n++) {
                    uint32_t b0, b1, b2, b3;      // keys wk + 8 n .., dims 32 k2 + 8 mi ..: the B fragments of two k steps
                    ldsm4(smem_u32(Ks + (wk + n * 8 + (lane & 7)) * LD + k2 * 32 + 8 * mi), b0, b1, b2, b3);
                    mma_f16_top(s[n], qh[2 * k2][0], qh[2 * k2][1], b0, b1);
                    mma_f16_top(s[n], ql[2 * k2][0], ql[2 * k2][1], b0, b1);
                    mma_f16_top(s[n], qh[2 * k2 + 1][0], qh[2 * k2 + 1][1], b2, b3);
                    mma_f16_top(s[n], ql[2 * k2 + 1][0], ql[2 * k2 + 1][1], b2, b3);
                }
            }
            float mx = m_w;
            #pragma unroll
            for (int n = 0; n < 2; n++) {
                const int key = wk + n * 8 + 2 * t;
                s[n][0] = key < cnt ? s[n][0] * scale : -CUDART_INF_F;
                s[n][1] = key + 1 < cnt ? s[n][1] * scale : -CUDART_INF_F;
                mx = fmaxf(mx, fmaxf(s[n][0], s[n][1]));
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float cf = expf(m_w - mx);       // 0 on the warp's first keys (key wk is inside the range, so mx is finite)
            m_w = mx;
            const float e00 = expf(s[0][0] - mx), e01 = expf(s[0][1] - mx), e10 = expf(s[1][0] - mx), e11 = expf(s[1][1] - mx);
            float sum = (e00 + e01) + (e10 + e11);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_w = l_w * cf + sum;
            uint32_t ph0, pl0, ph1, pl1;           // the probabilities of keys 0-7 / 8-15 of the warp's share as A fragments (row g)
            split_h2(e00, e01, ph0, pl0);
            split_h2(e10, e11, ph1, pl1);
            #pragma unroll
            for (int n = 0; n < D / 8; n++) { o[n][0] *= cf; o[n][1] *= cf; }
            #pragma unroll
            for (int n2 = 0; n2 < D / 16; n2++) {
                uint32_t b0, b1, b2, b3;          // keys wk + 8 (mi & 1) .., dims 16 n2 + 8 (mi >> 1) ..
                ldsm4_t(smem_u32(Vs + (wk + 8 * (mi & 1) + (lane & 7)) * LD + n2 * 16 + 8 * (mi >> 1)), b0, b1, b2, b3);
                mma_f16_top(o[2 * n2], ph0, ph1, b0, b1);
                mma_f16_top(o[2 * n2], pl0, pl1, b0, b1);
                mma_f16_top(o[2 * n2 + 1], ph0, ph1, b2, b3);
                mma_f16_top(o[2 * n2 + 1], pl0, pl1, b2, b3);
            }
        }
        attn_bar<WHOLE>();                        // the pair's stages are free again
        #pragma unroll
        for (int k = 0; k < 2; k++) {
            if (t2 + kStages + k < ntiles) fetch(t2 + kStages + k);
            cp_commit();
        }
    }
    cp_wait<0>();
    attn_bar<WHOLE>();
    // the warps' results side by side over the stages, [warp][head][2 + D], then per thread what the rest of the kernel works with: the (head, dim pair)
    // sums of OUT_IT outputs, and in warp w < GP the running maximum and sum of head w
    float * res = reinterpret_cast<float *>(stages);
    if (t == 0) { res[(warp * 8 + g) * RS] = m_w; res[(warp * 8 + g) * RS + 1] = l_w; }
    #pragma unroll
    for (int n = 0; n < D / 8; n++) *reinterpret_cast<float2 *>(res + (warp * 8 + g) * RS + 2 + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
    attn_bar<WHOLE>();
    float m_run = -CUDART_INF_F, l_run = 0.f;
    float acc[OUT_IT][2];
    auto weight = [&](int w, int hq, float M) { const float mw = res[(w * 8 + hq) * RS]; return mw == -CUDART_INF_F ? 0.f : expf(mw - M); };
    if (warp < GP) {
        #pragma unroll
        for (int w = 0; w < 8; w++) m_run = fmaxf(m_run, res[(w * 8 + warp) * RS]);
        #pragma unroll
        for (int w = 0; w < 8; w++) l_run += res[(w * 8 + warp) * RS + 1] * weight(w, warp, m_run);
    }
    #pragma unroll
    for (int it = 0; it < OUT_IT; it++) {
        const int idx = tid + it * kThreads;
        acc[it][0] = acc[it][1] = 0.f;
        if (idx < GP * D / 2) {
            const int hq = idx / (D / 2), dp = idx % (D / 2);
            float M = -CUDART_INF_F;
            #pragma unroll
            for (int w = 0; w < 8; w++) M = fmaxf(M, res[(w * 8 + hq) * RS]);
            #pragma unroll
            for (int w = 0; w < 8; w++) {
                const float f = weight(w, hq, M);
                const float2 v = *reinterpret_cast<const float2 *>(res + (w * 8 + hq) * RS + 2 + 2 * dp);
                acc[it][0] += v.x * f;
                acc[it][1] += v.y * f;
            }
        }
    }
    cp_wait<0>();
    // partial results (an empty range leaves sum = 0, which the merge skips)
    #pragma unroll
    for (int it = 0; it < OUT_IT; it++) {
        const int idx = tid + it * kThreads;
        if (idx < GP * D / 2) {
            const int hq = idx / (D / 2), dp = idx % (D / 2);
            if (hq < G) {
                float * dst = p.part + (int64_t(kvh * G + hq) * p.splits + split) * (2 + D) + 2;
                dst[2 * dp] = acc[it][0];
                dst[2 * dp + 1] = acc[it][1];
            }
        }
    }
    if (warp < G && lane == 0) {
        float * dst = p.part + (int64_t(kvh * G + warp) * p.splits + split) * (2 + D);
        dst[0] = m_run;
        dst[1] = l_run;
    }
    if (!p.counters) return;
    // the last block of this key/value head to get here merges: its own writes are ordered before the count, the others' are visible after it
    __shared__ int is_last;
    __threadfence();
    attn_bar<WHOLE>();
    if (tid == 0) {
        const int done = atomicAdd(p.counters + kvh, 1);
        is_last = done == n_splits - 1;
        if (is_last) p.counters[kvh] = 0;          // ready for the next step; nobody else touches it any more in this launch
    }
    attn_bar<WHOLE>();
    if (!is_last) return;
    __threadfence();
    // weights of the ranges, per head: warp w takes head w (the stage buffers are free now and hold them)
    float * wts = reinterpret_cast<float *>(stages);            // [GP][splits]
    float * tot = wts + GP * p.splits;                          // [GP]
    // Every load of the merge is issued before anything waits on one: the partial results sit in L2, a round trip there costs more than all the
    // arithmetic of the merge, and loops that load and add split by split would pay it once per split.
    if (warp < G) {
        const float * base = p.part + int64_t(kvh * G + warp) * p.splits * (2 + D);
        constexpr int kPerLane = 8;                                   // ranges per lane held in registers: up to 256 ranges
        float2 ml[kPerLane];
        #pragma unroll
        for (int k = 0; k < kPerLane; k++) {
            const int sp = lane + 32 * k;
            ml[k] = sp < p.splits ? __ldcg(reinterpret_cast<const float2 *>(base + sp * (2 + D))) : make_float2(-CUDART_INF_F, 0.f);
        }
        float mx = -CUDART_INF_F;
        #pragma unroll
        for (int k = 0; k < kPerLane; k++) if (ml[k].y > 0.f) mx = fmaxf(mx, ml[k].x);
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float total = 0.f;
        #pragma unroll
        for (int k = 0; k < kPerLane; k++) {
            const int sp = lane + 32 * k;
            if (sp < p.splits) {
                const float w = ml[k].y > 0.f ? expf(ml[k].x - mx) : 0.f;      // an empty range weighs nothing
                wts[warp * p.splits + sp] = w;
                total += ml[k].y * w;
            }
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane == 0) tot[warp] = total;
    }
    constexpr int kChunk = 16;                                        // ranges whose values are in flight together, per output
    float v[MERGE_IT][kChunk];
    float merged[MERGE_IT];
    #pragma unroll
    for (int it = 0; it < MERGE_IT; it++) merged[it] = 0.f;
    for (int sp0 = 0; sp0 < p.splits; sp0 += kChunk) {
        #pragma unroll
        for (int it = 0; it < MERGE_IT; it++) {
            const int idx = tid + it * kThreads;            // (head, element): a warp holds 32 consecutive elements of one head
            const int hq = idx / D, d = idx % D;
            const bool mine = idx < GP * D && hq < G;
            const float * col = p.part + int64_t(kvh * G + (mine ? hq : 0)) * p.splits * (2 + D) + 2 + d;
            #pragma unroll
            for (int k = 0; k < kChunk; k++) v[it][k] = (mine && sp0 + k < p.splits) ? __ldcg(col + (sp0 + k) * (2 + D)) : 0.f;
        }
        if (sp0 == 0) attn_bar<WHOLE>();                                // the weights are in shared memory (the first chunk's loads are already on their way)
        #pragma unroll
        for (int it = 0; it < MERGE_IT; it++) {
            const int idx = tid + it * kThreads;
            const int hq = idx / D;
            if (idx < GP * D && hq < G) {
                const float * w = wts + hq * p.splits + sp0;
                #pragma unroll
                for (int k = 0; k < kChunk; k++) if (sp0 + k < p.splits) merged[it] += v[it][k] * w[k];      // an empty range's values are finite (zeros), its weight 0
            }
        }
    }
    #pragma unroll
    for (int it = 0; it < MERGE_IT; it++) {
        const int idx = tid + it * kThreads;
        const int hq = idx / D, d = idx % D;
        if (idx < GP * D && hq < G) {
            const float r = merged[it] / tot[hq];
            p.out[(kvh * G + hq) * D + d] = r;
            if (p.out16) p.out16[(kvh * G + hq) * D + d] = __float2half_rn(r);
            if (p.xq) split_block(r, lane, ((kvh * G + hq) * D + d) / 32, p.s.n_head * D / 32, p.xq);
        }
    }
}


}  // namespace attn_decode
}  // namespace cuda
}  // namespace dooms
