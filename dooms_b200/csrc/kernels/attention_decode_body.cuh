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
constexpr int kStages = 2;

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
};

__device__ __forceinline__ void cp16(uint32_t dst, const void * src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

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
template <int D, int GP>
constexpr size_t attention_decode_smem_bytes() { return ((GP * D + GP * kTileKeys + GP) * 4 + 127) / 128 * 128 + size_t(kStages) * kTileKeys * (D * 4 + 16); }

template <int D, int GP, bool WHOLE>
__device__ __forceinline__ void attention_decode_body(const AttnDecodeParams & pp, const int kvh, const int split, const int n_splits, const int row, uint8_t * smem) {
    constexpr int KP = D * 2 + 16;                      // bytes between key rows in a stage: 16-byte loads of 8 consecutive rows fall on different banks
    constexpr int VP = D * 2;
    constexpr int STAGE = kTileKeys * (KP + VP);
    constexpr int HQ = kThreads / kTileKeys;            // threads per key in the score phase: 4, each with the heads hq, hq + 4
    constexpr int HPT = (GP + HQ - 1) / HQ;             // heads per thread there
    constexpr int OUT_IT = (GP * D / 2 + kThreads - 1) / kThreads;   // (head, dim pair) outputs per thread
    constexpr int MERGE_IT = (GP * D + kThreads - 1) / kThreads;     // single outputs per thread in the merge
    float * qs = reinterpret_cast<float *>(smem);                      // [GP][D], scaled
    float * sc = qs + GP * D;                                          // [GP][kTileKeys] scores, then probabilities
    float * corr = sc + GP * kTileKeys;                                // [GP]
    uint8_t * stages = smem + ((GP * D + GP * kTileKeys + GP) * 4 + 127) / 128 * 128;
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
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
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
        for (int i = tid; i < cnt * PIECES; i += kThreads) {
            const int r = i / PIECES, c = i % PIECES;
            cp16(base + r * KP + c * 16, p.kc + int64_t(j0 + r) * p.s.kv_stride + kvh * D + c * 8);
            cp16(base + kTileKeys * KP + r * VP + c * 16, p.vc + int64_t(j0 + r) * p.s.kv_stride + kvh * D + c * 8);
        }
    };
    if (ntiles > 0) fetch(0);
    cp_commit();
    if (ntiles > 1) fetch(1);
    cp_commit();

    // the group's queries: rotated (when asked), scaled
    const float scale = rsqrtf(float(D));
    for (int i = tid; i < GP * D / 2; i += kThreads) {
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
        qs[hq * D + e0] = r0 * scale;
        qs[hq * D + e1] = r1 * scale;
    }

    float m_run = -CUDART_INF_F, l_run = 0.f;      // of head `warp` (warps below GP)
    float acc[OUT_IT][2];
    #pragma unroll
    for (int it = 0; it < OUT_IT; it++) acc[it][0] = acc[it][1] = 0.f;

    for (int tile = 0; tile < ntiles; tile++) {
        const int j0 = j_begin + tile * kTileKeys, cnt = min(kTileKeys, j_end - j0);
        uint8_t * ks = stages + (tile % kStages) * STAGE;
        uint8_t * vs = ks + kTileKeys * KP;
        cp_wait<kStages - 1>();
        attn_bar<WHOLE>();
        if (fuse && pos >= j0 && pos < j0 + cnt) {
            // the new token's own key and value: into the cache and over the (stale) row that was just copied from it
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
                __half * row = reinterpret_cast<__half *>(ks + r * KP);
                dst[e0] = h0; dst[e1] = h1;
                row[e0] = h0; row[e1] = h1;
            } else if (tid >= 64 && tid < 64 + D) {
                const int e = tid - 64;
                const __half hv = __float2half_rn(__ldcg(p.qkv + (p.s.n_head + p.s.n_head_kv + kvh) * D + e));
                p.vc[int64_t(pos) * p.s.kv_stride + kvh * D + e] = hv;
                reinterpret_cast<__half *>(vs + r * VP)[e] = hv;
            }
            attn_bar<WHOLE>();
        }
        // scores: thread (key, hq) for heads hq, hq + HQ, ...
        {
            const int key = tid % kTileKeys, hq0 = tid / kTileKeys;
            float a[HPT];
            #pragma unroll
            for (int i = 0; i < HPT; i++) a[i] = 0.f;
            if (key < cnt && hq0 < G) {
                const uint4 * krow = reinterpret_cast<const uint4 *>(ks + key * KP);
                #pragma unroll 4
                for (int c = 0; c < D / 8; c++) {
                    const uint4 kv = krow[c];
                    const float2 k0 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.x)), k1 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.y));
                    const float2 k2 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.z)), k3 = __half22float2(*reinterpret_cast<const __half2 *>(&kv.w));
                    #pragma unroll
                    for (int i = 0; i < HPT; i++) {
                        if (hq0 + i * HQ < GP) {
                            const float4 qa = *reinterpret_cast<const float4 *>(qs + (hq0 + i * HQ) * D + c * 8);
                            const float4 qb = *reinterpret_cast<const float4 *>(qs + (hq0 + i * HQ) * D + c * 8 + 4);
                            a[i] += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y + qb.x * k2.x + qb.y * k2.y + qb.z * k3.x + qb.w * k3.y;
                        }
                    }
                }
            }
            #pragma unroll
            for (int i = 0; i < HPT; i++) if (hq0 + i * HQ < GP) sc[(hq0 + i * HQ) * kTileKeys + key] = key < cnt ? a[i] : -CUDART_INF_F;
        }
        attn_bar<WHOLE>();
        // running softmax: warp w owns head w
        if (warp < GP) {
            const float s0 = sc[warp * kTileKeys + lane], s1 = sc[warp * kTileKeys + 32 + lane];
            float mx = fmaxf(s0, s1);
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_new = fmaxf(m_run, mx);
            const float p0 = lane < cnt ? expf(s0 - m_new) : 0.f, p1 = 32 + lane < cnt ? expf(s1 - m_new) : 0.f;
            float sum = p0 + p1;
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float cf = expf(m_run - m_new);        // 0 on the first tile
            l_run = l_run * cf + sum;
            m_run = m_new;
            sc[warp * kTileKeys + lane] = p0;
            sc[warp * kTileKeys + 32 + lane] = p1;
            if (lane == 0) corr[warp] = cf;
        }
        attn_bar<WHOLE>();
        // values: thread owns (head, dim pair) outputs
        #pragma unroll
        for (int it = 0; it < OUT_IT; it++) {
            const int idx = tid + it * kThreads;
            if (idx < GP * D / 2) {
                const int hq = idx / (D / 2), dp = idx % (D / 2);
                const float cf = corr[hq];
                float a0 = acc[it][0] * cf, a1 = acc[it][1] * cf;
                const float * pr = sc + hq * kTileKeys;
                const __half2 * vcol = reinterpret_cast<const __half2 *>(vs) + dp;
                if (cnt == kTileKeys) {
                    #pragma unroll 4
                    for (int k = 0; k < kTileKeys; k += 4) {
                        const float4 pk = *reinterpret_cast<const float4 *>(pr + k);
                        const float2 v0 = __half22float2(vcol[(k + 0) * (D / 2)]), v1 = __half22float2(vcol[(k + 1) * (D / 2)]);
                        const float2 v2 = __half22float2(vcol[(k + 2) * (D / 2)]), v3 = __half22float2(vcol[(k + 3) * (D / 2)]);
                        a0 += pk.x * v0.x; a1 += pk.x * v0.y;
                        a0 += pk.y * v1.x; a1 += pk.y * v1.y;
                        a0 += pk.z * v2.x; a1 += pk.z * v2.y;
                        a0 += pk.w * v3.x; a1 += pk.w * v3.y;
                    }
                } else {
                    // rows past cnt hold old bytes: their probabilities are 0, but 0 x NaN is not
                    for (int k = 0; k < cnt; k++) {
                        const float2 v = __half22float2(vcol[k * (D / 2)]);
                        a0 += pr[k] * v.x; a1 += pr[k] * v.y;
                    }
                }
                acc[it][0] = a0;
                acc[it][1] = a1;
            }
        }
        attn_bar<WHOLE>();                       // the stage and the scores are free again
        if (tile + kStages < ntiles) fetch(tile + kStages);
        cp_commit();
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
