// Decode attention for one new token, grouped-query aware: the query heads that share a key/value head are processed together, so every cached key and value
// row is read from device memory once per step, in 16-byte coalesced asynchronous copies, by a grid of (key/value head, range of positions) blocks that
// covers all SMs. The kernel also does what used to be a launch of its own before it: it rotates the new token's query and key (rope_store,
// src/backend/metal/llama_kernels.h:521-545), writes the rotated key and the value into the f16 cache, and uses them from shared memory in the same pass.
// Each block leaves an unnormalised partial result (max, sum, values) per query head; the block that finishes a key/value head's last range merges the
// ranges of its query heads itself (attention_split / attention_combine, llama_kernels.h:860-929), or k_attention_combine does when no counters are given.
// The scores and the weighted sums run on the tensor cores (attention_decode_body.cuh).
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"
#include "xsplit.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

}  // namespace
}  // namespace cuda
}  // namespace dooms

#include "attention_decode_body.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::cuda::attn_decode;

namespace {

template <int D, int GP>
__global__ void __launch_bounds__(kThreads) k_attention_decode(const AttnDecodeParams pp) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_trigger();
    if (pp.l2_hint) {
        // The cached keys and values of earlier positions do not depend on the projection that runs before this kernel. While that projection's last
        // blocks drain, ask for this block's range of both caches to be brought to L2 (a hint: nothing is read into the SM). The position is read before
        // the kernel that may still be writing it is known to be complete, so it can be one step old; that shifts the hinted range by one row at most.
        const int pos = __ldcg(&pp.st->pos);
        const int n_keys = pp.n_keys_fixed > 0 ? pp.n_keys_fixed : pos + 1;
        const int tiles_total = (n_keys + kTileKeys - 1) / kTileKeys, tiles_per = (tiles_total + pp.splits - 1) / pp.splits;
        const int j_begin = min(n_keys, int(blockIdx.y) * tiles_per * kTileKeys), j_end = min(n_keys, j_begin + tiles_per * kTileKeys);
        constexpr int LINES = D * 2 / 128 > 0 ? D * 2 / 128 : 1;      // 128-byte lines per cached row of one head
        if (pos >= 0 && pos < (1 << 28)) {
            for (int i = threadIdx.x; i < (j_end - j_begin) * LINES; i += kThreads) {
                const int64_t at = int64_t(j_begin + i / LINES) * pp.s.kv_stride + int(blockIdx.x) * D + (i % LINES) * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pp.kc + at));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pp.vc + at));
            }
        }
    }
    pdl_wait();
    attention_decode_body<D, GP, true>(pp, int(blockIdx.x), int(blockIdx.y), int(gridDim.y), int(blockIdx.z), smem);
}

template <int D, int GP>
cudaError_t launch_one(const AttnDecodeParams & p, cudaStream_t stream) {
    constexpr size_t smem = attention_decode_smem_bytes<D, GP>();
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_attention_decode<D, GP>, int(smem), configured); e != cudaSuccess) return e;
    return launch_pdl(k_attention_decode<D, GP>, dim3(p.s.n_head_kv, p.splits, p.b_slot ? unsigned(p.b_rows) : 1u), dim3(kThreads), smem, stream, p);
}

template <int D>
cudaError_t launch_group(const AttnDecodeParams & p, int G, cudaStream_t stream) {
    if (G == 1) return launch_one<D, 1>(p, stream);
    if (G == 2) return launch_one<D, 2>(p, stream);
    if (G <= 4) return launch_one<D, 4>(p, stream);
    return launch_one<D, 8>(p, stream);
}

}  // namespace

bool attention_gqa_supported(const AttnShape & s) {
    return (s.head_dim == 64 || s.head_dim == 128) && s.n_head % s.n_head_kv == 0 && s.n_head / s.n_head_kv <= 8 && s.kv_stride % 8 == 0;
}

int attention_gqa_splits(int n_head_kv, int n_ctx) {
    // about one block per SM, and no more ranges than the context has tiles
    static const int per_sm = [] { const char * e = getenv("DOOMS_GQA_PER_SM"); return e ? std::max(1, atoi(e)) : 1; }();
    const int want = std::max(1, (sm_count() * per_sm + n_head_kv - 1) / n_head_kv);
    static const int fixed = [] { const char * e = getenv("DOOMS_GQA_SPLITS"); return e ? atoi(e) : 0; }();
    if (fixed > 0) return std::max(1, std::min(fixed, (n_ctx + kTileKeys - 1) / kTileKeys));
    return std::max(1, std::min(want, (n_ctx + kTileKeys - 1) / kTileKeys));
}

cudaError_t launch_attention_gqa(const float * qkv, void * kc, void * vc, float * part, const DevState * st, const double * inv_freq, int n_keys_fixed,
                                 int splits, const AttnShape & s, int * counters, float * out, void * xq, cudaStream_t stream, const void * rope_cs) {
    if (!attention_gqa_supported(s) || (!inv_freq && n_keys_fixed < 1) || (counters && !out) || (xq && !counters)) return cudaErrorInvalidValue;
    AttnDecodeParams p{qkv, static_cast<__half *>(kc), static_cast<__half *>(vc), part, st, inv_freq, n_keys_fixed, splits, s, counters, out,
                       static_cast<uint8_t *>(xq), static_cast<const float2 *>(rope_cs), nullptr, nullptr, 0, 0, 0, nullptr, 0};
    static const bool hint = [] { const char * e = getenv("DOOMS_ATTN_L2_HINT"); return !(e && *e == '0'); }();
    p.l2_hint = (hint && st && inv_freq) ? 1 : 0;
    return s.head_dim == 64 ? launch_group<64>(p, s.n_head / s.n_head_kv, stream) : launch_group<128>(p, s.n_head / s.n_head_kv, stream);
}

cudaError_t launch_attention_gqa_rows(const float * qkv, void * kc, void * vc, float * part, const double * inv_freq, int splits, const AttnShape & s, int * counters,
                                      float * out, void * out16, const BatchRows & rows, int n_rows, cudaStream_t stream) {
    if (!attention_gqa_supported(s) || !inv_freq || !counters || !out || n_rows < 1 || splits < 1) return cudaErrorInvalidValue;
    const AttnDecodeParams p{qkv, static_cast<__half *>(kc), static_cast<__half *>(vc), part, nullptr, inv_freq, 0, splits, s, counters, out, nullptr, nullptr,
                             rows.slot, rows.pos, n_rows, rows.slot_elems, int64_t(splits) * s.n_head * (2 + s.head_dim), static_cast<__half *>(out16)};
    return s.head_dim == 64 ? launch_group<64>(p, s.n_head / s.n_head_kv, stream) : launch_group<128>(p, s.n_head / s.n_head_kv, stream);
}

}  // namespace cuda
}  // namespace dooms
