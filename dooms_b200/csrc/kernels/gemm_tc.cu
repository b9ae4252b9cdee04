// Prefill GEMM on the 5th-generation tensor cores: Y[m][n] (+)= sum_k X[m][k] * W[n][k] with W in its GGUF block format, dequantized tile by tile into
// shared memory and multiplied with tcgen05.mma, accumulators in tensor memory.
//
//   * One block of threads computes 128 weight rows x up to 256 tokens. The weight tile is the MMA's A operand (M = 128: one weight row per TMEM lane), the
//     token tile its B operand (N = 128 or 256), both K-major f16 in the 128-byte swizzled layout; D[n][m] lives in 256 TMEM columns (gate/up: two
//     accumulators, all 512 columns).
//   * Per 64-wide k step: the token tile (f16 activations written by the producing kernel) arrives by TMA (cp.async.bulk.tensor.2d, one block of threads per copy); 256
//     producer threads read the weight rows' raw blocks from global memory (two threads per row; q4_0 rows in 144-byte groups of 16-byte loads), dequantize them to f16 exactly as the
//     reference's tiles do (half(Q::elem), src/backend/metal/llama_kernels.h:1027-1035, 197) and store them swizzled; one thread issues the four k = 16
//     MMAs and commits the stage back to the producers. Stages are handed over through mbarriers; every wait is bounded and reports failure instead of
//     hanging.
//   * Epilogue: the producer warps read their TMEM lanes (tcgen05.ld 32x32b), add bias / the residual, or apply silu(gate) * up, and write coalesced
//     rows of Y (f32) or of the f16 activation buffer the next GEMM reads.
//   * From 128 tokens per call a matrix is first written out as f16 rows (k_dequant_f16, or a copy the caller keeps) and both operands arrive by TMA; the
//     producer warps then only run the epilogue. On that route a block may take 256 weight rows (the second accumulator holds rows 128..255 against the
//     same token tile), the first token tiles of a product running as such blocks and the rest as plain tiles, whichever split needs the fewest waves.
//   * Two ways to deal a reduction over several blocks: a product of few weight rows against one token tile (a batched decode step) writes per-share sums
//     that launch_add_shares adds in a fixed order; a fused gate / up product whose tiles leave a nearly empty last wave runs the leftover tiles that way
//     and k_gate_up_combine applies the epilogue.
// Replaces matmul_bigq / matmul_gate_up_bigq and the dequant_half + matmul_big pair of the reference (llama_kernels.h:1320-1382, 1474-1480).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"
#include "quant.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kRowsW = 128;         // weight rows per block = MMA M
constexpr int kStepK = 64;          // k elements per stage: one 128-byte swizzle row of f16
constexpr int kProducerWarps = 8;   // two threads per weight row
constexpr int kThreads = (kProducerWarps + 2) * 32;   // + the TMA warp and the MMA warp
constexpr uint32_t kTileWBytes = kRowsW * kStepK * 2; // 16 KB

// ---- tcgen05 / TMA wrappers ----
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap * map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                   "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Polls the count of consumed steps (a word in shared memory that only grows) until it reaches `want`; bounded like mbar_wait.
__device__ __forceinline__ bool wait_consumed(uint32_t addr, int want) {
    for (uint32_t i = 0; i < kMaxPolls; i++) {
        uint32_t v;
        asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
        if (int(v) >= want) { __threadfence_block(); return true; }
    }
    return false;
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzled layout: rows of 128 bytes, groups of 8 rows 1024 bytes apart (the tile base is
// 1024-byte aligned). A k = 16 slice inside the 128-byte row is addressed by adding its byte offset to the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor, kind::f16: f32 accumulator, A and B of type `bf16 ? bf16 : f16`, both K-major, M = 128, N = n.
__host__ __device__ inline uint32_t idesc_f16(int n, bool bf16) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(kRowsW >> 4) << 24);
}

// ---- dequantization of one thread's 32 elements (elements k0 .. k0+31 of a weight row, k0 a multiple of 32) to four 16-byte chunks of f16 ----

// Generic: element by element with the block formulas, rounded to f16 as the reference's tiles are (half(Q::elem)).
template <int DT>
__device__ __forceinline__ void dequant32(const uint8_t * row, uint32_t k0, uint4 (&out)[4]) {
    #pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t w[4];
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 h = __floats2half2_rn(elem<DT>(row, k0 + 8 * c + 2 * i), elem<DT>(row, k0 + 8 * c + 2 * i + 1));
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        out[c] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// q4_0: one 18-byte block. (1024 + q) is built as an f16 bit pattern, 1032 subtracted (exact), the block scale multiplied in f16: the rounding of the exact
// product d (q - 8), the same value half(d * (q - 8)) has.
__device__ __forceinline__ uint32_t h2_sub_mul(uint32_t v, __half2 d2) {
    const __half2 k1032 = __half2half2(__ushort_as_half(0x6408));      // 1032.0
    const __half2 r = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&v), k1032), d2);
    return *reinterpret_cast<const uint32_t *>(&r);
}
// raw: the block's nine 16-bit words (scale, then the quants two bytes at a time)
__device__ __forceinline__ void dequant_q4_0_words(const uint16_t (&raw)[9], uint4 (&out)[4]) {
    const __half2 d2 = __half2half2(__ushort_as_half(raw[0]));
    uint32_t lo[8], hi[8];      // half2 pairs of elements (2i, 2i+1) and (16+2i, 16+2i+1)
    #pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t two = raw[1 + i];                                  // bytes 2i, 2i+1 of qs
        const uint32_t t = (two & 0xFFu) | ((two & 0xFF00u) << 8);        // [b0, 0, b1, 0]
        lo[i] = h2_sub_mul((t & 0x000F000Fu) | 0x64006400u, d2);
        hi[i] = h2_sub_mul(((t >> 4) & 0x000F000Fu) | 0x64006400u, d2);
    }
    out[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    out[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    out[2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    out[3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
}
template <>
__device__ __forceinline__ void dequant32<kQ4_0>(const uint8_t * row, uint32_t k0, uint4 (&out)[4]) {
    const uint16_t * b = reinterpret_cast<const uint16_t *>(row + size_t(k0 / 32) * 18);
    uint16_t raw[9];
    #pragma unroll
    for (int i = 0; i < 9; i++) raw[i] = __ldg(b + i);
    dequant_q4_0_words(raw, out);
}
// Block B (0..7) of a 256-element group held in registers as 36 32-bit words (144 bytes): its 16-bit words are 9 B .. 9 B + 8 of the group's 72.
template <int B>
__device__ __forceinline__ void dequant_q4_0_group(const uint32_t (&w)[36], uint4 (&out)[4]) {
    uint16_t raw[9];
    #pragma unroll
    for (int i = 0; i < 9; i++) {
        constexpr int base = 9 * B;
        raw[i] = uint16_t(((base + i) & 1) ? w[(base + i) >> 1] >> 16 : w[(base + i) >> 1] & 0xFFFFu);
    }
    dequant_q4_0_words(raw, out);
}

// q4_K: a 256-element super-block is 144 bytes too (d, dmin, 12 scale bytes, 128 quant bytes). k step J of the group = sub-blocks 2J (the low nibbles of
// quant bytes 32J .. 32J+31) and 2J+1 (their high nibbles); every value goes through the same f32 roundings as elem<kQ4_K> before it is rounded to f16.
template <int J>
__device__ __forceinline__ void dequant_q4_K_group(const uint32_t (&w)[36], uint4 (&out)[8]) {
    const float d = __half2float(__ushort_as_half(uint16_t(w[0] & 0xFFFFu))), dmin = __half2float(__ushort_as_half(uint16_t(w[0] >> 16)));
    auto qb = [&](int j) -> uint32_t { return (w[1 + j / 4] >> (8 * (j % 4))) & 0xFFu; };      // scale byte j (an index known at compile time)
    float ds[2], mm[2];
    #pragma unroll
    for (int s = 0; s < 2; s++) {
        const int c = 2 * J + s;
        uint32_t sc, mn;
        if (c < 4) { sc = qb(c) & 63u; mn = qb(c + 4) & 63u; }
        else { sc = (qb(c + 4) & 15u) | ((qb(c < 4 ? 0 : c - 4) >> 6) << 4); mn = (qb(c + 4) >> 4) | ((qb(c) >> 6) << 4); }
        ds[s] = __fmul_rn(d, float(sc));
        mm[s] = __fmul_rn(dmin, float(mn));
    }
    auto pair = [&](uint32_t q0, uint32_t q1, float dsc, float m) -> uint32_t {
        const __half2 h = __floats2half2_rn(__fsub_rn(__fmul_rn(dsc, float(q0)), m), __fsub_rn(__fmul_rn(dsc, float(q1)), m));
        return *reinterpret_cast<const uint32_t *>(&h);
    };
    #pragma unroll
    for (int c8 = 0; c8 < 4; c8++) {
        const uint32_t a = w[4 + 8 * J + 2 * c8], b = w[4 + 8 * J + 2 * c8 + 1];      // quant bytes 8 c8 .. 8 c8 + 7 of this step
        out[c8] = make_uint4(pair(a & 15u, (a >> 8) & 15u, ds[0], mm[0]), pair((a >> 16) & 15u, (a >> 24) & 15u, ds[0], mm[0]),
                             pair(b & 15u, (b >> 8) & 15u, ds[0], mm[0]), pair((b >> 16) & 15u, (b >> 24) & 15u, ds[0], mm[0]));
        out[4 + c8] = make_uint4(pair((a >> 4) & 15u, (a >> 12) & 15u, ds[1], mm[1]), pair((a >> 20) & 15u, a >> 28, ds[1], mm[1]),
                                 pair((b >> 4) & 15u, (b >> 12) & 15u, ds[1], mm[1]), pair((b >> 20) & 15u, b >> 28, ds[1], mm[1]));
    }
}

// Whole rows to f16, the value every tile of the fused kernel would hold (half(Q::elem)): one thread per 32 elements.
template <int DT>
__global__ void __launch_bounds__(256) k_dequant_f16(const uint8_t * W, __half * out, int64_t rows, int cols) {
    const int64_t units = rows * (cols / 32);
    const int64_t RB = row_bytes_of(DT, cols);
    for (int64_t u = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = u / (cols / 32);
        const uint32_t k0 = uint32_t(u - r * (cols / 32)) * 32u;
        uint4 v[4];
        dequant32<DT>(W + r * RB, k0, v);
        uint4 * dst = reinterpret_cast<uint4 *>(out + r * cols + k0);
        dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; dst[3] = v[3];
    }
}

struct GemmTcParams {
    const uint8_t * W;
    const uint8_t * W2;        // gate/up: the up matrix
    float * Y;                 // f32 output rows [m][y_stride] (nullptr when only the f16 output is wanted)
    __half * Y16;              // f16 output rows [m][y16_stride] (gate/up: the activations the down projection reads)
    const float * bias;
    int64_t N;                 // weight rows
    int K, M;                  // reduction length, tokens
    int64_t y_stride, y16_stride;
    uint32_t flags;
    int T;                     // tokens per block: 128 or 256
    int wide;                  // q4_0 / q4_K rows of whole 256-element groups at 16-byte aligned addresses: the producers load 144-byte groups with 16-byte loads
    int pair;                  // (the two-matrix kernel) the second matrix is the next 128 rows of W: one block computes 256 weight rows against its token tile
    int ks_per;                // k steps per block along gridDim.z (0: all of them, one block per tile); block z writes its sum to Y + z * split_stride
    int64_t split_stride;
    int tile0, tiles_n;        // the block's tile is tile0 + blockIdx.x: row tile = that % tiles_n, token tile = that / tiles_n
    float * gate_shares;       // (two matrices, ks_per > 0) the raw sums of block (x, z): [x][z][matrix][token of the tile][row of the tile] floats
    int32_t * error;
};

// Shared memory: [stage][W tile | W2 tile | X tile], then the mbarriers and the TMEM base address.
// PRE: the weights were dequantized to f16 rows beforehand (k_dequant_f16; the reference's dequant_half + matmul_big pair for large M,
// llama_kernels.h:1474-1480, metal_llama_decoder.mm:31): their tiles arrive by TMA like the token tile (wmap / w2map), the producer warps only run the
// epilogue, and the stage's single "full" barrier counts the bytes of all its tiles.
template <int DT, bool GATE, bool PRE>
__global__ void __launch_bounds__(kThreads, 1) k_gemm_tc(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                                                         const __grid_constant__ CUtensorMap w2map, const GemmTcParams p) {
    constexpr int NMAT = GATE ? 2 : 1;
    constexpr int STAGES = GATE ? 3 : 4;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_x_bytes = uint32_t(p.T) * 128u;
    const uint32_t stage_bytes = NMAT * kTileWBytes + tile_x_bytes;
    const uint32_t bars = smem0 + STAGES * stage_bytes;       // full_x[S], full_w[S], empty[S], acc_full
    const uint32_t full_x = bars, full_w = bars + 8 * STAGES, empty = bars + 16 * STAGES, acc_full = bars + 24 * STAGES, tmem_slot = acc_full + 8;
    const uint32_t consumed = tmem_slot + 4;       // steps whose stage is free again, counted by the tracker lane
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const bool pair = GATE && p.pair;
    const int tile = p.tile0 + int(blockIdx.x);
    const int64_t n0 = int64_t(tile % p.tiles_n) * (pair ? 2 * kRowsW : kRowsW);
    const int m0 = (tile / p.tiles_n) * p.T;
    // a share of the reduction (f16-row path only): k steps ks0 .. ks0 + ksteps - 1
    const int ks0 = p.ks_per > 0 ? int(blockIdx.z) * p.ks_per : 0;
    const int ksteps = p.ks_per > 0 ? min(p.K / kStepK - ks0, p.ks_per) : p.K / kStepK;
    const uint32_t ncols = GATE ? 512u : 256u;

    if (!(p.flags & kFlagLateDependents)) pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full_x + 8 * s, 1); mbar_init(full_w + 8 * s, p.wide ? kProducerWarps * 16 : kProducerWarps * 32); mbar_init(empty + 8 * s, 1); }
        mbar_init(acc_full, 1);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(consumed), "r"(0u) : "memory");
        mbar_init_fence();
    }
    if (warp == kProducerWarps + 1) {      // the MMA warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
    bool ok = true;
    pdl_wait();      // every thread: from here on the token rows, the residual rows and the weights' f16 copies are those the kernels before this one wrote

    if (PRE && warp < kProducerWarps) {
        // nothing to produce: the weight tiles come by TMA
    } else if (warp < kProducerWarps && (DT == kQ4_0 || DT == kQ4_K) && p.wide) {
        // ---- weight producers, q4_0 / q4_K rows of whole 256-element groups (144 bytes in both formats): the two threads of a row take the groups (four
        // k steps each) in turn (both threads on every step, half a tile row each, measured 22 % slower on q4_0). A group is
        // 144 consecutive bytes, fetched with nine 16-byte loads per matrix before anything is computed, so that the other thread's stores overlap this
        // thread's loads; the thread then fills its four stages, a whole 128-byte row of the tile per step. ----
        const int r = (warp & 3) * 32 + lane, half = warp >> 2;
        const int64_t row = min(n0 + r, p.N - 1);
        const int64_t RB = row_bytes_of(DT, p.K);
        const uint8_t * wrow[NMAT];
        wrow[0] = p.W + row * RB;
        if (GATE) wrow[NMAT - 1] = pair ? p.W + min(n0 + kRowsW + r, p.N - 1) * RB : p.W2 + row * RB;
        const uint32_t dst_row = uint32_t(r) * 128u;
        const int groups = ksteps / 4;
        for (int g = half; g < groups && ok; g += 2) {
            uint32_t raw[NMAT][36];
            #pragma unroll
            for (int mtx = 0; mtx < NMAT; mtx++) {
                const uint4 * src = reinterpret_cast<const uint4 *>(wrow[mtx] + size_t(ks0 / 4 + g) * 144);
                #pragma unroll
                for (int i = 0; i < 9; i++) {
                    const uint4 v = __ldg(src + i);
                    raw[mtx][4 * i] = v.x; raw[mtx][4 * i + 1] = v.y; raw[mtx][4 * i + 2] = v.z; raw[mtx][4 * i + 3] = v.w;
                }
            }
            auto step = [&]<int J>() {
                // A thread comes back to a stage only every eighth step while the stage's barrier completes a phase every STAGES steps: a parity wait
                // would be ambiguous, so these threads wait on the count of steps whose stage the tensor core has finished reading (see the tracker).
                const int ks = g * 4 + J, s = ks % STAGES;
                if (ks >= STAGES) ok = ok && wait_consumed(consumed, ks - STAGES + 1);
                if (!ok) return;
                #pragma unroll
                for (int mtx = 0; mtx < NMAT; mtx++) {
                    uint4 v[8];
                    if constexpr (DT == kQ4_K) {
                        dequant_q4_K_group<J>(raw[mtx], v);
                    } else {
                        dequant_q4_0_group<2 * J>(raw[mtx], reinterpret_cast<uint4 (&)[4]>(v[0]));
                        dequant_q4_0_group<2 * J + 1>(raw[mtx], reinterpret_cast<uint4 (&)[4]>(v[4]));
                    }
                    const uint32_t tile = smem0 + s * stage_bytes + mtx * kTileWBytes + dst_row;
                    #pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const uint32_t chunk = uint32_t(c) ^ uint32_t(r & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile + chunk * 16u), "r"(v[c].x), "r"(v[c].y), "r"(v[c].z), "r"(v[c].w) : "memory");
                    }
                }
                fence_async_smem();
                mbar_arrive(full_w + 8 * s);
            };
            step.template operator()<0>();
            step.template operator()<1>();
            step.template operator()<2>();
            step.template operator()<3>();
        }
    } else if (warp < kProducerWarps) {
        // ---- weight producers, any format: row r of the tile, elements 32 half .. 32 half + 31 of each k step ----
        const int r = (warp & 3) * 32 + lane, half = warp >> 2;
        const int64_t row = min(n0 + r, p.N - 1);
        const int64_t RB = row_bytes_of(DT, p.K);
        const uint8_t * wrow[NMAT];
        wrow[0] = p.W + row * RB;
        if (GATE) wrow[NMAT - 1] = pair ? p.W + min(n0 + kRowsW + r, p.N - 1) * RB : p.W2 + row * RB;
        const uint32_t dst_row = uint32_t(r) * 128u;
        for (int ks = 0; ks < ksteps && ok; ks++) {
            const int s = ks % STAGES;
            if (ks >= STAGES) ok = mbar_wait(empty + 8 * s, uint32_t(ks / STAGES - 1) & 1u);
            if (!ok) break;
            #pragma unroll
            for (int mtx = 0; mtx < NMAT; mtx++) {
                uint4 v[4];
                dequant32<DT>(wrow[mtx], uint32_t((ks0 + ks) * kStepK + half * 32), v);
                const uint32_t tile = smem0 + s * stage_bytes + mtx * kTileWBytes + dst_row;
                #pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint32_t chunk = uint32_t(half * 4 + c) ^ uint32_t(r & 7);
                    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(tile + chunk * 16u), "r"(v[c].x), "r"(v[c].y), "r"(v[c].z), "r"(v[c].w) : "memory");
                }
            }
            fence_async_smem();      // the generic-proxy stores above must be visible to the tensor core's (asynchronous proxy) reads
            mbar_arrive(full_w + 8 * s);
        }
    } else if (warp == kProducerWarps) {
        // ---- TMA producer: the token tile of each k step (rows past the activation buffer are filled with zeros by the copy) ----
        if (lane == 0) {
            for (int ks = 0; ks < ksteps && ok; ks++) {
                const int s = ks % STAGES;
                if (ks >= STAGES) ok = mbar_wait(empty + 8 * s, uint32_t(ks / STAGES - 1) & 1u);
                if (!ok) break;
                const uint32_t dst = smem0 + s * stage_bytes + NMAT * kTileWBytes;
                mbar_arrive_expect_tx(full_x + 8 * s, tile_x_bytes + (PRE ? NMAT * kTileWBytes : 0u));
                for (int part = 0; part < p.T / 128; part++) tma_load_2d(dst + part * 16384u, &xmap, (ks0 + ks) * kStepK, m0 + part * 128, full_x + 8 * s);
                if (PRE) {
                    tma_load_2d(smem0 + s * stage_bytes, &wmap, (ks0 + ks) * kStepK, int(n0), full_x + 8 * s);
                    if (GATE) tma_load_2d(smem0 + s * stage_bytes + kTileWBytes, &w2map, (ks0 + ks) * kStepK, int(n0) + (pair ? kRowsW : 0), full_x + 8 * s);
                }
            }
        } else if (lane == 1 && p.wide) {
            // ---- tracker: passes through every phase of the stages' "empty" barriers in order and publishes the number of steps consumed ----
            for (int ks = 0; ks < ksteps && ok; ks++) {
                ok = mbar_wait(empty + 8 * (ks % STAGES), uint32_t(ks / STAGES) & 1u);
                if (ok) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(consumed), "r"(uint32_t(ks + 1)) : "memory");
            }
        }
    } else {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = idesc_f16(p.T, false);
            for (int ks = 0; ks < ksteps && ok; ks++) {
                const int s = ks % STAGES;
                const uint32_t ph = uint32_t(ks / STAGES) & 1u;
                ok = mbar_wait(full_x + 8 * s, ph) && (PRE || mbar_wait(full_w + 8 * s, ph));
                if (!ok) break;
                tc_fence_after();
                const uint32_t wt = smem0 + s * stage_bytes, xt = wt + NMAT * kTileWBytes;
                #pragma unroll
                for (int kk = 0; kk < kStepK / 16; kk++) {
                    const uint64_t bdesc = smem_desc_sw128(xt + kk * 32);
                    #pragma unroll
                    for (int mtx = 0; mtx < NMAT; mtx++) {
                        tc_mma_f16(tmem_base + mtx * 256u, smem_desc_sw128(wt + mtx * kTileWBytes + kk * 32), bdesc, idesc, (ks | kk) ? 1u : 0u);
                    }
                }
                tc_commit(empty + 8 * s);      // arrives when the MMAs above have read the stage
            }
            if (ok) tc_commit(acc_full);       // ... and this one when every MMA has written the accumulators
        }
    }
    __syncwarp();
    ok = __all_sync(0xffffffffu, ok);

    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (its weight rows) and half of the token columns ----
    if (warp < kProducerWarps) {
        if (ok) ok = mbar_wait(acc_full, 0);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3, colhalf = warp >> 2;
            const int cols_per_warp = p.T / 2;
            float * const Y = p.Y ? p.Y + (p.ks_per > 0 ? int64_t(blockIdx.z) * p.split_stride : 0) : nullptr;
            if (GATE && !pair && p.gate_shares) {
                // a share of a gate / up tile's reduction: both raw sums go out as they are; k_gate_up_combine adds the shares and applies silu(g) * u
                float * dst = p.gate_shares + (int64_t(blockIdx.x) * gridDim.z + blockIdx.z) * 2 * p.T * kRowsW + q * 32 + lane;
                for (int c0 = colhalf * cols_per_warp; c0 < (colhalf + 1) * cols_per_warp; c0 += 32) {
                    uint32_t acc[32], acc2[32];
                    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c0);
                    tc_ld32(taddr, acc);
                    tc_ld32(taddr + 256u, acc2);
                    #pragma unroll
                    for (int j = 0; j < 32; j++) {
                        dst[int64_t(c0 + j) * kRowsW] = __uint_as_float(acc[j]);
                        dst[int64_t(p.T + c0 + j) * kRowsW] = __uint_as_float(acc2[j]);
                    }
                }
            } else
            // pair: the second accumulator holds the next 128 weight rows, with the same epilogue as the first
            for (int part = 0; part < (pair ? 2 : 1); part++) {
                const int64_t n = n0 + part * kRowsW + q * 32 + lane;
                const float bias = (p.flags & kFlagBias) && n < p.N ? p.bias[n] : 0.f;
                for (int c0 = colhalf * cols_per_warp; c0 < (colhalf + 1) * cols_per_warp; c0 += 32) {
                    if (m0 + c0 >= p.M) break;      // warp-uniform
                    uint32_t acc[32], acc2[32];
                    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c0) + uint32_t(part) * 256u;
                    // what the results are added to: all 32 loads of a lane are asked for before the first is used (one after another, each behind the
                    // store before it, they cost a memory latency apiece: 4 x 32 of them per tile)
                    float old[32];
                    const bool adds = Y && (p.flags & kFlagAccumulate) && n < p.N;
                    #pragma unroll
                    for (int j = 0; j < 32; j++) old[j] = (adds && m0 + c0 + j < p.M) ? __ldcg(Y + int64_t(m0 + c0 + j) * p.y_stride + n) : 0.f;
                    tc_ld32(taddr, acc);
                    if (GATE && !pair) tc_ld32(taddr + 256u, acc2);
                    if (n < p.N) {
                        #pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const int m = m0 + c0 + j;
                            if (m >= p.M) continue;
                            float v = __uint_as_float(acc[j]);
                            if (GATE && !pair) v = v / (1.f + expf(-v)) * __uint_as_float(acc2[j]);
                            else v += bias;
                            v += old[j];
                            if (Y) Y[int64_t(m) * p.y_stride + n] = v;
                            if (p.Y16) p.Y16[int64_t(m) * p.y16_stride + n] = __float2half_rn(v);
                        }
                    }
                }
            }
        }
    }
    if (!ok && lane == 0 && p.error) *p.error = 2;
    tc_fence_before();
    __syncthreads();
    if (warp == kProducerWarps + 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void * sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        }
    });
    return fn;
}

template <int DT, bool PRE>
cudaError_t launch_tiles(const CUtensorMap & map, const CUtensorMap & wmap, const CUtensorMap & w2map, const GemmTcParams & p, bool gate, int n_tiles, cudaStream_t stream) {
    const size_t stage = (gate ? 2 : 1) * size_t(kTileWBytes) + size_t(p.T) * 128;
    const size_t smem = (gate ? 3 : 4) * stage + 1024 + 256;
    const int k_blocks = p.ks_per > 0 ? (p.K / kStepK + p.ks_per - 1) / p.ks_per : 1;
    const dim3 grid(unsigned(n_tiles), 1u, unsigned(k_blocks));
    static std::atomic<uint64_t> configured[2];
    if (const cudaError_t e = gate ? allow_dynamic_smem(k_gemm_tc<DT, true, PRE>, 220 * 1024, configured[1])
                                   : allow_dynamic_smem(k_gemm_tc<DT, false, PRE>, 220 * 1024, configured[0]); e != cudaSuccess) return e;
    // launched early: the block's set-up (mbarriers, tensor memory) overlaps the end of the kernel before it
    if (gate) return launch_pdl(k_gemm_tc<DT, true, PRE>, grid, dim3(kThreads), smem, stream, map, wmap, w2map, p);
    return launch_pdl(k_gemm_tc<DT, false, PRE>, grid, dim3(kThreads), smem, stream, map, wmap, w2map, p);
}

// Adds the shares of the tiles tile0 .. tile0 + gridDim.x - 1 of a gate / up product in a fixed order and writes silu(gate) * up as f16 (the epilogue of
// the unsplit tile, matmul_gate_up_bigq, src/backend/metal/llama_kernels.h:1351-1382).
__global__ void __launch_bounds__(256) k_gate_up_combine(const float * shares, int n_shares, int tile0, int tiles_n, int T, float * Y, int64_t y_stride, __half * Y16,
                                                         int64_t y16_stride, int64_t N, int M) {
    pdl_trigger();
    pdl_wait();
    const int tile = tile0 + int(blockIdx.x);
    const int64_t n0 = int64_t(tile % tiles_n) * kRowsW;
    const int m0 = (tile / tiles_n) * T;
    const int64_t plane = int64_t(T) * kRowsW;
    const float * mine = shares + int64_t(blockIdx.x) * n_shares * 2 * plane;
    for (int idx = int(blockIdx.y) * 256 + int(threadIdx.x); idx < T * kRowsW; idx += int(gridDim.y) * 256) {
        const int j = idx / kRowsW, r = idx % kRowsW;
        float g = 0.f, u = 0.f;
        for (int z = 0; z < n_shares; z++) {
            g += __ldcg(mine + (int64_t(z) * 2) * plane + idx);
            u += __ldcg(mine + (int64_t(z) * 2 + 1) * plane + idx);
        }
        if (m0 + j < M && n0 + r < N) {
            const float v = g / (1.f + expf(-g)) * u;
            if (Y) Y[int64_t(m0 + j) * y_stride + n0 + r] = v;
            if (Y16) Y16[int64_t(m0 + j) * y16_stride + n0 + r] = __float2half_rn(v);
        }
    }
}

// All tiles of a product. A fused gate / up product whose tiles do not fill the last wave of blocks (896 tiles on 148 SMs: six waves and eight tiles) runs
// its leftover tiles with their reduction dealt over the idle SMs (shares of whole 256-element groups), so that the last wave is short instead of as long
// as the others; `scratch` holds the shares' raw sums until k_gate_up_combine has applied the epilogue.
template <int DT, bool PRE>
cudaError_t launch_dt(const CUtensorMap & map, const CUtensorMap & wmap, const CUtensorMap & w2map, GemmTcParams p, bool gate, cudaStream_t stream,
                      void * scratch = nullptr, size_t scratch_bytes = 0) {
    const int64_t rows_per_block = p.pair ? 2 * kRowsW : kRowsW;
    p.tiles_n = int((p.N + rows_per_block - 1) / rows_per_block);
    const int tiles = p.tiles_n * ((p.M + p.T - 1) / p.T);
    p.tile0 = 0;
    p.gate_shares = nullptr;
    static const bool tail_off = [] { const char * e = getenv("DOOMS_GEMM_TAIL"); return e && *e == '0'; }();
    const int sms = sm_count(), left = tiles % sms, ksteps = p.K / kStepK;
    int per = 0, shares = 0;
    if (!tail_off && gate && !p.pair && !PRE && p.ks_per == 0 && scratch && tiles > sms && left > 0 && left * 4 <= sms && ksteps >= 16 && ksteps % 4 == 0) {
        const int want = std::min(sms / left, ksteps / 4);
        per = ((ksteps / 4 + want - 1) / want) * 4;
        shares = (ksteps + per - 1) / per;
        if (shares < 2 || size_t(left) * shares * 2 * p.T * kRowsW * sizeof(float) > scratch_bytes) shares = 0;
    }
    if (shares == 0) return launch_tiles<DT, PRE>(map, wmap, w2map, p, gate, tiles, stream);
    cudaError_t e = launch_tiles<DT, PRE>(map, wmap, w2map, p, gate, tiles - left, stream);
    if (e != cudaSuccess) return e;
    GemmTcParams t = p;
    t.tile0 = tiles - left;
    t.ks_per = per;
    t.gate_shares = static_cast<float *>(scratch);
    e = launch_tiles<DT, PRE>(map, wmap, w2map, t, gate, left, stream);
    if (e != cudaSuccess) return e;
    return launch_pdl(k_gate_up_combine, dim3(unsigned(left), 16u), dim3(256), 0, stream, static_cast<const float *>(t.gate_shares), shares, t.tile0, p.tiles_n, p.T, p.Y,
                      p.y_stride, p.Y16, p.y16_stride, p.N, p.M);
}

template <int DT>
cudaError_t dequant_rows(const void * W, void * out, int64_t rows, int64_t cols, cudaStream_t stream) {
    const int64_t units = rows * (cols / 32);
    k_dequant_f16<DT><<<unsigned(std::min<int64_t>((units + 255) / 256, sm_count() * 16)), 256, 0, stream>>>(static_cast<const uint8_t *>(W), static_cast<__half *>(out), rows, int(cols));
    return cudaGetLastError();
}
cudaError_t dequant_rows_dt(int dt, const void * W, void * out, int64_t rows, int64_t cols, cudaStream_t stream) {
    switch (dt) {
        case kF16: return dequant_rows<kF16>(W, out, rows, cols, stream);
        case kQ4_0: return dequant_rows<kQ4_0>(W, out, rows, cols, stream);
        case kQ5_0: return dequant_rows<kQ5_0>(W, out, rows, cols, stream);
        case kQ8_0: return dequant_rows<kQ8_0>(W, out, rows, cols, stream);
        case kQ4_K: return dequant_rows<kQ4_K>(W, out, rows, cols, stream);
        case kQ6_K: return dequant_rows<kQ6_K>(W, out, rows, cols, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

static_assert(sizeof(TensorMap) == sizeof(CUtensorMap) && alignof(TensorMap) >= alignof(CUtensorMap), "TensorMap must hold a CUtensorMap");

cudaError_t make_activation_map(TensorMap * out, const void * base, int64_t rows, int64_t cols) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {cuuint32_t(kStepK), 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t make_rows_map(TensorMap * out, const void * base, int64_t rows, int64_t row_bytes, int box_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return cudaErrorNotSupported;
    if (row_bytes % 16 != 0 || box_bytes % 16 != 0 || box_bytes > 512 || box_rows < 1 || box_rows > 256 || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) return cudaErrorInvalidValue;
    const cuuint64_t dims[2] = {cuuint64_t(row_bytes / 2), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(row_bytes)};
    const cuuint32_t box[2] = {cuuint32_t(box_bytes / 2), cuuint32_t(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = fn(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// The f16-row path is taken from this many tokens on (see launch_gemm_tc).
static int pre_from_tokens() {
    static const int v = [] { const char * e = getenv("DOOMS_GEMM_PRE_FROM"); return e ? atoi(e) : 128; }();
    return v;
}

static int k_splits_of_rows16(int M, int64_t N, int64_t K);

int gemm_tc_k_splits(int dt, int M, int64_t N, int64_t K, bool gate, size_t w16_bytes) {
    const bool wide = (dt == kQ4_0 || dt == kQ4_K) && K % 256 == 0;
    const bool pre = w16_bytes >= size_t(N) * size_t(K) * 2 * (gate ? 2 : 1) && M >= pre_from_tokens() && dt != kF16 && !(wide && gate);
    if (gate || !pre) return 1;
    return k_splits_of_rows16(M, N, K);
}
int gemm_tc_rows16_k_splits(int M, int64_t N, int64_t K) { return k_splits_of_rows16(M, N, K); }

static int k_splits_of_rows16(int M, int64_t N, int64_t K) {
    static const bool off = [] { const char * e = getenv("DOOMS_GEMM_SPLIT_K"); return e && *e == '0'; }();
    if (off || K % kStepK != 0) return 1;
    const int T = M > 128 ? 256 : 128;
    const int64_t tiles = (N + kRowsW - 1) / kRowsW * ((M + T - 1) / T);
    const int ksteps = int(K / kStepK);
    // worth it when the tiles leave most SMs idle and every share still has a few k steps; shares of equal size, none empty
    int want = int(std::min<int64_t>(sm_count() / std::max<int64_t>(tiles, 1), ksteps / 4));
    if (tiles * 2 > sm_count() || want < 2) return 1;
    want = std::min(want, 32);
    const int per = (ksteps + want - 1) / want;
    return (ksteps + per - 1) / per;
}

bool gemm_tc_supported(int dt, const void * W, int64_t N, int64_t K) {
    (void)W;
    const bool type_ok = dt == kF16 || dt == kQ4_0 || dt == kQ5_0 || dt == kQ8_0 || dt == kQ4_K || dt == kQ6_K;
    return type_ok && N >= 1 && K >= kStepK && K % kStepK == 0;
}

// Both operands by TMA: the token rows behind xmap against weights that are f16 rows [N][K] in device memory (w2_16: the second matrix of a gate / up pair).
static cudaError_t launch_rows16(GemmTcParams p, const CUtensorMap & xmap, const __half * w16, const __half * w2_16, int M, int64_t N, int64_t K, int k_splits,
                                 int64_t split_stride, cudaStream_t stream) {
    const bool gate = w2_16 != nullptr;
    TensorMap wmap, w2map;
    cudaError_t e = make_activation_map(&wmap, w16, N, K);
    if (e == cudaSuccess) e = make_activation_map(&w2map, gate ? w2_16 : w16, N, K);
    if (e != cudaSuccess) return e;
    p.wide = 0;
    if (k_splits > 1) {
        const int ksteps = int(K / kStepK);
        p.ks_per = (ksteps + k_splits - 1) / k_splits;
        p.split_stride = split_stride;
    }
    // One matrix: a block may take 256 weight rows (two accumulators that share the token tile), which cuts what a block pulls out of L2 per flop by
    // a third. A block of 256 rows is taken to cost 1.5 plain tiles; the first `pair_tm` token tiles run as such blocks and the rest as plain tiles,
    // whichever split needs the least time in waves of one block per SM (the 8B qkv product, 48 x 8 plain tiles: six token tiles as 144 blocks of 256
    // rows, two as 96 plain tiles, 2.5 units of time against 3 either way alone).
    const CUtensorMap & wm = *reinterpret_cast<const CUtensorMap *>(&wmap), & w2m = *reinterpret_cast<const CUtensorMap *>(&w2map);
    if (gate || k_splits > 1 || N <= kRowsW) return launch_dt<kF16, true>(xmap, wm, w2m, p, gate, stream);
    static const int pair_mode = [] { const char * e = getenv("DOOMS_GEMM_PAIR"); return e ? atoi(e) : -1; }();      // 0: never, 1: always, -1: by the estimate
    const int token_tiles = (M + p.T - 1) / p.T, sms = sm_count();
    const int tiles_single = int((N + kRowsW - 1) / kRowsW), tiles_pair = int((N + 2 * kRowsW - 1) / (2 * kRowsW));
    int pair_tm = 0;
    if (pair_mode > 0) pair_tm = token_tiles;
    if (pair_mode < 0) {
        int64_t best = -1;
        for (int tm = 0; tm <= token_tiles; tm++) {
            const int64_t cost = int64_t((tiles_pair * tm + sms - 1) / sms) * 3 + int64_t((tiles_single * (token_tiles - tm) + sms - 1) / sms) * 2;
            if (best < 0 || cost < best) { best = cost; pair_tm = tm; }
        }
    }
    cudaError_t e2 = cudaSuccess;
    if (pair_tm > 0) {
        GemmTcParams q = p;
        q.pair = 1;
        q.tiles_n = tiles_pair;
        q.tile0 = 0;
        e2 = launch_tiles<kF16, true>(xmap, wm, w2m, q, true, tiles_pair * pair_tm, stream);
    }
    if (e2 == cudaSuccess && pair_tm < token_tiles) {
        GemmTcParams q = p;
        q.pair = 0;
        q.tiles_n = tiles_single;
        q.tile0 = tiles_single * pair_tm;
        e2 = launch_tiles<kF16, true>(xmap, wm, w2m, q, false, tiles_single * (token_tiles - pair_tm), stream);
    }
    return e2;
}

cudaError_t launch_gemm_tc_rows16(const void * W16, const void * W2_16, const TensorMap * xmap, float * Y, void * Y16, const float * bias, int M, int64_t N, int64_t K,
                                  int64_t y_stride, int64_t y16_stride, uint32_t flags, int32_t * error, cudaStream_t stream, int k_splits, int64_t split_stride) {
    if (!W16 || N < 1 || K < kStepK || K % kStepK != 0 || M < 1 || (reinterpret_cast<uintptr_t>(W16) & 15u) || (reinterpret_cast<uintptr_t>(W2_16) & 15u)) return cudaErrorInvalidValue;
    if (k_splits > 1 && (k_splits != k_splits_of_rows16(M, N, K) || W2_16 || !Y || Y16 || flags || split_stride < int64_t(M) * y_stride)) return cudaErrorInvalidValue;
    GemmTcParams p{nullptr, nullptr, Y, static_cast<__half *>(Y16), bias, N, int(K), M, y_stride, y16_stride, flags, M > 128 ? 256 : 128, 0, 0, 0, 0, 0, 0, nullptr, error};
    return launch_rows16(p, *reinterpret_cast<const CUtensorMap *>(xmap), static_cast<const __half *>(W16), static_cast<const __half *>(W2_16), M, N, K, k_splits,
                         split_stride, stream);
}

cudaError_t launch_dequant_rows16(int dt, const void * W, void * out, int64_t rows, int64_t cols, cudaStream_t stream) {
    if (!W || !out || rows < 1 || cols < 32 || cols % 32 != 0) return cudaErrorInvalidValue;
    return dequant_rows_dt(dt, W, out, rows, cols, stream);
}

cudaError_t launch_gemm_tc(int dt, const void * W, const void * W2, const TensorMap * xmap, float * Y, void * Y16, const float * bias, int M, int64_t N, int64_t K,
                           int64_t y_stride, int64_t y16_stride, uint32_t flags, int32_t * error, cudaStream_t stream, void * w16_scratch, size_t w16_bytes, int k_splits,
                           int64_t split_stride) {
    if (!gemm_tc_supported(dt, W, N, K) || M < 1) return cudaErrorInvalidValue;
    if (k_splits > 1 && (k_splits != gemm_tc_k_splits(dt, M, N, K, W2 != nullptr, w16_scratch ? w16_bytes : 0) || !Y || Y16 || flags || split_stride < int64_t(M) * y_stride)) {
        return cudaErrorInvalidValue;
    }
    GemmTcParams p{static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(W2), Y, static_cast<__half *>(Y16), bias, N, int(K), M, y_stride, y16_stride,
                   flags, M > 128 ? 256 : 128, 0, 0, 0, 0, 0, 0, nullptr, error};
    p.wide = (dt == kQ4_0 || dt == kQ4_K) && K % 256 == 0 && (reinterpret_cast<uintptr_t>(W) & 15u) == 0 && (!W2 || (reinterpret_cast<uintptr_t>(W2) & 15u) == 0) ? 1 : 0;
    const CUtensorMap & map = *reinterpret_cast<const CUtensorMap *>(xmap);
    const bool gate = W2 != nullptr;
    // Many tokens: dequantize the matrix once to f16 rows and let TMA feed both operands (the reference does the same from 320 tokens on,
    // metal_llama_decoder.mm:31); otherwise every token tile would redo the dequantization in its producer warps.
    const size_t need = size_t(N) * size_t(K) * 2 * (gate ? 2 : 1);
    // (from 128 tokens: a batched decode step of 256 rows on the 0.5B shape measured 6.4 ms with the weights dequantized by each block's producer warps
    // and 5.5 ms from f16 rows; with few blocks per matrix the producers' loads are a chain of memory latencies)
    const int pre_from = pre_from_tokens();
    // Measured on the 8B shapes: q4_0 / q4_K gate/up is faster fused (875 against 836 TFLOP/s: no f16 copy to write and read), everything else is faster
    // or much faster from f16 rows (ffn_down 961 against 925; q6_K 754 against 83).
    if (w16_scratch && need <= w16_bytes && M >= pre_from && dt != kF16 && !(p.wide && gate)) {
        __half * w16 = static_cast<__half *>(w16_scratch);
        cudaError_t e = dequant_rows_dt(dt, W, w16, N, K, stream);
        if (e == cudaSuccess && gate) e = dequant_rows_dt(dt, W2, w16 + size_t(N) * size_t(K), N, K, stream);
        if (e != cudaSuccess) return e;
        return launch_rows16(p, map, w16, gate ? w16 + size_t(N) * size_t(K) : nullptr, M, N, K, k_splits, split_stride, stream);
    }
    switch (dt) {
        case kF16: return launch_dt<kF16, false>(map, map, map, p, gate, stream);
        case kQ4_0: return launch_dt<kQ4_0, false>(map, map, map, p, gate, stream, w16_scratch, w16_bytes);
        case kQ5_0: return launch_dt<kQ5_0, false>(map, map, map, p, gate, stream);
        case kQ8_0: return launch_dt<kQ8_0, false>(map, map, map, p, gate, stream);
        case kQ4_K: return launch_dt<kQ4_K, false>(map, map, map, p, gate, stream, w16_scratch, w16_bytes);
        case kQ6_K: return launch_dt<kQ6_K, false>(map, map, map, p, gate, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cuda
}  // namespace dooms
