// Decode GEMV on q4_0 rows, built for HBM speed on B200.
//
// The work per weight has to stay near one instruction for the kernel to keep up with ~44 GB/s per SM, so the dot products run on the tensor cores'
// integer path and the CUDA cores only unpack nibbles and apply block scales:
//   * The input vector arrives pre-split (k_quantize_x): per 32-element block a power-of-two scale s and, for every element, the 28-bit fixed-point value
//     X = rint(x / s * 2^26) cut into four balanced base-128 digits (int8 "limbs"). Elements within 8x of the block's largest keep every f32 bit; the rest
//     are exact to 2^-27 of it, so the product sums are exact integers and the only rounding left is the f32 accumulation over blocks.
//   * A weight nibble q becomes the int8 value 16 (q - 8) with two logic ops per four weights (shift the nibble into the byte's high half, flip its top
//     bit), exactly the operand layout mma.m16n8k32.s8 wants for a q4_0 block: low nibbles are elements 0..15, high nibbles 16..31.
//   * One MMA per block: 16 rows x 32 elements x (4 limbs of this block | 4 limbs of the next block's slot). Two consecutive blocks accumulate into one
//     8-column fragment so that all 32 lanes have one (row, block, limb pair) to scale: acc += float(c_lo + 128 c_hi) * (d * s * 2^-30 or 2^-16).
//   * Each warp streams (16 rows x a chunk of the row) units through its own ring of shared-memory stages, filled with the rows' bytes exactly as they
//     lie in the GGUF file (18-byte blocks, 2-byte aligned; no repacking): by TMA tensor copies of 8 rows x 144 bytes with one mbarrier per stage and
//     warp (bounded polls) when rows are whole 256-element groups, otherwise by 16-byte asynchronous copies of aligned covers with a row stride in the
//     stage that keeps the 8 rows of a fragment on different banks. One block-wide barrier after the prologue, one before the epilogue.
//   * The kernel is launched early (programmatic dependent launch): it asks for its copy descriptors and its first weight stages before it waits for
//     the kernel that produces its input.
// The block formulas are the reference's (src/backend/metal/llama_kernels.h:1012-1040: value = d (q - 8)); matvec1q / gate_up1q there are the kernels this
// replaces (llama_kernels.h:1197-1269).
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <memory>
#include <vector>

#include "kernels.h"
#include "ptx.cuh"
#include "launch.cuh"
#include "xsplit.cuh"
#include "attention_decode_body.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kTileRows = 16;
constexpr int kMaxTilesPerBlockDev = 8;     // the table of per-warp sums holds this many 16-row tiles
constexpr int kBlockBytes = 18;
constexpr int kMaxPieces = 10;      // 16-byte pieces of a stage one lane copies: 16 rows x at most 20 pieces per row / 32 lanes

struct GemvQ40Params {
    const uint8_t * W;      // rows x (cols / 32) blocks
    const uint8_t * W2;     // gate/up: the second matrix (up); nullptr for a plain projection
    const uint8_t * xq;     // the split input: (cols / 32) x 128 limb bytes, then (cols / 32) x 2 floats; nullptr: the block splits x itself
    const float * x;        // the input as f32 (xq == nullptr)
    const float * gamma;    // with x: RMS-normalize it first, x[i] * rsqrt(mean(x^2) + eps) * gamma[i] (norm_vec, llama_kernels.h:1272-1286); nullptr: as it is
    float eps;
    // Optional (rows a multiple of 32): the output row is also left split for the next projection (xq layout for `rows` elements). The blocks count the rows
    // they have written per 32-row group in out_counters (rows / 32 zeroed ints, left zeroed); whoever completes a group splits it.
    uint8_t * xq_out;
    int * out_counters;
    // The RMS norm of the NEXT projection, moved to where its input is produced (both optional, with xq_out): the split that goes to xq_out is of
    // y[i] * gamma_out[i], and block b leaves the sum of its rows' y^2 in ss_out[b]. The consumer then takes xq as its input and ss_in (the producer's
    // ss_out, ss_n entries) and multiplies its own results by rsqrt(sum(ss_in) / cols + eps): W (s u) = s (W u), so the scale factor of the norm can wait
    // until after the product, and no block has to read, normalize and split the whole input for itself again.
    const float * gamma_out;
    float * ss_out;
    const float * ss_in;
    int ss_n;
    int32_t * error;        // optional mapped host word: set to 4 when a bounded wait for a tensor copy ran out (TMA variant)
    float * y;
    const float * bias;
    int64_t rows;
    int cols;
    uint32_t flags;
    int cbk;                // blocks per chunk (even)
    int nchunks;            // chunks per row
    int stride;             // bytes between the rows of a stage (multiple of 16, = 16 mod 128)
    int upr;                // 16-byte pieces copied per row of a stage (the aligned cover of a chunk)
    int rows_q, rows_r;     // units / grid and units % grid: block b has rows_q + (b < rows_r) units of row_unit rows starting at unit b rows_q + min(b, rows_r)
    int row_unit;
    uint32_t inv_upr, inv_nchunks;   // 65536 / d + 1: (j * inv) >> 16 = j / d for the small j divided here
};

// x[K] (f32) -> xq. One warp per 32-element block.
__global__ void __launch_bounds__(256) k_quantize_x(const float * x, int nb, uint8_t * xq) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x % 32;
    const int blk = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (blk >= nb) return;
    split_block(x[blk * 32 + lane], lane, blk, nb, xq);
}

// One pair of consecutive blocks (even block at byte PAIR * 36 of the chunk row, odd block 18 bytes later) of the lane's two rows. Rows and chunks start
// 4-byte aligned (an even number of 18-byte blocks each), so the even block's quants straddle two words and the odd block's are one aligned word.
template <int PAIR>
__device__ __forceinline__ void pair_step(uint32_t a0, uint32_t a1, uint32_t d0a, uint32_t d1a, uint32_t ba, uint32_t sa, bool first, float & acc0, float & acc1) {
    constexpr int O = PAIR * 36;
    const uint2 bv = lds64<PAIR * 256>(ba);
    const float sx = ldsf<PAIR * 16>(sa);
    const uint32_t e0 = __byte_perm(lds32<O>(a0), lds32<O + 4>(a0), 0x5432), e1 = __byte_perm(lds32<O>(a1), lds32<O + 4>(a1), 0x5432);
    const uint32_t o0 = lds32<O + 20>(a0), o1 = lds32<O + 20>(a1);
    const float d0 = half_bits_to_float(lds16<O>(d0a)), d1 = half_bits_to_float(lds16<O>(d1a));
    int c[4];
    mma_s8_16832_zero(c, lop3_and_xor(e0 << 4, 0xF0F0F0F0u, 0x80808080u), lop3_and_xor(e1 << 4, 0xF0F0F0F0u, 0x80808080u),
                      lop3_and_xor(e0, 0xF0F0F0F0u, 0x80808080u), lop3_and_xor(e1, 0xF0F0F0F0u, 0x80808080u), first ? bv.x : 0u, first ? bv.y : 0u);
    mma_s8_16832(c, lop3_and_xor(o0 << 4, 0xF0F0F0F0u, 0x80808080u), lop3_and_xor(o1 << 4, 0xF0F0F0F0u, 0x80808080u),
                 lop3_and_xor(o0, 0xF0F0F0F0u, 0x80808080u), lop3_and_xor(o1, 0xF0F0F0F0u, 0x80808080u), first ? 0u : bv.x, first ? 0u : bv.y);
    acc0 = fmaf(float(c[0] + 128 * c[1]), d0 * sx, acc0);
    acc1 = fmaf(float(c[2] + 128 * c[3]), d1 * sx, acc1);
}

// q4_K: a 256-element super-block is 144 bytes as well (d, dmin, 12 packed 6-bit scales / mins, 128 quant bytes), so rows, chunks and stages have the
// geometry of eight q4_0 blocks and only the unpacking differs. "Pair" J of a super-block = sub-blocks 2J (low nibbles of quant bytes 32J .. 32J+31) and
// 2J+1 (their high nibbles); value = d sc q - dmin m (Q4_K::elem, llama_kernels.h:1085-1110), so per sub-block the lane adds (d sc) (q . x) from the MMA
// and, once per row and sub-block, subtracts (dmin m) sum(x) with the sums of the input's 32-element blocks precomputed in shared memory.
// h0 / h1: the super-block's four header words of the lane's two rows. s = t >> 1: which sub-block of the pair this lane scales.
template <int J>
__device__ __forceinline__ void pair_step_k4(uint32_t a0, uint32_t a1, const uint4 & h0, const uint4 & h1, uint32_t ba, uint32_t sa, uint32_t suma, bool first,
                                             uint32_t s, bool low_pair, float & acc0, float & acc1) {
    const uint2 bv = lds64<J * 256>(ba);
    const float sx = ldsf<J * 16>(sa) * 16.f;                     // the split's factor assumes weights scaled by 16 (the q4_0 path); these are plain 0..15
    const uint32_t w00 = lds32<16 + 32 * J>(a0), w10 = lds32<32 + 32 * J>(a0), w01 = lds32<16 + 32 * J>(a1), w11 = lds32<32 + 32 * J>(a1);
    constexpr uint32_t M = 0x0F0F0F0Fu;
    int c[4] = {0, 0, 0, 0};
    mma_u8s8_16832(c, w00 & M, w01 & M, w10 & M, w11 & M, first ? bv.x : 0u, first ? bv.y : 0u);
    mma_u8s8_16832(c, (w00 >> 4) & M, (w01 >> 4) & M, (w10 >> 4) & M, (w11 >> 4) & M, first ? 0u : bv.x, first ? 0u : bv.y);
    // 6-bit scale and min of sub-block 2J + s (ggml's get_scale_min_k4): bytes 2J+s of the first two scale words for the first four sub-blocks, split
    // between the third word's nibbles and the top two bits of the first two words' bytes for the last four
    const uint32_t sh = 16u * (J & 1) + 8u * s;
    uint32_t sc0, mn0, sc1, mn1;
    if (J < 2) {
        sc0 = (h0.y >> sh) & 63u; mn0 = (h0.z >> sh) & 63u;
        sc1 = (h1.y >> sh) & 63u; mn1 = (h1.z >> sh) & 63u;
    } else {
        sc0 = ((h0.w >> sh) & 15u) | ((((h0.y >> sh) >> 6) & 3u) << 4); mn0 = (((h0.w >> sh) >> 4) & 15u) | ((((h0.z >> sh) >> 6) & 3u) << 4);
        sc1 = ((h1.w >> sh) & 15u) | ((((h1.y >> sh) >> 6) & 3u) << 4); mn1 = (((h1.w >> sh) >> 4) & 15u) | ((((h1.z >> sh) >> 6) & 3u) << 4);
    }
    const float d0 = half_bits_to_float(h0.x & 0xFFFFu), d1 = half_bits_to_float(h1.x & 0xFFFFu);
    acc0 = fmaf(float(c[0] + 128 * c[1]), d0 * float(sc0) * sx, acc0);
    acc1 = fmaf(float(c[2] + 128 * c[3]), d1 * float(sc1) * sx, acc1);
    if (low_pair) {      // one lane of the two that share the sub-block
        const float sum = ldsf<J * 8>(suma);
        acc0 = fmaf(-(half_bits_to_float(h0.x >> 16) * float(mn0)), sum, acc0);
        acc1 = fmaf(-(half_bits_to_float(h1.x >> 16) * float(mn1)), sum, acc1);
    }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Grid: one block per SM, each with an equal share of the rows (so every SM pulls the same number of bytes, to within a row). A block's rows form tiles of
// 16; the units of work are (tile, matrix, chunk of the row), dealt round-robin to the block's warps, each of which streams its units through its own ring
// of stages with 16-byte asynchronous copies (commit / wait groups: a waiting warp sleeps in hardware, there is no polling and nothing that can hang).
// A warp adds what it computed for a (tile, matrix) into its own slot of a small shared table; after one block-wide barrier the table's slots are summed
// in a fixed order, so the result does not depend on timing.
// TMA: the stages are filled by tensor copies (cp.async.bulk.tensor.2d over the matrix seen as rows of 16-bit words) instead of per-lane 16-byte copies.
// A copy's shared-memory destination has to be 128-byte aligned and its rows land densely, so the stage is cut into sub-stages of 16 rows x 144 bytes (one
// round of four pairs = eight blocks = one q4_K super-block): 144 bytes = 36 words = 4 banks more per row, which puts the 8 rows of a fragment on
// different banks, and 8 rows x 144 bytes = 1152 bytes keeps every copy's destination aligned. One elected lane issues two 8-row copies per sub-stage (one
// when the block's last tile has at most 8 rows) and the warp waits on its own mbarrier per stage (bounded). Blocks own multiples of 8 rows, so nothing
// outside a block's range is fetched; rows past the end of the matrix are zero-filled by the copy.
//
// The kernel's work is a device function so that two kernels run it: k_gemv_q4_0 (one projection per launch) and the fused decode step further down, which
// walks through all projections of all layers in one launch. FUSED: `block_index` / `n_blocks` stand for blockIdx.x / gridDim.x, the wait for the
// producer of the input is a grid-wide barrier (grid) instead of the launch dependency, the mbarriers are invalidated at the end so that the next phase
// can set them up again, and a block may own no rows at all.
// A barrier over all blocks of a cooperative launch. Arrivals are counted in one device word (zeroed by the launch's first kernel); the block whose
// arrival completes a round publishes the round's number in a second word, on a cache line of its own, and that is the word the others poll: the
// counter's line only ever sees the atomics. Waits are bounded: after one that ran out the block stops waiting at later barriers, reports through
// `error` (5) and runs to the end on whatever data it finds; the host discards the step.
struct GridBarrier {
    unsigned * words;          // [0]: arrivals; [32]: rounds completed
    int32_t * error;
    unsigned n_blocks;
    unsigned round = 0;
    bool broken = false;
};
constexpr uint32_t kGridPolls = 1u << 22;
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void grid_barrier(GridBarrier & g) {
    __syncthreads();
    if (threadIdx.x == 0) {
        g.round += 1;
        unsigned seen;
        // release: this block's writes (ordered before by the barrier above) are visible before its arrival is; acquire: the last arriver sees everyone's
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(g.words) : "memory");
        if (seen + 1 == g.round * g.n_blocks) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.words + 32), "r"(g.round) : "memory");
        } else if (!g.broken) {
            uint32_t polls = 0;
            while (ld_acquire_gpu(g.words + 32) < g.round) {
                if (++polls > kGridPolls) { g.broken = true; if (g.error) *g.error = 5; break; }
            }
        }
    }
    __syncthreads();
}

template <int WARPS, int STAGES, bool K4, bool TMA, bool FUSED>
__device__ __forceinline__ void gemv_q4_0_body(const CUtensorMap * mwp, const CUtensorMap * mw2p, const GemvQ40Params & p, uint8_t * smem, const int block_index,
                                               const int n_blocks, GridBarrier * grid) {
    (void)n_blocks;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const int nb = p.cols / 32;
    const int nmat = p.W2 ? 2 : 1;
    if constexpr (TMA) {      // the copy descriptors are on their way to the SM while the indices and the barriers are set up
        if (threadIdx.x == 32) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(mwp) : "memory");
            if (nmat == 2) asm volatile("prefetch.tensormap [%0];" ::"l"(mw2p) : "memory");
        }
    }
    const uint32_t RB = uint32_t(nb) * kBlockBytes;
    const uint32_t CB = uint32_t(p.cbk) * kBlockBytes;

    // this block's rows
    // rows are dealt in units of p.row_unit rows (1, or 8 with tensor copies): block b gets rows_q + (b < rows_r) units
    const int64_t R0 = (int64_t(block_index) * p.rows_q + min(block_index, p.rows_r)) * p.row_unit;
    const int nrows = int(max(int64_t(0), min(int64_t(p.rows_q + (block_index < p.rows_r ? 1 : 0)) * p.row_unit, p.rows - R0)));
    const int ntiles = (nrows + kTileRows - 1) / kTileRows;
    const int total_units = ntiles * nmat * p.nchunks;
    const int my_units = warp < total_units ? (total_units - warp - 1) / WARPS + 1 : 0;

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t xl = smem_base;                                                  // limbs: nb x 128, then the block scales: nb x 2 floats
    const uint32_t sxp = xl + uint32_t(nb) * 128u;
    const uint32_t stride = uint32_t(p.stride);
    constexpr uint32_t kSub = 16u * 144u;                                           // TMA: a sub-stage, 16 rows of eight blocks
    const uint32_t rounds = uint32_t(p.cbk) / 8u;
    const uint32_t stage_bytes = TMA ? rounds * kSub : uint32_t(kTileRows) * stride;
    const uint32_t sumx = sxp + uint32_t(nb) * 8u;                                   // q4_K: the sum of each 32-element block of the input
    const uint32_t stages_base = xl + ((uint32_t(nb) * 140u + 127u) & ~127u);
    const uint32_t my_stages = stages_base + uint32_t(warp) * STAGES * stage_bytes;
    float * partial = reinterpret_cast<float *>(smem + (stages_base - smem_base) + size_t(WARPS) * STAGES * stage_bytes);   // [tile][mat][warp][16]
    // TMA: this warp's mbarriers, one per stage, after the table (kMaxTilesPerBlock tiles of nmat matrices)
    const uint32_t bars = stages_base + uint32_t(WARPS) * STAGES * stage_bytes + uint32_t(kMaxTilesPerBlockDev * nmat * WARPS * kTileRows * 4) + uint32_t(warp) * STAGES * 8u;

    // Unit u of this warp is unit warp + u WARPS of the block: (tile * nmat + mat) = that / nchunks, chunk = that % nchunks. Going to the next unit adds
    // WARPS: a fixed step in the chunk index plus a carry.
    const int step_tm = int((uint32_t(WARPS) * p.inv_nchunks) >> 16), step_chunk = WARPS - step_tm * p.nchunks;
    int f_tm = int((uint32_t(warp) * p.inv_nchunks) >> 16), f_chunk = warp - f_tm * p.nchunks, f_slot = 0;      // the unit being fetched
    int u_tm = f_tm, u_chunk = f_chunk, u_slot = 0;                           // the unit being used

    // Stage copy: a stage is 16 rows x p.upr 16-byte pieces (the aligned cover of the chunk's bytes), dealt to the lanes in order, so that one instruction
    // copies 512 consecutive bytes of a row or two. Which (row, piece) a lane copies is the same for every stage: a table of packed (source offset from
    // the tile's first row << 13 | offset in the stage), built once, plus the pieces' rows as 4-bit fields: the block's last tile may have fewer than 16
    // rows, and the pieces of the missing ones are not copied (what those rows of the stage hold is computed on and dropped).
    uint32_t tab[kMaxPieces], piece_rows[2] = {0u, 0u};
    #pragma unroll
    for (int k = 0; k < (TMA ? 0 : kMaxPieces); k++) {
        const uint32_t j = uint32_t(lane) + 32u * k;
        const uint32_t row = (j * p.inv_upr) >> 16, col = j - row * uint32_t(p.upr);
        tab[k] = row < uint32_t(kTileRows) ? ((row * RB + col * 16u) << 13) | (row * stride + col * 16u) : 0xFFFFFFFFu;
        piece_rows[k / 8] |= (row & 15u) << (4 * (k % 8));
    }
    const int last_rows = nrows - 1 - (ntiles - 1) * kTileRows;      // the last tile's last row
    auto fetch = [&]() {
        const int tile = nmat == 2 ? f_tm >> 1 : f_tm, mat = nmat == 2 ? f_tm & 1 : 0;
        const uint8_t * base = (mat ? p.W2 : p.W) + (R0 + tile * kTileRows) * int64_t(RB) + uint32_t(f_chunk) * CB;      // the tile's first row, this chunk
        const uint32_t lo = uint32_t(reinterpret_cast<uintptr_t>(base));
        const uint32_t dst0 = my_stages + uint32_t(f_slot) * stage_bytes;
        if constexpr (TMA) {
            if (lane == 0) {
                const uint32_t halves = tile != ntiles - 1 ? 2u : uint32_t(last_rows + 8) / 8u;      // 8-row copies that hold rows of this block
                const uint32_t bar = bars + 8u * uint32_t(f_slot);
                mbar_arrive_expect_tx(bar, rounds * halves * (kSub / 2u));
                const CUtensorMap * m = mat ? mw2p : mwp;
                const int x = f_chunk * int(CB / 2u), y = int(R0) + tile * kTileRows;
                for (uint32_t r = 0; r < rounds; r++) {
                    for (uint32_t hb = 0; hb < halves; hb++) {
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(dst0 + r * kSub + hb * (kSub / 2u)), "l"(m), "r"(x + int(r) * 72), "r"(y + int(hb) * 8), "r"(bar) : "memory");
                    }
                }
            }
        } else if (tile != ntiles - 1) {
            #pragma unroll
            for (int k = 0; k < kMaxPieces; k++) {
                const uint32_t e = tab[k];
                if (e != 0xFFFFFFFFu) {
                    const uint32_t off = e >> 13;
                    cp_async16(dst0 + (e & 0x1FFFu), base + (int32_t(off) - int32_t((lo + off) & 15u)));
                }
            }
        } else {
            #pragma unroll
            for (int k = 0; k < kMaxPieces; k++) {
                const uint32_t e = tab[k];
                if (e != 0xFFFFFFFFu && int((piece_rows[k / 8] >> (4 * (k % 8))) & 15u) <= last_rows) {
                    const uint32_t off = e >> 13;
                    cp_async16(dst0 + (e & 0x1FFFu), base + (int32_t(off) - int32_t((lo + off) & 15u)));
                }
            }
        }
        f_chunk += step_chunk;
        f_tm += step_tm;
        if (f_chunk >= p.nchunks) { f_chunk -= p.nchunks; f_tm++; }
        if (++f_slot == STAGES) f_slot = 0;
    };

    int fetched = 0;
    bool arrived = true;
    if constexpr (TMA) {
        if (lane == 0) {
            for (int s2 = 0; s2 < STAGES; s2++) mbar_init(bars + 8u * s2, 1);
            mbar_init_fence();
        }
        __syncwarp();
    }
    // The first STAGES - 1 stages of weights are asked for at once: they do not depend on the kernel before this one, which may still be running (this
    // kernel is launched early, see launch.cuh). Only then wait for that kernel, and fetch the split input it (or one before it) wrote, as one more group.
    if constexpr (!FUSED) { if (!(p.flags & kFlagLateDependents)) pdl_trigger(); }
    #pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (fetched < my_units) { fetch(); fetched++; }
        cp_async_commit();
    }
    for (int i = threadIdx.x; i < ntiles * nmat * WARPS * kTileRows; i += WARPS * 32) partial[i] = 0.f;
    if constexpr (FUSED) grid_barrier(*grid);      // the phase before this one has written its results, everywhere
    else pdl_wait();
    __shared__ float norm_scale;
    if (p.xq) {
        for (uint32_t i = threadIdx.x; i < uint32_t(nb) * 136u / 16u; i += WARPS * 32) cp_async16(xl + i * 16u, p.xq + size_t(i) * 16);
        cp_async_commit();
        if (warp == 0) {
            // the producer's per-block sums of squares, added in a fixed order (lane l takes entries l, l + 32, ...; then the shuffle tree)
            float ss = 0.f;
            for (int i = lane; i < p.ss_n; i += 32) ss += __ldcg(p.ss_in + i);
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) norm_scale = p.ss_in ? rsqrtf(ss / float(p.cols) + p.eps) : 1.f;
        }
        cp_async_wait<0>();               // the split input has landed (this thread's part), and with it the first stages
    } else {
        // every block normalizes (when asked) and splits the whole input itself, while its first stages are on their way: a 16 KB read from L2 and about
        // forty instructions per 32 elements, instead of a launch of its own and a round trip through device memory
        __shared__ float red[WARPS];
        constexpr int kHeld = 16;              // blocks of the input a warp keeps in registers: inputs of up to 16 x WARPS x 32 elements make one pass
        if (nb <= kHeld * WARPS) {
            // one pass: every load (input and gains) is issued before anything waits, the sum of squares and the split both work from registers
            float v[kHeld], gm[kHeld];
            #pragma unroll
            for (int j = 0; j < kHeld; j++) {
                const int blk = warp + j * WARPS;
                v[j] = blk < nb ? __ldcg(p.x + blk * 32 + lane) : 0.f;
                gm[j] = (p.gamma && blk < nb) ? p.gamma[blk * 32 + lane] : 1.f;
            }
            float inv = 1.f;
            if (p.gamma) {
                float ss = 0.f;
                #pragma unroll
                for (int j = 0; j < kHeld; j++) ss += v[j] * v[j];
                #pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) red[warp] = ss;
                __syncthreads();
                float total = 0.f;
                #pragma unroll
                for (int w = 0; w < WARPS; w++) total += red[w];
                inv = rsqrtf(total / float(p.cols) + p.eps);
            }
            #pragma unroll
            for (int j = 0; j < kHeld; j++) {
                const int blk = warp + j * WARPS;
                if (blk < nb) split_block(p.gamma ? v[j] * inv * gm[j] : v[j], lane, blk, nb, smem);
            }
        } else {
            float inv = 1.f;
            if (p.gamma) {
                float ss = 0.f;
                for (int i = threadIdx.x; i < p.cols; i += WARPS * 32) { const float v = __ldcg(p.x + i); ss += v * v; }
                #pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) red[warp] = ss;
                __syncthreads();
                float total = 0.f;
                #pragma unroll
                for (int w = 0; w < WARPS; w++) total += red[w];
                inv = rsqrtf(total / float(p.cols) + p.eps);
            }
            for (int blk0 = warp; blk0 < nb; blk0 += WARPS * 8) {       // eight loads on their way before the first block is split
                float v[8], gm[8];
                #pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int blk = blk0 + j * WARPS;
                    v[j] = blk < nb ? __ldcg(p.x + blk * 32 + lane) : 0.f;
                    gm[j] = (p.gamma && blk < nb) ? p.gamma[blk * 32 + lane] : 1.f;
                }
                #pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int blk = blk0 + j * WARPS;
                    if (blk < nb) split_block(p.gamma ? v[j] * inv * gm[j] : v[j], lane, blk, nb, smem);
                }
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
    }
    __syncthreads();
    if (K4) {
        // sum of each input block from its digits: lane l holds four bytes of digit l / 8; X = S0 + 128 S1 + 128^2 S2 + 128^3 S3, times the block's factor
        for (int blk = warp; blk < nb; blk += WARPS) {
            const uint32_t w = lds32<0>(xl + uint32_t(blk) * 128u + uint32_t(lane) * 4u);
            int sd = __dp4a(int(w), 0x01010101, 0);
            sd += __shfl_xor_sync(0xffffffffu, sd, 1); sd += __shfl_xor_sync(0xffffffffu, sd, 2); sd += __shfl_xor_sync(0xffffffffu, sd, 4);
            const float s0 = float(__shfl_sync(0xffffffffu, sd, 0)), s1 = float(__shfl_sync(0xffffffffu, sd, 8));
            const float s2 = float(__shfl_sync(0xffffffffu, sd, 16)), s3 = float(__shfl_sync(0xffffffffu, sd, 24));
            if (lane == 0) {
                const float f = ldsf<0>(sxp + uint32_t(blk) * 8u) * 16.f;        // s 2^-26
                const float total = ((s3 * 128.f + s2) * 128.f + s1) * 128.f + s0;
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(sumx + uint32_t(blk) * 4u), "f"(total * f) : "memory");
            }
        }
        __syncthreads();
    }

    const bool first = g < 4;
    const uint32_t b_lane = xl + uint32_t(g >> 2) * 128u + uint32_t(g & 3) * 32u + uint32_t(t) * 8u;
    const uint32_t s_lane = sxp + uint32_t(t >> 1) * 8u + uint32_t(t & 1) * 4u;
    const uint32_t row_lane0 = uint32_t(g) * stride, row_lane1 = uint32_t(g + 8) * stride;
    const uint32_t w_lo = uint32_t(reinterpret_cast<uintptr_t>(p.W)) + uint32_t(R0) * RB, w2_lo = uint32_t(reinterpret_cast<uintptr_t>(p.W2)) + uint32_t(R0) * RB;
    const int npairs = p.cbk / 2;
    float acc0 = 0.f, acc1 = 0.f;
    int acc_tm = u_tm;
    // Adds the lane quad's sums for rows g, g + 8 of (tile, matrix) acc_tm into this warp's slot of the table.
    auto flush = [&]() {
        float s0 = acc0, s1 = acc1;
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if (t == 0) {
            float * dst = partial + (acc_tm * WARPS + warp) * kTileRows;
            dst[g] += s0;
            dst[g + 8] += s1;
        }
        acc0 = 0.f;
        acc1 = 0.f;
    };
    for (int u = 0; u < my_units; u++) {
        if constexpr (TMA) {
            if (arrived) arrived = mbar_wait(bars + 8u * uint32_t(u_slot), uint32_t(u / STAGES) & 1u);      // bounded; after a failure the rest runs on without waiting
        } else {
            cp_async_wait<STAGES - 2>();  // stage u has landed (this lane's pieces) ...
        }
        __syncwarp();                     // ... and every lane's; also: every lane is done reading the slot refilled next
        if (fetched < my_units) { fetch(); fetched++; }
        cp_async_commit();
        if (u_tm != acc_tm) { flush(); acc_tm = u_tm; }
        const int tile = nmat == 2 ? u_tm >> 1 : u_tm;
        // where the rows' bytes start inside their stage rows: the low four address bits of each row's chunk
        const int last = nrows - 1 - tile * kTileRows;
        const uint32_t lo = ((nmat == 2 && (u_tm & 1)) ? w2_lo : w_lo) + uint32_t(tile * kTileRows) * RB + uint32_t(u_chunk) * CB;
        const uint32_t st = my_stages + uint32_t(u_slot) * stage_bytes;
        const uint32_t row0 = TMA ? st + uint32_t(g) * 144u : st + row_lane0 + ((lo + uint32_t(min(g, last)) * RB) & 15u);
        const uint32_t row1 = TMA ? row0 + 8u * 144u : st + row_lane1 + ((lo + uint32_t(min(g + 8, last)) * RB) & 15u);
        constexpr uint32_t kRound = TMA ? kSub : 144u;      // from one round's bytes of a row to the next round's
        uint32_t a0 = row0 + 4u * t, a1 = row1 + 4u * t, d0a = row0 + 18u * (t >> 1), d1a = row1 + 18u * (t >> 1);
        uint32_t ba = b_lane + uint32_t(u_chunk * p.cbk) * 128u, sa = s_lane + uint32_t(u_chunk * p.cbk) * 8u;
        int pr = 0;
        if constexpr (K4) {
            // one super-block (four pairs) per round; its header words are read once per row
            uint32_t suma = sumx + uint32_t(u_chunk * p.cbk) * 4u + uint32_t(t >> 1) * 4u, h0a = row0, h1a = row1;
            #pragma unroll 1
            for (; pr + 4 <= npairs; pr += 4) {
                const uint4 h0 = lds128(h0a), h1 = lds128(h1a);
                pair_step_k4<0>(a0, a1, h0, h1, ba, sa, suma, first, uint32_t(t >> 1), (t & 1) == 0, acc0, acc1);
                pair_step_k4<1>(a0, a1, h0, h1, ba, sa, suma, first, uint32_t(t >> 1), (t & 1) == 0, acc0, acc1);
                pair_step_k4<2>(a0, a1, h0, h1, ba, sa, suma, first, uint32_t(t >> 1), (t & 1) == 0, acc0, acc1);
                pair_step_k4<3>(a0, a1, h0, h1, ba, sa, suma, first, uint32_t(t >> 1), (t & 1) == 0, acc0, acc1);
                a0 += kRound; a1 += kRound; h0a += kRound; h1a += kRound; ba += 1024; sa += 64; suma += 32;
            }
        } else {
            #pragma unroll 1
            for (; pr + 4 <= npairs; pr += 4) {
                pair_step<0>(a0, a1, d0a, d1a, ba, sa, first, acc0, acc1);
                pair_step<1>(a0, a1, d0a, d1a, ba, sa, first, acc0, acc1);
                pair_step<2>(a0, a1, d0a, d1a, ba, sa, first, acc0, acc1);
                pair_step<3>(a0, a1, d0a, d1a, ba, sa, first, acc0, acc1);
                a0 += kRound; a1 += kRound; d0a += kRound; d1a += kRound; ba += 1024; sa += 64;
            }
            #pragma unroll 1
            for (; pr < npairs; pr++) {
                pair_step<0>(a0, a1, d0a, d1a, ba, sa, first, acc0, acc1);
                a0 += 36; a1 += 36; d0a += 36; d1a += 36; ba += 256; sa += 16;
            }
        }
        u_chunk += step_chunk;
        u_tm += step_tm;
        if (u_chunk >= p.nchunks) { u_chunk -= p.nchunks; u_tm++; }
        if (++u_slot == STAGES) u_slot = 0;
    }
    cp_async_wait<0>();
    if (TMA && !arrived && lane == 0 && p.error) *p.error = 4;
    if (my_units > 0) flush();
    __syncthreads();
    // the rows of this block: the warps' shares summed in warp order, then the epilogue
    const float in_scale = (p.xq && p.ss_in) ? norm_scale : 1.f;      // written before the barrier above
    float sq = 0.f;
    for (int r = threadIdx.x; r < nrows; r += WARPS * 32) {
        const float * src = partial + size_t(r / kTileRows) * nmat * WARPS * kTileRows + (r % kTileRows);
        float s = 0.f, s2 = 0.f;
        #pragma unroll
        for (int w = 0; w < WARPS; w++) s += src[w * kTileRows];
        s *= in_scale;
        if (nmat == 2) {
            #pragma unroll
            for (int w = 0; w < WARPS; w++) s2 += src[(WARPS + w) * kTileRows];
            s = s / (1.f + expf(-s)) * (s2 * in_scale);
        }
        const int64_t row = R0 + r;
        if (p.flags & kFlagBias) s += p.bias[row];
        const float out = (p.flags & kFlagAccumulate) ? accumulate_base(__ldcg(p.y + row), p.flags) + s : s;
        p.y[row] = out;
        sq += out * out;
    }
    if (p.ss_out) {
        // this block's sum of squares: lanes, then warps, in a fixed order
        __shared__ float sq_warp[WARPS];
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) sq_warp[warp] = sq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.f;
            #pragma unroll
            for (int w = 0; w < WARPS; w++) total += sq_warp[w];
            p.ss_out[block_index] = total;
        }
    }
    if constexpr (FUSED) {
        __syncwarp();
        if (TMA && lane == 0) for (int s2 = 0; s2 < STAGES; s2++) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bars + 8u * s2) : "memory");
    }
    if (p.xq_out && nrows > 0) {
        __threadfence();              // this block's rows are visible before they are counted
        __syncthreads();
        const int64_t R1 = R0 + nrows;
        for (int64_t grp = R0 / 32 + warp; grp * 32 < R1; grp += WARPS) {
            const int mine = int(min(R1, grp * 32 + 32) - max(R0, grp * 32));
            int done = 0;
            if (lane == 0) {
                done = atomicAdd(p.out_counters + grp, mine) + mine == 32;
                if (done) p.out_counters[grp] = 0;      // complete: nobody adds to it again in this launch
            }
            if (__shfl_sync(0xffffffffu, done, 0)) {
                __threadfence();
                const float v = __ldcg(p.y + grp * 32 + lane);
                split_block(p.gamma_out ? v * p.gamma_out[grp * 32 + lane] : v, lane, int(grp), int(p.rows / 32), p.xq_out);
            }
        }
    }
}

template <int WARPS, int STAGES, bool K4, bool TMA>
__global__ void __launch_bounds__(WARPS * 32, 1) k_gemv_q4_0(const __grid_constant__ CUtensorMap mw, const __grid_constant__ CUtensorMap mw2, const GemvQ40Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    gemv_q4_0_body<WARPS, STAGES, K4, TMA, false>(&mw, &mw2, p, smem, int(blockIdx.x), int(gridDim.x), nullptr);
}

// ---- the fused decode step: every projection and every attention of all layers in ONE cooperative launch ----
// A decode step of one sequence is a chain of ~5 dependent kernels per layer, each a few microseconds long; between two of them the GPU drains, launches,
// warms up and refills its copy pipelines, which costs about as much as the kernels' own streaming. Here one block per SM stays resident for the whole
// step and walks through the phases (qkv projection, attention, attn_output, gate / up, ffn_down of every layer); where a launch boundary stood there is
// a grid-wide barrier, and every projection asks for its first weight stages BEFORE it waits at that barrier, so the weights keep arriving while the
// previous phase's last blocks finish. The phases run the same device code as the kernels of their own (gemv_q4_0_body, attention_decode_body).
constexpr int kFusedWarps = 16, kFusedStages = 2, kFusedThreads = kFusedWarps * 32;

struct FusedPhase {
    int32_t kind;              // 0: projection, 1: attention
    int32_t k4;                // projection: q4_K rows
    int32_t map_w, map_w2;     // projection: indices into the tensor map array
    GemvQ40Params g;
    attn_decode::AttnDecodeParams a;
};
struct FusedArgs {
    const FusedPhase * phases;
    const CUtensorMap * maps;
    int32_t n_phases;
    unsigned * barrier;        // two words 128 bytes apart, zeroed by the step's first kernel
    int32_t * error;
};

template <int D, int GP>
__global__ void __launch_bounds__(kFusedThreads, 1) k_decode_layers(const FusedArgs fa) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(16) FusedPhase ph[2];
    static_assert(sizeof(FusedPhase) % 4 == 0, "phases are copied word by word");
    constexpr int kWords = int(sizeof(FusedPhase) / 4);
    GridBarrier gb{fa.barrier, fa.error, gridDim.x};
    const int block = int(blockIdx.x), n_blocks = int(gridDim.x);
    auto stage_phase = [&](int i) {      // phase i's description into its shared-memory slot (a handful of words per thread)
        const uint32_t * src = reinterpret_cast<const uint32_t *>(fa.phases + i);
        uint32_t * dst = reinterpret_cast<uint32_t *>(&ph[i & 1]);
        for (int w = threadIdx.x; w < kWords; w += kFusedThreads) dst[w] = __ldg(src + w);
    };
    stage_phase(0);
    __syncthreads();
    for (int i = 0; i < fa.n_phases; i++) {
        if (i + 1 < fa.n_phases) stage_phase(i + 1);      // nobody reads that slot during this phase; the barrier at the phase's end publishes it
        const FusedPhase & cur = ph[i & 1];
        if (cur.kind == 0) {
            if (cur.k4) gemv_q4_0_body<kFusedWarps, kFusedStages, true, true, true>(fa.maps + cur.map_w, fa.maps + cur.map_w2, cur.g, smem, block, n_blocks, &gb);
            else gemv_q4_0_body<kFusedWarps, kFusedStages, false, true, true>(fa.maps + cur.map_w, fa.maps + cur.map_w2, cur.g, smem, block, n_blocks, &gb);
        } else {
            grid_barrier(gb);                              // q, k and v of this layer are complete
            const int nkv = cur.a.s.n_head_kv;
            if (threadIdx.x < attn_decode::kThreads && block < nkv * cur.a.splits) {
                attn_decode::attention_decode_body<D, GP, false>(cur.a, block % nkv, block / nkv, cur.a.splits, 0, smem);
            }
        }
        __syncthreads();                                   // the phase's shared memory is free, the next phase's description is in place
    }
}

constexpr size_t kSmemLimit = 224 * 1024;
constexpr int kMaxTilesPerBlock = kMaxTilesPerBlockDev;        // the table of per-warp sums holds this many 16-row tiles of two matrices
constexpr size_t partial_bytes(int warps, int nmat) { return size_t(kMaxTilesPerBlock) * nmat * warps * kTileRows * sizeof(float); }

struct Plan { int cbk, nchunks, stride, stages, warps; size_t smem; bool ok; };

// Chunks of an even number of blocks that divides the row; the row stride in a stage is an odd multiple of 16 bytes so that the 8 rows of a fragment fall
// on different banks.
constexpr int kMaxStages = 6;
// tma: stages of 16 rows x chunk with one mbarrier per stage and warp; chunks of 8 or 16 blocks, at most 4 stages.
Plan plan_for(int64_t cols, int nmat, bool k4, bool tma = false) {      // k4: q4_K rows, chunks of whole 256-element super-blocks (8 or 16 blocks)
    Plan best{};
    const int nb = int(cols / 32);
    if (cols % (k4 ? 256 : 64) != 0 || nb < 2) return best;
    const size_t fixed = (size_t(nb) * 140 + 127) & ~size_t(127);
    int64_t best_score = -1;
    for (int warps : {16, 8}) {
        for (int cbk = 2; cbk <= std::min(nb, 16); cbk += 2) {
            if (nb % cbk || ((k4 || tma) && cbk % 8)) continue;
            int stride = (cbk * kBlockBytes + 32 + 15) / 16 * 16;
            if (stride % 32 != 16) stride += 16;
            if ((cbk * kBlockBytes + 30) / 16 * kTileRows > kMaxPieces * 32 || kTileRows * stride >= (1 << 13)) continue;
            int stages = 0;
            const size_t stage = tma ? size_t(kTileRows) * cbk * kBlockBytes : size_t(kTileRows) * stride;
            for (int st = tma ? 4 : kMaxStages; st >= 2; st--) {
                if (fixed + size_t(warps) * st * stage + partial_bytes(warps, nmat) + (tma ? size_t(warps) * st * 8 : 0) <= kSmemLimit) { stages = st; break; }
            }
            if (!stages) continue;
            // Measured on B200 (8B shapes, back-to-back launches over distinct matrices): the kernel is bound by instruction issue and shared-memory
            // bandwidth more than by the bytes in flight, so the longest chunk (fewest per-unit fixed costs) wins, then 16 warps over 8, then stages.
            // (Two blocks of 8 warps per SM with half the ring each, so that one block's prologue and epilogue overlap the other's streaming, measured slower:
            // 22.0 against 20.9 us on the 8B gate / up shape, 1.92 against 1.83 ms per decode step.)
            const int64_t score = int64_t(cbk) * 1000 + (warps == 16 ? 100 : 0) + stages;
            if (score > best_score) {
                best_score = score;
                best = Plan{cbk, nb / cbk, stride, stages, warps, fixed + size_t(warps) * stages * stage + partial_bytes(warps, nmat) + (tma ? size_t(warps) * stages * 8 : 0), true};
            }
        }
    }
    return best;
}

struct Maps { CUtensorMap w, w2; };

// How a launch deals the rows to its blocks: one block per SM; more (whole multiples) only when a block's share would exceed the table of
// kMaxTilesPerBlock tiles. Rows go in units of 8 with tensor copies, else singly.
struct RowSplit { int grid, rows_q, rows_r, row_unit; };
RowSplit row_split(int64_t rows, bool tma) {
    const int sms = sm_count();
    const int64_t max_rows = int64_t(kMaxTilesPerBlock) * kTileRows;
    const int64_t waves = (rows + sms * max_rows - 1) / (sms * max_rows);
    const int row_unit = tma ? 8 : 1;
    const int64_t units = (rows + row_unit - 1) / row_unit;
    const int grid = int(std::min<int64_t>(sms * waves, units));
    return RowSplit{grid, int(units / grid), int(units % grid), row_unit};
}

bool takes_tma(int64_t rows, int64_t cols, int nmat, bool q4_k) {
    static const bool tma_off = [] { const char * e = getenv("DOOMS_GEMV_TMA"); return e && *e == '0'; }();
    return !tma_off && cols % 256 == 0 && rows < (int64_t(1) << 31) && plan_for(cols, nmat, q4_k, true).ok;
}

template <int WARPS, int STAGES, bool K4, bool TMA>
cudaError_t launch_with(const GemvQ40Params & p, const Maps & maps, size_t smem, unsigned grid, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_gemv_q4_0<WARPS, STAGES, K4, TMA>, int(kSmemLimit), configured); e != cudaSuccess) return e;
    static const bool early = [] { const char * e = getenv("DOOMS_PDL_GEMV"); return !(e && *e == '0'); }();
    return launch_pdl_if(early, k_gemv_q4_0<WARPS, STAGES, K4, TMA>, dim3(grid), dim3(WARPS * 32), smem, stream, maps.w, maps.w2, p);
}

template <int WARPS, bool K4>
cudaError_t launch_stages(const GemvQ40Params & p, const Maps & maps, bool tma, const Plan & pl, unsigned grid, cudaStream_t stream) {
    if (tma) {
        switch (pl.stages) {
            case 4: return launch_with<WARPS, 4, K4, true>(p, maps, pl.smem, grid, stream);
            case 3: return launch_with<WARPS, 3, K4, true>(p, maps, pl.smem, grid, stream);
            default: return launch_with<WARPS, 2, K4, true>(p, maps, pl.smem, grid, stream);
        }
    }
    switch (pl.stages) {
        case 6: return launch_with<WARPS, 6, K4, false>(p, maps, pl.smem, grid, stream);
        case 5: return launch_with<WARPS, 5, K4, false>(p, maps, pl.smem, grid, stream);
        case 4: return launch_with<WARPS, 4, K4, false>(p, maps, pl.smem, grid, stream);
        case 3: return launch_with<WARPS, 3, K4, false>(p, maps, pl.smem, grid, stream);
        default: return launch_with<WARPS, 2, K4, false>(p, maps, pl.smem, grid, stream);
    }
}

}  // namespace

bool gemv_q4_0_supported(const void * W, int64_t rows, int64_t cols) {
    return rows >= 1 && (reinterpret_cast<uintptr_t>(W) & 15u) == 0 && plan_for(cols, 1, false).ok;
}
bool gemv_q4_k_supported(const void * W, int64_t rows, int64_t cols) {
    return rows >= 1 && (reinterpret_cast<uintptr_t>(W) & 15u) == 0 && plan_for(cols, 2, true).ok;
}

int gemv_q4_0_blocks(int64_t rows, int64_t cols, bool gate_up, bool q4_k) {
    return row_split(rows, takes_tma(rows, cols, gate_up ? 2 : 1, q4_k)).grid;
}

size_t quantized_x_bytes(int64_t cols) { return size_t(cols / 32) * 136; }      // the kernel adds 4 bytes per block of its own in shared memory

cudaError_t launch_quantize_x(const float * x, int64_t cols, void * xq, cudaStream_t stream) {
    const int nb = int(cols / 32);
    return launch_pdl(k_quantize_x, dim3((nb + 7) / 8), dim3(256), 0, stream, x, nb, static_cast<uint8_t *>(xq));
}

cudaError_t launch_gemv_q4_0(const void * W, const void * W2, const void * xq, const float * x, const float * gamma, float eps, float * y, const float * bias,
                             int64_t rows, int64_t cols, uint32_t flags, bool q4_k, cudaStream_t stream, void * xq_out, int * out_counters, int32_t * error,
                             const GemvNormLink * link) {
    if (xq_out && (!out_counters || rows % 32 != 0)) return cudaErrorInvalidValue;
    if (link && ((link->gamma_out || link->ss_out) && !xq_out)) return cudaErrorInvalidValue;
    if (link && link->ss_in && !xq) return cudaErrorInvalidValue;
    // tensor copies when rows and chunks are whole 16-byte units (cols a multiple of 256) and the driver hands out the encoder; per-lane copies otherwise
    Maps maps{};
    bool tma = takes_tma(rows, cols, W2 ? 2 : 1, q4_k);
    if (tma) {
        const Plan tp = plan_for(cols, W2 ? 2 : 1, q4_k, true);
        const int64_t rb = cols / 32 * kBlockBytes;
        (void)tp;
        tma = make_rows_map(reinterpret_cast<TensorMap *>(&maps.w), W, rows, rb, 8 * kBlockBytes, 8) == cudaSuccess &&
              (!W2 || make_rows_map(reinterpret_cast<TensorMap *>(&maps.w2), W2, rows, rb, 8 * kBlockBytes, 8) == cudaSuccess);
    }
    const Plan pl = plan_for(cols, W2 ? 2 : 1, q4_k, tma);
    if (!pl.ok) return cudaErrorInvalidValue;
    GemvQ40Params p{static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(W2), static_cast<const uint8_t *>(xq), x, gamma, eps, static_cast<uint8_t *>(xq_out), out_counters,
                    link ? link->gamma_out : nullptr, link ? link->ss_out : nullptr, link ? link->ss_in : nullptr, link ? link->ss_n : 0, error, y, bias, rows, int(cols), flags,
                    pl.cbk, pl.nchunks, pl.stride, 0, 0, 0, 1, 0u, 0u};
    if (!xq && !x) return cudaErrorInvalidValue;
    // pieces per row: exactly the chunk when rows and chunks start on 16-byte boundaries, otherwise the widest aligned cover
    const int64_t row_bytes = cols / 32 * kBlockBytes;
    const int chunk_bytes = pl.cbk * kBlockBytes;
    p.upr = (row_bytes % 16 == 0 && chunk_bytes % 16 == 0) ? chunk_bytes / 16 : (chunk_bytes + 30) / 16;
    const RowSplit rs = row_split(rows, tma);
    const unsigned grid = unsigned(rs.grid);
    p.row_unit = rs.row_unit;
    p.rows_q = rs.rows_q;
    p.rows_r = rs.rows_r;
    p.inv_upr = 65536u / uint32_t(p.upr) + 1u;
    p.inv_nchunks = 65536u / uint32_t(pl.nchunks) + 1u;
    if (q4_k) return pl.warps == 16 ? launch_stages<16, true>(p, maps, tma, pl, grid, stream) : launch_stages<8, true>(p, maps, tma, pl, grid, stream);
    return pl.warps == 16 ? launch_stages<16, false>(p, maps, tma, pl, grid, stream) : launch_stages<8, false>(p, maps, tma, pl, grid, stream);
}

// ---- host side of the fused decode step ----
struct DecodeLayersPlan {
    FusedPhase * phases = nullptr;
    CUtensorMap * maps = nullptr;
    unsigned * barrier = nullptr;
    int n_phases = 0, blocks = 0, head_dim = 0, gp = 0;
    size_t smem = 0;
    int32_t * error = nullptr;
};

namespace {

// One projection's kernel arguments as the fused kernel runs it: tensor copies, kFusedWarps warps, kFusedStages stages, the rows dealt over `blocks`.
bool fused_projection(const FusedMatrix & m, const void * w2, int blocks, GemvQ40Params * out, size_t * smem) {
    const int nmat = w2 ? 2 : 1;
    if (!m.w || (reinterpret_cast<uintptr_t>(m.w) & 15u) || (w2 && (reinterpret_cast<uintptr_t>(w2) & 15u))) return false;
    if (!takes_tma(m.rows, m.cols, nmat, m.q4_k)) return false;
    const Plan pl = plan_for(m.cols, nmat, m.q4_k, true);
    if (!pl.ok || pl.warps != kFusedWarps || pl.stages != kFusedStages) return false;
    const int64_t units = (m.rows + 7) / 8;
    const int64_t per_block_rows = ((units + blocks - 1) / blocks) * 8;
    if (per_block_rows > int64_t(kMaxTilesPerBlock) * kTileRows) return false;      // the table of per-warp sums would not hold the block's tiles
    GemvQ40Params p{};
    p.W = static_cast<const uint8_t *>(m.w);
    p.W2 = static_cast<const uint8_t *>(w2);
    p.rows = m.rows;
    p.cols = int(m.cols);
    p.cbk = pl.cbk; p.nchunks = pl.nchunks; p.stride = pl.stride;
    p.upr = pl.cbk * kBlockBytes / 16;
    p.row_unit = 8;
    p.rows_q = int(units / blocks);
    p.rows_r = int(units % blocks);
    p.inv_upr = 65536u / uint32_t(p.upr) + 1u;
    p.inv_nchunks = 65536u / uint32_t(pl.nchunks) + 1u;
    *out = p;
    *smem = std::max(*smem, pl.smem);
    return true;
}

template <int D>
cudaError_t launch_fused_group(const DecodeLayersPlan & pl, const FusedArgs & fa, cudaStream_t stream) {
    void * args[] = {const_cast<FusedArgs *>(&fa)};
    auto go = [&](auto kernel) -> cudaError_t {
        static std::atomic<uint64_t> configured{0};
        if (const cudaError_t e = allow_dynamic_smem(kernel, int(kSmemLimit), configured); e != cudaSuccess) return e;
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), dim3(unsigned(pl.blocks)), dim3(kFusedThreads), args, pl.smem, stream);
    };
    switch (pl.gp) {
        case 1: return go(k_decode_layers<D, 1>);
        case 2: return go(k_decode_layers<D, 2>);
        case 4: return go(k_decode_layers<D, 4>);
        default: return go(k_decode_layers<D, 8>);
    }
}

}  // namespace

cudaError_t decode_layers_create(const FusedLayer * layers, int n_layers, const FusedBuffers & b, DecodeLayersPlan ** out) {
    *out = nullptr;
    int dev = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    const AttnShape & s = b.shape;
    if (!coop || n_layers < 1 || !attention_gqa_supported(s) || s.head_dim % 32 != 0) return cudaErrorNotSupported;
    const int blocks = sm_count();
    const int G = s.n_head / s.n_head_kv, gp = G == 1 ? 1 : G == 2 ? 2 : G <= 4 ? 4 : 8;
    const int splits = std::min(b.max_splits, blocks / s.n_head_kv);
    if (splits < 1) return cudaErrorNotSupported;
    std::vector<FusedPhase> phases;
    std::vector<CUtensorMap> maps;
    size_t smem = s.head_dim == 64 ? attn_decode::attention_decode_smem_bytes<64, 8>() : attn_decode::attention_decode_smem_bytes<128, 8>();
    auto add_map = [&](const FusedMatrix & m, const void * w) -> int {
        CUtensorMap tm;
        if (make_rows_map(reinterpret_cast<TensorMap *>(&tm), w, m.rows, m.cols / 32 * kBlockBytes, 8 * kBlockBytes, 8) != cudaSuccess) return -1;
        maps.push_back(tm);
        return int(maps.size()) - 1;
    };
    for (int l = 0; l < n_layers; l++) {
        const FusedLayer & L = layers[l];
        if (L.ffn_gate.rows != L.ffn_up.rows || L.ffn_gate.cols != L.ffn_up.cols || L.ffn_gate.q4_k != L.ffn_up.q4_k) return cudaErrorNotSupported;
        if (L.attn_output.rows % 32 != 0 || L.ffn_gate.rows % 32 != 0 || L.ffn_down.rows % 32 != 0 || !L.next_norm) return cudaErrorNotSupported;
        FusedPhase q{}, at{}, o{}, gu{}, dn{};
        // qkv: the first layer normalizes and splits x itself; the others take what the ffn_down before them prepared
        if (!fused_projection(L.qkv, nullptr, blocks, &q.g, &smem)) return cudaErrorNotSupported;
        q.k4 = L.qkv.q4_k;
        q.map_w = q.map_w2 = add_map(L.qkv, L.qkv.w);
        q.g.eps = b.eps;
        if (l == 0) { q.g.x = b.x; q.g.gamma = L.attn_norm; }
        else { q.g.xq = static_cast<const uint8_t *>(b.xq2); q.g.ss_in = b.norm_ss; q.g.ss_n = blocks; }
        q.g.y = b.qkv;
        q.g.bias = L.qkv_bias;
        q.g.flags = L.qkv_bias ? kFlagBias : 0u;
        q.g.error = b.error;
        // attention: rotation, cache write, ranges, merge; leaves the row split for attn_output
        at.kind = 1;
        at.a = attn_decode::AttnDecodeParams{b.qkv, static_cast<__half *>(L.kc), static_cast<__half *>(L.vc), b.part, b.state, b.inv_freq, 0, splits, s, b.attn_counters, b.attn,
                                             static_cast<uint8_t *>(b.xq), static_cast<const float2 *>(b.rope_cs), nullptr, nullptr, 0, 0, 0, nullptr};
        // attn_output: x += W attn; leaves x * (ffn_norm's gains) split, and the sums of squares, for gate / up
        if (!fused_projection(L.attn_output, nullptr, blocks, &o.g, &smem)) return cudaErrorNotSupported;
        o.k4 = L.attn_output.q4_k;
        o.map_w = o.map_w2 = add_map(L.attn_output, L.attn_output.w);
        o.g.eps = b.eps;
        o.g.xq = static_cast<const uint8_t *>(b.xq);
        o.g.y = b.x;
        o.g.flags = kFlagAccumulate;
        o.g.xq_out = static_cast<uint8_t *>(b.xq2); o.g.out_counters = b.norm_counters; o.g.gamma_out = L.ffn_norm; o.g.ss_out = b.norm_ss;
        o.g.error = b.error;
        // gate / up: h = silu(Wg xn) * (Wu xn); leaves h split for ffn_down
        if (!fused_projection(L.ffn_gate, L.ffn_up.w, blocks, &gu.g, &smem)) return cudaErrorNotSupported;
        gu.k4 = L.ffn_gate.q4_k;
        gu.map_w = add_map(L.ffn_gate, L.ffn_gate.w);
        gu.map_w2 = add_map(L.ffn_up, L.ffn_up.w);
        gu.g.eps = b.eps;
        gu.g.xq = static_cast<const uint8_t *>(b.xq2); gu.g.ss_in = b.norm_ss; gu.g.ss_n = blocks;
        gu.g.y = b.h;
        gu.g.xq_out = static_cast<uint8_t *>(b.xq); gu.g.out_counters = b.split_counters;
        gu.g.error = b.error;
        // ffn_down: x += W h; prepares the next norm (the next layer's attn_norm, or the output norm)
        if (!fused_projection(L.ffn_down, nullptr, blocks, &dn.g, &smem)) return cudaErrorNotSupported;
        dn.k4 = L.ffn_down.q4_k;
        dn.map_w = dn.map_w2 = add_map(L.ffn_down, L.ffn_down.w);
        dn.g.eps = b.eps;
        dn.g.xq = static_cast<const uint8_t *>(b.xq);
        dn.g.y = b.x;
        dn.g.flags = kFlagAccumulate;
        dn.g.xq_out = static_cast<uint8_t *>(b.xq2); dn.g.out_counters = b.norm_counters; dn.g.gamma_out = L.next_norm; dn.g.ss_out = b.norm_ss;
        dn.g.error = b.error;
        for (const FusedPhase * f : {&q, &o, &gu, &dn}) if (f->map_w < 0 || f->map_w2 < 0) return cudaErrorNotSupported;
        phases.insert(phases.end(), {q, at, o, gu, dn});
    }
    if (smem > kSmemLimit) return cudaErrorNotSupported;
    auto plan = std::make_unique<DecodeLayersPlan>();
    plan->n_phases = int(phases.size());
    plan->blocks = blocks;
    plan->head_dim = s.head_dim;
    plan->gp = gp;
    plan->smem = smem;
    plan->error = b.error;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&plan->phases), phases.size() * sizeof(FusedPhase));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&plan->maps), maps.size() * sizeof(CUtensorMap));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&plan->barrier), 256);
    if (e == cudaSuccess) e = cudaMemcpy(plan->phases, phases.data(), phases.size() * sizeof(FusedPhase), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(plan->maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(plan->barrier, 0, 256);
    if (e != cudaSuccess) { decode_layers_destroy(plan.release()); return e; }
    *out = plan.release();
    return cudaSuccess;
}

void decode_layers_destroy(DecodeLayersPlan * plan) {
    if (!plan) return;
    for (void * p : {(void *)plan->phases, (void *)plan->maps, (void *)plan->barrier}) if (p) cudaFree(p);
    delete plan;
}

int decode_layers_blocks(const DecodeLayersPlan * plan) { return plan->blocks; }
unsigned * decode_layers_barrier(const DecodeLayersPlan * plan) { return plan->barrier; }

cudaError_t launch_decode_layers(const DecodeLayersPlan * plan, cudaStream_t stream) {
    const FusedArgs fa{plan->phases, plan->maps, plan->n_phases, plan->barrier, plan->error};
    return plan->head_dim == 64 ? launch_fused_group<64>(*plan, fa, stream) : launch_fused_group<128>(*plan, fa, stream);
}

}  // namespace cuda
}  // namespace dooms
