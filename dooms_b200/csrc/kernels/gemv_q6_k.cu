// Decode GEMV for q6_K rows on the tensor cores' int8 path: y (+)= W x (+ bias), replacing matvec1q<Q6_K> (src/backend/metal/llama_kernels.h:1197-1230)
// with Q6_K::elem (llama_kernels.h:1145-1154): element i of a 256-element super-block is d * scales[i / 16] * (q - 32), q = the low nibble from ql and
// two high bits from qh. On the CUDA cores rebuilding q and multiplying in f32 costs ~6 instructions per weight and bounds the kernel at a sixth of the
// memory rate (gemv_blocks.cu). Here:
//   * the input vector arrives split as for the q4_0 kernel (xsplit.cuh: per 32-element block a power-of-two scale and four base-128 int8 digits);
//   * one m16n8k32 MMA takes 32 consecutive elements of 16 rows; its 8 columns are (16-element sub-block, digit): column c carries digit c % 4 of the
//     input's first 16 elements (c < 4) or last 16 (c >= 4) and zeros in the other half, so every (row, sub-block, digit) sum comes out on its own and can
//     take the sub-block's scale;
//   * the weights go in as two parts that add up to q - 32: the low nibbles, unsigned (0..15), and the high bit pairs shifted into place with the
//     offset folded in, signed (-32, -16, 0, 16): two MMAs into the same accumulator, a few logic operations per register instead of assembling q;
//   * rows stream through per-warp rings of shared-memory stages as they lie in the file (210-byte super-blocks at 2-byte alignment: 16-byte asynchronous
//     copies of the aligned cover; words that end up 2 bytes off a 4-byte boundary are read as two aligned words and a funnel shift), and the input's
//     digits and factors for a unit's super-blocks travel with the unit's rows (1088 bytes per super-block from L2), so that shared memory holds rings
//     for 16 warps whatever the row length.
// Integer sums are exact; the only rounding is that of the f32 scale factors and of the f32 accumulation over sub-blocks, as in the q4_0 kernel.
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kTileRows = 16, kBB = 210, kMaxPieces = 16, kMaxTilesPerBlock = 8;
constexpr size_t kSmemLimit = 224 * 1024;

struct GemvQ6kParams {
    const uint8_t * W;
    const uint8_t * xq;     // the split input: cols / 32 x 128 digit bytes, then cols / 32 x 2 floats
    float * y;
    const float * bias;
    int cols;
    uint32_t flags;
    int cbk, nchunks;       // super-blocks per chunk, chunks per row
    int stride, upr;        // bytes between the rows of a stage; 16-byte pieces copied per row
    int rows_q, rows_r;     // block b has rows_q + (b < rows_r) rows starting at b rows_q + min(b, rows_r)
    uint32_t inv_upr, inv_nchunks;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// The 32-bit word at a shared-memory byte address that is a multiple of 2: the two aligned words around it and a funnel shift.
// (Both loads always: the rows of a fragment differ in alignment, and a branch would split the warp.)
__device__ __forceinline__ uint32_t word_at(uint32_t addr, uint32_t shift) {      // shift = 16 when addr is 2 past a word boundary, else 0
    const uint32_t a = addr & ~3u;
    return __funnelshift_r(lds_u32(a), lds_u32(a + 4u), shift);
}

template <int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1) k_gemv_q6_k(const GemvQ6kParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const int nb32 = p.cols / 32;
    const uint32_t RB = uint32_t(p.cols / 256) * kBB;
    const uint32_t CB = uint32_t(p.cbk) * kBB;

    const int nrows = p.rows_q + (int(blockIdx.x) < p.rows_r ? 1 : 0);
    const int64_t R0 = int64_t(blockIdx.x) * p.rows_q + min(int(blockIdx.x), p.rows_r);
    const int ntiles = (nrows + kTileRows - 1) / kTileRows;
    const int total_units = ntiles * p.nchunks;
    const int my_units = warp < total_units ? (total_units - warp - 1) / WARPS + 1 : 0;

    // shared memory: the warps' stages (16 rows, then the digits of the chunk's input blocks, then their factors), the table of the warps' sums
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t stride = uint32_t(p.stride);
    const uint32_t rows_bytes = uint32_t(kTileRows) * stride;
    const uint32_t x_bytes = uint32_t(p.cbk) * 8u * 136u;             // 8 blocks of 32 elements per super-block: 128 digit bytes and 2 floats each
    const uint32_t stage_bytes = rows_bytes + x_bytes;
    const uint32_t stages_off = 0u;
    const uint32_t my_stages = smem_base + stages_off + uint32_t(warp) * STAGES * stage_bytes;
    float * partial = reinterpret_cast<float *>(smem + stages_off + size_t(WARPS) * STAGES * stage_bytes);      // [tile][warp][16]

    const int step_tile = int((uint32_t(WARPS) * p.inv_nchunks) >> 16), step_chunk = WARPS - step_tile * p.nchunks;
    int f_tile = int((uint32_t(warp) * p.inv_nchunks) >> 16), f_chunk = warp - f_tile * p.nchunks, f_slot = 0;      // the unit being fetched
    int u_tile = f_tile, u_chunk = f_chunk, u_slot = 0;                                                               // the unit being used

    // which (row, piece) of a stage this lane copies: packed (source offset from the tile's first row << 13 | offset in the stage), and the rows as 4-bit fields
    uint32_t tab[kMaxPieces], piece_rows[2] = {0u, 0u};
    #pragma unroll
    for (int k = 0; k < kMaxPieces; k++) {
        const uint32_t j = uint32_t(lane) + 32u * k;
        const uint32_t row = (j * p.inv_upr) >> 16, col = j - row * uint32_t(p.upr);
        tab[k] = row < uint32_t(kTileRows) ? ((row * RB + col * 16u) << 13) | (row * stride + col * 16u) : 0xFFFFFFFFu;
        piece_rows[k / 8] |= (row & 15u) << (4 * (k % 8));
    }
    const int last_rows = nrows - 1 - (ntiles - 1) * kTileRows;
    // the input's part of a unit: the digits of its 8 cbk blocks (contiguous in xq), then their factors
    auto fetch_x = [&](int chunk, int slot) {
        const uint32_t dst = my_stages + uint32_t(slot) * stage_bytes + rows_bytes;
        const uint32_t blk0 = uint32_t(chunk * p.cbk) * 8u, n_digit = uint32_t(p.cbk) * 64u, n_all = n_digit + uint32_t(p.cbk) * 4u;
        for (uint32_t i = lane; i < n_all; i += 32u) {
            const uint8_t * src = i < n_digit ? p.xq + size_t(blk0) * 128 + size_t(i) * 16 : p.xq + size_t(nb32) * 128 + size_t(blk0) * 8 + size_t(i - n_digit) * 16;
            cp_async16(dst + i * 16u, src);
        }
    };
    auto fetch = [&](bool with_x) {
        if (with_x) fetch_x(f_chunk, f_slot);
        const uint8_t * base = p.W + (R0 + f_tile * kTileRows) * int64_t(RB) + uint32_t(f_chunk) * CB;
        const uint32_t lo = uint32_t(reinterpret_cast<uintptr_t>(base));
        const uint32_t dst0 = my_stages + uint32_t(f_slot) * stage_bytes;
        const int limit = f_tile != ntiles - 1 ? kTileRows : last_rows;
        #pragma unroll
        for (int k = 0; k < kMaxPieces; k++) {
            const uint32_t e = tab[k];
            if (e != 0xFFFFFFFFu && int((piece_rows[k / 8] >> (4 * (k % 8))) & 15u) <= limit) {
                const uint32_t off = e >> 13;
                cp_async16(dst0 + (e & 0x1FFFu), base + (int32_t(off) - int32_t((lo + off) & 15u)));
            }
        }
        f_chunk += step_chunk;
        f_tile += step_tile;
        if (f_chunk >= p.nchunks) { f_chunk -= p.nchunks; f_tile++; }
        if (++f_slot == STAGES) f_slot = 0;
    };

    // The rows of the first STAGES - 1 units are asked for before the wait for the kernel that wrote the input; the input's parts of those units follow it.
    int fetched = 0;
    if (!(p.flags & kFlagLateDependents)) pdl_trigger();
    int first_chunk[STAGES - 1];
    #pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        first_chunk[s] = f_chunk;
        if (fetched < my_units) { fetch(false); fetched++; }
    }
    for (int i = threadIdx.x; i < ntiles * WARPS * kTileRows; i += WARPS * 32) partial[i] = 0.f;
    pdl_wait();
    #pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < fetched) fetch_x(first_chunk[s], s);
        cp_async_commit();
    }
    __syncthreads();      // the table of sums is zeroed

    const uint32_t w_lo = uint32_t(reinterpret_cast<uintptr_t>(p.W)) + uint32_t(R0) * RB;
    const int sub = t >> 1;                                  // the 16-element sub-block of an MMA's 32 elements whose sums this lane scales
    const float digits = (t & 1) ? 16384.f : 1.f;            // its two columns are digits 0, 1 or 2, 3
    const bool first = g < 4;                                // its B column carries the first sub-block's elements
    float acc0 = 0.f, acc1 = 0.f;
    int acc_tile = u_tile;
    auto flush = [&]() {
        float s0 = acc0, s1 = acc1;
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if (t == 0) {
            float * dst = partial + (acc_tile * WARPS + warp) * kTileRows;
            dst[g] += s0;
            dst[g + 8] += s1;
        }
        acc0 = 0.f;
        acc1 = 0.f;
    };
    for (int u = 0; u < my_units; u++) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (fetched < my_units) { fetch(true); fetched++; }
        cp_async_commit();
        if (u_tile != acc_tile) { flush(); acc_tile = u_tile; }
        const int last = nrows - 1 - u_tile * kTileRows;      // rows past it are not copied: the lanes of those rows compute on whatever the stage holds and drop it
        const uint32_t lo = w_lo + uint32_t(u_tile * kTileRows) * RB + uint32_t(u_chunk) * CB;
        const uint32_t st = my_stages + uint32_t(u_slot) * stage_bytes;
        const uint32_t xl = st + rows_bytes, sxp = xl + uint32_t(p.cbk) * 1024u;      // the unit's digits and factors
        const uint32_t src0 = lo + uint32_t(min(g, last)) * RB, src1 = lo + uint32_t(min(g + 8, last)) * RB;      // the rows' addresses in device memory
        uint32_t r0 = st + uint32_t(g) * stride + (src0 & 15u), r1 = st + uint32_t(g + 8) * stride + (src1 & 15u);
        for (int b = 0; b < p.cbk; b++, r0 += kBB, r1 += kBB) {
            const uint32_t sh0 = (r0 & 2u) * 8u, sh1 = (r1 & 2u) * 8u;
            const int xb = b * 8;                              // the super-block's first 32-element block among the unit's
            const float d0 = __half2float(__ushort_as_half(uint16_t(word_at(r0 + 208u, sh0)))), d1 = __half2float(__ushort_as_half(uint16_t(word_at(r1 + 208u, sh1))));
            #pragma unroll
            for (int n = 0; n < 2; n++) {                      // the halves of 128 elements
                // high bit pairs of elements 4t .. 4t+3 and 16+4t .. of each 32: one word each, shared by the half's four groups of 32
                const uint32_t h0a = word_at(r0 + 128u + 32u * n + 4u * t, sh0), h0b = word_at(r0 + 128u + 32u * n + 16u + 4u * t, sh0);
                const uint32_t h1a = word_at(r1 + 128u + 32u * n + 4u * t, sh1), h1b = word_at(r1 + 128u + 32u * n + 16u + 4u * t, sh1);
                // the sub-block scales of the half: bytes 8 n .. 8 n + 7 of the 16
                const uint32_t s0lo = word_at(r0 + 192u + 8u * n, sh0), s0hi = word_at(r0 + 196u + 8u * n, sh0);
                const uint32_t s1lo = word_at(r1 + 192u + 8u * n, sh1), s1hi = word_at(r1 + 196u + 8u * n, sh1);
                #pragma unroll
                for (int jl = 0; jl < 2; jl++) {               // low nibbles: group jl of 32; high nibbles: group jl + 2
                    const uint32_t q0a = word_at(r0 + 64u * n + 32u * jl + 4u * t, sh0), q0b = word_at(r0 + 64u * n + 32u * jl + 16u + 4u * t, sh0);
                    const uint32_t q1a = word_at(r1 + 64u * n + 32u * jl + 4u * t, sh1), q1b = word_at(r1 + 64u * n + 32u * jl + 16u + 4u * t, sh1);
                    #pragma unroll
                    for (int hi = 0; hi < 2; hi++) {
                        const int j = jl + 2 * hi;             // the group of 32 elements within the half
                        const int blk = xb + 4 * n + j;
                        uint2 bv;
                        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(bv.x), "=r"(bv.y) : "r"(xl + uint32_t(blk) * 128u + uint32_t(g & 3) * 32u + uint32_t(t) * 8u));
                        const uint32_t b0 = first ? bv.x : 0u, b1 = first ? 0u : bv.y;
                        int c[4] = {0, 0, 0, 0};
                        constexpr uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
                        // the low nibbles (unsigned), then the high bit pairs at bits 4, 5 with the offset folded in: (h >> 2 j) << 4 is 0, 16, 32 or 48; flipping
                        // bit 5 and copying it into bits 6, 7 makes the signed bytes -32, -16, 0, 16
                        mma_u8s8_16832(c, (hi ? q0a >> 4 : q0a) & M4, (hi ? q1a >> 4 : q1a) & M4, (hi ? q0b >> 4 : q0b) & M4, (hi ? q1b >> 4 : q1b) & M4, b0, b1);
                        const int lsh = 4 - 2 * j;             // 4, 2, 0, -2
                        auto high = [&](uint32_t h) {
                            const uint32_t v = lop3_and_xor(lsh >= 0 ? h << (lsh >= 0 ? lsh : 0) : h >> 2, M2, 0x20202020u);
                            return v + (v & 0x20202020u) * 6u;
                        };
                        mma_s8_16832(c, high(h0a), high(h1a), high(h0b), high(h1b), b0, b1);
                        // scale of sub-block 2 j + sub of the half: byte 2 j + sub of (lo, hi)
                        const int sbyte = 2 * j + sub;         // 0 .. 7; j is a constant after unrolling, sub is not
                        const uint32_t w0 = sbyte < 4 ? s0lo : s0hi, w1 = sbyte < 4 ? s1lo : s1hi;
                        const float sc0 = float(int(int8_t((w0 >> (8 * (sbyte & 3))) & 0xFFu))), sc1 = float(int(int8_t((w1 >> (8 * (sbyte & 3))) & 0xFFu)));
                        float f;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(sxp + uint32_t(blk) * 8u));
                        // sum((q - 32) x) of this lane's two digits (f: the block's s 2^-26 / 16)
                        const float fx = f * 16.f * digits;
                        acc0 = fmaf(d0 * sc0 * fx, float(c[0] + 128 * c[1]), acc0);
                        acc1 = fmaf(d1 * sc1 * fx, float(c[2] + 128 * c[3]), acc1);
                    }
                }
            }
        }
        u_chunk += step_chunk;
        u_tile += step_tile;
        if (u_chunk >= p.nchunks) { u_chunk -= p.nchunks; u_tile++; }
        if (++u_slot == STAGES) u_slot = 0;
    }
    cp_async_wait<0>();
    if (my_units > 0) flush();
    __syncthreads();
    for (int r = threadIdx.x; r < nrows; r += WARPS * 32) {
        const float * src = partial + size_t(r / kTileRows) * WARPS * kTileRows + (r % kTileRows);
        float s = 0.f;
        #pragma unroll
        for (int w = 0; w < WARPS; w++) s += src[w * kTileRows];
        const int64_t rr = R0 + r;
        if (p.flags & kFlagBias) s += p.bias[rr];
        p.y[rr] = (p.flags & kFlagAccumulate) ? accumulate_base(p.y[rr], p.flags) + s : s;
    }
}

struct Plan { int cbk, nchunks, stride, upr, stages, warps; size_t smem; bool ok; };

constexpr size_t partial_bytes(int warps) { return size_t(kMaxTilesPerBlock) * warps * kTileRows * sizeof(float); }

// Chunks of one or two super-blocks (their aligned cover has to fit the copy table); 16 warps, as many stages as fit.
Plan plan_for(int64_t cols) {
    Plan best{};
    if (cols % 256 != 0 || cols > 40960) return best;      // (the copy table packs 15 rows' byte offsets into 19 bits)
    const int nb = int(cols / 256);
    const size_t fixed = 0;
    int64_t best_score = -1;
    for (int warps : {16, 8}) {
        for (int cbk = 1; cbk <= 2; cbk++) {
            if (nb % cbk) continue;
            const int upr = (cbk * kBB + 30) / 16;
            if (upr * kTileRows > kMaxPieces * 32) continue;
            int stride = (upr * 16 + 16 + 15) / 16 * 16;
            if (stride % 32 != 16) stride += 16;
            if (kTileRows * stride >= (1 << 13)) continue;
            int stages = 0;
            const size_t stage = size_t(kTileRows) * stride + size_t(cbk) * 8 * 136;
            for (int st = 4; st >= 2; st--) if (fixed + size_t(warps) * st * stage + partial_bytes(warps) <= kSmemLimit) { stages = st; break; }
            if (!stages) continue;
            const int64_t score = (warps == 16 ? 1000 : 0) + cbk * 100 + stages;
            if (score > best_score) {
                best_score = score;
                best = Plan{cbk, nb / cbk, stride, upr, stages, warps, fixed + size_t(warps) * stages * stage + partial_bytes(warps), true};
            }
        }
    }
    return best;
}

template <int WARPS, int STAGES>
cudaError_t launch_with(const GemvQ6kParams & p, size_t smem, unsigned grid, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_gemv_q6_k<WARPS, STAGES>, int(kSmemLimit), configured); e != cudaSuccess) return e;
    return launch_pdl(k_gemv_q6_k<WARPS, STAGES>, dim3(grid), dim3(WARPS * 32), smem, stream, p);
}

}  // namespace

bool gemv_q6_k_supported(const void * W, int64_t rows, int64_t cols) {
    static const bool off = [] { const char * e = getenv("DOOMS_GEMV_Q6K"); return e && *e == '0'; }();
    return !off && rows >= 1 && rows < (int64_t(1) << 31) && (reinterpret_cast<uintptr_t>(W) & 15u) == 0 && plan_for(cols).ok;
}

cudaError_t launch_gemv_q6_k(const void * W, const void * xq, float * y, const float * bias, int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream) {
    if (!W || !xq || !y || !gemv_q6_k_supported(W, rows, cols) || (reinterpret_cast<uintptr_t>(xq) & 15u)) return cudaErrorInvalidValue;
    const Plan pl = plan_for(cols);
    GemvQ6kParams p{static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(xq), y, bias, int(cols), flags, pl.cbk, pl.nchunks, pl.stride, pl.upr, 0, 0, 0u, 0u};
    const int sms = sm_count();
    const int64_t max_rows = int64_t(kMaxTilesPerBlock) * kTileRows;
    const int64_t waves = (rows + sms * max_rows - 1) / (sms * max_rows);
    const unsigned grid = unsigned(std::min<int64_t>(sms * waves, rows));
    p.rows_q = int(rows / grid);
    p.rows_r = int(rows % grid);
    p.inv_upr = 65536u / uint32_t(p.upr) + 1u;
    p.inv_nchunks = 65536u / uint32_t(pl.nchunks) + 1u;
    if (pl.warps == 16) {
        switch (pl.stages) {
            case 4: return launch_with<16, 4>(p, pl.smem, grid, stream);
            case 3: return launch_with<16, 3>(p, pl.smem, grid, stream);
            default: return launch_with<16, 2>(p, pl.smem, grid, stream);
        }
    }
    switch (pl.stages) {
        case 4: return launch_with<8, 4>(p, pl.smem, grid, stream);
        case 3: return launch_with<8, 3>(p, pl.smem, grid, stream);
        default: return launch_with<8, 2>(p, pl.smem, grid, stream);
    }
}

}  // namespace cuda
}  // namespace dooms
