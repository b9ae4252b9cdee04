// Decode GEMV for the block formats and shapes that have no integer tensor-core path here (q5_0, q8_0, f16; q4_0, q4_K and q6_K when gemv_q4_0.cu /
// gemv_q6_k.cu do not take the shape): the same streaming skeleton as gemv_q4_0.cu, with the dot products on the CUDA cores in f32.
//   * One block per SM with an equal share of the rows; the units of work are (16-row tile, matrix, chunk of the row), dealt round-robin to the block's
//     warps; every warp streams its units through its own ring of shared-memory stages filled by 16-byte asynchronous copies of the rows' bytes exactly as
//     they lie in the GGUF file (blocks of 22, 34, 144, 210 bytes at 2-byte alignment: the copies are the aligned cover of the chunk).
//   * The input vector sits in shared memory as f32 (copied once per block), so a lane's reads of it are broadcasts.
//   * Within a unit a lane owns one row and every second 32-element group of the chunk: the formats' own dot-product folding (UnitDot, the reference's
//     Q::dot, src/backend/metal/llama_kernels.h:1036-1154) runs unchanged on the staged bytes.
//   * Per-warp sums go to a small shared table and are added in a fixed order after one barrier: results do not depend on timing.
// Replaces matvec1q / gate_up1q (llama_kernels.h:1197-1269) for these formats.
#include <cuda_fp16.h>

#include <algorithm>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"
#include "quant.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kTileRows = 16;
constexpr int kMaxPieces = 10;      // 16-byte pieces of a stage one lane copies
constexpr int kMaxTilesPerBlock = 8;
constexpr size_t kSmemLimit = 224 * 1024;

template <int DT> struct Fmt;
template <> struct Fmt<kF16> { static constexpr int BE = 32, BB = 64; };
template <> struct Fmt<kQ4_0> { static constexpr int BE = 32, BB = 18; };
template <> struct Fmt<kQ5_0> { static constexpr int BE = 32, BB = 22; };
template <> struct Fmt<kQ8_0> { static constexpr int BE = 32, BB = 34; };
template <> struct Fmt<kQ4_K> { static constexpr int BE = 256, BB = 144; };
template <> struct Fmt<kQ6_K> { static constexpr int BE = 256, BB = 210; };

struct GemvBlocksParams {
    const uint8_t * W;
    const uint8_t * W2;     // gate/up: the second matrix (up)
    const float * x;
    const float * gamma;    // optional: RMS-normalize x first
    float eps;
    float * y;
    const float * bias;
    int cols;
    uint32_t flags;
    int cbk, nchunks;       // blocks per chunk, chunks per row
    int stride, upr;        // bytes between the rows of a stage; 16-byte pieces copied per row
    int rows_q, rows_r;     // block b has rows_q + (b < rows_r) rows starting at b rows_q + min(b, rows_r)
    uint32_t inv_upr, inv_nchunks;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// The 32 input values of one group, fetched with eight 16-byte shared-memory loads (a broadcast: the lanes of a half-warp read the same group) and handed
// to the formats' dot products by index: after inlining the indices are constants and the values stay in registers.
struct GroupX {
    float v[32];
    uint32_t first;     // index of v[0] in the chunk
    __device__ __forceinline__ void load(const float * chunk, uint32_t group) {
        first = group * 32u;
        const float4 * src = reinterpret_cast<const float4 *>(chunk + first);
        #pragma unroll
        for (int i = 0; i < 8; i++) { const float4 t = src[i]; v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
    }
    __device__ __forceinline__ float operator()(uint32_t i) const { return v[i - first]; }
};

template <int DT, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1) k_gemv_blocks(const GemvBlocksParams p) {
    constexpr int BE = Fmt<DT>::BE, BB = Fmt<DT>::BB;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nmat = p.W2 ? 2 : 1;
    const uint32_t RB = uint32_t(p.cols / BE) * BB;
    const uint32_t CB = uint32_t(p.cbk) * BB;

    const int nrows = p.rows_q + (int(blockIdx.x) < p.rows_r ? 1 : 0);
    const int64_t R0 = int64_t(blockIdx.x) * p.rows_q + min(int(blockIdx.x), p.rows_r);
    const int ntiles = (nrows + kTileRows - 1) / kTileRows;
    const int total_units = ntiles * nmat * p.nchunks;
    const int my_units = warp < total_units ? (total_units - warp - 1) / WARPS + 1 : 0;

    float * xs = reinterpret_cast<float *>(smem);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t stride = uint32_t(p.stride);
    const uint32_t stage_bytes = uint32_t(kTileRows) * stride;
    const uint32_t stages_off = (uint32_t(p.cols) * 4u + 127u) & ~127u;
    const uint32_t my_stages_off = stages_off + uint32_t(warp) * STAGES * stage_bytes;
    const uint32_t my_stages = smem_base + my_stages_off;
    float * partial = reinterpret_cast<float *>(smem + stages_off + size_t(WARPS) * STAGES * stage_bytes);   // [tile][mat][warp][16]

    const int step_tm = int((uint32_t(WARPS) * p.inv_nchunks) >> 16), step_chunk = WARPS - step_tm * p.nchunks;
    int f_tm = int((uint32_t(warp) * p.inv_nchunks) >> 16), f_chunk = warp - f_tm * p.nchunks, f_slot = 0;      // the unit being fetched
    int u_tm = f_tm, u_chunk = f_chunk, u_slot = 0;                                                               // the unit being used

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
    auto fetch = [&]() {
        const int tile = nmat == 2 ? f_tm >> 1 : f_tm, mat = nmat == 2 ? f_tm & 1 : 0;
        const uint8_t * base = (mat ? p.W2 : p.W) + (R0 + tile * kTileRows) * int64_t(RB) + uint32_t(f_chunk) * CB;
        const uint32_t lo = uint32_t(reinterpret_cast<uintptr_t>(base));
        const uint32_t dst0 = my_stages + uint32_t(f_slot) * stage_bytes;
        const int limit = tile != ntiles - 1 ? kTileRows : last_rows;
        #pragma unroll
        for (int k = 0; k < kMaxPieces; k++) {
            const uint32_t e = tab[k];
            if (e != 0xFFFFFFFFu && int((piece_rows[k / 8] >> (4 * (k % 8))) & 15u) <= limit) {
                const uint32_t off = e >> 13;
                cp_async16(dst0 + (e & 0x1FFFu), base + (int32_t(off) - int32_t((lo + off) & 15u)));
            }
        }
        f_chunk += step_chunk;
        f_tm += step_tm;
        if (f_chunk >= p.nchunks) { f_chunk -= p.nchunks; f_tm++; }
        if (++f_slot == STAGES) f_slot = 0;
    };

    int fetched = 0;
    if (!(p.flags & kFlagLateDependents)) pdl_trigger();
    #pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (fetched < my_units) { fetch(); fetched++; }
        cp_async_commit();
    }
    for (int i = threadIdx.x; i < ntiles * nmat * WARPS * kTileRows; i += WARPS * 32) partial[i] = 0.f;
    pdl_wait();
    for (uint32_t i = threadIdx.x; i < uint32_t(p.cols) / 4u; i += WARPS * 32) cp_async16(smem_base + i * 16u, p.x + size_t(i) * 4);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (p.gamma) {
        // x[i] * rsqrt(mean(x^2) + eps) * gamma[i] (norm_vec, llama_kernels.h:1272-1286), in place in shared memory, by every block for itself
        __shared__ float red[WARPS];
        float ss = 0.f;
        for (int i = threadIdx.x; i < p.cols; i += WARPS * 32) ss += xs[i] * xs[i];
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float total = 0.f;
        #pragma unroll
        for (int w = 0; w < WARPS; w++) total += red[w];
        const float inv = rsqrtf(total / float(p.cols) + p.eps);
        for (int i = threadIdx.x; i < p.cols; i += WARPS * 32) xs[i] = xs[i] * inv * p.gamma[i];
        __syncthreads();
    }

    const int row = lane & 15, half = lane >> 4;
    constexpr int UPB = BE / 32;                  // 32-element groups per block
    const int groups = p.cbk * UPB;               // per chunk
    const uint32_t w_lo = uint32_t(reinterpret_cast<uintptr_t>(p.W)) + uint32_t(R0) * RB, w2_lo = uint32_t(reinterpret_cast<uintptr_t>(p.W2)) + uint32_t(R0) * RB;
    float acc = 0.f;
    int acc_tm = u_tm;
    auto flush = [&]() {
        const float s = acc + __shfl_xor_sync(0xffffffffu, acc, 16);
        if (half == 0) partial[(acc_tm * WARPS + warp) * kTileRows + row] += s;
        acc = 0.f;
    };
    for (int u = 0; u < my_units; u++) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        if (fetched < my_units) { fetch(); fetched++; }
        cp_async_commit();
        if (u_tm != acc_tm) { flush(); acc_tm = u_tm; }
        const int tile = nmat == 2 ? u_tm >> 1 : u_tm;
        const uint32_t lo = ((nmat == 2 && (u_tm & 1)) ? w2_lo : w_lo) + uint32_t(tile * kTileRows) * RB + uint32_t(u_chunk) * CB;
        // the lane's row of the stage; its bytes start at the low four address bits of the row's chunk
        const uint8_t * rp = smem + my_stages_off + uint32_t(u_slot) * stage_bytes + uint32_t(row) * stride + ((lo + uint32_t(row) * RB) & 15u);
        const float * chunk_x = xs + size_t(u_chunk) * p.cbk * BE;
        for (int gq = half; gq < groups; gq += 2) {
            GroupX X;
            X.load(chunk_x, uint32_t(gq));
            acc += UnitDot<DT>::dot(rp, uint32_t(gq), X);
        }
        u_chunk += step_chunk;
        u_tm += step_tm;
        if (u_chunk >= p.nchunks) { u_chunk -= p.nchunks; u_tm++; }
        if (++u_slot == STAGES) u_slot = 0;
    }
    cp_async_wait<0>();
    if (my_units > 0) flush();
    __syncthreads();
    for (int r = threadIdx.x; r < nrows; r += WARPS * 32) {
        const float * src = partial + size_t(r / kTileRows) * nmat * WARPS * kTileRows + (r % kTileRows);
        float s = 0.f, s2 = 0.f;
        #pragma unroll
        for (int w = 0; w < WARPS; w++) s += src[w * kTileRows];
        if (nmat == 2) {
            #pragma unroll
            for (int w = 0; w < WARPS; w++) s2 += src[(WARPS + w) * kTileRows];
            s = s / (1.f + expf(-s)) * s2;
        }
        const int64_t rr = R0 + r;
        if (p.flags & kFlagBias) s += p.bias[rr];
        p.y[rr] = (p.flags & kFlagAccumulate) ? accumulate_base(p.y[rr], p.flags) + s : s;
    }
}

struct Plan { int cbk, nchunks, stride, upr, stages, warps; size_t smem; bool ok; };

constexpr size_t partial_bytes(int warps, int nmat) { return size_t(kMaxTilesPerBlock) * nmat * warps * kTileRows * sizeof(float); }

// The longest chunk of whole blocks that divides the row and whose aligned cover fits the copy table; 16 warps when two stages fit, else 8.
Plan plan_for(int BE, int BB, int64_t cols, int nmat) {
    Plan best{};
    if (cols % BE != 0 || cols % 4 != 0) return best;
    const int nb = int(cols / BE);
    const size_t fixed = (size_t(cols) * 4 + 127) & ~size_t(127);
    const bool aligned = (int64_t(nb) * BB) % 16 == 0;
    int64_t best_score = -1;
    for (int warps : {16, 8}) {
        for (int cbk = 1; cbk <= nb; cbk++) {
            if (nb % cbk) continue;
            const int chunk = cbk * BB;
            const int upr = (aligned && chunk % 16 == 0) ? chunk / 16 : (chunk + 30) / 16;
            if (upr * kTileRows > kMaxPieces * 32) break;
            int stride = (upr * 16 + 16 + 15) / 16 * 16;
            if (stride % 32 != 16) stride += 16;
            if (kTileRows * stride >= (1 << 13)) break;
            int stages = 0;
            for (int st = 4; st >= 2; st--) if (fixed + size_t(warps) * st * kTileRows * stride + partial_bytes(warps, nmat) <= kSmemLimit) { stages = st; break; }
            if (!stages) continue;
            const int64_t score = int64_t(chunk) * 1000 + (warps == 16 ? 100 : 0) + stages;
            if (score > best_score) {
                best_score = score;
                best = Plan{cbk, nb / cbk, stride, upr, stages, warps, fixed + size_t(warps) * stages * kTileRows * stride + partial_bytes(warps, nmat), true};
            }
        }
    }
    return best;
}

template <int DT, int WARPS, int STAGES>
cudaError_t launch_with(const GemvBlocksParams & p, size_t smem, unsigned grid, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0};
    if (const cudaError_t e = allow_dynamic_smem(k_gemv_blocks<DT, WARPS, STAGES>, int(kSmemLimit), configured); e != cudaSuccess) return e;
    return launch_pdl(k_gemv_blocks<DT, WARPS, STAGES>, dim3(grid), dim3(WARPS * 32), smem, stream, p);
}

// One block per SM; more (whole multiples) only when a block's share would exceed the table of kMaxTilesPerBlock tiles.
unsigned grid_for(int64_t rows) {
    const int sms = sm_count();
    const int64_t max_rows = int64_t(kMaxTilesPerBlock) * kTileRows;
    const int64_t waves = (rows + sms * max_rows - 1) / (sms * max_rows);
    return unsigned(std::min<int64_t>(sms * waves, rows));
}

template <int DT>
cudaError_t launch_dt(GemvBlocksParams p, int64_t rows, cudaStream_t stream) {
    const Plan pl = plan_for(Fmt<DT>::BE, Fmt<DT>::BB, p.cols, p.W2 ? 2 : 1);
    if (!pl.ok) return cudaErrorInvalidValue;
    p.cbk = pl.cbk; p.nchunks = pl.nchunks; p.stride = pl.stride; p.upr = pl.upr;
    const unsigned grid = grid_for(rows);
    p.rows_q = int(rows / grid);
    p.rows_r = int(rows % grid);
    p.inv_upr = 65536u / uint32_t(p.upr) + 1u;
    p.inv_nchunks = 65536u / uint32_t(pl.nchunks) + 1u;
    if (pl.warps == 16) {
        switch (pl.stages) {
            case 4: return launch_with<DT, 16, 4>(p, pl.smem, grid, stream);
            case 3: return launch_with<DT, 16, 3>(p, pl.smem, grid, stream);
            default: return launch_with<DT, 16, 2>(p, pl.smem, grid, stream);
        }
    }
    switch (pl.stages) {
        case 4: return launch_with<DT, 8, 4>(p, pl.smem, grid, stream);
        case 3: return launch_with<DT, 8, 3>(p, pl.smem, grid, stream);
        default: return launch_with<DT, 8, 2>(p, pl.smem, grid, stream);
    }
}

int fmt_be(int dt) { return dt == kQ4_K || dt == kQ6_K ? 256 : 32; }
int fmt_bb(int dt) {
    switch (dt) {
        case kF16: return 64; case kQ4_0: return 18; case kQ5_0: return 22; case kQ8_0: return 34; case kQ4_K: return 144; case kQ6_K: return 210;
        default: return 0;
    }
}

}  // namespace

bool gemv_blocks_supported(int dt, const void * W, const void * x, int64_t rows, int64_t cols) {
    if (fmt_bb(dt) == 0 || rows < 1 || cols > 65536) return false;
    if ((reinterpret_cast<uintptr_t>(W) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    // the nchunks reciprocal is exact for the warp counts divided by it as long as nchunks is small or larger than the dividends; upr <= 20
    return plan_for(fmt_be(dt), fmt_bb(dt), cols, 2).ok;
}

cudaError_t launch_gemv_blocks(int dt, const void * W, const void * W2, const float * x, const float * gamma, float eps, float * y, const float * bias,
                               int64_t rows, int64_t cols, uint32_t flags, cudaStream_t stream) {
    GemvBlocksParams p{static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(W2), x, gamma, eps, y, bias, int(cols), flags, 0, 0, 0, 0, 0, 0, 0u, 0u};
    switch (dt) {
        case kF16: return launch_dt<kF16>(p, rows, stream);
        case kQ4_0: return launch_dt<kQ4_0>(p, rows, stream);
        case kQ5_0: return launch_dt<kQ5_0>(p, rows, stream);
        case kQ8_0: return launch_dt<kQ8_0>(p, rows, stream);
        case kQ4_K: return launch_dt<kQ4_K>(p, rows, stream);
        case kQ6_K: return launch_dt<kQ6_K>(p, rows, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace cuda
}  // namespace dooms
