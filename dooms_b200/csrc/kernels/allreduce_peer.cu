// The tensor-parallel decode step's all-reduce, fused with the residual add: x += sum over ranks of `partial`, for one row of a few thousand floats, as one
// launch over peer memory instead of an NCCL call plus an add. Every rank pushes its partial vector into a slot of every rank's inbox (plain stores over
// NVLink into memory mapped through CUDA IPC), then publishes a sequence number next to it; a rank sums its inbox in rank order once all the numbers
// of this round are there, so every rank computes the same bits. The reference has one GPU; this is the collective of its all-reduce-after-attn_output /
// after-ffn_down sharding (the reduction itself is src/backend/metal/llama_kernels.h's residual accumulate, flags & 2).
//
// Ordering: data stores, then a system-scope fence, then the flag (release); the reader polls the flag (acquire, system scope) and reads the inbox with
// loads that bypass L1. Consecutive rounds alternate between two inbox halves: a rank can only be one round ahead of a peer (it needs the peer's flag of
// the round before), so the half it overwrites has been read. Waits are bounded: after kMaxPolls polls the kernel records an error and returns.
#include <cuda_runtime.h>

#include "kernels.h"
#include "launch.cuh"

namespace dooms {
namespace cuda {

using namespace dooms::dev;

namespace {

constexpr int kThreads = 256;
constexpr int kFloatsPerBlock = kThreads * 4;
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ void st_release_sys(uint32_t * p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t * p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kThreads) k_allreduce_add(const PeerAllReduce p, const float * partial, float * x, int n) {
    pdl_trigger();
    pdl_wait();
    __shared__ int ok_all;
    const int tid = threadIdx.x, i = blockIdx.x * kFloatsPerBlock + tid * 4;
    const uint32_t seq = *reinterpret_cast<volatile uint32_t *>(p.round) + 1u;      // the same for every block: it is bumped after the last one has finished
    const uint32_t half = seq & 1u;
    if (tid == 0) ok_all = 1;
    if (i < n) {
        const float4 v = *reinterpret_cast<const float4 *>(partial + i);
        for (int r = 0; r < p.n; r++) {
            *reinterpret_cast<float4 *>(p.inbox[r] + (size_t(half) * p.n + p.rank) * p.max_floats + i) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.n) {
        st_release_sys(p.flags[tid] + (size_t(half) * p.n + p.rank) * kPeerMaxBlocks + blockIdx.x, seq);
        const uint32_t * mine = p.flags[p.rank] + (size_t(half) * p.n + tid) * kPeerMaxBlocks + blockIdx.x;
        bool ok = false;
        for (uint32_t k = 0; k < kMaxPolls; k++) if (ld_acquire_sys(mine) == seq) { ok = true; break; }
        if (!ok) { ok_all = 0; p.state->error = 3; if (p.host_error) *p.host_error = 3; }
    }
    __syncthreads();
    if (ok_all && i < n) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.n; r++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(p.inbox[p.rank] + (size_t(half) * p.n + r) * p.max_floats + i));
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        float4 * dst = reinterpret_cast<float4 *>(x + i);
        float4 o = *dst;
        o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
        *dst = o;
    }
    __syncthreads();
    if (tid == 0) {
        const unsigned done = atomicAdd(p.ticket, 1u);
        if (done == gridDim.x - 1) {
            *p.ticket = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(p.round) = seq;
        }
    }
}

}  // namespace

size_t peer_allreduce_inbox_bytes(int n_ranks, int max_floats) { return size_t(2) * n_ranks * max_floats * sizeof(float); }
size_t peer_allreduce_flag_bytes(int n_ranks) { return size_t(2) * n_ranks * kPeerMaxBlocks * sizeof(uint32_t); }

cudaError_t launch_allreduce_add(const PeerAllReduce & p, const float * partial, float * x, int n, cudaStream_t stream) {
    if (n < 1 || n % 4 != 0 || n > p.max_floats || p.n < 2 || p.n > kPeerMaxRanks) return cudaErrorInvalidValue;
    const int blocks = (n + kFloatsPerBlock - 1) / kFloatsPerBlock;
    if (blocks > kPeerMaxBlocks) return cudaErrorInvalidValue;
    return launch_pdl(k_allreduce_add, dim3(blocks), dim3(kThreads), 0, stream, p, partial, x, n);
}

}  // namespace cuda
}  // namespace dooms
