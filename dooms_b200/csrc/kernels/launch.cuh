#pragma once
// Programmatic dependent launch: a kernel launched through launch_pdl() may start while the kernel before it in the stream is still running. Every kernel
// launched this way calls pdl_wait() before it reads anything an earlier kernel wrote and before it writes anything (weights and other constants may be
// fetched earlier); it calls pdl_trigger() as soon as the next kernel may start its own prologue. Because each kernel waits for its predecessor to finish
// before it can finish itself, waiting for the immediate predecessor orders a kernel after everything earlier in the stream.
// The early trigger is only safe when the kernel that follows is one of these: a kernel of another library that is itself launched as a programmatic
// dependent but does not wait before it reads (NCCL's symmetric-memory collectives behaved that way) would see half-written input. A kernel whose output
// such a collective reads therefore skips its trigger (kFlagLateDependents in kernels.h) and releases its dependents by finishing.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>

namespace dooms {
namespace dev {
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
}  // namespace dev

namespace cuda {

// Multiprocessors of the current device, asked once per device (the launchers size their grids by it).
inline int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    const int slot = dev & 63;
    int n = cached[slot].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) { cudaGetLastError(); n = 148; }
        cached[slot].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Raises a kernel's dynamic shared-memory limit once per device. The attribute belongs to (function, device); `done` is one word per kernel instantiation
// (a function-local static at the call site) with a bit per device, so threads that drive different devices never undo each other's work.
template <class K>
cudaError_t allow_dynamic_smem(K kernel, int bytes, std::atomic<uint64_t> & done) {
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = uint64_t(1) << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
}

// Early launches are on unless DOOMS_PDL=0 is in the environment. With one 180-200 KB block per SM the next kernel's blocks cannot sit beside the running
// ones; what the early launch buys is that each SM starts the next kernel's block (its prologue and its first weight copies) the moment its own block of the
// running kernel exits, instead of after the slowest block of the grid plus a launch: measured on B200, the 8B-shape decode step went from 2.04 to 1.91 ms.
// Without the launch attribute the kernels' waits return at once and the trigger does nothing.
inline bool pdl_enabled() {
    static const bool on = [] { const char * e = getenv("DOOMS_PDL"); return !(e && *e == '0'); }();
    return on;
}

template <class... KArgs, class... Args>
cudaError_t launch_pdl_if(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = early && pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return launch_pdl_if(true, kernel, grid, block, smem, stream, args...);
}

}  // namespace cuda
}  // namespace dooms
