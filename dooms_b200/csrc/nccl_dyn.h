#pragma once
// NCCL bound at run time (dlopen), so that the library has no link-time dependency on it: a one-GPU process never loads it. Only the handful of entry
// points the tensor-parallel decoder uses are declared, with the signatures of nccl.h (NCCL 2.x).
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <string>

#include "status.h"

namespace dooms {

struct NcclUniqueId { char internal[128]; };
typedef struct ncclComm * NcclComm;

struct NcclApi {
    void * lib = nullptr;
    int (*GetUniqueId)(NcclUniqueId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char * (*GetErrorString)(int) = nullptr;
    // Optional (NCCL 2.27 and later): memory from NCCL's own allocator, registered with the communicator as a symmetric window. Collectives on buffers that
    // lie in such windows on every rank run NCCL's low-latency symmetric kernels; nullptr when the library is older.
    int (*MemAlloc)(void **, size_t) = nullptr;
    int (*MemFree)(void *) = nullptr;
    int (*CommWindowRegister)(NcclComm, void *, size_t, void **, int) = nullptr;
    int (*CommWindowDeregister)(NcclComm, void *) = nullptr;
    bool has_windows() const { return MemAlloc && MemFree && CommWindowRegister && CommWindowDeregister; }
    static constexpr int kFloat32 = 7, kInt8 = 0, kSum = 0;   // ncclFloat32, ncclInt8, ncclSum
    static constexpr int kWinCollSymmetric = 1;               // NCCL_WIN_COLL_SYMMETRIC
    static constexpr size_t kWinAlignment = 4096;             // NCCL_WIN_REQUIRED_ALIGNMENT
};

inline Status load_nccl(const char * path, NcclApi * api) {
    if (api->lib) return Status();
    const char * names[] = {path, "libnccl.so.2", "libnccl.so"};
    for (const char * n : names) {
        if (!n || !*n) continue;
        api->lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (api->lib) break;
    }
    if (!api->lib) return unsupported(std::string("cannot load NCCL (") + (path ? path : "libnccl.so.2") + "): " + dlerror());
    auto sym = [&](const char * s) { return dlsym(api->lib, s); };
    api->GetUniqueId = reinterpret_cast<decltype(api->GetUniqueId)>(sym("ncclGetUniqueId"));
    api->CommInitRank = reinterpret_cast<decltype(api->CommInitRank)>(sym("ncclCommInitRank"));
    api->CommDestroy = reinterpret_cast<decltype(api->CommDestroy)>(sym("ncclCommDestroy"));
    api->AllReduce = reinterpret_cast<decltype(api->AllReduce)>(sym("ncclAllReduce"));
    api->AllGather = reinterpret_cast<decltype(api->AllGather)>(sym("ncclAllGather"));
    api->GetErrorString = reinterpret_cast<decltype(api->GetErrorString)>(sym("ncclGetErrorString"));
    api->MemAlloc = reinterpret_cast<decltype(api->MemAlloc)>(sym("ncclMemAlloc"));
    api->MemFree = reinterpret_cast<decltype(api->MemFree)>(sym("ncclMemFree"));
    api->CommWindowRegister = reinterpret_cast<decltype(api->CommWindowRegister)>(sym("ncclCommWindowRegister"));
    api->CommWindowDeregister = reinterpret_cast<decltype(api->CommWindowDeregister)>(sym("ncclCommWindowDeregister"));
    if (!api->GetUniqueId || !api->CommInitRank || !api->CommDestroy || !api->AllReduce || !api->AllGather || !api->GetErrorString) {
        return unsupported("the NCCL library lacks an entry point this decoder needs");
    }
    return Status();
}

}  // namespace dooms
