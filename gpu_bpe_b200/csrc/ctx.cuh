// Context object: one GPU, one stream, optional NCCL communicator for sharded jobs.
#pragma once

#include <string>

#include "common.cuh"

namespace b200bpe {

struct NcclIdBlob { char bytes[128]; };

// NCCL entry points resolved at run time from the library the caller names, so that the
// process holds a single NCCL (the one its host framework already loaded).
struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, /*ncclUniqueId by value*/ NcclIdBlob, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};
struct Ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int cc = 0;
    int rank = 0, world = 1;
    NcclApi nccl;
    void* comm = nullptr;
};

b200bpe_status load_nccl(const char* path, NcclApi* api);

// Ask the L2 to keep [base, base + bytes) resident for the kernels launched on the context's
// stream from now on (a persisting access-policy window; captured graphs keep the window they
// were captured with).  The set-aside is capped, so a larger range is kept in proportion.
inline void set_persisting_window(Ctx* c, const void* base, size_t bytes) {
    int max_win = 0, max_persist = 0;
    cudaDeviceGetAttribute(&max_win, cudaDevAttrMaxAccessPolicyWindowSize, c->device);
    cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, c->device);
    const size_t want = bytes < (size_t)(max_win > 0 ? max_win : 0) ? bytes : (size_t)(max_win > 0 ? max_win : 0);
    if (want == 0 || max_persist <= 0) { cudaGetLastError(); return; }
    size_t set_aside = (size_t)max_persist;
    if (set_aside > ((size_t)64 << 20)) set_aside = (size_t)64 << 20;
    cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, set_aside);
    cudaStreamAttrValue attr{};
    attr.accessPolicyWindow.base_ptr = const_cast<void*>(base);
    attr.accessPolicyWindow.num_bytes = want;
    attr.accessPolicyWindow.hitRatio = want <= set_aside ? 1.0f : (float)set_aside / (float)want;
    attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    cudaStreamSetAttribute(c->stream, cudaStreamAttributeAccessPolicyWindow, &attr);
    cudaGetLastError();
}

}  // namespace b200bpe

struct b200bpe_ctx { b200bpe::Ctx c; };
