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

}  // namespace b200bpe

struct b200bpe_ctx { b200bpe::Ctx c; };
