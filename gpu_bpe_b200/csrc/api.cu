// Context management, status text and NCCL loading for libb200bpe.so.
#include <dlfcn.h>

#include <cstring>

#include "ctx.cuh"

namespace b200bpe {

static thread_local std::string g_last_error;
void set_last_error(const std::string& s) { g_last_error = s; }

b200bpe_status load_nccl(const char* path, NcclApi* api) {
    if (!path || !*path) { set_last_error("no NCCL library path given"); return B200BPE_ERR_BAD_ARG; }
    void* h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) { set_last_error(std::string("dlopen ") + path + ": " + dlerror()); return B200BPE_ERR_NCCL; }
    api->handle = h;
#define B2_SYM(field, name)                                                                   \
    *reinterpret_cast<void**>(&api->field) = dlsym(h, name);                                  \
    if (!api->field) { set_last_error(std::string("missing symbol ") + name); return B200BPE_ERR_NCCL; }
    B2_SYM(GetUniqueId, "ncclGetUniqueId")
    B2_SYM(CommInitRank, "ncclCommInitRank")
    B2_SYM(CommDestroy, "ncclCommDestroy")
    B2_SYM(AllReduce, "ncclAllReduce")
    B2_SYM(AllGather, "ncclAllGather")
    B2_SYM(Send, "ncclSend")
    B2_SYM(Recv, "ncclRecv")
    B2_SYM(GroupStart, "ncclGroupStart")
    B2_SYM(GroupEnd, "ncclGroupEnd")
    B2_SYM(GetErrorString, "ncclGetErrorString")
#undef B2_SYM
    return B200BPE_OK;
}

static b200bpe_status make_ctx(int device, b200bpe_ctx** out) {
    if (!out) return B200BPE_ERR_BAD_ARG;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        set_last_error("no CUDA device is visible; this library has no CPU path");
        return B200BPE_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    B2_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_last_error(std::string("device ") + prop.name + " is not sm_100; the kernels are built for sm_100a only");
        return B200BPE_ERR_NO_DEVICE;
    }
    b200bpe_ctx* c = new b200bpe_ctx();
    c->c.device = device;
    c->c.sm_count = prop.multiProcessorCount;
    c->c.cc = prop.major * 10 + prop.minor;
    cudaError_t e = cudaStreamCreateWithFlags(&c->c.stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete c; set_last_error(cudaGetErrorString(e)); return B200BPE_ERR_CUDA; }
    *out = c;
    return B200BPE_OK;
}

}  // namespace b200bpe

using namespace b200bpe;

extern "C" {

const char* b200bpe_status_str(b200bpe_status s) {
    switch (s) {
        case B200BPE_OK: return "ok";
        case B200BPE_ERR_BAD_ARG: return "bad argument";
        case B200BPE_ERR_CUDA: return "CUDA error";
        case B200BPE_ERR_NO_DEVICE: return "no sm_100 GPU available (there is no CPU fallback)";
        case B200BPE_ERR_EMPTY_CORPUS: return "No symbols to train on — corpus is empty after pre-processing";
        case B200BPE_ERR_TABLE_FULL: return "pair table full";
        case B200BPE_ERR_LOOKBACK_TIMEOUT: return "device-side wait timed out";
        case B200BPE_ERR_BAD_TRIE_MAGIC: return "Invalid trie magic";
        case B200BPE_ERR_BAD_TRIE_VERSION: return "Unsupported trie version";
        case B200BPE_ERR_TRUNCATED_TRIE: return "Truncated trie data";
        case B200BPE_ERR_CAPACITY: return "output buffer too small";
        case B200BPE_ERR_NCCL: return "NCCL error";
        case B200BPE_ERR_OOM: return "out of device memory";
        case B200BPE_ERR_INTERNAL: return "internal consistency check failed";
        default: return "unknown status";
    }
}

const char* b200bpe_last_error(void) { return g_last_error.c_str(); }

int32_t b200bpe_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return 0; }
    return count;
}

b200bpe_status b200bpe_ctx_create(int32_t device, b200bpe_ctx** out) { return make_ctx(device, out); }

b200bpe_status b200bpe_nccl_unique_id(const char* nccl_lib, uint8_t unique_id[128]) {
    if (!unique_id) return B200BPE_ERR_BAD_ARG;
    NcclApi api;
    b200bpe_status r = load_nccl(nccl_lib, &api);
    if (r) return r;
    NcclIdBlob id;
    std::memset(&id, 0, sizeof(id));
    int rc = api.GetUniqueId(&id);
    if (rc) { set_last_error(std::string("ncclGetUniqueId: ") + api.GetErrorString(rc)); return B200BPE_ERR_NCCL; }
    std::memcpy(unique_id, id.bytes, 128);
    return B200BPE_OK;
}

b200bpe_status b200bpe_ctx_create_dist(int32_t device, int32_t rank, int32_t world, const char* nccl_lib,
                                       const uint8_t unique_id[128], b200bpe_ctx** out) {
    if (world < 1 || rank < 0 || rank >= world || !unique_id) return B200BPE_ERR_BAD_ARG;
    b200bpe_ctx* c = nullptr;
    b200bpe_status r = make_ctx(device, &c);
    if (r) return r;
    c->c.rank = rank;
    c->c.world = world;
    if (world > 1) {
        r = load_nccl(nccl_lib, &c->c.nccl);
        if (r) { b200bpe_ctx_destroy(c); return r; }
        NcclIdBlob id;
        std::memcpy(id.bytes, unique_id, 128);
        int rc = c->c.nccl.CommInitRank(&c->c.comm, world, id, rank);
        if (rc) {
            set_last_error(std::string("ncclCommInitRank: ") + c->c.nccl.GetErrorString(rc));
            b200bpe_ctx_destroy(c);
            return B200BPE_ERR_NCCL;
        }
    }
    *out = c;
    return B200BPE_OK;
}

void b200bpe_ctx_destroy(b200bpe_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->c.device);
    if (c->c.comm && c->c.nccl.CommDestroy) c->c.nccl.CommDestroy(c->c.comm);
    if (c->c.stream) cudaStreamDestroy(c->c.stream);
    delete c;
}

b200bpe_status b200bpe_ctx_info(b200bpe_ctx* c, int32_t* sm_count, int32_t* cc, uint64_t* total_mem, uint64_t* free_mem) {
    if (!c) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(c->c.device));
    size_t f = 0, t = 0;
    B2_CUDA(cudaMemGetInfo(&f, &t));
    if (sm_count) *sm_count = c->c.sm_count;
    if (cc) *cc = c->c.cc;
    if (total_mem) *total_mem = t;
    if (free_mem) *free_mem = f;
    return B200BPE_OK;
}

b200bpe_status b200bpe_ctx_synchronize(b200bpe_ctx* c) {
    if (!c) return B200BPE_ERR_BAD_ARG;
    B2_CUDA(cudaSetDevice(c->c.device));
    B2_CUDA(cudaStreamSynchronize(c->c.stream));
    return B200BPE_OK;
}

}  // extern "C"
