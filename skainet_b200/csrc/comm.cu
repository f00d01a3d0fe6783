// NCCL binding by dlopen (see comm.cuh). Only the five entry points the decoder needs.
#include "comm.cuh"

#include <dlfcn.h>
#include <cstring>
#include <mutex>

namespace sk {

// Mirrors of the NCCL ABI pieces used here (stable across NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt8 = 0, ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

static NcclApi g_nccl;
static std::once_flag g_nccl_once;

static void load_nccl() {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) return;
    auto sym = [](const char* s) { return dlsym(g_nccl.handle, s); };
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId)) sym("ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank)) sym("ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy)) sym("ncclCommDestroy");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce)) sym("ncclAllReduce");
    g_nccl.AllGather = (decltype(g_nccl.AllGather)) sym("ncclAllGather");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString)) sym("ncclGetErrorString");
    g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllReduce && g_nccl.AllGather;
}

static int32_t nccl_ready() {
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.ok) { set_error("NCCL (libnccl.so.2) could not be loaded: tensor parallelism is unavailable"); return SKAINET_CUDA_ERR_COMM; }
    return SKAINET_CUDA_OK;
}
static int32_t nccl_fail(ncclResult_t r, const char* what) {
    set_error("NCCL error %d (%s) in %s", r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
    return SKAINET_CUDA_ERR_COMM;
}

struct Comm { ncclComm_t comm = nullptr; int rank = 0, world = 1; };

int32_t comm_unique_id(uint8_t* id128) {
    SK_TRY(nccl_ready());
    ncclUniqueId id;
    const ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != 0) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id128, id.internal, 128);
    return SKAINET_CUDA_OK;
}

int32_t comm_create(int rank, int world, const uint8_t* id128, Comm** out) {
    SK_TRY(nccl_ready());
    ncclUniqueId id;
    memcpy(id.internal, id128, 128);
    Comm* c = new Comm();
    c->rank = rank; c->world = world;
    const ncclResult_t r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r != 0) { delete c; return nccl_fail(r, "ncclCommInitRank"); }
    *out = c;
    return SKAINET_CUDA_OK;
}

void comm_destroy(Comm* c) {
    if (!c) return;
    if (c->comm && g_nccl.ok) g_nccl.CommDestroy(c->comm);
    delete c;
}

int32_t comm_all_reduce_sum(Comm* c, float* buf, int64_t n, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    const ncclResult_t r = g_nccl.AllReduce(buf, buf, (size_t) n, ncclFloat32, ncclSum, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllReduce");
}

int32_t comm_all_gather(Comm* c, const void* send, void* recv, int64_t nbytes, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    const ncclResult_t r = g_nccl.AllGather(send, recv, (size_t) nbytes, ncclInt8, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllGather");
}

}  // namespace sk
