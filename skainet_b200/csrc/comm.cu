// NCCL binding by dlopen (see comm.cuh), only the five entry points the decoder needs, plus a one-shot
// all-reduce over peer memory for the small sums of a decode step.
//
// One-shot all-reduce (n <= P2P_MAX_ELEMS floats): every rank owns an "inbox" of world slots (two copies,
// used alternately) and a flag word per (sender, CTA). A CTA stores its slice of the local vector into its
// slot of every peer's inbox (plain stores over NVLink), publishes a sequence number with a system-scope
// release store, waits (bounded) until every peer's number for this round has arrived, and sums the world
// slots in rank order, so all ranks get bit-identical results. Nothing is reset between rounds: numbers only
// grow, and a peer can be at most one round ahead, which the second inbox copy absorbs. Latency is one NVLink
// store round instead of NCCL's multi-step protocol: what matters for a 32 KB sum issued 160 times per token.
#include "comm.cuh"
#include "tma.cuh"
#include "actquant.cuh"

#include <cooperative_groups.h>

#include <dlfcn.h>
#include <cstring>
#include <mutex>
#include <vector>
#include <cstdlib>

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

constexpr int P2P_MAX_WORLD = 8;
constexpr int P2P_CTA_ELEMS = 1024;                 // floats per CTA (256 threads x float4)
constexpr int P2P_MAX_CTAS = 64;
constexpr int P2P_MAX_ELEMS = P2P_CTA_ELEMS * P2P_MAX_CTAS;
constexpr int P2P_SPIN_LIMIT = 1 << 25;             // several seconds of polling (ranks may enter their first step apart), then the kernel gives up and reports

// Per-rank region, identical layout on every rank:
//   inbox [2][world][P2P_MAX_ELEMS] float | flags [world][P2P_MAX_CTAS] int | seq [P2P_MAX_CTAS] int (local only)
struct P2PView {
    float* inbox[P2P_MAX_WORLD];    // base of each rank's channel as mapped into this process
    int rank, world;
};
static size_t p2p_channel_bytes(int world) {
    return (size_t) 2 * world * P2P_MAX_ELEMS * 4 + (size_t) world * P2P_MAX_CTAS * 4 + P2P_MAX_CTAS * 4;
}
// Two channels with the layout above: channel 0 for the plain all-reduce (slot = 1024 floats), channel 1 for the
// fused all-reduce + RMSNorm + quantize (slot = 2048 floats). Inside a channel a slot always covers the same
// floats, which is what lets the two inbox copies alternate safely; mixing slot sizes in one channel would not.
static size_t p2p_region_bytes(int world) { return 2 * ((p2p_channel_bytes(world) + 255) & ~(size_t) 255); }
__device__ __forceinline__ int* p2p_flags(float* base, int world) { return (int*) (base + (size_t) 2 * world * P2P_MAX_ELEMS); }

__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(P2PView v, float* __restrict__ buf, int n, int* __restrict__ timeout_flag) {
    __shared__ int s_seq;
    skd::pdl_launch_dependents();
    const int cta = blockIdx.x, world = v.world, rank = v.rank;
    float* mine = v.inbox[rank];
    int* my_flags = p2p_flags(mine, world);
    int* seq_slot = my_flags + world * P2P_MAX_CTAS + cta;
    const int i = cta * P2P_CTA_ELEMS + threadIdx.x * 4;          // this thread's float4
    const bool live = i < n;                                      // n is a multiple of 4
    // buf is the predecessor's output, and the round counter is the previous round's: nothing is read before
    // every earlier kernel of the stream has completed
    skd::pdl_wait();
    if (threadIdx.x == 0) s_seq = *seq_slot + 1;
    __syncthreads();
    const int seq = s_seq, par = seq & 1;
    float4 own = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        own = *reinterpret_cast<const float4*>(buf + i);
        for (int p = 0; p < world; ++p)
            if (p != rank) *reinterpret_cast<float4*>(v.inbox[p] + ((size_t) par * world + rank) * P2P_MAX_ELEMS + i) = own;
    }
    __syncthreads();
    if (threadIdx.x < world && (int) threadIdx.x != rank) {
        // publish: the barrier above ordered the CTA's stores before this thread; the fence and the release
        // store make them visible system-wide before the number is
        __threadfence_system();
        int* peer_flag = p2p_flags(v.inbox[threadIdx.x], world) + rank * P2P_MAX_CTAS + cta;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flag), "r"(seq) : "memory");
        // wait for the same peer's number (bounded)
        const int* f = my_flags + threadIdx.x * P2P_MAX_CTAS + cta;
        int got = 0, spins = 0;
        do {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(got) : "l"(f) : "memory");
        } while (got < seq && ++spins < P2P_SPIN_LIMIT);
        if (got < seq && timeout_flag) atomicExch(timeout_flag, 2);
    }
    __syncthreads();
    if (live) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < world; ++p) {
            const float4 x = p == rank ? own : __ldcg(reinterpret_cast<const float4*>(mine + ((size_t) par * world + p) * P2P_MAX_ELEMS + i));
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        *reinterpret_cast<float4*>(buf + i) = acc;
    }
    if (threadIdx.x == 0) *seq_slot = seq;
}

// All-reduce of rows of x over the group fused with what always follows it in the decoder: RMSNorm with weights
// gamma and the int8-per-256 activation quantizer. One thread-block cluster per row, one CTA per 2048 floats
// (256 threads x 8): exchange and sum as above (the sum is also written back to x, the residual stream), then the
// CTAs of the cluster add up their sums of squares through distributed shared memory and each normalises and
// quantizes its own 2048 values (one warp = one 256-block, as in prep_kernel).
constexpr int P2P_FUSED_CTA_ELEMS = 2048;
__global__ void __launch_bounds__(256)
allreduce_norm_quant_kernel(P2PView v, float* __restrict__ x, int n, const float* __restrict__ gamma, float eps, ActQ8K act,
                            int* __restrict__ timeout_flag) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ int s_seq;
    __shared__ float s_red[8];
    __shared__ float s_part;                           // this CTA's sum of squares, read by the whole cluster
    skd::pdl_launch_dependents();
    const int cs = gridDim.x, cx = blockIdx.x, row = blockIdx.y;
    const int cta = row * cs + cx, world = v.world, rank = v.rank;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* mine = v.inbox[rank];
    int* my_flags = p2p_flags(mine, world);
    int* seq_slot = my_flags + world * P2P_MAX_CTAS + cta;
    const int col = cx * P2P_FUSED_CTA_ELEMS + threadIdx.x * 8;           // this thread's 8 floats of the row
    const int64_t i = (int64_t) cta * P2P_FUSED_CTA_ELEMS + threadIdx.x * 8;   // ... and of the inbox
    float* xr = x + (size_t) row * n + col;
    skd::pdl_wait();
    if (threadIdx.x == 0) s_seq = *seq_slot + 1;
    __syncthreads();
    const int seq = s_seq, par = seq & 1;
    const float4 own0 = *reinterpret_cast<const float4*>(xr), own1 = *reinterpret_cast<const float4*>(xr + 4);
    for (int p = 0; p < world; ++p)
        if (p != rank) {
            float* dst = v.inbox[p] + ((size_t) par * world + rank) * P2P_MAX_ELEMS + i;
            *reinterpret_cast<float4*>(dst) = own0; *reinterpret_cast<float4*>(dst + 4) = own1;
        }
    __syncthreads();
    if (threadIdx.x < world && (int) threadIdx.x != rank) {
        __threadfence_system();
        int* peer_flag = p2p_flags(v.inbox[threadIdx.x], world) + rank * P2P_MAX_CTAS + cta;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flag), "r"(seq) : "memory");
        const int* f = my_flags + threadIdx.x * P2P_MAX_CTAS + cta;
        int got = 0, spins = 0;
        do {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(got) : "l"(f) : "memory");
        } while (got < seq && ++spins < P2P_SPIN_LIMIT);
        if (got < seq && timeout_flag) atomicExch(timeout_flag, 2);
    }
    __syncthreads();
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < world; ++p) {                  // rank order: every rank gets the same bits
        float4 u0 = own0, u1 = own1;
        if (p != rank) {
            const float* src = mine + ((size_t) par * world + p) * P2P_MAX_ELEMS + i;
            u0 = __ldcg(reinterpret_cast<const float4*>(src)); u1 = __ldcg(reinterpret_cast<const float4*>(src + 4));
        }
        a[0] += u0.x; a[1] += u0.y; a[2] += u0.z; a[3] += u0.w; a[4] += u1.x; a[5] += u1.y; a[6] += u1.z; a[7] += u1.w;
    }
    *reinterpret_cast<float4*>(xr) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(xr + 4) = make_float4(a[4], a[5], a[6], a[7]);
    if (threadIdx.x == 0) *seq_slot = seq;
    // sum of squares of the row: warp, CTA, cluster (fixed orders)
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += a[k] * a[k];
    ss = skd::warp_sum(ss);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += s_red[k];
        s_part = t;
    }
    cluster.sync();
    float total = 0.0f;
    for (int r = 0; r < cs; ++r) total += *cluster.map_shared_rank(&s_part, r);
    cluster.sync();                                    // nobody leaves while its shared memory may still be read
    const float nscale = 1.0f / sqrtf(total * (1.0f / (float) n) + eps);
    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + col)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + col + 4));
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = (a[k] * nscale) * g[k];
    const int blk = col >> 8;
    skd::quant_q8k_regs(a, act.q + (size_t) row * n + (size_t) blk * 256, act.d + (size_t) row * (n >> 8) + blk,
                        act.bsums + (size_t) row * (n >> 5) + (size_t) blk * 8, lane);
}

struct Comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    bool p2p = false;
    P2PView view = {};              // channel 0: plain all-reduce
    P2PView view_fused = {};        // channel 1: all-reduce + RMSNorm + quantize
    void* region = nullptr;          // this rank's region (cudaMalloc)
    void* peers[P2P_MAX_WORLD] = {}; // opened IPC mappings (null for self)
};

// Exchanges IPC handles of the per-rank regions through NCCL and maps every peer's region. Any failure
// leaves the communicator on NCCL only.
static void p2p_setup(Comm* c) {
    static const bool off = []() { const char* e = getenv("SKAINET_TP_ALLREDUCE"); return e && strcmp(e, "nccl") == 0; }();
    if (off || c->world < 2 || c->world > P2P_MAX_WORLD) return;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    const size_t bytes = p2p_region_bytes(c->world);
    if (cudaMalloc(&c->region, bytes) != cudaSuccess) { c->region = nullptr; cudaGetLastError(); return; }
    cudaMemset(c->region, 0, bytes);
    cudaIpcMemHandle_t h;
    void* d_send = nullptr; void* d_recv = nullptr;
    std::vector<cudaIpcMemHandle_t> all(c->world);
    bool ok = cudaIpcGetMemHandle(&h, c->region) == cudaSuccess && cudaMalloc(&d_send, sizeof(h)) == cudaSuccess &&
              cudaMalloc(&d_recv, sizeof(h) * c->world) == cudaSuccess;
    // every rank takes part in the gather even when its own preparation failed (a zero handle then fails to open)
    if (!ok) memset(&h, 0, sizeof(h));
    if (d_send && d_recv) {
        cudaMemcpy(d_send, &h, sizeof(h), cudaMemcpyHostToDevice);
        ok = g_nccl.AllGather(d_send, d_recv, sizeof(h), ncclInt8, c->comm, (cudaStream_t) 0) == 0 && ok;
        ok = cudaStreamSynchronize(0) == cudaSuccess && ok;
        cudaMemcpy(all.data(), d_recv, sizeof(h) * c->world, cudaMemcpyDeviceToHost);
    } else ok = false;
    cudaFree(d_send); cudaFree(d_recv);
    for (int p = 0; ok && p < c->world; ++p) {
        if (p == c->rank) { c->view.inbox[p] = (float*) c->region; continue; }
        if (cudaIpcOpenMemHandle(&c->peers[p], all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { ok = false; c->peers[p] = nullptr; break; }
        c->view.inbox[p] = (float*) c->peers[p];
    }
    // agree: the fast path is used only when every rank mapped every peer
    int* d_ok = nullptr;
    int mine = ok ? 1 : 0, sum = 0;
    if (cudaMalloc(&d_ok, sizeof(int)) == cudaSuccess) {
        float f = (float) mine;
        cudaMemcpy(d_ok, &f, sizeof(float), cudaMemcpyHostToDevice);
        if (g_nccl.AllReduce(d_ok, d_ok, 1, ncclFloat32, ncclSum, c->comm, (cudaStream_t) 0) == 0 && cudaStreamSynchronize(0) == cudaSuccess) {
            cudaMemcpy(&f, d_ok, sizeof(float), cudaMemcpyDeviceToHost);
            sum = (int) f;
        }
        cudaFree(d_ok);
    }
    cudaGetLastError();
    c->view.rank = c->rank; c->view.world = c->world;
    c->view_fused = c->view;
    const size_t ch = (p2p_channel_bytes(c->world) + 255) & ~(size_t) 255;
    for (int p = 0; p < c->world; ++p)
        if (c->view.inbox[p]) c->view_fused.inbox[p] = (float*) ((uint8_t*) c->view.inbox[p] + ch);
    c->p2p = sum == c->world;
}

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
    p2p_setup(c);
    *out = c;
    return SKAINET_CUDA_OK;
}

void comm_destroy(Comm* c) {
    if (!c) return;
    for (int p = 0; p < P2P_MAX_WORLD; ++p)
        if (c->peers[p]) cudaIpcCloseMemHandle(c->peers[p]);
    if (c->region) cudaFree(c->region);
    if (c->comm && g_nccl.ok) g_nccl.CommDestroy(c->comm);
    delete c;
}

int32_t comm_all_reduce_sum(Comm* c, float* buf, int64_t n, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    if (c->p2p && n <= P2P_MAX_ELEMS && n % 4 == 0 && ((uintptr_t) buf & 15) == 0) {
        const int ctas = (int) ((n + P2P_CTA_ELEMS - 1) / P2P_CTA_ELEMS);
        SK_CUDA(launch_pdl(allreduce_oneshot_kernel, dim3(ctas), dim3(256), 0, s, c->view, buf, (int) n, device_timeout_flag()));
        return SKAINET_CUDA_OK;
    }
    const ncclResult_t r = g_nccl.AllReduce(buf, buf, (size_t) n, ncclFloat32, ncclSum, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllReduce");
}

// In place: x[rows][n] <- sum over the group; act <- quantize(rmsnorm(x, gamma)). Returns 1 when the fused kernel
// does not apply (no peer mapping, shapes outside its slots): the caller then runs the two steps separately.
int32_t comm_all_reduce_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s) {
    static const bool off = []() { const char* e = getenv("SKAINET_TP_FUSE"); return e && strcmp(e, "0") == 0; }();
    if (off || !c || !c->p2p || n % P2P_FUSED_CTA_ELEMS != 0) return 1;
    const int cs = n / P2P_FUSED_CTA_ELEMS;
    if (cs > 8 || rows * cs > P2P_MAX_CTAS || (int64_t) rows * n > P2P_MAX_ELEMS || ((uintptr_t) x & 15) != 0) return 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs, rows); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = cs; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs; cfg.numAttrs = 2;
    SK_CUDA(cudaLaunchKernelEx(&cfg, allreduce_norm_quant_kernel, c->view_fused, x, n, gamma, eps, act, device_timeout_flag()));
    return SKAINET_CUDA_OK;
}

int32_t comm_all_gather(Comm* c, const void* send, void* recv, int64_t nbytes, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    const ncclResult_t r = g_nccl.AllGather(send, recv, (size_t) nbytes, ncclInt8, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllGather");
}

}  // namespace sk
