// NCCL binding by dlopen (see comm.cuh), only the entry points the decoder needs (setup, the arg-max gather, large sums),
// plus the group exchanges of a decode step over peer memory: an in-place sum of a small vector, and the gather of the
// rows a row-parallel matvec produced, fused with the RMSNorm and the activation quantizer that always follow it.
// The protocol (no flags: every word of an inbox carries its own arrival state) is described where the kernels are.
// Latency is one NVLink store instead of NCCL's multi-step protocol: what matters for a 32 KB sum issued 160 times per token.
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
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
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
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort)) sym("ncclCommAbort");
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

// ------------------------------------------------------------------------------------------------
// Peer-memory exchange without flags. Every 32-bit word of an inbox carries its own arrival state: an inbox
// is filled with a sentinel bit pattern, a sender stores plain data words over NVLink, and the receiver polls
// the words themselves until none is the sentinel (a data word that happens to equal it is replaced by another
// NaN pattern before it is sent). There is no flag, no fence and no second round trip: the cost of a sum is one
// NVLink store latency. The receiver puts the sentinel back as soon as it has read a word, so an inbox cleans
// itself; two inbox copies alternate by round because a fast peer may already send round r+1 while this rank
// still reads round r (it cannot reach r+2 before this rank has finished r: it needs this rank's r+1 data).
//
// Per-rank region, identical layout on every rank (peers map it through CUDA IPC):
//   channel A  [2][world][P2P_MAX_ELEMS] words   in-place all-reduce of a vector (allreduce_words_kernel)
//   channel B  [2][world][P2P_MAX_ELEMS] words   outputs of a row-parallel matvec, written by the matvec's own
//                                                epilogue (matvec_fused.cu / matvec_ring.cu) or by the receiving
//                                                kernel itself, summed + RMS-normalised + quantized on arrival
//   control    seqA[P2P_MAX_CTAS] | roundB | ticketB     (local only, zeroed)
// ------------------------------------------------------------------------------------------------
constexpr int P2P_CTA_ELEMS = 1024;                 // floats per CTA of the vector all-reduce (256 threads x float4)
constexpr int P2P_MAX_CTAS = P2P_MAX_ELEMS / P2P_CTA_ELEMS;
constexpr int P2P_SPIN_LIMIT = 1 << 24;             // seconds of polling (ranks may enter their first step apart), then the kernel gives up and reports
constexpr uint32_t P2P_SENTINEL = 0xFFFFFFFFu;
constexpr uint32_t P2P_SENTINEL_ALIAS = 0x7FFFFFFFu;   // what a data word equal to the sentinel is sent as (both are NaNs)

static size_t p2p_channel_bytes(int world) { return (size_t) 2 * world * P2P_MAX_ELEMS * 4; }
static size_t p2p_ctl_bytes() { return ((size_t) (P2P_MAX_CTAS + 2) * 4 + 255) & ~(size_t) 255; }
static size_t p2p_region_bytes(int world) { return 2 * p2p_channel_bytes(world) + p2p_ctl_bytes(); }

struct P2PView {
    uint32_t* chan[P2P_MAX_WORLD];   // base of one channel in each rank's region, as mapped into this process
    int* ctl;                        // this rank's control words
    int rank, world;
};

__device__ __forceinline__ uint32_t p2p_word(float v) {
    const uint32_t u = __float_as_uint(v);
    return u == P2P_SENTINEL ? P2P_SENTINEL_ALIAS : u;
}
__device__ __forceinline__ uint4 p2p_words(float4 v) { return make_uint4(p2p_word(v.x), p2p_word(v.y), p2p_word(v.z), p2p_word(v.w)); }
__device__ __forceinline__ uint4 ld_volatile_u4(const uint32_t* p) {
    uint4 r;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ bool p2p_pending(const uint4& r) { return r.x == P2P_SENTINEL || r.y == P2P_SENTINEL || r.z == P2P_SENTINEL || r.w == P2P_SENTINEL; }
// Waits (bounded) until the four words at p have all arrived, returns them and puts the sentinel back.
__device__ __forceinline__ float4 p2p_take(uint32_t* p, int* timeout_flag) {
    uint4 r = ld_volatile_u4(p);
    int spins = 0;
    while ((r.x == P2P_SENTINEL || r.y == P2P_SENTINEL || r.z == P2P_SENTINEL || r.w == P2P_SENTINEL) && ++spins < P2P_SPIN_LIMIT) r = ld_volatile_u4(p);
    if (spins >= P2P_SPIN_LIMIT && timeout_flag) atomicExch(timeout_flag, 2);
    *reinterpret_cast<uint4*>(p) = make_uint4(P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL);
    return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z), __uint_as_float(r.w));
}

// In-place sum of buf[n] over the group (n a multiple of 4, n <= P2P_MAX_ELEMS). CTA c owns floats
// [1024 c, 1024 (c+1)); its round counter picks the inbox copy. Slots are summed in rank order, so every rank
// gets the same bits.
__global__ void __launch_bounds__(256)
allreduce_words_kernel(P2PView v, float* __restrict__ buf, int n, int* __restrict__ timeout_flag) {
    __shared__ int s_seq;
    skd::pdl_launch_dependents();
    const int cta = blockIdx.x, world = v.world, rank = v.rank;
    int* seq_slot = v.ctl + cta;
    const int i = cta * P2P_CTA_ELEMS + threadIdx.x * 4;          // this thread's float4
    const bool live = i < n;
    // buf is the predecessor's output, and the round counter is the previous round's: nothing is read before
    // every earlier kernel of the stream has completed
    skd::pdl_wait();
    if (threadIdx.x == 0) s_seq = *seq_slot + 1;
    __syncthreads();
    const int seq = s_seq, par = seq & 1;
    if (live) {
        const float4 own = *reinterpret_cast<const float4*>(buf + i);
        const uint4 mine = p2p_words(own);
        for (int p = 0; p < world; ++p)
            if (p != rank) *reinterpret_cast<uint4*>(v.chan[p] + ((size_t) par * world + rank) * P2P_MAX_ELEMS + i) = mine;
        uint32_t* src0 = v.chan[rank] + (size_t) par * world * P2P_MAX_ELEMS + i;
        uint4 w[P2P_MAX_WORLD];
#pragma unroll
        for (int p = 0; p < P2P_MAX_WORLD; ++p)
            if (p < world && p != rank) w[p] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS);
        for (int spins = 0; ; ++spins) {
            bool missing = false;
#pragma unroll
            for (int p = 0; p < P2P_MAX_WORLD; ++p)
                if (p < world && p != rank && p2p_pending(w[p])) { w[p] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS); missing = true; }
            if (!missing) break;
            if (spins >= P2P_SPIN_LIMIT) { if (timeout_flag) atomicExch(timeout_flag, 2); break; }
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < P2P_MAX_WORLD; ++p)          // rank order: every rank gets the same bits
            if (p < world) {
                float4 x = own;
                if (p != rank) {
                    *reinterpret_cast<uint4*>(src0 + (size_t) p * P2P_MAX_ELEMS) = make_uint4(P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL);
                    x = make_float4(__uint_as_float(w[p].x), __uint_as_float(w[p].y), __uint_as_float(w[p].z), __uint_as_float(w[p].w));
                }
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
            }
        *reinterpret_cast<float4*>(buf + i) = acc;
    }
    if (threadIdx.x == 0) *seq_slot = seq;
}

// Sum over the group of the rows a row-parallel matvec produced, fused with what always follows it in the decoder:
// the sum is written to x (the residual stream), RMS-normalised with gamma and quantized to int8 per 256 for the
// next matvec. One thread-block cluster per row, one CTA per 2048 floats (256 threads x 8). With SEND the kernel
// first stores this rank's partial row (in x) into every inbox; without, the matvec's epilogue has already done
// so (matvec_fused.cu, matvec_ring.cu: EPI_PEER) and x is only written. The CTAs of the cluster add up their sums
// of squares through distributed shared memory. The CTA that finishes last advances the channel's round.
constexpr int P2P_FUSED_CTA_ELEMS = 2048;
template <bool SEND>
__global__ void __launch_bounds__(256)
gather_sum_norm_quant_kernel(P2PView v, float* __restrict__ x, int n, const float* __restrict__ gamma, float eps, ActQ8K act,
                             int* __restrict__ timeout_flag) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float s_red[8];
    __shared__ float s_parts[8];                       // the sums of squares of the cluster's CTAs (at most 8), each written by its owner
    skd::pdl_launch_dependents();
    const int cs = gridDim.x, cx = blockIdx.x, row = blockIdx.y;
    const int world = v.world, rank = v.rank;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int* round_ctr = v.ctl + P2P_MAX_CTAS;
    int* ticket = round_ctr + 1;
    const int col = cx * P2P_FUSED_CTA_ELEMS + threadIdx.x * 8;           // this thread's 8 floats of the row
    const int64_t i = (int64_t) row * n + col;                              // ... and of every inbox slot
    float* xr = x + i;
    skd::pdl_wait();
    const int par = *reinterpret_cast<volatile int*>(round_ctr) & 1;
    if (SEND) {
        const uint4 w0 = p2p_words(*reinterpret_cast<const float4*>(xr)), w1 = p2p_words(*reinterpret_cast<const float4*>(xr + 4));
        for (int p = 0; p < world; ++p) {
            uint32_t* dst = v.chan[p] + ((size_t) par * world + rank) * P2P_MAX_ELEMS + i;
            *reinterpret_cast<uint4*>(dst) = w0; *reinterpret_cast<uint4*>(dst + 4) = w1;
        }
    }
    // gamma does not depend on the peers: fetch it before the wait
    const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + col)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + col + 4));
    // every slot's words are requested at once; only the ones that have not arrived are asked for again
    uint32_t* src0 = v.chan[rank] + (size_t) par * world * P2P_MAX_ELEMS + i;
    uint4 w[2 * P2P_MAX_WORLD];
#pragma unroll
    for (int p = 0; p < P2P_MAX_WORLD; ++p)
        if (p < world) { w[2 * p] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS); w[2 * p + 1] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS + 4); }
    for (int spins = 0; ; ++spins) {
        bool missing = false;
#pragma unroll
        for (int p = 0; p < P2P_MAX_WORLD; ++p)
            if (p < world) {
                if (p2p_pending(w[2 * p])) { w[2 * p] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS); missing = true; }
                if (p2p_pending(w[2 * p + 1])) { w[2 * p + 1] = ld_volatile_u4(src0 + (size_t) p * P2P_MAX_ELEMS + 4); missing = true; }
            }
        if (!missing) break;
        if (spins >= P2P_SPIN_LIMIT) { if (timeout_flag) atomicExch(timeout_flag, 2); break; }
    }
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const uint4 sent = make_uint4(P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL, P2P_SENTINEL);
#pragma unroll
    for (int p = 0; p < P2P_MAX_WORLD; ++p)              // rank order: every rank gets the same bits
        if (p < world) {
            *reinterpret_cast<uint4*>(src0 + (size_t) p * P2P_MAX_ELEMS) = sent;          // the inbox cleans itself
            *reinterpret_cast<uint4*>(src0 + (size_t) p * P2P_MAX_ELEMS + 4) = sent;
            a[0] += __uint_as_float(w[2 * p].x); a[1] += __uint_as_float(w[2 * p].y); a[2] += __uint_as_float(w[2 * p].z); a[3] += __uint_as_float(w[2 * p].w);
            a[4] += __uint_as_float(w[2 * p + 1].x); a[5] += __uint_as_float(w[2 * p + 1].y); a[6] += __uint_as_float(w[2 * p + 1].z); a[7] += __uint_as_float(w[2 * p + 1].w);
        }
    *reinterpret_cast<float4*>(xr) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(xr + 4) = make_float4(a[4], a[5], a[6], a[7]);
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
        // this CTA's partial goes into slot cx of EVERY CTA of the cluster: after the one barrier below each CTA sums its own
        // copy, and nobody reads another CTA's shared memory afterwards (no second barrier before leaving)
        for (int r = 0; r < cs; ++r) *cluster.map_shared_rank(&s_parts[cx], r) = t;
    }
    cluster.sync();
    float total = 0.0f;
    for (int r = 0; r < cs; ++r) total += s_parts[r];
    const float nscale = 1.0f / sqrtf(total * (1.0f / (float) n) + eps);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = (a[k] * nscale) * g[k];
    const int blk = col >> 8;
    skd::quant_q8k_regs(a, act.q + (size_t) row * n + (size_t) blk * 256, act.d + (size_t) row * (n >> 8) + blk,
                        act.bsums + (size_t) row * (n >> 5) + (size_t) blk * 8, lane);
    // the last CTA of the launch to get here advances the round (every CTA has read it by then)
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1) == (int) (gridDim.x * gridDim.y) - 1) { *ticket = 0; *round_ctr = *round_ctr + 1; }
    }
}

struct Comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    bool p2p = false;
    P2PView view = {};              // channel A: plain all-reduce
    P2PView view_fused = {};        // channel B: row-parallel matvec outputs -> sum + RMSNorm + quantize
    void* region = nullptr;          // this rank's region (cudaMalloc)
    void* peers[P2P_MAX_WORLD] = {}; // opened IPC mappings (null for self)
};

// Exchanges IPC handles of the per-rank regions through NCCL and maps every peer's region. Every rank takes part in
// both collectives below whatever happened to its own preparation (a rank that returned early would leave the others
// waiting inside NCCL): a failed rank contributes a zeroed handle and a "no" vote, and the vote turns the peer-memory
// path off on all ranks together. SKAINET_TP_ALLREDUCE=nccl is such a "no" vote.
static int32_t p2p_setup(Comm* c) {
    if (c->world < 2 || c->world > P2P_MAX_WORLD) return SKAINET_CUDA_OK;      // the same decision on every rank
    const char* env = getenv("SKAINET_TP_ALLREDUCE");
    bool ok = !(env && strcmp(env, "nccl") == 0);
    // the exchange buffers come first: without them this rank could not even take part in the gather
    const size_t hsz = sizeof(cudaIpcMemHandle_t);
    uint8_t* xchg = nullptr;
    if (cudaMalloc((void**) &xchg, hsz * (c->world + 1) + 256) != cudaSuccess) {
        cudaGetLastError();
        if (g_nccl.CommAbort) g_nccl.CommAbort(c->comm);       // releases the peers' collectives with an error instead of a hang
        set_error("tensor-parallel setup: no device memory for the handle exchange");
        return SKAINET_CUDA_ERR_OOM;
    }
    uint8_t* d_send = xchg; uint8_t* d_recv = xchg + hsz; float* d_vote = (float*) (xchg + hsz * (c->world + 1));
    const size_t bytes = p2p_region_bytes(c->world);
    cudaIpcMemHandle_t h;
    memset(&h, 0, sizeof(h));
    if (ok) {
        if (cudaMalloc(&c->region, bytes) != cudaSuccess) { c->region = nullptr; cudaGetLastError(); ok = false; }
        else {
            cudaMemset(c->region, 0xFF, 2 * p2p_channel_bytes(c->world));                                      // inboxes: every word the sentinel
            cudaMemset((uint8_t*) c->region + 2 * p2p_channel_bytes(c->world), 0, p2p_ctl_bytes());              // counters
            if (cudaIpcGetMemHandle(&h, c->region) != cudaSuccess) { cudaGetLastError(); memset(&h, 0, sizeof(h)); ok = false; }
        }
    }
    std::vector<cudaIpcMemHandle_t> all(c->world);
    cudaMemcpy(d_send, &h, hsz, cudaMemcpyHostToDevice);
    bool gathered = g_nccl.AllGather(d_send, d_recv, hsz, ncclInt8, c->comm, (cudaStream_t) 0) == 0;
    gathered = cudaStreamSynchronize(0) == cudaSuccess && gathered;
    if (gathered) cudaMemcpy(all.data(), d_recv, hsz * c->world, cudaMemcpyDeviceToHost); else ok = false;
    uint32_t* base[P2P_MAX_WORLD] = {};
    for (int p = 0; ok && p < c->world; ++p) {
        if (p == c->rank) { base[p] = (uint32_t*) c->region; continue; }
        if (cudaIpcOpenMemHandle(&c->peers[p], all[p], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = false; c->peers[p] = nullptr; break; }
        base[p] = (uint32_t*) c->peers[p];
    }
    // agree: the fast path is used only when every rank mapped every peer
    float vote = ok ? 1.0f : 0.0f;
    int sum = 0;
    cudaMemcpy(d_vote, &vote, sizeof(float), cudaMemcpyHostToDevice);
    if (g_nccl.AllReduce(d_vote, d_vote, 1, ncclFloat32, ncclSum, c->comm, (cudaStream_t) 0) == 0 && cudaStreamSynchronize(0) == cudaSuccess) {
        cudaMemcpy(&vote, d_vote, sizeof(float), cudaMemcpyDeviceToHost);
        sum = (int) vote;
    }
    cudaFree(xchg);
    cudaGetLastError();
    c->p2p = sum == c->world;
    if (c->p2p) {
        c->view.rank = c->view_fused.rank = c->rank; c->view.world = c->view_fused.world = c->world;
        c->view.ctl = c->view_fused.ctl = (int*) ((uint8_t*) c->region + 2 * p2p_channel_bytes(c->world));
        for (int p = 0; p < c->world; ++p) {
            c->view.chan[p] = base[p];
            c->view_fused.chan[p] = (uint32_t*) ((uint8_t*) base[p] + p2p_channel_bytes(c->world));
        }
    }
    return SKAINET_CUDA_OK;
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
    const int32_t st = p2p_setup(c);
    if (st != SKAINET_CUDA_OK) { c->comm = nullptr; comm_destroy(c); return st; }
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
        SK_CUDA(launch_pdl(allreduce_words_kernel, dim3(ctas), dim3(256), 0, s, c->view, buf, (int) n, device_timeout_flag()));
        return SKAINET_CUDA_OK;
    }
    const ncclResult_t r = g_nccl.AllReduce(buf, buf, (size_t) n, ncclFloat32, ncclSum, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllReduce");
}

int32_t comm_all_reduce_sum_nccl(Comm* c, float* buf, int64_t n, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    const ncclResult_t r = g_nccl.AllReduce(buf, buf, (size_t) n, ncclFloat32, ncclSum, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllReduce");
}

static bool fused_shape_ok(const Comm* c, const float* x, int rows, int n) {
    if (!c || !c->p2p || n % P2P_FUSED_CTA_ELEMS != 0) return false;
    const int cs = n / P2P_FUSED_CTA_ELEMS;
    return cs <= 8 && (int64_t) rows * n <= P2P_MAX_ELEMS && ((uintptr_t) x & 15) == 0;
}

template <bool SEND>
static int32_t launch_gather(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s) {
    const int cs = n / P2P_FUSED_CTA_ELEMS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cs, rows); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = cs; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs; cfg.numAttrs = 2;
    SK_CUDA(cudaLaunchKernelEx(&cfg, gather_sum_norm_quant_kernel<SEND>, c->view_fused, x, n, gamma, eps, act, device_timeout_flag()));
    return SKAINET_CUDA_OK;
}

// In place: x[rows][n] <- sum over the group; act <- quantize(rmsnorm(x, gamma)). Returns 1 when the fused kernel
// does not apply (no peer mapping, shapes outside its slots): the caller then runs the two steps separately.
int32_t comm_all_reduce_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s) {
    static const bool off = []() { const char* e = getenv("SKAINET_TP_FUSE"); return e && strcmp(e, "0") == 0; }();
    if (off || !fused_shape_ok(c, x, rows, n)) return 1;
    return launch_gather<true>(c, x, rows, n, gamma, eps, act, s);
}

bool comm_peer_out(Comm* c, int rows, int n, PeerOut* out) {
    static const bool off = []() { const char* e = getenv("SKAINET_TP_FUSE"); return e && (strcmp(e, "0") == 0 || strcmp(e, "1") == 0); }();
    if (off || rows != 1 || !fused_shape_ok(c, nullptr, rows, n)) return false;
    for (int p = 0; p < c->world; ++p) out->inbox[p] = c->view_fused.chan[p];
    out->round = c->view_fused.ctl + P2P_MAX_CTAS;
    out->world = c->world; out->rank = c->rank;
    return true;
}

int32_t comm_gather_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s) {
    if (!fused_shape_ok(c, x, rows, n)) { set_error("comm_gather_norm_quant: shape outside the peer-memory path"); return SKAINET_CUDA_ERR_INVALID; }
    return launch_gather<false>(c, x, rows, n, gamma, eps, act, s);
}

int32_t comm_all_gather(Comm* c, const void* send, void* recv, int64_t nbytes, cudaStream_t s) {
    if (!c) { set_error("tensor-parallel model without a communicator (call llama_tp_init)"); return SKAINET_CUDA_ERR_COMM; }
    const ncclResult_t r = g_nccl.AllGather(send, recv, (size_t) nbytes, ncclInt8, c->comm, s);
    return r == 0 ? SKAINET_CUDA_OK : nccl_fail(r, "ncclAllGather");
}

}  // namespace sk
