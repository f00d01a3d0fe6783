// Collectives for tensor parallelism over NVLink/NVSwitch. NCCL is bound at run time (dlopen of
// libnccl.so.2: the copy PyTorch already loaded when the host is a torch process, the system one
// otherwise), so the library loads and runs single-GPU where NCCL is absent.
#pragma once
#include "common.cuh"

namespace sk {

struct Comm;

constexpr int P2P_MAX_WORLD = 8;
constexpr int P2P_MAX_ELEMS = 65536;                // floats per inbox slot (8 rows of 8192)

// Where the epilogue of a row-parallel matvec stores its output rows so that the group sum needs no separate send:
// slot `rank` of the current inbox copy of every rank (this one included), element index = output row. Words are
// self-validating (see comm.cu): a value whose bits equal the sentinel is sent as another NaN pattern.
struct PeerOut {
    uint32_t* inbox[P2P_MAX_WORLD];   // channel base in each rank's region, as mapped into this process
    const int* round;                 // this rank's round counter of the channel (its parity picks the inbox copy)
    int world = 0, rank = 0;          // world == 0: no peer output
};

int32_t comm_unique_id(uint8_t* id128);
int32_t comm_create(int rank, int world, const uint8_t* id128, Comm** out);
void comm_destroy(Comm* c);
// in place, fp32, sum over the group
int32_t comm_all_reduce_sum(Comm* c, float* buf, int64_t n, cudaStream_t s);
// the same sum through NCCL whatever the size (the measurement entry compares the two)
int32_t comm_all_reduce_sum_nccl(Comm* c, float* buf, int64_t n, cudaStream_t s);
// x[rows][n] <- group sum; act <- int8-per-256 quantization of rmsnorm(x, gamma). 1 = not applicable (do it in two steps)
struct ActQ8K;
int32_t comm_all_reduce_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s);
#ifdef __CUDACC__
// Four consecutive output rows (first row a multiple of 4) into slot `rank` of the inbox copy `par` of every rank.
__device__ __forceinline__ void peer_store4(const PeerOut& po, int par, int p, int row, float a, float b, float c, float d) {
    auto word = [](float v) { const uint32_t u = __float_as_uint(v); return u == 0xFFFFFFFFu ? 0x7FFFFFFFu : u; };
    uint32_t* dst = po.inbox[p] + ((size_t) par * po.world + po.rank) * P2P_MAX_ELEMS + row;
    *reinterpret_cast<uint4*>(dst) = make_uint4(word(a), word(b), word(c), word(d));
}
__device__ __forceinline__ void peer_store1(const PeerOut& po, int par, int p, int row, float a) {
    const uint32_t u = __float_as_uint(a);
    po.inbox[p][((size_t) par * po.world + po.rank) * P2P_MAX_ELEMS + row] = u == 0xFFFFFFFFu ? 0x7FFFFFFFu : u;
}
#endif

// The peer-output descriptor for a row-parallel matvec of `rows` activation rows by n outputs; false when the
// peer-memory path does not apply (then the matvec writes locally and comm_all_reduce_norm_quant sends).
bool comm_peer_out(Comm* c, int rows, int n, PeerOut* out);
// The receiving half alone: the matvec epilogues have stored every rank's partial rows through a PeerOut;
// x[rows][n] <- their sum, act <- int8-per-256 quantization of rmsnorm(x, gamma).
int32_t comm_gather_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s);
// recv[world][nbytes] <- send[nbytes] of every rank
int32_t comm_all_gather(Comm* c, const void* send, void* recv, int64_t nbytes, cudaStream_t s);

}  // namespace sk
