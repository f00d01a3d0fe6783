// Collectives for tensor parallelism over NVLink/NVSwitch. NCCL is bound at run time (dlopen of
// libnccl.so.2: the copy PyTorch already loaded when the host is a torch process, the system one
// otherwise), so the library loads and runs single-GPU where NCCL is absent.
#pragma once
#include "common.cuh"

namespace sk {

struct Comm;

int32_t comm_unique_id(uint8_t* id128);
int32_t comm_create(int rank, int world, const uint8_t* id128, Comm** out);
void comm_destroy(Comm* c);
// in place, fp32, sum over the group
int32_t comm_all_reduce_sum(Comm* c, float* buf, int64_t n, cudaStream_t s);
// x[rows][n] <- group sum; act <- int8-per-256 quantization of rmsnorm(x, gamma). 1 = not applicable (do it in two steps)
struct ActQ8K;
int32_t comm_all_reduce_norm_quant(Comm* c, float* x, int rows, int n, const float* gamma, float eps, ActQ8K act, cudaStream_t s);
// recv[world][nbytes] <- send[nbytes] of every rank
int32_t comm_all_gather(Comm* c, const void* send, void* recv, int64_t nbytes, cudaStream_t s);

}  // namespace sk
