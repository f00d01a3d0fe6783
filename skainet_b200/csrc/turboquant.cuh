// Interface of the TurboQuant KV codec kernels (turboquant.cu), used by the KV store (kvstore.cu).
#pragma once
#include "common.cuh"
#include <cuda_fp16.h>

namespace sk {

// One plane (keys or values) of a TurboQuant store: per (layer, position, head) vector, indexed
// ((layer * max_seq + position) * heads + head).
struct TqPlane {
    uint8_t* codes = nullptr;     // [vectors][packed_size(head_dim, bits)]
    float* scales = nullptr;      // [vectors][head_dim / 32]
    uint8_t* resid = nullptr;     // [vectors][packed_size(head_dim, rbits)]   (rbits > 0)
    float* rscale = nullptr;      // [vectors]                                  (rbits > 0)
    // Not part of a block: the sign sequences of the rotation (and of the 1-bit residual), kept beside the blocks when
    // non-null so that a read does not have to re-run the sequential generator per vector (head_dim / 8 bytes each).
    uint32_t* signs = nullptr;    // [vectors][head_dim / 32]
    uint32_t* rsigns = nullptr;   // [vectors][head_dim / 32]                   (rbits == 1)
    int bits = 4;                 // 2, 3, 4 or 8
    int rbits = 0;                // 0: rotation + scalar quantizer only; 1..4: with the residual stage
};

// BitPacker.packedSize; one bit per element for the 1-bit residual (QjlResidual.kt:36)
__host__ __device__ inline int tq_packed_size(int count, int bits) {
    return bits == 1 ? (count + 7) / 8 : bits == 2 ? (count + 3) / 4 : bits == 3 ? (count * 3 + 7) / 8 : bits == 4 ? (count + 1) / 2 : count;
}
// TurboQuantBlock.sizeInBytes: codes + scales + the 4-byte seed (+ the packed residual)
inline int64_t tq_block_bytes(int head_dim, int bits, int rbits) {
    return tq_packed_size(head_dim, bits) + (head_dim / 32) * 4 + 4 + (rbits ? tq_packed_size(head_dim, rbits) : 0);
}

// rows [heads][head_dim] fp32 (device) -> the blocks of (layer, pos, every head). seed_xor: 0 for keys, 0x5A5A5A5A for values.
int32_t launch_tq_encode(const float* rows, const TqPlane& pl, int layer, int pos, int heads, int head_dim, int max_seq, int32_t seed_xor, cudaStream_t s,
                         bool fixed_seed = false);      // fixed_seed: seed_xor is the seed itself (one-vector codec entries)
// positions [start_pos, start_pos + n) of a layer -> out [heads][n][head_dim] fp32 (device)
int32_t launch_tq_decode(const TqPlane& pl, int layer, int start_pos, int n, int heads, int head_dim, int max_seq, int32_t seed_xor, float* out, cudaStream_t s,
                         bool fixed_seed = false);
// the same rows rounded to binary16 (the layout the decode-attention kernel reads: [heads][n][head_dim])
int32_t launch_tq_decode_f16(const TqPlane& pl, int layer, int start_pos, int n, int heads, int head_dim, int max_seq, int32_t seed_xor, __half* out, cudaStream_t s);

}  // namespace sk
