// Measurement aid: a kernel that only READS a resident weight's planes (128-bit loads, every byte once,
// nothing computed). Timed by the bench next to the matvec over the same bytes, it gives the floor a
// launch of that size can reach on this GPU, which for small weights is well under the streaming peak.
#include "common.cuh"
#include "tma.cuh"

namespace sk {

__global__ void __launch_bounds__(512) probe_read_kernel(const uint4* __restrict__ a, size_t na, const uint4* __restrict__ b, size_t nb,
                                                         uint32_t* __restrict__ sink) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    uint32_t acc = 0;
    const size_t stride = (size_t) gridDim.x * blockDim.x, t = blockIdx.x * (size_t) blockDim.x + threadIdx.x;
    size_t i = t;
    for (; i + 3 * stride < na; i += 4 * stride) {
        const uint4 v0 = skd::ld_stream(a + i), v1 = skd::ld_stream(a + i + stride), v2 = skd::ld_stream(a + i + 2 * stride), v3 = skd::ld_stream(a + i + 3 * stride);
        acc ^= v0.x ^ v0.y ^ v0.z ^ v0.w ^ v1.x ^ v1.y ^ v1.z ^ v1.w ^ v2.x ^ v2.y ^ v2.z ^ v2.w ^ v3.x ^ v3.y ^ v3.z ^ v3.w;
    }
    for (; i < na; i += stride) { const uint4 v = skd::ld_stream(a + i); acc ^= v.x ^ v.y ^ v.z ^ v.w; }
    for (i = t; i < nb; i += stride) { const uint4 v = skd::ld_stream(b + i); acc ^= v.x ^ v.y ^ v.z ^ v.w; }
    if (acc == 0x9e3779b9u) sink[0] = acc;      // keeps the loads alive; practically never true
}

int32_t launch_probe_read(const Weight& w, uint32_t* sink, cudaStream_t s) {
    const size_t nblk = (size_t) w.rows * w.bpr;
    const size_t qs_b = w.enc == SKAINET_ENC_Q8_0 ? 32 : 128, hdr_b = w.enc == SKAINET_ENC_Q8_0 ? 2 : 16;
    if (w.enc == SKAINET_ENC_Q5_K || w.enc == SKAINET_ENC_Q6_K) {
        // four planes in one allocation (256-byte aligned, in this order): read the span from the first to the end of the last
        const uint8_t* end = w.enc == SKAINET_ENC_Q6_K ? (const uint8_t*) w.aux + nblk * 2 : (const uint8_t*) w.extra + nblk * 32;
        const size_t span = (size_t) (end - (const uint8_t*) w.qs);
        SK_CUDA(launch_pdl(probe_read_kernel, dim3(sm_count() * 4), dim3(512), 0, s, (const uint4*) w.qs, (span + 15) / 16, (const uint4*) w.hdr, (size_t) 0, sink));
        return SKAINET_CUDA_OK;
    }
    SK_CUDA(launch_pdl(probe_read_kernel, dim3(sm_count() * 4), dim3(512), 0, s, (const uint4*) w.qs, nblk * qs_b / 16,
                       (const uint4*) w.hdr, nblk * hdr_b / 16, sink));
    return SKAINET_CUDA_OK;
}

// Self-test of the failure path every kernel here shares: one thread waits on a shared-memory barrier that
// nothing ever completes. The wait is bounded, so the kernel gives up after its poll limit, raises the device
// flag and returns normally: no trap, no fault, the context stays usable.
__global__ void bounded_wait_selftest_kernel(int* __restrict__ timeout_flag, int* __restrict__ reached_end) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { skd::mbar_init(&bar, 1); skd::mbar_fence_init(); }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = skd::mbar_wait_bounded(&bar, 0, timeout_flag);
    __syncthreads();
    if (threadIdx.x == 0) *reached_end = ok ? 1 : 2;
}

int32_t launch_bounded_wait_selftest(int* reached_end, cudaStream_t s) {
    bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(device_timeout_flag(), reached_end);
    SK_CUDA(cudaGetLastError());
    return SKAINET_CUDA_OK;
}

}  // namespace sk
