// Streaming matvec for decode: the packed weight tile of a CTA arrives in shared memory by TMA bulk
// copies issued by one thread before anything else (so, under programmatic dependent launch, while
// the kernel that produces the activation is still running), the quantized activation is staged
// once per CTA, and each warp keeps its slice of the activation in registers across the rows it owns.
// Shared-memory reads are bank-conflict free by construction (rotated group order for the 128-byte
// code blocks, XOR-swizzled activation chunks), so the only per-byte work is unpack + dp4a.
//
// HBM-bound: algorithmic bytes per launch = rows*(cols/256)*144 (Q4_K) or rows*(cols/32)*34 (Q8_0)
// + activation + 4*rows; arithmetic identical to matvec.cu (see the reference citations there).
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"

namespace sk {

constexpr int MS_WARPS = 4;
constexpr int MS_THREADS = MS_WARPS * 32;
constexpr size_t MS_SMEM_BUDGET = 100 * 1024;   // two CTAs per SM: a successor's prefetch can overlap

static inline size_t up16(size_t x) { return (x + 15) & ~(size_t) 15; }

// ================================================================================================
// Q4_K
// ================================================================================================
// Tile of R = 4*RW rows. Warp w owns rows w, w+4, ... of the tile. A lane pair (slot = lane/2) owns
// block slot + 16*cg of the row in column group cg; lane parity h takes bytes [32g+16h, +16) of each
// 32-byte group g, visiting the groups in the order g = (k + slot) & 3 so that the eight lanes of a
// quarter-warp touch eight distinct 16-byte bank groups.
template <int M, int RW>
__global__ void __launch_bounds__(MS_THREADS)
q4k_matvec_stream_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, int rows, int bpr,
                         ActQ8K act, int cols, float* __restrict__ y, int* __restrict__ timeout_flag) {
    constexpr int R = MS_WARPS * RW;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* s_qs = smem;
    uint8_t* s_hdr = s_qs + (size_t) R * bpr * 128;
    int8_t* s_q8 = (int8_t*) (s_hdr + (size_t) R * bpr * 16);
    int16_t* s_bs = (int16_t*) (s_q8 + (size_t) M * cols);
    uint64_t* bar = (uint64_t*) ((uint8_t*) s_bs + (size_t) M * (cols / 16));

    const int row0 = blockIdx.x * R;
    const int nrows = min(R, rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        skd::mbar_init(bar, 1);
        skd::mbar_fence_init();
        const uint32_t bq = (uint32_t) nrows * bpr * 128, bh = (uint32_t) nrows * bpr * 16;
        skd::mbar_expect_tx(bar, bq + bh);
        skd::bulk_g2s(s_qs, qs + (size_t) row0 * bpr * 128, bq, bar);
        skd::bulk_g2s(s_hdr, hdr + (size_t) row0 * bpr * 16, bh, bar);
    }
    skd::pdl_launch_dependents();
    skd::pdl_wait();                       // the quantized activation is the predecessor's output

    // Stage the activation: int8 codes with 16-byte chunks XOR-swizzled per block pair, sub-block sums as is.
    {
        const int nchunks = M * (cols >> 4);
        for (int c = threadIdx.x; c < nchunks; c += MS_THREADS) {
            const int blk = c >> 4, ch = c & 15;           // block (of 256 codes) across all m, chunk inside it
            const int sw = ch ^ ((((blk % bpr) >> 1) & 1) << 1);
            *reinterpret_cast<uint4*>(s_q8 + (size_t) blk * 256 + sw * 16) = skd::ld_ro(act.q + (size_t) c * 16);
        }
        const int nb16 = M * (cols >> 8);                   // 16 bytes of bsums per block
        for (int c = threadIdx.x; c < nb16; c += MS_THREADS)
            *reinterpret_cast<uint4*>((uint8_t*) s_bs + (size_t) c * 16) = skd::ld_ro((const uint8_t*) act.bsums + (size_t) c * 16);
    }
    __syncthreads();
    if (!skd::mbar_wait_bounded(bar, 0, timeout_flag)) return;

    const int h = lane & 1, slot = lane >> 1, s1 = (slot >> 1) & 1;
    const int off_lo = ((h) ^ (s1 << 1)) * 16, off_hi = ((2 + h) ^ (s1 << 1)) * 16;   // swizzled chunk of (lo|hi, h)
    float acc[M][RW];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RW; ++r) acc[m][r] = 0.0f;

    const int ncg = (bpr + 15) >> 4;
    for (int cg = 0; cg < ncg; ++cg) {
        const int b = cg * 16 + slot;
        if (b >= bpr) continue;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            // this lane's activation slice for block b: 4 groups x (lo, hi) x 16 codes, in rotated group order
            uint4 a_lo[4], a_hi[4];
            const int8_t* qa = s_q8 + ((size_t) m * bpr + b) * 256;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int g = (k + slot) & 3;
                a_lo[k] = skd::lds128(qa + 64 * g + off_lo);
                a_hi[k] = skd::lds128(qa + 64 * g + off_hi);
            }
            const uint2 bs = *reinterpret_cast<const uint2*>(s_bs + ((size_t) m * bpr + b) * 8 + 4 * h);
            const float di = __ldg(act.d + (size_t) m * bpr + b);
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int rl = warp + MS_WARPS * r;
                if (rl >= nrows) continue;
                const size_t blk = (size_t) rl * bpr + b;
                const uint8_t* qp = s_qs + blk * 128 + h * 16;
                const uint4 hd = skd::lds128(s_hdr + blk * 16);
                const float d = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
                const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
                uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                skd::k4_unpack(hd.y, hd.z, hd.w, sc_lo, sc_hi, mn_lo, mn_hi);
                int sdot = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int g = (k + slot) & 3;
                    const uint4 w = skd::lds128(qp + 32 * g);
                    const uint32_t scw = ((g & 2) ? sc_hi : sc_lo) >> (16 * (g & 1));
                    int dl = 0, dh = 0;   // dh carries the high nibbles in place: 16 x the dot
                    dl = __dp4a((int) (w.x & 0x0f0f0f0fu), (int) a_lo[k].x, dl);
                    dl = __dp4a((int) (w.y & 0x0f0f0f0fu), (int) a_lo[k].y, dl);
                    dl = __dp4a((int) (w.z & 0x0f0f0f0fu), (int) a_lo[k].z, dl);
                    dl = __dp4a((int) (w.w & 0x0f0f0f0fu), (int) a_lo[k].w, dl);
                    dh = skd::dp4a_us(w.x & 0xf0f0f0f0u, a_hi[k].x, dh);
                    dh = skd::dp4a_us(w.y & 0xf0f0f0f0u, a_hi[k].y, dh);
                    dh = skd::dp4a_us(w.z & 0xf0f0f0f0u, a_hi[k].z, dh);
                    dh = skd::dp4a_us(w.w & 0xf0f0f0f0u, a_hi[k].w, dh);
                    sdot += (int) (scw & 0xff) * dl + (int) ((scw >> 8) & 0xff) * (dh >> 4);
                }
                const uint32_t mn = h ? mn_hi : mn_lo;      // lane h accounts the mins of sub-blocks 4h..4h+3
                const int msum = skd::byte_of(mn, 0) * (int) (short) (bs.x & 0xffff) + skd::byte_of(mn, 1) * (int) (short) (bs.x >> 16)
                               + skd::byte_of(mn, 2) * (int) (short) (bs.y & 0xffff) + skd::byte_of(mn, 3) * (int) (short) (bs.y >> 16);
                acc[m][r] += di * (d * (float) sdot - dmin * (float) msum);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const float v = skd::warp_sum(acc[m][r]);
            const int rl = warp + MS_WARPS * r;
            if (lane == 0 && rl < nrows) y[(size_t) m * rows + row0 + rl] = v;
        }
}

static size_t q4k_stream_smem(int M, int RW, int bpr, int cols) {
    return (size_t) MS_WARPS * RW * bpr * 144 + (size_t) M * cols + (size_t) M * (cols / 16) + 16;
}

template <int M, int RW>
static int32_t launch_q4k_stream(const Weight& w, ActQ8K act, float* y, int* flag, cudaStream_t s) {
    const size_t smem = q4k_stream_smem(M, RW, w.bpr, w.cols);
    SK_TRY(ensure_dynamic_smem((const void*) q4k_matvec_stream_kernel<M, RW>, (int) MS_SMEM_BUDGET + 4096));
    const int R = MS_WARPS * RW;
    SK_CUDA(launch_pdl(q4k_matvec_stream_kernel<M, RW>, dim3((w.rows + R - 1) / R), dim3(MS_THREADS), smem, s,
                       (const uint8_t*) w.qs, (const uint8_t*) w.hdr, w.rows, w.bpr, act, w.cols, y, flag));
    return SKAINET_CUDA_OK;
}

// ================================================================================================
// Q8_0
// ================================================================================================
// Tile of R = 4*RW rows of int8 codes plus their f16 scales. A lane owns 16-code chunks
// lane, lane+32, ... (eight per 4096-wide column group); consecutive lanes read consecutive 16 bytes.
template <int M, int RW>
__global__ void __launch_bounds__(MS_THREADS)
q8_0_matvec_stream_kernel(const int8_t* __restrict__ codes, const __half* __restrict__ scales, int rows, int cols,
                          ActSplit act, float* __restrict__ y, int* __restrict__ timeout_flag) {
    constexpr int R = MS_WARPS * RW;
    extern __shared__ __align__(128) uint8_t smem[];
    const int bpr = cols >> 5;
    int8_t* s_codes = (int8_t*) smem;
    __half* s_scales = (__half*) (s_codes + (size_t) R * cols);
    int8_t* s_hi = (int8_t*) (s_scales + (size_t) R * bpr);
    int8_t* s_lo = s_hi + (size_t) M * cols;
    float* s_dx = (float*) (s_lo + (size_t) M * cols);
    uint64_t* bar = (uint64_t*) (s_dx + (size_t) M * bpr);

    const int row0 = blockIdx.x * R;
    const int nrows = min(R, rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        skd::mbar_init(bar, 1);
        skd::mbar_fence_init();
        const uint32_t bc = (uint32_t) nrows * cols, bs = (uint32_t) nrows * bpr * 2;
        skd::mbar_expect_tx(bar, bc + bs);
        skd::bulk_g2s(s_codes, codes + (size_t) row0 * cols, bc, bar);
        skd::bulk_g2s(s_scales, scales + (size_t) row0 * bpr, bs, bar);
    }
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    {
        const int nchunks = M * (cols >> 4);
        for (int c = threadIdx.x; c < nchunks; c += MS_THREADS) {
            *reinterpret_cast<uint4*>(s_hi + (size_t) c * 16) = skd::ld_ro(act.hi + (size_t) c * 16);
            *reinterpret_cast<uint4*>(s_lo + (size_t) c * 16) = skd::ld_ro(act.lo + (size_t) c * 16);
        }
        for (int c = threadIdx.x; c < M * bpr; c += MS_THREADS) s_dx[c] = __ldg(act.d + c);
    }
    __syncthreads();
    if (!skd::mbar_wait_bounded(bar, 0, timeout_flag)) return;

    float acc[M][RW];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RW; ++r) acc[m][r] = 0.0f;

    const int nchunks = cols >> 4;
    for (int c0 = 0; c0 < nchunks; c0 += 256) {           // column group: 8 chunks per lane
#pragma unroll
        for (int m = 0; m < M; ++m) {
            uint4 ah[8], al[8];
            float dx[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = c0 + j * 32 + lane;
                if (c < nchunks) {
                    ah[j] = skd::lds128(s_hi + (size_t) m * cols + c * 16);
                    al[j] = skd::lds128(s_lo + (size_t) m * cols + c * 16);
                    dx[j] = s_dx[m * bpr + (c >> 1)];
                } else { ah[j] = make_uint4(0, 0, 0, 0); al[j] = ah[j]; dx[j] = 0.0f; }
            }
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int rl = warp + MS_WARPS * r;
                if (rl >= nrows) continue;
                const int8_t* wr = s_codes + (size_t) rl * cols;
                const __half* sr = s_scales + (size_t) rl * bpr;
                float a = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = c0 + j * 32 + lane;
                    if (c < nchunks) {
                        const uint4 w = skd::lds128(wr + c * 16);
                        int dh = 0, dl = 0;
                        dh = __dp4a((int) w.x, (int) ah[j].x, dh); dh = __dp4a((int) w.y, (int) ah[j].y, dh);
                        dh = __dp4a((int) w.z, (int) ah[j].z, dh); dh = __dp4a((int) w.w, (int) ah[j].w, dh);
                        dl = __dp4a((int) w.x, (int) al[j].x, dl); dl = __dp4a((int) w.y, (int) al[j].y, dl);
                        dl = __dp4a((int) w.z, (int) al[j].z, dl); dl = __dp4a((int) w.w, (int) al[j].w, dl);
                        a += (__half2float(sr[c >> 1]) * dx[j]) * (float) (dh * 128 + dl);
                    }
                }
                acc[m][r] += a;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const float v = skd::warp_sum(acc[m][r]);
            const int rl = warp + MS_WARPS * r;
            if (lane == 0 && rl < nrows) y[(size_t) m * rows + row0 + rl] = v;
        }
}

static size_t q8_stream_smem(int M, int RW, int cols) {
    const int bpr = cols / 32;
    return (size_t) MS_WARPS * RW * (cols + bpr * 2) + (size_t) M * (2 * cols + bpr * 4) + 16;
}

template <int M, int RW>
static int32_t launch_q8_stream(const Weight& w, ActSplit act, float* y, int* flag, cudaStream_t s) {
    const size_t smem = q8_stream_smem(M, RW, w.cols);
    SK_TRY(ensure_dynamic_smem((const void*) q8_0_matvec_stream_kernel<M, RW>, (int) MS_SMEM_BUDGET + 4096));
    const int R = MS_WARPS * RW;
    SK_CUDA(launch_pdl(q8_0_matvec_stream_kernel<M, RW>, dim3((w.rows + R - 1) / R), dim3(MS_THREADS), smem, s,
                       (const int8_t*) w.qs, (const __half*) w.hdr, w.rows, w.cols, act, y, flag));
    return SKAINET_CUDA_OK;
}

// ================================================================================================
// dispatch: picks rows-per-warp so the tile fits the shared-memory budget. Returns 1 when the shape
// is outside what the streaming kernels take (the caller then uses the direct-load kernels).
// ================================================================================================
#define SK_STREAM_CASE(FN, MM, ...)                         \
    switch (rw) {                                           \
        case 4: return FN<MM, 4>(__VA_ARGS__);              \
        case 2: return FN<MM, 2>(__VA_ARGS__);              \
        default: return FN<MM, 1>(__VA_ARGS__);             \
    }

int32_t launch_matvec_stream(const Weight& w, const void* act_scratch, int m_total, int m0, int mm, float* y, cudaStream_t s) {
    int* flag = device_timeout_flag();
    if (w.enc == SKAINET_ENC_Q4_K) {
        int rw = 4;
        while (rw >= 1 && q4k_stream_smem(mm, rw, w.bpr, w.cols) > MS_SMEM_BUDGET) rw >>= 1;
        if (rw < 1) return 1;
        // small matrices: prefer more CTAs than SMs over longer tiles
        while (rw > 1 && (w.rows + MS_WARPS * rw - 1) / (MS_WARPS * rw) < 2 * sm_count()) rw >>= 1;
        ActQ8K a = act_q8k_layout(const_cast<void*>(act_scratch), m_total, w.cols);
        a.q += (size_t) m0 * w.cols; a.d += (size_t) m0 * (w.cols / 256); a.bsums += (size_t) m0 * (w.cols / 32);
        switch (mm) {
            case 8: SK_STREAM_CASE(launch_q4k_stream, 8, w, a, y, flag, s)
            case 4: SK_STREAM_CASE(launch_q4k_stream, 4, w, a, y, flag, s)
            case 2: SK_STREAM_CASE(launch_q4k_stream, 2, w, a, y, flag, s)
            default: SK_STREAM_CASE(launch_q4k_stream, 1, w, a, y, flag, s)
        }
    }
    if (w.enc == SKAINET_ENC_Q8_0) {
        if (w.cols % 256 != 0) return 1;     // scale rows must be whole 16-byte units for the bulk copy
        int rw = 4;
        while (rw >= 1 && q8_stream_smem(mm, rw, w.cols) > MS_SMEM_BUDGET) rw >>= 1;
        if (rw < 1) return 1;
        while (rw > 1 && (w.rows + MS_WARPS * rw - 1) / (MS_WARPS * rw) < 2 * sm_count()) rw >>= 1;
        ActSplit a = act_split_layout(const_cast<void*>(act_scratch), m_total, w.cols);
        a.hi += (size_t) m0 * w.cols; a.lo += (size_t) m0 * w.cols; a.d += (size_t) m0 * (w.cols / 32);
        switch (mm) {
            case 8: SK_STREAM_CASE(launch_q8_stream, 8, w, a, y, flag, s)
            case 4: SK_STREAM_CASE(launch_q8_stream, 4, w, a, y, flag, s)
            case 2: SK_STREAM_CASE(launch_q8_stream, 2, w, a, y, flag, s)
            default: SK_STREAM_CASE(launch_q8_stream, 1, w, a, y, flag, s)
        }
    }
    return 1;
}

}  // namespace sk
