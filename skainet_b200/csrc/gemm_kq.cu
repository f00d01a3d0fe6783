// Batched rows for Q6_K and Q5_K weights (a prompt chunk or a decode batch) on the tensor cores. First part: Q6_K, nine and
// more int8-quantized activation rows, mma.sync m16n8k16 s8 x s8 -> s32. Second part (further down): Q5_K, five and more
// fp32 activation rows carried as two f16 terms, mma.sync m16n8k16 f16 -> f32.
//
// Arithmetic is the reference's native Q6_K path (native/src/q6k_matmul.c:155-215, rows of a batch being independent
// matvecs there, :289-357): per 16-element scale group an exact integer dot of (code - 32) with the activation codes,
// times the group's int8 scale, summed over the block's sixteen groups in int32; then d * d_in * float(sum) added block by
// block in fp32, in the reference's order, so every output is bit-identical to the single-row kernel and to the C code.
// One MMA is exactly one scale group: its A tile is 16 weight rows x the group's 16 codes, its B tile the same 16 codes
// of 8 activation rows; the scale is applied to the int32 result on the CUDA cores.
//
// CTA = 4 warps x 16 weight rows against 64 activation rows, looping over the 256-element super-blocks of the
// contraction through a cp.async pipeline of three or four stages:
//   weight stage     ql [rows][144 B] (128 B of low nibbles + pad), qh [rows][80 B] (64 B of high bits + pad),
//                    scales [rows][16 B]; the row strides make the A-fragment word reads (8 rows x 4 words) conflict free;
//   activation stage [64 rows][272 B]: 256 codes + pad (the B-fragment reads, 8 rows x 4 words, are conflict free), and
//                    the rows' fp32 block scales.
// A thread builds the A fragments straight from the staged bytes: for rows g and g + 8 of its warp, word t of the
// group's 16 low-nibble bytes (one ql word serves the groups 64 elements apart in its low and high nibbles) and word t of
// the 16 high-bit bytes (one qh word serves four groups), code - 32 by a byte-wise subtract.
// Grid (activation tiles, weight tiles): the CTAs sharing a weight tile are launched next to each other, so the weight
// is read from HBM once and from L2 for the other activation tiles.
#include "common.cuh"
#include "actquant.cuh"
#include "tma.cuh"

#include <cuda_fp16.h>

namespace sk {

namespace {

constexpr int KG_MT = 64, KG_NT = KG_MT / 8;
constexpr int KG_QL_STRIDE = 144, KG_QH_STRIDE = 80, KG_X_STRIDE = 272;
// stage layout for NW warps (16 NW weight rows): ql | qh | scales | activation codes | activation block scales
__host__ __device__ constexpr int kg_off_qh(int nw) { return nw * 16 * KG_QL_STRIDE; }
__host__ __device__ constexpr int kg_off_sc(int nw) { return kg_off_qh(nw) + nw * 16 * KG_QH_STRIDE; }
__host__ __device__ constexpr int kg_off_x(int nw) { return kg_off_sc(nw) + nw * 16 * 16; }
__host__ __device__ constexpr int kg_off_xd(int nw) { return kg_off_x(nw) + KG_MT * KG_X_STRIDE; }
__host__ __device__ constexpr int kg_stage(int nw) { return kg_off_xd(nw) + KG_MT * 4; }

__device__ __forceinline__ void kg_cp16(void* dst, const void* src, bool live) {
    const int n = live ? 16 : 0;                      // zero-fill when the row lies past the batch
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(skd::smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void kg_cp4(void* dst, const void* src, bool live) {
    const int n = live ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(skd::smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void kg_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void kg_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void kg_mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}

template <int NW, int NS>
__global__ void __launch_bounds__(NW * 32)
q6k_gemm_mma_kernel(const uint8_t* __restrict__ ql, const uint8_t* __restrict__ qh, const int8_t* __restrict__ sc, const uint8_t* __restrict__ dd,
                    int rows, int bpr, ActQ8K act, int m, float* y, const float* resid) {
    constexpr int KG_RT = NW * 16, NTHR = NW * 32;
    constexpr int KG_OFF_QH = kg_off_qh(NW), KG_OFF_SC = kg_off_sc(NW), KG_OFF_X = kg_off_x(NW), KG_OFF_XD = kg_off_xd(NW), KG_STAGE = kg_stage(NW);
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int col0 = blockIdx.x * KG_MT, row0 = blockIdx.y * KG_RT;
    const int cols = bpr * 256;
    skd::pdl_launch_dependents();
    skd::pdl_wait();                                   // the quantized activation rows are the preceding kernel's output

    auto load_stage = [&](int blk, int buf) {
        uint8_t* st = smem + (size_t) buf * KG_STAGE;
#pragma unroll
        for (int i = 0; i < 4; ++i) {                  // ql: 16 NW rows x 8 chunks
            const int c = tid + i * NTHR, r = c >> 3, ch = c & 7;
            const size_t pblk = (size_t) min(row0 + r, rows - 1) * bpr + blk;     // rows past the end repeat the last one (never stored)
            kg_cp16(st + r * KG_QL_STRIDE + ch * 16, ql + pblk * 128 + ch * 16, true);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {                  // qh: 16 NW rows x 4 chunks
            const int c = tid + i * NTHR, r = c >> 2, ch = c & 3;
            const size_t pblk = (size_t) min(row0 + r, rows - 1) * bpr + blk;
            kg_cp16(st + KG_OFF_QH + r * KG_QH_STRIDE + ch * 16, qh + pblk * 64 + ch * 16, true);
        }
        if (tid < KG_RT) {                             // the rows' sixteen int8 scales
            const size_t pblk = (size_t) min(row0 + tid, rows - 1) * bpr + blk;
            kg_cp16(st + KG_OFF_SC + tid * 16, sc + pblk * 16, true);
        } else {                                       // the activation rows' block scales
#pragma unroll
            for (int c = tid - KG_RT; c < KG_MT; c += NTHR - KG_RT) {
                const int col = col0 + c;
                kg_cp4(st + KG_OFF_XD + c * 4, act.d + (size_t) min(col, m - 1) * bpr + blk, col < m);
            }
        }
#pragma unroll
        for (int i = 0; i < KG_MT * 16 / NTHR; ++i) {  // activation codes: 64 rows x 16 chunks
            const int c = tid + i * NTHR, r = c >> 4, ch = c & 15, col = col0 + r;
            kg_cp16(st + KG_OFF_X + r * KG_X_STRIDE + ch * 16, act.q + (size_t) min(col, m - 1) * cols + (size_t) blk * 256 + ch * 16, col < m);
        }
        kg_commit();
    };

    float acc[KG_NT][4];
#pragma unroll
    for (int nt = 0; nt < KG_NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[nt][j] = 0.0f;

    const int ra = warp * 16 + g, rb = ra + 8;         // this thread's two weight rows within the tile
    const size_t grow_a = (size_t) min(row0 + ra, rows - 1) * bpr, grow_b = (size_t) min(row0 + rb, rows - 1) * bpr;

    // NS stages: block blk + NS - 1 is requested while block blk is worked on; one group is committed per iteration
    // (an empty one past the end), so "all but the newest NS - 2 groups complete" always means block blk has landed
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) { if (s < bpr) load_stage(s, s); else kg_commit(); }
    for (int blk = 0; blk < bpr; ++blk) {
        kg_wait<NS - 2>();
        __syncthreads();                               // block blk visible to all; everyone is done with block blk - 1, whose buffer is refilled now
        if (blk + NS - 1 < bpr) load_stage(blk + NS - 1, (blk + NS - 1) % NS); else kg_commit();
        const uint8_t* st = smem + (size_t) (blk % NS) * KG_STAGE;
        const float d_a = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(dd) + grow_a + blk)));
        const float d_b = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(dd) + grow_b + blk)));
        const uint4 sca = *reinterpret_cast<const uint4*>(st + KG_OFF_SC + ra * 16), scb = *reinterpret_cast<const uint4*>(st + KG_OFF_SC + rb * 16);
        const uint32_t scw_a[4] = {sca.x, sca.y, sca.z, sca.w}, scw_b[4] = {scb.x, scb.y, scb.z, scb.w};
        int isum[KG_NT][4];
#pragma unroll
        for (int nt = 0; nt < KG_NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) isum[nt][j] = 0;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t qh_a = *reinterpret_cast<const uint32_t*>(st + KG_OFF_QH + ra * KG_QH_STRIDE + 32 * n + 16 * h + 4 * t);
                const uint32_t qh_b = *reinterpret_cast<const uint32_t*>(st + KG_OFF_QH + rb * KG_QH_STRIDE + 32 * n + 16 * h + 4 * t);
#pragma unroll
                for (int par = 0; par < 2; ++par) {
                    const uint32_t ql_a = *reinterpret_cast<const uint32_t*>(st + ra * KG_QL_STRIDE + 64 * n + 32 * par + 16 * h + 4 * t);
                    const uint32_t ql_b = *reinterpret_cast<const uint32_t*>(st + rb * KG_QL_STRIDE + 64 * n + 32 * par + 16 * h + 4 * t);
#pragma unroll
                    for (int nib = 0; nib < 2; ++nib) {
                        const int q = par + 2 * nib, grp = 8 * n + 2 * q + h, e = 128 * n + 32 * q + 16 * h;      // scale group and its first element
                        const uint32_t a0 = __vsub4(((ql_a >> (4 * nib)) & 0x0f0f0f0fu) | (((qh_a >> (2 * q)) & 0x03030303u) << 4), 0x20202020u);
                        const uint32_t a1 = __vsub4(((ql_b >> (4 * nib)) & 0x0f0f0f0fu) | (((qh_b >> (2 * q)) & 0x03030303u) << 4), 0x20202020u);
                        const int s_a = (int) (int8_t) (scw_a[grp >> 2] >> (8 * (grp & 3))), s_b = (int) (int8_t) (scw_b[grp >> 2] >> (8 * (grp & 3)));
#pragma unroll
                        for (int nt = 0; nt < KG_NT; ++nt) {
                            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(st + KG_OFF_X + (nt * 8 + g) * KG_X_STRIDE + e + 4 * t);
                            int c[4] = {0, 0, 0, 0};
                            kg_mma_s8(c, a0, a1, b0);
                            isum[nt][0] += s_a * c[0]; isum[nt][1] += s_a * c[1]; isum[nt][2] += s_b * c[2]; isum[nt][3] += s_b * c[3];
                        }
                    }
                }
            }
        }
        // accumulator j of tile nt: weight row g + 8 (j >> 1), activation row 8 nt + 2 t + (j & 1)
        const float* xd = reinterpret_cast<const float*>(st + KG_OFF_XD);
#pragma unroll
        for (int nt = 0; nt < KG_NT; ++nt) {
            const float2 di = *reinterpret_cast<const float2*>(xd + nt * 8 + 2 * t);
            acc[nt][0] = __fadd_rn(acc[nt][0], __fmul_rn(__fmul_rn(d_a, di.x), (float) isum[nt][0]));
            acc[nt][1] = __fadd_rn(acc[nt][1], __fmul_rn(__fmul_rn(d_a, di.y), (float) isum[nt][1]));
            acc[nt][2] = __fadd_rn(acc[nt][2], __fmul_rn(__fmul_rn(d_b, di.x), (float) isum[nt][2]));
            acc[nt][3] = __fadd_rn(acc[nt][3], __fmul_rn(__fmul_rn(d_b, di.y), (float) isum[nt][3]));
        }
    }
    kg_wait<0>();
#pragma unroll
    for (int nt = 0; nt < KG_NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = row0 + warp * 16 + g + 8 * (j >> 1), col = col0 + nt * 8 + 2 * t + (j & 1);
            if (row < rows && col < m) {
                const size_t o = (size_t) col * rows + row;
                y[o] = resid ? __fadd_rn(resid[o], acc[nt][j]) : acc[nt][j];       // resid may be y itself: read and written by this thread only
            }
        }
    }
}

template <int NW, int NS>
int32_t launch_gemm_q6k_nw(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    const int smem = NS * kg_stage(NW);
    SK_TRY(ensure_dynamic_smem((const void*) q6k_gemm_mma_kernel<NW, NS>, smem));
    const dim3 grid((m + KG_MT - 1) / KG_MT, (w.rows + NW * 16 - 1) / (NW * 16));
    if (grid.y > 65535) return 1;
    SK_CUDA(launch_pdl(q6k_gemm_mma_kernel<NW, NS>, grid, dim3(NW * 32), (size_t) smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.extra, (const int8_t*) w.hdr,
                       (const uint8_t*) w.aux, w.rows, w.bpr, a, m, y, resid));
    return SKAINET_CUDA_OK;
}


// =====================================================================================================================
// Q5_K. The reference keeps fp32 activations for this format (native/src/q5k_matmul.c:93-215): per sub-block
// code_sum * (d * sc) - input_sum * (dmin * mn). On the tensor cores (mma.sync m16n8k16 f16 -> f32): the A operand carries
// code * sc (at most 31 * 63 = 1953, exact in f16; built as f16(1024 + code) * sc - 1024 * sc under one fused rounding), the
// B operand the activation as two f16 terms, hi = f16(x) and lo = f16(x - hi), one MMA each, so the product keeps fp32
// accuracy; a block's 32 MMAs accumulate sum_sb sc_sb * code_sum_sb, which d scales once, and the mins term
// sum_sb (dmin * mn_sb) * input_sum_sb is eight multiply-adds per output on the CUDA cores from per-32 sums of the fp32
// activation. The activation side (hi, lo, sums) is prepared once per call by act_f16split_kernel.
// Within an MMA the order of the 16 contraction elements is free as long as A and B agree: thread t takes elements
// 4 t .. 4 t + 3 of the group (one 32-bit word of nibbles and one of fifth bits per weight row, one 8-byte read of the
// activation row), elements 4 t, 4 t + 1 in the k slots 2 t, 2 t + 1 and elements 4 t + 2, 4 t + 3 in the slots 2 t + 8, 2 t + 9.
// CTA = 4 warps x 16 weight rows against 32 activation rows; stage = one super-block:
//   qs [64][144 B] | fifth bits [64][48 B] | headers [64][16 B] | hi [32][544 B] | lo [32][544 B] | sums [32][8 floats]
// (row strides chosen so that the word reads of eight rows and the 8-byte reads of eight activation rows are conflict free).
// =====================================================================================================================
constexpr int K5_WARPS = 4, K5_RT = K5_WARPS * 16, K5_MT = 32, K5_NT = K5_MT / 8, K5_THREADS = K5_WARPS * 32;
constexpr int K5_QS_STRIDE = 144, K5_QH_STRIDE = 48, K5_X_STRIDE = 544;
constexpr int K5_OFF_QH = K5_RT * K5_QS_STRIDE, K5_OFF_HDR = K5_OFF_QH + K5_RT * K5_QH_STRIDE, K5_OFF_XH = K5_OFF_HDR + K5_RT * 16;
constexpr int K5_OFF_XL = K5_OFF_XH + K5_MT * K5_X_STRIDE, K5_OFF_XS = K5_OFF_XL + K5_MT * K5_X_STRIDE, K5_STAGE = K5_OFF_XS + K5_MT * 32;

struct ActF16Split { const __half* hi; const __half* lo; const float* sums; };      // [m][cols], [m][cols], [m][cols / 32]
static inline size_t k5_align256(size_t x) { return (x + 255) & ~(size_t) 255; }
static ActF16Split act_f16split_layout(const void* scratch, int m, int cols) {
    ActF16Split a;
    const uint8_t* p = (const uint8_t*) scratch;
    a.hi = (const __half*) p; p += k5_align256((size_t) m * cols * 2);
    a.lo = (const __half*) p; p += k5_align256((size_t) m * cols * 2);
    a.sums = (const float*) p;
    return a;
}

// One warp per 256 activation elements: lane l holds elements 8 l .. 8 l + 7, four lanes make one 32-element sum.
__global__ void __launch_bounds__(256)
act_f16split_kernel(const float* __restrict__ x, int64_t nblocks, __half* __restrict__ hi, __half* __restrict__ lo, float* __restrict__ sums) {
    skd::pdl_launch_dependents();
    skd::pdl_wait();
    const int64_t blk = (blockIdx.x * (int64_t) blockDim.x + threadIdx.x) >> 5;
    if (blk >= nblocks) return;
    const int lane = threadIdx.x & 31;
    const float4 v0 = __ldg(reinterpret_cast<const float4*>(x + blk * 256) + 2 * lane), v1 = __ldg(reinterpret_cast<const float4*>(x + blk * 256) + 2 * lane + 1);
    const float e[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t ph[4], pl[4];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half h0 = __float2half_rn(e[2 * i]), h1 = __float2half_rn(e[2 * i + 1]);
        const __half l0 = __float2half_rn(e[2 * i] - __half2float(h0)), l1 = __float2half_rn(e[2 * i + 1] - __half2float(h1));
        ph[i] = (uint32_t) __half_as_ushort(h0) | ((uint32_t) __half_as_ushort(h1) << 16);
        pl[i] = (uint32_t) __half_as_ushort(l0) | ((uint32_t) __half_as_ushort(l1) << 16);
        sum += e[2 * i] + e[2 * i + 1];
    }
    *reinterpret_cast<uint4*>(hi + blk * 256 + 8 * lane) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
    *reinterpret_cast<uint4*>(lo + blk * 256 + 8 * lane) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if ((lane & 3) == 0) sums[blk * 8 + (lane >> 2)] = sum;
}

__device__ __forceinline__ void k5_mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two 5-bit codes (bytes `lo_byte`, `lo_byte + 1` of w) times the sub-block scale, as two f16: (1024 + code) * sc - 1024 * sc
__device__ __forceinline__ uint32_t k5_scaled_pair(uint32_t w, int pair, __half2 sc2, __half2 nsc2) {
    const uint32_t v = __byte_perm(w, 0u, pair ? 0x4342 : 0x4140) | 0x64006400u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&v), sc2, nsc2);
    return *reinterpret_cast<const uint32_t*>(&r);
}

template <int NS>
__global__ void __launch_bounds__(K5_THREADS)
q5k_gemm_mma_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ hdr, const uint8_t* __restrict__ qh, int rows, int bpr,
                    ActF16Split act, int m, float* __restrict__ y) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int col0 = blockIdx.x * K5_MT, row0 = blockIdx.y * K5_RT;
    const int cols = bpr * 256;
    skd::pdl_launch_dependents();
    skd::pdl_wait();                                   // the prepared activation is the preceding kernel's output

    auto load_stage = [&](int blk, int buf) {
        uint8_t* st = smem + (size_t) buf * K5_STAGE;
#pragma unroll
        for (int i = 0; i < 4; ++i) {                  // nibbles: 64 rows x 8 chunks
            const int c = tid + i * K5_THREADS, r = c >> 3, ch = c & 7;
            const size_t pblk = (size_t) min(row0 + r, rows - 1) * bpr + blk;     // rows past the end repeat the last one (never stored)
            kg_cp16(st + r * K5_QS_STRIDE + ch * 16, qs + pblk * 128 + ch * 16, true);
        }
        {                                              // fifth bits: 64 rows x 2 chunks
            const int r = tid >> 1, ch = tid & 1;
            const size_t pblk = (size_t) min(row0 + r, rows - 1) * bpr + blk;
            kg_cp16(st + K5_OFF_QH + r * K5_QH_STRIDE + ch * 16, qh + pblk * 32 + ch * 16, true);
        }
        if (tid < K5_RT) {                             // headers
            const size_t pblk = (size_t) min(row0 + tid, rows - 1) * bpr + blk;
            kg_cp16(st + K5_OFF_HDR + tid * 16, hdr + pblk * 16, true);
        } else {                                       // per-32 sums of the activation rows: 32 rows x 2 chunks
            const int c = tid - K5_RT, r = c >> 1, ch = c & 1, col = col0 + r;
            kg_cp16(st + K5_OFF_XS + r * 32 + ch * 16, act.sums + ((size_t) min(col, m - 1) * bpr + blk) * 8 + ch * 4, col < m);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {                  // hi and lo terms: 32 rows x 32 chunks each; rows past the batch are zero-filled
            const int c = tid + i * K5_THREADS, r = c >> 5, ch = c & 31, col = col0 + r;
            const size_t src = (size_t) min(col, m - 1) * cols + (size_t) blk * 256 + ch * 8;
            kg_cp16(st + K5_OFF_XH + r * K5_X_STRIDE + ch * 16, act.hi + src, col < m);
            kg_cp16(st + K5_OFF_XL + r * K5_X_STRIDE + ch * 16, act.lo + src, col < m);
        }
        kg_commit();
    };

    float acc[K5_NT][4];
#pragma unroll
    for (int nt = 0; nt < K5_NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[nt][j] = 0.0f;
    const int ra = warp * 16 + g, rb = ra + 8;         // this thread's two weight rows within the tile

#pragma unroll
    for (int s = 0; s < NS - 1; ++s) { if (s < bpr) load_stage(s, s); else kg_commit(); }
    for (int blk = 0; blk < bpr; ++blk) {
        kg_wait<NS - 2>();
        __syncthreads();                               // block blk visible to all; everyone is done with block blk - 1, whose buffer is refilled now
        if (blk + NS - 1 < bpr) load_stage(blk + NS - 1, (blk + NS - 1) % NS); else kg_commit();
        const uint8_t* st = smem + (size_t) (blk % NS) * K5_STAGE;
        // headers of the two rows: d, dmin, eight 6-bit scales and mins each
        float d[2], mnf[2][8];
        uint32_t scw[2][2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 hd = *reinterpret_cast<const uint4*>(st + K5_OFF_HDR + (r ? rb : ra) * 16);
            d[r] = __half2float(__ushort_as_half((unsigned short) (hd.x & 0xffff)));
            const float dmin = __half2float(__ushort_as_half((unsigned short) (hd.x >> 16)));
            uint32_t mn_lo, mn_hi;
            skd::k4_unpack(hd.y, hd.z, hd.w, scw[r][0], scw[r][1], mn_lo, mn_hi);
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) mnf[r][sb] = dmin * (float) skd::byte_of(sb < 4 ? mn_lo : mn_hi, sb & 3);
        }
        float cm[K5_NT][4];
#pragma unroll
        for (int nt = 0; nt < K5_NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) cm[nt][j] = 0.0f;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {               // elements 16 hh .. 16 hh + 15 of every 32-element run
            const uint32_t qh_a = *reinterpret_cast<const uint32_t*>(st + K5_OFF_QH + ra * K5_QH_STRIDE + 16 * hh + 4 * t);
            const uint32_t qh_b = *reinterpret_cast<const uint32_t*>(st + K5_OFF_QH + rb * K5_QH_STRIDE + 16 * hh + 4 * t);
#pragma unroll
            for (int run = 0; run < 4; ++run) {        // 32 bytes of nibbles: sub-block 2 run in the low, 2 run + 1 in the high nibbles
                const uint32_t ql_a = *reinterpret_cast<const uint32_t*>(st + ra * K5_QS_STRIDE + 32 * run + 16 * hh + 4 * t);
                const uint32_t ql_b = *reinterpret_cast<const uint32_t*>(st + rb * K5_QS_STRIDE + 32 * run + 16 * hh + 4 * t);
#pragma unroll
                for (int nib = 0; nib < 2; ++nib) {
                    const int sb = 2 * run + nib, e0 = 32 * sb + 16 * hh;
                    const uint32_t ca = ((ql_a >> (4 * nib)) & 0x0f0f0f0fu) | (((qh_a >> sb) & 0x01010101u) << 4);
                    const uint32_t cb = ((ql_b >> (4 * nib)) & 0x0f0f0f0fu) | (((qh_b >> sb) & 0x01010101u) << 4);
                    const __half sa = __int2half_rn((int) skd::byte_of(scw[0][sb >> 2], sb & 3)), sbh = __int2half_rn((int) skd::byte_of(scw[1][sb >> 2], sb & 3));
                    const __half2 sa2 = __half2half2(sa), sb2 = __half2half2(sbh);
                    const __half2 nsa2 = __hmul2(sa2, __float2half2_rn(-1024.0f)), nsb2 = __hmul2(sb2, __float2half2_rn(-1024.0f));
                    uint32_t a[4];
                    a[0] = k5_scaled_pair(ca, 0, sa2, nsa2);      // row g,     elements 4 t, 4 t + 1  (k slots 2 t, 2 t + 1)
                    a[1] = k5_scaled_pair(cb, 0, sb2, nsb2);      // row g + 8
                    a[2] = k5_scaled_pair(ca, 1, sa2, nsa2);      // row g,     elements 4 t + 2, 4 t + 3  (k slots 2 t + 8, 2 t + 9)
                    a[3] = k5_scaled_pair(cb, 1, sb2, nsb2);      // row g + 8
#pragma unroll
                    for (int nt = 0; nt < K5_NT; ++nt) {
                        const uint2 bh = *reinterpret_cast<const uint2*>(st + K5_OFF_XH + (nt * 8 + g) * K5_X_STRIDE + (e0 + 4 * t) * 2);
                        const uint2 bl = *reinterpret_cast<const uint2*>(st + K5_OFF_XL + (nt * 8 + g) * K5_X_STRIDE + (e0 + 4 * t) * 2);
                        k5_mma_f16(cm[nt], a, bh.x, bh.y);
                        k5_mma_f16(cm[nt], a, bl.x, bl.y);
                    }
                }
            }
        }
        // accumulator j of tile nt: weight row g + 8 (j >> 1), activation row 8 nt + 2 t + (j & 1)
#pragma unroll
        for (int nt = 0; nt < K5_NT; ++nt) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float* xs = reinterpret_cast<const float*>(st + K5_OFF_XS + (nt * 8 + 2 * t + c) * 32);
                const float4 s0 = *reinterpret_cast<const float4*>(xs), s1 = *reinterpret_cast<const float4*>(xs + 4);
                const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float ms = 0.0f;
#pragma unroll
                    for (int sb = 0; sb < 8; ++sb) ms += mnf[r][sb] * sv[sb];
                    acc[nt][2 * r + c] += d[r] * cm[nt][2 * r + c] - ms;
                }
            }
        }
    }
    kg_wait<0>();
#pragma unroll
    for (int nt = 0; nt < K5_NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = row0 + warp * 16 + g + 8 * (j >> 1), col = col0 + nt * 8 + 2 * t + (j & 1);
            if (row < rows && col < m) y[(size_t) col * rows + row] = acc[nt][j];
        }
    }
}

template <int NS>
int32_t launch_gemm_q5k_ns(const Weight& w, ActF16Split a, int m, float* y, cudaStream_t s) {
    const int smem = NS * K5_STAGE;
    SK_TRY(ensure_dynamic_smem((const void*) q5k_gemm_mma_kernel<NS>, smem));
    const dim3 grid((m + K5_MT - 1) / K5_MT, (w.rows + K5_RT - 1) / K5_RT);
    if (grid.y > 65535) return 1;
    SK_CUDA(launch_pdl(q5k_gemm_mma_kernel<NS>, grid, dim3(K5_THREADS), (size_t) smem, s, (const uint8_t*) w.qs, (const uint8_t*) w.hdr, (const uint8_t*) w.extra,
                       w.rows, w.bpr, a, m, y));
    return SKAINET_CUDA_OK;
}

}  // namespace

// y[m][w.rows] (= resid +) for a Q6_K weight and m quantized activation rows on the tensor cores. A grid that gives each SM at most
// one CTA has nothing but its own ring to hide the load latency behind: four stages there, three otherwise (two CTAs per
// SM). Measured per call on 37 MB / 55 MB weights, stages 2 / 3 / 4: 11008 x 4096 at 64 rows 64 / 43 / 52 us, at 512 rows
// 200 / 198 / 249; 4096 x 11008 at 64 rows 91 / 108 / 68, at 128 rows 167 / 110 / 69; 8192 x 8192 at 64 rows 123 / 82 / 53.
// Tiles of 32 weight rows (two warps) were slower throughout (the activation tile is reloaded twice as often).
int32_t launch_gemm_q6k(const Weight& w, ActQ8K a, int m, float* y, const float* resid, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q6_K || m < 1 || w.rows < 1 || w.bpr < 1) return 1;
    const int64_t ctas = (int64_t) ((m + KG_MT - 1) / KG_MT) * ((w.rows + 63) / 64);
    return ctas <= sm_count() ? launch_gemm_q6k_nw<4, 4>(w, a, m, y, resid, s) : launch_gemm_q6k_nw<4, 3>(w, a, m, y, resid, s);
}

}  // namespace sk

namespace sk {

size_t act_f16split_bytes(int m, int cols) {
    return 2 * k5_align256((size_t) m * cols * 2) + k5_align256((size_t) m * (cols / 32) * 4);
}

// x[m][cols] fp32 -> hi, lo (two f16 terms) and per-32 sums in `scratch` (act_f16split_bytes of it).
int32_t launch_act_f16split(const float* x, int m, int cols, void* scratch, cudaStream_t s) {
    if (m <= 0 || cols <= 0) return SKAINET_CUDA_OK;
    const ActF16Split a = act_f16split_layout(scratch, m, cols);
    const int64_t nb = (int64_t) m * (cols / 256);
    SK_CUDA(launch_pdl(act_f16split_kernel, dim3((unsigned) ((nb * 32 + 255) / 256)), dim3(256), 0, s, x, nb, (__half*) a.hi, (__half*) a.lo, (float*) a.sums));
    return SKAINET_CUDA_OK;
}

// y[m][w.rows] for a Q5_K weight and m activation rows prepared by launch_act_f16split. Two stages with two CTAs per SM
// where the grid is larger than the GPU, four stages where an SM gets at most one CTA (the rule measured on the Q6_K kernel).
int32_t launch_gemm_q5k(const Weight& w, const void* act_scratch, int m, float* y, cudaStream_t s) {
    if (w.enc != SKAINET_ENC_Q5_K || m < 1 || w.rows < 1 || w.bpr < 1 || !act_scratch) return 1;
    const ActF16Split a = act_f16split_layout(act_scratch, m, w.cols);
    const int64_t ctas = (int64_t) ((m + K5_MT - 1) / K5_MT) * ((w.rows + K5_RT - 1) / K5_RT);
    return ctas <= sm_count() ? launch_gemm_q5k_ns<4>(w, a, m, y, s) : launch_gemm_q5k_ns<2>(w, a, m, y, s);
}

}  // namespace sk
