// Batched rows for Q6_K weights (nine and more int8-quantized activation rows: a prompt chunk or a large decode
// batch) on the tensor cores, mma.sync m16n8k16 s8 x s8 -> s32.
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
