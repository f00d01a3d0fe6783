// A KV-cache store resident in HBM: the device counterpart of the reference's KvCacheStore contract
// (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/tensor/storage/KvCacheStore.kt:36-165)
// as DefaultKvCacheStore implements it (DefaultKvCacheStore.kt:12-18 layout, :76-103 appendToken, :105-131 read /
// evict, :170-177 ring slots, :235-263 wrapped read), with binary16 elements (the reference's configurable cache
// dtype, KvCacheStore.kt:58-74; f16 -> f32 is exact, so a read returns exactly what attention sees).
//
// Per layer: keys and values [heads][max_seq][head_dim] f16. Positions are absolute; with sliding_window the
// buffer is a ring (slot = position mod max_seq) that keeps the newest max_seq positions. The sequence length
// advances when the LAST layer has been appended, as in the reference. Attention over a window of positions
// reads the ring in place (one run, or two when the window crosses the end of the buffer): the decode-attention
// kernel maps key i to slot (start + i) mod max_seq, the device form of iterating a WindowedKV pair
// (skainet-lang/skainet-lang-core/src/commonMain/kotlin/sk/ainet/lang/memory/WindowedAttention.kt:32-80).
//
// A second kind of store keeps TurboQuant blocks instead of binary16 rows (TurboQuantKvCacheStore.kt:62-199; codec in
// turboquant.cu): dense only, one block per (layer, position, head); reads and attention decode the window first.
#include "common.cuh"
#include "turboquant.cuh"

#include <mutex>
#include <unordered_set>
#include <vector>

namespace sk {

namespace {

struct KvStore {
    int layers = 0, heads = 0, head_dim = 0, max_seq = 0;
    bool ring = false;
    int cur = 0;            // currentSeqLen: positions appended so far (absolute)
    int oldest = 0;         // oldest absolute position still held intact
    __half *k = nullptr, *v = nullptr;     // [layers][heads][max_seq][head_dim]
    bool tq = false;                       // TurboQuant blocks instead of binary16 rows
    TqPlane kq, vq;
    int32_t* d_len = nullptr;              // device int read by the attention kernel
    int device = 0;
    uint64_t magic = 0;
    size_t layer_elems() const { return (size_t) heads * max_seq * head_dim; }
    int slot_of(int pos) const { return ring ? pos % max_seq : pos; }
    int window_start() const { return std::max(oldest, ring ? std::max(cur - max_seq, 0) : 0); }
};

const uint64_t KV_MAGIC = 0x534b4b5653544full;
std::mutex g_kv_mu;
std::unordered_set<KvStore*> g_kvs;

KvStore* kv_from_handle(int64_t h) {
    KvStore* s = reinterpret_cast<KvStore*>(h);
    std::lock_guard<std::mutex> lk(g_kv_mu);
    if (!s || g_kvs.find(s) == g_kvs.end() || s->magic != KV_MAGIC) { set_error("unknown or freed KV store handle %lld", (long long) h); return nullptr; }
    return s;
}

// one token's [heads][head_dim] fp32 rows -> slot `slot` of every head, rounded to binary16 (nearest even)
__global__ void kv_append_kernel(const float* __restrict__ key, const float* __restrict__ value, __half* __restrict__ kc,
                                 __half* __restrict__ vc, int heads, int head_dim, int max_seq, int slot) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= heads * head_dim) return;
    const int h = i / head_dim, d = i % head_dim;
    const size_t dst = ((size_t) h * max_seq + slot) * head_dim + d;
    kc[dst] = __float2half_rn(key[i]);
    vc[dst] = __float2half_rn(value[i]);
}

// positions [start, start + n) of a layer plane -> out [heads][n][head_dim] fp32, oldest first (two runs when wrapped)
__global__ void kv_read_kernel(const __half* __restrict__ plane, float* __restrict__ out, int heads, int head_dim, int max_seq,
                               int start_slot, int n, int ring) {
    const int64_t total = (int64_t) heads * n * head_dim;
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int d = (int) (i % head_dim), p = (int) ((i / head_dim) % n), h = (int) (i / ((int64_t) head_dim * n));
        int slot = start_slot + p;
        if (ring && slot >= max_seq) slot -= max_seq;
        out[i] = __half2float(plane[((size_t) h * max_seq + slot) * head_dim + d]);
    }
}

__global__ void kv_set_int_kernel(int32_t* p, int32_t v) { *p = v; }

int32_t kv_use(KvStore* s) { return set_thread_device(s->device); }

void kv_release(KvStore* s) {
    cudaFree(s->k); cudaFree(s->v); cudaFree(s->d_len);
    for (TqPlane* p : {&s->kq, &s->vq}) { cudaFree(p->codes); cudaFree(p->scales); cudaFree(p->resid); cudaFree(p->rscale); cudaFree(p->signs); cudaFree(p->rsigns); }
}
constexpr int32_t TQ_VALUE_SEED_XOR = 0x5A5A5A5A;      // TurboQuantKvCacheStore.kt:86

}  // namespace
}  // namespace sk

using namespace sk;

extern "C" {

int32_t skainet_cuda_kv_create(int32_t n_layers, int32_t n_heads, int32_t head_dim, int32_t max_seq, int32_t sliding_window,
                               skainet_kv_t* out) {
    SK_REQUIRE(out != nullptr, "kv_create: null output");
    *out = 0;
    SK_REQUIRE(n_layers > 0 && n_heads > 0 && max_seq > 0, "kv_create: layers, heads and max_seq must be positive");
    SK_REQUIRE(head_dim == 64 || head_dim == 128, "kv_create: head_dim %d not in {64,128}", head_dim);
    SK_TRY(ensure_device());
    KvStore* s = new KvStore();
    s->layers = n_layers; s->heads = n_heads; s->head_dim = head_dim; s->max_seq = max_seq; s->ring = sliding_window != 0;
    cudaGetDevice(&s->device);
    const size_t n = (size_t) n_layers * s->layer_elems();
    cudaError_t e = cudaMalloc((void**) &s->k, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMalloc((void**) &s->v, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMalloc((void**) &s->d_len, sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemset(s->k, 0, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMemset(s->v, 0, n * sizeof(__half));
    if (e != cudaSuccess) {
        cudaFree(s->k); cudaFree(s->v); cudaFree(s->d_len);
        delete s;
        return cuda_fail(e, "kv_create", __FILE__, __LINE__);
    }
    s->magic = KV_MAGIC;
    { std::lock_guard<std::mutex> lk(g_kv_mu); g_kvs.insert(s); }
    *out = (skainet_kv_t) reinterpret_cast<intptr_t>(s);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_create_turboquant(int32_t n_layers, int32_t n_heads, int32_t head_dim, int32_t max_seq, int32_t key_bits,
                                          int32_t key_residual_bits, int32_t value_bits, int32_t value_residual_bits, skainet_kv_t* out) {
    SK_REQUIRE(out != nullptr, "kv_create_turboquant: null output");
    *out = 0;
    SK_REQUIRE(n_layers > 0 && n_heads > 0 && max_seq > 0, "kv_create_turboquant: layers, heads and max_seq must be positive");
    SK_REQUIRE(n_heads <= 65535, "kv_create_turboquant: %d heads above 65535", n_heads);
    SK_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256, "kv_create_turboquant: head_dim %d not in {32,64,128,256}", head_dim);
    for (int b : {key_bits, value_bits}) SK_REQUIRE(b == 2 || b == 3 || b == 4 || b == 8, "bits must be 2, 3, 4, or 8, got %d", b);
    for (int b : {key_residual_bits, value_residual_bits}) SK_REQUIRE(b >= 0 && b <= 4, "residualBits must be 1-4 (0: no residual stage), got %d", b);
    SK_TRY(ensure_device());
    KvStore* s = new KvStore();
    s->layers = n_layers; s->heads = n_heads; s->head_dim = head_dim; s->max_seq = max_seq; s->ring = false; s->tq = true;
    s->kq.bits = key_bits; s->kq.rbits = key_residual_bits; s->vq.bits = value_bits; s->vq.rbits = value_residual_bits;
    cudaGetDevice(&s->device);
    const size_t vectors = (size_t) n_layers * max_seq * n_heads;
    cudaError_t e = cudaMalloc((void**) &s->d_len, sizeof(int32_t));
    for (TqPlane* p : {&s->kq, &s->vq}) {
        if (e == cudaSuccess) e = cudaMalloc((void**) &p->codes, vectors * tq_packed_size(head_dim, p->bits));
        if (e == cudaSuccess) e = cudaMalloc((void**) &p->scales, vectors * (head_dim / 32) * sizeof(float));
        if (e == cudaSuccess && p->rbits) e = cudaMalloc((void**) &p->resid, vectors * tq_packed_size(head_dim, p->rbits));
        if (e == cudaSuccess && p->rbits) e = cudaMalloc((void**) &p->rscale, vectors * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc((void**) &p->signs, vectors * (head_dim / 32) * sizeof(uint32_t));
        if (e == cudaSuccess && p->rbits == 1) e = cudaMalloc((void**) &p->rsigns, vectors * (head_dim / 32) * sizeof(uint32_t));
    }
    if (e != cudaSuccess) {
        kv_release(s);
        delete s;
        return cuda_fail(e, "kv_create_turboquant", __FILE__, __LINE__);
    }
    s->magic = KV_MAGIC;
    { std::lock_guard<std::mutex> lk(g_kv_mu); g_kvs.insert(s); }
    *out = (skainet_kv_t) reinterpret_cast<intptr_t>(s);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_free(skainet_kv_t h) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    kv_use(s);
    cudaDeviceSynchronize();
    { std::lock_guard<std::mutex> lk(g_kv_mu); g_kvs.erase(s); }
    kv_release(s);
    s->magic = 0;
    delete s;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_append_dev(skainet_kv_t h, int32_t layer, const float* key_dev, const float* value_dev, skainet_stream_t stream) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(layer >= 0 && layer < s->layers, "kv_append: layer index %d out of range [0, %d)", layer, s->layers);
    SK_REQUIRE(s->ring || s->cur < s->max_seq, "kv_append: KV cache is full: currentSeqLen=%d, maxSeqLen=%d", s->cur, s->max_seq);
    SK_REQUIRE(key_dev && value_dev, "kv_append: null key or value");
    SK_TRY(kv_use(s));
    if (s->tq) {
        SK_TRY(launch_tq_encode(key_dev, s->kq, layer, s->cur, s->heads, s->head_dim, s->max_seq, 0, as_stream(stream)));
        SK_TRY(launch_tq_encode(value_dev, s->vq, layer, s->cur, s->heads, s->head_dim, s->max_seq, TQ_VALUE_SEED_XOR, as_stream(stream)));
        if (layer == s->layers - 1) s->cur += 1;
        return SKAINET_CUDA_OK;
    }
    const int n = s->heads * s->head_dim;
    const size_t off = (size_t) layer * s->layer_elems();
    kv_append_kernel<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(key_dev, value_dev, s->k + off, s->v + off, s->heads, s->head_dim,
                                                                    s->max_seq, s->slot_of(s->cur));
    SK_CUDA(cudaGetLastError());
    if (layer == s->layers - 1) s->cur += 1;            // the sequence advances with the last layer
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_append(skainet_kv_t h, int32_t layer, const float* key_host, const float* value_host) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(key_host && value_host, "kv_append: null key or value");
    SK_TRY(kv_use(s));
    std::lock_guard<std::mutex> lk(twin_mutex());
    const size_t n = (size_t) s->heads * s->head_dim;
    void* staged = nullptr;
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_A, 2 * n * sizeof(float), &staged));
    SK_CUDA(cudaMemcpyAsync(staged, key_host, n * sizeof(float), cudaMemcpyHostToDevice, nullptr));
    SK_CUDA(cudaMemcpyAsync((float*) staged + n, value_host, n * sizeof(float), cudaMemcpyHostToDevice, nullptr));
    SK_TRY(skainet_cuda_kv_append_dev(h, layer, (const float*) staged, (const float*) staged + n, nullptr));
    SK_CUDA(cudaStreamSynchronize(nullptr));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_read(skainet_kv_t h, int32_t layer, int32_t which, int32_t start_pos, int32_t end_pos, float* host_out) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(layer >= 0 && layer < s->layers, "kv_read: layer index %d out of range [0, %d)", layer, s->layers);
    SK_REQUIRE(which == 0 || which == 1, "kv_read: which must be 0 (keys) or 1 (values)");
    SK_REQUIRE(start_pos >= s->window_start() && start_pos <= end_pos, "kv_read: invalid range: startPos=%d, endPos=%d, oldest held position=%d",
               start_pos, end_pos, s->window_start());
    SK_REQUIRE(end_pos <= s->cur, "kv_read: endPos=%d exceeds currentSeqLen=%d", end_pos, s->cur);
    const int n = end_pos - start_pos;
    if (n == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(host_out != nullptr, "kv_read: null output");
    SK_TRY(kv_use(s));
    const size_t total = (size_t) s->heads * n * s->head_dim;
    float* tmp = nullptr;
    SK_CUDA(cudaMalloc((void**) &tmp, total * sizeof(float)));
    cudaError_t e = cudaSuccess;
    if (s->tq) {
        const int32_t st = launch_tq_decode(which == 0 ? s->kq : s->vq, layer, start_pos, n, s->heads, s->head_dim, s->max_seq,
                                            which == 0 ? 0 : TQ_VALUE_SEED_XOR, tmp, nullptr);
        if (st != SKAINET_CUDA_OK) { cudaFree(tmp); return st; }
    } else {
        const __half* plane = (which == 0 ? s->k : s->v) + (size_t) layer * s->layer_elems();
        kv_read_kernel<<<(unsigned) std::min<size_t>((total + 255) / 256, 4096), 256>>>(plane, tmp, s->heads, s->head_dim, s->max_seq, s->slot_of(start_pos), n,
                                                                                         s->ring ? 1 : 0);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(host_out, tmp, total * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(tmp);
    if (e != cudaSuccess) return cuda_fail(e, "kv_read", __FILE__, __LINE__);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_evict(skainet_kv_t h, int32_t from_pos) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(from_pos >= 0 && from_pos <= s->cur, "kv_evict: fromPos=%d out of range [0, %d]", from_pos, s->cur);
    SK_REQUIRE(from_pos >= s->window_start(), "kv_evict: fromPos=%d lies before the oldest position the ring still holds (%d)", from_pos, s->window_start());
    SK_TRY(kv_use(s));
    SK_CUDA(cudaDeviceSynchronize());
    // positions the ring had already overwritten do not come back when the sequence is shortened
    s->oldest = s->window_start();
    if (!s->tq && (!s->ring || s->cur <= s->max_seq)) {
        // a cache that has not wrapped: zero the evicted tail of every head, as the reference does
        const size_t count = (size_t) (s->max_seq - from_pos) * s->head_dim * sizeof(__half);
        for (int l = 0; l < s->layers && count > 0; ++l)
            for (int hd = 0; hd < s->heads; ++hd) {
                const size_t off = (size_t) l * s->layer_elems() + ((size_t) hd * s->max_seq + from_pos) * s->head_dim;
                SK_CUDA(cudaMemsetAsync(s->k + off, 0, count, nullptr));
                SK_CUDA(cudaMemsetAsync(s->v + off, 0, count, nullptr));
            }
        SK_CUDA(cudaStreamSynchronize(nullptr));
    }
    s->cur = from_pos;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_clear(skainet_kv_t h) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(kv_use(s));
    SK_CUDA(cudaDeviceSynchronize());
    if (!s->tq) {
        const size_t n = (size_t) s->layers * s->layer_elems() * sizeof(__half);
        SK_CUDA(cudaMemset(s->k, 0, n));
        SK_CUDA(cudaMemset(s->v, 0, n));
    }
    s->cur = 0; s->oldest = 0;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_info(skainet_kv_t h, int64_t* out8) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(out8 != nullptr, "kv_info: null output");
    out8[0] = s->cur; out8[1] = s->window_start(); out8[2] = s->max_seq; out8[3] = s->layers; out8[4] = s->heads; out8[5] = s->head_dim;
    out8[6] = s->ring ? 1 : 0;
    out8[7] = (int64_t) (2 * (size_t) s->layers * s->layer_elems() * sizeof(__half));     // physical bytes, keys + values
    if (s->tq) {        // what the reference's memoryReport counts: the blocks of the positions held (TurboQuantKvCacheStore.kt:139-150)
        out8[6] = 2;
        out8[7] = (int64_t) s->layers * s->cur * s->heads * (tq_block_bytes(s->head_dim, s->kq.bits, s->kq.rbits) + tq_block_bytes(s->head_dim, s->vq.bits, s->vq.rbits));
    }
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_kv_attn_decode_dev(skainet_kv_t h, int32_t layer, const float* q_dev, float* out_dev, int32_t q_heads,
                                        int32_t from_pos, int32_t to_pos, float scale, skainet_stream_t stream) {
    KvStore* s = kv_from_handle(h);
    if (!s) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(layer >= 0 && layer < s->layers, "kv_attn_decode: layer index %d out of range [0, %d)", layer, s->layers);
    SK_REQUIRE(q_heads > 0 && q_heads % s->heads == 0, "kv_attn_decode: query heads %d not a multiple of the cache's %d heads", q_heads, s->heads);
    const int G = q_heads / s->heads;
    SK_REQUIRE(s->tq || G == 1 || G == 2 || G == 4 || G == 8, "kv_attn_decode: query heads per cache head %d not in {1,2,4,8}", G);
    // the token being decoded counts once its slot of this layer is written, i.e. up to currentSeqLen + 1 before the last layer's append
    const int cur_incl = std::min(s->cur + 1, s->ring ? INT32_MAX : s->max_seq);
    SK_REQUIRE(to_pos <= cur_incl, "kv_attn_decode: window end %d exceeds currentSeqLen=%d (+1 for the token in flight)", to_pos, s->cur);
    const int oldest = std::max(s->oldest, s->ring ? std::max(to_pos - s->max_seq, 0) : 0);
    SK_REQUIRE(from_pos >= oldest && from_pos < to_pos, "kv_attn_decode: window [%d, %d) is empty or starts before the oldest held position (%d)",
               from_pos, to_pos, oldest);
    SK_REQUIRE(q_dev && out_dev, "kv_attn_decode: null pointer");
    SK_REQUIRE(((uintptr_t) q_dev & 15) == 0, "kv_attn_decode: q must be 16-byte aligned");
    SK_TRY(kv_use(s));
    cudaStream_t st = as_stream(stream);
    const int len = to_pos - from_pos;
    const float sc0 = scale != 0.0f ? scale : 1.0f / sqrtf((float) s->head_dim);
    if (s->tq) {
        SK_REQUIRE(to_pos <= s->cur, "kv_attn_decode: a TurboQuant store attends appended positions only (window end %d, currentSeqLen %d)", to_pos, s->cur);
        const size_t plane = (size_t) s->heads * len * s->head_dim;
        void* win = nullptr;
        if ((G == 1 || G == 2 || G == 4 || G == 8) && (s->head_dim == 64 || s->head_dim == 128)) {
            // the window's blocks decoded to binary16 rows [heads][len][head_dim], then the split-K decode attention over them
            // (the rounding the binary16 store applies to every row it holds)
            SK_TRY(scratch_get(st, SCRATCH_FUSED, 2 * plane * sizeof(__half), &win));
            __half* kh = (__half*) win; __half* vh = kh + plane;
            SK_TRY(launch_tq_decode_f16(s->kq, layer, from_pos, len, s->heads, s->head_dim, s->max_seq, 0, kh, st));
            SK_TRY(launch_tq_decode_f16(s->vq, layer, from_pos, len, s->heads, s->head_dim, s->max_seq, TQ_VALUE_SEED_XOR, vh, st));
            void* scratch = nullptr;
            SK_TRY(scratch_get(st, SCRATCH_ATTN, attn_scratch_bytes(1, q_heads, s->head_dim, len), &scratch));
            kv_set_int_kernel<<<1, 1, 0, st>>>(s->d_len, len);
            SK_CUDA(cudaGetLastError());
            return launch_attn_decode_ring(q_dev, kh, vh, out_dev, q_heads, s->heads, s->head_dim, len, s->d_len, len, sc0, 0, 0, scratch, st);
        }
        // other head sizes / group sizes: fp32 rows [heads][len][head_dim] (what readKeys / readValues return), attended in fp32
        SK_TRY(scratch_get(st, SCRATCH_FUSED, 2 * plane * sizeof(float), &win));
        float* kw = (float*) win; float* vw = kw + plane;
        SK_TRY(launch_tq_decode(s->kq, layer, from_pos, len, s->heads, s->head_dim, s->max_seq, 0, kw, st));
        SK_TRY(launch_tq_decode(s->vq, layer, from_pos, len, s->heads, s->head_dim, s->max_seq, TQ_VALUE_SEED_XOR, vw, st));
        return launch_sdpa_f32(q_dev, kw, vw, out_dev, 1, q_heads, s->heads, 1, len, s->head_dim, sc0, 1, 0, 0, nullptr, nullptr, 1, 1, 1, 1, st);
    }
    void* scratch = nullptr;
    SK_TRY(scratch_get(st, SCRATCH_ATTN, attn_scratch_bytes(1, q_heads, s->head_dim, len), &scratch));
    kv_set_int_kernel<<<1, 1, 0, st>>>(s->d_len, len);
    SK_CUDA(cudaGetLastError());
    const size_t off = (size_t) layer * s->layer_elems();
    const float sc = scale != 0.0f ? scale : 1.0f / sqrtf((float) s->head_dim);          // 0 means 1/sqrt(headDim), as WindowedAttention.decodeStep
    return launch_attn_decode_ring(q_dev, s->k + off, s->v + off, out_dev, q_heads, s->heads, s->head_dim, s->max_seq, s->d_len, len, sc,
                                   s->slot_of(from_pos), s->ring ? s->max_seq : 0, scratch, st);
}

}  // extern "C"
