// The C ABI of libskainet_cuda (include/skainet_cuda.h): argument validation, error reporting,
// the resident-weight registry, per-stream scratch, and the host-pointer twins of the reference's
// native entry points, which are thin wrappers over the resident API (upload, run, read back).
#include "common.cuh"
#include <cstdlib>
#include "matvec_fused.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_set>
#include <vector>

namespace sk {

// ---- errors ----------------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int32_t cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    set_error("CUDA error %d (%s) at %s:%d in %s", (int) e, cudaGetErrorString(e), file, line, what);
    if (e == cudaErrorMemoryAllocation) { cudaGetLastError(); return SKAINET_CUDA_ERR_OOM; }
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) return SKAINET_CUDA_ERR_NODEVICE;
    return SKAINET_CUDA_ERR_CUDA;
}

// ---- device ------------------------------------------------------------------------------------------------
static std::mutex g_mu;
static int g_dev_count = -2;                    // -2 = not probed
static thread_local int t_device = 0;
static thread_local bool t_device_set = false;
static int g_sm_count[64] = {0};

static int probe_devices() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev_count != -2) return g_dev_count;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; set_error("no CUDA device: %s", cudaGetErrorString(e)); }
    g_dev_count = n;
    return n;
}

int32_t ensure_device() {
    const int n = probe_devices();
    if (n <= 0) { set_error("no usable CUDA device (this library has no CPU fallback)"); return SKAINET_CUDA_ERR_NODEVICE; }
    if (!t_device_set) {
        if (t_device >= n) { set_error("device %d out of range (%d present)", t_device, n); return SKAINET_CUDA_ERR_NODEVICE; }
        SK_CUDA(cudaSetDevice(t_device));
        cudaDeviceProp p;
        SK_CUDA(cudaGetDeviceProperties(&p, t_device));
        if (p.major < 10) {
            set_error("device %d is sm_%d%d; this library is built for sm_100a only", t_device, p.major, p.minor);
            return SKAINET_CUDA_ERR_NODEVICE;
        }
        if (t_device < 64) g_sm_count[t_device] = p.multiProcessorCount;
        t_device_set = true;
    }
    return SKAINET_CUDA_OK;
}

// The CUDA device current on the calling thread (what every launch of this thread targets).
static int current_device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) { cudaGetLastError(); d = 0; }
    return d;
}

int sm_count() {
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return 148;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) g_sm_count[dev] = n;
        else cudaGetLastError();
    }
    return g_sm_count[dev] > 0 ? g_sm_count[dev] : 148;
}

// Makes `device` current on this thread and records it as the thread's device, so that later calls of the
// thread (flag, SM count, scratch) all refer to the device its kernels really run on.
int32_t set_thread_device(int device) {
    SK_TRY(ensure_device());
    if (device != t_device || current_device() != device) {
        SK_CUDA(cudaSetDevice(device));
        t_device = device;
    }
    return SKAINET_CUDA_OK;
}

static std::map<std::pair<int, const void*>, int> g_smem_attr;
int32_t ensure_dynamic_smem(const void* kernel, int bytes) {
    const int dev = current_device();
    std::lock_guard<std::mutex> lk(g_mu);
    int& have = g_smem_attr[{dev, kernel}];
    if (have >= bytes) return SKAINET_CUDA_OK;
    SK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    have = bytes;
    return SKAINET_CUDA_OK;
}

// One int per device, set by kernels whose bounded waits give up (1 = a wait on an asynchronous copy or
// tensor-core barrier, 2 = a wait on a tensor-parallel peer). Keyed on the device that is current when it is
// asked for, and allocated with that device current, so a kernel never receives a flag that lives on another GPU.
static int* g_timeout_flag[64] = {nullptr};
int* device_timeout_flag() {
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_timeout_flag[dev]) {
        int* p = nullptr;
        if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cudaMemset(p, 0, sizeof(int));
        g_timeout_flag[dev] = p;
    }
    return g_timeout_flag[dev];
}

// Turns a raised flag value into the status and message the entry points return.
int32_t timeout_status(int value) {
    if (value == 0) return SKAINET_CUDA_OK;
    if (value == 2) set_error("a kernel's bounded wait on a tensor-parallel peer ran out (a rank is late or gone); the step's outputs are not valid");
    else set_error("a kernel's bounded wait on an asynchronous copy or tensor-core barrier ran out; its outputs are not valid");
    return SKAINET_CUDA_ERR_TIMEOUT;
}

// ---- weight registry ---------------------------------------------------------------------------------------
static const uint64_t WEIGHT_MAGIC = 0x534b57454947ull;
static std::unordered_set<Weight*> g_weights;

Weight* weight_from_handle(skainet_weight_t h) {
    Weight* w = reinterpret_cast<Weight*>(h);
    std::lock_guard<std::mutex> lk(g_mu);
    if (w == nullptr || g_weights.find(w) == g_weights.end() || w->magic != WEIGHT_MAGIC) {
        set_error("unknown or freed weight handle %lld", (long long) h);
        return nullptr;
    }
    return w;
}

static inline size_t a256(size_t x) { return (x + 255) & ~(size_t) 255; }

static int32_t validate_geometry(int enc, int rows, int cols, const char* who) {
    SK_REQUIRE(block_bytes(enc) != 0, "%s: unknown encoding %d", who, enc);
    SK_REQUIRE(rows >= 0 && cols >= 0, "%s: negative shape [%d, %d]", who, rows, cols);
    SK_REQUIRE(cols % block_elems(enc) == 0, "%s: inputDim must be a multiple of %d; got %d", who, block_elems(enc), cols);
    return SKAINET_CUDA_OK;
}

// Allocates the planes of a [rows, cols] weight (one allocation, 256-byte aligned planes).
int32_t weight_alloc(int enc, int rows, int cols, Weight** out) {
    SK_TRY(ensure_device());
    Weight* w = new Weight();
    w->enc = enc; w->rows = rows; w->cols = cols; w->bpr = cols / block_elems(enc);
    const size_t nb = (size_t) rows * w->bpr;
    w->packed_bytes = (int64_t) (nb * block_bytes(enc));
    size_t s_qs = 0, s_hdr = 0, s_extra = 0, s_aux = 0;
    switch (enc) {
        case SKAINET_ENC_Q8_0: s_qs = nb * 32; s_hdr = nb * 2; break;
        case SKAINET_ENC_Q4_K: s_qs = nb * 128; s_hdr = nb * 16; break;
        case SKAINET_ENC_Q5_K: s_qs = nb * 128; s_hdr = nb * 16; s_extra = nb * 32; break;
        default:               s_qs = nb * 128; s_hdr = nb * 16; s_extra = nb * 64; s_aux = nb * 2; break;
    }
    const size_t total = a256(s_qs) + a256(s_hdr) + a256(s_extra) + a256(s_aux) + 256;
    cudaError_t e = cudaMalloc(&w->base, total);
    if (e != cudaSuccess) { delete w; return cuda_fail(e, "cudaMalloc(weight)", __FILE__, __LINE__); }
    uint8_t* p = (uint8_t*) w->base;
    w->qs = p; p += a256(s_qs);
    w->hdr = p; p += a256(s_hdr);
    w->extra = s_extra ? p : nullptr; p += a256(s_extra);
    w->aux = s_aux ? p : nullptr;
    cudaGetDevice(&w->device);
    w->magic = WEIGHT_MAGIC;
    { std::lock_guard<std::mutex> lk(g_mu); g_weights.insert(w); }
    *out = w;
    return SKAINET_CUDA_OK;
}

skainet_weight_t weight_to_handle(Weight* w) { return (skainet_weight_t) reinterpret_cast<intptr_t>(w); }

void weight_release(Weight* w) {
    { std::lock_guard<std::mutex> lk(g_mu); g_weights.erase(w); }
    if (w->base) cudaFree(w->base);
    w->magic = 0;
    delete w;
}

// ---- per-stream scratch ---------------------------------------------------------------------------------------
struct ScratchBuf { void* p = nullptr; size_t n = 0; };
static std::map<std::pair<int, cudaStream_t>, std::vector<ScratchBuf>> g_scratch;

int32_t scratch_get(cudaStream_t stream, int slot, size_t nbytes, void** out) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    auto& v = g_scratch[{dev, stream}];
    if (v.empty()) v.resize(SCRATCH_SLOTS);
    ScratchBuf& b = v[slot];
    if (b.n < nbytes) {
        // Growing frees the old buffer: wait for work that may still read it.
        if (b.p) { SK_CUDA(cudaStreamSynchronize(stream)); cudaFree(b.p); b.p = nullptr; b.n = 0; }
        const size_t want = std::max(nbytes, (size_t) 1 << 16);
        cudaError_t e = cudaMalloc(&b.p, want);
        if (e != cudaSuccess) { b.p = nullptr; return cuda_fail(e, "cudaMalloc(scratch)", __FILE__, __LINE__); }
        b.n = want;
    }
    *out = b.p;
    return SKAINET_CUDA_OK;
}

size_t scratch_capacity(cudaStream_t stream, int slot) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_scratch.find({dev, stream});
    return it == g_scratch.end() || it->second.empty() ? 0 : it->second[slot].n;
}

void scratch_release(cudaStream_t stream) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_scratch.find({dev, stream});
    if (it == g_scratch.end()) return;
    for (auto& b : it->second) if (b.p) cudaFree(b.p);
    g_scratch.erase(it);
}

// Host twins share the default stream's staging buffers: one twin call at a time per process.
static std::mutex g_twin_mu;
std::mutex& twin_mutex() { return g_twin_mu; }
#define SK_TWIN_LOCK() std::lock_guard<std::mutex> _twin_lk(::sk::g_twin_mu)

// A host twin's device staging: upload `n` bytes into a scratch slot of the default stream.
static int32_t stage_in(int slot, const void* host, size_t n, void** dev) {
    SK_TRY(scratch_get(nullptr, slot, std::max<size_t>(n, 16), dev));
    if (n) SK_CUDA(cudaMemcpyAsync(*dev, host, n, cudaMemcpyHostToDevice, nullptr));
    return SKAINET_CUDA_OK;
}

}  // namespace sk

using namespace sk;

// =====================================================================================================
extern "C" {

const char* skainet_cuda_last_error(void) { return g_err; }
const char* skainet_cuda_version(void) { return "skainet-backend-cuda 0.1 (sm_100a)"; }

int32_t skainet_cuda_device_count(void) { return probe_devices(); }

int32_t skainet_cuda_set_device(int32_t device) {
    const int n = probe_devices();
    if (n <= 0) { set_error("no usable CUDA device"); return SKAINET_CUDA_ERR_NODEVICE; }
    SK_REQUIRE(device >= 0 && device < n, "set_device: %d out of range (%d present)", device, n);
    t_device = device;
    t_device_set = false;
    return ensure_device();
}

int32_t skainet_cuda_device_info(int64_t* out4) {
    SK_REQUIRE(out4 != nullptr, "device_info: null output");
    SK_TRY(ensure_device());
    cudaDeviceProp p;
    SK_CUDA(cudaGetDeviceProperties(&p, t_device));
    out4[0] = p.multiProcessorCount; out4[1] = p.l2CacheSize; out4[2] = (int64_t) p.totalGlobalMem; out4[3] = p.major * 10 + p.minor;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_device_status(void) {
    SK_TRY(ensure_device());
    int* flag = device_timeout_flag();
    if (!flag) return SKAINET_CUDA_OK;
    int v = 0;
    SK_CUDA(cudaMemcpy(&v, flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) cudaMemset(flag, 0, sizeof(int));
    return timeout_status(v);
}

int32_t skainet_cuda_selftest_bounded_wait(int32_t* outcome) {
    SK_REQUIRE(outcome != nullptr, "selftest_bounded_wait: null output");
    SK_TRY(ensure_device());
    SK_REQUIRE(device_timeout_flag() != nullptr, "selftest_bounded_wait: the device flag is unavailable");
    int* d = nullptr;
    SK_CUDA(cudaMalloc((void**) &d, sizeof(int)));
    cudaMemset(d, 0, sizeof(int));
    int32_t st = launch_bounded_wait_selftest(d, (cudaStream_t) 0);
    int v = 0;
    if (st == SKAINET_CUDA_OK && cudaMemcpy(&v, d, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) st = cuda_fail(cudaGetLastError(), "cudaMemcpy", __FILE__, __LINE__);
    cudaFree(d);
    *outcome = v;
    return st;
}

// ---- resident API ---------------------------------------------------------------------------------------------
int32_t skainet_cuda_malloc(void** dev_ptr, int64_t nbytes) {
    SK_REQUIRE(dev_ptr != nullptr && nbytes >= 0, "malloc: bad arguments");
    SK_TRY(ensure_device());
    *dev_ptr = nullptr;
    if (nbytes == 0) return SKAINET_CUDA_OK;
    SK_CUDA(cudaMalloc(dev_ptr, (size_t) nbytes));
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_free(void* dev_ptr) {
    if (dev_ptr) SK_CUDA(cudaFree(dev_ptr));
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_memcpy_h2d(void* dst, const void* src, int64_t n, skainet_stream_t stream) {
    SK_REQUIRE(n >= 0 && (n == 0 || (dst && src)), "memcpy_h2d: bad arguments");
    SK_TRY(ensure_device());
    if (n) SK_CUDA(cudaMemcpyAsync(dst, src, (size_t) n, cudaMemcpyHostToDevice, as_stream(stream)));
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_memcpy_d2h(void* dst, const void* src, int64_t n, skainet_stream_t stream) {
    SK_REQUIRE(n >= 0 && (n == 0 || (dst && src)), "memcpy_d2h: bad arguments");
    SK_TRY(ensure_device());
    if (n) {
        SK_CUDA(cudaMemcpyAsync(dst, src, (size_t) n, cudaMemcpyDeviceToHost, as_stream(stream)));
        SK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    }
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_stream_create(skainet_stream_t* out) {
    SK_REQUIRE(out != nullptr, "stream_create: null output");
    SK_TRY(ensure_device());
    cudaStream_t s;
    SK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = (skainet_stream_t) s;
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_stream_destroy(skainet_stream_t stream) {
    if (stream) {
        SK_CUDA(cudaStreamSynchronize(as_stream(stream)));
        scratch_release(as_stream(stream));          // the stream's scratch goes with it
        SK_CUDA(cudaStreamDestroy(as_stream(stream)));
    }
    return SKAINET_CUDA_OK;
}
int32_t skainet_cuda_stream_sync(skainet_stream_t stream) {
    SK_TRY(ensure_device());
    SK_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return SKAINET_CUDA_OK;
}

static int32_t weight_build(const uint8_t* bytes, bool on_device, int64_t nbytes, int32_t enc, int32_t rows, int32_t cols,
                            int32_t order, skainet_weight_t* out) {
    SK_REQUIRE(out != nullptr, "weight_upload: null output");
    *out = 0;
    SK_TRY(validate_geometry(enc, rows, cols, "weight_upload"));
    SK_REQUIRE(order == SKAINET_ORDER_ROW_MAJOR || order == SKAINET_ORDER_INPUT_MAJOR, "weight_upload: unknown order %d", order);
    const int64_t need = (int64_t) rows * (cols / block_elems(enc)) * block_bytes(enc);
    SK_REQUIRE(nbytes == need, "weight_upload: %lld bytes given, [%d, %d] needs %lld", (long long) nbytes, rows, cols, (long long) need);
    SK_REQUIRE(need == 0 || bytes != nullptr, "weight_upload: null bytes");
    Weight* w = nullptr;
    SK_TRY(weight_alloc(enc, rows, cols, &w));
    int32_t st = SKAINET_CUDA_OK;
    if (need > 0) {
        void* staged = nullptr;
        const uint8_t* src = bytes;
        if (!on_device) {
            cudaError_t e = cudaMalloc(&staged, (size_t) need + 16);
            if (e != cudaSuccess) { weight_release(w); return cuda_fail(e, "cudaMalloc(staging)", __FILE__, __LINE__); }
            e = cudaMemcpy(staged, bytes, (size_t) need, cudaMemcpyHostToDevice);
            if (e != cudaSuccess) { cudaFree(staged); weight_release(w); return cuda_fail(e, "cudaMemcpy(weight)", __FILE__, __LINE__); }
            src = (const uint8_t*) staged;
        } else if (((uintptr_t) bytes & 1) != 0) {
            weight_release(w);
            set_error("weight_from_device: device bytes must be 2-byte aligned");
            return SKAINET_CUDA_ERR_INVALID;
        }
        st = launch_split_planes(src, *w, order, nullptr);
        if (st == SKAINET_CUDA_OK) {
            cudaError_t e = cudaStreamSynchronize(nullptr);
            if (e != cudaSuccess) st = cuda_fail(e, "split planes", __FILE__, __LINE__);
        }
        if (staged) cudaFree(staged);
    }
    if (st != SKAINET_CUDA_OK) { weight_release(w); return st; }
    *out = (skainet_weight_t) reinterpret_cast<intptr_t>(w);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_weight_upload(const uint8_t* host_bytes, int64_t nbytes, int32_t enc, int32_t rows, int32_t cols,
                                   int32_t order, skainet_weight_t* out) {
    return weight_build(host_bytes, false, nbytes, enc, rows, cols, order, out);
}
int32_t skainet_cuda_weight_from_device(const uint8_t* dev_bytes, int64_t nbytes, int32_t enc, int32_t rows, int32_t cols,
                                        int32_t order, skainet_weight_t* out) {
    return weight_build(dev_bytes, true, nbytes, enc, rows, cols, order, out);
}

int32_t skainet_cuda_weight_synth(int32_t enc, int32_t rows, int32_t cols, uint64_t seed, float std, int32_t mode,
                                  skainet_weight_t* out) {
    SK_REQUIRE(out != nullptr, "weight_synth: null output");
    *out = 0;
    SK_TRY(validate_geometry(enc, rows, cols, "weight_synth"));
    SK_REQUIRE(enc == SKAINET_ENC_Q4_K || enc == SKAINET_ENC_Q8_0, "weight_synth: encoding %d not supported", enc);
    SK_REQUIRE(mode == 0 || mode == 1, "weight_synth: mode %d", mode);
    Weight* w = nullptr;
    SK_TRY(weight_alloc(enc, rows, cols, &w));
    int32_t st = launch_synth(*w, seed, std, mode, 0, 0, cols, nullptr);
    if (st == SKAINET_CUDA_OK) {
        cudaError_t e = cudaStreamSynchronize(nullptr);
        if (e != cudaSuccess) st = cuda_fail(e, "weight_synth", __FILE__, __LINE__);
    }
    if (st != SKAINET_CUDA_OK) { weight_release(w); return st; }
    *out = (skainet_weight_t) reinterpret_cast<intptr_t>(w);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_weight_export(skainet_weight_t h, uint8_t* host_bytes, int64_t nbytes) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(nbytes == w->packed_bytes, "weight_export: %lld bytes given, weight holds %lld", (long long) nbytes, (long long) w->packed_bytes);
    if (nbytes == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(host_bytes != nullptr, "weight_export: null output");
    SK_TRY(ensure_device());
    void* tmp = nullptr;
    SK_CUDA(cudaMalloc(&tmp, (size_t) nbytes + 16));
    int32_t st = launch_join_planes(*w, (uint8_t*) tmp, nullptr);
    if (st == SKAINET_CUDA_OK) {
        cudaError_t e = cudaMemcpy(host_bytes, tmp, (size_t) nbytes, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = cuda_fail(e, "weight_export copy", __FILE__, __LINE__);
    }
    cudaFree(tmp);
    return st;
}

int32_t skainet_cuda_weight_info(skainet_weight_t h, int64_t* out4) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(out4 != nullptr, "weight_info: null output");
    out4[0] = w->enc; out4[1] = w->rows; out4[2] = w->cols; out4[3] = w->packed_bytes;
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_weight_free(skainet_weight_t h) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    weight_release(w);
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_weight_dequant(skainet_weight_t h, float* dev_out, skainet_stream_t stream) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(dev_out != nullptr || w->rows * (int64_t) w->cols == 0, "weight_dequant: null output");
    SK_TRY(ensure_device());
    return launch_dequant_weight(*w, dev_out, as_stream(stream));
}

constexpr int MATMUL_PROLOGUE_MAX_COLS = 12288;

int32_t skainet_cuda_matmul_dev(skainet_weight_t h, const float* x_dev, int32_t m, float* y_dev, int32_t act_mode,
                                skainet_stream_t stream) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_REQUIRE(m >= 0, "matmul: negative row count %d", m);
    SK_REQUIRE(act_mode == SKAINET_ACT_NATIVE || act_mode == SKAINET_ACT_F32, "matmul: unknown activation mode %d", act_mode);
    if (m == 0 || w->rows == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(x_dev != nullptr && y_dev != nullptr, "matmul: null activation or output");
    SK_REQUIRE(((uintptr_t) x_dev & 15) == 0, "matmul: the activation must be 16-byte aligned");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    if (w->cols == 0) { SK_CUDA(cudaMemsetAsync(y_dev, 0, sizeof(float) * (size_t) m * w->rows, s)); return SKAINET_CUDA_OK; }
    // One activation row of a Q4_K weight of 4 MB or more: a single launch, the ring kernel quantizes the row in its own
    // prologue (once per SM) while the first weight stages are in flight (config 2: 5.7 / 7.2 us per matvec against
    // 8.0 / 8.4 us for a quantizer launch followed by the matvec).
    if (m == 1 && act_mode == SKAINET_ACT_NATIVE && w->enc == SKAINET_ENC_Q4_K && w->cols <= MATMUL_PROLOGUE_MAX_COLS && matvec_uses_ring(*w, PREP_F32)) {
        MatvecIn in; in.x = x_dev;
        const int32_t st = launch_matvec_fused(*w, in, PREP_F32, y_dev, nullptr, s);
        if (st != 1) return st;
    }
    void* scratch = nullptr;
    const size_t need = act_scratch_bytes(w->enc, act_mode, m, w->cols);
    if (need) SK_TRY(scratch_get(s, SCRATCH_ACT, need, &scratch));
    SK_TRY(launch_act_quant(w->enc, act_mode, x_dev, m, w->cols, scratch, s));
    // Otherwise one row = quantizer launch, then the streaming matvec over the quantized row. In the one-tile kernel
    // (small weights, Q8_0) quantizing in every CTA's prologue measured slower (Q8_0 4096 x 4096: 7.2 against 6.8 us):
    // every CTA pulls the fp32 row out of L2 again.
    if (m == 1 && act_mode == SKAINET_ACT_NATIVE && (w->enc == SKAINET_ENC_Q4_K || w->enc == SKAINET_ENC_Q8_0)) {
        MatvecIn in;
        if (w->enc == SKAINET_ENC_Q8_0) in.split = act_split_layout(scratch, 1, w->cols); else in.q8 = act_q8k_layout(scratch, 1, w->cols);
        const int32_t st = launch_matvec_fused(*w, in, PREP_QUANTIZED, y_dev, nullptr, s);
        if (st != 1) return st;
    }
    return launch_matvec(*w, x_dev, scratch, m, y_dev, act_mode, s);
}

int32_t skainet_cuda_probe_read_dev(skainet_weight_t h, skainet_stream_t stream) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    SK_TRY(ensure_device());
    void* sink = nullptr;
    SK_TRY(scratch_get(as_stream(stream), SCRATCH_FUSED2, 64, &sink));
    return launch_probe_read(*w, (uint32_t*) sink, as_stream(stream));
}

int32_t skainet_cuda_matvec_fused_dev(skainet_weight_t h, const float* x_dev, const float* gamma_dev, float eps,
                                      const float* resid_dev, float* y_dev, skainet_stream_t stream) {
    Weight* w = weight_from_handle(h);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    if (w->rows == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(x_dev != nullptr && y_dev != nullptr, "matvec_fused: null activation or output");
    SK_REQUIRE((((uintptr_t) x_dev | (uintptr_t) gamma_dev) & 15) == 0, "matvec_fused: x and gamma must be 16-byte aligned");
    SK_REQUIRE(w->cols > 0, "matvec_fused: empty input dimension");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    MatvecIn in; in.x = x_dev; in.gamma = gamma_dev; in.eps = eps;
    const int32_t st = launch_matvec_fused(*w, in, gamma_dev ? PREP_NORM_F32 : PREP_F32, y_dev, resid_dev, s);
    if (st != 1) return st;
    // shapes the fused kernel does not take: the same result from the general kernels
    const float* xin = x_dev;
    if (gamma_dev) {
        void* tmp = nullptr;
        SK_TRY(scratch_get(s, SCRATCH_FUSED, sizeof(float) * (size_t) w->cols, &tmp));
        SK_TRY(launch_rms_norm(x_dev, gamma_dev, (float*) tmp, 1, w->cols, eps, s));
        xin = (const float*) tmp;
    }
    float* yout = y_dev;
    if (resid_dev) {
        void* tmp = nullptr;
        SK_TRY(scratch_get(s, SCRATCH_FUSED2, sizeof(float) * (size_t) w->rows, &tmp));
        yout = (float*) tmp;
    }
    void* scratch = nullptr;
    const size_t need = act_scratch_bytes(w->enc, SKAINET_ACT_NATIVE, 1, w->cols);
    if (need) SK_TRY(scratch_get(s, SCRATCH_ACT, need, &scratch));
    SK_TRY(launch_act_quant(w->enc, SKAINET_ACT_NATIVE, xin, 1, w->cols, scratch, s));
    SK_TRY(launch_matvec(*w, xin, scratch, 1, yout, SKAINET_ACT_NATIVE, s));
    if (resid_dev) SK_TRY(launch_binary(0, resid_dev, 0, yout, 0, y_dev, w->rows, 1, s));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_rms_norm_dev(const float* in, const float* gamma, float* out, int32_t rows, int32_t cols, float eps,
                                  skainet_stream_t stream) {
    if (rows <= 0 || cols <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(in && out, "rms_norm: null pointer");
    SK_TRY(ensure_device());
    return launch_rms_norm(in, gamma, out, rows, cols, eps, as_stream(stream));
}
int32_t skainet_cuda_unary_dev(int32_t op, const float* in, float* out, int64_t n, skainet_stream_t stream) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(op >= 0 && op <= 6, "unary: unknown op %d", op);
    SK_REQUIRE(in && out, "unary: null pointer");
    SK_TRY(ensure_device());
    return launch_unary(op, in, out, n, as_stream(stream));
}
int32_t skainet_cuda_binary_dev(int32_t op, const float* a, int32_t am, const float* b, int32_t bm, float* out, int64_t n,
                                int32_t inner, skainet_stream_t stream) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(op >= 0 && op <= 3, "binary: unknown op %d", op);
    SK_REQUIRE(am >= 0 && am <= 2 && bm >= 0 && bm <= 2, "binary: unknown operand mode");
    SK_REQUIRE(a && b && out, "binary: null pointer");
    SK_TRY(ensure_device());
    return launch_binary(op, a, am, b, bm, out, n, inner, as_stream(stream));
}
int32_t skainet_cuda_swiglu_dev(const float* gate, const float* up, float* out, int64_t n, skainet_stream_t stream) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(gate && up && out, "swiglu: null pointer");
    SK_TRY(ensure_device());
    return launch_swiglu(gate, up, out, n, as_stream(stream));
}
int32_t skainet_cuda_rope_dev(float* x, const int32_t* positions, int32_t rows, int32_t heads, int32_t head_dim, float theta,
                              int32_t mode, skainet_stream_t stream) {
    if (rows <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope: head_dim %d must be even", head_dim);
    SK_REQUIRE(mode == 0 || mode == 1, "rope: unknown mode %d", mode);
    SK_REQUIRE(x && positions, "rope: null pointer");
    SK_TRY(ensure_device());
    return launch_rope(x, positions, rows, heads, head_dim, theta, mode, as_stream(stream));
}
int32_t skainet_cuda_argmax_dev(const float* x, int32_t rows, int32_t cols, int32_t* out_idx, skainet_stream_t stream) {
    if (rows <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(cols > 0, "argmax: empty rows");
    SK_REQUIRE(x && out_idx, "argmax: null pointer");
    SK_TRY(ensure_device());
    return launch_argmax(x, rows, cols, out_idx, as_stream(stream));
}
int32_t skainet_cuda_embed_dev(skainet_weight_t table, const int32_t* ids_dev, int32_t n, float* out, skainet_stream_t stream) {
    Weight* w = weight_from_handle(table);
    if (!w) return SKAINET_CUDA_ERR_HANDLE;
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(ids_dev && out, "embed: null pointer");
    SK_TRY(ensure_device());
    return launch_embed(*w, ids_dev, n, out, as_stream(stream));
}
int32_t skainet_cuda_f32_to_f16_dev(const float* in, uint16_t* out, int64_t n, skainet_stream_t stream) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(in && out, "f32_to_f16: null pointer");
    SK_TRY(ensure_device());
    return launch_f32_to_f16(in, out, n, as_stream(stream));
}

int32_t skainet_cuda_sdpa_dev(const float* q, const float* k, const float* v, float* out, int32_t batch, int32_t heads, int32_t kv_heads,
                              int32_t seq_q, int32_t seq_kv, int32_t head_dim, float scale, int32_t causal, int32_t window, int32_t right_context,
                              const int32_t* lengths_dev, const float* mask_dev, int32_t mask_b, int32_t mask_h, int32_t mask_q, int32_t mask_k,
                              skainet_stream_t stream) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || seq_q <= 0 || head_dim <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(q && out, "sdpa: null pointer");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    if (seq_kv <= 0) { SK_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * (size_t) batch * heads * seq_q * head_dim, s)); return SKAINET_CUDA_OK; }
    SK_REQUIRE(k && v, "sdpa: null pointer");
    SK_REQUIRE(heads % kv_heads == 0, "sdpa: heads %d not a multiple of kv_heads %d", heads, kv_heads);
    SK_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256, "sdpa: head_dim %d not in {32,64,128,256}", head_dim);
    if (mask_dev) {
        SK_REQUIRE((mask_b == 1 || mask_b == batch) && (mask_h == 1 || mask_h == heads || mask_h == kv_heads) &&
                   (mask_q == 1 || mask_q == seq_q) && (mask_k == 1 || mask_k == seq_kv), "sdpa: mask dims do not broadcast");
    }
    return launch_sdpa_f32(q, k, v, out, batch, heads, kv_heads, seq_q, seq_kv, head_dim, scale, causal, window, right_context, lengths_dev,
                           mask_dev, mask_b, mask_h, mask_q, mask_k, s);
}

int32_t skainet_cuda_attn_decode_dev(const float* q, const uint16_t* k_cache, const uint16_t* v_cache, float* out,
                                     int32_t batch, int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t cache_stride,
                                     const int32_t* kv_len_dev, int32_t max_kv_len, float scale, int32_t window,
                                     skainet_stream_t stream) {
    if (batch <= 0 || heads <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(kv_heads > 0 && heads % kv_heads == 0, "attn_decode: heads %d not a multiple of kv_heads %d", heads, kv_heads);
    SK_REQUIRE(head_dim == 64 || head_dim == 128, "attn_decode: head_dim %d not in {64,128}", head_dim);
    SK_REQUIRE(max_kv_len >= 0 && cache_stride >= max_kv_len, "attn_decode: cache_stride %lld < max_kv_len %d", (long long) cache_stride, max_kv_len);
    SK_REQUIRE(q && k_cache && v_cache && out && kv_len_dev, "attn_decode: null pointer");
    SK_REQUIRE((((uintptr_t) q | (uintptr_t) k_cache | (uintptr_t) v_cache) & 15) == 0, "attn_decode: q/k/v must be 16-byte aligned");
    SK_TRY(ensure_device());
    cudaStream_t s = as_stream(stream);
    void* scratch = nullptr;
    SK_TRY(scratch_get(s, SCRATCH_ATTN, attn_scratch_bytes(batch, heads, head_dim, std::max(1, max_kv_len)), &scratch));
    return launch_attn_decode(q, (const __half*) k_cache, (const __half*) v_cache, out, batch, heads, kv_heads, head_dim,
                              cache_stride, kv_len_dev, max_kv_len, scale, window, scratch, s);
}

// ---- drop-in twins (host pointers) ------------------------------------------------------------------------------
int32_t skainet_cuda_smoke_double(const float* input, float* output, int32_t length) {
    if (length <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(input && output, "smoke_double: null pointer");
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    void *din, *dout;
    SK_TRY(stage_in(SCRATCH_TWIN_A, input, sizeof(float) * (size_t) length, &din));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_B, sizeof(float) * (size_t) length, &dout));
    SK_TRY(launch_smoke((const float*) din, (float*) dout, length, nullptr));
    SK_CUDA(cudaMemcpy(output, dout, sizeof(float) * (size_t) length, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

// One host matvec: upload activation and weight, run, read back. The per-call weight upload mirrors the
// reference FFM path (which copies the whole weight off-heap per call,
// skainet-backends/skainet-backend-native-cpu/src/jvmMain/kotlin/sk/ainet/exec/kernel/NativeQ4KMatmulKernel.kt:61-74);
// callers that care about speed upload once and use skainet_cuda_matmul_dev.
static int32_t host_matvec(int enc, int order, const float* input, int32_t input_offset, const uint8_t* weight,
                           int32_t weight_byte_offset, int32_t input_dim, int32_t output_dim, float* output, int32_t output_offset) {
    const char* who = enc == SKAINET_ENC_Q4_K ? "q4k_matmul" : enc == SKAINET_ENC_Q8_0 ? "q8_0_matmul" : enc == SKAINET_ENC_Q6_K ? "q6k_matmul" : "q5k_matmul";
    SK_REQUIRE(input_dim < 0 || input_dim % block_elems(enc) == 0, "%s: inputDim must be a multiple of %d; got %d", who, block_elems(enc), input_dim);
    if (output_dim <= 0) return SKAINET_CUDA_OK;
    if (input_dim <= 0) {
        // Q8_0 zeroes the output (q8_0_matmul.c:175-179); the native K-quant kernels leave it untouched (q4k_matmul.c:326,
        // q6k_matmul.c:284, q5k_matmul.c:264).
        if (enc == SKAINET_ENC_Q8_0) { SK_REQUIRE(output, "%s: null output", who); memset(output + output_offset, 0, sizeof(float) * (size_t) output_dim); }
        return SKAINET_CUDA_OK;
    }
    SK_REQUIRE(input && weight && output, "%s: null pointer", who);
    SK_REQUIRE(input_offset >= 0 && weight_byte_offset >= 0 && output_offset >= 0, "%s: negative offset", who);
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    skainet_weight_t h = 0;
    const int64_t nbytes = (int64_t) output_dim * (input_dim / block_elems(enc)) * block_bytes(enc);
    SK_TRY(skainet_cuda_weight_upload(weight + weight_byte_offset, nbytes, enc, output_dim, input_dim, order, &h));
    void *dx = nullptr, *dy = nullptr;
    int32_t st = stage_in(SCRATCH_TWIN_A, input + input_offset, sizeof(float) * (size_t) input_dim, &dx);
    if (st == SKAINET_CUDA_OK) st = scratch_get(nullptr, SCRATCH_TWIN_B, sizeof(float) * (size_t) output_dim, &dy);
    if (st == SKAINET_CUDA_OK) st = skainet_cuda_matmul_dev(h, (const float*) dx, 1, (float*) dy, SKAINET_ACT_NATIVE, nullptr);
    if (st == SKAINET_CUDA_OK) {
        cudaError_t e = cudaMemcpy(output + output_offset, dy, sizeof(float) * (size_t) output_dim, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = cuda_fail(e, "matvec read-back", __FILE__, __LINE__);
    }
    skainet_cuda_weight_free(h);
    return st;
}

int32_t skainet_cuda_q4k_matmul(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q4_K, SKAINET_ORDER_INPUT_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q4k_matmul_rm(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q4_K, SKAINET_ORDER_ROW_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q8_0_matmul(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q8_0, SKAINET_ORDER_INPUT_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q8_0_matmul_rm(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q8_0, SKAINET_ORDER_ROW_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q6k_matmul(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q6_K, SKAINET_ORDER_INPUT_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q6k_matmul_rm(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q6_K, SKAINET_ORDER_ROW_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q5k_matmul(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q5_K, SKAINET_ORDER_INPUT_MAJOR, in, io, w, wo, k, n, out, oo);
}
int32_t skainet_cuda_q5k_matmul_rm(const float* in, int32_t io, const uint8_t* w, int32_t wo, int32_t k, int32_t n, float* out, int32_t oo) {
    return host_matvec(SKAINET_ENC_Q5_K, SKAINET_ORDER_ROW_MAJOR, in, io, w, wo, k, n, out, oo);
}

int32_t skainet_cuda_f32_rms_norm(const float* in, const float* gamma, float* out, int32_t rows, int32_t cols, float eps) {
    if (rows <= 0 || cols <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(in && out, "rms_norm: null pointer");
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    const size_t n = sizeof(float) * (size_t) rows * cols;
    void *din, *dg = nullptr, *dout;
    SK_TRY(stage_in(SCRATCH_TWIN_A, in, n, &din));
    if (gamma) SK_TRY(stage_in(SCRATCH_TWIN_B, gamma, sizeof(float) * (size_t) cols, &dg));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_C, n, &dout));
    SK_TRY(launch_rms_norm((const float*) din, (const float*) dg, (float*) dout, rows, cols, eps, nullptr));
    SK_CUDA(cudaMemcpy(out, dout, n, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_f32_sdpa(const float* q, const float* k, const float* v, float* out, int32_t batch, int32_t heads,
                              int32_t kv_heads, int32_t seq_q, int32_t seq_kv, int32_t head_dim, float scale, int32_t causal,
                              int32_t window, int32_t right_context, const int32_t* lengths, const float* mask,
                              int32_t mask_b, int32_t mask_h, int32_t mask_q, int32_t mask_k) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || seq_q <= 0 || head_dim <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(q && out, "sdpa: null pointer");
    const size_t nq = sizeof(float) * (size_t) batch * heads * seq_q * head_dim;
    if (seq_kv <= 0) { memset(out, 0, nq); return SKAINET_CUDA_OK; }   // f32_fused.c:384-387
    SK_REQUIRE(k && v, "sdpa: null pointer");
    SK_REQUIRE(heads % kv_heads == 0, "sdpa: heads %d not a multiple of kv_heads %d", heads, kv_heads);
    SK_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256, "sdpa: head_dim %d not in {32,64,128,256}", head_dim);
    if (mask) {
        SK_REQUIRE((mask_b == 1 || mask_b == batch) && (mask_h == 1 || mask_h == heads || mask_h == kv_heads) &&
                   (mask_q == 1 || mask_q == seq_q) && (mask_k == 1 || mask_k == seq_kv), "sdpa: mask dims do not broadcast");
    }
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    const size_t nkv = sizeof(float) * (size_t) batch * kv_heads * seq_kv * head_dim;
    void *dq, *dk, *dv, *dout, *dl = nullptr, *dm = nullptr;
    SK_TRY(stage_in(SCRATCH_TWIN_A, q, nq, &dq));
    SK_TRY(stage_in(SCRATCH_TWIN_B, k, nkv, &dk));
    SK_TRY(stage_in(SCRATCH_TWIN_C, v, nkv, &dv));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_D, nq, &dout));
    if (lengths) SK_TRY(stage_in(SCRATCH_TWIN_E, lengths, sizeof(int32_t) * (size_t) batch, &dl));
    if (mask) SK_TRY(stage_in(SCRATCH_TWIN_F, mask, sizeof(float) * (size_t) mask_b * mask_h * mask_q * mask_k, &dm));
    SK_TRY(launch_sdpa_f32((const float*) dq, (const float*) dk, (const float*) dv, (float*) dout, batch, heads, kv_heads, seq_q,
                           seq_kv, head_dim, scale, causal, window, right_context, (const int32_t*) dl, (const float*) dm,
                           mask_b, mask_h, mask_q, mask_k, nullptr));
    SK_CUDA(cudaMemcpy(out, dout, nq, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_f32_unary(int32_t op, const float* in, float* out, int32_t n) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(op >= 0 && op <= 6, "unary: unknown op %d", op);
    SK_REQUIRE(in && out, "unary: null pointer");
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    void *din, *dout;
    SK_TRY(stage_in(SCRATCH_TWIN_A, in, sizeof(float) * (size_t) n, &din));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_B, sizeof(float) * (size_t) n, &dout));
    SK_TRY(launch_unary(op, (const float*) din, (float*) dout, n, nullptr));
    SK_CUDA(cudaMemcpy(out, dout, sizeof(float) * (size_t) n, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_f32_binary(int32_t op, const float* a, int32_t am, const float* b, int32_t bm, float* out, int32_t n, int32_t inner) {
    if (n <= 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(op >= 0 && op <= 3, "binary: unknown op %d", op);
    SK_REQUIRE(am >= 0 && am <= 2 && bm >= 0 && bm <= 2, "binary: unknown operand mode");
    SK_REQUIRE(a && b && out, "binary: null pointer");
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    const int in_ = inner > 0 ? inner : 1;
    const size_t na = am == 0 ? n : (am == 1 ? 1 : std::min(n, in_)), nb = bm == 0 ? n : (bm == 1 ? 1 : std::min(n, in_));
    void *da, *db, *dout;
    SK_TRY(stage_in(SCRATCH_TWIN_A, a, sizeof(float) * na, &da));
    SK_TRY(stage_in(SCRATCH_TWIN_B, b, sizeof(float) * nb, &db));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_C, sizeof(float) * (size_t) n, &dout));
    SK_TRY(launch_binary(op, (const float*) da, am, (const float*) db, bm, (float*) dout, n, in_, nullptr));
    SK_CUDA(cudaMemcpy(out, dout, sizeof(float) * (size_t) n, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

int32_t skainet_cuda_dequant(int32_t enc, const uint8_t* packed, int64_t nblocks, float* out) {
    SK_REQUIRE(block_bytes(enc) != 0, "dequant: unknown encoding %d", enc);
    SK_REQUIRE(nblocks >= 0, "dequant: negative block count");
    if (nblocks == 0) return SKAINET_CUDA_OK;
    SK_REQUIRE(packed && out, "dequant: null pointer");
    SK_TRY(ensure_device());
    SK_TWIN_LOCK();
    const size_t nin = (size_t) nblocks * block_bytes(enc), nout = sizeof(float) * (size_t) nblocks * block_elems(enc);
    void *din, *dout;
    SK_TRY(stage_in(SCRATCH_TWIN_A, packed, nin, &din));
    SK_TRY(scratch_get(nullptr, SCRATCH_TWIN_B, nout, &dout));
    SK_TRY(launch_dequant_canonical(enc, (const uint8_t*) din, nblocks, (float*) dout, nullptr));
    SK_CUDA(cudaMemcpy(out, dout, nout, cudaMemcpyDeviceToHost));
    return SKAINET_CUDA_OK;
}

}  // extern "C"
