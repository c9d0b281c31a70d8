// extern "C" surface of libntb200: argument validation in the order the reference performs it, routing
// between the tcgen05 and CUDA-core GEMMs, the stream-ordered storage pool and the host-buffer variants.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "internal.h"

namespace ntb200 {

namespace {
thread_local char t_error[512] = "";
thread_local const char* t_route = "none";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_pool_in_use{0}, g_pool_high{0};
std::mutex g_pool_mu;
struct Block { void* ptr; size_t bytes; };
std::vector<Block> g_blocks;  // live pool allocations (for byte accounting)
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t err, const char* what) {
    const int code = (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver) ? NTB200_ERR_NO_DEVICE
                     : (err == cudaErrorMemoryAllocation)                              ? NTB200_ERR_ALLOC
                                                                                       : NTB200_ERR_CUDA;
    return fail(code, "%s: %s", what, cudaGetErrorString(err));
}

size_t dtype_size(int dtype) {
    switch (dtype) {
        case NTB200_F32: case NTB200_I32: case NTB200_U32: case NTB200_C32: return 4;
        case NTB200_F16: case NTB200_BF16: case NTB200_I16: case NTB200_U16: return 2;
        case NTB200_I8: case NTB200_U8: return 1;
        case NTB200_I64: case NTB200_F64: case NTB200_C64: return 8;
        case NTB200_C128: return 16;
    }
    return 0;
}

const char* dtype_name(int dtype) {
    static const char* names[] = {"Float32", "Float16", "BFloat16", "int8", "int16", "int32",
                                  "int64",   "Float64", "uint8",    "uint16", "uint32", "Complex64", "Complex128", "Complex32"};
    return (dtype >= 0 && dtype <= NTB200_C32) ? names[dtype] : "unknown";
}

void count_launch(int n) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }
void note_route(const char* name) { t_route = name; }

// The stream-ordered pool keeps freed blocks instead of returning them to the driver at every synchronisation
// (the default release threshold of 0 turns each allocate/free pair into a real cudaMalloc/cudaFree).
void keep_pool_memory() {
    static std::atomic<bool> done[64];   // zero-initialised; host threads may race here, setting it twice is harmless
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || done[dev].load(std::memory_order_acquire)) return;
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
        unsigned long long keep = ~0ull;
        (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    (void)cudaGetLastError();
    done[dev].store(true, std::memory_order_release);
}

int sm_count() {
    static std::atomic<int> cached[64];  // zero-initialised
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// ---- scratch of the library's own kernels ------------------------------------------------------------
// Hi/lo copies of the Float32 split, limb planes, partial tiles of K slices.  A block is kept per (device, stream)
// and handed to the next call on that stream: work on one stream runs in order, so the next kernel that writes the
// block starts after the last one that read it, and a GEMM call makes no cudaMallocAsync / cudaFreeAsync once its
// stream has a block that is large enough.  Blocks above the keep limit (NTB200_SCRATCH_KEEP_MB, default 512) are
// allocated and freed in stream order per call, as are blocks for a second host thread launching on the same stream
// at the same moment.
namespace {
struct ScratchBlock { int dev; cudaStream_t stream; void* ptr; size_t bytes; bool busy; uint64_t last_use; };
std::mutex g_scratch_mu;
std::vector<ScratchBlock> g_scratch;
uint64_t g_scratch_tick = 0;
std::atomic<uint64_t> g_scratch_acquires{0}, g_scratch_allocs{0};
constexpr size_t kScratchCacheEntries = 16;
size_t scratch_keep_limit() {
    static const size_t limit = [] {
        const char* e = getenv("NTB200_SCRATCH_KEEP_MB");
        const long v = e ? atol(e) : 512;
        return size_t(v < 0 ? 0 : v) << 20;
    }();
    return limit;
}
}  // namespace

int scratch_acquire(void** out, size_t bytes, cudaStream_t stream) {
    *out = nullptr;
    if (bytes == 0) bytes = 256;
    bytes = (bytes + ((size_t(1) << 20) - 1)) & ~((size_t(1) << 20) - 1);   // whole MiB: a slightly larger next call still fits
    g_scratch_acquires.fetch_add(1, std::memory_order_relaxed);
    int dev = 0;
    NTB200_CUDA(cudaGetDevice(&dev));
    const bool keep = bytes <= scratch_keep_limit();
    void* stale = nullptr;
    if (keep) {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        for (auto& b : g_scratch)
            if (b.dev == dev && b.stream == stream && !b.busy) {
                if (b.bytes >= bytes) {
                    b.busy = true;
                    b.last_use = ++g_scratch_tick;
                    *out = b.ptr;
                    return NTB200_OK;
                }
                stale = b.ptr;     // too small: replaced below (freed in stream order, after its last reader)
                b = g_scratch.back();
                g_scratch.pop_back();
                break;
            }
    }
    if (stale) (void)cudaFreeAsync(stale, stream);
    keep_pool_memory();
    g_scratch_allocs.fetch_add(1, std::memory_order_relaxed);
    NTB200_CUDA(cudaMallocAsync(out, bytes, stream));
    if (keep) {
        void* evict = nullptr;
        {
            std::lock_guard<std::mutex> lk(g_scratch_mu);
            if (g_scratch.size() >= kScratchCacheEntries) {   // drop the idle block that has not been used for longest
                size_t victim = g_scratch.size();
                for (size_t i = 0; i < g_scratch.size(); ++i)
                    if (!g_scratch[i].busy && (victim == g_scratch.size() || g_scratch[i].last_use < g_scratch[victim].last_use)) victim = i;
                if (victim < g_scratch.size()) {
                    evict = g_scratch[victim].ptr;
                    g_scratch[victim] = g_scratch.back();
                    g_scratch.pop_back();
                }
            }
            if (g_scratch.size() < kScratchCacheEntries) g_scratch.push_back({dev, stream, *out, bytes, true, ++g_scratch_tick});
        }
        if (evict) (void)cudaFree(evict);   // owned by another stream, which may be gone: the synchronising free is the safe one
    }
    return NTB200_OK;
}

void scratch_release(void* ptr, cudaStream_t stream) {
    if (!ptr) return;
    {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        for (auto& b : g_scratch)
            if (b.ptr == ptr) {
                b.busy = false;
                return;
            }
    }
    (void)cudaFreeAsync(ptr, stream);
}

namespace {

// Validation shared by every GEMM entry point, then routing.
int run_gemm(GemmArgs g, int route, cudaStream_t stream) {
    if (dtype_size(g.dtype) == 0) return fail(NTB200_ERR_UNSUPPORTED, "matmult: unknown dtype %d", g.dtype);
    if (g.m < 0 || g.n < 0 || g.k < 0 || g.batch < 0) return fail(NTB200_ERR_INVALID_ARG, "matmult: negative extent");
    if (g.m == 0 || g.n == 0 || g.batch == 0) return NTB200_OK;
    const bool tables = g.a_ptrs || g.b_ptrs || g.c_ptrs;
    if (tables && !(g.a_ptrs && g.b_ptrs && g.c_ptrs)) return fail(NTB200_ERR_INVALID_ARG, "matmult: incomplete pointer tables");
    if (!tables && (!g.c || (g.k > 0 && (!g.a || !g.b)))) return fail(NTB200_ERR_INVALID_ARG, "matmult: null operand");
    if (g.k == 0) {
        if (g.accumulate && !g.bias) return NTB200_OK;  // C += 0
        return launch_fill_c(g, stream);
    }
    // Complex64 / Complex128: the reference's componentwise chains, CUDA-core route only.
    if (g.dtype == NTB200_C64 || g.dtype == NTB200_C128 || g.dtype == NTB200_C32) {
        if (route == NTB200_ROUTE_TENSOR) return fail(NTB200_ERR_UNSUPPORTED, "matmult: complex dtypes run on the CUDA-core route only");
        route = NTB200_ROUTE_SIMT;
    }
    // Float32: the exact one-chain CUDA-core kernel for small problems (and always with NTB200_FP32_MODE=ffma);
    // three-TF32-product tensor-core kernel (within 1e-5 relative Frobenius error) once the problem is large
    // enough to pay for the split pass.
    const bool wide_int = g.dtype == NTB200_I32 || g.dtype == NTB200_U32 || g.dtype == NTB200_I16 || g.dtype == NTB200_U16;
    if (wide_int && route == NTB200_ROUTE_AUTO && double(g.m) * double(g.n) * double(g.k) * double(g.batch) < 6.0e7)
        route = NTB200_ROUTE_SIMT;   // ten limb GEMMs and a split pass only pay off on large problems
    if (g.dtype == NTB200_F32 && route == NTB200_ROUTE_AUTO) {
        static const bool ffma_only = [] { const char* e = getenv("NTB200_FP32_MODE"); return e && std::strcmp(e, "ffma") == 0; }();
        if (ffma_only || double(g.m) * double(g.n) * double(g.k) * double(g.batch) < 6.0e7) route = NTB200_ROUTE_SIMT;
    }
    // Callers that may not allocate: the routes that copy their operands first (Float32 hi/lo parts, integer limb
    // planes) need scratch, so these dtypes stay on the CUDA-core kernel; the weight-streaming kernels and K slices
    // (fp32 partial tiles) are skipped below and in launch_umma_gemm.
    if (g.no_alloc && (g.dtype == NTB200_F32 || wide_int)) {
        if (route == NTB200_ROUTE_TENSOR) return fail(NTB200_ERR_UNSUPPORTED, "matmult: the tcgen05 route of %s needs scratch memory", dtype_name(g.dtype));
        route = NTB200_ROUTE_SIMT;
    }
    // one or two rows against a large 16-bit weight matrix are bound by reading the weights once: the tensor-core
    // kernel that slices K over a cluster does that in one launch; shapes it does not take stream the weights on
    // CUDA cores
    if (route == NTB200_ROUTE_AUTO && !g.no_alloc && gemv_supported(g) && !umma_cluster_k_would_run(g)) return launch_gemv(g, stream);
    if (route != NTB200_ROUTE_SIMT) {
        const char* why = nullptr;
        if (umma_supported(g, &why)) {
            const int rc = launch_umma_gemm(g, stream);
            if (rc != NTB200_ERR_UNSUPPORTED || route == NTB200_ROUTE_TENSOR) return rc;
        } else if (route == NTB200_ROUTE_TENSOR) {
            return fail(NTB200_ERR_UNSUPPORTED, "matmult: tcgen05 route refused (%s)", why ? why : "?");
        }
    }
    return launch_simt_gemm(g, stream);
}

// The reference's raw-pointer contract (nt_matmult.h:6-10) as strides.
GemmArgs raw_contract(int dtype, const void* A, const void* B, void* C, int64_t a_rows, int64_t a_cols, int64_t b_cols,
                      bool ta, bool tb, int accumulate) {
    GemmArgs g{};
    g.dtype = dtype;
    g.accumulate = accumulate;
    g.f16_rounding = NTB200_F16_ROUND_ONCE;
    g.m = a_rows; g.k = a_cols; g.n = b_cols; g.batch = 1;
    g.a = A; g.a_rs = ta ? 1 : a_cols; g.a_cs = ta ? a_rows : 1; g.a_bs = a_rows * a_cols;
    g.b = B; g.b_rs = tb ? 1 : b_cols; g.b_cs = tb ? a_cols : 1; g.b_bs = a_cols * b_cols;
    g.c = C; g.c_rs = b_cols; g.c_bs = a_rows * b_cols;
    return g;
}

int check_raw_dims(int64_t a_rows, int64_t a_cols, int64_t b_rows, int64_t b_cols) {
    if (a_rows < 0 || a_cols < 0 || b_rows < 0 || b_cols < 0) return fail(NTB200_ERR_INVALID_ARG, "matmult: negative extent");
    if (a_cols != b_rows)
        return fail(NTB200_ERR_INVALID_ARG, "Expected second tensor rows to be %lld when it was %lld", (long long)a_cols,
                    (long long)b_rows);
    return NTB200_OK;
}

// ---- host-buffer pipeline ------------------------------------------------------------------------
struct Lane {
    cudaStream_t stream = nullptr;
    void* buf[3] = {nullptr, nullptr, nullptr};
    size_t cap[3] = {0, 0, 0};
};
constexpr int kLanes = 3;
struct HostCtx {
    Lane lanes[kLanes];
    void* shared_b = nullptr;  // an operand every chunk reuses
    size_t shared_cap = 0;
};
std::mutex g_host_mu;
HostCtx g_host_ctx[64];

int ensure(void** p, size_t* cap, size_t bytes) {
    if (*cap >= bytes) return NTB200_OK;
    if (*p) NTB200_CUDA(cudaFree(*p));
    *p = nullptr; *cap = 0;
    NTB200_CUDA(cudaMalloc(p, bytes));
    *cap = bytes;
    return NTB200_OK;
}

}  // namespace

int route_gemm(const GemmArgs& g, int route, cudaStream_t stream) { return run_gemm(g, route, stream); }

int conv2d_forward(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch, int64_t channels,
                   int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                   int64_t pw, int64_t dh, int64_t dw, bool no_alloc, cudaStream_t stream) {
    if (dtype_size(dtype) == 0) return fail(NTB200_ERR_UNSUPPORTED, "conv2d: unknown dtype %d", dtype);
    if (sh < 1 || sw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d stride cannot be less than 1");
    if (dh < 1 || dw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d dilation cannot be less than 1");
    if (ph < 0 || pw < 0) return fail(NTB200_ERR_INVALID_ARG, "Conv2d padding cannot be less than 0");
    if (batch < 0 || channels <= 0 || cout <= 0 || height <= 0 || width <= 0 || kh <= 0 || kw <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "conv2d: bad extent");
    const int64_t hc = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int64_t wc = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    if (hc <= 0 || wc <= 0) return fail(NTB200_ERR_INVALID_ARG, "conv2d: calculated output size (%lld, %lld) must be at least one", (long long)hc, (long long)wc);
    if (batch == 0) return NTB200_OK;
    if (!x || !w || !out || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d: null pointer");
    const int64_t L = hc * wc, ck = channels * kh * kw;
    // 16-bit floats with stride 1 and whole 64-channel blocks: gather the GEMM's operand from a channels-last copy of
    // the input instead of writing the column matrix (the workspace holds that copy and the reordered weights).
    const Conv2dShape shape{dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, hc, wc};
    if (conv2d_implicit_supported(shape, ntb200_conv2d_workspace_bytes(dtype, batch, channels, height, width, kh, kw, sh,
                                                                       sw, ph, pw, dh, dw))) {
        const int rc_implicit = launch_conv2d_implicit(shape, x, w, out, workspace, stream);
        if (rc_implicit != NTB200_ERR_UNSUPPORTED) return rc_implicit;
    }
    // The column matrix is written densely ([B][ck][L]); out[b] (cout x L) = w2d (cout x ck) . col[b] (ck x L),
    // which is the reference's matmult(col, w2d, true, true) followed by its row/col swap, with the same
    // ascending-ck order for every output element.
    int rc = ntb200_im2col(dtype, x, workspace, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream);
    if (rc) return rc;
    GemmArgs g{};
    g.dtype = dtype; g.accumulate = 0; g.f16_rounding = NTB200_F16_ROUND_ONCE;
    g.m = cout; g.n = L; g.k = ck; g.batch = batch;
    g.a = w; g.a_rs = ck; g.a_cs = 1; g.a_bs = 0;
    g.b = workspace; g.b_rs = L; g.b_cs = 1; g.b_bs = ck * L;
    g.c = out; g.c_rs = L; g.c_bs = cout * L;
    g.no_alloc = no_alloc ? 1 : 0;
    return run_gemm(g, NTB200_ROUTE_AUTO, stream);
}

}  // namespace ntb200

using namespace ntb200;

extern "C" {

const char* ntb200_version(void) { return "ntb200 0.1 (sm_100a)"; }
const char* ntb200_last_error_string(void) { return t_error; }
uint64_t ntb200_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* ntb200_last_gemm_route(void) { return t_route; }

int ntb200_device_count(int* count) {
    if (!count) return fail(NTB200_ERR_INVALID_ARG, "device_count: null pointer");
    *count = 0;
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) { *count = 0; return cuda_fail(e, "cudaGetDeviceCount"); }
    return NTB200_OK;
}
int ntb200_set_device(int device) { NTB200_CUDA(cudaSetDevice(device)); return NTB200_OK; }
int ntb200_get_device(int* device) {
    if (!device) return fail(NTB200_ERR_INVALID_ARG, "get_device: null pointer");
    NTB200_CUDA(cudaGetDevice(device));
    return NTB200_OK;
}
int ntb200_selftest_wait_timeout(unsigned int limit_ms, void* stream) {
    if (limit_ms == 0 || limit_ms > 1000) return fail(NTB200_ERR_INVALID_ARG, "selftest_wait_timeout: limit must be 1..1000 ms");
    return launch_wait_timeout_selftest(1000000ull * limit_ms, static_cast<cudaStream_t>(stream));
}
int ntb200_check_device_status(void* stream) { return read_device_status(static_cast<cudaStream_t>(stream)); }

int ntb200_malloc_async(void** ptr, size_t bytes, void* stream) {
    if (!ptr) return fail(NTB200_ERR_INVALID_ARG, "malloc_async: null pointer");
    *ptr = nullptr;
    if (bytes == 0) return NTB200_OK;
    keep_pool_memory();
    NTB200_CUDA(cudaMallocAsync(ptr, bytes, static_cast<cudaStream_t>(stream)));
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        g_blocks.push_back({*ptr, bytes});
    }
    const uint64_t now = g_pool_in_use.fetch_add(bytes) + bytes;
    uint64_t hw = g_pool_high.load();
    while (now > hw && !g_pool_high.compare_exchange_weak(hw, now)) {}
    return NTB200_OK;
}
int ntb200_free_async(void* ptr, void* stream) {
    if (!ptr) return NTB200_OK;
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        for (size_t i = 0; i < g_blocks.size(); ++i)
            if (g_blocks[i].ptr == ptr) {
                g_pool_in_use.fetch_sub(g_blocks[i].bytes);
                g_blocks[i] = g_blocks.back();
                g_blocks.pop_back();
                break;
            }
    }
    NTB200_CUDA(cudaFreeAsync(ptr, static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}
int ntb200_pool_stats(uint64_t* bytes_in_use, uint64_t* high_water) {
    if (bytes_in_use) *bytes_in_use = g_pool_in_use.load();
    if (high_water) *high_water = g_pool_high.load();
    return NTB200_OK;
}
int ntb200_scratch_stats(uint64_t* retained_bytes, uint64_t* acquisitions, uint64_t* allocations) {
    if (retained_bytes) {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        uint64_t total = 0;
        for (const auto& b : g_scratch) total += b.bytes;
        *retained_bytes = total;
    }
    if (acquisitions) *acquisitions = g_scratch_acquires.load();
    if (allocations) *allocations = g_scratch_allocs.load();
    return NTB200_OK;
}
int ntb200_scratch_release_all(void) {
    std::vector<void*> idle;
    {
        std::lock_guard<std::mutex> lk(g_scratch_mu);
        for (size_t i = 0; i < g_scratch.size();)
            if (!g_scratch[i].busy) {
                idle.push_back(g_scratch[i].ptr);
                g_scratch[i] = g_scratch.back();
                g_scratch.pop_back();
            } else {
                ++i;
            }
    }
    for (void* p : idle) NTB200_CUDA(cudaFree(p));   // waits for the work that still uses the block
    return NTB200_OK;
}
int ntb200_device_pool_usage(uint64_t* used_now, uint64_t* used_high, uint64_t* reserved_now, int reset_high) {
    int dev = 0;
    NTB200_CUDA(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    NTB200_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    if (reset_high) {
        unsigned long long zero = 0;
        NTB200_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &zero));
    }
    unsigned long long v = 0;
    if (used_now) { NTB200_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &v)); *used_now = v; }
    if (used_high) { NTB200_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemHigh, &v)); *used_high = v; }
    if (reserved_now) { NTB200_CUDA(cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &v)); *reserved_now = v; }
    return NTB200_OK;
}
int ntb200_memset_async(void* ptr, int value, size_t bytes, void* stream) {
    if (bytes == 0) return NTB200_OK;
    NTB200_CUDA(cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}
int ntb200_memcpy_h2d_async(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return NTB200_OK;
    NTB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}
int ntb200_memcpy_d2h_async(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return NTB200_OK;
    NTB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}
int ntb200_memcpy_d2d_async(void* dst, const void* src, size_t bytes, void* stream) {
    if (bytes == 0) return NTB200_OK;
    NTB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}
int ntb200_stream_synchronize(void* stream) {
    NTB200_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return NTB200_OK;
}

static int gemm_from_desc(const ntb200_gemm_desc* d, const ntb200_gemm_epilogue* ep, void* const* peer_c, int n_peers, void* stream,
                          int64_t relu_row_stride = 0, int peers_get_relu = 0) {
    if (!d) return fail(NTB200_ERR_INVALID_ARG, "gemm: null descriptor");
    GemmArgs g{};
    if (n_peers < 0 || n_peers > 7) return fail(NTB200_ERR_INVALID_ARG, "gemm_push: between 0 and 7 peers");
    if (n_peers > 0 && !peer_c) return fail(NTB200_ERR_INVALID_ARG, "gemm_push: null peer table");
    g.n_peers = n_peers;
    for (int t = 0; t < n_peers; ++t) {
        if (!peer_c[t]) return fail(NTB200_ERR_INVALID_ARG, "gemm_push: null peer pointer");
        g.peer_c[t] = peer_c[t];
    }
    g.dtype = d->dtype; g.accumulate = d->accumulate ? 1 : 0; g.f16_rounding = d->f16_rounding;
    g.m = d->m; g.n = d->n; g.k = d->k; g.batch = d->batch;
    g.a = d->a; g.a_rs = d->a_row_stride; g.a_cs = d->a_col_stride; g.a_bs = d->a_batch_stride;
    g.b = d->b; g.b_rs = d->b_row_stride; g.b_cs = d->b_col_stride; g.b_bs = d->b_batch_stride;
    g.c = d->c; g.c_rs = d->c_row_stride; g.c_bs = d->c_batch_stride;
    g.bias = d->bias; g.bias_rs = d->bias_row_stride; g.bias_cs = d->bias_col_stride; g.bias_bs = d->bias_batch_stride;
    if (ep) { g.relu_out = ep->relu_out; g.mask_src = ep->relu_mask_src; }
    g.relu_rs = relu_row_stride; g.relu_bs = 0; g.peers_get_relu = peers_get_relu;
    if ((g.relu_out || g.mask_src) && d->route == NTB200_ROUTE_SIMT)
        return fail(NTB200_ERR_UNSUPPORTED, "gemm: fused ReLU epilogues need the tcgen05 route");
    if (g.c_rs < g.n && g.m > 1) return fail(NTB200_ERR_INVALID_ARG, "gemm: C row stride %lld is smaller than n %lld", (long long)g.c_rs, (long long)g.n);
    int route = d->route;
    // per-K-tile fp16 rounding only exists on the CUDA-core route
    if (g.dtype == NTB200_F16 && g.f16_rounding == NTB200_F16_ROUND_PER_KTILE) {
        if (route == NTB200_ROUTE_TENSOR) return fail(NTB200_ERR_UNSUPPORTED, "gemm: per-K-tile fp16 rounding needs the CUDA-core route");
        route = NTB200_ROUTE_SIMT;
    }
    if (g.relu_out || g.mask_src) route = NTB200_ROUTE_TENSOR;
    if (n_peers > 0) {
        if (route == NTB200_ROUTE_SIMT) return fail(NTB200_ERR_UNSUPPORTED, "gemm_push needs the tcgen05 route");
        route = NTB200_ROUTE_TENSOR;
    }
    return run_gemm(g, route, static_cast<cudaStream_t>(stream));
}

int ntb200_host_alloc(void** ptr, size_t bytes) {
    if (!ptr) return fail(NTB200_ERR_INVALID_ARG, "host_alloc: null pointer");
    *ptr = nullptr;
    if (bytes == 0) return NTB200_OK;
    NTB200_CUDA(cudaHostAlloc(ptr, bytes, cudaHostAllocPortable));
    return NTB200_OK;
}
int ntb200_host_free(void* ptr) {
    if (ptr) NTB200_CUDA(cudaFreeHost(ptr));
    return NTB200_OK;
}
int ntb200_host_register(void* ptr, size_t bytes) {
    if (!ptr || bytes == 0) return fail(NTB200_ERR_INVALID_ARG, "host_register: null pointer or zero size");
    NTB200_CUDA(cudaHostRegister(ptr, bytes, cudaHostRegisterPortable));
    return NTB200_OK;
}
int ntb200_host_unregister(void* ptr) {
    if (ptr) NTB200_CUDA(cudaHostUnregister(ptr));
    return NTB200_OK;
}

int ntb200_gemm(const ntb200_gemm_desc* d, void* stream) { return gemm_from_desc(d, nullptr, nullptr, 0, stream); }

int ntb200_gemm_fused(const ntb200_gemm_desc* d, const ntb200_gemm_epilogue* ep, void* stream) {
    return gemm_from_desc(d, ep, nullptr, 0, stream);
}

int ntb200_gemm_push(const ntb200_gemm_desc* d, void* const* peer_c, int n_peers, void* stream) {
    return gemm_from_desc(d, nullptr, peer_c, n_peers, stream);
}

int ntb200_gemm_push_relu(const ntb200_gemm_desc* d, void* relu_out, int64_t relu_row_stride, void* const* peer_relu,
                          int n_peers, void* stream) {
    if (!d) return fail(NTB200_ERR_INVALID_ARG, "gemm_push_relu: null descriptor");
    if (!relu_out) return fail(NTB200_ERR_INVALID_ARG, "gemm_push_relu: null ReLU output");
    if (d->batch != 1) return fail(NTB200_ERR_INVALID_ARG, "gemm_push_relu takes one 2-D problem");
    if (relu_row_stride < d->n) return fail(NTB200_ERR_INVALID_ARG, "gemm_push_relu: ReLU row stride %lld is smaller than n %lld",
                                            (long long)relu_row_stride, (long long)d->n);
    ntb200_gemm_epilogue ep{relu_out, nullptr};
    return gemm_from_desc(d, &ep, peer_relu, n_peers, stream, relu_row_stride, 1);
}

int ntb200_peer_alloc(void** ptr, size_t bytes) {
    if (!ptr) return fail(NTB200_ERR_INVALID_ARG, "peer_alloc: null pointer");
    *ptr = nullptr;
    if (bytes == 0) return fail(NTB200_ERR_INVALID_ARG, "peer_alloc: zero bytes");
    NTB200_CUDA(cudaMalloc(ptr, bytes));
    NTB200_CUDA(cudaMemset(*ptr, 0, bytes));
    return NTB200_OK;
}
int ntb200_peer_free(void* ptr) {
    if (ptr) NTB200_CUDA(cudaFree(ptr));
    return NTB200_OK;
}
int ntb200_peer_export(const void* ptr, unsigned char handle[64]) {
    if (!ptr || !handle) return fail(NTB200_ERR_INVALID_ARG, "peer_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    NTB200_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
    std::memcpy(handle, &h, 64);
    return NTB200_OK;
}
int ntb200_peer_import(const unsigned char handle[64], void** ptr) {
    if (!ptr || !handle) return fail(NTB200_ERR_INVALID_ARG, "peer_import: null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    NTB200_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return NTB200_OK;
}
int ntb200_peer_release(void* ptr) {
    if (ptr) NTB200_CUDA(cudaIpcCloseMemHandle(ptr));
    return NTB200_OK;
}

int ntb200_matmult(int dtype, const void* A, const void* B, void* C, int64_t a_rows, int64_t a_cols, int64_t b_rows,
                   int64_t b_cols, int transpose_a, int transpose_b, void* stream) {
    if (int rc = check_raw_dims(a_rows, a_cols, b_rows, b_cols)) return rc;
    GemmArgs g = raw_contract(dtype, A, B, C, a_rows, a_cols, b_cols, transpose_a != 0, transpose_b != 0, 1);
    return run_gemm(g, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream));
}

int ntb200_matmult_batch(int dtype, const void* const* A, const void* const* B, void* const* C, int64_t batches,
                         int64_t a_rows, int64_t a_cols, int64_t b_rows, int64_t b_cols, int transpose_a,
                         int transpose_b, void* stream) {
    if (int rc = check_raw_dims(a_rows, a_cols, b_rows, b_cols)) return rc;
    if (batches < 0) return fail(NTB200_ERR_INVALID_ARG, "matmult_batch: negative batch count");
    if (batches == 0) return NTB200_OK;
    if (!A || !B || !C) return fail(NTB200_ERR_INVALID_ARG, "matmult_batch: null pointer table");
    const size_t es = dtype_size(dtype);
    if (!es) return fail(NTB200_ERR_UNSUPPORTED, "matmult_batch: unknown dtype %d", dtype);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GemmArgs g = raw_contract(dtype, A[0], B[0], C[0], a_rows, a_cols, b_cols, transpose_a != 0, transpose_b != 0, 1);
    g.batch = batches;
    // Equally spaced pointers (the common case: one tensor split along its batch axis) -> one strided launch.
    auto spacing = [&](const void* const* p, int64_t* stride) {
        if (batches == 1) { *stride = 0; return true; }
        const ptrdiff_t d = static_cast<const char*>(p[1]) - static_cast<const char*>(p[0]);
        if (d < 0 || d % ptrdiff_t(es)) return false;
        for (int64_t i = 2; i < batches; ++i)
            if (static_cast<const char*>(p[i]) - static_cast<const char*>(p[i - 1]) != d) return false;
        *stride = d / ptrdiff_t(es);
        return true;
    };
    int64_t sa, sb, sc;
    if (spacing(A, &sa) && spacing(B, &sb) && spacing(reinterpret_cast<const void* const*>(C), &sc) &&
        (batches == 1 || sc >= a_rows * b_cols)) {
        g.a_bs = sa; g.b_bs = sb; g.c_bs = sc;
        return run_gemm(g, NTB200_ROUTE_AUTO, s);
    }
    // Irregular pointers: device pointer tables, CUDA-core route.
    void* table = nullptr;
    const size_t tbytes = size_t(batches) * sizeof(void*);
    if (int rc = scratch_acquire(&table, 3 * tbytes, s)) return rc;
    char* t = static_cast<char*>(table);
    cudaError_t e = cudaMemcpyAsync(t, A, tbytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t + tbytes, B, tbytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t + 2 * tbytes, C, tbytes, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) { scratch_release(table, s); return cuda_fail(e, "pointer table upload"); }
    // the host arrays may be reused by the caller as soon as we return, so this branch waits for the upload
    // (it therefore cannot run inside a stream capture; equally spaced pointers above never come here)
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { scratch_release(table, s); return cuda_fail(e, "pointer table upload"); }
    g.a_ptrs = reinterpret_cast<const void* const*>(t);
    g.b_ptrs = reinterpret_cast<const void* const*>(t + tbytes);
    g.c_ptrs = reinterpret_cast<void* const*>(t + 2 * tbytes);
    int rc = run_gemm(g, NTB200_ROUTE_SIMT, s);
    scratch_release(table, s);
    return rc;
}

int ntb200_matmult_host(int dtype, const void* A, const void* B, void* C, int64_t batches, int64_t a_rows,
                        int64_t a_cols, int64_t b_rows, int64_t b_cols, int transpose_a, int transpose_b,
                        int accumulate) {
    if (int rc = check_raw_dims(a_rows, a_cols, b_rows, b_cols)) return rc;
    if (batches < 0) return fail(NTB200_ERR_INVALID_ARG, "matmult_host: negative batch count");
    accumulate = accumulate ? 1 : 0;
    const size_t es = dtype_size(dtype);
    if (!es) return fail(NTB200_ERR_UNSUPPORTED, "matmult_host: unknown dtype %d", dtype);
    if (batches == 0 || a_rows == 0 || b_cols == 0) return NTB200_OK;
    if (!A || !B || !C) return fail(NTB200_ERR_INVALID_ARG, "matmult_host: null pointer");
    int dev = 0;
    NTB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NTB200_ERR_UNSUPPORTED, "matmult_host: device index out of range");
    std::lock_guard<std::mutex> lk(g_host_mu);
    HostCtx& ctx = g_host_ctx[dev];
    for (auto& l : ctx.lanes)
        if (!l.stream) NTB200_CUDA(cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking));

    const size_t a_item = size_t(a_rows) * a_cols * es, b_item = size_t(a_cols) * b_cols * es,
                 c_item = size_t(a_rows) * b_cols * es;
    int rc = NTB200_OK;
    if (batches > 1) {
        // chunks of whole batch items; each lane: upload A,B,C -> multiply -> download C
        const int64_t per = std::max<int64_t>(1, (batches + 31) / 32);   // short pipeline fill and drain
        int lane_i = 0;
        for (int64_t b0 = 0; b0 < batches && rc == NTB200_OK; b0 += per, lane_i = (lane_i + 1) % kLanes) {
            const int64_t nb = std::min(per, batches - b0);
            Lane& l = ctx.lanes[lane_i];
            if ((rc = ensure(&l.buf[0], &l.cap[0], a_item * per))) break;
            if ((rc = ensure(&l.buf[1], &l.cap[1], b_item * per))) break;
            if ((rc = ensure(&l.buf[2], &l.cap[2], c_item * per))) break;
            const char* ha = static_cast<const char*>(A) + b0 * a_item;
            const char* hb = static_cast<const char*>(B) + b0 * b_item;
            char* hc = static_cast<char*>(C) + b0 * c_item;
            NTB200_CUDA(cudaMemcpyAsync(l.buf[0], ha, a_item * nb, cudaMemcpyHostToDevice, l.stream));
            NTB200_CUDA(cudaMemcpyAsync(l.buf[1], hb, b_item * nb, cudaMemcpyHostToDevice, l.stream));
            if (accumulate) NTB200_CUDA(cudaMemcpyAsync(l.buf[2], hc, c_item * nb, cudaMemcpyHostToDevice, l.stream));
            GemmArgs g = raw_contract(dtype, l.buf[0], l.buf[1], l.buf[2], a_rows, a_cols, b_cols, transpose_a != 0,
                                      transpose_b != 0, accumulate);
            g.batch = nb;
            rc = run_gemm(g, NTB200_ROUTE_AUTO, l.stream);
            if (rc) break;
            NTB200_CUDA(cudaMemcpyAsync(hc, l.buf[2], c_item * nb, cudaMemcpyDeviceToHost, l.stream));
        }
    } else {
        // one matrix: B is uploaded once; A and C travel in row slabs when A's rows are contiguous
        if ((rc = ensure(&ctx.shared_b, &ctx.shared_cap, b_item))) return rc;
        cudaStream_t s0 = ctx.lanes[0].stream;
        NTB200_CUDA(cudaMemcpyAsync(ctx.shared_b, B, b_item, cudaMemcpyHostToDevice, s0));
        NTB200_CUDA(cudaStreamSynchronize(s0));
        const bool slab = !transpose_a && a_rows >= 1024;
        const int64_t rows_per = slab ? ((a_rows + 7) / 8 + 127) / 128 * 128 : a_rows;
        int lane_i = 0;
        for (int64_t r0 = 0; r0 < a_rows && rc == NTB200_OK; r0 += rows_per, lane_i = (lane_i + 1) % kLanes) {
            const int64_t nr = std::min(rows_per, a_rows - r0);
            Lane& l = ctx.lanes[lane_i];
            if ((rc = ensure(&l.buf[0], &l.cap[0], size_t(rows_per) * a_cols * es))) break;
            if ((rc = ensure(&l.buf[2], &l.cap[2], size_t(rows_per) * b_cols * es))) break;
            const char* ha = static_cast<const char*>(A) + size_t(r0) * a_cols * es;
            char* hc = static_cast<char*>(C) + size_t(r0) * b_cols * es;
            NTB200_CUDA(cudaMemcpyAsync(l.buf[0], ha, size_t(nr) * a_cols * es, cudaMemcpyHostToDevice, l.stream));
            if (accumulate)
                NTB200_CUDA(cudaMemcpyAsync(l.buf[2], hc, size_t(nr) * b_cols * es, cudaMemcpyHostToDevice, l.stream));
            GemmArgs g = raw_contract(dtype, l.buf[0], ctx.shared_b, l.buf[2], nr, a_cols, b_cols, transpose_a != 0,
                                      transpose_b != 0, accumulate);
            rc = run_gemm(g, NTB200_ROUTE_AUTO, l.stream);
            if (rc) break;
            NTB200_CUDA(cudaMemcpyAsync(hc, l.buf[2], size_t(nr) * b_cols * es, cudaMemcpyDeviceToHost, l.stream));
        }
    }
    for (auto& l : ctx.lanes) {
        cudaError_t e = cudaStreamSynchronize(l.stream);
        if (e != cudaSuccess && rc == NTB200_OK) rc = cuda_fail(e, "matmult_host: stream synchronize");
    }
    return rc;
}

size_t ntb200_conv2d_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                     int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                     int64_t dh, int64_t dw) {
    if (sh < 1 || sw < 1) return 0;
    const int64_t hc = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int64_t wc = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    if (hc <= 0 || wc <= 0 || batch <= 0 || channels <= 0) return 0;
    const int64_t L = hc * wc;
    return size_t(batch) * size_t(channels * kh * kw) * size_t(L) * dtype_size(dtype);
}

int ntb200_conv2d(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch, int64_t channels,
                  int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                  int64_t ph, int64_t pw, int64_t dh, int64_t dw, void* stream) {
    return conv2d_forward(dtype, x, w, out, workspace, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw,
                          false, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
