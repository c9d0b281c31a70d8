// Internal declarations shared by the translation units of libntb200.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "../../include/ntb200.h"

namespace ntb200 {

// Error text of the calling thread; returns `code` so call sites can `return fail(...)`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
int cuda_fail(cudaError_t err, const char* what);
#define NTB200_CUDA(expr)                                            \
    do {                                                             \
        cudaError_t e__ = (expr);                                    \
        if (e__ != cudaSuccess) return ::ntb200::cuda_fail(e__, #expr); \
    } while (0)

size_t dtype_size(int dtype);
const char* dtype_name(int dtype);
void count_launch(int n = 1);
void note_route(const char* name);
int sm_count();  // multiprocessors of the current device (cached per device)
void keep_pool_memory();  // once per device: the stream-ordered pool retains freed blocks
// Scratch for the library's own kernels, from a block kept per (device, stream) where one fits; `release` hands the
// block back for the next call on that stream (the kernels already queued keep using it in stream order).
int scratch_acquire(void** ptr, size_t bytes, cudaStream_t stream);
void scratch_release(void* ptr, cudaStream_t stream);

// A GEMM after validation: C[b] = (accumulate ? C[b] : 0) + bias + A[b].B[b]; strides in elements.
struct GemmArgs {
    int dtype;
    int accumulate;
    int f16_rounding;
    int64_t m, n, k, batch;
    const void* a; int64_t a_rs, a_cs, a_bs;
    const void* b; int64_t b_rs, b_cs, b_bs;
    void* c; int64_t c_rs, c_bs;
    const void* bias; int64_t bias_rs, bias_cs, bias_bs;
    // optional device pointer tables (batch entries each); when set they replace a/b/c + batch strides
    const void* const* a_ptrs = nullptr;
    const void* const* b_ptrs = nullptr;
    void* const* c_ptrs = nullptr;
    // fused elementwise neighbours (tcgen05 route, 16-bit): tensors with exactly C's layout
    void* relu_out = nullptr;        // also write max(C, 0) here
    int64_t relu_rs = 0, relu_bs = 0;  // strides of relu_out when they differ from C's (0: exactly C's layout; TMA-store epilogue only)
    int peers_get_relu = 0;          // the peer copies receive relu_out's values instead of C's
    const void* mask_src = nullptr;  // zero the result where this tensor is negative
    // peer-mapped copies of C on other GPUs that receive every finished tile as well (tcgen05 route only)
    int n_peers = 0;
    void* peer_c[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // the caller may not allocate: only routes that need no scratch memory (no operand copies, no K slices, no
    // weight-streaming partial sums)
    int no_alloc = 0;
};

// tcgen05 route.  Returns NTB200_ERR_UNSUPPORTED (without touching the error text) when the operands
// cannot be expressed as TMA tensor maps, so the caller can route elsewhere.
bool umma_supported(const GemmArgs& g, const char** why);
int launch_umma_gemm(const GemmArgs& g, cudaStream_t stream);
// Few rows of 16-bit floats against a large weight matrix: would the automatic route slice K over a thread-block
// cluster (one launch, weights read once at close to the HBM rate)?
bool umma_cluster_k_would_run(const GemmArgs& g);
int read_device_status(cudaStream_t stream);
int launch_wait_timeout_selftest(unsigned long long limit_ns, cudaStream_t stream);

// Pieces of the tcgen05 GEMM translation unit that the implicit convolution shares.
unsigned int* device_status_word();   // device address of the status word raised by bounded waits (nullptr on error)
int max_resident_pairs(const void* kernel, uint32_t smem_bytes);   // CTA pairs of `kernel` resident at once
void* tensor_map_encoder();           // cuTensorMapEncodeTiled from the driver, or nullptr

// conv2d geometry after validation (ho, wo = output extent).
struct Conv2dShape {
    int dtype;
    int64_t batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, ho, wo;
};
// Convolution straight from a channels-last copy of the input (16-bit floats, stride 1, channels % 64 == 0).
// `launch` returns NTB200_ERR_UNSUPPORTED before launching anything when the tensor maps cannot be built.
bool conv2d_implicit_supported(const Conv2dShape& s, size_t workspace_bytes);
int launch_conv2d_implicit(const Conv2dShape& s, const void* x, const void* w, void* out, void* workspace,
                           cudaStream_t stream);
// Kernel gradient of the same convolution without a column matrix (16-bit floats, stride 1, channels and output
// channels multiples of 64).  `bytes` is the workspace it needs (0: shape not supported); `launch` returns
// NTB200_ERR_UNSUPPORTED before launching anything when it cannot run.
size_t conv2d_dkernel_implicit_bytes(const Conv2dShape& s);
int launch_conv2d_dkernel_implicit(const Conv2dShape& s, const void* x, const void* grad, void* d_kernel,
                                   void* workspace, int accumulate, cudaStream_t stream);

// One or two rows of 16-bit floats against a large weight matrix: CUDA-core kernels that stream the weights.
bool gemv_supported(const GemmArgs& g);
int launch_gemv(const GemmArgs& g, cudaStream_t stream);

// CUDA-core route: every dtype, every stride pattern.
int launch_simt_gemm(const GemmArgs& g, cudaStream_t stream);

// ntb200_conv2d's body; `no_alloc` keeps its GEMM on routes that need no scratch memory.
int conv2d_forward(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch, int64_t channels,
                   int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                   int64_t pw, int64_t dh, int64_t dw, bool no_alloc, cudaStream_t stream);

// The route decision every GEMM of the library goes through (tcgen05, CUDA cores or a plain fill of C).
int route_gemm(const GemmArgs& g, int route, cudaStream_t stream);

// K == 0 or pure bias/zero fill of C.
int launch_fill_c(const GemmArgs& g, cudaStream_t stream);

}  // namespace ntb200
