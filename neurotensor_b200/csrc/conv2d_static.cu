// conv2d for callers that may not allocate device memory.
//
// ntb200_conv2d needs scratch for the im2col column matrix and leaves its allocation to the caller.  Some
// callers cannot provide it: a host application that has already handed the whole device heap to its own
// allocator (so a further cudaMalloc fails), or one running in a phase where it forbids itself cudaMalloc
// because that call synchronises the device.  For them this file keeps ONE fixed scratch buffer inside the
// library: a file-scope device array that every GPU loading the library holds until the process exits.
// Nothing here, nor anything it calls, uses cudaMalloc, cudaFree, the stream-ordered pool or any other
// allocating routine: the GEMM under the convolution is told so (GemmArgs::no_alloc) and keeps to the routes that
// need no scratch of their own.  Float32, Int16 and Int32 therefore run on the CUDA-core kernel whatever their size
// (their tensor-core routes first write hi/lo or limb copies of the operands), and 16-bit problems never take K
// slices or the weight-streaming kernels (both leave fp32 partial sums in scratch).
//
// The CUDA runtime creates a module's device storage when the module is first used (lazy loading, the default
// since CUDA 12): the 32 MiB behind this array are taken at this entry point's first call on a device, or at
// library load with CUDA_MODULE_LOADING=EAGER.  A caller that hands the whole heap to its own allocator makes
// that first call (any valid tiny problem) beforehand, or sets the variable.
#include <mutex>

#include "internal.h"

namespace {

// The column matrix of one call must fit here: batch * channels*kh*kw * Ho*Wo * sizeof(element) <= 32 MiB.
constexpr size_t kScratchBytes = size_t(NTB200_CONV2D_STATIC_SCRATCH_BYTES);
static __device__ __align__(256) unsigned char g_conv2d_scratch[kScratchBytes];

// In host code `g_conv2d_scratch` is only a stand-in for the device array, not a device address; the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
std::mutex g_mu;
void* g_scratch_ptr[64] = {nullptr};

int scratch_for_current_device(void** out) {
    int dev = 0;
    NTB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ntb200::fail(NTB200_ERR_UNSUPPORTED, "conv2d_static_scratch: device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_conv2d_scratch);
        if (e == cudaErrorMemoryAllocation)
            return ntb200::fail(NTB200_ERR_ALLOC,
                                "conv2d_static_scratch: no device memory left for the library's built-in %zu-byte scratch array; "
                                "make the first call on each device before the application takes the whole heap, or run with "
                                "CUDA_MODULE_LOADING=EAGER", kScratchBytes);
        if (e != cudaSuccess) return ntb200::cuda_fail(e, "cudaGetSymbolAddress(conv2d scratch)");
        if (!p) return ntb200::fail(NTB200_ERR_CUDA, "conv2d_static_scratch: the scratch array has no device address");
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return NTB200_OK;
}

}  // namespace

extern "C" int ntb200_conv2d_static_scratch(int dtype, const void* x, const void* w, void* out, int64_t batch,
                                            int64_t channels, int64_t height, int64_t width, int64_t cout,
                                            int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                            int64_t dh, int64_t dw, void* stream) {
    if (ntb200::dtype_size(dtype) == 0) return ntb200::fail(NTB200_ERR_UNSUPPORTED, "conv2d_static_scratch: unknown dtype %d", dtype);
    if (sh < 1 || sw < 1) return ntb200::fail(NTB200_ERR_INVALID_ARG, "Conv2d stride cannot be less than 1");
    const size_t need = ntb200_conv2d_workspace_bytes(dtype, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw);
    if (need > kScratchBytes)
        return ntb200::fail(NTB200_ERR_INVALID_ARG,
                            "conv2d_static_scratch: the column matrix needs %zu bytes but the built-in scratch holds %zu; "
                            "use ntb200_conv2d with a caller-provided workspace",
                            need, kScratchBytes);
    void* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;
    // im2col writes every element of the column matrix it uses (zeros where a tap falls in the padding), so
    // whatever an earlier call left in the scratch never reaches the result and nothing has to be cleared.
    return ntb200::conv2d_forward(dtype, x, w, out, scratch, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh,
                                  dw, /*no_alloc=*/true, static_cast<cudaStream_t>(stream));
}
