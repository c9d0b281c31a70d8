// conv2d backward, groups == 1: the image gradient (conv_dimage) and the kernel gradient (conv_dkernel) of
// nt/functional/tensor_files/conv.cpp:318-346 and :444-471.
//
// Reference structure:
//   d_image  = col2im( matmult(w2d, grad, true, false) )                  w2d = w viewed [Cout, C*kh*kw]
//   d_kernel += sum over the batch of matmult(grad[b], col[b], false, true)   col = unfold2d(image)
//
// Both are kept as the general route (every dtype, every geometry).  For 16-bit floats with stride 1 the image
// gradient takes a shorter way: it is itself a stride-1 convolution of grad with the kernel flipped in both spatial
// directions and its two channel axes swapped, with padding d*(k-1) - p, so it runs through ntb200_conv2d and, where
// that applies, its implicit GEMM: no [B, C*kh*kw, L] gradient column matrix is written and gathered back.
#include <algorithm>
#include <cstdlib>

#include "internal.h"

namespace ntb200 {
namespace {

inline size_t round256(size_t v) { return (v + 255u) & ~size_t(255); }

// wf[c][co][i][j] = w[co][c][kh-1-i][kw-1-j]
template <typename T>
__global__ void flip_kernel_kernel(const T* __restrict__ w, T* __restrict__ wf, int cout, int channels, int kh, int kw,
                                   long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int j = int(idx % kw);
    long long r = idx / kw;
    const int i = int(r % kh);
    r /= kh;
    const int co = int(r % cout);
    const long long c = r / cout;
    wf[idx] = w[(((long long)co * channels + c) * kh + (kh - 1 - i)) * kw + (kw - 1 - j)];
}

struct Geometry {
    int64_t ho, wo, L, ck;
};

int check_geometry(const char* who, int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                   int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                   int64_t dw, Geometry* g) {
    if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16)
        return fail(NTB200_ERR_UNSUPPORTED, "%s: gradients are computed for Float32, Float16 and BFloat16 (got %s)", who,
                    dtype_name(dtype));
    if (sh < 1 || sw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d stride cannot be less than 1");
    if (dh < 1 || dw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d dilation cannot be less than 1");
    if (ph < 0 || pw < 0) return fail(NTB200_ERR_INVALID_ARG, "Conv2d padding cannot be less than 0");
    if (batch < 0 || channels <= 0 || cout <= 0 || height <= 0 || width <= 0 || kh <= 0 || kw <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    g->ho = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    g->wo = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    if (g->ho <= 0 || g->wo <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: calculated output size (%lld, %lld) must be at least one", who,
                    (long long)g->ho, (long long)g->wo);
    g->L = g->ho * g->wo;
    g->ck = channels * kh * kw;
    return NTB200_OK;
}

// The image gradient as a convolution of grad: possible when stride is 1 and the flipped padding is not negative.
bool image_as_convolution(int dtype, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                          int64_t dw) {
    if (dtype != NTB200_F16 && dtype != NTB200_BF16) return false;   // other dtypes keep the reference's summation order
    return sh == 1 && sw == 1 && dh * (kh - 1) - ph >= 0 && dw * (kw - 1) - pw >= 0;
}

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

size_t ntb200_conv2d_backward_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                              int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                                              int64_t pw, int64_t dh, int64_t dw) {
    const size_t es = dtype_size(dtype);
    if (es == 0 || sh < 1 || sw < 1 || batch <= 0 || channels <= 0 || cout <= 0) return 0;
    const int64_t ho = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int64_t wo = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    if (ho <= 0 || wo <= 0) return 0;
    const size_t col = size_t(batch) * size_t(channels * kh * kw) * size_t(ho * wo) * es;      // both general routes
    const size_t per_image = size_t(batch) * size_t(cout) * size_t(channels * kh * kw) * es;   // kernel gradient
    // ... and a region of its own for the batch sum that `accumulate` adds to d_kernel afterwards
    size_t need = round256(col) + round256(per_image) + size_t(cout) * size_t(channels * kh * kw) * es;
    if (image_as_convolution(dtype, kh, kw, sh, sw, ph, pw, dh, dw)) {
        const size_t conv_ws = ntb200_conv2d_workspace_bytes(dtype, batch, cout, ho, wo, kh, kw, 1, 1, dh * (kh - 1) - ph,
                                                             dw * (kw - 1) - pw, dh, dw);
        need = std::max(need, round256(conv_ws) + size_t(cout) * size_t(channels * kh * kw) * es);
    }
    const Conv2dShape shape{dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, ho, wo};
    need = std::max(need, conv2d_dkernel_implicit_bytes(shape));
    return need;
}

int ntb200_conv2d_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 int64_t batch, int64_t channels, int64_t height, int64_t width, int64_t cout,
                                 int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                                 int64_t dw, void* stream) {
    Geometry g;
    if (int rc = check_geometry("conv2d_backward_image", dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph,
                                pw, dh, dw, &g))
        return rc;
    if (batch == 0) return NTB200_OK;
    if (!grad || !w || !d_image || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d_backward_image: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // NTB200_CONV_EXPLICIT=1 keeps the reference's structure (GEMM, then col2im) for comparisons
    const char* env = getenv("NTB200_CONV_EXPLICIT");
    if (!(env && env[0] == '1') && image_as_convolution(dtype, kh, kw, sh, sw, ph, pw, dh, dw)) {
        const int64_t fph = dh * (kh - 1) - ph, fpw = dw * (kw - 1) - pw;
        const size_t conv_ws = ntb200_conv2d_workspace_bytes(dtype, batch, cout, g.ho, g.wo, kh, kw, 1, 1, fph, fpw, dh, dw);
        void* wf = static_cast<char*>(workspace) + round256(conv_ws);
        const long long total = (long long)cout * g.ck;
        flip_kernel_kernel<uint16_t><<<unsigned((total + 255) / 256), 256, 0, s>>>(
            static_cast<const uint16_t*>(w), static_cast<uint16_t*>(wf), int(cout), int(channels), int(kh), int(kw), total);
        count_launch();
        NTB200_CUDA(cudaGetLastError());
        // grad [B, Cout, Ho, Wo] convolved with wf [C, Cout, kh, kw] gives [B, C, H, W]
        return ntb200_conv2d(dtype, grad, wf, d_image, workspace, batch, cout, g.ho, g.wo, channels, kh, kw, 1, 1, fph, fpw,
                             dh, dw, stream);
    }

    // d_col[b] (CK x L) = w2d^T (CK x Cout) . grad[b] (Cout x L), then the adjoint of im2col
    GemmArgs a{};
    a.dtype = dtype; a.accumulate = 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
    a.m = g.ck; a.n = g.L; a.k = cout; a.batch = batch;
    a.a = w; a.a_rs = 1; a.a_cs = g.ck; a.a_bs = 0;
    a.b = grad; a.b_rs = g.L; a.b_cs = 1; a.b_bs = cout * g.L;
    a.c = workspace; a.c_rs = g.L; a.c_bs = g.ck * g.L;
    if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, s)) return rc;
    return ntb200_col2im(dtype, workspace, d_image, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream);
}

int ntb200_conv2d_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace,
                                  int accumulate, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                  int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                  int64_t dh, int64_t dw, void* stream) {
    Geometry g;
    if (int rc = check_geometry("conv2d_backward_kernel", dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph,
                                pw, dh, dw, &g))
        return rc;
    if (batch == 0) return NTB200_OK;
    if (!x || !grad || !d_kernel || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d_backward_kernel: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype_size(dtype);
    {   // 16-bit floats, stride 1: the implicit GEMM over channels-last copies (no column matrix)
        const Conv2dShape shape{dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, g.ho, g.wo};
        const int rc = launch_conv2d_dkernel_implicit(shape, x, grad, d_kernel, workspace, accumulate, s);
        if (rc != NTB200_ERR_UNSUPPORTED) return rc;
    }
    void* col = workspace;
    void* per_image = static_cast<char*>(workspace) + round256(size_t(batch) * size_t(g.ck) * size_t(g.L) * es);
    if (int rc = ntb200_im2col(dtype, x, col, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream)) return rc;
    // per_image[b] (Cout x CK) = grad[b] (Cout x L) . col[b]^T (L x CK)
    const bool direct = batch == 1;     // one image: the product is the gradient (added to d_kernel when asked)
    GemmArgs a{};
    a.dtype = dtype; a.accumulate = direct ? (accumulate != 0) : 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
    a.m = cout; a.n = g.ck; a.k = g.L; a.batch = batch;
    a.a = grad; a.a_rs = g.L; a.a_cs = 1; a.a_bs = cout * g.L;
    a.b = col; a.b_rs = 1; a.b_cs = g.L; a.b_bs = g.ck * g.L;
    a.c = direct ? d_kernel : per_image; a.c_rs = g.ck; a.c_bs = cout * g.ck;
    if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, s)) return rc;
    if (direct) return NTB200_OK;
    // the reference's .view(batch, -1).sum(0): column sums of [B, Cout*CK]
    if (!accumulate) return ntb200_column_sum(dtype, per_image, d_kernel, batch, cout * g.ck, stream);
    // the batch sum gets a region of its own behind the per-image gradients: it can be larger than the column matrix
    // (a 1 x 1 output with more filters than images), which the summing blocks are still reading next door
    void* summed = static_cast<char*>(per_image) + round256(size_t(batch) * size_t(cout) * size_t(g.ck) * es);
    if (int rc = ntb200_column_sum(dtype, per_image, summed, batch, cout * g.ck, stream)) return rc;
    return ntb200_add_inplace(dtype, d_kernel, summed, cout * g.ck, stream);
}

}  // extern "C"
