// conv2d with groups > 1, forward and backward (nt/functional/tensor_files/conv.cpp:97-118, 328-337, 453-461).
//
// The reference splits the column matrix into `groups` row blocks (C/groups * kh*kw rows each) and the kernel
// into `groups` blocks of Cout/groups filters, multiplies block by block (as one tensor-of-tensors batch) and
// interleaves the results back into [B, Cout, Ho, Wo].  Here the column matrix of the whole image is written
// once; group g's rows are the contiguous block starting at row g * (C/groups) * kh*kw, and its filters, outputs
// and gradients are contiguous channel ranges, so every group is one batched GEMM on offset pointers with the
// whole tensor's batch strides.  Nothing is copied or re-ordered.  groups == 1 forwards to the ungrouped entry
// points (and their implicit-GEMM routes).
#include <algorithm>

#include "internal.h"

namespace ntb200 {
namespace {

inline size_t round256(size_t v) { return (v + 255u) & ~size_t(255); }

struct Grouped {
    int64_t ho, wo, L, cg, coutg, ckg;   // per group: channels, filters, column rows
};

int check_grouped(const char* who, int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                  int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                  int64_t dw, int64_t groups, Grouped* g) {
    if (dtype_size(dtype) == 0) return fail(NTB200_ERR_UNSUPPORTED, "%s: unknown dtype %d", who, dtype);
    if (groups < 1) return fail(NTB200_ERR_INVALID_ARG, "Expected groups for a convolution to be greater than 0 but got %lld", (long long)groups);
    if (sh < 1 || sw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d stride cannot be less than 1");
    if (dh < 1 || dw < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv2d dilation cannot be less than 1");
    if (ph < 0 || pw < 0) return fail(NTB200_ERR_INVALID_ARG, "Conv2d padding cannot be less than 0");
    if (batch < 0 || channels <= 0 || cout <= 0 || height <= 0 || width <= 0 || kh <= 0 || kw <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    if (channels % groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected image channels to be divisible by groups in Conv2d but got %lld %% %lld != 0",
                    (long long)channels, (long long)groups);
    if (cout % groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected kernel filters to be divisible by groups in Conv2d but got %lld %% %lld != 0",
                    (long long)cout, (long long)groups);
    g->ho = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    g->wo = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    if (g->ho <= 0 || g->wo <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: calculated output size (%lld, %lld) must be at least one", who,
                    (long long)g->ho, (long long)g->wo);
    g->L = g->ho * g->wo;
    g->cg = channels / groups;
    g->coutg = cout / groups;
    g->ckg = g->cg * kh * kw;
    return NTB200_OK;
}

inline const char* at(const void* p, int64_t elements, size_t es) { return static_cast<const char*>(p) + size_t(elements) * es; }
inline char* at(void* p, int64_t elements, size_t es) { return static_cast<char*>(p) + size_t(elements) * es; }

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

size_t ntb200_conv2d_grouped_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                             int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                                             int64_t pw, int64_t dh, int64_t dw, int64_t groups) {
    if (groups < 1 || channels % groups || cout % groups) return 0;
    const size_t fwd = ntb200_conv2d_workspace_bytes(dtype, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw);
    if (fwd == 0) return 0;
    if (groups == 1)
        return std::max(fwd, ntb200_conv2d_backward_workspace_bytes(dtype, batch, channels, height, width, cout, kh, kw, sh,
                                                                    sw, ph, pw, dh, dw));
    // column matrix + the per-image kernel gradients [B, Cout, (C/groups)*kh*kw] + their batch sum (accumulate)
    const size_t per_image = size_t(batch) * size_t(cout) * size_t(channels / groups * kh * kw) * dtype_size(dtype);
    return round256(fwd) + round256(per_image) + size_t(cout) * size_t(channels / groups * kh * kw) * dtype_size(dtype);
}

int ntb200_conv2d_grouped(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch,
                          int64_t channels, int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw,
                          int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, int64_t groups,
                          void* stream) {
    Grouped g;
    if (int rc = check_grouped("conv2d", dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, groups, &g))
        return rc;
    if (groups == 1)
        return ntb200_conv2d(dtype, x, w, out, workspace, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw, dh, dw, stream);
    if (batch == 0) return NTB200_OK;
    if (!x || !w || !out || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d: null pointer");
    const size_t es = dtype_size(dtype);
    if (int rc = ntb200_im2col(dtype, x, workspace, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream)) return rc;
    for (int64_t gi = 0; gi < groups; ++gi) {   // out_g[b] (coutg x L) = w_g (coutg x ckg) . col_g[b] (ckg x L)
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = g.coutg; a.n = g.L; a.k = g.ckg; a.batch = batch;
        a.a = at(w, gi * g.coutg * g.ckg, es); a.a_rs = g.ckg; a.a_cs = 1; a.a_bs = 0;
        a.b = at(static_cast<const void*>(workspace), gi * g.ckg * g.L, es); a.b_rs = g.L; a.b_cs = 1; a.b_bs = groups * g.ckg * g.L;
        a.c = at(out, gi * g.coutg * g.L, es); a.c_rs = g.L; a.c_bs = cout * g.L;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    return NTB200_OK;
}

int ntb200_conv2d_grouped_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                         int64_t batch, int64_t channels, int64_t height, int64_t width, int64_t cout,
                                         int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                         int64_t dh, int64_t dw, int64_t groups, void* stream) {
    Grouped g;
    if (int rc = check_grouped("conv2d_backward_image", dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw,
                               dh, dw, groups, &g))
        return rc;
    if (groups == 1)
        return ntb200_conv2d_backward_image(dtype, grad, w, d_image, workspace, batch, channels, height, width, cout, kh, kw,
                                            sh, sw, ph, pw, dh, dw, stream);
    if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16)
        return fail(NTB200_ERR_UNSUPPORTED, "conv2d_backward_image: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    if (batch == 0) return NTB200_OK;
    if (!grad || !w || !d_image || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d_backward_image: null pointer");
    const size_t es = dtype_size(dtype);
    for (int64_t gi = 0; gi < groups; ++gi) {   // d_col_g[b] (ckg x L) = w_g^T (ckg x coutg) . grad_g[b] (coutg x L)
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = g.ckg; a.n = g.L; a.k = g.coutg; a.batch = batch;
        a.a = at(w, gi * g.coutg * g.ckg, es); a.a_rs = 1; a.a_cs = g.ckg; a.a_bs = 0;
        a.b = at(grad, gi * g.coutg * g.L, es); a.b_rs = g.L; a.b_cs = 1; a.b_bs = cout * g.L;
        a.c = at(workspace, gi * g.ckg * g.L, es); a.c_rs = g.L; a.c_bs = groups * g.ckg * g.L;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    return ntb200_col2im(dtype, workspace, d_image, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream);
}

int ntb200_conv2d_grouped_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace,
                                          int accumulate, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                          int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                                          int64_t pw, int64_t dh, int64_t dw, int64_t groups, void* stream) {
    Grouped g;
    if (int rc = check_grouped("conv2d_backward_kernel", dtype, batch, channels, height, width, cout, kh, kw, sh, sw, ph, pw,
                               dh, dw, groups, &g))
        return rc;
    if (groups == 1)
        return ntb200_conv2d_backward_kernel(dtype, x, grad, d_kernel, workspace, accumulate, batch, channels, height, width,
                                             cout, kh, kw, sh, sw, ph, pw, dh, dw, stream);
    if (dtype != NTB200_F32 && dtype != NTB200_F16 && dtype != NTB200_BF16)
        return fail(NTB200_ERR_UNSUPPORTED, "conv2d_backward_kernel: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    if (batch == 0) return NTB200_OK;
    if (!x || !grad || !d_kernel || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv2d_backward_kernel: null pointer");
    const size_t es = dtype_size(dtype);
    const int64_t ck = groups * g.ckg;
    void* col = workspace;
    void* per_image = at(workspace, 0, es) + round256(size_t(batch) * size_t(ck) * size_t(g.L) * es);
    if (int rc = ntb200_im2col(dtype, x, col, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, stream)) return rc;
    const bool direct = batch == 1;
    for (int64_t gi = 0; gi < groups; ++gi) {   // per_image_g[b] (coutg x ckg) = grad_g[b] (coutg x L) . col_g[b]^T
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = direct ? (accumulate != 0) : 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = g.coutg; a.n = g.ckg; a.k = g.L; a.batch = batch;
        a.a = at(grad, gi * g.coutg * g.L, es); a.a_rs = g.L; a.a_cs = 1; a.a_bs = cout * g.L;
        a.b = at(static_cast<const void*>(col), gi * g.ckg * g.L, es); a.b_rs = 1; a.b_cs = g.L; a.b_bs = ck * g.L;
        a.c = at(direct ? d_kernel : per_image, gi * g.coutg * g.ckg, es); a.c_rs = g.ckg; a.c_bs = cout * g.ckg;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    if (direct) return NTB200_OK;
    if (!accumulate) return ntb200_column_sum(dtype, per_image, d_kernel, batch, cout * g.ckg, stream);
    // the batch sum has its own region behind the per-image gradients (it can be larger than the column matrix)
    void* summed = static_cast<char*>(per_image) + round256(size_t(batch) * size_t(cout) * size_t(g.ckg) * es);
    if (int rc = ntb200_column_sum(dtype, per_image, summed, batch, cout * g.ckg, stream)) return rc;
    return ntb200_add_inplace(dtype, d_kernel, summed, cout * g.ckg, stream);
}

}  // extern "C"
