// nt::functional -- matmult, matmult_cT, linear, conv2d, unfold2d and the handful of helpers the Linear / conv2d
// path uses, with the reference's signatures (nt/functional/tensor_files/matmult.h:10-13, conv.h, colim_transform.h)
// and the reference's checks in the reference's order (matmult.cpp:14-25, matmult_cpu.cpp:51-93,137-143,863-1005).
// Every function is a thin translation of nt::Tensor views into calls on the C ABI of libntb200.so.
#pragma once
#include <cmath>
#include <cstdio>
#include <fstream>

#include "Tensor.h"

namespace nt {
namespace functional {

inline Tensor zeros(SizeRef shape, DType dt = DType::Float32, DeviceType dev = DeviceType::CUDA) {
    return Tensor(std::move(shape), dt, dev);
}
inline Tensor zeros_like(const Tensor& t) { return Tensor(t.shape(), t.dtype(), t.device()); }

namespace detail {

struct Operand {
    Tensor keep;  // owns a contiguous copy when one had to be made
    const void* ptr;
    int64_t rows, cols, rs, cs, batch, bs;
};

// Last two dims as a strided matrix, leading dims folded into one batch stride (copy only if they cannot be).
inline Operand operand_of(const Tensor& t) {
    Operand o{};
    Tensor v = t;
    const int64_t lead = t.dims() - 2;
    bool foldable = true;
    for (int64_t i = 0; i + 1 < lead; ++i) foldable = foldable && t.stride(i) == t.stride(i + 1) * t.shape()[i + 1];
    if (!foldable) v = t.contiguous();
    o.keep = v;
    o.ptr = v.data_ptr();
    o.rows = v.shape()[-2];
    o.cols = v.shape()[-1];
    o.rs = v.stride(-2);
    o.cs = v.stride(-1);
    o.batch = 1;
    for (int64_t i = 0; i < lead; ++i) o.batch *= v.shape()[i];
    o.bs = (lead > 0 && o.batch > 1) ? v.stride(lead - 1) : 0;
    return o;
}

// determine_transposes (matmult_cpu.cpp:51-93): inner dimensions for the four flag combinations.
inline void check_inner(const Tensor& a, const Tensor& b, bool ta, bool tb, int64_t& m, int64_t& k, int64_t& n) {
    m = ta ? a.shape()[-1] : a.shape()[-2];
    k = ta ? a.shape()[-2] : a.shape()[-1];
    const int64_t k2 = tb ? b.shape()[-1] : b.shape()[-2];
    n = tb ? b.shape()[-2] : b.shape()[-1];
    utils::throw_exception(k == k2, "Expected second tensor rows to be ", k, " when it was ", k2, " (shapes ", a.shape(), " and ",
                           b.shape(), ", transpose_a=", ta, ", transpose_b=", tb, ")");
}

inline void check_operands(const Tensor& a, const Tensor& b) {
    utils::throw_exception(!a.is_null() && !b.is_null(), "matmult got a null tensor");
    utils::throw_exception(a.dtype() != DType::Bool && b.dtype() != DType::Bool, "Expected a number type for matmult but got Bool");
    utils::throw_exception(a.dtype() == b.dtype(), "Expected both tensors to have the same dtype for matmult but got ",
                           dtype_name(a.dtype()), " and ", dtype_name(b.dtype()));
    utils::throw_exception(a.dims() >= 2 && b.dims() >= 2, "Expected tensors of at least 2 dims for matmult but got ", a.dims(),
                           "D and ", b.dims(), "D");
    utils::throw_exception(a.device() == b.device(), "Expected both tensors on the same device");
}

// Leading (batch) shape of the result: equal on the shared suffix; a 2-D operand is repeated over the other's batch
// (the reference repeat_()s it, matmult_cpu.cpp:883).
inline std::vector<int64_t> batch_shape(const Tensor& a, const Tensor& b) {
    std::vector<int64_t> la(a.shape().Vec().begin(), a.shape().Vec().end() - 2);
    std::vector<int64_t> lb(b.shape().Vec().begin(), b.shape().Vec().end() - 2);
    if (la.empty()) return lb;
    if (lb.empty()) return la;
    utils::throw_exception(la == lb, "Expected batch dims to match but got ", a.shape(), " and ", b.shape());
    return la;
}

inline Tensor& run(const Tensor& a, const Tensor& b, Tensor& c, bool ta, bool tb, bool accumulate, const Tensor* bias) {
    int64_t m, k, n;
    check_inner(a, b, ta, tb, m, k, n);
    if (a.device() == DeviceType::CPU) {
        // Host tensors: the reference's own raw-pointer contract, staged through the device by the library.
        utils::throw_exception(bias == nullptr, "linear on host tensors: move the tensors to DeviceType::CUDA");
        Tensor ac = a.contiguous(), bc = b.contiguous();
        const int64_t batches = ac.dims() > 2 ? ac.numel() / (ac.shape()[-1] * ac.shape()[-2]) : 1;
        const int64_t bbatches = bc.dims() > 2 ? bc.numel() / (bc.shape()[-1] * bc.shape()[-2]) : 1;
        utils::throw_exception(batches == bbatches, "host matmult needs equal batch counts; move the tensors to DeviceType::CUDA");
        utils::check(ntb200_matmult_host(dtype_code(a.dtype()), ac.data_ptr(), bc.data_ptr(), c.data_ptr(), batches, m, k, k, n, ta, tb,
                                         accumulate));
        return c;
    }
    Operand oa = operand_of(a), ob = operand_of(b);
    ntb200_gemm_desc d{};
    d.dtype = dtype_code(a.dtype());
    d.route = NTB200_ROUTE_AUTO;
    d.accumulate = accumulate ? 1 : 0;
    d.f16_rounding = NTB200_F16_ROUND_ONCE;
    d.m = m; d.n = n; d.k = k;
    d.batch = std::max(oa.batch, ob.batch);
    d.a = oa.ptr; d.a_row_stride = ta ? oa.cs : oa.rs; d.a_col_stride = ta ? oa.rs : oa.cs;
    d.a_batch_stride = oa.batch > 1 ? oa.bs : 0;
    d.b = ob.ptr; d.b_row_stride = tb ? ob.cs : ob.rs; d.b_col_stride = tb ? ob.rs : ob.cs;
    d.b_batch_stride = ob.batch > 1 ? ob.bs : 0;
    d.c = c.data_ptr(); d.c_row_stride = n; d.c_batch_stride = m * n;
    Tensor bias_keep;
    if (bias && !bias->is_null()) {
        utils::throw_exception(bias->dtype() == a.dtype(), "Expected bias to have dtype ", dtype_name(a.dtype()));
        bias_keep = bias->contiguous();
        d.bias = bias_keep.data_ptr();
        if (bias_keep.numel() == n) {            // [N] or [1,N]: broadcast over rows and batch
            d.bias_row_stride = 0; d.bias_col_stride = 1; d.bias_batch_stride = 0;
        } else if (bias_keep.numel() == m * n) { // [M,N]: broadcast over the batch
            d.bias_row_stride = n; d.bias_col_stride = 1; d.bias_batch_stride = 0;
        } else if (bias_keep.numel() == d.batch * m * n) {
            d.bias_row_stride = n; d.bias_col_stride = 1; d.bias_batch_stride = m * n;
        } else {
            utils::throw_error("bias of shape ", bias->shape(), " cannot be broadcast to the output ", c.shape());
        }
    }
    utils::check(ntb200_gemm(&d, nullptr));
    return c;
}

inline SizeRef result_shape(const Tensor& a, const Tensor& b, bool ta, bool tb) {
    int64_t m, k, n;
    check_inner(a, b, ta, tb, m, k, n);
    std::vector<int64_t> s = batch_shape(a, b);
    s.push_back(m);
    s.push_back(n);
    return SizeRef(s);
}

}  // namespace detail

// C = op(A).op(B) into a new tensor (matmult.cpp:14-18).
inline Tensor matmult(const Tensor& a, const Tensor& b, bool trans_a = false, bool trans_b = false) {
    detail::check_operands(a, b);
    Tensor c(detail::result_shape(a, b, trans_a, trans_b), a.dtype(), a.device());
    detail::run(a, b, c, trans_a, trans_b, /*accumulate=*/false, nullptr);
    return c;
}

// c += op(A).op(B) into the caller's tensor, which must be mutable, contiguous, of the right dtype and shape
// (matmult.cpp:20-25, matmult_cpu.cpp:137-143).
inline Tensor& matmult(const Tensor& a, const Tensor& b, Tensor& c, bool trans_a = false, bool trans_b = false) {
    detail::check_operands(a, b);
    utils::throw_exception(!c.is_null(), "matmult got a null output tensor");
    utils::throw_exception(c.is_mutable(), "Output tensor in matmult must be mutable");
    utils::throw_exception(c.is_contiguous(), "Expected the output tensor of matmult to be contiguous");
    utils::throw_exception(c.dtype() == a.dtype(), "Expected the output tensor of matmult to have dtype ", dtype_name(a.dtype()));
    const SizeRef want = detail::result_shape(a, b, trans_a, trans_b);
    utils::throw_exception(c.shape() == want, "Expected the output tensor of matmult to have shape ", want, " but got ", c.shape());
    return detail::run(a, b, c, trans_a, trans_b, /*accumulate=*/true, nullptr);
}

// Tensor-of-tensors operands (DType::TensorObj in the reference, matmult_cpu.cpp:1240-1558): two lists of equal
// length, one shape and dtype per list; result[i] = matmult(a[i], b[i]).  Every (item, batch) pair is one entry of
// the pointer tables of a single ntb200_matmult_batch call (equally spaced pointers run as one strided launch).
// Device tensors only.  Checks follow subT_check (matmult_cpu.cpp:1486-1513).
inline std::vector<Tensor> matmult(const std::vector<Tensor>& a, const std::vector<Tensor>& b, bool trans_a = false,
                                   bool trans_b = false) {
    utils::throw_exception(a.size() == b.size(), "Expected both tensors to have the same number of sub-tensors, going to have these "
                           "multiplied in a list-like fashion, but got ", a.size(), " and ", b.size(), " tensors");
    std::vector<Tensor> out;
    if (a.empty()) return out;
    for (size_t i = 1; i < a.size(); ++i) {
        utils::throw_exception(a[i].shape() == a[0].shape(), "Expected all tensors in list of tensors to have the same shape, but a has a "
                               "tensor of shape ", a[0].shape(), " and ", a[i].shape());
        utils::throw_exception(b[i].shape() == b[0].shape(), "Expected all tensors in list of tensors to have the same shape, but b has a "
                               "tensor of shape ", b[0].shape(), " and ", b[i].shape());
        utils::throw_exception(a[i].dtype() == a[0].dtype() && b[i].dtype() == a[0].dtype(),
                               "Expected all tensors in list of tensors to have the same dtype (", dtype_name(a[0].dtype()), ")");
    }
    detail::check_operands(a[0], b[0]);
    utils::throw_exception(a[0].device() != DeviceType::CPU, "matmult on lists of tensors: move the tensors to DeviceType::CUDA");
    int64_t m, k, n;
    detail::check_inner(a[0], b[0], trans_a, trans_b, m, k, n);
    const SizeRef item_shape = detail::result_shape(a[0], b[0], trans_a, trans_b);
    const int64_t ar = a[0].shape()[-2], ac = a[0].shape()[-1], br = b[0].shape()[-2], bc = b[0].shape()[-1];
    const int64_t a_inner = a[0].numel() / (ar * ac), b_inner = b[0].numel() / (br * bc);
    const int64_t inner = std::max(a_inner, b_inner);
    const size_t es = dtype_size(a[0].dtype());
    std::vector<Tensor> keep;   // contiguous copies stay alive until the call returns
    std::vector<const void*> pa, pb;
    std::vector<void*> pc;
    for (size_t i = 0; i < a.size(); ++i) {
        keep.push_back(a[i].contiguous());
        const char* base_a = static_cast<const char*>(keep.back().data_ptr());
        keep.push_back(b[i].contiguous());
        const char* base_b = static_cast<const char*>(keep.back().data_ptr());
        Tensor c(item_shape, a[0].dtype(), a[0].device());   // zero-filled: the raw contract accumulates
        char* base_c = static_cast<char*>(c.data_ptr());
        for (int64_t j = 0; j < inner; ++j) {
            pa.push_back(base_a + (j % a_inner) * ar * ac * es);
            pb.push_back(base_b + (j % b_inner) * br * bc * es);
            pc.push_back(base_c + j * m * n * es);
        }
        out.push_back(c);
    }
    // the raw contract takes the logical extents of op(a) and op(b); the flags say how they are stored
    utils::check(ntb200_matmult_batch(dtype_code(a[0].dtype()), pa.data(), pb.data(), pc.data(), int64_t(pa.size()), m, k, k, n,
                                      trans_a, trans_b, nullptr));
    utils::check(ntb200_stream_synchronize(nullptr));
    return out;
}

inline Tensor matmult_cT(const Tensor& a, const Tensor& b) { return matmult(a, b, false, true); }

// op(x).op(w) + bias; a null bias is a plain matmult (matmult.cpp:27-32).  The bias is the value the accumulation
// starts from, exactly as cpu::linear preloads C with it (matmult_cpu.cpp:1637-1647).
inline Tensor linear(const Tensor& input, const Tensor& weight, const Tensor& bias, bool trans_input = false,
                     bool trans_weight = false) {
    if (bias.is_null()) return matmult(input, weight, trans_input, trans_weight);
    detail::check_operands(input, weight);
    Tensor c(detail::result_shape(input, weight, trans_input, trans_weight), input.dtype(), input.device());
    detail::run(input, weight, c, trans_input, trans_weight, false, &bias);
    return c;
}

struct ConvArgs {
    int64_t sh = 1, sw = 1, ph = 0, pw = 0, dh = 1, dw = 1;
};

namespace detail {
inline Tensor as_batched_image(const Tensor& x) {
    utils::throw_exception(x.dims() >= 3, "Expected input tensor to have dims greater than or equal to 3 but got ", x.dims(), "D");
    Tensor c = x.contiguous();
    return c.view({-1, x.shape()[-3], x.shape()[-2], x.shape()[-1]});
}
inline void check_conv_args(const ConvArgs& g) {
    utils::throw_exception(g.sh >= 1 && g.sw >= 1, "Conv2d stride cannot be less than 1");
    utils::throw_exception(g.dh >= 1 && g.dw >= 1, "Conv2d dilation cannot be less than 1");
    utils::throw_exception(g.ph >= 0 && g.pw >= 0, "Conv2d padding cannot be less than 0");
}
inline int64_t out_size(int64_t size, int64_t k, int64_t s, int64_t p, int64_t d) { return (size + 2 * p - d * (k - 1) - 1) / s + 1; }
}  // namespace detail

// unfold2d(x, kernel, dilation, padding, stride, transpose_out = true) -> [B, C*kh*kw, L]
// (colim_transform.cpp:565-588).
inline Tensor unfold2d(const Tensor& x, int64_t kh, int64_t kw, const ConvArgs& g = {}) {
    utils::throw_exception(!x.is_null(), "unfold2d got a null tensor");
    detail::check_conv_args(g);
    Tensor im = detail::as_batched_image(x);
    const int64_t B = im.shape()[0], C = im.shape()[1], H = im.shape()[2], W = im.shape()[3];
    const int64_t ho = detail::out_size(H, kh, g.sh, g.ph, g.dh), wo = detail::out_size(W, kw, g.sw, g.pw, g.dw);
    utils::throw_exception(ho > 0 && wo > 0, "calculated shape of the array of sliding blocks as (", ho, ", ", wo,
                           "), but its components must be at least one");
    Tensor col({B, C * kh * kw, ho * wo}, x.dtype(), DeviceType::CUDA);
    utils::check(ntb200_im2col(dtype_code(x.dtype()), im.data_ptr(), col.data_ptr(), B, C, H, W, kh, kw, g.sh, g.sw, g.ph, g.pw, g.dh,
                               g.dw, nullptr));
    return col;
}

// unfold2d_backward (colim_transform.cpp:592-653): column-matrix gradient -> image gradient [B, C, H, W].
inline Tensor unfold2d_backward(const Tensor& dcol, int64_t H, int64_t W, int64_t kh, int64_t kw, const ConvArgs& g = {}) {
    Tensor dc = dcol.contiguous();
    const int64_t B = dc.shape()[0], C = dc.shape()[1] / (kh * kw);
    Tensor im({B, C, H, W}, dcol.dtype(), DeviceType::CUDA);
    utils::check(ntb200_col2im(dtype_code(dcol.dtype()), dc.data_ptr(), im.data_ptr(), B, C, H, W, kh, kw, g.sh, g.sw, g.ph, g.pw, g.dh,
                               g.dw, nullptr));
    return im;
}

// conv2d (conv.cpp:69-119) -> [B, Cout, Ho, Wo]; kernel is [Cout, C/groups, kh, kw].
inline Tensor conv2d(const Tensor& image, const Tensor& kernel, const ConvArgs& g = {}, int64_t groups = 1) {
    utils::throw_exception(!image.is_null() && !kernel.is_null(), "conv2d got a null tensor");
    utils::throw_exception(image.dims() >= 3, "Expected to get a 3D or greater tensor as the input for a 2d convolution, but got ",
                           image.dims(), "D");
    utils::throw_exception(kernel.dims() == 3 || kernel.dims() == 4,
                           "Expected to get a 4D or 3D tensor as the kernel for a 2d convolution, but got ", kernel.dims(), "D");
    utils::throw_exception(image.dtype() == kernel.dtype(), "Expected both kernel and image to have the same dtype for conv2d but got ",
                           dtype_name(kernel.dtype()), " and ", dtype_name(image.dtype()));
    detail::check_conv_args(g);
    utils::throw_exception(groups >= 1, "Expected groups for a convolution to be greater than 0 but got ", groups);
    Tensor im = detail::as_batched_image(image);
    Tensor w = kernel.contiguous();
    if (w.dims() == 3) w = w.view({1, w.shape()[0], w.shape()[1], w.shape()[2]});
    const int64_t B = im.shape()[0], C = im.shape()[1], H = im.shape()[2], W = im.shape()[3];
    const int64_t cout = w.shape()[0], kh = w.shape()[2], kw = w.shape()[3];
    utils::throw_exception(C % groups == 0, "Expected image channels to be divisible by groups in Conv2d but got ", C, " % ", groups,
                           " != 0");
    utils::throw_exception(w.shape()[1] * groups == C, "Expected kernel rows times groups to be equal to rows of image Conv2d but got ",
                           w.shape()[1], " * ", groups, " != ", C);
    const int64_t ho = detail::out_size(H, kh, g.sh, g.ph, g.dh), wo = detail::out_size(W, kw, g.sw, g.pw, g.dw);
    utils::throw_exception(ho > 0 && wo > 0, "conv2d: calculated output size must be at least one");
    const int code = dtype_code(image.dtype());
    const size_t need = ntb200_conv2d_grouped_workspace_bytes(code, B, C, H, W, cout, kh, kw, g.sh, g.sw, g.ph, g.pw, g.dh, g.dw, groups);
    Tensor ws({int64_t(need)}, DType::uint8, DeviceType::CUDA);
    Tensor out({B, cout, ho, wo}, image.dtype(), DeviceType::CUDA);
    utils::check(ntb200_conv2d_grouped(code, im.data_ptr(), w.data_ptr(), out.data_ptr(), ws.data_ptr(), B, C, H, W, cout, kh, kw, g.sh,
                                       g.sw, g.ph, g.pw, g.dh, g.dw, groups, nullptr));
    return out;
}

// conv1d (conv.cpp:13-67): [B, C, W] with a [Cout, C/groups, k] kernel, the one-row case of conv2d.
inline Tensor conv1d(const Tensor& image, const Tensor& kernel, int64_t stride = 1, int64_t padding = 0, int64_t dilation = 1,
                     int64_t groups = 1) {
    utils::throw_exception(image.dims() >= 2, "Expected to get a 2D or greater tensor as the input for a 1d convolution, but got ",
                           image.dims(), "D");
    utils::throw_exception(kernel.dims() == 2 || kernel.dims() == 3,
                           "Expected to get a 3D or 2D tensor as the kernel for a 1d convolution, but got ", kernel.dims(), "D");
    Tensor im = image.contiguous().view({-1, image.shape()[-2], 1, image.shape()[-1]});
    Tensor w = kernel.contiguous();
    w = w.dims() == 2 ? w.view({1, w.shape()[0], 1, w.shape()[1]}) : w.view({w.shape()[0], w.shape()[1], 1, w.shape()[2]});
    ConvArgs a;
    a.sw = stride; a.pw = padding; a.dw = dilation;
    Tensor out = conv2d(im, w, a, groups);
    return out.view({out.shape()[0], out.shape()[1], out.shape()[3]});
}

// conv_transpose2d (conv.cpp:614-672): x [B, Cin, Hi, Wi], kernel [Cin, Cout/groups, kh, kw] -> [B, Cout, Ho, Wo].  It is
// the image gradient of the convolution with the same kernel, evaluated with x in the place of the gradient.
inline Tensor conv_transpose2d(const Tensor& image, const Tensor& kernel, const ConvArgs& g = {}, int64_t out_pad_h = 0,
                               int64_t out_pad_w = 0, int64_t groups = 1) {
    utils::throw_exception(!image.is_null() && !kernel.is_null(), "conv_transpose2d got a null tensor");
    utils::throw_exception(image.dims() >= 3, "Expected to get a 3D or greater tensor as the input for a conv2d transpose, but got ",
                           image.dims(), "D");
    utils::throw_exception(kernel.dims() == 3 || kernel.dims() == 4,
                           "Expected to get a 3D or 4D tensor as the kernel for a conv2d transpose, but got ", kernel.dims(), "D");
    utils::throw_exception(image.dtype() == kernel.dtype(),
                           "Expected both kernel and image to have the same dtype for conv2d transpose but got ", dtype_name(kernel.dtype()),
                           " and ", dtype_name(image.dtype()));
    detail::check_conv_args(g);
    utils::throw_exception(out_pad_h >= 0 && out_pad_w >= 0, "Conv2d Transpose output_padding cannot be less than 0");
    utils::throw_exception(out_pad_h < g.sh && out_pad_w < g.sw, "conv_transpose2d: output_padding must be smaller than the stride");
    utils::throw_exception(groups >= 1, "Expected groups for a convolution to be greater than 0 but got ", groups);
    Tensor im = detail::as_batched_image(image);
    Tensor w = kernel.contiguous();
    if (w.dims() == 3) w = w.view({1, w.shape()[0], w.shape()[1], w.shape()[2]});
    const int64_t B = im.shape()[0], cin = im.shape()[1], hi = im.shape()[2], wi = im.shape()[3];
    utils::throw_exception(cin == w.shape()[0], "Expected image channels to be the same as the kernel batches for conv_transpose2d but got ",
                           im.shape(), " and ", w.shape());
    utils::throw_exception(cin % groups == 0, "Expected image channels to be divisible by groups in Conv2d Transpose but got ", cin, " % ",
                           groups, " != 0");
    const int64_t cout = w.shape()[1] * groups, kh = w.shape()[2], kw = w.shape()[3];
    const int64_t ho = (hi - 1) * g.sh - 2 * g.ph + g.dh * (kh - 1) + 1 + out_pad_h;
    const int64_t wo = (wi - 1) * g.sw - 2 * g.pw + g.dw * (kw - 1) + 1 + out_pad_w;
    utils::throw_exception(ho > 0 && wo > 0, "conv_transpose2d: calculated output size must be at least one");
    const int code = dtype_code(image.dtype());
    const size_t need = ntb200_conv2d_grouped_workspace_bytes(code, B, cout, ho, wo, cin, kh, kw, g.sh, g.sw, g.ph, g.pw, g.dh, g.dw, groups);
    Tensor ws({int64_t(need)}, DType::uint8, DeviceType::CUDA);
    Tensor out({B, cout, ho, wo}, image.dtype(), DeviceType::CUDA);
    utils::check(ntb200_conv2d_grouped_backward_image(code, im.data_ptr(), w.data_ptr(), out.data_ptr(), ws.data_ptr(), B, cout, ho, wo, cin,
                                                      kh, kw, g.sh, g.sw, g.ph, g.pw, g.dh, g.dw, groups, nullptr));
    return out;
}

// relu(x) = clamp(x, 0, none) (nn/functional/activation_functions.cpp:210-212).
inline Tensor relu(const Tensor& x) {
    Tensor xc = x.contiguous();
    Tensor y(x.shape(), x.dtype(), DeviceType::CUDA);
    utils::check(ntb200_relu(dtype_code(x.dtype()), xc.data_ptr(), y.data_ptr(), x.numel(), nullptr));
    return y;
}

// allclose(a, b, rtol = 1e-5, atol = 1e-8) (nt/functional/tensor_files/compare.h:34); compared on the host in fp64.
inline bool allclose(const Tensor& a, const Tensor& b, double rtol = 1e-5, double atol = 1e-8) {
    if (a.shape() != b.shape()) return false;
    Tensor af = a.device() == DeviceType::CUDA ? a.to(DType::Float32) : a;
    Tensor bf = b.device() == DeviceType::CUDA ? b.to(DType::Float32) : b;
    utils::throw_exception(af.dtype() == DType::Float32 && bf.dtype() == DType::Float32, "allclose compares Float32-convertible tensors");
    std::vector<float> va = af.to_vector<float>(), vb = bf.to_vector<float>();
    for (size_t i = 0; i < va.size(); ++i)
        if (!(std::fabs(double(va[i]) - double(vb[i])) <= atol + rtol * std::fabs(double(vb[i])))) return false;
    return true;
}

// Minimal NumPy .npy I/O for Float32 C-order arrays (nt/functional/tensor_files/numpy.h:8-9), enough for the
// reference's golden fixtures.
inline Tensor from_numpy(const std::string& path, DeviceType dev = DeviceType::CUDA) {
    std::ifstream f(path, std::ios::binary);
    utils::throw_exception(bool(f), "from_numpy: cannot open ", path);
    char magic[8];
    f.read(magic, 8);
    utils::throw_exception(f && std::memcmp(magic, "\x93NUMPY", 6) == 0, "from_numpy: ", path, " is not a .npy file");
    uint32_t hlen = 0;
    if (magic[6] == 1) { uint16_t h16; f.read(reinterpret_cast<char*>(&h16), 2); hlen = h16; }
    else f.read(reinterpret_cast<char*>(&hlen), 4);
    std::string header(hlen, ' ');
    f.read(header.data(), hlen);
    utils::throw_exception(header.find("'<f4'") != std::string::npos, "from_numpy: only little-endian float32 is supported");
    utils::throw_exception(header.find("'fortran_order': False") != std::string::npos, "from_numpy: only C order is supported");
    const size_t l = header.find('(', header.find("'shape'")), r = header.find(')', l);
    std::vector<int64_t> shape;
    int64_t cur = -1;
    for (size_t i = l + 1; i <= r; ++i) {
        const char ch = header[i];
        if (ch >= '0' && ch <= '9') cur = (cur < 0 ? 0 : cur * 10) + (ch - '0');
        else if (cur >= 0) { shape.push_back(cur); cur = -1; }
    }
    SizeRef s(shape);
    std::vector<float> data(size_t(s.multiply()));
    f.read(reinterpret_cast<char*>(data.data()), std::streamsize(data.size() * 4));
    utils::throw_exception(bool(f), "from_numpy: ", path, " is truncated");
    return Tensor::from_host(data.data(), s, DType::Float32, dev);
}

inline void to_numpy(const Tensor& t, const std::string& path) {
    utils::throw_exception(t.dtype() == DType::Float32, "to_numpy: only Float32 is supported");
    std::vector<float> v = t.to_vector<float>();
    std::string shape = "(";
    for (int64_t i = 0; i < t.dims(); ++i) shape += std::to_string(t.shape()[i]) + ",";
    shape += ")";
    std::string header = "{'descr': '<f4', 'fortran_order': False, 'shape': " + shape + ", }";
    while ((10 + header.size() + 1) % 64) header += ' ';
    header += '\n';
    std::ofstream f(path, std::ios::binary);
    f.write("\x93NUMPY\x01\x00", 8);
    const uint16_t hl = uint16_t(header.size());
    f.write(reinterpret_cast<const char*>(&hl), 2);
    f.write(header.data(), std::streamsize(header.size()));
    f.write(reinterpret_cast<const char*>(v.data()), std::streamsize(v.size() * 4));
}

}  // namespace functional
}  // namespace nt
