// nt::TensorGrad, nt::layers::Linear, nt::loss::MSE -- the slice of NeuroTensor's dynamic autograd that
// layers::Linear forward + backward needs, over device tensors.  Mirrors:
//   TensorGrad / graph walk      nt/nn/TensorGrad.h:72-175, nt/nn/AutoGrad.cpp:7-25,75-101,164-180
//   matmult / linear backward    nt/nn/functional/matmult.cpp:37-63,253-273   (flags only, no transposes materialised)
//   relu = clamp(x, 0) backward  nt/nn/functional/min_max.cpp:40-63
//   conv2d backward              nt/functional/tensor_files/conv.cpp:318-346,444-471
//   layers::Linear               nt/nn/layers/Linear.h:10-20, Linear.cpp:10-24  (Weight stored [in, out])
//   loss::MSE, ScalarGrad        nt/nn/Loss.cpp:49-55, nt/nn/ScalarGrad.cpp:28-39
#pragma once
#include <functional>
#include <random>
#include <unordered_set>

#include "functional.h"

namespace nt {

namespace detail {
struct GraphNode {
    Tensor tensor;
    Tensor grad;
    bool requires_grad = true;
    bool grad_is_borrowed = false;  // first gradient is adopted by reference (AutoGrad.cpp:7-25)
    std::vector<std::shared_ptr<GraphNode>> parents;
    std::function<void(const Tensor&, std::vector<std::shared_ptr<GraphNode>>&)> backward_fn;

    void accumulate_gradient(const Tensor& g) {
        if (!requires_grad) return;
        Tensor incoming = g;
        if (incoming.shape() != tensor.shape() && incoming.numel() != tensor.numel()) {
            // broadcast-reduce to this node's shape (bias gradients)
            Tensor reduced(tensor.shape(), tensor.dtype(), DeviceType::CUDA);
            reduced += incoming;
            incoming = reduced;
        } else if (incoming.shape() != tensor.shape()) {
            incoming = incoming.contiguous().view(tensor.shape().Vec());
        }
        if (grad.is_null()) {
            grad = incoming;
            grad_is_borrowed = true;
            return;
        }
        if (grad_is_borrowed) {  // do not write into a tensor someone else may still hold
            grad = grad.clone();
            grad_is_borrowed = false;
        }
        grad += incoming;
    }
};
}  // namespace detail

using GraphParents = std::vector<std::shared_ptr<detail::GraphNode>>;

class TensorGrad {
    std::shared_ptr<detail::GraphNode> node_;

   public:
    TensorGrad() : node_(std::make_shared<detail::GraphNode>()) { node_->requires_grad = false; }
    TensorGrad(Tensor t, bool grad_required = true) : node_(std::make_shared<detail::GraphNode>()) {
        node_->tensor = std::move(t);
        node_->requires_grad = grad_required;
    }
    Tensor& detach() { return node_->tensor; }
    const Tensor& detach() const { return node_->tensor; }
    const SizeRef& shape() const { return node_->tensor.shape(); }
    DType dtype() const { return node_->tensor.dtype(); }
    bool is_null() const { return node_->tensor.is_null(); }
    bool track_grad() const { return node_->requires_grad; }
    const Tensor& grad() const {
        utils::throw_exception(!node_->grad.is_null(), "Gradient has not been computed; call backward first");
        return node_->grad;
    }
    bool has_grad() const { return !node_->grad.is_null(); }
    void zero_grad() { node_->grad = Tensor(); node_->grad_is_borrowed = false; }
    const std::shared_ptr<detail::GraphNode>& node() const { return node_; }

    static TensorGrad make_result(Tensor value, std::vector<std::shared_ptr<detail::GraphNode>> parents,
                                  std::function<void(const Tensor&, std::vector<std::shared_ptr<detail::GraphNode>>&)> fn) {
        bool any = false;
        for (auto& p : parents) any = any || p->requires_grad;
        TensorGrad r(std::move(value), any);
        if (any) {
            r.node_->parents = std::move(parents);
            r.node_->backward_fn = std::move(fn);
        }
        return r;
    }

    // AutoGrad::backward (AutoGrad.cpp:164-180): seed this node, then run every node's backward function once, in
    // reverse topological order of a depth-first walk (AutoGrad.cpp:75-101).
    void backward(const Tensor& grad) {
        utils::throw_exception(grad.shape() == shape() || grad.numel() == node_->tensor.numel(),
                               "Expected the gradient's shape ", grad.shape(), " to match the tensor's ", shape());
        node_->accumulate_gradient(grad);
        std::vector<detail::GraphNode*> order;
        std::unordered_set<detail::GraphNode*> seen;
        std::function<void(detail::GraphNode*)> visit = [&](detail::GraphNode* n) {
            if (!seen.insert(n).second) return;
            for (auto& p : n->parents) visit(p.get());
            order.push_back(n);
        };
        visit(node_.get());
        for (auto it = order.rbegin(); it != order.rend(); ++it) {
            detail::GraphNode* n = *it;
            if (n->backward_fn && !n->grad.is_null()) n->backward_fn(n->grad, n->parents);
        }
    }
};

namespace functional {

// matmult with gradient tracking.  dA = ta ? matmult(B, g, tb, true) : matmult(g, B, false, !tb);
//                                  dB = tb ? matmult(g, A, true, ta) : matmult(A, g, !ta, false)   (matmult.cpp:37-63)
inline TensorGrad matmult(const TensorGrad& a, const TensorGrad& b, bool trans_a = false, bool trans_b = false) {
    Tensor A = a.detach(), B = b.detach();
    // A 2-D right operand is shared by the whole batch: fold the batch into the rows so its gradient needs no
    // separate reduction (same sums as the reference's repeat_ + sum_as).
    const bool fold = !trans_a && A.dims() > 2 && B.dims() == 2;
    const SizeRef a_shape = A.shape();
    if (fold) A = A.contiguous().flatten_leading();
    Tensor out = matmult(A, B, trans_a, trans_b);
    if (fold) {
        std::vector<int64_t> s(a_shape.Vec().begin(), a_shape.Vec().end() - 1);
        s.push_back(out.shape()[-1]);
        out = out.view(s);
    }
    return TensorGrad::make_result(out, {a.node(), b.node()},
        [A, B, trans_a, trans_b, fold, a_shape](const Tensor& g_in, GraphParents& parents) {
            Tensor g = fold ? g_in.contiguous().flatten_leading() : g_in;
            if (parents[0]->requires_grad) {
                Tensor dA = trans_a ? matmult(B, g, trans_b, true) : matmult(g, B, false, !trans_b);
                if (fold) dA = dA.view(a_shape.Vec());
                parents[0]->accumulate_gradient(dA);
            }
            if (parents[1]->requires_grad) {
                Tensor dB = trans_b ? matmult(g, A, true, trans_a) : matmult(A, g, !trans_a, false);
                parents[1]->accumulate_gradient(dB);
            }
        });
}

// linear with gradient tracking; the bias gradient is the incoming gradient reduced to the bias's shape
// (matmult.cpp:253-273).
inline TensorGrad linear(const TensorGrad& input, const TensorGrad& weight, const TensorGrad& bias, bool trans_input = false,
                         bool trans_weight = false) {
    if (bias.is_null()) return matmult(input, weight, trans_input, trans_weight);
    Tensor X = input.detach(), W = weight.detach();
    const bool fold = !trans_input && X.dims() > 2 && W.dims() == 2;
    const SizeRef x_shape = X.shape();
    if (fold) X = X.contiguous().flatten_leading();
    Tensor out = linear(X, W, bias.detach(), trans_input, trans_weight);
    if (fold) {
        std::vector<int64_t> s(x_shape.Vec().begin(), x_shape.Vec().end() - 1);
        s.push_back(out.shape()[-1]);
        out = out.view(s);
    }
    return TensorGrad::make_result(out, {input.node(), weight.node(), bias.node()},
        [X, W, trans_input, trans_weight, fold, x_shape](const Tensor& g_in, GraphParents& parents) {
            Tensor g = fold ? g_in.contiguous().flatten_leading() : g_in;
            if (parents[0]->requires_grad) {
                Tensor dX = trans_input ? matmult(W, g, trans_weight, true) : matmult(g, W, false, !trans_weight);
                if (fold) dX = dX.view(x_shape.Vec());
                parents[0]->accumulate_gradient(dX);
            }
            if (parents[1]->requires_grad) {
                Tensor dW = trans_weight ? matmult(g, X, true, trans_input) : matmult(X, g, !trans_input, false);
                parents[1]->accumulate_gradient(dW);
            }
            if (parents[2]->requires_grad) parents[2]->accumulate_gradient(g);
        });
}

inline TensorGrad relu(const TensorGrad& x) {
    Tensor X = x.detach().contiguous();
    return TensorGrad::make_result(relu(X), {x.node()},
        [X](const Tensor& g, GraphParents& parents) {
            Tensor gc = g.contiguous();
            Tensor gi(X.shape(), X.dtype(), DeviceType::CUDA);
            utils::check(ntb200_relu_backward(dtype_code(X.dtype()), X.data_ptr(), gc.data_ptr(), gi.data_ptr(), X.numel(), nullptr));
            parents[0]->accumulate_gradient(gi);
        });
}

// conv2d with gradient tracking, groups == 1.  d_image = col2im(matmult(w2d, g, true, false)) (conv.cpp:343-345);
// d_kernel = sum over the batch of matmult(g, col, false, true) (conv.cpp:467).  Both gradients are computed by the
// library's conv2d backward entry points on one shared workspace.
inline TensorGrad conv2d(const TensorGrad& image, const TensorGrad& kernel, const ConvArgs& args = {}, int64_t groups = 1) {
    Tensor X = image.detach(), W = kernel.detach();
    Tensor out = conv2d(X, W, args, groups);
    return TensorGrad::make_result(out, {image.node(), kernel.node()},
        [X, W, args, groups](const Tensor& g_in, GraphParents& parents) {
            Tensor im = detail::as_batched_image(X).contiguous();
            Tensor w4 = W.contiguous();
            if (w4.dims() == 3) w4 = w4.view({1, w4.shape()[0], w4.shape()[1], w4.shape()[2]});
            const int64_t B = im.shape()[0], C = im.shape()[1], H = im.shape()[2], Wd = im.shape()[3];
            const int64_t cout = w4.shape()[0], kh = w4.shape()[2], kw = w4.shape()[3];
            Tensor g = g_in.contiguous();
            const int code = dtype_code(X.dtype());
            const size_t need = ntb200_conv2d_grouped_workspace_bytes(code, B, C, H, Wd, cout, kh, kw, args.sh, args.sw, args.ph,
                                                                      args.pw, args.dh, args.dw, groups);
            Tensor ws({int64_t(need)}, DType::uint8, DeviceType::CUDA);
            if (parents[0]->requires_grad) {
                Tensor dx({B, C, H, Wd}, X.dtype(), DeviceType::CUDA);
                utils::check(ntb200_conv2d_grouped_backward_image(code, g.data_ptr(), w4.data_ptr(), dx.data_ptr(), ws.data_ptr(), B, C,
                                                                  H, Wd, cout, kh, kw, args.sh, args.sw, args.ph, args.pw, args.dh,
                                                                  args.dw, groups, nullptr));
                parents[0]->accumulate_gradient(dx.view(X.shape().Vec()));
            }
            if (parents[1]->requires_grad) {
                Tensor dw(w4.shape(), W.dtype(), DeviceType::CUDA);
                utils::check(ntb200_conv2d_grouped_backward_kernel(code, im.data_ptr(), g.data_ptr(), dw.data_ptr(), ws.data_ptr(), 0, B,
                                                                   C, H, Wd, cout, kh, kw, args.sh, args.sw, args.ph, args.pw, args.dh,
                                                                   args.dw, groups, nullptr));
                parents[1]->accumulate_gradient(dw.view(W.shape().Vec()));
            }
        });
}

}  // namespace functional

// Seeded normal initialisation on the host (the reference's randn is a softmax of random integers seeded from
// std::random_device -- nt/functional/tensor_files/rand.cpp:51-55 -- and cannot be reproduced; tests need seeds).
inline Tensor randn_seeded(SizeRef shape, DType dt, uint64_t seed, double stddev = 1.0) {
    std::mt19937_64 gen(seed);
    std::normal_distribution<float> dist(0.f, float(stddev));
    std::vector<float> v(size_t(shape.multiply()));
    for (auto& x : v) x = dist(gen);
    Tensor t = Tensor::from_host(v.data(), std::move(shape), DType::Float32);
    return dt == DType::Float32 ? t : t.to(dt);
}

namespace layers {
// y = x . Weight + Bias with Weight stored [in, out] (not [out, in]); both parameters are immutable tensors that
// track gradients (Linear.cpp:10-24).
class Linear {
   public:
    bool use_bias;
    TensorGrad Weight, Bias;
    Linear(int64_t in_channels, int64_t out_channels, bool use_bias = true, DType dt = DType::Float32, uint64_t seed = 0)
        : use_bias(use_bias),
          Weight(randn_seeded({in_channels, out_channels}, dt, seed * 2 + 1, 1.0 / std::sqrt(double(in_channels)))),
          Bias(use_bias ? TensorGrad(randn_seeded({out_channels}, dt, seed * 2 + 2, 0.01)) : TensorGrad()) {
        Weight.detach().set_mutability(false);
        if (use_bias) Bias.detach().set_mutability(false);
    }
    TensorGrad forward(const TensorGrad& x) { return functional::linear(x, Weight, Bias); }
    TensorGrad operator()(const TensorGrad& x) { return forward(x); }
};
// Conv2D (nn/layers/Conv2D.cpp:11-44): Weight [out, in / groups, kh, kw], Bias [out, 1, 1]; forward is
// conv2d(x, Weight, stride, padding, dilation, groups) + Bias, the bias being a separate elementwise step whose
// gradient is the sum of the output gradient over the batch and the pixels.
class Conv2D {
   public:
    bool use_bias;
    int64_t groups, in_channels, out_channels;
    functional::ConvArgs args;
    TensorGrad Weight, Bias;
    Conv2D(int64_t in_channels, int64_t out_channels, int64_t kh, int64_t kw, functional::ConvArgs args = {}, int64_t groups = 1,
           bool use_bias = true, DType dt = DType::Float32, uint64_t seed = 0)
        : use_bias(use_bias), groups(groups), in_channels(in_channels), out_channels(out_channels), args(args),
          Weight(randn_seeded({out_channels, in_channels / (groups > 0 ? groups : 1), kh, kw}, dt, seed * 2 + 1,
                              1.0 / std::sqrt(double(in_channels / (groups > 0 ? groups : 1) * kh * kw)))),
          Bias(use_bias ? TensorGrad(randn_seeded({out_channels, 1, 1}, dt, seed * 2 + 2, 0.01)) : TensorGrad()) {
        utils::throw_exception(groups >= 1 && out_channels % groups == 0, "Expected in channels to be divisible by groups");
        utils::throw_exception(in_channels % groups == 0, "Expected in channels to be divisible by groups");
        Weight.detach().set_mutability(false);
        if (use_bias) Bias.detach().set_mutability(false);
    }
    TensorGrad forward(const TensorGrad& x) {
        utils::throw_exception(x.shape()[-3] == in_channels, "Expected input tensor to have channel size of ", in_channels, " but got ",
                               x.shape());
        TensorGrad outp = functional::conv2d(x, Weight, args, groups);
        if (!use_bias) return outp;
        Tensor y = outp.detach().clone();
        const int64_t B = y.shape()[0], C = y.shape()[1], inner = y.numel() / (B * C);
        utils::check(ntb200_bias_add_channels(dtype_code(y.dtype()), y.data_ptr(), Bias.detach().data_ptr(), B, C, inner, nullptr));
        return TensorGrad::make_result(y, {outp.node(), Bias.node()}, [B, C, inner](const Tensor& g, GraphParents& parents) {
            if (parents[0]->requires_grad) parents[0]->accumulate_gradient(g);
            if (parents[1]->requires_grad) {
                Tensor gc = g.contiguous();
                Tensor db({C, 1, 1}, g.dtype(), DeviceType::CUDA);
                utils::check(ntb200_sum_channels(dtype_code(g.dtype()), gc.data_ptr(), db.data_ptr(), B, C, inner, nullptr));
                parents[1]->accumulate_gradient(db);
            }
        });
    }
    TensorGrad operator()(const TensorGrad& x) { return forward(x); }
};
}  // namespace layers

namespace optimizers {
// optimizers::SGD and optimizers::Adam (nn/Optimizers.h:12-62, Optimizers.cpp:8-98) over an explicit parameter list
// (the reference collects the list by reflection over a Module).  step() updates every parameter that tracks a
// gradient and has one, with one kernel per parameter, then drops the gradients as erase_grad_tracking does.
class SGD {
    std::vector<TensorGrad> parameters_;
    double learning_rate_;

   public:
    explicit SGD(std::vector<TensorGrad> params, double lr = 0.01) : parameters_(std::move(params)), learning_rate_(lr) {}
    void step() {
        for (auto& p : parameters_) {
            if (p.is_null() || !p.track_grad() || !p.has_grad()) continue;
            Tensor g = p.grad().contiguous();
            utils::check(ntb200_sgd_step(dtype_code(p.dtype()), p.detach().data_ptr(), g.data_ptr(), p.detach().numel(),
                                         learning_rate_, nullptr));
        }
        zero_grad();
    }
    void zero_grad() {
        for (auto& p : parameters_)
            if (!p.is_null()) p.zero_grad();
    }
};

class Adam {
    std::vector<TensorGrad> parameters_;
    double learning_rate_, beta1_, beta2_, epsilon_;
    std::vector<Tensor> m_, v_;
    int64_t t_ = 0;   // never advanced, as in the reference

   public:
    explicit Adam(std::vector<TensorGrad> params, double lr = 0.001, double beta1 = 0.9, double beta2 = 0.999,
                  double epsilon = 1e-8)
        : parameters_(std::move(params)), learning_rate_(lr), beta1_(beta1), beta2_(beta2), epsilon_(epsilon),
          m_(parameters_.size()), v_(parameters_.size()) {}
    void step() {
        for (size_t i = 0; i < parameters_.size(); ++i) {
            TensorGrad& p = parameters_[i];
            if (p.is_null() || !p.track_grad() || !p.has_grad()) continue;
            if (m_[i].is_null()) m_[i] = functional::zeros(p.shape(), p.dtype());
            if (v_[i].is_null()) v_[i] = functional::zeros(p.shape(), p.dtype());
            Tensor g = p.grad().contiguous();
            utils::check(ntb200_adam_step(dtype_code(p.dtype()), p.detach().data_ptr(), g.data_ptr(), m_[i].data_ptr(),
                                          v_[i].data_ptr(), p.detach().numel(), learning_rate_, beta1_, beta2_, epsilon_, t_,
                                          nullptr));
        }
        zero_grad();
    }
    void zero_grad() {
        for (auto& p : parameters_)
            if (!p.is_null()) p.zero_grad();
    }
};
}  // namespace optimizers

// A scalar loss that remembers the gradient to send back (ScalarGrad.h:18-40).
class ScalarGrad {
    double item_;
    TensorGrad parent_;

   public:
    Tensor grad;
    ScalarGrad(double item, Tensor g, TensorGrad parent) : item_(item), parent_(std::move(parent)), grad(std::move(g)) {}
    double item() const { return item_; }
    void backward() { parent_.backward(grad); }
};

namespace loss {
// loss = sum((o - t)^2) / numel, dx = 2 (o - t) / numel (Loss.cpp:49-55).
inline ScalarGrad MSE(const TensorGrad& output, const Tensor& target) {
    const Tensor& o = output.detach();
    utils::throw_exception(o.shape() == target.shape() && o.dtype() == target.dtype(), "MSE: output and target must match");
    Tensor oc = o.contiguous(), tc = target.contiguous();
    Tensor dx(o.shape(), o.dtype(), DeviceType::CUDA);
    Tensor loss_t({1}, DType::Float32, DeviceType::CUDA);
    utils::check(ntb200_mse(dtype_code(o.dtype()), oc.data_ptr(), tc.data_ptr(), dx.data_ptr(), static_cast<float*>(loss_t.data_ptr()),
                            o.numel(), nullptr));
    float v = 0.f;
    loss_t.to_host(&v);
    return ScalarGrad(double(v), dx, output);
}
}  // namespace loss

}  // namespace nt
