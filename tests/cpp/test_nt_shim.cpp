// C++ tests of the nt:: host surface, written the way the reference writes its own tests
// (tests/src/test_macros.h:68-93: named cases that must not throw).  Cases mirror tests/src/matmult_test.cpp:10-307,
// tests/src/linear_autograd_test.cpp:128-149, tests/src/conv_autograd_test.cpp:249-374 and
// tests/src/col_im_autograd_test.cpp:77-116, reading the reference's committed golden .npy vectors.
//   usage: test_nt_shim <dir with the golden .npy files>
#include <nt/nt.h>

#include <cstdio>
#include <iostream>
#include <thread>

static int g_failed = 0, g_run = 0;
template <class F>
void run_test(const char* name, F&& f) {
    ++g_run;
    try {
        f();
        std::printf("PASS %s\n", name);
    } catch (const std::exception& e) {
        ++g_failed;
        std::printf("FAIL %s: %s\n", name, e.what());
    }
    // the reference's harness also fails a case that leaks tracked memory (test_macros.h:72-85)
    uint64_t in_use = 0;
    ntb200_pool_stats(&in_use, nullptr);
    if (in_use != 0) {
        ++g_failed;
        std::printf("FAIL %s: %llu bytes still allocated from the pool\n", name, (unsigned long long)in_use);
    }
}
#define REQUIRE(cond) nt::utils::throw_exception((cond), "requirement failed: " #cond " (line ", __LINE__, ")")
template <class F>
bool throws_invalid_argument(F&& f) {
    try { f(); } catch (const std::invalid_argument&) { return true; }
    return false;
}

using nt::DType;
using nt::DeviceType;
using nt::SizeRef;
using nt::Tensor;
using nt::TensorGrad;
namespace fn = nt::functional;

int main(int argc, char** argv) {
    const std::string gold = argc > 1 ? std::string(argv[1]) + "/" : "tests/golden/reference_autograd_data/";

    run_test("matmult shapes, 2-D and batched, all flag combinations", [] {
        Tensor a = nt::randn_seeded({3, 4, 5}, DType::Float32, 1), b = nt::randn_seeded({3, 5, 2}, DType::Float32, 2);
        REQUIRE(fn::matmult(a, b).shape() == SizeRef({3, 4, 2}));
        REQUIRE(fn::matmult(a[0], b[0]).shape() == SizeRef({4, 2}));
        Tensor at = nt::randn_seeded({3, 5, 4}, DType::Float32, 3), bt = nt::randn_seeded({3, 2, 5}, DType::Float32, 4);
        REQUIRE(fn::matmult(at, b, true, false).shape() == SizeRef({3, 4, 2}));
        REQUIRE(fn::matmult(a, bt, false, true).shape() == SizeRef({3, 4, 2}));
        REQUIRE(fn::matmult(at, bt, true, true).shape() == SizeRef({3, 4, 2}));
        REQUIRE(fn::matmult_cT(a, bt).shape() == SizeRef({3, 4, 2}));
        // bigger a / bigger b: the 2-D operand is repeated over the batch
        REQUIRE(fn::matmult(a, b[0]).shape() == SizeRef({3, 4, 2}));
        REQUIRE(fn::matmult(a[0], b).shape() == SizeRef({3, 4, 2}));
    });

    run_test("batched matmult equals per-item matmult", [] {
        Tensor a = nt::randn_seeded({4, 33, 20}, DType::Float32, 5), b = nt::randn_seeded({4, 20, 17}, DType::Float32, 6);
        Tensor o = fn::matmult(a, b);
        for (int64_t i = 0; i < 4; ++i) {
            std::vector<float> whole = o[i].to_vector<float>(), single = fn::matmult(a[i], b[i]).to_vector<float>();
            REQUIRE(whole == single);  // bit for bit
        }
    });

    run_test("matmult tensors: lists of tensors multiply pairwise (no bigger, Ta, Tb, bigger a)", [] {
        // the cases of the reference's tests/src/matmult_test.cpp:108-190, with its own check all(o1 == o[i])
        struct Case { SizeRef a, b; bool ta, tb; };
        const Case cases[] = {{{5, 2, 3, 4}, {5, 2, 4, 3}, false, false}, {{5, 2, 4, 3}, {5, 2, 4, 3}, true, false},
                              {{5, 2, 4, 3}, {5, 2, 4, 3}, false, true},  {{5, 2, 4, 3}, {5, 4, 3}, true, false},
                              {{5, 2, 4, 3}, {5, 4, 3}, false, true}};
        int seed = 40;
        for (const Case& c : cases) {
            Tensor a = nt::randn_seeded(c.a, DType::Float32, ++seed), b = nt::randn_seeded(c.b, DType::Float32, ++seed);
            std::vector<Tensor> al, bl;
            for (int64_t i = 0; i < 5; ++i) { al.push_back(a[i]); bl.push_back(b[i]); }
            std::vector<Tensor> o = fn::matmult(al, bl, c.ta, c.tb);
            REQUIRE(o.size() == 5);
            for (int64_t i = 0; i < 5; ++i) {
                Tensor o1 = fn::matmult(al[size_t(i)], bl[size_t(i)], c.ta, c.tb);
                REQUIRE(o[size_t(i)].shape() == o1.shape());
                REQUIRE(o[size_t(i)].to_vector<float>() == o1.to_vector<float>());
            }
            // the same lists in another order: pointers no longer equally spaced
            std::vector<Tensor> as = {al[3], al[0], al[4], al[1], al[2]}, bs = {bl[3], bl[0], bl[4], bl[1], bl[2]};
            std::vector<Tensor> os = fn::matmult(as, bs, c.ta, c.tb);
            REQUIRE(os[0].to_vector<float>() == o[3].to_vector<float>());
            REQUIRE(os[4].to_vector<float>() == o[2].to_vector<float>());
        }
        Tensor x = nt::randn_seeded({2, 3, 4}, DType::Float32, 60);
        REQUIRE(throws_invalid_argument([&] { fn::matmult(std::vector<Tensor>{x, x}, std::vector<Tensor>{x}); }));
        REQUIRE(throws_invalid_argument([&] { fn::matmult(std::vector<Tensor>{x}, std::vector<Tensor>{x}); }));   // 4 != 3
    });

    run_test("transpose is an O(1) view and matmult reads it in place", [] {
        Tensor a = nt::randn_seeded({2, 128, 192}, DType::Float32, 7).to(DType::Float16);
        Tensor bs = nt::randn_seeded({2, 256, 192}, DType::Float32, 8).to(DType::Float16);
        Tensor bview = bs.transpose(-1, -2);
        REQUIRE(bview.shares_storage_with(bs) && !bview.is_contiguous() && bview.shape() == SizeRef({2, 192, 256}));
        uint64_t before = ntb200_kernel_launch_count();
        Tensor c1 = fn::matmult(a, bview);
        REQUIRE(ntb200_kernel_launch_count() == before + 1);  // one GEMM, no copy kernel
        REQUIRE(std::string(ntb200_last_gemm_route()) == "umma_f16");
        Tensor c2 = fn::matmult(a, bs, false, true);
        REQUIRE(c1.to_vector<uint16_t>() == c2.to_vector<uint16_t>());
        REQUIRE(bview.contiguous().is_contiguous() && !bview.contiguous().shares_storage_with(bs));
    });

    run_test("matmult with an out tensor accumulates and validates it", [] {
        Tensor a = nt::randn_seeded({6, 8}, DType::Float32, 9), b = nt::randn_seeded({8, 4}, DType::Float32, 10);
        Tensor c = fn::matmult(a, b);
        Tensor twice = c.clone();
        Tensor& r = fn::matmult(a, b, twice);
        REQUIRE(&r == &twice);
        std::vector<float> v1 = c.to_vector<float>(), v2 = twice.to_vector<float>();
        for (size_t i = 0; i < v1.size(); ++i) REQUIRE(std::fabs(v2[i] - 2 * v1[i]) <= 1e-5f * std::fabs(v1[i]) + 1e-6f);
        Tensor wrong = fn::zeros({6, 5});
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, b, wrong); }));
        Tensor frozen = fn::zeros({6, 4});
        frozen.set_mutability(false);
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, b, frozen); }));
        Tensor strided = fn::zeros({4, 6}).transpose(0, 1);
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, b, strided); }));
    });

    run_test("errors are std::invalid_argument raised before any launch", [] {
        Tensor a = fn::zeros({4, 5}), b = fn::zeros({4, 5});
        uint64_t before = ntb200_kernel_launch_count();
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, b); }));
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, fn::zeros({5, 3}, DType::Float16)); }));
        REQUIRE(throws_invalid_argument([&] { fn::matmult(a, Tensor::Null()); }));
        REQUIRE(throws_invalid_argument([&] { fn::matmult(fn::zeros({4, 5}, DType::Bool), fn::zeros({5, 4}, DType::Bool)); }));
        REQUIRE(throws_invalid_argument([&] { fn::matmult(fn::zeros({2, 4, 5}), fn::zeros({3, 5, 4})); }));
        REQUIRE(ntb200_kernel_launch_count() == before);
    });

    run_test("int8 matmult wraps modulo 256 and returns int8", [] {
        std::vector<int8_t> ha(16 * 32), hb(32 * 8);
        for (size_t i = 0; i < ha.size(); ++i) ha[i] = int8_t((i * 37 + 11) % 251 - 125);
        for (size_t i = 0; i < hb.size(); ++i) hb[i] = int8_t((i * 53 + 7) % 241 - 120);
        Tensor a = Tensor::from_host(ha.data(), {16, 32}, DType::int8), b = Tensor::from_host(hb.data(), {32, 8}, DType::int8);
        Tensor c = fn::matmult(a, b);
        REQUIRE(c.dtype() == DType::int8);
        std::vector<int8_t> got = c.to_vector<int8_t>();
        for (int i = 0; i < 16; ++i)
            for (int j = 0; j < 8; ++j) {
                int acc = 0;
                for (int k = 0; k < 32; ++k) acc += int(ha[i * 32 + k]) * int(hb[k * 8 + j]);
                REQUIRE(got[i * 8 + j] == int8_t(uint8_t(acc)));
            }
    });

    run_test("host tensors go through the raw-pointer contract", [] {
        Tensor a = nt::randn_seeded({5, 40, 24}, DType::Float32, 11), b = nt::randn_seeded({5, 24, 56}, DType::Float32, 12);
        Tensor dev = fn::matmult(a, b);
        Tensor host = fn::matmult(a.to(DeviceType::CPU), b.to(DeviceType::CPU));
        REQUIRE(host.device() == DeviceType::CPU);
        REQUIRE(host.to_vector<float>() == dev.to_vector<float>());
    });

    run_test("Linear Autograd test (golden)", [&] {
        TensorGrad x(fn::from_numpy(gold + "linear_input.npy"), true);
        Tensor grad = fn::from_numpy(gold + "linear_grad.npy");
        TensorGrad w(fn::from_numpy(gold + "linear_weight.npy"), true), b(fn::from_numpy(gold + "linear_bias.npy"), true);
        TensorGrad o = fn::linear(x, w, b, false, true);
        REQUIRE(o.shape() == SizeRef({3, 4, 3}));
        o.backward(grad);
        REQUIRE(fn::allclose(x.grad(), fn::from_numpy(gold + "linear_xgrad.npy")));
        REQUIRE(fn::allclose(w.grad(), fn::from_numpy(gold + "linear_wgrad.npy")));
        REQUIRE(fn::allclose(b.grad(), fn::from_numpy(gold + "linear_bgrad.npy")));
    });

    for (const char* ext : {"", "_batched"}) {
        const std::string e = ext;
        run_test(("Conv2d Autograd test (golden)" + e).c_str(), [&] {
            TensorGrad x(fn::from_numpy(gold + "conv2d_input" + e + ".npy"), true);
            TensorGrad w(fn::from_numpy(gold + "conv2d_weight" + e + ".npy"), true);
            fn::ConvArgs args;
            args.ph = args.pw = 1;
            TensorGrad o = fn::conv2d(x, w, args);
            REQUIRE(fn::allclose(o.detach(), fn::from_numpy(gold + "conv2d_output" + e + ".npy")));
            o.backward(fn::from_numpy(gold + "conv2d_grad" + e + ".npy"));
            REQUIRE(fn::allclose(x.grad(), fn::from_numpy(gold + "conv2d_xgrad" + e + ".npy")));
            REQUIRE(fn::allclose(w.grad(), fn::from_numpy(gold + "conv2d_wgrad" + e + ".npy")));
        });
    }

    for (const std::string e : {"_grouped", "_grouped_batched"}) {
        run_test(("Conv2d Autograd test, groups = 2 (golden)" + e).c_str(), [&] {
            TensorGrad x(fn::from_numpy(gold + "conv2d_input" + e + ".npy"), true), w(fn::from_numpy(gold + "conv2d_weight" + e + ".npy"), true);
            TensorGrad o = fn::conv2d(x, w, fn::ConvArgs{}, 2);
            REQUIRE(fn::allclose(o.detach(), fn::from_numpy(gold + "conv2d_output" + e + ".npy")));
            o.backward(fn::from_numpy(gold + "conv2d_grad" + e + ".npy"));
            REQUIRE(fn::allclose(x.grad(), fn::from_numpy(gold + "conv2d_xgrad" + e + ".npy")));
            REQUIRE(fn::allclose(w.grad(), fn::from_numpy(gold + "conv2d_wgrad" + e + ".npy")));
        });
    }
    run_test("conv1d and conv_transpose2d (golden)", [&] {
        Tensor o1 = fn::conv1d(fn::from_numpy(gold + "conv1d_input_batched.npy"), fn::from_numpy(gold + "conv1d_weight_batched.npy"), 1, 1);
        REQUIRE(fn::allclose(o1, fn::from_numpy(gold + "conv1d_output_batched.npy")));
        fn::ConvArgs a;
        a.sh = a.sw = 2; a.ph = a.pw = 1;
        Tensor o2 = fn::conv_transpose2d(fn::from_numpy(gold + "conv_transpose2d_input_batched.npy"),
                                         fn::from_numpy(gold + "conv_transpose2d_weight_batched.npy"), a, 1, 1);
        REQUIRE(fn::allclose(o2, fn::from_numpy(gold + "conv_transpose2d_output_batched.npy")));
        fn::ConvArgs b;
        b.ph = b.pw = 1;
        Tensor o3 = fn::conv_transpose2d(fn::from_numpy(gold + "conv_transpose2d_input_grouped.npy"),
                                         fn::from_numpy(gold + "conv_transpose2d_weight_grouped.npy"), b, 0, 0, 5);
        REQUIRE(fn::allclose(o3, fn::from_numpy(gold + "conv_transpose2d_output_grouped.npy")));
    });

    run_test("layers::Conv2D: convolution plus per-channel bias, and the three gradients", [] {
        fn::ConvArgs a;
        a.ph = a.pw = 1;
        nt::layers::Conv2D conv(6, 8, 3, 3, a, 2, true, DType::Float32, 21);
        REQUIRE(conv.Weight.shape() == SizeRef({8, 3, 3, 3}) && conv.Bias.shape() == SizeRef({8, 1, 1}));
        Tensor xt = nt::randn_seeded({2, 6, 5, 7}, DType::Float32, 22);
        TensorGrad x(xt, true);
        TensorGrad y = conv(x);
        REQUIRE(y.shape() == SizeRef({2, 8, 5, 7}));
        // forward = conv2d without bias + bias per channel
        Tensor plain = fn::conv2d(xt, conv.Weight.detach(), a, 2);
        auto yv = y.detach().to_vector<float>(), pv = plain.to_vector<float>(), bv = conv.Bias.detach().to_vector<float>();
        bool fwd = true;
        for (size_t i = 0; i < yv.size(); ++i) fwd = fwd && (yv[i] == pv[i] + bv[(i / 35) % 8]);
        REQUIRE(fwd);
        Tensor g = nt::randn_seeded({2, 8, 5, 7}, DType::Float32, 23);
        y.backward(g);
        auto gv = g.to_vector<float>(), db = conv.Bias.grad().to_vector<float>();
        REQUIRE(conv.Bias.grad().shape() == SizeRef({8, 1, 1}));
        bool bias_ok = true;
        for (int c = 0; c < 8; ++c) {
            double s = 0;
            for (int b = 0; b < 2; ++b)
                for (int i = 0; i < 35; ++i) s += gv[(b * 8 + c) * 35 + i];
            bias_ok = bias_ok && std::fabs(db[c] - s) <= 1e-4 * (1.0 + std::fabs(s));
        }
        REQUIRE(bias_ok);
        REQUIRE(conv.Weight.grad().shape() == SizeRef({8, 3, 3, 3}) && x.grad().shape() == SizeRef({2, 6, 5, 7}));
    });

    run_test("unfold2d (golden)", [&] {
        Tensor x = fn::from_numpy(gold + "unfold_input.npy");
        fn::ConvArgs args;
        args.ph = args.pw = 1; args.sh = args.sw = 2; args.dh = 1; args.dw = 2;
        Tensor col = fn::unfold2d(x, 3, 2, args);
        REQUIRE(fn::allclose(col, fn::from_numpy(gold + "unfold_output.npy"), 0, 0));
        Tensor dx = fn::unfold2d_backward(fn::from_numpy(gold + "unfold_grad.npy"), 8, 8, 3, 2, args);
        REQUIRE(fn::allclose(dx, fn::from_numpy(gold + "unfold_input_grad.npy")));
    });

    run_test("MLP through layers::Linear, relu and loss::MSE: forward + backward", [] {
        const int64_t B = 64, D = 48, H = 96;
        nt::layers::Linear l1(D, H, true, DType::Float32, 1), l2(H, D, true, DType::Float32, 2);
        REQUIRE(l1.Weight.shape() == SizeRef({D, H}) && !l1.Weight.detach().is_mutable());
        Tensor xt = nt::randn_seeded({B, D}, DType::Float32, 3), target = nt::randn_seeded({B, D}, DType::Float32, 4);
        TensorGrad x(xt, true);
        TensorGrad y = l2(fn::relu(l1(x)));
        nt::ScalarGrad loss = nt::loss::MSE(y, target);
        loss.backward();
        // plain fp64 restatement on the host
        auto X = xt.to_vector<float>(), T = target.to_vector<float>();
        auto W1 = l1.Weight.detach().to_vector<float>(), B1 = l1.Bias.detach().to_vector<float>();
        auto W2 = l2.Weight.detach().to_vector<float>(), B2 = l2.Bias.detach().to_vector<float>();
        std::vector<double> Hh(B * H), A(B * H), Y(B * D), dY(B * D), dA(B * H, 0.0), dW2(H * D, 0.0), dW1(D * H, 0.0), dX(B * D, 0.0);
        double lossv = 0;
        for (int64_t i = 0; i < B; ++i)
            for (int64_t j = 0; j < H; ++j) {
                double s = B1[j];
                for (int64_t k = 0; k < D; ++k) s += double(X[i * D + k]) * W1[k * H + j];
                Hh[i * H + j] = s;
                A[i * H + j] = s > 0 ? s : 0;
            }
        for (int64_t i = 0; i < B; ++i)
            for (int64_t j = 0; j < D; ++j) {
                double s = B2[j];
                for (int64_t k = 0; k < H; ++k) s += A[i * H + k] * W2[k * D + j];
                Y[i * D + j] = s;
                const double d = s - T[i * D + j];
                lossv += d * d;
                dY[i * D + j] = 2 * d / double(B * D);
            }
        lossv /= double(B * D);
        for (int64_t i = 0; i < B; ++i)
            for (int64_t k = 0; k < H; ++k) {
                double s = 0;
                for (int64_t j = 0; j < D; ++j) { s += dY[i * D + j] * W2[k * D + j]; dW2[k * D + j] += A[i * H + k] * dY[i * D + j]; }
                dA[i * H + k] = Hh[i * H + k] < 0 ? 0 : s;
            }
        for (int64_t i = 0; i < B; ++i)
            for (int64_t k = 0; k < D; ++k) {
                double s = 0;
                for (int64_t j = 0; j < H; ++j) { s += dA[i * H + j] * W1[k * H + j]; dW1[k * H + j] += double(X[i * D + k]) * dA[i * H + j]; }
                dX[i * D + k] = s;
            }
        auto close = [](const std::vector<float>& got, const std::vector<double>& exp) {
            double num = 0, den = 0;
            for (size_t i = 0; i < got.size(); ++i) { num += (got[i] - exp[i]) * (got[i] - exp[i]); den += exp[i] * exp[i]; }
            return std::sqrt(num / (den > 0 ? den : 1)) <= 1e-5;
        };
        REQUIRE(std::fabs(loss.item() - lossv) <= 1e-5 * lossv);
        REQUIRE(close(y.detach().to_vector<float>(), Y));
        REQUIRE(close(l2.Weight.grad().to_vector<float>(), dW2));
        REQUIRE(close(l1.Weight.grad().to_vector<float>(), dW1));
        REQUIRE(close(x.grad().to_vector<float>(), dX));
        REQUIRE(l1.Bias.grad().shape() == SizeRef({H}) && l2.Bias.grad().shape() == SizeRef({D}));
    });

    run_test("BFloat16 MLP step runs on tensor cores", [] {
        nt::layers::Linear l1(256, 512, true, DType::BFloat16, 5), l2(512, 256, true, DType::BFloat16, 6);
        TensorGrad x(nt::randn_seeded({256, 256}, DType::BFloat16, 7), false);
        Tensor target = nt::randn_seeded({256, 256}, DType::BFloat16, 8);
        TensorGrad y = l2(fn::relu(l1(x)));
        REQUIRE(std::string(ntb200_last_gemm_route()).rfind("umma_bf16", 0) == 0);   // any of the tensor-core routes
        nt::ScalarGrad loss = nt::loss::MSE(y, target);
        REQUIRE(std::isfinite(loss.item()) && loss.item() > 0);
        loss.backward();
        REQUIRE(l1.Weight.grad().shape() == SizeRef({256, 512}) && l2.Weight.grad().shape() == SizeRef({512, 256}));
        REQUIRE(!x.has_grad());  // the input does not track a gradient
    });

    run_test("optimizers::SGD and optimizers::Adam make a train step: the loss goes down and the updates are the reference's", [] {
        const int64_t B = 32, D = 16, H = 24;
        nt::layers::Linear l1(D, H, true, DType::Float32, 11), l2(H, D, true, DType::Float32, 12);
        Tensor xt = nt::randn_seeded({B, D}, DType::Float32, 13), target = nt::randn_seeded({B, D}, DType::Float32, 14);
        TensorGrad x(xt, false);
        nt::optimizers::SGD sgd({l1.Weight, l1.Bias, l2.Weight, l2.Bias}, 0.05);
        double first = 0, last = 0;
        for (int it = 0; it < 20; ++it) {
            nt::ScalarGrad loss = nt::loss::MSE(l2(fn::relu(l1(x))), target);
            if (it == 0) first = loss.item();
            last = loss.item();
            loss.backward();
            if (it == 0) {   // one SGD update by hand, in float like the reference: w -= clip(g, -10, 10) * lr
                auto w = l2.Weight.detach().to_vector<float>(), g = l2.Weight.grad().to_vector<float>();
                sgd.step();
                auto w_new = l2.Weight.detach().to_vector<float>();
                bool same = true;
                for (size_t i = 0; i < w.size(); ++i) {
                    const float gi = std::fmin(std::fmax(g[i], -10.f), 10.f) * 0.05f;
                    same = same && (w_new[i] == w[i] - gi);
                }
                REQUIRE(same);
                REQUIRE(!l2.Weight.has_grad());   // step() drops the gradients
            } else {
                sgd.step();
            }
        }
        REQUIRE(last < first);
        // Adam, first step from zero moments: m = (1-b1) g, v = (1-b2) g^2, update = lr m / (sqrt(v) + eps)
        nt::optimizers::Adam adam({l1.Weight, l1.Bias, l2.Weight, l2.Bias}, 0.001);
        nt::ScalarGrad loss = nt::loss::MSE(l2(fn::relu(l1(x))), target);
        loss.backward();
        auto w = l1.Weight.detach().to_vector<float>(), g = l1.Weight.grad().to_vector<float>();
        adam.step();
        auto w_new = l1.Weight.detach().to_vector<float>();
        double worst = 0;
        for (size_t i = 0; i < w.size(); ++i) {
            const double m = (1 - 0.9) * g[i], v = (1 - 0.999) * double(g[i]) * g[i];
            const double u = 0.001 * m / (std::sqrt(v) + 1e-8);
            worst = std::fmax(worst, std::fabs((double(w[i]) - u) - w_new[i]));
        }
        REQUIRE(worst <= 1e-6);
    });

    run_test("named-argument forms (nt/nt.h:812-850; conv calls as in tests/src/conv_autograd_test.cpp:140,266)", [&] {
        Tensor a = nt::randn_seeded({4, 6}, DType::Float32, 31), b = nt::randn_seeded({5, 6}, DType::Float32, 32);
        const auto plain = fn::matmult(a, b, false, true).to_vector<float>();
        REQUIRE(nt::matmult(a, b, nt::transpose_b = true).to_vector<float>() == plain);
        REQUIRE(nt::matmult(nt::other = b, nt::input = a, nt::transpose_b = true).to_vector<float>() == plain);
        REQUIRE(nt::matmult(a, b, nullptr, false, true).to_vector<float>() == plain);
        Tensor c = fn::zeros({4, 5});
        Tensor r = nt::matmult(a, b, nt::out = c, nt::transpose_b = true);       // C += op(A).op(B) into the caller's tensor
        REQUIRE(r.shares_storage_with(c) && c.to_vector<float>() == plain);
        Tensor bias = nt::randn_seeded({5}, DType::Float32, 33);
        REQUIRE(nt::linear(a, b, bias, nt::transpose_b = true).to_vector<float>() == fn::linear(a, b, bias, false, true).to_vector<float>());
        REQUIRE(nt::linear(nt::input = a, nt::weight = b, nt::bias = bias, nt::transpose_b = true).shape() == SizeRef({4, 5}));
        // the same forms on TensorGrad, with the reference's conv2d golden case written the way its test writes it
        using namespace nt;   // stride = 1, padding = 1
        TensorGrad x(fn::from_numpy(gold + "conv2d_input.npy"), true), w(fn::from_numpy(gold + "conv2d_weight.npy"), true);
        TensorGrad o = nt::conv2d(x, w, stride = 1, padding = 1);
        REQUIRE(fn::allclose(o.detach(), fn::from_numpy(gold + "conv2d_output.npy")));
        o.backward(fn::from_numpy(gold + "conv2d_grad.npy"));
        REQUIRE(fn::allclose(x.grad(), fn::from_numpy(gold + "conv2d_xgrad.npy")));
        REQUIRE(fn::allclose(w.grad(), fn::from_numpy(gold + "conv2d_wgrad.npy")));
        Tensor o1 = nt::conv1d(fn::from_numpy(gold + "conv1d_input_batched.npy"), fn::from_numpy(gold + "conv1d_weight_batched.npy"),
                               stride = 1, padding = 1);
        REQUIRE(fn::allclose(o1, fn::from_numpy(gold + "conv1d_output_batched.npy")));
        TensorGrad xg(fn::from_numpy(gold + "conv2d_input_grouped.npy"), true), wg(fn::from_numpy(gold + "conv2d_weight_grouped.npy"), true);
        REQUIRE(fn::allclose(nt::conv2d(xg, wg, stride = 1, groups = 2).detach(), fn::from_numpy(gold + "conv2d_output_grouped.npy")));
    });

    run_test("nt::distributed on one rank: shard arithmetic and a column block gathered at an offset", [&] {
        namespace ds = nt::distributed;
        int64_t covered = 0;
        for (int r = 0; r < 8; ++r) {
            auto [s0, n] = ds::shard(16384, 8, r, 8);
            REQUIRE(s0 == covered && n == 2048);
            covered += n;
        }
        REQUIRE(ds::shard(5, 2, 0).second == 3 && ds::shard(5, 2, 1).first == 3);
        REQUIRE(throws_invalid_argument([&] { ds::shard(5, 2, 2); }));
        ds::Communicator comm(0, 1);
        Tensor x = nt::randn_seeded({200, 96}, DType::Float32, 41).to(DType::Float16);
        Tensor w = nt::randn_seeded({96, 136}, DType::Float32, 42).to(DType::Float16);
        Tensor bias = nt::randn_seeded({136}, DType::Float32, 43).to(DType::Float16);
        ds::GatheredMatrix full(comm, 200, 400, DType::Float16);
        Tensor pre;
        Tensor act = ds::linear_allgather(comm, x, w, bias, full, 128, &pre);
        Tensor expect = fn::linear(x, w, bias);
        REQUIRE(pre.to_vector<uint16_t>() == expect.to_vector<uint16_t>());
        REQUIRE(act.columns(128, 136).contiguous().to_vector<uint16_t>() == fn::relu(expect).to_vector<uint16_t>());
        Tensor plain = ds::linear_allgather(comm, x, w, bias, full, 0);
        REQUIRE(plain.columns(0, 136).contiguous().to_vector<uint16_t>() == expect.to_vector<uint16_t>());
        // two row blocks of the same product, the second through another communicator, give the same matrix
        ds::Communicator comm2(0, 1);
        ds::GatheredMatrix blocks(comm, 200, 136, DType::Float16);
        ds::linear_allgather(comm, x.rows(0, 128), w, bias, blocks, 0, nullptr, 0);
        Tensor both = ds::linear_allgather(comm2, x.rows(128, 72), w, bias, blocks, 0, nullptr, 128);
        REQUIRE(both.contiguous().to_vector<uint16_t>() == expect.to_vector<uint16_t>());
        REQUIRE(throws_invalid_argument([&] { ds::linear_allgather(comm, x, w, bias, blocks, 0, nullptr, 8); }));
        comm.barrier();
        nt::cuda::synchronize();
    });

    int n_devices = 0;
    ntb200_device_count(&n_devices);
    if (n_devices >= 2) {
        run_test("nt::distributed, two ranks as two host threads on two GPUs: Linear + ReLU gathered by the GEMM epilogues", [&] {
            namespace ds = nt::distributed;
            ds::ThreadExchange exchange(2);
            std::string errors[2];
            auto worker = [&](int rank) {
                try {
                    nt::utils::check(ntb200_set_device(rank));
                    ds::ThreadExchange::Rank me{&exchange, rank};
                    ds::Communicator comm(rank, 2, ds::ThreadExchange::callback, &me);
                    // same seeds on both ranks: replicated operands agree
                    Tensor x = nt::randn_seeded({4096, 512}, DType::Float32, 51).to(DType::BFloat16);
                    Tensor w = nt::randn_seeded({512, 4096}, DType::Float32, 52).to(DType::BFloat16);
                    Tensor bias = nt::randn_seeded({4096}, DType::Float32, 53).to(DType::BFloat16);
                    Tensor whole = fn::relu(fn::linear(x, w, bias));
                    auto [c0, cn] = comm.shard(4096, 8);
                    ds::GatheredMatrix bufs[2] = {ds::GatheredMatrix(comm, 4096, 4096, DType::BFloat16),
                                                  ds::GatheredMatrix(comm, 4096, 4096, DType::BFloat16)};
                    for (int step = 0; step < 6; ++step) {
                        Tensor pre;
                        Tensor act = ds::linear_allgather(comm, x, w.columns(c0, cn), bias.view({1, 4096}).columns(c0, cn), bufs[step & 1], c0, &pre);
                        nt::cuda::synchronize();
                        if (act.to_vector<uint16_t>() != whole.to_vector<uint16_t>()) throw std::runtime_error("gathered activation differs from the unsharded one");
                    }
                    comm.barrier();
                    nt::cuda::synchronize();
                    nt::utils::check(ntb200_check_device_status(nullptr));
                } catch (const std::exception& e) {
                    errors[rank] = e.what();
                }
            };
            std::thread t0(worker, 0), t1(worker, 1);
            t0.join();
            t1.join();
            nt::utils::check(ntb200_set_device(0));
            REQUIRE(errors[0].empty() && errors[1].empty());
        });
    }

    nt::utils::check(ntb200_check_device_status(nullptr));
    std::printf("%d of %d cases failed\n", g_failed, g_run);
    return g_failed ? 1 : 0;
}
