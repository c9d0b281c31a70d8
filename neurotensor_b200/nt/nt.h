// Umbrella header of the nt:: host surface over libntb200 (see Tensor.h, functional.h, nn.h, distributed.h), and the
// named-argument forms of the reference's user-facing header (nt/nt.h:812-850 for matmult and linear; the conv
// family is called as nt::conv2d(x, w, stride = 1, padding = 1) throughout the reference's tests,
// tests/src/conv_autograd_test.cpp:140,266):
//
//     nt::matmult(a, b)                                    nt::matmult(input = a, other = b, transpose_b = true)
//     nt::matmult(a, b, out = c)                           nt::linear(x, w, bias, transpose_b = true)
//     nt::conv2d(x, w, stride = 1, padding = 1)            nt::conv1d(x, w, stride = 1, groups = 2)
//
// Arguments are positional in the reference's order, then named in any order; every function works on nt::Tensor and
// on nt::TensorGrad alike.  Giving an argument twice, a positional argument after a named one, or a name the function
// does not have is a compile-time error.
#pragma once
#include <tuple>
#include <type_traits>
#include <utility>

#include "Tensor.h"
#include "functional.h"
#include "nn.h"
#include "distributed.h"

namespace nt {
namespace named {

template <class Tag, class T>
struct Arg {
    T value;   // a reference (lvalue or rvalue) to what the caller wrote; lives for the full call expression
};
template <class Tag>
struct Name {
    constexpr Name() = default;
    template <class T>
    constexpr Arg<Tag, T&&> operator=(T&& v) const { return Arg<Tag, T&&>{std::forward<T>(v)}; }
};

template <class T> struct is_named : std::false_type {};
template <class Tag, class T> struct is_named<Arg<Tag, T>> : std::true_type {};
template <class Tag, class T> struct has_tag : std::false_type {};
template <class Tag, class T> struct has_tag<Tag, Arg<Tag, T>> : std::true_type {};
template <class T, class... Tags> struct tag_in : std::false_type {};
template <class Tag, class T, class... Tags> struct tag_in<Arg<Tag, T>, Tags...> : std::disjunction<std::is_same<Tag, Tags>...> {};

template <class... A>
constexpr size_t leading_positional() {
    size_t n = 0;
    bool named_seen = false;
    ((named_seen = named_seen || is_named<std::decay_t<A>>::value, n += named_seen ? 0 : 1), ...);
    return n;
}
template <class... A>
constexpr bool positional_after_named() {
    bool named_seen = false, bad = false;
    ((bad = bad || (named_seen && !is_named<std::decay_t<A>>::value), named_seen = named_seen || is_named<std::decay_t<A>>::value), ...);
    return bad;
}
template <class Tag, class... A>
constexpr size_t count_tag() { return (size_t(0) + ... + (has_tag<Tag, std::decay_t<A>>::value ? 1 : 0)); }
template <class Tag, class... A>
constexpr size_t tag_index() {
    size_t i = 0, found = sizeof...(A);
    ((found = (found == sizeof...(A) && has_tag<Tag, std::decay_t<A>>::value) ? i : found, ++i), ...);
    return found;
}

template <class T>
T& as_lvalue(T&& v) { return v; }

// The value of slot (Tag, position Pos) among `args`: the named argument if given, else the Pos-th positional one, else `def`.
template <class Tag, size_t Pos, class Default, class... A>
decltype(auto) pick(Default&& def, std::tuple<A...>& args) {
    static_assert(count_tag<Tag, A...>() <= 1, "named argument given twice");
    constexpr size_t ti = tag_index<Tag, A...>();
    if constexpr (ti < sizeof...(A)) {
        static_assert(Pos >= leading_positional<A...>(), "argument given both by position and by name");
        return as_lvalue(std::get<ti>(args).value);
    } else if constexpr (Pos < leading_positional<A...>()) {
        return as_lvalue(std::get<Pos>(args));
    } else {
        return std::decay_t<Default>(std::forward<Default>(def));   // by value: the default is a temporary of the caller
    }
}
template <class Tag, size_t Pos, class... A>
constexpr bool given() { return tag_index<Tag, A...>() < sizeof...(A) || Pos < leading_positional<A...>(); }

template <size_t MaxPositional, class... Tags>
struct Signature {
    template <class... A>
    static constexpr void check() {
        static_assert(!positional_after_named<A...>(), "positional arguments come before named ones");
        static_assert(leading_positional<A...>() <= MaxPositional, "too many positional arguments");
        static_assert(((!is_named<std::decay_t<A>>::value || tag_in<std::decay_t<A>, Tags...>::value) && ...),
                      "this function has no argument of that name");
    }
};

// stride / padding / dilation: one number for both directions, or {height, width}
struct Pair2 {
    int64_t h, w;
    Pair2(int64_t v) : h(v), w(v) {}
    Pair2(int v) : h(v), w(v) {}
    Pair2(int64_t a, int64_t b) : h(a), w(b) {}
    Pair2(std::pair<int64_t, int64_t> p) : h(p.first), w(p.second) {}
};

struct input_t {}; struct other_t {}; struct out_t {}; struct transpose_a_t {}; struct transpose_b_t {};
struct weight_t {}; struct bias_t {}; struct image_t {}; struct kernel_t {}; struct stride_t {}; struct padding_t {};
struct dilation_t {}; struct groups_t {}; struct output_padding_t {};
}  // namespace named

inline constexpr named::Name<named::input_t> input{};
inline constexpr named::Name<named::other_t> other{};
inline constexpr named::Name<named::out_t> out{};
inline constexpr named::Name<named::transpose_a_t> transpose_a{};
inline constexpr named::Name<named::transpose_b_t> transpose_b{};
inline constexpr named::Name<named::weight_t> weight{};
inline constexpr named::Name<named::bias_t> bias{};
inline constexpr named::Name<named::image_t> image{};
inline constexpr named::Name<named::kernel_t> kernel{};
inline constexpr named::Name<named::stride_t> stride{};
inline constexpr named::Name<named::padding_t> padding{};
inline constexpr named::Name<named::dilation_t> dilation{};
inline constexpr named::Name<named::groups_t> groups{};
inline constexpr named::Name<named::output_padding_t> output_padding{};

// matmult(input, other, out = nullptr, transpose_a = false, transpose_b = false)      (nt/nt.h:812-841)
template <class... A>
auto matmult(A&&... a) {
    using namespace named;
    Signature<5, input_t, other_t, out_t, transpose_a_t, transpose_b_t>::check<A...>();
    static_assert(given<input_t, 0, A...>() && given<other_t, 1, A...>(), "matmult needs input and other");
    std::tuple<A&&...> args(std::forward<A>(a)...);
    decltype(auto) x = pick<input_t, 0>(nullptr, args);
    decltype(auto) y = pick<other_t, 1>(nullptr, args);
    decltype(auto) o = pick<out_t, 2>(nullptr, args);
    const bool ta = pick<transpose_a_t, 3>(false, args), tb = pick<transpose_b_t, 4>(false, args);
    if constexpr (std::is_same_v<std::decay_t<decltype(o)>, std::nullptr_t>) return functional::matmult(x, y, ta, tb);
    else return std::decay_t<decltype(o)>(functional::matmult(x, y, o, ta, tb));
}

// linear(input, weight, bias, transpose_a = false, transpose_b = false)               (nt/nt.h:844-850)
template <class... A>
auto linear(A&&... a) {
    using namespace named;
    Signature<5, input_t, weight_t, bias_t, transpose_a_t, transpose_b_t>::check<A...>();
    static_assert(given<input_t, 0, A...>() && given<weight_t, 1, A...>() && given<bias_t, 2, A...>(), "linear needs input, weight and bias");
    std::tuple<A&&...> args(std::forward<A>(a)...);
    return functional::linear(pick<input_t, 0>(nullptr, args), pick<weight_t, 1>(nullptr, args), pick<bias_t, 2>(nullptr, args),
                              bool(pick<transpose_a_t, 3>(false, args)), bool(pick<transpose_b_t, 4>(false, args)));
}

// conv2d(image, kernel, stride = 1, padding = 0, dilation = 1, groups = 1)            (nt/functional/tensor_files/conv.h)
template <class... A>
auto conv2d(A&&... a) {
    using namespace named;
    Signature<6, image_t, kernel_t, stride_t, padding_t, dilation_t, groups_t>::check<A...>();
    static_assert(given<image_t, 0, A...>() && given<kernel_t, 1, A...>(), "conv2d needs image and kernel");
    std::tuple<A&&...> args(std::forward<A>(a)...);
    const Pair2 s = pick<stride_t, 2>(Pair2(1), args), p = pick<padding_t, 3>(Pair2(0), args), d = pick<dilation_t, 4>(Pair2(1), args);
    functional::ConvArgs g;
    g.sh = s.h; g.sw = s.w; g.ph = p.h; g.pw = p.w; g.dh = d.h; g.dw = d.w;
    return functional::conv2d(pick<image_t, 0>(nullptr, args), pick<kernel_t, 1>(nullptr, args), g, int64_t(pick<groups_t, 5>(int64_t(1), args)));
}

// conv1d(image, kernel, stride = 1, padding = 0, dilation = 1, groups = 1)
template <class... A>
auto conv1d(A&&... a) {
    using namespace named;
    Signature<6, image_t, kernel_t, stride_t, padding_t, dilation_t, groups_t>::check<A...>();
    static_assert(given<image_t, 0, A...>() && given<kernel_t, 1, A...>(), "conv1d needs image and kernel");
    std::tuple<A&&...> args(std::forward<A>(a)...);
    return functional::conv1d(pick<image_t, 0>(nullptr, args), pick<kernel_t, 1>(nullptr, args), int64_t(pick<stride_t, 2>(int64_t(1), args)),
                              int64_t(pick<padding_t, 3>(int64_t(0), args)), int64_t(pick<dilation_t, 4>(int64_t(1), args)),
                              int64_t(pick<groups_t, 5>(int64_t(1), args)));
}

// conv_transpose2d(image, kernel, stride = 1, padding = 0, output_padding = 0, dilation = 1, groups = 1)
template <class... A>
auto conv_transpose2d(A&&... a) {
    using namespace named;
    Signature<7, image_t, kernel_t, stride_t, padding_t, output_padding_t, dilation_t, groups_t>::check<A...>();
    static_assert(given<image_t, 0, A...>() && given<kernel_t, 1, A...>(), "conv_transpose2d needs image and kernel");
    std::tuple<A&&...> args(std::forward<A>(a)...);
    const Pair2 s = pick<stride_t, 2>(Pair2(1), args), p = pick<padding_t, 3>(Pair2(0), args), op = pick<output_padding_t, 4>(Pair2(0), args),
                d = pick<dilation_t, 5>(Pair2(1), args);
    functional::ConvArgs g;
    g.sh = s.h; g.sw = s.w; g.ph = p.h; g.pw = p.w; g.dh = d.h; g.dw = d.w;
    return functional::conv_transpose2d(pick<image_t, 0>(nullptr, args), pick<kernel_t, 1>(nullptr, args), g, op.h, op.w,
                                        int64_t(pick<groups_t, 6>(int64_t(1), args)));
}

}  // namespace nt
