// Parameter updates of nt::optimizers::SGD and nt::optimizers::Adam (nt/nn/Optimizers.cpp:8-17 and :68-98) as one
// elementwise kernel each.
//
// The reference builds every update from whole-tensor operations in the parameter's dtype, so each intermediate is
// rounded to that dtype.  The kernels follow the same operation sequence and round after every operation (the
// __f*_rn intrinsics are never contracted into FMAs; 16-bit types are rounded to their format after each step), so
// a Float32 or Float16 update is bit-identical to the reference's arithmetic.  BFloat16 is not a dtype of the
// reference; it gets the same sequence with bf16 roundings.
//
//   SGD::step    g' = clip(g, -10, 10) * lr ;  p -= g'
//   Adam::step   m = (m * beta1 + (1 - beta1)) * g          (as written in the reference: the moment estimate is
//                v = (v * beta2 + (1 - beta2)) * g^2         scaled by the gradient, not blended with it)
//                m_hat = m / (1 - beta1)^t ;  v_hat = v / (1 - beta2)^t      t is the optimizer's step counter,
//                u = clip(lr * m_hat / (sqrt(v_hat) + eps), -10, 10) ;  p -= u   which the reference leaves at 0
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>

#include "internal.h"

namespace ntb200 {
namespace {

template <typename T> struct Fmt;
template <> struct Fmt<float> {
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float x) { *p = x; }
    static float from_double(double x) { return float(x); }
};
template <> struct Fmt<__half> {
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ void store(__half* p, float x) { *p = __float2half_rn(x); }
    static float from_double(double x) { return __half2float(__double2half(x)); }
};
template <> struct Fmt<__nv_bfloat16> {
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
    static float from_double(double x) { return __bfloat162float(__double2bfloat16(x)); }
};

// Division and square root for the 16-bit formats.  The sequence to reproduce is the correctly rounded Float32 result,
// then one rounding to the 16-bit format (which, Float32 having more than twice the 16-bit formats' precision plus
// two bits, is the correctly rounded 16-bit result of the operation).  The hardware approximations are within two
// ulps (division) and one ulp (root) of the exact Float32 result, so whenever the approximation moved four ulps down
// and four ulps up rounds to one and the same 16-bit value, that value is the answer: rounding is monotonic and the
// exact result lies in between.  Otherwise (the approximation sits next to a rounding boundary of the narrow format:
// one element in a few thousand; or it is a NaN, or so small that the approximation itself may flush) the exact
// instruction is issued.  The result is the same always; subnormal 16-bit results take the fast path too.
template <typename T>
__device__ __forceinline__ bool settled(float q, float& rounded) {
    const uint32_t bits = __float_as_uint(q);
    const float lo = Fmt<T>::round(__uint_as_float(bits - 4u)), hi = Fmt<T>::round(__uint_as_float(bits + 4u));
    rounded = hi;
    return lo == hi && fabsf(q) > 1e-36f;   // false for NaNs; an approximation of a Float32 subnormal is not trusted
}
template <typename T>
__device__ __forceinline__ float div_rounded(float num, float den) {
    if constexpr (sizeof(T) == 2) {
        const float a = fabsf(den);
        if (a > 1e-30f && a < 1e30f) {
            if (num == 0.f) return __fdiv_rn(num, den) ;            // a signed zero: exact and cheap enough
            float r;
            if (settled<T>(__fdividef(num, den), r)) return r;
        }
    }
    return Fmt<T>::round(__fdiv_rn(num, den));
}
template <typename T>
__device__ __forceinline__ float sqrt_rounded(float x) {
    if constexpr (sizeof(T) == 2) {
        if (x > 1e-30f && x < 1e30f) {
            float q, r;
            asm("sqrt.approx.f32 %0, %1;" : "=f"(q) : "f"(x));
            if (settled<T>(q, r)) return r;
        }
    }
    return Fmt<T>::round(__fsqrt_rn(x));
}

// std::clamp as the reference's clamp_ applies it (nt/functional/cpu/min_max.cpp:66-101): a NaN stays a NaN
__device__ __forceinline__ float clip10(float x) { return x < -10.f ? -10.f : (10.f < x ? 10.f : x); }

// Elements per 16-byte vector, and a register view of one vector.
template <typename T> struct Vec {
    static constexpr int kN = 16 / int(sizeof(T));
    union { uint4 raw; T e[16 / sizeof(T)]; };
};

template <typename T>
__device__ __forceinline__ float sgd_one(float p, float g, float lr) {
    using F = Fmt<T>;
    return F::round(__fsub_rn(p, F::round(__fmul_rn(clip10(g), lr))));
}

// One 16-byte vector per thread and pass; the last n % kN elements are done one by one by the first threads.
template <typename T>
__global__ void sgd_step_kernel(T* __restrict__ param, const T* __restrict__ grad, long long n, float lr, int vec) {
    using F = Fmt<T>;
    constexpr int kN = Vec<T>::kN;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
    const long long nvec = vec ? n / kN : 0;
    for (long long i = tid; i < nvec; i += nthreads) {
        Vec<T> p, g;
        p.raw = reinterpret_cast<const uint4*>(param)[i];
        g.raw = reinterpret_cast<const uint4*>(grad)[i];
#pragma unroll
        for (int j = 0; j < kN; ++j) F::store(&p.e[j], sgd_one<T>(F::load(&p.e[j]), F::load(&g.e[j]), lr));
        reinterpret_cast<uint4*>(param)[i] = p.raw;
    }
    for (long long i = nvec * kN + tid; i < n; i += nthreads)
        F::store(param + i, sgd_one<T>(F::load(param + i), F::load(grad + i), lr));
}

struct AdamScalars {   // every scalar already rounded to the tensor's dtype, as Scalar -> T conversion does
    float lr, beta1, beta2, one_minus_beta1, one_minus_beta2, eps, corr1, corr2;
};

// Division by exactly 1 (the reference's bias correction while its step counter is 0) leaves every value as it is.
template <typename T>
__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamScalars& k) {
    using F = Fmt<T>;
    float mi = F::round(__fmul_rn(m, k.beta1));
    mi = F::round(__fadd_rn(mi, k.one_minus_beta1));
    mi = F::round(__fmul_rn(mi, g));
    const float g2 = F::round(__fmul_rn(g, g));
    float vi = F::round(__fmul_rn(v, k.beta2));
    vi = F::round(__fadd_rn(vi, k.one_minus_beta2));
    vi = F::round(__fmul_rn(vi, g2));
    m = mi;
    v = vi;
    const float m_hat = k.corr1 == 1.f ? mi : div_rounded<T>(mi, k.corr1);
    const float v_hat = k.corr2 == 1.f ? vi : div_rounded<T>(vi, k.corr2);
    const float num = F::round(__fmul_rn(k.lr, m_hat));
    const float den = F::round(__fadd_rn(sqrt_rounded<T>(v_hat), k.eps));
    const float u = clip10(div_rounded<T>(num, den));
    p = F::round(__fsub_rn(p, u));
}

// Eight 16-bit elements at once.  Every product and sum of the update is one correctly rounded operation in the
// tensor's own format, which is exactly what the packed hardware instructions deliver (the _rn forms are never
// contracted into an FMA); only the root and the two divisions go through Float32, lane by lane.
template <typename T> struct Packed;
template <> struct Packed<__half> {
    using T2 = __half2;
    static __device__ __forceinline__ T2 make(float x) { return __float2half2_rn(x); }
    static __device__ __forceinline__ float lo(T2 v) { return __low2float(v); }
    static __device__ __forceinline__ float hi(T2 v) { return __high2float(v); }
    static __device__ __forceinline__ T2 pack(float a, float b) { return __floats2half2_rn(a, b); }
};
template <> struct Packed<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ T2 make(float x) { return __float2bfloat162_rn(x); }
    static __device__ __forceinline__ float lo(T2 v) { return __low2float(v); }
    static __device__ __forceinline__ float hi(T2 v) { return __high2float(v); }
    static __device__ __forceinline__ T2 pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
};

template <typename T>
__device__ __forceinline__ void adam_pair(typename Packed<T>::T2& p, typename Packed<T>::T2 g, typename Packed<T>::T2& m,
                                          typename Packed<T>::T2& v, const AdamScalars& k) {
    using P = Packed<T>;
    using T2 = typename P::T2;
    T2 mi = __hmul2_rn(m, P::make(k.beta1));
    mi = __hadd2_rn(mi, P::make(k.one_minus_beta1));
    mi = __hmul2_rn(mi, g);
    const T2 g2 = __hmul2_rn(g, g);
    T2 vi = __hmul2_rn(v, P::make(k.beta2));
    vi = __hadd2_rn(vi, P::make(k.one_minus_beta2));
    vi = __hmul2_rn(vi, g2);
    m = mi;
    v = vi;
    const T2 m_hat = k.corr1 == 1.f ? mi : P::pack(div_rounded<T>(P::lo(mi), k.corr1), div_rounded<T>(P::hi(mi), k.corr1));
    const T2 v_hat = k.corr2 == 1.f ? vi : P::pack(div_rounded<T>(P::lo(vi), k.corr2), div_rounded<T>(P::hi(vi), k.corr2));
    const T2 num = __hmul2_rn(P::make(k.lr), m_hat);
    const T2 root = P::pack(sqrt_rounded<T>(P::lo(v_hat)), sqrt_rounded<T>(P::hi(v_hat)));
    const T2 den = __hadd2_rn(root, P::make(k.eps));
    const T2 u = P::pack(clip10(div_rounded<T>(P::lo(num), P::lo(den))), clip10(div_rounded<T>(P::hi(num), P::hi(den))));
    p = __hsub2_rn(p, u);
}

template <typename T>
__global__ void adam_step_kernel(T* __restrict__ param, const T* __restrict__ grad, T* __restrict__ m, T* __restrict__ v,
                                 long long n, AdamScalars k, int vec) {
    using F = Fmt<T>;
    constexpr int kN = Vec<T>::kN;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
    const long long nvec = vec ? n / kN : 0;
    for (long long i = tid; i < nvec; i += nthreads) {
        Vec<T> p, g, mm, vv;
        p.raw = reinterpret_cast<const uint4*>(param)[i];
        g.raw = reinterpret_cast<const uint4*>(grad)[i];
        mm.raw = reinterpret_cast<const uint4*>(m)[i];
        vv.raw = reinterpret_cast<const uint4*>(v)[i];
        if constexpr (sizeof(T) == 2) {
            using T2 = typename Packed<T>::T2;
            T2* p2 = reinterpret_cast<T2*>(&p.raw);
            T2* m2 = reinterpret_cast<T2*>(&mm.raw);
            T2* v2 = reinterpret_cast<T2*>(&vv.raw);
            const T2* g2 = reinterpret_cast<const T2*>(&g.raw);
#pragma unroll
            for (int j = 0; j < kN / 2; ++j) adam_pair<T>(p2[j], g2[j], m2[j], v2[j], k);
        } else {
#pragma unroll
            for (int j = 0; j < kN; ++j) {
                float pj = F::load(&p.e[j]), mj = F::load(&mm.e[j]), vj = F::load(&vv.e[j]);
                adam_one<T>(pj, F::load(&g.e[j]), mj, vj, k);
                F::store(&p.e[j], pj);
                F::store(&mm.e[j], mj);
                F::store(&vv.e[j], vj);
            }
        }
        reinterpret_cast<uint4*>(param)[i] = p.raw;
        reinterpret_cast<uint4*>(m)[i] = mm.raw;
        reinterpret_cast<uint4*>(v)[i] = vv.raw;
    }
    for (long long i = nvec * kN + tid; i < n; i += nthreads) {
        float pj = F::load(param + i), mj = F::load(m + i), vj = F::load(v + i);
        adam_one<T>(pj, F::load(grad + i), mj, vj, k);
        F::store(param + i, pj);
        F::store(m + i, mj);
        F::store(v + i, vj);
    }
}

inline int all_aligned16(const void* a, const void* b, const void* c = nullptr, const void* d = nullptr) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d)) % 16) == 0;
}

template <typename T>
void launch_adam(void* param, const void* grad, void* m, void* v, int64_t n, double learning_rate, double beta1,
                 double beta2, double epsilon, int64_t t, int grid, cudaStream_t s) {
    AdamScalars k;
    k.lr = Fmt<T>::from_double(learning_rate);
    k.beta1 = Fmt<T>::from_double(beta1);
    k.beta2 = Fmt<T>::from_double(beta2);
    k.one_minus_beta1 = Fmt<T>::from_double(1 - beta1);
    k.one_minus_beta2 = Fmt<T>::from_double(1 - beta2);
    k.eps = Fmt<T>::from_double(epsilon);
    k.corr1 = Fmt<T>::from_double(std::pow(1 - beta1, double(t)));
    k.corr2 = Fmt<T>::from_double(std::pow(1 - beta2, double(t)));
    adam_step_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(param), static_cast<const T*>(grad), static_cast<T*>(m),
                                             static_cast<T*>(v), n, k, all_aligned16(param, grad, m, v));
}

int grid_for_elements(int64_t n) {
    const int64_t blocks = (n + 2047) / 2048;   // about one 16-byte vector per thread, capped at 16 blocks per SM
    const int64_t cap = int64_t(sm_count()) * 16;
    return int(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace
}  // namespace ntb200

using namespace ntb200;

#define NTB200_OPT_SWITCH(dtype, CALL)                                                                            \
    switch (dtype) {                                                                                              \
        case NTB200_F32: { using T = float; CALL; break; }                                                        \
        case NTB200_F16: { using T = __half; CALL; break; }                                                       \
        case NTB200_BF16: { using T = __nv_bfloat16; CALL; break; }                                               \
        default: return fail(NTB200_ERR_UNSUPPORTED, "%s: dtype %s is not a float type of this engine", __func__, \
                             dtype_name(dtype));                                                                  \
    }

extern "C" {

int ntb200_sgd_step(int dtype, void* param, const void* grad, int64_t n, double learning_rate, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "sgd_step: negative size");
    if (n == 0) return NTB200_OK;
    if (!param || !grad) return fail(NTB200_ERR_INVALID_ARG, "sgd_step: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NTB200_OPT_SWITCH(dtype, (sgd_step_kernel<T><<<grid_for_elements(n), 256, 0, s>>>(
                                 static_cast<T*>(param), static_cast<const T*>(grad), n, Fmt<T>::from_double(learning_rate),
                                 all_aligned16(param, grad))));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_adam_step(int dtype, void* param, const void* grad, void* m, void* v, int64_t n, double learning_rate,
                     double beta1, double beta2, double epsilon, int64_t t, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "adam_step: negative size");
    if (n == 0) return NTB200_OK;
    if (!param || !grad || !m || !v) return fail(NTB200_ERR_INVALID_ARG, "adam_step: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NTB200_OPT_SWITCH(dtype, (launch_adam<T>(param, grad, m, v, n, learning_rate, beta1, beta2, epsilon, t, grid_for_elements(n), s)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

}  // extern "C"
