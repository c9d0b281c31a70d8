// CUDA-core GEMM for every dtype and every stride pattern: Float32 / Float64 (one ascending-k fused
// multiply-add chain per output element, which is exactly the order of the reference's microkernel,
// nt/functional/cpu/matmult/nt_matmult_simde.hpp:338-340), Int16/Int32/Int64 and their unsigned twins
// (wrapping multiply-add, nt/mp/simde_traits/simde_traits_avx2.h:444-485,523-540,810-865), and the route
// Float16 / BFloat16 / Int8 take when their operands cannot be described by a TMA tensor map.
//
// 128 x 128 output tile per CTA, 256 threads, 8 x 8 accumulators per thread held as two 4-wide halves so
// shared-memory reads are conflict-free; K is consumed in blocks staged through double-buffered shared
// memory with the next block prefetched into registers.  No split-K: the k order of every output is
// ascending, so Float32 results do not depend on the launch geometry.
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace ntb200 {
namespace {

constexpr int kBM = 128, kBN = 128, kThreads = 256;

struct SimtParams {
    long long m, n, k, batch;
    const void* a; long long a_rs, a_cs, a_bs;
    const void* b; long long b_rs, b_cs, b_bs;
    void* c; long long c_rs, c_bs;
    const void* bias; long long bias_rs, bias_cs, bias_bs;
    const void* const* a_ptrs; const void* const* b_ptrs; void* const* c_ptrs;
    int accumulate, round_per_ktile;
    int vec_ok;  // 4-byte dtype, 16-byte aligned bases, every non-unit stride a multiple of 4 elements
};

template <class T> struct Num;
template <> struct Num<float> {
    using Acc = float;
    static __device__ __forceinline__ Acc widen(float v) { return v; }
    static __device__ __forceinline__ float narrow(Acc v) { return v; }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return fmaf(a, b, c); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
template <> struct Num<double> {
    using Acc = double;
    static __device__ __forceinline__ Acc widen(double v) { return v; }
    static __device__ __forceinline__ double narrow(Acc v) { return v; }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return ::fma(a, b, c); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
template <> struct Num<__half> {
    using Acc = float;
    static __device__ __forceinline__ Acc widen(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half narrow(Acc v) { return __float2half_rn(v); }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return fmaf(a, b, c); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Num<__nv_bfloat16> {
    using Acc = float;
    static __device__ __forceinline__ Acc widen(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 narrow(Acc v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return fmaf(a, b, c); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
// Complex64 / Complex128 as the reference's SIMD traits treat them: a pair of independent lanes.  fmadd on the
// interleaved vector multiplies re with re and im with im (simde_traits_avx2.h:996-998, 1107-1109).
template <class F> struct Cplx {
    F re, im;
    Cplx() = default;
    __host__ __device__ explicit Cplx(int) : re(F(0)), im(F(0)) {}
    __host__ __device__ Cplx(F r, F i) : re(r), im(i) {}
};
template <class F> __device__ __forceinline__ Cplx<F> operator+(Cplx<F> a, Cplx<F> b) { return Cplx<F>(a.re + b.re, a.im + b.im); }
template <> struct Num<Cplx<float>> {
    using Acc = Cplx<float>;
    static __device__ __forceinline__ Acc widen(Acc v) { return v; }
    static __device__ __forceinline__ Acc narrow(Acc v) { return v; }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return Acc(fmaf(a.re, b.re, c.re), fmaf(a.im, b.im, c.im)); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
template <> struct Num<Cplx<double>> {
    using Acc = Cplx<double>;
    static __device__ __forceinline__ Acc widen(Acc v) { return v; }
    static __device__ __forceinline__ Acc narrow(Acc v) { return v; }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return Acc(::fma(a.re, b.re, c.re), ::fma(a.im, b.im, c.im)); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
// Complex32 (a pair of Float16): the reference's traits widen the interleaved halves to floats, multiply lane by lane
// and round the running sums back to Float16 whenever its K tile ends, every 8 k-steps for this type
// (simde_traits_avx2.h:1270-1300: pack size 4, so a tile is 8 wide; load = cvtph_ps, store = cvtps_ph).
struct CplxH {
    __half re, im;
};
template <> struct Num<CplxH> {
    using Acc = Cplx<float>;
    static __device__ __forceinline__ Acc widen(CplxH v) { return Acc(__half2float(v.re), __half2float(v.im)); }
    static __device__ __forceinline__ CplxH narrow(Acc v) { CplxH r; r.re = __float2half_rn(v.re); r.im = __float2half_rn(v.im); return r; }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return Acc(fmaf(a.re, b.re, c.re), fmaf(a.im, b.im, c.im)); }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return Acc(__half2float(__float2half_rn(v.re)), __half2float(__float2half_rn(v.im))); }
};
template <class U, class A> struct IntNum {
    using Acc = A;
    static __device__ __forceinline__ Acc widen(U v) { return Acc(v); }
    static __device__ __forceinline__ U narrow(Acc v) { return U(v); }
    static __device__ __forceinline__ Acc fma(Acc a, Acc b, Acc c) { return a * b + c; }
    static __device__ __forceinline__ Acc round_tile(Acc v) { return v; }
};
template <> struct Num<uint8_t> : IntNum<uint8_t, uint32_t> {};
template <> struct Num<uint16_t> : IntNum<uint16_t, uint32_t> {};
template <> struct Num<uint32_t> : IntNum<uint32_t, uint32_t> {};
template <> struct Num<unsigned long long> : IntNum<unsigned long long, unsigned long long> {};

// One CTA per SM by register count (231 registers for Float32).  More warps per SM do not help: holding a thread to
// 128 registers (__launch_bounds__(256, 2), two CTAs per SM, a few spills) gave 41.7 against 45.7 TFLOP/s at 4096^3,
// and a Float32-only variant with 64 x 128 tiles, 128 threads and three CTAs per SM at 168 registers (twelve warps,
// no spills, same chains) gave 43.3 against 44.9 (30.4 against 38.4 at 2048^3).
template <class T>
__global__ void __launch_bounds__(kThreads)
simt_gemm_kernel(const SimtParams p) {
    using N = Num<T>;
    using Acc = typename N::Acc;
    constexpr int BK = sizeof(Acc) >= 16 ? 4 : (sizeof(Acc) == 8 ? 8 : 16);
    constexpr int kLoads = kBM * BK / kThreads;  // elements of each operand tile per thread
    // +4 elements of padding per row: rows stay 16-byte aligned for vector reads, and the transposing stores of a
    // K-contiguous operand (16 consecutive k of one row per half-warp) spread over the banks instead of hitting one
    constexpr int kPad = 4;
    __shared__ __align__(16) Acc As[2][BK][kBM + kPad];
    __shared__ __align__(16) Acc Bs[2][BK][kBN + kPad];

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const long long bidx = blockIdx.z;
    const long long m0 = (long long)blockIdx.y * kBM, n0 = (long long)blockIdx.x * kBN;
    const T* A = p.a_ptrs ? static_cast<const T*>(p.a_ptrs[bidx]) : static_cast<const T*>(p.a) + bidx * p.a_bs;
    const T* B = p.b_ptrs ? static_cast<const T*>(p.b_ptrs[bidx]) : static_cast<const T*>(p.b) + bidx * p.b_bs;
    T* C = p.c_ptrs ? static_cast<T*>(p.c_ptrs[bidx]) : static_cast<T*>(p.c) + bidx * p.c_bs;

    // Loader geometry: walk the unit-stride direction with consecutive threads.
    const bool a_k_fast = (p.a_cs == 1 && p.a_rs != 1);
    const bool b_k_fast = (p.b_rs == 1 && p.b_cs != 1);

    // Interior tiles of 4-byte dtypes with 16-byte aligned operands take 16-byte global loads (two per operand per
    // thread and K block instead of eight scalar ones); edge tiles and everything else take the scalar path.  The
    // values and their k order are the same either way.
    constexpr bool kVecCapable = sizeof(T) == 4 && sizeof(Acc) == 4 && BK == 16;
    const bool vec_tile = kVecCapable && p.vec_ok && m0 + kBM <= p.m && n0 + kBN <= p.n;

    Acc ra[kLoads], rb[kLoads];
    auto fetch = [&](long long k0) {
        if constexpr (kVecCapable) {
            if (vec_tile && k0 + BK <= p.k) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int v = tid + i * kThreads;   // 0..511: one float4 each
                    float4 qa, qb;
                    if (a_k_fast) qa = *reinterpret_cast<const float4*>(A + (m0 + (v >> 2)) * p.a_rs + k0 + (v & 3) * 4);
                    else qa = *reinterpret_cast<const float4*>(A + (k0 + (v >> 5)) * p.a_cs + m0 + (v & 31) * 4);
                    if (b_k_fast) qb = *reinterpret_cast<const float4*>(B + (n0 + (v >> 2)) * p.b_cs + k0 + (v & 3) * 4);
                    else qb = *reinterpret_cast<const float4*>(B + (k0 + (v >> 5)) * p.b_rs + n0 + (v & 31) * 4);
                    const Acc* pa = reinterpret_cast<const Acc*>(&qa);
                    const Acc* pb = reinterpret_cast<const Acc*>(&qb);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { ra[i * 4 + j] = pa[j]; rb[i * 4 + j] = pb[j]; }
                }
                return true;
            }
        }
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            const int e = tid + i * kThreads;
            int mm, kk;
            if (a_k_fast) { kk = e % BK; mm = e / BK; } else { mm = e % kBM; kk = e / kBM; }
            const long long gm = m0 + mm, gk = k0 + kk;
            ra[i] = (gm < p.m && gk < p.k) ? N::widen(A[gm * p.a_rs + gk * p.a_cs]) : Acc(0);
            int nn, kb;
            if (b_k_fast) { kb = e % BK; nn = e / BK; } else { nn = e % kBN; kb = e / kBN; }
            const long long gn = n0 + nn, gkb = k0 + kb;
            rb[i] = (gn < p.n && gkb < p.k) ? N::widen(B[gkb * p.b_rs + gn * p.b_cs]) : Acc(0);
        }
        return false;
    };
    auto stash = [&](int buf, bool vec) {
        if constexpr (kVecCapable) {
            if (vec) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int v = tid + i * kThreads;
                    if (a_k_fast) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) As[buf][(v & 3) * 4 + j][v >> 2] = ra[i * 4 + j];
                    } else {
                        *reinterpret_cast<float4*>(&As[buf][v >> 5][(v & 31) * 4]) = *reinterpret_cast<const float4*>(&ra[i * 4]);
                    }
                    if (b_k_fast) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) Bs[buf][(v & 3) * 4 + j][v >> 2] = rb[i * 4 + j];
                    } else {
                        *reinterpret_cast<float4*>(&Bs[buf][v >> 5][(v & 31) * 4]) = *reinterpret_cast<const float4*>(&rb[i * 4]);
                    }
                }
                return;
            }
        }
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            const int e = tid + i * kThreads;
            int mm, kk;
            if (a_k_fast) { kk = e % BK; mm = e / BK; } else { mm = e % kBM; kk = e / kBM; }
            As[buf][kk][mm] = ra[i];
            int nn, kb;
            if (b_k_fast) { kb = e % BK; nn = e / BK; } else { nn = e % kBN; kb = e / kBN; }
            Bs[buf][kb][nn] = rb[i];
        }
    };

    // rows ty*4 + {0..3} and 64 + ty*4 + {0..3}; columns tx*4 + {0..3} and 64 + tx*4 + {0..3}
    Acc acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            Acc v = Acc(0);
            if (row < p.m && col < p.n) {
                // the chain starts from the bias (linear) or from the previous C (the C += contract)
                if (p.accumulate) v = N::widen(C[row * p.c_rs + col]);
                if (p.bias) {
                    const Acc bv = N::widen(static_cast<const T*>(p.bias)[bidx * p.bias_bs + row * p.bias_rs + col * p.bias_cs]);
                    v = p.accumulate ? Acc(v + bv) : bv;
                }
            }
            acc[i][j] = v;
        }
    }

    const long long kblocks = (p.k + BK - 1) / BK;
    bool fetched_vec = false;
    if (kblocks > 0) {
        fetched_vec = fetch(0);
        stash(0, fetched_vec);
    }
    __syncthreads();
    for (long long kb = 0; kb < kblocks; ++kb) {
        const int buf = int(kb & 1);
        if (kb + 1 < kblocks) fetched_vec = fetch((kb + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            Acc af[8], bf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                af[i] = As[buf][kk][ty * 4 + i];
                af[4 + i] = As[buf][kk][64 + ty * 4 + i];
                bf[i] = Bs[buf][kk][tx * 4 + i];
                bf[4 + i] = Bs[buf][kk][64 + tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = N::fma(af[i], bf[j], acc[i][j]);
        }
        if (p.round_per_ktile) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = N::round_tile(acc[i][j]);
        }
        if (kb + 1 < kblocks) stash(buf ^ 1, fetched_vec);
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long col = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (col < p.n) C[row * p.c_rs + col] = N::narrow(acc[i][j]);
        }
    }
}

// C = (accumulate ? C : 0) + bias when there is nothing to contract (K == 0).
template <class T>
__global__ void fill_c_kernel(const SimtParams p) {
    using N = Num<T>;
    using Acc = typename N::Acc;
    const long long total = p.m * p.n * p.batch;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long col = i % p.n, row = (i / p.n) % p.m, b = i / (p.n * p.m);
        T* C = p.c_ptrs ? static_cast<T*>(p.c_ptrs[b]) : static_cast<T*>(p.c) + b * p.c_bs;
        Acc v = Acc(0);
        if (p.accumulate) v = N::widen(C[row * p.c_rs + col]);
        if (p.bias) {
            const Acc bv = N::widen(static_cast<const T*>(p.bias)[b * p.bias_bs + row * p.bias_rs + col * p.bias_cs]);
            v = p.accumulate ? Acc(v + bv) : bv;
        }
        C[row * p.c_rs + col] = N::narrow(v);
    }
}

SimtParams to_params(const GemmArgs& g) {
    SimtParams p{};
    p.m = g.m; p.n = g.n; p.k = g.k; p.batch = g.batch;
    p.a = g.a; p.a_rs = g.a_rs; p.a_cs = g.a_cs; p.a_bs = g.a_bs;
    p.b = g.b; p.b_rs = g.b_rs; p.b_cs = g.b_cs; p.b_bs = g.b_bs;
    p.c = g.c; p.c_rs = g.c_rs; p.c_bs = g.c_bs;
    p.bias = g.bias; p.bias_rs = g.bias_rs; p.bias_cs = g.bias_cs; p.bias_bs = g.bias_bs;
    p.a_ptrs = g.a_ptrs; p.b_ptrs = g.b_ptrs; p.c_ptrs = g.c_ptrs;
    p.accumulate = g.accumulate;
    auto al16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    auto m4 = [](long long v) { return v % 4 == 0; };
    const bool a_ok = (g.a_cs == 1 && g.a_rs != 1) ? m4(g.a_rs) : (g.a_rs == 1 && m4(g.a_cs));
    const bool b_ok = (g.b_rs == 1 && g.b_cs != 1) ? m4(g.b_cs) : (g.b_cs == 1 && m4(g.b_rs));
    p.vec_ok = (dtype_size(g.dtype) == 4 && !g.a_ptrs && al16(g.a) && al16(g.b) && a_ok && b_ok && m4(g.a_bs) && m4(g.b_bs)) ? 1 : 0;
    // Complex32 always rounds at the reference's K-tile edges (the kernel's K block for this type is the reference's tile, 8)
    p.round_per_ktile = ((g.dtype == NTB200_F16 && g.f16_rounding == NTB200_F16_ROUND_PER_KTILE) || g.dtype == NTB200_C32) ? 1 : 0;
    return p;
}

template <class T>
int launch_typed(const GemmArgs& g, cudaStream_t stream, bool fill_only) {
    const SimtParams p = to_params(g);
    if (fill_only) {
        const long long total = g.m * g.n * g.batch;
        const int blocks = int(std::min<long long>((total + 255) / 256, 148 * 8));
        fill_c_kernel<T><<<blocks, 256, 0, stream>>>(p);
    } else {
        // gridDim.z is limited to 65535: slice larger batches
        const long long gx = (g.n + kBN - 1) / kBN, gy = (g.m + kBM - 1) / kBM;
        if (gy > 65535) return fail(NTB200_ERR_UNSUPPORTED, "M too large for the CUDA-core route");
        for (long long b0 = 0; b0 < g.batch; b0 += 65535) {
            SimtParams q = p;
            const long long nb = std::min<long long>(65535, g.batch - b0);
            q.batch = nb;
            if (q.a_ptrs) { q.a_ptrs += b0; q.b_ptrs += b0; q.c_ptrs += b0; }
            else {
                q.a = static_cast<const char*>(p.a) + b0 * p.a_bs * sizeof(T);
                q.b = static_cast<const char*>(p.b) + b0 * p.b_bs * sizeof(T);
                q.c = static_cast<char*>(p.c) + b0 * p.c_bs * sizeof(T);
                if (q.bias) q.bias = static_cast<const char*>(p.bias) + b0 * p.bias_bs * sizeof(T);
            }
            simt_gemm_kernel<T><<<dim3(unsigned(gx), unsigned(gy), unsigned(nb)), kThreads, 0, stream>>>(q);
            count_launch();
        }
        NTB200_CUDA(cudaGetLastError());
        return NTB200_OK;
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int dispatch(const GemmArgs& g, cudaStream_t stream, bool fill_only) {
    switch (g.dtype) {
        case NTB200_F32: return launch_typed<float>(g, stream, fill_only);
        case NTB200_F64: return launch_typed<double>(g, stream, fill_only);
        case NTB200_F16: return launch_typed<__half>(g, stream, fill_only);
        case NTB200_BF16: return launch_typed<__nv_bfloat16>(g, stream, fill_only);
        case NTB200_I8: case NTB200_U8: return launch_typed<uint8_t>(g, stream, fill_only);
        case NTB200_I16: case NTB200_U16: return launch_typed<uint16_t>(g, stream, fill_only);
        case NTB200_I32: case NTB200_U32: return launch_typed<uint32_t>(g, stream, fill_only);
        case NTB200_I64: return launch_typed<unsigned long long>(g, stream, fill_only);
        case NTB200_C64: return launch_typed<Cplx<float>>(g, stream, fill_only);
        case NTB200_C128: return launch_typed<Cplx<double>>(g, stream, fill_only);
        case NTB200_C32: return launch_typed<CplxH>(g, stream, fill_only);
    }
    return fail(NTB200_ERR_UNSUPPORTED, "unknown dtype %d", g.dtype);
}

}  // namespace

int launch_simt_gemm(const GemmArgs& g, cudaStream_t stream) {
    note_route("simt");
    return dispatch(g, stream, false);
}

int launch_fill_c(const GemmArgs& g, cudaStream_t stream) {
    note_route("fill");
    return dispatch(g, stream, true);
}

}  // namespace ntb200
