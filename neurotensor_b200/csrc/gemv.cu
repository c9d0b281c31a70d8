// Products with one or two rows, Float16 / BFloat16: out[m][n] = bias + sum_k a[m][k] * w(k, n).
//
// These are bound by reading the weight matrix once from HBM, and the tensor-core kernels cannot read it in long
// runs (their operand tiles are rows of 128 bytes).  Here every warp reads whole 512-byte runs of the weights along
// their contiguous direction with 16-byte loads, multiplies on the CUDA cores in fp32 and leaves fp32 partial sums
// per K slab; gemv_reduce_kernel adds the slabs in order, adds the bias / the previous C and rounds once (the same
// "fp32 accumulate, one rounding" contract as the tensor-core route, with a different summation order).
//   weights [K, N] (N contiguous, the layout of layers::Linear's Weight): a thread owns 8 neighbouring columns;
//   weights [N, K] (K contiguous, i.e. a transposed-view operand): a warp owns a row and reduces over its lanes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include <cstdlib>

#include "internal.h"

namespace ntb200 {
namespace {

constexpr int kGemvMaxRows = 2;    // measured: from four rows on the multiplies cost as much as the tensor route's slower reads
constexpr int kSlabKN = 64;      // K rows per block, [K, N] weights
constexpr int kSlabNK = 2048;    // K columns per block, [N, K] weights

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// partial[slab][m][n]; grid (ceil(n / 2048), slabs), 256 threads, thread t owns columns col0 + 8 t .. + 8.
template <typename T, int M>
__global__ void __launch_bounds__(256)
gemv_kn_kernel(const T* __restrict__ a, long long a_rs, const T* __restrict__ w, long long w_rs, float* __restrict__ partial,
               long long n, long long k) {
    __shared__ float xs[M][kSlabKN];
    const long long k0 = (long long)blockIdx.y * kSlabKN;
    const int kn = int(min((long long)kSlabKN, k - k0));
    for (int i = threadIdx.x; i < M * kSlabKN; i += 256) {
        const int m = i / kSlabKN, kk = i - m * kSlabKN;
        xs[m][kk] = kk < kn ? to_f(a[m * a_rs + k0 + kk]) : 0.f;
    }
    __syncthreads();
    const long long col = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
    if (col >= n) return;
    float acc[M][8];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][j] = 0.f;
    const T* wp = w + k0 * w_rs + col;
#pragma unroll 8
    for (int kk = 0; kk < kn; ++kk) {
        const uint4 v = *reinterpret_cast<const uint4*>(wp + (long long)kk * w_rs);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float wf = to_f(e[j]);
#pragma unroll
            for (int m = 0; m < M; ++m) acc[m][j] = fmaf(xs[m][kk], wf, acc[m][j]);
        }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
        float* dst = partial + ((long long)blockIdx.y * M + m) * n + col;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[m][4], acc[m][5], acc[m][6], acc[m][7]);
    }
}

// grid (ceil(n / 64), slabs), 256 threads = 8 warps, each warp owns 8 rows of w (output columns).
template <typename T, int M>
__global__ void __launch_bounds__(256)
gemv_nk_kernel(const T* __restrict__ a, long long a_rs, const T* __restrict__ w, long long w_rs, float* __restrict__ partial,
               long long n, long long k) {
    // a's slab, element kk kept at [kk & 7][kk >> 3]: a lane that holds weights kk = 8 q .. 8 q + 7 then reads
    // xs[m][j][q], and the 32 lanes of a warp (consecutive q) hit 32 different banks
    __shared__ float xs[M][8][kSlabNK / 8];
    const long long k0 = (long long)blockIdx.y * kSlabNK;
    const int kn = int(min((long long)kSlabNK, k - k0));     // a multiple of 8 (k is)
    for (int i = threadIdx.x; i < M * kSlabNK; i += 256) {
        const int m = i / kSlabNK, kk = i - m * kSlabNK;
        xs[m][kk & 7][kk >> 3] = kk < kn ? to_f(a[m * a_rs + k0 + kk]) : 0.f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = 0; r < 8; r += 2) {   // two rows at a time: sixteen 16-byte loads in flight per lane
        const long long col = (long long)blockIdx.x * 64 + warp * 8 + r;
        if (col >= n) break;
        const bool two = col + 1 < n;
        const T* wp0 = w + col * w_rs + k0;
        const T* wp1 = two ? wp0 + w_rs : wp0;
        float acc0[M], acc1[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
#pragma unroll 8
        for (int kk = lane * 8; kk < kn; kk += 256) {
            const uint4 v0 = *reinterpret_cast<const uint4*>(wp0 + kk);
            const uint4 v1 = *reinterpret_cast<const uint4*>(wp1 + kk);
            const T* e0 = reinterpret_cast<const T*>(&v0);
            const T* e1 = reinterpret_cast<const T*>(&v1);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w0 = to_f(e0[j]), w1 = to_f(e1[j]);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float xv = xs[m][j][kk >> 3];
                    acc0[m] = fmaf(xv, w0, acc0[m]);
                    acc1[m] = fmaf(xv, w1, acc1[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float s0 = acc0[m], s1 = acc1[m];
            for (int off = 16; off; off >>= 1) {
                s0 += __shfl_xor_sync(0xffffffffu, s0, off);
                s1 += __shfl_xor_sync(0xffffffffu, s1, off);
            }
            if (lane == 0) {
                partial[((long long)blockIdx.y * M + m) * n + col] = s0;
                if (two) partial[((long long)blockIdx.y * M + m) * n + col + 1] = s1;
            }
        }
    }
}

// Eight lanes per output: lane g adds slabs g, g + 8, ... (eight independent loads in flight at a time), the eight
// sums are combined in a fixed order by shuffles, and lane 0 adds the bias / previous C and rounds once.
template <typename T>
__global__ void __launch_bounds__(256)
gemv_reduce_kernel(const float* __restrict__ partial, int slabs, int rows, long long n, T* __restrict__ c, long long c_rs,
                   const T* __restrict__ bias, long long bias_rs, long long bias_cs, int accumulate) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int g = threadIdx.x & 7;
    const bool live = i < (long long)rows * n;
    const long long m = live ? i / n : 0, col = live ? i - m * n : 0;
    const float* pp = partial + m * n + col;
    const long long step = (long long)rows * n;
    float s = 0.f;
    if (live) {
        int sl = g;
        for (; sl + 56 < slabs; sl += 64) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = pp[(long long)(sl + 8 * u) * step];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
        }
        for (; sl < slabs; sl += 8) s += pp[(long long)sl * step];
    }
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if (live && g == 0) {
        if (bias) s += to_f(bias[m * bias_rs + col * bias_cs]);
        if (accumulate) s += to_f(c[m * c_rs + col]);
        c[m * c_rs + col] = from_f<T>(s);
    }
}

template <typename T, int M>
int launch_gemv_rows(const GemmArgs& g, bool kn_layout, cudaStream_t stream) {
    const long long slab = kn_layout ? kSlabKN : kSlabNK;
    const int slabs = int((g.k + slab - 1) / slab);
    float* partial = nullptr;
    if (int rc = scratch_acquire(reinterpret_cast<void**>(&partial), size_t(slabs) * M * size_t(g.n) * sizeof(float), stream)) return rc;
    const T* a = static_cast<const T*>(g.a);
    const T* w = static_cast<const T*>(g.b);
    if (kn_layout)
        gemv_kn_kernel<T, M><<<dim3(unsigned((g.n + 2047) / 2048), unsigned(slabs)), 256, 0, stream>>>(a, g.a_rs, w, g.b_rs, partial, g.n, g.k);
    else
        gemv_nk_kernel<T, M><<<dim3(unsigned((g.n + 63) / 64), unsigned(slabs)), 256, 0, stream>>>(a, g.a_rs, w, g.b_cs, partial, g.n, g.k);
    const long long outputs = (long long)g.m * g.n;
    gemv_reduce_kernel<T><<<unsigned((outputs * 8 + 255) / 256), 256, 0, stream>>>(partial, slabs, M, g.n, static_cast<T*>(g.c), g.c_rs,
                                                                               static_cast<const T*>(g.bias), g.bias_rs, g.bias_cs,
                                                                               g.accumulate);
    count_launch(2);
    cudaError_t e = cudaGetLastError();
    scratch_release(partial, stream);
    if (e != cudaSuccess) return cuda_fail(e, "gemv kernels");
    note_route("gemv_simt");
    return NTB200_OK;
}

}  // namespace

// One 2-D problem with one or two rows, 16-bit floats, K-contiguous A, weights contiguous along N or along K with
// 16-byte aligned rows, plain epilogue.
bool gemv_supported(const GemmArgs& g) {
    static const bool disabled = [] { const char* e = getenv("NTB200_NO_GEMV"); return e && e[0] == '1'; }();   // A/B measurements
    if (disabled) return false;
    if (g.dtype != NTB200_F16 && g.dtype != NTB200_BF16) return false;
    if (g.batch != 1 || g.m < 1 || g.m > kGemvMaxRows || g.k < 512 || g.n < 512) return false;
    if (g.a_ptrs || g.b_ptrs || g.c_ptrs || g.relu_out || g.mask_src || g.n_peers) return false;
    if (g.a_cs != 1 && g.k != 1) return false;
    if (g.n % 8 || g.k % 8 || reinterpret_cast<uintptr_t>(g.b) % 16) return false;
    if (g.k > (int64_t(1) << 30) || g.n > (int64_t(1) << 30) || g.a_rs < 0 || g.b_rs < 0 || g.b_cs < 0) return false;
    const bool kn = g.b_cs == 1 && g.b_rs % 8 == 0 && g.b_rs >= g.n;
    const bool nk = g.b_rs == 1 && g.b_cs % 8 == 0 && g.b_cs >= g.k;
    const long long slabs = kn ? (g.k + kSlabKN - 1) / kSlabKN : (g.k + kSlabNK - 1) / kSlabNK;
    return (kn || nk) && slabs <= 65535;
}

int launch_gemv(const GemmArgs& g, cudaStream_t stream) {
    const bool kn = g.b_cs == 1 && g.b_rs % 8 == 0 && g.b_rs >= g.n;
    GemmArgs q = g;
#define NTB200_GEMV(T)                                                                  \
    switch (g.m) {                                                                      \
        case 1: return launch_gemv_rows<T, 1>(q, kn, stream);                           \
        default: return launch_gemv_rows<T, 2>(q, kn, stream);                          \
    }
    if (g.dtype == NTB200_F16) { NTB200_GEMV(__half) }
    NTB200_GEMV(__nv_bfloat16)
#undef NTB200_GEMV
}

}  // namespace ntb200
