// Memory-bound neighbours of the GEMM on the Linear / conv2d path: im2col and its adjoint, ReLU and its
// mask backward, MSE, the bias-gradient column sum, gradient accumulation, strided copy and dtype
// conversion.  All are HBM-bound byte movers: coalesced along the innermost dimension, grid-stride loops
// sized in multiples of the SM count.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "internal.h"

namespace ntb200 {
namespace {

inline int grid_for(long long n, int per_block) {
    const long long want = (n + per_block - 1) / per_block;
    return int(std::max<long long>(1, std::min<long long>(want, (long long)sm_count() * 16)));
}

template <class T> struct F;
template <> struct F<float> {
    static __device__ __forceinline__ float ld(float v) { return v; }
    static __device__ __forceinline__ float st(float v) { return v; }
};
template <> struct F<__half> {
    static __device__ __forceinline__ float ld(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half st(float v) { return __float2half_rn(v); }
};
template <> struct F<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 st(float v) { return __float2bfloat16_rn(v); }
};

struct ConvGeom {
    long long batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, hc, wc;
};

// Column-matrix writer.  Each thread produces V = 16 / sizeof(T) consecutive output pixels of one column-matrix row
// (one (channel, tap) pair of one image) and writes them with a single 16-byte store; consecutive threads write
// consecutive 16-byte segments, so stores are fully coalesced, and for unit stride the loads of a warp cover a
// contiguous run of the image.  The (batch, row, pixel) decomposition is done once per vector in index type I
// (32-bit whenever the element counts allow it).  T is an unsigned integer of the element's size: pure byte moves.
template <class T, class I, int V>
__global__ void im2col_kernel(const T* __restrict__ im, T* __restrict__ col, const ConvGeom g) {
    const I L = I(g.hc * g.wc), ccol = I(g.channels * g.kh * g.kw), wc = I(g.wc), kw = I(g.kw), kh = I(g.kh);
    const I vec_per_row = L / V;  // V divides L on this path (V == 1 otherwise)
    const I total_vec = I(g.batch) * ccol * vec_per_row;
    const I height = I(g.height), width = I(g.width);
    const I sh = I(g.sh), sw = I(g.sw), ph = I(g.ph), pw = I(g.pw), dh = I(g.dh), dw = I(g.dw);
    for (I v = I(blockIdx.x) * I(blockDim.x) + I(threadIdx.x); v < total_vec; v += I(gridDim.x) * I(blockDim.x)) {
        const I lv = v % vec_per_row, row = v / vec_per_row;   // row = b * ccol + c
        const I c = row % ccol, b = row / ccol;
        const I w_off = c % kw, h_off = (c / kw) % kh, c_im = c / (kh * kw);
        const I l0 = lv * V;
        I h = l0 / wc, w = l0 - h * wc;
        const T* plane = im + (I(b) * I(g.channels) + c_im) * height * width;
        __align__(16) T out[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const I hp = h * sh - ph + h_off * dh, wp = w * sw - pw + w_off * dw;
            T val = T(0);
            if (hp >= 0 && hp < height && wp >= 0 && wp < width) val = plane[hp * width + wp];
            out[j] = val;
            if (++w == wc) { w = 0; ++h; }
        }
        T* dst = col + row * L + l0;
        if constexpr (V * sizeof(T) == 16) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(out);
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) dst[j] = out[j];
        }
    }
}

// Same result, staged through shared memory: one CTA owns one (image, channel) plane, reads it from HBM once with
// coalesced loads, and writes the kh*kw column-matrix rows that are built from it (each a shifted, zero-padded
// copy of the plane) with 16-byte stores.  Global loads drop by kh*kw and the kernel is bound by the column-matrix
// write.  Requires the output width to be a multiple of the vector width V, so a vector never straddles two output
// rows: a thread keeps one vector column and walks down the output rows, so the inner loop has no division and a
// single row test per vector.
template <class T, int V>
__global__ void im2col_plane_kernel(const T* __restrict__ im, T* __restrict__ col, const ConvGeom g) {
    extern __shared__ __align__(16) unsigned char plane_raw[];
    T* plane = reinterpret_cast<T*>(plane_raw);
    const int c_im = blockIdx.x, b = blockIdx.y;
    const int height = int(g.height), width = int(g.width), wc = int(g.wc), hc = int(g.hc), L = hc * wc;
    const int kh = int(g.kh), kw = int(g.kw);
    const int sh = int(g.sh), sw = int(g.sw), ph = int(g.ph), pw = int(g.pw), dh = int(g.dh), dw = int(g.dw);
    const int plane_elems = height * width;
    const T* src = im + ((long long)b * g.channels + c_im) * plane_elems;
    if ((reinterpret_cast<uintptr_t>(src) % 16 == 0) && (plane_elems % V == 0)) {
        for (int i = threadIdx.x; i < plane_elems / V; i += blockDim.x)
            reinterpret_cast<uint4*>(plane)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < plane_elems; i += blockDim.x) plane[i] = src[i];
    }
    __syncthreads();
    const int vec_per_wrow = wc / V;                       // vectors per output row
    const int rows_per_pass = blockDim.x / vec_per_wrow;   // >= 1 (checked by the launcher)
    const int hv = threadIdx.x / vec_per_wrow, wv = threadIdx.x - hv * vec_per_wrow;
    if (hv >= rows_per_pass) return;
    const int w0 = wv * V;
    T* dst_base = col + ((long long)b * g.channels + c_im) * (kh * kw) * (long long)L + w0;
    for (int h_off = 0; h_off < kh; ++h_off) {
        for (int w_off = 0; w_off < kw; ++w_off) {
            T* dst_tap = dst_base + (long long)(h_off * kw + w_off) * L;
            const int wp0 = w0 * sw - pw + w_off * dw;
            for (int h = hv; h < hc; h += rows_per_pass) {
                const int hp = h * sh - ph + h_off * dh;
                __align__(16) T out[V];
                if constexpr (sizeof(T) == 2) {
                    // unit stride, the whole vector inside the row: 8 consecutive 2-byte pixels come from 4 aligned
                    // 32-bit shared loads, or from 5 of them and a funnel shift when the run starts on an odd pixel
                    if (sw == 1 && hp >= 0 && hp < height && wp0 >= 0 && wp0 + V <= width) {
                        const int e0 = hp * width + wp0;
                        const uint32_t* words = reinterpret_cast<const uint32_t*>(plane) + (e0 >> 1);
                        uint32_t o[4];
                        if ((e0 & 1) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) o[j] = words[j];
                        } else {
                            uint32_t w5[5];
#pragma unroll
                            for (int j = 0; j < 5; ++j) w5[j] = words[j];
#pragma unroll
                            for (int j = 0; j < 4; ++j) o[j] = __funnelshift_r(w5[j], w5[j + 1], 16);
                        }
                        *reinterpret_cast<uint4*>(dst_tap + h * wc) = make_uint4(o[0], o[1], o[2], o[3]);
                        continue;
                    }
                }
                if (hp >= 0 && hp < height) {
                    const T* row = plane + hp * width;
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const int wp = wp0 + j * sw;
                        out[j] = (unsigned(wp) < unsigned(width)) ? row[wp] : T(0);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) out[j] = T(0);
                }
                *reinterpret_cast<uint4*>(dst_tap + h * wc) = *reinterpret_cast<const uint4*>(out);
            }
        }
    }
}

template <class T>
void launch_im2col(const void* im, void* col, const ConvGeom& g, cudaStream_t s) {
    constexpr int V = 16 / int(sizeof(T));
    const long long L = g.hc * g.wc, total = g.batch * g.channels * g.kh * g.kw * L;
    const long long im_elems = g.batch * g.channels * g.height * g.width;
    const bool small = total < (1ll << 31) && im_elems < (1ll << 31);
    const bool vec = (L % V == 0) && (reinterpret_cast<uintptr_t>(col) % 16 == 0);
    const long long work = vec ? total / V : total;
    const int blocks = grid_for(work, 256);
    const T* src = static_cast<const T*>(im);
    T* dst = static_cast<T*>(col);
    const long long plane_bytes = g.height * g.width * (long long)sizeof(T);
    if (vec && small && plane_bytes <= 40 * 1024 && g.batch <= 65535 && g.kh * g.kw > 1 && g.wc % V == 0 && g.wc / V <= 256) {
        im2col_plane_kernel<T, V><<<dim3(unsigned(g.channels), unsigned(g.batch)), 256, size_t((plane_bytes + 15) / 16 * 16 + 16), s>>>(src, dst, g);
        return;
    }
    if (vec && small) im2col_kernel<T, int, V><<<blocks, 256, 0, s>>>(src, dst, g);
    else if (vec) im2col_kernel<T, long long, V><<<blocks, 256, 0, s>>>(src, dst, g);
    else if (small) im2col_kernel<T, int, 1><<<blocks, 256, 0, s>>>(src, dst, g);
    else im2col_kernel<T, long long, 1><<<blocks, 256, 0, s>>>(src, dst, g);
}

// Gather form of col2im: each image element sums the taps that read it (no atomics, deterministic).
template <class T>
__global__ void col2im_kernel(const T* __restrict__ col, T* __restrict__ im, const ConvGeom g) {
    const long long total = g.batch * g.channels * g.height * g.width;
    const long long L = g.hc * g.wc, ccol = g.channels * g.kh * g.kw;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long w = i % g.width, h = (i / g.width) % g.height;
        const long long c_im = (i / (g.width * g.height)) % g.channels, b = i / (g.width * g.height * g.channels);
        float acc = 0.f;
        for (long long ki = 0; ki < g.kh; ++ki) {
            const long long hn = h + g.ph - ki * g.dh;
            if (hn < 0 || hn % g.sh) continue;
            const long long hc = hn / g.sh;
            if (hc >= g.hc) continue;
            for (long long kj = 0; kj < g.kw; ++kj) {
                const long long wn = w + g.pw - kj * g.dw;
                if (wn < 0 || wn % g.sw) continue;
                const long long wc = wn / g.sw;
                if (wc >= g.wc) continue;
                const long long c = (c_im * g.kh + ki) * g.kw + kj;
                acc += F<T>::ld(col[(b * ccol + c) * L + hc * g.wc + wc]);
            }
        }
        im[i] = F<T>::st(acc);
    }
}

// 16-byte vector forms of the elementwise kernels (n a multiple of the vector width, pointers 16-byte aligned).
template <class T> struct Vec16 { static constexpr int N = 16 / int(sizeof(T)); T v[N]; };

template <class T>
__global__ void relu_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, long long nvec) {
    using VT = Vec16<T>;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        uint4 raw = x[i];
        VT& a = *reinterpret_cast<VT*>(&raw);
#pragma unroll
        for (int j = 0; j < VT::N; ++j)
            if (F<T>::ld(a.v[j]) < 0.f) a.v[j] = F<T>::st(0.f);
        y[i] = raw;
    }
}
template <class T>
__global__ void relu_backward_vec_kernel(const uint4* __restrict__ x, const uint4* __restrict__ go, uint4* __restrict__ gi,
                                         long long nvec) {
    using VT = Vec16<T>;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        uint4 rx = x[i], rg = go[i];
        const VT& a = *reinterpret_cast<const VT*>(&rx);
        VT& g = *reinterpret_cast<VT*>(&rg);
#pragma unroll
        for (int j = 0; j < VT::N; ++j)
            if (F<T>::ld(a.v[j]) < 0.f) g.v[j] = F<T>::st(0.f);
        gi[i] = rg;
    }
}
template <class T>
__global__ void add_inplace_vec_kernel(uint4* __restrict__ y, const uint4* __restrict__ x, long long nvec) {
    using VT = Vec16<T>;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        uint4 ry = y[i], rx = x[i];
        VT& a = *reinterpret_cast<VT*>(&ry);
        const VT& b = *reinterpret_cast<const VT*>(&rx);
#pragma unroll
        for (int j = 0; j < VT::N; ++j) a.v[j] = F<T>::st(F<T>::ld(a.v[j]) + F<T>::ld(b.v[j]));
        y[i] = ry;
    }
}
inline bool vec_ok(long long n, int elem_size, const void* a, const void* b = nullptr, const void* c = nullptr) {
    auto al = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    return n % (16 / elem_size) == 0 && al(a) && al(b) && al(c);
}

template <class T>
__global__ void relu_kernel(const T* __restrict__ x, T* __restrict__ y, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = F<T>::ld(x[i]);
        y[i] = v < 0.f ? F<T>::st(0.f) : x[i];
    }
}
// grad_in = grad_out where clamp left x unchanged (x >= 0), else 0 (the "before != after" mask).
template <class T>
__global__ void relu_backward_kernel(const T* __restrict__ x, const T* __restrict__ go, T* __restrict__ gi, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        gi[i] = F<T>::ld(x[i]) < 0.f ? F<T>::st(0.f) : go[i];
}

template <class T>
__global__ void mse_kernel(const T* __restrict__ o, const T* __restrict__ t, T* __restrict__ grad, float* __restrict__ loss,
                           long long n, float inv_n) {
    float local = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float d = F<T>::ld(o[i]) - F<T>::ld(t[i]);
        local += d * d;
        if (grad) grad[i] = F<T>::st(2.f * d * inv_n);
    }
    __shared__ float red[32];
    for (int off = 16; off; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (threadIdx.x == 0) atomicAdd(loss, v * inv_n);
    }
}

// The gradient of mse_kernel alone, for a [rows, cols] block of a larger matrix (row strides in elements): the same
// expression, with the element count of the WHOLE matrix the loss is taken over.
template <class T>
__global__ void mse_grad_block_kernel(const T* __restrict__ o, long long o_rs, const T* __restrict__ t, long long t_rs,
                                      T* __restrict__ grad, long long g_rs, long long rows, long long cols, float inv_n) {
    const long long total = rows * cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols, c = i - r * cols;
        const float d = F<T>::ld(o[r * o_rs + c]) - F<T>::ld(t[r * t_rs + c]);
        grad[r * g_rs + c] = F<T>::st(2.f * d * inv_n);
    }
}

// out[c] = sum_r grad[r][c]; block = 32 columns x 32 row lanes, one block per 32 columns.
template <class T>
__global__ void column_sum_kernel(const T* __restrict__ g, T* __restrict__ out, long long rows, long long cols) {
    __shared__ float red[32][33];
    const long long c = (long long)blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (c < cols)
        for (long long r = threadIdx.y; r < rows; r += 32) acc += F<T>::ld(g[r * cols + c]);
    red[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < cols) {
        float s = 0.f;
        for (int r = 0; r < 32; ++r) s += red[r][threadIdx.x];
        out[c] = F<T>::st(s);
    }
}

// Column sums of a 16-bit matrix with 16-byte loads: a warp covers 256 columns of one row (512 contiguous bytes),
// the block's 8 row lanes walk its slab of rows, and every (column block, row slab) leaves one fp32 partial row;
// column_sum_final_kernel adds the slabs in order and rounds once.
template <class T>
__global__ void __launch_bounds__(256)
column_sum_partial_kernel(const T* __restrict__ g, float* __restrict__ partial, long long rows, long long cols, long long rows_per_slab) {
    __shared__ float red[8][256 + 8];
    const long long c0 = ((long long)blockIdx.x * 32 + threadIdx.x) * 8;
    const long long r_begin = (long long)blockIdx.y * rows_per_slab, r_end = min(rows, r_begin + rows_per_slab);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (c0 < cols) {
        for (long long r = r_begin + threadIdx.y; r < r_end; r += 8) {
            const uint4 v = *reinterpret_cast<const uint4*>(g + r * cols + c0);
            const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += F<T>::ld(e[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x * 8 + j] = acc[j];
    __syncthreads();
    const int t = threadIdx.y * 32 + threadIdx.x;   // 256 threads, one column of the block each
    const long long c = (long long)blockIdx.x * 256 + t;
    if (c < cols) {
        float s = 0.f;
#pragma unroll
        for (int y = 0; y < 8; ++y) s += red[y][t];
        partial[(long long)blockIdx.y * cols + c] = s;
    }
}
template <class T>
__global__ void column_sum_final_kernel(const float* __restrict__ partial, T* __restrict__ out, int slabs, long long cols) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int i = 0; i < slabs; ++i) s += partial[(long long)i * cols + c];
    out[c] = F<T>::st(s);
}

// x[b][c][i] += bias[c] in place: the `outp + Bias` of layers::Conv2D with Bias shaped [C, 1, 1].
template <class T>
__global__ void bias_add_channels_kernel(T* __restrict__ x, const T* __restrict__ bias, long long total, long long channels,
                                         long long inner) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long c = (i / inner) % channels;
        x[i] = F<T>::st(F<T>::ld(x[i]) + F<T>::ld(bias[c]));
    }
}
// Eight 16-bit elements per thread when a channel's run is a multiple of 8 elements (one channel per vector).
template <class T>
__global__ void bias_add_channels_vec_kernel(uint4* __restrict__ x, const T* __restrict__ bias, long long nvec, long long channels,
                                             long long inner_vec) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        const float b = F<T>::ld(bias[(i / inner_vec) % channels]);
        uint4 v = x[i];
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int j = 0; j < int(16 / sizeof(T)); ++j) e[j] = F<T>::st(F<T>::ld(e[j]) + b);
        x[i] = v;
    }
}
// out[c] = sum over b and i of g[b][c][i] (the bias gradient of layers::Conv2D): one block per channel, fp32 sums.
template <class T>
__global__ void __launch_bounds__(256)
sum_channels_kernel(const T* __restrict__ g, T* __restrict__ out, long long batch, long long channels, long long inner) {
    const long long c = blockIdx.x;
    float acc = 0.f;
    for (long long b = 0; b < batch; ++b) {
        const T* row = g + (b * channels + c) * inner;
        for (long long i = threadIdx.x; i < inner; i += blockDim.x) acc += F<T>::ld(row[i]);
    }
    __shared__ float red[8];
    for (int off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < 8; ++w) s += red[w];
        out[c] = F<T>::st(s);
    }
}

template <class T>
__global__ void add_inplace_kernel(T* __restrict__ y, const T* __restrict__ x, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] = F<T>::st(F<T>::ld(y[i]) + F<T>::ld(x[i]));
}
__global__ void add_inplace_i32_kernel(unsigned int* __restrict__ y, const unsigned int* __restrict__ x, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] += x[i];
}

// 32 x 32 tiled strided copy through shared memory: coalesced on both sides whichever stride is the unit one.
template <class T>
__global__ void copy_strided_kernel(T* __restrict__ dst, const T* __restrict__ src, long long rows, long long cols,
                                    long long sbs, long long srs, long long scs) {
    __shared__ T tile[32][33];
    const long long b = blockIdx.z;
    const long long r0 = (long long)blockIdx.y * 32, c0 = (long long)blockIdx.x * 32;
    const T* s = src + b * sbs;
    T* d = dst + b * rows * cols;
    if (scs == 1 || srs != 1) {
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + j, c = c0 + threadIdx.x;
            if (r < rows && c < cols) tile[j][threadIdx.x] = s[r * srs + c * scs];
        }
    } else {  // rows are the unit-stride direction of the source: read along rows
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + threadIdx.x, c = c0 + j;
            if (r < rows && c < cols) tile[threadIdx.x][j] = s[r * srs + c * scs];
        }
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const long long r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) d[r * cols + c] = tile[j][threadIdx.x];
    }
}

// Rows that are contiguous in the source (unit column stride): plain 16-byte row copies, coalesced on both sides.
// dst is dense [batch][rows][cols]; one grid-stride loop over all 16-byte vectors.
__global__ void copy_rows_kernel(uint4* __restrict__ dst, const unsigned char* __restrict__ src, long long total_vec,
                                 long long rows, long long vec_per_row, long long batch_stride_bytes, long long row_stride_bytes) {
    for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total_vec; v += (long long)gridDim.x * blockDim.x) {
        const long long c = v % vec_per_row, t = v / vec_per_row;
        const long long r = t % rows, b = t / rows;
        dst[v] = *reinterpret_cast<const uint4*>(src + b * batch_stride_bytes + r * row_stride_bytes + c * 16);
    }
}

template <class D, class S>
__global__ void convert_kernel(D* __restrict__ dst, const S* __restrict__ src, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = F<D>::st(F<S>::ld(src[i]));
}

bool geom(ConvGeom* g, int64_t batch, int64_t channels, int64_t height, int64_t width, int64_t kh, int64_t kw, int64_t sh,
          int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    if (batch < 0 || channels < 0 || height <= 0 || width <= 0 || kh <= 0 || kw <= 0 || sh < 1 || sw < 1 || ph < 0 ||
        pw < 0 || dh < 1 || dw < 1)
        return false;
    *g = ConvGeom{batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw, 0, 0};
    g->hc = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    g->wc = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    return g->hc > 0 && g->wc > 0;
}

#define NTB200_FLOAT_SWITCH(dtype, CALL)                                   \
    switch (dtype) {                                                       \
        case NTB200_F32: { using T = float; CALL; break; }                 \
        case NTB200_F16: { using T = __half; CALL; break; }                \
        case NTB200_BF16: { using T = __nv_bfloat16; CALL; break; }        \
        default: return fail(NTB200_ERR_UNSUPPORTED, "%s: dtype %s is not a float type of this engine", __func__, dtype_name(dtype)); \
    }

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

int ntb200_im2col(int dtype, const void* im, void* col, int64_t batch, int64_t channels, int64_t height, int64_t width,
                  int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw,
                  void* stream) {
    ConvGeom g;
    if (!geom(&g, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw))
        return fail(NTB200_ERR_INVALID_ARG, "im2col: bad geometry (calculated sliding-block shape must be at least one)");
    const long long total = g.batch * g.channels * g.kh * g.kw * g.hc * g.wc;
    if (total == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "im2col: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype_size(dtype)) {
        case 1: launch_im2col<uint8_t>(im, col, g, s); break;
        case 2: launch_im2col<uint16_t>(im, col, g, s); break;
        case 4: launch_im2col<uint32_t>(im, col, g, s); break;
        case 8: launch_im2col<unsigned long long>(im, col, g, s); break;
        default: return fail(NTB200_ERR_UNSUPPORTED, "im2col: unknown dtype %d", dtype);
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_col2im(int dtype, const void* col, void* im, int64_t batch, int64_t channels, int64_t height, int64_t width,
                  int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw,
                  void* stream) {
    ConvGeom g;
    if (!geom(&g, batch, channels, height, width, kh, kw, sh, sw, ph, pw, dh, dw))
        return fail(NTB200_ERR_INVALID_ARG, "col2im: bad geometry");
    const long long total = g.batch * g.channels * g.height * g.width;
    if (total == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "col2im: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(total, 256);
    NTB200_FLOAT_SWITCH(dtype, (col2im_kernel<T><<<blocks, 256, 0, s>>>((const T*)col, (T*)im, g)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_relu(int dtype, const void* x, void* y, int64_t n, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "relu: negative size");
    if (n == 0) return NTB200_OK;
    if (!x || !y) return fail(NTB200_ERR_INVALID_ARG, "relu: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(n, 1024);
    if (vec_ok(n, int(dtype_size(dtype)), x, y)) {
        const long long nvec = n / (16 / (long long)dtype_size(dtype));
        const int vb = grid_for(nvec, 256);
        NTB200_FLOAT_SWITCH(dtype, (relu_vec_kernel<T><<<vb, 256, 0, s>>>((const uint4*)x, (uint4*)y, nvec)));
    } else {
        NTB200_FLOAT_SWITCH(dtype, (relu_kernel<T><<<blocks, 256, 0, s>>>((const T*)x, (T*)y, n)));
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_relu_backward(int dtype, const void* x, const void* grad_out, void* grad_in, int64_t n, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "relu_backward: negative size");
    if (n == 0) return NTB200_OK;
    if (!x || !grad_out || !grad_in) return fail(NTB200_ERR_INVALID_ARG, "relu_backward: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(n, 1024);
    if (vec_ok(n, int(dtype_size(dtype)), x, grad_out, grad_in)) {
        const long long nvec = n / (16 / (long long)dtype_size(dtype));
        const int vb = grid_for(nvec, 256);
        NTB200_FLOAT_SWITCH(dtype, (relu_backward_vec_kernel<T><<<vb, 256, 0, s>>>((const uint4*)x, (const uint4*)grad_out, (uint4*)grad_in, nvec)));
    } else {
        NTB200_FLOAT_SWITCH(dtype, (relu_backward_kernel<T><<<blocks, 256, 0, s>>>((const T*)x, (const T*)grad_out, (T*)grad_in, n)));
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_mse(int dtype, const void* out, const void* target, void* grad, float* loss, int64_t n, void* stream) {
    if (n <= 0) return fail(NTB200_ERR_INVALID_ARG, "mse: size must be positive");
    if (!out || !target || !loss) return fail(NTB200_ERR_INVALID_ARG, "mse: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NTB200_CUDA(cudaMemsetAsync(loss, 0, sizeof(float), s));
    const int blocks = grid_for(n, 2048);
    const float inv_n = 1.0f / float(n);
    NTB200_FLOAT_SWITCH(dtype, (mse_kernel<T><<<blocks, 256, 0, s>>>((const T*)out, (const T*)target, (T*)grad, loss, n, inv_n)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_mse_grad_block(int dtype, const void* out, int64_t out_row_stride, const void* target, int64_t target_row_stride,
                          void* grad, int64_t grad_row_stride, int64_t rows, int64_t cols, int64_t n_total, void* stream) {
    if (rows < 0 || cols < 0 || n_total <= 0) return fail(NTB200_ERR_INVALID_ARG, "mse_grad_block: bad size");
    if (rows == 0 || cols == 0) return NTB200_OK;
    if (!out || !target || !grad) return fail(NTB200_ERR_INVALID_ARG, "mse_grad_block: null pointer");
    if (out_row_stride < cols || target_row_stride < cols || grad_row_stride < cols)
        return fail(NTB200_ERR_INVALID_ARG, "mse_grad_block: a row stride is shorter than the block's rows");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(rows * cols, 2048);
    const float inv_n = 1.0f / float(n_total);
    NTB200_FLOAT_SWITCH(dtype, (mse_grad_block_kernel<T><<<blocks, 256, 0, s>>>((const T*)out, out_row_stride, (const T*)target, target_row_stride,
                                                                               (T*)grad, grad_row_stride, rows, cols, inv_n)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_column_sum(int dtype, const void* grad, void* out, int64_t rows, int64_t cols, void* stream) {
    if (rows < 0 || cols < 0) return fail(NTB200_ERR_INVALID_ARG, "column_sum: negative size");
    if (cols == 0) return NTB200_OK;
    if (!grad || !out) return fail(NTB200_ERR_INVALID_ARG, "column_sum: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Large 16-bit matrices (bias gradients of wide layers): two passes with 16-byte loads and the rows spread
    // over enough blocks to fill the GPU.
    if (dtype_size(dtype) == 2 && cols % 8 == 0 && reinterpret_cast<uintptr_t>(grad) % 16 == 0 && rows * cols >= (int64_t(1) << 22)) {
        const int64_t col_blocks = (cols + 255) / 256;
        int64_t slabs = std::max<int64_t>(1, std::min<int64_t>((rows + 63) / 64, (int64_t(sm_count()) * 8 + col_blocks - 1) / col_blocks));
        slabs = std::min<int64_t>(slabs, 65535);
        const int64_t rows_per_slab = (rows + slabs - 1) / slabs;
        slabs = (rows + rows_per_slab - 1) / rows_per_slab;
        float* partial = nullptr;
        if (int rc = scratch_acquire(reinterpret_cast<void**>(&partial), size_t(slabs) * size_t(cols) * sizeof(float), s)) return rc;
        const dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(slabs), 1);
        const dim3 block(32, 8, 1);
        cudaError_t e = cudaSuccess;
        if (dtype == NTB200_F16) {
            column_sum_partial_kernel<__half><<<grid, block, 0, s>>>((const __half*)grad, partial, rows, cols, rows_per_slab);
            column_sum_final_kernel<__half><<<unsigned((cols + 255) / 256), 256, 0, s>>>(partial, (__half*)out, int(slabs), cols);
        } else {
            column_sum_partial_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16*)grad, partial, rows, cols, rows_per_slab);
            column_sum_final_kernel<__nv_bfloat16><<<unsigned((cols + 255) / 256), 256, 0, s>>>(partial, (__nv_bfloat16*)out, int(slabs), cols);
        }
        e = cudaGetLastError();
        scratch_release(partial, s);
        count_launch(2);
        if (e != cudaSuccess) return cuda_fail(e, "column_sum kernels");
        return NTB200_OK;
    }
    const dim3 block(32, 32);
    const unsigned blocks = unsigned((cols + 31) / 32);
    NTB200_FLOAT_SWITCH(dtype, (column_sum_kernel<T><<<blocks, block, 0, s>>>((const T*)grad, (T*)out, rows, cols)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_add_inplace(int dtype, void* y, const void* x, int64_t n, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "add_inplace: negative size");
    if (n == 0) return NTB200_OK;
    if (!x || !y) return fail(NTB200_ERR_INVALID_ARG, "add_inplace: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(n, 1024);
    if (dtype == NTB200_I32 || dtype == NTB200_U32) {
        add_inplace_i32_kernel<<<blocks, 256, 0, s>>>((unsigned int*)y, (const unsigned int*)x, n);
    } else {
        if (vec_ok(n, int(dtype_size(dtype)), x, y)) {
            const long long nvec = n / (16 / (long long)dtype_size(dtype));
            const int vb = grid_for(nvec, 256);
            NTB200_FLOAT_SWITCH(dtype, (add_inplace_vec_kernel<T><<<vb, 256, 0, s>>>((uint4*)y, (const uint4*)x, nvec)));
        } else {
            NTB200_FLOAT_SWITCH(dtype, (add_inplace_kernel<T><<<blocks, 256, 0, s>>>((T*)y, (const T*)x, n)));
        }
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_copy_strided_2d(int dtype, void* dst, const void* src, int64_t batch, int64_t rows, int64_t cols,
                           int64_t src_batch_stride, int64_t src_row_stride, int64_t src_col_stride, void* stream) {
    if (batch < 0 || rows < 0 || cols < 0) return fail(NTB200_ERR_INVALID_ARG, "copy_strided_2d: negative size");
    if (batch == 0 || rows == 0 || cols == 0) return NTB200_OK;
    if (!dst || !src) return fail(NTB200_ERR_INVALID_ARG, "copy_strided_2d: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long es = (long long)dtype_size(dtype);
    if (es && src_col_stride == 1 && (cols * es) % 16 == 0 && (src_row_stride * es) % 16 == 0 && (src_batch_stride * es) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(dst) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0) {
        const long long vpr = cols * es / 16, total_vec = batch * rows * vpr;
        copy_rows_kernel<<<grid_for(total_vec, 256), 256, 0, s>>>(static_cast<uint4*>(dst), static_cast<const unsigned char*>(src),
                                                                 total_vec, rows, vpr, src_batch_stride * es, src_row_stride * es);
        count_launch();
        NTB200_CUDA(cudaGetLastError());
        return NTB200_OK;
    }
    if (batch > 65535 || (rows + 31) / 32 > 65535) return fail(NTB200_ERR_UNSUPPORTED, "copy_strided_2d: too many tiles");
    const dim3 grid(unsigned((cols + 31) / 32), unsigned((rows + 31) / 32), unsigned(batch));
    const dim3 block(32, 8);
    switch (dtype_size(dtype)) {
        case 1: copy_strided_kernel<uint8_t><<<grid, block, 0, s>>>((uint8_t*)dst, (const uint8_t*)src, rows, cols, src_batch_stride, src_row_stride, src_col_stride); break;
        case 2: copy_strided_kernel<uint16_t><<<grid, block, 0, s>>>((uint16_t*)dst, (const uint16_t*)src, rows, cols, src_batch_stride, src_row_stride, src_col_stride); break;
        case 4: copy_strided_kernel<uint32_t><<<grid, block, 0, s>>>((uint32_t*)dst, (const uint32_t*)src, rows, cols, src_batch_stride, src_row_stride, src_col_stride); break;
        case 8: copy_strided_kernel<unsigned long long><<<grid, block, 0, s>>>((unsigned long long*)dst, (const unsigned long long*)src, rows, cols, src_batch_stride, src_row_stride, src_col_stride); break;
        default: return fail(NTB200_ERR_UNSUPPORTED, "copy_strided_2d: unknown dtype %d", dtype);
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_bias_add_channels(int dtype, void* x, const void* bias, int64_t batch, int64_t channels, int64_t inner, void* stream) {
    if (batch < 0 || channels <= 0 || inner < 0) return fail(NTB200_ERR_INVALID_ARG, "bias_add_channels: bad extent");
    const int64_t total = batch * channels * inner;
    if (total == 0) return NTB200_OK;
    if (!x || !bias) return fail(NTB200_ERR_INVALID_ARG, "bias_add_channels: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t per = 16 / int64_t(dtype_size(dtype) ? dtype_size(dtype) : 16);
    if ((dtype == NTB200_F32 || dtype == NTB200_F16 || dtype == NTB200_BF16) && inner % per == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        const int64_t nvec = total / per;
        NTB200_FLOAT_SWITCH(dtype, (bias_add_channels_vec_kernel<T><<<grid_for(nvec, 256), 256, 0, s>>>((uint4*)x, (const T*)bias, nvec, channels, inner / per)));
    } else {
        NTB200_FLOAT_SWITCH(dtype, (bias_add_channels_kernel<T><<<grid_for(total, 1024), 256, 0, s>>>((T*)x, (const T*)bias, total, channels, inner)));
    }
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_sum_channels(int dtype, const void* grad, void* out, int64_t batch, int64_t channels, int64_t inner, void* stream) {
    if (batch < 0 || channels <= 0 || inner < 0) return fail(NTB200_ERR_INVALID_ARG, "sum_channels: bad extent");
    if (!grad || !out) return fail(NTB200_ERR_INVALID_ARG, "sum_channels: null pointer");
    if (channels > 2147483647) return fail(NTB200_ERR_INVALID_ARG, "sum_channels: too many channels");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NTB200_FLOAT_SWITCH(dtype, (sum_channels_kernel<T><<<unsigned(channels), 256, 0, s>>>((const T*)grad, (T*)out, batch, channels, inner)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_convert(int dst_dtype, void* dst, int src_dtype, const void* src, int64_t n, void* stream) {
    if (n < 0) return fail(NTB200_ERR_INVALID_ARG, "convert: negative size");
    if (n == 0) return NTB200_OK;
    if (!dst || !src) return fail(NTB200_ERR_INVALID_ARG, "convert: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = grid_for(n, 1024);
#define NTB200_CVT(DT, ST, D, S) \
    if (dst_dtype == DT && src_dtype == ST) { convert_kernel<D, S><<<blocks, 256, 0, s>>>((D*)dst, (const S*)src, n); } else
    NTB200_CVT(NTB200_F32, NTB200_F16, float, __half)
    NTB200_CVT(NTB200_F32, NTB200_BF16, float, __nv_bfloat16)
    NTB200_CVT(NTB200_F16, NTB200_F32, __half, float)
    NTB200_CVT(NTB200_BF16, NTB200_F32, __nv_bfloat16, float)
    NTB200_CVT(NTB200_F16, NTB200_BF16, __half, __nv_bfloat16)
    NTB200_CVT(NTB200_BF16, NTB200_F16, __nv_bfloat16, __half)
    NTB200_CVT(NTB200_F32, NTB200_F32, float, float)
    NTB200_CVT(NTB200_F16, NTB200_F16, __half, __half)
    NTB200_CVT(NTB200_BF16, NTB200_BF16, __nv_bfloat16, __nv_bfloat16)
    { return fail(NTB200_ERR_UNSUPPORTED, "convert: %s -> %s is not supported", dtype_name(src_dtype), dtype_name(dst_dtype)); }
#undef NTB200_CVT
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

}  // extern "C"
