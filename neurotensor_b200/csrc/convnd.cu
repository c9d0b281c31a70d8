// convnd / conv_transposend for any number of spatial dimensions (nt/functional/tensor_files/conv.cpp:177-262 forward,
// :747-860 transposed; unfoldnd / unfoldnd_backward in nt/functional/cpu/unfoldnd.cpp and unfoldnd_backward.cpp).
//
// The reference's N-D convolution is the same chain as its 1-, 2- and 3-D ones: unfoldnd writes the column matrix
// col[b][(c, k_0 .. k_{N-1})][(o_0 .. o_{N-1})], every group is one matmult(col_g, w_g, true, true) and the result is
// swapped back to channel-major.  Here the column matrix is written once by im2colnd_kernel (mixed-radix decode of
// the row and the output position, extents in a by-value struct), every group is one batched GEMM on offset
// pointers, and the image gradient gathers the gradient column matrix back (col2imnd_kernel: one thread per image
// element sums the taps that reach it in ascending tap order: no atomics, deterministic).  conv_transposend is the
// image-gradient call with the input in the place of the gradient.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace ntb200 {
namespace {

constexpr int MAXD = NTB200_CONVND_MAX_DIMS;

struct GeoN {
    int dims;
    long long batch, channels;
    long long size[MAXD], k[MAXD], s[MAXD], p[MAXD], d[MAXD], o[MAXD];
    long long L, taps, ck, volume;   // prod(o), prod(k), channels*taps, prod(size)
};

inline size_t round256(size_t v) { return (v + 255u) & ~size_t(255); }

template <typename T>
__global__ void im2colnd_kernel(const T* __restrict__ im, T* __restrict__ col, const GeoN g, long long total) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        long long l = idx % g.L;
        long long r = idx / g.L;
        long long row = r % g.ck;
        const long long b = r / g.ck;
        const long long c = row / g.taps;
        long long tap = row % g.taps;
        long long off = 0, scale = 1;
        bool inside = true;
        for (int i = g.dims - 1; i >= 0; --i) {   // innermost dimension first
            const long long oi = l % g.o[i]; l /= g.o[i];
            const long long ki = tap % g.k[i]; tap /= g.k[i];
            const long long xi = oi * g.s[i] - g.p[i] + ki * g.d[i];
            inside = inside && xi >= 0 && xi < g.size[i];
            off += xi * scale;
            scale *= g.size[i];
        }
        col[idx] = inside ? im[(b * g.channels + c) * g.volume + off] : T(0);
    }
}

template <typename T> __device__ __forceinline__ float as_float(T v);
template <> __device__ __forceinline__ float as_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// im[b][c][x_0 .. x_{N-1}] = sum over the taps k and output positions o with o_i*s_i - p_i + k_i*d_i == x_i for every i
// of col[b][(c, k)][o]; taps in ascending order of their flattened index.
template <typename T>
__global__ void col2imnd_kernel(const T* __restrict__ col, T* __restrict__ im, const GeoN g, long long total) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        long long x[MAXD];
        long long r = idx;
        for (int i = g.dims - 1; i >= 0; --i) { x[i] = r % g.size[i]; r /= g.size[i]; }
        const long long c = r % g.channels, b = r / g.channels;
        float acc = 0.f;
        for (long long tap = 0; tap < g.taps; ++tap) {
            long long t = tap, l = 0, scale = 1;
            bool hit = true;
            for (int i = g.dims - 1; i >= 0 && hit; --i) {
                const long long ki = t % g.k[i]; t /= g.k[i];
                const long long ti = x[i] + g.p[i] - ki * g.d[i];
                if (ti < 0 || ti % g.s[i]) { hit = false; break; }
                const long long oi = ti / g.s[i];
                if (oi >= g.o[i]) { hit = false; break; }
                l += oi * scale;
                scale *= g.o[i];
            }
            if (hit) acc += as_float(col[(b * g.ck + c * g.taps + tap) * g.L + l]);
        }
        im[idx] = from_float<T>(acc);
    }
}

int make_geo(const char* who, const ntb200_convnd_geom* q, GeoN* g) {
    if (!q) return fail(NTB200_ERR_INVALID_ARG, "%s: null geometry", who);
    if (q->dims < 1) return fail(NTB200_ERR_INVALID_ARG, "Error, cannot do a dynamic ConvND where N < 0 got (N = %lld)", (long long)q->dims);
    if (q->dims > MAXD) return fail(NTB200_ERR_UNSUPPORTED, "%s: at most %d spatial dimensions (got %lld)", who, MAXD, (long long)q->dims);
    g->dims = int(q->dims);
    if (q->batch < 0 || q->channels <= 0) return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    g->batch = q->batch; g->channels = q->channels;
    g->L = g->taps = g->volume = 1;
    for (int i = 0; i < g->dims; ++i) {
        if (q->stride[i] < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv%dD stride cannot be less than 1", g->dims);
        if (q->dilation[i] < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv%dD dilation cannot be less than 1", g->dims);
        if (q->padding[i] < 0) return fail(NTB200_ERR_INVALID_ARG, "Conv%dD padding cannot be less than 0", g->dims);
        if (q->size[i] <= 0 || q->kernel[i] <= 0) return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
        g->size[i] = q->size[i]; g->k[i] = q->kernel[i]; g->s[i] = q->stride[i]; g->p[i] = q->padding[i]; g->d[i] = q->dilation[i];
        g->o[i] = (g->size[i] + 2 * g->p[i] - g->d[i] * (g->k[i] - 1) - 1) / g->s[i] + 1;
        if (g->o[i] <= 0)
            return fail(NTB200_ERR_INVALID_ARG, "%s: calculated output size %lld of dimension %d must be at least one", who, g->o[i], i);
        g->L *= g->o[i]; g->taps *= g->k[i]; g->volume *= g->size[i];
    }
    for (int i = g->dims; i < MAXD; ++i) { g->size[i] = g->k[i] = g->s[i] = g->d[i] = g->o[i] = 1; g->p[i] = 0; }
    g->ck = g->channels * g->taps;
    return NTB200_OK;
}

int check_groups(const char* who, const ntb200_convnd_geom* q) {
    if (q->groups < 1) return fail(NTB200_ERR_INVALID_ARG, "Expected groups for a convolution to be greater than 0 but got %lld", (long long)q->groups);
    if (q->cout <= 0) return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    if (q->channels % q->groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected image channels to be divisible by groups in Conv%lldd but got %lld %% %lld != 0",
                    (long long)q->dims, (long long)q->channels, (long long)q->groups);
    if (q->cout % q->groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected kernel filters to be divisible by groups in Conv%lldd but got %lld %% %lld != 0",
                    (long long)q->dims, (long long)q->cout, (long long)q->groups);
    return NTB200_OK;
}

int grid_for_total(long long total) {
    const long long blocks = (total + 255) / 256, cap = (long long)sm_count() * 32;
    return int(std::max<long long>(1, std::min(blocks, cap)));
}

inline const char* at(const void* p, long long elements, size_t es) { return static_cast<const char*>(p) + size_t(elements) * es; }
inline char* at(void* p, long long elements, size_t es) { return static_cast<char*>(p) + size_t(elements) * es; }

bool float_dtype(int dtype) { return dtype == NTB200_F32 || dtype == NTB200_F16 || dtype == NTB200_BF16; }

}  // namespace
}  // namespace ntb200

using namespace ntb200;

#define NTB200_SIZE_SWITCH(es, CALL)                                   \
    switch (es) {                                                      \
        case 1: { using T = uint8_t; CALL; break; }                    \
        case 2: { using T = uint16_t; CALL; break; }                   \
        case 4: { using T = uint32_t; CALL; break; }                   \
        case 8: { using T = unsigned long long; CALL; break; }         \
        default: return fail(NTB200_ERR_UNSUPPORTED, "column matrix: elements of 1, 2, 4 or 8 bytes (got %d)", int(es)); \
    }

extern "C" {

int ntb200_im2colnd(int dtype, const void* im, void* col, const ntb200_convnd_geom* geom, void* stream) {
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(NTB200_ERR_UNSUPPORTED, "im2colnd: unknown dtype %d", dtype);
    GeoN g;
    if (int rc = make_geo("im2colnd", geom, &g)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "im2colnd: null pointer");
    const long long total = g.batch * g.ck * g.L;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // a pure copy: elements are moved as raw words of their size
    NTB200_SIZE_SWITCH(es, (im2colnd_kernel<T><<<grid_for_total(total), 256, 0, s>>>(static_cast<const T*>(im), static_cast<T*>(col), g, total)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_col2imnd(int dtype, const void* col, void* im, const ntb200_convnd_geom* geom, void* stream) {
    if (!float_dtype(dtype)) return fail(NTB200_ERR_UNSUPPORTED, "col2imnd: Float32, Float16 and BFloat16 only (got %s)", dtype_name(dtype));
    GeoN g;
    if (int rc = make_geo("col2imnd", geom, &g)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "col2imnd: null pointer");
    const long long total = g.batch * g.channels * g.volume;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for_total(total);
    if (dtype == NTB200_F32) col2imnd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(col), static_cast<float*>(im), g, total);
    else if (dtype == NTB200_F16) col2imnd_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(col), static_cast<__half*>(im), g, total);
    else col2imnd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(col), static_cast<__nv_bfloat16*>(im), g, total);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

size_t ntb200_convnd_workspace_bytes(int dtype, const ntb200_convnd_geom* geom) {
    const size_t es = dtype_size(dtype);
    GeoN g;
    if (es == 0 || !geom || geom->groups < 1 || geom->cout <= 0 || make_geo("convnd", geom, &g) != NTB200_OK) return 0;
    if (geom->channels % geom->groups || geom->cout % geom->groups) return 0;
    // column matrix + the per-image kernel gradients [B, Cout, (C/groups)*taps] + their batch sum (accumulate)
    return round256(size_t(g.batch) * size_t(g.ck) * size_t(g.L) * es) +
           round256(size_t(g.batch) * size_t(geom->cout) * size_t(g.ck / geom->groups) * es) +
           size_t(geom->cout) * size_t(g.ck / geom->groups) * es;
}

int ntb200_convnd(int dtype, const void* x, const void* w, void* out, void* workspace, const ntb200_convnd_geom* geom,
                  void* stream) {
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(NTB200_ERR_UNSUPPORTED, "convnd: unknown dtype %d", dtype);
    GeoN g;
    if (int rc = make_geo("convnd", geom, &g)) return rc;
    if (int rc = check_groups("convnd", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!x || !w || !out || !workspace) return fail(NTB200_ERR_INVALID_ARG, "convnd: null pointer");
    if (int rc = ntb200_im2colnd(dtype, x, workspace, geom, stream)) return rc;
    const long long groups = geom->groups, coutg = geom->cout / groups, ckg = g.ck / groups;
    for (long long gi = 0; gi < groups; ++gi) {   // out_g[b] (coutg x L) = w_g (coutg x ckg) . col_g[b] (ckg x L)
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = coutg; a.n = g.L; a.k = ckg; a.batch = g.batch;
        a.a = at(w, gi * coutg * ckg, es); a.a_rs = ckg; a.a_cs = 1; a.a_bs = 0;
        a.b = at(static_cast<const void*>(workspace), gi * ckg * g.L, es); a.b_rs = g.L; a.b_cs = 1; a.b_bs = g.ck * g.L;
        a.c = at(out, gi * coutg * g.L, es); a.c_rs = g.L; a.c_bs = geom->cout * g.L;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    return NTB200_OK;
}

int ntb200_convnd_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 const ntb200_convnd_geom* geom, void* stream) {
    if (!float_dtype(dtype))
        return fail(NTB200_ERR_UNSUPPORTED, "convnd_backward_image: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    const size_t es = dtype_size(dtype);
    GeoN g;
    if (int rc = make_geo("convnd_backward_image", geom, &g)) return rc;
    if (int rc = check_groups("convnd_backward_image", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!grad || !w || !d_image || !workspace) return fail(NTB200_ERR_INVALID_ARG, "convnd_backward_image: null pointer");
    const long long groups = geom->groups, coutg = geom->cout / groups, ckg = g.ck / groups;
    for (long long gi = 0; gi < groups; ++gi) {   // d_col_g[b] (ckg x L) = w_g^T (ckg x coutg) . grad_g[b] (coutg x L)
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = ckg; a.n = g.L; a.k = coutg; a.batch = g.batch;
        a.a = at(w, gi * coutg * ckg, es); a.a_rs = 1; a.a_cs = ckg; a.a_bs = 0;
        a.b = at(grad, gi * coutg * g.L, es); a.b_rs = g.L; a.b_cs = 1; a.b_bs = geom->cout * g.L;
        a.c = at(workspace, gi * ckg * g.L, es); a.c_rs = g.L; a.c_bs = g.ck * g.L;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    return ntb200_col2imnd(dtype, workspace, d_image, geom, stream);
}

int ntb200_convnd_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace, int accumulate,
                                  const ntb200_convnd_geom* geom, void* stream) {
    if (!float_dtype(dtype))
        return fail(NTB200_ERR_UNSUPPORTED, "convnd_backward_kernel: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    const size_t es = dtype_size(dtype);
    GeoN g;
    if (int rc = make_geo("convnd_backward_kernel", geom, &g)) return rc;
    if (int rc = check_groups("convnd_backward_kernel", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!x || !grad || !d_kernel || !workspace) return fail(NTB200_ERR_INVALID_ARG, "convnd_backward_kernel: null pointer");
    const long long groups = geom->groups, coutg = geom->cout / groups, ckg = g.ck / groups;
    void* col = workspace;
    void* per_image = at(workspace, 0, es) + round256(size_t(g.batch) * size_t(g.ck) * size_t(g.L) * es);
    if (int rc = ntb200_im2colnd(dtype, x, col, geom, stream)) return rc;
    const bool direct = g.batch == 1;
    for (long long gi = 0; gi < groups; ++gi) {   // per_image_g[b] (coutg x ckg) = grad_g[b] (coutg x L) . col_g[b]^T
        GemmArgs a{};
        a.dtype = dtype; a.accumulate = direct ? (accumulate != 0) : 0; a.f16_rounding = NTB200_F16_ROUND_ONCE;
        a.m = coutg; a.n = ckg; a.k = g.L; a.batch = g.batch;
        a.a = at(grad, gi * coutg * g.L, es); a.a_rs = g.L; a.a_cs = 1; a.a_bs = geom->cout * g.L;
        a.b = at(static_cast<const void*>(col), gi * ckg * g.L, es); a.b_rs = 1; a.b_cs = g.L; a.b_bs = g.ck * g.L;
        a.c = at(direct ? d_kernel : per_image, gi * coutg * ckg, es); a.c_rs = ckg; a.c_bs = geom->cout * ckg;
        if (int rc = route_gemm(a, NTB200_ROUTE_AUTO, static_cast<cudaStream_t>(stream))) return rc;
    }
    if (direct) return NTB200_OK;
    if (!accumulate) return ntb200_column_sum(dtype, per_image, d_kernel, g.batch, geom->cout * ckg, stream);
    // the batch sum has its own region behind the per-image gradients (it can be larger than the column matrix)
    void* summed = static_cast<char*>(per_image) + round256(size_t(g.batch) * size_t(geom->cout) * size_t(ckg) * es);
    if (int rc = ntb200_column_sum(dtype, per_image, summed, g.batch, geom->cout * ckg, stream)) return rc;
    return ntb200_add_inplace(dtype, d_kernel, summed, geom->cout * ckg, stream);
}

}  // extern "C"
