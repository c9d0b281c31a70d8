// conv3d, forward and backward, with groups (nt/functional/tensor_files/conv.cpp:122-174 forward; conv_dimage /
// conv_dkernel dim == 3 cases; unfold3d / unfold3d_backward in colim_transform.cpp:661-800 and
// nt/functional/cpu/unfold3d.cpp).
//
// Same structure as the 2-D case: the column matrix col[b][(c, kz, ky, kx)][(z, y, x)] is written once
// (im2col3d_kernel), every group is one batched GEMM on offset pointers, and the image gradient gathers the
// gradient column matrix back (col2im3d_kernel: one thread per image element sums the taps that reach it, so there
// are no atomics and the result is deterministic).  conv_transpose3d is the image-gradient call with the input in
// the place of the gradient.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace ntb200 {
namespace {

struct Geo3 {
    long long batch, channels, depth, height, width;
    long long kd, kh, kw, sd, sh, sw, pd, ph, pw, dd, dh, dw;
    long long od, oh, ow;     // output extent
    long long L, taps, ck;    // od*oh*ow, kd*kh*kw, channels*taps
};

inline size_t round256(size_t v) { return (v + 255u) & ~size_t(255); }

template <typename T>
__global__ void im2col3d_kernel(const T* __restrict__ im, T* __restrict__ col, Geo3 g, long long total) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long l = idx % g.L;
        long long r = idx / g.L;
        const long long row = r % g.ck;
        const long long b = r / g.ck;
        const long long x = l % g.ow, y = (l / g.ow) % g.oh, z = l / (g.ow * g.oh);
        const long long kx = row % g.kw, ky = (row / g.kw) % g.kh, kz = (row / (g.kw * g.kh)) % g.kd, c = row / g.taps;
        const long long iz = z * g.sd - g.pd + kz * g.dd, iy = y * g.sh - g.ph + ky * g.dh, ix = x * g.sw - g.pw + kx * g.dw;
        T v = T(0);
        if (iz >= 0 && iz < g.depth && iy >= 0 && iy < g.height && ix >= 0 && ix < g.width)
            v = im[(((b * g.channels + c) * g.depth + iz) * g.height + iy) * g.width + ix];
        col[idx] = v;
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

// im[b][c][iz][iy][ix] = sum over the taps (kz, ky, kx) and output positions (z, y, x) with
// z*sd - pd + kz*dd == iz (and likewise for y, x) of col[b][(c, kz, ky, kx)][(z, y, x)]; taps in ascending order.
template <typename T>
__global__ void col2im3d_kernel(const T* __restrict__ col, T* __restrict__ im, Geo3 g, long long total) {
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long ix = idx % g.width, iy = (idx / g.width) % g.height, iz = (idx / (g.width * g.height)) % g.depth;
        const long long c = (idx / (g.width * g.height * g.depth)) % g.channels, b = idx / (g.width * g.height * g.depth * g.channels);
        float acc = 0.f;
        for (long long kz = 0; kz < g.kd; ++kz) {
            const long long tz = iz + g.pd - kz * g.dd;
            if (tz < 0 || tz % g.sd) continue;
            const long long z = tz / g.sd;
            if (z >= g.od) continue;
            for (long long ky = 0; ky < g.kh; ++ky) {
                const long long ty = iy + g.ph - ky * g.dh;
                if (ty < 0 || ty % g.sh) continue;
                const long long y = ty / g.sh;
                if (y >= g.oh) continue;
                for (long long kx = 0; kx < g.kw; ++kx) {
                    const long long tx = ix + g.pw - kx * g.dw;
                    if (tx < 0 || tx % g.sw) continue;
                    const long long x = tx / g.sw;
                    if (x >= g.ow) continue;
                    const long long row = ((c * g.kd + kz) * g.kh + ky) * g.kw + kx;
                    acc += as_float(col[(b * g.ck + row) * g.L + (z * g.oh + y) * g.ow + x]);
                }
            }
        }
        im[idx] = from_float<T>(acc);
    }
}

int make_geo(const char* who, const ntb200_conv3d_geom* q, Geo3* g) {
    if (!q) return fail(NTB200_ERR_INVALID_ARG, "%s: null geometry", who);
    if (q->stride[0] < 1 || q->stride[1] < 1 || q->stride[2] < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv3d stride cannot be less than 1");
    if (q->dilation[0] < 1 || q->dilation[1] < 1 || q->dilation[2] < 1) return fail(NTB200_ERR_INVALID_ARG, "Conv3d dilation cannot be less than 1");
    if (q->padding[0] < 0 || q->padding[1] < 0 || q->padding[2] < 0) return fail(NTB200_ERR_INVALID_ARG, "Conv3d padding cannot be less than 0");
    if (q->batch < 0 || q->channels <= 0 || q->depth <= 0 || q->height <= 0 || q->width <= 0 || q->kernel[0] <= 0 ||
        q->kernel[1] <= 0 || q->kernel[2] <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    g->batch = q->batch; g->channels = q->channels; g->depth = q->depth; g->height = q->height; g->width = q->width;
    g->kd = q->kernel[0]; g->kh = q->kernel[1]; g->kw = q->kernel[2];
    g->sd = q->stride[0]; g->sh = q->stride[1]; g->sw = q->stride[2];
    g->pd = q->padding[0]; g->ph = q->padding[1]; g->pw = q->padding[2];
    g->dd = q->dilation[0]; g->dh = q->dilation[1]; g->dw = q->dilation[2];
    g->od = (g->depth + 2 * g->pd - g->dd * (g->kd - 1) - 1) / g->sd + 1;
    g->oh = (g->height + 2 * g->ph - g->dh * (g->kh - 1) - 1) / g->sh + 1;
    g->ow = (g->width + 2 * g->pw - g->dw * (g->kw - 1) - 1) / g->sw + 1;
    if (g->od <= 0 || g->oh <= 0 || g->ow <= 0)
        return fail(NTB200_ERR_INVALID_ARG, "%s: calculated output size (%lld, %lld, %lld) must be at least one", who, g->od, g->oh, g->ow);
    g->L = g->od * g->oh * g->ow;
    g->taps = g->kd * g->kh * g->kw;
    g->ck = g->channels * g->taps;
    return NTB200_OK;
}

int check_groups(const char* who, const ntb200_conv3d_geom* q) {
    if (q->groups < 1) return fail(NTB200_ERR_INVALID_ARG, "Expected groups for a convolution to be greater than 0 but got %lld", (long long)q->groups);
    if (q->cout <= 0) return fail(NTB200_ERR_INVALID_ARG, "%s: bad extent", who);
    if (q->channels % q->groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected image channels to be divisible by groups in Conv3d but got %lld %% %lld != 0",
                    (long long)q->channels, (long long)q->groups);
    if (q->cout % q->groups)
        return fail(NTB200_ERR_INVALID_ARG, "Expected kernel filters to be divisible by groups in Conv3d but got %lld %% %lld != 0",
                    (long long)q->cout, (long long)q->groups);
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

int ntb200_im2col3d(int dtype, const void* im, void* col, const ntb200_conv3d_geom* geom, void* stream) {
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(NTB200_ERR_UNSUPPORTED, "im2col3d: unknown dtype %d", dtype);
    Geo3 g;
    if (int rc = make_geo("im2col3d", geom, &g)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "im2col3d: null pointer");
    const long long total = g.batch * g.ck * g.L;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // a pure copy: elements are moved as raw words of their size
    NTB200_SIZE_SWITCH(es, (im2col3d_kernel<T><<<grid_for_total(total), 256, 0, s>>>(static_cast<const T*>(im), static_cast<T*>(col), g, total)));
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_col2im3d(int dtype, const void* col, void* im, const ntb200_conv3d_geom* geom, void* stream) {
    if (!float_dtype(dtype)) return fail(NTB200_ERR_UNSUPPORTED, "col2im3d: Float32, Float16 and BFloat16 only (got %s)", dtype_name(dtype));
    Geo3 g;
    if (int rc = make_geo("col2im3d", geom, &g)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!im || !col) return fail(NTB200_ERR_INVALID_ARG, "col2im3d: null pointer");
    const long long total = g.batch * g.channels * g.depth * g.height * g.width;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = grid_for_total(total);
    if (dtype == NTB200_F32) col2im3d_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(col), static_cast<float*>(im), g, total);
    else if (dtype == NTB200_F16) col2im3d_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(col), static_cast<__half*>(im), g, total);
    else col2im3d_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(col), static_cast<__nv_bfloat16*>(im), g, total);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

size_t ntb200_conv3d_workspace_bytes(int dtype, const ntb200_conv3d_geom* geom) {
    const size_t es = dtype_size(dtype);
    Geo3 g;
    if (es == 0 || !geom || geom->groups < 1 || geom->cout <= 0 || make_geo("conv3d", geom, &g) != NTB200_OK) return 0;
    if (geom->channels % geom->groups || geom->cout % geom->groups) return 0;
    // column matrix + the per-image kernel gradients [B, Cout, (C/groups)*taps] + their batch sum (accumulate)
    return round256(size_t(g.batch) * size_t(g.ck) * size_t(g.L) * es) +
           round256(size_t(g.batch) * size_t(geom->cout) * size_t(g.ck / geom->groups) * es) +
           size_t(geom->cout) * size_t(g.ck / geom->groups) * es;
}

int ntb200_conv3d(int dtype, const void* x, const void* w, void* out, void* workspace, const ntb200_conv3d_geom* geom,
                  void* stream) {
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(NTB200_ERR_UNSUPPORTED, "conv3d: unknown dtype %d", dtype);
    Geo3 g;
    if (int rc = make_geo("conv3d", geom, &g)) return rc;
    if (int rc = check_groups("conv3d", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!x || !w || !out || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv3d: null pointer");
    if (int rc = ntb200_im2col3d(dtype, x, workspace, geom, stream)) return rc;
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

int ntb200_conv3d_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 const ntb200_conv3d_geom* geom, void* stream) {
    if (!float_dtype(dtype))
        return fail(NTB200_ERR_UNSUPPORTED, "conv3d_backward_image: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    const size_t es = dtype_size(dtype);
    Geo3 g;
    if (int rc = make_geo("conv3d_backward_image", geom, &g)) return rc;
    if (int rc = check_groups("conv3d_backward_image", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!grad || !w || !d_image || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv3d_backward_image: null pointer");
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
    return ntb200_col2im3d(dtype, workspace, d_image, geom, stream);
}

int ntb200_conv3d_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace, int accumulate,
                                  const ntb200_conv3d_geom* geom, void* stream) {
    if (!float_dtype(dtype))
        return fail(NTB200_ERR_UNSUPPORTED, "conv3d_backward_kernel: gradients are computed for Float32, Float16 and BFloat16 (got %s)",
                    dtype_name(dtype));
    const size_t es = dtype_size(dtype);
    Geo3 g;
    if (int rc = make_geo("conv3d_backward_kernel", geom, &g)) return rc;
    if (int rc = check_groups("conv3d_backward_kernel", geom)) return rc;
    if (g.batch == 0) return NTB200_OK;
    if (!x || !grad || !d_kernel || !workspace) return fail(NTB200_ERR_INVALID_ARG, "conv3d_backward_kernel: null pointer");
    const long long groups = geom->groups, coutg = geom->cout / groups, ckg = g.ck / groups;
    void* col = workspace;
    void* per_image = at(workspace, 0, es) + round256(size_t(g.batch) * size_t(g.ck) * size_t(g.L) * es);
    if (int rc = ntb200_im2col3d(dtype, x, col, geom, stream)) return rc;
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
