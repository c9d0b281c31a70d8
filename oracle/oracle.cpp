// TEST INFRASTRUCTURE ONLY -- CPU oracle for the NeuroTensor dense-contraction path.
//
// A from-scratch CPU restatement of the *numerics* of the reference's matmult, used only as the
// checker in tests, in the smoke test and as the timed CPU baseline of the benchmark.  Nothing in
// the shipped library links, loads or calls this file.
//
// Parity status: the Float32 path is pinned against the reference's own committed golden vectors
// (linear_*.npy, conv2d_*.npy, unfold_*.npy from tests/autograd_data, see tests/golden/).  For
// Float16 / integer / BFloat16 results the reference's tests hold no golden vector: "parity
// unpinned" by tests; those paths encode the source semantics cited below.
//
// What is restated (paths are relative to the reference project root):
//   * nt/functional/cpu/matmult/nt_matmult.hpp:124-225   loop nest: for each K tile of TILE = 2 x
//     SIMD pack width, every TILE x TILE output tile is LOADED from C, updated by an ascending-k
//     chain of fmadd, and STORED back to C.  The raw-pointer contract is C += op(A) . op(B) with
//     row-major contiguous operands and post-transpose logical dims (nt_matmult.h:6-10).
//   * nt/functional/cpu/matmult/nt_matmult_simde.hpp:301-350  the microkernel (load C, fmadd, store C).
//   * nt/mp/simde_traits/simde_traits_avx2.h  per-dtype load / fmadd / store:
//       float    (:250-256)   fused multiply-add in fp32, TILE 16
//       double   (:366-368)   fused multiply-add in fp64, TILE 8
//       float16  (:1133-1135 load = cvtph_ps, :1160-1165 store = cvtps_ph RNE, :1230-1236 fp32 fmadd)
//                -> fp32 chain inside a 16-wide K tile, running sum rounded to fp16 at every tile edge
//       int8/16/32/64 (:650-670, :810-865, :444-485, :523-540) mullo + add -> arithmetic mod 2^bits
//   * nt/functional/cpu/matmult/nt_matmult.hpp:228-235   batches are independent, same flags for all.
//   * nt/functional/cpu/unfold2d.cpp:12-165   im2col index arithmetic (channel-major, then kh, kw).
//   * BFloat16 has no dtype in the reference (nt/dtype/compatible/DTypeDeclareMacros.h:5-9); the
//     oracle for it is the Float32 chain on exactly-widened inputs, rounded once to bf16 at the end.
//
// Because every output element is one sequential-k chain whose only rounding points are fixed by
// the dtype's TILE, the result does not depend on the blocking or threading chosen here.

#include <immintrin.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

enum DType : int { F32 = 0, F16 = 1, BF16 = 2, I8 = 3, I16 = 4, I32 = 5, I64 = 6, F64 = 7, U8 = 8, U16 = 9, U32 = 10,
                   F16_TILE8 = 100 /* one lane of Complex32: Float16 with a K tile of 8 */ };

inline float half_to_float(uint16_t h) { return _cvtsh_ss(h); }
inline uint16_t float_to_half(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT); }
inline float bf16_to_float(uint16_t h) {
    uint32_t u = uint32_t(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);  // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);                                         // round to nearest even
    return uint16_t(u >> 16);
}

template <class F>
void parallel_rows(int64_t n, int nthreads, F&& f) {
    nthreads = int(std::max<int64_t>(1, std::min<int64_t>(nthreads, n)));
    if (nthreads == 1) { f(0, n); return; }
    std::vector<std::thread> pool;
    int64_t chunk = (n + nthreads - 1) / nthreads;
    chunk = (chunk + 3) / 4 * 4;
    for (int64_t s = 0; s < n; s += chunk) pool.emplace_back([&, s] { f(s, std::min(n, s + chunk)); });
    for (auto& t : pool) t.join();
}

// ---- floating point (fp32 chain) -------------------------------------------------------------
enum class FloatKind { f32, f16, bf16, f16_tile8 };

template <FloatKind KIND>
struct FloatIO;
template <>
struct FloatIO<FloatKind::f32> {
    using T = float;
    static float widen(T v) { return v; }
    static T narrow(float v) { return v; }
    static constexpr bool round_each_tile = false;
    static constexpr int tile = 16;
};
template <>
struct FloatIO<FloatKind::f16> {
    using T = uint16_t;
    static float widen(T v) { return half_to_float(v); }
    static T narrow(float v) { return float_to_half(v); }
    static constexpr bool round_each_tile = true;   // C tile is stored as fp16 after every K tile
    static constexpr int tile = 16;
};
// One lane of a Complex32 matmult: Float16 values, but the reference's K tile for complex_32 is 8 wide (pack size 4,
// nt/mp/simde_traits/simde_traits_avx2.h:1273-1275), so the running sum is rounded to Float16 every 8 k-steps.
template <>
struct FloatIO<FloatKind::f16_tile8> {
    using T = uint16_t;
    static float widen(T v) { return half_to_float(v); }
    static T narrow(float v) { return float_to_half(v); }
    static constexpr bool round_each_tile = true;
    static constexpr int tile = 8;
};
template <>
struct FloatIO<FloatKind::bf16> {
    using T = uint16_t;
    static float widen(T v) { return bf16_to_float(v); }
    static T narrow(float v) { return float_to_bf16(v); }
    static constexpr bool round_each_tile = false;
    static constexpr int tile = 16;
};

inline __m256 round_through_half(__m256 v) {
    return _mm256_cvtph_ps(_mm256_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT));
}

// Ap: [M][Kp] widened op(A) (zero padded to Kp, a multiple of 16).  Bp: [Kp][Np] widened op(B),
// Np a multiple of 16.  One ascending-k fused-multiply-add chain per output element.
template <FloatKind KIND>
void float_rows(const float* Ap, const float* Bp, typename FloatIO<KIND>::T* C, int64_t N, int64_t K,
                int64_t Kp, int64_t Np, int64_t r0, int64_t r1) {
    using IO = FloatIO<KIND>;
    constexpr int TILE = IO::tile, MR = 4;
    (void)K;
    for (int64_t j0 = 0; j0 < Np; j0 += 16) {
        const int64_t jn = std::min<int64_t>(16, N - j0);
        for (int64_t i0 = r0; i0 < r1; i0 += MR) {
            const int mr = int(std::min<int64_t>(MR, r1 - i0));
            alignas(32) float cbuf[MR][16];
            for (int r = 0; r < MR; ++r)
                for (int j = 0; j < 16; ++j)
                    cbuf[r][j] = (r < mr && j < jn) ? IO::widen(C[(i0 + r) * N + j0 + j]) : 0.0f;
            __m256 acc[MR][2];
            for (int r = 0; r < MR; ++r) {
                acc[r][0] = _mm256_load_ps(&cbuf[r][0]);
                acc[r][1] = _mm256_load_ps(&cbuf[r][8]);
            }
            const float* a_row[MR];
            for (int r = 0; r < MR; ++r) a_row[r] = Ap + (i0 + std::min(r, mr - 1)) * Kp;
            for (int64_t k0 = 0; k0 < Kp; k0 += TILE) {
                for (int kk = 0; kk < TILE; ++kk) {
                    const float* brow = Bp + (k0 + kk) * Np + j0;
                    const __m256 b0 = _mm256_loadu_ps(brow), b1 = _mm256_loadu_ps(brow + 8);
                    for (int r = 0; r < MR; ++r) {
                        const __m256 a = _mm256_broadcast_ss(a_row[r] + k0 + kk);
                        acc[r][0] = _mm256_fmadd_ps(a, b0, acc[r][0]);
                        acc[r][1] = _mm256_fmadd_ps(a, b1, acc[r][1]);
                    }
                }
                if (IO::round_each_tile)
                    for (int r = 0; r < MR; ++r) {
                        acc[r][0] = round_through_half(acc[r][0]);
                        acc[r][1] = round_through_half(acc[r][1]);
                    }
            }
            for (int r = 0; r < MR; ++r) {
                _mm256_store_ps(&cbuf[r][0], acc[r][0]);
                _mm256_store_ps(&cbuf[r][8], acc[r][1]);
            }
            for (int r = 0; r < mr; ++r)
                for (int j = 0; j < jn; ++j) C[(i0 + r) * N + j0 + j] = IO::narrow(cbuf[r][j]);
        }
    }
}

template <FloatKind KIND>
void float_gemm(const void* A_, const void* B_, void* C_, int64_t M, int64_t K, int64_t N, bool ta, bool tb,
                int nthreads) {
    using IO = FloatIO<KIND>;
    using T = typename IO::T;
    const T* A = static_cast<const T*>(A_);
    const T* B = static_cast<const T*>(B_);
    T* C = static_cast<T*>(C_);
    if (M == 0 || N == 0 || K == 0) return;
    const int64_t Kp = (K + 15) / 16 * 16, Np = (N + 15) / 16 * 16;
    std::vector<float> Ap(size_t(M) * Kp, 0.0f), Bp(size_t(Kp) * Np, 0.0f);
    // op(A)[i][k]: stored [M][K] when !ta, [K][M] when ta (nt_matmult.hpp:109-122 reads it transposed).
    parallel_rows(M, nthreads, [&](int64_t s, int64_t e) {
        for (int64_t i = s; i < e; ++i)
            for (int64_t k = 0; k < K; ++k) Ap[i * Kp + k] = IO::widen(ta ? A[k * M + i] : A[i * K + k]);
    });
    parallel_rows(K, nthreads, [&](int64_t s, int64_t e) {
        for (int64_t k = s; k < e; ++k)
            for (int64_t j = 0; j < N; ++j) Bp[k * Np + j] = IO::widen(tb ? B[j * K + k] : B[k * N + j]);
    });
    parallel_rows(M, nthreads,
                  [&](int64_t s, int64_t e) { float_rows<KIND>(Ap.data(), Bp.data(), C, N, K, Kp, Np, s, e); });
}

void double_gemm(const double* A, const double* B, double* C, int64_t M, int64_t K, int64_t N, bool ta, bool tb,
                 int nthreads) {
    if (M == 0 || N == 0 || K == 0) return;
    std::vector<double> Bp(size_t(K) * N);
    for (int64_t k = 0; k < K; ++k)
        for (int64_t j = 0; j < N; ++j) Bp[k * N + j] = tb ? B[j * K + k] : B[k * N + j];
    parallel_rows(M, nthreads, [&](int64_t s, int64_t e) {
        std::vector<double> acc(N);
        for (int64_t i = s; i < e; ++i) {
            for (int64_t j = 0; j < N; ++j) acc[j] = C[i * N + j];
            for (int64_t k = 0; k < K; ++k) {
                const double a = ta ? A[k * M + i] : A[i * K + k];
                const double* b = &Bp[k * N];
                for (int64_t j = 0; j < N; ++j) acc[j] = __builtin_fma(a, b[j], acc[j]);
            }
            for (int64_t j = 0; j < N; ++j) C[i * N + j] = acc[j];
        }
    });
}

// ---- integers: products and sums wrap in the element width ------------------------------------
// Sum mod 2^32 (or 2^64) truncated to the element width equals the sum taken mod 2^width at every
// step, so one wide wrapping accumulator reproduces mullo+add in the narrow type; signed and
// unsigned share the low bits.
template <class T, class Acc>
void int_gemm(const void* A_, const void* B_, void* C_, int64_t M, int64_t K, int64_t N, bool ta, bool tb,
              int nthreads) {
    const T* A = static_cast<const T*>(A_);
    const T* B = static_cast<const T*>(B_);
    T* C = static_cast<T*>(C_);
    if (M == 0 || N == 0 || K == 0) return;
    std::vector<Acc> Bp(size_t(K) * N);
    parallel_rows(K, nthreads, [&](int64_t s, int64_t e) {
        for (int64_t k = s; k < e; ++k)
            for (int64_t j = 0; j < N; ++j) Bp[k * N + j] = Acc(tb ? B[j * K + k] : B[k * N + j]);
    });
    parallel_rows(M, nthreads, [&](int64_t s, int64_t e) {
        std::vector<Acc> acc(N);
        for (int64_t i = s; i < e; ++i) {
            for (int64_t j = 0; j < N; ++j) acc[j] = Acc(C[i * N + j]);
            for (int64_t k = 0; k < K; ++k) {
                const Acc a = Acc(ta ? A[k * M + i] : A[i * K + k]);
                const Acc* b = &Bp[k * N];
                for (int64_t j = 0; j < N; ++j) acc[j] += a * b[j];
            }
            for (int64_t j = 0; j < N; ++j) C[i * N + j] = T(acc[j]);
        }
    });
}

int dispatch(int dtype, const void* A, const void* B, void* C, int64_t M, int64_t K, int64_t N, bool ta, bool tb,
             int nthreads) {
    switch (dtype) {
        case F32: float_gemm<FloatKind::f32>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case F16: float_gemm<FloatKind::f16>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case BF16: float_gemm<FloatKind::bf16>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case F16_TILE8: float_gemm<FloatKind::f16_tile8>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case F64:
            double_gemm(static_cast<const double*>(A), static_cast<const double*>(B), static_cast<double*>(C), M, K, N,
                        ta, tb, nthreads);
            return 0;
        case I8: case U8: int_gemm<uint8_t, uint32_t>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case I16: case U16: int_gemm<uint16_t, uint32_t>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case I32: case U32: int_gemm<uint32_t, uint32_t>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
        case I64: int_gemm<uint64_t, uint64_t>(A, B, C, M, K, N, ta, tb, nthreads); return 0;
    }
    return 1;
}

int elem_size(int dtype) {
    switch (dtype) {
        case F32: case I32: case U32: return 4;
        case F16: case BF16: case I16: case U16: case F16_TILE8: return 2;
        case I8: case U8: return 1;
        case I64: case F64: return 8;
    }
    return 0;
}

}  // namespace

extern "C" {

// Mirrors nt_matmult<T> (nt/functional/cpu/matmult/nt_matmult.h:6-7): C += op(A).op(B); a_rows/a_cols and
// b_rows/b_cols are the logical dims AFTER the transposes (a_cols == b_rows); all row-major contiguous.
int oracle_matmult(int dtype, const void* A, const void* B, void* C, int64_t a_rows, int64_t a_cols, int64_t b_rows,
                   int64_t b_cols, int transpose_a, int transpose_b, int nthreads) {
    if (a_cols != b_rows || a_rows < 0 || a_cols < 0 || b_cols < 0) return 2;
    return dispatch(dtype, A, B, C, a_rows, a_cols, b_cols, transpose_a != 0, transpose_b != 0, nthreads);
}

// Mirrors nt_matmult_batch<T> (nt_matmult.h:9-10, nt_matmult.hpp:228-235): serial over the batch.
int oracle_matmult_batch(int dtype, const void* const* A, const void* const* B, void* const* C, int64_t batches,
                         int64_t a_rows, int64_t a_cols, int64_t b_rows, int64_t b_cols, int transpose_a,
                         int transpose_b, int nthreads) {
    for (int64_t b = 0; b < batches; ++b) {
        int rc = oracle_matmult(dtype, A[b], B[b], C[b], a_rows, a_cols, b_rows, b_cols, transpose_a, transpose_b,
                                nthreads);
        if (rc) return rc;
    }
    return 0;
}

// im2col with the reference's layout (nt/functional/cpu/unfold2d.cpp:12-165): col[b][c][h*Wc + w] with
// c = (c_im * kh + h_off) * kw + w_off, zero where the tap falls in the padding.  `col` must be zeroed
// by the caller exactly as functional::unfold2d does (colim_transform.cpp:579).
int oracle_im2col(int dtype, const void* im, void* col, int64_t batch, int64_t channels, int64_t height,
                  int64_t width, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                  int64_t dw) {
    const int es = elem_size(dtype);
    if (!es) return 1;
    const int64_t Hc = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int64_t Wc = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    const int64_t Ccol = channels * kh * kw;
    const char* src = static_cast<const char*>(im);
    char* dst = static_cast<char*>(col);
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t c = 0; c < Ccol; ++c) {
            const int64_t w_off = c % kw, h_off = (c / kw) % kh, c_im = c / kh / kw;
            for (int64_t h = 0; h < Hc; ++h) {
                const int64_t hp = h * sh - ph + h_off * dh;
                if (hp < 0 || hp >= height) continue;
                for (int64_t w = 0; w < Wc; ++w) {
                    const int64_t wp = w * sw - pw + w_off * dw;
                    if (wp < 0 || wp >= width) continue;
                    std::memcpy(dst + (((b * Ccol + c) * Hc + h) * Wc + w) * es,
                                src + (((b * channels + c_im) * height + hp) * width + wp) * es, es);
                }
            }
        }
    return 0;
}

// col2im for Float32 (nt/functional/cpu/unfold2d_backward.cpp): scatter-add of the column matrix back
// to the image, the adjoint of oracle_im2col.  `im` must be zeroed by the caller.
int oracle_col2im_f32(const float* col, float* im, int64_t batch, int64_t channels, int64_t height, int64_t width,
                      int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw) {
    const int64_t Hc = (height + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
    const int64_t Wc = (width + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
    const int64_t Ccol = channels * kh * kw;
    for (int64_t b = 0; b < batch; ++b)
        for (int64_t c = 0; c < Ccol; ++c) {
            const int64_t w_off = c % kw, h_off = (c / kw) % kh, c_im = c / kh / kw;
            for (int64_t h = 0; h < Hc; ++h) {
                const int64_t hp = h * sh - ph + h_off * dh;
                if (hp < 0 || hp >= height) continue;
                for (int64_t w = 0; w < Wc; ++w) {
                    const int64_t wp = w * sw - pw + w_off * dw;
                    if (wp < 0 || wp >= width) continue;
                    im[((b * channels + c_im) * height + hp) * width + wp] += col[((b * Ccol + c) * Hc + h) * Wc + w];
                }
            }
        }
    return 0;
}

int oracle_hardware_threads() { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
