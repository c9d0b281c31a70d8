// conv2d without a column matrix, for Float16 / BFloat16 with stride 1.
//
// The reference computes conv2d as unfold2d (im2col) followed by a matmult of the weights with the column matrix
// (NeuroTensor/functional/tensor_files/conv.cpp, conv2d; unfold2d in functional/tensor_files/fold.cpp).  The column
// matrix is kh*kw times the size of the input, and writing then re-reading it costs more than the GEMM itself on
// this GPU.  Here the GEMM's B operand is gathered from the input directly:
//
//   * the input is first copied to channels-last order, xt[b][h][w][c] (one pass over the input, not kh*kw);
//   * the weights are reordered to wp[cout][tap][c], tap = i*kw + j, so that K runs tap-major;
//   * K block (tap, c0..c0+63) of the B operand for the output pixels of rows h0..h0+r-1 is then the box
//     xt[b][h0 + i*dh - ph .. +r][j*dw - pw .. +Wo][c0 .. +64], which ONE 4-D TMA load fetches: its innermost
//     coordinate (c0) is a multiple of 64 elements, so the 16-byte start rule holds for every tap, the spatial shift
//     sits on outer coordinates that have no alignment rule, and positions outside the image are zero-filled by the
//     copy engine, which is exactly the convolution's zero padding;
//   * in shared memory the box is r*Wo rows of 128 bytes, i.e. a K-major operand tile with the 128-byte swizzle, the
//     same layout the GEMM kernels feed to tcgen05.mma.
//
// One CTA pair (cta_group::2) owns 256 output channels x (2*r*Wo) output pixels of one image; the even CTA issues the
// MMAs, both load and both run the epilogue.  Sums run over K in tap-major order instead of the reference's
// channel-major order; the accumulator is fp32 either way and the result is rounded once.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "internal.h"
#include "sm100_ptx.cuh"

namespace ntb200 {
namespace {

constexpr int kConvThreads = 192;                      // warp 0 loads, warp 1 issues MMAs, warps 2-5 store
constexpr int kConvStages = 5;                         // the loads are not latency bound: 4 to 7 stages time the same
constexpr uint32_t kConvOperandBytes = 128 * 128;      // 128 rows of 128 bytes
constexpr uint32_t kConvStageBytes = 2 * kConvOperandBytes;
constexpr uint32_t kConvStagingBytes = 65536;          // output staging: 4 epilogue warps x 8 chunks of 32 rows x 64 bytes
constexpr uint32_t kConvSmemBytes = kConvStages * kConvStageBytes + kConvStagingBytes + 256 + 1024;
constexpr uint32_t kConvTmemCols = 512;                // two accumulators of up to 256 columns

struct ConvParams {
    int cout, L, batch;
    int tiles_m, tiles_n, total_tiles;
    int c_blocks;          // channels / 64
    int k_blocks;          // kh * kw * c_blocks
    int kw, dh, dw, ph, pw;
    int rows_per_cta;      // output rows whose pixels one CTA stages per K block
    int wo;
    int bn;                // output pixels per tile = 2 * rows_per_cta * wo (multiple of 16, at most 256)
    uint32_t b_bytes;      // rows_per_cta * wo * 128
    uint32_t idesc;
    int out_bf16;
    int vec_ok;            // rows of the output start on 16-byte boundaries
    int tma_store;         // tiles leave through shared memory and TMA stores (bn a multiple of 32, aligned rows)
    void* out;
    unsigned int* status;  // device status word raised when a bounded wait runs out
};

__device__ __forceinline__ void conv_timeout(const ConvParams& p, volatile uint32_t* abort_flag, unsigned int where) {
    *abort_flag = 1;
    atomicExch(p.status, 0x100u | where);
}

__device__ __forceinline__ void conv_tile_coords(const ConvParams& p, int t, int& b, int& mi, int& ni) {
    const int per_image = p.tiles_m * p.tiles_n;
    b = t / per_image;
    const int r = t - b * per_image;
    mi = r / p.tiles_n;
    ni = r - mi * p.tiles_n;
}

__device__ __forceinline__ uint32_t pack16(float lo, float hi, int bf16) {
    if (bf16)
        return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
               (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
    return uint32_t(__half_as_ushort(__float2half_rn(lo))) | (uint32_t(__half_as_ushort(__float2half_rn(hi))) << 16);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kConvThreads, 1)
conv2d_implicit_pair_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                            const __grid_constant__ CUtensorMap tma_out, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t staging_base = smem_base + kConvStages * kConvStageBytes;
    uint8_t* bar_gen = smem_gen + kConvStages * kConvStageBytes + kConvStagingBytes;
    const uint32_t bar_base = staging_base + kConvStagingBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kConvStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kConvStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kConvStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * kConvStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        if (p.tma_store) tma_prefetch_desc(&tma_out);
        for (int s = 0; s < kConvStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);   // one arrival per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tma_w);
        tma_prefetch_desc(&tma_x);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kConvTmemCols);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.total_tiles; t += npairs) {
                int b, mi, ni;
                conv_tile_coords(p, t, b, mi, ni);
                const int m0 = mi * 256 + int(rank) * 128;
                const int h0 = (ni * 2 + int(rank)) * p.rows_per_cta;
                int tap_i = 0, tap_j = 0, cb = 0;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        conv_timeout(p, abort_flag, 0x21);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * kConvStageBytes;
                    const uint32_t b_dst = a_dst + kConvOperandBytes;
                    const uint32_t bar = full_bar(stage);
                    if (leader) mbar_expect_tx(bar, 2 * (kConvOperandBytes + p.b_bytes));
                    tma_load_3d_pair(a_dst, &tma_w, bar, kb * 64, m0, 0);
                    tma_load_4d_pair(b_dst, &tma_x, bar, cb * 64, tap_j * p.dw - p.pw, h0 + tap_i * p.dh - p.ph, b);
                    if (++cb == p.c_blocks) {
                        cb = 0;
                        if (++tap_j == p.kw) { tap_j = 0; ++tap_i; }
                    }
                    if (++stage == kConvStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {  // every stage released: all loads of this CTA have landed and been consumed
                for (int s = 0; s < kConvStages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { conv_timeout(p, abort_flag, 0x22); break; }
                    if (++stage == kConvStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA only)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.total_tiles; t += npairs) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    conv_timeout(p, abort_flag, 0x23);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        conv_timeout(p, abort_flag, 0x24);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_base + stage * kConvStageBytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(a_addr + kConvOperandBytes, 16, 1024);
#pragma unroll
                    for (int k = 0; k < 4; ++k)   // 16 elements (32 bytes) of K per instruction
                        umma<MmaKind::f16, 2>(d_tmem, a_desc + uint64_t(2 * k), b_desc + uint64_t(2 * k), p.idesc,
                                              (kb | k) != 0);
                    umma_commit_pair(empty_bar(stage), 3);
                    if (++stage == kConvStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(acc), 3);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int quad = warp & 3;
        const int row_in_tile = int(rank) * 128 + quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = pair; t < p.total_tiles; t += npairs) {
            int b, mi, ni;
            conv_tile_coords(p, t, b, mi, ni);
            bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) conv_timeout(p, abort_flag, 0x25);
                break;
            }
            tcgen05_fence_after();
            const int row = mi * 256 + row_in_tile;
            const int n0 = ni * p.bn;
            const int n_end = min(p.L, n0 + p.bn);
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * 256);
            if (p.tma_store) {
                // 32-column chunks leave through this warp's staging buffers (32 rows x 64 bytes each, 64-byte swizzle:
                // the 16-byte piece q of row r sits at piece q ^ ((r >> 1) & 3)) and one TMA store per chunk, which
                // clips at the end of the image's pixels.  bn is a multiple of 32 here, so no chunk crosses into the
                // next tile.
                const uint32_t staging = staging_base + uint32_t(quad) * 16384u;
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
#pragma unroll 1
                for (int cc = 0; cc * 32 < p.bn; ++cc) {
                    const int col0 = n0 + cc * 32;
                    if (col0 >= n_end) break;   // uniform across the CTA
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + uint32_t(cc * 32), v);
                    tmem_ld_wait();
                    const uint32_t buf = staging + uint32_t(cc) * 2048u;
                    const uint32_t row_smem = buf + uint32_t(lane) * 64u;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t w0 = pack16(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]), p.out_bf16);
                        const uint32_t w1 = pack16(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]), p.out_bf16);
                        const uint32_t w2 = pack16(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]), p.out_bf16);
                        const uint32_t w3 = pack16(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]), p.out_bf16);
                        const uint32_t piece = uint32_t(q) ^ uint32_t((lane >> 1) & 3);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_smem + (piece << 4)), "r"(w0), "r"(w1),
                                     "r"(w2), "r"(w3) : "memory");
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tma_out, buf, col0, mi * 256 + int(rank) * 128 + quad * 32, b);
                        tma_store_commit();
                    }
                }
            } else {
            uint16_t* out_row = static_cast<uint16_t*>(p.out) + ((long long)b * p.cout + row) * (long long)p.L;
#pragma unroll 1
            for (int cc = 0; cc * 32 < p.bn; ++cc) {
                const int col0 = n0 + cc * 32;
                if (col0 >= n_end) break;   // uniform across the CTA
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + uint32_t(cc * 32), v);
                tmem_ld_wait();
                if (row >= p.cout) continue;
                uint16_t* dst = out_row + col0;
                if (p.vec_ok && col0 + 32 <= n_end) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        o.x = pack16(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]), p.out_bf16);
                        o.y = pack16(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]), p.out_bf16);
                        o.z = pack16(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]), p.out_bf16);
                        o.w = pack16(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]), p.out_bf16);
                        *reinterpret_cast<uint4*>(dst + 8 * q) = o;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < n_end) dst[j] = uint16_t(pack16(__uint_as_float(v[j]), 0.f, p.out_bf16));
                }
            }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();
    }

    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kConvTmemCols);
    }
}

// One launch prepares both operands.
//   blocks [0, tr_blocks): x[b][c][hw] -> xt[b][hw][c], 16-bit elements, one 64 x 64 tile per block through shared
//     memory so that both the reads (along hw) and the writes (along c) are contiguous.  kVec: hw is even and the
//     bases are 4-byte aligned, so every access moves two elements and a warp moves 128 contiguous bytes.  Channel c
//     is kept in tile row (c >> 1) + 32 * (c & 1): the two halves of an output word then sit in rows that differ by
//     32, and with a row stride of 33 words the 32 lanes of a warp read 32 different banks.
//   the remaining blocks: w[cout][c][tap] -> wp[cout][tap][c].
template <int kVec>
__global__ void __launch_bounds__(256)
conv_prepare_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ xt, int channels, int hw, int tiles_p,
                    int tiles_c, int tr_blocks, const uint16_t* __restrict__ w, uint16_t* __restrict__ wp, int taps,
                    long long w_total) {
    if (int(blockIdx.x) >= tr_blocks) {
        const long long idx = (long long)(blockIdx.x - tr_blocks) * 256 + threadIdx.x;
        if (idx >= w_total) return;
        const int c = int(idx % channels);
        const long long r = idx / channels;
        const int t = int(r % taps);
        const long long co = r / taps;
        wp[idx] = w[(co * channels + c) * taps + t];
        return;
    }
    __shared__ __align__(16) uint32_t tile[64][33];
    const int pt = int(blockIdx.x) % tiles_p;
    const int rest = int(blockIdx.x) / tiles_p;
    const int ct = rest % tiles_c, b = rest / tiles_c;
    const size_t image = size_t(b) * size_t(channels) * size_t(hw);
    const int c0 = ct * 64, p0 = pt * 64;
    if constexpr (kVec == 8) {
        // hw is a multiple of 8 and the bases are 16-byte aligned: 16-byte loads (8 pixels of one channel) and
        // 16-byte stores (8 channels of one pixel).  The tile keeps 128-byte rows [channel][64 pixels] whose
        // 16-byte chunks are XOR-ed with bits 3..5 of the channel, so the eight channels one output vector needs
        // (same pixel, channels 8*cw .. 8*cw+7 for the eight cw of a quarter warp) come from different banks.
        uint4* t128 = reinterpret_cast<uint4*>(&tile[0][0]);          // [64 rows][8 chunks]
        const uint16_t* t16 = reinterpret_cast<const uint16_t*>(&tile[0][0]);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int c = idx >> 3, chunk = idx & 7;
            if (p0 + 8 * chunk < hw)
                t128[c * 8 + (chunk ^ ((c >> 3) & 7))] =
                    *reinterpret_cast<const uint4*>(x + image + size_t(c0 + c) * hw + p0 + 8 * chunk);
        }
        __syncthreads();
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int pp = idx >> 3, cw = idx & 7;
            if (p0 + pp < hw) {
                uint32_t v[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int ce = 8 * cw + 2 * q;   // channels ce, ce + 1: same (c >> 3), so the same chunk swizzle
                    const int at = (((pp >> 3) ^ cw) << 3) + (pp & 7);
                    v[q] = uint32_t(t16[ce * 64 + at]) | (uint32_t(t16[(ce + 1) * 64 + at]) << 16);
                }
                *reinterpret_cast<uint4*>(xt + image + size_t(p0 + pp) * channels + c0 + 8 * cw) =
                    make_uint4(v[0], v[1], v[2], v[3]);
            }
        }
    } else if constexpr (kVec == 2) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int c = idx >> 5, pw = idx & 31;
            if (p0 + 2 * pw < hw)
                tile[(c >> 1) + 32 * (c & 1)][pw] =
                    *reinterpret_cast<const uint32_t*>(x + image + size_t(c0 + c) * hw + p0 + 2 * pw);
        }
        __syncthreads();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int pp = idx >> 5, cw = idx & 31;   // channels 2*cw and 2*cw + 1 of pixel pp
            if (p0 + pp < hw) {
                const uint32_t even = tile[cw][pp >> 1], odd = tile[cw + 32][pp >> 1];
                const uint32_t word = (pp & 1) ? ((even >> 16) | (odd & 0xffff0000u)) : ((even & 0xffffu) | (odd << 16));
                *reinterpret_cast<uint32_t*>(xt + image + size_t(p0 + pp) * channels + c0 + 2 * cw) = word;
            }
        }
    } else {
        uint16_t* t16 = reinterpret_cast<uint16_t*>(&tile[0][0]);   // [64][66] elements
#pragma unroll
        for (int it = 0; it < 16; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int c = idx >> 6, pp = idx & 63;
            if (p0 + pp < hw) t16[c * 66 + pp] = x[image + size_t(c0 + c) * hw + p0 + pp];
        }
        __syncthreads();
#pragma unroll
        for (int it = 0; it < 16; ++it) {
            const int idx = it * 256 + int(threadIdx.x);
            const int pp = idx >> 6, c = idx & 63;
            if (p0 + pp < hw) xt[image + size_t(p0 + pp) * channels + c0 + c] = t16[c * 66 + pp];
        }
    }
}

// NTB200_DIRECT_STORES=1 keeps the per-thread global stores in the epilogue (for A/B measurements).
bool direct_stores() {
    const char* e = getenv("NTB200_DIRECT_STORES");
    return e && e[0] == '1';
}

// NTB200_CONV_EXPLICIT=1 keeps every convolution on the column-matrix path (read per call, for A/B comparisons).
bool force_explicit() {
    const char* e = getenv("NTB200_CONV_EXPLICIT");
    return e && e[0] == '1';
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline size_t round256(size_t v) { return (v + 255u) & ~size_t(255); }

}  // namespace

// Output rows per CTA: the most rows whose pixels fill at most 128 operand rows in whole groups of eight.
static int conv_rows_per_cta(int64_t wo) {
    for (int64_t r = 128 / wo; r >= 1; --r)
        if ((r * wo) % 8 == 0) return int(r);
    return 0;
}

bool conv2d_implicit_supported(const Conv2dShape& s, size_t workspace_bytes) {
    if (force_explicit()) return false;
    if (s.dtype != NTB200_F16 && s.dtype != NTB200_BF16) return false;
    if (s.sh != 1 || s.sw != 1) return false;
    if (s.channels % 64 != 0) return false;
    if (s.kh * s.kw == 1 && s.ph == 0 && s.pw == 0) return false;   // the column matrix IS the input: nothing to save
    if (s.wo < 1 || s.wo > 128 || conv_rows_per_cta(s.wo) == 0) return false;
    const int64_t lim = int64_t(1) << 30;
    if (s.batch >= lim || s.channels * s.kh * s.kw >= lim || s.height >= lim || s.width >= lim || s.cout >= lim ||
        s.ho * s.wo >= lim)
        return false;
    if (s.ph >= lim || s.pw >= lim || s.dh * s.kh >= lim || s.dw * s.kw >= lim) return false;
    const size_t es = 2;
    const size_t need = round256(size_t(s.batch) * s.channels * s.height * s.width * es) +
                        size_t(s.cout) * s.channels * s.kh * s.kw * es;
    return need <= workspace_bytes;
}

int launch_conv2d_implicit(const Conv2dShape& s, const void* x, const void* w, void* out, void* workspace,
                           cudaStream_t stream) {
    const size_t es = 2;
    const int64_t taps = s.kh * s.kw, ck = s.channels * taps, L = s.ho * s.wo;
    uint16_t* xt = static_cast<uint16_t*>(workspace);
    uint16_t* wp = reinterpret_cast<uint16_t*>(static_cast<char*>(workspace) +
                                               round256(size_t(s.batch) * s.channels * s.height * s.width * es));
    if (reinterpret_cast<uintptr_t>(workspace) % 256 || reinterpret_cast<uintptr_t>(out) % 2 ||
        reinterpret_cast<uintptr_t>(x) % 2 || reinterpret_cast<uintptr_t>(w) % 2)
        return NTB200_ERR_UNSUPPORTED;

    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
    if (!enc) return NTB200_ERR_UNSUPPORTED;
    const CUtensorMapDataType dt = s.dtype == NTB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const int rows = conv_rows_per_cta(s.wo);

    CUtensorMap map_w, map_x;
    {
        cuuint64_t dims[3] = {cuuint64_t(ck), cuuint64_t(s.cout), 1};
        cuuint64_t strides[2] = {cuuint64_t(ck) * es, cuuint64_t(ck) * es * cuuint64_t(s.cout)};
        strides[1] = (strides[1] + 15u) & ~cuuint64_t(15);
        cuuint32_t box[3] = {64, 128, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&map_w, dt, 3, wp, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return NTB200_ERR_UNSUPPORTED;
    }
    {
        cuuint64_t dims[4] = {cuuint64_t(s.channels), cuuint64_t(s.width), cuuint64_t(s.height), cuuint64_t(s.batch)};
        cuuint64_t strides[3] = {cuuint64_t(s.channels) * es, cuuint64_t(s.channels) * es * cuuint64_t(s.width),
                                 cuuint64_t(s.channels) * es * cuuint64_t(s.width) * cuuint64_t(s.height)};
        cuuint32_t box[4] = {64, cuuint32_t(s.wo), cuuint32_t(rows), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&map_x, dt, 4, xt, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return NTB200_ERR_UNSUPPORTED;
    }

    ConvParams p{};
    CUtensorMap map_out = map_w;
    p.tma_store = 0;
    if ((2 * rows * s.wo) % 32 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 && L % 8 == 0 && !direct_stores()) {
        cuuint64_t dims[3] = {cuuint64_t(L), cuuint64_t(s.cout), cuuint64_t(s.batch)};
        cuuint64_t strides[2] = {cuuint64_t(L) * es, cuuint64_t(L) * es * cuuint64_t(s.cout)};
        cuuint32_t box[3] = {32, 32, 1};
        cuuint32_t estr[3] = {1, 1, 1};
        p.tma_store = enc(&map_out, dt, 3, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    p.cout = int(s.cout); p.L = int(L); p.batch = int(s.batch);
    p.tiles_m = int((s.cout + 255) / 256);
    p.tiles_n = int((s.ho + 2 * rows - 1) / (2 * rows));
    const int64_t total = int64_t(p.tiles_m) * p.tiles_n * s.batch;
    if (total >= (int64_t(1) << 30)) return NTB200_ERR_UNSUPPORTED;
    p.total_tiles = int(total);
    p.c_blocks = int(s.channels / 64);
    p.k_blocks = int(taps) * p.c_blocks;
    p.kw = int(s.kw); p.dh = int(s.dh); p.dw = int(s.dw); p.ph = int(s.ph); p.pw = int(s.pw);
    p.rows_per_cta = rows;
    p.wo = int(s.wo);
    p.bn = 2 * rows * int(s.wo);
    p.b_bytes = uint32_t(rows) * uint32_t(s.wo) * 128u;
    const uint32_t fmt = s.dtype == NTB200_F16 ? 0u : 1u;
    p.idesc = make_instr_desc(1, fmt, fmt, false, false, 256, uint32_t(p.bn));
    p.out_bf16 = s.dtype == NTB200_BF16;
    p.vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (L % 8 == 0);
    p.out = out;
    p.status = device_status_word();
    if (!p.status) return NTB200_ERR_UNSUPPORTED;

    // Nothing has been launched before this point: UNSUPPORTED above lets the caller take the column-matrix path.
    const int hw = int(s.height * s.width);
    const int tiles_p = (hw + 63) / 64, tiles_c = int(s.channels / 64);
    const long long tr_blocks = (long long)tiles_p * tiles_c * s.batch;
    const long long w_total = (long long)s.cout * ck;
    const long long blocks = tr_blocks + (w_total + 255) / 256;
    if (blocks >= (int64_t(1) << 31)) return NTB200_ERR_UNSUPPORTED;
    const uintptr_t x_addr = reinterpret_cast<uintptr_t>(x);
    auto prepare = (hw % 8 == 0 && x_addr % 16 == 0) ? conv_prepare_kernel<8>
                   : (hw % 2 == 0 && x_addr % 4 == 0) ? conv_prepare_kernel<2>
                                                       : conv_prepare_kernel<0>;
    prepare<<<unsigned(blocks), 256, 0, stream>>>(static_cast<const uint16_t*>(x), xt, int(s.channels), hw, tiles_p,
                                                  tiles_c, int(tr_blocks), static_cast<const uint16_t*>(w), wp,
                                                  int(taps), w_total);
    count_launch();
    NTB200_CUDA(cudaGetLastError());

    cudaError_t e = cudaFuncSetAttribute(conv2d_implicit_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(kConvSmemBytes));
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(conv2d_implicit_pair_kernel)");
    static int resident[64] = {0};
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (resident[dev] == 0)
        resident[dev] = max_resident_pairs(reinterpret_cast<const void*>(conv2d_implicit_pair_kernel), kConvSmemBytes);
    const int pairs = std::min(p.total_tiles, resident[dev]);
    conv2d_implicit_pair_kernel<<<2 * pairs, kConvThreads, kConvSmemBytes, stream>>>(map_w, map_x, map_out, p);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    note_route("conv2d-implicit-umma-pair");
    return NTB200_OK;
}

// ---- kernel gradient -----------------------------------------------------------------------------------
// d_kernel[co][c][i][j] = sum over images b and output pixels (y, x) of
//     grad[b][co][y][x] * image[b][c][y + i*dh - ph][x + j*dw - pw]          (conv.cpp:444-471 without the column matrix)
// As a GEMM: M = co, N = (tap, c), K = (b, y, x).  With channels-last copies of grad and of the image, both
// operands have their M / N index contiguous and the pixels as rows, i.e. they are MN-major operand tiles:
//   A chunk = gt[b][y0 .. +r][0 .. Wo][co0 .. +64]                      r*Wo pixel rows of 128 bytes
//   B chunk = xt[b][y0 + i*dh - ph .. +r][j*dw - pw .. +Wo][c0 .. +64]  the same pixels, shifted by the tap
// each fetched by one 4-D TMA box (zero-filled outside the image).  One stage holds r*Wo pixels of K for the
// 2 x 64 output channels and 2 x 64 (tap, c) columns of one CTA; the pair's UMMA is 256 x 256 x 16.  There are only
// (Cout/256) x (taps*C/256) output tiles, so K is also split over groups of images: every (group, tile) is one work
// item with its own fp32 partial result, and dkernel_reduce_kernel adds the groups, restores the [co][c][tap]
// order and rounds once.
namespace {

constexpr uint32_t kDkSmemLimit = 232448 - 2048;   // dynamic shared memory per CTA minus barriers and alignment slack

struct DkParams {
    int cout, channels, taps, n_total;   // n_total = taps * channels
    int tiles_m, tiles_n, groups, images_per_group, batch, total_items;
    int row_blocks;                       // ceil(Ho / rows)
    int rows, ksteps;                     // output rows per stage; rows * Wo / 16
    uint32_t chunk_bytes;                 // rows * Wo * 128
    uint32_t stage_bytes;                 // 4 chunks
    int stages;
    int kw, dh, dw, ph, pw;
    uint32_t idesc;
    float* partial;                       // [groups][cout][n_total]
    unsigned int* status;
};

__device__ __forceinline__ void dk_timeout(const DkParams& p, volatile uint32_t* abort_flag, unsigned int where) {
    *abort_flag = 1;
    atomicExch(p.status, 0x100u | where);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kConvThreads, 1)
conv2d_dkernel_pair_kernel(const __grid_constant__ CUtensorMap tma_g, const __grid_constant__ CUtensorMap tma_x,
                           const DkParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const int stages = p.stages;
    uint8_t* bar_gen = smem_gen + stages * p.stage_bytes;
    const uint32_t bar_base = smem_base + stages * p.stage_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (stages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * stages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * stages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * stages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tma_g);
        tma_prefetch_desc(&tma_x);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kConvTmemCols);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before();
    cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.total_items; t += npairs) {
                const int g = t / tiles, r = t - g * tiles;
                const int mi = r / p.tiles_n, ni = r - mi * p.tiles_n;
                const int co0 = mi * 256 + int(rank) * 128;
                int c0[2], sh_y[2], sh_x[2];
#pragma unroll
                for (int q = 0; q < 2; ++q) {   // the two 64-wide (tap, c) chunks this CTA stages
                    const int nidx = ((ni * 2 + int(rank)) * 2 + q) * 64;
                    const int tap = nidx / p.channels;
                    c0[q] = nidx - tap * p.channels;
                    const int ti = tap / p.kw, tj = tap - ti * p.kw;
                    sh_y[q] = ti * p.dh - p.ph;
                    sh_x[q] = tj * p.dw - p.pw;
                }
                const int img_end = min(p.batch, (g + 1) * p.images_per_group);
                for (int img = g * p.images_per_group; ok && img < img_end; ++img) {
                    for (int rb = 0; rb < p.row_blocks; ++rb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                            dk_timeout(p, abort_flag, 0x31);
                            ok = false;
                            break;
                        }
                        const uint32_t a_dst = smem_base + stage * p.stage_bytes;
                        const uint32_t b_dst = a_dst + 2 * p.chunk_bytes;
                        const uint32_t bar = full_bar(stage);
                        if (leader) mbar_expect_tx(bar, 2 * p.stage_bytes);
                        const int y0 = rb * p.rows;
                        tma_load_4d_pair(a_dst, &tma_g, bar, co0, 0, y0, img);
                        tma_load_4d_pair(a_dst + p.chunk_bytes, &tma_g, bar, co0 + 64, 0, y0, img);
                        tma_load_4d_pair(b_dst, &tma_x, bar, c0[0], sh_x[0], y0 + sh_y[0], img);
                        tma_load_4d_pair(b_dst + p.chunk_bytes, &tma_x, bar, c0[1], sh_x[1], y0 + sh_y[1], img);
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (ok) {
                for (int s = 0; s < stages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { dk_timeout(p, abort_flag, 0x32); break; }
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA only)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.total_items; t += npairs) {
                const int g = t / tiles;
                const int n_img = min(p.batch, (g + 1) * p.images_per_group) - g * p.images_per_group;
                const int n_stages = n_img * p.row_blocks;
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    dk_timeout(p, abort_flag, 0x33);
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int it = 0; it < n_stages; ++it) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        dk_timeout(p, abort_flag, 0x34);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_base + stage * p.stage_bytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, p.chunk_bytes, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(a_addr + 2 * p.chunk_bytes, p.chunk_bytes, 1024);
                    for (int k = 0; k < p.ksteps; ++k)   // 16 pixel rows (2048 bytes) per instruction
                        umma<MmaKind::f16, 2>(d_tmem, a_desc + uint64_t(k * 128), b_desc + uint64_t(k * 128), p.idesc,
                                              (it | k) != 0);
                    umma_commit_pair(empty_bar(stage), 3);
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(acc), 3);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs): fp32 partials
        const int quad = warp & 3;
        const int row_in_tile = int(rank) * 128 + quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = pair; t < p.total_items; t += npairs) {
            const int g = t / tiles, r = t - g * tiles;
            const int mi = r / p.tiles_n, ni = r - mi * p.tiles_n;
            bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) dk_timeout(p, abort_flag, 0x35);
                break;
            }
            tcgen05_fence_after();
            const int row = mi * 256 + row_in_tile;
            const int n0 = ni * 256;
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * 256);
            float* out_row = p.partial + ((long long)g * p.cout + row) * (long long)p.n_total;
#pragma unroll 1
            for (int cc = 0; cc < 8; ++cc) {
                const int col0 = n0 + cc * 32;
                if (col0 >= p.n_total) break;   // n_total is a multiple of 64: chunks are whole
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + uint32_t(cc * 32), v);
                tmem_ld_wait();
                if (row >= p.cout) continue;
                float4* dst = reinterpret_cast<float4*>(out_row + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    dst[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                         __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kConvTmemCols);
    }
}

// d_kernel[co][c][tap] (+)= sum over groups of partial[g][co][tap * C + c], rounded once.
__global__ void dkernel_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ dk, int groups,
                                      long long per_group, int n_total, int channels, int taps, int bf16, int accumulate) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per_group) return;
    float sum = 0.f;
    for (int g = 0; g < groups; ++g) sum += partial[(long long)g * per_group + idx];
    const long long co = idx / n_total;
    const int n = int(idx - co * n_total);
    const int tap = n / channels, c = n - tap * channels;
    uint16_t* dst = dk + (co * channels + c) * taps + tap;
    if (accumulate)
        sum += bf16 ? __bfloat162float(__ushort_as_bfloat16(*dst)) : __half2float(__ushort_as_half(*dst));
    *dst = uint16_t(pack16(sum, 0.f, bf16));
}

// Output rows per stage for the kernel gradient: the most rows whose pixels are at most 128 and a multiple of 16.
int dk_rows_per_stage(int64_t wo) {
    for (int64_t r = 128 / wo; r >= 1; --r)
        if ((r * wo) % 16 == 0) return int(r);
    return 0;
}

struct DkPlan {
    int rows, groups, images_per_group, tiles_m, tiles_n;
    size_t xt_bytes, gt_bytes, partial_bytes;
};

bool dk_plan(const Conv2dShape& s, DkPlan* out) {
    if (s.dtype != NTB200_F16 && s.dtype != NTB200_BF16) return false;
    if (s.sh != 1 || s.sw != 1) return false;
    if (s.channels % 64 != 0 || s.cout % 64 != 0) return false;
    if (s.wo < 1 || s.wo > 128) return false;
    const int rows = dk_rows_per_stage(s.wo);
    if (rows == 0) return false;
    const int64_t lim = int64_t(1) << 30;
    if (s.batch >= lim || s.channels * s.kh * s.kw >= lim || s.height >= lim || s.width >= lim || s.cout >= lim ||
        s.ho * s.wo >= lim || s.ph >= lim || s.pw >= lim || s.dh * s.kh >= lim || s.dw * s.kw >= lim)
        return false;
    out->rows = rows;
    out->tiles_m = int((s.cout + 255) / 256);
    out->tiles_n = int((s.channels * s.kh * s.kw + 255) / 256);
    const int64_t tiles = int64_t(out->tiles_m) * out->tiles_n;
    if (tiles >= lim) return false;
    const int pairs = std::max(1, sm_count() / 2);
    int64_t groups = std::max<int64_t>(1, std::min<int64_t>(s.batch, pairs / tiles));
    out->images_per_group = int((s.batch + groups - 1) / groups);
    out->groups = int((s.batch + out->images_per_group - 1) / out->images_per_group);
    out->xt_bytes = round256(size_t(s.batch) * s.channels * s.height * s.width * 2);
    out->gt_bytes = round256(size_t(s.batch) * s.cout * s.ho * s.wo * 2);
    out->partial_bytes = size_t(out->groups) * s.cout * s.channels * s.kh * s.kw * 4;
    return true;
}

}  // namespace

size_t conv2d_dkernel_implicit_bytes(const Conv2dShape& s) {
    DkPlan pl;
    if (!dk_plan(s, &pl)) return 0;
    return pl.xt_bytes + pl.gt_bytes + pl.partial_bytes;
}

int launch_conv2d_dkernel_implicit(const Conv2dShape& s, const void* x, const void* grad, void* d_kernel,
                                   void* workspace, int accumulate, cudaStream_t stream) {
    DkPlan pl;
    if (force_explicit() || !dk_plan(s, &pl)) return NTB200_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) % 256) return NTB200_ERR_UNSUPPORTED;
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
    if (!enc) return NTB200_ERR_UNSUPPORTED;
    const size_t es = 2;
    uint16_t* xt = static_cast<uint16_t*>(workspace);
    uint16_t* gt = reinterpret_cast<uint16_t*>(static_cast<char*>(workspace) + pl.xt_bytes);
    float* partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + pl.xt_bytes + pl.gt_bytes);
    const CUtensorMapDataType dt = s.dtype == NTB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;

    auto encode4 = [&](CUtensorMap* map, void* base, int64_t ch, int64_t wd, int64_t ht) {
        cuuint64_t dims[4] = {cuuint64_t(ch), cuuint64_t(wd), cuuint64_t(ht), cuuint64_t(s.batch)};
        cuuint64_t strides[3] = {cuuint64_t(ch) * es, cuuint64_t(ch) * es * cuuint64_t(wd),
                                 cuuint64_t(ch) * es * cuuint64_t(wd) * cuuint64_t(ht)};
        cuuint32_t box[4] = {64, cuuint32_t(s.wo), cuuint32_t(pl.rows), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        return enc(map, dt, 4, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    };
    CUtensorMap map_g, map_x;
    if (!encode4(&map_g, gt, s.cout, s.wo, s.ho) || !encode4(&map_x, xt, s.channels, s.width, s.height))
        return NTB200_ERR_UNSUPPORTED;

    DkParams p{};
    p.cout = int(s.cout); p.channels = int(s.channels); p.taps = int(s.kh * s.kw);
    p.n_total = p.taps * p.channels;
    p.tiles_m = pl.tiles_m; p.tiles_n = pl.tiles_n;
    p.groups = pl.groups; p.images_per_group = pl.images_per_group; p.batch = int(s.batch);
    p.total_items = pl.groups * pl.tiles_m * pl.tiles_n;
    p.rows = pl.rows;
    p.row_blocks = int((s.ho + pl.rows - 1) / pl.rows);
    p.ksteps = int(pl.rows * s.wo / 16);
    p.chunk_bytes = uint32_t(pl.rows * s.wo) * 128u;
    p.stage_bytes = 4 * p.chunk_bytes;
    p.stages = int(std::min<uint32_t>(8, kDkSmemLimit / p.stage_bytes));
    p.kw = int(s.kw); p.dh = int(s.dh); p.dw = int(s.dw); p.ph = int(s.ph); p.pw = int(s.pw);
    const uint32_t fmt = s.dtype == NTB200_F16 ? 0u : 1u;
    p.idesc = make_instr_desc(1, fmt, fmt, true, true, 256, 256);
    p.partial = partial;
    p.status = device_status_word();
    if (!p.status || p.stages < 2) return NTB200_ERR_UNSUPPORTED;

    // channels-last copies of the image and of the gradient (nothing was launched before this point)
    auto copy_channels_last = [&](const void* src, uint16_t* dst, int64_t ch, int64_t hw64) -> int {
        const int hw = int(hw64);
        const int tiles_p = (hw + 63) / 64, tiles_c = int(ch / 64);
        const long long blocks = (long long)tiles_p * tiles_c * s.batch;
        if (blocks >= (int64_t(1) << 31)) return fail(NTB200_ERR_INVALID_ARG, "conv2d_backward_kernel: too many tiles");
        const uintptr_t addr = reinterpret_cast<uintptr_t>(src);
        auto prepare = (hw % 8 == 0 && addr % 16 == 0) ? conv_prepare_kernel<8>
                       : (hw % 2 == 0 && addr % 4 == 0) ? conv_prepare_kernel<2>
                                                        : conv_prepare_kernel<0>;
        prepare<<<unsigned(blocks), 256, 0, stream>>>(static_cast<const uint16_t*>(src), dst, int(ch), hw, tiles_p, tiles_c,
                                                      int(blocks), nullptr, nullptr, 1, 0);
        count_launch();
        NTB200_CUDA(cudaGetLastError());
        return NTB200_OK;
    };
    if (int rc = copy_channels_last(x, xt, s.channels, s.height * s.width)) return rc;
    if (int rc = copy_channels_last(grad, gt, s.cout, s.ho * s.wo)) return rc;

    const uint32_t smem = uint32_t(p.stages) * p.stage_bytes + 256 + 1024;
    cudaError_t e = cudaFuncSetAttribute(conv2d_dkernel_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(conv2d_dkernel_pair_kernel)");
    const int pairs = std::min(p.total_items, std::max(1, sm_count() / 2));
    conv2d_dkernel_pair_kernel<<<2 * pairs, kConvThreads, smem, stream>>>(map_g, map_x, p);
    count_launch();
    NTB200_CUDA(cudaGetLastError());

    const long long per_group = (long long)s.cout * p.n_total;
    dkernel_reduce_kernel<<<unsigned((per_group + 255) / 256), 256, 0, stream>>>(
        partial, static_cast<uint16_t*>(d_kernel), p.groups, per_group, p.n_total, p.channels, p.taps,
        s.dtype == NTB200_BF16, accumulate != 0);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    note_route("conv2d-dkernel-implicit-umma-pair");
    return NTB200_OK;
}

}  // namespace ntb200
