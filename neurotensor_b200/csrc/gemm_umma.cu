// tcgen05 GEMMs.  Replace the packed simde/TBB kernels of nt/functional/cpu/matmult/nt_matmult.hpp:124-235 for
//   Float16 / BFloat16   fp32 accumulation in tensor memory, one rounding at the end
//   Int8 / UInt8         s32 accumulation, truncated to 8 bits (arithmetic mod 2^8)
//   Float32              three TF32 products per multiply on hi/lo split copies, two-level accumulation
//   Int32 / UInt32       products of 8-bit limbs, shifted and added modulo 2^32 by the epilogue
//
// Two kernels with the same roles.  `umma_gemm_pair_kernel`: a cluster of two CTAs (the two SMs of a TPC) computes a
// 256 x 256 tile with tcgen05.mma.cta_group::2; `umma_gemm_kernel<BN>`: one CTA per 128 x BN tile, for problems too
// small to fill the machine with pair tiles.  Both are persistent (one CTA per SM) with 192 threads:
//   warp 0      TMA producer   - one lane issues cp.async.bulk.tensor loads of the A and B tiles of a K block
//                                into a ring of shared-memory stages (128-byte swizzle), signalling `full`
//   warp 1      MMA issuer     - allocates tensor memory; one lane issues tcgen05.mma per 32 bytes of K,
//                                tcgen05.commit releases the stage (`empty`) and, after the last K block,
//                                publishes the accumulator (`tmem_full`)
//   warps 2..5  epilogue       - tcgen05.ld the accumulator (each warp owns a 32-lane quadrant), add bias /
//                                previous C, apply the optional ReLU outputs, convert, store (also into peer GPUs'
//                                copies of C when asked); then hand the accumulator back.  In the pair kernel the
//                                8- and 16-bit outputs leave through a swizzled shared-memory staging buffer and
//                                TMA stores of 128-byte row segments instead of per-thread global stores
// (the Float32 split kernels run 8 epilogue warps that keep running sums in registers).
// Two accumulators (2 x 256 columns of TMEM) let the epilogue of tile i overlap the main loop of tile i+1.
//
// Transposed and strided views never get copied: an operand whose unit stride runs along K is staged
// K-major, one whose unit stride runs along M (or N) is staged MN-major in 128-byte-wide chunks; the
// difference is carried by the TMA tensor map, the shared-memory descriptor and one bit of the
// instruction descriptor.  Tails in M, N and K are zero-filled by TMA and masked at the store.
// Every wait is bounded; a wait that runs out raises the device status word and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "internal.h"
#include "sm100_ptx.cuh"

namespace ntb200 {

// Raised (never cleared by kernels) when a bounded wait ran out.  Low byte = which wait.
__device__ unsigned int g_device_status = 0;

namespace {

constexpr int kBM = 128;
constexpr int kThreads = 192;
constexpr int kThreadsSplit = 320;  // Float32 split kernels: 8 epilogue warps hold the running sums in registers
constexpr int kTmemCols = 512;

enum OutKind : int { kOutF16 = 0, kOutBF16 = 1, kOutI8 = 2, kOutF32 = 3, kOutU32 = 4, kOutU16 = 5 };

struct UmmaParams {
    int m, n, k, batch;
    int tiles_m, tiles_n, k_blocks, group_m;
    int chunk_blocks;        // K blocks accumulated in tensor memory before the epilogue takes the partial sum
    int total_tiles;
    int block_k;             // elements per K block (128 bytes of K)
    uint32_t idesc;
    int a_mn_major, b_mn_major;
    int a_chunks, b_chunks;  // TMA loads per stage for an MN-major operand
    int chunk_mn;            // MN extent of one such load (128 bytes)
    uint32_t chunk_bytes;    // block_k * 128
    uint32_t a_lbo, b_lbo;   // leading byte offset of the shared-memory descriptor
    uint32_t a_kstep, b_kstep;  // start-address increment (16-byte units) per 32 bytes of K
    int a_batch_mul, b_batch_mul;  // 0 when the operand is shared by the whole batch
    void* c;
    long long c_rs, c_bs;
    const void* bias;
    long long bias_rs, bias_cs, bias_bs;
    int accumulate, out_kind, c_vec_ok;
    // Copies of C in other GPUs' memory (peer-mapped): the epilogue stores every finished tile there too.
    int n_peers;
    long long peer_offset[7];   // byte distance from this GPU's C to peer i's C (same layout)
    // Fused elementwise neighbours (16-bit outputs): tensors laid out exactly like C, given as byte offsets from C.
    int has_relu_out, has_mask;
    int shift;                   // kOutU32 / kOutU16: the s32 accumulator is shifted left by this much before it is added
    int tma_store;               // pair kernel, 16-bit outputs: tiles leave through shared memory and TMA stores
    int lean_ok;                 // pair kernel: a C with nothing fused may take the lean epilogue
    int peers_relu;              // TMA-store epilogue: the peer copies receive the fused ReLU output instead of C
    // Stage geometry of the single-CTA kernel (run-time: a problem with few rows stages only those rows of A and
    // spends the shared memory on more stages instead; the unused rows of the 128-row MMA operand alias whatever follows
    // in shared memory and only feed accumulator rows that are never stored)
    int s_stages;
    uint32_t s_a_bytes;          // bytes reserved per copy of the A tile (a multiple of 1024)
    uint32_t s_stage_bytes;      // A copies + B copies
    uint32_t s_stage_tx;         // bytes the TMA loads of one stage deliver
    long long relu_out_offset;   // second output: max(C, 0)
    long long mask_offset;       // input h: the result is zeroed where h < 0 (ReLU backward)
};

// Tensor maps of the peer-mapped copies of C (TMA-store epilogue of ntb200_gemm_push); only the first n_peers are valid.
struct PeerMaps {
    CUtensorMap m[7];
};

// kSplit: every operand is staged twice (high and low part of a Float32 split into two TF32 values).
template <int BN, bool kSplit = false>
struct Tile {
    static constexpr uint32_t kABytes = kBM * 128;
    static constexpr uint32_t kBBytes = BN * 128;
    static constexpr uint32_t kStageBytes = (kSplit ? 2u : 1u) * (kABytes + kBBytes);
    static constexpr int kStages = int(196608u / kStageBytes);   // 4 / 6 / 8 stages, half of that when split
    static constexpr int kMaxStages = 24;                        // ring length when few rows of A are staged
    static constexpr uint32_t kBarrierBytes = 512;               // 2 * kMaxStages + 4 barriers, TMEM slot, abort flag
    static constexpr uint32_t kRingBudget = 196608u + 16384u;    // shared memory the ring (plus one A tile of slack) may take
};

__device__ __forceinline__ void raise_timeout(volatile uint32_t* abort_flag, unsigned int where) {
    *abort_flag = 1;
    atomicExch(&g_device_status, 0x100u | where);
}

// n / d for 0 <= n < 2^22 and d >= 1 through the Float32 reciprocal (both are exact as floats, the quotient is off by
// less than one, one correction step): a quarter of the instructions of an integer division.  Every role of every
// CTA runs the tile scheduler once per tile, and for tiles with one or two K blocks it was a fifth of the tile's time.
__device__ __forceinline__ int small_div(int n, int d) {
    int q = __float2int_rz(__fdividef(__int2float_rn(n), __int2float_rn(d)));
    const int r = n - q * d;
    if (r < 0) --q;
    else if (r >= d) ++q;
    return q;
}

__device__ __forceinline__ void tile_coords(const UmmaParams& p, int t, int& b, int& mi, int& ni) {
    const int per_batch = p.tiles_m * p.tiles_n;
    const int group = p.group_m * p.tiles_n;
    if (p.total_tiles < (1 << 22)) {
        b = small_div(t, per_batch);
        const int r = t - b * per_batch;
        const int g = small_div(r, group);
        const int first_m = g * p.group_m;
        const int gm = min(p.group_m, p.tiles_m - first_m);
        const int w = r - g * group;
        ni = small_div(w, gm);
        mi = first_m + (w - ni * gm);
        return;
    }
    b = t / per_batch;
    const int r = t - b * per_batch;
    const int g = r / group;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, p.tiles_m - first_m);
    const int w = r - g * group;
    mi = first_m + w % gm;
    ni = w / gm;
}

__device__ __forceinline__ float to_float_bits16(uint32_t bits, int out_kind) {
    return out_kind == kOutF16 ? __half2float(__ushort_as_half((unsigned short)bits))
                               : __bfloat162float(__ushort_as_bfloat16((unsigned short)bits));
}
__device__ __forceinline__ uint32_t from_float_bits16(float v, int out_kind) {
    return out_kind == kOutF16 ? (uint32_t)__half_as_ushort(__float2half_rn(v))
                               : (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Two fp32 values rounded to nearest-even and packed (first value in the low half): one cvt.rn.{f16x2,bf16x2}.f32.
__device__ __forceinline__ uint32_t pack2_bits16(float lo, float hi, int out_kind) {
    if (out_kind == kOutF16) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Stores 32 consecutive Float32 results of one row (bias and previous C added first).
__device__ __forceinline__ void store_chunk_f32(const UmmaParams& p, int b, int row, int col0, const float* f_in) {
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = f_in[j];
    if (p.bias) {
        const float* bias = static_cast<const float*>(p.bias) + (long long)b * p.bias_bs + (long long)row * p.bias_rs;
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.n) f[j] += bias[(long long)(col0 + j) * p.bias_cs];
    }
    float* dst = static_cast<float*>(p.c) + (long long)b * p.c_bs + (long long)row * p.c_rs + col0;
    if (col0 + 32 <= p.n && p.c_vec_ok) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float4 o = make_float4(f[4 * q], f[4 * q + 1], f[4 * q + 2], f[4 * q + 3]);
            if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(dst + 4 * q);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(dst + 4 * q) = o;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.n) dst[j] = p.accumulate ? dst[j] + f[j] : f[j];
    }
}

// Two-level accumulation for the Float32 split kernels.  The tensor core adds into its fp32 accumulator with
// truncation, so a long chain drifts (about 2e-8 of the sum per MMA); the MMA warp therefore hands over a partial sum
// every `chunk_blocks` K blocks and the epilogue threads add the partial sums in registers with round-to-nearest.
template <int HC>
__device__ __forceinline__ void drain_partial(uint32_t taddr, float (&run)[HC], bool first) {
#pragma unroll
    for (int cc = 0; cc < HC / 32; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + uint32_t(cc * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
            run[cc * 32 + j] = first ? __uint_as_float(v[j]) : run[cc * 32 + j] + __uint_as_float(v[j]);
    }
}
template <int HC>
__device__ __forceinline__ void store_running(const UmmaParams& p, const float (&run)[HC], int b, int row, int col_base) {
    if (row >= p.m) return;
#pragma unroll
    for (int cc = 0; cc < HC / 32; ++cc)
        if (col_base + cc * 32 < p.n) store_chunk_f32(p, b, row, col_base + cc * 32, &run[cc * 32]);
}

// Epilogue of one 128-row accumulator slice: thread `row` of the tile reads its TMEM lane 32 columns at a time,
// adds the bias and / or the previous C, converts and stores.  `tmem_acc` already carries the warp's lane quadrant
// and the accumulator's first column.  Executed by whole warps (tcgen05.ld is warp-collective).
template <int BN>
__device__ __forceinline__ void epilogue_tile(const UmmaParams& p, uint32_t tmem_acc, int b, int row, int n0) {
    const int es = (p.out_kind == kOutI8) ? 1 : ((p.out_kind == kOutF32 || p.out_kind == kOutU32) ? 4 : 2);   // kOutU16: 2
    const bool row_ok = row < p.m;
    uint8_t* c_row = static_cast<uint8_t*>(p.c) + ((long long)b * p.c_bs + (long long)row * p.c_rs) * es;
#pragma unroll 1
    for (int cc = 0; cc < BN / 32; ++cc) {
        const int col0 = n0 + cc * 32;
        if (col0 >= p.n) break;  // uniform across the CTA
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_acc + uint32_t(cc * 32), v);
        tmem_ld_wait();
        if (!row_ok) continue;
        const bool full_chunk = (col0 + 32 <= p.n);
        if (p.out_kind == kOutI8) {
            // s32 accumulators; keep the low 8 bits (wrap), adding bias / previous C first
            if (p.bias) {
                const int8_t* bias = static_cast<const int8_t*>(p.bias) + (long long)b * p.bias_bs +
                                     (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) v[j] += (uint32_t)(int)bias[(long long)(col0 + j) * p.bias_cs];
            }
            uint8_t* dst = c_row + col0;
            if (full_chunk && p.c_vec_ok) {
                uint32_t packed[8];
                if (p.accumulate) {
                    const uint4 o0 = *reinterpret_cast<const uint4*>(dst);
                    const uint4 o1 = *reinterpret_cast<const uint4*>(dst + 16);
                    const uint32_t old[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += (old[j >> 2] >> (8 * (j & 3))) & 0xffu;
                }
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    packed[q] = (v[4 * q] & 0xffu) | ((v[4 * q + 1] & 0xffu) << 8) |
                                ((v[4 * q + 2] & 0xffu) << 16) | ((v[4 * q + 3] & 0xffu) << 24);
                *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) {
                        uint32_t x = v[j];
                        if (p.accumulate) x += dst[j];
                        dst[j] = (uint8_t)x;
                    }
            }
        } else if (p.out_kind == kOutU32) {
            // one limb product of a 32-bit integer GEMM: (acc << shift) joins C modulo 2^32
            uint32_t* dst = reinterpret_cast<uint32_t*>(c_row) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] <<= p.shift;
            if (p.bias) {
                const uint32_t* bias = static_cast<const uint32_t*>(p.bias) + (long long)b * p.bias_bs + (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) v[j] += bias[(long long)(col0 + j) * p.bias_cs];
            }
            if (full_chunk && p.c_vec_ok) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    uint4 o = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    if (p.accumulate) {
                        const uint4 old = *reinterpret_cast<const uint4*>(dst + 4 * q);
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    *reinterpret_cast<uint4*>(dst + 4 * q) = o;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
            }
        } else if (p.out_kind == kOutU16) {
            // one limb product of a 16-bit integer GEMM: (acc << shift) joins C modulo 2^16
            uint16_t* dst = reinterpret_cast<uint16_t*>(c_row) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] <<= p.shift;
            if (p.bias) {
                const uint16_t* bias = static_cast<const uint16_t*>(p.bias) + (long long)b * p.bias_bs + (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) v[j] += bias[(long long)(col0 + j) * p.bias_cs];
            }
            if (full_chunk && p.c_vec_ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
                    if (p.accumulate) {
                        const uint4 old = *reinterpret_cast<const uint4*>(dst + 8 * q);
                        const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            v[8 * q + 2 * j] += ow[j] & 0xffffu;
                            v[8 * q + 2 * j + 1] += ow[j] >> 16;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) w[j] = (v[8 * q + 2 * j] & 0xffffu) | (v[8 * q + 2 * j + 1] << 16);
                    *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) dst[j] = uint16_t(p.accumulate ? dst[j] + v[j] : v[j]);
            }
        } else if (p.out_kind == kOutF32) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            store_chunk_f32(p, b, row, col0, f);
        } else {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            if (p.bias) {
                const uint16_t* bias = static_cast<const uint16_t*>(p.bias) + (long long)b * p.bias_bs +
                                       (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) f[j] += to_float_bits16(bias[(long long)(col0 + j) * p.bias_cs], p.out_kind);
            }
            uint16_t* dst = reinterpret_cast<uint16_t*>(c_row) + col0;
            if (full_chunk && p.c_vec_ok) {
                if (p.accumulate) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * q);
                        const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            f[8 * q + 2 * j] += to_float_bits16(w[j] & 0xffffu, p.out_kind);
                            f[8 * q + 2 * j + 1] += to_float_bits16(w[j] >> 16, p.out_kind);
                        }
                    }
                }
                if (p.has_mask) {   // ReLU backward: no gradient where the forward input was negative
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 hq = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(dst + 8 * q) + p.mask_offset);
                        const uint32_t hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (to_float_bits16(hw[j] & 0xffffu, p.out_kind) < 0.f) f[8 * q + 2 * j] = 0.f;
                            if (to_float_bits16(hw[j] >> 16, p.out_kind) < 0.f) f[8 * q + 2 * j + 1] = 0.f;
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        w[j] = from_float_bits16(f[8 * q + 2 * j], p.out_kind) |
                               (from_float_bits16(f[8 * q + 2 * j + 1], p.out_kind) << 16);
                    const uint4 packed = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(dst + 8 * q) = packed;
                    if (p.has_relu_out) {   // second output: the activation, negatives (of the ROUNDED value) cleared
                        uint32_t r[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t lo = w[j] & 0xffffu, hi = w[j] >> 16;
                            r[j] = (to_float_bits16(lo, p.out_kind) < 0.f ? 0u : lo) |
                                   ((to_float_bits16(hi, p.out_kind) < 0.f ? 0u : hi) << 16);
                        }
                        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(dst + 8 * q) + p.relu_out_offset) =
                            make_uint4(r[0], r[1], r[2], r[3]);
                    }
                    // the same 16 bytes into every peer's copy of C (plain stores over NVLink)
                    for (int t = 0; t < p.n_peers; ++t)
                        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(dst + 8 * q) + p.peer_offset[t]) = packed;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) {
                        float x = f[j];
                        if (p.accumulate) x += to_float_bits16(dst[j], p.out_kind);
                        if (p.has_mask &&
                            to_float_bits16(*reinterpret_cast<const uint16_t*>(reinterpret_cast<const char*>(dst + j) + p.mask_offset),
                                            p.out_kind) < 0.f)
                            x = 0.f;
                        const uint16_t r16 = (uint16_t)from_float_bits16(x, p.out_kind);
                        dst[j] = r16;
                        if (p.has_relu_out)
                            *reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(dst + j) + p.relu_out_offset) =
                                to_float_bits16(r16, p.out_kind) < 0.f ? uint16_t(0) : r16;
                        for (int t = 0; t < p.n_peers; ++t)
                            *reinterpret_cast<uint16_t*>(reinterpret_cast<char*>(dst + j) + p.peer_offset[t]) = r16;
                    }
            }
        }
    }
}

// Epilogue of one warp's 32 x BN slice leaving through shared memory (16-bit and 8-bit outputs): every thread
// converts its row 32 columns at a time and writes them into the warp's staging buffer, laid out as sub-tiles of
// 32 rows x 128 bytes with the 128-byte swizzle (conflict-free for the 16-byte writes of 32 different rows); each
// finished sub-tile is handed to one TMA store, which writes whole 128-byte row segments and clips at the edges
// of C.  Bias, the previous C (accumulate) and the ReLU-backward mask are applied in registers first (the latter two
// read with the thread's own 16-byte loads); the fused ReLU output is a second sub-tile and a second store.
// `staging` is this warp's 16 KB = four 4 KB sub-tile buffers; a buffer is rewritten only after the store that
// last used it has finished reading it.
// `extra.apply<parity>(v, cc)` may change the 32 accumulator values of chunk cc before they are converted (K slices of a
// cluster add the other slices' partial sums there; parity = cc & 1, a constant, for hooks that keep one register set
// per parity); the default does nothing.
struct NoExtra {
    template <int kParity> __device__ __forceinline__ void apply(uint32_t (&)[32], int) const {}
};

template <int BN, class Extra = NoExtra>
__device__ __forceinline__ void epilogue_tile_tma(const UmmaParams& p, const CUtensorMap* tma_c, const CUtensorMap* tma_relu,
                                                  const PeerMaps* peers, uint32_t tmem_acc, uint32_t staging, int b, int row0,
                                                  int lane, int n0, const Extra extra = Extra()) {
    const int row = row0 + lane;
    const bool row_ok = row < p.m;
    const bool i8 = p.out_kind == kOutI8;
    const int es = i8 ? 1 : 2;
    const int per_sub = i8 ? 4 : 2;              // 32-column chunks per 128-byte sub-tile row
    const int pieces = i8 ? 2 : 4;               // 16-byte pieces one chunk contributes to a row
    const uint8_t* c_row = static_cast<const uint8_t*>(p.c) + ((long long)b * p.c_bs + (long long)row * p.c_rs) * es;
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
    // One 32-column chunk of this thread's row: convert, stage in shared memory, hand finished sub-tiles to TMA.
    auto process = [&](uint32_t (&v)[32], int cc) {
        const int col0 = n0 + cc * 32;
        const int sub = i8 ? (cc >> 2) : (cc >> 1), in_sub = cc - sub * per_sub;
        const int buf_c = p.has_relu_out ? ((2 * sub) & 3) : sub;
        if (p.has_relu_out && in_sub == 0 && sub >= 2) {   // buffers of sub-tile (sub - 2) come round again
            if (lane == 0) tma_store_wait_read_but2();
            __syncwarp();
        }
        const bool full_chunk = col0 + 32 <= p.n;
        uint32_t w[16];                            // the chunk's 32 outputs, packed (16-bit: 16 words, 8-bit: 8 words)
        if (i8) {
            if (p.bias && row_ok) {
                const int8_t* bias = static_cast<const int8_t*>(p.bias) + (long long)b * p.bias_bs + (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) v[j] += (uint32_t)(int)bias[(long long)(col0 + j) * p.bias_cs];
            }
            if (p.accumulate && row_ok) {
                if (full_chunk) {
                    const uint4 o0 = *reinterpret_cast<const uint4*>(c_row + col0);
                    const uint4 o1 = *reinterpret_cast<const uint4*>(c_row + col0 + 16);
                    const uint32_t old[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += (old[j >> 2] >> (8 * (j & 3))) & 0xffu;
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.n) v[j] += c_row[col0 + j];
                }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
                w[q] = (v[4 * q] & 0xffu) | ((v[4 * q + 1] & 0xffu) << 8) | ((v[4 * q + 2] & 0xffu) << 16) |
                       ((v[4 * q + 3] & 0xffu) << 24);
        } else {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            if (p.bias && row_ok) {
                const uint16_t* bias = static_cast<const uint16_t*>(p.bias) + (long long)b * p.bias_bs + (long long)row * p.bias_rs;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) f[j] += to_float_bits16(bias[(long long)(col0 + j) * p.bias_cs], p.out_kind);
            }
            if ((p.accumulate || p.has_mask) && row_ok) {
                const uint8_t* src = c_row + (long long)col0 * 2 + (p.has_mask ? p.mask_offset : 0);
                if (full_chunk) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 o = *reinterpret_cast<const uint4*>(src + 16 * q);
                        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float lo = to_float_bits16(ow[j] & 0xffffu, p.out_kind), hi = to_float_bits16(ow[j] >> 16, p.out_kind);
                            if (p.has_mask) {   // ReLU backward: no gradient where the forward input was negative
                                if (lo < 0.f) f[8 * q + 2 * j] = 0.f;
                                if (hi < 0.f) f[8 * q + 2 * j + 1] = 0.f;
                            } else {
                                f[8 * q + 2 * j] += lo;
                                f[8 * q + 2 * j + 1] += hi;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.n) {
                            const float o = to_float_bits16(reinterpret_cast<const uint16_t*>(src)[j], p.out_kind);
                            if (p.has_mask) { if (o < 0.f) f[j] = 0.f; } else f[j] += o;
                        }
                }
            }
            if (p.out_kind == kOutF16) {   // decided once per chunk, not once per pair of values
#pragma unroll
                for (int q = 0; q < 16; ++q) w[q] = pack2_bits16(f[2 * q], f[2 * q + 1], kOutF16);
            } else {
#pragma unroll
                for (int q = 0; q < 16; ++q) w[q] = pack2_bits16(f[2 * q], f[2 * q + 1], kOutBF16);
            }
        }
        const uint32_t row_c = staging + uint32_t(buf_c) * 4096u + uint32_t(lane) * 128u;
        for (int q = 0; q < pieces; ++q) {
            const uint32_t chunk = uint32_t(in_sub * pieces + q) ^ uint32_t(lane & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_c + (chunk << 4)), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                         "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
        }
        if (p.has_relu_out) {   // second output: the activation, negatives (of the ROUNDED value) cleared
            const uint32_t row_r = row_c + 4096u;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t lo = w[4 * q + j] & 0xffffu, hi = w[4 * q + j] >> 16;
                    r[j] = (to_float_bits16(lo, p.out_kind) < 0.f ? 0u : lo) | ((to_float_bits16(hi, p.out_kind) < 0.f ? 0u : hi) << 16);
                }
                const uint32_t chunk = uint32_t(in_sub * 4 + q) ^ uint32_t(lane & 7);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_r + (chunk << 4)), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                             "r"(r[3]) : "memory");
            }
        }
        if (in_sub == per_sub - 1 || col0 + 32 >= p.n) {   // the sub-tile is complete (or C ends inside it)
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                const int x0 = n0 + sub * per_sub * 32;
                tma_store_3d(tma_c, staging + uint32_t(buf_c) * 4096u, x0, row0, b);
                // the same sub-tile into every peer's copy: whole 128-byte row segments over NVLink
                if (!p.peers_relu)
                    for (int t = 0; t < p.n_peers; ++t) tma_store_3d(&peers->m[t], staging + uint32_t(buf_c) * 4096u, x0, row0, b);
                tma_store_commit();
                if (p.has_relu_out) {
                    tma_store_3d(tma_relu, staging + uint32_t(buf_c + 1) * 4096u, x0, row0, b);
                    if (p.peers_relu)
                        for (int t = 0; t < p.n_peers; ++t)
                            tma_store_3d(&peers->m[t], staging + uint32_t(buf_c + 1) * 4096u, x0, row0, b);
                    tma_store_commit();
                }
            }
        }
    };
    // The tensor-memory load of the next chunk is in flight while the current one is converted and staged (two
    // register sets, the loop unrolled by two so that both are addressed statically).  Loads past the last column of
    // C read accumulator columns that are never used; no load is left outstanding on return.
    constexpr int kChunks = BN / 32;
    static_assert(kChunks % 2 == 0, "the chunk loop is unrolled by two");
    uint32_t va[32], vb[32];
    tmem_ld_32x32b_x32(tmem_acc, va);
#pragma unroll 1
    for (int cc = 0; cc < kChunks; cc += 2) {
        if (n0 + cc * 32 >= p.n) break;  // uniform across the CTA
        tmem_ld_wait();
        tmem_ld_32x32b_x32(tmem_acc + uint32_t((cc + 1) * 32), vb);
        extra.template apply<0>(va, cc);
        process(va, cc);
        tmem_ld_wait();
        if (cc + 2 < kChunks) tmem_ld_32x32b_x32(tmem_acc + uint32_t((cc + 2) * 32), va);
        if (n0 + (cc + 1) * 32 < p.n) {
            extra.template apply<1>(vb, cc + 1);
            process(vb, cc + 1);
        }
    }
    tmem_ld_wait();
}

// The same for the commonest case: a 16-bit C with nothing fused (no bias, previous C, mask, second output or peer
// copy), NSUB sub-tiles of 64 columns.  Nothing is decided per value and little per chunk, so the warp issues a
// fraction of the instructions of the general epilogue.  kDouble keeps the next chunk's tensor-memory load in flight
// during the conversion (two register sets); the sixteen-warp instantiation, whose 96 registers per thread do not
// hold two chunks without spilling, takes one chunk at a time and lets the quadrant's other warps cover the latency.
// `staging` is NSUB x 4 KB; a sub-tile is handed to its TMA store as soon as its two chunks are staged.
template <int NSUB, bool kDouble>
__device__ __forceinline__ void epilogue_plain(const UmmaParams& p, const CUtensorMap* tma_c, uint32_t tmem_acc, uint32_t staging,
                                               int b, int row0, int lane, int n0) {
    if (n0 >= p.n) return;   // uniform across the CTA
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
    constexpr int kChunks = 2 * NSUB;
    const bool f16 = p.out_kind == kOutF16;
    auto emit = [&](const uint32_t (&v)[32], int cc) {
        uint32_t w[16];
        if (f16) {
#pragma unroll
            for (int q = 0; q < 16; ++q) w[q] = pack2_bits16(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]), kOutF16);
        } else {
#pragma unroll
            for (int q = 0; q < 16; ++q) w[q] = pack2_bits16(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]), kOutBF16);
        }
        const uint32_t sub = staging + uint32_t(cc >> 1) * 4096u;
        const uint32_t row_c = sub + uint32_t(lane) * 128u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t chunk = uint32_t((cc & 1) * 4 + q) ^ uint32_t(lane & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_c + (chunk << 4)), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                         "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
        }
        if ((cc & 1) || n0 + (cc + 1) * 32 >= p.n) {   // the sub-tile is complete, or C ends inside it (the store clips)
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(tma_c, sub, n0 + (cc >> 1) * 64, row0, b);
                tma_store_commit();
            }
        }
    };
    if constexpr (!kDouble) {
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
            if (n0 + cc * 32 >= p.n) break;
            uint32_t v[32];
            tmem_ld_32x32b_x32(tmem_acc + uint32_t(cc * 32), v);
            tmem_ld_wait();
            emit(v, cc);
        }
    } else {
        uint32_t va[32], vb[32];
        tmem_ld_32x32b_x32(tmem_acc, va);
#pragma unroll
        for (int cc = 0; cc < kChunks; cc += 2) {
            if (n0 + cc * 32 >= p.n) break;
            tmem_ld_wait();
            tmem_ld_32x32b_x32(tmem_acc + uint32_t((cc + 1) * 32), vb);   // past the last column of C: never used
            emit(va, cc);
            tmem_ld_wait();
            if (cc + 2 < kChunks) tmem_ld_32x32b_x32(tmem_acc + uint32_t((cc + 2) * 32), va);
            if (n0 + (cc + 1) * 32 < p.n) emit(vb, cc + 1);
        }
        tmem_ld_wait();
    }
}

template <MmaKind kKind, int BN, bool kSplit>
__global__ void __launch_bounds__(kSplit ? kThreadsSplit : kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_a_lo, const __grid_constant__ CUtensorMap tma_b_lo,
                 const UmmaParams p) {
    using T = Tile<BN, kSplit>;
    const int kStages = p.s_stages;   // run-time ring length (the name is kept from when it was a constant)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // the ring, then one A tile of slack (the last stage's 128-row operand view may run past its trimmed A region)
    const uint32_t ring_bytes = uint32_t(kStages) * p.s_stage_bytes + T::kABytes;
    uint8_t* bar_gen = smem_gen + ring_bytes;
    const uint32_t bar_base = smem_base + ring_bytes;
    // barrier layout (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kSplit ? 8 : 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                int b, mi, ni;
                tile_coords(p, t, b, mi, ni);
                const int m0 = mi * kBM, n0 = ni * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        raise_timeout(abort_flag, 1);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * p.s_stage_bytes;
                    const uint32_t b_dst = a_dst + (kSplit ? 2u : 1u) * p.s_a_bytes;
                    const uint32_t bar = full_bar(stage);
                    mbar_expect_tx(bar, p.s_stage_tx);
                    const int k0 = kb * p.block_k;
                    if constexpr (kSplit) {  // the split copies are dense and K-major
                        tma_load_3d(a_dst + p.s_a_bytes, &tma_a_lo, bar, k0, m0, b * p.a_batch_mul);
                        tma_load_3d(b_dst + T::kBBytes, &tma_b_lo, bar, k0, n0, b * p.b_batch_mul);
                    }
                    if (!p.a_mn_major) {
                        tma_load_3d(a_dst, &tma_a, bar, k0, m0, b * p.a_batch_mul);
                    } else {
                        for (int c = 0; c < p.a_chunks; ++c)
                            tma_load_3d(a_dst + c * p.chunk_bytes, &tma_a, bar, m0 + c * p.chunk_mn, k0,
                                        b * p.a_batch_mul);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d(b_dst, &tma_b, bar, k0, n0, b * p.b_batch_mul);
                    } else {
                        for (int c = 0; c < p.b_chunks; ++c)
                            tma_load_3d(b_dst + c * p.chunk_bytes, &tma_b, bar, n0 + c * p.chunk_mn, k0,
                                        b * p.b_batch_mul);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            // Leave no copy in flight behind us: wait (bounded) until the consumer has released every stage,
            // which implies every load issued above has landed.
            if (ok) {
                for (int s = 0; s < kStages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { raise_timeout(abort_flag, 2); break; }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x)
            for (int kb0 = 0; ok && kb0 < p.k_blocks; kb0 += p.chunk_blocks) {   // one accumulator per K chunk
                const int kb_end = min(p.k_blocks, kb0 + p.chunk_blocks);
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    raise_timeout(abort_flag, 3);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb_end; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        raise_timeout(abort_flag, 4);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_base + stage * p.s_stage_bytes;
                    const uint32_t b_addr = a_addr + (kSplit ? 2u : 1u) * p.s_a_bytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, p.a_lbo, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(b_addr, p.b_lbo, 1024);
                    if constexpr (kSplit) {
                        // a.b ~ a_lo.b_hi + a_hi.b_lo + a_hi.b_hi, all into the same fp32 accumulator
                        const uint64_t a_lo = make_smem_desc_sw128(a_addr + p.s_a_bytes, p.a_lbo, 1024);
                        const uint64_t b_lo = make_smem_desc_sw128(b_addr + T::kBBytes, p.b_lbo, 1024);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t ka = uint64_t(k * p.a_kstep), kbs = uint64_t(k * p.b_kstep);
                            umma<kKind, 1>(d_tmem, a_lo + ka, b_desc + kbs, p.idesc, ((kb - kb0) | k) != 0);
                            umma<kKind, 1>(d_tmem, a_desc + ka, b_lo + kbs, p.idesc, 1);
                            umma<kKind, 1>(d_tmem, a_desc + ka, b_desc + kbs, p.idesc, 1);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<kKind, 1>(d_tmem, a_desc + uint64_t(k * p.a_kstep), b_desc + uint64_t(k * p.b_kstep),
                                           p.idesc, ((kb - kb0) | k) != 0);
                    }
                    umma_commit<1>(empty_bar(stage));  // stage is free once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit<1>(tfull_bar(acc));        // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else if constexpr (kSplit) {
        // ------------------------------------------------------------------ epilogue, Float32 split: 8 warps, each
        // thread keeps the running sums of one row x BN/2 columns in registers
        constexpr int HC = BN / 2;
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int row_in_tile = quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        float run[HC];
        bool alive = true;
        for (int t = blockIdx.x; alive && t < p.total_tiles; t += gridDim.x) {
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            for (int kb0 = 0; kb0 < p.k_blocks; kb0 += p.chunk_blocks) {
                bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) raise_timeout(abort_flag, 6);
                    alive = false;
                    break;
                }
                tcgen05_fence_after();
                drain_partial<HC>(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + half * HC), run, kb0 == 0);
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (alive) store_running<HC>(p, run, b, mi * kBM + row_in_tile, ni * BN + half * HC);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        const int row_in_tile = quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) raise_timeout(abort_flag, 5);
                break;
            }
            tcgen05_fence_after();
            epilogue_tile<BN>(p, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN), b,
                              mi * kBM + row_in_tile, ni * BN);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// ---- pair kernel: two CTAs (the two SMs of a TPC, one cluster) share a 256 x 256 tile ------------------------
// tcgen05.mma.cta_group::2 computes rows [0,128) of the tile in the even CTA's tensor memory and rows [128,256)
// in the odd CTA's; each CTA stages only its own 128 rows of A and its own 128 of the tile's 256 B columns, so a
// K block costs each SM 32 KB of L2 traffic instead of 48 KB and the ring holds 6 stages instead of 4.
//   * both CTAs run a producer; every load credits the EVEN CTA's `full` barrier, whose producer posts the byte
//     count of both halves;
//   * only the even CTA issues MMAs; its commits are delivered to `empty` / `tmem_full` in BOTH CTAs;
//   * both CTAs run the epilogue on their own TMEM lanes and hand the accumulator back by arriving on the even
//     CTA's `tmem_empty` (8 arrivals: 4 warps x 2 CTAs).
// The loads are per-CTA copies of this GPU's own memory (no multicast).
constexpr uint32_t kPairOperandBytes = 128 * 128;                 // 128 rows (or 128 bytes of MN x block_k rows)
template <bool kSplit>
struct PairTile {
    static constexpr uint32_t kStageBytes = (kSplit ? 4u : 2u) * kPairOperandBytes;   // per CTA
    // Four to seven stages run at the same speed (the loads are not latency bound), so the plain kernel keeps five and
    // gives 64 KB to the output staging buffer of the TMA-store epilogue; the split kernel has three 64 KB stages.
    static constexpr int kStages = kSplit ? 3 : 5;
    static constexpr uint32_t kStagingBytes = kSplit ? 0u : 65536u;                   // 4 warps x 32 rows x 256 x 2 bytes
    static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kStagingBytes + 256 + 1024;
};

// kEpi = 8 (16- and 8-bit outputs through TMA stores, no second output): two epilogue warps per lane quadrant, each
// taking 128 of the tile's 256 columns, for shallow K where the epilogue, not the main loop, bounds a tile.
template <MmaKind kKind, bool kSplit, int kEpi = 4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kSplit ? kThreadsSplit : 64 + 32 * kEpi, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ CUtensorMap tma_a_lo, const __grid_constant__ CUtensorMap tma_b_lo,
                      const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_relu,
                      const __grid_constant__ PeerMaps tma_peers, const UmmaParams p) {
    constexpr int BN = 256;
    constexpr int kStages = PairTile<kSplit>::kStages;
    constexpr uint32_t kPairStageBytes = PairTile<kSplit>::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr uint32_t kStagingBytes = PairTile<kSplit>::kStagingBytes;
    const uint32_t staging_base = smem_base + kStages * kPairStageBytes;   // 1024-byte aligned
    uint8_t* bar_gen = smem_gen + kStages * kPairStageBytes + kStagingBytes;
    const uint32_t bar_base = staging_base + kStagingBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * kStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kSplit ? 16 : 2 * kEpi);   // one arrival per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        if (p.tma_store) tma_prefetch_desc(&tma_c);
        if (p.tma_store && p.has_relu_out) tma_prefetch_desc(&tma_relu);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before();
    cluster_sync_all();  // barriers of both CTAs are initialised before anything signals them remotely
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
                tile_coords(p, t, b, mi, ni);
                const int m0 = mi * 256 + int(rank) * 128, n0 = ni * BN + int(rank) * 128;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        raise_timeout(abort_flag, 0x11);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_base + stage * kPairStageBytes;
                    const uint32_t b_dst = a_dst + (kSplit ? 2u : 1u) * kPairOperandBytes;
                    const uint32_t bar = full_bar(stage);
                    if (leader) mbar_expect_tx(bar, 2 * kPairStageBytes);
                    const int k0 = kb * p.block_k;
                    if constexpr (kSplit) {
                        tma_load_3d_pair(a_dst + kPairOperandBytes, &tma_a_lo, bar, k0, m0, b * p.a_batch_mul);
                        tma_load_3d_pair(b_dst + kPairOperandBytes, &tma_b_lo, bar, k0, n0, b * p.b_batch_mul);
                    }
                    if (!p.a_mn_major) {
                        tma_load_3d_pair(a_dst, &tma_a, bar, k0, m0, b * p.a_batch_mul);
                    } else {
                        for (int c = 0; c < p.a_chunks; ++c)
                            tma_load_3d_pair(a_dst + c * p.chunk_bytes, &tma_a, bar, m0 + c * p.chunk_mn, k0,
                                             b * p.a_batch_mul);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d_pair(b_dst, &tma_b, bar, k0, n0, b * p.b_batch_mul);
                    } else {
                        for (int c = 0; c < p.b_chunks; ++c)
                            tma_load_3d_pair(b_dst + c * p.chunk_bytes, &tma_b, bar, n0 + c * p.chunk_mn, k0,
                                             b * p.b_batch_mul);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {  // drain: every stage released means every load of this CTA has landed and been consumed
                for (int s = 0; s < kStages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { raise_timeout(abort_flag, 0x12); break; }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
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
            for (int t = pair; ok && t < p.total_tiles; t += npairs)
            for (int kb0 = 0; ok && kb0 < p.k_blocks; kb0 += p.chunk_blocks) {
                const int kb_end = min(p.k_blocks, kb0 + p.chunk_blocks);
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) {
                    raise_timeout(abort_flag, 0x13);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb_end; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        raise_timeout(abort_flag, 0x14);
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_base + stage * kPairStageBytes;
                    const uint32_t b_addr = a_addr + (kSplit ? 2u : 1u) * kPairOperandBytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, p.a_lbo, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(b_addr, p.b_lbo, 1024);
                    if constexpr (kSplit) {
                        const uint64_t a_lo = make_smem_desc_sw128(a_addr + kPairOperandBytes, p.a_lbo, 1024);
                        const uint64_t b_lo = make_smem_desc_sw128(b_addr + kPairOperandBytes, p.b_lbo, 1024);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t ka = uint64_t(k * p.a_kstep), kbs = uint64_t(k * p.b_kstep);
                            umma<kKind, 2>(d_tmem, a_lo + ka, b_desc + kbs, p.idesc, ((kb - kb0) | k) != 0);
                            umma<kKind, 2>(d_tmem, a_desc + ka, b_lo + kbs, p.idesc, 1);
                            umma<kKind, 2>(d_tmem, a_desc + ka, b_desc + kbs, p.idesc, 1);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<kKind, 2>(d_tmem, a_desc + uint64_t(k * p.a_kstep), b_desc + uint64_t(k * p.b_kstep),
                                           p.idesc, ((kb - kb0) | k) != 0);
                    }
                    umma_commit_pair(empty_bar(stage), 3);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(acc), 3);
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else if constexpr (kSplit) {
        // ------------------------------------------------------------------ epilogue, Float32 split (both CTAs)
        constexpr int HC = BN / 2;
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int row_in_tile = int(rank) * 128 + quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        float run[HC];
        bool alive = true;
        for (int t = pair; alive && t < p.total_tiles; t += npairs) {
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            for (int kb0 = 0; kb0 < p.k_blocks; kb0 += p.chunk_blocks) {
                bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) raise_timeout(abort_flag, 0x16);
                    alive = false;
                    break;
                }
                tcgen05_fence_after();
                drain_partial<HC>(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + half * HC), run, kb0 == 0);
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(tempty_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
            if (alive) store_running<HC>(p, run, b, mi * 256 + row_in_tile, ni * BN + half * HC);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int quad = warp & 3;
        const int row_in_tile = int(rank) * 128 + quad * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = pair; t < p.total_tiles; t += npairs) {
            int b, mi, ni;
            tile_coords(p, t, b, mi, ni);
            bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) raise_timeout(abort_flag, 0x15);
                break;
            }
            tcgen05_fence_after();
            // a 16-bit C with nothing fused takes the lean epilogue (NTB200_GENERAL_EPILOGUE=1 sets p.lean_ok to 0)
            const bool plain = p.tma_store && p.lean_ok && !p.bias && !p.accumulate && !p.has_mask && !p.has_relu_out &&
                               p.n_peers == 0 && p.out_kind != kOutI8;
            if constexpr (!kSplit && kEpi == 16) {
                const int quarter = (warp - 2) >> 2;   // four warps per lane quadrant, 64 columns (one 128-byte sub-tile) each
                if (plain)
                    epilogue_plain<1, false>(p, &tma_c, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + quarter * 64),
                                             staging_base + uint32_t(warp - 2) * 4096u, b, mi * 256 + int(rank) * 128 + quad * 32, lane,
                                             ni * BN + quarter * 64);
                else if (p.tma_store)
                    epilogue_tile_tma<64>(p, &tma_c, &tma_relu, &tma_peers,
                                          tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + quarter * 64),
                                          staging_base + uint32_t(warp - 2) * 4096u, b, mi * 256 + int(rank) * 128 + quad * 32,
                                          lane, ni * BN + quarter * 64);
                else
                    epilogue_tile<64>(p, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + quarter * 64), b,
                                      mi * 256 + row_in_tile, ni * BN + quarter * 64);
            } else if constexpr (!kSplit && kEpi == 8) {
                const int half = (warp - 2) >> 2;   // warps 2-5: columns 0-127, warps 6-9: columns 128-255
                if (plain)
                    epilogue_plain<2, true>(p, &tma_c, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + half * 128),
                                            staging_base + uint32_t(warp - 2) * 8192u, b, mi * 256 + int(rank) * 128 + quad * 32, lane,
                                            ni * BN + half * 128);
                else if (p.tma_store)
                    epilogue_tile_tma<128>(p, &tma_c, &tma_relu, &tma_peers,
                                           tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + half * 128),
                                           staging_base + uint32_t(warp - 2) * 8192u, b, mi * 256 + int(rank) * 128 + quad * 32,
                                           lane, ni * BN + half * 128);
                else
                    epilogue_tile<128>(p, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN + half * 128), b,
                                       mi * 256 + row_in_tile, ni * BN + half * 128);
            } else if constexpr (!kSplit) {
                if (plain)
                    epilogue_plain<BN / 64, true>(p, &tma_c, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN),
                                                  staging_base + uint32_t(quad) * 16384u, b, mi * 256 + int(rank) * 128 + quad * 32, lane,
                                                  ni * BN);
                else if (p.tma_store)
                    epilogue_tile_tma<BN>(p, &tma_c, &tma_relu, &tma_peers, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN),
                                          staging_base + uint32_t(quad) * 16384u, b, mi * 256 + int(rank) * 128 + quad * 32,
                                          lane, ni * BN);
                else
                    epilogue_tile<BN>(p, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN), b,
                                      mi * 256 + row_in_tile, ni * BN);
            } else {
                epilogue_tile<BN>(p, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN), b,
                                  mi * 256 + row_in_tile, ni * BN);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();   // the last tiles' stores are complete before the CTA leaves
    }

    // ---------------------------------------------------------------------- teardown
    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}


// ---- K slices inside a thread-block cluster ---------------------------------------------------------------------
// Few rows against a large weight matrix are bound by reading the weights once, and a CTA streams them fastest on
// wide tiles (bytes per issued instruction), of which a narrow output has too few to occupy every SM.  Here the S
// CTAs of a cluster work on ONE 128 x BN output tile, each on its own slice of K: CTA r accumulates its partial tile
// in tensor memory, spills it as fp32 into its own shared memory (over the operand ring, which is idle by then), and
// after a cluster barrier CTA r adds columns [r BN/S, (r+1) BN/S) of all S partial tiles in slice order through
// distributed shared memory, adds the bias and the previous C, rounds once and stores.  One launch, no partial tile
// ever travels through HBM, and the sum order is fixed (slice 0, 1, ..., S-1), so results are reproducible.
// Not persistent: one tile per cluster.  Roles as in umma_gemm_kernel; every wait is bounded.
struct ClusterKParams {
    UmmaParams u;          // geometry, operands, epilogue inputs (batch == 1)
    int slices;            // S = cluster size
    int blocks_per_slice;  // K blocks per slice (the last slice may have fewer, never zero)
    int pitch;             // floats per row of a partial tile in shared memory (BN + 4)
    int rows_live;         // rows of a tile that can hold results (min(128, m)), rounded up to 32
    int c_wide_ok;         // C and its rows are 8-byte aligned: four results leave in one store
    float* exchange;       // pair clusters: scratch the partial tiles cross the K slices through (L2-resident); null = distributed shared memory
    int c_tma_ok;          // pair clusters: C can be written by TMA stores (16-byte aligned rows), see plan_store
};

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_addr, uint32_t cta_rank) {
    float4 v;
    asm volatile(
        "{\n\t.reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %4, %5;\n\t"
        "ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [remote];\n\t}"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(local_addr), "r"(cta_rank) : "memory");
    return v;
}


// Sum of the S partial tiles of a cluster for this CTA's share of the columns, then bias, previous C, one rounding and
// the store.  The partial tiles sit at the same shared-memory offset (`tile_base`, row pitch cp.pitch floats) in the S
// CTAs with ranks rank_first, rank_first + rank_stride, ...; they are added in that order.  A read of a neighbour's
// shared memory takes several hundred cycles, so every thread first issues the reads of U items x S slices and only
// then starts adding: the latency is paid once per batch, not once per read.
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

template <int S, int U>
__device__ __forceinline__ void cluster_reduce_store(const UmmaParams& p, const ClusterKParams& cp, uint32_t tile_base, int rows,
                                                     int m_base, int n_base, int col_first, int cols_mine, uint32_t rank_first,
                                                     uint32_t rank_stride, int my_slice) {
    const int groups = cols_mine >> 2;
    const int items = rows * groups;
    const int threads = int(blockDim.x);
    for (int base = threadIdx.x; base < items; base += threads * U) {
        float4 v[U][S];
        int row[U], gcol[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * threads;
            const bool live = i < items;
            row[u] = live ? i / groups : 0;
            gcol[u] = live ? (i - row[u] * groups) * 4 + col_first : col_first;
            const uint32_t addr = tile_base + uint32_t(row[u] * cp.pitch + gcol[u]) * 4u;
#pragma unroll
            for (int sl = 0; sl < S; ++sl)     // this CTA's own partial is a plain shared-memory read; only the others cross the cluster
                v[u][sl] = sl == my_slice ? ld_shared_f4(addr) : ld_cluster_f4(addr, rank_first + uint32_t(sl) * rank_stride);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * threads;
            const int col = n_base + gcol[u];
            if (i >= items || col >= p.n) continue;
            float4 acc = v[u][0];
#pragma unroll
            for (int sl = 1; sl < S; ++sl) { acc.x += v[u][sl].x; acc.y += v[u][sl].y; acc.z += v[u][sl].z; acc.w += v[u][sl].w; }
            float f[4] = {acc.x, acc.y, acc.z, acc.w};
            const int grow = m_base + row[u];
            uint16_t* dst = static_cast<uint16_t*>(p.c) + (long long)grow * p.c_rs + col;
            const uint16_t* bias = static_cast<const uint16_t*>(p.bias);
            uint32_t r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (col + j < p.n) {
                    if (bias) f[j] += to_float_bits16(bias[(long long)grow * p.bias_rs + (long long)(col + j) * p.bias_cs], p.out_kind);
                    if (p.accumulate) f[j] += to_float_bits16(dst[j], p.out_kind);
                }
                r[j] = from_float_bits16(f[j], p.out_kind);
            }
            if (cp.c_wide_ok && col + 4 <= p.n) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(r[0] | (r[1] << 16), r[2] | (r[3] << 16));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (col + j < p.n) dst[j] = uint16_t(r[j]);
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_cluster_k_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const ClusterKParams cp) {
    using T = Tile<BN, false>;
    const UmmaParams& p = cp.u;
    const int kStages = p.s_stages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t ring_bytes = uint32_t(kStages) * p.s_stage_bytes + T::kABytes;
    uint8_t* bar_gen = smem_gen + ring_bytes;
    const uint32_t bar_base = smem_base + ring_bytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * kStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * kStages + 1));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int tile = blockIdx.x / cp.slices;
    const int mi = tile / p.tiles_n, ni = tile - mi * p.tiles_n;
    const int m0 = mi * kBM, n0 = ni * BN;
    const int kb_begin = int(rank) * cp.blocks_per_slice;
    const int kb_end = min(p.k_blocks, kb_begin + cp.blocks_per_slice);

    // One K block into one stage (thread 0 only: it is the producer, before and after the block-wide barrier).
    auto load_stage = [&](int kb, int stage) {
        const uint32_t a_dst = smem_base + stage * p.s_stage_bytes;
        const uint32_t b_dst = a_dst + p.s_a_bytes;
        const uint32_t bar = full_bar(stage);
        mbar_expect_tx(bar, p.s_stage_tx);
        const int k0 = kb * p.block_k;
        if (!p.a_mn_major) {
            tma_load_3d(a_dst, &tma_a, bar, k0, m0, 0);
        } else {
            for (int c = 0; c < p.a_chunks; ++c) tma_load_3d(a_dst + c * p.chunk_bytes, &tma_a, bar, m0 + c * p.chunk_mn, k0, 0);
        }
        if (!p.b_mn_major) {
            tma_load_3d(b_dst, &tma_b, bar, k0, n0, 0);
        } else {
            for (int c = 0; c < p.b_chunks; ++c) tma_load_3d(b_dst + c * p.chunk_bytes, &tma_b, bar, n0 + c * p.chunk_mn, k0, 0);
        }
    };
    // The first loads leave before the tensor-memory allocation and the block-wide barrier: every barrier they use is
    // this CTA's own and was initialised by this very thread, the ring is empty, and the weights' first bytes are what
    // the kernel waits for longest.
    int prefilled = 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        prefilled = min(min(4, kStages), kb_end - kb_begin);
        for (int i = 0; i < prefilled; ++i) load_stage(kb_begin + i, i);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_slot)), BN);
        tmem_relinquish<1>();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer: this slice's K blocks
        if (lane == 0) {
            int stage = prefilled == kStages ? 0 : prefilled;       // the stages filled before the barrier come first
            uint32_t phase = prefilled == kStages ? 1u : 0u;
            bool ok = true;
            for (int kb = kb_begin + prefilled; kb < kb_end; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    raise_timeout(abort_flag, 0x21);
                    ok = false;
                    break;
                }
                load_stage(kb, stage);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) {   // leave no copy in flight: every stage released means every load has landed and been consumed
                for (int s = 0; s < kStages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { raise_timeout(abort_flag, 0x22); break; }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    raise_timeout(abort_flag, 0x24);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_base + stage * p.s_stage_bytes;
                const uint64_t a_desc = make_smem_desc_sw128(a_addr, p.a_lbo, 1024);
                const uint64_t b_desc = make_smem_desc_sw128(a_addr + p.s_a_bytes, p.b_lbo, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma<MmaKind::f16, 1>(tmem_base, a_desc + uint64_t(k * p.a_kstep), b_desc + uint64_t(k * p.b_kstep), p.idesc,
                                          ((kb - kb_begin) | k) != 0);
                umma_commit<1>(empty_bar(stage));
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit<1>(tfull_bar);   // this slice's partial tile is complete
        }
    }
    __syncwarp();   // the other lanes of the producer and MMA warps wait here until their lane 0 is through its loop
    {
        // ------------------------------------------------------------------ spill the partial tile to shared memory
        // A warp reads the 32 tensor-memory lanes of quadrant warp % 4, so rows 0-63 have two warps each (0 and 4, 1
        // and 5: the producer and MMA warps are free by now) and share their chunks; with few rows, where only the
        // first quadrants hold results, that halves the longest serial piece of the kernel's tail.
        const int quad = warp & 3;
        const int part = warp >> 2, parts = quad < 2 ? 2 : 1;
        bool ok = mbar_wait(tfull_bar, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) raise_timeout(abort_flag, 0x25);
        } else if (quad * 32 < cp.rows_live) {
            tcgen05_fence_after();
            // the ring is idle (every MMA has completed, so every load has been consumed): the partial tile goes there
            float* dst = reinterpret_cast<float*>(smem_gen) + (quad * 32 + lane) * cp.pitch;
#pragma unroll 1
            for (int cc = part; cc < BN / 32; cc += parts) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(cc * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    *reinterpret_cast<float4*>(dst + cc * 32 + 4 * q) =
                        make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
            }
            tcgen05_fence_before();
        }
    }

    // ---------------------------------------------------------------------- reduce across the cluster
    __syncwarp();
    cluster_sync_all();   // every CTA's partial tile is in its shared memory (or its abort flag is up)
    if (*abort_flag == 0) {
        const int cols_mine = BN / cp.slices;               // a multiple of 4 (BN 128 / 256, S <= 8)
        const int rows = min(kBM, p.m - m0);
        const int col_first = int(rank) * cols_mine;
        switch (cp.slices) {
            case 2: cluster_reduce_store<2, 8>(p, cp, smem_base, rows, m0, n0, col_first, cols_mine, 0u, 1u, int(rank)); break;
            case 4: cluster_reduce_store<4, 4>(p, cp, smem_base, rows, m0, n0, col_first, cols_mine, 0u, 1u, int(rank)); break;
            default: cluster_reduce_store<8, 2>(p, cp, smem_base, rows, m0, n0, col_first, cols_mine, 0u, 1u, int(rank)); break;
        }
    }
    // nobody leaves while a neighbour may still read its shared memory
    tcgen05_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<1>(tmem_base, BN);
    }
}

// Pair clusters, exchange through L2: the epilogue warp of lane quadrant `quad` adds, for the 32-column chunks this CTA
// owns, its own partial (tensor memory) and the partials the other S - 1 slices left in scratch, in slice order, and
// writes the sums into the staged tile in shared memory (row pitch cp.pitch floats).  A scratch region holds one CTA's
// 128 x 256 partial as [quad][chunk][piece][lane] float4: the thread that owns a row writes and reads 16-byte pieces
// that neighbour its warp's other lanes, so every warp access covers whole 512-byte runs.
constexpr int kExchangeRegion = 4 * 8 * 8 * 32;   // float4 per CTA

template <int S>
__device__ __forceinline__ void pair_cluster_sum_chunks(const ClusterKParams& cp, uint32_t tmem_base, float* staged, int quad, int lane,
                                                        int tile, int slice, uint32_t half) {
    constexpr int kChunks = 8 / S;
    const float4* regions = reinterpret_cast<const float4*>(cp.exchange) + size_t(tile) * (2 * S) * kExchangeRegion;
    float* dst = staged + (quad * 32 + lane) * cp.pitch;
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
        const int cc = slice * kChunks + i;
        float4 r[S][8];
#pragma unroll
        for (int sl = 0; sl < S; ++sl) {
            if (sl == slice) continue;
            const float4* src = regions + size_t(2 * sl + int(half)) * kExchangeRegion + ((quad * 8 + cc) * 8) * 32 + lane;
#pragma unroll
            for (int q = 0; q < 8; ++q) r[sl][q] = __ldcg(src + q * 32);
        }
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(cc * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 own = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                           __uint_as_float(v[4 * q + 3]));
            float4 acc = slice == 0 ? own : r[0][q];
#pragma unroll
            for (int sl = 1; sl < S; ++sl) {
                const float4 t = sl == slice ? own : r[sl][q];
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            *reinterpret_cast<float4*>(dst + cc * 32 + 4 * q) = acc;
        }
    }
}


// The same sum as pair_cluster_sum_chunks, as the hook of epilogue_tile_tma: the chunk's own partial arrives in `v`
// (tensor memory), the other slices' partials are read from scratch, and the slice-ordered sum replaces `v`.
template <int S>
struct ExchangeAdd {
    const float4* regions;   // the 2 S regions of this tile
    int quad, lane, slice, half, chunk0;
    template <int kParity> __device__ __forceinline__ void apply(uint32_t (&v)[32], int cc) const {
        float4 r[S][8];
#pragma unroll
        for (int sl = 0; sl < S; ++sl) {
            if (sl == slice) continue;
            const float4* src = regions + size_t(2 * sl + half) * kExchangeRegion + ((quad * 8 + chunk0 + cc) * 8) * 32 + lane;
#pragma unroll
            for (int q = 0; q < 8; ++q) r[sl][q] = __ldcg(src + q * 32);
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 own = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                           __uint_as_float(v[4 * q + 3]));
            float4 acc = slice == 0 ? own : r[0][q];
#pragma unroll
            for (int sl = 1; sl < S; ++sl) {
                const float4 t = sl == slice ? own : r[sl][q];
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            v[4 * q] = __float_as_uint(acc.x); v[4 * q + 1] = __float_as_uint(acc.y);
            v[4 * q + 2] = __float_as_uint(acc.z); v[4 * q + 3] = __float_as_uint(acc.w);
        }
    }
};

// ---- K slices of CTA pairs inside one cluster ---------------------------------------------------------------------
// A few hundred rows against a large weight matrix give fewer 256 x 256 tiles than the GPU has CTA pairs, and an SM
// takes in operands from L2 at a fixed rate (about 64 bytes per clock), so the time of a tile is its K blocks times
// that rate whatever else happens: the only way to finish sooner is more SMs on the same tile.  Here a cluster of
// 2 S CTAs = S pairs computes ONE 256 x 256 tile, pair s on K slice s (tcgen05.mma.cta_group::2 exactly as in
// umma_gemm_pair_kernel: even CTA rows 0-127, odd CTA rows 128-255, each staging its own halves of A and B).  Every
// CTA then spills its 128 x 256 fp32 partial tile into its own shared memory (over the idle ring), and after a
// cluster barrier the S CTAs that hold the same rows each add one S-th of the columns over all S slices, in slice
// order, through distributed shared memory; bias and previous C are added, the sum is rounded once and stored.
// One launch, no partial tile in HBM, reproducible sum order.  One tile per cluster (not persistent).
// Two slices, two chunks per warp: the other slice's partials of both chunks are requested before the first
// tensor-memory load is waited for, so the L2 latency is paid once (set r[parity][piece] with load()).
struct ExchangePair {
    float4 r[2][8];
    int slice;
    __device__ __forceinline__ void load(const float4* regions, int quad, int lane, int half, int chunk0) {
        const float4* src = regions + size_t(2 * (slice ^ 1) + half) * kExchangeRegion + ((quad * 8 + chunk0) * 8) * 32 + lane;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int q = 0; q < 8; ++q) r[c][q] = __ldcg(src + (c * 8 + q) * 32);
    }
    template <int kParity> __device__ __forceinline__ void apply(uint32_t (&v)[32], int) const {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 own = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                           __uint_as_float(v[4 * q + 3]));
            const float4 oth = r[kParity][q];
            const float4 first = slice == 0 ? own : oth, second = slice == 0 ? oth : own;   // slice order: 0 then 1
            v[4 * q] = __float_as_uint(first.x + second.x); v[4 * q + 1] = __float_as_uint(first.y + second.y);
            v[4 * q + 2] = __float_as_uint(first.z + second.z); v[4 * q + 3] = __float_as_uint(first.w + second.w);
        }
    }
};

constexpr int kPairClusterThreads = 256;   // eight warps, two per lane quadrant; lane 0 of warps 0 and 1 feed and issue the main loop first

template <int kDummy>
__global__ void __launch_bounds__(kPairClusterThreads, 1)
umma_gemm_pair_cluster_k_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                                const __grid_constant__ CUtensorMap tma_c, const ClusterKParams cp) {
    constexpr int BN = 256;
    constexpr int kStages = 6;
    constexpr uint32_t kStageBytes = 2u * kPairOperandBytes;   // per CTA: its 128 rows of A, its 128 columns of B
    const UmmaParams& p = cp.u;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* bar_gen = smem_gen + kStages * kStageBytes;
    const uint32_t bar_base = smem_base + kStages * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * kStages);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * kStages + 1));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const uint32_t half = rank & 1u;              // 0: rows 0-127 of the tile (the pair's MMA leader), 1: rows 128-255
    const int slice = int(rank >> 1);
    const bool leader = half == 0;
    const int tile = blockIdx.x / (2 * cp.slices);
    const int mi = tile / p.tiles_n, ni = tile - mi * p.tiles_n;
    const int m0 = mi * 256 + int(half) * 128, n0_pair = ni * BN;
    const int kb_begin = slice * cp.blocks_per_slice;
    const int kb_end = min(p.k_blocks, kb_begin + cp.blocks_per_slice);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tma_a);
        tma_prefetch_desc(&tma_b);
        if (cp.c_tma_ok) tma_prefetch_desc(&tma_c);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_slot)), BN);
        tmem_relinquish<2>();
    }
    tcgen05_fence_before();
    cluster_sync_all();  // barriers of every CTA are initialised before anything signals them remotely
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (every CTA, its own halves)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const int n0 = n0_pair + int(half) * 128;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    raise_timeout(abort_flag, 0x31);
                    ok = false;
                    break;
                }
                const uint32_t a_dst = smem_base + stage * kStageBytes;
                const uint32_t b_dst = a_dst + kPairOperandBytes;
                const uint32_t bar = full_bar(stage);
                if (leader) mbar_expect_tx(bar, 2 * kStageBytes);   // both CTAs' loads credit the even CTA's barrier
                const int k0 = kb * p.block_k;
                if (!p.a_mn_major) {
                    tma_load_3d_pair(a_dst, &tma_a, bar, k0, m0, 0);
                } else {
                    for (int c = 0; c < p.a_chunks; ++c) tma_load_3d_pair(a_dst + c * p.chunk_bytes, &tma_a, bar, m0 + c * p.chunk_mn, k0, 0);
                }
                if (!p.b_mn_major) {
                    tma_load_3d_pair(b_dst, &tma_b, bar, k0, n0, 0);
                } else {
                    for (int c = 0; c < p.b_chunks; ++c) tma_load_3d_pair(b_dst + c * p.chunk_bytes, &tma_b, bar, n0 + c * p.chunk_mn, k0, 0);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) {
                for (int s = 0; s < kStages; ++s) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { raise_timeout(abort_flag, 0x32); break; }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (even CTA of each pair)
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint16_t pair_mask = uint16_t(3u << (rank & ~1u));   // the two CTAs of this pair, by rank in the cluster
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    raise_timeout(abort_flag, 0x34);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_base + stage * kStageBytes;
                const uint64_t a_desc = make_smem_desc_sw128(a_addr, p.a_lbo, 1024);
                const uint64_t b_desc = make_smem_desc_sw128(a_addr + kPairOperandBytes, p.b_lbo, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma<MmaKind::f16, 2>(tmem_base, a_desc + uint64_t(k * p.a_kstep), b_desc + uint64_t(k * p.b_kstep), p.idesc,
                                          ((kb - kb_begin) | k) != 0);
                umma_commit_pair(empty_bar(stage), pair_mask);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit_pair(tfull_bar, pair_mask);
        }
    }
    __syncwarp();   // the other lanes of the producer and MMA warps wait here, without issuing, until their lane 0 is done
    {
        // ------------------------------------------------------------------ all eight warps: this CTA's 128 x 256 partial tile
        // (one tile per cluster, so the epilogue never overlaps a main loop and the two role warps can join it)
        const int quad = warp & 3, part = warp >> 2;   // two warps per lane quadrant
        bool ok = mbar_wait(tfull_bar, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) raise_timeout(abort_flag, 0x35);
        } else {
            tcgen05_fence_after();
            if (cp.exchange) {
                // the chunks other slices own leave for their owners through L2 (coalesced 16-byte pieces, see above)
                float4* mine = reinterpret_cast<float4*>(cp.exchange) + (size_t(blockIdx.x) * 4 + quad) * (8 * 8 * 32) + lane;
                const int chunks_per_slice = 8 / cp.slices;
                int turn = 0;
#pragma unroll 1
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc / chunks_per_slice == slice) continue;
                    if ((turn++ & 1) != part) continue;           // the quadrant's two warps take the foreign chunks in turn
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(cc * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        __stcg(mine + (cc * 8 + q) * 32,
                               make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
                }
            } else {
                float* dst = reinterpret_cast<float*>(smem_gen) + (quad * 32 + lane) * cp.pitch;
#pragma unroll 1
                for (int cc = part; cc < BN / 32; cc += 2) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(cc * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4*>(dst + cc * 32 + 4 * q) =
                            make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                }
            }
            tcgen05_fence_before();
        }
    }

    // ---------------------------------------------------------------------- reduce across the slices
    __syncwarp();
    cluster_sync_all();
    if (*abort_flag == 0) {
        // the S CTAs with this row half share the tile's 256 columns: this one takes columns [slice, slice + 1) * 256 / S
        const int cols_mine = BN / cp.slices;
        const int rows = max(0, min(128, p.m - m0));
        if (cp.exchange && cp.c_tma_ok) {
            // sums are formed in registers, converted, staged 32 rows x 128 bytes at a time over the idle ring and leave
            // as TMA stores (whole 128-byte row segments): no copy-out pass
            {
                tcgen05_fence_after();
                const int quad = warp & 3, part = warp >> 2;
                const float4* regions = reinterpret_cast<const float4*>(cp.exchange) + size_t(tile) * (2 * cp.slices) * kExchangeRegion;
                const uint32_t staging = smem_base + uint32_t(warp) * 4096u;    // one 32-row x 128-byte sub-tile per warp
                if (cp.slices == 2) {      // 128 columns: each of the quadrant's two warps takes 64 of them (two chunks)
                    const int col = slice * cols_mine + part * 64;
                    ExchangePair ex;
                    ex.slice = slice;
                    ex.load(regions, quad, lane, int(half), col / 32);
                    epilogue_tile_tma<64>(p, &tma_c, &tma_c, nullptr, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(col), staging, 0,
                                          m0 + quad * 32, lane, n0_pair + col, ex);
                } else if (part == 0) {   // 64 columns = one sub-tile: one warp per quadrant
                    const int col = slice * cols_mine;
                    epilogue_tile_tma<64>(p, &tma_c, &tma_c, nullptr, tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(col), staging, 0,
                                          m0 + quad * 32, lane, n0_pair + col, ExchangeAdd<4>{regions, quad, lane, slice, int(half), slice * 2});
                }
                if (lane == 0) tma_store_wait_all();
                tcgen05_fence_before();
            }
        } else if (cp.exchange) {
            if (warp < 4) {
                tcgen05_fence_after();
                if (cp.slices == 2) pair_cluster_sum_chunks<2>(cp, tmem_base, reinterpret_cast<float*>(smem_gen), warp & 3, lane, tile, slice, half);
                else pair_cluster_sum_chunks<4>(cp, tmem_base, reinterpret_cast<float*>(smem_gen), warp & 3, lane, tile, slice, half);
                tcgen05_fence_before();
            }
            __syncthreads();
            // the staged sums leave with bias, previous C and one rounding, coalesced along the rows
            cluster_reduce_store<1, 8>(p, cp, smem_base, rows, m0, n0_pair, slice * cols_mine, cols_mine, 0u, 0u, 0);
        } else if (cp.slices == 2) {
            cluster_reduce_store<2, 8>(p, cp, smem_base, rows, m0, n0_pair, slice * cols_mine, cols_mine, half, 2u, slice);
        } else {
            cluster_reduce_store<4, 4>(p, cp, smem_base, rows, m0, n0_pair, slice * cols_mine, cols_mine, half, 2u, slice);
        }
    }
    tcgen05_fence_before();
    cluster_sync_all();   // nobody leaves while a neighbour may still read its shared memory or signal its barriers
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc<2>(tmem_base, BN);
    }
}

// ---- host side ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoded tensor maps of the calling thread's most recent operands.  cuTensorMapEncodeTiled costs about a
// microsecond of host time per map and a GEMM needs three to five; a training or inference loop presents the same
// pointers, shapes and strides again and again.  The map depends on nothing but these arguments.
struct MapKey {
    const void* ptr;
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    int32_t dt, swizzle;
};
CUresult encode_cached(CUtensorMap* out, CUtensorMapDataType dt, void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
                       const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return CUDA_ERROR_NOT_SUPPORTED;
    constexpr int kEntries = 32;
    struct Entry { MapKey key; CUtensorMap map; bool used; };
    thread_local Entry cache[kEntries] = {};
    thread_local int next = 0;
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    key.ptr = ptr;
    for (int i = 0; i < 3; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    key.strides[0] = strides[0]; key.strides[1] = strides[1];
    key.dt = int32_t(dt); key.swizzle = int32_t(swizzle);
    for (int i = 0; i < kEntries; ++i)
        if (cache[i].used && std::memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
            *out = cache[i].map;
            return CUDA_SUCCESS;
        }
    cuuint32_t elem_strides[3] = {1, 1, 1};
    const CUresult r = enc(out, dt, 3, ptr, dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        Entry& e = cache[next];
        next = (next + 1) % kEntries;
        e.key = key; e.map = *out; e.used = true;
    }
    return r;
}

struct OperandPlan {
    bool mn_major = false;
    int batch_mul = 1;
    CUtensorMap map;
};

inline uint64_t round16(uint64_t v) { return (v + 15u) & ~uint64_t(15); }

// An operand is logically [mn_extent, k_extent] with element strides (mn_stride, k_stride) and a batch stride.
// Returns nullptr on success, else the reason the operand cannot be staged by TMA.
const char* plan_operand(const void* ptr, int es, CUtensorMapDataType dt, int64_t mn, int64_t k, int64_t mn_stride,
                         int64_t k_stride, int64_t batch, int64_t batch_stride, int tile_mn, int block_k,
                         OperandPlan* out) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return "operand base is not 16-byte aligned";
    if (mn_stride < 0 || k_stride < 0 || batch_stride < 0) return "negative stride";
    const bool k_unit = (k_stride == 1 || k == 1);
    const bool mn_unit = (mn_stride == 1 || mn == 1);
    auto aligned = [&](int64_t stride) { return (stride * es) % 16 == 0; };
    bool k_major_ok = k_unit && (mn == 1 || aligned(mn_stride));
    bool mn_major_ok = mn_unit && (k == 1 || aligned(k_stride));
    if (!k_major_ok && !mn_major_ok) return "no unit stride with a 16-byte aligned other stride";
    if (batch > 1 && batch_stride != 0 && !aligned(batch_stride)) return "batch stride is not 16-byte aligned";
    out->mn_major = !k_major_ok;
    const bool batched = batch > 1 && batch_stride != 0;
    out->batch_mul = batched ? 1 : 0;
    const int64_t inner = out->mn_major ? mn : k;
    const int64_t outer = out->mn_major ? k : mn;
    int64_t outer_stride = out->mn_major ? k_stride : mn_stride;
    if (outer == 1) outer_stride = int64_t(round16(uint64_t(inner) * es)) / es;
    if (inner > (int64_t(1) << 31) || outer > (int64_t(1) << 31)) return "extent too large for a tensor map";
    cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(outer), cuuint64_t(batched ? batch : 1)};
    cuuint64_t strides[2] = {cuuint64_t(outer_stride) * es,
                             batched ? cuuint64_t(batch_stride) * es
                                     : round16(cuuint64_t(outer_stride) * es * cuuint64_t(outer))};
    if (strides[0] % 16 || strides[1] % 16) return "stride is not 16-byte aligned";
    if (strides[0] >= (cuuint64_t(1) << 40) || strides[1] >= (cuuint64_t(1) << 40)) return "stride too large";
    cuuint32_t box[3];
    if (out->mn_major) {
        box[0] = cuuint32_t(128 / es);
        box[1] = cuuint32_t(block_k);
    } else {
        box[0] = cuuint32_t(block_k);
        box[1] = cuuint32_t(tile_mn);
    }
    box[2] = 1;
    if (!encode_fn()) return "cuTensorMapEncodeTiled is not available from the driver";
    const CUresult r = encode_cached(&out->map, dt, const_cast<void*>(ptr), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (r != CUDA_SUCCESS) return "cuTensorMapEncodeTiled rejected the operand";
    return nullptr;
}

// NTB200_NO_PAIR=1 keeps every GEMM on the single-CTA kernel (for A/B measurements).
const bool g_disable_pair = [] { const char* e = getenv("NTB200_NO_PAIR"); return e && e[0] == '1'; }();

// NTB200_FULL_A_TILE=1 always stages all 128 rows of A in the single-CTA kernel (for A/B measurements).
const bool g_four_epilogue_warps = [] { const char* e = getenv("NTB200_FOUR_EPILOGUE_WARPS"); return e && e[0] == '1'; }();
const bool g_full_a_tile = [] { const char* e = getenv("NTB200_FULL_A_TILE"); return e && e[0] == '1'; }();
// NTB200_TUNE=1 at load time makes every launch re-read NTB200_FORCE_BN (64 / 128 / 256), NTB200_FORCE_SPLITS (K slices)
// and NTB200_NO_PAIR from the environment: the knobs the tile heuristics were fitted with.
const bool g_tune = [] { const char* e = getenv("NTB200_TUNE"); return e && e[0] == '1'; }();
int tune_int(const char* name) {
    if (!g_tune) return 0;
    const char* e = getenv(name);
    return e ? atoi(e) : 0;
}

// NTB200_DIRECT_STORES=1 keeps the per-thread global stores in every epilogue (for A/B measurements).
const bool g_direct_stores = [] { const char* e = getenv("NTB200_DIRECT_STORES"); return e && e[0] == '1'; }();

// K blocks per partial sum of the Float32 split kernels (NTB200_TF32_CHUNK overrides it for measurements).
const int g_split_chunk_blocks = [] {
    const char* e = getenv("NTB200_TF32_CHUNK");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 8;
}();

bool dtype_on_tensor_cores(int dtype) {
    return dtype == NTB200_F16 || dtype == NTB200_BF16 || dtype == NTB200_I8 || dtype == NTB200_U8 || dtype == NTB200_F32 ||
           dtype == NTB200_I32 || dtype == NTB200_U32 || dtype == NTB200_I16 || dtype == NTB200_U16;
}

// Cheap structural test (no driver call): can both operands be staged?
const char* operands_stageable(const GemmArgs& g) {
    if (!dtype_on_tensor_cores(g.dtype)) return "dtype has no tensor-core kernel";
    if (g.a_ptrs || g.b_ptrs || g.c_ptrs) return "pointer-table batches run on the CUDA-core route";
    if (g.m <= 0 || g.n <= 0 || g.k <= 0 || g.batch <= 0) return "empty problem";
    if (g.dtype == NTB200_I32 || g.dtype == NTB200_U32 || g.dtype == NTB200_I16 || g.dtype == NTB200_U16) {   // limb planes are copies too; each limb GEMM must be exact in s32
        if (g.m > (int64_t(1) << 30) || g.n > (int64_t(1) << 30)) return "extent too large";
        if (g.a_rs < 0 || g.a_cs < 0 || g.a_bs < 0 || g.b_rs < 0 || g.b_cs < 0 || g.b_bs < 0) return "negative stride";
        return nullptr;
    }
    if (g.dtype == NTB200_F32) {  // operands are copied (split) first, so any strides do
        if (g.m > (int64_t(1) << 30) || g.n > (int64_t(1) << 30) || g.k > (int64_t(1) << 30)) return "extent too large";
        if (g.a_rs < 0 || g.a_cs < 0 || g.a_bs < 0 || g.b_rs < 0 || g.b_cs < 0 || g.b_bs < 0) return "negative stride";
        if ((g.m + 31) / 32 + (g.n + 31) / 32 > 65535) return "operands too tall for the split pass";
        return nullptr;
    }
    const int es = int(dtype_size(g.dtype));
    // s32 accumulation is exact (no overflow) while k * 2^14 < 2^31
    if (es == 1 && g.k > 131071) return "int8 K too large for exact s32 accumulation";
    if (g.m > (int64_t(1) << 30) || g.n > (int64_t(1) << 30) || g.k > (int64_t(1) << 30)) return "extent too large";
    auto check = [&](const void* ptr, int64_t mn, int64_t k, int64_t mn_s, int64_t k_s, int64_t bs) -> const char* {
        if (reinterpret_cast<uintptr_t>(ptr) % 16) return "operand base is not 16-byte aligned";
        if (mn_s < 0 || k_s < 0 || bs < 0) return "negative stride";
        const bool k_major_ok = (k_s == 1 || k == 1) && (mn == 1 || (mn_s * es) % 16 == 0);
        const bool mn_major_ok = (mn_s == 1 || mn == 1) && (k == 1 || (k_s * es) % 16 == 0);
        if (!k_major_ok && !mn_major_ok) return "no unit stride with a 16-byte aligned other stride";
        if (g.batch > 1 && bs != 0 && (bs * es) % 16) return "batch stride is not 16-byte aligned";
        return nullptr;
    };
    if (const char* w = check(g.a, g.m, g.k, g.a_rs, g.a_cs, g.a_bs)) return w;
    if (const char* w = check(g.b, g.n, g.k, g.b_cs, g.b_rs, g.b_bs)) return w;
    const int64_t tiles = ((g.m + kBM - 1) / kBM) * ((g.n + 63) / 64) * g.batch;
    if (tiles > (int64_t(1) << 30)) return "too many tiles";
    return nullptr;
}

struct Maps {
    OperandPlan a, b, a_lo, b_lo;
    CUtensorMap c, relu;   // outputs of the TMA-store epilogue (valid when UmmaParams::tma_store is set)
    PeerMaps peers;
};

// Tensor map of C [batch][m][n] (1- or 2-byte elements) for store boxes of 128 bytes x 32 rows with the 128-byte swizzle.
bool plan_store(void* c, CUtensorMapDataType dt, int es_bytes, int64_t m, int64_t n, int64_t batch, int64_t c_rs, int64_t c_bs,
                CUtensorMap* out) {
    const uint64_t es = uint64_t(es_bytes);
    if (reinterpret_cast<uintptr_t>(c) % 16 || (uint64_t(c_rs) * es) % 16) return false;
    if (batch > 1 && (uint64_t(c_bs) * es) % 16) return false;
    if (c_rs < n || c_rs <= 0 || (batch > 1 && c_bs <= 0)) return false;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    cuuint64_t dims[3] = {cuuint64_t(n), cuuint64_t(m), cuuint64_t(batch > 1 ? batch : 1)};
    cuuint64_t strides[2] = {cuuint64_t(c_rs) * es, batch > 1 ? cuuint64_t(c_bs) * es : round16(cuuint64_t(c_rs) * es * cuuint64_t(m))};
    if (strides[0] >= (cuuint64_t(1) << 40) || strides[1] >= (cuuint64_t(1) << 40)) return false;
    cuuint32_t box[3] = {cuuint32_t(128 / es), 32, 1};   // 128 bytes of columns x 32 rows
    return encode_cached(out, dt, c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) == CUDA_SUCCESS;
}

template <MmaKind kKind, int BN, bool kSplit>
int launch_instance(const Maps& m, const UmmaParams& p_in, int grid, int a_rows_staged, cudaStream_t stream) {
    using T = Tile<BN, kSplit>;
    UmmaParams p = p_in;
    // Stage geometry: all 128 rows of A, or only the `a_rows_staged` (8 / 16 / 32 / 64) the problem has, with the
    // shared memory saved going into a longer ring (more bytes of B in flight for memory-bound, few-row problems).
    const uint32_t copies = kSplit ? 2u : 1u;
    p.s_a_bytes = uint32_t(a_rows_staged) * 128u;
    p.s_stage_bytes = copies * (p.s_a_bytes + T::kBBytes);
    p.s_stage_tx = p.s_stage_bytes;
    p.s_stages = int(std::min<uint32_t>(uint32_t(T::kMaxStages), (T::kRingBudget - T::kABytes) / p.s_stage_bytes));
    const uint32_t smem = uint32_t(p.s_stages) * p.s_stage_bytes + T::kABytes + T::kBarrierBytes + 1024;
    // the attribute is per device and per instantiation: the largest size this instantiation can ask for, set once
    static std::atomic<bool> attr_set[64];
    int dev_i = 0;
    (void)cudaGetDevice(&dev_i);
    if (dev_i < 0 || dev_i >= 64) dev_i = 0;
    if (!attr_set[dev_i].load(std::memory_order_acquire)) {
        const uint32_t max_smem = T::kRingBudget + T::kBarrierBytes + 1024;
        cudaError_t e = cudaFuncSetAttribute(umma_gemm_kernel<kKind, BN, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(max_smem));
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma_gemm_kernel)");
        attr_set[dev_i].store(true, std::memory_order_release);
    }
    umma_gemm_kernel<kKind, BN, kSplit><<<grid, kSplit ? kThreadsSplit : kThreads, smem, stream>>>(m.a.map, m.b.map, m.a_lo.map, m.b_lo.map, p);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

// Number of CTA pairs that can be resident at once (one pair per TPC).
int resident_pairs_query(const void* kernel, uint32_t smem_bytes) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(sm_count() & ~1), 1, 1);
    cfg.blockDim = dim3(kThreadsSplit, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = sm_count() / 2;
    }
    return std::min(n, sm_count() / 2);
}

// How many clusters of `cluster_size` CTAs of `kernel` the current device can hold at once (cached per call site).
int active_clusters_query(const void* kernel, uint32_t smem_bytes, int cluster_size, int threads) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(cluster_size * 64), 1, 1);
    cfg.blockDim = dim3(unsigned(threads), 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = unsigned(cluster_size);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

template <MmaKind kKind, bool kSplit, int kEpi = 4>
int launch_pair_instance(const Maps& m, const UmmaParams& p, cudaStream_t stream) {
    // Shallow K, plain TMA-store epilogue: the instantiations with eight or sixteen epilogue warps (the epilogue, not
    // the main loop, bounds a tile, and its throughput grows with the warps that run it)
    if constexpr (!kSplit && kEpi == 4) {
        if (p.tma_store && !p.has_relu_out && p.k_blocks <= 6 && !g_four_epilogue_warps) {
            static const int forced = [] { const char* e = getenv("NTB200_EPILOGUE_WARPS"); return e ? atoi(e) : 0; }();
            // A C with nothing fused leaves through the lean epilogue, and with it four warps (two chunks in flight, no
            // register pressure) are as fast as eight and faster than sixteen at every depth: [8192, k]^T x [k, 8192] at
            // k = 16 / 128 / 256 / 384 takes 0.0255 / 0.0282 / 0.0414 / 0.0541 ms on four warps against 0.0279 / 0.0357 /
            // 0.0491 / 0.0622 ms on sixteen and 0.0258 / 0.0308 / 0.0448 / 0.0571 ms on eight.  The wider instantiations
            // remain for the general epilogue (bias, previous C, mask), whose chunks are several times as long.
            const bool plain = p.lean_ok && !p.bias && !p.accumulate && !p.has_mask && p.n_peers == 0 && p.out_kind != kOutI8;
            const int warps = forced == 8 || forced == 16 ? forced : (plain ? 4 : (p.k_blocks <= 2 ? 16 : 8));   // general epilogue: 16 warps win up to two K blocks
            if (warps == 16) return launch_pair_instance<kKind, kSplit, 16>(m, p, stream);
            if (warps == 8) return launch_pair_instance<kKind, kSplit, 8>(m, p, stream);
        }
    }
    constexpr uint32_t smem = PairTile<kSplit>::kSmemBytes;
    cudaError_t e = cudaFuncSetAttribute(umma_gemm_pair_kernel<kKind, kSplit, kEpi>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma_gemm_pair_kernel)");
    static int cached[64] = {0};  // per instantiation, per device
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0)
        cached[dev] = resident_pairs_query(reinterpret_cast<const void*>(umma_gemm_pair_kernel<kKind, kSplit, kEpi>), smem);
    const int pairs = std::min(p.total_tiles, cached[dev]);
    umma_gemm_pair_kernel<kKind, kSplit, kEpi><<<2 * pairs, kSplit ? kThreadsSplit : 64 + 32 * kEpi, smem, stream>>>(m.a.map, m.b.map, m.a_lo.map, m.b_lo.map, m.c, m.relu, m.peers, p);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

// ---- Float32 as three TF32 products ------------------------------------------------------------------
// x = hi + lo with hi = x rounded to TF32 (10 explicit mantissa bits) and lo = x - hi (exact in fp32), so that
// a.b = a_hi.b_hi + a_hi.b_lo + a_lo.b_hi + O(2^-21 |a||b|).  The pre-pass writes hi and lo as dense K-major
// matrices [batch][rows][k_padded], whatever the strides of the source view, so the GEMM only ever sees one layout.
struct SplitJob {
    const float* src;
    float* hi;
    float* lo;
    long long rows, batch, sbs, srs, scs;
    int row_blocks;   // ceil(rows / 32)
};

// One launch splits both operands: blockIdx.y below a.row_blocks works on A, the rest on B.
__global__ void split_tf32_kernel(SplitJob ja, SplitJob jb, long long cols, long long cols_padded) {
    const bool second = int(blockIdx.y) >= ja.row_blocks;
    const SplitJob& job = second ? jb : ja;
    if ((long long)blockIdx.z >= job.batch) return;
    const float* __restrict__ src = job.src;
    float* __restrict__ hi = job.hi;
    float* __restrict__ lo = job.lo;
    const long long rows = job.rows, sbs = job.sbs, srs = job.srs, scs = job.scs;
    const int by = int(blockIdx.y) - (second ? ja.row_blocks : 0);
    __shared__ float tile[32][33];
    const long long b = blockIdx.z;
    const long long r0 = (long long)by * 32, c0 = (long long)blockIdx.x * 32;
    const float* s = src + b * sbs;
    const bool read_along_cols = (scs == 1 || srs != 1);
    if (read_along_cols) {
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + j, c = c0 + threadIdx.x;
            tile[j][threadIdx.x] = (r < rows && c < cols) ? s[r * srs + c * scs] : 0.f;
        }
    } else {  // rows are the unit-stride direction of the source
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + threadIdx.x, c = c0 + j;
            tile[threadIdx.x][j] = (r < rows && c < cols) ? s[r * srs + c * scs] : 0.f;
        }
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        const long long r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols_padded) {
            const float x = tile[j][threadIdx.x];
            uint32_t h;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
            const float hf = __uint_as_float(h);
            const float l = (isfinite(x) && isfinite(hf)) ? x - hf : 0.f;
            const long long o = (b * rows + r) * cols_padded + c;
            hi[o] = hf;
            lo[o] = l;
        }
    }
}

struct Planned {
    int es;
    CUtensorMapDataType dt;
    MmaKind kind;
    int out_kind;
    uint32_t d_fmt, in_fmt;
    bool split;
    const char* route;
    int shift = 0;
};

// Operands as the tensor-map planner sees them: logical [mn, k] with element strides and a batch stride.
struct Side {
    const void* ptr;
    int64_t mn_stride, k_stride, bs;
};

// A tile shape decided by the caller (the 16-bit cost model below) instead of the heuristics inside launch_planned.
struct TileChoice {
    bool pair;
    int bn;
};

int launch_planned(const GemmArgs& g, const Planned& pl, const Side& a, const Side& b, const Side* a_lo, const Side* b_lo,
                   cudaStream_t stream, const TileChoice* choice = nullptr) {
    const int es = pl.es;
    const int block_k = 128 / es;
    // Tile width: the widest one that still gives every SM a tile.
    const int sms = sm_count();
    const int64_t tiles_m = (g.m + kBM - 1) / kBM;
    int bn = 64;
    for (int cand : {256, 128, 64}) {
        bn = cand;
        if (g.n > cand / 2 && tiles_m * ((g.n + cand - 1) / cand) * g.batch >= sms) break;
    }
    if (g.n <= 64) bn = 64;
    else if (g.n <= 128 && bn > 128) bn = 128;
    // Float32 split kernel: 64-wide tiles only pay while 128-wide ones would leave more than half of the SMs idle
    // (measured: [512, 4096] x [4096, 4096] 0.211 -> 0.156 ms, [256, 8192] x [8192, 8192] 0.517 -> 0.411 ms on 128-wide
    // tiles; 1024^3, 64 tiles of 128 columns, stays on 64-wide ones at 0.035 ms)
    if (pl.split && bn == 64 && g.n > 64 && tiles_m * ((g.n + 127) / 128) * g.batch * 2 >= sms) bn = 128;

    // Large problems run on CTA pairs (256 x 256 tiles); anything with fewer pair tiles than TPCs keeps the
    // single-CTA kernel, whose narrower tiles spread small problems over more SMs.
    const int64_t pair_tiles = ((g.m + 255) / 256) * ((g.n + 255) / 256) * g.batch;
    // (the Float32 split kernel, whose K blocks are three MMAs deep, already pays from 60 % of a wave:
    // [768, 4096] x [4096, 4096] 0.229 -> 0.202 ms)
    bool use_pair = !g_disable_pair && g.m > 128 && g.n > 128 && pair_tiles * 5 >= (sms / 2) * (pl.split ? 3 : 4);   // >= 80 % of one wave
    if (choice) {
        use_pair = choice->pair && g.m > 128 && g.n > 128;
        if (!use_pair) bn = choice->bn;
    }
    if (g_tune) {
        if (tune_int("NTB200_NO_PAIR") == 1) use_pair = false;
        if (tune_int("NTB200_NO_PAIR") == 2) use_pair = g.m > 128 && g.n > 128;
        const int f = tune_int("NTB200_FORCE_BN");
        if (!use_pair && (f == 64 || f == 128 || f == 256)) bn = f;
    }
    if (use_pair) bn = 256;

    Maps maps;
    if (const char* w = plan_operand(a.ptr, es, pl.dt, g.m, g.k, a.mn_stride, a.k_stride, g.batch, a.bs, kBM, block_k, &maps.a))
        return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route, A: %s", w);
    // Few rows (one M tile of at most 64 rows, K-major A): stage only those rows and run a longer ring, so that a
    // memory-bound problem keeps more bytes of B in flight.
    int a_rows_staged = kBM;
    if (!use_pair && !pl.split && g.m <= 64 && !maps.a.mn_major && !g_full_a_tile) {
        a_rows_staged = g.m <= 8 ? 8 : (g.m <= 16 ? 16 : (g.m <= 32 ? 32 : 64));
        if (const char* w = plan_operand(a.ptr, es, pl.dt, g.m, g.k, a.mn_stride, a.k_stride, g.batch, a.bs, a_rows_staged, block_k, &maps.a))
            return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route, A: %s", w);
    }
    if (const char* w = plan_operand(b.ptr, es, pl.dt, g.n, g.k, b.mn_stride, b.k_stride, g.batch, b.bs, use_pair ? 128 : bn,
                                     block_k, &maps.b))
        return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route, B: %s", w);
    // An N-major operand is staged in chunks of 128 bytes of N: 8-bit tiles cannot be narrower than one chunk.
    // (The tensor map of an N-major operand does not depend on the tile width, so the plan stays valid.)
    if (maps.b.mn_major && bn < 128 / es) bn = 128 / es;
    if (pl.split) {
        if (const char* w = plan_operand(a_lo->ptr, es, pl.dt, g.m, g.k, a_lo->mn_stride, a_lo->k_stride, g.batch, a_lo->bs, kBM,
                                         block_k, &maps.a_lo))
            return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route, A (low part): %s", w);
        if (const char* w = plan_operand(b_lo->ptr, es, pl.dt, g.n, g.k, b_lo->mn_stride, b_lo->k_stride, g.batch, b_lo->bs,
                                         use_pair ? 128 : bn, block_k, &maps.b_lo))
            return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route, B (low part): %s", w);
        if (maps.a.mn_major || maps.b.mn_major || maps.a_lo.mn_major || maps.b_lo.mn_major)
            return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route: split operands must be K-major");
    } else {
        maps.a_lo = maps.a;
        maps.b_lo = maps.b;
    }

    UmmaParams p{};
    p.m = int(g.m); p.n = int(g.n); p.k = int(g.k); p.batch = int(g.batch);
    p.tiles_m = use_pair ? int((g.m + 255) / 256) : int(tiles_m);
    p.tiles_n = int((g.n + bn - 1) / bn);
    p.k_blocks = int((g.k + block_k - 1) / block_k);
    // Float32 split: hand over a partial sum every `g_split_chunk_blocks` K blocks (32 k each)
    p.chunk_blocks = pl.split ? g_split_chunk_blocks : p.k_blocks;
    p.group_m = 8;
    p.total_tiles = int(int64_t(p.tiles_m) * p.tiles_n * g.batch);
    p.block_k = block_k;
    p.idesc = make_instr_desc(pl.d_fmt, pl.in_fmt, pl.in_fmt, maps.a.mn_major, maps.b.mn_major, use_pair ? 256u : uint32_t(kBM),
                              uint32_t(bn));
    p.a_mn_major = maps.a.mn_major; p.b_mn_major = maps.b.mn_major;
    p.chunk_mn = 128 / es;
    p.chunk_bytes = uint32_t(block_k) * 128u;
    p.a_chunks = kBM / p.chunk_mn;
    p.b_chunks = (use_pair ? 128 : bn) / p.chunk_mn;
    // K-major: rows are 128 bytes, 8-row groups 1024 bytes apart, +32 bytes per MMA along K.
    // MN-major: each K row of a chunk is 128 bytes of MN, 8-row groups 1024 bytes apart (SBO), chunks
    // `chunk_bytes` apart (LBO), and one MMA consumes 32/es K rows.
    p.a_lbo = maps.a.mn_major ? p.chunk_bytes : 16u;
    p.b_lbo = maps.b.mn_major ? p.chunk_bytes : 16u;
    const uint32_t mn_kstep = uint32_t(32 / es) * 128u / 16u;
    p.a_kstep = maps.a.mn_major ? mn_kstep : 2u;
    p.b_kstep = maps.b.mn_major ? mn_kstep : 2u;
    p.a_batch_mul = maps.a.batch_mul; p.b_batch_mul = maps.b.batch_mul;
    p.c = g.c; p.c_rs = g.c_rs; p.c_bs = g.c_bs;
    p.bias = g.bias; p.bias_rs = g.bias_rs; p.bias_cs = g.bias_cs; p.bias_bs = g.bias_bs;
    p.accumulate = g.accumulate;
    p.out_kind = pl.out_kind;
    p.shift = pl.shift;
    p.has_relu_out = g.relu_out != nullptr;
    p.has_mask = g.mask_src != nullptr;
    p.relu_out_offset = g.relu_out ? static_cast<const char*>(g.relu_out) - static_cast<const char*>(g.c) : 0;
    p.mask_offset = g.mask_src ? static_cast<const char*>(g.mask_src) - static_cast<const char*>(g.c) : 0;
    if ((g.relu_out || g.mask_src) && pl.out_kind != kOutF16 && pl.out_kind != kOutBF16)
        return fail(NTB200_ERR_UNSUPPORTED, "fused ReLU epilogues are implemented for Float16 / BFloat16 outputs");
    if ((g.relu_out || g.mask_src) && g.accumulate)
        return fail(NTB200_ERR_UNSUPPORTED, "fused ReLU epilogues do not combine with accumulate");
    p.n_peers = g.n_peers;
    for (int t = 0; t < g.n_peers; ++t)
        p.peer_offset[t] = static_cast<const char*>(g.peer_c[t]) - static_cast<const char*>(g.c);
    if (g.n_peers > 0 && pl.out_kind != kOutF16 && pl.out_kind != kOutBF16)
        return fail(NTB200_ERR_UNSUPPORTED, "peer stores are implemented for Float16 / BFloat16 outputs");
    const int ces = int(dtype_size(g.dtype));
    p.c_vec_ok = (reinterpret_cast<uintptr_t>(g.c) % 16 == 0) && ((g.c_rs * ces) % 16 == 0) &&
                 (g.batch == 1 || (g.c_bs * ces) % 16 == 0);
    // Pair kernel, 16-bit and 8-bit outputs: finished tiles leave through shared memory and TMA stores, peer copies
    // of C included (plain TMA stores into peer-mapped memory; no load ever touches a peer).
    maps.c = maps.a.map;
    maps.relu = maps.a.map;
    p.tma_store = 0;
    const bool out16 = pl.out_kind == kOutF16 || pl.out_kind == kOutBF16;
    if (use_pair && !pl.split && (out16 || pl.out_kind == kOutI8) && !g_direct_stores) {
        const int64_t relu_rs = g.relu_rs ? g.relu_rs : g.c_rs, relu_bs = g.relu_rs ? g.relu_bs : g.c_bs;
        const bool peers_relu = g.peers_get_relu && g.relu_out;
        bool ok = plan_store(g.c, pl.dt, out16 ? 2 : 1, g.m, g.n, g.batch, g.c_rs, g.c_bs, &maps.c);
        for (int t = 0; ok && t < g.n_peers; ++t)   // peer-mapped copies with the layout of the tensor they mirror
            ok = plan_store(g.peer_c[t], pl.dt, out16 ? 2 : 1, g.m, g.n, g.batch, peers_relu ? relu_rs : g.c_rs,
                            peers_relu ? relu_bs : g.c_bs, &maps.peers.m[t]);
        if (ok && g.relu_out) ok = plan_store(g.relu_out, pl.dt, 2, g.m, g.n, g.batch, relu_rs, relu_bs, &maps.relu);
        p.peers_relu = peers_relu ? 1 : 0;
        if (ok && g.mask_src) ok = reinterpret_cast<uintptr_t>(g.mask_src) % 16 == 0;
        p.tma_store = ok ? 1 : 0;
        static const bool general_only = [] { const char* e = getenv("NTB200_GENERAL_EPILOGUE"); return e && e[0] == '1'; }();
        p.lean_ok = general_only ? 0 : 1;
    }
    if (!p.tma_store && g.relu_out && ((g.relu_rs && g.relu_rs != g.c_rs) || g.peers_get_relu))
        return fail(NTB200_ERR_UNSUPPORTED,
                    "tcgen05 route: a ReLU output with its own strides (or pushed to peers) needs the TMA-store epilogue "
                    "(problem of at least 74 tiles of 256 x 256, 16-byte aligned rows)");
    const int grid = int(std::min<int64_t>(p.total_tiles, sms));
    note_route(pl.route);
    if (pl.kind == MmaKind::tf32) {
        if (use_pair) return launch_pair_instance<MmaKind::tf32, true>(maps, p, stream);
        if (bn == 256) return launch_instance<MmaKind::tf32, 256, true>(maps, p, grid, a_rows_staged, stream);
        if (bn == 128) return launch_instance<MmaKind::tf32, 128, true>(maps, p, grid, a_rows_staged, stream);
        return launch_instance<MmaKind::tf32, 64, true>(maps, p, grid, a_rows_staged, stream);
    }
    if (pl.kind == MmaKind::i8) {
        if (use_pair) return launch_pair_instance<MmaKind::i8, false>(maps, p, stream);
        if (bn == 256) return launch_instance<MmaKind::i8, 256, false>(maps, p, grid, a_rows_staged, stream);
        if (bn == 128) return launch_instance<MmaKind::i8, 128, false>(maps, p, grid, a_rows_staged, stream);
        return launch_instance<MmaKind::i8, 64, false>(maps, p, grid, a_rows_staged, stream);
    }
    if (use_pair) return launch_pair_instance<MmaKind::f16, false>(maps, p, stream);
    if (bn == 256) return launch_instance<MmaKind::f16, 256, false>(maps, p, grid, a_rows_staged, stream);
    if (bn == 128) return launch_instance<MmaKind::f16, 128, false>(maps, p, grid, a_rows_staged, stream);
    return launch_instance<MmaKind::f16, 64, false>(maps, p, grid, a_rows_staged, stream);
}

// Float32: split both operands into dense K-major hi/lo copies in pool scratch, then one GEMM with three TF32
// products per K step.  The scratch is returned to the pool in stream order.
int launch_f32_split(const GemmArgs& g, cudaStream_t stream) {
    const int64_t kp = (g.k + 3) & ~int64_t(3);  // rows of the copies stay 16-byte aligned
    const int64_t a_batch = (g.batch > 1 && g.a_bs != 0) ? g.batch : 1;
    const int64_t b_batch = (g.batch > 1 && g.b_bs != 0) ? g.batch : 1;
    if (a_batch > 65535 || b_batch > 65535) return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route: batch too large for the Float32 split pass");
    const size_t a_elems = size_t(a_batch) * size_t(g.m) * size_t(kp), b_elems = size_t(b_batch) * size_t(g.n) * size_t(kp);
    float* scratch = nullptr;
    if (int rc = scratch_acquire(reinterpret_cast<void**>(&scratch), 2 * (a_elems + b_elems) * sizeof(float), stream)) return rc;
    float* a_hi = scratch;
    float* a_lo = a_hi + a_elems;
    float* b_hi = a_lo + a_elems;
    float* b_lo = b_hi + b_elems;
    const dim3 block(32, 8);
    // B is logically [k, n]; its copy is [n][k]: rows = n (source stride b_cs), columns = k (source stride b_rs)
    const SplitJob ja{static_cast<const float*>(g.a), a_hi, a_lo, g.m, a_batch, g.a_bs, g.a_rs, g.a_cs, int((g.m + 31) / 32)};
    const SplitJob jb{static_cast<const float*>(g.b), b_hi, b_lo, g.n, b_batch, g.b_bs, g.b_cs, g.b_rs, int((g.n + 31) / 32)};
    if (int64_t(ja.row_blocks) + jb.row_blocks > 65535) {
        scratch_release(scratch, stream);
        return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route: operand too tall for the Float32 split pass");
    }
    split_tf32_kernel<<<dim3(unsigned((kp + 31) / 32), unsigned(ja.row_blocks + jb.row_blocks), unsigned(std::max(a_batch, b_batch))),
                        block, 0, stream>>>(ja, jb, g.k, kp);
    count_launch();
    cudaError_t e = cudaGetLastError();
    int rc = NTB200_OK;
    if (e != cudaSuccess) {
        rc = cuda_fail(e, "split_tf32_kernel");
    } else {
        const Planned pl{4, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, MmaKind::tf32, kOutF32, 1u, 2u, true, "umma_3xtf32"};
        const Side sa{a_hi, kp, 1, a_batch > 1 ? g.m * kp : 0}, sal{a_lo, kp, 1, a_batch > 1 ? g.m * kp : 0};
        const Side sb{b_hi, kp, 1, b_batch > 1 ? g.n * kp : 0}, sbl{b_lo, kp, 1, b_batch > 1 ? g.n * kp : 0};
        rc = launch_planned(g, pl, sa, sb, &sal, &sbl, stream);
    }
    scratch_release(scratch, stream);
    return rc;
}

// ---- Int32 / UInt32 as products of 8-bit limbs ----------------------------------------------------------
// x = x0 + x1 2^8 + x2 2^16 + x3 2^24 with unsigned 8-bit limbs (the top limb's sign does not matter modulo 2^32), so
// a.b mod 2^32 = sum over s = 0..3 of 2^(8s) * sum over i + j = s of (a_i . b_j)  mod 2^32.
// The pre-pass writes, per K chunk of Kc columns, the four limb planes of a row side by side:
//     A row: [a_0 | a_1 | a_2 | a_3],   B^T row: [b_3 | b_2 | b_1 | b_0]        (each Kc bytes, K-major)
// so that sum_{i+j=s} a_i . b_j is ONE 8-bit GEMM of depth (s+1) Kc: the first s+1 planes of the A row against the
// last s+1 planes of the B row.  Four kind::i8 GEMMs per K chunk, whose exact s32 sums ((s+1) Kc 255^2 < 2^31) are
// shifted and added into C by the epilogue.  Bit-exact with the reference's mullo_epi32 / add_epi32
// (nt/mp/simde_traits/simde_traits_avx2.h:444-485) by construction.
constexpr int64_t kLimbChunkK = 8192;

template <typename Src, int kLimbs>
__global__ void split_limbs_kernel(const Src* __restrict__ src, uint8_t* __restrict__ limbs, long long rows, long long cols,
                                   long long kc, long long nchunks, int reverse, long long sbs, long long srs, long long scs) {
    __shared__ uint32_t tile[32][33];
    const long long b = blockIdx.z;
    const long long r0 = (long long)blockIdx.y * 32, c0 = (long long)blockIdx.x * 32;
    const Src* s = src + b * sbs;
    if (scs == 1 || srs != 1) {
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + j, c = c0 + threadIdx.x;
            tile[j][threadIdx.x] = (r < rows && c < cols) ? s[r * srs + c * scs] : 0u;
        }
    } else {
        for (int j = threadIdx.y; j < 32; j += 8) {
            const long long r = r0 + threadIdx.x, c = c0 + j;
            tile[threadIdx.x][j] = (r < rows && c < cols) ? s[r * srs + c * scs] : 0u;
        }
    }
    __syncthreads();
    const long long row_bytes = nchunks * kLimbs * kc;
    for (int j = threadIdx.y; j < 32; j += 8) {
        const long long r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < nchunks * kc) {
            const uint32_t x = tile[j][threadIdx.x];   // zero beyond `cols`: the padding columns contribute nothing
            uint8_t* row = limbs + (b * rows + r) * row_bytes + (c / kc) * kLimbs * kc + (c % kc);
#pragma unroll
            for (int l = 0; l < kLimbs; ++l) row[(reverse ? kLimbs - 1 - l : l) * kc] = uint8_t(x >> (8 * l));
        }
    }
}

// kLimbs = 4: Int32 / UInt32 (four GEMMs per K chunk); kLimbs = 2: Int16 / UInt16 (two), the same scheme modulo 2^16.
template <typename Src, int kLimbs>
int launch_int_limbs(const GemmArgs& g, cudaStream_t stream) {
    const int64_t kp = (g.k + 15) & ~int64_t(15);
    const int64_t kc = std::min(kp, kLimbChunkK), nchunks = (kp + kc - 1) / kc;
    const int64_t row_bytes = nchunks * kLimbs * kc;
    const int64_t a_batch = (g.batch > 1 && g.a_bs != 0) ? g.batch : 1;
    const int64_t b_batch = (g.batch > 1 && g.b_bs != 0) ? g.batch : 1;
    if (a_batch > 65535 || b_batch > 65535) return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route: batch too large for the limb split pass");
    const size_t a_bytes = size_t(a_batch) * size_t(g.m) * size_t(row_bytes), b_bytes = size_t(b_batch) * size_t(g.n) * size_t(row_bytes);
    uint8_t* scratch = nullptr;
    if (int rc = scratch_acquire(reinterpret_cast<void**>(&scratch), a_bytes + b_bytes, stream)) return rc;
    uint8_t* a_limbs = scratch;
    uint8_t* b_limbs = scratch + a_bytes;
    const dim3 block(32, 8);
    const unsigned gx = unsigned((nchunks * kc + 31) / 32);
    split_limbs_kernel<Src, kLimbs><<<dim3(gx, unsigned((g.m + 31) / 32), unsigned(a_batch)), block, 0, stream>>>(
        static_cast<const Src*>(g.a), a_limbs, g.m, g.k, kc, nchunks, 0, g.a_bs, g.a_rs, g.a_cs);
    split_limbs_kernel<Src, kLimbs><<<dim3(gx, unsigned((g.n + 31) / 32), unsigned(b_batch)), block, 0, stream>>>(
        static_cast<const Src*>(g.b), b_limbs, g.n, g.k, kc, nchunks, 1, g.b_bs, g.b_cs, g.b_rs);
    count_launch(2);
    cudaError_t e = cudaGetLastError();
    int rc = e == cudaSuccess ? NTB200_OK : cuda_fail(e, "split_limbs_kernel");
    bool first = true;
    for (int64_t ch = 0; ch < nchunks && rc == NTB200_OK; ++ch)
        for (int sh = 0; sh < kLimbs && rc == NTB200_OK; ++sh) {
            Planned pl{1, CU_TENSOR_MAP_DATA_TYPE_UINT8, MmaKind::i8, kLimbs == 4 ? kOutU32 : kOutU16, 2u, 0u, false,
                       kLimbs == 4 ? "umma_i32_limbs" : "umma_i16_limbs"};
            pl.shift = 8 * sh;
            GemmArgs part = g;
            part.k = (sh + 1) * kc;                         // planes 0..sh of A against planes sh..0 of B
            if (!first) { part.accumulate = 1; part.bias = nullptr; }
            const Side sa{a_limbs + ch * kLimbs * kc, row_bytes, 1, a_batch > 1 ? g.m * row_bytes : 0};
            const Side sb{b_limbs + ch * kLimbs * kc + (kLimbs - 1 - sh) * kc, row_bytes, 1, b_batch > 1 ? g.n * row_bytes : 0};
            rc = launch_planned(part, pl, sa, sb, nullptr, nullptr, stream);
            first = false;
        }
    scratch_release(scratch, stream);
    return rc;
}

// ---- few-row products of 16-bit floats: K split over the "batch" axis of the same kernel -------------------
// One elected thread issues every TMA load and every MMA of a CTA, and each of those instructions costs it some
// 50 to 100 cycles, so a CTA turns over one 64-deep K block in about 550 cycles whatever the tile's width: a
// [16, 8192] x [8192, 8192] product on 128 tiles of 128 x 64 streams its weights at 15 bytes per clock and SM
// (2.9 TB/s in all), well under what HBM delivers.  Wider tiles move more bytes per instruction but leave SMs idle
// when there are few of them.  So the K axis is cut into S slices that run as S "batches" of the ordinary kernel
// (A and B are strided views, nothing is copied), each writing an fp32 partial tile; a small second kernel adds the
// S partials in order, then the bias and the previous C, and rounds once, like the one-pass epilogue does.
const bool g_no_splitk = [] { const char* e = getenv("NTB200_NO_SPLITK"); return e && e[0] == '1'; }();

int pick_k_splits(const GemmArgs& g) {
    if (g_no_splitk || g.no_alloc || g.batch != 1 || g.m > kBM || g.relu_out || g.mask_src || g.n_peers > 0) return 1;
    if (g.k % 64 != 0 || g.n % 4 != 0) return 1;
    // measured: no gain (or a loss, once the partial tiles weigh against the weights) below 4096 deep or 32 MB of weights
    if (g.k < 4096 || g.n * g.k < (int64_t(1) << 24)) return 1;
    const int sms = sm_count();
    const int64_t tiles = (g.n + 127) / 128;               // 128-wide tiles: 16 KB of B per K block
    if (tiles >= sms) return 1;
    int best = 1;
    for (int s = 2; s <= 16; s *= 2) {
        if (g.k % (64 * s) != 0 || g.k / s < 512) break;
        best = s;
        if (tiles * s >= sms) break;
    }
    return best;
}

// More than 128 rows of 16-bit floats: tile shape and K slices by a small cost model, in microseconds.  One K block
// of a tile costs its CTA (or CTA pair) a fixed time that hardly depends on the tile's width below 256 columns (the
// issue cost above), so what matters is the number of waves of tiles, the K blocks each tile runs through, and, with
// K slices, the fp32 partial tiles that are written and read back.  The constants are fitted to a sweep of
// m = 129 .. 1536 against weight matrices 2048 .. 11008 wide and deep (tile kind x slices, CUDA events over
// back-to-back launches, so the fixed part includes the launch).
struct F16Plan {
    TileChoice tile;
    int splits;
    bool valid;
    double us = 1e30;   // the model's estimate for the chosen combination
};

F16Plan plan_f16_tiles(const GemmArgs& g, int es = 2) {
    F16Plan best{{false, 64}, 1, false};
    if (g.m <= kBM) return best;   // few rows: pick_k_splits and the heuristics in launch_planned
    const int sms = sm_count();
    const int block_k = 128 / es;  // 8-bit operands: 128 deep K blocks, the same four MMAs and the same cycles
    const double kb = double((g.k + block_k - 1) / block_k);
    const bool fused = g.relu_out || g.mask_src || g.n_peers > 0;
    const bool may_split = es == 2 && !g_no_splitk && !g.no_alloc && g.batch == 1 && !fused && g.n % 4 == 0;   // the reduce kernel is 16-bit
    const double dram_us = double(g.batch) * (double(g.m) * g.k + double(g.k) * g.n + double(g.m) * g.n) * es / 4.5e6;
    struct Cand { bool pair; int bn; double fixed_us, us_per_k_block; };   // launch + fill + last epilogue; main loop
    const Cand cands[] = {{true, 256, 11.0, 0.35}, {false, 256, 13.0, 0.39}, {false, 128, 10.0, 0.34}, {false, 64, 10.0, 0.30}};
    double best_us = 1e30;
    for (const Cand& c : cands) {
        if (c.pair && (g_disable_pair || g.n <= 128)) continue;
        if (!c.pair && c.bn > 64 && g.n <= c.bn / 2) continue;          // a tile more than twice as wide as C
        if (fused && !c.pair && g.n > 128) continue;                     // fused epilogues keep the TMA-store kernel
        const int64_t tiles = (c.pair ? ((g.m + 255) / 256) * ((g.n + 255) / 256)
                                      : ((g.m + kBM - 1) / kBM) * ((g.n + c.bn - 1) / c.bn)) * g.batch;
        const int units = c.pair ? sms / 2 : sms;
        for (int s = 1; s <= 16; s *= 2) {
            if (s > 1 && (!may_split || g.k % (64 * s) != 0 || g.k / s < 512)) break;
            const double waves = double((tiles * s + units - 1) / units);
            double us = c.fixed_us + std::max(waves * (kb / s) * c.us_per_k_block, dram_us);
            if (s > 1) us += 3.0 + double(s) * double(g.m) * double(g.n) * 8.0 / 4.0e6;   // partial tiles out and back in (mostly L2)
            if (us < best_us * 0.97) {   // candidates come in order of preference: a later one has to be clearly better
                best_us = us;
                best = F16Plan{{c.pair, c.bn}, s, true, us};
            }
        }
    }
    return best;
}

template <int kOutKind>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, long long slab, int m, int n, uint16_t* c,
                                     long long c_rs, const uint16_t* bias, long long bias_rs, long long bias_cs, int accumulate,
                                     int wide_stores) {
    const int n4 = n >> 2;                                  // n is a multiple of 4
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)m * n4) return;
    const int row = int(idx / n4), col = int(idx % n4) * 4;
    const float* src = partial + (long long)row * n + col;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(src + s * slab);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float f[4] = {acc.x, acc.y, acc.z, acc.w};
    uint16_t* dst = c + (long long)row * c_rs + col;
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (bias) f[j] += to_float_bits16(bias[(long long)row * bias_rs + (long long)(col + j) * bias_cs], kOutKind);
        if (accumulate) f[j] += to_float_bits16(dst[j], kOutKind);
        r[j] = from_float_bits16(f[j], kOutKind);
    }
    if (wide_stores) {   // C and its rows are 8-byte aligned
        *reinterpret_cast<uint2*>(dst) = make_uint2(r[0] | (r[1] << 16), r[2] | (r[3] << 16));
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = uint16_t(r[j]);
    }
}

int launch_f16_split_k(const GemmArgs& g, const Planned& pl16, int splits, const TileChoice* choice, cudaStream_t stream) {
    const int64_t slab = g.m * g.n, kslice = g.k / splits;
    float* partial = nullptr;
    if (int rc = scratch_acquire(reinterpret_cast<void**>(&partial), size_t(splits) * size_t(slab) * sizeof(float), stream)) return rc;
    GemmArgs part = g;
    part.batch = splits;
    part.k = kslice;
    part.c = partial; part.c_rs = g.n; part.c_bs = slab;
    part.bias = nullptr; part.accumulate = 0;
    Planned pl = pl16;
    pl.out_kind = kOutF32;
    pl.route = g.dtype == NTB200_F16 ? "umma_f16_splitk" : "umma_bf16_splitk";
    const Side a{g.a, g.a_rs, g.a_cs, kslice * g.a_cs}, b{g.b, g.b_cs, g.b_rs, kslice * g.b_rs};
    int rc = launch_planned(part, pl, a, b, nullptr, nullptr, stream, choice);
    if (rc == NTB200_OK) {
        const long long work = (long long)g.m * (g.n / 4);
        const unsigned blocks = unsigned((work + 255) / 256);
        uint16_t* c = static_cast<uint16_t*>(g.c);
        const uint16_t* bias = static_cast<const uint16_t*>(g.bias);
        const int wide_stores = (reinterpret_cast<uintptr_t>(g.c) % 8 == 0 && g.c_rs % 4 == 0) ? 1 : 0;
        if (g.dtype == NTB200_F16)
            splitk_reduce_kernel<kOutF16><<<blocks, 256, 0, stream>>>(partial, splits, slab, int(g.m), int(g.n), c, g.c_rs, bias,
                                                                     g.bias_rs, g.bias_cs, g.accumulate, wide_stores);
        else
            splitk_reduce_kernel<kOutBF16><<<blocks, 256, 0, stream>>>(partial, splits, slab, int(g.m), int(g.n), c, g.c_rs, bias,
                                                                      g.bias_rs, g.bias_cs, g.accumulate, wide_stores);
        count_launch();
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_fail(e, "splitk_reduce_kernel");
    }
    scratch_release(partial, stream);
    return rc;
}


// K slices inside a cluster (umma_gemm_cluster_k_kernel): one launch for few-row products of 16-bit floats.
// Returns NTB200_ERR_UNSUPPORTED (nothing launched, error text untouched) when the shape does not fit the scheme.
const bool g_no_cluster_k = [] { const char* e = getenv("NTB200_NO_CLUSTER_K"); return e && e[0] == '1'; }();

template <int BN>
int launch_cluster_k_instance(const Maps& maps, ClusterKParams cp, int a_rows_staged, int clusters, cudaStream_t stream) {
    using T = Tile<BN, false>;
    UmmaParams& p = cp.u;
    p.s_a_bytes = uint32_t(a_rows_staged) * 128u;
    p.s_stage_bytes = p.s_a_bytes + T::kBBytes;
    p.s_stage_tx = p.s_stage_bytes;
    p.s_stages = int(std::min<uint32_t>(uint32_t(T::kMaxStages), (T::kRingBudget - T::kABytes) / p.s_stage_bytes));
    const uint32_t ring = uint32_t(p.s_stages) * p.s_stage_bytes + T::kABytes;
    if (uint32_t(cp.rows_live) * uint32_t(cp.pitch) * 4u > ring) return NTB200_ERR_UNSUPPORTED;   // the partial tile lives in the ring
    const uint32_t smem = ring + T::kBarrierBytes + 1024;
    auto kernel = umma_gemm_cluster_k_kernel<BN>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(umma_gemm_cluster_k_kernel)");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(clusters * cp.slices), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = unsigned(cp.slices);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, maps.a.map, maps.b.map, cp);
    if (e != cudaSuccess) return cuda_fail(e, "umma_gemm_cluster_k_kernel launch");
    count_launch();
    return NTB200_OK;
}

// Tile width and slice count for the cluster scheme, with an estimate of its run time in microseconds (same units
// and fitted per-K-block costs as plan_f16_tiles).  valid = false: the shape does not fit.
struct ClusterKPlan {
    int bn, slices;
    double us;
    bool valid;
};

int cluster_k_capacity(int bn, int slices) {
    static std::atomic<int> cached[64][2][9];
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || slices < 1 || slices > 8) return 0;
    const int bi = bn == 256 ? 1 : 0;
    int v = cached[dev][bi][slices].load(std::memory_order_relaxed);
    if (v == 0) {
        using T256 = Tile<256, false>;
        const uint32_t smem = T256::kRingBudget + T256::kBarrierBytes + 1024;   // the largest the kernel asks for
        const void* kernel = bn == 256 ? reinterpret_cast<const void*>(umma_gemm_cluster_k_kernel<256>)
                                       : reinterpret_cast<const void*>(umma_gemm_cluster_k_kernel<128>);
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        v = active_clusters_query(kernel, smem, slices, kThreads);
        cached[dev][bi][slices].store(v > 0 ? v : -1, std::memory_order_relaxed);
    }
    return v > 0 ? v : 0;
}

ClusterKPlan plan_cluster_k(const GemmArgs& g, int es) {
    ClusterKPlan best{0, 0, 1e30, false};
    if (g_no_cluster_k || g.no_alloc || g.batch != 1 || g.relu_out || g.mask_src || g.n_peers > 0) return best;
    if (g.k < 2048 || g.n * g.k < (int64_t(1) << 23)) return best;
    const int block_k = 128 / es;
    const int k_blocks = int((g.k + block_k - 1) / block_k);
    const int sms = sm_count();
    const int64_t tiles_m = (g.m + kBM - 1) / kBM;
    const double dram_us = (double(g.m) * g.k + double(g.k) * g.n + double(g.m) * g.n) * es / 4.5e6;
    // as many CTAs as fit in one wave, wide tiles first (bytes per issued instruction)
    for (int bn : {256, 128}) {
        if (g.n <= bn / 2) continue;
        const int64_t tiles = tiles_m * ((g.n + bn - 1) / bn);
        const double us_per_k_block = bn == 256 ? 0.39 : 0.34;
        for (int sl : {8, 4, 2}) {
            if (k_blocks / sl < 4) continue;
            const int bps = (k_blocks + sl - 1) / sl;
            if ((sl - 1) * bps >= k_blocks) continue;         // an empty last slice
            const int64_t ctas = tiles * sl;
            if (ctas > sms || ctas * 2 < sms) continue;       // one wave, and not a mostly idle GPU
            const int cap = cluster_k_capacity(bn, sl);       // clusters of this size the GPU holds at once (GPC boundaries)
            if (cap > 0 && tiles > cap) continue;
            const double us = 8.0 + std::max(double(bps) * us_per_k_block, dram_us) + 1.5;
            if (us < best.us * 0.97) best = ClusterKPlan{bn, sl, us, true};
        }
    }
    return best;
}

int launch_f16_cluster_k(const GemmArgs& g, const Planned& pl16, const ClusterKPlan& plan, cudaStream_t stream) {
    if (!plan.valid) return NTB200_ERR_UNSUPPORTED;
    const int es = pl16.es, block_k = 128 / es;
    const int k_blocks = int((g.k + block_k - 1) / block_k);
    const int bn = plan.bn, slices = plan.slices;
    Maps maps;
    int a_rows_staged = kBM;
    {
        OperandPlan probe;
        if (plan_operand(g.a, es, pl16.dt, g.m, g.k, g.a_rs, g.a_cs, 1, 0, kBM, block_k, &probe)) return NTB200_ERR_UNSUPPORTED;
        if (!probe.mn_major && g.m <= 64 && !g_full_a_tile) a_rows_staged = g.m <= 8 ? 8 : (g.m <= 16 ? 16 : (g.m <= 32 ? 32 : 64));
    }
    const int tiles_m = int((g.m + kBM - 1) / kBM);
    if (plan_operand(g.a, es, pl16.dt, g.m, g.k, g.a_rs, g.a_cs, 1, 0, a_rows_staged, block_k, &maps.a)) return NTB200_ERR_UNSUPPORTED;
    if (plan_operand(g.b, es, pl16.dt, g.n, g.k, g.b_cs, g.b_rs, 1, 0, bn, block_k, &maps.b)) return NTB200_ERR_UNSUPPORTED;
    ClusterKParams cp{};
    UmmaParams& p = cp.u;
    p.m = int(g.m); p.n = int(g.n); p.k = int(g.k); p.batch = 1;
    p.tiles_m = tiles_m; p.tiles_n = int((g.n + bn - 1) / bn);
    p.k_blocks = k_blocks; p.chunk_blocks = k_blocks; p.group_m = 8; p.total_tiles = p.tiles_m * p.tiles_n;
    p.block_k = block_k;
    p.idesc = make_instr_desc(pl16.d_fmt, pl16.in_fmt, pl16.in_fmt, maps.a.mn_major, maps.b.mn_major, uint32_t(kBM), uint32_t(bn));
    p.a_mn_major = maps.a.mn_major; p.b_mn_major = maps.b.mn_major;
    p.chunk_mn = 128 / es;
    p.chunk_bytes = uint32_t(block_k) * 128u;
    p.a_chunks = kBM / p.chunk_mn;
    p.b_chunks = bn / p.chunk_mn;
    p.a_lbo = maps.a.mn_major ? p.chunk_bytes : 16u;
    p.b_lbo = maps.b.mn_major ? p.chunk_bytes : 16u;
    const uint32_t mn_kstep = uint32_t(32 / es) * 128u / 16u;
    p.a_kstep = maps.a.mn_major ? mn_kstep : 2u;
    p.b_kstep = maps.b.mn_major ? mn_kstep : 2u;
    p.c = g.c; p.c_rs = g.c_rs; p.c_bs = g.c_bs;
    p.bias = g.bias; p.bias_rs = g.bias_rs; p.bias_cs = g.bias_cs; p.bias_bs = g.bias_bs;
    p.accumulate = g.accumulate;
    p.out_kind = pl16.out_kind;
    cp.slices = slices;
    cp.blocks_per_slice = (k_blocks + slices - 1) / slices;
    if ((slices - 1) * cp.blocks_per_slice >= k_blocks) return NTB200_ERR_UNSUPPORTED;   // an empty last slice
    cp.pitch = bn + 4;
    cp.rows_live = int(std::min<int64_t>(kBM, (g.m + 31) / 32 * 32));   // every M tile but the last is full
    cp.c_wide_ok = (reinterpret_cast<uintptr_t>(g.c) % 8 == 0 && g.c_rs % 4 == 0) ? 1 : 0;
    const int rc = bn == 256 ? launch_cluster_k_instance<256>(maps, cp, a_rows_staged, p.total_tiles, stream)
                             : launch_cluster_k_instance<128>(maps, cp, a_rows_staged, p.total_tiles, stream);
    if (rc == NTB200_OK) note_route(g.dtype == NTB200_F16 ? "umma_f16_clusterk" : "umma_bf16_clusterk");
    return rc;
}


constexpr uint32_t kPairClusterSmem = 6u * 2u * kPairOperandBytes + 512u + 1024u;

// Clusters of S pairs that fit the device at once, S = 2 / 4 (cluster of 4 / 8 CTAs); 0 = unknown or none.
int pair_cluster_capacity(int slices) {
    static std::atomic<int> cached[64][5];
    int dev = 0;
    (void)cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || slices < 1 || slices > 4) return 0;
    int v = cached[dev][slices].load(std::memory_order_relaxed);
    if (v == 0) {
        auto kernel = umma_gemm_pair_cluster_k_kernel<0>;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairClusterSmem)) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        v = active_clusters_query(reinterpret_cast<const void*>(kernel), kPairClusterSmem, 2 * slices, kPairClusterThreads);
        cached[dev][slices].store(v > 0 ? v : -1, std::memory_order_relaxed);
    }
    return v > 0 ? v : 0;
}

struct PairClusterPlan {
    int slices;
    double us;
    bool valid;
};

// More than 128 rows of 16-bit floats, fewer 256 x 256 tiles than half the pairs: S pairs per tile.
PairClusterPlan plan_pair_cluster_k(const GemmArgs& g, int es) {
    PairClusterPlan best{0, 1e30, false};
    static const bool disabled = [] { const char* e = getenv("NTB200_NO_PAIR_CLUSTER_K"); return e && e[0] == '1'; }();
    if (disabled || g_disable_pair || es != 2 || g.no_alloc || g.batch != 1 || g.relu_out || g.mask_src || g.n_peers > 0) return best;
    if (g.m <= kBM || g.n <= 128) return best;
    const int block_k = 128 / es;
    const int k_blocks = int((g.k + block_k - 1) / block_k);
    const int64_t tiles = ((g.m + 255) / 256) * ((g.n + 255) / 256);
    const double dram_us = (double(g.m) * g.k + double(g.k) * g.n + double(g.m) * g.n) * es / 4.5e6;
    for (int sl : {4, 2}) {
        if (k_blocks / sl < 4) continue;
        const int bps = (k_blocks + sl - 1) / sl;
        if ((sl - 1) * bps >= k_blocks) continue;
        const int cap = pair_cluster_capacity(sl);
        if (cap <= 0 || tiles > cap) continue;                 // one wave only: the point is to finish a tile sooner
        const double us = 7.0 + std::max(double(bps) * 0.29, dram_us) + 2.0;
        if (us < best.us * 0.97) best = PairClusterPlan{sl, us, true};
    }
    return best;
}

int launch_f16_pair_cluster_k(const GemmArgs& g, const Planned& pl16, const PairClusterPlan& plan, cudaStream_t stream) {
    if (!plan.valid) return NTB200_ERR_UNSUPPORTED;
    const int es = pl16.es, block_k = 128 / es;
    Maps maps;
    if (plan_operand(g.a, es, pl16.dt, g.m, g.k, g.a_rs, g.a_cs, 1, 0, kBM, block_k, &maps.a)) return NTB200_ERR_UNSUPPORTED;
    if (plan_operand(g.b, es, pl16.dt, g.n, g.k, g.b_cs, g.b_rs, 1, 0, 128, block_k, &maps.b)) return NTB200_ERR_UNSUPPORTED;
    ClusterKParams cp{};
    UmmaParams& p = cp.u;
    p.m = int(g.m); p.n = int(g.n); p.k = int(g.k); p.batch = 1;
    p.tiles_m = int((g.m + 255) / 256); p.tiles_n = int((g.n + 255) / 256);
    p.k_blocks = int((g.k + block_k - 1) / block_k); p.chunk_blocks = p.k_blocks; p.group_m = 8;
    p.total_tiles = p.tiles_m * p.tiles_n;
    p.block_k = block_k;
    p.idesc = make_instr_desc(pl16.d_fmt, pl16.in_fmt, pl16.in_fmt, maps.a.mn_major, maps.b.mn_major, 256u, 256u);
    p.a_mn_major = maps.a.mn_major; p.b_mn_major = maps.b.mn_major;
    p.chunk_mn = 128 / es;
    p.chunk_bytes = uint32_t(block_k) * 128u;
    p.a_chunks = kBM / p.chunk_mn;
    p.b_chunks = 128 / p.chunk_mn;
    p.a_lbo = maps.a.mn_major ? p.chunk_bytes : 16u;
    p.b_lbo = maps.b.mn_major ? p.chunk_bytes : 16u;
    const uint32_t mn_kstep = uint32_t(32 / es) * 128u / 16u;
    p.a_kstep = maps.a.mn_major ? mn_kstep : 2u;
    p.b_kstep = maps.b.mn_major ? mn_kstep : 2u;
    p.c = g.c; p.c_rs = g.c_rs; p.c_bs = g.c_bs;
    p.bias = g.bias; p.bias_rs = g.bias_rs; p.bias_cs = g.bias_cs; p.bias_bs = g.bias_bs;
    p.accumulate = g.accumulate;
    p.out_kind = pl16.out_kind;
    cp.slices = plan.slices;
    cp.blocks_per_slice = (p.k_blocks + plan.slices - 1) / plan.slices;
    cp.pitch = 256 + 4;
    cp.rows_live = 128;
    cp.c_wide_ok = (reinterpret_cast<uintptr_t>(g.c) % 8 == 0 && g.c_rs % 4 == 0) ? 1 : 0;
    if (uint32_t(128 * cp.pitch * 4) > 6u * 2u * kPairOperandBytes) return NTB200_ERR_UNSUPPORTED;   // the partial tile lives in the ring
    // The partial tiles cross the slices through scratch that stays in L2 (128 KB per CTA, at most one wave of CTAs);
    // NTB200_PAIR_CLUSTER_DSMEM=1 keeps the exchange through distributed shared memory instead.
    static const bool dsmem = [] { const char* e = getenv("NTB200_PAIR_CLUSTER_DSMEM"); return e && e[0] == '1'; }();
    void* exchange = nullptr;
    if (!dsmem) {
        const size_t bytes = size_t(p.total_tiles) * 2 * plan.slices * kExchangeRegion * sizeof(float4);
        if (scratch_acquire(&exchange, bytes, stream) != NTB200_OK) exchange = nullptr;   // the distributed-shared-memory exchange needs none
    }
    cp.exchange = static_cast<float*>(exchange);
    CUtensorMap map_c = maps.a.map;   // a valid map either way; used only when c_tma_ok
    static const bool copy_out = [] { const char* e = getenv("NTB200_PAIR_CLUSTER_COPY_OUT"); return e && e[0] == '1'; }();
    cp.c_tma_ok = (exchange && !copy_out && !g_direct_stores && plan_store(g.c, pl16.dt, 2, g.m, g.n, 1, g.c_rs, g.c_bs, &map_c)) ? 1 : 0;
    auto kernel = umma_gemm_pair_cluster_k_kernel<0>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(p.total_tiles * 2 * plan.slices), 1, 1);
    cfg.blockDim = dim3(kPairClusterThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairClusterSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = unsigned(2 * plan.slices);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, maps.a.map, maps.b.map, map_c, cp);
    if (exchange) scratch_release(exchange, stream);
    if (e != cudaSuccess) return cuda_fail(e, "umma_gemm_pair_cluster_k_kernel launch");
    count_launch();
    note_route(g.dtype == NTB200_F16 ? "umma_f16_pairclusterk" : "umma_bf16_pairclusterk");
    return NTB200_OK;
}

}  // namespace

bool umma_cluster_k_would_run(const GemmArgs& g) {
    if (g.dtype != NTB200_F16 && g.dtype != NTB200_BF16) return false;
    if (g.m > kBM || operands_stageable(g) != nullptr) return false;
    return plan_cluster_k(g, 2).valid;
}

bool umma_supported(const GemmArgs& g, const char** why) {
    const char* w = operands_stageable(g);
    if (why) *why = w;
    return w == nullptr;
}

int launch_umma_gemm(const GemmArgs& g, cudaStream_t stream) {
    if (const char* w = operands_stageable(g)) return fail(NTB200_ERR_UNSUPPORTED, "tcgen05 route: %s", w);
    if (g.dtype == NTB200_F32) return launch_f32_split(g, stream);
    if (g.dtype == NTB200_I32 || g.dtype == NTB200_U32) return launch_int_limbs<uint32_t, 4>(g, stream);
    if (g.dtype == NTB200_I16 || g.dtype == NTB200_U16) return launch_int_limbs<uint16_t, 2>(g, stream);
    const int es = int(dtype_size(g.dtype));
    const bool is_i8 = es == 1;
    Planned pl;
    pl.es = es;
    pl.dt = g.dtype == NTB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
            : g.dtype == NTB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    pl.kind = is_i8 ? MmaKind::i8 : MmaKind::f16;
    pl.out_kind = is_i8 ? kOutI8 : (g.dtype == NTB200_F16 ? kOutF16 : kOutBF16);
    pl.d_fmt = is_i8 ? 2u : 1u;
    pl.in_fmt = g.dtype == NTB200_BF16 ? 1u : (g.dtype == NTB200_I8 ? 1u : 0u);
    pl.split = false;
    pl.route = is_i8 ? "umma_i8" : (g.dtype == NTB200_F16 ? "umma_f16" : "umma_bf16");
    const TileChoice* choice = nullptr;
    F16Plan plan{};
    if (is_i8) {
        plan = plan_f16_tiles(g, 1);
        if (plan.valid && !tune_int("NTB200_OLD_PLAN")) choice = &plan.tile;
    } else {
        int splits = pick_k_splits(g);
        plan = plan_f16_tiles(g);
        if (plan.valid && !tune_int("NTB200_OLD_PLAN")) {
            choice = &plan.tile;
            splits = plan.splits;
        }
        if (const int f = tune_int("NTB200_FORCE_SPLITS")) {
            choice = nullptr;
            splits = (!g.no_alloc && g.batch == 1 && !g.relu_out && !g.mask_src && g.n_peers == 0 && g.n % 4 == 0 && g.k % (64 * f) == 0) ? f : 1;
        }
        if (!tune_int("NTB200_FORCE_SPLITS")) {
            // K slices inside a cluster (one launch): always for few rows; for more rows when its estimate beats the
            // planner's best tile kind / slice count by a margin
            // K slices inside a cluster (one launch): single-CTA tiles for few rows; S CTA pairs per 256 x 256 tile for
            // more rows, when that beats the planner's best tile kind / slice count
            if (g.m <= kBM) {
                const ClusterKPlan ck = plan_cluster_k(g, es);
                if (ck.valid) {
                    const int rc = launch_f16_cluster_k(g, pl, ck, stream);
                    if (rc != NTB200_ERR_UNSUPPORTED) return rc;
                }
            } else {
                const PairClusterPlan pk = plan_pair_cluster_k(g, es);
                if (pk.valid && (!plan.valid || pk.us < plan.us)) {
                    const int rc = launch_f16_pair_cluster_k(g, pl, pk, stream);
                    if (rc != NTB200_ERR_UNSUPPORTED) return rc;
                }
            }
        }
        if (splits > 1) return launch_f16_split_k(g, pl, splits, choice, stream);
    }
    const Side a{g.a, g.a_rs, g.a_cs, g.a_bs}, b{g.b, g.b_cs, g.b_rs, g.b_bs};
    return launch_planned(g, pl, a, b, nullptr, nullptr, stream, choice);
}

// Self-test of the bounded-wait plumbing: one thread waits on an mbarrier that nothing ever signals, with a short
// limit; the wait must give up, raise the device status word and let the kernel return normally.
__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_barrier_init();
        if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_ns)) raise_timeout(&abort_flag, 0x7f);
    }
}

int launch_wait_timeout_selftest(unsigned long long limit_ns, cudaStream_t stream) {
    wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(limit_ns);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

unsigned int* device_status_word() {
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_device_status) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return static_cast<unsigned int*>(addr);
}

void* tensor_map_encoder() { return reinterpret_cast<void*>(encode_fn()); }

int max_resident_pairs(const void* kernel, uint32_t smem_bytes) { return resident_pairs_query(kernel, smem_bytes); }

int read_device_status(cudaStream_t stream) {
    NTB200_CUDA(cudaStreamSynchronize(stream));
    unsigned int st = 0;
    NTB200_CUDA(cudaMemcpyFromSymbol(&st, g_device_status, sizeof(st)));
    if (st) {
        unsigned int zero = 0;
        NTB200_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero)));
        return fail(NTB200_ERR_TIMEOUT, "a device-side wait ran out (code 0x%x)", st);
    }
    return NTB200_OK;
}

}  // namespace ntb200
