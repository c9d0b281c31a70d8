/* ntb200 -- C ABI of the B200 (sm_100a) dense-contraction engine behind NeuroTensor's matmult path.
 *
 * Plain C, plain pointers and sizes: this is the boundary a NeuroTensor build binds instead of its CPU
 * GEMM templates.  Every entry point returns an ntb200_status (0 = ok) and never throws; the text of the
 * last failure on the calling thread is available from ntb200_last_error_string().
 *
 * Unless a function says "host", pointers are DEVICE pointers valid on the current CUDA device, `stream`
 * is a cudaStream_t passed as void* (NULL = the legacy default stream) and calls are asynchronous on it.
 * There is no CPU fallback anywhere: without a usable CUDA device every compute entry point fails with
 * NTB200_ERR_NO_DEVICE / NTB200_ERR_CUDA.
 *
 * File:line citations name the reference interface (NeuroTensor, paths relative to its project root)
 * that each entry point replaces.
 */
#ifndef NTB200_H_
#define NTB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types.  Output and accumulation follow the reference: the result has the operands' dtype;
 * integers wrap modulo 2^bits (signed and unsigned share kernels); F16/BF16 accumulate in fp32. */
typedef enum ntb200_dtype {
    NTB200_F32 = 0,
    NTB200_F16 = 1,
    NTB200_BF16 = 2, /* not a dtype of the reference; added for this engine */
    NTB200_I8 = 3,
    NTB200_I16 = 4,
    NTB200_I32 = 5,
    NTB200_I64 = 6,
    NTB200_F64 = 7,
    NTB200_U8 = 8,
    NTB200_U16 = 9,
    NTB200_U32 = 10,
    /* Complex64 / Complex128 (interleaved re, im).  The reference's GEMM traits for these types are the plain float /
     * double vector operations on the interleaved lanes (nt/mp/simde_traits/simde_traits_avx2.h:915-1000,1029-1110:
     * broadcast = set1 of the pair, fmadd = _mm256_fmadd_ps / _pd), so its matmult multiplies real parts with real
     * parts and imaginary parts with imaginary parts: C.re = A.re B.re, C.im = A.im B.im, each an exact sequential FMA
     * chain.  These codes reproduce exactly that (bit for bit), on the CUDA-core route; they are NOT the mathematical
     * complex product. */
    NTB200_C64 = 11,
    NTB200_C128 = 12, /* the reference's own Complex128 matmult leaves C untouched (its load / store switch has no case for
                       * this type's tile size of 4, nt/functional/cpu/matmult/nt_matmult_macros.h:413-438); this code
                       * computes the lane-wise product its traits define, like NTB200_C64 */
    NTB200_C32 = 13   /* Complex32, a pair of Float16: lane-wise like the other two, fp32 within a K tile of 8, the running
                       * sums rounded to Float16 at every tile edge (simde_traits_avx2.h:1270-1300); CUDA-core route */
} ntb200_dtype;

typedef enum ntb200_status {
    NTB200_OK = 0,
    NTB200_ERR_INVALID_ARG = 1,  /* what the reference reports as std::invalid_argument */
    NTB200_ERR_UNSUPPORTED = 2,  /* dtype / layout this engine does not cover */
    NTB200_ERR_ALLOC = 3,
    NTB200_ERR_CUDA = 4,
    NTB200_ERR_TIMEOUT = 5,      /* a bounded device-side wait ran out (see ntb200_check_device_status) */
    NTB200_ERR_NO_DEVICE = 6
} ntb200_status;

/* Which kernel family a GEMM is routed to.  AUTO picks tcgen05 tensor cores for F16/BF16/I8/U8 when the
 * operands can be described by a TMA tensor map (unit stride along rows or columns, 16-byte aligned base
 * and other strides) and the CUDA-core kernel otherwise. */
typedef enum ntb200_route {
    NTB200_ROUTE_AUTO = 0,
    NTB200_ROUTE_TENSOR = 1,  /* fail with NTB200_ERR_UNSUPPORTED if tcgen05 cannot take it */
    NTB200_ROUTE_SIMT = 2     /* CUDA-core kernel: one ascending-k chain per output element */
} ntb200_route;

/* F16 rounding on the CUDA-core route.  The reference rounds the running sum to fp16 after every 16
 * k-steps (nt/mp/simde_traits/simde_traits_avx2.h:1133-1165 with nt/functional/cpu/matmult/nt_matmult.hpp:196);
 * NTB200_F16_ROUND_PER_KTILE reproduces that bit for bit, NTB200_F16_ROUND_ONCE keeps fp32 to the end. */
typedef enum ntb200_f16_rounding { NTB200_F16_ROUND_ONCE = 0, NTB200_F16_ROUND_PER_KTILE = 1 } ntb200_f16_rounding;

/* General strided, batched GEMM:  C[b] = (accumulate ? C[b] : 0) + bias + A[b] . B[b]
 * A is m x k, B is k x n, C is m x n (column stride 1).  Strides are in ELEMENTS; a transposed view is a
 * pair of swapped strides, never a copy.  A batch stride of 0 repeats the operand over the batch. */
typedef struct ntb200_gemm_desc {
    int32_t dtype;      /* ntb200_dtype */
    int32_t route;      /* ntb200_route */
    int32_t accumulate; /* 0: overwrite C, 1: C += (the reference's raw-pointer contract) */
    int32_t f16_rounding;
    int64_t m, n, k, batch;
    const void* a; int64_t a_row_stride, a_col_stride, a_batch_stride;
    const void* b; int64_t b_row_stride, b_col_stride, b_batch_stride;
    void* c;       int64_t c_row_stride, c_batch_stride;
    const void* bias; /* optional (NULL = none); same dtype */
    int64_t bias_row_stride, bias_col_stride, bias_batch_stride;
} ntb200_gemm_desc;

/* ---- library / device ---------------------------------------------------------------------------- */
const char* ntb200_version(void);
const char* ntb200_last_error_string(void);
int ntb200_device_count(int* count);
int ntb200_set_device(int device);
int ntb200_get_device(int* device);
/* Number of this library's kernels launched by the process so far (all threads, all devices). */
uint64_t ntb200_kernel_launch_count(void);
/* Name of the kernel family the most recent GEMM on this thread was routed to ("umma_f16", "simt", ...). */
const char* ntb200_last_gemm_route(void);
/* Synchronises `stream` and reports NTB200_ERR_TIMEOUT if any kernel since the last check gave up a wait. */
int ntb200_check_device_status(void* stream);

/* Failure-path self-test (no counterpart in the reference): launches a one-thread kernel that waits, for at most
 * `limit_ms` (1..1000), on a barrier nothing signals.  The wait gives up, the kernel returns normally, and the next
 * ntb200_check_device_status reports NTB200_ERR_TIMEOUT once; the context stays usable.  Exercises the same bounded
 * wait every GEMM role uses, without faulting or hanging anything. */
int ntb200_selftest_wait_timeout(unsigned int limit_ms, void* stream);

/* ---- storage: replaces DeviceCPU::allocate / release (nt/memory/device.cpp:46-92) with a stream-ordered
 * pool (cudaMallocAsync) on the current device. ---------------------------------------------------------- */
int ntb200_malloc_async(void** ptr, size_t bytes, void* stream);
int ntb200_free_async(void* ptr, void* stream);
int ntb200_memset_async(void* ptr, int value, size_t bytes, void* stream);
int ntb200_memcpy_h2d_async(void* dst_device, const void* src_host, size_t bytes, void* stream);
int ntb200_memcpy_d2h_async(void* dst_host, const void* src_device, size_t bytes, void* stream);
int ntb200_memcpy_d2d_async(void* dst_device, const void* src_device, size_t bytes, void* stream);
int ntb200_stream_synchronize(void* stream);
/* Page-locked host memory for tensors that stay on the CPU side of the boundary: what DeviceCPU::allocate /
 * release (nt/memory/device.cpp:46-92, 64-byte aligned_alloc) should call so that ntb200_matmult_host copies
 * run asynchronously at full PCIe speed.  ntb200_host_register pins memory the application already owns. */
int ntb200_host_alloc(void** ptr, size_t bytes);
int ntb200_host_free(void* ptr);
int ntb200_host_register(void* ptr, size_t bytes);
int ntb200_host_unregister(void* ptr);
/* Bytes currently held / high-water mark of the pool: the device counterpart of
 * nt::utils::getAllocatedMemory (nt/memory/track_memory.h:23-35).  Counts ntb200_malloc_async blocks. */
int ntb200_pool_stats(uint64_t* bytes_in_use, uint64_t* high_water);
/* Scratch of the library's own kernels (no counterpart in the reference, whose pack buffers are static arrays,
 * nt/functional/cpu/matmult/nt_matmult_macros.h:60-71).  Routes that copy or slice their operands (Float32 as three
 * TF32 products, integer limb planes, K slices, weight streaming) take a block from the stream-ordered pool and keep
 * it for the next call on the same (device, stream), so a GEMM call allocates nothing once its stream is warm.
 * Blocks above NTB200_SCRATCH_KEEP_MB (environment, default 512) are allocated and freed per call.
 * scratch_stats: bytes kept right now, blocks handed out so far, and how many of those needed a new allocation.
 * scratch_release_all: returns every idle kept block to the pool (waits for the kernels still using them). */
int ntb200_scratch_stats(uint64_t* retained_bytes, uint64_t* acquisitions, uint64_t* allocations);
int ntb200_scratch_release_all(void);
/* The current device's default stream-ordered pool as the CUDA runtime accounts for it: bytes handed out now, their
 * high-water mark (reset_high != 0 first resets the mark to zero) and bytes the pool holds from the driver.  Every
 * allocation this library makes on a compute path goes through that pool, so a caller can check that a call
 * allocated nothing. */
int ntb200_device_pool_usage(uint64_t* used_now, uint64_t* used_high, uint64_t* reserved_now, int reset_high);

/* Optional fused neighbours of Linear for ntb200_gemm_fused (F16 / BF16 on the tensor-core route, accumulate = 0).
 * Both tensors have exactly C's layout (same row and batch strides); a NULL member is simply not used.
 * relu_out:      a second output, relu(C) = clamp(C, 0, none) of the rounded result (nn/functional/min_max.cpp:40-63),
 *                so one launch yields the pre-activation C and the activation;
 * relu_mask_src: the forward input h of a ReLU; the result is zeroed where h < 0, which is the clamp backward
 *                applied to the gradient this GEMM produces (dH = mask(dA)). */
typedef struct ntb200_gemm_epilogue {
    void* relu_out;
    const void* relu_mask_src;
} ntb200_gemm_epilogue;

/* ---- GEMM ----------------------------------------------------------------------------------------- */
int ntb200_gemm(const ntb200_gemm_desc* desc, void* stream);
/* ntb200_gemm with the fused epilogue members above (`epilogue` may be NULL: then identical to ntb200_gemm). */
int ntb200_gemm_fused(const ntb200_gemm_desc* desc, const ntb200_gemm_epilogue* epilogue, void* stream);

/* Multi-GPU (no counterpart in the reference, which has a single CPU device).  ntb200_gemm_push is ntb200_gemm
 * whose epilogue stores every finished tile of C into this GPU's C AND into up to 7 peer-mapped copies of C on
 * other GPUs (same layout, plain stores over NVLink): the all-gather of an N-sharded GEMM fused into the GEMM.
 * F16 / BF16, tcgen05 route only.  The kernel does not wait for anybody; the caller orders the ranks with one
 * collective (a barrier) before any rank reads its gathered buffer, and must not let a rank overwrite a buffer
 * that a slower peer may still be reading (alternate two buffers).
 * The peer_* helpers allocate buffers that can be mapped into other processes (cudaMalloc + CUDA IPC): export
 * gives a 64-byte handle to send to the peers, import maps a peer's buffer here and enables peer access. */
int ntb200_gemm_push(const ntb200_gemm_desc* desc, void* const* peer_c, int n_peers, void* stream);
/* Linear + ReLU of an N-sharded layer in one launch: desc->c receives the pre-activation block (kept by its owner
 * for the backward mask), and max(c, 0) goes to relu_out (row stride relu_row_stride, normally the block's place in
 * this GPU's full activation buffer) and to the same place in up to 7 peer-mapped activation buffers.  One 2-D
 * problem, F16 / BF16, at least 74 tiles of 256 x 256, 16-byte aligned rows.  Ordering rules as for ntb200_gemm_push. */
int ntb200_gemm_push_relu(const ntb200_gemm_desc* desc, void* relu_out, int64_t relu_row_stride, void* const* peer_relu,
                          int n_peers, void* stream);
int ntb200_peer_alloc(void** ptr, size_t bytes);
int ntb200_peer_free(void* ptr);
int ntb200_peer_export(const void* ptr, unsigned char handle[64]);
int ntb200_peer_import(const unsigned char handle[64], void** ptr);
int ntb200_peer_release(void* ptr);

/* ---- the multi-GPU partitioner (no counterpart in the reference: its only device is the CPU,
 * nt/memory/DeviceEnum.h:6-10).  One rank per GPU of one NVLink domain (up to 8): one process per rank, or one host
 * thread per rank inside one process.  No communication library is linked: ranks exchange 88-byte buffer records at
 * set-up through the caller's all-gather callback (torch.distributed, MPI, a socket; a shared array between threads),
 * data crosses NVLink as stores from the GEMM epilogues into peer-mapped buffers, and ranks are ordered by a flag
 * exchange kernel whose polls are bounded (two seconds, then NTB200_ERR_TIMEOUT from ntb200_check_device_status).
 *
 *   ntb200_dist_shard            which units of `total` belong to `rank`: contiguous blocks of `align` units, the first
 *                                (blocks % world) ranks one block more.  Batched matmult shards its batch with
 *                                align = 1 and needs nothing else: items are independent
 *                                (nt/functional/cpu/matmult/nt_matmult.hpp:228-235 is a serial loop over them).
 *                                A GEMM split over its output columns uses align = 8 (16-byte rows of 2-byte types).
 *   ntb200_dist_init             collective over all ranks, with the rank's device current; `exchange` gathers
 *                                `bytes` bytes of every rank, rank-major, into `recv` and returns 0 (may be NULL for one rank).
 *   ntb200_dist_buffer_create    collective: `bytes` on every rank, each block mapped into every rank (zero-filled).
 *                                Two calls of `exchange`: the 88-byte records, then one status word per rank, so a
 *                                rank that cannot allocate or map makes the call fail on EVERY rank (nobody is left
 *                                waiting in a later collective); ntb200_dist_init creates one small buffer this way.
 *   ntb200_dist_gemm_allgather   this rank's column block of C = bias + A.B goes to columns [col0, col0 + n) of the
 *                                gathered [m, gathered_row_stride] matrix in EVERY rank's buffer, stored by the GEMM's
 *                                epilogue, followed by ntb200_dist_barrier on the same stream: when work queued after
 *                                the call runs, every rank's block has arrived here.  relu != 0: desc->c keeps the
 *                                pre-activation block [m, n] and the gathered matrix receives max(C, 0) (Linear + ReLU
 *                                of a column-sharded layer in one launch).  F16 / BF16; desc->c is ignored when relu == 0.
 *                                A rank must not start the next gather into the same buffer while a slower rank may
 *                                still read the previous one: alternate two buffers.
 *   ntb200_dist_allgather_columns the same gather for a block that already exists (any dtype).
 *   ntb200_dist_barrier          orders the ranks on `stream` (asynchronous for the host).  A rank whose peer does not
 *                                arrive within the limit (default 2000 ms, ntb200_dist_set_barrier_limit_ms) gives up:
 *                                the kernel returns, ntb200_check_device_status reports NTB200_ERR_TIMEOUT, the context
 *                                stays usable, and the late peer's own barrier call still completes against the count
 *                                this rank left behind, so the ranks are in step again afterwards. */
typedef struct ntb200_dist_comm ntb200_dist_comm;
typedef struct ntb200_dist_buffer ntb200_dist_buffer;
typedef int (*ntb200_allgather_fn)(void* ctx, const void* send, void* recv, size_t bytes);
int ntb200_dist_shard(int64_t total, int world, int rank, int64_t align, int64_t* start, int64_t* count);
int ntb200_dist_init(ntb200_dist_comm** comm, int rank, int world, ntb200_allgather_fn exchange, void* ctx);
int ntb200_dist_destroy(ntb200_dist_comm* comm);
int ntb200_dist_rank(const ntb200_dist_comm* comm);
int ntb200_dist_world(const ntb200_dist_comm* comm);
int ntb200_dist_buffer_create(ntb200_dist_comm* comm, size_t bytes, ntb200_dist_buffer** buffer);
int ntb200_dist_buffer_destroy(ntb200_dist_buffer* buffer);
void* ntb200_dist_buffer_ptr(const ntb200_dist_buffer* buffer);   /* this rank's block (device pointer) */
int ntb200_dist_barrier(ntb200_dist_comm* comm, void* stream);
int ntb200_dist_set_barrier_limit_ms(ntb200_dist_comm* comm, unsigned int limit_ms);
int ntb200_dist_gemm_allgather(ntb200_dist_comm* comm, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                               int64_t gathered_row_stride, int64_t col0, int relu, void* stream);
/* The same with the block placed at row `row0` of the gathered matrix: row blocks of one matrix can be gathered
 * one after the other, or at the same time on two streams - each stream then needs a communicator of its own (its
 * own flags), while `gathered` may have been created by either. */
int ntb200_dist_gemm_allgather_at(ntb200_dist_comm* comm, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                                  int64_t gathered_row_stride, int64_t row0, int64_t col0, int relu, void* stream);
/* The same without the closing flag exchange: the block is on its way to every rank when the call returns (in stream
 * order), and nothing may read the other ranks' blocks before an ntb200_dist_barrier on the same communicator.  For
 * callers with work that needs only this rank's own block in the meantime. */
int ntb200_dist_gemm_push_at(ntb200_dist_comm* comm, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                             int64_t gathered_row_stride, int64_t row0, int64_t col0, int relu, void* stream);
int ntb200_dist_allgather_columns(ntb200_dist_comm* comm, int dtype, const void* block, int64_t rows, int64_t cols,
                                  int64_t block_row_stride, ntb200_dist_buffer* gathered, int64_t gathered_row_stride,
                                  int64_t col0, void* stream);

/* Replaces nt_matmult<T> (nt/functional/cpu/matmult/nt_matmult.h:6-7; call sites
 * nt/functional/cpu/matmult_cpu.cpp:118,150): C += op(A).op(B), row-major contiguous, a_rows/a_cols and
 * b_rows/b_cols are the logical dims AFTER the transposes (a_cols == b_rows); with transpose_a the
 * buffer holds A as [a_cols][a_rows].  Device pointers. */
int ntb200_matmult(int dtype, const void* A, const void* B, void* C, int64_t a_rows, int64_t a_cols, int64_t b_rows,
                   int64_t b_cols, int transpose_a, int transpose_b, void* stream);

/* Replaces nt_matmult_batch<T> (nt_matmult.h:9-10; call sites matmult_cpu.cpp:740,851): host arrays of
 * `batches` device pointers, same dims and flags for every item.  Equally spaced pointers run as one
 * strided launch; anything else runs through a device pointer table. */
int ntb200_matmult_batch(int dtype, const void* const* A, const void* const* B, void* const* C, int64_t batches,
                         int64_t a_rows, int64_t a_cols, int64_t b_rows, int64_t b_cols, int transpose_a,
                         int transpose_b, void* stream);

/* The same two contracts with HOST buffers, exactly the pointers the reference's CPU templates receive:
 * operands are staged to the device through pinned memory, multiplied there and C is copied back.
 * `batches` contiguous items (A: batches x a-matrix, ...); synchronous.  accumulate = 1 is the templates'
 * C += contract (C is uploaded first); accumulate = 0 overwrites C without uploading it, for the call sites
 * that have just zero-filled C (matmult_cpu.cpp:110,707).  Copies and compute of successive chunks overlap
 * on separate streams; pinned host buffers make the copies asynchronous. */
int ntb200_matmult_host(int dtype, const void* A, const void* B, void* C, int64_t batches, int64_t a_rows,
                        int64_t a_cols, int64_t b_rows, int64_t b_cols, int transpose_a, int transpose_b,
                        int accumulate);

/* ---- linear: replaces cpu::linear (nt/functional/cpu/matmult_cpu.cpp:1624-1714), which preloads C with
 * the broadcast bias and then accumulates the GEMM.  Expressed through ntb200_gemm with `bias` set. ----- */

/* ---- conv2d path -------------------------------------------------------------------------------------
 * Replaces cpu::unfold2d_ / im2col_cpu (nt/functional/cpu/unfold2d.cpp:12-165,219-235):
 * col[b][(c*kh + i)*kw + j][h*Wc + w] = im[b][c][h*sh - ph + i*dh][w*sw - pw + j*dw] (0 in the padding). */
int ntb200_im2col(int dtype, const void* im, void* col, int64_t batch, int64_t channels, int64_t height,
                  int64_t width, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                  int64_t dw, void* stream);
/* Replaces unfold2d_backward / col2im (nt/functional/tensor_files/colim_transform.cpp:592-653): the
 * adjoint of ntb200_im2col; `im` is overwritten.  F32, F16, BF16. */
int ntb200_col2im(int dtype, const void* col, void* im, int64_t batch, int64_t channels, int64_t height,
                  int64_t width, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                  int64_t dw, void* stream);
/* Replaces functional::conv2d for groups == 1 (nt/functional/tensor_files/conv.cpp:69-96):
 * out[B, Cout, Ho, Wo] = unfold2d(x) contracted with w[Cout, C*kh*kw].  `workspace` must hold
 * ntb200_conv2d_workspace_bytes(...) bytes (the column matrix).  F16 / BF16 with stride 1 and channels a
 * multiple of 64 skip the column matrix: the workspace then holds a channels-last copy of x and the
 * reordered weights, and the fp32 sums run tap-major before the single rounding. */
size_t ntb200_conv2d_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                     int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                                     int64_t dh, int64_t dw);
int ntb200_conv2d(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch,
                  int64_t channels, int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh,
                  int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, void* stream);

/* conv2d backward, groups == 1.  Replaces conv_dimage (nt/functional/tensor_files/conv.cpp:318-346):
 *   d_image[B, C, H, W] = col2im( w2d^T . grad )       grad is [B, Cout, Ho, Wo]; d_image is overwritten
 * and conv_dkernel (conv.cpp:444-471):
 *   d_kernel[Cout, C, kh, kw] (+)= sum over the batch of grad[b] . unfold2d(x)[b]^T
 * (`accumulate` != 0 adds to d_kernel as the reference's `d_kernel +=` does).  F32, F16, BF16.  `workspace` must
 * hold ntb200_conv2d_backward_workspace_bytes(...) bytes; one size serves both calls.  For F16 / BF16 with
 * stride 1 the image gradient is evaluated as a convolution of grad with the flipped kernel (no gradient
 * column matrix), which sums in a different order than col2im. */
size_t ntb200_conv2d_backward_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height,
                                              int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh,
                                              int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw);
int ntb200_conv2d_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 int64_t batch, int64_t channels, int64_t height, int64_t width, int64_t cout,
                                 int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
                                 int64_t dw, void* stream);
int ntb200_conv2d_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace,
                                  int accumulate, int64_t batch, int64_t channels, int64_t height, int64_t width,
                                  int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                                  int64_t pw, int64_t dh, int64_t dw, void* stream);

/* conv2d with groups, forward and backward (conv.cpp:97-118, 328-337, 453-461): w is [Cout, C/groups, kh, kw];
 * group g maps input channels [g*C/groups, (g+1)*C/groups) to filters [g*Cout/groups, (g+1)*Cout/groups).
 * Same arguments as the ungrouped calls plus `groups`; groups == 1 forwards to them.  One workspace size
 * (ntb200_conv2d_grouped_workspace_bytes) serves the three calls.  conv1d is the H == 1, kh == 1 case;
 * conv_transpose2d(x, w) is ntb200_conv2d_grouped_backward_image with x in the place of grad, and its own
 * gradients are ntb200_conv2d_grouped (for x) and ntb200_conv2d_grouped_backward_kernel with the roles of
 * image and gradient exchanged (for w). */
size_t ntb200_conv2d_grouped_workspace_bytes(int dtype, int64_t batch, int64_t channels, int64_t height,
                                             int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh,
                                             int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw,
                                             int64_t groups);
int ntb200_conv2d_grouped(int dtype, const void* x, const void* w, void* out, void* workspace, int64_t batch,
                          int64_t channels, int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw,
                          int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, int64_t groups,
                          void* stream);
int ntb200_conv2d_grouped_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                         int64_t batch, int64_t channels, int64_t height, int64_t width,
                                         int64_t cout, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph,
                                         int64_t pw, int64_t dh, int64_t dw, int64_t groups, void* stream);
int ntb200_conv2d_grouped_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel,
                                          void* workspace, int accumulate, int64_t batch, int64_t channels,
                                          int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw,
                                          int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw,
                                          int64_t groups, void* stream);

/* ---- conv3d -------------------------------------------------------------------------------------------
 * functional::conv3d / unfold3d and their backward (nt/functional/tensor_files/conv.cpp:122-174 and the dim == 3
 * cases of conv_dimage / conv_dkernel; colim_transform.cpp:661-800).  x is [B, C, D, H, W], w is
 * [Cout, C/groups, kd, kh, kw]; the three-element arrays are ordered (depth, height, width).  The column matrix
 * is col[b][((c*kd + kz)*kh + ky)*kw + kx][(z*Ho + y)*Wo + x].  One workspace size serves the three conv3d calls.
 * conv_transpose3d(x, w) is ntb200_conv3d_backward_image with x in the place of grad (as in the 2-D case).
 * This struct is frozen: new inputs get new entry points. */
typedef struct ntb200_conv3d_geom {
    int64_t batch, channels, depth, height, width, cout, groups;
    int64_t kernel[3], stride[3], padding[3], dilation[3];
} ntb200_conv3d_geom;
int ntb200_im2col3d(int dtype, const void* im, void* col, const ntb200_conv3d_geom* geom, void* stream);
int ntb200_col2im3d(int dtype, const void* col, void* im, const ntb200_conv3d_geom* geom, void* stream);
size_t ntb200_conv3d_workspace_bytes(int dtype, const ntb200_conv3d_geom* geom);
int ntb200_conv3d(int dtype, const void* x, const void* w, void* out, void* workspace, const ntb200_conv3d_geom* geom,
                  void* stream);
int ntb200_conv3d_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 const ntb200_conv3d_geom* geom, void* stream);
int ntb200_conv3d_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace,
                                  int accumulate, const ntb200_conv3d_geom* geom, void* stream);

/* ---- convnd ---------------------------------------------------------------------------------------------
 * functional::convnd / conv_transposend / unfoldnd for any number N of spatial dimensions
 * (nt/functional/tensor_files/conv.cpp:177-262 and :747-860; nt/functional/cpu/unfoldnd.cpp,
 * unfoldnd_backward.cpp), 1 <= N <= NTB200_CONVND_MAX_DIMS.  x is [B, C, size_0 .. size_{N-1}], w is
 * [Cout, C/groups, kernel_0 .. kernel_{N-1}]; the arrays hold one entry per spatial dimension, outermost
 * first, entries past dims are ignored.  The column matrix is col[b][(c, k_0 .. k_{N-1})][(o_0 .. o_{N-1})],
 * both index groups flattened row-major - for N = 1, 2, 3 exactly the layouts of unfold1d/2d/3d, which is what
 * the reference's own tests assert of unfoldnd (tests/src/col_im_tests.cpp:47-83).  One workspace size serves
 * the three calls.  conv_transposend(x, w) is ntb200_convnd_backward_image with x in the place of grad.
 * This struct is frozen: new inputs get new entry points. */
#define NTB200_CONVND_MAX_DIMS 8
typedef struct ntb200_convnd_geom {
    int64_t dims, batch, channels, cout, groups;
    int64_t size[NTB200_CONVND_MAX_DIMS], kernel[NTB200_CONVND_MAX_DIMS], stride[NTB200_CONVND_MAX_DIMS],
            padding[NTB200_CONVND_MAX_DIMS], dilation[NTB200_CONVND_MAX_DIMS];
} ntb200_convnd_geom;
int ntb200_im2colnd(int dtype, const void* im, void* col, const ntb200_convnd_geom* geom, void* stream);
int ntb200_col2imnd(int dtype, const void* col, void* im, const ntb200_convnd_geom* geom, void* stream);
size_t ntb200_convnd_workspace_bytes(int dtype, const ntb200_convnd_geom* geom);
int ntb200_convnd(int dtype, const void* x, const void* w, void* out, void* workspace, const ntb200_convnd_geom* geom,
                  void* stream);
int ntb200_convnd_backward_image(int dtype, const void* grad, const void* w, void* d_image, void* workspace,
                                 const ntb200_convnd_geom* geom, void* stream);
int ntb200_convnd_backward_kernel(int dtype, const void* x, const void* grad, void* d_kernel, void* workspace,
                                  int accumulate, const ntb200_convnd_geom* geom, void* stream);

/* ntb200_conv2d for callers that cannot allocate device memory.  No counterpart in the reference, which
 * allocates its column matrix on the CPU heap as it goes.  Some users of this library cannot do the
 * device-side equivalent: their application has given the whole device heap to its own allocator, so a
 * cudaMalloc from anywhere else fails, or they are in a phase in which they do not allow themselves
 * cudaMalloc because it synchronises the device.  This variant takes the same inputs and output as
 * ntb200_conv2d but no workspace: the column matrix lives in a fixed array of
 * NTB200_CONV2D_STATIC_SCRATCH_BYTES inside the library, which every GPU that loads the library holds until
 * the process exits.  The call (and everything under it) uses no cudaMalloc / cudaFree / pool allocation: its GEMM
 * keeps to the routes that need no scratch of their own, so Float32, Int16 and Int32 run on the CUDA-core kernel
 * whatever their size (bit-exact, slower than ntb200_conv2d on large problems) and 16-bit floats never take K
 * slices or the weight-streaming kernels.
 *   - A problem whose column matrix (ntb200_conv2d_workspace_bytes) is larger than the array is refused with
 *     NTB200_ERR_INVALID_ARG and a message naming both sizes; nothing is launched.
 *   - The first call on each device looks up the array's device address (one cudaGetSymbolAddress with that
 *     device current).  With CUDA's lazy module loading
 *     (the default) the runtime also creates the array's 32 MiB of device storage at that moment, which fails with
 *     NTB200_ERR_ALLOC if the application has already taken the whole heap: make the first call (any tiny valid
 *     problem) before that, or run with CUDA_MODULE_LOADING=EAGER so the storage exists from library load on.
 *   - All calls on a device share the one array, and it keeps the previous call's contents.  Each call rewrites
 *     every element it reads, so stale contents never reach a result, but two calls that overlap on the GPU
 *     (different streams, no ordering between them) race on it: order them. */
#define NTB200_CONV2D_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int ntb200_conv2d_static_scratch(int dtype, const void* x, const void* w, void* out, int64_t batch, int64_t channels,
                                 int64_t height, int64_t width, int64_t cout, int64_t kh, int64_t kw, int64_t sh,
                                 int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, void* stream);

/* ---- elementwise neighbours of the GEMM in Linear forward/backward ----------------------------------
 * relu = clamp(x, 0, none) and its mask backward (nt/nn/functional/min_max.cpp:40-63). */
int ntb200_relu(int dtype, const void* x, void* y, int64_t n, void* stream);
int ntb200_relu_backward(int dtype, const void* x, const void* grad_out, void* grad_in, int64_t n, void* stream);
/* loss::MSE (nt/nn/Loss.cpp:49-55): *loss (float, device) = sum((o-t)^2)/n ; grad = 2(o-t)/n in `dtype`. */
int ntb200_mse(int dtype, const void* out, const void* target, void* grad, float* loss, int64_t n, void* stream);
/* The gradient alone for a [rows, cols] block of a larger matrix (row strides in elements; n_total = the element count
 * of the whole matrix the loss is taken over): the same values ntb200_mse writes there.  A rank that owns a column
 * block of the output can start on its weight gradient before the other ranks' blocks have arrived. */
int ntb200_mse_grad_block(int dtype, const void* out, int64_t out_row_stride, const void* target, int64_t target_row_stride,
                          void* grad, int64_t grad_row_stride, int64_t rows, int64_t cols, int64_t n_total, void* stream);
/* Bias gradient: column sums of grad[rows, cols] -> out[cols], the broadcast-reduce that
 * Tensor::operator+= / sum_as performs for dBias (nt/functional/tensor_files/operators.cpp:178-186). */
int ntb200_column_sum(int dtype, const void* grad, void* out, int64_t rows, int64_t cols, void* stream);
/* y += x elementwise: GraphNode::accumulate_gradient (nt/nn/AutoGrad.cpp:7-25). */
int ntb200_add_inplace(int dtype, void* y, const void* x, int64_t n, void* stream);
/* Parameter updates of the reference's optimizers, one launch per parameter tensor; F32, F16, BF16.
 * Every intermediate is rounded to the tensor's dtype, as the reference's whole-tensor operations do.
 *   optimizers::SGD::step (nt/nn/Optimizers.cpp:8-17):  param -= clip(grad, -10, 10) * learning_rate
 *   optimizers::Adam::step (nt/nn/Optimizers.cpp:68-98), exactly as written there:
 *     m = (m*beta1 + (1-beta1)) * grad;  v = (v*beta2 + (1-beta2)) * grad^2;
 *     param -= clip(learning_rate * (m / (1-beta1)^t) / (sqrt(v / (1-beta2)^t) + epsilon), -10, 10)
 *   `t` is the optimizer's step counter (the reference never advances it from 0).  grad is not modified. */
int ntb200_sgd_step(int dtype, void* param, const void* grad, int64_t n, double learning_rate, void* stream);
int ntb200_adam_step(int dtype, void* param, const void* grad, void* m, void* v, int64_t n, double learning_rate,
                     double beta1, double beta2, double epsilon, int64_t t, void* stream);
/* layers::Conv2D adds its bias [C, 1, 1] to the convolution's output as a separate elementwise operation
 * (nt/nn/layers/Conv2D.cpp:34-44): x[b][c][i] += bias[c] in place, and the bias gradient is the sum of the output
 * gradient over the batch and the pixels, out[c] = sum_b sum_i grad[b][c][i].  F32, F16, BF16. */
int ntb200_bias_add_channels(int dtype, void* x, const void* bias, int64_t batch, int64_t channels, int64_t inner,
                             void* stream);
int ntb200_sum_channels(int dtype, const void* grad, void* out, int64_t batch, int64_t channels, int64_t inner,
                        void* stream);
/* dst[rows, cols] (contiguous) = src viewed with the given element strides: Tensor::contiguous(). */
int ntb200_copy_strided_2d(int dtype, void* dst, const void* src, int64_t batch, int64_t rows, int64_t cols,
                           int64_t src_batch_stride, int64_t src_row_stride, int64_t src_col_stride, void* stream);
/* dst = convert(src) between F32, F16, BF16: Tensor::to(DType). */
int ntb200_convert(int dst_dtype, void* dst, int src_dtype, const void* src, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NTB200_H_ */
