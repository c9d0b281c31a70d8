// Multi-GPU partitioner behind the C ABI: one rank per GPU (one process each, or one host thread each inside a
// single process), no dependency on any communication library.  The reference is a single-device CPU library
// (nt/memory/DeviceEnum.h:6-10), so nothing here replaces reference code; the contract is the partitioning the
// matmult path admits:
//   * batched matmult: the batch is cut into contiguous ranges (ntb200_dist_shard), no exchange at all;
//   * one large GEMM: B and C are cut by columns; where the next operation needs whole rows of C, the GEMM's own
//     epilogue stores its column block into every rank's copy of C (TMA stores over NVLink into peer-mapped
//     buffers), and a flag exchange orders the ranks before anybody reads the gathered rows.
//
// Symmetric buffers.  ntb200_dist_buffer_create allocates the same number of bytes on every rank and maps every
// rank's block into every other rank (CUDA IPC between processes, plain peer access between threads of one process).
// The 88-byte descriptors travel through the caller's all-gather callback: torch.distributed, MPI, a socket, or a
// shared array when the ranks are threads.
//
// Ordering.  ntb200_dist_barrier launches a one-block kernel on the caller's stream: thread r publishes this rank's
// barrier count into rank r's flag array (a system-scope release store, after the kernels queued before it on the
// stream, whose peer stores are therefore visible first) and then polls, for at most two seconds, its own flag array
// for rank r's count (system-scope acquire loads).  A poll that runs out raises the device status word that
// ntb200_check_device_status reports as NTB200_ERR_TIMEOUT and the kernel returns; nothing waits without a bound.
// Only stores and 4-byte flag loads of this GPU's own memory are involved: no load of any kind reads peer memory.
#include <cuda_fp16.h>
#include <unistd.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "internal.h"

struct ntb200_dist_buffer;

struct ntb200_dist_comm {
    int rank = 0, world = 1, device = 0;
    ntb200_allgather_fn exchange = nullptr;
    void* ctx = nullptr;
    ntb200_dist_buffer* flags = nullptr;   // [kMaxRanks] unsigned counters per rank, in a symmetric buffer
    unsigned int epoch = 0;
    unsigned long long barrier_limit_ns = 2000000000ull;
    std::mutex mu;
};

struct ntb200_dist_buffer {
    ntb200_dist_comm* comm = nullptr;
    size_t bytes = 0;
    void* base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // by rank; [rank] is local
    bool ipc[8] = {false, false, false, false, false, false, false, false};                     // opened through CUDA IPC
};

namespace ntb200 {
namespace {

constexpr int kMaxRanks = 8;

struct BufferBlob {          // what one rank tells the others about its block
    int64_t pid;
    int32_t device;
    int32_t reserved;
    uint64_t address;
    unsigned char ipc[64];
};
static_assert(sizeof(BufferBlob) == 88, "exchange record size");

struct FlagTable {
    unsigned int* slot[kMaxRanks];   // slot[r]: this rank's entry in rank r's flag array (slot[rank]: own array base)
};

__global__ void dist_barrier_kernel(FlagTable table, unsigned int* own, int rank, int world, unsigned int epoch,
                                    unsigned long long limit_ns, unsigned int* status) {
    const int r = threadIdx.x;
    if (r >= world || r == rank) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(table.slot[r]), "r"(epoch) : "memory");
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(own + r) : "memory");
        if (int(seen - epoch) >= 0) break;          // the peer has reached this barrier (or is already one ahead)
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > limit_ns) {                  // give up: report, do not hang
            atomicExch(status, 0x200u | unsigned(r));
            break;
        }
        __nanosleep(200);
    }
}

// dst blocks (this rank's buffer and every peer's) receive src[m][n_bytes] at the same place: 16-byte pieces.
struct PushTargets {
    char* base[kMaxRanks];
    int count;
};
__global__ void push_block_kernel(const char* __restrict__ src, long long src_row_bytes, PushTargets t, long long dst_row_bytes,
                                  long long rows, long long pieces_per_row) {
    const long long total = rows * pieces_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / pieces_per_row, piece = i - row * pieces_per_row;
        const uint4 v = *reinterpret_cast<const uint4*>(src + row * src_row_bytes + piece * 16);
        for (int d = 0; d < t.count; ++d) *reinterpret_cast<uint4*>(t.base[d] + row * dst_row_bytes + piece * 16) = v;
    }
}
// 16-bit floats: max(x, 0) of a contiguous-row block into every target (the activation of a layer whose
// pre-activation block stays with its owner).  Negative zero and NaN pass as clamp(x, 0, none) passes them.
template <bool kBf16>
__global__ void push_relu16_kernel(const unsigned short* __restrict__ src, long long src_row_elems, PushTargets t,
                                   long long dst_row_bytes, long long rows, long long cols) {
    const long long total = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / cols, col = i - row * cols;
        unsigned short v = src[row * src_row_elems + col];
        const float f = kBf16 ? __uint_as_float(unsigned(v) << 16) : __half2float(__ushort_as_half(v));
        if (f < 0.f) v = 0;
        for (int d = 0; d < t.count; ++d) *reinterpret_cast<unsigned short*>(t.base[d] + row * dst_row_bytes + col * 2) = v;
    }
}
__global__ void push_block_bytes_kernel(const char* __restrict__ src, long long src_row_bytes, PushTargets t, long long dst_row_bytes,
                                        long long rows, long long row_bytes) {
    const long long total = rows * row_bytes;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / row_bytes, b = i - row * row_bytes;
        const char v = src[row * src_row_bytes + b];
        for (int d = 0; d < t.count; ++d) t.base[d][row * dst_row_bytes + b] = v;
    }
}

int check_comm(const ntb200_dist_comm* c, const char* who) {
    if (!c) return fail(NTB200_ERR_INVALID_ARG, "%s: null communicator", who);
    int dev = -1;
    NTB200_CUDA(cudaGetDevice(&dev));
    if (dev != c->device)
        return fail(NTB200_ERR_INVALID_ARG, "%s: the communicator belongs to device %d but device %d is current", who, c->device, dev);
    return NTB200_OK;
}

}  // namespace
}  // namespace ntb200

using namespace ntb200;

extern "C" {

int ntb200_dist_shard(int64_t total, int world, int rank, int64_t align, int64_t* start, int64_t* count) {
    if (!start || !count) return fail(NTB200_ERR_INVALID_ARG, "dist_shard: null pointer");
    if (world < 1 || rank < 0 || rank >= world) return fail(NTB200_ERR_INVALID_ARG, "dist_shard: bad rank %d for world size %d", rank, world);
    if (total < 0 || align < 1) return fail(NTB200_ERR_INVALID_ARG, "dist_shard: negative total or alignment below 1");
    // blocks of `align` units are dealt out contiguously; the first (blocks % world) ranks get one more
    const int64_t blocks = (total + align - 1) / align;
    const int64_t base = blocks / world, extra = blocks % world;
    const int64_t first = rank * base + (rank < extra ? rank : extra);
    const int64_t mine = base + (rank < extra ? 1 : 0);
    const int64_t s = first * align;
    int64_t e = (first + mine) * align;
    if (e > total) e = total;
    *start = s < total ? s : total;
    *count = e > *start ? e - *start : 0;
    return NTB200_OK;
}

int ntb200_dist_buffer_create(ntb200_dist_comm* comm, size_t bytes, ntb200_dist_buffer** out) {
    if (!out) return fail(NTB200_ERR_INVALID_ARG, "dist_buffer_create: null pointer");
    *out = nullptr;
    if (int rc = check_comm(comm, "dist_buffer_create")) return rc;
    if (bytes == 0) return fail(NTB200_ERR_INVALID_ARG, "dist_buffer_create: zero bytes");
    ntb200_dist_buffer* b = new ntb200_dist_buffer();
    b->comm = comm;
    b->bytes = bytes;
    // Every rank makes the same two exchanges whatever happens to it: a rank that cannot allocate or cannot map a peer
    // says so in the second one, and then all ranks fail together instead of one leaving the others in a collective.
    void* local = nullptr;
    cudaError_t e = cudaMalloc(&local, bytes);
    if (e == cudaSuccess) e = cudaMemset(local, 0, bytes);
    int rc = NTB200_OK;
    if (e != cudaSuccess) {
        if (local) cudaFree(local);
        local = nullptr;
        rc = cuda_fail(e, "dist_buffer_create: cudaMalloc");
        if (comm->world == 1) { delete b; return rc; }
    }
    b->base[comm->rank] = local;
    if (comm->world == 1) { *out = b; return NTB200_OK; }
    BufferBlob mine{};
    mine.pid = int64_t(getpid());
    mine.device = comm->device;
    mine.address = reinterpret_cast<uint64_t>(local);
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "IPC handle size");
    if (local) {
        e = cudaIpcGetMemHandle(&h, local);
        if (e == cudaSuccess) std::memcpy(mine.ipc, &h, 64);
        else (void)cudaGetLastError();                   // ranks inside one process do not need the handle
    }
    std::vector<BufferBlob> all(size_t(comm->world));
    const int xrc = comm->exchange(comm->ctx, &mine, all.data(), sizeof(BufferBlob));
    if (xrc != 0) {                                      // the transport itself failed: nothing more can be agreed on
        if (local) cudaFree(local);
        delete b;
        return fail(NTB200_ERR_INVALID_ARG, "dist_buffer_create: the all-gather callback failed with %d", xrc);
    }
    for (int r = 0; r < comm->world && rc == NTB200_OK; ++r) {
        if (r == comm->rank) continue;
        const BufferBlob& o = all[size_t(r)];
        if (o.address == 0) break;                       // that rank has no block; it reports the failure below
        if (o.pid == mine.pid) {                         // a thread of this process: plain peer access
            if (o.device != comm->device) {
                e = cudaDeviceEnablePeerAccess(o.device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); e = cudaSuccess; }
                if (e != cudaSuccess) { rc = cuda_fail(e, "dist_buffer_create: cudaDeviceEnablePeerAccess"); break; }
            }
            b->base[r] = reinterpret_cast<void*>(o.address);
        } else {
            cudaIpcMemHandle_t oh;
            std::memcpy(&oh, o.ipc, 64);
            void* p = nullptr;
            e = cudaIpcOpenMemHandle(&p, oh, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { rc = cuda_fail(e, "dist_buffer_create: cudaIpcOpenMemHandle"); break; }
            b->base[r] = p;
            b->ipc[r] = true;
        }
    }
    int32_t status = rc, statuses[kMaxRanks] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int yrc = comm->exchange(comm->ctx, &status, statuses, sizeof(int32_t));
    int failed_rank = -1;
    for (int r = 0; r < comm->world && failed_rank < 0; ++r)
        if (statuses[r] != NTB200_OK) failed_rank = r;
    if (rc != NTB200_OK || yrc != 0 || failed_rank >= 0) {
        for (int r = 0; r < comm->world; ++r)
            if (b->ipc[r] && b->base[r]) cudaIpcCloseMemHandle(b->base[r]);
        if (local) cudaFree(local);
        delete b;
        if (rc != NTB200_OK) return rc;                  // this rank's own error text stands
        if (yrc != 0) return fail(NTB200_ERR_INVALID_ARG, "dist_buffer_create: the all-gather callback failed with %d", yrc);
        return fail(statuses[failed_rank], "dist_buffer_create: rank %d could not allocate or map its peers", failed_rank);
    }
    *out = b;
    return NTB200_OK;
}

int ntb200_dist_buffer_destroy(ntb200_dist_buffer* b) {
    if (!b) return NTB200_OK;
    const int world = b->comm ? b->comm->world : 1, rank = b->comm ? b->comm->rank : 0;
    for (int r = 0; r < world; ++r)
        if (r != rank && b->ipc[r] && b->base[r]) (void)cudaIpcCloseMemHandle(b->base[r]);
    if (b->base[rank]) (void)cudaFree(b->base[rank]);
    (void)cudaGetLastError();
    delete b;
    return NTB200_OK;
}

void* ntb200_dist_buffer_ptr(const ntb200_dist_buffer* b) { return (b && b->comm) ? b->base[b->comm->rank] : nullptr; }

int ntb200_dist_init(ntb200_dist_comm** out, int rank, int world, ntb200_allgather_fn exchange, void* ctx) {
    if (!out) return fail(NTB200_ERR_INVALID_ARG, "dist_init: null pointer");
    *out = nullptr;
    if (world < 1 || world > kMaxRanks) return fail(NTB200_ERR_INVALID_ARG, "dist_init: world size %d (1..%d ranks of one NVLink domain)", world, kMaxRanks);
    if (rank < 0 || rank >= world) return fail(NTB200_ERR_INVALID_ARG, "dist_init: bad rank %d for world size %d", rank, world);
    if (world > 1 && !exchange) return fail(NTB200_ERR_INVALID_ARG, "dist_init: more than one rank needs an all-gather callback");
    ntb200_dist_comm* c = new ntb200_dist_comm();
    c->rank = rank; c->world = world; c->exchange = exchange; c->ctx = ctx;
    cudaError_t e = cudaGetDevice(&c->device);
    if (e != cudaSuccess) { delete c; return cuda_fail(e, "dist_init: cudaGetDevice"); }
    if (world > 1) {
        if (int rc = ntb200_dist_buffer_create(c, kMaxRanks * sizeof(unsigned int), &c->flags)) { delete c; return rc; }
    }
    *out = c;
    return NTB200_OK;
}

int ntb200_dist_destroy(ntb200_dist_comm* c) {
    if (!c) return NTB200_OK;
    if (c->flags) ntb200_dist_buffer_destroy(c->flags);
    delete c;
    return NTB200_OK;
}

int ntb200_dist_rank(const ntb200_dist_comm* c) { return c ? c->rank : -1; }
int ntb200_dist_world(const ntb200_dist_comm* c) { return c ? c->world : 0; }

int ntb200_dist_set_barrier_limit_ms(ntb200_dist_comm* c, unsigned int limit_ms) {
    if (!c) return fail(NTB200_ERR_INVALID_ARG, "dist_set_barrier_limit_ms: null communicator");
    if (limit_ms == 0 || limit_ms > 60000) return fail(NTB200_ERR_INVALID_ARG, "dist_set_barrier_limit_ms: 1..60000 ms");
    std::lock_guard<std::mutex> lk(c->mu);
    c->barrier_limit_ns = 1000000ull * limit_ms;
    return NTB200_OK;
}

int ntb200_dist_barrier(ntb200_dist_comm* c, void* stream) {
    if (int rc = check_comm(c, "dist_barrier")) return rc;
    if (c->world == 1) return NTB200_OK;
    unsigned int* status = device_status_word();
    if (!status) return fail(NTB200_ERR_CUDA, "dist_barrier: the device status word is not available");
    unsigned int epoch;
    unsigned long long limit_ns;
    {
        std::lock_guard<std::mutex> lk(c->mu);
        epoch = ++c->epoch;
        limit_ns = c->barrier_limit_ns;
    }
    FlagTable t{};
    for (int r = 0; r < c->world; ++r) t.slot[r] = static_cast<unsigned int*>(c->flags->base[r]) + c->rank;
    dist_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, static_cast<unsigned int*>(c->flags->base[c->rank]), c->rank,
                                                                       c->world, epoch, limit_ns, status);
    count_launch();
    NTB200_CUDA(cudaGetLastError());
    return NTB200_OK;
}

int ntb200_dist_gemm_allgather(ntb200_dist_comm* c, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                               int64_t gathered_row_stride, int64_t col0, int relu, void* stream) {
    if (gathered && gathered->comm != c)
        return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: the buffer belongs to another communicator");
    return ntb200_dist_gemm_allgather_at(c, desc, gathered, gathered_row_stride, 0, col0, relu, stream);
}

int ntb200_dist_gemm_allgather_at(ntb200_dist_comm* c, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                                  int64_t gathered_row_stride, int64_t row0, int64_t col0, int relu, void* stream) {
    if (int rc = ntb200_dist_gemm_push_at(c, desc, gathered, gathered_row_stride, row0, col0, relu, stream)) return rc;
    return ntb200_dist_barrier(c, stream);
}

int ntb200_dist_gemm_push_at(ntb200_dist_comm* c, const ntb200_gemm_desc* desc, ntb200_dist_buffer* gathered,
                             int64_t gathered_row_stride, int64_t row0, int64_t col0, int relu, void* stream) {
    if (int rc = check_comm(c, "dist_gemm_allgather")) return rc;
    if (!desc || !gathered) return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: null pointer");
    // the buffer may come from another communicator of the same ranks (row blocks of one matrix gathered on two
    // streams need two sets of flags, i.e. two communicators, and one buffer)
    if (!gathered->comm || gathered->comm->world != c->world || gathered->comm->rank != c->rank)
        return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: the buffer belongs to a communicator of other ranks");
    if (row0 < 0) return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: negative row offset");
    const size_t es = dtype_size(desc->dtype);
    if (desc->dtype != NTB200_F16 && desc->dtype != NTB200_BF16)
        return fail(NTB200_ERR_UNSUPPORTED, "dist_gemm_allgather: Float16 / BFloat16 (got %s)", dtype_name(desc->dtype));
    if (desc->batch != 1) return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather takes one 2-D problem");
    if (col0 < 0 || gathered_row_stride < col0 + desc->n)
        return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: columns [%lld, %lld) do not fit rows of %lld", (long long)col0,
                    (long long)(col0 + desc->n), (long long)gathered_row_stride);
    if (size_t(row0 + desc->m) * size_t(gathered_row_stride) * es > gathered->bytes)
        return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: rows [%lld, %lld) of %lld elements do not fit the %zu-byte buffer",
                    (long long)row0, (long long)(row0 + desc->m), (long long)gathered_row_stride, gathered->bytes);
    const size_t block_offset = (size_t(row0) * size_t(gathered_row_stride) + size_t(col0)) * es;
    void* peers[kMaxRanks];
    int n_peers = 0;
    for (int r = 0; r < c->world; ++r)
        if (r != c->rank) peers[n_peers++] = static_cast<char*>(gathered->base[r]) + block_offset;
    void* local_block = static_cast<char*>(gathered->base[c->rank]) + block_offset;
    int rc;
    if (relu) {
        // desc->c keeps the pre-activation block; the activation goes into every rank's gathered buffer
        if (!desc->c) return fail(NTB200_ERR_INVALID_ARG, "dist_gemm_allgather: relu needs desc->c for the pre-activation block");
        rc = ntb200_gemm_push_relu(desc, local_block, gathered_row_stride, peers, n_peers, stream);
    } else {
        ntb200_gemm_desc d = *desc;
        d.c = local_block;
        d.c_row_stride = gathered_row_stride;
        d.c_batch_stride = 0;
        d.route = NTB200_ROUTE_TENSOR;
        rc = ntb200_gemm_push(&d, peers, n_peers, stream);
    }
    if (rc == NTB200_ERR_UNSUPPORTED) {
        // Too small (or too oddly laid out) for the epilogue that stores to peers: multiply locally on whatever
        // route takes the operands, then push the block with a copy kernel.
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        PushTargets t{};
        const long long dst_rb = gathered_row_stride * (long long)es;
        const int blocks = sm_count() * 4;
        if (relu) {
            ntb200_gemm_desc d = *desc;
            d.route = NTB200_ROUTE_AUTO;
            if ((rc = ntb200_gemm(&d, stream))) return rc;
            for (int r = 0; r < c->world; ++r) t.base[t.count++] = static_cast<char*>(gathered->base[r]) + block_offset;
            if (desc->dtype == NTB200_BF16)
                push_relu16_kernel<true><<<blocks, 256, 0, s>>>(static_cast<const unsigned short*>(desc->c), desc->c_row_stride, t, dst_rb, desc->m, desc->n);
            else
                push_relu16_kernel<false><<<blocks, 256, 0, s>>>(static_cast<const unsigned short*>(desc->c), desc->c_row_stride, t, dst_rb, desc->m, desc->n);
        } else {
            ntb200_gemm_desc d = *desc;
            d.c = local_block;
            d.c_row_stride = gathered_row_stride;
            d.c_batch_stride = 0;
            d.route = NTB200_ROUTE_AUTO;
            if ((rc = ntb200_gemm(&d, stream))) return rc;
            for (int r = 0; r < c->world; ++r)
                if (r != c->rank) t.base[t.count++] = static_cast<char*>(gathered->base[r]) + block_offset;
            if (t.count > 0)
                push_block_bytes_kernel<<<blocks, 256, 0, s>>>(static_cast<const char*>(local_block), dst_rb, t, dst_rb, desc->m, desc->n * (long long)es);
        }
        count_launch();
        NTB200_CUDA(cudaGetLastError());
        rc = NTB200_OK;
    }
    return rc;
}

int ntb200_dist_allgather_columns(ntb200_dist_comm* c, int dtype, const void* block, int64_t rows, int64_t cols,
                                  int64_t block_row_stride, ntb200_dist_buffer* gathered, int64_t gathered_row_stride,
                                  int64_t col0, void* stream) {
    if (int rc = check_comm(c, "dist_allgather_columns")) return rc;
    const size_t es = dtype_size(dtype);
    if (!es) return fail(NTB200_ERR_UNSUPPORTED, "dist_allgather_columns: unknown dtype %d", dtype);
    if (!gathered || gathered->comm != c) return fail(NTB200_ERR_INVALID_ARG, "dist_allgather_columns: bad buffer");
    if (rows < 0 || cols < 0 || col0 < 0 || block_row_stride < cols || gathered_row_stride < col0 + cols)
        return fail(NTB200_ERR_INVALID_ARG, "dist_allgather_columns: bad extents");
    if (size_t(rows) * size_t(gathered_row_stride) * es > gathered->bytes)
        return fail(NTB200_ERR_INVALID_ARG, "dist_allgather_columns: the rows do not fit the buffer");
    if (rows > 0 && cols > 0) {
        if (!block) return fail(NTB200_ERR_INVALID_ARG, "dist_allgather_columns: null block");
        PushTargets t{};
        for (int r = 0; r < c->world; ++r) t.base[t.count++] = static_cast<char*>(gathered->base[r]) + size_t(col0) * es;
        const long long row_bytes = cols * (long long)es, src_rb = block_row_stride * (long long)es, dst_rb = gathered_row_stride * (long long)es;
        const bool vec = row_bytes % 16 == 0 && src_rb % 16 == 0 && dst_rb % 16 == 0 && (size_t(col0) * es) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(block) % 16 == 0;
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const int blocks = sm_count() * 4;
        if (vec) push_block_kernel<<<blocks, 256, 0, s>>>(static_cast<const char*>(block), src_rb, t, dst_rb, rows, row_bytes / 16);
        else push_block_bytes_kernel<<<blocks, 256, 0, s>>>(static_cast<const char*>(block), src_rb, t, dst_rb, rows, row_bytes);
        count_launch();
        NTB200_CUDA(cudaGetLastError());
    }
    return ntb200_dist_barrier(c, stream);
}

}  // extern "C"
