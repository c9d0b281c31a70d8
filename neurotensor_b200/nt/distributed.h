// nt::distributed -- the multi-GPU partitioner of the matmult path for C++ callers, over ntb200_dist_* of the C ABI.
// New: the reference has one device, the CPU (nt/memory/DeviceEnum.h:6-10).  One rank per GPU; ranks are processes
// (give Communicator an all-gather callback over whatever the application already uses to talk between them) or host
// threads of one process (ThreadExchange below is that callback for threads).
//
//   batched matmult     every rank multiplies its own items (shard), nothing is exchanged;
//   one large GEMM      split over the output columns: linear_allgather computes this rank's column block and the
//                       GEMM's epilogue stores it into every rank's GatheredMatrix, where the next operation finds
//                       whole rows.  Alternate two GatheredMatrix objects from step to step.
#pragma once
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "Tensor.h"
#include "functional.h"

namespace nt {
namespace distributed {

// Contiguous share [start, start + count) of `total` units for `rank`, in blocks of `align` units.
inline std::pair<int64_t, int64_t> shard(int64_t total, int world, int rank, int64_t align = 1) {
    int64_t start = 0, count = 0;
    utils::check(ntb200_dist_shard(total, world, rank, align, &start, &count));
    return {start, count};
}

// All-gather between the threads of one process: every rank thread calls gather() with its record and leaves with
// everybody's.  One object shared by the ranks; pass `&exchange` as ctx and ThreadExchange::callback as the function.
class ThreadExchange {
    std::mutex mu_;
    std::condition_variable cv_;
    std::vector<char> slots_;
    int world_, arrived_ = 0, generation_ = 0;

   public:
    explicit ThreadExchange(int world) : world_(world) {}
    // rank r's record goes to slot r: ranks register in the order of their rank numbers' first call
    struct Rank { ThreadExchange* ex; int rank; };
    static int callback(void* ctx, const void* send, void* recv, size_t bytes) {
        Rank* r = static_cast<Rank*>(ctx);
        return r->ex->gather(r->rank, send, recv, bytes);
    }
    int gather(int rank, const void* send, void* recv, size_t bytes) {
        std::unique_lock<std::mutex> lk(mu_);
        if (slots_.size() != bytes * size_t(world_)) slots_.assign(bytes * size_t(world_), 0);
        std::memcpy(slots_.data() + size_t(rank) * bytes, send, bytes);
        const int gen = generation_;
        if (++arrived_ == world_) {
            arrived_ = 0;
            ++generation_;
            std::memcpy(recv, slots_.data(), slots_.size());
            done_copy_ = slots_;
            cv_.notify_all();
            return 0;
        }
        cv_.wait(lk, [&] { return generation_ != gen; });
        std::memcpy(recv, done_copy_.data(), done_copy_.size());
        return 0;
    }

   private:
    std::vector<char> done_copy_;
};

class Communicator {
    ntb200_dist_comm* c_ = nullptr;

   public:
    // Collective: every rank constructs its communicator at the same time, with its own device current.
    Communicator(int rank, int world, ntb200_allgather_fn exchange = nullptr, void* ctx = nullptr) {
        utils::check(ntb200_dist_init(&c_, rank, world, exchange, ctx));
    }
    ~Communicator() { ntb200_dist_destroy(c_); }
    Communicator(const Communicator&) = delete;
    Communicator& operator=(const Communicator&) = delete;
    int rank() const { return ntb200_dist_rank(c_); }
    int world() const { return ntb200_dist_world(c_); }
    ntb200_dist_comm* handle() const { return c_; }
    void barrier() { utils::check(ntb200_dist_barrier(c_, nullptr)); }
    std::pair<int64_t, int64_t> shard(int64_t total, int64_t align = 1) const { return distributed::shard(total, world(), rank(), align); }
};

// A [rows, cols] matrix that exists on every rank and into which every rank's GEMM epilogue can store its columns.
class GatheredMatrix {
    ntb200_dist_buffer* b_ = nullptr;
    int64_t rows_, cols_;
    DType dtype_;

   public:
    GatheredMatrix(Communicator& comm, int64_t rows, int64_t cols, DType dt) : rows_(rows), cols_(cols), dtype_(dt) {
        utils::check(ntb200_dist_buffer_create(comm.handle(), size_t(rows) * size_t(cols) * dtype_size(dt), &b_));
    }
    ~GatheredMatrix() { ntb200_dist_buffer_destroy(b_); }
    GatheredMatrix(const GatheredMatrix&) = delete;
    GatheredMatrix& operator=(const GatheredMatrix&) = delete;
    ntb200_dist_buffer* handle() const { return b_; }
    int64_t rows() const { return rows_; }
    int64_t cols() const { return cols_; }
    // This rank's copy as a tensor (a view: the buffer must outlive it).
    Tensor local() const { return Tensor::adopt(ntb200_dist_buffer_ptr(b_), SizeRef({rows_, cols_}), dtype_); }
};

// This rank's column block  bias + x . w_cols  lands in columns [col0, col0 + n) of `out` on every rank; on return
// (in stream order) `out.local()` holds every rank's block.  With `pre_activation` the block itself is kept there
// ([m, n], for the ReLU backward mask) and `out` receives max(block, 0): Linear + ReLU of a column-sharded layer.
// `row0`: the block goes to rows [row0, row0 + m) of the gathered matrix (row blocks of one matrix gathered one after
// the other; `out` may have been created through another communicator of the same ranks).
inline Tensor linear_allgather(Communicator& comm, const Tensor& x, const Tensor& w_cols, const Tensor& bias_cols, GatheredMatrix& out,
                               int64_t col0, Tensor* pre_activation = nullptr, int64_t row0 = 0) {
    utils::throw_exception(!x.is_null() && !w_cols.is_null(), "linear_allgather got a null tensor");
    utils::throw_exception(x.dims() == 2 && w_cols.dims() == 2, "linear_allgather takes 2-D operands");
    utils::throw_exception(x.dtype() == w_cols.dtype(), "Expected both tensors to have the same dtype for matmult");
    utils::throw_exception(x.shape()[1] == w_cols.shape()[0], "Expected second tensor rows to be ", x.shape()[1], " when it was ",
                           w_cols.shape()[0]);
    const int64_t m = x.shape()[0], k = x.shape()[1], n = w_cols.shape()[1];
    utils::throw_exception(row0 >= 0 && row0 + m <= out.rows() && col0 >= 0 && col0 + n <= out.cols(),
                           "linear_allgather: the block does not fit the gathered matrix");
    ntb200_gemm_desc d{};
    d.dtype = dtype_code(x.dtype());
    d.route = NTB200_ROUTE_TENSOR;
    d.m = m; d.n = n; d.k = k; d.batch = 1;
    d.a = x.data_ptr(); d.a_row_stride = x.stride(0); d.a_col_stride = x.stride(1);
    d.b = w_cols.data_ptr(); d.b_row_stride = w_cols.stride(0); d.b_col_stride = w_cols.stride(1);
    if (!bias_cols.is_null()) {
        utils::throw_exception(bias_cols.numel() == n && bias_cols.dtype() == x.dtype(), "linear_allgather: bias must hold the block's ", n, " columns");
        d.bias = bias_cols.data_ptr(); d.bias_col_stride = bias_cols.stride(-1);
    }
    if (pre_activation) {
        *pre_activation = Tensor(SizeRef({m, n}), x.dtype());
        d.c = pre_activation->data_ptr(); d.c_row_stride = n;
    }
    utils::check(ntb200_dist_gemm_allgather_at(comm.handle(), &d, out.handle(), out.cols(), row0, col0, pre_activation ? 1 : 0, nullptr));
    return out.local();
}

}  // namespace distributed
}  // namespace nt
