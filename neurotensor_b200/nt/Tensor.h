// nt::Tensor -- the slice of NeuroTensor's tensor type that the matmult / Linear / conv2d path touches, with
// device-resident storage.  Mirrors nt/Tensor.h:66-448 and nt/refs/SizeRef of the reference for: construction from
// (shape, dtype), shape/dims/numel/dtype/device, data_ptr, is_contiguous/is_null/is_mutable, view, transpose,
// contiguous, clone, to(DType), to(DeviceType), operator+=.  Differences by design:
//   * storage lives on DeviceType::CUDA in the library's stream-ordered pool (ntb200_malloc_async) -- the reference
//     has DeviceType::CPU only (nt/memory/DeviceEnum.h:6-10);
//   * a view is (offset, strides) over shared storage instead of a table of per-element pointers
//     (nt/functional/tensor_files/transpose.cpp:843-894), so transpose(-1,-2) is O(1) and matmult reads it in place;
//   * errors are std::invalid_argument thrown before any device work, like nt::utils::throw_exception.
// Header-only C++17; links against libntb200.so only.
#pragma once
#include <ntb200.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <initializer_list>
#include <memory>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace nt {

enum class DType { Float32, Float16, BFloat16, int8, int16, int32, int64, Float64, uint8, uint16, uint32, Bool };
enum class DeviceType { CPU, CUDA };

namespace utils {
template <class... Args>
[[noreturn]] inline void throw_error(Args&&... args) {
    std::ostringstream os;
    (os << ... << args);
    throw std::invalid_argument(os.str());
}
template <class... Args>
inline void throw_exception(bool ok, Args&&... args) {
    if (!ok) throw_error(std::forward<Args>(args)...);
}
inline void check(int rc) {
    if (rc != NTB200_OK) throw std::invalid_argument(ntb200_last_error_string());
}
}  // namespace utils

inline int dtype_code(DType dt) {
    switch (dt) {
        case DType::Float32: return NTB200_F32;
        case DType::Float16: return NTB200_F16;
        case DType::BFloat16: return NTB200_BF16;
        case DType::int8: return NTB200_I8;
        case DType::int16: return NTB200_I16;
        case DType::int32: return NTB200_I32;
        case DType::int64: return NTB200_I64;
        case DType::Float64: return NTB200_F64;
        case DType::uint8: return NTB200_U8;
        case DType::uint16: return NTB200_U16;
        case DType::uint32: return NTB200_U32;
        case DType::Bool: break;
    }
    utils::throw_error("Expected a number type but got Bool");
}
inline size_t dtype_size(DType dt) {
    switch (dt) {
        case DType::Float32: case DType::int32: case DType::uint32: return 4;
        case DType::Float16: case DType::BFloat16: case DType::int16: case DType::uint16: return 2;
        case DType::int8: case DType::uint8: case DType::Bool: return 1;
        case DType::int64: case DType::Float64: return 8;
    }
    return 0;
}
inline const char* dtype_name(DType dt) {
    static const char* n[] = {"Float32", "Float16", "BFloat16", "int8", "int16", "int32",
                              "int64",   "Float64", "uint8",    "uint16", "uint32", "Bool"};
    return n[int(dt)];
}

// Shape with Python-style negative indexing (nt/refs/SizeRef.h).
class SizeRef {
    std::vector<int64_t> d_;

   public:
    SizeRef() = default;
    SizeRef(std::initializer_list<int64_t> l) : d_(l) {}
    explicit SizeRef(std::vector<int64_t> v) : d_(std::move(v)) {}
    int64_t size() const { return int64_t(d_.size()); }
    int64_t operator[](int64_t i) const {
        if (i < 0) i += size();
        utils::throw_exception(i >= 0 && i < size(), "SizeRef index ", i, " out of range for ", size(), " dims");
        return d_[size_t(i)];
    }
    int64_t multiply(int64_t from = 0) const {
        int64_t n = 1;
        for (int64_t i = from; i < size(); ++i) n *= d_[size_t(i)];
        return n;
    }
    const std::vector<int64_t>& Vec() const { return d_; }
    bool operator==(const SizeRef& o) const { return d_ == o.d_; }
    bool operator!=(const SizeRef& o) const { return d_ != o.d_; }
    SizeRef transpose(int64_t a, int64_t b) const {
        std::vector<int64_t> v = d_;
        if (a < 0) a += size();
        if (b < 0) b += size();
        std::swap(v[size_t(a)], v[size_t(b)]);
        return SizeRef(v);
    }
    std::string str() const {
        std::ostringstream os;
        os << "{";
        for (size_t i = 0; i < d_.size(); ++i) os << (i ? "," : "") << d_[i];
        os << "}";
        return os.str();
    }
};
inline std::ostream& operator<<(std::ostream& os, const SizeRef& s) { return os << s.str(); }

namespace detail {
// Ref-counted block: the counterpart of the reference's DeviceHolder / Bucket pair (nt/memory/device.h:23-116).
struct Storage {
    void* ptr = nullptr;
    size_t bytes = 0;
    DeviceType device = DeviceType::CUDA;
    Storage(size_t n, DeviceType dev) : bytes(n), device(dev) {
        if (n == 0) return;
        if (dev == DeviceType::CUDA) {
            utils::check(ntb200_malloc_async(&ptr, n, nullptr));
        } else {
            // page-locked (and therefore at least 64-byte aligned like DeviceCPU, device.cpp:39-41): host tensors feed
            // ntb200_matmult_host, whose copies are asynchronous only from pinned memory
            utils::check(ntb200_host_alloc(&ptr, n));
        }
    }
    // Memory that somebody else owns (the reference's Bucket adopts an external pointer with a deleter the same way,
    // nt/memory/bucket.cpp:149-166); `release` runs when the last tensor viewing it goes away.
    std::function<void(void*)> release;
    Storage(void* external, size_t n, DeviceType dev, std::function<void(void*)> deleter)
        : ptr(external), bytes(n), device(dev), release(std::move(deleter)) {}
    ~Storage() {
        if (!ptr) return;
        if (release) { release(ptr); return; }
        if (device == DeviceType::CUDA) ntb200_free_async(ptr, nullptr);
        else ntb200_host_free(ptr);
    }
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
};
inline std::vector<int64_t> contiguous_strides(const SizeRef& s) {
    std::vector<int64_t> st(size_t(s.size()), 1);
    for (int64_t i = s.size() - 2; i >= 0; --i) st[size_t(i)] = st[size_t(i + 1)] * s[i + 1];
    return st;
}
}  // namespace detail

namespace cuda {
// The device path is asynchronous on the default stream; host reads synchronise through this.
inline void synchronize() { utils::check(ntb200_stream_synchronize(nullptr)); }
}  // namespace cuda

class Tensor {
    std::shared_ptr<detail::Storage> storage_;
    int64_t offset_ = 0;  // elements
    SizeRef shape_;
    std::vector<int64_t> strides_;  // elements
    DType dtype_ = DType::Float32;
    bool mutable_ = true;

   public:
    Tensor() = default;  // the null tensor
    static Tensor Null() { return Tensor(); }
    // Zero-initialised, like the reference's zeros-backed results (matmult_cpu.cpp:110).
    explicit Tensor(SizeRef shape, DType dt = DType::Float32, DeviceType dev = DeviceType::CUDA)
        : storage_(std::make_shared<detail::Storage>(size_t(shape.multiply()) * dtype_size(dt), dev)),
          shape_(std::move(shape)),
          strides_(detail::contiguous_strides(shape_)),
          dtype_(dt) {
        if (storage_->bytes) {
            if (dev == DeviceType::CUDA) utils::check(ntb200_memset_async(storage_->ptr, 0, storage_->bytes, nullptr));
            else std::memset(storage_->ptr, 0, storage_->bytes);
        }
    }
    // Contiguous tensor filled from host memory.
    static Tensor from_host(const void* src, SizeRef shape, DType dt, DeviceType dev = DeviceType::CUDA) {
        Tensor t(std::move(shape), dt, dev);
        const size_t n = size_t(t.numel()) * dtype_size(dt);
        if (n == 0) return t;
        if (dev == DeviceType::CUDA) {
            utils::check(ntb200_memcpy_h2d_async(t.data_ptr(), src, n, nullptr));
            cuda::synchronize();  // `src` may be a temporary
        } else {
            std::memcpy(t.data_ptr(), src, n);
        }
        return t;
    }

    // A contiguous tensor over memory owned elsewhere; `deleter` (may be empty) runs when the last view is gone.
    static Tensor adopt(void* ptr, SizeRef shape, DType dt, DeviceType dev = DeviceType::CUDA,
                        std::function<void(void*)> deleter = [](void*) {}) {
        Tensor t;
        t.storage_ = std::make_shared<detail::Storage>(ptr, size_t(shape.multiply()) * dtype_size(dt), dev, std::move(deleter));
        t.shape_ = std::move(shape);
        t.strides_ = detail::contiguous_strides(t.shape_);
        t.dtype_ = dt;
        return t;
    }
    // Columns [c0, c0 + n) of a 2-D tensor: a strided view sharing the storage.
    Tensor columns(int64_t c0, int64_t n) const {
        utils::throw_exception(dims() == 2 && c0 >= 0 && n >= 0 && c0 + n <= shape_[1], "columns: range outside the tensor");
        Tensor t = *this;
        t.shape_ = SizeRef({shape_[0], n});
        t.offset_ = offset_ + c0 * strides_[1];
        return t;
    }
    // Rows [r0, r0 + n) of a tensor (first dimension): a view sharing the storage.
    Tensor rows(int64_t r0, int64_t n) const {
        utils::throw_exception(dims() >= 1 && r0 >= 0 && n >= 0 && r0 + n <= shape_[0], "rows: range outside the tensor");
        Tensor t = *this;
        std::vector<int64_t> s = shape_.Vec();
        s[0] = n;
        t.shape_ = SizeRef(s);
        t.offset_ = offset_ + r0 * strides_[0];
        return t;
    }

    bool is_null() const { return !storage_; }
    const SizeRef& shape() const { return shape_; }
    int64_t dims() const { return shape_.size(); }
    int64_t numel() const { return is_null() ? 0 : shape_.multiply(); }
    DType dtype() const { return dtype_; }
    DeviceType device() const { return storage_ ? storage_->device : DeviceType::CPU; }
    bool is_mutable() const { return mutable_; }
    Tensor& set_mutability(bool m) { mutable_ = m; return *this; }
    const std::vector<int64_t>& strides() const { return strides_; }
    int64_t stride(int64_t i) const { return strides_[size_t(i < 0 ? i + dims() : i)]; }
    void* data_ptr() const {
        return storage_ ? static_cast<char*>(storage_->ptr) + offset_ * int64_t(dtype_size(dtype_)) : nullptr;
    }
    bool is_contiguous() const {
        if (is_null()) return true;
        int64_t expect = 1;
        for (int64_t i = dims() - 1; i >= 0; --i) {
            if (shape_[i] != 1 && strides_[size_t(i)] != expect) return false;
            expect *= shape_[i];
        }
        return true;
    }
    bool shares_storage_with(const Tensor& o) const { return storage_ && storage_ == o.storage_; }

    // view: same storage, new shape (one -1 allowed); the tensor must be contiguous.
    Tensor view(std::vector<int64_t> dims_) const {
        utils::throw_exception(!is_null(), "Cannot view a null tensor");
        utils::throw_exception(is_contiguous(), "view needs a contiguous tensor; call contiguous() first");
        int64_t known = 1, infer = -1;
        for (size_t i = 0; i < dims_.size(); ++i) {
            if (dims_[i] == -1) {
                utils::throw_exception(infer < 0, "only one dimension of a view can be -1");
                infer = int64_t(i);
            } else {
                known *= dims_[i];
            }
        }
        if (infer >= 0) {
            utils::throw_exception(known != 0 && numel() % known == 0, "view shape is not compatible with ", numel(), " elements");
            dims_[size_t(infer)] = numel() / known;
            known *= dims_[size_t(infer)];
        }
        utils::throw_exception(known == numel(), "view of ", numel(), " elements as a shape with ", known);
        Tensor t = *this;
        t.shape_ = SizeRef(std::move(dims_));
        t.strides_ = detail::contiguous_strides(t.shape_);
        return t;
    }
    Tensor view(std::initializer_list<int64_t> l) const { return view(std::vector<int64_t>(l)); }
    Tensor flatten_leading() const {  // [d0, ..., dn-1, c] -> [d0*...*dn-1, c]
        return view({-1, shape_[-1]});
    }
    // transpose: swaps two dims of the VIEW -- O(1), shares memory, generally non-contiguous afterwards.
    Tensor transpose(int64_t a, int64_t b) const {
        utils::throw_exception(!is_null(), "Cannot transpose a null tensor");
        if (a < 0) a += dims();
        if (b < 0) b += dims();
        utils::throw_exception(a >= 0 && a < dims() && b >= 0 && b < dims(), "transpose dims out of range");
        Tensor t = *this;
        t.shape_ = shape_.transpose(a, b);
        std::swap(t.strides_[size_t(a)], t.strides_[size_t(b)]);
        return t;
    }
    // Sub-tensor along the first dim (a batch item); shares storage.
    Tensor operator[](int64_t i) const {
        utils::throw_exception(dims() >= 1 && i >= 0 && i < shape_[0], "index out of range");
        Tensor t = *this;
        std::vector<int64_t> s(shape_.Vec().begin() + 1, shape_.Vec().end());
        t.shape_ = SizeRef(s);
        t.strides_.assign(strides_.begin() + 1, strides_.end());
        t.offset_ = offset_ + i * strides_[0];
        return t;
    }

    Tensor contiguous() const;
    Tensor clone() const;
    Tensor to(DType dt) const;
    Tensor to(DeviceType dev) const;
    Tensor& operator+=(const Tensor& other);

    // Copies the (contiguous form of the) tensor to host memory, synchronising first.
    void to_host(void* dst) const;
    template <class T>
    std::vector<T> to_vector() const {
        utils::throw_exception(sizeof(T) == dtype_size(dtype_), "to_vector: element size mismatch");
        std::vector<T> v(static_cast<size_t>(numel()), T());
        to_host(v.data());
        return v;
    }
};

inline Tensor Tensor::contiguous() const {
    if (is_null() || is_contiguous()) return *this;
    return clone();
}

inline Tensor Tensor::clone() const {
    if (is_null()) return Tensor();
    Tensor out(shape_, dtype_, device());
    if (numel() == 0) return out;
    const size_t es = dtype_size(dtype_);
    if (is_contiguous()) {
        if (device() == DeviceType::CUDA)
            utils::check(ntb200_memcpy_d2d_async(out.data_ptr(), data_ptr(), size_t(numel()) * es, nullptr));
        else
            std::memcpy(out.data_ptr(), data_ptr(), size_t(numel()) * es);
        return out;
    }
    // strided source: fold leading dims into one batch stride when possible, else copy item by item
    utils::throw_exception(dims() >= 2, "clone of a non-contiguous 1-D view is not supported");
    const int64_t rows = shape_[-2], cols = shape_[-1], rs = stride(-2), cs = stride(-1);
    const int64_t lead = dims() - 2;
    int64_t batch = 1;
    for (int64_t i = 0; i < lead; ++i) batch *= shape_[i];
    bool foldable = true;
    for (int64_t i = 0; i + 1 < lead; ++i) foldable = foldable && strides_[size_t(i)] == strides_[size_t(i + 1)] * shape_[i + 1];
    if (device() == DeviceType::CUDA && (foldable || lead == 0)) {
        const int64_t bs = lead ? strides_[size_t(lead - 1)] : 0;
        for (int64_t b0 = 0; b0 < batch; b0 += 65535) {
            const int64_t nb = std::min<int64_t>(65535, batch - b0);
            utils::check(ntb200_copy_strided_2d(dtype_code(dtype_), static_cast<char*>(out.data_ptr()) + b0 * rows * cols * int64_t(es),
                                                static_cast<const char*>(data_ptr()) + b0 * bs * int64_t(es), nb, rows, cols, bs, rs,
                                                cs, nullptr));
        }
        return out;
    }
    if (device() == DeviceType::CPU) {
        std::vector<int64_t> idx(size_t(dims()), 0);
        char* dst = static_cast<char*>(out.data_ptr());
        const char* src = static_cast<const char*>(data_ptr());
        for (int64_t n = 0, total = numel(); n < total; ++n) {
            int64_t off = 0;
            for (int64_t d = 0; d < dims(); ++d) off += idx[size_t(d)] * strides_[size_t(d)];
            std::memcpy(dst + n * int64_t(es), src + off * int64_t(es), es);
            for (int64_t d = dims() - 1; d >= 0; --d) {
                if (++idx[size_t(d)] < shape_[d]) break;
                idx[size_t(d)] = 0;
            }
        }
        return out;
    }
    // device, leading dims not foldable: recurse over the first dim
    for (int64_t i = 0; i < shape_[0]; ++i) {
        Tensor piece = (*this)[i].clone();
        utils::check(ntb200_memcpy_d2d_async(static_cast<char*>(out.data_ptr()) + i * piece.numel() * int64_t(es), piece.data_ptr(),
                                             size_t(piece.numel()) * es, nullptr));
    }
    return out;
}

inline Tensor Tensor::to(DeviceType dev) const {
    if (is_null() || dev == device()) return *this;
    Tensor src = contiguous();
    Tensor out(shape_, dtype_, dev);
    const size_t n = size_t(numel()) * dtype_size(dtype_);
    if (n) {
        if (dev == DeviceType::CUDA) utils::check(ntb200_memcpy_h2d_async(out.data_ptr(), src.data_ptr(), n, nullptr));
        else utils::check(ntb200_memcpy_d2h_async(out.data_ptr(), src.data_ptr(), n, nullptr));
        cuda::synchronize();
    }
    out.mutable_ = mutable_;
    return out;
}

inline Tensor Tensor::to(DType dt) const {
    if (is_null() || dt == dtype_) return *this;
    utils::throw_exception(device() == DeviceType::CUDA, "dtype conversion runs on the device; move the tensor with to(DeviceType::CUDA) first");
    Tensor src = contiguous();
    Tensor out(shape_, dt, DeviceType::CUDA);
    utils::check(ntb200_convert(dtype_code(dt), out.data_ptr(), dtype_code(dtype_), src.data_ptr(), numel(), nullptr));
    return out;
}

inline void Tensor::to_host(void* dst) const {
    if (numel() == 0) return;
    Tensor src = contiguous();
    const size_t n = size_t(numel()) * dtype_size(dtype_);
    if (device() == DeviceType::CUDA) {
        utils::check(ntb200_memcpy_d2h_async(dst, src.data_ptr(), n, nullptr));
        cuda::synchronize();
    } else {
        std::memcpy(dst, src.data_ptr(), n);
    }
}

// this += other.  When `other` has extra leading rows (shape [..., n] against this [n]) they are summed away first:
// the broadcast-reduce rule of Tensor::operator+= -> sum_as (nt/functional/tensor_files/operators.cpp:175-186).
inline Tensor& Tensor::operator+=(const Tensor& other) {
    utils::throw_exception(!is_null() && !other.is_null(), "operator+= on a null tensor");
    utils::throw_exception(is_mutable(), "Can only perform operator+= on a mutable tensor");
    utils::throw_exception(dtype_ == other.dtype_, "Expected dtypes to match in operator+= but got ", dtype_name(dtype_), " and ", dtype_name(other.dtype_));
    utils::throw_exception(device() == DeviceType::CUDA && other.device() == DeviceType::CUDA, "operator+= runs on the device");
    utils::throw_exception(is_contiguous(), "operator+= needs a contiguous destination");
    Tensor o = other.contiguous();
    if (o.numel() == numel()) {
        utils::check(ntb200_add_inplace(dtype_code(dtype_), data_ptr(), o.data_ptr(), numel(), nullptr));
        return *this;
    }
    utils::throw_exception(numel() > 0 && o.numel() % numel() == 0 && o.shape()[-1] == shape_[-1] && dims() == 1,
                           "Shapes ", shape_, " and ", o.shape(), " are not compatible for operator+=");
    Tensor reduced(shape_, dtype_, DeviceType::CUDA);
    utils::check(ntb200_column_sum(dtype_code(dtype_), o.data_ptr(), reduced.data_ptr(), o.numel() / numel(), numel(), nullptr));
    utils::check(ntb200_add_inplace(dtype_code(dtype_), data_ptr(), reduced.data_ptr(), numel(), nullptr));
    return *this;
}

}  // namespace nt
