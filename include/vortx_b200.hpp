/*
 * vortx_b200.hpp — the host side of vortx's matmul path in C++17, header only, over the C ABI of
 * vortx_b200.h / vortx_b200_host.h.
 *
 * vortx's host code is Rust; this header mirrors the types a vortx program touches on this path —
 * same names, same argument meaning, same failure points — for hosts written in C++:
 *   TensorLayout                          src/shapes.rs:49-533
 *   GpuBackend, GpuBuffer<T>              khal's backend surface as vortx uses it (src/tensor/tensor_impl.rs:69,105,715)
 *   Tensor<T>, TensorRef<T>, TensorMut<T> src/tensor/tensor_impl.rs:117-121, tensor_ref.rs:11-151, tensor_mut.rs:10-163
 *   Gemm, Reduce, OpAssign, Repeat, Contiguous   src/linalg/{gemm,reduce,op_assign,repeat,contiguous}.rs
 *   QuantizedMatrix, Gemv, GemvBatch      no reference counterpart (block-quantised weights)
 * Where the reference panics (assert_eq! on shapes, out-of-range axes) these throw: ShapeMismatch for
 * Gemm::dispatch's shape asserts (src/linalg/gemm.rs:70-104), Error otherwise.  Where the reference returns
 * None (unsqueeze, broadcast) these return an empty std::optional.  Nothing here computes on the host: a
 * missing library or GPU is an exception, never a fallback.
 */
#ifndef VORTX_B200_HPP
#define VORTX_B200_HPP

#include <array>
#include <cstdint>
#include <initializer_list>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "vortx_b200_host.h"

namespace vortx {

struct Error : std::runtime_error {
    vx_status status;
    Error(vx_status s, const std::string& what) : std::runtime_error(what), status(s) {}
};
/* Gemm::dispatch's assert_eq! failures — src/linalg/gemm.rs:70-104. */
struct ShapeMismatch : Error {
    using Error::Error;
};

inline void check(vx_status s) {
    if (s == VX_OK) return;
    const std::string msg = vx_last_error();
    if (s == VX_ERR_SHAPE) throw ShapeMismatch(s, msg);
    throw Error(s, msg);
}

/* ------------------------------------------------------------------ TensorLayout ---- */
/* src/shapes.rs:49-60. */
struct TensorLayout {
    vx_layout l{};

    TensorLayout() = default;
    explicit TensorLayout(const vx_layout& raw) : l(raw) {}

    /* src/shapes.rs:85-99 */
    static TensorLayout contiguous(std::initializer_list<uint32_t> size) {
        return contiguous(std::vector<uint32_t>(size));
    }
    static TensorLayout contiguous(const std::vector<uint32_t>& size) {
        TensorLayout out;
        check(vx_layout_contiguous(size.data(), (uint32_t)size.size(), &out.l));
        return out;
    }
    uint32_t rank() const { return l.rank; }
    uint32_t offset() const { return l.offset; }
    uint32_t size(uint32_t i) const { return l.size[i]; }
    uint32_t stride(uint32_t i) const { return l.stride[i]; }
    /* src/shapes.rs:527-533 */
    uint64_t len() const { return vx_layout_len(&l); }
    /* src/shapes.rs:20-47 */
    vx_shape into_gpu() const {
        vx_shape s;
        check(vx_layout_to_shape(&l, &s));
        return s;
    }
    TensorLayout canonicalize() const { return apply([&](vx_layout* o) { return vx_layout_canonicalize(&l, o); }); }
    TensorLayout transpose(uint32_t a, uint32_t b) const {
        return apply([&](vx_layout* o) { return vx_layout_transpose(&l, a, b, o); });
    }
    TensorLayout transpose_last_dims() const {
        return apply([&](vx_layout* o) { return vx_layout_transpose_last_dims(&l, o); });
    }
    TensorLayout permute(const std::array<uint32_t, 4>& p) const {
        return apply([&](vx_layout* o) { return vx_layout_permute(&l, p.data(), o); });
    }
    TensorLayout permute_ggml(const std::array<uint32_t, 4>& p) const {
        return apply([&](vx_layout* o) { return vx_layout_permute_ggml(&l, p.data(), o); });
    }
    TensorLayout index(uint32_t i) const { return apply([&](vx_layout* o) { return vx_layout_index(&l, i, o); }); }
    TensorLayout squeeze() const { return apply([&](vx_layout* o) { return vx_layout_squeeze(&l, o); }); }
    TensorLayout squeeze_axis(uint32_t axis) const {
        return apply([&](vx_layout* o) { return vx_layout_squeeze_axis(&l, axis, o); });
    }
    /* src/shapes.rs:161-175 — None when the rank is already 4 or the axis is beyond the rank. */
    std::optional<TensorLayout> unsqueeze(uint32_t axis) const {
        TensorLayout out;
        const vx_status s = vx_layout_unsqueeze(&l, axis, &out.l);
        if (s == VX_ERR_UNSUPPORTED) return std::nullopt;
        check(s);
        return out;
    }
    TensorLayout reshape(const std::vector<uint32_t>& shape) const {
        return apply([&](vx_layout* o) { return vx_layout_reshape(&l, shape.data(), (uint32_t)shape.size(), o); });
    }
    /* src/shapes.rs:407-441 — strides that are not given are derived. */
    TensorLayout view(uint32_t offset, const std::vector<uint32_t>& shape,
                      const std::vector<std::optional<uint32_t>>& stride = {}) const {
        std::vector<uint32_t> values(stride.size(), 0);
        std::vector<uint8_t> set(stride.size(), 0);
        for (size_t i = 0; i < stride.size(); ++i)
            if (stride[i]) {
                values[i] = *stride[i];
                set[i] = 1;
            }
        return apply([&](vx_layout* o) {
            return vx_layout_view(&l, offset, shape.data(), (uint32_t)shape.size(), values.data(), set.data(),
                                  (uint32_t)stride.size(), o);
        });
    }
    TensorLayout narrow(uint32_t axis, uint32_t first, uint32_t count) const {
        return apply([&](vx_layout* o) { return vx_layout_narrow(&l, axis, first, count, o); });
    }
    TensorLayout matrix(uint32_t id) const { return apply([&](vx_layout* o) { return vx_layout_matrix(&l, id, o); }); }
    TensorLayout columns(uint32_t first, uint32_t count) const {
        return apply([&](vx_layout* o) { return vx_layout_columns(&l, first, count, o); });
    }
    TensorLayout column(uint32_t i) const { return columns(i, 1); }
    TensorLayout rows(uint32_t first, uint32_t count) const {
        return apply([&](vx_layout* o) { return vx_layout_rows(&l, first, count, o); });
    }
    TensorLayout row(uint32_t i) const { return rows(i, 1); }
    bool is_contiguous() const { return vx_layout_is_contiguous(&l) != 0; }
    /* src/shapes.rs:346-389 — None when the shapes cannot be broadcast. */
    static std::optional<std::pair<TensorLayout, TensorLayout>> broadcast(const TensorLayout& a, const TensorLayout& b) {
        TensorLayout oa, ob;
        const vx_status s = vx_layout_broadcast(&a.l, &b.l, &oa.l, &ob.l);
        if (s == VX_ERR_SHAPE) return std::nullopt;
        check(s);
        return std::make_pair(oa, ob);
    }

private:
    template <class F>
    TensorLayout apply(F&& f) const {
        TensorLayout out;
        check(f(&out.l));
        return out;
    }
};

/* ------------------------------------------------------------- backend and buffers ---- */
/* One CUDA context + stream: GpuBackend::Cuda(Cuda::new(i)) — src/linalg/gemm.rs:353. */
class GpuBackend {
public:
    explicit GpuBackend(int device = 0) { check(vx_context_create(device, &ctx_)); }
    GpuBackend(const GpuBackend&) = delete;
    GpuBackend& operator=(const GpuBackend&) = delete;
    ~GpuBackend() {
        if (ctx_) vx_context_destroy(ctx_);
    }
    vx_context* ctx() const { return ctx_; }
    /* backend.synchronize() — src/linalg/gemm.rs:421; also reports a device-side wait that ran out. */
    void synchronize() const { check(vx_synchronize(ctx_)); }
    uint64_t launch_count() const {
        uint64_t n = 0;
        check(vx_context_launch_count(ctx_, &n));
        return n;
    }
    void set_option(const char* key, int64_t value) const { check(vx_set_option(ctx_, key, value)); }

private:
    vx_context* ctx_ = nullptr;
};

/* khal's GpuBuffer<T> as vortx holds it: a device allocation of `len` elements; frees on drop. */
template <class T>
class GpuBuffer {
public:
    GpuBuffer() = default;
    /* backend.uninit_buffer(len, usage) — src/tensor/tensor_impl.rs:69 */
    GpuBuffer(const GpuBackend& backend, size_t len) : ctx_(backend.ctx()), len_(len) {
        void* p = nullptr;
        check(vx_alloc(ctx_, (len ? len : 1) * sizeof(T), &p));
        ptr_ = static_cast<T*>(p);
    }
    /* backend.init_buffer(data, usage) — src/tensor/tensor_impl.rs:105 */
    GpuBuffer(const GpuBackend& backend, const T* data, size_t len) : GpuBuffer(backend, len) {
        if (len) check(vx_upload(ctx_, ptr_, data, len * sizeof(T)));
    }
    GpuBuffer(GpuBuffer&& o) noexcept : ctx_(o.ctx_), ptr_(o.ptr_), len_(o.len_) { o.ptr_ = nullptr; }
    GpuBuffer& operator=(GpuBuffer&& o) noexcept {
        if (this != &o) {
            release();
            ctx_ = o.ctx_;
            ptr_ = o.ptr_;
            len_ = o.len_;
            o.ptr_ = nullptr;
        }
        return *this;
    }
    GpuBuffer(const GpuBuffer&) = delete;
    GpuBuffer& operator=(const GpuBuffer&) = delete;
    ~GpuBuffer() { release(); }

    T* ptr() const { return ptr_; }
    size_t len() const { return len_; }
    /* backend.write_buffer(buf, offset, data) — src/tensor/tensor_impl.rs:715 */
    void write(size_t offset, const T* data, size_t n) const {
        if (offset + n > len_) throw Error(VX_ERR_OUT_OF_BOUNDS, "write_buffer past the end of the buffer");
        if (n) check(vx_upload(ctx_, ptr_ + offset, data, n * sizeof(T)));
    }
    /* backend.slow_read_buffer(buf, host) — src/linalg/gemm.rs:423-426 (blocking) */
    std::vector<T> read() const {
        std::vector<T> host(len_);
        if (len_) check(vx_download(ctx_, host.data(), ptr_, len_ * sizeof(T)));
        return host;
    }

private:
    void release() {
        if (ptr_ && ctx_) vx_free(ctx_, ptr_);
        ptr_ = nullptr;
    }
    vx_context* ctx_ = nullptr;
    T* ptr_ = nullptr;
    size_t len_ = 0;
};

/* ------------------------------------------------------------------------ views ---- */
/* The layout modifiers of src/tensor/tensor_macro.rs:1-125, shared by TensorRef and TensorMut. */
template <class Derived, class T>
struct ViewOps {
    TensorLayout layout_;
    T* base_ = nullptr;   // base of the underlying buffer (no offset): raw_buffer(), tensor_ref.rs:106-108
    size_t cap_ = 0;      // its length in elements

    const TensorLayout& layout() const { return layout_; }
    uint32_t rank() const { return layout_.rank(); }
    uint32_t size(uint32_t i) const { return layout_.size(i); }
    uint32_t stride(uint32_t i) const { return layout_.stride(i); }
    uint64_t len() const { return layout_.len(); }
    bool is_contiguous() const { return layout_.is_contiguous(); }
    /* buffer(): slice(offset..) — src/tensor/tensor_ref.rs:101-103 */
    T* buffer() const { return base_ + layout_.offset(); }
    T* raw_buffer() const { return base_; }
    size_t raw_len() const { return cap_; }

    Derived transpose(uint32_t a, uint32_t b) const { return with(layout_.transpose(a, b)); }
    Derived transpose_last_dims() const { return with(layout_.transpose_last_dims()); }
    Derived permute(const std::array<uint32_t, 4>& p) const { return with(layout_.permute(p)); }
    Derived canonicalize() const { return with(layout_.canonicalize()); }
    Derived reshape(const std::vector<uint32_t>& s) const { return with(layout_.reshape(s)); }
    Derived view(uint32_t offset, const std::vector<uint32_t>& shape,
                 const std::vector<std::optional<uint32_t>>& stride = {}) const {
        return with(layout_.view(offset, shape, stride));
    }
    Derived narrow(uint32_t axis, uint32_t first, uint32_t n) const { return with(layout_.narrow(axis, first, n)); }
    Derived matrix(uint32_t id) const { return with(layout_.matrix(id)); }
    Derived columns(uint32_t first, uint32_t n) const { return with(layout_.columns(first, n)); }
    Derived column(uint32_t i) const { return with(layout_.column(i)); }
    Derived rows(uint32_t first, uint32_t n) const { return with(layout_.rows(first, n)); }
    Derived row(uint32_t i) const { return with(layout_.row(i)); }
    Derived index(uint32_t i) const { return with(layout_.index(i)); }
    Derived squeeze() const { return with(layout_.squeeze()); }

private:
    Derived with(const TensorLayout& l) const {
        Derived d;
        d.layout_ = l;
        d.base_ = base_;
        d.cap_ = cap_;
        return d;
    }
};
template <class T> struct TensorRef : ViewOps<TensorRef<T>, const T> {};
template <class T> struct TensorMut : ViewOps<TensorMut<T>, T> {
    TensorRef<T> as_ref() const {
        TensorRef<T> r;
        r.layout_ = this->layout_;
        r.base_ = this->base_;
        r.cap_ = this->cap_;
        return r;
    }
};

/* The owning tensor — src/tensor/tensor_impl.rs:117-121; matrices are row-major (:543-555). */
template <class T>
class Tensor {
public:
    static Tensor matrix(const GpuBackend& b, uint32_t nrows, uint32_t ncols, const std::vector<T>& data) {
        if (data.size() != (size_t)nrows * ncols) throw Error(VX_ERR_INVALID_ARGUMENT, "matrix data size mismatch");
        return Tensor({nrows, ncols}, GpuBuffer<T>(b, data.data(), data.size()));
    }
    static Tensor matrix_uninit(const GpuBackend& b, uint32_t nrows, uint32_t ncols) {
        return Tensor({nrows, ncols}, GpuBuffer<T>(b, (size_t)nrows * ncols));
    }
    static Tensor vector(const GpuBackend& b, const std::vector<T>& data) {
        return Tensor({(uint32_t)data.size()}, GpuBuffer<T>(b, data.data(), data.size()));
    }
    static Tensor vector_uninit(const GpuBackend& b, uint32_t len) { return Tensor({len}, GpuBuffer<T>(b, len)); }
    static Tensor scalar(const GpuBackend& b, T value) { return Tensor({}, GpuBuffer<T>(b, &value, 1)); }
    static Tensor tensor_uninit(const GpuBackend& b, const std::vector<uint32_t>& shape) {
        size_t n = 1;
        for (uint32_t s : shape) n *= s;
        return Tensor(shape, GpuBuffer<T>(b, n));
    }

    uint32_t rank() const { return (uint32_t)shape_.size(); }
    const std::vector<uint32_t>& shape() const { return shape_; }
    uint64_t len() const { return layout().len(); }
    TensorLayout layout() const { return TensorLayout::contiguous(shape_); }
    const GpuBuffer<T>& buffer() const { return buffer_; }
    TensorRef<T> as_view() const {
        TensorRef<T> r;
        r.layout_ = layout();
        r.base_ = buffer_.ptr();
        r.cap_ = buffer_.len();
        return r;
    }
    TensorMut<T> as_view_mut() {
        TensorMut<T> m;
        m.layout_ = layout();
        m.base_ = buffer_.ptr();
        m.cap_ = buffer_.len();
        return m;
    }
    std::vector<T> read() const { return buffer_.read(); }

private:
    Tensor(std::vector<uint32_t> shape, GpuBuffer<T> buffer) : shape_(std::move(shape)), buffer_(std::move(buffer)) {}
    std::vector<uint32_t> shape_;
    GpuBuffer<T> buffer_;
};

/* --------------------------------------------------------------------- operators ---- */
/* src/linalg/gemm.rs:34-321.  out = lhs * rhs, batched over the two leading dimensions, any strides. */
struct Gemm {
    /* Gemm::dispatch — :47-187: seven shape asserts (ShapeMismatch), then tiled iff M >= 32 || N >= 32. */
    static void dispatch(const GpuBackend& b, const TensorMut<float>& out, const TensorRef<float>& lhs,
                         const TensorRef<float>& rhs) {
        go(b, VX_DISPATCH, out, lhs, rhs);
    }
    /* :190-246 and :249-305: forced kernels, no asserts. */
    static void dispatch_naive(const GpuBackend& b, const TensorMut<float>& out, const TensorRef<float>& lhs,
                               const TensorRef<float>& rhs) {
        go(b, VX_DISPATCH_NAIVE, out, lhs, rhs);
    }
    static void dispatch_tiled(const GpuBackend& b, const TensorMut<float>& out, const TensorRef<float>& lhs,
                               const TensorRef<float>& rhs) {
        go(b, VX_DISPATCH_TILED, out, lhs, rhs);
    }
    /* Same asserts as dispatch, then the tcgen05 TF32 kernel (no reference counterpart). */
    static void dispatch_tf32(const GpuBackend& b, const TensorMut<float>& out, const TensorRef<float>& lhs,
                              const TensorRef<float>& rhs) {
        go(b, VX_DISPATCH_TF32, out, lhs, rhs);
    }
    /* 1 naive, 2 SIMT vector, 3 tcgen05, 4 SIMT generic strides */
    static int last_kernel(const GpuBackend& b) {
        int32_t k = 0;
        check(vx_gemm_last_kernel(b.ctx(), &k));
        return k;
    }

private:
    static void go(const GpuBackend& b, vx_dispatch_kind kind, const TensorMut<float>& out, const TensorRef<float>& lhs,
                   const TensorRef<float>& rhs) {
        check(vx_gemm_dispatch(b.ctx(), kind, out.raw_buffer(), &out.layout().l, out.raw_len(), lhs.raw_buffer(),
                               &lhs.layout().l, lhs.raw_len(), rhs.raw_buffer(), &rhs.layout().l, rhs.raw_len()));
    }
};

/* src/linalg/reduce.rs:16-30 */
enum class ReduceVariant { Sum = VX_REDUCE_SUM, Prod = VX_REDUCE_PROD, Min = VX_REDUCE_MIN, Max = VX_REDUCE_MAX,
                           SqNorm = VX_REDUCE_SQNORM };
/* Reduce::launch — src/linalg/reduce.rs:79-207: the w axis of the canonical input into output[0]. */
struct Reduce {
    static void launch(const GpuBackend& b, ReduceVariant variant, const TensorRef<float>& input,
                       const TensorMut<float>& output, vx_reduce_mode mode = VX_REDUCE_ORDERED) {
        const vx_shape s = input.layout().canonicalize().into_gpu();
        check(vx_reduce(b.ctx(), (vx_reduce_op)variant, VX_F32, mode, input.buffer(), &s,
                        input.raw_len() - input.layout().offset(), output.buffer()));
    }
};

/* src/linalg/op_assign.rs:12-24 */
enum class OpAssignVariant { Add = VX_OP_ADD, Sub = VX_OP_SUB, Mul = VX_OP_MUL, Div = VX_OP_DIV, Copy = VX_OP_COPY };
/* OpAssign::launch — src/linalg/op_assign.rs:38-143: a op= b with b broadcast to a. */
struct OpAssign {
    static void launch(const GpuBackend& b, OpAssignVariant variant, const TensorMut<float>& a, const TensorRef<float>& rhs) {
        check(vx_op_assign_dispatch(b.ctx(), (vx_op)variant, 0, a.raw_buffer(), &a.layout().l, a.raw_len(), rhs.raw_buffer(),
                                    &rhs.layout().l, rhs.raw_len()));
    }
};
/* Repeat::launch — src/linalg/repeat.rs:24-88 */
struct Repeat {
    static void launch(const GpuBackend& b, const TensorMut<float>& destination, const TensorRef<float>& source) {
        check(vx_op_assign_dispatch(b.ctx(), VX_OP_COPY, 1, destination.raw_buffer(), &destination.layout().l,
                                    destination.raw_len(), source.raw_buffer(), &source.layout().l, source.raw_len()));
    }
};
/* Contiguous::launch — src/linalg/contiguous.rs:24-129 (4-byte elements). */
struct Contiguous {
    static void launch(const GpuBackend& b, const TensorMut<float>& out, const TensorRef<float>& tensor) {
        for (uint32_t i = 0; i < 4; ++i)
            if (out.layout().canonicalize().size(i) != tensor.layout().canonicalize().size(i))
                throw ShapeMismatch(VX_ERR_SHAPE, "Contiguous: source and destination sizes differ");
        if (!out.is_contiguous()) throw Error(VX_ERR_INVALID_ARGUMENT, "Output tensor must be contiguous.");
        const vx_shape s = tensor.layout().canonicalize().into_gpu();
        check(vx_contiguous(b.ctx(), out.buffer(), out.raw_len() - out.layout().offset(), tensor.raw_buffer(), &s,
                            tensor.raw_len(), tensor.layout().offset()));
    }
};

/* ---------------------------------------------------------- block-quantised weights ---- */
/* Device-resident Q8_0 / Q4_0 matrix (no reference counterpart). */
class QuantizedMatrix {
public:
    /* Quantises `w` (rows x cols, row-major, cols % 32 == 0) on the host and uploads it. */
    QuantizedMatrix(const GpuBackend& b, vx_qtype type, const std::vector<float>& w, size_t rows, size_t cols)
        : ctx_(b.ctx()), rows_(rows), cols_(cols) {
        if (w.size() != rows * cols) throw Error(VX_ERR_INVALID_ARGUMENT, "weight data size mismatch");
        std::vector<uint8_t> blocks(rows * (cols / 32) * vx_qblock_bytes(type));
        check(vx_quantize(type, w.data(), rows, cols, blocks.data()));
        check(vx_qweights_upload(ctx_, type, blocks.data(), rows, cols, &w_));
    }
    QuantizedMatrix(const QuantizedMatrix&) = delete;
    QuantizedMatrix& operator=(const QuantizedMatrix&) = delete;
    ~QuantizedMatrix() {
        if (w_) vx_qweights_free(ctx_, w_);
    }
    const vx_qweights* handle() const { return w_; }
    size_t rows() const { return rows_; }
    size_t cols() const { return cols_; }

private:
    vx_context* ctx_;
    vx_qweights* w_ = nullptr;
    size_t rows_, cols_;
};

/* y = W x for `batch` contiguous vectors. */
struct Gemv {
    static void dispatch(const GpuBackend& b, const TensorMut<float>& y, const QuantizedMatrix& w, const TensorRef<float>& x,
                         size_t batch = 1) {
        if (x.len() < batch * w.cols() || y.len() < batch * w.rows())
            throw ShapeMismatch(VX_ERR_SHAPE, "Gemv: x or y shorter than batch vectors");
        check(vx_gemv_q(b.ctx(), w.handle(), x.buffer(), w.cols(), y.buffer(), w.rows(), batch));
    }
};

/* A fixed list of products in one persistent launch (vx_gemv_batch). */
class GemvBatch {
public:
    GemvBatch(const GpuBackend& b, const std::vector<vx_gemv_op>& ops) : ctx_(b.ctx()) {
        check(vx_gemv_batch_create(ctx_, ops.data(), ops.size(), &batch_));
    }
    GemvBatch(const GemvBatch&) = delete;
    GemvBatch& operator=(const GemvBatch&) = delete;
    ~GemvBatch() {
        if (batch_) vx_gemv_batch_free(ctx_, batch_);
    }
    void launch() const { check(vx_gemv_batch_launch(ctx_, batch_)); }
    const vx_gemv_batch* handle() const { return batch_; }

private:
    vx_context* ctx_;
    vx_gemv_batch* batch_ = nullptr;
};

}  // namespace vortx
#endif /* VORTX_B200_HPP */
