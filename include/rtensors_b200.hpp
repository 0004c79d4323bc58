// rtensors_b200.hpp -- C++17 host-side mirror of the reference's API for the hot path, on top of the
// C ABI in rt_b200.h.  Header only; link with -lrt_b200 (no CUDA headers needed by the caller).
//
// It restates, with the reference's names and argument meaning:
//   MetaTensor {shape, strides, offset}, Slice            src/core/meta.rs:155-159, src/core/slice.rs:9-52
//   trait Backend (the methods on the hot path) as class Cuda   src/backend/mod.rs:216-472
//   TensorBase<T, B>: constructors, views, operators, reductions, mean_l1_loss
//                                                           src/core/primitives.rs:367-484, src/core/tensor.rs:66-105,
//                                                           418-524, src/ops/{scalar,unary,broadcast,reduction}
// Errors are exceptions carrying the library status (TensorError variants map to status codes).
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "rt_b200.h"

namespace rtb200 {

struct TensorError : std::runtime_error {
    int code;
    TensorError(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};
inline void check(int rc) {
    if (rc != RTB_OK) throw TensorError(rc, rtb_last_error_string());
}

template <typename T> struct DTypeOf;
#define RTB200_DT(T, CODE) template <> struct DTypeOf<T> { static constexpr int value = CODE; };
RTB200_DT(uint8_t, RTB_U8) RTB200_DT(int8_t, RTB_I8) RTB200_DT(uint16_t, RTB_U16) RTB200_DT(int16_t, RTB_I16)
RTB200_DT(uint32_t, RTB_U32) RTB200_DT(int32_t, RTB_I32) RTB200_DT(uint64_t, RTB_U64) RTB200_DT(int64_t, RTB_I64)
RTB200_DT(float, RTB_F32) RTB200_DT(double, RTB_F64) RTB200_DT(bool, RTB_BOOL)
RTB200_DT(unsigned __int128, RTB_U128) RTB200_DT(__int128, RTB_I128)
#undef RTB200_DT

enum class BinaryOpType { Add = 0, Sub = 1, Mul = 2, Div = 3 };
// codes of ReductionOpTypes::get_code (src/ops/reduction/mod.rs:160-175); Variance also covers Stdev
enum class ReductionOpTypes { Sum = 1, Prod = 2, Max = 3, Min = 4, Mean = 5, Variance = 6, LogSumExp = 7, Norm = 8, ArgMax = 9, ArgMin = 10 };
enum class NormType { L1 = 1, L2 = 2 };

struct Slice {
    std::optional<size_t> start, end;
    ptrdiff_t step_ = 1;
    static Slice full() { return Slice{}; }
    static Slice range(size_t a, size_t b) { return Slice{a, b, a > b ? -1 : 1}; }  // From<Range<usize>>
    static Slice index(size_t i) { return Slice{i, i, 1}; }                          // From<usize>
    Slice step(ptrdiff_t s) const { Slice r = *this; r.step_ = s; return r; }
    Slice from(size_t s) const { Slice r = *this; r.start = s; return r; }
    Slice to(size_t e) const { Slice r = *this; r.end = e; return r; }
};

struct MetaTensor {
    std::vector<size_t> shape;
    std::vector<ptrdiff_t> strides;
    size_t offset = 0;

    static MetaTensor contiguous(std::vector<size_t> shape) {
        MetaTensor m;
        m.shape = std::move(shape);
        m.strides.resize(m.shape.size());
        rtb_meta_contiguous_strides(m.shape.size(), m.shape.data(), m.strides.data());
        return m;
    }
    size_t rank() const { return shape.size(); }
    size_t size() const { size_t n = 1; for (size_t s : shape) n *= s; return n; }
    bool is_contiguous() const { return rtb_meta_is_contiguous(rank(), shape.data(), strides.data()) != 0; }
    MetaTensor slice(size_t dim, const Slice &s) const {
        MetaTensor o;
        o.shape.resize(rank() ? rank() : 1); o.strides.resize(rank() ? rank() : 1);
        size_t r = 0;
        check(rtb_meta_slice(rank(), shape.data(), strides.data(), offset, dim, s.start.has_value(), s.start.value_or(0),
                             s.end.has_value(), s.end.value_or(0), s.step_, &r, o.shape.data(), o.strides.data(), &o.offset));
        o.shape.resize(r); o.strides.resize(r);
        return o;
    }
    MetaTensor permute(const std::vector<size_t> &dims) const {
        MetaTensor o = *this;
        check(rtb_meta_permute(rank(), shape.data(), strides.data(), dims.size(), dims.data(), o.shape.data(), o.strides.data()));
        return o;
    }
    // view_as_inner (src/core/tensor.rs:328-355): contiguous views only, equal element count
    MetaTensor view_as(std::vector<size_t> new_shape) const {
        MetaTensor o = MetaTensor::contiguous(std::move(new_shape));
        if (!is_contiguous()) throw TensorError(RTB_ERR_NONCONTIG, "Cannot view_as non contiguous tensor");
        if (o.size() != size()) throw TensorError(RTB_ERR_SHAPE, "Invalid size for initial shape");
        o.offset = offset;
        return o;
    }
    MetaTensor transpose() const {
        std::vector<size_t> dims(rank());
        for (size_t k = 0; k < rank(); ++k) dims[k] = rank() - 1 - k;
        return permute(dims);
    }
    MetaTensor unsqueeze(size_t dim) const {
        MetaTensor o;
        o.offset = offset; o.shape.resize(rank() + 1); o.strides.resize(rank() + 1);
        check(rtb_meta_unsqueeze(rank(), shape.data(), strides.data(), dim, o.shape.data(), o.strides.data()));
        return o;
    }
    MetaTensor squeeze(ptrdiff_t dim = -1) const {
        MetaTensor o = *this;
        size_t r = 0;
        if (rank() == 0) return o;
        check(rtb_meta_squeeze(rank(), shape.data(), strides.data(), dim, &r, o.shape.data(), o.strides.data()));
        o.shape.resize(r); o.strides.resize(r);
        return o;
    }
};

// ---- Backend ------------------------------------------------------------------------------------
class Cuda {
  public:
    explicit Cuda(int device = 0) { check(rtb_ctx_create(device, &ctx_)); }
    ~Cuda() { rtb_ctx_destroy(ctx_); }
    Cuda(const Cuda &) = delete;
    Cuda &operator=(const Cuda &) = delete;
    rtb_ctx *ctx() const { return ctx_; }
    void sync() const { check(rtb_ctx_sync(ctx_)); }

    template <typename T> struct Buf {
        T *ptr = nullptr;
        size_t len = 0;
        const Cuda *owner = nullptr;
        ~Buf() { if (ptr && owner) rtb_free(owner->ctx(), ptr); }
    };
    template <typename T> using BufPtr = std::shared_ptr<Buf<T>>;

    template <typename T> BufPtr<T> alloc(size_t len) const {  // uninitialised
        auto b = std::make_shared<Buf<T>>();
        void *p = nullptr;
        check(rtb_alloc(ctx_, (len ? len : 1) * sizeof(T), &p));
        b->ptr = static_cast<T *>(p); b->len = len; b->owner = this;
        return b;
    }
    template <typename T> BufPtr<T> alloc_from_slice(const std::vector<T> &src) const {
        auto b = alloc<T>(src.size());
        if (!src.empty()) check(rtb_h2d(ctx_, b->ptr, src.data(), src.size() * sizeof(T)));
        sync();  // the host vector may go away
        return b;
    }
    template <typename T> std::vector<T> dump(const Buf<T> &b) const {
        std::vector<T> out(b.len);
        if (b.len) check(rtb_d2h(ctx_, out.data(), b.ptr, b.len * sizeof(T)));
        return out;
    }
    template <typename T> size_t len(const Buf<T> &b) const { return b.len; }
    // Backend::copy_from_slice / copy_range_within (src/backend/mod.rs:227-228; checks as in src/backend/cpu.rs:151-183)
    template <typename T> void copy_from_slice(Buf<T> &dst, const std::vector<T> &src) const {
        if (dst.len != src.size()) throw TensorError(RTB_ERR_SHAPE, "Buffer size mismatch in copy_from_slice");
        if (!src.empty()) check(rtb_h2d(ctx_, dst.ptr, src.data(), src.size() * sizeof(T)));
        sync();
    }
    template <typename T> void copy_range_within(Buf<T> &dst, const Buf<T> &src, size_t dst_offset, size_t src_offset, size_t n) const {
        if (dst_offset + n > dst.len || src_offset + n > src.len)
            throw TensorError(RTB_ERR_BOUNDS, "Index out of bounds in copy_range_within");
        if (n) check(rtb_d2d(ctx_, dst.ptr + dst_offset, src.ptr + src_offset, n * sizeof(T)));
    }
    template <typename T> T read(const Buf<T> &b, size_t offset) const {
        if (offset >= b.len) throw TensorError(RTB_ERR_BOUNDS, "Index out of bounds for buffer");
        T v;
        check(rtb_d2h(ctx_, &v, b.ptr + offset, sizeof(T)));
        return v;
    }
    template <typename T> void write(Buf<T> &b, size_t offset, T v) const {
        if (offset >= b.len) throw TensorError(RTB_ERR_BOUNDS, "Index out of bounds for buffer");
        check(rtb_h2d(ctx_, b.ptr + offset, &v, sizeof(T)));
        sync();
    }
    template <typename T> BufPtr<T> copy(const Buf<T> &b) const {
        auto o = alloc<T>(b.len);
        if (b.len) check(rtb_d2d(ctx_, o->ptr, b.ptr, b.len * sizeof(T)));
        return o;
    }

    template <typename T> void scalar_apply(Buf<T> &buf, BinaryOpType op, T value, const MetaTensor &m) const {
        check(rtb_meta_check_extent(m.rank(), m.shape.data(), m.strides.data(), m.offset, buf.len));
        check(rtb_scalar_op(ctx_, DTypeOf<T>::value, (int)op, buf.ptr, &value, m.rank(), m.shape.data(), m.strides.data(), m.offset));
    }
    template <typename T> void scalar_apply_add(Buf<T> &b, T v, const MetaTensor &m) const { scalar_apply(b, BinaryOpType::Add, v, m); }
    template <typename T> void scalar_apply_sub(Buf<T> &b, T v, const MetaTensor &m) const { scalar_apply(b, BinaryOpType::Sub, v, m); }
    template <typename T> void scalar_apply_mul(Buf<T> &b, T v, const MetaTensor &m) const { scalar_apply(b, BinaryOpType::Mul, v, m); }
    template <typename T> void scalar_apply_div(Buf<T> &b, T v, const MetaTensor &m) const { scalar_apply(b, BinaryOpType::Div, v, m); }

    template <typename T> void apply_unary(Buf<T> &buf, int unop, const MetaTensor &m) const {
        check(rtb_meta_check_extent(m.rank(), m.shape.data(), m.strides.data(), m.offset, buf.len));
        check(rtb_unary_op(ctx_, DTypeOf<T>::value, unop, buf.ptr, m.rank(), m.shape.data(), m.strides.data(), m.offset));
    }
    template <typename T> void apply_neg(Buf<T> &b, const MetaTensor &m) const { apply_unary(b, RTB_NEG, m); }
    template <typename T> void apply_relu(Buf<T> &b, const MetaTensor &m) const { apply_unary(b, RTB_RELU, m); }
    template <typename T> void apply_abs(Buf<T> &b, const MetaTensor &m) const { apply_unary(b, RTB_ABS, m); }
    template <typename T> void apply_sign(Buf<T> &b, const MetaTensor &m) const { apply_unary(b, RTB_SIGN, m); }

    template <typename T> void fill(Buf<T> &buf, T value, const MetaTensor &m) const {
        check(rtb_meta_check_extent(m.rank(), m.shape.data(), m.strides.data(), m.offset, buf.len));
        check(rtb_fill(ctx_, DTypeOf<T>::value, buf.ptr, &value, m.rank(), m.shape.data(), m.strides.data(), m.offset));
    }
    // Backend::broadcast: all three metas carry the output shape; dst may be left (in place)
    template <typename T>
    void broadcast(const Buf<T> &l, const MetaTensor &lm, const Buf<T> &r, const MetaTensor &rm, Buf<T> &d,
                   const MetaTensor &dm, BinaryOpType op) const {
        check(rtb_meta_check_extent(lm.rank(), lm.shape.data(), lm.strides.data(), lm.offset, l.len));
        check(rtb_meta_check_extent(rm.rank(), rm.shape.data(), rm.strides.data(), rm.offset, r.len));
        check(rtb_meta_check_extent(dm.rank(), dm.shape.data(), dm.strides.data(), dm.offset, d.len));
        check(rtb_broadcast(ctx_, DTypeOf<T>::value, (int)op, l.ptr, lm.strides.data(), lm.offset, r.ptr, rm.strides.data(),
                            rm.offset, d.ptr, dm.strides.data(), dm.offset, dm.rank(), dm.shape.data()));
    }
    template <typename T>
    void apply_reduce_contiguous_flat(const Buf<T> &src, Buf<T> &dst, size_t start, size_t len, ReductionOpTypes op) const {
        if (start + len > src.len) throw TensorError(RTB_ERR_BOUNDS, "flat reduction range exceeds the buffer");
        check(rtb_reduce_flat(ctx_, DTypeOf<T>::value, (int)op, src.ptr, start, len, dst.ptr));
    }
    template <typename T>
    void apply_reduce(const Buf<T> &src, const MetaTensor &sm, Buf<T> &dst, size_t dim, ReductionOpTypes op) const {
        if (!sm.is_contiguous()) throw TensorError(RTB_ERR_NONCONTIG, "Reduction over non-contiguous tensors is not implemented yet.");
        if (sm.rank() == 1) return apply_reduce_contiguous_flat(src, dst, sm.offset, sm.size(), op);
        size_t outer = 1, inner = 1;
        for (size_t k = 0; k < dim; ++k) outer *= sm.shape[k];
        for (size_t k = dim + 1; k < sm.rank(); ++k) inner *= sm.shape[k];
        check(rtb_reduce_axis(ctx_, DTypeOf<T>::value, (int)op, src.ptr, sm.offset, outer, sm.shape[dim], inner, dst.ptr));
    }
    // any reduction code over a view, the op's settings alongside (variance / std / norm); Out is T,
    // or uint64_t for ArgMax / ArgMin.  axis < 0 reduces everything.
    template <typename T, typename Out>
    void reduce_view(const Buf<T> &src, const MetaTensor &m, ptrdiff_t axis, ReductionOpTypes op, Buf<Out> &dst, bool unbiased = true,
                     bool is_std = false, NormType norm = NormType::L2) const {
        check(rtb_meta_check_extent(m.rank(), m.shape.data(), m.strides.data(), m.offset, src.len));
        rtb_reduce_settings st{unbiased, is_std, (int)norm};
        check(rtb_reduce_view_ex(ctx_, DTypeOf<T>::value, (int)op, &st, src.ptr, m.rank(), m.shape.data(), m.strides.data(), m.offset,
                                 axis, dst.ptr));
    }
    // Backend::convert (src/backend/mod.rs:234): dst[i] = src[i] as N, both buffers of equal length
    template <typename T, typename N> void convert(const Buf<T> &src, Buf<N> &dst) const {
        if (src.len != dst.len) throw TensorError(RTB_ERR_SHAPE, "Buffer size mismatch in convert");
        check(rtb_convert(ctx_, DTypeOf<T>::value, DTypeOf<N>::value, src.ptr, dst.ptr, src.len));
    }
    // dense per-element map of a view (relu / abs / leaky_relu gradient maps, reciprocal), kind = RTB_MASK_*
    template <typename T> void grad_mask(const Buf<T> &src, const MetaTensor &m, int kind, Buf<T> &dst, T value = T()) const {
        check(rtb_meta_check_extent(m.rank(), m.shape.data(), m.strides.data(), m.offset, src.len));
        check(rtb_grad_mask(ctx_, DTypeOf<T>::value, kind, &value, src.ptr, m.rank(), m.shape.data(), m.strides.data(), m.offset, dst.ptr));
    }
    template <typename T> void copy_view(const Buf<T> &src, const MetaTensor &m, Buf<T> &dst) const {
        check(rtb_copy_view(ctx_, DTypeOf<T>::value, src.ptr, m.rank(), m.shape.data(), m.strides.data(), m.offset, dst.ptr));
    }
    // one dense layer's `+ bias`, relu and relu gradient map in one pass over a dense (rows, cols) activation
    template <typename T> void bias_relu_mask(Buf<T> &z, const Buf<T> &bias, Buf<T> &mask, size_t rows, size_t cols) const {
        if (z.len < rows * cols || mask.len < rows * cols || bias.len < cols) throw TensorError(RTB_ERR_BOUNDS, "bias_relu_mask: buffer too small");
        check(rtb_bias_relu_mask(ctx_, DTypeOf<T>::value, z.ptr, bias.ptr, mask.ptr, rows, cols));
    }

    // ---- tensors in HOST memory (rtb_host_*): the context's upload and download lanes overlap a tensor's
    //      upload, the kernels and the copy-out of results; every call enqueues, host_wait() completes.
    //      The reference uploads and dumps whole tensors with blocking copies (src/backend/cuda.rs:668-680,
    //      770-788).  HostVec<T> is page-locked memory from the library. -------------------------------------
    template <typename T> struct HostVec {
        T *ptr = nullptr;
        size_t len = 0;
        explicit HostVec(size_t n) : len(n) { check(rtb_host_alloc(n * sizeof(T), (void **)&ptr)); }
        HostVec(const std::vector<T> &v) : HostVec(v.size()) { std::copy(v.begin(), v.end(), ptr); }
        HostVec(const HostVec &) = delete;
        HostVec &operator=(const HostVec &) = delete;
        ~HostVec() { rtb_host_free(ptr); }
        T &operator[](size_t i) { return ptr[i]; }
        const T &operator[](size_t i) const { return ptr[i]; }
        std::vector<T> to_vector() const { return std::vector<T>(ptr, ptr + len); }
    };
    // `l op r` with both operand buffers in host memory; out receives indices [begin, end) of the
    // outermost output dim, row-major
    template <typename T>
    void host_broadcast(const HostVec<T> &l, const MetaTensor &lm, const HostVec<T> &r, const MetaTensor &rm, BinaryOpType op,
                        HostVec<T> &out, size_t begin, size_t end) const;
    template <typename T, typename Out>
    void host_reduce_view(const HostVec<T> &src, const MetaTensor &m, ptrdiff_t axis, ReductionOpTypes op, HostVec<Out> &dst,
                          bool unbiased = true, bool is_std = false, NormType norm = NormType::L2) const {
        rtb_reduce_settings st{unbiased, is_std, (int)norm};
        size_t n_out = 1;
        for (size_t d = 0; d < m.rank(); ++d)
            if (axis >= 0 && (ptrdiff_t)d != axis) n_out *= m.shape[d];
        if (dst.len < n_out) throw TensorError(RTB_ERR_BOUNDS, "host_reduce_view: the result does not fit");
        check(rtb_host_reduce_view(ctx_, DTypeOf<T>::value, (int)op, &st, src.ptr, src.len, m.rank(), m.shape.data(), m.strides.data(),
                                   m.offset, axis, dst.ptr));
    }
    // the primitives: a pool block that is being uploaded (the compute stream waits for it at host_ready),
    // a scratch block, a copy-out behind the work enqueued so far, and the block's return to the pool
    template <typename T> T *host_stage_in(const HostVec<T> &src) const {
        void *dev = nullptr;
        check(rtb_host_stage_in(ctx_, src.ptr, src.len * sizeof(T), &dev));
        return (T *)dev;
    }
    template <typename T> T *host_scratch(size_t n) const {
        void *dev = nullptr;
        check(rtb_host_scratch(ctx_, n * sizeof(T), &dev));
        return (T *)dev;
    }
    void host_ready(const void *dev) const { check(rtb_host_ready(ctx_, dev)); }
    template <typename T> void host_stage_out(const T *dev, HostVec<T> &dst, size_t n) const {
        if (n > dst.len) throw TensorError(RTB_ERR_BOUNDS, "host_stage_out: the host buffer is too small");
        check(rtb_host_stage_out(ctx_, dev, dst.ptr, n * sizeof(T)));
    }
    void host_release(void *dev) const { check(rtb_host_release(ctx_, dev)); }
    void host_join() const { check(rtb_host_join(ctx_)); }
    void host_wait() const { check(rtb_host_wait(ctx_)); }

    // ---- several GPUs: one Cuda per device (one process per GPU, or one host thread per device); the
    //      reference has a single device (`// TODO multiple devices`, src/backend/cuda.rs:155-162).  All
    //      mg_* device calls are collective: same calls, same order, on every rank. ------------------------
    static std::vector<unsigned char> mg_unique_id() {
        std::vector<unsigned char> id(RTB_MG_ID_BYTES);
        check(rtb_mg_unique_id(id.data()));
        return id;
    }
    void mg_init(int nranks, int rank, const std::vector<unsigned char> &id) const { check(rtb_mg_init(ctx_, nranks, rank, id.data())); }
    void mg_finalize() const { check(rtb_mg_finalize(ctx_)); }
    int mg_world() const { int n = 1; check(rtb_mg_info(ctx_, &n, nullptr, nullptr)); return n; }
    int mg_rank() const { int r = 0; check(rtb_mg_info(ctx_, nullptr, &r, nullptr)); return r; }
    bool mg_peer_mapped() const { int m = 0; check(rtb_mg_info(ctx_, nullptr, nullptr, &m)); return m != 0; }
    unsigned mg_status() const { unsigned b = 0; check(rtb_mg_status(ctx_, &b)); return b; }
    void mg_realign() const { check(rtb_mg_realign(ctx_)); }
    void mg_set_wait_ns(uint64_t ns) const { check(rtb_mg_set_wait_ns(ctx_, ns)); }
    // full reduction of a tensor whose flat range is split across the ranks: src holds this rank's local_len elements
    template <typename T>
    void mg_reduce_flat(const Buf<T> &src, size_t start, size_t local_len, size_t global_len, ReductionOpTypes op, Buf<T> &dst) const {
        if (start + local_len > src.len) throw TensorError(RTB_ERR_BOUNDS, "flat reduction range exceeds the buffer");
        check(rtb_mg_reduce_flat(ctx_, DTypeOf<T>::value, (int)op, src.ptr, start, local_len, global_len, dst.ptr));
    }
    // axis reduction whose reduced dim is split: this rank holds r_local of global_r rows of a dense [outer, r, inner] block
    template <typename T>
    void mg_reduce_axis(const Buf<T> &src, size_t offset, size_t outer, size_t r_local, size_t inner, size_t global_r,
                        ReductionOpTypes op, Buf<T> &dst) const {
        check(rtb_mg_reduce_axis(ctx_, DTypeOf<T>::value, (int)op, src.ptr, offset, outer, r_local, inner,
                                 (ptrdiff_t)(r_local * inner), (ptrdiff_t)inner, global_r, dst.ptr));
    }
    template <typename T> void mg_combine(Buf<T> &buf, size_t n, ReductionOpTypes op, size_t mean_count = 0) const {
        check(rtb_mg_combine(ctx_, DTypeOf<T>::value, (int)op, buf.ptr, n, mean_count));
    }
    template <typename T> void mg_allreduce(Buf<T> &buf, size_t n, ReductionOpTypes op, bool overlap = false) const {
        check((overlap ? rtb_mg_allreduce_begin : rtb_mg_allreduce)(ctx_, DTypeOf<T>::value, (int)op, buf.ptr, n, 0));
    }
    void mg_allreduce_join() const { check(rtb_mg_allreduce_join(ctx_)); }

  private:
    rtb_ctx *ctx_ = nullptr;
};

inline void broadcast_params(const MetaTensor &a, const MetaTensor &b, std::vector<size_t> &shape,
                             std::vector<ptrdiff_t> &sa, std::vector<ptrdiff_t> &sb) {
    size_t r = a.rank() > b.rank() ? a.rank() : b.rank(), out_r = 0;
    shape.assign(r ? r : 1, 0); sa.assign(r ? r : 1, 0); sb.assign(r ? r : 1, 0);
    check(rtb_broadcast_params(a.rank(), a.shape.data(), a.strides.data(), b.rank(), b.shape.data(), b.strides.data(), &out_r,
                               shape.data(), sa.data(), sb.data()));
    shape.resize(out_r); sa.resize(out_r); sb.resize(out_r);
}

template <typename T>
void Cuda::host_broadcast(const HostVec<T> &l, const MetaTensor &lm, const HostVec<T> &r, const MetaTensor &rm, BinaryOpType op,
                          HostVec<T> &out, size_t begin, size_t end) const {
    std::vector<size_t> shape;
    std::vector<ptrdiff_t> sl, sr;
    broadcast_params(lm, rm, shape, sl, sr);
    size_t per = 1;
    for (size_t d = 1; d < shape.size(); ++d) per *= shape[d];
    if (end < begin || out.len < (end - begin) * per) throw TensorError(RTB_ERR_BOUNDS, "host_broadcast: the result does not fit");
    check(rtb_host_broadcast(ctx_, DTypeOf<T>::value, (int)op, l.ptr, l.len, sl.data(), lm.offset, r.ptr, r.len, sr.data(), rm.offset,
                             out.ptr, shape.size(), shape.data(), begin, end));
}

// ---- TensorBase<T, Cuda> (owned tensors and views share this type; views share the buffer) -------
template <typename T> class TensorBase {
  public:
    using Buf = typename Cuda::template Buf<T>;
    const Cuda *backend = nullptr;
    std::shared_ptr<Buf> buf;
    MetaTensor meta;

    static TensorBase from_buf(const Cuda &b, const std::vector<T> &data, std::vector<size_t> shape) {
        MetaTensor m = MetaTensor::contiguous(std::move(shape));
        if (m.size() != data.size()) throw TensorError(RTB_ERR_SHAPE, "Element count mismatch");
        return TensorBase{&b, b.alloc_from_slice(data), m};
    }
    static TensorBase full(const Cuda &b, std::vector<size_t> shape, T v) {
        MetaTensor m = MetaTensor::contiguous(std::move(shape));
        TensorBase t{&b, b.alloc<T>(m.size()), m};
        b.fill(*t.buf, v, m);
        return t;
    }
    static TensorBase zeros(const Cuda &b, std::vector<size_t> shape) { return full(b, std::move(shape), T(0)); }
    static TensorBase ones(const Cuda &b, std::vector<size_t> shape) { return full(b, std::move(shape), T(1)); }
    static TensorBase scalar(const Cuda &b, T v) { return from_buf(b, {v}, {}); }
    static TensorBase column(const Cuda &b, const std::vector<T> &v) { return from_buf(b, v, {v.size()}); }
    static TensorBase row(const Cuda &b, const std::vector<T> &v) { return from_buf(b, v, {1, v.size()}); }

    const std::vector<size_t> &shape() const { return meta.shape; }
    const std::vector<ptrdiff_t> &strides() const { return meta.strides; }
    size_t offset() const { return meta.offset; }
    size_t size() const { return meta.size(); }
    bool is_contiguous() const { return meta.is_contiguous(); }

    TensorBase view_of(MetaTensor m) const { return TensorBase{backend, buf, std::move(m)}; }
    TensorBase slice(size_t dim, const Slice &s) const { return view_of(meta.slice(dim, s)); }
    TensorBase permute(const std::vector<size_t> &dims) const { return view_of(meta.permute(dims)); }
    TensorBase squeeze() const { return view_of(meta.squeeze()); }
    TensorBase unsqueeze(size_t dim) const { return view_of(meta.unsqueeze(dim)); }

    TensorBase contiguous() const {
        MetaTensor m = MetaTensor::contiguous(meta.shape);
        TensorBase t{backend, backend->template alloc<T>(m.size()), m};
        if (m.size()) backend->copy_view(*buf, meta, *t.buf);
        return t;
    }
    TensorBase owned() const { return contiguous(); }
    TensorBase view_as(std::vector<size_t> shape) const { return view_of(meta.view_as(std::move(shape))); }
    TensorBase transpose() const { return view_of(meta.transpose()); }
    // contiguous() then view_as: always a fresh buffer (src/core/tensor.rs:238-243)
    TensorBase reshape(std::vector<size_t> shape) const {
        TensorBase c = contiguous();
        c.meta = c.meta.view_as(std::move(shape));
        return c;
    }
    void fill(T v) { backend->fill(*buf, v, meta); }
    // alloc + convert of the whole buffer, meta cloned (src/core/primitives.rs:527-538)
    template <typename N> TensorBase<N> into_dtype() const {
        TensorBase<N> t{backend, backend->template alloc<N>(buf->len), meta};
        backend->convert(*buf, *t.buf);
        return t;
    }
    std::vector<T> cpu() const {
        TensorBase c = contiguous();
        std::vector<T> all = backend->dump(*c.buf);
        all.resize(size());
        return all;
    }
    T item() const {
        if (size() != 1) throw TensorError(RTB_ERR_SHAPE, "item() needs a single-element tensor");
        return backend->read(*buf, meta.offset);
    }
    T get(const std::vector<size_t> &coord) const {
        size_t o = meta.offset;
        for (size_t k = 0; k < coord.size(); ++k) o += (ptrdiff_t)coord[k] * meta.strides[k];
        return backend->read(*buf, o);
    }
    void set(const std::vector<size_t> &coord, T v) {
        size_t o = meta.offset;
        for (size_t k = 0; k < coord.size(); ++k) o += (ptrdiff_t)coord[k] * meta.strides[k];
        backend->write(*buf, o, v);
    }

    // tensor (op) tensor: broadcast into a fresh row-major tensor
    TensorBase binary(const TensorBase &rhs, BinaryOpType op) const {
        std::vector<size_t> shape; std::vector<ptrdiff_t> sa, sb;
        broadcast_params(meta, rhs.meta, shape, sa, sb);
        MetaTensor dm = MetaTensor::contiguous(shape);
        TensorBase out{backend, backend->template alloc<T>(dm.size()), dm};
        backend->broadcast(*buf, MetaTensor{shape, sa, meta.offset}, *rhs.buf, MetaTensor{shape, sb, rhs.meta.offset}, *out.buf, dm, op);
        return out;
    }
    TensorBase &assign(const TensorBase &rhs, BinaryOpType op) {
        std::vector<size_t> shape; std::vector<ptrdiff_t> sa, sb;
        broadcast_params(meta, rhs.meta, shape, sa, sb);
        if (shape != meta.shape) throw TensorError(RTB_ERR_BROADCAST, "Incompatible shapes for in-place op");
        MetaTensor ma{shape, sa, meta.offset};
        backend->broadcast(*buf, ma, *rhs.buf, MetaTensor{shape, sb, rhs.meta.offset}, *buf, ma, op);
        return *this;
    }
    TensorBase operator+(const TensorBase &r) const { return binary(r, BinaryOpType::Add); }
    TensorBase operator-(const TensorBase &r) const { return binary(r, BinaryOpType::Sub); }
    TensorBase operator*(const TensorBase &r) const { return binary(r, BinaryOpType::Mul); }
    TensorBase operator/(const TensorBase &r) const { return binary(r, BinaryOpType::Div); }
    TensorBase &operator+=(const TensorBase &r) { return assign(r, BinaryOpType::Add); }
    TensorBase &operator-=(const TensorBase &r) { return assign(r, BinaryOpType::Sub); }
    TensorBase &operator*=(const TensorBase &r) { return assign(r, BinaryOpType::Mul); }
    TensorBase &operator/=(const TensorBase &r) { return assign(r, BinaryOpType::Div); }
    // tensor (op) scalar: copy, then in place (src/ops/scalar/add.rs:93-97)
    TensorBase scalar_op(T v, BinaryOpType op) const { TensorBase t = owned(); t.backend->scalar_apply(*t.buf, op, v, t.meta); return t; }
    TensorBase operator+(T v) const { return scalar_op(v, BinaryOpType::Add); }
    TensorBase operator-(T v) const { return scalar_op(v, BinaryOpType::Sub); }
    TensorBase operator*(T v) const { return scalar_op(v, BinaryOpType::Mul); }
    TensorBase operator/(T v) const { return scalar_op(v, BinaryOpType::Div); }
    TensorBase &operator+=(T v) { backend->scalar_apply(*buf, BinaryOpType::Add, v, meta); return *this; }
    TensorBase &operator-=(T v) { backend->scalar_apply(*buf, BinaryOpType::Sub, v, meta); return *this; }
    TensorBase &operator*=(T v) { backend->scalar_apply(*buf, BinaryOpType::Mul, v, meta); return *this; }
    TensorBase &operator/=(T v) { backend->scalar_apply(*buf, BinaryOpType::Div, v, meta); return *this; }

    TensorBase &relu_inplace() { backend->apply_relu(*buf, meta); return *this; }
    TensorBase &abs_inplace() { backend->apply_abs(*buf, meta); return *this; }
    TensorBase &sign_inplace() { backend->apply_sign(*buf, meta); return *this; }
    TensorBase &neg_inplace() { backend->apply_neg(*buf, meta); return *this; }
    TensorBase relu() const { TensorBase t = owned(); t.relu_inplace(); return t; }
    TensorBase abs() const { TensorBase t = owned(); t.abs_inplace(); return t; }
    TensorBase sign() const { TensorBase t = owned(); t.sign_inplace(); return t; }
    TensorBase neg() const { TensorBase t = owned(); t.neg_inplace(); return t; }
    TensorBase grad_map(int kind, T value = T()) const {
        MetaTensor m = MetaTensor::contiguous(meta.shape);
        TensorBase t{backend, backend->template alloc<T>(m.size()), m};
        if (m.size()) backend->grad_mask(*buf, meta, kind, *t.buf, value);
        return t;
    }
    TensorBase leaky_relu_grad_map(T slope) const { return grad_map(RTB_MASK_LEAKY_RELU, slope); }  // src/ops/scalar/mod.rs:149-166
    TensorBase reciprocal_map() const { return grad_map(RTB_MASK_RECIPROCAL); }                    // src/ops/broadcast/div.rs:583-587
    TensorBase relu_grad_map() const { return grad_map(RTB_MASK_RELU); }
    TensorBase abs_grad_map() const { return grad_map(RTB_MASK_ABS); }

    // reductions: a non-contiguous view is copied first; `_at` keeps the reduced dim as size 1
    TensorBase reduce(ReductionOpTypes op) const {
        TensorBase t = is_contiguous() ? *this : contiguous();
        TensorBase out{backend, backend->template alloc<T>(1), MetaTensor::contiguous({})};
        backend->apply_reduce_contiguous_flat(*t.buf, *out.buf, t.meta.offset, t.size(), op);
        return out;
    }
    TensorBase reduce_at(size_t axis, ReductionOpTypes op) const {
        TensorBase t = is_contiguous() ? *this : contiguous();
        if (axis >= t.meta.rank()) throw TensorError(RTB_ERR_DIM, "axis out of range");
        std::vector<size_t> os = t.meta.shape;
        os[axis] = 1;
        MetaTensor om = MetaTensor::contiguous(os);
        TensorBase out{backend, backend->template alloc<T>(om.size()), om};
        if (om.size()) backend->apply_reduce(*t.buf, t.meta, *out.buf, axis, op);
        return out;
    }
    TensorBase sum() const { return reduce(ReductionOpTypes::Sum); }
    TensorBase mean() const { return reduce(ReductionOpTypes::Mean); }
    TensorBase max() const { return reduce(ReductionOpTypes::Max); }
    TensorBase min() const { return reduce(ReductionOpTypes::Min); }
    TensorBase prod() const { return reduce(ReductionOpTypes::Prod); }
    TensorBase sum_at(size_t a) const { return reduce_at(a, ReductionOpTypes::Sum); }
    TensorBase mean_at(size_t a) const { return reduce_at(a, ReductionOpTypes::Mean); }
    TensorBase max_at(size_t a) const { return reduce_at(a, ReductionOpTypes::Max); }
    TensorBase min_at(size_t a) const { return reduce_at(a, ReductionOpTypes::Min); }
    TensorBase prod_at(size_t a) const { return reduce_at(a, ReductionOpTypes::Prod); }

    // The reductions only the reference's CUDA backend implements (ReductionOp / TotalReductionOp,
    // src/ops/reduction/mod.rs:199-250, 413-510); any view, no copy where its layout allows.
    template <typename Out>
    TensorBase<Out> reduce_ex(ptrdiff_t axis, ReductionOpTypes op, bool unbiased = true, bool is_std = false,
                              NormType norm = NormType::L2) const {
        if (axis >= (ptrdiff_t)meta.rank()) throw TensorError(RTB_ERR_DIM, "axis out of range");
        std::vector<size_t> os;
        if (axis >= 0) { os = meta.shape; os[axis] = 1; }
        MetaTensor om = MetaTensor::contiguous(os);
        TensorBase<Out> out{backend, backend->template alloc<Out>(om.size() ? om.size() : 1), om};
        if (om.size()) backend->reduce_view(*buf, meta, axis, op, *out.buf, unbiased, is_std, norm);
        return out;
    }
    TensorBase var_at(size_t a) const { return reduce_ex<T>((ptrdiff_t)a, ReductionOpTypes::Variance, true); }
    TensorBase pop_var_at(size_t a) const { return reduce_ex<T>((ptrdiff_t)a, ReductionOpTypes::Variance, false); }
    TensorBase std_at(size_t a, bool unbiased) const { return reduce_ex<T>((ptrdiff_t)a, ReductionOpTypes::Variance, unbiased, true); }
    TensorBase norm_at(size_t a, NormType n) const { return reduce_ex<T>((ptrdiff_t)a, ReductionOpTypes::Norm, true, false, n); }
    TensorBase l1_norm_at(size_t a) const { return norm_at(a, NormType::L1); }
    TensorBase l2_norm_at(size_t a) const { return norm_at(a, NormType::L2); }
    TensorBase logsumexp_at(size_t a) const { return reduce_ex<T>((ptrdiff_t)a, ReductionOpTypes::LogSumExp); }
    TensorBase<uint64_t> argmax_at(size_t a) const { return reduce_ex<uint64_t>((ptrdiff_t)a, ReductionOpTypes::ArgMax); }
    TensorBase<uint64_t> argmin_at(size_t a) const { return reduce_ex<uint64_t>((ptrdiff_t)a, ReductionOpTypes::ArgMin); }
    TensorBase var() const { return reduce_ex<T>(-1, ReductionOpTypes::Variance, true); }
    TensorBase pop_var() const { return reduce_ex<T>(-1, ReductionOpTypes::Variance, false); }
    TensorBase std(bool unbiased) const { return reduce_ex<T>(-1, ReductionOpTypes::Variance, unbiased, true); }
    TensorBase norm(NormType n) const { return reduce_ex<T>(-1, ReductionOpTypes::Norm, true, false, n); }
    TensorBase l1_norm() const { return norm(NormType::L1); }
    TensorBase l2_norm() const { return norm(NormType::L2); }
    TensorBase logsumexp() const { return reduce_ex<T>(-1, ReductionOpTypes::LogSumExp); }
    TensorBase<uint64_t> argmax() const { return reduce_ex<uint64_t>(-1, ReductionOpTypes::ArgMax); }
    TensorBase<uint64_t> argmin() const { return reduce_ex<uint64_t>(-1, ReductionOpTypes::ArgMin); }
};

// mean(|input - target|) as a rank-0 tensor (src/ops/broadcast/l1.rs:79-84), fused
template <typename T> TensorBase<T> mean_l1_loss(const TensorBase<T> &input, const TensorBase<T> &target) {
    if (input.shape() != target.shape()) throw TensorError(RTB_ERR_SHAPE, "mean_l1_loss needs equal shapes");
    TensorBase<T> a = input.is_contiguous() ? input : input.contiguous();
    TensorBase<T> b = target.is_contiguous() ? target : target.contiguous();
    TensorBase<T> out{input.backend, input.backend->template alloc<T>(1), MetaTensor::contiguous({})};
    check(rtb_l1_loss(input.backend->ctx(), DTypeOf<T>::value, a.buf->ptr + a.meta.offset, b.buf->ptr + b.meta.offset, a.size(), 0,
                      out.buf->ptr, nullptr));
    return out;
}

}  // namespace rtb200
