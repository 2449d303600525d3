/*
 * Expressions that address a tensor by axis number or by a begin/end box:
 *
 *   range(start, stop, step, repeat)                    a generated vector
 *   slice(src, begin, end)                              a box of an n-d tensor (also an l-value)
 *   reduce_with_axis<Reducer, mask>(src, axis)          fold one axis away (or report the arg-index)
 *   reduce_keepdim<Reducer, mask>(src, axis)            the same, the axis stays with extent 1
 *   broadcast_with_axis(src, axis, size)                insert a repeated axis after `axis`
 *   broadcast_keepdim(src, axis, size)                  repeat an axis of extent 1
 *   broadcast_multi_axes(src, axes, sizes)              repeat several axes of extent 1
 *   broadcast_to(src, target_shape)                     the same, from the target shape
 *
 * Names, signatures, result shapes and the order in which a reduction visits its axis follow
 * dmlc/mshadow's mshadow/extension/range.h (:24-115), slice_ex.h (:20-132), reduce_with_axis.h
 * (:20-133) and broadcast_with_axis.h (:22-255).  The plans here split linear indices with
 * precomputed reciprocals, and the reductions walk their axis by stepping (row, column) of the
 * source instead of dividing at every element.
 */
#ifndef MSHADOW_EXTENSION_AXIS_H_
#define MSHADOW_EXTENSION_AXIS_H_

#include <cmath>
#include <vector>

#include "../engine/check.h"
#include "../engine/fastdiv.h"

namespace mshadow {
namespace expr {

// ------------------------------------------------------------------------------------------
// range
// ------------------------------------------------------------------------------------------
template <typename DType>
struct RangeExp : public Exp<RangeExp<DType>, DType, type::kMapper> {
  const DType start_, stop_, step_;
  const int repeat_;
  RangeExp(DType start, DType stop, DType step, int repeat)
      : start_(start), stop_(stop), step_(step), repeat_(repeat) {}
};

/*! \brief start, start + step, ... up to (not including) stop, every value `repeat` times */
template <typename DType>
inline RangeExp<DType> range(DType start, DType stop, DType step = 1, int repeat = 1) {
  return RangeExp<DType>(start, stop, step, repeat);
}

template <typename DType>
class Plan<RangeExp<DType>, DType> {
 public:
  explicit Plan(const RangeExp<DType> &e) : start_(e.start_), step_(e.step_), by_repeat_(e.repeat_) {}
  MSHADOW_XINLINE DType Eval(index_t, index_t x) const {
    return detail::AddRN<DType>(start_, detail::MulRN<DType>(static_cast<DType>(static_cast<int>(by_repeat_.Quot(x))), step_));
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    Pack<DType> r;
#pragma unroll
    for (int l = 0; l < Pack<DType>::kLanes; ++l) r.v[l] = Eval(y, x + l);
    return r;
  }
#endif

 private:
  const DType start_, step_;
  const FastDiv by_repeat_;
};

template <typename DType>
inline Plan<RangeExp<DType>, DType> MakePlan(const RangeExp<DType> &exp) {
  return Plan<RangeExp<DType>, DType>(exp);
}

/*! \brief number of elements range(start, stop, step, repeat) produces */
template <typename DType>
inline int RangeOutSize(DType start, DType stop, DType step, int repeat) {
  return repeat * ((stop - start - 1) / step + 1);
}
template <>
inline int RangeOutSize<float>(float start, float stop, float step, int repeat) {
  return repeat * static_cast<int>(
                      std::ceil((static_cast<double>(stop) - static_cast<double>(start)) / static_cast<double>(step)));
}
template <>
inline int RangeOutSize<double>(double start, double stop, double step, int repeat) {
  return repeat * static_cast<int>(std::ceil((stop - start) / step));
}

template <int dim, typename DType>
struct ShapeCheck<dim, RangeExp<DType> > {
  inline static Shape<dim> Check(const RangeExp<DType> &t) {
    CHECK(dim == 1) << "RangeExp only support 1 dimension output, received " << dim;
    CHECK(t.step_ != 0) << "RangeExp does not support step=0, received " << t.step_;
    CHECK(t.repeat_ > 0) << "RangeExp only supports repeat > 0, received " << t.repeat_;
    if (t.step_ > 0) {
      CHECK(t.start_ < t.stop_) << "RangeExp does not support (start, stop, step) = (" << t.start_ << "," << t.stop_
                                << "," << t.step_ << ")";
    } else {
      CHECK(t.start_ > t.stop_) << "RangeExp does not support (start, stop, step)= (" << t.start_ << "," << t.stop_
                                << "," << t.step_ << ")";
    }
    Shape<dim> s;
    s[0] = RangeOutSize<DType>(t.start_, t.stop_, t.step_, t.repeat_);
    return s;
  }
};
template <typename DType>
struct ExpInfo<RangeExp<DType> > {
  static const int kDim = 1;
  static const int kDevMask = 0xffff;
};
template <typename DType>
struct PackInfo<RangeExp<DType> > {
  static const bool kPass = true;
};
template <typename DType>
struct PackAlign<RangeExp<DType> > {
  inline static bool Check(const RangeExp<DType> &) { return true; }
};

// ------------------------------------------------------------------------------------------
// slice(src, begin, end): the box [begin, end) of an n-d tensor; usable on the left of an assignment
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct SliceExExp : public TRValue<SliceExExp<SrcExp, Device, DType, srcdim>, Device, srcdim, DType> {
  const SrcExp &src_;
  Shape<srcdim> src_shape_;
  Shape<srcdim> shape_;
  const Shape<srcdim> begin_;
  const Shape<srcdim> end_;
  SliceExExp(const SrcExp &src, Shape<srcdim> begin, Shape<srcdim> end) : src_(src), begin_(begin), end_(end) {
    src_shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    for (int i = 0; i < srcdim; ++i) {
      CHECK(begin_[i] <= end_[i] && end_[i] <= src_shape_[i]) << "The slice went out of range";
      shape_[i] = end_[i] - begin_[i];
    }
    CHECK_LT(static_cast<uint64_t>(src_shape_.Size()), uint64_t(1) << 31) << "slice: tensor too large for 32-bit indexing";
  }
  template <typename E, int etype>
  inline void operator=(const expr::Exp<E, DType, etype> &exp) {
    this->__assign(exp);
  }
  inline void operator=(const DType &exp) { this->__assign(exp); }
};

template <typename SrcExp, typename Device, typename DType, int srcdim>
inline SliceExExp<SrcExp, Device, DType, srcdim> slice(const TRValue<SrcExp, Device, srcdim, DType> &src,
                                                       Shape<srcdim> begin, Shape<srcdim> end) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim == srcdim>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return SliceExExp<SrcExp, Device, DType, srcdim>(src.self(), begin, end);
}

template <typename SrcExp, typename Device, typename DType, int srcdim>
struct ShapeCheck<srcdim, SliceExExp<SrcExp, Device, DType, srcdim> > {
  inline static Shape<srcdim> Check(const SliceExExp<SrcExp, Device, DType, srcdim> &t) { return t.shape_; }
};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct StreamInfo<Device, SliceExExp<SrcExp, Device, DType, srcdim> > {
  inline static Stream<Device> *Get(const SliceExExp<SrcExp, Device, DType, srcdim> &t) {
    return StreamInfo<Device, SrcExp>::Get(t.src_);
  }
};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct ExpInfo<SliceExExp<SrcExp, Device, DType, srcdim> > {
  static const int kDim = ExpInfo<SrcExp>::kDim;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask;
};

template <typename SrcExp, typename Device, typename DType, int srcdim>
class Plan<SliceExExp<SrcExp, Device, DType, srcdim>, DType> {
 public:
  explicit Plan(const SliceExExp<SrcExp, Device, DType, srcdim> &e) : src_(MakePlan(e.src_)), col_begin_(e.begin_[srcdim - 1]) {
    uint32_t stride = 1;
    row_begin_ = 0;
    for (int k = srcdim - 2; k >= 0; --k) {
      by_extent_[k] = FastDiv(e.shape_[k]);
      stride_[k] = stride;
      row_begin_ += stride * e.begin_[k];
      stride *= e.src_shape_[k];
    }
  }
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const { return src_.Eval(SrcRow(i), j + col_begin_); }
  MSHADOW_XINLINE DType &REval(index_t i, index_t j) { return src_.REval(SrcRow(i), j + col_begin_); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    return src_.EvalPack(SrcRow(i), j + col_begin_);
  }
  __device__ __forceinline__ void StorePack(index_t i, index_t j, const Pack<DType> &v) {
    src_.StorePack(SrcRow(i), j + col_begin_, v);
  }
#endif

 private:
  /*! \brief row of the source that holds row i of the box */
  MSHADOW_XINLINE index_t SrcRow(index_t i) const {
    uint32_t rest = i, row = row_begin_;
#pragma unroll
    for (int k = srcdim - 2; k >= 0; --k) {
      uint32_t q;
      row += stride_[k] * by_extent_[k].DivMod(rest, &q);
      rest = q;
    }
    return row;
  }
  Plan<SrcExp, DType> src_;
  FastDiv by_extent_[srcdim > 1 ? srcdim - 1 : 1];
  uint32_t stride_[srcdim > 1 ? srcdim - 1 : 1];
  uint32_t row_begin_;
  const index_t col_begin_;
};

template <typename SrcExp, typename Device, typename DType, int srcdim>
struct PackInfo<SliceExExp<SrcExp, Device, DType, srcdim> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct PackAlign<SliceExExp<SrcExp, Device, DType, srcdim> > {
  inline static bool Check(const SliceExExp<SrcExp, Device, DType, srcdim> &e) {
    return e.begin_[srcdim - 1] % Pack<DType>::kLanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// reduce_with_axis / reduce_keepdim
// ------------------------------------------------------------------------------------------
template <typename Reducer, typename SrcExp, typename DType, int dimsrc, bool mask, int dimdst>
struct ReduceWithAxisExp
    : public MakeTensorExp<ReduceWithAxisExp<Reducer, SrcExp, DType, dimsrc, mask, dimdst>, SrcExp, dimdst, DType> {
  const SrcExp &src_;
  index_t last_dst_dim_;  // extent of the result's last dimension
  index_t trailing_;      // product of the source extents behind the axis
  index_t size_;          // extent of the axis
  index_t last_;          // extent of the source's last dimension
  ReduceWithAxisExp(const SrcExp &src, int axis) : src_(src) {
    const bool keepdim = (dimsrc == dimdst);
    CHECK(dimsrc > axis && axis >= 0) << "reduce axis out of bound";
    const Shape<dimsrc> src_shape = ShapeCheck<dimsrc, SrcExp>::Check(src_);
    CHECK_LT(static_cast<uint64_t>(src_shape.Size()), uint64_t(1) << 31) << "reduce_with_axis: tensor too large for 32-bit indexing";
    for (int i = 0; i < axis; ++i) this->shape_[i] = src_shape[i];
    size_ = src_shape[axis];
    trailing_ = 1;
    if (!keepdim) {
      for (int i = axis + 1; i < dimsrc; ++i) {
        trailing_ *= src_shape[i];
        this->shape_[i - 1] = src_shape[i];
      }
    } else {
      this->shape_[axis] = 1;
      for (int i = axis + 1; i < dimsrc; ++i) {
        trailing_ *= src_shape[i];
        this->shape_[i] = src_shape[i];
      }
    }
    last_ = src_shape[dimsrc - 1];
    last_dst_dim_ = this->shape_[dimdst - 1];
  }
};

/*! \brief fold `axis` away; with mask the result is the position along the axis that last changed the fold */
template <typename Reducer, bool mask, typename SrcExp, typename DType, int etype>
inline ReduceWithAxisExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim, mask, ExpInfo<SrcExp>::kDim - 1> reduce_with_axis(
    const Exp<SrcExp, DType, etype> &src, int axis) {
  return ReduceWithAxisExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim, mask, ExpInfo<SrcExp>::kDim - 1>(src.self(), axis);
}
template <typename Reducer, bool mask, typename SrcExp, typename DType, int etype>
inline ReduceWithAxisExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim, mask, ExpInfo<SrcExp>::kDim> reduce_keepdim(
    const Exp<SrcExp, DType, etype> &src, int axis) {
  return ReduceWithAxisExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim, mask, ExpInfo<SrcExp>::kDim>(src.self(), axis);
}

template <typename Reducer, typename SrcExp, typename DType, int dimsrc, bool mask, int dimdst>
class Plan<ReduceWithAxisExp<Reducer, SrcExp, DType, dimsrc, mask, dimdst>, DType> {
 public:
  explicit Plan(const ReduceWithAxisExp<Reducer, SrcExp, DType, dimsrc, mask, dimdst> &e)
      : src_(MakePlan(e.src_)), last_dst_dim_(e.last_dst_dim_), size_(e.size_), by_trailing_(e.trailing_),
        by_last_(e.last_), row_step_(e.trailing_ / e.last_), col_step_(e.trailing_ % e.last_) {}
  /*!
   * \brief element number lin = (outer, inner) of the result folds source elements
   *  (outer * size + k) * trailing + inner for k = 0 .. size-1, in that order; consecutive k are
   *  `trailing` elements apart, which is a fixed (row, column) step of the source matrix
   */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t outer, row;
    const uint32_t inner = by_trailing_.DivMod(i * last_dst_dim_ + j, &outer);
    uint32_t col = by_last_.DivMod(outer * size_ * by_trailing_.div + inner, &row);
    DType res;
    Reducer::SetInitValue(res);
    uint32_t idx = 0;
    for (uint32_t k = 0; k < static_cast<uint32_t>(size_); ++k) {
      const DType before = res;
      Reducer::Reduce(res, src_.Eval(row, col));
      if (mask && before != res) idx = k;
      row += row_step_;
      col += col_step_;
      if (col >= by_last_.div) {
        col -= by_last_.div;
        ++row;
      }
    }
    return mask ? static_cast<DType>(static_cast<int>(idx)) : res;
  }

 private:
  Plan<SrcExp, DType> src_;
  const index_t last_dst_dim_, size_;
  const FastDiv by_trailing_, by_last_;
  const uint32_t row_step_, col_step_;
};

// ------------------------------------------------------------------------------------------
// broadcast_with_axis / broadcast_keepdim
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dimsrc, int dimdst>
struct BroadcastWithAxisExp
    : public MakeTensorExp<BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst>, SrcExp, dimdst, DType> {
  const SrcExp &src_;
  index_t dst_last_;  // extent of the result's last dimension
  index_t trailing_;  // product of the extents behind the repeated axis
  index_t size_;      // extent of the repeated axis
  index_t last_;      // extent of the source's last dimension
  BroadcastWithAxisExp(const SrcExp &src, const int axis, const index_t size) : src_(src), size_(size) {
    const bool keepdim = (dimsrc == dimdst);
    const Shape<dimsrc> src_shape = ShapeCheck<dimsrc, SrcExp>::Check(src_);
    trailing_ = 1;
    if (!keepdim) {
      CHECK(dimsrc > axis && axis >= -1) << "broadcast axis (no keepdim) out of bound, axis must be between -1 and"
                                         << dimsrc - 1 << ", given=" << axis << ".";
      for (int i = 0; i <= axis; ++i) this->shape_[i] = src_shape[i];
      this->shape_[axis + 1] = size_;
      for (int i = axis + 1; i < dimsrc; ++i) {
        trailing_ *= src_shape[i];
        this->shape_[i + 1] = src_shape[i];
      }
    } else {
      CHECK(dimdst > axis && axis >= 0) << "broadcast axis (keepdim) out of bound, axis must be between 0 and"
                                        << dimdst - 1 << ", given=" << axis << ".";
      CHECK_EQ(src_shape[axis], 1U) << "Size of the dimension of the broadcasting axis must be 1 when keepdim is on, "
                                    << "src_shape[" << axis << "]=" << src_shape[axis] << ".";
      for (int i = 0; i <= axis - 1; ++i) this->shape_[i] = src_shape[i];
      this->shape_[axis] = size_;
      for (int i = axis + 1; i < dimdst; ++i) {
        trailing_ *= src_shape[i];
        this->shape_[i] = src_shape[i];
      }
    }
    last_ = src_shape[dimsrc - 1];
    dst_last_ = this->shape_[dimdst - 1];
    CHECK_LT(static_cast<uint64_t>(this->shape_.Size()), uint64_t(1) << 31) << "broadcast_with_axis: result too large for 32-bit indexing";
  }
};

template <typename SrcExp, typename DType, int etype>
inline BroadcastWithAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim + 1> broadcast_with_axis(
    const Exp<SrcExp, DType, etype> &src, const int axis, const index_t size) {
  return BroadcastWithAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim + 1>(src.self(), axis, size);
}
template <typename SrcExp, typename DType, int etype>
inline BroadcastWithAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim> broadcast_keepdim(
    const Exp<SrcExp, DType, etype> &src, const int axis, const index_t size) {
  return BroadcastWithAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim>(src.self(), axis, size);
}

template <typename SrcExp, typename DType, int dimsrc, int dimdst>
class Plan<BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst>, DType> {
 public:
  explicit Plan(const BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst> &e)
      : src_(MakePlan(e.src_)), dst_last_(e.dst_last_), by_trailing_(e.trailing_), by_size_(e.size_), by_last_(e.last_) {}
  /*! \brief result element (outer, repeat, inner) is source element (outer, inner) */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t t, row;
    const uint32_t inner = by_trailing_.DivMod(i * dst_last_ + j, &t);
    const uint32_t col = by_last_.DivMod(by_size_.Quot(t) * by_trailing_.div + inner, &row);
    return src_.Eval(row, col);
  }
#ifdef __CUDACC__
  /*! \brief a group stays inside one (outer, repeat) block when every extent involved is a multiple of the group */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    uint32_t t, row;
    const uint32_t inner = by_trailing_.DivMod(i * dst_last_ + j, &t);
    const uint32_t col = by_last_.DivMod(by_size_.Quot(t) * by_trailing_.div + inner, &row);
    return src_.EvalPack(row, col);
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const index_t dst_last_;
  const FastDiv by_trailing_, by_size_, by_last_;
};

template <typename SrcExp, typename DType, int dimsrc, int dimdst>
struct PackInfo<BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimsrc, int dimdst>
struct PackAlign<BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst> > {
  inline static bool Check(const BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst> &e) {
    const index_t lanes = Pack<DType>::kLanes;
    return e.trailing_ % lanes == 0 && e.last_ % lanes == 0 && e.dst_last_ % lanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// broadcast_multi_axes / broadcast_to.  TShape is any type with ndim(), operator[] and a
// constructor from an iterator range (the callers' dynamic shape type).
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dimsrc>
struct BroadcastWithMultiAxesExp
    : public MakeTensorExp<BroadcastWithMultiAxesExp<SrcExp, DType, dimsrc>, SrcExp, dimsrc, DType> {
  const SrcExp &src_;
  index_t dst_last_;
  index_t axesnum_;
  Shape<dimsrc> trailings_;  // per repeated axis: product of the result's extents behind it
  Shape<dimsrc> sizes_;      // per repeated axis: its extent in the result
  index_t last_;
  template <typename TShape>
  BroadcastWithMultiAxesExp(const SrcExp &src, const TShape &axes, const TShape &sizes) : src_(src) {
    const Shape<dimsrc> src_shape = ShapeCheck<dimsrc, SrcExp>::Check(src_);
    CHECK(axes.ndim() == sizes.ndim()) << "ndim of axes and sizes must be equal.";
    axesnum_ = axes.ndim();
    CHECK(axesnum_ <= dimsrc) << "Number of broadcasting axes must be smaller than the source ndim, number of axes="
                              << axesnum_ << " dimsrc=" << dimsrc;
    for (index_t i = 0; i < axesnum_; i++) {
      CHECK(dimsrc > static_cast<int>(axes[i]) && static_cast<int>(axes[i]) >= 0)
          << "broadcast axis (keepdim) out of bound, all axes must be between 0 and" << dimsrc - 1 << ", given axes[" << i
          << "] = " << axes[i] << ".";
      CHECK_EQ(src_shape[axes[i]], 1U) << "Size of the dimension of the broadcasting axis must be 1, src_shape["
                                       << axes[i] << "]=" << src_shape[axes[i]] << ".";
      if (i < axesnum_ - 1) {
        CHECK(axes[i] < axes[i + 1]) << "The given axes must be in increasing order.";
      }
    }
    for (index_t i = 0; i < dimsrc; i++) {
      this->shape_[i] = src_shape[i];
      sizes_[i] = 1;
      trailings_[i] = 1;
    }
    for (index_t i = 0; i < axesnum_; i++) {
      this->shape_[axes[i]] = sizes[i];
      sizes_[i] = sizes[i];
    }
    for (index_t i = 0; i < axesnum_; i++) {
      trailings_[i] = 1;
      for (index_t j = axes[i] + 1; j < dimsrc; ++j) trailings_[i] *= this->shape_[j];
    }
    last_ = src_shape[dimsrc - 1];
    dst_last_ = this->shape_[dimsrc - 1];
    CHECK_LT(static_cast<uint64_t>(this->shape_.Size()), uint64_t(1) << 31) << "broadcast_multi_axes: result too large for 32-bit indexing";
  }
};

template <typename SrcExp, typename DType, int etype, typename TShape>
inline BroadcastWithMultiAxesExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> broadcast_multi_axes(
    const Exp<SrcExp, DType, etype> &src, const TShape &axes, const TShape &sizes) {
  return BroadcastWithMultiAxesExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), axes, sizes);
}

/*! \brief every dimension whose extent differs from the target's must have extent 1 in src */
template <typename SrcExp, typename DType, int etype, typename TShape>
inline BroadcastWithMultiAxesExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> broadcast_to(const Exp<SrcExp, DType, etype> &src,
                                                                                    const TShape &target_shape) {
  static const size_t dimsrc = ExpInfo<SrcExp>::kDim;
  CHECK_EQ(static_cast<size_t>(target_shape.ndim()), dimsrc);
  std::vector<index_t> axes_vec, sizes_vec;
  const Shape<dimsrc> src_shape = ShapeCheck<dimsrc, SrcExp>::Check(src.self());
  for (size_t i = 0; i < dimsrc; ++i) {
    if (src_shape[i] != static_cast<index_t>(target_shape[i])) {
      CHECK_EQ(src_shape[i], 1U) << "broadcasting axis must have size 1, received shape=" << src_shape;
      axes_vec.push_back(i);
      sizes_vec.push_back(target_shape[i]);
    }
  }
  const TShape axes = TShape(axes_vec.begin(), axes_vec.end());
  const TShape sizes = TShape(sizes_vec.begin(), sizes_vec.end());
  return BroadcastWithMultiAxesExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), axes, sizes);
}

template <typename SrcExp, typename DType, int dimsrc>
class Plan<BroadcastWithMultiAxesExp<SrcExp, DType, dimsrc>, DType> {
 public:
  explicit Plan(const BroadcastWithMultiAxesExp<SrcExp, DType, dimsrc> &e)
      : src_(MakePlan(e.src_)), dst_last_(e.dst_last_), axesnum_(e.axesnum_), by_last_(e.last_) {
    for (int p = 0; p < dimsrc; ++p) {
      by_trailing_[p] = FastDiv(e.trailings_[p]);
      by_size_[p] = FastDiv(e.sizes_[p]);
    }
  }
  /*! \brief the repeated axes are taken out of the linear index one after the other, first axis first */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t indx = i * dst_last_ + j;
#pragma unroll
    for (int p = 0; p < dimsrc; ++p) {
      if (p < static_cast<int>(axesnum_)) {
        uint32_t t;
        const uint32_t inner = by_trailing_[p].DivMod(indx, &t);
        indx = by_size_[p].Quot(t) * by_trailing_[p].div + inner;
      }
    }
    uint32_t row;
    const uint32_t col = by_last_.DivMod(indx, &row);
    return src_.Eval(row, col);
  }

 private:
  Plan<SrcExp, DType> src_;
  const index_t dst_last_, axesnum_;
  const FastDiv by_last_;
  FastDiv by_trailing_[dimsrc], by_size_[dimsrc];
};

// cheap per-element plans; the reductions stay out (their Eval walks a whole axis)
template <typename DType>
struct LaneInfo<RangeExp<DType> > {
  static const bool kPass = true;
};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct LaneInfo<SliceExExp<SrcExp, Device, DType, srcdim> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimsrc, int dimdst>
struct LaneInfo<BroadcastWithAxisExp<SrcExp, DType, dimsrc, dimdst> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimsrc>
struct LaneInfo<BroadcastWithMultiAxesExp<SrcExp, DType, dimsrc> > : public LaneInfo<SrcExp> {};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_AXIS_H_
