/*
 * Index-remapping expressions: the value at (row, column) of the result is the value of a
 * source expression at remapped coordinates.  None of them computes anything; all of them are
 * pure data movement and evaluate bit-exactly.
 *
 *   reshape(src, shape)            same elements, another shape          (l-value: no)
 *   slice<dim>(src, begin, end)    a range of one dimension              (l-value: yes)
 *   concat<dim>(a, b)              a followed by b along one dimension   (l-value: yes)
 *   swapaxis<a1, a2>(src)          two dimensions exchanged, a2 < a1
 *   transpose(src, axes)           any permutation of the dimensions
 *   pad(src, y[, x])               zero border around the last two dimensions
 *   crop(src, shape[, y0, x0])     a window of the last two dimensions (centred by default)
 *   mirror(src)                    last dimension reversed
 *   flip(src, dim)                 one dimension reversed                (l-value: yes)
 *
 * Names, factory signatures, result shapes and checks follow dmlc/mshadow's
 * mshadow/extension/{reshape,slice,concat,swapaxis,transpose,pad,crop,mirror,flip}.h.  What
 * differs is how a plan finds its source coordinates:
 *   - every division or remainder by a launch-constant extent is a multiplication by a
 *     precomputed reciprocal (FastDiv) instead of an integer divide per element;
 *   - where the remapping keeps 16-byte groups of the last dimension together (reshape between
 *     aligned widths, slices and concatenations on an aligned boundary, swaps and permutations
 *     that leave the last dimension in place, aligned crops, mirror) the plan also serves
 *     EvalPack, so that expressions containing it stay on the 128-bit kernel.  The run-time half
 *     of that decision is in PackAlign;
 *   - `dst = transpose(tensor, axes)` and `dst = swapaxis<last, a>(tensor)` on dense fp32/any-type
 *     GPU tensors, when the permutation moves the last axis, run in a dedicated kernel that turns
 *     64 x 64 tiles round in shared memory (gpu/transpose.cuh) instead of reading the source with a
 *     large stride.
 */
#ifndef MSHADOW_EXTENSION_REMAP_H_
#define MSHADOW_EXTENSION_REMAP_H_

#include <algorithm>

#include "../engine/check.h"
#include "../engine/fastdiv.h"
#if MSHADOW_USE_CUDA && defined(__CUDACC__)
#include <type_traits>

#include "../gpu/transpose.cuh"
#endif

namespace mshadow {
namespace expr {

namespace remapdetail {
/*! \brief FastDiv is exact for 31-bit numbers: every linear index of the result has to fit */
template <int dim>
inline void CheckIndexRange(const Shape<dim> &shape, const char *what) {
  uint64_t n = 1;
  for (int i = 0; i < dim; ++i) n *= shape[i];
  CHECK_LT(n, (uint64_t(1) << 31)) << what << ": tensor too large for 32-bit indexing";
}
}  // namespace remapdetail

// ------------------------------------------------------------------------------------------
// reshape (dmlc/mshadow: mshadow/extension/reshape.h:15-84)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dimdst, int dimsrc>
struct ReshapeExp : public MakeTensorExp<ReshapeExp<SrcExp, DType, dimdst, dimsrc>, SrcExp, dimdst, DType> {
  const SrcExp &src_;
  index_t ishapex_;  // last extent of the source
  ReshapeExp(const SrcExp &src, Shape<dimdst> shape) : src_(src) {
    const Shape<dimsrc> ishape = ShapeCheck<dimsrc, SrcExp>::Check(src_);
    CHECK_EQ(ishape.Size(), shape.Size()) << "reshape size must match";
    remapdetail::CheckIndexRange(shape, "reshape");
    ishapex_ = ishape[dimsrc - 1];
    this->shape_ = shape;
  }
};

template <typename SrcExp, typename DType, int etype, int dimdst>
inline ReshapeExp<SrcExp, DType, dimdst, ExpInfo<SrcExp>::kDim> reshape(const Exp<SrcExp, DType, etype> &src,
                                                                        Shape<dimdst> oshape) {
  return ReshapeExp<SrcExp, DType, dimdst, ExpInfo<SrcExp>::kDim>(src.self(), oshape);
}

template <typename SrcExp, typename DType, int dimdst, int dimsrc>
class Plan<ReshapeExp<SrcExp, DType, dimdst, dimsrc>, DType> {
 public:
  explicit Plan(const ReshapeExp<SrcExp, DType, dimdst, dimsrc> &e)
      : src_(MakePlan(e.src_)), oshapex_(e.shape_[dimdst - 1]), by_ishapex_(e.ishapex_) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    uint32_t row;
    const uint32_t col = by_ishapex_.DivMod(y * oshapex_ + x, &row);
    return src_.Eval(row, col);
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    uint32_t row;
    const uint32_t col = by_ishapex_.DivMod(y * oshapex_ + x, &row);
    return src_.EvalPack(row, col);
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const index_t oshapex_;
  const FastDiv by_ishapex_;
};

template <typename SrcExp, typename DType, int dimdst, int dimsrc>
struct PackInfo<ReshapeExp<SrcExp, DType, dimdst, dimsrc> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimdst, int dimsrc>
struct PackAlign<ReshapeExp<SrcExp, DType, dimdst, dimsrc> > {
  inline static bool Check(const ReshapeExp<SrcExp, DType, dimdst, dimsrc> &e) {
    // groups of the result must coincide with groups of the source
    const index_t lanes = Pack<DType>::kLanes;
    return e.shape_[dimdst - 1] % lanes == 0 && e.ishapex_ % lanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// slice (dmlc/mshadow: mshadow/extension/slice.h:15-153); usable on the left of an assignment
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct SliceExp : public TRValue<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice>, Device, srcdim, DType> {
  static const int dimslice = srcdim - dimsrc_m_slice;
  const SrcExp &src_;
  index_t ch_begin_;
  index_t ch_old_;
  Shape<srcdim> shape_;
  SliceExp(const SrcExp &src, index_t begin, index_t end) : src_(src), ch_begin_(begin) {
    shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    ch_old_ = shape_[dimslice];
    CHECK(begin < shape_[dimslice] && end <= shape_[dimslice]) << "The slice went out of range";
    remapdetail::CheckIndexRange(shape_, "slice");
    shape_[dimslice] = end - begin;
  }
  template <typename E, int etype>
  inline void operator=(const expr::Exp<E, DType, etype> &exp) {
    this->__assign(exp);
  }
  inline void operator=(const DType &exp) { this->__assign(exp); }
};

template <int sdim, typename SrcExp, typename Device, typename DType, int srcdim>
inline SliceExp<SrcExp, Device, DType, srcdim, srcdim - sdim> slice(const TRValue<SrcExp, Device, srcdim, DType> &src,
                                                                    index_t begin, index_t end) {
  TypeCheckPass<sdim < srcdim && ExpInfo<SrcExp>::kDim == srcdim>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return SliceExp<SrcExp, Device, DType, srcdim, srcdim - sdim>(src.self(), begin, end);
}

template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct ShapeCheck<srcdim, SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > {
  inline static Shape<srcdim> Check(const SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> &t) {
    return t.shape_;
  }
};
template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct StreamInfo<Device, SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > {
  inline static Stream<Device> *Get(const SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> &t) {
    return StreamInfo<Device, SrcExp>::Get(t.src_);
  }
};
template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct ExpInfo<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > {
  static const int kDim = ExpInfo<SrcExp>::kDim;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask;
};

template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
class Plan<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice>, DType> {
 public:
  static const int dimslice = srcdim - dimsrc_m_slice;
  static const bool kLast = dimsrc_m_slice == 1;  // the sliced dimension is the last one
  explicit Plan(const SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> &e)
      : src_(MakePlan(e.src_)), by_height_(kLast ? 1 : e.shape_.ProdShape(dimslice + 1, srcdim - 1)),
        by_ch_(e.shape_[dimslice]), ch_begin_(e.ch_begin_), ch_old_(e.ch_old_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    return kLast ? src_.Eval(i, j + ch_begin_) : src_.Eval(SrcRow(i), j);
  }
  MSHADOW_XINLINE DType &REval(index_t i, index_t j) {
    return kLast ? src_.REval(i, j + ch_begin_) : src_.REval(SrcRow(i), j);
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    return kLast ? src_.EvalPack(i, j + ch_begin_) : src_.EvalPack(SrcRow(i), j);
  }
  __device__ __forceinline__ void StorePack(index_t i, index_t j, const Pack<DType> &v) {
    if (kLast) src_.StorePack(i, j + ch_begin_, v);
    else src_.StorePack(SrcRow(i), j, v);
  }
#endif

 private:
  /*! \brief row (b, c, y) of the slice is row (b, c + begin, y) of the source */
  MSHADOW_XINLINE index_t SrcRow(index_t i) const {
    uint32_t t, b;
    const uint32_t y = by_height_.DivMod(i, &t);
    const uint32_t c = by_ch_.DivMod(t, &b);
    return (b * ch_old_ + c + ch_begin_) * by_height_.div + y;
  }
  Plan<SrcExp, DType> src_;
  const FastDiv by_height_, by_ch_;
  const index_t ch_begin_, ch_old_;
};

template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct PackInfo<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct PackAlign<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > {
  inline static bool Check(const SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> &e) {
    const bool boundary_ok = dimsrc_m_slice != 1 || e.ch_begin_ % Pack<DType>::kLanes == 0;
    return boundary_ok && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// concat (dmlc/mshadow: mshadow/extension/concat.h:15-191); usable on the left of an assignment
// ------------------------------------------------------------------------------------------
template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct ConcatExp
    : public TRValue<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat>, Device, srcdim, DType> {
  static const int dimcat = srcdim - dimsrc_m_cat;
  const LhsExp &src1_;
  const RhsExp &src2_;
  index_t dcat_src1_;
  index_t dcat_src2_;
  Shape<srcdim> shape_;
  ConcatExp(const LhsExp &src1, const RhsExp &src2) : src1_(src1), src2_(src2) {
    const Shape<srcdim> sshape1 = ShapeCheck<srcdim, LhsExp>::Check(src1_);
    const Shape<srcdim> sshape2 = ShapeCheck<srcdim, RhsExp>::Check(src2_);
    for (int i = 0; i < srcdim; ++i) {
      if (i != dimcat) CHECK_EQ(sshape1[i], sshape2[i]) << "ConcatExp: shape mismatch";
    }
    shape_ = sshape1;
    shape_[dimcat] = sshape1[dimcat] + sshape2[dimcat];
    dcat_src1_ = sshape1[dimcat];
    dcat_src2_ = sshape2[dimcat];
    remapdetail::CheckIndexRange(shape_, "concat");
  }
  template <typename E, int etype>
  inline void operator=(const expr::Exp<E, DType, etype> &exp) {
    this->__assign(exp);
  }
  inline void operator=(const DType &exp) { this->__assign(exp); }
};

template <int cdim, typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim>
inline ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, srcdim - cdim> concat(
    const TRValue<LhsExp, Device, srcdim, DType> &src1, const TRValue<RhsExp, Device, srcdim, DType> &src2) {
  TypeCheckPass<ExpInfo<LhsExp>::kDim == ExpInfo<RhsExp>::kDim>::Error_Expression_Does_Not_Meet_Dimension_Req();
  TypeCheckPass<cdim < srcdim && ExpInfo<LhsExp>::kDim == srcdim>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, srcdim - cdim>(src1.self(), src2.self());
}

template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct ShapeCheck<srcdim, ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  inline static Shape<srcdim> Check(const ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> &t) {
    return t.shape_;
  }
};
template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct StreamInfo<Device, ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  inline static Stream<Device> *Get(const ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> &t) {
    Stream<Device> *lhs = StreamInfo<Device, LhsExp>::Get(t.src1_);
    Stream<Device> *rhs = StreamInfo<Device, RhsExp>::Get(t.src2_);
    return lhs != rhs ? NULL : lhs;  // operands on different streams: no stream to order the write on
  }
};
template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct ExpInfo<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  static const int kDim = checkdetail::JoinDim(ExpInfo<LhsExp>::kDim, ExpInfo<RhsExp>::kDim);
  static const int kDevMask = ExpInfo<LhsExp>::kDevMask & ExpInfo<RhsExp>::kDevMask;
};

template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
class Plan<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat>, DType> {
 public:
  static const int dimcat = srcdim - dimsrc_m_cat;
  static const bool kLast = dimsrc_m_cat == 1;  // joined along the last dimension
  explicit Plan(const ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> &e)
      : src1_(MakePlan(e.src1_)), src2_(MakePlan(e.src2_)),
        by_height_(kLast ? 1 : e.shape_.ProdShape(dimcat + 1, srcdim - 1)), by_ch_(e.shape_[dimcat]),
        ch_src1_(e.dcat_src1_), ch_src2_(e.dcat_src2_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    if (kLast) return j < ch_src1_ ? src1_.Eval(i, j) : src2_.Eval(i, j - ch_src1_);
    bool first;
    const index_t row = SrcRow(i, &first);
    return first ? src1_.Eval(row, j) : src2_.Eval(row, j);
  }
  MSHADOW_XINLINE DType &REval(index_t i, index_t j) {
    if (kLast) return j < ch_src1_ ? src1_.REval(i, j) : src2_.REval(i, j - ch_src1_);
    bool first;
    const index_t row = SrcRow(i, &first);
    return first ? src1_.REval(row, j) : src2_.REval(row, j);
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    if (kLast) return j < ch_src1_ ? src1_.EvalPack(i, j) : src2_.EvalPack(i, j - ch_src1_);
    bool first;
    const index_t row = SrcRow(i, &first);
    return first ? src1_.EvalPack(row, j) : src2_.EvalPack(row, j);
  }
  __device__ __forceinline__ void StorePack(index_t i, index_t j, const Pack<DType> &v) {
    if (kLast) {
      if (j < ch_src1_) src1_.StorePack(i, j, v);
      else src2_.StorePack(i, j - ch_src1_, v);
      return;
    }
    bool first;
    const index_t row = SrcRow(i, &first);
    if (first) src1_.StorePack(row, j, v);
    else src2_.StorePack(row, j, v);
  }
#endif

 private:
  /*! \brief row (b, c, y) of the result lives in the first operand while c < its extent */
  MSHADOW_XINLINE index_t SrcRow(index_t i, bool *first) const {
    uint32_t t, b;
    const uint32_t y = by_height_.DivMod(i, &t);
    const uint32_t c = by_ch_.DivMod(t, &b);
    *first = c < ch_src1_;
    return *first ? (b * ch_src1_ + c) * by_height_.div + y : (b * ch_src2_ + c - ch_src1_) * by_height_.div + y;
  }
  Plan<LhsExp, DType> src1_;
  Plan<RhsExp, DType> src2_;
  const FastDiv by_height_, by_ch_;
  const index_t ch_src1_, ch_src2_;
};

template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct PackInfo<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  static const bool kPass = PackInfo<LhsExp>::kPass && PackInfo<RhsExp>::kPass;
};
template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct PackAlign<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  inline static bool Check(const ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> &e) {
    const bool boundary_ok = dimsrc_m_cat != 1 || e.dcat_src1_ % Pack<DType>::kLanes == 0;
    return boundary_ok && PackAlign<LhsExp>::Check(e.src1_) && PackAlign<RhsExp>::Check(e.src2_);
  }
};

// ------------------------------------------------------------------------------------------
// swapaxis<a1, a2>, a2 < a1 (dmlc/mshadow: mshadow/extension/swapaxis.h:15-107)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dimsrc, int m_a1, int a2>
struct SwapAxisExp : public MakeTensorExp<SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2>, SrcExp, dimsrc, DType> {
  static const int a1 = dimsrc - m_a1;
  const SrcExp &src_;
  explicit SwapAxisExp(const SrcExp &src) : src_(src) {
    this->shape_ = ShapeCheck<dimsrc, SrcExp>::Check(src);
    remapdetail::CheckIndexRange(this->shape_, "swapaxis");
    std::swap(this->shape_[a1], this->shape_[a2]);
  }
};

template <int a1, int a2, typename SrcExp, typename DType, int etype>
inline SwapAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim - a1, a2> swapaxis(
    const Exp<SrcExp, DType, etype> &src) {
  typedef ExpInfo<SrcExp> Info;
  TypeCheckPass<Info::kDim >= a1 + 1 && Info::kDim >= a2 + 1 && a2 < a1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return SwapAxisExp<SrcExp, DType, ExpInfo<SrcExp>::kDim, ExpInfo<SrcExp>::kDim - a1, a2>(src.self());
}

/*!
 * \brief result coordinates (.., n, c.., z, y.., x) with n on axis a2 and z on axis a1 read the
 *  source at (.., z, c.., n, y.., x).  When a1 is the last axis there is no trailing (y.., x)
 *  part and the column itself is swapped with n.
 */
template <typename SrcExp, typename DType, int dimsrc, int m_a1, int a2>
class Plan<SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2>, DType> {
 public:
  static const int a1 = dimsrc - m_a1;
  static const bool kLast = m_a1 == 1;  // the last axis takes part in the swap
  explicit Plan(const SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2> &e)
      : src_(MakePlan(e.src_)), by_y_(kLast ? 1 : e.shape_.ProdShape(a1 + 1, dimsrc - 1)),
        by_z_(kLast ? 1 : e.shape_[a1]), by_c_(e.shape_.ProdShape(a2 + 1, kLast ? dimsrc - 1 : a1)),
        by_n_(e.shape_[a2]), shapex_(e.shape_[dimsrc - 1]) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    if (kLast) {
      uint32_t t, outer;
      const uint32_t c = by_c_.DivMod(i, &t);
      const uint32_t n = by_n_.DivMod(t, &outer);
      return src_.Eval((outer * shapex_ + j) * by_c_.div + c, n);
    }
    return src_.Eval(SrcRow(i), j);
  }
#ifdef __CUDACC__
  /*! \brief only reached when the last axis stays in place (PackInfo is false otherwise) */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const { return src_.EvalPack(SrcRow(i), j); }
#endif

 private:
  MSHADOW_XINLINE index_t SrcRow(index_t i) const {
    uint32_t t1, t2, t3, outer;
    const uint32_t y = by_y_.DivMod(i, &t1);
    const uint32_t z = by_z_.DivMod(t1, &t2);
    const uint32_t c = by_c_.DivMod(t2, &t3);
    const uint32_t n = by_n_.DivMod(t3, &outer);
    return (((outer * by_z_.div + z) * by_c_.div + c) * by_n_.div + n) * by_y_.div + y;
  }
  Plan<SrcExp, DType> src_;
  const FastDiv by_y_, by_z_, by_c_, by_n_;
  const index_t shapex_;
};

template <typename SrcExp, typename DType, int dimsrc, int m_a1, int a2>
struct PackInfo<SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2> > {
  static const bool kPass = m_a1 != 1 && PackInfo<SrcExp>::kPass;
};
template <typename SrcExp, typename DType, int dimsrc, int m_a1, int a2>
struct PackAlign<SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2> > {
  inline static bool Check(const SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2> &e) {
    return PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// transpose(src, axes): result axis k is source axis axes[k]
// (dmlc/mshadow: mshadow/extension/transpose.h:15-92)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dimsrc>
struct TransposeExExp : public MakeTensorExp<TransposeExExp<SrcExp, DType, dimsrc>, SrcExp, dimsrc, DType> {
  const SrcExp &src_;
  const Shape<dimsrc> axes_;
  Shape<dimsrc> dst_in_src_stride_;  // for every result axis, the distance of its steps in the dense source
  index_t src_stride_;               // last extent of the source
  TransposeExExp(const SrcExp &src, Shape<dimsrc> axes) : src_(src), axes_(axes) {
    const Shape<dimsrc> src_shape = ShapeCheck<dimsrc, SrcExp>::Check(src);
    remapdetail::CheckIndexRange(src_shape, "transpose");
    src_stride_ = src_shape[dimsrc - 1];
    Shape<dimsrc> src_stride;
    src_stride[dimsrc - 1] = 1;
    for (int i = dimsrc - 2; i >= 0; --i) src_stride[i] = src_shape[i + 1] * src_stride[i + 1];
    bool seen[dimsrc] = {};
    for (int i = 0; i < dimsrc; ++i) {
      CHECK_LT(axes[i], static_cast<index_t>(dimsrc)) << "transpose: axes must be a permutation, got " << axes;
      seen[axes[i]] = true;
      dst_in_src_stride_[i] = src_stride[axes[i]];
      this->shape_[i] = src_shape[axes[i]];
    }
    for (int i = 0; i < dimsrc; ++i) CHECK(seen[i]) << "transpose: axes must be a permutation, got " << axes;
  }
};

template <typename SrcExp, typename DType, int etype>
inline TransposeExExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> transpose(const Exp<SrcExp, DType, etype> &src,
                                                                      Shape<ExpInfo<SrcExp>::kDim> axes) {
  return TransposeExExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), axes);
}

template <typename SrcExp, typename DType, int dimsrc>
class Plan<TransposeExExp<SrcExp, DType, dimsrc>, DType> {
 public:
  explicit Plan(const TransposeExExp<SrcExp, DType, dimsrc> &e)
      : src_(MakePlan(e.src_)), by_src_stride_(e.src_stride_), dst_in_src_stride_(e.dst_in_src_stride_) {
    for (int k = 0; k < dimsrc; ++k) by_extent_[k] = FastDiv(e.shape_[k]);
  }
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t row;
    const uint32_t col = by_src_stride_.DivMod(SrcOffset(i, j), &row);
    return src_.Eval(row, col);
  }
#ifdef __CUDACC__
  /*! \brief only reached when the last axis stays in place (see PackAlign) */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    uint32_t row;
    const uint32_t col = by_src_stride_.DivMod(SrcOffset(i, j), &row);
    return src_.EvalPack(row, col);
  }
#endif

 private:
  /*! \brief offset of result element (i, j) in the dense source */
  MSHADOW_XINLINE index_t SrcOffset(index_t i, index_t j) const {
    index_t idx = j * dst_in_src_stride_[dimsrc - 1];
#pragma unroll
    for (int k = dimsrc - 2; k >= 0; --k) {
      uint32_t q;
      idx += by_extent_[k].DivMod(i, &q) * dst_in_src_stride_[k];
      i = q;
    }
    return idx;
  }
  Plan<SrcExp, DType> src_;
  const FastDiv by_src_stride_;
  FastDiv by_extent_[dimsrc];
  const Shape<dimsrc> dst_in_src_stride_;
};

template <typename SrcExp, typename DType, int dimsrc>
struct PackInfo<TransposeExExp<SrcExp, DType, dimsrc> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimsrc>
struct PackAlign<TransposeExExp<SrcExp, DType, dimsrc> > {
  inline static bool Check(const TransposeExExp<SrcExp, DType, dimsrc> &e) {
    // groups of the last axis survive only a permutation of the other axes
    return e.axes_[dimsrc - 1] == static_cast<index_t>(dimsrc - 1) &&
           e.src_stride_ % Pack<DType>::kLanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// pad (dmlc/mshadow: mshadow/extension/pad.h:15-108): zeros around the last two dimensions
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int srcdim>
struct PaddingExp : public MakeTensorExp<PaddingExp<SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  index_t pad_y_, pad_x_, src_height_, src_width_;
  PaddingExp(const SrcExp &src, index_t pad_y, index_t pad_x) : src_(src), pad_y_(pad_y), pad_x_(pad_x) {
    this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    src_height_ = this->shape_[srcdim - 2];
    src_width_ = this->shape_[srcdim - 1];
    this->shape_[srcdim - 2] += pad_y * 2;
    this->shape_[srcdim - 1] += pad_x * 2;
    remapdetail::CheckIndexRange(this->shape_, "pad");
  }
};

template <typename SrcExp, typename DType, int etype>
inline PaddingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> pad(const Exp<SrcExp, DType, etype> &src, index_t pad_y,
                                                            index_t pad_x) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return PaddingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), pad_y, pad_x);
}
template <typename SrcExp, typename DType, int etype>
inline PaddingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> pad(const Exp<SrcExp, DType, etype> &src, index_t pad) {
  return mshadow::expr::pad(src, pad, pad);
}

template <typename SrcExp, typename DType, int srcdim>
class Plan<PaddingExp<SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const PaddingExp<SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), pad_y_(e.pad_y_), pad_x_(e.pad_x_), by_new_height_(e.shape_[srcdim - 2]),
        src_height_(e.src_height_), src_width_(e.src_width_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t c;
    const uint32_t y = by_new_height_.DivMod(i, &c);
    // in unsigned arithmetic "above / left of the image" wraps to a huge value: one comparison per axis
    const uint32_t h = y - static_cast<uint32_t>(pad_y_), w = static_cast<uint32_t>(j) - static_cast<uint32_t>(pad_x_);
    return (h < static_cast<uint32_t>(src_height_) && w < static_cast<uint32_t>(src_width_))
               ? src_.Eval(c * src_height_ + h, w)
               : static_cast<DType>(0);
  }

 private:
  Plan<SrcExp, DType> src_;
  const index_t pad_y_, pad_x_;
  const FastDiv by_new_height_;
  const index_t src_height_, src_width_;
};

// ------------------------------------------------------------------------------------------
// crop (dmlc/mshadow: mshadow/extension/crop.h:15-116): a window of the last two dimensions
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int srcdim>
struct CroppingExp : public MakeTensorExp<CroppingExp<SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  index_t pad_height_, pad_width_, src_height_;
  /*! \brief centred window */
  CroppingExp(const SrcExp &src, Shape<2> cshape) : src_(src) {
    this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    CHECK_GE(this->shape_[srcdim - 2], cshape[0]) << "CroppingExp: height requirement not met";
    CHECK_GE(this->shape_[srcdim - 1], cshape[1]) << "CroppingExp: width requirement not met";
    remapdetail::CheckIndexRange(this->shape_, "crop");
    pad_height_ = (this->shape_[srcdim - 2] - cshape[0]) / 2;
    pad_width_ = (this->shape_[srcdim - 1] - cshape[1]) / 2;
    src_height_ = this->shape_[srcdim - 2];
    this->shape_[srcdim - 2] = cshape[0];
    this->shape_[srcdim - 1] = cshape[1];
  }
  /*! \brief window starting at (start_height, start_width) */
  CroppingExp(const SrcExp &src, Shape<2> cshape, index_t start_height, index_t start_width)
      : src_(src), pad_height_(start_height), pad_width_(start_width) {
    this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    CHECK_GE(this->shape_[srcdim - 2], cshape[0] + start_height) << "CroppingExp: height requirement not met";
    CHECK_GE(this->shape_[srcdim - 1], cshape[1] + start_width) << "CroppingExp: width requirement not met";
    remapdetail::CheckIndexRange(this->shape_, "crop");
    src_height_ = this->shape_[srcdim - 2];
    this->shape_[srcdim - 2] = cshape[0];
    this->shape_[srcdim - 1] = cshape[1];
  }
};

template <typename SrcExp, typename DType, int etype>
inline CroppingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> crop(const Exp<SrcExp, DType, etype> &src, Shape<2> oshape) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return CroppingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), oshape);
}
template <typename SrcExp, typename DType, int etype>
inline CroppingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> crop(const Exp<SrcExp, DType, etype> &src, Shape<2> oshape,
                                                              index_t start_height, index_t start_width) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return CroppingExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), oshape, start_height, start_width);
}

template <typename SrcExp, typename DType, int srcdim>
class Plan<CroppingExp<SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const CroppingExp<SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), pad_height_(e.pad_height_), pad_width_(e.pad_width_),
        by_new_height_(e.shape_[srcdim - 2]), src_height_(e.src_height_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const { return src_.Eval(SrcRow(i), j + pad_width_); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    return src_.EvalPack(SrcRow(i), j + pad_width_);
  }
#endif

 private:
  MSHADOW_XINLINE index_t SrcRow(index_t i) const {
    uint32_t c;
    const uint32_t y = by_new_height_.DivMod(i, &c);
    return c * src_height_ + y + pad_height_;
  }
  Plan<SrcExp, DType> src_;
  const index_t pad_height_, pad_width_;
  const FastDiv by_new_height_;
  const index_t src_height_;
};

template <typename SrcExp, typename DType, int srcdim>
struct PackInfo<CroppingExp<SrcExp, DType, srcdim> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int srcdim>
struct PackAlign<CroppingExp<SrcExp, DType, srcdim> > {
  inline static bool Check(const CroppingExp<SrcExp, DType, srcdim> &e) {
    return e.pad_width_ % Pack<DType>::kLanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// mirror (dmlc/mshadow: mshadow/extension/mirror.h:15-59): last dimension reversed
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int srcdim>
struct MirroringExp : public MakeTensorExp<MirroringExp<SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  explicit MirroringExp(const SrcExp &src) : src_(src) { this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_); }
};

template <typename SrcExp, typename DType, int etype>
inline MirroringExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> mirror(const Exp<SrcExp, DType, etype> &src) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return MirroringExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self());
}

template <typename SrcExp, typename DType, int srcdim>
class Plan<MirroringExp<SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const MirroringExp<SrcExp, DType, srcdim> &e) : src_(MakePlan(e.src_)), width_(e.shape_[srcdim - 1]) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const { return src_.Eval(i, width_ - j - 1); }
#ifdef __CUDACC__
  /*! \brief the group at column j is the source group ending at width - j, lanes reversed */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    constexpr int kLanes = Pack<DType>::kLanes;
    const Pack<DType> s = src_.EvalPack(i, width_ - j - kLanes);
    Pack<DType> r;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) r.v[l] = s.v[kLanes - 1 - l];
    return r;
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const index_t width_;
};

template <typename SrcExp, typename DType, int srcdim>
struct PackInfo<MirroringExp<SrcExp, DType, srcdim> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int srcdim>
struct PackAlign<MirroringExp<SrcExp, DType, srcdim> > {
  inline static bool Check(const MirroringExp<SrcExp, DType, srcdim> &e) {
    return e.shape_[srcdim - 1] % Pack<DType>::kLanes == 0 && PackAlign<SrcExp>::Check(e.src_);
  }
};

// ------------------------------------------------------------------------------------------
// flip (dmlc/mshadow: mshadow/extension/flip.h:15-129): one dimension reversed; an l-value
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct FlipExp : public TRValue<FlipExp<SrcExp, Device, DType, srcdim>, Device, srcdim, DType> {
  const SrcExp &src_;
  index_t trailing_;  // elements per step of the flipped dimension
  index_t stride_;    // extent of the flipped dimension
  index_t stride_j_;  // last extent
  Shape<srcdim> shape_;
  FlipExp(const SrcExp &src, int dim) : src_(src) {
    shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    CHECK(dim >= 0 && dim < srcdim) << "flip: dimension out of range";
    remapdetail::CheckIndexRange(shape_, "flip");
    stride_ = shape_[dim];
    stride_j_ = shape_[srcdim - 1];
    trailing_ = 1;
    for (int i = dim + 1; i < srcdim; ++i) trailing_ *= shape_[i];
  }
  template <typename E, int etype>
  inline void operator=(const expr::Exp<E, DType, etype> &exp) {
    this->__assign(exp);
  }
  inline void operator=(const DType &exp) { this->__assign(exp); }
};

template <typename SrcExp, typename Device, typename DType, int srcdim>
inline FlipExp<SrcExp, Device, DType, srcdim> flip(const TRValue<SrcExp, Device, srcdim, DType> &src, int dim) {
  return FlipExp<SrcExp, Device, DType, srcdim>(src.self(), dim);
}

template <typename SrcExp, typename Device, typename DType, int srcdim>
struct ShapeCheck<srcdim, FlipExp<SrcExp, Device, DType, srcdim> > {
  inline static Shape<srcdim> Check(const FlipExp<SrcExp, Device, DType, srcdim> &t) { return t.shape_; }
};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct StreamInfo<Device, FlipExp<SrcExp, Device, DType, srcdim> > {
  inline static Stream<Device> *Get(const FlipExp<SrcExp, Device, DType, srcdim> &t) {
    return StreamInfo<Device, SrcExp>::Get(t.src_);
  }
};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct ExpInfo<FlipExp<SrcExp, Device, DType, srcdim> > {
  static const int kDim = ExpInfo<SrcExp>::kDim;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask;
};

template <typename SrcExp, typename Device, typename DType, int srcdim>
class Plan<FlipExp<SrcExp, Device, DType, srcdim>, DType> {
 public:
  explicit Plan(const FlipExp<SrcExp, Device, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), by_stride_j_(e.stride_j_), by_trailing_(e.trailing_), by_stride_(e.stride_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t row;
    const uint32_t col = by_stride_j_.DivMod(SrcOffset(i, j), &row);
    return src_.Eval(row, col);
  }
  MSHADOW_XINLINE DType &REval(index_t i, index_t j) {
    uint32_t row;
    const uint32_t col = by_stride_j_.DivMod(SrcOffset(i, j), &row);
    return src_.REval(row, col);
  }

 private:
  /*! \brief linear offset (high, x, low) -> (high, extent - 1 - x, low) */
  MSHADOW_XINLINE index_t SrcOffset(index_t i, index_t j) const {
    uint32_t t, high;
    const uint32_t low = by_trailing_.DivMod(i * by_stride_j_.div + j, &t);
    const uint32_t x = by_stride_.DivMod(t, &high);
    return (high * by_stride_.div + by_stride_.div - 1 - x) * by_trailing_.div + low;
  }
  Plan<SrcExp, DType> src_;
  const FastDiv by_stride_j_, by_trailing_, by_stride_;
};

// every plan of this file is pure index arithmetic around its source's Eval
template <typename SrcExp, typename DType, int dimdst, int dimsrc>
struct LaneInfo<ReshapeExp<SrcExp, DType, dimdst, dimsrc> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename Device, typename DType, int srcdim, int dimsrc_m_slice>
struct LaneInfo<SliceExp<SrcExp, Device, DType, srcdim, dimsrc_m_slice> > : public LaneInfo<SrcExp> {};
template <typename LhsExp, typename RhsExp, typename Device, typename DType, int srcdim, int dimsrc_m_cat>
struct LaneInfo<ConcatExp<LhsExp, RhsExp, Device, DType, srcdim, dimsrc_m_cat> > {
  static const bool kPass = LaneInfo<LhsExp>::kPass && LaneInfo<RhsExp>::kPass;
};
template <typename SrcExp, typename DType, int dimsrc, int m_a1, int a2>
struct LaneInfo<SwapAxisExp<SrcExp, DType, dimsrc, m_a1, a2> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimsrc>
struct LaneInfo<TransposeExExp<SrcExp, DType, dimsrc> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int srcdim>
struct LaneInfo<PaddingExp<SrcExp, DType, srcdim> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int srcdim>
struct LaneInfo<CroppingExp<SrcExp, DType, srcdim> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename DType, int srcdim>
struct LaneInfo<MirroringExp<SrcExp, DType, srcdim> > : public LaneInfo<SrcExp> {};
template <typename SrcExp, typename Device, typename DType, int srcdim>
struct LaneInfo<FlipExp<SrcExp, Device, DType, srcdim> > : public LaneInfo<SrcExp> {};

}  // namespace expr

#if MSHADOW_USE_CUDA && defined(__CUDACC__)
namespace cuda {

namespace remapdetail {
/*! \brief tiled kernel when tensors are dense and have at most five dimensions, else the generic route */
template <typename DType, int dim, typename E>
inline void PermuteOrGeneric(Tensor<gpu, dim, DType> *dst, const E &e, const Tensor<gpu, dim, DType> &src,
                             const Shape<dim> &axes, Shape<dim> dshape, cudaStream_t stream, std::true_type) {
  if (src.CheckContiguous() && dst->CheckContiguous() && dst->dptr_ != src.dptr_ &&
      TiledPermuteLaunch<DType, dim>(dst->dptr_, src.dptr_, src.shape_, axes, stream)) {
    return;
  }
  MapGeneric<sv::saveto, DType>(dst, e, dshape, stream);
}
template <typename DType, int dim, typename E>
inline void PermuteOrGeneric(Tensor<gpu, dim, DType> *dst, const E &e, const Tensor<gpu, dim, DType> &,
                             const Shape<dim> &, Shape<dim> dshape, cudaStream_t stream, std::false_type) {
  MapGeneric<sv::saveto, DType>(dst, e, dshape, stream);
}
}  // namespace remapdetail

// `dst = transpose(tensor, axes)`: permutations that move the last axis go through shared-memory tiles
template <typename DType, int dim>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, DType>, expr::TransposeExExp<Tensor<gpu, dim, DType>, DType, dim>, DType,
                   dim> {
  typedef expr::TransposeExExp<Tensor<gpu, dim, DType>, DType, dim> E;
  inline static void Run(Tensor<gpu, dim, DType> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    if (e.axes_[dim - 1] != static_cast<index_t>(dim - 1)) {
      remapdetail::PermuteOrGeneric<DType, dim>(dst, e, e.src_, e.axes_, dshape, stream,
                                                std::integral_constant<bool, (dim >= 2 && dim <= 5)>());
    } else {
      MapGeneric<sv::saveto, DType>(dst, e, dshape, stream);
    }
  }
};

// `dst = swapaxis<last, a2>(tensor)`
template <typename DType, int dim, int a2>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, DType>, expr::SwapAxisExp<Tensor<gpu, dim, DType>, DType, dim, 1, a2>,
                   DType, dim> {
  typedef expr::SwapAxisExp<Tensor<gpu, dim, DType>, DType, dim, 1, a2> E;
  inline static void Run(Tensor<gpu, dim, DType> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    Shape<dim> axes;
    for (int k = 0; k < dim; ++k) axes[k] = k;
    axes[dim - 1] = a2;
    axes[a2] = dim - 1;
    remapdetail::PermuteOrGeneric<DType, dim>(dst, e, e.src_, axes, dshape, stream,
                                              std::integral_constant<bool, (dim >= 2 && dim <= 5)>());
  }
};

}  // namespace cuda
#endif  // MSHADOW_USE_CUDA && __CUDACC__

}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_REMAP_H_
