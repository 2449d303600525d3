/*
 * Expressions that pick rows or elements by an index vector, and nearest-neighbour upsampling:
 *
 *   take(index, weight)                    out(y, x) = weight(index[y], x)      (embedding look-up, the
 *                                                                                forward of AddTakeGrad)
 *   take_grad(index, grad, input_dim)      out(r, x) = sum over i with index[i] == r of grad(i, x)
 *   one_hot_encode(index, num_choices)     out(y, x) = (x == index[y])
 *   mat_choose_row_element(mat, index)     out(y)    = mat(y, index[y])
 *   mat_fill_row_element(mat, val, index)  out(y, x) = x == index[y] ? val[y] : mat(y, x)
 *   mask(rowmask, mat)                     out(y, x) = mat(y, x) * rowmask[y]
 *   upsampling_nearest(src, scale)         out(.., y, x) = src(.., y / scale, x / scale)
 *
 * Names, signatures, shapes and checks follow dmlc/mshadow's mshadow/extension/{take, take_grad,
 * one_hot, choose, fill, mask, spatial_upsampling_nearest}.h; index vectors hold integers stored
 * in the element type, as there.  take and mask keep 16-byte groups of the last dimension
 * together, so they also serve EvalPack and expressions built on them stay on the 128-bit kernel.
 */
#ifndef MSHADOW_EXTENSION_SELECT_H_
#define MSHADOW_EXTENSION_SELECT_H_

#include "../engine/check.h"
#include "../engine/fastdiv.h"

namespace mshadow {
namespace expr {

// ------------------------------------------------------------------------------------------
// take (dmlc/mshadow: mshadow/extension/take.h:15-96)
// ------------------------------------------------------------------------------------------
template <typename IndexExp, typename SrcExp, typename DType>
struct TakeExp : public Exp<TakeExp<IndexExp, SrcExp, DType>, DType, type::kChainer> {
  const IndexExp &index_;
  const SrcExp &src_;
  TakeExp(const IndexExp &index, const SrcExp &src) : index_(index), src_(src) {}
};

template <typename IndexExp, typename SrcExp, typename DType, int e1, int e2>
inline TakeExp<IndexExp, SrcExp, DType> take(const Exp<IndexExp, DType, e1> &index, const Exp<SrcExp, DType, e2> &src) {
  return TakeExp<IndexExp, SrcExp, DType>(index.self(), src.self());
}

template <typename IndexExp, typename SrcExp, typename DType>
class Plan<TakeExp<IndexExp, SrcExp, DType>, DType> {
 public:
  explicit Plan(const TakeExp<IndexExp, SrcExp, DType> &e) : index_(MakePlan(e.index_)), src_(MakePlan(e.src_)) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return static_cast<DType>(src_.Eval(static_cast<index_t>(index_.Eval(0, y)), x));
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    return src_.EvalPack(static_cast<index_t>(index_.Eval(0, y)), x);
  }
#endif

 private:
  Plan<IndexExp, DType> index_;
  Plan<SrcExp, DType> src_;
};

template <typename IndexExp, typename SrcExp, typename DType>
inline Plan<TakeExp<IndexExp, SrcExp, DType>, DType> MakePlan(const TakeExp<IndexExp, SrcExp, DType> &exp) {
  return Plan<TakeExp<IndexExp, SrcExp, DType>, DType>(exp);
}
template <int dim, typename IndexExp, typename SrcExp, typename DType>
struct ShapeCheck<dim, TakeExp<IndexExp, SrcExp, DType> > {
  inline static Shape<dim> Check(const TakeExp<IndexExp, SrcExp, DType> &t) {
    CHECK(dim == 2) << "TakeExp only support 2D output";
    const Shape<1> dshape = ShapeCheck<1, IndexExp>::Check(t.index_);
    const Shape<2> wshape = ShapeCheck<2, SrcExp>::Check(t.src_);
    Shape<dim> ret;
    ret[0] = dshape[0];
    ret[1] = wshape[1];
    return ret;
  }
};
template <typename IndexExp, typename SrcExp, typename DType>
struct ExpInfo<TakeExp<IndexExp, SrcExp, DType> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<IndexExp>::kDevMask;
};
template <typename IndexExp, typename SrcExp, typename DType>
struct PackInfo<TakeExp<IndexExp, SrcExp, DType> > : public PackInfo<SrcExp> {};
template <typename IndexExp, typename SrcExp, typename DType>
struct PackAlign<TakeExp<IndexExp, SrcExp, DType> > {
  inline static bool Check(const TakeExp<IndexExp, SrcExp, DType> &e) { return PackAlign<SrcExp>::Check(e.src_); }
};

// ------------------------------------------------------------------------------------------
// take_grad (dmlc/mshadow: mshadow/extension/take_grad.h:15-108): the expression form of the
// embedding gradient; every output element walks the whole batch, in batch order
// ------------------------------------------------------------------------------------------
template <typename IndexExp, typename SrcExp, typename DType>
struct TakeGradExp : public Exp<TakeGradExp<IndexExp, SrcExp, DType>, DType, type::kChainer> {
  const IndexExp &index_;
  const SrcExp &src_;
  const index_t input_dim_;
  TakeGradExp(const IndexExp &index, const SrcExp &src, const index_t input_dim)
      : index_(index), src_(src), input_dim_(input_dim) {}
};

template <typename IndexExp, typename SrcExp, typename DType, int e1, int e2>
inline TakeGradExp<IndexExp, SrcExp, DType> take_grad(const Exp<IndexExp, DType, e1> &index,
                                                      const Exp<SrcExp, DType, e2> &src, const index_t input_dim) {
  return TakeGradExp<IndexExp, SrcExp, DType>(index.self(), src.self(), input_dim);
}

template <typename IndexExp, typename SrcExp, typename DType>
class Plan<TakeGradExp<IndexExp, SrcExp, DType>, DType> {
 public:
  explicit Plan(const TakeGradExp<IndexExp, SrcExp, DType> &e)
      : index_(MakePlan(e.index_)), src_(MakePlan(e.src_)), batch_size_(ShapeCheck<1, IndexExp>::Check(e.index_)[0]) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    DType ret = 0.f;
    for (index_t i = 0; i < batch_size_; ++i) {
      if (static_cast<index_t>(index_.Eval(0, i)) == y) ret = detail::AddRN<DType>(ret, static_cast<DType>(src_.Eval(i, x)));
    }
    return ret;
  }

 private:
  Plan<IndexExp, DType> index_;
  Plan<SrcExp, DType> src_;
  const index_t batch_size_;
};

template <typename IndexExp, typename SrcExp, typename DType>
inline Plan<TakeGradExp<IndexExp, SrcExp, DType>, DType> MakePlan(const TakeGradExp<IndexExp, SrcExp, DType> &exp) {
  return Plan<TakeGradExp<IndexExp, SrcExp, DType>, DType>(exp);
}
template <int dim, typename IndexExp, typename SrcExp, typename DType>
struct ShapeCheck<dim, TakeGradExp<IndexExp, SrcExp, DType> > {
  inline static Shape<dim> Check(const TakeGradExp<IndexExp, SrcExp, DType> &t) {
    CHECK(dim == 2) << "TakeGradExp only support 2D output";
    const Shape<2> gshape = ShapeCheck<2, SrcExp>::Check(t.src_);
    Shape<dim> ret;
    ret[0] = t.input_dim_;
    ret[1] = gshape[1];
    return ret;
  }
};
template <typename IndexExp, typename SrcExp, typename DType>
struct ExpInfo<TakeGradExp<IndexExp, SrcExp, DType> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<IndexExp>::kDevMask;
};

// ------------------------------------------------------------------------------------------
// one_hot_encode (dmlc/mshadow: mshadow/extension/one_hot.h:15-85)
// ------------------------------------------------------------------------------------------
template <typename IndexExp, typename DType>
struct OneHotEncodeExp : public Exp<OneHotEncodeExp<IndexExp, DType>, DType, type::kChainer> {
  const IndexExp &index_;
  index_t num_choices_;
  OneHotEncodeExp(const IndexExp &index, index_t num_choices) : index_(index), num_choices_(num_choices) {}
};

template <typename IndexExp, typename IDType, int e1>
inline OneHotEncodeExp<IndexExp, default_real_t> one_hot_encode(const Exp<IndexExp, IDType, e1> &index,
                                                                index_t num_choices) {
  TypeCheckPass<ExpInfo<IndexExp>::kDim == 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return OneHotEncodeExp<IndexExp, default_real_t>(index.self(), num_choices);
}

template <typename IndexExp, typename DType>
class Plan<OneHotEncodeExp<IndexExp, DType>, DType> {
 public:
  explicit Plan(const OneHotEncodeExp<IndexExp, DType> &e) : index_(MakePlan(e.index_)) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return static_cast<DType>(x == static_cast<index_t>(index_.Eval(0, y)));
  }

 private:
  Plan<IndexExp, DType> index_;
};

template <typename IndexExp, typename DType>
inline Plan<OneHotEncodeExp<IndexExp, DType>, DType> MakePlan(const OneHotEncodeExp<IndexExp, DType> &exp) {
  return Plan<OneHotEncodeExp<IndexExp, DType>, DType>(exp);
}
template <int dim, typename IndexExp, typename DType>
struct ShapeCheck<dim, OneHotEncodeExp<IndexExp, DType> > {
  inline static Shape<dim> Check(const OneHotEncodeExp<IndexExp, DType> &t) {
    CHECK(dim == 2) << "OneHotEncodeExp only support 2 dimension output";
    const Shape<1> shape = ShapeCheck<1, IndexExp>::Check(t.index_);
    Shape<dim> ret;
    ret[0] = shape[0];
    ret[1] = t.num_choices_;
    return ret;
  }
};
template <typename IndexExp, typename DType>
struct ExpInfo<OneHotEncodeExp<IndexExp, DType> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<IndexExp>::kDevMask;
};

// ------------------------------------------------------------------------------------------
// mat_choose_row_element (dmlc/mshadow: mshadow/extension/choose.h:15-88)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename IndexExp, typename DType>
struct MatChooseRowElementExp : public Exp<MatChooseRowElementExp<SrcExp, IndexExp, DType>, DType, type::kChainer> {
  const SrcExp &src_;
  const IndexExp &index_;
  MatChooseRowElementExp(const SrcExp &src, const IndexExp &index) : src_(src), index_(index) {}
};

template <typename SrcExp, typename IndexExp, typename DType, typename IDType, int e1, int e2>
inline MatChooseRowElementExp<SrcExp, IndexExp, DType> mat_choose_row_element(const Exp<SrcExp, DType, e1> &src,
                                                                              const Exp<IndexExp, IDType, e2> &index) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim == 2 && ExpInfo<IndexExp>::kDim == 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return MatChooseRowElementExp<SrcExp, IndexExp, DType>(src.self(), index.self());
}

/*! \brief the result is a vector, evaluated as a single row: column x picks from matrix row x */
template <typename SrcExp, typename IndexExp, typename DType>
class Plan<MatChooseRowElementExp<SrcExp, IndexExp, DType>, DType> {
 public:
  explicit Plan(const MatChooseRowElementExp<SrcExp, IndexExp, DType> &e)
      : src_(MakePlan(e.src_)), index_(MakePlan(e.index_)) {}
  MSHADOW_XINLINE DType Eval(index_t, index_t x) const {
    return src_.Eval(x, static_cast<index_t>(index_.Eval(0, x)));
  }

 private:
  Plan<SrcExp, DType> src_;
  Plan<IndexExp, DType> index_;
};

template <typename SrcExp, typename IndexExp, typename DType>
inline Plan<MatChooseRowElementExp<SrcExp, IndexExp, DType>, DType> MakePlan(
    const MatChooseRowElementExp<SrcExp, IndexExp, DType> &exp) {
  return Plan<MatChooseRowElementExp<SrcExp, IndexExp, DType>, DType>(exp);
}
template <int dim, typename SrcExp, typename IndexExp, typename DType>
struct ShapeCheck<dim, MatChooseRowElementExp<SrcExp, IndexExp, DType> > {
  inline static Shape<dim> Check(const MatChooseRowElementExp<SrcExp, IndexExp, DType> &t) {
    CHECK(dim == 1) << "MatChooseRowElementExp only support 1 dimension output";
    const Shape<2> shape1 = ShapeCheck<2, SrcExp>::Check(t.src_);
    const Shape<dim> shape2 = ShapeCheck<dim, IndexExp>::Check(t.index_);
    CHECK_EQ(shape1[0], shape2[0]) << "mat_choose_row_element index length and number of rows in matrix";
    return shape2;
  }
};
template <typename SrcExp, typename IndexExp, typename DType>
struct ExpInfo<MatChooseRowElementExp<SrcExp, IndexExp, DType> > {
  static const int kDim = 1;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask & ExpInfo<IndexExp>::kDevMask;
};

// ------------------------------------------------------------------------------------------
// mat_fill_row_element (dmlc/mshadow: mshadow/extension/fill.h:15-101)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename ValExp, typename IndexExp, typename DType>
struct MatFillRowElementExp
    : public Exp<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType>, DType, type::kChainer> {
  const SrcExp &src_;
  const ValExp &val_;
  const IndexExp &index_;
  MatFillRowElementExp(const SrcExp &src, const ValExp &val, const IndexExp &index)
      : src_(src), val_(val), index_(index) {}
};

template <typename SrcExp, typename ValExp, typename IndexExp, typename SDType, typename VDType, typename IDType, int e1,
          int e2, int e3>
inline MatFillRowElementExp<SrcExp, ValExp, IndexExp, SDType> mat_fill_row_element(const Exp<SrcExp, SDType, e1> &src,
                                                                                  const Exp<ValExp, VDType, e2> &val,
                                                                                  const Exp<IndexExp, IDType, e3> &index) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim == 2 && ExpInfo<ValExp>::kDim == 1 &&
                ExpInfo<IndexExp>::kDim == 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return MatFillRowElementExp<SrcExp, ValExp, IndexExp, SDType>(src.self(), val.self(), index.self());
}

template <typename SrcExp, typename ValExp, typename IndexExp, typename DType>
class Plan<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType>, DType> {
 public:
  explicit Plan(const MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> &e)
      : src_(MakePlan(e.src_)), val_(MakePlan(e.val_)), index_(MakePlan(e.index_)) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return static_cast<index_t>(index_.Eval(0, y)) == x ? static_cast<DType>(val_.Eval(0, y))
                                                        : static_cast<DType>(src_.Eval(y, x));
  }

 private:
  Plan<SrcExp, DType> src_;
  Plan<ValExp, DType> val_;
  Plan<IndexExp, DType> index_;
};

template <typename SrcExp, typename ValExp, typename IndexExp, typename DType>
inline Plan<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType>, DType> MakePlan(
    const MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> &exp) {
  return Plan<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType>, DType>(exp);
}
template <int dim, typename SrcExp, typename ValExp, typename IndexExp, typename DType>
struct ShapeCheck<dim, MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> > {
  inline static Shape<dim> Check(const MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> &t) {
    CHECK(dim == 2) << "MatFillRowElementExp only support 2 dimension output";
    const Shape<2> shape_src = ShapeCheck<2, SrcExp>::Check(t.src_);
    const Shape<1> shape_val = ShapeCheck<1, ValExp>::Check(t.val_);
    const Shape<1> shape_index = ShapeCheck<1, IndexExp>::Check(t.index_);
    CHECK((shape_src[0] == shape_index[0]) && (shape_index[0] == shape_val[0]))
        << "mat_fill_row_element index length, val length and number of rows in matrix";
    Shape<dim> ret;
    ret[0] = shape_src[0];
    ret[1] = shape_src[1];
    return ret;
  }
};
template <typename SrcExp, typename ValExp, typename IndexExp, typename DType>
struct ExpInfo<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask & ExpInfo<ValExp>::kDevMask & ExpInfo<IndexExp>::kDevMask;
};

// ------------------------------------------------------------------------------------------
// mask (dmlc/mshadow: mshadow/extension/mask.h:15-95): every row scaled by its entry of a vector
// ------------------------------------------------------------------------------------------
template <typename IndexExp, typename SrcExp, typename DType>
struct MaskExp : public Exp<MaskExp<IndexExp, SrcExp, DType>, DType, type::kChainer> {
  const IndexExp &index_;
  const SrcExp &src_;
  MaskExp(const IndexExp &index, const SrcExp &src) : index_(index), src_(src) {}
};

template <typename IndexExp, typename SrcExp, typename DType, int e1, int e2>
inline MaskExp<IndexExp, SrcExp, DType> mask(const Exp<IndexExp, DType, e1> &index, const Exp<SrcExp, DType, e2> &src) {
  return MaskExp<IndexExp, SrcExp, DType>(index.self(), src.self());
}

template <typename IndexExp, typename SrcExp, typename DType>
class Plan<MaskExp<IndexExp, SrcExp, DType>, DType> {
 public:
  explicit Plan(const MaskExp<IndexExp, SrcExp, DType> &e) : index_(MakePlan(e.index_)), src_(MakePlan(e.src_)) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return static_cast<DType>(detail::MulRN<DType>(src_.Eval(y, x), index_.Eval(0, y)));
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    Pack<DType> r = src_.EvalPack(y, x);
    const DType m = index_.Eval(0, y);
#pragma unroll
    for (int l = 0; l < Pack<DType>::kLanes; ++l) r.v[l] = detail::MulRN<DType>(r.v[l], m);
    return r;
  }
#endif

 private:
  Plan<IndexExp, DType> index_;
  Plan<SrcExp, DType> src_;
};

template <typename IndexExp, typename SrcExp, typename DType>
inline Plan<MaskExp<IndexExp, SrcExp, DType>, DType> MakePlan(const MaskExp<IndexExp, SrcExp, DType> &exp) {
  return Plan<MaskExp<IndexExp, SrcExp, DType>, DType>(exp);
}
template <int dim, typename IndexExp, typename SrcExp, typename DType>
struct ShapeCheck<dim, MaskExp<IndexExp, SrcExp, DType> > {
  inline static Shape<dim> Check(const MaskExp<IndexExp, SrcExp, DType> &t) {
    CHECK(dim == 2) << "MaskExp only support 2D output";
    const Shape<1> dshape = ShapeCheck<1, IndexExp>::Check(t.index_);
    const Shape<2> wshape = ShapeCheck<2, SrcExp>::Check(t.src_);
    CHECK_EQ(dshape[0], wshape[0]) << "MaskExp require inputs in same first dimention";
    Shape<dim> ret;
    ret[0] = wshape[0];
    ret[1] = wshape[1];
    return ret;
  }
};
template <typename IndexExp, typename SrcExp, typename DType>
struct ExpInfo<MaskExp<IndexExp, SrcExp, DType> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<IndexExp>::kDevMask;
};
template <typename IndexExp, typename SrcExp, typename DType>
struct PackInfo<MaskExp<IndexExp, SrcExp, DType> > : public PackInfo<SrcExp> {};
template <typename IndexExp, typename SrcExp, typename DType>
struct PackAlign<MaskExp<IndexExp, SrcExp, DType> > {
  inline static bool Check(const MaskExp<IndexExp, SrcExp, DType> &e) { return PackAlign<SrcExp>::Check(e.src_); }
};

// ------------------------------------------------------------------------------------------
// upsampling_nearest (dmlc/mshadow: mshadow/extension/spatial_upsampling_nearest.h:15-68)
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int srcdim>
struct UpSamplingNearestExp : public MakeTensorExp<UpSamplingNearestExp<SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  index_t scale_;
  UpSamplingNearestExp(const SrcExp &src, index_t scale) : src_(src), scale_(scale) {
    CHECK_GE(scale, 1) << "upsampling_nearest: scale must be positive";
    this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    this->shape_[srcdim - 2] *= scale_;
    this->shape_[srcdim - 1] *= scale_;
  }
};

template <typename SrcExp, typename DType, int etype>
inline UpSamplingNearestExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> upsampling_nearest(const Exp<SrcExp, DType, etype> &src,
                                                                                     index_t scale) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return UpSamplingNearestExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), scale);
}

template <typename SrcExp, typename DType, int srcdim>
class Plan<UpSamplingNearestExp<SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const UpSamplingNearestExp<SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), by_scale_(e.scale_), by_new_height_(e.shape_[srcdim - 2]),
        src_height_(e.shape_[srcdim - 2] / e.scale_) {}
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t c;
    const uint32_t y = by_new_height_.DivMod(i, &c);
    return src_.Eval(c * src_height_ + by_scale_.Quot(y), by_scale_.Quot(j));
  }

 private:
  Plan<SrcExp, DType> src_;
  const FastDiv by_scale_, by_new_height_;
  const index_t src_height_;
};

// one or two look-ups per element; take_grad stays out (its Eval walks the whole batch)
template <typename IndexExp, typename SrcExp, typename DType>
struct LaneInfo<TakeExp<IndexExp, SrcExp, DType> > {
  static const bool kPass = LaneInfo<IndexExp>::kPass && LaneInfo<SrcExp>::kPass;
};
template <typename IndexExp, typename DType>
struct LaneInfo<OneHotEncodeExp<IndexExp, DType> > : public LaneInfo<IndexExp> {};
template <typename SrcExp, typename IndexExp, typename DType>
struct LaneInfo<MatChooseRowElementExp<SrcExp, IndexExp, DType> > {
  static const bool kPass = LaneInfo<IndexExp>::kPass && LaneInfo<SrcExp>::kPass;
};
template <typename SrcExp, typename ValExp, typename IndexExp, typename DType>
struct LaneInfo<MatFillRowElementExp<SrcExp, ValExp, IndexExp, DType> > {
  static const bool kPass = LaneInfo<IndexExp>::kPass && LaneInfo<SrcExp>::kPass && LaneInfo<ValExp>::kPass;
};
template <typename IndexExp, typename SrcExp, typename DType>
struct LaneInfo<MaskExp<IndexExp, SrcExp, DType> > {
  static const bool kPass = LaneInfo<IndexExp>::kPass && LaneInfo<SrcExp>::kPass;
};
template <typename SrcExp, typename DType, int srcdim>
struct LaneInfo<UpSamplingNearestExp<SrcExp, DType, srcdim> > : public LaneInfo<SrcExp> {};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_SELECT_H_
