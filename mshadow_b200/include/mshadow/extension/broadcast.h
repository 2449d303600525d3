/*
 * Broadcasting a vector along one dimension of a higher-dimensional shape:
 *   broadcast<dimcast>(vec, shape)   value at (.., i_dimcast, ..) is vec[i_dimcast]
 *   repmat(vec, nrow)                = broadcast<1>(vec, Shape2(nrow, len)): every row is vec
 * Expression type, factory functions and plan semantics follow dmlc/mshadow's
 * mshadow/extension/broadcast.h (:24-148).  In addition the plans take part in the 128-bit
 * evaluation path: a last-dimension broadcast serves a 16-byte group with one aligned load
 * of the vector, any other broadcast with one scalar load replicated over the group.
 */
#ifndef MSHADOW_EXTENSION_BROADCAST_H_
#define MSHADOW_EXTENSION_BROADCAST_H_

#include "../engine/check.h"

namespace mshadow {
namespace expr {

/*!
 * \tparam dimdst dimension of the result
 * \tparam dimdst_m_cast dimdst minus the dimension that the vector runs along
 */
template <typename SrcExp, typename DType, int dimdst, int dimdst_m_cast>
struct Broadcast1DExp
    : public MakeTensorExp<Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast>, SrcExp, dimdst, DType> {
  const SrcExp &src_;
  Broadcast1DExp(const SrcExp &src, Shape<dimdst> shape) : src_(src) { this->shape_ = shape; }
};

template <int dimcast, typename SrcExp, typename DType, int etype, int dimdst>
inline Broadcast1DExp<SrcExp, DType, dimdst, dimdst - dimcast> broadcast(const Exp<SrcExp, DType, etype> &src,
                                                                         Shape<dimdst> shape) {
  TypeCheckPass<dimcast < dimdst && ExpInfo<SrcExp>::kDim == 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  typedef ShapeCheck<1, SrcExp> ShapeCheckDim1SrcExp;
  CHECK_EQ(ShapeCheckDim1SrcExp::Check(src.self())[0], shape[dimcast]) << "broadcast, shape mismatch";
  return Broadcast1DExp<SrcExp, DType, dimdst, dimdst - dimcast>(src.self(), shape);
}

template <typename SrcExp, typename DType, int etype>
inline Broadcast1DExp<SrcExp, DType, 2, 1> repmat(const Exp<SrcExp, DType, etype> &src, index_t nrow) {
  return broadcast<1>(src, Shape2(nrow, ShapeCheck<1, SrcExp>::Check(src.self())[0]));
}

/*! \brief the vector runs along a dimension other than the last: one value per row */
template <typename SrcExp, typename DType, int dimdst, int dimdst_m_cast>
class Plan<Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast>, DType> {
 public:
  static const int dimcast = dimdst - dimdst_m_cast;
  explicit Plan(const Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast> &e)
      : src_(MakePlan(e.src_)), ystride_(e.shape_.ProdShape(dimcast + 1, dimdst - 1)), length_(e.shape_[dimcast]) {
    TypeCheckPass<dimcast != dimdst - 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
  }
  MSHADOW_XINLINE DType Eval(index_t y, index_t) const { return src_.Eval(0, (y / ystride_) % length_); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t) const {
    const DType v = src_.Eval(0, (y / ystride_) % length_);
    Pack<DType> r;
#pragma unroll
    for (int i = 0; i < Pack<DType>::kLanes; ++i) r.v[i] = v;
    return r;
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const index_t ystride_, length_;
};

/*! \brief the vector runs along the last dimension: column x of every row is vec[x] */
template <typename SrcExp, typename DType, int dimdst>
class Plan<Broadcast1DExp<SrcExp, DType, dimdst, 1>, DType> {
 public:
  explicit Plan(const Broadcast1DExp<SrcExp, DType, dimdst, 1> &e) : src_(MakePlan(e.src_)) {}
  MSHADOW_XINLINE DType Eval(index_t, index_t x) const { return src_.Eval(0, x); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t, index_t x) const { return src_.EvalPack(0, x); }
#endif

 private:
  Plan<SrcExp, DType> src_;
};

// Broadcasts keep an expression on the 128-bit path as long as their source is.  They are
// position-dependent, so they never take part in the single-long-row traversal (FlatInfo
// stays false).
template <typename SrcExp, typename DType, int dimdst, int dimdst_m_cast>
struct PackInfo<Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast> > : public PackInfo<SrcExp> {};
template <typename SrcExp, typename DType, int dimdst, int dimdst_m_cast>
struct PackAlign<Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast> > {
  inline static bool Check(const Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast> &e) {
    return PackAlign<SrcExp>::Check(e.src_);
  }
};
template <typename SrcExp, typename DType, int dimdst, int dimdst_m_cast>
struct LaneInfo<Broadcast1DExp<SrcExp, DType, dimdst, dimdst_m_cast> > : public LaneInfo<SrcExp> {};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_BROADCAST_H_
