/*
 * Reduction of an expression to a vector, keeping one dimension:
 *   sumall_except_dim<d>(e)          sum over every dimension but d
 *   reduce_except_dim<d, Reducer>(e) the same with any reducer
 *   sum_rows(m)                      column sums of a matrix (= sumall_except_dim<1>)
 * and `scale * reduction` / `reduction * scale`, which fold the factor into the reduction.
 * Interface as in dmlc/mshadow's mshadow/extension/reduceto1d.h (:22-101) and
 * mshadow/expr_scalar-inl.h (:36-47).  Keeping the last dimension routes to
 * MapReduceKeepLowest, keeping any other to MapReduceKeepHighDim.
 */
#ifndef MSHADOW_EXTENSION_REDUCETO1D_H_
#define MSHADOW_EXTENSION_REDUCETO1D_H_

#include "../engine/check.h"

namespace mshadow {
namespace expr {

/*! \tparam m_dimkeep dimension of the source minus the kept dimension (1 = keep the last) */
template <typename SrcExp, typename DType, typename Reducer, int m_dimkeep>
struct ReduceTo1DExp : public Exp<ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep>, DType, type::kComplex> {
  const SrcExp &src_;
  DType scale_;
  ReduceTo1DExp(const SrcExp &src, DType scale) : src_(src), scale_(scale) {}
};

template <int dimkeep, typename SrcExp, typename DType, int etype>
inline ReduceTo1DExp<SrcExp, DType, red::sum, ExpInfo<SrcExp>::kDim - dimkeep> sumall_except_dim(
    const Exp<SrcExp, DType, etype> &exp) {
  return ReduceTo1DExp<SrcExp, DType, red::sum, ExpInfo<SrcExp>::kDim - dimkeep>(exp.self(), DType(1));
}
template <int dimkeep, typename Reducer, typename SrcExp, typename DType, int etype>
inline ReduceTo1DExp<SrcExp, DType, Reducer, ExpInfo<SrcExp>::kDim - dimkeep> reduce_except_dim(
    const Exp<SrcExp, DType, etype> &exp) {
  return ReduceTo1DExp<SrcExp, DType, Reducer, ExpInfo<SrcExp>::kDim - dimkeep>(exp.self(), DType(1));
}
template <typename SrcExp, typename DType, int etype>
inline ReduceTo1DExp<SrcExp, DType, red::sum, 1> sum_rows(const Exp<SrcExp, DType, etype> &exp) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim == 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return sumall_except_dim<1>(exp);
}

template <typename SrcExp, typename DType, typename Reducer, int m_dimkeep>
inline ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep> operator*(
    const ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep> &e, typename exprdetail::NoDeduce<DType>::Type scale) {
  return ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep>(e.src_, e.scale_ * scale);
}
template <typename SrcExp, typename DType, typename Reducer, int m_dimkeep>
inline ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep> operator*(
    typename exprdetail::NoDeduce<DType>::Type scale, const ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep> &e) {
  return ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep>(e.src_, scale * e.scale_);
}

template <typename SV, typename Device, typename DType, typename SrcExp, typename Reducer, int m_dimkeep>
struct ExpComplexEngine<SV, Tensor<Device, 1, DType>, ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep>, DType> {
  static const int dimkeep = ExpInfo<SrcExp>::kDim - m_dimkeep;
  inline static void Eval(Tensor<Device, 1, DType> *dst, const ReduceTo1DExp<SrcExp, DType, Reducer, m_dimkeep> &exp) {
    TypeCheckPass<m_dimkeep != 1>::Error_Expression_Does_Not_Meet_Dimension_Req();
    MapReduceKeepHighDim<SV, Reducer, dimkeep>(dst, exp.src_, exp.scale_);
  }
};
template <typename SV, typename Device, typename DType, typename SrcExp, typename Reducer>
struct ExpComplexEngine<SV, Tensor<Device, 1, DType>, ReduceTo1DExp<SrcExp, DType, Reducer, 1>, DType> {
  inline static void Eval(Tensor<Device, 1, DType> *dst, const ReduceTo1DExp<SrcExp, DType, Reducer, 1> &exp) {
    MapReduceKeepLowest<SV, Reducer>(dst, exp.src_, exp.scale_);
  }
};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_REDUCETO1D_H_
