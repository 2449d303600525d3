/*
 * Compile-time and run-time checks that stand between an expression and a kernel launch:
 *   ExpInfo / TypeCheck   dimension and device inference (compile time)
 *   ShapeCheck            shape agreement (run time, CHECK on mismatch)
 *   StreamInfo            which stream an l-value evaluates on
 *   PackInfo / PackAlign  whether an expression may use the 128-bit path, and whether the
 *                         actual pointers and strides allow it for this call
 *   FlatInfo / FlatCheck  whether the whole evaluation may be treated as one long row
 *   ExpEngine             dispatch of `dst (op)= exp` to MapExp or to a complex engine
 * The first three and ExpEngine mirror dmlc/mshadow's mshadow/expr_engine-inl.h (:236-479),
 * whose names extension authors specialise; the Pack* and Flat* traits are specific to
 * this engine (their closest relative in the reference is the CPU-only PacketCheck /
 * PacketAlignCheck pair in mshadow/packet-inl.h:300-388).
 */
#ifndef MSHADOW_ENGINE_CHECK_H_
#define MSHADOW_ENGINE_CHECK_H_

#include "./plan.h"

namespace mshadow {
namespace expr {

// ----------------------------------------------------------------------------------------
// static inference of dimension (-1 = inconsistent) and of the devices an expression lives on
// ----------------------------------------------------------------------------------------
template <typename E>
struct ExpInfo {
  static const int kDim = -1;
  static const int kDevMask = 0;
};
template <typename DType>
struct ExpInfo<ScalarExp<DType> > {
  static const int kDim = 0;
  static const int kDevMask = 0xffff;
};
template <typename E, typename DType>
struct ExpInfo<TransposeExp<E, DType> > : public ExpInfo<E> {};
template <typename DstDType, typename SrcDType, typename EType, int etype>
struct ExpInfo<TypecastExp<DstDType, SrcDType, EType, etype> > : public ExpInfo<EType> {};
template <typename Device, int dim, typename DType>
struct ExpInfo<Tensor<Device, dim, DType> > {
  static const int kDim = dim;
  static const int kDevMask = Device::kDevMask;
};
template <typename T, typename SrcExp, int dim, typename DType>
struct ExpInfo<MakeTensorExp<T, SrcExp, dim, DType> > {
  static const int kDimSrc = ExpInfo<SrcExp>::kDim;
  static const int kDim = kDimSrc >= 0 ? dim : -1;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask;
};
template <typename OP, typename TA, typename DType, int etype>
struct ExpInfo<UnaryMapExp<OP, TA, DType, etype> > : public ExpInfo<TA> {};

namespace checkdetail {
/*! \brief dimension of a map over two operands; a 0-d (scalar) operand adapts to the other */
constexpr int JoinDim(int a, int b) {
  return (a < 0 || b < 0) ? -1 : (a == 0 ? b : ((b == 0 || a == b) ? a : -1));
}
}  // namespace checkdetail

template <typename OP, typename TA, typename TB, typename DType, int etype>
struct ExpInfo<BinaryMapExp<OP, TA, TB, DType, etype> > {
  static const int kDimLhs = ExpInfo<TA>::kDim;
  static const int kDimRhs = ExpInfo<TB>::kDim;
  static const int kDim = checkdetail::JoinDim(kDimLhs, kDimRhs);
  static const int kDevMask = ExpInfo<TA>::kDevMask & ExpInfo<TB>::kDevMask;
};
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct ExpInfo<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  static const int kDimItem1 = ExpInfo<TA>::kDim;
  static const int kDimItem2 = ExpInfo<TB>::kDim;
  static const int kDimItem3 = ExpInfo<TC>::kDim;
  static const int kDim = kDimItem1;
  static const int kDevMask =
      ExpInfo<TA>::kDevMask & ExpInfo<TB>::kDevMask & ExpInfo<TC>::kDevMask;
};

/*! \brief can expression E be assigned / reduced to a `dim`-d container on Device? */
template <typename Device, int dim, typename DType, typename E>
struct TypeCheck {
  static const int kExpDim = ExpInfo<E>::kDim;
  static const bool kDevPass = (ExpInfo<E>::kDevMask & Device::kDevMask) != 0;
  static const bool kMapPass = (kExpDim == 0 || kExpDim == dim) && kDevPass;
  static const bool kRedPass = (kExpDim > dim) && kDevPass;
};
/*! \brief a failed check names the missing member function in the compiler's message */
template <bool kPass>
struct TypeCheckPass;
template <>
struct TypeCheckPass<false> {};
template <>
struct TypeCheckPass<true> {
  inline static void Error_All_Tensor_in_Exp_Must_Have_Same_Type() {}
  inline static void Error_TypeCheck_Not_Pass_For_Reduce_Exp() {}
  inline static void Error_Expression_Does_Not_Meet_Dimension_Req() {}
};

// ----------------------------------------------------------------------------------------
// stream of an l-value
// ----------------------------------------------------------------------------------------
template <typename Device, typename E>
struct StreamInfo {
  inline static Stream<Device> *Get(const E &t);
};
template <int dim, typename Device, typename DType>
struct StreamInfo<Device, Tensor<Device, dim, DType> > {
  inline static Stream<Device> *Get(const Tensor<Device, dim, DType> &t) { return t.stream_; }
};

// ----------------------------------------------------------------------------------------
// run-time shape agreement; a scalar reports the all-zero shape, which matches anything
// ----------------------------------------------------------------------------------------
template <int dim, typename E>
struct ShapeCheck {
  inline static Shape<dim> Check(const E &t);
};
template <int dim, typename DType>
struct ShapeCheck<dim, ScalarExp<DType> > {
  inline static Shape<dim> Check(const ScalarExp<DType> &) {
    Shape<dim> s;
    for (int i = 0; i < dim; ++i) s[i] = 0;
    return s;
  }
};
template <int dim, typename DstDType, typename SrcDType, typename EType, int etype>
struct ShapeCheck<dim, TypecastExp<DstDType, SrcDType, EType, etype> > {
  inline static Shape<dim> Check(const TypecastExp<DstDType, SrcDType, EType, etype> &e) {
    return ShapeCheck<dim, EType>::Check(e.exp);
  }
};
template <int dim, typename E, typename DType>
struct ShapeCheck<dim, TransposeExp<E, DType> > {
  inline static Shape<dim> Check(const TransposeExp<E, DType> &e) {
    static_assert(dim == 2, "transpose is defined for matrices");
    const Shape<dim> s = ShapeCheck<dim, E>::Check(e.exp);
    Shape<dim> r;
    r[0] = s[1];
    r[1] = s[0];
    return r;
  }
};
template <int dim, typename Device, typename DType>
struct ShapeCheck<dim, Tensor<Device, dim, DType> > {
  inline static Shape<dim> Check(const Tensor<Device, dim, DType> &t) { return t.shape_; }
};
template <int dim, typename SrcExp, typename T, typename DType>
struct ShapeCheck<dim, MakeTensorExp<T, SrcExp, dim, DType> > {
  inline static Shape<dim> Check(const MakeTensorExp<T, SrcExp, dim, DType> &t) { return t.shape_; }
};
template <int dim, typename OP, typename TA, typename DType, int etype>
struct ShapeCheck<dim, UnaryMapExp<OP, TA, DType, etype> > {
  inline static Shape<dim> Check(const UnaryMapExp<OP, TA, DType, etype> &t) {
    return ShapeCheck<dim, TA>::Check(t.src_);
  }
};
template <int dim, typename OP, typename TA, typename TB, typename DType, int etype>
struct ShapeCheck<dim, BinaryMapExp<OP, TA, TB, DType, etype> > {
  inline static Shape<dim> Check(const BinaryMapExp<OP, TA, TB, DType, etype> &t) {
    const Shape<dim> l = ShapeCheck<dim, TA>::Check(t.lhs_);
    const Shape<dim> r = ShapeCheck<dim, TB>::Check(t.rhs_);
    if (l[0] == 0) return r;
    if (r[0] == 0) return l;
    CHECK_EQ(l, r) << "BinaryMapExp: Shapes of operands are not the same, "
                   << "Shape1=" << l << ", Shape2=" << r;
    return l;
  }
};
template <int dim, typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct ShapeCheck<dim, TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  inline static Shape<dim> Check(const TernaryMapExp<OP, TA, TB, TC, DType, etype> &t) {
    const Shape<dim> s1 = ShapeCheck<dim, TA>::Check(t.item1_);
    const Shape<dim> s2 = ShapeCheck<dim, TB>::Check(t.item2_);
    const Shape<dim> s3 = ShapeCheck<dim, TC>::Check(t.item3_);
    const bool same = (s1 == s2) && (s2 == s3);
    CHECK(same) << "TernaryMapExp: Shapes of operands are not the same, "
                << "Shape1=" << s1 << ", Shape2=" << s2 << ", Shape3=" << s3;
    return s1;
  }
};

// ----------------------------------------------------------------------------------------
// 128-bit path eligibility.
//   PackInfo<E>::kPass   compile time: every node of E knows EvalPack
//   PackAlign<E>::Check  run time: every tensor leaf has a 16-byte aligned base and a
//                        row stride that keeps rows 16-byte aligned
//   FlatInfo<E>::kPass   compile time: E's value at (y,x) depends only on the linear element
//                        offset, so dense operands may be walked as one long row
//   FlatCheck<E>::Check  run time: every tensor leaf is dense (stride_ == last extent)
// ----------------------------------------------------------------------------------------
template <typename E>
struct PackInfo {
  static const bool kPass = false;
};
template <typename E>
struct FlatInfo {
  static const bool kPass = false;
};
template <typename E>
struct PackAlign {
  inline static bool Check(const E &) { return false; }
};
template <typename E>
struct FlatCheck {
  inline static bool Check(const E &) { return false; }
};

// an extension expression seen through its MakeTensorExp base
template <typename T, typename SrcExp, int dim, typename DType>
struct PackInfo<MakeTensorExp<T, SrcExp, dim, DType> > : public PackInfo<T> {};
template <typename T, typename SrcExp, int dim, typename DType>
struct PackAlign<MakeTensorExp<T, SrcExp, dim, DType> > {
  inline static bool Check(const MakeTensorExp<T, SrcExp, dim, DType> &e) {
    return PackAlign<T>::Check(e.real_self());
  }
};

template <typename DType>
struct PackInfo<ScalarExp<DType> > {
  static const bool kPass = true;
};
template <typename DType>
struct FlatInfo<ScalarExp<DType> > {
  static const bool kPass = true;
};
template <typename DType>
struct PackAlign<ScalarExp<DType> > {
  inline static bool Check(const ScalarExp<DType> &) { return true; }
};
template <typename DType>
struct FlatCheck<ScalarExp<DType> > {
  inline static bool Check(const ScalarExp<DType> &) { return true; }
};

template <int dim, typename DType>
struct PackInfo<Tensor<gpu, dim, DType> > {
  static const bool kPass = (16 % sizeof(DType) == 0) && sizeof(DType) <= 8;
};
template <int dim, typename DType>
struct FlatInfo<Tensor<gpu, dim, DType> > {
  static const bool kPass = true;
};
template <int dim, typename DType>
struct PackAlign<Tensor<gpu, dim, DType> > {
  inline static bool Check(const Tensor<gpu, dim, DType> &t) {
    const bool base_ok = reinterpret_cast<uintptr_t>(t.dptr_) % 16 == 0;
    const bool single_row = t.shape_.FlatTo2D()[0] <= 1;
    return base_ok && (single_row || (t.stride_ * sizeof(DType)) % 16 == 0);
  }
};
template <int dim, typename DType>
struct FlatCheck<Tensor<gpu, dim, DType> > {
  inline static bool Check(const Tensor<gpu, dim, DType> &t) { return t.CheckContiguous(); }
};

template <typename OP, typename TA, typename DType, int etype>
struct PackInfo<UnaryMapExp<OP, TA, DType, etype> > : public PackInfo<TA> {};
template <typename OP, typename TA, typename DType, int etype>
struct FlatInfo<UnaryMapExp<OP, TA, DType, etype> > : public FlatInfo<TA> {};
template <typename OP, typename TA, typename DType, int etype>
struct PackAlign<UnaryMapExp<OP, TA, DType, etype> > {
  inline static bool Check(const UnaryMapExp<OP, TA, DType, etype> &e) {
    return PackAlign<TA>::Check(e.src_);
  }
};
template <typename OP, typename TA, typename DType, int etype>
struct FlatCheck<UnaryMapExp<OP, TA, DType, etype> > {
  inline static bool Check(const UnaryMapExp<OP, TA, DType, etype> &e) {
    return FlatCheck<TA>::Check(e.src_);
  }
};

template <typename OP, typename TA, typename TB, typename DType, int etype>
struct PackInfo<BinaryMapExp<OP, TA, TB, DType, etype> > {
  static const bool kPass = PackInfo<TA>::kPass && PackInfo<TB>::kPass;
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct FlatInfo<BinaryMapExp<OP, TA, TB, DType, etype> > {
  static const bool kPass = FlatInfo<TA>::kPass && FlatInfo<TB>::kPass;
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct PackAlign<BinaryMapExp<OP, TA, TB, DType, etype> > {
  inline static bool Check(const BinaryMapExp<OP, TA, TB, DType, etype> &e) {
    return PackAlign<TA>::Check(e.lhs_) && PackAlign<TB>::Check(e.rhs_);
  }
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct FlatCheck<BinaryMapExp<OP, TA, TB, DType, etype> > {
  inline static bool Check(const BinaryMapExp<OP, TA, TB, DType, etype> &e) {
    return FlatCheck<TA>::Check(e.lhs_) && FlatCheck<TB>::Check(e.rhs_);
  }
};

template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct PackInfo<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  static const bool kPass = PackInfo<TA>::kPass && PackInfo<TB>::kPass && PackInfo<TC>::kPass;
};
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct FlatInfo<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  static const bool kPass = FlatInfo<TA>::kPass && FlatInfo<TB>::kPass && FlatInfo<TC>::kPass;
};
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct PackAlign<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  inline static bool Check(const TernaryMapExp<OP, TA, TB, TC, DType, etype> &e) {
    return PackAlign<TA>::Check(e.item1_) && PackAlign<TB>::Check(e.item2_) &&
           PackAlign<TC>::Check(e.item3_);
  }
};
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct FlatCheck<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  inline static bool Check(const TernaryMapExp<OP, TA, TB, TC, DType, etype> &e) {
    return FlatCheck<TA>::Check(e.item1_) && FlatCheck<TB>::Check(e.item2_) &&
           FlatCheck<TC>::Check(e.item3_);
  }
};

// ----------------------------------------------------------------------------------------
// dispatch of an assignment
// ----------------------------------------------------------------------------------------
/*! \brief expressions of kind kComplex specialise this with their own evaluation routine */
template <typename SV, typename RV, typename E, typename DType>
struct ExpComplexEngine {
  inline static void Eval(RV *dst, const E &exp);
};

template <typename SV, typename RV, typename DType>
struct ExpEngine {
  template <typename E>
  inline static void Eval(RV *dst, const Exp<E, DType, type::kMapper> &exp) {
    MapExp<SV>(dst, exp);
  }
  template <typename E>
  inline static void Eval(RV *dst, const Exp<E, DType, type::kChainer> &exp) {
    MapExp<SV>(dst, exp);
  }
  template <typename E>
  inline static void Eval(RV *dst, const Exp<E, DType, type::kRValue> &exp) {
    MapExp<SV>(dst, exp);
  }
  template <typename E>
  inline static void Eval(RV *dst, const Exp<E, DType, type::kComplex> &exp) {
    ExpComplexEngine<SV, RV, E, DType>::Eval(dst->ptrself(), exp.self());
  }
};

// ----------------------------------------------------------------------------------------
// LaneInfo<E>::kPass: every node of E is a cheap, side-effect free Eval(y, x) (arithmetic and
// index remapping, no loop over other elements).  For such an expression without EvalPack the
// map kernel still writes the destination in 16-byte groups, each put together from element
// evaluations.  Expressions whose Eval walks many elements (reductions, take_grad) stay out:
// one thread would serialise several such walks.  Unknown (user-defined) expressions default
// to false.
// ----------------------------------------------------------------------------------------
template <typename E>
struct LaneInfo {
  static const bool kPass = false;
};
template <typename T, typename SrcExp, int dim, typename DType>
struct LaneInfo<MakeTensorExp<T, SrcExp, dim, DType> > : public LaneInfo<T> {};
template <typename DType>
struct LaneInfo<ScalarExp<DType> > {
  static const bool kPass = true;
};
template <typename Device, int dim, typename DType>
struct LaneInfo<Tensor<Device, dim, DType> > {
  static const bool kPass = true;
};
template <typename DstDType, typename SrcDType, typename EType, int etype>
struct LaneInfo<TypecastExp<DstDType, SrcDType, EType, etype> > : public LaneInfo<EType> {};
template <typename OP, typename TA, typename DType, int etype>
struct LaneInfo<UnaryMapExp<OP, TA, DType, etype> > : public LaneInfo<TA> {};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct LaneInfo<BinaryMapExp<OP, TA, TB, DType, etype> > {
  static const bool kPass = LaneInfo<TA>::kPass && LaneInfo<TB>::kPass;
};
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct LaneInfo<TernaryMapExp<OP, TA, TB, TC, DType, etype> > {
  static const bool kPass = LaneInfo<TA>::kPass && LaneInfo<TB>::kPass && LaneInfo<TC>::kPass;
};

}  // namespace expr

#if MSHADOW_USE_CUDA
namespace cuda {
/*!
 * \brief chooses the kernel for `dst <Saver>= exp` on the GPU.  The primary template (in
 *  gpu/engine.cuh) serves every expression through the generic map kernels; extension
 *  headers specialise it for expressions that have a dedicated kernel.
 */
template <typename Saver, typename R, typename E, typename DType, int dim>
struct MapDispatch;
/*! \brief the generic route: 128-bit kernel when the expression and the operands allow it */
template <typename Saver, typename DType, typename R, typename E, int dim>
inline void MapGeneric(R *dst, const E &exp, Shape<dim> dshape, cudaStream_t stream);
}  // namespace cuda
#endif

}  // namespace mshadow
#endif  // MSHADOW_ENGINE_CHECK_H_
