/*
 * Symbolic expression nodes of the mshadow API.  Nothing here computes: `A * B + 0.5f * C`
 * only builds a tree of references that the engine later turns into one GPU kernel.
 *
 * Node types, their public members and the operator set follow dmlc/mshadow's
 * mshadow/expression.h (:60-413) and mshadow/expr_scalar-inl.h (:36-162) so that user
 * code and user-defined extension expressions keep compiling.  Two things are done
 * differently here: the scalar overloads are templates that accept any arithmetic
 * right- or left-hand value for every element type (the reference re-includes a file once
 * per scalar type), and matrix products (dot) are not part of this engine.
 */
#ifndef MSHADOW_EXPRESSION_H_
#define MSHADOW_EXPRESSION_H_

#include <type_traits>

#include "./base.h"

namespace mshadow {
namespace expr {

/*! \brief what kind of node an expression is; a bit mask, wider kinds include narrower ones */
namespace type {
const int kRValue = 0;   // a container that can be assigned to
const int kMapper = 1;   // element-wise: value at (y,x) depends on operands at (y,x) only
const int kChainer = 3;  // index-remapping: value at (y,x) may read operands anywhere
const int kComplex = 7;  // needs its own evaluation routine (reductions)
}  // namespace type

template <typename Saver, typename RValue, typename DType>
struct ExpEngine;

/*! \brief CRTP root of every expression */
template <typename SubType, typename DType, int exp_type>
struct Exp {
  inline const SubType &self() const { return *static_cast<const SubType *>(this); }
  inline SubType *ptrself() { return static_cast<SubType *>(this); }
};

/*! \brief a constant; converts implicitly from the element type */
template <typename DType>
struct ScalarExp : public Exp<ScalarExp<DType>, DType, type::kMapper> {
  DType scalar_;
  ScalarExp(DType scalar) : scalar_(scalar) {}  // NOLINT(*)
};
template <typename DType>
inline ScalarExp<DType> scalar(DType s) {
  return ScalarExp<DType>(s);
}

/*! \brief element type conversion */
template <typename DstDType, typename SrcDType, typename EType, int etype>
struct TypecastExp : public Exp<TypecastExp<DstDType, SrcDType, EType, etype>, DstDType, etype> {
  const EType &exp;
  explicit TypecastExp(const EType &e) : exp(e) {}
};
template <typename DstDType, typename SrcDType, typename EType, int etype>
inline TypecastExp<DstDType, SrcDType, EType, (etype | type::kMapper)> tcast(
    const Exp<EType, SrcDType, etype> &exp) {
  return TypecastExp<DstDType, SrcDType, EType, (etype | type::kMapper)>(exp.self());
}

/*! \brief transposed view of a container */
template <typename EType, typename DType>
struct TransposeExp : public Exp<TransposeExp<EType, DType>, DType, type::kChainer> {
  const EType &exp;
  explicit TransposeExp(const EType &e) : exp(e) {}
  inline const EType &T() const { return exp; }
};

/*! \brief base of assignable containers: routes every assignment form to the engine */
template <typename Container, typename DType>
class RValueExp : public Exp<Container, DType, type::kRValue> {
 public:
  inline const TransposeExp<Container, DType> T() const {
    return TransposeExp<Container, DType>(this->self());
  }
  inline Container &operator+=(DType s) { return Apply<sv::plusto>(scalar<DType>(s)); }
  inline Container &operator-=(DType s) { return Apply<sv::minusto>(scalar<DType>(s)); }
  inline Container &operator*=(DType s) { return Apply<sv::multo>(scalar<DType>(s)); }
  inline Container &operator/=(DType s) { return Apply<sv::divto>(scalar<DType>(s)); }
  template <typename E, int etype>
  inline Container &operator+=(const Exp<E, DType, etype> &e) { return Apply<sv::plusto>(e); }
  template <typename E, int etype>
  inline Container &operator-=(const Exp<E, DType, etype> &e) { return Apply<sv::minusto>(e); }
  template <typename E, int etype>
  inline Container &operator*=(const Exp<E, DType, etype> &e) { return Apply<sv::multo>(e); }
  template <typename E, int etype>
  inline Container &operator/=(const Exp<E, DType, etype> &e) { return Apply<sv::divto>(e); }
  /*! \brief `dst = scalar`; called by the containers' operator= */
  inline Container &__assign(DType s) { return Apply<sv::saveto>(scalar<DType>(s)); }
  /*! \brief `dst = expression`; called by the containers' operator= */
  template <typename E, int etype>
  inline Container &__assign(const Exp<E, DType, etype> &e) { return Apply<sv::saveto>(e); }
  /*! \brief `dst = expression of another element type` */
  template <typename E, int etype, typename OtherDType>
  inline Container &__assign(const Exp<E, OtherDType, etype> &e) {
    ExpEngine<sv::saveto, Container, DType>::Eval(this->ptrself(), e.self());
    return *(this->ptrself());
  }

 private:
  template <typename Saver, typename E, int etype>
  inline Container &Apply(const Exp<E, DType, etype> &e) {
    ExpEngine<Saver, Container, DType>::Eval(this->ptrself(), e.self());
    return *(this->ptrself());
  }
};

// ------------------------------- element-wise maps -------------------------------------

template <typename OP, typename TA, typename DType, int etype>
struct UnaryMapExp : public Exp<UnaryMapExp<OP, TA, DType, etype>, DType, etype> {
  const TA &src_;
  explicit UnaryMapExp(const TA &src) : src_(src) {}
};

template <typename OP, typename TA, typename TB, typename DType, int etype>
struct BinaryMapExp : public Exp<BinaryMapExp<OP, TA, TB, DType, etype>, DType, etype> {
  const TA &lhs_;
  const TB &rhs_;
  explicit BinaryMapExp(const TA &lhs, const TB &rhs) : lhs_(lhs), rhs_(rhs) {}
};

template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
struct TernaryMapExp : public Exp<TernaryMapExp<OP, TA, TB, TC, DType, etype>, DType, etype> {
  const TA &item1_;
  const TB &item2_;
  const TC &item3_;
  explicit TernaryMapExp(const TA &i1, const TB &i2, const TC &i3)
      : item1_(i1), item2_(i2), item3_(i3) {}
};

template <typename OP, typename TA, typename DType, int ta>
inline UnaryMapExp<OP, TA, DType, (ta | type::kMapper)> MakeExp(const Exp<TA, DType, ta> &src) {
  return UnaryMapExp<OP, TA, DType, (ta | type::kMapper)>(src.self());
}
template <typename OP, typename TA, typename TB, typename DType, int ta, int tb>
inline BinaryMapExp<OP, TA, TB, DType, (ta | tb | type::kMapper)> MakeExp(
    const Exp<TA, DType, ta> &lhs, const Exp<TB, DType, tb> &rhs) {
  return BinaryMapExp<OP, TA, TB, DType, (ta | tb | type::kMapper)>(lhs.self(), rhs.self());
}
template <typename OP, typename TA, typename TB, typename TC, typename DType, int ta, int tb,
          int tc>
inline TernaryMapExp<OP, TA, TB, TC, DType, (ta | tb | tc | type::kMapper)> MakeExp(
    const Exp<TA, DType, ta> &i1, const Exp<TB, DType, tb> &i2, const Exp<TC, DType, tc> &i3) {
  return TernaryMapExp<OP, TA, TB, TC, DType, (ta | tb | tc | type::kMapper)>(i1.self(), i2.self(),
                                                                              i3.self());
}

/*! \brief apply a user functor `struct OP { static DType Map(...); }` element-wise */
template <typename OP, typename TA, typename DType, int ta>
inline UnaryMapExp<OP, TA, DType, (ta | type::kMapper)> F(const Exp<TA, DType, ta> &src) {
  return MakeExp<OP>(src);
}
template <typename OP, typename TA, typename TB, typename DType, int ta, int tb>
inline BinaryMapExp<OP, TA, TB, DType, (ta | tb | type::kMapper)> F(const Exp<TA, DType, ta> &lhs,
                                                                   const Exp<TB, DType, tb> &rhs) {
  return MakeExp<OP>(lhs, rhs);
}
template <typename OP, typename TA, typename TB, typename TC, typename DType, int ta, int tb,
          int tc>
inline TernaryMapExp<OP, TA, TB, TC, DType, (ta | tb | tc | type::kMapper)> F(
    const Exp<TA, DType, ta> &i1, const Exp<TB, DType, tb> &i2, const Exp<TC, DType, tc> &i3) {
  return MakeExp<OP>(i1, i2, i3);
}

namespace exprdetail {
/*! \brief parameter type that takes no part in template argument deduction */
template <typename T>
struct NoDeduce {
  typedef T Type;
};
}  // namespace exprdetail

// The four arithmetic operators, each in three forms: expression (op) expression,
// expression (op) scalar, scalar (op) expression.  In the scalar forms the element type is
// deduced from the expression alone, so `A * 2`, `A * 2.0f` and `0.5 * A` all work.
#define MSHADOW_B200_ARITH_OPERATOR_(SYM, OPNAME)                                               \
  template <typename TA, typename TB, typename DType, int ta, int tb>                           \
  inline BinaryMapExp<op::OPNAME, TA, TB, DType, (ta | tb | type::kMapper)> operator SYM(       \
      const Exp<TA, DType, ta> &lhs, const Exp<TB, DType, tb> &rhs) {                           \
    return MakeExp<op::OPNAME>(lhs, rhs);                                                       \
  }                                                                                             \
  template <typename TA, typename DType, int ta>                                                \
  inline BinaryMapExp<op::OPNAME, TA, ScalarExp<DType>, DType, (ta | type::kMapper)>            \
  operator SYM(const Exp<TA, DType, ta> &lhs,                                                   \
               const typename exprdetail::NoDeduce<ScalarExp<DType> >::Type &rhs) {             \
    return MakeExp<op::OPNAME>(lhs, rhs);                                                       \
  }                                                                                             \
  template <typename TB, typename DType, int tb>                                                \
  inline BinaryMapExp<op::OPNAME, ScalarExp<DType>, TB, DType, (tb | type::kMapper)>            \
  operator SYM(const typename exprdetail::NoDeduce<ScalarExp<DType> >::Type &lhs,               \
               const Exp<TB, DType, tb> &rhs) {                                                 \
    return MakeExp<op::OPNAME>(lhs, rhs);                                                       \
  }

MSHADOW_B200_ARITH_OPERATOR_(+, plus)
MSHADOW_B200_ARITH_OPERATOR_(-, minus)
MSHADOW_B200_ARITH_OPERATOR_(*, mul)
MSHADOW_B200_ARITH_OPERATOR_(/, div)
#undef MSHADOW_B200_ARITH_OPERATOR_

/*! \brief user functor with one scalar operand */
template <typename OP, typename TA, typename DType, int ta>
inline BinaryMapExp<OP, TA, ScalarExp<DType>, DType, (ta | type::kMapper)> F(
    const Exp<TA, DType, ta> &lhs, const typename exprdetail::NoDeduce<ScalarExp<DType> >::Type &rhs) {
  return MakeExp<OP>(lhs, rhs);
}
template <typename OP, typename TB, typename DType, int tb>
inline BinaryMapExp<OP, ScalarExp<DType>, TB, DType, (tb | type::kMapper)> F(
    const typename exprdetail::NoDeduce<ScalarExp<DType> >::Type &lhs, const Exp<TB, DType, tb> &rhs) {
  return MakeExp<OP>(lhs, rhs);
}

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXPRESSION_H_
