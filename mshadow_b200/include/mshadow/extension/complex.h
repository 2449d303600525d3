/*
 * Complex arithmetic on tensors whose last dimension interleaves real and imaginary parts
 * (re0, im0, re1, im1, ...):
 *
 *   complex_mul_cc / _cr / _rc (a, b)   product of complex x complex, complex x real, real x complex
 *   complex_div_cc / _cr / _rc (a, b)   quotient, likewise
 *   conj(a), complex_exchange(a)        conjugate; real and imaginary part swapped
 *   complex_pad_imag(r)                 real tensor -> complex tensor with zero imaginary part
 *   complex_toreal(a), complex_abs_square(a), complex_sum_real_imag(a)   complex -> real
 *
 * Function names, operand layouts, shape rules and the operator structs `op::complex::*` with
 * their RealMap / ImagMap members follow dmlc/mshadow's mshadow/extension/complex.h (:14-114 the
 * operators, :130-303 the expression types and functions, :307-365 the shape rules, :370-489 the
 * plans), so user-written complex operators keep working through ComplexF<>.  The arithmetic
 * inside the built-in operators rounds every product, sum and quotient separately, as the
 * reference's CPU build does, so results are bit-identical on the GPU.
 *
 * An element of the result is either the real or the imaginary part of one complex number; which
 * one is decided by the parity of its column.  All plans are cheap per element (two to four
 * look-ups), so on the GPU they are evaluated four columns per thread with one 16-byte store.
 */
#ifndef MSHADOW_EXTENSION_COMPLEX_H_
#define MSHADOW_EXTENSION_COMPLEX_H_

#include <type_traits>

#include "../engine/check.h"

namespace mshadow {
namespace op {
namespace complex {
enum BinaryCalculationType { kBinaryCC, kBinaryCR, kBinaryRC };
enum UnitaryCalculationType { kUnitaryC2R, kUnitaryC2C, kUnitaryR2C };

/*! \brief (ar + i ai) (br + i bi) */
struct mul {
  template <typename DType>
  MSHADOW_XINLINE static DType RealMap(DType ar, DType ai, DType br, DType bi) {
    return detail::SubRN<DType>(detail::MulRN<DType>(ar, br), detail::MulRN<DType>(ai, bi));
  }
  template <typename DType>
  MSHADOW_XINLINE static DType ImagMap(DType ar, DType ai, DType br, DType bi) {
    return detail::AddRN<DType>(detail::MulRN<DType>(ar, bi), detail::MulRN<DType>(br, ai));
  }
};
/*! \brief (ar + i ai) / (br + i bi) */
struct div {
  template <typename DType>
  MSHADOW_XINLINE static DType RealMap(DType ar, DType ai, DType br, DType bi) {
    return detail::DivRN<DType>(detail::AddRN<DType>(detail::MulRN<DType>(ar, br), detail::MulRN<DType>(ai, bi)),
                                detail::AddRN<DType>(detail::MulRN<DType>(br, br), detail::MulRN<DType>(bi, bi)));
  }
  template <typename DType>
  MSHADOW_XINLINE static DType ImagMap(DType ar, DType ai, DType br, DType bi) {
    return detail::DivRN<DType>(detail::SubRN<DType>(detail::MulRN<DType>(br, ai), detail::MulRN<DType>(ar, bi)),
                                detail::AddRN<DType>(detail::MulRN<DType>(br, br), detail::MulRN<DType>(bi, bi)));
  }
};
// complex -> complex: (ri, rj) and (ii, ij) are the positions of the real and the imaginary part in `src`
struct conjugate {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj, index_t, index_t) {
    return src.Eval(ri, rj);
  }
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType ImagMap(const expr::Plan<TA, DType> &src, index_t, index_t, index_t ii, index_t ij) {
    return -src.Eval(ii, ij);
  }
};
struct exchange {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t, index_t, index_t ii, index_t ij) {
    return src.Eval(ii, ij);
  }
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType ImagMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj, index_t, index_t) {
    return src.Eval(ri, rj);
  }
};
// real -> complex
struct pad_imag {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj) {
    return src.Eval(ri, rj);
  }
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType ImagMap(const expr::Plan<TA, DType> &, index_t, index_t) {
    return static_cast<DType>(0);
  }
};
// complex -> real
struct toreal {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj, index_t, index_t) {
    return src.Eval(ri, rj);
  }
};
struct abs_square {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj, index_t ii,
                                       index_t ij) {
    const DType re = src.Eval(ri, rj), im = src.Eval(ii, ij);
    return detail::AddRN<DType>(detail::MulRN<DType>(re, re), detail::MulRN<DType>(im, im));
  }
};
struct sum_real_imag {
  template <typename TA, typename DType>
  MSHADOW_XINLINE static DType RealMap(const expr::Plan<TA, DType> &src, index_t ri, index_t rj, index_t ii,
                                       index_t ij) {
    return detail::AddRN<DType>(src.Eval(ri, rj), src.Eval(ii, ij));
  }
};
}  // namespace complex
}  // namespace op

namespace expr {

/*! \brief binary complex expression; calctype says which operands are complex */
template <int calctype, typename OP, typename TA, typename TB, typename DType, int etype>
struct ComplexBinaryMapExp : public Exp<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype>, DType, etype> {
  const TA &lhs_;
  const TB &rhs_;
  ComplexBinaryMapExp(const TA &lhs, const TB &rhs) : lhs_(lhs), rhs_(rhs) {}
};
/*! \brief unary complex expression; calctype says whether source and result are complex */
template <int calctype, typename OP, typename TA, typename DType, int etype>
struct ComplexUnitaryExp : public Exp<ComplexUnitaryExp<calctype, OP, TA, DType, etype>, DType, etype> {
  const TA &src_;
  explicit ComplexUnitaryExp(const TA &src) : src_(src) {}
};

template <int calctype, typename OP, typename TA, typename TB, typename DType, int ta, int tb>
inline ComplexBinaryMapExp<calctype, OP, TA, TB, DType, (ta | tb | type::kMapper)> ComplexF(const Exp<TA, DType, ta> &lhs,
                                                                                          const Exp<TB, DType, tb> &rhs) {
  return ComplexBinaryMapExp<calctype, OP, TA, TB, DType, (ta | tb | type::kMapper)>(lhs.self(), rhs.self());
}
template <int calctype, typename OP, typename SrcExp, typename DType, int e1>
inline ComplexUnitaryExp<calctype, OP, SrcExp, DType, (e1 | type::kMapper)> ComplexF(const Exp<SrcExp, DType, e1> &src) {
  return ComplexUnitaryExp<calctype, OP, SrcExp, DType, (e1 | type::kMapper)>(src.self());
}

#define MSHADOW_B200_COMPLEX_BINARY_(NAME, CALC, OP)                                                          \
  template <typename TA, typename TB, typename DType, int ta, int tb>                                         \
  inline ComplexBinaryMapExp<op::complex::CALC, op::complex::OP, TA, TB, DType, (ta | tb | type::kMapper)> NAME( \
      const Exp<TA, DType, ta> &lhs, const Exp<TB, DType, tb> &rhs) {                                          \
    return ComplexF<op::complex::CALC, op::complex::OP>(lhs, rhs);                                            \
  }
MSHADOW_B200_COMPLEX_BINARY_(complex_mul_cc, kBinaryCC, mul)
MSHADOW_B200_COMPLEX_BINARY_(complex_mul_cr, kBinaryCR, mul)
MSHADOW_B200_COMPLEX_BINARY_(complex_mul_rc, kBinaryRC, mul)
MSHADOW_B200_COMPLEX_BINARY_(complex_div_cc, kBinaryCC, div)
MSHADOW_B200_COMPLEX_BINARY_(complex_div_cr, kBinaryCR, div)
MSHADOW_B200_COMPLEX_BINARY_(complex_div_rc, kBinaryRC, div)
#undef MSHADOW_B200_COMPLEX_BINARY_

#define MSHADOW_B200_COMPLEX_UNARY_(NAME, CALC, OP)                                                          \
  template <typename SrcExp, typename DType, int e1>                                                        \
  inline ComplexUnitaryExp<op::complex::CALC, op::complex::OP, SrcExp, DType, (e1 | type::kMapper)> NAME(    \
      const Exp<SrcExp, DType, e1> &src) {                                                                  \
    return ComplexF<op::complex::CALC, op::complex::OP>(src);                                               \
  }
MSHADOW_B200_COMPLEX_UNARY_(conj, kUnitaryC2C, conjugate)
MSHADOW_B200_COMPLEX_UNARY_(complex_exchange, kUnitaryC2C, exchange)
MSHADOW_B200_COMPLEX_UNARY_(complex_pad_imag, kUnitaryR2C, pad_imag)
MSHADOW_B200_COMPLEX_UNARY_(complex_toreal, kUnitaryC2R, toreal)
MSHADOW_B200_COMPLEX_UNARY_(complex_abs_square, kUnitaryC2R, abs_square)
MSHADOW_B200_COMPLEX_UNARY_(complex_sum_real_imag, kUnitaryC2R, sum_real_imag)
#undef MSHADOW_B200_COMPLEX_UNARY_

// ------------------------------------------------------------------------------------------
// shapes: a complex operand is twice as wide as a real one; complex widths must be even
// ------------------------------------------------------------------------------------------
template <int dim, int calctype, typename OP, typename TA, typename TB, typename DType, int etype>
struct ShapeCheck<dim, ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype> > {
  inline static Shape<dim> Check(const ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype> &t) {
    const Shape<dim> lhs = ShapeCheck<dim, TA>::Check(t.lhs_), rhs = ShapeCheck<dim, TB>::Check(t.rhs_);
    if (lhs[0] == 0) return rhs;
    if (rhs[0] == 0) return lhs;
    if (calctype == op::complex::kBinaryCC) {
      CHECK_EQ(lhs, rhs) << "ComplexBinaryMapExp (CC): Shapes of operands are not the same.";
      CHECK_EQ(lhs[dim - 1] % 2, 0) << "ComplexBinaryMapExp (CC): Shape of the last dimension is not even. "
                                    << "We must have real part + imaginary part.";
      return lhs;
    }
    const char *kind = calctype == op::complex::kBinaryCR ? "CR" : "RC";
    CHECK(calctype == op::complex::kBinaryCR || calctype == op::complex::kBinaryRC)
        << "ComplexBinaryMapExp: Unexpected Calculation Type!";
    const Shape<dim> &wide = calctype == op::complex::kBinaryCR ? lhs : rhs;
    const Shape<dim> &narrow = calctype == op::complex::kBinaryCR ? rhs : lhs;
    for (int i = 0; i < dim - 1; ++i) {
      CHECK_EQ(wide[i], narrow[i]) << "ComplexBinaryMapExp (" << kind << "): Shapes of operands are not the same.";
    }
    CHECK_EQ(wide[dim - 1], narrow[dim - 1] * 2) << "ComplexBinaryMapExp (" << kind << "): Shapes of operands do not match.";
    return wide;
  }
};
template <int dim, int calctype, typename OP, typename TA, typename DType, int etype>
struct ShapeCheck<dim, ComplexUnitaryExp<calctype, OP, TA, DType, etype> > {
  inline static Shape<dim> Check(const ComplexUnitaryExp<calctype, OP, TA, DType, etype> &t) {
    Shape<dim> s = ShapeCheck<dim, TA>::Check(t.src_);
    CHECK_EQ(s[dim - 1] % 2, 0) << "ComplexUnitaryExp: Shape of the last dimension is not even. "
                                << "We must have real + imaginary.";
    CHECK(calctype == op::complex::kUnitaryC2C || calctype == op::complex::kUnitaryC2R ||
          calctype == op::complex::kUnitaryR2C)
        << "ComplexUnitaryExp: Unexpected Calculation Type!";
    if (calctype == op::complex::kUnitaryC2R) s[dim - 1] /= 2;
    if (calctype == op::complex::kUnitaryR2C) s[dim - 1] *= 2;
    return s;
  }
};
template <int calctype, typename OP, typename TA, typename TB, typename DType, int etype>
struct ExpInfo<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype> > {
  static const int kDimLhs = ExpInfo<TA>::kDim;
  static const int kDimRhs = ExpInfo<TB>::kDim;
  static const int kDim = (kDimLhs >= 0 && kDimRhs >= 0)
                              ? (kDimLhs == 0 ? kDimRhs : ((kDimRhs == 0 || kDimLhs == kDimRhs) ? kDimLhs : -1))
                              : -1;
  static const int kDevMask = ExpInfo<TA>::kDevMask & ExpInfo<TB>::kDevMask;
};
template <int calctype, typename OP, typename TA, typename DType, int etype>
struct ExpInfo<ComplexUnitaryExp<calctype, OP, TA, DType, etype> > {
  static const int kDim = ExpInfo<TA>::kDim;
  static const int kDevMask = ExpInfo<TA>::kDevMask;
};

// ------------------------------------------------------------------------------------------
// plans: column x of the result is part (x & 1) of complex number x / 2 of its row
// ------------------------------------------------------------------------------------------
template <int calctype, typename OP, typename TA, typename TB, int etype, typename DType>
class Plan<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype>, DType> {
 public:
  Plan(const Plan<TA, DType> &lhs, const Plan<TB, DType> &rhs) : lhs_(lhs), rhs_(rhs) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    const index_t re = x & ~static_cast<index_t>(1), im = re + 1, half = x >> 1;
    const DType zero = static_cast<DType>(0);
    // a real operand supplies (value, 0)
    const DType ar = calctype == op::complex::kBinaryRC ? lhs_.Eval(y, half) : lhs_.Eval(y, re);
    const DType ai = calctype == op::complex::kBinaryRC ? zero : lhs_.Eval(y, im);
    const DType br = calctype == op::complex::kBinaryCR ? rhs_.Eval(y, half) : rhs_.Eval(y, re);
    const DType bi = calctype == op::complex::kBinaryCR ? zero : rhs_.Eval(y, im);
    return (x & 1) == 0 ? OP::RealMap(ar, ai, br, bi) : OP::ImagMap(ar, ai, br, bi);
  }
#ifdef __CUDACC__
  /*! \brief complex x complex only: a 16-byte group holds whole (re, im) pairs of both operands */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    const Pack<DType> a = lhs_.EvalPack(y, x), b = rhs_.EvalPack(y, x);
    Pack<DType> r;
#pragma unroll
    for (int p = 0; p < Pack<DType>::kLanes; p += 2) {
      r.v[p] = OP::RealMap(a.v[p], a.v[p + 1], b.v[p], b.v[p + 1]);
      r.v[p + 1] = OP::ImagMap(a.v[p], a.v[p + 1], b.v[p], b.v[p + 1]);
    }
    return r;
  }
#endif

 private:
  Plan<TA, DType> lhs_;
  Plan<TB, DType> rhs_;
};

// complex x complex reads both operands at the result's own positions: 16-byte groups, and one
// long row where the operands are dense (widths are even, so parity survives the flattening)
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct PackInfo<ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> > {
  static const bool kPass = PackInfo<TA>::kPass && PackInfo<TB>::kPass;
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct PackAlign<ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> > {
  inline static bool Check(const ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> &e) {
    return PackAlign<TA>::Check(e.lhs_) && PackAlign<TB>::Check(e.rhs_);
  }
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct FlatInfo<ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> > {
  static const bool kPass = FlatInfo<TA>::kPass && FlatInfo<TB>::kPass;
};
template <typename OP, typename TA, typename TB, typename DType, int etype>
struct FlatCheck<ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> > {
  inline static bool Check(const ComplexBinaryMapExp<op::complex::kBinaryCC, OP, TA, TB, DType, etype> &e) {
    return FlatCheck<TA>::Check(e.lhs_) && FlatCheck<TB>::Check(e.rhs_);
  }
};

template <int calctype, typename OP, typename TA, int etype, typename DType>
class Plan<ComplexUnitaryExp<calctype, OP, TA, DType, etype>, DType> {
 public:
  explicit Plan(const Plan<TA, DType> &src) : src_(src) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const { return Part(y, x, std::integral_constant<int, calctype>()); }

 private:
  MSHADOW_XINLINE DType Part(index_t y, index_t x, std::integral_constant<int, op::complex::kUnitaryC2C>) const {
    const index_t re = x & ~static_cast<index_t>(1);
    return (x & 1) == 0 ? OP::RealMap(src_, y, re, y, re + 1) : OP::ImagMap(src_, y, re, y, re + 1);
  }
  MSHADOW_XINLINE DType Part(index_t y, index_t x, std::integral_constant<int, op::complex::kUnitaryR2C>) const {
    return (x & 1) == 0 ? OP::RealMap(src_, y, x >> 1) : OP::ImagMap(src_, y, x >> 1);
  }
  MSHADOW_XINLINE DType Part(index_t y, index_t x, std::integral_constant<int, op::complex::kUnitaryC2R>) const {
    return OP::RealMap(src_, y, x * 2, y, x * 2 + 1);
  }
  Plan<TA, DType> src_;
};

template <int calctype, typename OP, typename TA, typename TB, typename DType, int etype>
inline Plan<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype>, DType> MakePlan(
    const ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype> &e) {
  return Plan<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype>, DType>(MakePlan(e.lhs_), MakePlan(e.rhs_));
}
template <int calctype, typename OP, typename TA, typename DType, int etype>
inline Plan<ComplexUnitaryExp<calctype, OP, TA, DType, etype>, DType> MakePlan(
    const ComplexUnitaryExp<calctype, OP, TA, DType, etype> &e) {
  return Plan<ComplexUnitaryExp<calctype, OP, TA, DType, etype>, DType>(MakePlan(e.src_));
}

// cheap per element: results leave in 16-byte groups assembled from element evaluations
template <int calctype, typename OP, typename TA, typename TB, typename DType, int etype>
struct LaneInfo<ComplexBinaryMapExp<calctype, OP, TA, TB, DType, etype> > {
  static const bool kPass = LaneInfo<TA>::kPass && LaneInfo<TB>::kPass;
};
template <int calctype, typename OP, typename TA, typename DType, int etype>
struct LaneInfo<ComplexUnitaryExp<calctype, OP, TA, DType, etype> > : public LaneInfo<TA> {};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_COMPLEX_H_
