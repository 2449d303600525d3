/*
 * The fixed set of axis- and box-addressed expressions behind msb_axis_case_f32, written once
 * for both devices: the C ABI instantiates it for gpu, the host conformance library for cpu.
 * The case list is documented at the declaration of msb_axis_case_f32.
 */
#ifndef MSHADOW_B200_CSRC_AXIS_CASES_H_
#define MSHADOW_B200_CSRC_AXIS_CASES_H_

#include <cstdint>
#include <vector>

#include "mshadow/tensor.h"

namespace msb_axis {

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

const int kNumCases = 11;

/*! \brief a minimal dynamic shape, the kind of type broadcast_multi_axes / broadcast_to are templated on */
struct DynShape {
  std::vector<index_t> v;
  DynShape() {}
  template <typename It>
  DynShape(It b, It e) : v(b, e) {}
  index_t ndim() const { return static_cast<index_t>(v.size()); }
  index_t operator[](size_t i) const { return v[i]; }
};

template <typename xpu, int dim>
inline Tensor<xpu, dim, float> Dense(const float *p, Shape<dim> s, Stream<xpu> *stream) {
  return Tensor<xpu, dim, float>(const_cast<float *>(p), s, s[dim - 1], stream);
}

inline void Box(int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, Shape<4> *b, Shape<4> *e) {
  *b = Shape4(p0 % n, p1 % c, p0 % h, p1 % w);
  *e = Shape4(n, c, (*b)[2] + (h - (*b)[2] + 1) / 2, w);
}

template <int dim>
inline int PutShape(Shape<dim> s, int64_t o[4]) {
  for (int i = 0; i < 4; ++i) o[i] = i < dim ? s[i] : 1;
  return dim;
}

/*! \brief cheap argument screening, so that the expressions' own checks only see sane extents */
inline bool ArgsOk(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1) {
  const int64_t lim = int64_t(1) << 30;
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || n * c * h * w >= lim) return false;
  if (p0 <= -lim || p0 >= lim || p1 < 0 || p1 >= lim) return false;
  switch (id) {
    case 0: case 1: return p1 >= 1 && p1 < (int64_t(1) << 24);
    case 2: case 3: return p0 >= 0;
    case 4: case 5: case 6: return p0 >= 0 && p0 < 4;
    case 7: return p0 >= 0 && p0 < 4 && p1 >= 1 && n * c * h * w * p1 < lim;
    case 8: return p1 >= 1 && n * h * w * p1 < lim;
    case 9: return p0 >= 1 && p1 >= 1 && n * h * p0 * p1 < lim;
    default: return p0 >= 1 && p1 >= 1 && c * w * p0 * p1 < lim;
  }
}

/*! \brief extents of the result (from the expression objects themselves); returns their number */
template <typename xpu>
inline int ResultShape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t o[4]) {
  Stream<xpu> *none = nullptr;
  const Tensor<xpu, 4, float> a = Dense<xpu>(nullptr, Shape4(n, c, h, w), none);
  Shape<4> b, e;
  Box(n, c, h, w, p0, p1, &b, &e);
  std::vector<index_t> ax(2), sz(4);
  switch (id) {
    case 0: return PutShape(ShapeCheck<1, RangeExp<float> >::Check(range<float>(p0, p0 + p1, 0.5f, 2)), o);
    case 1: return PutShape(ShapeCheck<1, RangeExp<float> >::Check(range<float>(p0 + p1, p0, -1.5f, 1)), o);
    case 2: return PutShape(slice(a, b, e).shape_, o);
    case 3: return PutShape(a.shape_, o);
    case 4: return PutShape(reduce_with_axis<red::sum, false>(a, p0).shape_, o);
    case 5: return PutShape(reduce_with_axis<red::maximum, true>(a, p0).shape_, o);
    case 6: return PutShape(reduce_keepdim<red::minimum, false>(a, p0).shape_, o);
    case 7: return PutShape(broadcast_with_axis(Dense<xpu>(nullptr, Shape3(n * c, h, w), none), p0 - 1, p1).shape_, o);
    case 8: return PutShape(broadcast_keepdim(slice<1>(a, 0, 1), 1, p1).shape_, o);
    case 9:
      sz[0] = n; sz[1] = p0; sz[2] = h; sz[3] = p1;
      return PutShape(broadcast_to(Dense<xpu>(nullptr, Shape4(n, 1, h, 1), none), DynShape(sz.begin(), sz.end())).shape_, o);
    default:
      ax[0] = 0; ax[1] = 2; sz.resize(2); sz[0] = p0; sz[1] = p1;
      return PutShape(broadcast_multi_axes(Dense<xpu>(nullptr, Shape4(1, c, 1, w), none), DynShape(ax.begin(), ax.end()),
                                           DynShape(sz.begin(), sz.end())).shape_, o);
  }
}

/*! \brief evaluates case `id` into dense `dst` on `stream` */
template <typename xpu>
inline void Run(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                Stream<xpu> *stream) {
  int64_t o[4];
  ResultShape<xpu>(id, n, c, h, w, p0, p1, o);
  const Tensor<xpu, 4, float> a = Dense<xpu>(A, Shape4(n, c, h, w), stream);
  Tensor<xpu, 4, float> d4 = Dense<xpu>(dst, Shape4(o[0], o[1], o[2], o[3]), stream);
  Tensor<xpu, 3, float> d3 = Dense<xpu>(dst, Shape3(o[0], o[1], o[2]), stream);
  Tensor<xpu, 1, float> d1 = Dense<xpu>(dst, Shape1(o[0]), stream);
  Shape<4> b, e;
  Box(n, c, h, w, p0, p1, &b, &e);
  std::vector<index_t> ax(2), sz(4);
  switch (id) {
    case 0: d1 = range<float>(p0, p0 + p1, 0.5f, 2); break;
    case 1: d1 = range<float>(p0 + p1, p0, -1.5f, 1); break;
    case 2: d4 = slice(a, b, e); break;
    case 3:
      d4 = a * 2.0f;
      slice(d4, b, e) = slice(a, b, e) + 1.0f;
      break;
    case 4: d3 = reduce_with_axis<red::sum, false>(a, p0); break;
    case 5: d3 = reduce_with_axis<red::maximum, true>(a, p0); break;
    case 6: d4 = reduce_keepdim<red::minimum, false>(a, p0); break;
    case 7: d4 = broadcast_with_axis(Dense<xpu>(A, Shape3(n * c, h, w), stream), p0 - 1, p1); break;
    case 8: d4 = broadcast_keepdim(slice<1>(a, 0, 1), 1, p1); break;
    case 9:
      sz[0] = n; sz[1] = p0; sz[2] = h; sz[3] = p1;
      d4 = broadcast_to(Dense<xpu>(A, Shape4(n, 1, h, 1), stream), DynShape(sz.begin(), sz.end()));
      break;
    default:
      ax[0] = 0; ax[1] = 2; sz.resize(2); sz[0] = p0; sz[1] = p1;
      d4 = broadcast_multi_axes(Dense<xpu>(A, Shape4(1, c, 1, w), stream), DynShape(ax.begin(), ax.end()),
                                DynShape(sz.begin(), sz.end()));
      break;
  }
}

}  // namespace msb_axis
#endif  // MSHADOW_B200_CSRC_AXIS_CASES_H_
