/*
 * C entry points around the UNMODIFIED reference CPU evaluator -- TEST INFRASTRUCTURE ONLY.
 *
 * This file contains no arithmetic of its own: every function wraps caller memory in
 * mshadow::Tensor<cpu,...> handles and calls the reference's public API, so that the
 * results are, by construction, what dmlc/mshadow computes on the CPU.  It is compiled
 * against the reference headers where they lie (include path only; see the Makefile)
 * into oracle/_ref/libmshadow_ref.so, which is used to pin oracle.c, to generate the
 * fixtures under tests/golden/, and as the timed CPU baseline of the benchmark.
 *
 * The exported names are those of oracle.h with a ref_ prefix.
 */
#define ORC_PREFIX ref_
#include "oracle.h"

#include <cmath>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "mshadow/tensor.h"

using namespace mshadow;
using namespace mshadow::expr;

namespace {

typedef Tensor<cpu, 1, float> T1;
typedef Tensor<cpu, 2, float> T2;
typedef Tensor<cpu, 4, float> T4;

inline T2 mat(const float *p, int64_t rows, int64_t cols, int64_t ld) {
  return T2(const_cast<float *>(p), Shape2(rows, cols), static_cast<index_t>(ld), NULL);
}
inline T1 vec(const float *p, int64_t n) {
  return T1(const_cast<float *>(p), Shape1(n), static_cast<index_t>(n), NULL);
}
inline T4 img(const float *p, int64_t n, int64_t c, int64_t h, int64_t w, int64_t ld) {
  return T4(const_cast<float *>(p), Shape4(n, c, h, w), static_cast<index_t>(ld), NULL);
}

/* user-defined operators in the style of guide/defop.cpp and guide/README.md:152-157 */
struct sigmoid {
  MSHADOW_XINLINE static float Map(float a) { return 1.0f / (1.0f + expf(-a)); }
};
struct clip_mul {
  MSHADOW_XINLINE static float Map(float a, float b) { return a > b ? a * b : b; }
};
struct fma3 {
  MSHADOW_XINLINE static float Map(float a, float b, float c) { return a * b + c; }
};
struct square {
  MSHADOW_XINLINE static float Map(float a) { return a * a; }
};

/* the functors of a local-response-normalisation layer written against the reference */
struct power {
  MSHADOW_XINLINE static float Map(float a, float b) { return powf(a, b); }
};
struct power_by_roots {
  MSHADOW_XINLINE static float Map(float a, float b) {
    if (b != -0.75f && b != -1.75f) return powf(a, b);
    const float r = sqrtf(a);
    float t = r * sqrtf(r);
    if (b == -1.75f) t = t * a;
    return 1.0f / t;
  }
};

template <typename Power>
void lrn_forward_impl(T4 out, T4 norm, const T4 &src, int nsize, float salpha, float beta, float knorm) {
  norm = chpool<red::sum>(F<square>(src), nsize) * salpha + knorm;
  out = src * F<Power>(norm, -beta);
}
template <typename Power>
void lrn_backward_impl(T4 gsrc, const T4 &gout, const T4 &src, const T4 &norm, int nsize, float salpha, float beta) {
  gsrc = gout * F<Power>(norm, -beta);
  gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<Power>(norm, -beta - 1.0f), nsize) * src;
}

template <typename Reducer>
void keep_lowest(T1 d, const T2 &s, float scale, int saver) {
  switch (saver) {
    case 0: MapReduceKeepLowest<sv::saveto, Reducer>(&d, s, scale); break;
    case 1: MapReduceKeepLowest<sv::plusto, Reducer>(&d, s, scale); break;
    case 2: MapReduceKeepLowest<sv::minusto, Reducer>(&d, s, scale); break;
    case 3: MapReduceKeepLowest<sv::multo, Reducer>(&d, s, scale); break;
    default: MapReduceKeepLowest<sv::divto, Reducer>(&d, s, scale); break;
  }
}

template <typename Reducer>
void keep_dim1(T1 d, const T4 &s, float scale, int saver) {
  switch (saver) {
    case 0: MapReduceKeepHighDim<sv::saveto, Reducer, 1>(&d, s, scale); break;
    case 1: MapReduceKeepHighDim<sv::plusto, Reducer, 1>(&d, s, scale); break;
    case 2: MapReduceKeepHighDim<sv::minusto, Reducer, 1>(&d, s, scale); break;
    case 3: MapReduceKeepHighDim<sv::multo, Reducer, 1>(&d, s, scale); break;
    default: MapReduceKeepHighDim<sv::divto, Reducer, 1>(&d, s, scale); break;
  }
}

}  // namespace

extern "C" {

void ref_expr_case(int id, float *dst, const float *A, const float *B, const float *C,
                   const float *bias, int64_t rows, int64_t cols, int64_t ld_dst, int64_t ld_a,
                   int64_t ld_b, int64_t ld_c) {
  T2 d = mat(dst, rows, cols, ld_dst);
  T2 a = mat(A, rows, cols, ld_a), b = mat(B, rows, cols, ld_b), c = mat(C, rows, cols, ld_c);
  switch (id) {
    case 0: d = F<sigmoid>(a * b + 0.5f * c) + repmat(vec(bias, cols), rows); break;
    case 1: d += a * 2.0f - b / c; break;
    case 2: d = F<clip_mul>(a, b) * c; break;
    case 3: d *= a + 1.5f; break;
    case 4: d -= a * b; break;
    case 5: d /= c * c + 1.0f; break;
    case 6: d = 3.25f; break;
    case 7: d = F<fma3>(a, b, c); break;
    case 8: d = broadcast<0>(vec(bias, rows), d.shape_) * a + b; break;
    default: d = F<square>(a - 1.0f) / (b * b + 2.0f) + c; break;
  }
}

void ref_reduce_keep_lowest(float *dst, const float *src, int64_t rows, int64_t cols,
                            int64_t ld, float scale, int saver, int reducer) {
  T1 d = vec(dst, cols);
  T2 s = mat(src, rows, cols, ld);
  if (reducer == 0) keep_lowest<red::sum>(d, s, scale, saver);
  else if (reducer == 1) keep_lowest<red::maximum>(d, s, scale, saver);
  else keep_lowest<red::minimum>(d, s, scale, saver);
}

void ref_reduce_keep_highdim(float *dst, const float *src, int64_t n, int64_t c, int64_t h,
                             int64_t w, int64_t ld, float scale, int saver, int reducer) {
  T1 d = vec(dst, c);
  T4 s = img(src, n, c, h, w, ld);
  if (reducer == 0) keep_dim1<red::sum>(d, s, scale, saver);
  else if (reducer == 1) keep_dim1<red::maximum>(d, s, scale, saver);
  else keep_dim1<red::minimum>(d, s, scale, saver);
}

void ref_softmax(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst,
                 int64_t ld_src) {
  Softmax(mat(dst, rows, cols, ld_dst), mat(src, rows, cols, ld_src));
}

void ref_softmax_grad(float *dst, const float *src, const float *label, int64_t rows,
                      int64_t cols, int64_t ld_dst, int64_t ld_src, int mode,
                      float ignore_label, float alpha) {
  T2 d = mat(dst, rows, cols, ld_dst), s = mat(src, rows, cols, ld_src);
  T1 l = vec(label, rows);
  switch (mode & 3) {
    case 0: SoftmaxGrad(d, s, l); break;
    case 1: SmoothSoftmaxGrad(d, s, l, alpha); break;
    case 2: SoftmaxGrad(d, s, l, ignore_label); break;
    default: SmoothSoftmaxGrad(d, s, l, ignore_label, alpha); break;
  }
}

void ref_pool(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky,
              int kx, int sy, int sx, int64_t ld_src, int64_t ld_dst, int reducer) {
  const int64_t ph = (h - ky) / sy + 1, pw = (w - kx) / sx + 1;
  T4 s = img(src, 1, planes, h, w, ld_src), d = img(dst, 1, planes, ph, pw, ld_dst);
  if (reducer == 0) d = pool<red::sum>(s, ky, kx, sy, sx);
  else if (reducer == 1) d = pool<red::maximum>(s, ky, kx, sy, sx);
  else d = pool<red::minimum>(s, ky, kx, sy, sx);
}

void ref_unpool(float *dst, const float *src, const float *pooled, const float *gpooled,
                int64_t planes, int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx,
                int sy, int sx, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst,
                int reducer) {
  T4 s = img(src, 1, planes, h, w, ld_src), d = img(dst, 1, planes, h, w, ld_dst);
  T4 p = img(pooled, 1, planes, ph, pw, ld_pooled), g = img(gpooled, 1, planes, ph, pw, ld_pooled);
  if (reducer == 0) d = unpool<red::sum>(s, p, g, ky, kx, sy, sx);
  else if (reducer == 1) d = unpool<red::maximum>(s, p, g, ky, kx, sy, sx);
  else d = unpool<red::minimum>(s, p, g, ky, kx, sy, sx);
}

void ref_chpool(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                int nsize, int stride, int pad, int64_t ld_src, int64_t ld_dst, int reducer) {
  const int64_t co = (c - nsize + pad * 2 + 1) / stride;
  T4 s = img(src, n, c, h, w, ld_src), d = img(dst, n, co, h, w, ld_dst);
  if (reducer == 0) d = chpool<red::sum>(s, nsize, stride, pad);
  else if (reducer == 1) d = chpool<red::maximum>(s, nsize, stride, pad);
  else d = chpool<red::minimum>(s, nsize, stride, pad);
}

void ref_ch_unpool(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t n,
                   int64_t c, int64_t pc, int64_t h, int64_t w, int nsize, int stride, int pad, int64_t ld_src,
                   int64_t ld_pooled, int64_t ld_dst, int reducer) {
  T4 s = img(src, n, c, h, w, ld_src), d = img(dst, n, c, h, w, ld_dst);
  T4 p = img(pooled, n, pc, h, w, ld_pooled), g = img(gpooled, n, pc, h, w, ld_pooled);
  if (reducer == 0) d = ch_unpool<red::sum>(s, p, g, nsize, stride, pad);
  else if (reducer == 1) d = ch_unpool<red::maximum>(s, p, g, nsize, stride, pad);
  else d = ch_unpool<red::minimum>(s, p, g, nsize, stride, pad);
}

void ref_lrn_forward(float *out, float *norm, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int nsize,
                     float salpha, float beta, float knorm, int power_kind) {
  T4 o = img(out, n, c, h, w, w), nm = img(norm, n, c, h, w, w), s = img(src, n, c, h, w, w);
  if (power_kind == 0) lrn_forward_impl<power>(o, nm, s, nsize, salpha, beta, knorm);
  else lrn_forward_impl<power_by_roots>(o, nm, s, nsize, salpha, beta, knorm);
}

void ref_lrn_backward(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n, int64_t c,
                      int64_t h, int64_t w, int nsize, float salpha, float beta, int power_kind) {
  T4 g = img(gsrc, n, c, h, w, w), go = img(gout, n, c, h, w, w), s = img(src, n, c, h, w, w),
     nm = img(norm, n, c, h, w, w);
  if (power_kind == 0) lrn_backward_impl<power>(g, go, s, nm, nsize, salpha, beta);
  else lrn_backward_impl<power_by_roots>(g, go, s, nm, nsize, salpha, beta);
}

void ref_addtakegrad(float *dst, const int32_t *index, const float *src, int64_t k, int64_t d,
                     int64_t nidx, int64_t ld_dst, int64_t ld_src) {
  Tensor<cpu, 1, int32_t> idx(const_cast<int32_t *>(index), Shape1(nidx), nidx, NULL);
  AddTakeGrad(mat(dst, k, d, ld_dst), idx, mat(src, nidx, d, ld_src));
}

void ref_addtakegrad_largebatch(float *dst, const int32_t *sorted, const int32_t *index,
                                const float *src, int64_t k, int64_t d, int64_t nidx) {
  Tensor<cpu, 1, int32_t> s(const_cast<int32_t *>(sorted), Shape1(nidx), nidx, NULL);
  Tensor<cpu, 1, int32_t> i(const_cast<int32_t *>(index), Shape1(nidx), nidx, NULL);
  AddTakeGradLargeBatch(mat(dst, k, d, d), s, i, mat(src, nidx, d, d));
}

void ref_sort_by_key(int32_t *keys, int32_t *values, int64_t n, int ascend) {
  Tensor<cpu, 1, int32_t> k(keys, Shape1(n), n, NULL), v(values, Shape1(n), n, NULL);
  SortByKey(k, v, ascend != 0);
}

void ref_softmax3d(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos,
                   int64_t ld_dst, int64_t ld_src) {
  typedef Tensor<cpu, 3, float> T3;
  T3 d(dst, Shape3(batch, classes, npos), static_cast<index_t>(ld_dst), NULL);
  T3 s(const_cast<float *>(src), Shape3(batch, classes, npos), static_cast<index_t>(ld_src), NULL);
  Softmax(d, s);
}

void ref_softmax_grad3d(float *dst, const float *src, const float *label, int64_t batch,
                        int64_t classes, int64_t npos, int64_t ld_dst, int64_t ld_src,
                        int64_t ld_label, int mode, float ignore_label, float alpha) {
  typedef Tensor<cpu, 3, float> T3;
  T3 d(dst, Shape3(batch, classes, npos), static_cast<index_t>(ld_dst), NULL);
  T3 s(const_cast<float *>(src), Shape3(batch, classes, npos), static_cast<index_t>(ld_src), NULL);
  T2 l = mat(label, batch, npos, ld_label);
  switch (mode & 3) {
    case 0: SoftmaxGrad(d, s, l); break;
    case 1: SmoothSoftmaxGrad(d, s, l, alpha); break;
    case 2: SoftmaxGrad(d, s, l, ignore_label); break;
    default: SmoothSoftmaxGrad(d, s, l, ignore_label, alpha); break;
  }
}

void ref_index_fill(float *dst, const int32_t *index, const float *src, int64_t d, int64_t nidx,
                    int64_t ld_dst, int64_t ld_src) {
  /* the destination's row count is not consulted by the reference; any bound >= max(index)+1 serves */
  int64_t k = 1;
  for (int64_t y = 0; y < nidx; ++y) k = index[y] + 1 > k ? index[y] + 1 : k;
  Tensor<cpu, 1, int32_t> idx(const_cast<int32_t *>(index), Shape1(nidx), nidx, NULL);
  IndexFill(mat(dst, k, d, ld_dst), idx, mat(src, nidx, d, ld_src));
}

void ref_vectorized_sort(float *values, int32_t *segments, int64_t n) {
  Tensor<cpu, 1, float> v(values, Shape1(n), n, NULL);
  Tensor<cpu, 1, int32_t> s(segments, Shape1(n), n, NULL);
  VectorizedSort(v, s);
}

void ref_remap_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                     int64_t o[4]) {
  /* shapes come from the reference's own expression objects */
  float dummy = 0.0f;
  T4 a = img(&dummy, n, c, h, w, w);
  Shape<4> s = a.shape_;
  switch (id) {
    case 0: s = reshape(a, Shape4(n, h, c, w)).shape_; break;
    case 1: s = slice<1>(a, p0, p1).shape_; break;
    case 2: s = slice<3>(a, p0, p1).shape_; break;
    case 3: s = concat<1>(a, a).shape_; break;
    case 4: s = concat<3>(a, a).shape_; break;
    case 5: s = swapaxis<2, 1>(a).shape_; break;
    case 6: s = swapaxis<3, 1>(a).shape_; break;
    case 7: s = transpose(a, Shape4(0, 2, 1, 3)).shape_; break;
    case 8: s = transpose(a, Shape4(3, 1, 0, 2)).shape_; break;
    case 9: s = pad(a, p0, p1).shape_; break;
    case 10: s = crop(a, Shape2(p0, p1)).shape_; break;
    case 11: s = crop(a, Shape2(p0, p1), h - p0, w - p1).shape_; break;
    case 15: s[0] = 2 * n; break;
    default: break;
  }
  for (int i = 0; i < 4; ++i) o[i] = s[i];
}

void ref_remap_case(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c,
                    int64_t h, int64_t w, int64_t p0, int64_t p1) {
  int64_t o[4];
  ref_remap_shape(id, n, c, h, w, p0, p1, o);
  T4 a = img(A, n, c, h, w, w), b = img(B, n, c, h, w, w);
  T4 d = img(dst, o[0], o[1], o[2], o[3], o[3]);
  switch (id) {
    case 0: d = reshape(a, Shape4(n, h, c, w)); break;
    case 1: d = slice<1>(a, p0, p1); break;
    case 2: d = slice<3>(a, p0, p1); break;
    case 3: d = concat<1>(a, b); break;
    case 4: d = concat<3>(a, b); break;
    case 5: d = swapaxis<2, 1>(a); break;
    case 6: d = swapaxis<3, 1>(a); break;
    case 7: d = transpose(a, Shape4(0, 2, 1, 3)); break;
    case 8: d = transpose(a, Shape4(3, 1, 0, 2)); break;
    case 9: d = pad(a, p0, p1); break;
    case 10: d = crop(a, Shape2(p0, p1)); break;
    case 11: d = crop(a, Shape2(p0, p1), h - p0, w - p1); break;
    case 12: d = mirror(a); break;
    case 13: d = flip(a, 1); break;
    case 14:
      Copy(d, b);
      slice<1>(d, p0, p1) = slice<1>(a, p0, p1) + 1.0f;
      break;
    case 15: {
      T4 d1 = img(dst, n, c, h, w, w), d2 = img(dst + n * c * h * w, n, c, h, w, w);
      concat<1>(d1, d2) = F<op::identity>(concat<1>(b, a));
    } break;
    default: d = crop(pad(a, p0, p1), Shape2(h, w)) + mirror(a); break;
  }
}

void ref_select_case(int id, float *dst, const float *A, const float *B, const float *idx_r,
                     const float *idx_c, int64_t rows, int64_t cols, int64_t p0) {
  T2 a = mat(A, rows, cols, cols), b = mat(B, rows, cols, cols);
  T1 ir = vec(idx_r, rows), ic = vec(idx_c, rows), val = vec(B, rows);
  T2 d = mat(dst, rows, cols, cols);
  switch (id) {
    case 0: d = take(ir, a); break;
    case 1: d = one_hot_encode(ic, cols); break;
    case 2: {
      T1 d1 = vec(dst, rows);
      d1 = mat_choose_row_element(a, ic);
    } break;
    case 3: d = mat_fill_row_element(a, val, ic); break;
    case 4: d = mask(ic, a); break;
    case 5: {
      T2 up = mat(dst, rows * p0, cols * p0, cols * p0);
      up = upsampling_nearest(a, p0);
    } break;
    case 6: d = take_grad(ir, a, rows); break;
    default: d = take(ir, a) * b + one_hot_encode(ic, cols); break;
  }
}

void ref_unpack_patch2col(float *matp, const float *imgp, int64_t n, int64_t c, int64_t h, int64_t w,
                          int psy, int psx, int sy, int sx, int dy, int dx) {
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  T2 m = mat(matp, (int64_t)psy * psx * c, oh * ow * n, oh * ow * n);
  m = unpack_patch2col(img(imgp, n, c, h, w, w), psy, psx, sy, sx, dy, dx);
}

void ref_pack_col2patch(float *imgp, const float *matp, int64_t n, int64_t c, int64_t h, int64_t w,
                        int psy, int psx, int sy, int sx, int dy, int dx) {
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  T4 d = img(imgp, n, c, h, w, w);
  d = pack_col2patch(mat(matp, (int64_t)psy * psx * c, oh * ow * n, oh * ow * n), d.shape_, psy, psx, sy, sx, dy, dx);
}

extern "C++" {
namespace {
/* stand-in for the callers' dynamic shape type that broadcast_multi_axes / broadcast_to are templated on */
struct DynShape {
  std::vector<index_t> v;
  DynShape() {}
  template <typename It>
  DynShape(It b, It e) : v(b, e) {}
  index_t ndim() const { return static_cast<index_t>(v.size()); }
  index_t operator[](size_t i) const { return v[i]; }
};
inline std::ostream &operator<<(std::ostream &os, const DynShape &s) {
  for (size_t i = 0; i < s.v.size(); ++i) os << (i ? "," : "(") << s.v[i];
  return os << ")";
}
inline void axis_box(int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, Shape<4> *b, Shape<4> *e) {
  *b = Shape4(p0 % n, p1 % c, p0 % h, p1 % w);
  *e = Shape4(n, c, (*b)[2] + (h - (*b)[2] + 1) / 2, w);
}
template <int dim>
inline Tensor<cpu, dim, float> dense(const float *p, Shape<dim> s) {
  return Tensor<cpu, dim, float>(const_cast<float *>(p), s, s[dim - 1], NULL);
}
template <int dim>
inline int put_shape(Shape<dim> s, int64_t o[4]) {
  for (int i = 0; i < 4; ++i) o[i] = i < dim ? s[i] : 1;
  return dim;
}
}  // namespace
}  // extern "C++"

int ref_axis_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t o[4]) {
  /* shapes come from the reference's own expression objects */
  float dummy = 0.0f;
  T4 a = img(&dummy, n, c, h, w, w);
  Shape<4> b, e;
  axis_box(n, c, h, w, p0, p1, &b, &e);
  std::vector<index_t> ax(2), sz(2);
  switch (id) {
    case 0: return put_shape(ShapeCheck<1, RangeExp<float> >::Check(range<float>(p0, p0 + p1, 0.5f, 2)), o);
    case 1: return put_shape(ShapeCheck<1, RangeExp<float> >::Check(range<float>(p0 + p1, p0, -1.5f, 1)), o);
    case 2: return put_shape(slice(a, b, e).shape_, o);
    case 3: return put_shape(a.shape_, o);
    case 4: return put_shape(reduce_with_axis<red::sum, false>(a, p0).shape_, o);
    case 5: return put_shape(reduce_with_axis<red::maximum, true>(a, p0).shape_, o);
    case 6: return put_shape(reduce_keepdim<red::minimum, false>(a, p0).shape_, o);
    case 7: return put_shape(broadcast_with_axis(dense(&dummy, Shape3(n * c, h, w)), p0 - 1, p1).shape_, o);
    case 8: return put_shape(broadcast_keepdim(slice<1>(a, 0, 1), 1, p1).shape_, o);
    case 9: {
      sz.resize(4);
      sz[0] = n; sz[1] = p0; sz[2] = h; sz[3] = p1;
      return put_shape(broadcast_to(dense(&dummy, Shape4(n, 1, h, 1)), DynShape(sz.begin(), sz.end())).shape_, o);
    }
    default:
      ax[0] = 0; ax[1] = 2; sz[0] = p0; sz[1] = p1;
      return put_shape(broadcast_multi_axes(dense(&dummy, Shape4(1, c, 1, w)), DynShape(ax.begin(), ax.end()),
                                            DynShape(sz.begin(), sz.end())).shape_, o);
  }
}

void ref_axis_case(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0,
                   int64_t p1) {
  int64_t o[4];
  ref_axis_shape(id, n, c, h, w, p0, p1, o);
  T4 a = img(A, n, c, h, w, w);
  T4 d4 = dense(dst, Shape4(o[0], o[1], o[2], o[3]));
  Tensor<cpu, 3, float> d3 = dense(dst, Shape3(o[0], o[1], o[2]));
  T1 d1 = vec(dst, o[0]);
  Shape<4> b, e;
  axis_box(n, c, h, w, p0, p1, &b, &e);
  std::vector<index_t> ax(2), sz(2);
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
    case 7: d4 = broadcast_with_axis(dense(A, Shape3(n * c, h, w)), p0 - 1, p1); break;
    case 8: d4 = broadcast_keepdim(slice<1>(a, 0, 1), 1, p1); break;
    case 9:
      sz.resize(4);
      sz[0] = n; sz[1] = p0; sz[2] = h; sz[3] = p1;
      d4 = broadcast_to(dense(A, Shape4(n, 1, h, 1)), DynShape(sz.begin(), sz.end()));
      break;
    default:
      ax[0] = 0; ax[1] = 2; sz[0] = p0; sz[1] = p1;
      d4 = broadcast_multi_axes(dense(A, Shape4(1, c, 1, w)), DynShape(ax.begin(), ax.end()),
                                DynShape(sz.begin(), sz.end()));
      break;
  }
}

void ref_complex_case(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols) {
  T2 a = mat(A, rows, cols, cols), b = mat(B, rows, cols, cols);
  T2 ah = mat(A, rows, cols / 2, cols / 2), bh = mat(B, rows, cols / 2, cols / 2);
  T2 d = mat(dst, rows, cols, cols), dh = mat(dst, rows, cols / 2, cols / 2);
  switch (id) {
    case 0: d = complex_mul_cc(a, b); break;
    case 1: d = complex_mul_cr(a, bh); break;
    case 2: d = complex_mul_rc(ah, b); break;
    case 3: d = complex_div_cc(a, b); break;
    case 4: d = complex_div_cr(a, bh); break;
    case 5: d = complex_div_rc(ah, b); break;
    case 6: d = conj(a); break;
    case 7: d = complex_exchange(a); break;
    case 8: d = complex_pad_imag(ah); break;
    case 9: dh = complex_toreal(a); break;
    case 10: dh = complex_abs_square(a); break;
    case 11: dh = complex_sum_real_imag(a); break;
    default: d = complex_mul_cc(conj(a), b) + complex_pad_imag(complex_abs_square(b)) * 0.5f; break;
  }
}

int ref_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void ref_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

}  // extern "C"
