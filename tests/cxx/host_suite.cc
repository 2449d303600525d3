/*
 * Host-side conformance library: the engine's headers evaluated on Tensor<cpu>, compiled by
 * g++ without CUDA.  An expression plan's Eval(y, x) is the same code on both devices, so the
 * index arithmetic of every index-remapping plan can be checked here, on a machine without a
 * GPU, against the CPU oracle.  Test code only; not part of the product library.
 */
#include <cstdint>
#include <cstring>
#include <string>

#include "mshadow/tensor.h"
#include "../../mshadow_b200/csrc/axis_cases.h"
#include "../../mshadow_b200/csrc/complex_cases.h"

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

namespace {
typedef Tensor<cpu, 4, float> H4;
std::string g_error;

inline H4 Img(const float *p, int64_t n, int64_t c, int64_t h, int64_t w) {
  return H4(const_cast<float *>(p), Shape4(n, c, h, w), static_cast<index_t>(w), nullptr);
}

Shape<4> RemapShape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1) {
  const H4 a = Img(nullptr, n, c, h, w);
  switch (id) {
    case 0: return reshape(a, Shape4(n, h, c, w)).shape_;
    case 1: return slice<1>(a, p0, p1).shape_;
    case 2: return slice<3>(a, p0, p1).shape_;
    case 3: return concat<1>(a, a).shape_;
    case 4: return concat<3>(a, a).shape_;
    case 5: return swapaxis<2, 1>(a).shape_;
    case 6: return swapaxis<3, 1>(a).shape_;
    case 7: return transpose(a, Shape4(0, 2, 1, 3)).shape_;
    case 8: return transpose(a, Shape4(3, 1, 0, 2)).shape_;
    case 9: return pad(a, p0, p1).shape_;
    case 10: return crop(a, Shape2(p0, p1)).shape_;
    case 11: return crop(a, Shape2(p0, p1), h - p0, w - p1).shape_;
    case 15: return Shape4(2 * n, c, h, w);
    default: return a.shape_;
  }
}
}  // namespace

extern "C" {

const char *hostmsb_last_error(void) { return g_error.c_str(); }

/* the cases of msb_select_case_f32, on host memory; returns 0, or 1 when a CHECK of the engine fired */
int hostmsb_select_case(int id, float *dst, const float *A, const float *B, const float *idx_r, const float *idx_c,
                        int64_t rows, int64_t cols, int64_t p0) {
  typedef Tensor<cpu, 2, float> H2;
  typedef Tensor<cpu, 1, float> H1;
  try {
    const H2 a(const_cast<float *>(A), Shape2(rows, cols)), b(const_cast<float *>(B), Shape2(rows, cols));
    const H1 ir(const_cast<float *>(idx_r), Shape1(rows)), ic(const_cast<float *>(idx_c), Shape1(rows));
    const H1 val(const_cast<float *>(B), Shape1(rows));
    H2 d(dst, Shape2(rows, cols));
    switch (id) {
      case 0: d = take(ir, a); break;
      case 1: d = one_hot_encode(ic, cols); break;
      case 2: {
        H1 d1(dst, Shape1(rows));
        d1 = mat_choose_row_element(a, ic);
      } break;
      case 3: d = mat_fill_row_element(a, val, ic); break;
      case 4: d = mask(ic, a); break;
      case 5: {
        H2 up(dst, Shape2(rows * p0, cols * p0));
        up = upsampling_nearest(a, p0);
      } break;
      case 6: d = take_grad(ir, a, rows); break;
      default: d = take(ir, a) * b + one_hot_encode(ic, cols); break;
    }
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

/* patch <-> column conversion on host memory; direction 0 = unpack (img -> mat), 1 = pack (mat -> img) */
int hostmsb_patch(int direction, float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int psy,
                  int psx, int sy, int sx, int dy, int dx) {
  typedef Tensor<cpu, 2, float> H2;
  try {
    const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
    const Shape<2> mshape = Shape2(static_cast<index_t>(psy) * psx * c, oh * ow * n);
    if (direction == 0) {
      H2 m(dst, mshape);
      m = unpack_patch2col(Img(src, n, c, h, w), psy, psx, sy, sx, dy, dx);
    } else {
      H4 d = Img(dst, n, c, h, w);
      d = pack_col2patch(H2(const_cast<float *>(src), mshape), d.shape_, psy, psx, sy, sx, dy, dx);
    }
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

/* binary16 conversions of mshadow::half::half_t as the host performs them */
void hostmsb_half_from_float(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = mshadow::half::half_t(src[i]).half_;
}
void hostmsb_half_to_float(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = static_cast<float>(mshadow::half::half_t::Binary(src[i]));
}
/* dst = a * b + a * 0.5 - b / (a * a + 2) on binary16 host tensors, every operation rounded to half */
void hostmsb_half_expr(const uint16_t *a, const uint16_t *b, uint16_t *dst, int64_t rows, int64_t cols) {
  typedef mshadow::half::half_t H;
  Tensor<cpu, 2, H> A(reinterpret_cast<H *>(const_cast<uint16_t *>(a)), Shape2(rows, cols));
  Tensor<cpu, 2, H> B(reinterpret_cast<H *>(const_cast<uint16_t *>(b)), Shape2(rows, cols));
  Tensor<cpu, 2, H> D(reinterpret_cast<H *>(dst), Shape2(rows, cols));
  D = A * B + A * H(0.5f) - B / (A * A + H(2.0f));
}

/* the cases of msb_complex_case_f32, on host memory; returns 0, 1 when a CHECK of the engine fired, 2 when the
   arguments are outside the domain */
int hostmsb_complex_case(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols) {
  if (!msb_complex::ArgsOk(id, rows, cols)) return 2;
  try {
    msb_complex::Run<cpu>(id, dst, A, B, rows, cols, static_cast<Stream<cpu> *>(nullptr));
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

/* a complex product of operands whose widths do not match: the shape rule must fire */
int hostmsb_complex_shape_error(void) {
  float buf[24] = {0};
  Tensor<cpu, 2, float> a(buf, Shape2(2, 6)), b(buf, Shape2(2, 4)), d(buf + 12, Shape2(2, 6));
  try {
    d = complex_mul_cr(a, b);  // a real operand must be half as wide as the complex one
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

/* reciprocal division against `/` and `%`: returns the number of (divisor, number) pairs that disagree */
int64_t hostmsb_fastdiv_mismatches(const uint32_t *divisors, int64_t ndiv, const uint32_t *numbers, int64_t nnum) {
  int64_t bad = 0;
  for (int64_t i = 0; i < ndiv; ++i) {
    const FastDiv f(divisors[i]);
    const uint32_t d = divisors[i];
    for (int64_t j = 0; j < nnum + 6; ++j) {
      // the caller's numbers, and for every divisor its own multiples and their neighbours
      const uint64_t around = static_cast<uint64_t>(d) * ((1u << 31) / d);
      const uint32_t n = j < nnum ? numbers[j]
                                  : static_cast<uint32_t>(j - nnum < 3 ? d - 1 + (j - nnum) : around - 2 + (j - nnum - 3));
      if (n >= (1u << 31)) continue;
      uint32_t q;
      const uint32_t r = f.DivMod(n, &q);
      bad += (q != n / d) || (r != n % d) || (f.Quot(n) != n / d);
    }
  }
  return bad;
}

/* the cases of msb_axis_case_f32, on host memory (dst == NULL: shape query only); returns 0, 1 when a CHECK of
   the engine fired, 2 when the arguments are outside the case's domain */
int hostmsb_axis_case(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0,
                      int64_t p1, int64_t *out_shape, int *out_ndim) {
  if (id < 0 || id >= msb_axis::kNumCases || !msb_axis::ArgsOk(id, n, c, h, w, p0, p1)) return 2;
  try {
    *out_ndim = msb_axis::ResultShape<cpu>(id, n, c, h, w, p0, p1, out_shape);
    if (dst != nullptr) msb_axis::Run<cpu>(id, dst, A, n, c, h, w, p0, p1, static_cast<Stream<cpu> *>(nullptr));
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

/* the cases of msb_remap_case_f32, on host memory; returns 0, or 1 when a CHECK of the engine fired */
int hostmsb_remap_case(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c, int64_t h,
                       int64_t w, int64_t p0, int64_t p1, int64_t *out_shape) {
  try {
    const Shape<4> o = RemapShape(id, n, c, h, w, p0, p1);
    for (int i = 0; i < 4; ++i) out_shape[i] = o[i];
    if (dst == nullptr) return 0;  // shape query
    const H4 a = Img(A, n, c, h, w), b = Img(B, n, c, h, w);
    H4 d = Img(dst, o[0], o[1], o[2], o[3]);
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
        std::memcpy(dst, B, sizeof(float) * n * c * h * w);
        slice<1>(d, p0, p1) = slice<1>(a, p0, p1) + 1.0f;
        break;
      case 15: {
        H4 d1 = Img(dst, n, c, h, w), d2 = Img(dst + n * c * h * w, n, c, h, w);
        concat<1>(d1, d2) = F<op::identity>(concat<1>(b, a));
      } break;
      default: d = crop(pad(a, p0, p1), Shape2(h, w)) + mirror(a); break;
    }
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
  return 0;
}

}  // extern "C"
