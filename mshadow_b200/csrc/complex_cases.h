/*
 * The fixed set of complex-arithmetic expressions behind msb_complex_case_f32, written once for
 * both devices: the C ABI instantiates it for gpu, the host conformance library for cpu.  The
 * case list is documented at the declaration of msb_complex_case_f32.
 */
#ifndef MSHADOW_B200_CSRC_COMPLEX_CASES_H_
#define MSHADOW_B200_CSRC_COMPLEX_CASES_H_

#include <cstdint>

#include "mshadow/tensor.h"

namespace msb_complex {

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

const int kNumCases = 13;

/*! \brief width of the result of case `id` on rows x cols operands (cols counts floats) */
inline int64_t ResultCols(int id, int64_t cols) { return (id >= 9 && id <= 11) ? cols / 2 : cols; }

/*! \brief cols must be a multiple of 4: pairs everywhere, and pairs again after halving */
inline bool ArgsOk(int id, int64_t rows, int64_t cols) {
  return id >= 0 && id < kNumCases && rows > 0 && cols > 0 && cols % 4 == 0 && rows * cols < (int64_t(1) << 30);
}

template <typename xpu>
inline void Run(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols, Stream<xpu> *stream) {
  typedef Tensor<xpu, 2, float> M;
  const M a(const_cast<float *>(A), Shape2(rows, cols), cols, stream), b(const_cast<float *>(B), Shape2(rows, cols), cols, stream);
  // real operands: the first rows * cols / 2 floats of the same buffers, seen as rows x cols/2
  const M ah(const_cast<float *>(A), Shape2(rows, cols / 2), cols / 2, stream);
  const M bh(const_cast<float *>(B), Shape2(rows, cols / 2), cols / 2, stream);
  M d(dst, Shape2(rows, cols), cols, stream), dh(dst, Shape2(rows, cols / 2), cols / 2, stream);
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

}  // namespace msb_complex
#endif  // MSHADOW_B200_CSRC_COMPLEX_CASES_H_
