/*
 * Division of an index by a divisor that is fixed for a whole kernel launch, without a divide
 * instruction.  Index-remapping plans split a linear row index into coordinates for every
 * element; an integer divide costs tens of instructions on the GPU, this costs three (multiply
 * high, add, shift) and has no special case.  The reference's plans use `/` and `%` (e.g.
 * mshadow/extension/swapaxis.h:72-84).
 */
#ifndef MSHADOW_ENGINE_FASTDIV_H_
#define MSHADOW_ENGINE_FASTDIV_H_

#include <stdint.h>

#include "../base.h"

namespace mshadow {
namespace expr {

/*!
 * \brief exact quotient and remainder of a 32-bit number by a fixed divisor d (Granlund and
 *  Montgomery's round-up multiplier): with l = ceil(log2 d) and mul = floor(2^(32+l) / d) + 1 - 2^32,
 *  n / d = (mulhi(n, mul) + n) >> l.  The engine indexes below 2^31, where the sum cannot carry
 *  out of 32 bits.
 */
struct FastDiv {
  uint32_t mul;
  uint32_t shift;
  uint32_t div;
  FastDiv() : mul(1), shift(0), div(1) {}
  explicit FastDiv(uint32_t d) : div(d == 0 ? 1 : d) {
    shift = 0;
    while ((1ull << shift) < div) ++shift;
    // 2^(32+shift) / div without 128-bit arithmetic: shift <= 32, so split off the power of two
    const uint64_t two32 = 1ull << 32;
    const uint64_t pow = 1ull << shift;              // div <= pow < 2 * div
    const uint64_t q = (two32 * (pow - div)) / div;  // floor(2^32 * (pow - div) / div), below 2^32
    mul = static_cast<uint32_t>(q + 1);              // floor(2^32 * pow / div) + 1 - 2^32
  }
  MSHADOW_XINLINE uint32_t Quot(uint32_t n) const {
#ifdef __CUDA_ARCH__
    return (__umulhi(n, mul) + n) >> shift;
#else
    return static_cast<uint32_t>((((static_cast<uint64_t>(n) * mul) >> 32) + n) >> shift);
#endif
  }
  /*! \brief q = n / div, returns n % div */
  MSHADOW_XINLINE uint32_t DivMod(uint32_t n, uint32_t *q) const {
    *q = Quot(n);
    return n - *q * div;
  }
};

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_ENGINE_FASTDIV_H_
