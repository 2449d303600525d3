/*
 * Division of an index by a divisor that is fixed for a whole kernel launch, without a divide
 * instruction.  Index-remapping plans split a linear row index into coordinates for every
 * element; an integer divide costs tens of instructions on the GPU, a multiply-high and a shift
 * cost two.  The reference's plans use `/` and `%` (e.g. mshadow/extension/swapaxis.h:72-84).
 */
#ifndef MSHADOW_ENGINE_FASTDIV_H_
#define MSHADOW_ENGINE_FASTDIV_H_

#include <stdint.h>

#include "../base.h"

namespace mshadow {
namespace expr {

/*! \brief exact quotient and remainder of a non-negative 31-bit number by a fixed divisor */
struct FastDiv {
  uint32_t mul;
  uint32_t shift;
  uint32_t div;
  FastDiv() : mul(0), shift(0), div(1) {}
  explicit FastDiv(uint32_t d) : div(d == 0 ? 1 : d) {
    // q = (n * mul) >> (31 + ceil(log2 d)) is exact for all n < 2^31 (round-up method)
    uint32_t lg = 0;
    while ((1ull << lg) < div) ++lg;
    shift = 31 + lg;
    mul = static_cast<uint32_t>(((1ull << shift) + div - 1) / div);
  }
  MSHADOW_XINLINE uint32_t Quot(uint32_t n) const {
    return div == 1 ? n : static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> shift);
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
