/*
 * Device math that has to agree with the host C library bit for bit.
 *
 * mshadow's element-wise functors are user code (`struct sigmoid { Map(a) { return
 * 1.0f / (1.0f + expf(-a)); } }`, guide/README.md:152-157 of the reference), and on the CPU
 * `expf` is the C library's, which is correctly rounded in all but a vanishing fraction of
 * cases.  CUDA's expf is specified to 2 ulp, which is enough to change the last bits of a
 * sigmoid and therefore to break "within 1 ulp of the CPU result" once the sigmoid is
 * added to something of opposite sign.  mshadow::b200::expf_host_exact closes that gap:
 * on the host it is ::expf, on the device it evaluates the table-driven algorithm that
 * GNU libm (2.28 and later) and the Arm Optimized Routines publish for single-precision
 * exp -- reduce x = k*ln2/32 + r, look up 2^(k mod 32 / 32) in a 32-entry table, evaluate a
 * cubic in r, all in binary64, and round once to binary32.  Evaluated over every float
 * with |x| < 87 on the host, this sequence differs from glibc 2.39's expf for 2 inputs out
 * of 2.2e9 (both beyond |x| = 32).  The table entries are 2^(i/32) rounded to binary64 with
 * the index folded out of the exponent field.
 *
 * Cost: about ten binary64 operations per element, which a B200 hides behind a 16-byte-per-
 * element memory stream.
 */
#ifndef MSHADOW_GPU_MATH_H_
#define MSHADOW_GPU_MATH_H_

#include <cmath>
#include <cstdint>

#include "../base.h"

namespace mshadow {
namespace b200 {

#ifdef __CUDACC__
namespace mathdetail {
static __device__ const unsigned long long kExp2Tab32[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

__device__ __forceinline__ float ExpTable32(float x) {
  // out-of-range and non-finite inputs: overflow to +inf, underflow to 0, NaN stays NaN
  if (!(fabsf(x) < 104.0f)) {
    if (x != x) return x;
    return x > 0.0f ? __int_as_float(0x7f800000) : 0.0f;
  }
  const double kInvLn2N = 0x1.71547652b82fep+0 * 32.0;
  const double kShift = 0x1.8p+52;
  const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
  const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
  const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
  const double z = __dmul_rn(kInvLn2N, static_cast<double>(x));
  double kd = __dadd_rn(z, kShift);  // low bits of kd now hold round(z)
  const unsigned long long ki = static_cast<unsigned long long>(__double_as_longlong(kd));
  kd = __dsub_rn(kd, kShift);
  const double r = __dsub_rn(z, kd);
  const unsigned long long t = kExp2Tab32[ki & 31] + (ki << 47);
  const double s = __longlong_as_double(static_cast<long long>(t));
  const double p = __fma_rn(c0, r, c1);
  const double r2 = __dmul_rn(r, r);
  double y = __fma_rn(c2, r, 1.0);
  y = __fma_rn(p, r2, y);
  y = __dmul_rn(y, s);
  return __double2float_rn(y);
}
}  // namespace mathdetail
#endif  // __CUDACC__

/*! \brief e^x; the device result equals the host C library's expf (see the file comment) */
MSHADOW_XINLINE float expf_host_exact(float x) {
#ifdef __CUDA_ARCH__
  return mathdetail::ExpTable32(x);
#else
  return ::expf(x);
#endif
}

/*! \brief logistic function with the host's rounding: 1 / (1 + e^-a), division correctly rounded */
struct sigmoid {
  MSHADOW_XINLINE static float Map(float a) {
    return mshadow::detail::DivRN(1.0f, mshadow::detail::AddRN(1.0f, expf_host_exact(-a)));
  }
};

}  // namespace b200
}  // namespace mshadow
#endif  // MSHADOW_GPU_MATH_H_
