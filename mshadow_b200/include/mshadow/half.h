/*
 * IEEE binary16 element type for tensors: mshadow::half::half_t, with the interface of
 * dmlc/mshadow's mshadow/half.h (:75-240): construction from the arithmetic types, conversion
 * to float, + - * / and comparisons carried out in float and rounded back (round to nearest
 * even), compound assignment, Binary() for raw bit patterns.
 *
 * For the evaluation engine a half_t tensor is just another element type: the fused
 * element-wise kernel moves EIGHT of them per 16-byte group (Pack<half_t>::kLanes == 8), every
 * functor sees half_t operands and computes through the operators below, and the result is
 * rounded once per operation, exactly as on the host.  On the device the conversions are the
 * hardware's (cvt.rn.f16.f32 / cvt.f32.f16); on the host they are done in integer arithmetic
 * with the same rounding, so host and device agree bit for bit.
 */
#ifndef MSHADOW_HALF_H_
#define MSHADOW_HALF_H_

#include <stdint.h>
#include <string.h>

#include <type_traits>

#include "./base.h"

#if MSHADOW_USE_CUDA
#include <cuda_fp16.h>
#endif

namespace mshadow {
namespace half {

namespace halfdetail {
/*! \brief float -> binary16 bits, round to nearest even, on the host */
inline uint16_t FloatToBitsHost(float value) {
  uint32_t f;
  memcpy(&f, &value, sizeof(f));
  const uint16_t sign = static_cast<uint16_t>((f >> 16) & 0x8000u);
  const uint32_t mag = f & 0x7fffffffu;
  if (mag >= 0x7f800000u) {  // infinity or NaN (NaN keeps a quiet payload bit)
    return static_cast<uint16_t>(sign | 0x7c00u | (mag > 0x7f800000u ? 0x0200u | ((mag >> 13) & 0x03ffu) : 0u));
  }
  if (mag >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);  // rounds to infinity (>= 65520)
  if (mag < 0x33000001u) return sign;                                     // rounds to zero (<= 2^-25)
  const int32_t exp = static_cast<int32_t>(mag >> 23) - 127;
  uint32_t mant = (mag & 0x007fffffu) | 0x00800000u;
  uint32_t shift;
  uint32_t base;
  if (exp < -14) {  // subnormal result: value = mant * 2^(exp-23), unit 2^-24
    shift = static_cast<uint32_t>(-exp - 1);  // 13 + (-14 - exp)
    base = 0;
  } else {
    shift = 13;
    base = static_cast<uint32_t>(exp + 15) << 10;
    mant &= 0x007fffffu;
  }
  uint32_t half = base + (mant >> shift);
  const uint32_t rem = mant & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half & 1u))) ++half;  // a carry into the exponent is the right result
  return static_cast<uint16_t>(sign | half);
}
/*! \brief binary16 bits -> float, exact, on the host */
inline float BitsToFloatHost(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu, mant = h & 0x03ffu;
  uint32_t f;
  if (exp == 0x1fu) {
    f = sign | 0x7f800000u | (mant << 13);
  } else if (exp != 0) {
    f = sign | ((exp + 112u) << 23) | (mant << 13);
  } else if (mant == 0) {
    f = sign;
  } else {  // subnormal: normalise
    uint32_t m = mant, e = 113;
    while ((m & 0x0400u) == 0) {
      m <<= 1;
      --e;
    }
    f = sign | (e << 23) | ((m & 0x03ffu) << 13);
  }
  float out;
  memcpy(&out, &f, sizeof(out));
  return out;
}
}  // namespace halfdetail

class MSHADOW_ALIGNED(2) half_t {
 public:
  uint16_t half_;

  MSHADOW_XINLINE half_t() {}
  MSHADOW_XINLINE half_t(const float &value) : half_(FromFloat(value)) {}  // NOLINT(*) implicit, as in the reference
  MSHADOW_XINLINE explicit half_t(const double &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const int8_t &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const uint8_t &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const int32_t &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const uint32_t &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const int64_t &value) : half_(FromFloat(static_cast<float>(value))) {}
  MSHADOW_XINLINE explicit half_t(const uint64_t &value) : half_(FromFloat(static_cast<float>(value))) {}

  /*! \brief the value whose bit pattern is `bits` */
  MSHADOW_XINLINE static half_t Binary(uint16_t bits) {
    half_t r;
    r.half_ = bits;
    return r;
  }
  MSHADOW_XINLINE operator float() const { return ToFloat(half_); }  // NOLINT(*)

  MSHADOW_XINLINE half_t operator+() const { return *this; }
  MSHADOW_XINLINE half_t operator-() const { return Binary(static_cast<uint16_t>(half_ ^ 0x8000u)); }
  template <typename T>
  MSHADOW_XINLINE half_t &operator+=(const T &a) {
    return *this = half_t(static_cast<float>(*this) + static_cast<float>(a));
  }
  template <typename T>
  MSHADOW_XINLINE half_t &operator-=(const T &a) {
    return *this = half_t(static_cast<float>(*this) - static_cast<float>(a));
  }
  template <typename T>
  MSHADOW_XINLINE half_t &operator*=(const T &a) {
    return *this = half_t(static_cast<float>(*this) * static_cast<float>(a));
  }
  template <typename T>
  MSHADOW_XINLINE half_t &operator/=(const T &a) {
    return *this = half_t(static_cast<float>(*this) / static_cast<float>(a));
  }

 private:
  MSHADOW_XINLINE static uint16_t FromFloat(float value) {
#if defined(__CUDA_ARCH__)
    return __half_as_ushort(__float2half_rn(value));
#else
    return halfdetail::FloatToBitsHost(value);
#endif
  }
  MSHADOW_XINLINE static float ToFloat(uint16_t bits) {
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half(bits));
#else
    return halfdetail::BitsToFloatHost(bits);
#endif
  }
};

// arithmetic and comparisons (with half_t or any arithmetic type on the other side): in float,
// one rounding back to half per operation.  The
// products and sums go through the no-contraction helpers, so `a * b + c` on half_t is two
// roundings to float and two to half on either device.
#define MSHADOW_B200_HALF_ARITH_(OP, FN)                                                                        \
  MSHADOW_XINLINE half_t operator OP(half_t a, half_t b) {                                                      \
    return half_t(detail::FN<float>(static_cast<float>(a), static_cast<float>(b)));                             \
  }                                                                                                             \
  template <typename T, typename = typename std::enable_if<std::is_arithmetic<T>::value>::type>                 \
  MSHADOW_XINLINE half_t operator OP(half_t a, T b) {                                                           \
    return half_t(detail::FN<float>(static_cast<float>(a), static_cast<float>(b)));                             \
  }                                                                                                             \
  template <typename T, typename = typename std::enable_if<std::is_arithmetic<T>::value>::type>                 \
  MSHADOW_XINLINE half_t operator OP(T a, half_t b) {                                                           \
    return half_t(detail::FN<float>(static_cast<float>(a), static_cast<float>(b)));                             \
  }
MSHADOW_B200_HALF_ARITH_(+, AddRN)
MSHADOW_B200_HALF_ARITH_(-, SubRN)
MSHADOW_B200_HALF_ARITH_(*, MulRN)
MSHADOW_B200_HALF_ARITH_(/, DivRN)
#undef MSHADOW_B200_HALF_ARITH_

#define MSHADOW_B200_HALF_COMPARE_(OP)                                                                          \
  MSHADOW_XINLINE bool operator OP(half_t a, half_t b) { return static_cast<float>(a) OP static_cast<float>(b); } \
  template <typename T, typename = typename std::enable_if<std::is_arithmetic<T>::value>::type>                 \
  MSHADOW_XINLINE bool operator OP(half_t a, T b) {                                                             \
    return static_cast<float>(a) OP static_cast<float>(b);                                                      \
  }                                                                                                             \
  template <typename T, typename = typename std::enable_if<std::is_arithmetic<T>::value>::type>                 \
  MSHADOW_XINLINE bool operator OP(T a, half_t b) {                                                             \
    return static_cast<float>(a) OP static_cast<float>(b);                                                      \
  }
MSHADOW_B200_HALF_COMPARE_(>)
MSHADOW_B200_HALF_COMPARE_(<)
MSHADOW_B200_HALF_COMPARE_(>=)
MSHADOW_B200_HALF_COMPARE_(<=)
MSHADOW_B200_HALF_COMPARE_(==)
MSHADOW_B200_HALF_COMPARE_(!=)
#undef MSHADOW_B200_HALF_COMPARE_

/*! \brief largest and lowest finite values */
#define MSHADOW_HALF_MAX mshadow::half::half_t::Binary(0x7BFF)
#define MSHADOW_HALF_MIN mshadow::half::half_t::Binary(0xFBFF)

}  // namespace half

template <>
struct DataType<half::half_t> {
  static const int kFlag = kFloat16;
  static const int kLanes = 1;
};

namespace red {
namespace limits {
template <>
MSHADOW_XINLINE half::half_t MinValue<half::half_t>() {
  return MSHADOW_HALF_MIN;
}
template <>
MSHADOW_XINLINE half::half_t MaxValue<half::half_t>() {
  return MSHADOW_HALF_MAX;
}
}  // namespace limits
}  // namespace red

}  // namespace mshadow
#endif  // MSHADOW_HALF_H_
