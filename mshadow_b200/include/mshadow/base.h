/*
 * Build configuration, scalar types and the functor vocabulary (op::, sv::, red::) of the
 * mshadow API, re-implemented for the B200 evaluation engine.  Names, template parameters
 * and semantics follow dmlc/mshadow's mshadow/base.h (macros :49-276, index_t :288-292,
 * type flags :306-413, op:: :483-537, sv:: :539-602, red:: :604-862) so that user code
 * written against it compiles unchanged; the bodies are new.
 *
 * One deliberate difference: on the device, the float and double arithmetic functors use
 * round-to-nearest intrinsics that the compiler may not contract into fused multiply-adds.
 * mshadow's CPU evaluator performs a*b+c as two rounded operations; keeping that on the GPU
 * is what makes `+ - * /` expressions bit-identical between the two devices.
 */
#ifndef MSHADOW_BASE_H_
#define MSHADOW_BASE_H_

#include <cfloat>
#include <climits>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <functional>
#include <sstream>
#include <string>

// ---------------------------------------------------------------------------------------
// configuration switches (same names and defaults as the reference where they matter here)
// ---------------------------------------------------------------------------------------
#ifndef MSHADOW_STAND_ALONE
#define MSHADOW_STAND_ALONE 0
#endif
#ifndef MSHADOW_ALLOC_PAD
#define MSHADOW_ALLOC_PAD true
#endif
#ifndef MSHADOW_MIN_PAD_RATIO
#define MSHADOW_MIN_PAD_RATIO 2
#endif
#ifndef MSHADOW_FORCE_STREAM
#define MSHADOW_FORCE_STREAM 1
#endif
#ifndef MSHADOW_USE_CUDA
#if MSHADOW_STAND_ALONE
#define MSHADOW_USE_CUDA 0
#else
#define MSHADOW_USE_CUDA 1
#endif
#endif
#ifndef MSHADOW_INT64_TENSOR_SIZE
#define MSHADOW_INT64_TENSOR_SIZE 0
#endif
// BLAS / cuDNN / cuSOLVER bridges are not part of this engine
#ifndef MSHADOW_USE_CBLAS
#define MSHADOW_USE_CBLAS 0
#endif
#ifndef MSHADOW_USE_MKL
#define MSHADOW_USE_MKL 0
#endif
#ifndef MSHADOW_USE_CUDNN
#define MSHADOW_USE_CUDNN 0
#endif
#ifndef MSHADOW_USE_CUSOLVER
#define MSHADOW_USE_CUSOLVER 0
#endif
#define MSHADOW_IN_CXX11 1

#if MSHADOW_USE_CUDA
#include <cuda_runtime.h>
#endif

#ifdef MSHADOW_XINLINE
#error "MSHADOW_XINLINE must not be defined"
#endif
#define MSHADOW_FORCE_INLINE inline __attribute__((always_inline))
#ifdef __CUDACC__
#define MSHADOW_XINLINE MSHADOW_FORCE_INLINE __device__ __host__
#else
#define MSHADOW_XINLINE MSHADOW_FORCE_INLINE
#endif
#define MSHADOW_CINLINE MSHADOW_FORCE_INLINE
#define MSHADOW_CONSTEXPR constexpr
#define MSHADOW_ALIGNED(x) __attribute__((aligned(x)))
#define MSHADOW_THROW_EXCEPTION noexcept(false)
#define MSHADOW_NO_EXCEPTION noexcept(true)
#ifndef MSHADOW_DEFAULT_DTYPE
#define MSHADOW_DEFAULT_DTYPE = ::mshadow::default_real_t
#endif

#include "./logging.h"

/*! \brief abort (or throw) with the CUDA error string when a runtime call fails */
#define MSHADOW_CUDA_CALL(func)                                           \
  {                                                                       \
    cudaError_t msh_err_ = (func);                                        \
    CHECK(msh_err_ == cudaSuccess) << "CUDA: " << cudaGetErrorString(msh_err_); \
  }

namespace mshadow {

const unsigned kRandBufferSize = 1000000;
const float kPi = 3.1415926f;

#if MSHADOW_INT64_TENSOR_SIZE == 1
typedef int64_t index_t;
#else
typedef int32_t index_t;
#endif
typedef index_t openmp_index_t;
typedef float default_real_t;

/*! \brief run-time tag of an element type */
enum TypeFlag {
  kFloat32 = 0,
  kFloat64 = 1,
  kFloat16 = 2,
  kUint8 = 3,
  kInt32 = 4,
  kInt8 = 5,
  kInt64 = 6,
};

template <typename DType>
struct DataType;
#define MSHADOW_B200_DATATYPE_(T, FLAG, LANES)   \
  template <>                                    \
  struct DataType<T> {                           \
    static const int kFlag = FLAG;               \
    static const int kLanes = LANES;             \
  }
MSHADOW_B200_DATATYPE_(float, kFloat32, 1);
MSHADOW_B200_DATATYPE_(double, kFloat64, 1);
MSHADOW_B200_DATATYPE_(uint8_t, kUint8, 1);
MSHADOW_B200_DATATYPE_(int8_t, kInt8, 1);
MSHADOW_B200_DATATYPE_(int32_t, kInt32, 1);
MSHADOW_B200_DATATYPE_(int64_t, kInt64, 1);
#undef MSHADOW_B200_DATATYPE_

/*! \brief layout tags kept for source compatibility */
enum LayoutFlag { kNCHW = 0, kNHWC, kCHWN, kNCW = 1 << 3, kNWC, kCWN, kNCDHW = 1 << 5, kNDHWC, kCDHWN };

namespace detail {
// Arithmetic that the device compiler may not fuse.  Host code relies on the translation
// unit being compiled without contraction, as the reference CPU build is.
template <typename T>
MSHADOW_XINLINE T AddRN(T a, T b) { return a + b; }
template <typename T>
MSHADOW_XINLINE T SubRN(T a, T b) { return a - b; }
template <typename T>
MSHADOW_XINLINE T MulRN(T a, T b) { return a * b; }
template <typename T>
MSHADOW_XINLINE T DivRN(T a, T b) { return a / b; }
#ifdef __CUDA_ARCH__
template <>
MSHADOW_XINLINE float AddRN<float>(float a, float b) { return __fadd_rn(a, b); }
template <>
MSHADOW_XINLINE float SubRN<float>(float a, float b) { return __fsub_rn(a, b); }
template <>
MSHADOW_XINLINE float MulRN<float>(float a, float b) { return __fmul_rn(a, b); }
template <>
MSHADOW_XINLINE float DivRN<float>(float a, float b) { return __fdiv_rn(a, b); }
template <>
MSHADOW_XINLINE double AddRN<double>(double a, double b) { return __dadd_rn(a, b); }
template <>
MSHADOW_XINLINE double SubRN<double>(double a, double b) { return __dsub_rn(a, b); }
template <>
MSHADOW_XINLINE double MulRN<double>(double a, double b) { return __dmul_rn(a, b); }
template <>
MSHADOW_XINLINE double DivRN<double>(double a, double b) { return __ddiv_rn(a, b); }
#endif
}  // namespace detail

/*! \brief binary element operators usable in expressions */
namespace op {
struct mul {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType a, DType b) { return detail::MulRN(a, b); }
};
struct plus {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType a, DType b) { return detail::AddRN(a, b); }
};
struct minus {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType a, DType b) { return detail::SubRN(a, b); }
};
struct div {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType a, DType b) { return detail::DivRN(a, b); }
};
struct right {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType, DType b) { return b; }
};
struct identity {
  template <typename DType>
  MSHADOW_XINLINE static DType Map(DType a) { return a; }
};
}  // namespace op

/*! \brief how a computed value is merged into the destination element */
namespace sv {
struct saveto {
  template <typename DType>
  MSHADOW_XINLINE static void Save(DType &a, DType b) { a = b; }  // NOLINT(*)
  MSHADOW_XINLINE static default_real_t AlphaBLAS() { return 1.0f; }
  MSHADOW_XINLINE static default_real_t BetaBLAS() { return 0.0f; }
  typedef op::right OPType;
};
struct plusto {
  template <typename DType>
  MSHADOW_XINLINE static void Save(DType &a, DType b) { a = detail::AddRN(a, b); }  // NOLINT(*)
  MSHADOW_XINLINE static default_real_t AlphaBLAS() { return 1.0f; }
  MSHADOW_XINLINE static default_real_t BetaBLAS() { return 1.0f; }
  typedef op::plus OPType;
};
struct minusto {
  template <typename DType>
  MSHADOW_XINLINE static void Save(DType &a, DType b) { a = detail::SubRN(a, b); }  // NOLINT(*)
  MSHADOW_XINLINE static default_real_t AlphaBLAS() { return -1.0f; }
  MSHADOW_XINLINE static default_real_t BetaBLAS() { return 1.0f; }
  typedef op::minus OPType;
};
struct multo {
  template <typename DType>
  MSHADOW_XINLINE static void Save(DType &a, DType b) { a = detail::MulRN(a, b); }  // NOLINT(*)
  typedef op::mul OPType;
};
struct divto {
  template <typename DType>
  MSHADOW_XINLINE static void Save(DType &a, DType b) { a = detail::DivRN(a, b); }  // NOLINT(*)
  typedef op::div OPType;
};
}  // namespace sv

/*! \brief reducers: the fold, its identity value and its partial derivative */
namespace red {
namespace limits {
template <typename DType>
MSHADOW_XINLINE DType MinValue();
template <>
MSHADOW_XINLINE float MinValue<float>() { return -FLT_MAX; }
template <>
MSHADOW_XINLINE double MinValue<double>() { return -DBL_MAX; }
template <>
MSHADOW_XINLINE uint8_t MinValue<uint8_t>() { return 0; }
template <>
MSHADOW_XINLINE int8_t MinValue<int8_t>() { return SCHAR_MIN; }
template <>
MSHADOW_XINLINE int32_t MinValue<int32_t>() { return INT_MIN; }
template <>
MSHADOW_XINLINE int64_t MinValue<int64_t>() { return LLONG_MIN; }
template <typename DType>
MSHADOW_XINLINE DType MaxValue();
template <>
MSHADOW_XINLINE float MaxValue<float>() { return FLT_MAX; }
template <>
MSHADOW_XINLINE double MaxValue<double>() { return DBL_MAX; }
template <>
MSHADOW_XINLINE uint8_t MaxValue<uint8_t>() { return UCHAR_MAX; }
template <>
MSHADOW_XINLINE int8_t MaxValue<int8_t>() { return SCHAR_MAX; }
template <>
MSHADOW_XINLINE int32_t MaxValue<int32_t>() { return INT_MAX; }
template <>
MSHADOW_XINLINE int64_t MaxValue<int64_t>() { return LLONG_MAX; }
}  // namespace limits

struct sum {
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src) {  // NOLINT(*)
    dst = detail::AddRN<DType>(dst, src);
  }
  /*! \brief register-friendly overload, chosen for non-volatile accumulators */
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(DType &dst, DType src) {  // NOLINT(*)
    dst = detail::AddRN<DType>(dst, src);
  }
  /*! \brief compensated (Kahan) accumulation */
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src,  // NOLINT(*)
                                     volatile DType &residual) {               // NOLINT(*)
    DType y = detail::SubRN<DType>(src, residual);
    DType t = detail::AddRN<DType>(dst, y);
    residual = detail::SubRN<DType>(detail::SubRN<DType>(t, dst), y);
    dst = t;
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &src_val) {  // NOLINT(*)
    Reduce(dst_val, src_val);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &dst_residual,  // NOLINT(*)
                                    volatile DType &src_val, volatile DType &src_residual) {  // NOLINT(*)
    // two-sum of the values, then fold both running residuals into the error term
    const DType a = dst_val, b = src_val;
    const DType s = detail::AddRN<DType>(a, b);
    const DType bv = detail::SubRN<DType>(s, a);
    const DType err = detail::AddRN<DType>(detail::SubRN<DType>(a, detail::SubRN<DType>(s, bv)),
                                           detail::SubRN<DType>(b, bv));
    const DType carry = detail::AddRN<DType>(detail::AddRN<DType>(err, dst_residual), src_residual);
    const DType total = detail::AddRN<DType>(s, carry);
    dst_val = total;
    dst_residual = detail::SubRN<DType>(carry, detail::SubRN<DType>(total, s));
  }
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &, volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static DType PartialGrad(DType, DType) { return 1; }
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv) { initv = 0; }  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv, DType &residual) {  // NOLINT(*)
    initv = 0;
    residual = 0;
  }
};

struct maximum {
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src) {  // NOLINT(*)
    const DType a = dst, b = src;
    dst = a < b ? b : a;
  }
  /*! \brief register-friendly overload, chosen for non-volatile accumulators */
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(DType &dst, DType src) {  // NOLINT(*)
    dst = dst < src ? src : dst;
  }
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src,  // NOLINT(*)
                                     volatile DType &) {                       // NOLINT(*)
    Reduce(dst, src);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &src_val) {  // NOLINT(*)
    Reduce(dst_val, src_val);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &,  // NOLINT(*)
                                    volatile DType &src_val, volatile DType &) {  // NOLINT(*)
    Reduce(dst_val, src_val);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &, volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static DType PartialGrad(DType redres, DType redsrc) {
    return redres == redsrc ? 1 : 0;
  }
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv) { initv = limits::MinValue<DType>(); }  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv, DType &) { SetInitValue(initv); }  // NOLINT(*)
};

struct minimum {
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src) {  // NOLINT(*)
    const DType a = dst, b = src;
    dst = b < a ? b : a;
  }
  /*! \brief register-friendly overload, chosen for non-volatile accumulators */
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(DType &dst, DType src) {  // NOLINT(*)
    dst = src < dst ? src : dst;
  }
  template <typename DType>
  MSHADOW_XINLINE static void Reduce(volatile DType &dst, volatile DType src,  // NOLINT(*)
                                     volatile DType &) {                       // NOLINT(*)
    Reduce(dst, src);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &src_val) {  // NOLINT(*)
    Reduce(dst_val, src_val);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Merge(volatile DType &dst_val, volatile DType &,  // NOLINT(*)
                                    volatile DType &src_val, volatile DType &) {  // NOLINT(*)
    Reduce(dst_val, src_val);
  }
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void Finalize(volatile DType &, volatile DType &) {}  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static DType PartialGrad(DType redres, DType redsrc) {
    return redres == redsrc ? 1 : 0;
  }
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv) { initv = limits::MaxValue<DType>(); }  // NOLINT(*)
  template <typename DType>
  MSHADOW_XINLINE static void SetInitValue(DType &initv, DType &) { SetInitValue(initv); }  // NOLINT(*)
};
}  // namespace red

/*! \brief run `...` with DType bound to the C++ type that a TypeFlag names */
#define MSHADOW_TYPE_SWITCH(type, DType, ...)                        \
  switch (type) {                                                    \
    case mshadow::kFloat32: { typedef float DType; {__VA_ARGS__} } break;   \
    case mshadow::kFloat64: { typedef double DType; {__VA_ARGS__} } break;  \
    case mshadow::kUint8: { typedef uint8_t DType; {__VA_ARGS__} } break;   \
    case mshadow::kInt8: { typedef int8_t DType; {__VA_ARGS__} } break;     \
    case mshadow::kInt32: { typedef int32_t DType; {__VA_ARGS__} } break;   \
    case mshadow::kInt64: { typedef int64_t DType; {__VA_ARGS__} } break;   \
    default: LOG(FATAL) << "Unknown type enum " << type;             \
  }
#define MSHADOW_REAL_TYPE_SWITCH(type, DType, ...)                   \
  switch (type) {                                                    \
    case mshadow::kFloat32: { typedef float DType; {__VA_ARGS__} } break;   \
    case mshadow::kFloat64: { typedef double DType; {__VA_ARGS__} } break;  \
    default: LOG(FATAL) << "This operation only supports real types, not " << type; \
  }

/*! \brief size in bytes of the type a TypeFlag names */
inline size_t mshadow_sizeof(int type) {
  size_t size = 0;
  MSHADOW_TYPE_SWITCH(type, DType, size = sizeof(DType););
  return size;
}

}  // namespace mshadow
#endif  // MSHADOW_BASE_H_
