/*
 * LRNForward / LRNBackward: local response normalisation across channels as single passes.
 *
 * dmlc/mshadow has no LRN function; layers compose it from chpool<red::sum> and user functors
 * (mshadow/extension/channel_pool.h:77-104, the gradient of the pooling being
 * channel_unpool.h:102-133).  These two functions evaluate exactly those compositions,
 *
 *   LRNForward<Power>(out, norm, src, nsize, salpha, beta, knorm):
 *     norm = chpool<red::sum>(F<square>(src), nsize) * salpha + knorm;   square(a) = a * a
 *     out  = src * F<Power>(norm, -beta);
 *   LRNBackward<Power>(gsrc, gout, src, norm, nsize, salpha, beta):
 *     gsrc  = gout * F<Power>(norm, -beta);
 *     gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<Power>(norm, -beta - 1.0f), nsize) * src;
 *
 * with every product and sum rounded separately and in that order.  On the GPU they run the
 * fused kernels of gpu/lrn.cuh when the tensors are dense, 16-byte aligned, the plane a multiple
 * of four elements, nsize 3, 5 or 7 and there are at least 2 * nsize channels; otherwise (and on
 * the CPU) the expressions themselves are evaluated.  `norm` may be an empty tensor (dptr_ ==
 * NULL) in LRNForward when the fused kernel applies; the backward pass needs it.
 */
#ifndef MSHADOW_EXTENSION_LRN_H_
#define MSHADOW_EXTENSION_LRN_H_

#include <cmath>

#include "./pooling.h"
#if MSHADOW_USE_CUDA && defined(__CUDACC__)
#include "../gpu/lrn.cuh"
#endif

namespace mshadow {
namespace b200 {
/*! \brief a * a */
struct square {
  MSHADOW_XINLINE static float Map(float a) { return mshadow::detail::MulRN(a, a); }
};
/*! \brief base ^ exponent by the C library (host) / CUDA (device): results may differ in the last bits */
struct power {
  MSHADOW_XINLINE static float Map(float base, float exponent) { return powf(base, exponent); }
};
/*!
 * \brief base ^ exponent for the exponents -0.75 and -1.75 (the usual beta = 0.75) from square
 *  roots, products and one division, all correctly rounded operations: the same bits on every
 *  device.  Other exponents fall back to powf.
 */
struct power_by_roots {
  MSHADOW_XINLINE static float Map(float base, float exponent) {
    if (exponent != -0.75f && exponent != -1.75f) return powf(base, exponent);
#ifdef __CUDA_ARCH__
    const float r = __fsqrt_rn(base);
    float t = __fmul_rn(r, __fsqrt_rn(r));  // base ^ 0.75
    if (exponent == -1.75f) t = __fmul_rn(t, base);
    return __frcp_rn(t);  // the correctly rounded reciprocal is the correctly rounded 1.0f / t
#else
    const float r = sqrtf(base);
    float t = r * sqrtf(r);
    if (exponent == -1.75f) t = t * base;
    return 1.0f / t;
#endif
  }
};
/*!
 * \brief base ^ exponent for positive bases by the GPU's fast exp2 / log2 units (about 2^-21
 *  relative error); on the host, powf.  For layers that accept results within tolerance: with it
 *  the LRN kernels are bound by memory instead of by the arithmetic of an exactly rounded power.
 */
struct power_fast {
  MSHADOW_XINLINE static float Map(float base, float exponent) {
#ifdef __CUDA_ARCH__
    return __powf(base, exponent);
#else
    return powf(base, exponent);
#endif
  }
};
}  // namespace b200

namespace lrndetail {
template <typename Power, typename xpu>
inline void ForwardByExpressions(Tensor<xpu, 4, float> out, Tensor<xpu, 4, float> norm, const Tensor<xpu, 4, float> &src,
                                 int nsize, float salpha, float beta, float knorm) {
  using namespace mshadow::expr;  // NOLINT(*)
  CHECK(norm.dptr_ != NULL) << "LRNForward: this shape is evaluated through expressions and needs the norm tensor";
  norm = chpool<red::sum>(F<b200::square>(src), nsize) * salpha + knorm;
  out = src * F<Power>(norm, -beta);
}
template <typename Power, typename xpu>
inline void BackwardByExpressions(Tensor<xpu, 4, float> gsrc, const Tensor<xpu, 4, float> &gout,
                                  const Tensor<xpu, 4, float> &src, const Tensor<xpu, 4, float> &norm, int nsize,
                                  float salpha, float beta) {
  using namespace mshadow::expr;  // NOLINT(*)
  gsrc = gout * F<Power>(norm, -beta);
  gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<Power>(norm, -beta - 1.0f), nsize) * src;
}
}  // namespace lrndetail

template <typename Power>
inline void LRNForward(Tensor<cpu, 4, float> out, Tensor<cpu, 4, float> norm, const Tensor<cpu, 4, float> &src,
                       int nsize, float salpha, float beta, float knorm) {
  CHECK_EQ(out.shape_, src.shape_) << "LRNForward: shape mismatch";
  lrndetail::ForwardByExpressions<Power>(out, norm, src, nsize, salpha, beta, knorm);
}
template <typename Power>
inline void LRNBackward(Tensor<cpu, 4, float> gsrc, const Tensor<cpu, 4, float> &gout, const Tensor<cpu, 4, float> &src,
                        const Tensor<cpu, 4, float> &norm, int nsize, float salpha, float beta) {
  CHECK_EQ(gsrc.shape_, src.shape_) << "LRNBackward: shape mismatch";
  lrndetail::BackwardByExpressions<Power>(gsrc, gout, src, norm, nsize, salpha, beta);
}

#if MSHADOW_USE_CUDA && defined(__CUDACC__)
template <typename Power>
inline void LRNForward(Tensor<gpu, 4, float> out, Tensor<gpu, 4, float> norm, const Tensor<gpu, 4, float> &src,
                       int nsize, float salpha, float beta, float knorm) {
  CHECK_EQ(out.shape_, src.shape_) << "LRNForward: shape mismatch";
  CHECK(norm.dptr_ == NULL || norm.shape_ == src.shape_) << "LRNForward: shape mismatch";
  CHECK(nsize % 2 == 1) << "LRNForward: the window must be odd";
  const int64_t plane = static_cast<int64_t>(src.size(2)) * src.size(3);
  const bool dense = out.CheckContiguous() && src.CheckContiguous() && (norm.dptr_ == NULL || norm.CheckContiguous());
  if (dense && cuda::lrndetail::Supported(nsize, src.size(1), plane, out.dptr_, src.dptr_, norm.dptr_, NULL)) {
    cuda::LrnForwardLaunch<Power>(out.dptr_, norm.dptr_, src.dptr_, src.size(0), src.size(1), plane, nsize, salpha, beta,
                                  knorm, Stream<gpu>::GetStream(out.stream_));
  } else {
    lrndetail::ForwardByExpressions<Power>(out, norm, src, nsize, salpha, beta, knorm);
  }
}
template <typename Power>
inline void LRNBackward(Tensor<gpu, 4, float> gsrc, const Tensor<gpu, 4, float> &gout, const Tensor<gpu, 4, float> &src,
                        const Tensor<gpu, 4, float> &norm, int nsize, float salpha, float beta) {
  CHECK_EQ(gsrc.shape_, src.shape_) << "LRNBackward: shape mismatch";
  CHECK(gout.shape_ == src.shape_ && norm.shape_ == src.shape_) << "LRNBackward: shape mismatch";
  CHECK(nsize % 2 == 1) << "LRNBackward: the window must be odd";
  const int64_t plane = static_cast<int64_t>(src.size(2)) * src.size(3);
  const bool dense = gsrc.CheckContiguous() && gout.CheckContiguous() && src.CheckContiguous() && norm.CheckContiguous();
  if (dense && cuda::lrndetail::Supported(nsize, src.size(1), plane, gsrc.dptr_, gout.dptr_, src.dptr_, norm.dptr_)) {
    cuda::LrnBackwardLaunch<Power>(gsrc.dptr_, gout.dptr_, src.dptr_, norm.dptr_, src.size(0), src.size(1), plane, nsize,
                                   salpha, beta, Stream<gpu>::GetStream(gsrc.stream_));
  } else {
    lrndetail::BackwardByExpressions<Power>(gsrc, gout, src, norm, nsize, salpha, beta);
  }
}
#endif

}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_LRN_H_
