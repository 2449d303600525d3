/*
 * Pooling expressions:
 *   pool<Reducer>(src, ksize_y, ksize_x, kstride_y, kstride_x)     spatial window reduce
 *   pool<Reducer>(src, pshape, ...)                                 same, output size given
 *   unpool<Reducer>(data_src, data_pooled, grad_pooled, ...)        its gradient
 *   chpool<Reducer>(src, nsize [, stride, pad])                     window over channels
 * Expression types, factory functions, shape rules and Plan::Eval semantics follow
 * dmlc/mshadow's mshadow/extension/spatial_pool.h (:20-149), spatial_unpool.h (:20-132) and
 * channel_pool.h (:21-104), so any composition with other expressions evaluates as there,
 * through the generic map kernel.
 *
 * New: when the operands are plain fp32 GPU tensors and the destination is assigned with
 * `=`, evaluation is routed to the dedicated kernels of gpu/pool.cuh (shared-memory staged
 * planes, register-ring channel march) instead of the generic kernel.
 */
#ifndef MSHADOW_EXTENSION_POOLING_H_
#define MSHADOW_EXTENSION_POOLING_H_

#include <algorithm>

#include "../engine/check.h"
#if MSHADOW_USE_CUDA && defined(__CUDACC__)
#include "../gpu/pool.cuh"
#endif

namespace mshadow {
namespace expr {

// ------------------------------------------------------------------------------------------
// spatial pooling
// ------------------------------------------------------------------------------------------
template <typename Reducer, typename SrcExp, typename DType, int srcdim>
struct PoolingExp : public MakeTensorExp<PoolingExp<Reducer, SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  index_t ksize_y_, ksize_x_, kstride_y_, kstride_x_;
  index_t src_height_, src_width_;
  /*! \brief output extent floor((in - k) / s) + 1: no padding, a ragged border is dropped */
  PoolingExp(const SrcExp &src, index_t ksize_y, index_t ksize_x, index_t kstride_y, index_t kstride_x)
      : src_(src), ksize_y_(ksize_y), ksize_x_(ksize_x), kstride_y_(kstride_y), kstride_x_(kstride_x) {
    Init();
    this->shape_[srcdim - 2] = (src_height_ - ksize_y) / kstride_y + 1;
    this->shape_[srcdim - 1] = (src_width_ - ksize_x) / kstride_x + 1;
  }
  /*! \brief output extent chosen by the caller; windows are clipped at the image border */
  PoolingExp(const SrcExp &src, Shape<2> pshape, index_t ksize_y, index_t ksize_x, index_t kstride_y,
             index_t kstride_x)
      : src_(src), ksize_y_(ksize_y), ksize_x_(ksize_x), kstride_y_(kstride_y), kstride_x_(kstride_x) {
    Init();
    this->shape_[srcdim - 2] = pshape[0];
    this->shape_[srcdim - 1] = pshape[1];
  }

 private:
  inline void Init() {
    const Shape<srcdim> sshape = ShapeCheck<srcdim, SrcExp>::Check(src_);
    CHECK(sshape[srcdim - 1] >= ksize_x_ && sshape[srcdim - 2] >= ksize_y_)
        << "PoolingExp: kernel must be smaller than image";
    src_height_ = sshape[srcdim - 2];
    src_width_ = sshape[srcdim - 1];
    this->shape_ = sshape;
  }
};

template <typename Reducer, typename SrcExp, typename DType, int etype>
inline PoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> pool(const Exp<SrcExp, DType, etype> &src,
                                                                      index_t ksize_y, index_t ksize_x,
                                                                      index_t kstride_y, index_t kstride_x) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return PoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), ksize_y, ksize_x, kstride_y,
                                                                   kstride_x);
}
template <typename Reducer, typename SrcExp, typename DType, int etype>
inline PoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> pool(const Exp<SrcExp, DType, etype> &src,
                                                                      Shape<2> pshape, index_t ksize_y,
                                                                      index_t ksize_x, index_t kstride_y,
                                                                      index_t kstride_x) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return PoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), pshape, ksize_y, ksize_x, kstride_y,
                                                                   kstride_x);
}

template <typename Reducer, typename SrcExp, typename DType, int srcdim>
class Plan<PoolingExp<Reducer, SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const PoolingExp<Reducer, SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), ky_(e.ksize_y_), kx_(e.ksize_x_), sy_(e.kstride_y_), sx_(e.kstride_x_),
        in_h_(e.src_height_), in_w_(e.src_width_), out_h_(e.shape_[srcdim - 2]) {}
  /*! \brief row i of the matrix view is (plane i / out_h, output row i % out_h) */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    const index_t plane = i / out_h_, py = i - plane * out_h_;
    const index_t y_lo = py * sy_, x_lo = j * sx_;
    const index_t y_hi = y_lo + ky_ < in_h_ ? y_lo + ky_ : in_h_;
    const index_t x_hi = x_lo + kx_ < in_w_ ? x_lo + kx_ : in_w_;
    DType res;
    Reducer::SetInitValue(res);
    for (index_t y = y_lo; y < y_hi; ++y)
      for (index_t x = x_lo; x < x_hi; ++x) Reducer::Reduce(res, src_.Eval(plane * in_h_ + y, x));
    return res;
  }

 private:
  Plan<SrcExp, DType> src_;
  const index_t ky_, kx_, sy_, sx_, in_h_, in_w_, out_h_;
};

// ------------------------------------------------------------------------------------------
// gradient of spatial pooling
// ------------------------------------------------------------------------------------------
template <typename Reducer, typename SrcExp, typename DType, int srcdim>
struct UnPoolingExp : public MakeTensorExp<UnPoolingExp<Reducer, SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &data_src_;
  const SrcExp &data_pooled_;
  const SrcExp &grad_pooled_;
  index_t pshape_y_, pshape_x_;
  index_t ksize_y_, ksize_x_, kstride_y_, kstride_x_;
  UnPoolingExp(const SrcExp &data_src, const SrcExp &data_pooled, const SrcExp &grad_pooled, index_t ksize_y,
               index_t ksize_x, index_t kstride_y, index_t kstride_x)
      : data_src_(data_src), data_pooled_(data_pooled), grad_pooled_(grad_pooled), ksize_y_(ksize_y),
        ksize_x_(ksize_x), kstride_y_(kstride_y), kstride_x_(kstride_x) {
    typedef ShapeCheck<srcdim, SrcExp> Check;
    const Shape<srcdim> pshape = Check::Check(grad_pooled);
    CHECK_EQ(pshape, Check::Check(data_pooled)) << "UnPoolingExp: pooled shape mismatch";
    const Shape<srcdim> sshape = Check::Check(data_src);
    for (int k = 0; k < srcdim - 2; ++k) {
      CHECK_EQ(pshape[k], sshape[k]) << "UnPoolingExp: pool and src shape mismatch";
    }
    pshape_x_ = pshape[srcdim - 1];
    pshape_y_ = pshape[srcdim - 2];
    this->shape_ = sshape;
  }
};

template <typename Reducer, typename SrcExp, typename DType, int etype>
inline UnPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> unpool(const Exp<SrcExp, DType, etype> &data_src,
                                                                          const Exp<SrcExp, DType, etype> &data_pooled,
                                                                          const Exp<SrcExp, DType, etype> &grad_pooled,
                                                                          index_t ksize_y, index_t ksize_x,
                                                                          index_t kstride_y, index_t kstride_x) {
  return UnPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(data_src.self(), data_pooled.self(),
                                                                     grad_pooled.self(), ksize_y, ksize_x, kstride_y,
                                                                     kstride_x);
}

template <typename Reducer, typename SrcExp, typename DType, int srcdim>
class Plan<UnPoolingExp<Reducer, SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const UnPoolingExp<Reducer, SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.data_src_)), pooled_(MakePlan(e.data_pooled_)), grad_(MakePlan(e.grad_pooled_)),
        in_h_(e.shape_[srcdim - 2]), out_h_(e.pshape_y_), out_w_(e.pshape_x_), ky_(e.ksize_y_), kx_(e.ksize_x_),
        sy_(e.kstride_y_), sx_(e.kstride_x_) {}
  /*!
   * \brief sum, over the pooling windows that cover input pixel (y, x) in row-major window
   *  order, of PartialGrad(input, pooled) * pooled gradient; starts from zero
   */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    const index_t plane = i / in_h_, y = i - plane * in_h_, x = j;
    const DType v = src_.Eval(i, j);
    const index_t py_lo = y < ky_ ? 0 : (y - ky_ + sy_) / sy_;
    const index_t px_lo = x < kx_ ? 0 : (x - kx_ + sx_) / sx_;
    index_t py_hi = (y + sy_) / sy_, px_hi = (x + sx_) / sx_;
    if (py_hi > out_h_) py_hi = out_h_;
    if (px_hi > out_w_) px_hi = out_w_;
    DType val = static_cast<DType>(0);
    for (index_t py = py_lo; py < py_hi; ++py)
      for (index_t px = px_lo; px < px_hi; ++px) {
        const index_t row = plane * out_h_ + py;
        val = detail::AddRN<DType>(val, detail::MulRN<DType>(Reducer::PartialGrad(v, pooled_.Eval(row, px)),
                                                             grad_.Eval(row, px)));
      }
    return val;
  }

 private:
  Plan<SrcExp, DType> src_, pooled_, grad_;
  const index_t in_h_, out_h_, out_w_, ky_, kx_, sy_, sx_;
};

// ------------------------------------------------------------------------------------------
// pooling over a window of channels (local response normalisation building block)
// ------------------------------------------------------------------------------------------
template <typename Reducer, typename SrcExp, typename DType, int srcdim>
struct ChannelPoolingExp
    : public MakeTensorExp<ChannelPoolingExp<Reducer, SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &src_;
  index_t nsize_, stride_, pad_, src_channel_;
  ChannelPoolingExp(const SrcExp &src, index_t nsize, index_t stride, index_t pad)
      : src_(src), nsize_(nsize), stride_(stride), pad_(pad) {
    this->shape_ = ShapeCheck<srcdim, SrcExp>::Check(src_);
    this->src_channel_ = this->shape_[srcdim - 3];
    CHECK_GE(this->shape_[srcdim - 3], nsize_) << "chpool: local size must be smaller than nchannels";
    this->shape_[srcdim - 3] = (this->src_channel_ - nsize + pad * 2 + 1) / stride;
  }
};

template <typename Reducer, typename SrcExp, typename DType, int etype>
inline ChannelPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> chpool(const Exp<SrcExp, DType, etype> &src,
                                                                               index_t nsize) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 3>::Error_Expression_Does_Not_Meet_Dimension_Req();
  CHECK_EQ(nsize % 2, 1U) << "chpool: if no pad is specified, local size must be odd";
  return ChannelPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), nsize, 1, nsize / 2);
}
template <typename Reducer, typename SrcExp, typename DType, int etype>
inline ChannelPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> chpool(const Exp<SrcExp, DType, etype> &src,
                                                                               index_t nsize, index_t stride,
                                                                               index_t pad) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 3>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return ChannelPoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(src.self(), nsize, stride, pad);
}

template <typename Reducer, typename SrcExp, typename DType, int srcdim>
class Plan<ChannelPoolingExp<Reducer, SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const ChannelPoolingExp<Reducer, SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.src_)), out_c_(e.shape_[srcdim - 3]), h_(e.shape_[srcdim - 2]), nsize_(e.nsize_),
        stride_(e.stride_), pad_(e.pad_), in_c_(e.src_channel_) {}
  /*!
   * \brief reduce source channels [c*stride - pad, c*stride - pad + nsize), clipped below at 0
   *  and above at the OUTPUT channel count (the reference's clamp), in ascending order
   */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    const index_t t = i / h_, y = i - t * h_;
    const index_t n = t / out_c_, c = t - n * out_c_;
    const index_t lo = c * stride_ < pad_ ? 0 : c * stride_ - pad_;
    const index_t top = c * stride_ - pad_ + nsize_;
    const index_t hi = top < out_c_ ? top : out_c_;
    DType res;
    Reducer::SetInitValue(res);
    for (index_t cc = lo; cc < hi; ++cc) Reducer::Reduce(res, src_.Eval((n * in_c_ + cc) * h_ + y, j));
    return res;
  }

 private:
  Plan<SrcExp, DType> src_;
  const index_t out_c_, h_, nsize_, stride_, pad_, in_c_;
};

// ------------------------------------------------------------------------------------------
// gradient of channel pooling (dmlc/mshadow: mshadow/extension/channel_unpool.h:20-133)
// ------------------------------------------------------------------------------------------
template <typename Reducer, typename SrcExp, typename DType, int srcdim>
struct ChannelUnpoolingExp
    : public MakeTensorExp<ChannelUnpoolingExp<Reducer, SrcExp, DType, srcdim>, SrcExp, srcdim, DType> {
  const SrcExp &data_src_;
  const SrcExp &data_pooled_;
  const SrcExp &grad_pooled_;
  index_t pchannel_, nsize_, kstride_, pad_;
  ChannelUnpoolingExp(const SrcExp &data_src, const SrcExp &data_pooled, const SrcExp &grad_pooled, index_t nsize,
                      index_t kstride, index_t pad)
      : data_src_(data_src), data_pooled_(data_pooled), grad_pooled_(grad_pooled), nsize_(nsize), kstride_(kstride),
        pad_(pad) {
    typedef ShapeCheck<srcdim, SrcExp> Check;
    const Shape<srcdim> pshape = Check::Check(grad_pooled);
    CHECK_EQ(pshape, Check::Check(data_pooled)) << "ChannelUnPoolingExp: data and grad shape mismatch";
    const Shape<srcdim> sshape = Check::Check(data_src);
    for (int k = 0; k < srcdim; ++k) {
      if (k == 1) continue;  // the channel extent is the one that pooling changes
      CHECK_EQ(pshape[k], sshape[k]) << "ChannelUnPoolingExp: pooled tensor and src tensor shape mismatch"
                                     << pshape[k] << " vs " << sshape[k];
    }
    pchannel_ = pshape[1];
    this->shape_ = sshape;
  }
};

template <typename Reducer, typename SrcExp, typename DType, int etype>
inline ChannelUnpoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> ch_unpool(
    const Exp<SrcExp, DType, etype> &data_src, const Exp<SrcExp, DType, etype> &data_pooled,
    const Exp<SrcExp, DType, etype> &grad_pooled, index_t nsize, index_t stride, index_t pad) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 3>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return ChannelUnpoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim>(data_src.self(), data_pooled.self(),
                                                                            grad_pooled.self(), nsize, stride, pad);
}
template <typename Reducer, typename SrcExp, typename DType, int etype>
inline ChannelUnpoolingExp<Reducer, SrcExp, DType, ExpInfo<SrcExp>::kDim> ch_unpool(
    const Exp<SrcExp, DType, etype> &data_src, const Exp<SrcExp, DType, etype> &data_pooled,
    const Exp<SrcExp, DType, etype> &grad_pooled, index_t nsize) {
  return ch_unpool<Reducer>(data_src, data_pooled, grad_pooled, nsize, 1, nsize / 2);
}

template <typename Reducer, typename SrcExp, typename DType, int srcdim>
class Plan<ChannelUnpoolingExp<Reducer, SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const ChannelUnpoolingExp<Reducer, SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.data_src_)), pooled_(MakePlan(e.data_pooled_)), grad_(MakePlan(e.grad_pooled_)),
        c_(e.shape_[srcdim - 3]), h_(e.shape_[srcdim - 2]), pc_(e.pchannel_), nsize_(e.nsize_), stride_(e.kstride_),
        pad_(e.pad_) {}
  /*!
   * \brief sum over the pooled channels whose window contains source channel c, in ascending
   *  order from zero, of PartialGrad(src, pooled) * grad; the upper clamp is the SOURCE
   *  channel count, as in the reference
   */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    const DType v = src_.Eval(i, j);
    const index_t t = i / h_, y = i - t * h_;
    const index_t n = t / c_, c = t - n * c_;
    const index_t lo = c < nsize_ - pad_ ? 0 : (c - (nsize_ - pad_) + stride_) / stride_;
    index_t hi = (c + pad_ + stride_) / stride_;
    if (hi > c_) hi = c_;
    DType val = static_cast<DType>(0);
    for (index_t cc = lo; cc < hi; ++cc) {
      const index_t row = (n * pc_ + cc) * h_ + y;
      val = detail::AddRN<DType>(
          val, detail::MulRN<DType>(Reducer::PartialGrad(v, pooled_.Eval(row, j)), grad_.Eval(row, j)));
    }
    return val;
  }

 private:
  Plan<SrcExp, DType> src_, pooled_, grad_;
  const index_t c_, h_, pc_, nsize_, stride_, pad_;
};

}  // namespace expr

#if MSHADOW_USE_CUDA && defined(__CUDACC__)
namespace cuda {

// `dst = pool<Reducer>(tensor, ...)` on fp32 GPU tensors
template <typename Reducer, int dim>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, float>, expr::PoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim>,
                   float, dim> {
  typedef expr::PoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim> E;
  inline static void Run(Tensor<gpu, dim, float> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    const Tensor<gpu, dim, float> &src = e.src_;
    const index_t ph = dshape[dim - 2], pw = dshape[dim - 1];
    const bool standard_shape = ph == (e.src_height_ - e.ksize_y_) / e.kstride_y_ + 1 &&
                                pw == (e.src_width_ - e.ksize_x_) / e.kstride_x_ + 1;
    if (standard_shape && PoolPlanesFit(e.src_height_, e.src_width_, ph, pw, false)) {
      PoolPlanesLaunch<Reducer>(dst->dptr_, src.dptr_, dshape.ProdShape(0, dim - 2), e.src_height_, e.src_width_,
                                e.ksize_y_, e.ksize_x_, e.kstride_y_, e.kstride_x_, src.stride_, dst->stride_, stream);
      return;
    }
    // planes beyond shared memory: bands of whole rows
    const BandPlan bp = standard_shape ? PlanPoolBands(e.src_height_, e.src_width_, ph, e.ksize_y_, e.kstride_y_)
                                       : BandPlan{0, 0, 0, 0, false};
    if (bp.ok) {
      PoolBandsLaunch<Reducer>(dst->dptr_, src.dptr_, dshape.ProdShape(0, dim - 2), e.src_height_, e.src_width_,
                               e.ksize_y_, e.ksize_x_, e.kstride_y_, e.kstride_x_, src.stride_, dst->stride_, bp, stream);
    } else {
      MapGeneric<sv::saveto, float>(dst, e, dshape, stream);
    }
  }
};

// `dst = unpool<Reducer>(src, pooled, grad, ...)` on fp32 GPU tensors
template <typename Reducer, int dim>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, float>,
                   expr::UnPoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim>, float, dim> {
  typedef expr::UnPoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim> E;
  inline static void Run(Tensor<gpu, dim, float> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    const Tensor<gpu, dim, float> &src = e.data_src_, &pooled = e.data_pooled_, &grad = e.grad_pooled_;
    const index_t h = dshape[dim - 2], w = dshape[dim - 1];
    if (pooled.stride_ == grad.stride_ && PoolPlanesFit(h, w, e.pshape_y_, e.pshape_x_, true)) {
      UnpoolPlanesLaunch<Reducer>(dst->dptr_, src.dptr_, pooled.dptr_, grad.dptr_, dshape.ProdShape(0, dim - 2), h, w,
                                  e.pshape_y_, e.pshape_x_, e.ksize_y_, e.ksize_x_, e.kstride_y_, e.kstride_x_,
                                  src.stride_, pooled.stride_, dst->stride_, stream);
      return;
    }
    const BandPlan bp = pooled.stride_ == grad.stride_
                            ? PlanUnpoolBands(h, w, e.pshape_y_, e.pshape_x_, e.ksize_y_, e.kstride_y_)
                            : BandPlan{0, 0, 0, 0, false};
    if (bp.ok) {
      UnpoolBandsLaunch<Reducer>(dst->dptr_, src.dptr_, pooled.dptr_, grad.dptr_, dshape.ProdShape(0, dim - 2), h, w,
                                 e.pshape_y_, e.pshape_x_, e.ksize_y_, e.ksize_x_, e.kstride_y_, e.kstride_x_,
                                 src.stride_, pooled.stride_, dst->stride_, bp, stream);
    } else {
      MapGeneric<sv::saveto, float>(dst, e, dshape, stream);
    }
  }
};

// `dst = chpool<Reducer>(tensor, nsize)` on dense fp32 GPU tensors
template <typename Reducer, int dim>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, float>,
                   expr::ChannelPoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim>, float, dim> {
  typedef expr::ChannelPoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim> E;
  inline static void Run(Tensor<gpu, dim, float> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    const Tensor<gpu, dim, float> &src = e.src_;
    const index_t images = dshape.ProdShape(0, dim - 3);
    if (ChannelPoolSupported(e.nsize_, e.stride_, e.pad_) && src.CheckContiguous() && dst->CheckContiguous() &&
        images < 65536) {
      ChannelPoolLaunch<Reducer>(dst->dptr_, src.dptr_, images, e.src_channel_, dshape[dim - 2], dshape[dim - 1],
                                 e.nsize_, stream);
    } else {
      MapGeneric<sv::saveto, float>(dst, e, dshape, stream);
    }
  }
};

// `dst = ch_unpool<Reducer>(src, pooled, grad, nsize)` on dense fp32 GPU tensors
template <typename Reducer, int dim>
struct MapDispatch<sv::saveto, Tensor<gpu, dim, float>,
                   expr::ChannelUnpoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim>, float, dim> {
  typedef expr::ChannelUnpoolingExp<Reducer, Tensor<gpu, dim, float>, float, dim> E;
  inline static void Run(Tensor<gpu, dim, float> *dst, const E &e, Shape<dim> dshape, cudaStream_t stream) {
    const Tensor<gpu, dim, float> &src = e.data_src_, &pooled = e.data_pooled_, &grad = e.grad_pooled_;
    const index_t images = dshape.ProdShape(0, dim - 3);
    if (ChannelUnpoolSupported(e.nsize_, e.kstride_, e.pad_) && e.pchannel_ == dshape[dim - 3] &&
        src.CheckContiguous() && pooled.CheckContiguous() && grad.CheckContiguous() && dst->CheckContiguous() &&
        images < 65536) {
      ChannelUnpoolLaunch<Reducer>(dst->dptr_, src.dptr_, pooled.dptr_, grad.dptr_, images, dshape[dim - 3],
                                   dshape[dim - 2], dshape[dim - 1], e.nsize_, stream);
    } else {
      MapGeneric<sv::saveto, float>(dst, e, dshape, stream);
    }
  }
};

}  // namespace cuda
#endif  // MSHADOW_USE_CUDA && __CUDACC__

}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_POOLING_H_
