/*
 * GPU implementations of the evaluation entry points declared in tensor.h: MapExp,
 * MapReduceKeepLowest, MapReduceKeepHighDim, and the function-form operators Softmax,
 * SoftmaxGrad (four variants), AddTakeGrad, AddTakeGradLargeBatch and SortByKey.
 * Host-side checks and error behaviour follow the reference (mshadow/tensor_gpu-inl.h:
 * 101-243 and the launch wrappers in mshadow/cuda/tensor_gpu-inl.cuh); what is launched is
 * described in map.cuh, reduce.cuh, softmax.cuh, pool.cuh and embed.cuh.
 *
 * All work is enqueued on the destination's stream and returns immediately.
 */
#ifndef MSHADOW_GPU_ENGINE_CUH_
#define MSHADOW_GPU_ENGINE_CUH_

#include <type_traits>

#include "./embed.cuh"
#include "./map.cuh"
#include "./reduce.cuh"
#include "./softmax.cuh"

namespace mshadow {
namespace cuda {

/*!
 * \brief the generic route of `dst <Saver>= exp`, decided per call:
 *  1. expression and destination both serve 16-byte groups and all pointers, strides and slice
 *     boundaries are aligned: the 128-bit kernel (walked as one long row where every operand is
 *     dense and the expression position-independent);
 *  2. only the destination does, and the expression is cheap per element (expr::LaneInfo): the
 *     128-bit kernel with groups assembled from element evaluations, which keeps one index
 *     split and one wide store per four floats;
 *  3. otherwise one element per thread.
 */
template <typename Saver, typename DType, typename R, typename E, int dim>
inline void MapGeneric(R *dst, const E &exp, Shape<dim> dshape, cudaStream_t stream) {
  const Shape<2> flat = dshape.FlatTo2D();
  if constexpr (expr::PackInfo<R>::kPass) {
    if (expr::PackAlign<R>::Check(*dst)) {
      if constexpr (expr::PackInfo<E>::kPass) {
        if (expr::PackAlign<E>::Check(exp)) {
          const bool one_row = expr::FlatInfo<E>::kPass && expr::FlatInfo<R>::kPass && expr::FlatCheck<E>::Check(exp) &&
                               expr::FlatCheck<R>::Check(*dst);
          MapPlanPacked<Saver, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), flat, one_row, stream);
          return;
        }
      }
      if constexpr (expr::LaneInfo<E>::kPass && MSHADOW_B200_MAP_HYBRID) {
        MapPlanPacked<Saver, DType, false>(expr::MakePlan(*dst), expr::MakePlan(exp), flat, false, stream);
        return;
      }
    }
  }
  MapPlanScalar<Saver, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), flat, stream);
}

template <typename Saver, typename R, typename E, typename DType, int dim>
struct MapDispatch {
  inline static void Run(R *dst, const E &exp, Shape<dim> dshape, cudaStream_t stream) {
    MapGeneric<Saver, DType>(dst, exp, dshape, stream);
  }
};

/*!
 * \brief an assignment sees an extension expression through its MakeTensorExp base (that is
 *  the type `dst = pool<...>(...)` deduces); dispatch on the real expression type
 */
template <typename Saver, typename R, typename T, typename SrcExp, int dim, typename DType>
struct MapDispatch<Saver, R, expr::MakeTensorExp<T, SrcExp, dim, DType>, DType, dim> {
  inline static void Run(R *dst, const expr::MakeTensorExp<T, SrcExp, dim, DType> &exp, Shape<dim> dshape,
                         cudaStream_t stream) {
    MapDispatch<Saver, R, T, DType, dim>::Run(dst, exp.real_self(), dshape, stream);
  }
};

}  // namespace cuda

template <typename Saver, typename R, int dim, typename DType, typename E, int etype>
inline void MapExp(TRValue<R, gpu, dim, DType> *dst, const expr::Exp<E, DType, etype> &exp) {
  expr::TypeCheckPass<expr::TypeCheck<gpu, dim, DType, E>::kMapPass>::Error_All_Tensor_in_Exp_Must_Have_Same_Type();
  const Shape<dim> eshape = expr::ShapeCheck<dim, E>::Check(exp.self());
  const Shape<dim> dshape = expr::ShapeCheck<dim, R>::Check(dst->self());
  CHECK(eshape[0] == 0 || eshape == dshape) << "Assignment: Shape of Tensors are not consistent with target, "
                                            << "eshape: " << eshape << " dshape:" << dshape;
  const cudaStream_t stream = Stream<gpu>::GetStream(expr::StreamInfo<gpu, R>::Get(dst->self()));
  cuda::MapDispatch<Saver, R, E, DType, dim>::Run(dst->ptrself(), exp.self(), dshape, stream);
}

namespace cuda {
template <typename Saver, typename Reducer, typename DType, typename R, typename E>
inline void KeepLowestGo(R *dst, const E &exp, Shape<2> eshape, DType scale, cudaStream_t stream, std::true_type) {
  constexpr int kLanes = expr::Pack<DType>::kLanes;
  if (eshape[1] % kLanes == 0 && expr::PackAlign<E>::Check(exp)) {
    ReduceKeepLowestLaunch<Saver, Reducer, kLanes, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), eshape, scale,
                                                          stream);
  } else {
    ReduceKeepLowestLaunch<Saver, Reducer, 1, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), eshape, scale, stream);
  }
}
template <typename Saver, typename Reducer, typename DType, typename R, typename E>
inline void KeepLowestGo(R *dst, const E &exp, Shape<2> eshape, DType scale, cudaStream_t stream, std::false_type) {
  ReduceKeepLowestLaunch<Saver, Reducer, 1, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), eshape, scale, stream);
}

template <typename Saver, typename Reducer, typename DType, typename R, typename E>
inline void KeepHighDimGo(R *dst, const E &exp, Shape<4> pshape, DType scale, cudaStream_t stream, std::true_type) {
  constexpr int kLanes = expr::Pack<DType>::kLanes;
  auto splan = expr::MakePlan(exp);
  if (expr::FlatCheck<E>::Check(exp) && expr::PackAlign<E>::Check(exp) &&
      (static_cast<int64_t>(pshape[2]) * pshape[3]) % kLanes == 0) {
    // dense operands of a position-independent expression: every (n, c) plane is one long row
    const index_t plane = pshape[2] * pshape[3];
    splan.Reflow(plane);
    ReduceKeepHighDimLaunch<Saver, Reducer, kLanes, DType>(expr::MakePlan(*dst), splan,
                                                           Shape4(pshape[0], pshape[1], 1, plane), scale, stream);
  } else if (pshape[3] % kLanes == 0 && expr::PackAlign<E>::Check(exp)) {
    ReduceKeepHighDimLaunch<Saver, Reducer, kLanes, DType>(expr::MakePlan(*dst), splan, pshape, scale, stream);
  } else {
    ReduceKeepHighDimLaunch<Saver, Reducer, 1, DType>(expr::MakePlan(*dst), splan, pshape, scale, stream);
  }
}
template <typename Saver, typename Reducer, typename DType, typename R, typename E>
inline void KeepHighDimGo(R *dst, const E &exp, Shape<4> pshape, DType scale, cudaStream_t stream, std::false_type) {
  ReduceKeepHighDimLaunch<Saver, Reducer, 1, DType>(expr::MakePlan(*dst), expr::MakePlan(exp), pshape, scale, stream);
}
}  // namespace cuda

template <typename Saver, typename Reducer, typename R, typename DType, typename E, int etype>
inline void MapReduceKeepLowest(TRValue<R, gpu, 1, DType> *dst, const expr::Exp<E, DType, etype> &exp, DType scale) {
  expr::TypeCheckPass<expr::TypeCheck<gpu, 1, DType, E>::kRedPass>::Error_TypeCheck_Not_Pass_For_Reduce_Exp();
  const Shape<2> eshape = expr::ShapeCheck<expr::ExpInfo<E>::kDim, E>::Check(exp.self()).FlatTo2D();
  const Shape<1> dshape = expr::ShapeCheck<1, R>::Check(dst->self());
  CHECK_EQ(eshape[1], dshape[0]) << "MapReduceKeepLowest::reduction dimension do not match";
  CHECK_NE(eshape[0], 0U) << "can not reduce over empty tensor";
  const cudaStream_t stream = Stream<gpu>::GetStream(expr::StreamInfo<gpu, R>::Get(dst->self()));
  if (eshape[1] == 0) return;
  cuda::KeepLowestGo<Saver, Reducer, DType>(dst->ptrself(), exp.self(), eshape, scale, stream,
                                            std::integral_constant<bool, expr::PackInfo<E>::kPass>());
}

template <typename Saver, typename Reducer, int dimkeep, typename R, typename DType, typename E, int etype>
inline void MapReduceKeepHighDim(TRValue<R, gpu, 1, DType> *dst, const expr::Exp<E, DType, etype> &exp,
                                 DType scale) {
  expr::TypeCheckPass<expr::TypeCheck<gpu, dimkeep, DType, E>::kRedPass>::Error_TypeCheck_Not_Pass_For_Reduce_Exp();
  typedef Shape<expr::ExpInfo<E>::kDim> EShape;
  const EShape eshape = expr::ShapeCheck<expr::ExpInfo<E>::kDim, E>::Check(exp.self());
  const Shape<1> dshape = expr::ShapeCheck<1, R>::Check(dst->self());
  CHECK_EQ(eshape[dimkeep], dshape[0]) << "MapReduceKeepHighDim::reduction dimension do not match";
  // (everything before the kept dimension, kept, everything between it and the last, last)
  const Shape<4> pshape = Shape4(eshape.ProdShape(0, dimkeep), eshape[dimkeep],
                                 eshape.ProdShape(dimkeep + 1, EShape::kSubdim), eshape[EShape::kSubdim]);
  const cudaStream_t stream = Stream<gpu>::GetStream(expr::StreamInfo<gpu, R>::Get(dst->self()));
  if (pshape[1] == 0) return;
  cuda::KeepHighDimGo<Saver, Reducer, DType>(
      dst->ptrself(), exp.self(), pshape, scale, stream,
      std::integral_constant<bool, expr::PackInfo<E>::kPass && expr::FlatInfo<E>::kPass>());
}

// ------------------------------- function-form operators ------------------------------------

inline void Softmax(Tensor<gpu, 2, float> dst, const Tensor<gpu, 2, float> &src) {
  CHECK_EQ(dst.shape_, src.shape_) << "Softmax: shape mismatch";
  cuda::SoftmaxLaunch(dst.dptr_, src.dptr_, dst.size(0), dst.size(1), dst.stride_, src.stride_,
                      Stream<gpu>::GetStream(dst.stream_));
}
namespace cuda {
inline void SoftmaxGradCheck(const Tensor<gpu, 2, float> &dst, const Tensor<gpu, 2, float> &src,
                             const Tensor<gpu, 1, float> &label) {
  CHECK_EQ(dst.shape_, src.shape_) << "SoftmaxGrad: shape mismatch";
  CHECK_EQ(dst.size(0), label.size(0)) << "SoftmaxGrad: label shape mismatch";
}
}  // namespace cuda

inline void SoftmaxGrad(Tensor<gpu, 2, float> dst, const Tensor<gpu, 2, float> &src,
                        const Tensor<gpu, 1, float> &label) {
  cuda::SoftmaxGradCheck(dst, src, label);
  cuda::SoftmaxGradLaunch(dst.dptr_, src.dptr_, label.dptr_, dst.size(0), dst.size(1), dst.stride_, src.stride_, 0,
                          0.0f, 0.0f, Stream<gpu>::GetStream(dst.stream_));
}
inline void SoftmaxGrad(const Tensor<gpu, 2, float> &dst, const Tensor<gpu, 2, float> &src,
                        const Tensor<gpu, 1, float> &label, const float &ignore_label) {
  cuda::SoftmaxGradCheck(dst, src, label);
  cuda::SoftmaxGradLaunch(dst.dptr_, src.dptr_, label.dptr_, dst.size(0), dst.size(1), dst.stride_, src.stride_, 2,
                          ignore_label, 0.0f, Stream<gpu>::GetStream(dst.stream_));
}
inline void SmoothSoftmaxGrad(Tensor<gpu, 2, float> dst, const Tensor<gpu, 2, float> &src,
                              const Tensor<gpu, 1, float> &label, const float alpha) {
  cuda::SoftmaxGradCheck(dst, src, label);
  cuda::SoftmaxGradLaunch(dst.dptr_, src.dptr_, label.dptr_, dst.size(0), dst.size(1), dst.stride_, src.stride_, 1,
                          0.0f, alpha, Stream<gpu>::GetStream(dst.stream_));
}
inline void SmoothSoftmaxGrad(const Tensor<gpu, 2, float> &dst, const Tensor<gpu, 2, float> &src,
                              const Tensor<gpu, 1, float> &label, const float &ignore_label, const float alpha) {
  cuda::SoftmaxGradCheck(dst, src, label);
  cuda::SoftmaxGradLaunch(dst.dptr_, src.dptr_, label.dptr_, dst.size(0), dst.size(1), dst.stride_, src.stride_, 3,
                          ignore_label, alpha, Stream<gpu>::GetStream(dst.stream_));
}

/*! \brief softmax over the middle axis of (batch, classes, positions); mshadow/tensor_gpu-inl.h:163-167 */
inline void Softmax(Tensor<gpu, 3, float> dst, const Tensor<gpu, 3, float> &src) {
  CHECK_EQ(dst.shape_, src.shape_) << "Softmax: shape mismatch";
  cuda::Softmax3DLaunch(dst.dptr_, src.dptr_, dst.size(0), dst.size(1), dst.size(2), dst.stride_, src.stride_,
                        Stream<gpu>::GetStream(dst.stream_));
}
namespace cuda {
inline void SoftmaxGrad3DGo(const Tensor<gpu, 3, float> &dst, const Tensor<gpu, 3, float> &src,
                            const Tensor<gpu, 2, float> &label, int mode, float ignore_label, float alpha) {
  CHECK_EQ(dst.shape_, src.shape_) << "SoftmaxGrad: shape mismatch";
  CHECK_EQ(dst.size(0), label.size(0)) << "SoftmaxGrad: label shape mismatch";
  CHECK_EQ(dst.size(2), label.size(1)) << "SoftmaxGrad: label shape mismatch";
  SoftmaxGrad3DLaunch(dst.dptr_, src.dptr_, label.dptr_, dst.size(0), dst.size(1), dst.size(2), dst.stride_,
                      src.stride_, label.stride_, mode, ignore_label, alpha, Stream<gpu>::GetStream(dst.stream_));
}
}  // namespace cuda
/*! \brief 3-D gradient forms, label(y, n) per position; mshadow/tensor_gpu-inl.h:201-214, tensor_cpu-inl.h:370-462 */
inline void SoftmaxGrad(const Tensor<gpu, 3, float> &dst, const Tensor<gpu, 3, float> &src,
                        const Tensor<gpu, 2, float> &label) {
  cuda::SoftmaxGrad3DGo(dst, src, label, 0, 0.0f, 0.0f);
}
inline void SoftmaxGrad(const Tensor<gpu, 3, float> &dst, const Tensor<gpu, 3, float> &src,
                        const Tensor<gpu, 2, float> &label, const float &ignore_label) {
  cuda::SoftmaxGrad3DGo(dst, src, label, 2, ignore_label, 0.0f);
}
inline void SmoothSoftmaxGrad(const Tensor<gpu, 3, float> &dst, const Tensor<gpu, 3, float> &src,
                              const Tensor<gpu, 2, float> &label, const float alpha) {
  cuda::SoftmaxGrad3DGo(dst, src, label, 1, 0.0f, alpha);
}
inline void SmoothSoftmaxGrad(const Tensor<gpu, 3, float> &dst, const Tensor<gpu, 3, float> &src,
                              const Tensor<gpu, 2, float> &label, const float &ignore_label, const float alpha) {
  cuda::SoftmaxGrad3DGo(dst, src, label, 3, ignore_label, alpha);
}

/*!
 * \brief dst = Softmax(logits) - onehot(label) in one pass over memory: what
 *  `Softmax(p, logits); SoftmaxGrad(dst, p, label);` computes, for loss layers that only
 *  need the gradient.  Not part of the reference API; it saves the write and re-read of p.
 */
inline void SoftmaxGradFused(Tensor<gpu, 2, float> dst, const Tensor<gpu, 2, float> &logits,
                             const Tensor<gpu, 1, float> &label) {
  cuda::SoftmaxGradCheck(dst, logits, label);
  cuda::SoftmaxLaunch(dst.dptr_, logits.dptr_, dst.size(0), dst.size(1), dst.stride_, logits.stride_,
                      Stream<gpu>::GetStream(dst.stream_), label.dptr_);
}

inline void AddTakeGrad(Tensor<gpu, 2, float> dst, const Tensor<gpu, 1, int32_t> &index,
                        const Tensor<gpu, 2, float> &src) {
  CHECK_EQ(dst.size(1), src.size(1)) << "AddTakeGrad: shape of src mismatch";
  CHECK_EQ(index.size(0), src.size(0)) << "AddTakeGrad: shape of index/src mismatch";
  cuda::AddTakeGradLaunch(dst.dptr_, dst.stride_, index.dptr_, src.dptr_, src.stride_, dst.size(0), index.size(0),
                          dst.size(1), Stream<gpu>::GetStream(dst.stream_));
}

inline void AddTakeGradLargeBatch(Tensor<gpu, 2, float> dst, const Tensor<gpu, 1, int32_t> &sorted,
                                  const Tensor<gpu, 1, int32_t> &index, const Tensor<gpu, 2, float> &src) {
  CHECK_EQ(dst.CheckContiguous(), true);
  CHECK_EQ(sorted.CheckContiguous(), true);
  CHECK_EQ(index.CheckContiguous(), true);
  CHECK_EQ(src.CheckContiguous(), true);
  CHECK_EQ(dst.size(1), src.size(1)) << "AddTakeGradLargeBatch: shape of src mismatch";
  CHECK_EQ(sorted.size(0), index.size(0)) << "AddTakeGradLargeBatch: shape of sorted/index mismatch";
  cuda::AddTakeGradLargeBatchLaunch(dst.dptr_, dst.stride_, sorted.dptr_, index.dptr_, src.dptr_, src.stride_,
                                    sorted.size(0), dst.size(1), Stream<gpu>::GetStream(dst.stream_));
}

template <typename KDType, typename VDType>
inline void SortByKey(Tensor<gpu, 1, KDType> keys, Tensor<gpu, 1, VDType> values, bool is_ascend = true) {
  CHECK_EQ(keys.CheckContiguous(), true);
  CHECK_EQ(values.CheckContiguous(), true);
  CHECK_EQ(keys.size(0), values.size(0)) << "The sizes of key/value are not equal! keys_size: " << keys.size(0)
                                         << "values_size: " << values.size(0);
  cuda::SortPairsLaunch(keys.dptr_, values.dptr_, keys.size(0), is_ascend, Stream<gpu>::GetStream(keys.stream_));
}

/*!
 * \brief dst[index[y]] = src[y] (mshadow/tensor_gpu-inl.h:237-242).  Where several entries name one
 *  row the result is the CPU's (the last entry stays), not the reference kernel's race.
 */
inline void IndexFill(Tensor<gpu, 2, float> dst, const Tensor<gpu, 1, int32_t> &index,
                      const Tensor<gpu, 2, float> &src) {
  CHECK_EQ(dst.CheckContiguous(), true);
  CHECK_EQ(index.CheckContiguous(), true);
  CHECK_EQ(src.CheckContiguous(), true);
  CHECK_EQ(dst.size(1), src.size(1)) << "IndexFill: shape mismatch";
  CHECK_EQ(index.size(0), src.size(0)) << "IndexFill: shape mismatch";
  cuda::IndexFillLaunch(dst.dptr_, dst.stride_, index.dptr_, src.dptr_, src.stride_, dst.size(0), index.size(0),
                        dst.size(1), Stream<gpu>::GetStream(dst.stream_));
}

/*!
 * \brief sort `values` inside each run of equal `segments` (ascending on entry) by two stable
 *  pair sorts, as mshadow/tensor_cpu-inl.h:562-567 does on either device
 */
template <typename VDType, typename SDType>
inline void VectorizedSort(Tensor<gpu, 1, VDType> values, Tensor<gpu, 1, SDType> segments) {
  SortByKey(values, segments, true);
  SortByKey(segments, values, true);
}

}  // namespace mshadow
#endif  // MSHADOW_GPU_ENGINE_CUH_
