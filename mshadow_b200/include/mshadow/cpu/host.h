/*
 * Host-side tensors: allocation, copies and a plain element-wise evaluator.
 *
 * This engine computes on the GPU; `Tensor<cpu, ...>` exists so that user code can stage
 * inputs and read back results through the same API as with dmlc/mshadow
 * (mshadow/tensor_cpu-inl.h:19-201): InitTensorEngine<cpu>, AllocSpace / FreeSpace / NewTensor,
 * AllocHost<gpu> (page-locked), Copy, and `host_tensor = expression` evaluated by a scalar
 * loop so that initialisation code such as `t = 0.0f` works on either device.  Reductions
 * and the function-form operators are GPU-only; nothing on the GPU path ever runs here.
 */
#ifndef MSHADOW_CPU_HOST_H_
#define MSHADOW_CPU_HOST_H_

#include <cstdlib>
#include <cstring>

#include "../engine/check.h"

namespace mshadow {

template <>
inline void InitTensorEngine<cpu>(int) {}
template <>
inline void ShutdownTensorEngine<cpu>() {}
template <>
inline void SetDevice<cpu>(int) {}
template <>
inline Stream<cpu> *NewStream<cpu>(bool, bool, int) {
  return new Stream<cpu>();
}
template <>
inline void DeleteStream<cpu>(Stream<cpu> *stream) {
  delete stream;
}

namespace hostdetail {
/*! \brief rows padded to 16 bytes, base aligned to 64 */
inline void *AlignedRows(size_t *pitch_bytes, size_t row_bytes, size_t rows) {
  const size_t pitch = (row_bytes + 15) / 16 * 16;
  *pitch_bytes = pitch;
  void *p = nullptr;
  const size_t total = pitch * rows;
  const int rc = posix_memalign(&p, 64, total == 0 ? 64 : total);
  CHECK(rc == 0 && p != nullptr) << "AllocSpace: out of host memory";
  return p;
}
}  // namespace hostdetail

template <int dim, typename DType>
inline void AllocSpace(Tensor<cpu, dim, DType> *obj, bool pad) {
  size_t pitch = 0;
  const Shape<2> flat = obj->shape_.FlatTo2D();
  if (pad) {
    obj->dptr_ = static_cast<DType *>(hostdetail::AlignedRows(&pitch, flat[1] * sizeof(DType), flat[0]));
    obj->stride_ = static_cast<index_t>(pitch / sizeof(DType));
  } else {
    obj->stride_ = obj->size(dim - 1);
    obj->dptr_ = static_cast<DType *>(
        hostdetail::AlignedRows(&pitch, static_cast<size_t>(flat[0]) * flat[1] * sizeof(DType), 1));
  }
}
template <int dim, typename DType>
inline void FreeSpace(Tensor<cpu, dim, DType> *obj) {
  free(obj->dptr_);
  obj->dptr_ = NULL;
}

#if MSHADOW_USE_CUDA
/*! \brief page-locked host memory for fast, truly asynchronous device copies */
template <typename xpu, int dim, typename DType>
inline void AllocHost(Tensor<cpu, dim, DType> *obj) {
  obj->stride_ = obj->size(dim - 1);
  void *p = nullptr;
  MSHADOW_CUDA_CALL(cudaMallocHost(&p, static_cast<size_t>(obj->MSize()) * sizeof(DType), cudaHostAllocPortable));
  obj->dptr_ = static_cast<DType *>(p);
}
template <typename xpu, int dim, typename DType>
inline void FreeHost(Tensor<cpu, dim, DType> *obj) {
  CHECK(obj->dptr_ != NULL) << "FreeHost:: double free";
  MSHADOW_CUDA_CALL(cudaFreeHost(obj->dptr_));
  obj->dptr_ = NULL;
}
#endif

template <int dim, typename DType>
inline void Copy(Tensor<cpu, dim, DType> dst_nd, const Tensor<cpu, dim, DType> &src_nd, Stream<cpu> *) {
  CHECK_EQ(dst_nd.shape_, src_nd.shape_) << "Copy:shape mismatch:" << dst_nd.shape_ << " vs " << src_nd.shape_;
  const Tensor<cpu, 2, DType> dst = dst_nd.FlatTo2D(), src = src_nd.FlatTo2D();
  if (dst.CheckContiguous() && src.CheckContiguous()) {
    memcpy(dst.dptr_, src.dptr_, sizeof(DType) * static_cast<size_t>(dst.size(0)) * dst.size(1));
    return;
  }
  for (index_t y = 0; y < dst.size(0); ++y) {
    memcpy(dst.dptr_ + static_cast<size_t>(y) * dst.stride_, src.dptr_ + static_cast<size_t>(y) * src.stride_,
           sizeof(DType) * dst.size(1));
  }
}

/*! \brief host evaluation of `dst <Saver>= exp`, one element at a time */
template <typename Saver, typename R, int dim, typename DType, typename E, int etype>
inline void MapExp(TRValue<R, cpu, dim, DType> *dst, const expr::Exp<E, DType, etype> &exp) {
  expr::TypeCheckPass<expr::TypeCheck<cpu, dim, DType, E>::kMapPass>::Error_All_Tensor_in_Exp_Must_Have_Same_Type();
  const Shape<dim> eshape = expr::ShapeCheck<dim, E>::Check(exp.self());
  const Shape<dim> dshape = expr::ShapeCheck<dim, R>::Check(dst->self());
  CHECK(eshape[0] == 0 || eshape == dshape) << "Assignment: Shape of Tensors are not consistent with target, "
                                            << "eshape: " << eshape << " dshape:" << dshape;
  const Shape<2> flat = dshape.FlatTo2D();
  expr::Plan<R, DType> dplan = expr::MakePlan(dst->self());
  const expr::Plan<E, DType> splan = expr::MakePlan(exp.self());
  for (index_t y = 0; y < flat[0]; ++y)
    for (index_t x = 0; x < flat[1]; ++x) Saver::template Save<DType>(dplan.REval(y, x), splan.Eval(y, x));
}

template <typename Device, typename DType, int dim>
inline Tensor<Device, dim, DType> NewTensor(const Shape<dim> &shape, DType initv, bool pad, Stream<Device> *stream) {
  Tensor<Device, dim, DType> obj(shape);
  obj.stream_ = stream;
  AllocSpace(&obj, pad);
  MapExp<sv::saveto>(&obj, expr::ScalarExp<DType>(initv));
  return obj;
}

}  // namespace mshadow
#endif  // MSHADOW_CPU_HOST_H_
