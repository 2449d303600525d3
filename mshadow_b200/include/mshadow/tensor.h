/*
 * Data handles of the mshadow API -- Shape, Stream, Tensor -- and the declarations of every
 * free function of the lazy-evaluation path.  Including this header pulls in the whole
 * engine, exactly as `#include <mshadow/tensor.h>` does for dmlc/mshadow.
 *
 * The public surface (type names, members dptr_/shape_/stride_/stream_, constructors,
 * function signatures) follows mshadow/tensor.h of the reference (:50-179 Shape, :364-382
 * Stream, :390-392 TRValue, :400-614 Tensor, :625-1050 functions).  The implementation is
 * new and targets one device generation: NVIDIA B200 (sm_100a).
 */
#ifndef MSHADOW_TENSOR_H_
#define MSHADOW_TENSOR_H_

#include <iostream>
#include <string>

#include "./base.h"
#include "./half.h"
#include "./expression.h"

namespace mshadow {

/*! \brief device tag: host memory */
struct cpu {
  static const bool kDevCPU = true;
  static const int kDevMask = 1 << 0;
};
/*! \brief device tag: CUDA device memory */
struct gpu {
  static const bool kDevCPU = false;
  static const int kDevMask = 1 << 1;
};

template <int ndim>
struct Shape;
template <int ndim>
inline std::ostream &operator<<(std::ostream &os, const Shape<ndim> &shape);

/*! \brief extents of a tensor, highest dimension first */
template <int dimension>
struct Shape {
  static const int kDimension = dimension;
  static const int kSubdim = dimension - 1;
  index_t shape_[kDimension];

  MSHADOW_XINLINE Shape() {}
  MSHADOW_XINLINE Shape(const Shape<kDimension> &s) {
#pragma unroll
    for (int i = 0; i < kDimension; ++i) shape_[i] = s[i];
  }
  MSHADOW_XINLINE Shape<kDimension> &operator=(const Shape<kDimension> &s) {
#pragma unroll
    for (int i = 0; i < kDimension; ++i) shape_[i] = s[i];
    return *this;
  }
  MSHADOW_XINLINE index_t &operator[](int idx) { return shape_[idx]; }
  MSHADOW_XINLINE const index_t &operator[](int idx) const { return shape_[idx]; }
  MSHADOW_XINLINE bool operator==(const Shape<kDimension> &s) const {
    bool same = true;
#pragma unroll
    for (int i = 0; i < kDimension; ++i) same = same && (shape_[i] == s.shape_[i]);
    return same;
  }
  MSHADOW_XINLINE bool operator!=(const Shape<kDimension> &s) const { return !(*this == s); }
  /*! \brief product of extents [dimstart, dimend) */
  MSHADOW_XINLINE index_t ProdShape(int dimstart, int dimend) const {
    index_t n = 1;
    for (int i = dimstart; i < dimend; ++i) n *= shape_[i];
    return n;
  }
  MSHADOW_XINLINE index_t Size() const { return ProdShape(0, kDimension); }
  MSHADOW_XINLINE Shape<1> FlatTo1D() const {
    Shape<1> s;
    s[0] = Size();
    return s;
  }
  /*! \brief (product of all but the last extent, last extent) */
  MSHADOW_XINLINE Shape<2> FlatTo2D() const {
    Shape<2> s;
    s[1] = shape_[kDimension - 1];
    s[0] = ProdShape(0, kDimension - 1);
    return s;
  }
  /*! \brief drop the highest dimension */
  MSHADOW_XINLINE Shape<kSubdim> SubShape() const {
    Shape<kSubdim> s;
#pragma unroll
    for (int i = 0; i < kSubdim; ++i) s.shape_[i] = shape_[i + 1];
    return s;
  }
  template <int dimstart, int dimend>
  MSHADOW_XINLINE Shape<dimend - dimstart> Slice() const {
    Shape<dimend - dimstart> s;
#pragma unroll
    for (int i = dimstart; i < dimend; ++i) s[i - dimstart] = shape_[i];
    return s;
  }
  template <int dim>
  friend std::ostream &operator<<(std::ostream &os, const Shape<dim> &shape);
};

MSHADOW_XINLINE Shape<1> Shape1(index_t s0) {
  Shape<1> s;
  s[0] = s0;
  return s;
}
MSHADOW_XINLINE Shape<2> Shape2(index_t s0, index_t s1) {
  Shape<2> s;
  s[0] = s0;
  s[1] = s1;
  return s;
}
MSHADOW_XINLINE Shape<3> Shape3(index_t s0, index_t s1, index_t s2) {
  Shape<3> s;
  s[0] = s0;
  s[1] = s1;
  s[2] = s2;
  return s;
}
MSHADOW_XINLINE Shape<4> Shape4(index_t s0, index_t s1, index_t s2, index_t s3) {
  Shape<4> s;
  s[0] = s0;
  s[1] = s1;
  s[2] = s2;
  s[3] = s3;
  return s;
}
MSHADOW_XINLINE Shape<5> Shape5(index_t s0, index_t s1, index_t s2, index_t s3, index_t s4) {
  Shape<5> s;
  s[0] = s0;
  s[1] = s1;
  s[2] = s2;
  s[3] = s3;
  s[4] = s4;
  return s;
}

template <int ndim>
inline std::ostream &operator<<(std::ostream &os, const Shape<ndim> &shape) {
  os << '(';
  for (int i = 0; i < ndim; ++i) {
    if (i != 0) os << ',';
    os << shape[i];
  }
  if (ndim == 1) os << ',';
  os << ')';
  return os;
}

/*! \brief execution queue of a device; the host one does nothing */
template <typename Device>
struct Stream {
  inline void Wait() {}
  inline bool CheckIdle() { return true; }
  inline void CreateBlasHandle() {}
};

/*! \brief common base of everything that behaves like a tensor l-value */
template <typename Container, typename Device, int dimension, typename DType>
struct TRValue : public expr::RValueExp<Container, DType> {};

/*!
 * \brief non-owning view of `dimension`-d data on `Device`.
 *  Rows of the last dimension are `stride_` elements apart; all other dimensions are dense.
 */
template <typename Device, int dimension, typename DType MSHADOW_DEFAULT_DTYPE>
struct Tensor : public TRValue<Tensor<Device, dimension, DType>, Device, dimension, DType> {
 public:
  static const bool kDevCPU = Device::kDevCPU;
  static const int kSubdim = dimension - 1;
  DType *dptr_ = nullptr;
  Shape<dimension> shape_;
  index_t stride_;
  Stream<Device> *stream_;

  MSHADOW_XINLINE Tensor() : stream_(NULL) {}
  MSHADOW_XINLINE explicit Tensor(const Shape<dimension> &shape) : shape_(shape), stream_(NULL) {}
  MSHADOW_XINLINE Tensor(DType *dptr, const Shape<dimension> &shape)
      : dptr_(dptr), shape_(shape), stride_(shape[kSubdim]), stream_(NULL) {}
  MSHADOW_XINLINE Tensor(DType *dptr, const Shape<dimension> &shape, Stream<Device> *stream)
      : dptr_(dptr), shape_(shape), stride_(shape[kSubdim]), stream_(stream) {}
  MSHADOW_XINLINE Tensor(DType *dptr, const Shape<dimension> &shape, index_t stride,
                         Stream<Device> *stream)
      : dptr_(dptr), shape_(shape), stride_(stride), stream_(stream) {}

  inline void set_stream(Stream<Device> *stream) { this->stream_ = stream; }
  /*! \brief elements spanned from dimension `startdim` on, padding included */
  template <int startdim>
  MSHADOW_XINLINE index_t MemSize() const {
    index_t n = this->stride_;
#pragma unroll
    for (int i = startdim; i < kSubdim; ++i) n *= this->shape_[i];
    return n;
  }
  MSHADOW_XINLINE bool CheckContiguous() const { return this->shape_[dimension - 1] == stride_; }
  MSHADOW_XINLINE index_t MSize() const { return this->MemSize<0>(); }
  MSHADOW_XINLINE index_t size(int idx) const { return shape_[idx]; }
  MSHADOW_XINLINE Tensor<Device, 1, DType> FlatTo1D() const {
    return Tensor<Device, 1, DType>(dptr_, shape_.FlatTo1D(), stride_, stream_);
  }
  MSHADOW_XINLINE Tensor<Device, 2, DType> FlatTo2D() const {
    return Tensor<Device, 2, DType>(dptr_, shape_.FlatTo2D(), stride_, stream_);
  }
  MSHADOW_XINLINE Tensor<Device, kSubdim, DType> operator[](index_t idx) const {
    return Tensor<Device, kSubdim, DType>(dptr_ + this->MemSize<1>() * idx, shape_.SubShape(),
                                          stride_, stream_);
  }
  /*! \brief sub-range [begin, end) of the highest dimension */
  MSHADOW_XINLINE Tensor<Device, dimension, DType> Slice(index_t begin, index_t end) const {
    Shape<dimension> s = this->shape_;
    s[0] = end - begin;
    return Tensor<Device, dimension, DType>(dptr_ + this->MemSize<1>() * begin, s, stride_,
                                            stream_);
  }
  inline Tensor<Device, dimension, DType> &operator=(const Tensor<Device, dimension, DType> &t) {
    dptr_ = t.dptr_;
    shape_ = t.shape_;
    stride_ = t.stride_;
    stream_ = t.stream_;
    return *this;
  }
  MSHADOW_XINLINE Tensor(const Tensor<Device, dimension, DType> &t)
      : dptr_(t.dptr_), shape_(t.shape_), stride_(t.stride_), stream_(t.stream_) {}
  template <typename E, int etype>
  inline Tensor<Device, dimension, DType> &operator=(const expr::Exp<E, DType, etype> &e) {
    return this->__assign(e);
  }
  inline Tensor<Device, dimension, DType> &operator=(const DType &s) { return this->__assign(s); }
};

/*! \brief 1-d tensors index to elements, and slices keep a dense stride */
template <typename Device, typename DType>
struct Tensor<Device, 1, DType> : public TRValue<Tensor<Device, 1, DType>, Device, 1, DType> {
 public:
  DType *dptr_ = nullptr;
  Shape<1> shape_;
  index_t stride_;
  Stream<Device> *stream_;

  MSHADOW_XINLINE Tensor() : stream_(NULL) {}
  MSHADOW_XINLINE explicit Tensor(const Shape<1> &shape) : shape_(shape), stream_(NULL) {}
  MSHADOW_XINLINE Tensor(DType *dptr, Shape<1> shape)
      : dptr_(dptr), shape_(shape), stride_(shape[0]), stream_(NULL) {}
  MSHADOW_XINLINE Tensor(DType *dptr, Shape<1> shape, Stream<Device> *stream)
      : dptr_(dptr), shape_(shape), stride_(shape[0]), stream_(stream) {}
  MSHADOW_XINLINE Tensor(DType *dptr, Shape<1> shape, index_t stride, Stream<Device> *stream)
      : dptr_(dptr), shape_(shape), stride_(stride), stream_(stream) {}

  inline void set_stream(Stream<Device> *stream) { this->stream_ = stream; }
  MSHADOW_XINLINE Tensor<Device, 1, DType> FlatTo1D() const { return *this; }
  MSHADOW_XINLINE Tensor<Device, 2, DType> FlatTo2D() const {
    return Tensor<Device, 2, DType>(dptr_, shape_.FlatTo2D(), stride_, stream_);
  }
  MSHADOW_XINLINE Tensor<Device, 1, DType> Slice(index_t begin, index_t end) const {
    Shape<1> s;
    s[0] = end - begin;
    return Tensor<Device, 1, DType>(dptr_ + begin, s, s[0], stream_);
  }
  MSHADOW_XINLINE bool CheckContiguous() const { return true; }
  MSHADOW_XINLINE index_t MSize() const { return shape_[0]; }
  MSHADOW_XINLINE index_t size(index_t i) const { return shape_[0]; }
  MSHADOW_XINLINE DType &operator[](index_t idx) { return dptr_[idx]; }
  MSHADOW_XINLINE const DType &operator[](index_t idx) const { return dptr_[idx]; }
  inline Tensor<Device, 1, DType> &operator=(const Tensor<Device, 1, DType> &t) {
    dptr_ = t.dptr_;
    shape_ = t.shape_;
    stride_ = t.stride_;
    stream_ = t.stream_;
    return *this;
  }
  MSHADOW_XINLINE Tensor(const Tensor<Device, 1, DType> &t)
      : dptr_(t.dptr_), shape_(t.shape_), stride_(t.stride_), stream_(t.stream_) {}
  template <typename E, int etype>
  inline Tensor<Device, 1, DType> &operator=(const expr::Exp<E, DType, etype> &e) {
    return this->__assign(e);
  }
  inline Tensor<Device, 1, DType> &operator=(const DType &s) { return this->__assign(s); }
};

// ------------------------------------------------------------------------------------
// engine life cycle, streams, memory
// ------------------------------------------------------------------------------------
template <typename Device>
inline void InitTensorEngine(int device_id = 0);
template <typename Device>
inline void ShutdownTensorEngine();
template <typename Device>
inline void SetDevice(int devid);
/*! \brief the BLAS / DNN handle requests are accepted and ignored: this engine has no BLAS bridge */
template <typename Device>
inline Stream<Device> *NewStream(bool create_blas_handle, bool create_dnn_handle, int dev_id = -1);
template <typename Device>
inline Stream<Device> *NewStream(int dev_id) {
  return NewStream<Device>(true, false, dev_id);
}
template <typename Device>
inline void DeleteStream(Stream<Device> *stream);

template <int dim, typename DType>
inline void AllocSpace(Tensor<cpu, dim, DType> *obj, bool pad = MSHADOW_ALLOC_PAD);
template <int dim, typename DType>
inline void AllocSpace(Tensor<gpu, dim, DType> *obj, bool pad = MSHADOW_ALLOC_PAD);
template <int dim, typename DType>
inline void FreeSpace(Tensor<cpu, dim, DType> *obj);
template <int dim, typename DType>
inline void FreeSpace(Tensor<gpu, dim, DType> *obj);
template <typename Device, typename DType, int dim>
inline Tensor<Device, dim, DType> NewTensor(const Shape<dim> &shape, DType initv,
                                            bool pad = MSHADOW_ALLOC_PAD,
                                            Stream<Device> *stream = NULL);

/*! \brief row-wise copies that honour both strides; device copies are asynchronous on `stream` */
template <int dim, typename DType>
inline void Copy(Tensor<cpu, dim, DType> dst, const Tensor<cpu, dim, DType> &src,
                 Stream<cpu> *stream = NULL);
template <int dim, typename DType>
inline void Copy(Tensor<cpu, dim, DType> dst, const Tensor<gpu, dim, DType> &src,
                 Stream<gpu> *stream = NULL);
template <int dim, typename DType>
inline void Copy(Tensor<gpu, dim, DType> dst, const Tensor<cpu, dim, DType> &src,
                 Stream<gpu> *stream = NULL);
template <int dim, typename DType>
inline void Copy(Tensor<gpu, dim, DType> dst, const Tensor<gpu, dim, DType> &src,
                 Stream<gpu> *stream = NULL);

// ------------------------------------------------------------------------------------
// expression evaluation entry points
// ------------------------------------------------------------------------------------
/*! \brief dst <Saver>= exp, element-wise, on the destination's device */
template <typename Saver, typename R, int dim, typename DType, typename E, int etype>
inline void MapExp(TRValue<R, cpu, dim, DType> *dst, const expr::Exp<E, DType, etype> &exp);
template <typename Saver, typename R, int dim, typename DType, typename E, int etype>
inline void MapExp(TRValue<R, gpu, dim, DType> *dst, const expr::Exp<E, DType, etype> &exp);
/*! \brief dst[x] <Saver>= scale * Reducer over y of exp(y, x) */
template <typename Saver, typename Reducer, typename R, typename DType, typename E, int etype>
inline void MapReduceKeepLowest(TRValue<R, gpu, 1, DType> *dst,
                                const expr::Exp<E, DType, etype> &exp, DType scale = 1);
/*! \brief dst[c] <Saver>= scale * Reducer over everything but dimension `dimkeep` */
template <typename Saver, typename Reducer, int dimkeep, typename R, typename DType, typename E,
          int etype>
inline void MapReduceKeepHighDim(TRValue<R, gpu, 1, DType> *dst,
                                 const expr::Exp<E, DType, etype> &exp, DType scale = 1);

}  // namespace mshadow

#include "./engine/plan.h"
#include "./engine/check.h"
#if MSHADOW_USE_CUDA
#include "./gpu/runtime.h"
#endif
#include "./extension.h"
#include "./cpu/host.h"
#if MSHADOW_USE_CUDA && defined(__CUDACC__)
#include "./gpu/engine.cuh"
#endif
#include "./tensor_container.h"

#endif  // MSHADOW_TENSOR_H_
