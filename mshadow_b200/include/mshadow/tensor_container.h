/*
 * TensorContainer: a Tensor that owns its memory and can be resized.
 * Interface after dmlc/mshadow's mshadow/tensor_container.h (:21-206), minus binary
 * save/load (serialisation is outside this engine).  Memory only ever grows: Resize keeps the
 * allocation when the new shape fits.
 */
#ifndef MSHADOW_TENSOR_CONTAINER_H_
#define MSHADOW_TENSOR_CONTAINER_H_

#include "./tensor.h"

namespace mshadow {

template <typename Device, int dimension, typename DType = default_real_t>
class TensorContainer : public Tensor<Device, dimension, DType> {
 public:
  typedef Tensor<Device, dimension, DType> Base;

  explicit TensorContainer(bool pad = MSHADOW_ALLOC_PAD) : pad_(pad) {
    this->dptr_ = data_.dptr_ = NULL;
    this->shape_[0] = 0;
    this->stride_ = 0;
    data_.stride_ = 0;
    data_.shape_[0] = 0;
  }
  explicit TensorContainer(const Shape<dimension> &shape) : pad_(MSHADOW_ALLOC_PAD) {
    data_.dptr_ = NULL;
    Allocate(shape);
  }
  TensorContainer(const Shape<dimension> &shape, DType initv) : pad_(MSHADOW_ALLOC_PAD) {
    data_.dptr_ = NULL;
    Allocate(shape);
    (*this) = initv;
  }
  /*! \brief deep copy */
  TensorContainer(const TensorContainer<Device, dimension, DType> &src) : pad_(src.pad_) {
    data_.dptr_ = NULL;
    this->dptr_ = NULL;
    this->stream_ = src.stream_;
    if (src.dptr_ != NULL) {
      Allocate(src.shape_);
      Copy(*this, src, this->stream_);
    }
  }
  ~TensorContainer() { Release(); }

  /*! \brief change the shape; contents are unspecified afterwards */
  inline void Resize(const Shape<dimension> &shape) {
    const Shape<2> want = shape.FlatTo2D();
    if (data_.dptr_ != NULL && want[1] <= data_.shape_[1] && want[0] <= data_.shape_[0]) {
      this->shape_ = shape;
      this->stride_ = data_.stride_;
      this->dptr_ = data_.dptr_;
    } else {
      Allocate(shape);
    }
  }
  inline void Resize(const Shape<dimension> &shape, DType initv) {
    Resize(shape);
    (*this) = initv;
  }
  inline void set_pad(bool pad) { pad_ = pad; }
  /*! \brief give the memory back; the container becomes empty */
  inline void Release() {
    if (data_.dptr_ != NULL) {
      this->shape_[0] = 0;
      this->stride_ = 0;
      data_.stride_ = 0;
      data_.shape_[0] = 0;
      FreeSpace(&data_);
      data_.dptr_ = this->dptr_ = NULL;
    }
  }

  inline Base &operator=(DType s) { return this->__assign(s); }
  template <typename E, int etype>
  inline Base &operator=(const expr::Exp<E, DType, etype> &e) {
    return this->__assign(e);
  }
  inline TensorContainer &operator=(const TensorContainer &src) {
    if (this != &src) {
      Resize(src.shape_);
      Copy(*this, src, this->stream_);
    }
    return *this;
  }

 private:
  inline void Allocate(const Shape<dimension> &shape) {
    if (data_.dptr_ != NULL) Release();
    data_.shape_ = shape.FlatTo2D();
    AllocSpace(&data_, pad_);
    this->dptr_ = data_.dptr_;
    this->shape_ = shape;
    this->stride_ = pad_ ? data_.stride_ : data_.size(1);
  }
  bool pad_;
  /*! \brief the allocation, viewed as a matrix */
  Tensor<Device, 2, DType> data_;
};

}  // namespace mshadow
#endif  // MSHADOW_TENSOR_CONTAINER_H_
