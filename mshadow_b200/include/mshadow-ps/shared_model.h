/*
 * ISharedModel: the interface through which replicated tensors are synchronised across GPUs,
 * as in dmlc/mshadow's mshadow-ps (mshadow-ps/mshadow_ps.h:37-258).  Implementations:
 * NcclModel (mshadow_ps.h) and PeerModel (peer_model.h).
 */
#ifndef MSHADOW_PS_SHARED_MODEL_H_
#define MSHADOW_PS_SHARED_MODEL_H_

#include <functional>
#include <vector>

#include "../mshadow/tensor.h"

namespace mshadow {
namespace ps {

/*! \brief interface of a synchronised key -> tensor store; see the file comment */
template <typename xpu, typename DType MSHADOW_DEFAULT_DTYPE>
class ISharedModel {
 public:
  /*! \brief called after a pull's data has been enqueued; may enqueue more work on `stream` */
  typedef void(CallbackFunction)(Stream<xpu> *stream, void *arg);
  virtual ~ISharedModel() {}
  virtual void SetParam(const char *, const char *) {}
  virtual void Init(const std::vector<int> &) {}
  inline void Init() {
    std::vector<int> dev;
    dev.push_back(0);
    this->Init(dev);
  }
  template <int dim>
  inline void InitKey(Shape<dim> shape, int key, int devid) {
    this->InitKey_(shape.FlatTo2D(), key, devid);
  }
  virtual void PullWait(int key, int devid) = 0;
  /*!
   * \brief device-side PullWait: work enqueued on `stream` after this call runs after the last
   *  pull of `key` has completed; the host does not block (an extension of the reference
   *  interface, for consumers that stay on the GPU).  The default falls back to PullWait.
   */
  virtual void PullFence(int key, int devid, Stream<xpu> *stream) {
    (void)stream;
    this->PullWait(key, devid);
  }
  template <int dim>
  inline void CheckWeight(Tensor<xpu, dim, DType> data, int key, int devid) {
    this->CheckWeight_(data.FlatTo2D(), key, devid);
  }
  template <int dim>
  inline void SetWeight(Tensor<xpu, dim, DType> data, int key, int devid) {
    this->SetWeight_(data.FlatTo2D(), key, devid);
  }
  template <int dim>
  inline void Push(Tensor<xpu, dim, DType> data, int key, int devid, int priority = 0) {
    this->Push_(data.FlatTo2D(), key, devid, priority);
  }
  template <int dim>
  inline void PullReq(Tensor<xpu, dim, DType> data, int key, int devid, int priority = 0,
                      CallbackFunction callback = NULL, void *callback_arg = NULL) {
    this->PullReq_(data.FlatTo2D(), key, devid, priority, callback, callback_arg);
  }
  template <int dim>
  inline void PullReq(Tensor<xpu, dim, DType> data, int key, int devid, int priority,
                      std::function<void(Stream<xpu> *stream)> callback) {
    auto *held = new std::function<void(Stream<xpu> *stream)>(callback);
    this->PullReq(data, key, devid, priority, InvokeLambda_, held);
  }
  virtual void SetWeight_(Tensor<xpu, 2, DType> data, int key, int devid) = 0;
  virtual void CheckWeight_(Tensor<xpu, 2, DType> data, int key, int devid) = 0;

 protected:
  virtual void InitKey_(Shape<2> shape, int key, int devid) = 0;
  virtual void Push_(Tensor<xpu, 2, DType> data, int key, int devid, int priority = 0) = 0;
  virtual void PullReq_(Tensor<xpu, 2, DType> data, int key, int devid, int priority, CallbackFunction callback,
                        void *callback_arg) = 0;

 private:
  inline static void InvokeLambda_(Stream<xpu> *stream, void *fun) {
    auto *fp = static_cast<std::function<void(Stream<xpu> *stream)> *>(fun);
    (*fp)(stream);
    delete fp;
  }
};

}  // namespace ps
}  // namespace mshadow
#endif  // MSHADOW_PS_SHARED_MODEL_H_
