/*
 * Synchronisation of replicated tensors across GPUs: the ISharedModel interface of
 * dmlc/mshadow's mshadow-ps (mshadow-ps/mshadow_ps.h:37-258) with one implementation,
 * NcclModel, built for NVLink/NVSwitch machines.
 *
 * The reference's LocalModel (mshadow-ps/ps_local-inl.h) lives in ONE process, runs one host
 * thread per device, copies every pushed tensor to pinned host memory, sums there and copies
 * the sum back to every device.  NcclModel keeps the interface and the semantics
 *     Push(data, key)      contribute `data` to the sum stored under `key`
 *     PullReq(data, key)   ask for that sum to be written into `data`, then run a callback
 *     PullWait(key)        block the host until the request has completed
 * but runs as one process per GPU, and the sum is one NCCL all-reduce on device memory over
 * NVLink: nothing is staged through the host.  Work is ordered without host synchronisation:
 * Push makes the model's communication stream wait (by an event) for what the tensor's own
 * stream has enqueued so far; the all-reduce, the copy into the requester's tensor and whatever
 * the callback enqueues run on the communication stream; PullWait waits for the event recorded
 * after them.
 *
 * Set-up (before Init): SetParam("world_size", n), SetParam("rank", r), and
 * SetParam("nccl_id", hex) with the identifier that NcclModel<DType>::NewUniqueIdHex()
 * returned on ONE rank and that the application handed to the others (file, socket, MPI, a
 * launcher's store: the model does not care).  Init takes the one device this process drives.
 * With world_size 1 (the default) no identifier is needed.
 *
 * Differences from the reference, all deliberate: a process drives one device, so the `devid`
 * arguments must name that device; `priority` is accepted and ignored (a single in-order
 * communication stream); server-side updaters (IModelUpdater, "update_on_server") are not
 * provided: every rank receives the plain sum.
 */
#ifndef MSHADOW_PS_H_
#define MSHADOW_PS_H_

#include <nccl.h>

#include <cstring>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "../mshadow/tensor.h"
#include "./shared_model.h"
#include "./peer_model.h"

namespace mshadow {
namespace ps {

#define MSHADOW_NCCL_CALL(call)                                                                   \
  {                                                                                               \
    const ncclResult_t nccl_status_ = (call);                                                     \
    CHECK_EQ(nccl_status_, ncclSuccess) << "NCCL: " << ncclGetErrorString(nccl_status_);         \
  }

namespace psdetail {
template <typename DType>
struct NcclType;
template <>
struct NcclType<float> {
  static const ncclDataType_t kType = ncclFloat32;
};
template <>
struct NcclType<double> {
  static const ncclDataType_t kType = ncclFloat64;
};
template <>
struct NcclType<int32_t> {
  static const ncclDataType_t kType = ncclInt32;
};

#ifdef __CUDACC__
/*! \brief counts elements that differ between two dense buffers (for CheckWeight) */
template <typename DType>
__global__ void CountMismatchKernel(const DType *a, const DType *b, size_t n, unsigned long long *count) {
  unsigned long long local = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    local += a[i] != b[i];
  }
  if (local != 0) atomicAdd(count, local);
}
#endif
}  // namespace psdetail

/*! \brief all-reduce implementation of ISharedModel<gpu, DType>; one instance per process and device */
template <typename DType>
class NcclModel : public ISharedModel<gpu, DType> {
 public:
  typedef typename ISharedModel<gpu, DType>::CallbackFunction CallbackFunction;
  NcclModel() : rank_(0), world_(1), device_(-1), comm_(NULL), ready_(false) { comm_stream_.stream_ = NULL; }
  virtual ~NcclModel() { this->Destroy(); }

  /*! \brief identifier for a new group of ranks, as 256 hexadecimal digits; call on one rank */
  static std::string NewUniqueIdHex() {
    ncclUniqueId id;
    MSHADOW_NCCL_CALL(ncclGetUniqueId(&id));
    static const char *digits = "0123456789abcdef";
    std::string hex(2 * NCCL_UNIQUE_ID_BYTES, '0');
    for (int i = 0; i < NCCL_UNIQUE_ID_BYTES; ++i) {
      const unsigned char b = static_cast<unsigned char>(id.internal[i]);
      hex[2 * i] = digits[b >> 4];
      hex[2 * i + 1] = digits[b & 15];
    }
    return hex;
  }

  virtual void SetParam(const char *name, const char *val) {
    if (!strcmp(name, "rank")) rank_ = atoi(val);
    if (!strcmp(name, "world_size")) world_ = atoi(val);
    if (!strcmp(name, "nccl_id")) id_hex_ = val;
  }

  virtual void Init(const std::vector<int> &devices) {
    CHECK_EQ(devices.size(), 1U) << "NcclModel drives one device per process; start one process per GPU";
    CHECK(!ready_) << "NcclModel: Init called twice";
    CHECK(world_ >= 1 && rank_ >= 0 && rank_ < world_) << "NcclModel: rank " << rank_ << " of " << world_;
    device_ = devices[0];
    MSHADOW_CUDA_CALL(cudaSetDevice(device_));
    ncclUniqueId id;
    if (world_ == 1 && id_hex_.empty()) {
      MSHADOW_NCCL_CALL(ncclGetUniqueId(&id));
    } else {
      CHECK_EQ(id_hex_.size(), static_cast<size_t>(2 * NCCL_UNIQUE_ID_BYTES)) << "NcclModel: nccl_id missing or malformed";
      for (int i = 0; i < NCCL_UNIQUE_ID_BYTES; ++i) {
        id.internal[i] = static_cast<char>(HexValue(id_hex_[2 * i]) * 16 + HexValue(id_hex_[2 * i + 1]));
      }
    }
    MSHADOW_NCCL_CALL(ncclCommInitRank(&comm_, world_, id, rank_));
    MSHADOW_CUDA_CALL(cudaStreamCreateWithFlags(&comm_stream_.stream_, cudaStreamNonBlocking));
    ready_ = true;
  }

  virtual void PullWait(int key, int devid) {
    Entry &e = this->Find(key, devid);
    if (e.pull_pending) {
      MSHADOW_CUDA_CALL(cudaEventSynchronize(e.pull_done));
      e.pull_pending = false;
    }
  }

  virtual void PullFence(int key, int devid, Stream<gpu> *stream) {
    Entry &e = this->Find(key, devid);
    if (e.pull_pending) MSHADOW_CUDA_CALL(cudaStreamWaitEvent(Stream<gpu>::GetStream(stream), e.pull_done, 0));
  }

  /*! \brief every rank's `data` becomes rank 0's */
  virtual void SetWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
    Entry &e = this->Find(key, devid);
    CHECK_EQ(data.shape_, e.shape) << "SetWeight: shape differs from InitKey";
    this->OrderAfter(data.stream_, &e);
    this->Gather(e.buffer, data);
    MSHADOW_NCCL_CALL(ncclBroadcast(e.buffer, e.buffer, e.shape.Size(), psdetail::NcclType<DType>::kType, 0, comm_,
                                    comm_stream_.stream_));
    this->Scatter(data, e.buffer);
    MSHADOW_CUDA_CALL(cudaStreamSynchronize(comm_stream_.stream_));
  }

  /*! \brief CHECKs that `data` equals rank 0's copy bit for bit */
  virtual void CheckWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
#ifdef __CUDACC__
    Entry &e = this->Find(key, devid);
    CHECK_EQ(data.shape_, e.shape) << "CheckWeight: shape differs from InitKey";
    const size_t n = e.shape.Size();
    DType *mine = NULL, *root = NULL;
    unsigned long long *count = NULL;
    MSHADOW_CUDA_CALL(cudaMalloc(&mine, 2 * n * sizeof(DType) + sizeof(unsigned long long)));
    root = mine + n;
    count = reinterpret_cast<unsigned long long *>(root + n);
    this->OrderAfter(data.stream_, &e);
    MSHADOW_CUDA_CALL(cudaMemsetAsync(count, 0, sizeof(unsigned long long), comm_stream_.stream_));
    this->Gather(mine, data);
    MSHADOW_NCCL_CALL(ncclBroadcast(mine, root, n, psdetail::NcclType<DType>::kType, 0, comm_, comm_stream_.stream_));
    const int grid = n < 256 * 1024 ? static_cast<int>((n + 255) / 256) : 1024;
    psdetail::CountMismatchKernel<DType><<<grid, 256, 0, comm_stream_.stream_>>>(mine, root, n, count);
    unsigned long long bad = 0;
    MSHADOW_CUDA_CALL(cudaMemcpyAsync(&bad, count, sizeof(bad), cudaMemcpyDeviceToHost, comm_stream_.stream_));
    MSHADOW_CUDA_CALL(cudaStreamSynchronize(comm_stream_.stream_));
    MSHADOW_CUDA_CALL(cudaFree(mine));
    CHECK_EQ(bad, 0ULL) << "CheckWeight: key " << key << " differs from rank 0 in " << bad << " elements";
#else
    LOG(FATAL) << "CheckWeight needs a CUDA translation unit";
#endif
  }

 protected:
  virtual void InitKey_(Shape<2> shape, int key, int devid) {
    CHECK(ready_) << "NcclModel: Init has not been called";
    CHECK_EQ(devid, device_) << "NcclModel: this process drives device " << device_;
    CHECK(entries_.find(key) == entries_.end()) << "NcclModel: key " << key << " initialised twice";
    Entry e;
    e.shape = shape;
    e.pull_pending = false;
    MSHADOW_CUDA_CALL(cudaSetDevice(device_));
    MSHADOW_CUDA_CALL(cudaMalloc(&e.buffer, (shape.Size() > 0 ? shape.Size() : 1) * sizeof(DType)));
    MSHADOW_CUDA_CALL(cudaEventCreateWithFlags(&e.pushed, cudaEventDisableTiming));
    MSHADOW_CUDA_CALL(cudaEventCreateWithFlags(&e.pull_done, cudaEventDisableTiming));
    entries_[key] = e;
  }

  virtual void Push_(Tensor<gpu, 2, DType> data, int key, int devid, int) {
    Entry &e = this->Find(key, devid);
    CHECK_EQ(data.shape_, e.shape) << "Push: shape differs from InitKey";
    this->OrderAfter(data.stream_, &e);
    const DType *send = data.dptr_;
    if (!data.CheckContiguous()) {  // pitched rows: pack them into the key's buffer first
      this->Gather(e.buffer, data);
      send = e.buffer;
    }
    MSHADOW_NCCL_CALL(ncclAllReduce(send, e.buffer, e.shape.Size(), psdetail::NcclType<DType>::kType, ncclSum, comm_,
                                    comm_stream_.stream_));
  }

  virtual void PullReq_(Tensor<gpu, 2, DType> data, int key, int devid, int, CallbackFunction callback,
                        void *callback_arg) {
    Entry &e = this->Find(key, devid);
    CHECK_EQ(data.shape_, e.shape) << "PullReq: shape differs from InitKey";
    // the requester may still be using `data` on its own stream (it usually is: it just pushed it)
    this->OrderAfter(data.stream_, &e);
    this->Scatter(data, e.buffer);
    if (callback != NULL) callback(&comm_stream_, callback_arg);
    MSHADOW_CUDA_CALL(cudaEventRecord(e.pull_done, comm_stream_.stream_));
    e.pull_pending = true;
  }

 private:
  struct Entry {
    Shape<2> shape;
    DType *buffer;       // dense rows x cols: the last sum of this key
    cudaEvent_t pushed;  // marks the requester's stream at Push / PullReq
    cudaEvent_t pull_done;
    bool pull_pending;
  };

  static int HexValue(char c) { return c >= 'a' ? c - 'a' + 10 : (c >= 'A' ? c - 'A' + 10 : c - '0'); }

  Entry &Find(int key, int devid) {
    CHECK(ready_) << "NcclModel: Init has not been called";
    CHECK_EQ(devid, device_) << "NcclModel: this process drives device " << device_;
    typename std::map<int, Entry>::iterator it = entries_.find(key);
    CHECK(it != entries_.end()) << "NcclModel: key " << key << " has not been initialised";
    return it->second;
  }
  /*! \brief the communication stream continues only after what `user` has enqueued so far */
  void OrderAfter(Stream<gpu> *user, Entry *e) {
    const cudaStream_t s = Stream<gpu>::GetStream(user);
    MSHADOW_CUDA_CALL(cudaEventRecord(e->pushed, s));
    MSHADOW_CUDA_CALL(cudaStreamWaitEvent(comm_stream_.stream_, e->pushed, 0));
  }
  void Gather(DType *dense, const Tensor<gpu, 2, DType> &src) {
    if (src.shape_.Size() == 0) return;
    MSHADOW_CUDA_CALL(cudaMemcpy2DAsync(dense, src.size(1) * sizeof(DType), src.dptr_, src.stride_ * sizeof(DType),
                                        src.size(1) * sizeof(DType), src.size(0), cudaMemcpyDeviceToDevice,
                                        comm_stream_.stream_));
  }
  void Scatter(Tensor<gpu, 2, DType> dst, const DType *dense) {
    if (dst.shape_.Size() == 0) return;
    MSHADOW_CUDA_CALL(cudaMemcpy2DAsync(dst.dptr_, dst.stride_ * sizeof(DType), dense, dst.size(1) * sizeof(DType),
                                        dst.size(1) * sizeof(DType), dst.size(0), cudaMemcpyDeviceToDevice,
                                        comm_stream_.stream_));
  }
  void Destroy() {
    if (!ready_) return;
    cudaSetDevice(device_);
    cudaStreamSynchronize(comm_stream_.stream_);
    for (typename std::map<int, Entry>::iterator it = entries_.begin(); it != entries_.end(); ++it) {
      cudaFree(it->second.buffer);
      cudaEventDestroy(it->second.pushed);
      cudaEventDestroy(it->second.pull_done);
    }
    entries_.clear();
    ncclCommDestroy(comm_);
    cudaStreamDestroy(comm_stream_.stream_);
    ready_ = false;
  }

  int rank_, world_, device_;
  std::string id_hex_;
  ncclComm_t comm_;
  Stream<gpu> comm_stream_;
  std::map<int, Entry> entries_;
  bool ready_;
};

/*!
 * \brief factory with the reference's name (mshadow-ps/mshadow_ps.h:339-356).  "local" -- the
 *  type the reference's examples ask for -- and "nccl" both give the all-reduce model; "peer"
 *  gives the peer-store model for small tensors (peer_model.h).
 */
template <typename xpu, typename DType>
inline ISharedModel<xpu, DType> *CreateSharedModel(const char *type);
template <>
inline ISharedModel<gpu, float> *CreateSharedModel<gpu, float>(const char *type) {
  if (!strcmp("local", type) || !strcmp("nccl", type)) return new NcclModel<float>();
  if (!strcmp("peer", type)) return new PeerModel<float>();
  LOG(FATAL) << "unknown server type " << type;
  return NULL;
}

}  // namespace ps
}  // namespace mshadow
#endif  // MSHADOW_PS_H_
