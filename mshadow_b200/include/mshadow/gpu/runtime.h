/*
 * Host-side GPU runtime of the engine: Stream<gpu>, engine life cycle, device memory,
 * copies, launch-geometry helpers and the library-owned scratch buffers.
 *
 * The API follows dmlc/mshadow's mshadow/stream_gpu-inl.h (:18-211) and
 * mshadow/tensor_gpu-inl.h (:14-92).  Differences: there is no BLAS / cuDNN / cuSOLVER
 * handle (matrix products are outside this engine; the creation flags are accepted and
 * ignored), and kernels that need scratch memory obtain it from a per-(device, stream)
 * cache kept here, so that the "operators allocate no temporaries" contract of the
 * reference (README.md:19-20) still holds from the caller's point of view.
 */
#ifndef MSHADOW_GPU_RUNTIME_H_
#define MSHADOW_GPU_RUNTIME_H_

#include <cuda_runtime.h>

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#include "../tensor.h"
#include "../engine/fastdiv.h"
#include "./tuning.h"

namespace mshadow {
namespace gpu_rt {
/*! \brief number of kernels this engine has launched in the process (all threads, all devices) */
inline std::atomic<long long> &LaunchCounter() {
  static std::atomic<long long> count(0);
  return count;
}
}  // namespace gpu_rt
}  // namespace mshadow

/*! \brief check that the launch just issued was accepted by the driver, and count it */
#define MSHADOW_CUDA_POST_KERNEL_CHECK(name)                                              \
  {                                                                                       \
    cudaError_t msh_err_ = cudaPeekAtLastError();                                         \
    CHECK_EQ(msh_err_, cudaSuccess) << "Name: " << #name << " ErrStr:" << cudaGetErrorString(msh_err_); \
    ::mshadow::gpu_rt::LaunchCounter().fetch_add(1, std::memory_order_relaxed);           \
  }

namespace mshadow {
namespace gpu_rt {
#ifdef __CUDACC__
/*!
 * \brief launch of a kernel that begins with GridDependencySync(): when the operation before it
 *  in the stream is a kernel, its CTAs may be placed on the SMs while that kernel drains, run up
 *  to GridDependencySync() and wait there until it has completed and its memory is visible.  The
 *  launch gap between the two kernels (a few microseconds, a fifth of the time of a kernel that
 *  processes an eighth of a benchmark tensor) overlaps the tail of the first.  Only kernels that
 *  call GridDependencySync() before their first access to global memory may be launched this way.
 */
template <typename... KArgs, typename... Args>
inline void LaunchAfterDrain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = MSHADOW_B200_EARLY_LAUNCH ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

/*! \brief lets the next kernel of the stream be placed early, then waits for the previous one: first statements of a kernel launched with LaunchAfterDrain */
__device__ __forceinline__ void GridDependencySync() {
#if MSHADOW_B200_EARLY_LAUNCH
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
#endif  // __CUDACC__
}  // namespace gpu_rt
}  // namespace mshadow

namespace mshadow {

/*! \brief execution queue of a CUDA device */
template <>
struct Stream<gpu> {
  cudaStream_t stream_;
  int dev_id;
  Stream() : stream_(0), dev_id(0) {}
  inline void Wait() { MSHADOW_CUDA_CALL(cudaStreamSynchronize(stream_)); }
  inline bool CheckIdle() {
    const cudaError_t err = cudaStreamQuery(stream_);
    if (err == cudaSuccess) return true;
    if (err == cudaErrorNotReady) return false;
    LOG(FATAL) << cudaGetErrorString(err);
    return false;
  }
  inline void CreateBlasHandle() {}
  /*! \brief raw stream of a possibly-null Stream pointer; null is fatal under MSHADOW_FORCE_STREAM */
  inline static cudaStream_t GetStream(Stream<gpu> *stream) {
    if (stream == NULL) {
#if MSHADOW_FORCE_STREAM
      LOG(FATAL) << "Default GPU stream was used when MSHADOW_FORCE_STREAM was on";
#endif
      return 0;
    }
    return stream->stream_;
  }
};

namespace gpu_rt {

/*! \brief properties of the current device that launch heuristics need; queried once per device */
struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
  int l2_bytes;
};

inline const DeviceInfo &CurrentDevice() {
  static std::mutex mu;
  static std::map<int, DeviceInfo> cache;
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(dev);
  if (it == cache.end()) {
    DeviceInfo info;
    MSHADOW_CUDA_CALL(cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev));
    MSHADOW_CUDA_CALL(
        cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    MSHADOW_CUDA_CALL(cudaDeviceGetAttribute(&info.l2_bytes, cudaDevAttrL2CacheSize, dev));
    it = cache.insert(std::make_pair(dev, info)).first;
  }
  return it->second;
}

/*!
 * \brief scratch buffers, one per (device, stream, owner), grown on demand and never shrunk.
 *  Work that uses a buffer is ordered on its stream, so one buffer per stream is race-free;
 *  growing synchronises that stream before the old buffer is released.  The engine's own
 *  operators use owner kEngine; a buffer handed out to a caller (owner kCaller) is a different
 *  one, so that no later operator on the stream overwrites or reallocates it.
 */
class Scratch {
 public:
  enum Owner { kEngine = 0, kCaller = 1 };
  static void *Get(cudaStream_t stream, size_t bytes, Owner owner = kEngine) {
    int dev = 0;
    MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(Mutex());
    Slot &slot = Table()[Key(dev, stream, owner)];
    if (slot.bytes < bytes) {
      if (slot.ptr != nullptr) {
        MSHADOW_CUDA_CALL(cudaStreamSynchronize(stream));
        MSHADOW_CUDA_CALL(cudaFree(slot.ptr));
        slot.ptr = nullptr;
        slot.bytes = 0;
      }
      size_t want = bytes + bytes / 2;
      want = (want + 255) / 256 * 256;
      MSHADOW_CUDA_CALL(cudaMalloc(&slot.ptr, want));
      slot.bytes = want;
    }
    return slot.ptr;
  }
  /*! \brief bytes currently held for (current device, stream, owner); 0 if none */
  static size_t Held(cudaStream_t stream, Owner owner = kEngine) {
    int dev = 0;
    MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(Mutex());
    auto it = Table().find(Key(dev, stream, owner));
    return it == Table().end() ? 0 : it->second.bytes;
  }
  /*! \brief release the buffers of one stream on the current device (stream == all: every buffer) */
  static void Release(bool all, cudaStream_t stream) {
    int dev = 0;
    if (!all) MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(Mutex());
    auto &table = Table();
    for (auto it = table.begin(); it != table.end();) {
      if (all || (it->first.dev == dev && it->first.stream == stream)) {
        if (it->second.ptr != nullptr) {
          int cur = 0;
          cudaGetDevice(&cur);
          cudaSetDevice(it->first.dev);
          cudaFree(it->second.ptr);
          cudaSetDevice(cur);
        }
        it = table.erase(it);
      } else {
        ++it;
      }
    }
  }

 private:
  struct Slot {
    void *ptr = nullptr;
    size_t bytes = 0;
  };
  struct Key {
    int dev;
    cudaStream_t stream;
    int owner;
    Key(int d, cudaStream_t s, int o) : dev(d), stream(s), owner(o) {}
    bool operator<(const Key &b) const {
      if (dev != b.dev) return dev < b.dev;
      if (stream != b.stream) return stream < b.stream;
      return owner < b.owner;
    }
  };
  static std::mutex &Mutex() {
    static std::mutex mu;
    return mu;
  }
  static std::map<Key, Slot> &Table() {
    static std::map<Key, Slot> table;
    return table;
  }
};

#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
/*!
 * \brief checked build: the first access that a tensor leaf refused on the current device since
 *  the last call (this translation unit's kernels), after waiting for the device; clears the record.
 * \return true if there was one; then *offset is the element offset from the tensor's base,
 *  *width the number of elements of the access and *limit the extent of the tensor's storage
 */
inline bool TakeBoundsViolation(long long *offset, int *width, long long *limit) {
  expr::plandetail::BoundsRecord rec;
  MSHADOW_CUDA_CALL(cudaDeviceSynchronize());
  MSHADOW_CUDA_CALL(cudaMemcpyFromSymbol(&rec, expr::plandetail::g_bounds_record, sizeof(rec)));
  if (rec.hit == 0) return false;
  const expr::plandetail::BoundsRecord clean = {0, 0, 0, 0};
  MSHADOW_CUDA_CALL(cudaMemcpyToSymbol(expr::plandetail::g_bounds_record, &clean, sizeof(clean)));
  *offset = rec.offset;
  *width = rec.width;
  *limit = rec.limit;
  return true;
}
#endif

/*!
 * \brief one int per device in which a kernel records that a bounded wait gave up
 *  (see gpu/tma.cuh); allocated on first use, lives as long as the process
 */
inline int *StatusWord() {
  static std::mutex mu;
  static std::map<int, int *> words;
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  auto it = words.find(dev);
  if (it == words.end()) {
    int *p = nullptr;
    MSHADOW_CUDA_CALL(cudaMalloc(&p, sizeof(int)));
    MSHADOW_CUDA_CALL(cudaMemset(p, 0, sizeof(int)));
    it = words.insert(std::make_pair(dev, p)).first;
  }
  return it->second;
}

/*!
 * \brief one page-locked int per host thread, into which msb-style waits copy the device's status
 *  word on the stream they wait for; allocated on the thread's first use, lives as long as the process
 */
inline int *StatusMirror() {
  thread_local int *mirror = nullptr;
  if (mirror == nullptr) {
    MSHADOW_CUDA_CALL(cudaHostAlloc(reinterpret_cast<void **>(&mirror), sizeof(int), cudaHostAllocPortable));
  }
  return mirror;
}

#ifdef __CUDACC__
/*!
 * \brief CTAs of `kernel` (with `threads` threads and `smem` bytes of dynamic shared memory) that
 *  one SM of the current device keeps resident; at least 1.  Looked up once per (device, kernel)
 *  and kept under a lock, so that host threads driving different devices can share the library.
 */
template <typename Kernel>
inline int ResidentPerSM(Kernel kernel, int threads, size_t smem = 0) {
  static std::mutex mu;
  static std::map<std::pair<int, const void *>, int> cache;
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  const std::pair<int, const void *> key(dev, reinterpret_cast<const void *>(kernel));
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    int per_sm = 0;
    MSHADOW_CUDA_CALL(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem));
    it = cache.insert(std::make_pair(key, per_sm < 1 ? 1 : per_sm)).first;
  }
  return it->second;
}
#endif

/*! \brief exact division of an index by a divisor fixed per launch, without a divide instruction */
typedef expr::FastDiv FastDiv;

inline int CeilDiv(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

#ifdef __CUDACC__
/*!
 * \brief load that bypasses L1 (data written by other CTAs of the same launch), for any element
 *  type of 1, 2, 4, 8 or 16 bytes; the intrinsic itself only knows the built-in types
 */
template <typename T>
__device__ __forceinline__ T LoadCg(const T *p) {
  static_assert(sizeof(T) == 1 || sizeof(T) == 2 || sizeof(T) == 4 || sizeof(T) == 8 || sizeof(T) == 16,
                "LoadCg: unsupported element size");
  T r;
  if (sizeof(T) == 1) {
    const unsigned char v = __ldcg(reinterpret_cast<const unsigned char *>(p));
    memcpy(&r, &v, sizeof(T) == 1 ? 1 : 0);
  } else if (sizeof(T) == 2) {
    const unsigned short v = __ldcg(reinterpret_cast<const unsigned short *>(p));
    memcpy(&r, &v, sizeof(T) == 2 ? 2 : 0);
  } else if (sizeof(T) == 4) {
    const unsigned int v = __ldcg(reinterpret_cast<const unsigned int *>(p));
    memcpy(&r, &v, sizeof(T) == 4 ? 4 : 0);
  } else if (sizeof(T) == 8) {
    const unsigned long long v = __ldcg(reinterpret_cast<const unsigned long long *>(p));
    memcpy(&r, &v, sizeof(T) == 8 ? 8 : 0);
  } else {
    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(p));
    memcpy(&r, &v, sizeof(T) == 16 ? 16 : 0);
  }
  return r;
}
#endif

}  // namespace gpu_rt

template <>
inline void InitTensorEngine<gpu>(int dev_id) {
  int device_count = 0;
  cudaGetDeviceCount(&device_count);
  CHECK_GT(device_count, 0) << "Cannot find CUDA device. Please check CUDA-Configuration";
  const int device_id = dev_id < 0 ? 0 : dev_id;
  CHECK_LT(device_id, device_count) << "Incorrect Device ID";
  MSHADOW_CUDA_CALL(cudaSetDevice(device_id));
  gpu_rt::CurrentDevice();
}
template <>
inline void ShutdownTensorEngine<gpu>() {
  gpu_rt::Scratch::Release(true, 0);
}
template <>
inline void SetDevice<gpu>(int devid) {
  MSHADOW_CUDA_CALL(cudaSetDevice(devid));
}
template <>
inline Stream<gpu> *NewStream<gpu>(bool, bool, int dev_id) {
  Stream<gpu> *st = new Stream<gpu>();
  MSHADOW_CUDA_CALL(cudaStreamCreate(&st->stream_));
  if (dev_id < 0) {
    MSHADOW_CUDA_CALL(cudaGetDevice(&st->dev_id));
  } else {
    st->dev_id = dev_id;
  }
  return st;
}
template <>
inline void DeleteStream<gpu>(Stream<gpu> *stream) {
  if (stream == NULL) return;
  gpu_rt::Scratch::Release(false, stream->stream_);
  MSHADOW_CUDA_CALL(cudaStreamDestroy(stream->stream_));
  delete stream;
}

template <int dim, typename DType>
inline void AllocSpace(Tensor<gpu, dim, DType> *obj, bool pad) {
  size_t pitch = 0;
  const Shape<2> flat = obj->shape_.FlatTo2D();
  if (pad && obj->size(dim - 1) >= MSHADOW_MIN_PAD_RATIO * 32) {
    MSHADOW_CUDA_CALL(cudaMallocPitch(reinterpret_cast<void **>(&obj->dptr_), &pitch,
                                      flat[1] * sizeof(DType), flat[0]));
    obj->stride_ = static_cast<index_t>(pitch / sizeof(DType));
  } else {
    obj->stride_ = obj->size(dim - 1);
    MSHADOW_CUDA_CALL(cudaMalloc(reinterpret_cast<void **>(&obj->dptr_),
                                 static_cast<size_t>(flat[0]) * flat[1] * sizeof(DType)));
  }
}
template <int dim, typename DType>
inline void FreeSpace(Tensor<gpu, dim, DType> *obj) {
  MSHADOW_CUDA_CALL(cudaFree(obj->dptr_));
  obj->dptr_ = NULL;
}

namespace gpu_rt {
template <typename A, typename B, int dim, typename DType>
inline void CopyRows(Tensor<A, dim, DType> dst_nd, Tensor<B, dim, DType> src_nd, cudaMemcpyKind kind,
                     Stream<gpu> *stream) {
  CHECK_EQ(dst_nd.shape_, src_nd.shape_) << "Copy:shape mismatch";
  const Tensor<A, 2, DType> dst = dst_nd.FlatTo2D();
  const Tensor<B, 2, DType> src = src_nd.FlatTo2D();
  const cudaStream_t s = Stream<gpu>::GetStream(stream);
  if (dst.CheckContiguous() && src.CheckContiguous()) {
    MSHADOW_CUDA_CALL(cudaMemcpyAsync(dst.dptr_, src.dptr_,
                                      static_cast<size_t>(dst.size(0)) * dst.size(1) * sizeof(DType),
                                      kind, s));
  } else {
    MSHADOW_CUDA_CALL(cudaMemcpy2DAsync(dst.dptr_, dst.stride_ * sizeof(DType), src.dptr_,
                                        src.stride_ * sizeof(DType), dst.size(1) * sizeof(DType),
                                        dst.size(0), kind, s));
  }
  // a copy issued without a stream behaves synchronously, as in the reference
  if (stream == NULL) MSHADOW_CUDA_CALL(cudaStreamSynchronize(0));
}
}  // namespace gpu_rt

template <int dim, typename DType>
inline void Copy(Tensor<cpu, dim, DType> dst, const Tensor<gpu, dim, DType> &src, Stream<gpu> *stream) {
  gpu_rt::CopyRows(dst, src, cudaMemcpyDeviceToHost, stream);
}
template <int dim, typename DType>
inline void Copy(Tensor<gpu, dim, DType> dst, const Tensor<cpu, dim, DType> &src, Stream<gpu> *stream) {
  gpu_rt::CopyRows(dst, src, cudaMemcpyHostToDevice, stream);
}
template <int dim, typename DType>
inline void Copy(Tensor<gpu, dim, DType> dst, const Tensor<gpu, dim, DType> &src, Stream<gpu> *stream) {
  gpu_rt::CopyRows(dst, src, cudaMemcpyDeviceToDevice, stream);
}

}  // namespace mshadow
#endif  // MSHADOW_GPU_RUNTIME_H_
