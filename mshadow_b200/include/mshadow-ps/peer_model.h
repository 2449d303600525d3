/*
 * PeerModel: the ISharedModel interface (Push / PullReq / PullWait, see mshadow_ps.h) for small,
 * latency-bound tensors, built on plain stores into the other GPUs' memory over NVLink.
 *
 * The reference's LocalModel (mshadow-ps/ps_local-inl.h:443-461, 625-662, 700-736) copies each
 * pushed tensor to the host, sums on a CPU thread and copies the sum back.  An all-reduce
 * library removes the host but still costs a communication kernel that sits on the SMs beside
 * the compute kernels while it waits for its peers.  For a few thousand floats neither is
 * needed.  Every rank owns a window of device memory that its peers map (CUDA IPC).  For a key
 * of n elements the window holds `depth` slots of world x n elements and world flags per slot:
 *
 *   Push(data, key)     step s of the key: one kernel stores `data` into row `rank` of slot
 *                       s % depth of EVERY rank's window (its own included), fences, and sets
 *                       flag[s % depth][rank] = s + 1 there.  It never waits for anybody.
 *   PullReq(data, key)  one kernel waits until all world flags of slot s % depth hold s + 1
 *                       (bounded: see below), then adds the world rows in rank order,
 *                       ((r0 + r1) + r2) + ..., and writes the sum to `data`.
 *
 * Both kernels run on the tensor's own stream, so there is no communication stream, no event
 * hand-over and nothing resident on the SMs between the two.  Every rank adds the same rows in
 * the same order: all ranks receive bit-identical sums, run after run.
 *
 * Slot reuse.  A rank may enqueue Push of step s + a before PullReq of step s (to overlap the
 * exchange with its next kernels).  A peer's store for step j lands in the slot that step
 * j - depth used, so that step must have been pulled here already; following the stream orders
 * of both ranks this holds when  depth >= 2 + 2 a.  The default depth 4 allows a = 1 (push the
 * next step, then pull the previous one); a = 0 needs depth 2.
 *
 * Waiting is bounded.  The pull kernel polls for at most `wait_limit_ms` (default 2000) of the
 * device timer.  When that runs out it writes nothing to `data`, records a status that
 * PullWait turns into an error, and returns; the context stays usable.
 *
 * Set-up: SetParam("rank" / "world_size" / "window_bytes" / "depth" / "wait_limit_ms"),
 * Init({device}) allocates and clears the window; ExportHandleHex() gives 128 hexadecimal
 * digits that the application hands to every other rank (as it does with NCCL's identifier);
 * SetParam("peer_handles", all world handles concatenated in rank order) and Connect() map
 * the peers' windows.  All ranks must call InitKey with the same keys and shapes in the same
 * order (the window is carved up in that order) and use a key from one stream at a time.
 * Before destroying a model the application makes sure (a barrier of its own) that no peer
 * still pushes into it.
 *
 * Only ordinary loads and stores touch peer memory: no multicast of any kind, no bulk-copy
 * engine, no library kernel is ever handed a peer pointer.
 */
#ifndef MSHADOW_PS_PEER_MODEL_H_
#define MSHADOW_PS_PEER_MODEL_H_

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "./shared_model.h"

namespace mshadow {
namespace ps {
namespace peerdetail {

const int kMaxWorld = 16;
const int kHandleBytes = 64;  // sizeof(cudaIpcMemHandle_t)
const int kStatusPeerTimeout = 2;
const unsigned kPushThreads = 512;
const unsigned kPushElemsPerCta = 8192;  // per peer: 32 KB of floats, four 16-byte stores a thread
const unsigned kPullThreads = 256;
const unsigned kPullElemsPerCta = 2048;

/*! \brief what the push kernel needs; passed by value */
template <typename DType>
struct PushArgs {
  const DType *src;
  uint32_t rows, cols, ld;   // the caller's matrix (ld elements between rows)
  DType *dst[kMaxWorld];     // row `rank` of the step's slot in every rank's window
  uint32_t *flag[kMaxWorld]; // flag[slot][rank] in every rank's window
  uint32_t *tickets;         // the key's world counters in this rank's own memory (zero between launches)
  uint32_t seq1;             // step + 1
  int world;
};

/*! \brief what the pull kernel needs */
template <typename DType>
struct PullArgs {
  DType *dst;
  uint32_t rows, cols, ld;
  const DType *slot;         // this rank's slot of the step: world rows, row_stride elements apart
  uint32_t row_stride;
  const uint32_t *flags;     // its world flags
  uint32_t seq1;
  int world;
  int root_only;             // 1: copy row 0 instead of summing (SetWeight)
  unsigned long long limit_ns;
  int *status;               // set to kStatusPeerTimeout when the wait gives up
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long GlobalNanos() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t LoadAcquireSys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void StoreReleaseSys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

/*!
 * \brief grid (chunks, world): CTA (x, p) stores its chunk of the caller's tensor into rank p's
 *  window; the last CTA of a peer to finish publishes the step's flag there.
 */
template <typename DType, bool kVec>
__global__ void __launch_bounds__(kPushThreads) PeerPushKernel(const PushArgs<DType> a) {
  const int p = blockIdx.y;
  const uint32_t n = a.rows * a.cols;
  const uint32_t begin = blockIdx.x * kPushElemsPerCta;
  uint32_t end = begin + kPushElemsPerCta;
  if (end > n) end = n;
  DType *out = a.dst[p];
  if (kVec) {
    // dense source, 16-byte aligned on both sides, n a multiple of the group
    constexpr uint32_t kGroup = 16 / sizeof(DType);
    const uint4 *src4 = reinterpret_cast<const uint4 *>(a.src);
    uint4 *dst4 = reinterpret_cast<uint4 *>(out);
    for (uint32_t g = begin / kGroup + threadIdx.x; g < end / kGroup; g += kPushThreads) dst4[g] = src4[g];
  } else {
    for (uint32_t i = begin + threadIdx.x; i < end; i += kPushThreads) {
      const uint32_t r = i / a.cols;
      out[i] = a.src[static_cast<size_t>(r) * a.ld + (i - r * a.cols)];
    }
  }
  // every thread's stores are ordered before the flag: fence, meet, then one thread publishes
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (gridDim.x > 1) {
    const uint32_t arrived = atomicAdd(&a.tickets[p], 1u);
    if (arrived + 1 != gridDim.x) return;
    a.tickets[p] = 0;  // the next launch on this stream starts from zero again
    __threadfence_system();
  }
  StoreReleaseSys(a.flag[p], a.seq1);
}

/*!
 * \brief waits (bounded) for the world flags of the step, then folds the world rows in rank
 *  order.  Each CTA polls for itself, so CTAs never wait for one another.
 */
template <typename DType>
__global__ void __launch_bounds__(kPullThreads) PeerPullKernel(const PullArgs<DType> a) {
  __shared__ int ok_all;
  if (threadIdx.x == 0) ok_all = 1;
  __syncthreads();
  if (threadIdx.x < static_cast<unsigned>(a.world)) {
    bool ok = false;
    unsigned long long start = 0;
    // bounded twice: by the device timer, and by a poll count that no wait of limit_ns can reach
    // (a poll is a round trip to the L2, several hundred nanoseconds)
    const unsigned long long max_spins = a.limit_ns / 64 + 4096;
    for (unsigned long long spin = 1; !ok && spin <= max_spins; ++spin) {
      const uint32_t v = LoadAcquireSys(a.flags + threadIdx.x);
      ok = static_cast<int32_t>(v - a.seq1) >= 0;
      if (!ok && (spin & 63u) == 0) {  // the timer is first read after 64 vain polls
        const unsigned long long now = GlobalNanos();
        if (start == 0) start = now;
        else if (now - start > a.limit_ns) break;
      }
    }
    if (!ok) ok_all = 0;
  }
  __syncthreads();
  if (ok_all == 0) {
    if (threadIdx.x == 0) {  // mapped host memory: a plain store and a system-wide fence
      *static_cast<volatile int *>(a.status) = kStatusPeerTimeout;
      __threadfence_system();
    }
    return;
  }
  const uint32_t n = a.rows * a.cols;
  const uint32_t begin = blockIdx.x * kPullElemsPerCta;
  uint32_t end = begin + kPullElemsPerCta;
  if (end > n) end = n;
  for (uint32_t i = begin + threadIdx.x; i < end; i += kPullThreads) {
    // the rows were written by other GPUs: read them past the L1, which nothing keeps coherent
    DType sum = gpu_rt::LoadCg(a.slot + i);
    if (!a.root_only) {
      DType v[kMaxWorld];
#pragma unroll
      for (int q = 1; q < kMaxWorld; ++q) {
        if (q < a.world) v[q] = gpu_rt::LoadCg(a.slot + static_cast<size_t>(q) * a.row_stride + i);
      }
#pragma unroll
      for (int q = 1; q < kMaxWorld; ++q) {
        if (q < a.world) sum = sum + v[q];
      }
    }
    const uint32_t r = i / a.cols;
    a.dst[static_cast<size_t>(r) * a.ld + (i - r * a.cols)] = sum;
  }
}

/*! \brief counts elements that differ between two dense buffers (CheckWeight) */
template <typename DType>
__global__ void PeerCountMismatchKernel(const DType *a, const DType *b, size_t n, unsigned long long *count) {
  unsigned long long local = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    local += a[i] != b[i];
  }
  if (local != 0) atomicAdd(count, local);
}
#endif  // __CUDACC__

inline size_t RoundUp(size_t v, size_t to) { return (v + to - 1) / to * to; }

}  // namespace peerdetail

/*! \brief peer-store implementation of ISharedModel<gpu, DType>; one instance per process and device */
template <typename DType>
class PeerModel : public ISharedModel<gpu, DType> {
 public:
  typedef typename ISharedModel<gpu, DType>::CallbackFunction CallbackFunction;
  PeerModel()
      : rank_(0), world_(1), device_(-1), depth_(4), wait_limit_ms_(2000), window_bytes_(size_t(16) << 20),
        window_(NULL), used_(0), status_host_(NULL), status_dev_(NULL), ready_(false),
        connected_(false) {
    for (int p = 0; p < peerdetail::kMaxWorld; ++p) peer_[p] = NULL, opened_[p] = false;
  }
  virtual ~PeerModel() { this->Destroy(); }

  virtual void SetParam(const char *name, const char *val) {
    if (!strcmp(name, "rank")) rank_ = atoi(val);
    if (!strcmp(name, "world_size")) world_ = atoi(val);
    if (!strcmp(name, "depth")) depth_ = atoi(val);
    if (!strcmp(name, "wait_limit_ms")) wait_limit_ms_ = atoi(val);
    if (!strcmp(name, "window_bytes")) window_bytes_ = static_cast<size_t>(atoll(val));
    if (!strcmp(name, "peer_handles")) peer_handles_hex_ = val;
  }

  virtual void Init(const std::vector<int> &devices) {
    CHECK_EQ(devices.size(), 1U) << "PeerModel drives one device per process; start one process per GPU";
    CHECK(!ready_) << "PeerModel: Init called twice";
    CHECK(world_ >= 1 && world_ <= peerdetail::kMaxWorld && rank_ >= 0 && rank_ < world_)
        << "PeerModel: rank " << rank_ << " of " << world_ << " (at most " << peerdetail::kMaxWorld << " ranks)";
    CHECK(depth_ >= 2 && depth_ <= 64) << "PeerModel: depth must be within 2..64";
    CHECK(wait_limit_ms_ >= 1 && wait_limit_ms_ <= 600000) << "PeerModel: wait_limit_ms must be within 1..600000";
    CHECK(window_bytes_ >= 4096) << "PeerModel: window_bytes too small";
    device_ = devices[0];
    MSHADOW_CUDA_CALL(cudaSetDevice(device_));
    window_bytes_ = peerdetail::RoundUp(window_bytes_, 256);
    MSHADOW_CUDA_CALL(cudaMalloc(&window_, window_bytes_));
    MSHADOW_CUDA_CALL(cudaMemset(window_, 0, window_bytes_));
    // the status word lives in mapped host memory: a timed-out kernel writes it, the host reads it
    // without a copy (and therefore without touching any stream)
    MSHADOW_CUDA_CALL(cudaHostAlloc(reinterpret_cast<void **>(&status_host_), sizeof(int), cudaHostAllocMapped));
    *status_host_ = 0;
    MSHADOW_CUDA_CALL(cudaHostGetDevicePointer(reinterpret_cast<void **>(&status_dev_), status_host_, 0));
    MSHADOW_CUDA_CALL(cudaDeviceSynchronize());  // the window is clear before anybody can learn its handle
    peer_[rank_] = static_cast<char *>(window_);
    ready_ = true;
    connected_ = world_ == 1;
  }

  /*! \brief this rank's window as 128 hexadecimal digits, to be handed to every other rank */
  std::string ExportHandleHex() {
    CHECK(ready_) << "PeerModel: Init has not been called";
    cudaIpcMemHandle_t h;
    MSHADOW_CUDA_CALL(cudaIpcGetMemHandle(&h, window_));
    static const char *digits = "0123456789abcdef";
    const unsigned char *b = reinterpret_cast<const unsigned char *>(&h);
    std::string hex(2 * peerdetail::kHandleBytes, '0');
    for (int i = 0; i < peerdetail::kHandleBytes; ++i) {
      hex[2 * i] = digits[b[i] >> 4];
      hex[2 * i + 1] = digits[b[i] & 15];
    }
    return hex;
  }

  /*!
   * \brief map the windows named by SetParam("peer_handles", ...).  A handle equal to this
   *  rank's own stands for this rank's window (a process cannot open its own handle); tests use
   *  that to build a group whose other members never answer.
   */
  void Connect() {
    CHECK(ready_) << "PeerModel: Init has not been called";
    CHECK(!connected_ || world_ == 1) << "PeerModel: Connect called twice";
    if (world_ == 1) return;
    const size_t per = 2 * peerdetail::kHandleBytes;
    CHECK_EQ(peer_handles_hex_.size(), per * world_) << "PeerModel: peer_handles must hold " << world_ << " handles";
    const std::string mine = this->ExportHandleHex();
    MSHADOW_CUDA_CALL(cudaSetDevice(device_));
    for (int p = 0; p < world_; ++p) {
      const std::string hex = peer_handles_hex_.substr(p * per, per);
      if (p == rank_) {
        CHECK(hex == mine) << "PeerModel: entry " << p << " of peer_handles is not this rank's handle";
        continue;
      }
      if (hex == mine) {
        peer_[p] = static_cast<char *>(window_);
        continue;
      }
      cudaIpcMemHandle_t h;
      unsigned char *b = reinterpret_cast<unsigned char *>(&h);
      for (int i = 0; i < peerdetail::kHandleBytes; ++i) b[i] = HexValue(hex[2 * i]) * 16 + HexValue(hex[2 * i + 1]);
      void *ptr = NULL;
      MSHADOW_CUDA_CALL(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
      peer_[p] = static_cast<char *>(ptr);
      opened_[p] = true;
    }
    connected_ = true;
  }

  virtual void PullWait(int key, int devid) {
    Entry &e = this->Find(key, devid);
    if (e.pull_pending) {
      MSHADOW_CUDA_CALL(cudaEventSynchronize(e.pull_done));
      e.pull_pending = false;
    }
    this->CheckStatus();
  }

  /*! \brief every rank's `data` becomes rank 0's (synchronous) */
  virtual void SetWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
    Entry &e = this->Find(key, devid);
    this->PushStep(data, &e);
    this->PullStep(data, &e, 1);
    MSHADOW_CUDA_CALL(cudaStreamSynchronize(Stream<gpu>::GetStream(data.stream_)));
    this->CheckStatus();
  }

  /*! \brief CHECKs that `data` equals rank 0's copy bit for bit (synchronous) */
  virtual void CheckWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
#ifdef __CUDACC__
    Entry &e = this->Find(key, devid);
    const size_t n = e.shape.Size();
    const cudaStream_t s = Stream<gpu>::GetStream(data.stream_);
    DType *mine = NULL;
    MSHADOW_CUDA_CALL(cudaMalloc(&mine, 2 * (n > 0 ? n : 1) * sizeof(DType) + sizeof(unsigned long long)));
    DType *root = mine + n;
    unsigned long long *count = reinterpret_cast<unsigned long long *>(root + n);
    MSHADOW_CUDA_CALL(cudaMemsetAsync(count, 0, sizeof(unsigned long long), s));
    Tensor<gpu, 2, DType> dense_mine(mine, e.shape, e.shape[1], data.stream_);
    Tensor<gpu, 2, DType> dense_root(root, e.shape, e.shape[1], data.stream_);
    if (n > 0) {
      MSHADOW_CUDA_CALL(cudaMemcpy2DAsync(mine, e.shape[1] * sizeof(DType), data.dptr_, data.stride_ * sizeof(DType),
                                          e.shape[1] * sizeof(DType), e.shape[0], cudaMemcpyDeviceToDevice, s));
    }
    this->PushStep(dense_mine, &e);
    this->PullStep(dense_root, &e, 1);
    const int grid = n < 256 * 1024 ? static_cast<int>((n + 255) / 256) : 1024;
    if (n > 0) peerdetail::PeerCountMismatchKernel<DType><<<grid, 256, 0, s>>>(mine, root, n, count);
    unsigned long long bad = 0;
    MSHADOW_CUDA_CALL(cudaMemcpyAsync(&bad, count, sizeof(bad), cudaMemcpyDeviceToHost, s));
    MSHADOW_CUDA_CALL(cudaStreamSynchronize(s));
    MSHADOW_CUDA_CALL(cudaFree(mine));
    this->CheckStatus();
    CHECK_EQ(bad, 0ULL) << "CheckWeight: key " << key << " differs from rank 0 in " << bad << " elements";
#else
    LOG(FATAL) << "CheckWeight needs a CUDA translation unit";
#endif
  }

  /*! \brief bytes of the window that InitKey has handed out so far */
  size_t WindowUsed() const { return used_; }

 protected:
  virtual void InitKey_(Shape<2> shape, int key, int devid) {
    CHECK(ready_) << "PeerModel: Init has not been called";
    CHECK_EQ(devid, device_) << "PeerModel: this process drives device " << device_;
    CHECK(entries_.find(key) == entries_.end()) << "PeerModel: key " << key << " initialised twice";
    CHECK_LT(static_cast<uint64_t>(shape[0]) * shape[1], uint64_t(1) << 31) << "PeerModel: tensor too large";
    Entry e;
    e.shape = shape;
    e.push_seq = e.pull_seq = 0;
    e.pull_pending = false;
    const size_t n = shape.Size();
    e.row_bytes = peerdetail::RoundUp((n > 0 ? n : 1) * sizeof(DType), 256);
    e.flag_offset = used_;
    // flags of all slots, then the push kernel's ticket counters (used by this rank only)
    e.ticket_offset = used_ + static_cast<size_t>(depth_) * peerdetail::kMaxWorld * sizeof(uint32_t);
    e.data_offset = peerdetail::RoundUp(e.ticket_offset + peerdetail::kMaxWorld * sizeof(uint32_t), 256);
    const size_t end = e.data_offset + static_cast<size_t>(depth_) * world_ * e.row_bytes;
    CHECK_LE(end, window_bytes_) << "PeerModel: key " << key << " does not fit the window of " << window_bytes_
                                 << " bytes (SetParam(\"window_bytes\", ...) before Init)";
    used_ = end;
    MSHADOW_CUDA_CALL(cudaEventCreateWithFlags(&e.pull_done, cudaEventDisableTiming));
    entries_[key] = e;
  }

  virtual void Push_(Tensor<gpu, 2, DType> data, int key, int devid, int) {
    Entry &e = this->Find(key, devid);
    this->PushStep(data, &e);
  }

  virtual void PullReq_(Tensor<gpu, 2, DType> data, int key, int devid, int, CallbackFunction callback,
                        void *callback_arg) {
    Entry &e = this->Find(key, devid);
    this->PullStep(data, &e, 0);
    if (callback != NULL) callback(data.stream_, callback_arg);
    MSHADOW_CUDA_CALL(cudaEventRecord(e.pull_done, Stream<gpu>::GetStream(data.stream_)));
    e.pull_pending = true;
  }

 private:
  struct Entry {
    Shape<2> shape;
    size_t flag_offset, ticket_offset, data_offset, row_bytes;  // within every rank's window
    uint32_t push_seq, pull_seq;
    cudaEvent_t pull_done;
    bool pull_pending;
  };

  static unsigned char HexValue(char c) {
    return static_cast<unsigned char>(c >= 'a' ? c - 'a' + 10 : (c >= 'A' ? c - 'A' + 10 : c - '0'));
  }

  Entry &Find(int key, int devid) {
    CHECK(ready_) << "PeerModel: Init has not been called";
    CHECK_EQ(devid, device_) << "PeerModel: this process drives device " << device_;
    typename std::map<int, Entry>::iterator it = entries_.find(key);
    CHECK(it != entries_.end()) << "PeerModel: key " << key << " has not been initialised";
    return it->second;
  }

  void CheckStatus() {
    if (status_host_ != NULL && *static_cast<volatile int *>(status_host_) != 0) {
      const int code = *static_cast<volatile int *>(status_host_);
      *static_cast<volatile int *>(status_host_) = 0;
      LOG(FATAL) << "PeerModel: timeout: a pull gave up waiting for its peers after " << wait_limit_ms_
                 << " ms (status " << code << "); its destination was left unchanged";
    }
  }

  void PushStep(const Tensor<gpu, 2, DType> &data, Entry *e) {
#ifdef __CUDACC__
    CHECK(connected_) << "PeerModel: Connect has not been called";
    CHECK_EQ(data.shape_, e->shape) << "Push: shape differs from InitKey";
    CHECK_LE(e->push_seq - e->pull_seq, static_cast<uint32_t>(depth_ / 2 - 1))
        << "Push: too many steps pushed ahead of their pulls for depth " << depth_;
    const size_t n = e->shape.Size();
    const uint32_t slot = e->push_seq % static_cast<uint32_t>(depth_);
    peerdetail::PushArgs<DType> a;
    a.src = data.dptr_;
    a.rows = e->shape[0];
    a.cols = e->shape[1];
    a.ld = data.stride_;
    a.tickets = reinterpret_cast<uint32_t *>(peer_[rank_] + e->ticket_offset);
    a.seq1 = e->push_seq + 1;
    a.world = world_;
    for (int p = 0; p < peerdetail::kMaxWorld; ++p) {
      const int q = p < world_ ? p : 0;
      a.dst[p] = reinterpret_cast<DType *>(peer_[q] + e->data_offset +
                                           (static_cast<size_t>(slot) * world_ + rank_) * e->row_bytes);
      a.flag[p] = reinterpret_cast<uint32_t *>(peer_[q] + e->flag_offset) + slot * peerdetail::kMaxWorld + rank_;
    }
    const unsigned chunks = n == 0 ? 1 : static_cast<unsigned>((n + peerdetail::kPushElemsPerCta - 1) /
                                                                peerdetail::kPushElemsPerCta);
    const bool vec = data.CheckContiguous() && (n * sizeof(DType)) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(data.dptr_) % 16 == 0 &&
                     peerdetail::kPushElemsPerCta % (16 / sizeof(DType)) == 0;
    const cudaStream_t s = Stream<gpu>::GetStream(data.stream_);
    const dim3 grid(chunks, world_);
    if (vec) {
      peerdetail::PeerPushKernel<DType, true><<<grid, peerdetail::kPushThreads, 0, s>>>(a);
    } else {
      peerdetail::PeerPushKernel<DType, false><<<grid, peerdetail::kPushThreads, 0, s>>>(a);
    }
    MSHADOW_CUDA_POST_KERNEL_CHECK(PeerPushKernel);
    e->push_seq += 1;
#else
    LOG(FATAL) << "PeerModel needs a CUDA translation unit";
#endif
  }

  void PullStep(Tensor<gpu, 2, DType> data, Entry *e, int root_only) {
#ifdef __CUDACC__
    CHECK_EQ(data.shape_, e->shape) << "PullReq: shape differs from InitKey";
    CHECK_LT(e->pull_seq, e->push_seq) << "PullReq: nothing pushed under this key that was not pulled already";
    const size_t n = e->shape.Size();
    const uint32_t slot = e->pull_seq % static_cast<uint32_t>(depth_);
    peerdetail::PullArgs<DType> a;
    a.dst = data.dptr_;
    a.rows = e->shape[0];
    a.cols = e->shape[1] > 0 ? e->shape[1] : 1;
    a.ld = data.stride_;
    a.slot = reinterpret_cast<const DType *>(peer_[rank_] + e->data_offset + static_cast<size_t>(slot) * world_ * e->row_bytes);
    a.flags = reinterpret_cast<const uint32_t *>(peer_[rank_] + e->flag_offset) + slot * peerdetail::kMaxWorld;
    a.row_stride = static_cast<uint32_t>(e->row_bytes / sizeof(DType));
    a.seq1 = e->pull_seq + 1;
    a.world = world_;
    a.root_only = root_only;
    a.limit_ns = static_cast<unsigned long long>(wait_limit_ms_) * 1000000ull;
    a.status = status_dev_;
    const unsigned ctas = n == 0 ? 1 : static_cast<unsigned>((n + peerdetail::kPullElemsPerCta - 1) /
                                                              peerdetail::kPullElemsPerCta);
    peerdetail::PeerPullKernel<DType>
        <<<ctas, peerdetail::kPullThreads, 0, Stream<gpu>::GetStream(data.stream_)>>>(a);
    MSHADOW_CUDA_POST_KERNEL_CHECK(PeerPullKernel);
    e->pull_seq += 1;
#else
    LOG(FATAL) << "PeerModel needs a CUDA translation unit";
#endif
  }

  void Destroy() {
    if (!ready_) return;
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (typename std::map<int, Entry>::iterator it = entries_.begin(); it != entries_.end(); ++it) {
      cudaEventDestroy(it->second.pull_done);
    }
    entries_.clear();
    for (int p = 0; p < world_; ++p) {
      if (opened_[p]) cudaIpcCloseMemHandle(peer_[p]);
      opened_[p] = false;
    }
    cudaFree(window_);
    cudaFreeHost(status_host_);
    window_ = NULL;
    ready_ = false;
  }

  int rank_, world_, device_, depth_, wait_limit_ms_;
  size_t window_bytes_;
  void *window_;
  size_t used_;
  int *status_host_, *status_dev_;
  char *peer_[peerdetail::kMaxWorld];
  bool opened_[peerdetail::kMaxWorld];
  std::string peer_handles_hex_;
  std::map<int, Entry> entries_;
  bool ready_, connected_;
};

}  // namespace ps
}  // namespace mshadow
#endif  // MSHADOW_PS_PEER_MODEL_H_
