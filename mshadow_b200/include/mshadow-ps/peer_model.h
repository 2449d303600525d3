/*
 * PeerModel: the ISharedModel interface (Push / PullReq / PullWait, see shared_model.h) for small,
 * latency-bound tensors of 4-byte elements, built on plain stores into the other GPUs' memory
 * over NVLink.
 *
 * The reference's LocalModel (mshadow-ps/ps_local-inl.h:443-461, 625-662, 700-736) copies each
 * pushed tensor to the host, sums on a CPU thread and copies the sum back.  An all-reduce
 * library removes the host but still costs a communication kernel that sits on the SMs beside
 * the compute kernels while it waits for its peers.  For a few thousand floats neither is
 * needed.  Every rank owns a window of device memory that its peers map (CUDA IPC).  For a key
 * of n elements the window holds `depth` slots of world rows of n 64-bit words.  A word carries
 * one element and the tag of the step it belongs to, and is written by one naturally aligned
 * 64-bit store, which is never torn: whoever reads the tag has the element.  So the protocol
 * needs no flags, no fences and nobody who knows when "everything" has arrived:
 *
 *   Push(data, key)     step s of the key: one kernel stores (data[i], s + 1) into row `rank` of
 *                       slot s % depth of EVERY rank's window (its own included).  It never waits.
 *   PullReq(data, key)  one kernel reads, per element, the world words of slot s % depth until
 *                       all carry tag s + 1 (bounded: see below), adds the world values in rank
 *                       order, ((r0 + r1) + r2) + ..., and writes the sum to `data`.
 *   NextSink(key, ...)  instead of Push: hands out the addresses and the tag of step s as a
 *                       gpu_rt::PeerSink, with which a reduction kernel delivers its results to
 *                       all ranks from the thread that computes them (mshadow/gpu/peer_sink.h).
 *                       Several reductions may fill disjoint segments of one step's row.
 *
 * By default the kernels run on the tensor's own stream: no communication stream, no event
 * hand-over, nothing resident on the SMs between a push and its pull.  With
 * SetParam("own_stream", "1") they run on a stream of the model instead, ordered behind the
 * tensor's stream by an event at every call, so that the exchange (a few microseconds of launch
 * gaps and NVLink round trips) proceeds beside the caller's next kernels; the caller then leaves
 * a pushed tensor alone until its step has been pulled and uses PullWait or PullFence before it
 * touches the result.  Every rank adds the same rows in the same order: all ranks receive
 * bit-identical sums, run after run.
 *
 * Slot reuse.  A rank may enqueue Push of step s + a before PullReq of step s (to overlap the
 * exchange with its next kernels).  A peer's store for step j lands in the slot that step
 * j - depth used, so that step must have been pulled here already; following the stream orders
 * of both ranks this holds when  depth >= 2 + 2 a.  The default depth 4 allows a = 1 (push the
 * next step, then pull the previous one); a = 0 needs depth 2.  Push refuses to run further ahead.
 *
 * Waiting is bounded.  The pull kernel polls for at most `wait_limit_ms` (default 2000) of the
 * device timer.  When that runs out it records a status that PullWait turns into an error and
 * returns; elements whose words had not all arrived are not written.  The context stays usable.
 *
 * Set-up: SetParam("rank" / "world_size" / "window_bytes" / "depth" / "wait_limit_ms" / "own_stream"),
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

#include "../mshadow/gpu/peer_sink.h"
#include "./shared_model.h"

namespace mshadow {
namespace ps {
namespace peerdetail {

const int kMaxWorld = gpu_rt::kPeerMaxWorld;
const int kHandleBytes = 64;  // sizeof(cudaIpcMemHandle_t)
const int kStatusPeerTimeout = 2;
const unsigned kPushThreads = 256;
const unsigned kPullThreads = 256;
typedef unsigned long long Word;

/*! \brief what the pull kernel needs */
template <typename DType>
struct PullArgs {
  DType *dst;
  uint32_t rows, cols, ld;   // the caller's matrix (ld elements between rows)
  const Word *slot;          // this rank's slot of the step: world rows, row_stride words apart
  uint32_t row_stride;
  uint32_t tag;              // step + 1
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
__device__ __forceinline__ Word LoadWord(const Word *p) {
  Word v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

/*! \brief one thread per element: the caller's element i, tagged, goes into every rank's window */
template <typename DType>
__global__ void __launch_bounds__(kPushThreads)
PeerPushKernel(const DType *src, uint32_t rows, uint32_t cols, uint32_t ld, const gpu_rt::PeerSink sink) {
  const uint32_t i = blockIdx.x * kPushThreads + threadIdx.x;
  if (i >= rows * cols) return;
  const uint32_t r = ld == cols ? 0 : i / cols;
  sink.Put(i, src[static_cast<size_t>(r) * ld + (i - r * cols)]);
}

/*!
 * \brief one thread per element: reads the element's world words until all carry the step's tag
 *  (bounded), adds the values in rank order, stores the sum.  Threads wait for their own words
 *  only, so neither threads nor CTAs wait for one another.
 */
template <typename DType>
__global__ void __launch_bounds__(kPullThreads) PeerPullKernel(const PullArgs<DType> a) {
  const uint32_t i = blockIdx.x * kPullThreads + threadIdx.x;
  if (i >= a.rows * a.cols) return;
  const int world = a.root_only ? 1 : a.world;
  Word w[kMaxWorld];
  uint32_t waiting = (1u << world) - 1u;
  unsigned long long start = 0;
  // bounded twice: by the device timer, and by a poll count that no wait of limit_ns can reach
  // (a poll is a round trip to the L2, several hundred nanoseconds)
  const unsigned long long max_spins = a.limit_ns / 64 + 4096;
  for (unsigned long long spin = 1; waiting != 0 && spin <= max_spins; ++spin) {
#pragma unroll
    for (int q = 0; q < kMaxWorld; ++q) {
      if ((waiting >> q) & 1u) w[q] = LoadWord(a.slot + static_cast<size_t>(q) * a.row_stride + i);
    }
#pragma unroll
    for (int q = 0; q < kMaxWorld; ++q) {
      if (((waiting >> q) & 1u) && static_cast<uint32_t>(w[q] >> 32) == a.tag) waiting &= ~(1u << q);
    }
    if (waiting != 0 && (spin & 63u) == 0) {  // the timer is first read after 64 vain polls
      const unsigned long long now = GlobalNanos();
      if (start == 0) start = now;
      else if (now - start > a.limit_ns) break;
    }
  }
  if (waiting != 0) {  // mapped host memory: a plain store and a system-wide fence
    *static_cast<volatile int *>(a.status) = kStatusPeerTimeout;
    __threadfence_system();
    return;
  }
  DType sum;
  uint32_t bits = static_cast<uint32_t>(w[0]);
  memcpy(&sum, &bits, 4);
#pragma unroll
  for (int q = 1; q < kMaxWorld; ++q) {
    if (q < world) {
      DType v;
      bits = static_cast<uint32_t>(w[q]);
      memcpy(&v, &bits, 4);
      sum = sum + v;
    }
  }
  const uint32_t r = a.ld == a.cols ? 0 : i / a.cols;
  a.dst[static_cast<size_t>(r) * a.ld + (i - r * a.cols)] = sum;
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
  static_assert(sizeof(DType) == 4, "PeerModel carries 4-byte elements (a word is element + tag)");
  typedef typename ISharedModel<gpu, DType>::CallbackFunction CallbackFunction;
  PeerModel()
      : rank_(0), world_(1), device_(-1), depth_(4), wait_limit_ms_(2000), window_bytes_(size_t(64) << 20),
        window_(NULL), used_(0), status_host_(NULL), status_dev_(NULL), own_stream_(0), ready_(false),
        connected_(false) {
    comm_.stream_ = NULL;
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
    if (!strcmp(name, "own_stream")) own_stream_ = atoi(val);
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
    MSHADOW_CUDA_CALL(cudaMemset(window_, 0, window_bytes_));  // tag 0 belongs to no step
    // the status word lives in mapped host memory: a timed-out kernel writes it, the host reads it
    // without a copy (and therefore without touching any stream)
    MSHADOW_CUDA_CALL(cudaHostAlloc(reinterpret_cast<void **>(&status_host_), sizeof(int), cudaHostAllocMapped));
    *status_host_ = 0;
    MSHADOW_CUDA_CALL(cudaHostGetDevicePointer(reinterpret_cast<void **>(&status_dev_), status_host_, 0));
    if (own_stream_) MSHADOW_CUDA_CALL(cudaStreamCreateWithFlags(&comm_.stream_, cudaStreamNonBlocking));
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

  /*!
   * \brief instead of Push: the sink through which a reduction kernel delivers `count` results,
   *  starting at element `offset` of the key's row, to all ranks.  The first call of a step
   *  (offset 0) opens it; segments must together cover the whole row before the step is pulled.
   */
  gpu_rt::PeerSink NextSink(int key, int devid, uint32_t offset, uint32_t count) {
    Entry &e = this->Find(key, devid);
    CHECK(connected_) << "PeerModel: Connect has not been called";
    CHECK_LE(static_cast<size_t>(offset) + count, e.shape.Size()) << "NextSink: segment beyond the key's extent";
    if (offset == 0) this->OpenStep(&e);
    CHECK_GT(e.push_seq, 0U) << "NextSink: the first segment of a step starts at offset 0";
    return this->SinkOf(e, e.push_seq - 1, offset, count);
  }

  virtual void PullWait(int key, int devid) {
    Entry &e = this->Find(key, devid);
    if (e.pull_pending) {
      MSHADOW_CUDA_CALL(cudaEventSynchronize(e.pull_done));
      e.pull_pending = false;
    }
    this->CheckStatus();
  }

  virtual void PullFence(int key, int devid, Stream<gpu> *stream) {
    Entry &e = this->Find(key, devid);
    if (e.pull_pending) MSHADOW_CUDA_CALL(cudaStreamWaitEvent(Stream<gpu>::GetStream(stream), e.pull_done, 0));
  }

  /*! \brief every rank's `data` becomes rank 0's (synchronous) */
  virtual void SetWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
    Entry &e = this->Find(key, devid);
    const cudaStream_t s = this->WorkStream(data.stream_, &e);
    this->PushStep(data, &e, s);
    this->PullStep(data, &e, 1, s);
    MSHADOW_CUDA_CALL(cudaStreamSynchronize(s));
    this->CheckStatus();
  }

  /*! \brief CHECKs that `data` equals rank 0's copy bit for bit (synchronous) */
  virtual void CheckWeight_(Tensor<gpu, 2, DType> data, int key, int devid) {
#ifdef __CUDACC__
    Entry &e = this->Find(key, devid);
    const size_t n = e.shape.Size();
    const cudaStream_t s = this->WorkStream(data.stream_, &e);
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
    this->PushStep(dense_mine, &e, s);
    this->PullStep(dense_root, &e, 1, s);
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

  /*! \brief bytes of the window that InitKey and ReserveRaw have handed out so far */
  size_t WindowUsed() const { return used_; }

  /*!
   * \brief sets `bytes` of every rank's window aside for the caller's own kernels and returns
   *  their offset.  All ranks make the same calls in the same order, so the offset is the same
   *  everywhere.  What travels through such a region, and how its readers learn that it has
   *  arrived, is the caller's business; a key pushed after the writing kernels, on the same stream,
   *  is a completion signal: its words are stored after those kernels have finished.
   */
  size_t ReserveRaw(size_t bytes) {
    CHECK(ready_) << "PeerModel: Init has not been called";
    const size_t offset = peerdetail::RoundUp(used_, 256);
    CHECK_LE(offset + bytes, window_bytes_) << "PeerModel: a region of " << bytes << " bytes does not fit the window of "
                                            << window_bytes_ << " bytes (SetParam(\"window_bytes\", ...) before Init)";
    used_ = offset + bytes;
    return offset;
  }

  /*! \brief address, in this process, of byte `offset` of rank p's window (plain loads and stores only) */
  void *WindowOf(int p, size_t offset) const {
    CHECK(connected_) << "PeerModel: Connect has not been called";
    CHECK(p >= 0 && p < world_) << "PeerModel: rank " << p << " of " << world_;
    CHECK_LE(offset, window_bytes_) << "PeerModel: offset beyond the window";
    return peer_[p] + offset;
  }

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
    e.row_bytes = peerdetail::RoundUp((n > 0 ? n : 1) * sizeof(peerdetail::Word), 256);
    e.data_offset = used_;
    const size_t end = e.data_offset + static_cast<size_t>(depth_) * world_ * e.row_bytes;
    CHECK_LE(end, window_bytes_) << "PeerModel: key " << key << " does not fit the window of " << window_bytes_
                                 << " bytes (SetParam(\"window_bytes\", ...) before Init)";
    used_ = end;
    MSHADOW_CUDA_CALL(cudaEventCreateWithFlags(&e.pull_done, cudaEventDisableTiming));
    MSHADOW_CUDA_CALL(cudaEventCreateWithFlags(&e.ordered, cudaEventDisableTiming));
    entries_[key] = e;
  }

  virtual void Push_(Tensor<gpu, 2, DType> data, int key, int devid, int) {
    Entry &e = this->Find(key, devid);
    this->PushStep(data, &e, this->WorkStream(data.stream_, &e));
  }

  virtual void PullReq_(Tensor<gpu, 2, DType> data, int key, int devid, int, CallbackFunction callback,
                        void *callback_arg) {
    Entry &e = this->Find(key, devid);
    // ordered behind everything the requester has enqueued: its use of `data`, and the kernels
    // that deliver this rank's own contribution through a sink
    const cudaStream_t s = this->WorkStream(data.stream_, &e);
    this->PullStep(data, &e, 0, s);
    if (callback != NULL) callback(own_stream_ ? &comm_ : data.stream_, callback_arg);
    MSHADOW_CUDA_CALL(cudaEventRecord(e.pull_done, s));
    e.pull_pending = true;
  }

 private:
  struct Entry {
    Shape<2> shape;
    size_t data_offset, row_bytes;  // within every rank's window
    uint32_t push_seq, pull_seq;
    cudaEvent_t pull_done;
    cudaEvent_t ordered;  // marks the caller's stream when work moves to the model's own stream
    bool pull_pending;
  };

  /*! \brief the stream a call's kernels run on: the caller's, or the model's own ordered behind it */
  cudaStream_t WorkStream(Stream<gpu> *user, Entry *e) {
    const cudaStream_t s = Stream<gpu>::GetStream(user);
    if (!own_stream_) return s;
    MSHADOW_CUDA_CALL(cudaEventRecord(e->ordered, s));
    MSHADOW_CUDA_CALL(cudaStreamWaitEvent(comm_.stream_, e->ordered, 0));
    return comm_.stream_;
  }

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
                 << " ms (status " << code << "); elements that had not arrived were not written";
    }
  }

  /*! \brief a new step of the key begins: refuse to run further ahead of the pulls than the slots allow */
  void OpenStep(Entry *e) {
    CHECK_LE(e->push_seq - e->pull_seq, static_cast<uint32_t>(depth_ / 2 - 1))
        << "Push: too many steps pushed ahead of their pulls for depth " << depth_;
    e->push_seq += 1;
  }

  /*! \brief where `count` elements from `offset` of step `seq` go in every rank's window */
  gpu_rt::PeerSink SinkOf(const Entry &e, uint32_t seq, uint32_t offset, uint32_t count) const {
    gpu_rt::PeerSink sink;
    const uint32_t slot = seq % static_cast<uint32_t>(depth_);
    for (int p = 0; p < world_; ++p) {
      sink.row[p] = reinterpret_cast<peerdetail::Word *>(peer_[p] + e.data_offset +
                                                         (static_cast<size_t>(slot) * world_ + rank_) * e.row_bytes) +
                    offset;
    }
    sink.tag = seq + 1;
    sink.count = count;
    sink.world = world_;
    return sink;
  }

  void PushStep(const Tensor<gpu, 2, DType> &data, Entry *e, cudaStream_t stream) {
#ifdef __CUDACC__
    CHECK(connected_) << "PeerModel: Connect has not been called";
    CHECK_EQ(data.shape_, e->shape) << "Push: shape differs from InitKey";
    this->OpenStep(e);
    const size_t n = e->shape.Size();
    if (n == 0) return;
    const gpu_rt::PeerSink sink = this->SinkOf(*e, e->push_seq - 1, 0, static_cast<uint32_t>(n));
    const unsigned ctas = static_cast<unsigned>((n + peerdetail::kPushThreads - 1) / peerdetail::kPushThreads);
    peerdetail::PeerPushKernel<DType><<<ctas, peerdetail::kPushThreads, 0, stream>>>(
        data.dptr_, e->shape[0], e->shape[1], data.stride_, sink);
    MSHADOW_CUDA_POST_KERNEL_CHECK(PeerPushKernel);
#else
    LOG(FATAL) << "PeerModel needs a CUDA translation unit";
#endif
  }

  void PullStep(Tensor<gpu, 2, DType> data, Entry *e, int root_only, cudaStream_t stream) {
#ifdef __CUDACC__
    CHECK_EQ(data.shape_, e->shape) << "PullReq: shape differs from InitKey";
    CHECK_LT(e->pull_seq, e->push_seq) << "PullReq: nothing pushed under this key that was not pulled already";
    const size_t n = e->shape.Size();
    const uint32_t slot = e->pull_seq % static_cast<uint32_t>(depth_);
    e->pull_seq += 1;
    if (n == 0) return;
    peerdetail::PullArgs<DType> a;
    a.dst = data.dptr_;
    a.rows = e->shape[0];
    a.cols = e->shape[1];
    a.ld = data.stride_;
    a.slot = reinterpret_cast<const peerdetail::Word *>(peer_[rank_] + e->data_offset +
                                                        static_cast<size_t>(slot) * world_ * e->row_bytes);
    a.row_stride = static_cast<uint32_t>(e->row_bytes / sizeof(peerdetail::Word));
    a.tag = e->pull_seq;  // already advanced: step + 1
    a.world = world_;
    a.root_only = root_only;
    a.limit_ns = static_cast<unsigned long long>(wait_limit_ms_) * 1000000ull;
    a.status = status_dev_;
    const unsigned ctas = static_cast<unsigned>((n + peerdetail::kPullThreads - 1) / peerdetail::kPullThreads);
    peerdetail::PeerPullKernel<DType><<<ctas, peerdetail::kPullThreads, 0, stream>>>(a);
    MSHADOW_CUDA_POST_KERNEL_CHECK(PeerPullKernel);
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
      cudaEventDestroy(it->second.ordered);
    }
    if (comm_.stream_ != NULL) cudaStreamDestroy(comm_.stream_);
    comm_.stream_ = NULL;
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
  int own_stream_;
  Stream<gpu> comm_;
  char *peer_[peerdetail::kMaxWorld];
  bool opened_[peerdetail::kMaxWorld];
  std::string peer_handles_hex_;
  std::map<int, Entry> entries_;
  bool ready_, connected_;
};

}  // namespace ps
}  // namespace mshadow
#endif  // MSHADOW_PS_PEER_MODEL_H_
