/*
 * C ABI around mshadow::ps::NcclModel<float> and mshadow::ps::PeerModel<float> (see
 * mshadow_b200_ps.h for the contract).  A handle is a pointer to the ISharedModel base, so the
 * tensor calls are the same for both models.
 * A separate shared object, so that the single-GPU library carries no NCCL dependency.
 */
#include "mshadow_b200_ps.h"

#include <cstdio>
#include <string>

#include "mshadow-ps/mshadow_ps.h"

using namespace mshadow;  // NOLINT(*)

namespace {

thread_local std::string g_ps_error;

int FailPs(const std::string &msg) {
  g_ps_error = msg;
  return 1;
}

typedef ps::ISharedModel<gpu, float> Model;
typedef ps::NcclModel<float> NcclImpl;
typedef ps::PeerModel<float> PeerImpl;

/*! \brief the caller's matrix as a tensor on the caller's stream */
struct View {
  Stream<gpu> stream;
  Tensor<gpu, 2, float> tensor;
  View(const float *p, int64_t rows, int64_t cols, int64_t ld, void *s)
      : tensor(const_cast<float *>(p), Shape2(rows, cols), static_cast<index_t>(ld), NULL) {
    stream.stream_ = static_cast<cudaStream_t>(s);
    tensor.stream_ = &stream;
  }
};

bool ShapeOk(int64_t rows, int64_t cols, int64_t ld) {
  return rows >= 0 && cols >= 0 && ld >= cols && rows < (int64_t(1) << 31) && cols < (int64_t(1) << 31) &&
         rows * cols < (int64_t(1) << 31);
}

}  // namespace

#define PS_BEGIN try {
#define PS_END                      \
  }                                 \
  catch (const std::exception &e) { \
    return FailPs(e.what());        \
  }                                 \
  return 0;

extern "C" {

const char *msb_ps_last_error(void) { return g_ps_error.c_str(); }

int msb_ps_new_unique_id(char *hex, int64_t capacity) {
  if (hex == NULL || capacity < 2 * NCCL_UNIQUE_ID_BYTES + 1) return FailPs("msb_ps_new_unique_id: buffer too small");
  PS_BEGIN
  const std::string s = NcclImpl::NewUniqueIdHex();
  snprintf(hex, static_cast<size_t>(capacity), "%s", s.c_str());
  PS_END
}

int msb_ps_create(int rank, int world, const char *id_hex, int device, msb_ps_t *out) {
  if (out == NULL) return FailPs("msb_ps_create: null pointer");
  if (world < 1 || rank < 0 || rank >= world) return FailPs("msb_ps_create: rank outside [0, world)");
  if (world > 1 && id_hex == NULL) return FailPs("msb_ps_create: an identifier is needed for more than one process");
  NcclImpl *m = NULL;
  try {
    m = new NcclImpl();
    char num[32];
    snprintf(num, sizeof(num), "%d", rank);
    m->SetParam("rank", num);
    snprintf(num, sizeof(num), "%d", world);
    m->SetParam("world_size", num);
    if (id_hex != NULL) m->SetParam("nccl_id", id_hex);
    m->Init(std::vector<int>(1, device));
  } catch (const std::exception &e) {
    delete m;
    return FailPs(e.what());
  }
  *out = static_cast<Model *>(m);
  return 0;
}

int msb_ps_peer_create(int rank, int world, int device, int64_t window_bytes, int depth, int wait_limit_ms,
                       int own_stream, msb_ps_t *out) {
  if (out == NULL) return FailPs("msb_ps_peer_create: null pointer");
  if (world < 1 || rank < 0 || rank >= world) return FailPs("msb_ps_peer_create: rank outside [0, world)");
  PeerImpl *m = NULL;
  try {
    m = new PeerImpl();
    char num[32];
    snprintf(num, sizeof(num), "%d", rank);
    m->SetParam("rank", num);
    snprintf(num, sizeof(num), "%d", world);
    m->SetParam("world_size", num);
    if (window_bytes > 0) {
      snprintf(num, sizeof(num), "%lld", static_cast<long long>(window_bytes));
      m->SetParam("window_bytes", num);
    }
    if (depth > 0) {
      snprintf(num, sizeof(num), "%d", depth);
      m->SetParam("depth", num);
    }
    if (wait_limit_ms > 0) {
      snprintf(num, sizeof(num), "%d", wait_limit_ms);
      m->SetParam("wait_limit_ms", num);
    }
    m->SetParam("own_stream", own_stream ? "1" : "0");
    m->Init(std::vector<int>(1, device));
  } catch (const std::exception &e) {
    delete m;
    return FailPs(e.what());
  }
  *out = static_cast<Model *>(m);
  return 0;
}

int msb_ps_peer_handle(msb_ps_t model, char *hex, int64_t capacity) {
  PeerImpl *m = dynamic_cast<PeerImpl *>(static_cast<Model *>(model));
  if (m == NULL) return FailPs("msb_ps_peer_handle: not a peer model");
  if (hex == NULL || capacity < 2 * ps::peerdetail::kHandleBytes + 1) return FailPs("msb_ps_peer_handle: buffer too small");
  PS_BEGIN
  const std::string s = m->ExportHandleHex();
  snprintf(hex, static_cast<size_t>(capacity), "%s", s.c_str());
  PS_END
}

int msb_ps_peer_connect(msb_ps_t model, const char *all_handles_hex) {
  PeerImpl *m = dynamic_cast<PeerImpl *>(static_cast<Model *>(model));
  if (m == NULL) return FailPs("msb_ps_peer_connect: not a peer model");
  if (all_handles_hex == NULL) return FailPs("msb_ps_peer_connect: null pointer");
  PS_BEGIN
  m->SetParam("peer_handles", all_handles_hex);
  m->Connect();
  PS_END
}

int msb_ps_peer_next_sink(msb_ps_t model, int key, int64_t offset, int64_t count, msb_peer_sink_t *out) {
  PeerImpl *m = dynamic_cast<PeerImpl *>(static_cast<Model *>(model));
  if (m == NULL) return FailPs("msb_ps_peer_next_sink: not a peer model");
  if (out == NULL) return FailPs("msb_ps_peer_next_sink: null pointer");
  if (offset < 0 || count < 0 || offset + count >= (int64_t(1) << 31)) return FailPs("msb_ps_peer_next_sink: extent out of range");
  static_assert(sizeof(msb_peer_sink_t) == sizeof(gpu_rt::PeerSink), "msb_peer_sink_t must mirror gpu_rt::PeerSink");
  PS_BEGIN
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  const gpu_rt::PeerSink sink = m->NextSink(key, dev, static_cast<uint32_t>(offset), static_cast<uint32_t>(count));
  for (int p = 0; p < MSB_PEER_MAX_WORLD; ++p) out->row[p] = sink.row[p];
  out->tag = sink.tag;
  out->count = sink.count;
  out->world = sink.world;
  PS_END
}

int msb_ps_peer_reserve(msb_ps_t model, int64_t bytes, int64_t *offset) {
  PeerImpl *m = dynamic_cast<PeerImpl *>(static_cast<Model *>(model));
  if (m == NULL) return FailPs("msb_ps_peer_reserve: not a peer model");
  if (offset == NULL || bytes < 0) return FailPs("msb_ps_peer_reserve: bad argument");
  PS_BEGIN
  *offset = static_cast<int64_t>(m->ReserveRaw(static_cast<size_t>(bytes)));
  PS_END
}

int msb_ps_peer_window(msb_ps_t model, int rank, int64_t offset, void **ptr) {
  PeerImpl *m = dynamic_cast<PeerImpl *>(static_cast<Model *>(model));
  if (m == NULL) return FailPs("msb_ps_peer_window: not a peer model");
  if (ptr == NULL || offset < 0) return FailPs("msb_ps_peer_window: bad argument");
  PS_BEGIN
  *ptr = m->WindowOf(rank, static_cast<size_t>(offset));
  PS_END
}

int msb_ps_destroy(msb_ps_t model) {
  PS_BEGIN
  delete static_cast<Model *>(model);
  PS_END
}

int msb_ps_init_key(msb_ps_t model, int key, int64_t rows, int64_t cols) {
  if (model == NULL) return FailPs("msb_ps_init_key: null model");
  if (!ShapeOk(rows, cols, cols)) return FailPs("msb_ps_init_key: extent out of range");
  PS_BEGIN
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  static_cast<Model *>(model)->InitKey(Shape2(rows, cols), key, dev);
  PS_END
}

#define PS_TENSOR_CALL(NAME, CALL)                                                                    \
  if (model == NULL || (data == NULL && rows * cols > 0)) return FailPs(NAME ": null pointer");      \
  if (!ShapeOk(rows, cols, ld)) return FailPs(NAME ": extent out of range");                         \
  PS_BEGIN                                                                                            \
  int dev = 0;                                                                                        \
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));                                                             \
  View v(data, rows, cols, ld, stream);                                                               \
  static_cast<Model *>(model)->CALL;                                                                  \
  PS_END

int msb_ps_push(msb_ps_t model, const float *data, int64_t rows, int64_t cols, int64_t ld, int key, void *stream) {
  PS_TENSOR_CALL("msb_ps_push", Push(v.tensor, key, dev))
}

int msb_ps_pull_req(msb_ps_t model, float *data, int64_t rows, int64_t cols, int64_t ld, int key, void *stream) {
  PS_TENSOR_CALL("msb_ps_pull_req", PullReq(v.tensor, key, dev))
}

int msb_ps_pull_wait(msb_ps_t model, int key) {
  if (model == NULL) return FailPs("msb_ps_pull_wait: null model");
  PS_BEGIN
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  static_cast<Model *>(model)->PullWait(key, dev);
  PS_END
}

int msb_ps_pull_fence(msb_ps_t model, int key, void *stream) {
  if (model == NULL) return FailPs("msb_ps_pull_fence: null model");
  PS_BEGIN
  int dev = 0;
  MSHADOW_CUDA_CALL(cudaGetDevice(&dev));
  Stream<gpu> st;
  st.stream_ = static_cast<cudaStream_t>(stream);
  static_cast<Model *>(model)->PullFence(key, dev, &st);
  PS_END
}

int msb_ps_set_weight(msb_ps_t model, float *data, int64_t rows, int64_t cols, int64_t ld, int key, void *stream) {
  PS_TENSOR_CALL("msb_ps_set_weight", SetWeight(v.tensor, key, dev))
}

int msb_ps_check_weight(msb_ps_t model, const float *data, int64_t rows, int64_t cols, int64_t ld, int key,
                        void *stream) {
  PS_TENSOR_CALL("msb_ps_check_weight", CheckWeight(v.tensor, key, dev))
}

}  // extern "C"
