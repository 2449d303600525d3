/*
 * extern "C" layer of the B200 mshadow engine (declared in include/mshadow_b200.h).
 *
 * Every entry point validates its arguments, wraps the raw pointers in mshadow::Tensor
 * handles and calls the header-level C++ API, which holds all kernels.  The translation
 * unit is compiled with DMLC_LOG_FATAL_THROW=1, so a failed CHECK inside the C++ API
 * surfaces here as a dmlc::Error; it is turned into a status code and a thread-local
 * message.  Nothing in this file computes on the host and there is no fallback path: if
 * the CUDA runtime or the device is unusable the call fails with MSB_ERR_CUDA.
 */
#include "mshadow_b200.h"

#include <string>

#include "mshadow/tensor.h"
#include "mshadow/gpu/math.h"
#include "./axis_cases.h"
#include "./complex_cases.h"

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

namespace {

thread_local std::string g_last_error;

int Fail(int code, const std::string &msg) {
  g_last_error = msg;
  return code;
}

/*! \brief a Stream<gpu> that wraps a caller-owned cudaStream_t for the duration of one call */
struct BorrowedStream {
  Stream<gpu> s;
  explicit BorrowedStream(msb_stream_t raw) { s.stream_ = static_cast<cudaStream_t>(raw); }
  Stream<gpu> *get() { return &s; }
};

typedef Tensor<gpu, 1, float> G1;
typedef Tensor<gpu, 2, float> G2;
typedef Tensor<gpu, 3, float> G3;
typedef Tensor<gpu, 4, float> G4;

inline G2 Mat(const float *p, int64_t r, int64_t c, int64_t ld, Stream<gpu> *s) {
  return G2(const_cast<float *>(p), Shape2(r, c), static_cast<index_t>(ld), s);
}
inline G1 Vec(const float *p, int64_t n, Stream<gpu> *s) {
  return G1(const_cast<float *>(p), Shape1(n), static_cast<index_t>(n), s);
}
inline G4 Img(const float *p, int64_t n, int64_t c, int64_t h, int64_t w, int64_t ld, Stream<gpu> *s) {
  return G4(const_cast<float *>(p), Shape4(n, c, h, w), static_cast<index_t>(ld), s);
}
inline G3 Planes(const float *p, int64_t n, int64_t h, int64_t w, int64_t ld, Stream<gpu> *s) {
  return G3(const_cast<float *>(p), Shape3(n, h, w), static_cast<index_t>(ld), s);
}

inline bool FitsIndex(int64_t v) { return v >= 0 && v <= 0x7fffffffLL; }
/*! \brief a leading dimension covers its row and fits the 32-bit stride field of a Tensor */
inline bool LdOk(int64_t ld, int64_t width) { return ld >= width && FitsIndex(ld); }

// user-style functors for the exported expression cases (cf. guide/defop.cpp of the reference)
struct clip_mul {
  MSHADOW_XINLINE static float Map(float a, float b) { return a > b ? a * b : b; }
};
struct fma3 {
  MSHADOW_XINLINE static float Map(float a, float b, float c) { return a * b + c; }
};
struct square {
  MSHADOW_XINLINE static float Map(float a) { return a * a; }
};

template <typename Reducer>
void KeepLowest(G1 d, const G2 &s, float scale, int saver) {
  switch (saver) {
    case 0: MapReduceKeepLowest<sv::saveto, Reducer>(&d, s, scale); break;
    case 1: MapReduceKeepLowest<sv::plusto, Reducer>(&d, s, scale); break;
    case 2: MapReduceKeepLowest<sv::minusto, Reducer>(&d, s, scale); break;
    case 3: MapReduceKeepLowest<sv::multo, Reducer>(&d, s, scale); break;
    default: MapReduceKeepLowest<sv::divto, Reducer>(&d, s, scale); break;
  }
}
template <typename Reducer>
void KeepDim1(G1 d, const G4 &s, float scale, int saver) {
  switch (saver) {
    case 0: MapReduceKeepHighDim<sv::saveto, Reducer, 1>(&d, s, scale); break;
    case 1: MapReduceKeepHighDim<sv::plusto, Reducer, 1>(&d, s, scale); break;
    case 2: MapReduceKeepHighDim<sv::minusto, Reducer, 1>(&d, s, scale); break;
    case 3: MapReduceKeepHighDim<sv::multo, Reducer, 1>(&d, s, scale); break;
    default: MapReduceKeepHighDim<sv::divto, Reducer, 1>(&d, s, scale); break;
  }
}

}  // namespace

namespace msb_internal {
/*! \brief lets the library's other translation units report through msb_last_error() */
void SetLastError(const char *message) { g_last_error = message; }
}  // namespace msb_internal

// Every entry that launches work runs inside an NVTX range named after the function, so that a
// timeline shows the C ABI call around its kernels.  Without a profiler attached a range costs a
// few nanoseconds; -DMSHADOW_B200_NVTX=0 compiles them out.
#ifndef MSHADOW_B200_NVTX
#define MSHADOW_B200_NVTX 1
#endif
#if MSHADOW_B200_NVTX
#include <nvtx3/nvToolsExt.h>
namespace {
struct TraceRange {
  explicit TraceRange(const char *name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
};
}  // namespace
#define MSB_TRACE_RANGE_ TraceRange msb_trace_range_(__func__);
#else
#define MSB_TRACE_RANGE_
#endif

#define MSB_GUARD_BEGIN MSB_TRACE_RANGE_ try {
#define MSB_GUARD_END                                        \
  }                                                          \
  catch (const dmlc::Error &e) {                             \
    const std::string what = e.what();                       \
    const bool cuda = what.find("CUDA") != std::string::npos || what.find("ErrStr") != std::string::npos; \
    return Fail(cuda ? MSB_ERR_CUDA : MSB_ERR_SHAPE, what);  \
  }                                                          \
  catch (const std::exception &e) {                          \
    return Fail(MSB_ERR_MEMORY, e.what());                   \
  }                                                          \
  return MSB_OK;

#define MSB_REQUIRE(cond, code, msg) \
  if (!(cond)) return Fail(code, std::string(__func__) + ": " + msg)

extern "C" {

const char *msb_last_error(void) { return g_last_error.c_str(); }
int msb_version(void) { return 100; }
int64_t msb_launch_count(void) { return gpu_rt::LaunchCounter().load(); }

int msb_init(int device) {
  MSB_GUARD_BEGIN
  InitTensorEngine<gpu>(device);
  MSB_GUARD_END
}
int msb_set_device(int device) {
  MSB_GUARD_BEGIN
  SetDevice<gpu>(device);
  MSB_GUARD_END
}
int msb_shutdown(void) {
  MSB_GUARD_BEGIN
  ShutdownTensorEngine<gpu>();
  MSB_GUARD_END
}
int msb_stream_create(msb_stream_t *out) {
  MSB_REQUIRE(out != nullptr, MSB_ERR_ARGUMENT, "null output");
  cudaStream_t s;
  const cudaError_t err = cudaStreamCreate(&s);
  if (err != cudaSuccess) return Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
  *out = s;
  return MSB_OK;
}
int msb_stream_destroy(msb_stream_t stream) {
  MSB_GUARD_BEGIN
  gpu_rt::Scratch::Release(false, static_cast<cudaStream_t>(stream));
  MSHADOW_CUDA_CALL(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  MSB_GUARD_END
}
int msb_stream_wait(msb_stream_t stream) {
  // A kernel whose bounded wait ran out leaves a mark in the device's status word.  The word is
  // read on the waited stream itself (into page-locked memory), so that waiting on one stream does
  // not wait for work on the others.
  MSB_TRACE_RANGE_
  try {
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    int *word = gpu_rt::StatusWord();
    int *seen = gpu_rt::StatusMirror();
    *seen = 0;
    MSHADOW_CUDA_CALL(cudaMemcpyAsync(seen, word, sizeof(int), cudaMemcpyDeviceToHost, s));
    const cudaError_t err = cudaStreamSynchronize(s);
    if (err != cudaSuccess) return Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
    const int flag = *seen;
    if (flag != 0) {
      MSHADOW_CUDA_CALL(cudaMemsetAsync(word, 0, sizeof(int), s));
      MSHADOW_CUDA_CALL(cudaStreamSynchronize(s));
      return Fail(MSB_ERR_TIMEOUT, "a device-side bounded wait gave up (status " + std::to_string(flag) + ")");
    }
  } catch (const dmlc::Error &e) {
    return Fail(MSB_ERR_CUDA, e.what());
  } catch (const std::exception &e) {
    return Fail(MSB_ERR_MEMORY, e.what());
  }
  return MSB_OK;
}
namespace {
__global__ void WaitThatNothingSignalsKernel(int *status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  mshadow::cuda::tma::BarrierInit(&bar, 1);  // one arrival expected; none will come
  if (!mshadow::cuda::tma::WaitBounded(&bar, 0, limit_ns)) {
    atomicExch(status, mshadow::cuda::tma::kStatusBulkCopyTimeout);
  }
}
}  // namespace

int msb_selftest_bounded_wait(int limit_ms, msb_stream_t stream) {
  MSB_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, MSB_ERR_ARGUMENT, "limit_ms must be within 1..1000");
  MSB_GUARD_BEGIN
  WaitThatNothingSignalsKernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      gpu_rt::StatusWord(), static_cast<unsigned long long>(limit_ms) * 1000000ull);
  MSHADOW_CUDA_POST_KERNEL_CHECK(WaitThatNothingSignalsKernel);
  MSB_GUARD_END
}

int msb_stream_idle(msb_stream_t stream, int *idle) {
  MSB_REQUIRE(idle != nullptr, MSB_ERR_ARGUMENT, "null output");
  const cudaError_t err = cudaStreamQuery(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess && err != cudaErrorNotReady) return Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
  *idle = err == cudaSuccess;
  return MSB_OK;
}

int msb_alloc_space(void **dptr_out, int64_t *ld_out, int64_t rows, int64_t cols, int64_t elem_size, int pad) {
  MSB_REQUIRE(dptr_out != nullptr && ld_out != nullptr, MSB_ERR_ARGUMENT, "null output");
  MSB_REQUIRE(rows >= 0 && cols >= 0 && elem_size > 0, MSB_ERR_ARGUMENT, "negative size");
  void *p = nullptr;
  size_t pitch = 0;
  cudaError_t err;
  if (pad && cols >= MSHADOW_MIN_PAD_RATIO * 32) {
    err = cudaMallocPitch(&p, &pitch, cols * elem_size, rows);
    *ld_out = static_cast<int64_t>(pitch / elem_size);
  } else {
    const size_t bytes = static_cast<size_t>(rows) * cols * elem_size;
    err = cudaMalloc(&p, bytes == 0 ? 1 : bytes);
    *ld_out = cols;
  }
  if (err != cudaSuccess) return Fail(MSB_ERR_MEMORY, cudaGetErrorString(err));
  *dptr_out = p;
  return MSB_OK;
}
int msb_free_space(void *dptr) {
  const cudaError_t err = cudaFree(dptr);
  return err == cudaSuccess ? MSB_OK : Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
}
int msb_alloc_host(void **ptr_out, int64_t bytes) {
  MSB_REQUIRE(ptr_out != nullptr && bytes >= 0, MSB_ERR_ARGUMENT, "bad argument");
  const cudaError_t err = cudaMallocHost(ptr_out, bytes == 0 ? 1 : bytes, cudaHostAllocPortable);
  return err == cudaSuccess ? MSB_OK : Fail(MSB_ERR_MEMORY, cudaGetErrorString(err));
}
int msb_free_host(void *ptr) {
  const cudaError_t err = cudaFreeHost(ptr);
  return err == cudaSuccess ? MSB_OK : Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
}
int msb_copy_2d(void *dst, int64_t ld_dst, const void *src, int64_t ld_src, int64_t rows, int64_t cols,
                int64_t elem_size, int kind, msb_stream_t stream) {
  MSB_REQUIRE(kind >= 1 && kind <= 3, MSB_ERR_ARGUMENT, "kind must be 1 (h2d), 2 (d2h) or 3 (d2d)");
  MSB_REQUIRE(rows >= 0 && cols >= 0 && LdOk(ld_dst, cols) && LdOk(ld_src, cols), MSB_ERR_SHAPE, "bad extents");
  if (rows == 0 || cols == 0) return MSB_OK;
  MSB_REQUIRE(dst != nullptr && src != nullptr, MSB_ERR_ARGUMENT, "null pointer");
  const cudaMemcpyKind k =
      kind == 1 ? cudaMemcpyHostToDevice : (kind == 2 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice);
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  if (ld_dst == cols && ld_src == cols) {
    err = cudaMemcpyAsync(dst, src, static_cast<size_t>(rows) * cols * elem_size, k, s);
  } else {
    err = cudaMemcpy2DAsync(dst, ld_dst * elem_size, src, ld_src * elem_size, cols * elem_size, rows, k, s);
  }
  return err == cudaSuccess ? MSB_OK : Fail(MSB_ERR_CUDA, cudaGetErrorString(err));
}
int msb_workspace(msb_stream_t stream, int64_t bytes, void **out) {
  MSB_REQUIRE(out != nullptr && bytes >= 0, MSB_ERR_ARGUMENT, "bad argument");
  MSB_GUARD_BEGIN
  // the caller's buffer is not the one the operators park their partial results in
  *out = gpu_rt::Scratch::Get(static_cast<cudaStream_t>(stream), static_cast<size_t>(bytes), gpu_rt::Scratch::kCaller);
  MSB_GUARD_END
}

int msb_scratch_bytes(msb_stream_t stream, int64_t *engine_bytes, int64_t *caller_bytes) {
  MSB_REQUIRE(engine_bytes != nullptr && caller_bytes != nullptr, MSB_ERR_ARGUMENT, "null output");
  MSB_GUARD_BEGIN
  *engine_bytes = static_cast<int64_t>(gpu_rt::Scratch::Held(static_cast<cudaStream_t>(stream), gpu_rt::Scratch::kEngine));
  *caller_bytes = static_cast<int64_t>(gpu_rt::Scratch::Held(static_cast<cudaStream_t>(stream), gpu_rt::Scratch::kCaller));
  MSB_GUARD_END
}

int msb_expr_case_f32(int id, float *dst, const float *A, const float *B, const float *C, const float *bias,
                      int64_t rows, int64_t cols, int64_t ld_dst, int64_t ld_a, int64_t ld_b, int64_t ld_c,
                      msb_stream_t stream) {
  MSB_REQUIRE(id >= 0 && id <= 9, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(FitsIndex(rows) && FitsIndex(cols) && FitsIndex(rows * cols), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(LdOk(ld_dst, cols) && LdOk(ld_a, cols) && LdOk(ld_b, cols) && LdOk(ld_c, cols), MSB_ERR_SHAPE, "stride < width");
  if (rows == 0 || cols == 0) return MSB_OK;
  MSB_REQUIRE(dst && A && B && C && bias, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G2 d = Mat(dst, rows, cols, ld_dst, st.get());
  const G2 a = Mat(A, rows, cols, ld_a, st.get()), b = Mat(B, rows, cols, ld_b, st.get()),
           c = Mat(C, rows, cols, ld_c, st.get());
  switch (id) {
    case 0: d = F<b200::sigmoid>(a * b + 0.5f * c) + repmat(Vec(bias, cols, st.get()), rows); break;
    case 1: d += a * 2.0f - b / c; break;
    case 2: d = F<clip_mul>(a, b) * c; break;
    case 3: d *= a + 1.5f; break;
    case 4: d -= a * b; break;
    case 5: d /= c * c + 1.0f; break;
    case 6: d = 3.25f; break;
    case 7: d = F<fma3>(a, b, c); break;
    case 8: d = broadcast<0>(Vec(bias, rows, st.get()), d.shape_) * a + b; break;
    default: d = F<square>(a - 1.0f) / (b * b + 2.0f) + c; break;
  }
  MSB_GUARD_END
}

static_assert(sizeof(msb_peer_sink_t) == sizeof(gpu_rt::PeerSink) && MSB_PEER_MAX_WORLD == gpu_rt::kPeerMaxWorld,
              "msb_peer_sink_t must mirror gpu_rt::PeerSink");

/*! \brief the C sink as the engine's; NULL or world 0 gives none */
static bool ToPeerSink(const msb_peer_sink_t *in, gpu_rt::PeerSink *out) {
  if (in == nullptr || in->world == 0) return true;
  if (in->world < 0 || in->world > MSB_PEER_MAX_WORLD) return false;
  for (int p = 0; p < in->world; ++p) {
    if (in->row[p] == nullptr) return false;
    out->row[p] = in->row[p];
  }
  out->tag = in->tag;
  out->count = in->count;
  out->world = in->world;
  return true;
}

int msb_reduce_keep_lowest_f32(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld, float scale,
                               int saver, int reducer, msb_stream_t stream) {
  return msb_reduce_keep_lowest_f32_sink(dst, src, rows, cols, ld, scale, saver, reducer, nullptr, stream);
}

int msb_reduce_keep_lowest_f32_sink(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld, float scale,
                                    int saver, int reducer, const msb_peer_sink_t *csink, msb_stream_t stream) {
  gpu_rt::PeerSink sink;
  MSB_REQUIRE(ToPeerSink(csink, &sink), MSB_ERR_ARGUMENT, "malformed peer sink");
  MSB_REQUIRE(sink.world == 0 || static_cast<int64_t>(sink.count) == cols, MSB_ERR_SHAPE,
              "the peer sink expects a different number of results");
  MSB_REQUIRE(saver >= 0 && saver <= 4 && reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown selector");
  MSB_REQUIRE(FitsIndex(rows) && FitsIndex(cols) && FitsIndex(rows * cols) && LdOk(ld, cols), MSB_ERR_SHAPE,
              "extent out of range");
  MSB_REQUIRE(rows > 0, MSB_ERR_SHAPE, "can not reduce over empty tensor");
  if (cols == 0) return MSB_OK;
  MSB_REQUIRE(dst && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const G1 d = Vec(dst, cols, st.get());
  const G2 s = Mat(src, rows, cols, ld, st.get());
  gpu_rt::PeerSinkScope scope(sink.world > 0 ? &sink : nullptr);
  if (reducer == 0) KeepLowest<red::sum>(d, s, scale, saver);
  else if (reducer == 1) KeepLowest<red::maximum>(d, s, scale, saver);
  else KeepLowest<red::minimum>(d, s, scale, saver);
  MSB_GUARD_END
}

int msb_reduce_keep_highdim_f32(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int64_t ld,
                                float scale, int saver, int reducer, msb_stream_t stream) {
  return msb_reduce_keep_highdim_f32_sink(dst, src, n, c, h, w, ld, scale, saver, reducer, nullptr, stream);
}

int msb_reduce_keep_highdim_f32_sink(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                                     int64_t ld, float scale, int saver, int reducer, const msb_peer_sink_t *csink,
                                     msb_stream_t stream) {
  gpu_rt::PeerSink sink;
  MSB_REQUIRE(ToPeerSink(csink, &sink), MSB_ERR_ARGUMENT, "malformed peer sink");
  MSB_REQUIRE(sink.world == 0 || static_cast<int64_t>(sink.count) == c, MSB_ERR_SHAPE,
              "the peer sink expects a different number of results");
  MSB_REQUIRE(saver >= 0 && saver <= 4 && reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown selector");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(c) && FitsIndex(h) && FitsIndex(w) && LdOk(ld, w), MSB_ERR_SHAPE,
              "extent out of range");
  MSB_REQUIRE(FitsIndex(n * c) && FitsIndex(n * c * h) && FitsIndex(n * c * h * w), MSB_ERR_SHAPE, "tensor too large");
  if (c == 0) return MSB_OK;
  MSB_REQUIRE(dst && (src || n * h * w == 0), MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const G1 d = Vec(dst, c, st.get());
  const G4 s = Img(src, n, c, h, w, ld, st.get());
  gpu_rt::PeerSinkScope scope(sink.world > 0 ? &sink : nullptr);
  if (reducer == 0) KeepDim1<red::sum>(d, s, scale, saver);
  else if (reducer == 1) KeepDim1<red::maximum>(d, s, scale, saver);
  else KeepDim1<red::minimum>(d, s, scale, saver);
  MSB_GUARD_END
}

int msb_softmax_f32(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst, int64_t ld_src,
                    msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(rows) && FitsIndex(cols) && LdOk(ld_dst, cols) && LdOk(ld_src, cols), MSB_ERR_SHAPE,
              "extent out of range");
  if (rows == 0 || cols == 0) return MSB_OK;
  MSB_REQUIRE(dst && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  Softmax(Mat(dst, rows, cols, ld_dst, st.get()), Mat(src, rows, cols, ld_src, st.get()));
  MSB_GUARD_END
}

int msb_softmax_grad_f32(float *dst, const float *src, const float *label, int64_t rows, int64_t cols,
                         int64_t ld_dst, int64_t ld_src, int mode, float ignore_label, float alpha,
                         msb_stream_t stream) {
  MSB_REQUIRE(mode >= 0 && mode <= 3, MSB_ERR_ARGUMENT, "mode must be 0..3");
  MSB_REQUIRE(FitsIndex(rows) && FitsIndex(cols) && FitsIndex(rows * cols) && LdOk(ld_dst, cols) && LdOk(ld_src, cols),
              MSB_ERR_SHAPE, "extent out of range");
  if (rows == 0 || cols == 0) return MSB_OK;
  MSB_REQUIRE(dst && src && label, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G2 d = Mat(dst, rows, cols, ld_dst, st.get());
  const G2 s = Mat(src, rows, cols, ld_src, st.get());
  const G1 l = Vec(label, rows, st.get());
  switch (mode) {
    case 0: SoftmaxGrad(d, s, l); break;
    case 1: SmoothSoftmaxGrad(d, s, l, alpha); break;
    case 2: SoftmaxGrad(d, s, l, ignore_label); break;
    default: SmoothSoftmaxGrad(d, s, l, ignore_label, alpha); break;
  }
  MSB_GUARD_END
}

int msb_softmax_grad_fused_f32(float *dst, const float *logits, const float *label, int64_t rows, int64_t cols,
                               int64_t ld_dst, int64_t ld_src, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(rows) && FitsIndex(cols) && LdOk(ld_dst, cols) && LdOk(ld_src, cols), MSB_ERR_SHAPE,
              "extent out of range");
  if (rows == 0 || cols == 0) return MSB_OK;
  MSB_REQUIRE(dst && logits && label, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  SoftmaxGradFused(Mat(dst, rows, cols, ld_dst, st.get()), Mat(logits, rows, cols, ld_src, st.get()),
                   Vec(label, rows, st.get()));
  MSB_GUARD_END
}

int msb_pool_f32(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky, int kx, int sy, int sx,
                 int64_t ld_src, int64_t ld_dst, int reducer, msb_stream_t stream) {
  MSB_REQUIRE(reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown reducer");
  MSB_REQUIRE(ky > 0 && kx > 0 && sy > 0 && sx > 0, MSB_ERR_ARGUMENT, "window and stride must be positive");
  MSB_REQUIRE(FitsIndex(planes) && FitsIndex(h) && FitsIndex(w) && FitsIndex(planes * h) && FitsIndex(planes * h * w),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(h >= ky && w >= kx, MSB_ERR_SHAPE, "PoolingExp: kernel must be smaller than image");
  const int64_t ph = (h - ky) / sy + 1, pw = (w - kx) / sx + 1;
  MSB_REQUIRE(LdOk(ld_src, w) && LdOk(ld_dst, pw), MSB_ERR_SHAPE, "stride < width");
  if (planes == 0) return MSB_OK;
  MSB_REQUIRE(dst && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G3 d = Planes(dst, planes, ph, pw, ld_dst, st.get());
  const G3 s = Planes(src, planes, h, w, ld_src, st.get());
  if (reducer == 0) d = pool<red::sum>(s, ky, kx, sy, sx);
  else if (reducer == 1) d = pool<red::maximum>(s, ky, kx, sy, sx);
  else d = pool<red::minimum>(s, ky, kx, sy, sx);
  MSB_GUARD_END
}

int msb_unpool_f32(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t planes, int64_t h,
                   int64_t w, int64_t ph, int64_t pw, int ky, int kx, int sy, int sx, int64_t ld_src,
                   int64_t ld_pooled, int64_t ld_dst, int reducer, msb_stream_t stream) {
  MSB_REQUIRE(reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown reducer");
  MSB_REQUIRE(ky > 0 && kx > 0 && sy > 0 && sx > 0, MSB_ERR_ARGUMENT, "window and stride must be positive");
  MSB_REQUIRE(FitsIndex(planes) && FitsIndex(h) && FitsIndex(w) && FitsIndex(planes * h) && FitsIndex(planes * h * w) &&
                  FitsIndex(ph) && FitsIndex(pw),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(LdOk(ld_src, w) && LdOk(ld_dst, w) && LdOk(ld_pooled, pw), MSB_ERR_SHAPE, "stride < width");
  if (planes == 0 || h * w == 0) return MSB_OK;
  MSB_REQUIRE(dst && src && (ph * pw == 0 || (pooled && gpooled)), MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G3 d = Planes(dst, planes, h, w, ld_dst, st.get());
  const G3 s = Planes(src, planes, h, w, ld_src, st.get());
  const G3 p = Planes(pooled, planes, ph, pw, ld_pooled, st.get()), g = Planes(gpooled, planes, ph, pw, ld_pooled, st.get());
  if (reducer == 0) d = unpool<red::sum>(s, p, g, ky, kx, sy, sx);
  else if (reducer == 1) d = unpool<red::maximum>(s, p, g, ky, kx, sy, sx);
  else d = unpool<red::minimum>(s, p, g, ky, kx, sy, sx);
  MSB_GUARD_END
}

int msb_chpool_f32(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int nsize, int stride,
                   int pad, int64_t ld_src, int64_t ld_dst, int reducer, msb_stream_t stream) {
  MSB_REQUIRE(reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown reducer");
  MSB_REQUIRE(nsize > 0 && stride > 0 && pad >= 0, MSB_ERR_ARGUMENT, "bad window");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(c) && FitsIndex(h) && FitsIndex(w) && FitsIndex(n * c * h) &&
                  FitsIndex(n * c * h * w),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(c >= nsize, MSB_ERR_SHAPE, "chpool: local size must be smaller than nchannels");
  MSB_REQUIRE(LdOk(ld_src, w) && LdOk(ld_dst, w), MSB_ERR_SHAPE, "stride < width");
  const int64_t co = (c - nsize + pad * 2 + 1) / stride;
  if (n * co * h * w == 0) return MSB_OK;
  MSB_REQUIRE(dst && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G4 d = Img(dst, n, co, h, w, ld_dst, st.get());
  const G4 s = Img(src, n, c, h, w, ld_src, st.get());
  if (reducer == 0) d = chpool<red::sum>(s, nsize, stride, pad);
  else if (reducer == 1) d = chpool<red::maximum>(s, nsize, stride, pad);
  else d = chpool<red::minimum>(s, nsize, stride, pad);
  MSB_GUARD_END
}

int msb_ch_unpool_f32(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t n, int64_t c,
                      int64_t pc, int64_t h, int64_t w, int nsize, int stride, int pad, int64_t ld_src,
                      int64_t ld_pooled, int64_t ld_dst, int reducer, msb_stream_t stream) {
  MSB_REQUIRE(reducer >= 0 && reducer <= 2, MSB_ERR_ARGUMENT, "unknown reducer");
  MSB_REQUIRE(nsize > 0 && stride > 0 && pad >= 0, MSB_ERR_ARGUMENT, "bad window");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(c) && FitsIndex(pc) && FitsIndex(h) && FitsIndex(w) && FitsIndex(n * c * h) &&
                  FitsIndex(n * c * h * w) && FitsIndex(n * pc * h * w),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(LdOk(ld_src, w) && LdOk(ld_dst, w) && LdOk(ld_pooled, w), MSB_ERR_SHAPE, "stride < width");
  if (n * c * h * w == 0) return MSB_OK;
  {
    const int64_t top = (c - 1 + pad + stride) / stride;
    MSB_REQUIRE((top < c ? top : c) <= pc, MSB_ERR_SHAPE, "window reaches past the pooled channels");
  }
  MSB_REQUIRE(dst && src && pooled && gpooled, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G4 d = Img(dst, n, c, h, w, ld_dst, st.get());
  const G4 s = Img(src, n, c, h, w, ld_src, st.get());
  const G4 p = Img(pooled, n, pc, h, w, ld_pooled, st.get()), g = Img(gpooled, n, pc, h, w, ld_pooled, st.get());
  if (reducer == 0) d = ch_unpool<red::sum>(s, p, g, nsize, stride, pad);
  else if (reducer == 1) d = ch_unpool<red::maximum>(s, p, g, nsize, stride, pad);
  else d = ch_unpool<red::minimum>(s, p, g, nsize, stride, pad);
  MSB_GUARD_END
}

int msb_lrn_forward_f32(float *out, float *norm, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int nsize,
                        float salpha, float beta, float knorm, int power_kind, msb_stream_t stream) {
  MSB_REQUIRE(nsize > 0 && nsize % 2 == 1, MSB_ERR_ARGUMENT, "the window must be odd and positive");
  MSB_REQUIRE(power_kind >= 0 && power_kind <= 2, MSB_ERR_ARGUMENT, "power_kind must be 0 (powf), 1 (roots) or 2 (fast)");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(c) && FitsIndex(h) && FitsIndex(w) && FitsIndex(n * c * h) &&
                  FitsIndex(n * c * h * w),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(c >= nsize, MSB_ERR_SHAPE, "chpool: local size must be smaller than nchannels");
  if (n * c * h * w == 0) return MSB_OK;
  MSB_REQUIRE(out && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G4 o = Img(out, n, c, h, w, w, st.get());
  G4 nm = Img(norm, n, c, h, w, w, st.get());
  const G4 s = Img(src, n, c, h, w, w, st.get());
  if (power_kind == 0) LRNForward<b200::power>(o, nm, s, nsize, salpha, beta, knorm);
  else if (power_kind == 1) LRNForward<b200::power_by_roots>(o, nm, s, nsize, salpha, beta, knorm);
  else LRNForward<b200::power_fast>(o, nm, s, nsize, salpha, beta, knorm);
  MSB_GUARD_END
}

int msb_lrn_backward_f32(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n, int64_t c,
                         int64_t h, int64_t w, int nsize, float salpha, float beta, int power_kind,
                         msb_stream_t stream) {
  MSB_REQUIRE(nsize > 0 && nsize % 2 == 1, MSB_ERR_ARGUMENT, "the window must be odd and positive");
  MSB_REQUIRE(power_kind >= 0 && power_kind <= 2, MSB_ERR_ARGUMENT, "power_kind must be 0 (powf), 1 (roots) or 2 (fast)");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(c) && FitsIndex(h) && FitsIndex(w) && FitsIndex(n * c * h) &&
                  FitsIndex(n * c * h * w),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(c >= nsize, MSB_ERR_SHAPE, "chpool: local size must be smaller than nchannels");
  if (n * c * h * w == 0) return MSB_OK;
  MSB_REQUIRE(gsrc && gout && src && norm, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  G4 g = Img(gsrc, n, c, h, w, w, st.get());
  const G4 go = Img(gout, n, c, h, w, w, st.get()), s = Img(src, n, c, h, w, w, st.get()),
           nm = Img(norm, n, c, h, w, w, st.get());
  if (power_kind == 0) LRNBackward<b200::power>(g, go, s, nm, nsize, salpha, beta);
  else if (power_kind == 1) LRNBackward<b200::power_by_roots>(g, go, s, nm, nsize, salpha, beta);
  else LRNBackward<b200::power_fast>(g, go, s, nm, nsize, salpha, beta);
  MSB_GUARD_END
}

int msb_addtakegrad_f32_i32(float *dst, const int32_t *index, const float *src, int64_t k, int64_t d, int64_t nidx,
                            int64_t ld_dst, int64_t ld_src, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(k) && FitsIndex(d) && FitsIndex(nidx) && LdOk(ld_dst, d) && LdOk(ld_src, d), MSB_ERR_SHAPE,
              "extent out of range");
  MSB_REQUIRE(k > 0 || nidx == 0, MSB_ERR_SHAPE, "empty table");
  if (nidx == 0 || d == 0) return MSB_OK;
  MSB_REQUIRE(dst && index && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const Tensor<gpu, 1, int32_t> idx(const_cast<int32_t *>(index), Shape1(nidx), nidx, st.get());
  AddTakeGrad(Mat(dst, k, d, ld_dst, st.get()), idx, Mat(src, nidx, d, ld_src, st.get()));
  MSB_GUARD_END
}

int msb_addtakegrad_largebatch_f32_i32(float *dst, const int32_t *sorted, const int32_t *index, const float *src,
                                       int64_t k, int64_t d, int64_t nidx, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(k) && FitsIndex(d) && FitsIndex(nidx), MSB_ERR_SHAPE, "extent out of range");
  if (nidx == 0 || d == 0) return MSB_OK;
  MSB_REQUIRE(dst && sorted && index && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const Tensor<gpu, 1, int32_t> s(const_cast<int32_t *>(sorted), Shape1(nidx), nidx, st.get());
  const Tensor<gpu, 1, int32_t> i(const_cast<int32_t *>(index), Shape1(nidx), nidx, st.get());
  AddTakeGradLargeBatch(Mat(dst, k, d, d, st.get()), s, i, Mat(src, nidx, d, d, st.get()));
  MSB_GUARD_END
}

int msb_sort_by_key_i32(int32_t *keys, int32_t *values, int64_t n, int ascend, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n), MSB_ERR_SHAPE, "extent out of range");
  if (n == 0) return MSB_OK;
  MSB_REQUIRE(keys && values, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  Tensor<gpu, 1, int32_t> k(keys, Shape1(n), n, st.get()), v(values, Shape1(n), n, st.get());
  SortByKey(k, v, ascend != 0);
  MSB_GUARD_END
}

int msb_sort_by_key_lowbits_i32(int32_t *keys, int32_t *values, int64_t n, int bits, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(bits >= 1 && bits <= 31, MSB_ERR_ARGUMENT, "1 to 31 key bits");
  if (n <= 1) return MSB_OK;
  MSB_REQUIRE(keys && values, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  cudaStream_t cs = Stream<gpu>::GetStream(st.get());
  char *scratch = static_cast<char *>(mshadow::gpu_rt::Scratch::Get(cs, mshadow::cuda::sortdetail::ScratchBytes(n)));
  const mshadow::cuda::sortdetail::Source as_given = {0};
  mshadow::cuda::sortdetail::SortPairs<int32_t, int32_t>(keys, values, keys, n, bits, true, as_given, scratch, cs);
  MSB_GUARD_END
}

int msb_frequent_rows_i32(int32_t *rows_out, int32_t *counts_out, const int32_t *sorted, int64_t n, int64_t count,
                          msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n) && count >= 0 && count <= n, MSB_ERR_SHAPE, "extent out of range");
  if (count == 0) return MSB_OK;
  MSB_REQUIRE(rows_out && counts_out && sorted, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  cudaStream_t cs = Stream<gpu>::GetStream(st.get());
  using mshadow::cuda::sortdetail::Align256;
  const size_t ib = Align256(static_cast<size_t>(n) * 4);
  const size_t sort_bytes = mshadow::cuda::sortdetail::ScratchBytes(n);
  char *base = static_cast<char *>(mshadow::gpu_rt::Scratch::Get(cs, 2 * ib + sort_bytes));
  int32_t *lens = reinterpret_cast<int32_t *>(base), *rows = reinterpret_cast<int32_t *>(base + ib);
  mshadow::cuda::RunLengthLaunch(lens, rows, sorted, n, cs);
  // run lengths in descending order, stable: equal counts stay in ascending row order
  int bits = 1;
  while (bits < 31 && (int64_t(1) << bits) <= n) ++bits;
  const mshadow::cuda::sortdetail::Source as_given = {0};
  mshadow::cuda::sortdetail::SortPairs<int32_t, int32_t>(lens, rows, lens, n, bits, false, as_given, base + 2 * ib, cs);
  MSHADOW_CUDA_CALL(cudaMemcpyAsync(counts_out, lens, count * 4, cudaMemcpyDeviceToDevice, cs));
  MSHADOW_CUDA_CALL(cudaMemcpyAsync(rows_out, rows, count * 4, cudaMemcpyDeviceToDevice, cs));
  MSB_GUARD_END
}

int msb_run_index_i32(int32_t *run_of, int32_t *run_keys, uint32_t *total, const int32_t *sorted, int64_t n,
                      msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(total, MSB_ERR_ARGUMENT, "null pointer");
  MSB_REQUIRE(n == 0 || (run_of && run_keys && sorted), MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  mshadow::cuda::RunIndexLaunch(run_of, run_keys, total, sorted, n, Stream<gpu>::GetStream(st.get()));
  MSB_GUARD_END
}

int msb_run_bounds_i32(int32_t *first, const int32_t *run_keys, const uint32_t *total, int world, int64_t per_owner,
                       msb_stream_t stream) {
  MSB_REQUIRE(world >= 1 && world <= mshadow::cuda::routedetail::kMaxOwners, MSB_ERR_ARGUMENT, "1 to 16 owners");
  MSB_REQUIRE(FitsIndex(per_owner) && per_owner >= 1 && FitsIndex(per_owner * world), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(first && run_keys && total, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  mshadow::cuda::RunBoundsLaunch(first, run_keys, total, world, static_cast<int32_t>(per_owner),
                                 Stream<gpu>::GetStream(st.get()));
  MSB_GUARD_END
}

int msb_run_keys_to_owners_i32(int32_t *const *key_blocks, const int32_t *first, const int32_t *run_keys, int64_t n,
                               int world, int64_t per_owner, msb_stream_t stream) {
  MSB_REQUIRE(world >= 1 && world <= mshadow::cuda::routedetail::kMaxOwners, MSB_ERR_ARGUMENT, "1 to 16 owners");
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(per_owner) && per_owner >= 1, MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(key_blocks && first && run_keys, MSB_ERR_ARGUMENT, "null pointer");
  mshadow::cuda::routedetail::OwnerBlocks<int32_t> to;
  for (int q = 0; q < mshadow::cuda::routedetail::kMaxOwners; ++q) to.base[q] = q < world ? key_blocks[q] : nullptr;
  for (int q = 0; q < world; ++q) MSB_REQUIRE(to.base[q] != nullptr, MSB_ERR_ARGUMENT, "null block");
  to.first = first;
  to.world = world;
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  mshadow::cuda::RunKeysToOwnersLaunch(to, run_keys, n, static_cast<int32_t>(per_owner), Stream<gpu>::GetStream(st.get()));
  MSB_GUARD_END
}

int msb_take_sum_to_owners_f32_i32(float *const *row_blocks, const int32_t *first, const int32_t *run_of,
                                   const int32_t *index, const float *src, int64_t d, int64_t nidx, int world,
                                   msb_stream_t stream) {
  MSB_REQUIRE(world >= 1 && world <= mshadow::cuda::routedetail::kMaxOwners, MSB_ERR_ARGUMENT, "1 to 16 owners");
  MSB_REQUIRE(FitsIndex(d) && FitsIndex(nidx), MSB_ERR_SHAPE, "extent out of range");
  if (nidx == 0 || d == 0) return MSB_OK;
  MSB_REQUIRE(row_blocks && first && run_of && index && src, MSB_ERR_ARGUMENT, "null pointer");
  mshadow::cuda::routedetail::RowRoute route;
  for (int q = 0; q < mshadow::cuda::routedetail::kMaxOwners; ++q) route.base[q] = q < world ? row_blocks[q] : nullptr;
  for (int q = 0; q < world; ++q) {
    MSB_REQUIRE(route.base[q] != nullptr, MSB_ERR_ARGUMENT, "null block");
    MSB_REQUIRE(reinterpret_cast<uintptr_t>(route.base[q]) % 16 == 0, MSB_ERR_ARGUMENT, "blocks must be 16-byte aligned");
  }
  route.first = first;
  route.world = world;
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  mshadow::cuda::AddTakeGradLargeBatchLaunch(nullptr, d, run_of, index, src, d, nidx, d, Stream<gpu>::GetStream(st.get()),
                                             true, &route);
  MSB_GUARD_END
}

int msb_route_cyclic_hot_i32(int32_t *keys_out, int32_t *rows_out, uint32_t *totals, const int32_t *sorted,
                             const int32_t *index, int64_t n, const int32_t *hot, int64_t hot_count, int world,
                             int rank, int64_t src_begin, int64_t src_end, int64_t hot_base, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n) && FitsIndex(src_begin) && FitsIndex(src_end) && FitsIndex(hot_base) && hot_count >= 0 &&
                  hot_count <= mshadow::cuda::routedetail::kMaxHot,
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(world >= 1 && rank >= 0 && rank < world, MSB_ERR_ARGUMENT, "rank outside the group");
  MSB_REQUIRE(totals, MSB_ERR_ARGUMENT, "null pointer");
  MSB_REQUIRE(n == 0 || (keys_out && rows_out && sorted && index), MSB_ERR_ARGUMENT, "null pointer");
  MSB_REQUIRE(hot_count == 0 || hot, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  mshadow::cuda::RouteCyclicHotLaunch(keys_out, rows_out, totals, sorted, index, n, hot, static_cast<int>(hot_count),
                                      world, rank, static_cast<int32_t>(src_begin), static_cast<int32_t>(src_end),
                                      static_cast<int32_t>(hot_base), Stream<gpu>::GetStream(st.get()));
  MSB_GUARD_END
}

int msb_softmax3d_f32(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos, int64_t ld_dst,
                      int64_t ld_src, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(batch) && FitsIndex(classes) && FitsIndex(npos) && FitsIndex(batch * classes) &&
                  FitsIndex(batch * classes * npos) && LdOk(ld_dst, npos) && LdOk(ld_src, npos),
              MSB_ERR_SHAPE, "extent out of range");
  if (batch == 0 || classes == 0 || npos == 0) return MSB_OK;
  MSB_REQUIRE(dst && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  Tensor<gpu, 3, float> d(dst, Shape3(batch, classes, npos), static_cast<index_t>(ld_dst), st.get());
  const Tensor<gpu, 3, float> s(const_cast<float *>(src), Shape3(batch, classes, npos), static_cast<index_t>(ld_src),
                                st.get());
  Softmax(d, s);
  MSB_GUARD_END
}

int msb_softmax_grad3d_f32(float *dst, const float *src, const float *label, int64_t batch, int64_t classes,
                           int64_t npos, int64_t ld_dst, int64_t ld_src, int64_t ld_label, int mode,
                           float ignore_label, float alpha, msb_stream_t stream) {
  MSB_REQUIRE(mode >= 0 && mode <= 3, MSB_ERR_ARGUMENT, "mode must be 0..3");
  MSB_REQUIRE(FitsIndex(batch) && FitsIndex(classes) && FitsIndex(npos) && FitsIndex(batch * classes) &&
                  FitsIndex(batch * classes * npos) && LdOk(ld_dst, npos) && LdOk(ld_src, npos) && LdOk(ld_label, npos),
              MSB_ERR_SHAPE, "extent out of range");
  if (batch == 0 || classes == 0 || npos == 0) return MSB_OK;
  MSB_REQUIRE(dst && src && label, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const Tensor<gpu, 3, float> d(dst, Shape3(batch, classes, npos), static_cast<index_t>(ld_dst), st.get());
  const Tensor<gpu, 3, float> s(const_cast<float *>(src), Shape3(batch, classes, npos), static_cast<index_t>(ld_src),
                                st.get());
  const G2 l = Mat(label, batch, npos, ld_label, st.get());
  switch (mode) {
    case 0: SoftmaxGrad(d, s, l); break;
    case 1: SmoothSoftmaxGrad(d, s, l, alpha); break;
    case 2: SoftmaxGrad(d, s, l, ignore_label); break;
    default: SmoothSoftmaxGrad(d, s, l, ignore_label, alpha); break;
  }
  MSB_GUARD_END
}

int msb_index_fill_f32_i32(float *dst, const int32_t *index, const float *src, int64_t k, int64_t d, int64_t nidx,
                           msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(k) && FitsIndex(d) && FitsIndex(nidx) && FitsIndex(k * d) && FitsIndex(nidx * d),
              MSB_ERR_SHAPE, "extent out of range");
  if (nidx == 0 || d == 0 || k == 0) return MSB_OK;
  MSB_REQUIRE(dst && index && src, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const Tensor<gpu, 1, int32_t> idx(const_cast<int32_t *>(index), Shape1(nidx), nidx, st.get());
  IndexFill(Mat(dst, k, d, d, st.get()), idx, Mat(src, nidx, d, d, st.get()));
  MSB_GUARD_END
}

namespace {
typedef Tensor<gpu, 4, float> G4;
inline G4 Img(const float *p, int64_t n, int64_t c, int64_t h, int64_t w, Stream<gpu> *s) {
  return G4(const_cast<float *>(p), Shape4(n, c, h, w), static_cast<index_t>(w), s);
}
/*! \brief result shape of an index-remapping case, from the expression objects themselves */
inline Shape<4> RemapShape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1) {
  const G4 a = Img(nullptr, n, c, h, w, nullptr);
  switch (id) {
    case 0: return reshape(a, Shape4(n, h, c, w)).shape_;
    case 1: return slice<1>(a, p0, p1).shape_;
    case 2: return slice<3>(a, p0, p1).shape_;
    case 3: return concat<1>(a, a).shape_;
    case 4: return concat<3>(a, a).shape_;
    case 5: return swapaxis<2, 1>(a).shape_;
    case 6: return swapaxis<3, 1>(a).shape_;
    case 7: return transpose(a, Shape4(0, 2, 1, 3)).shape_;
    case 8: return transpose(a, Shape4(3, 1, 0, 2)).shape_;
    case 9: return pad(a, p0, p1).shape_;
    case 10: return crop(a, Shape2(p0, p1)).shape_;
    case 11: return crop(a, Shape2(p0, p1), h - p0, w - p1).shape_;
    case 15: return Shape4(2 * n, c, h, w);
    default: return a.shape_;
  }
}
inline bool RemapArgsOk(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1) {
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || p0 < 0 || p1 < 0) return false;
  if (!FitsIndex(n * c) || !FitsIndex(n * c * h) || !FitsIndex(2 * n * c * h * w)) return false;
  if (id == 9 || id == 16) return FitsIndex(n * c * (h + 2 * p0) * (w + 2 * p1));
  return true;
}
}  // namespace

int msb_remap_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t *out_shape) {
  MSB_REQUIRE(id >= 0 && id <= 16, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(RemapArgsOk(id, n, c, h, w, p0, p1), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(out_shape != nullptr, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  const Shape<4> s = RemapShape(id, n, c, h, w, p0, p1);
  for (int i = 0; i < 4; ++i) out_shape[i] = s[i];
  MSB_GUARD_END
}

int msb_remap_case_f32(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c, int64_t h, int64_t w,
                       int64_t p0, int64_t p1, msb_stream_t stream) {
  MSB_REQUIRE(id >= 0 && id <= 16, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(RemapArgsOk(id, n, c, h, w, p0, p1), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(dst && A && B, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const Shape<4> o = RemapShape(id, n, c, h, w, p0, p1);
  const G4 a = Img(A, n, c, h, w, st.get()), b = Img(B, n, c, h, w, st.get());
  G4 d = Img(dst, o[0], o[1], o[2], o[3], st.get());
  switch (id) {
    case 0: d = reshape(a, Shape4(n, h, c, w)); break;
    case 1: d = slice<1>(a, p0, p1); break;
    case 2: d = slice<3>(a, p0, p1); break;
    case 3: d = concat<1>(a, b); break;
    case 4: d = concat<3>(a, b); break;
    case 5: d = swapaxis<2, 1>(a); break;
    case 6: d = swapaxis<3, 1>(a); break;
    case 7: d = transpose(a, Shape4(0, 2, 1, 3)); break;
    case 8: d = transpose(a, Shape4(3, 1, 0, 2)); break;
    case 9: d = pad(a, p0, p1); break;
    case 10: d = crop(a, Shape2(p0, p1)); break;
    case 11: d = crop(a, Shape2(p0, p1), h - p0, w - p1); break;
    case 12: d = mirror(a); break;
    case 13: d = flip(a, 1); break;
    case 14:
      Copy(d, b, st.get());
      slice<1>(d, p0, p1) = slice<1>(a, p0, p1) + 1.0f;
      break;
    case 15: {
      G4 d1 = Img(dst, n, c, h, w, st.get()), d2 = Img(dst + n * c * h * w, n, c, h, w, st.get());
      concat<1>(d1, d2) = F<op::identity>(concat<1>(b, a));
    } break;
    default: d = crop(pad(a, p0, p1), Shape2(h, w)) + mirror(a); break;
  }
  MSB_GUARD_END
}

int msb_select_case_f32(int id, float *dst, const float *A, const float *B, const float *idx_r, const float *idx_c,
                        int64_t rows, int64_t cols, int64_t p0, msb_stream_t stream) {
  MSB_REQUIRE(id >= 0 && id <= 7, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(rows > 0 && cols > 0 && FitsIndex(rows) && FitsIndex(cols) && FitsIndex(rows * cols) && p0 >= 1 &&
                  (id != 5 || FitsIndex(rows * cols * p0 * p0)),
              MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(dst && A && B && idx_r && idx_c, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const G2 a = Mat(A, rows, cols, cols, st.get()), b = Mat(B, rows, cols, cols, st.get());
  const G1 ir = Vec(idx_r, rows, st.get()), ic = Vec(idx_c, rows, st.get()), val = Vec(B, rows, st.get());
  G2 d = Mat(dst, rows, cols, cols, st.get());
  switch (id) {
    case 0: d = take(ir, a); break;
    case 1: d = one_hot_encode(ic, cols); break;
    case 2: {
      G1 d1 = Vec(dst, rows, st.get());
      d1 = mat_choose_row_element(a, ic);
    } break;
    case 3: d = mat_fill_row_element(a, val, ic); break;
    case 4: d = mask(ic, a); break;
    case 5: {
      G2 up = Mat(dst, rows * p0, cols * p0, cols * p0, st.get());
      up = upsampling_nearest(a, p0);
    } break;
    case 6: d = take_grad(ir, a, rows); break;
    default: d = take(ir, a) * b + one_hot_encode(ic, cols); break;
  }
  MSB_GUARD_END
}

namespace {
inline bool PatchArgsOk(int64_t n, int64_t c, int64_t h, int64_t w, int psy, int psx, int sy, int sx, int dy, int dx) {
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || psy <= 0 || psx <= 0 || sy <= 0 || sx <= 0 || dy <= 0 || dx <= 0) return false;
  if (!FitsIndex(n * c) || !FitsIndex(n * c * h) || !FitsIndex(n * c * h * w)) return false;
  if (dy * (psy - 1) + 1 > h || dx * (psx - 1) + 1 > w) return false;
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  return FitsIndex(static_cast<int64_t>(psy) * psx * c) && FitsIndex(oh * ow * n) &&
         FitsIndex(static_cast<int64_t>(psy) * psx * c * oh * ow * n);
}
}  // namespace

int msb_unpack_patch2col_f32(float *mat, const float *img, int64_t n, int64_t c, int64_t h, int64_t w, int psy, int psx,
                             int sy, int sx, int dy, int dx, msb_stream_t stream) {
  MSB_REQUIRE(PatchArgsOk(n, c, h, w, psy, psx, sy, sx, dy, dx), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(mat && img, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  G2 m = Mat(mat, static_cast<int64_t>(psy) * psx * c, oh * ow * n, oh * ow * n, st.get());
  m = unpack_patch2col(Img(img, n, c, h, w, st.get()), psy, psx, sy, sx, dy, dx);
  MSB_GUARD_END
}

int msb_pack_col2patch_f32(float *img, const float *mat, int64_t n, int64_t c, int64_t h, int64_t w, int psy, int psx,
                           int sy, int sx, int dy, int dx, msb_stream_t stream) {
  MSB_REQUIRE(PatchArgsOk(n, c, h, w, psy, psx, sy, sx, dy, dx), MSB_ERR_SHAPE, "extent out of range");
  MSB_REQUIRE(mat && img, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  G4 d = Img(img, n, c, h, w, st.get());
  d = pack_col2patch(Mat(mat, static_cast<int64_t>(psy) * psx * c, oh * ow * n, oh * ow * n, st.get()), d.shape_, psy,
                     psx, sy, sx, dy, dx);
  MSB_GUARD_END
}

int msb_axis_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t *out_shape,
                   int *out_ndim) {
  MSB_REQUIRE(id >= 0 && id < msb_axis::kNumCases, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(msb_axis::ArgsOk(id, n, c, h, w, p0, p1), MSB_ERR_SHAPE, "extent or parameter out of range");
  MSB_REQUIRE(out_shape != nullptr && out_ndim != nullptr, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  *out_ndim = msb_axis::ResultShape<gpu>(id, n, c, h, w, p0, p1, out_shape);
  MSB_GUARD_END
}

int msb_axis_case_f32(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0,
                      int64_t p1, msb_stream_t stream) {
  MSB_REQUIRE(id >= 0 && id < msb_axis::kNumCases, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(msb_axis::ArgsOk(id, n, c, h, w, p0, p1), MSB_ERR_SHAPE, "extent or parameter out of range");
  MSB_REQUIRE(dst && (A || id < 2), MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  msb_axis::Run<gpu>(id, dst, A, n, c, h, w, p0, p1, st.get());
  MSB_GUARD_END
}

int msb_complex_case_f32(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols,
                         msb_stream_t stream) {
  MSB_REQUIRE(id >= 0 && id < msb_complex::kNumCases, MSB_ERR_ARGUMENT, "unknown expression id");
  MSB_REQUIRE(msb_complex::ArgsOk(id, rows, cols), MSB_ERR_SHAPE, "extent out of range (cols must be a multiple of 4)");
  MSB_REQUIRE(dst && A && B, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  msb_complex::Run<gpu>(id, dst, A, B, rows, cols, st.get());
  MSB_GUARD_END
}

int msb_vectorized_sort_f32_i32(float *values, int32_t *segments, int64_t n, msb_stream_t stream) {
  MSB_REQUIRE(FitsIndex(n), MSB_ERR_SHAPE, "extent out of range");
  if (n == 0) return MSB_OK;
  MSB_REQUIRE(values && segments, MSB_ERR_ARGUMENT, "null pointer");
  MSB_GUARD_BEGIN
  BorrowedStream st(stream);
  Tensor<gpu, 1, float> v(values, Shape1(n), n, st.get());
  Tensor<gpu, 1, int32_t> s(segments, Shape1(n), n, st.get());
  VectorizedSort(v, s);
  MSB_GUARD_END
}

}  // extern "C"
