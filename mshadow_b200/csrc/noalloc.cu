/*
 * Column sum without any allocation.
 *
 * msb_reduce_keep_lowest_f32() splits the rows of its input over many thread-block clusters
 * and parks one partial row per cluster in a scratch matrix, which the library normally
 * takes from a cudaMalloc'ed, per-stream cache.  Some callers must not trigger an
 * allocation at the moment they call us: code that runs while a memory pool is frozen,
 * inside another framework's "no allocation" region, on a real-time path where cudaMalloc's
 * implicit device synchronisation is unacceptable, or in a process whose device memory was
 * handed out up front and where a late cudaMalloc would simply fail.  For them this file
 * offers one entry point, msb_reduce_keep_lowest_sum_f32_noalloc(), whose scratch matrix is
 * a fixed array in the library's device image.
 *
 * What callers need to know:
 *   - the array holds kNoAllocScratchFloats floats (1 MiB).  Every GPU that loads the
 *     library carries it from load to exit, used or not.  A call whose partial rows would
 *     not fit (clusters x columns floats; on a 148-SM B200 that takes an input more than a
 *     hundred thousand columns wide) is rejected with MSB_ERR_SHAPE before anything is
 *     launched.
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) and the SM count.  That first call is a set-up call: make it
 *     before starting any stream capture.  Later calls only launch kernels.
 *   - all calls share the one array, also across streams.  Nothing in it has to start at
 *     zero (each launch overwrites exactly the rows it later reads), so stale contents are
 *     harmless, but two calls that execute on the GPU at the same time overwrite each
 *     other's partial rows.  Serialise them: one stream, or events between streams.
 *   - no cudaMalloc, cudaFree or other allocating routine is called, on the host or for
 *     the device; inputs and outputs are the caller's.
 * The arithmetic, launch geometry and result are those of msb_reduce_keep_lowest_f32 with
 * saver 0 (assign) and reducer 0 (sum).
 */
#include "mshadow_b200.h"

#include <mutex>
#include <string>

#include "mshadow/tensor.h"

namespace msb_internal {
void SetLastError(const char *message);  // defined next to msb_last_error()
}

namespace {

const size_t kNoAllocScratchFloats = size_t(1) << 18;  // 1 MiB
const int kMaxDevices = 64;

// In host code this name is only a handle for the runtime's symbol table, never a device
// address: kernels receive the pointer that cudaGetSymbolAddress returns for it.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

struct PerDevice {
  bool ready;
  float *scratch;
  uint32_t slots_vec;     // resident CTAs of the 128-bit kernel on this device
  uint32_t slots_scalar;  // ... and of the element-at-a-time kernel
};

typedef mshadow::expr::Plan<mshadow::Tensor<mshadow::gpu, 1, float>, float> DPlan;
typedef mshadow::expr::Plan<mshadow::Tensor<mshadow::gpu, 2, float>, float> SPlan;
#define MSB_NOALLOC_KERNEL(LANES) \
  mshadow::cuda::ReduceKeepLowestKernel<mshadow::sv::saveto, mshadow::red::sum, LANES, float, DPlan, SPlan>
PerDevice g_dev[kMaxDevices];
std::mutex g_dev_mutex;

int FailNoAlloc(int code, const char *msg) {
  char text[256];
  snprintf(text, sizeof(text), "msb_reduce_keep_lowest_sum_f32_noalloc: %s", msg);
  msb_internal::SetLastError(text);  // read back through msb_last_error()
  return code;
}

/*! \brief once per device, with that device current: resolve the scratch array and the SM count */
int SetUpDevice(int dev, PerDevice *out) {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_dev[dev].ready) {
    float *ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_scratch);
    if (err != cudaSuccess || ptr == nullptr) return FailNoAlloc(MSB_ERR_CUDA, cudaGetErrorString(err));
    int sms = 0, per_sm_vec = 0, per_sm_scalar = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess || sms <= 0) return FailNoAlloc(MSB_ERR_CUDA, cudaGetErrorString(err));
    // the same occupancy figures the allocating entry point plans its grid with
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_vec, MSB_NOALLOC_KERNEL(4),
                                                        mshadow::cuda::kRedLowThreads, 0);
    if (err == cudaSuccess)
      err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_scalar, MSB_NOALLOC_KERNEL(1),
                                                          mshadow::cuda::kRedLowThreads, 0);
    if (err != cudaSuccess) return FailNoAlloc(MSB_ERR_CUDA, cudaGetErrorString(err));
    g_dev[dev].scratch = ptr;
    g_dev[dev].slots_vec = static_cast<uint32_t>(per_sm_vec < 1 ? 1 : per_sm_vec) * sms;
    g_dev[dev].slots_scalar = static_cast<uint32_t>(per_sm_scalar < 1 ? 1 : per_sm_scalar) * sms;
    g_dev[dev].ready = true;
  }
  *out = g_dev[dev];
  return MSB_OK;
}

}  // namespace

extern "C" int msb_reduce_keep_lowest_sum_f32_noalloc(float *dst, const float *src, int64_t rows, int64_t cols,
                                                       int64_t ld, float scale, msb_stream_t stream) {
  using namespace mshadow;  // NOLINT(*)
  if (rows <= 0) return FailNoAlloc(MSB_ERR_SHAPE, "can not reduce over empty tensor");
  if (cols < 0 || ld < cols || ld > 0x7fffffffLL || rows > 0x7fffffffLL || cols > 0x7fffffffLL ||
      rows * cols > 0x7fffffffLL)
    return FailNoAlloc(MSB_ERR_SHAPE, "extent out of range");
  if (cols == 0) return MSB_OK;
  if (dst == nullptr || src == nullptr) return FailNoAlloc(MSB_ERR_ARGUMENT, "null pointer");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FailNoAlloc(MSB_ERR_CUDA, "no current CUDA device");
  if (dev < 0 || dev >= kMaxDevices) return FailNoAlloc(MSB_ERR_ARGUMENT, "device ordinal beyond 63");
  PerDevice pd;
  const int rc = SetUpDevice(dev, &pd);
  if (rc != MSB_OK) return rc;

  // Nothing below may leave through the C boundary as an exception: the planning helper and the
  // plan constructors CHECK their arguments, and a failed CHECK throws in this build.
  try {
  // same 128-bit eligibility rule and the same split as the allocating entry point
  const bool vec = cols % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && (rows == 1 || ld % 4 == 0);
  const int lanes = vec ? 4 : 1;
  const uint32_t col_tiles = static_cast<uint32_t>((cols + mshadow::cuda::kRedLowThreads * lanes - 1) /
                                                   (mshadow::cuda::kRedLowThreads * lanes));
  const mshadow::cuda::reddetail::Split sp = mshadow::cuda::reddetail::PlanKeepLowest(
      static_cast<uint32_t>(rows), col_tiles, vec ? pd.slots_vec : pd.slots_scalar);
  float *partial = nullptr;
  if (sp.clusters > 1) {
    if (static_cast<size_t>(sp.clusters) * static_cast<size_t>(cols) > kNoAllocScratchFloats)
      return FailNoAlloc(MSB_ERR_SHAPE, "input needs more than the 1 MiB built-in scratch; use msb_reduce_keep_lowest_f32");
    partial = pd.scratch;
  }
  Stream<gpu> st;
  st.stream_ = static_cast<cudaStream_t>(stream);
  const Tensor<gpu, 1, float> d(dst, Shape1(cols), static_cast<index_t>(cols), &st);
  const Tensor<gpu, 2, float> s(const_cast<float *>(src), Shape2(rows, cols), static_cast<index_t>(ld), &st);
  const DPlan dplan = expr::MakePlan(d);
  const SPlan splan = expr::MakePlan(s);
  const dim3 grid(col_tiles, sp.chunks), block(mshadow::cuda::kRedLowThreads);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st.stream_;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = sp.cluster;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const uint32_t urows = static_cast<uint32_t>(rows), ucols = static_cast<uint32_t>(cols);
  const gpu_rt::PeerSink no_sink;  // results stay on this GPU
  cudaError_t err;
  if (vec) {
    err = cudaLaunchKernelEx(&cfg, MSB_NOALLOC_KERNEL(4), dplan, splan, urows, ucols, sp.per_chunk, scale, partial,
                             no_sink);
  } else {
    err = cudaLaunchKernelEx(&cfg, MSB_NOALLOC_KERNEL(1), dplan, splan, urows, ucols, sp.per_chunk, scale, partial,
                             no_sink);
  }
  if (err != cudaSuccess) return FailNoAlloc(MSB_ERR_CUDA, cudaGetErrorString(err));
  gpu_rt::LaunchCounter().fetch_add(1, std::memory_order_relaxed);
  if (partial != nullptr) {
    mshadow::cuda::ReduceFinishKernel<sv::saveto, red::sum, float, DPlan>
        <<<(ucols + 255) / 256, 256, 0, st.stream_>>>(dplan, partial, sp.clusters, ucols, scale, no_sink);
    err = cudaPeekAtLastError();
    if (err != cudaSuccess) return FailNoAlloc(MSB_ERR_CUDA, cudaGetErrorString(err));
    gpu_rt::LaunchCounter().fetch_add(1, std::memory_order_relaxed);
  }
  } catch (const std::exception &e) {
    return FailNoAlloc(MSB_ERR_SHAPE, e.what());
  }
  return MSB_OK;
}
