/*
 * Local response normalisation across channels, forward and backward, each as ONE pass.
 *
 * With dmlc/mshadow an LRN layer is written as expressions around the channel pooling of
 * mshadow/extension/channel_pool.h:77-104 (and, for the gradient of that pooling,
 * channel_unpool.h:102-133, which for red::sum is the same window sum applied to the incoming
 * gradient):
 *
 *   norm = chpool<red::sum>(F<square>(src), nsize) * salpha + knorm;
 *   out  = src * F<power>(norm, -beta);
 *
 *   gsrc  = gout * F<power>(norm, -beta);
 *   gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<power>(norm, -beta - 1.0f), nsize) * src;
 *
 * Through the generic evaluator each chpool output walks its window in global memory, and the
 * statements are separate sweeps: 20 and 36 bytes of traffic per element.  Here a thread
 * marches over the channels of its four pixels with the window in registers while a producer
 * thread streams the channel planes through a shared-memory ring by bulk asynchronous copies
 * (the scheme of ChannelPoolStagedKernel in pool.cuh, same full / empty barrier pairs per slot),
 * and applies the surrounding arithmetic on the way: 8 bytes per element forward (12 when `norm`
 * is kept for the backward pass), 16 backward.
 *
 * Every product and sum is rounded on its own and taken in the order in which the expressions
 * above evaluate (window sums in ascending channel order from zero), so with a `Power` functor
 * whose arithmetic is the same on both sides the result equals the CPU evaluation of the
 * expressions bit for bit.  `Power` is user code, as `square` and `power` are in a layer written
 * against the reference: any struct with  static float Map(float base, float exponent).
 */
#ifndef MSHADOW_GPU_LRN_CUH_
#define MSHADOW_GPU_LRN_CUH_

#include "./runtime.h"
#include "./tma.cuh"

namespace mshadow {
namespace cuda {

namespace lrndetail {
const uint32_t kMaxRing = 16;
// pixels per tile: 31 consumer warps of 128 pixels and the producer warp make a 1024-thread CTA
// (measured on (256,256,56,56): whole planes of 3136 pixels 0.61 ms forward, half planes 0.78 ms)
const uint32_t kMaxTilePx = MSHADOW_B200_LRN_TILE_PX;
const int kMaxThreads = kMaxTilePx / 4 + 32;

/*! \brief what both kernels share: the CTA's tile, its channel segment and the slot barriers */
struct Geometry {
  uint32_t channels, plane, tile_px, tiles_per_plane, seg_len, ring;
};
}  // namespace lrndetail

/*!
 * \brief forward.  CTA = (image, pixel tile) x channel segment; warps 0 .. n-2 consume, four
 *  adjacent pixels per thread, the last warp produces.  Dynamic shared memory: ring * tile_px floats.
 *  `norm` may be null.
 */
template <typename Power, int NSIZE>
__global__ void __launch_bounds__(lrndetail::kMaxThreads, 1)
LrnForwardKernel(float *dst, float *norm, const float *src, lrndetail::Geometry g, float salpha, float beta,
                 float knorm, int *status) {
  constexpr int kPad = NSIZE / 2;
  extern __shared__ __align__(16) float slots[];
  __shared__ uint64_t full[lrndetail::kMaxRing], empty[lrndetail::kMaxRing];
  const uint32_t image_idx = blockIdx.x / g.tiles_per_plane;
  const uint32_t px0 = (blockIdx.x - image_idx * g.tiles_per_plane) * g.tile_px;
  const uint32_t len = min(g.tile_px, g.plane - px0);
  const uint32_t c_begin = blockIdx.y * g.seg_len;
  const uint32_t c_end = min(g.channels, c_begin + g.seg_len);
  const int64_t base = static_cast<int64_t>(image_idx) * g.channels * g.plane + px0;
  const uint32_t nsteps = (c_end - c_begin) + 2 * kPad;
  const uint32_t consumer_warps = (blockDim.x >> 5) - 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (uint32_t j = 0; j < g.ring; ++j) {
      tma::BarrierInit(&full[j], 1);
      tma::BarrierInit(&empty[j], consumer_warps);
    }
  }
  __syncthreads();
  if (warp == consumer_warps) {
    if (lane != 0) return;
    uint32_t slot = 0, use = 0;  // counted, not s % ring and s / ring: no divisions in the march
    for (uint32_t s = 0; s < nsteps; ++s) {
      if (use > 0 && !tma::WaitBounded(&empty[slot], (use - 1) & 1u)) {
        atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      const int64_t ch = static_cast<int64_t>(c_begin) - kPad + s;
      if (ch >= 0 && ch < static_cast<int64_t>(g.channels)) {
        tma::BarrierExpect(&full[slot], len * 4u);
        tma::BulkLoad(slots + static_cast<size_t>(slot) * g.tile_px, src + base + ch * g.plane, len * 4u, &full[slot]);
      } else {
        tma::BarrierArrive(&full[slot]);  // keeps the slot's turn: see ChannelPoolStagedKernel
      }
      if (++slot == g.ring) {
        slot = 0;
        ++use;
      }
    }
    return;
  }
  const bool mine = threadIdx.x * 4 < len;
  float win[NSIZE][4];
#pragma unroll
  for (int j = 0; j < NSIZE; ++j) win[j][0] = win[j][1] = win[j][2] = win[j][3] = 0.0f;
  const float neg_beta = -beta;
  uint32_t slot = 0, lap = 0;
  // 32-bit bookkeeping: the channel of a step as an unsigned number (one before the tensor wraps and
  // fails the one comparison), slot and output addresses advanced by additions
  uint32_t ch = c_begin - kPad;
  const float *my_slot = slots + threadIdx.x * 4;
  int64_t at = base + static_cast<int64_t>(c_begin) * g.plane + threadIdx.x * 4;
  for (uint32_t s0 = 0; s0 < nsteps; s0 += NSIZE) {
#pragma unroll
    for (int j = 0; j < NSIZE; ++j) {
      const uint32_t s = s0 + j;
      if (s < nsteps) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // a channel outside the tensor adds 0 * 0
        if (!tma::WaitBounded(&full[slot], lap & 1u)) {
          if (lane == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
          return;
        }
        if (ch < g.channels && mine) {
          v = *reinterpret_cast<const float4 *>(my_slot);
        }
        __syncwarp();
        if (lane == 0) tma::BarrierArrive(&empty[slot]);
        win[j][0] = v.x, win[j][1] = v.y, win[j][2] = v.z, win[j][3] = v.w;
        if (s >= 2 * kPad && mine) {
          // output channel ch - kPad: squares of the last NSIZE channels, oldest first, from zero
          float o[4], nrm[4];
#pragma unroll
          for (int l = 0; l < 4; ++l) {
            float sum = 0.0f;
#pragma unroll
            for (int t = 1; t <= NSIZE; ++t) {
              const float a = win[(j + t) % NSIZE][l];
              sum = __fadd_rn(sum, __fmul_rn(a, a));
            }
            nrm[l] = __fadd_rn(__fmul_rn(sum, salpha), knorm);
            o[l] = __fmul_rn(win[(j + 1 + kPad) % NSIZE][l], Power::Map(nrm[l], neg_beta));
          }
          __stcs(reinterpret_cast<float4 *>(dst + at), make_float4(o[0], o[1], o[2], o[3]));
          if (norm != nullptr) __stcs(reinterpret_cast<float4 *>(norm + at), make_float4(nrm[0], nrm[1], nrm[2], nrm[3]));
          at += g.plane;
        }
        ++ch;
        my_slot += g.tile_px;
        if (++slot == g.ring) {
          slot = 0;
          ++lap;
          my_slot = slots + threadIdx.x * 4;
        }
      }
    }
  }
}

/*!
 * \brief backward.  A slot holds the tile of three planes of one channel: incoming gradient,
 *  source and norm.  The window keeps t(c) = (gout * src) * power(norm, -beta - 1); the values of
 *  the centre channel are read again from its slot, which is therefore released NSIZE/2 steps
 *  after it was first read.  Dynamic shared memory: 3 * ring * tile_px floats.
 */
template <typename Power, int NSIZE>
__global__ void __launch_bounds__(lrndetail::kMaxThreads, 1)
LrnBackwardKernel(float *gsrc, const float *gout, const float *src, const float *norm, lrndetail::Geometry g,
                  float scale, float beta, int *status) {
  constexpr int kPad = NSIZE / 2;
  extern __shared__ __align__(16) float slots[];
  __shared__ uint64_t full[lrndetail::kMaxRing], empty[lrndetail::kMaxRing];
  const uint32_t image_idx = blockIdx.x / g.tiles_per_plane;
  const uint32_t px0 = (blockIdx.x - image_idx * g.tiles_per_plane) * g.tile_px;
  const uint32_t len = min(g.tile_px, g.plane - px0);
  const uint32_t c_begin = blockIdx.y * g.seg_len;
  const uint32_t c_end = min(g.channels, c_begin + g.seg_len);
  const int64_t base = static_cast<int64_t>(image_idx) * g.channels * g.plane + px0;
  const uint32_t nsteps = (c_end - c_begin) + 2 * kPad;
  const uint32_t consumer_warps = (blockDim.x >> 5) - 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t slot_floats = static_cast<size_t>(3) * g.tile_px;
  if (threadIdx.x == 0) {
    for (uint32_t j = 0; j < g.ring; ++j) {
      tma::BarrierInit(&full[j], 1);
      tma::BarrierInit(&empty[j], consumer_warps);
    }
  }
  __syncthreads();
  if (warp == consumer_warps) {
    if (lane != 0) return;
    uint32_t slot = 0, use = 0;
    for (uint32_t s = 0; s < nsteps; ++s) {
      if (use > 0 && !tma::WaitBounded(&empty[slot], (use - 1) & 1u)) {
        atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      const int64_t ch = static_cast<int64_t>(c_begin) - kPad + s;
      if (ch >= 0 && ch < static_cast<int64_t>(g.channels)) {
        float *at = slots + slot * slot_floats;
        const int64_t from = base + ch * g.plane;
        tma::BarrierExpect(&full[slot], 3u * len * 4u);
        tma::BulkLoad(at, gout + from, len * 4u, &full[slot]);
        tma::BulkLoad(at + g.tile_px, src + from, len * 4u, &full[slot]);
        tma::BulkLoad(at + 2 * g.tile_px, norm + from, len * 4u, &full[slot]);
      } else {
        tma::BarrierArrive(&full[slot]);
      }
      if (++slot == g.ring) {
        slot = 0;
        ++use;
      }
    }
    return;
  }
  const bool mine = threadIdx.x * 4 < len;
  float win[NSIZE][4];
#pragma unroll
  for (int j = 0; j < NSIZE; ++j) win[j][0] = win[j][1] = win[j][2] = win[j][3] = 0.0f;
  const float neg_beta = -beta, neg_beta_1 = -beta - 1.0f;
  uint32_t slot = 0, lap = 0;  // ring position of step s, and of step s - kPad (the centre channel's slot)
  uint32_t centre = 0;
  // 32-bit bookkeeping as in the forward kernel
  uint32_t ch = c_begin - kPad;
  const float *my_slot = slots + threadIdx.x * 4, *my_centre = my_slot;
  float *my_out = gsrc + base + static_cast<int64_t>(c_begin) * g.plane + threadIdx.x * 4;
  for (uint32_t s0 = 0; s0 < nsteps; s0 += NSIZE) {
#pragma unroll
    for (int j = 0; j < NSIZE; ++j) {
      const uint32_t s = s0 + j;
      if (s < nsteps) {
        if (!tma::WaitBounded(&full[slot], lap & 1u)) {
          if (lane == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
          return;
        }
        float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // a channel outside the tensor adds nothing
        if (ch < g.channels && mine) {
          const float *at = my_slot;
          const float4 gv = *reinterpret_cast<const float4 *>(at);
          const float4 xv = *reinterpret_cast<const float4 *>(at + g.tile_px);
          const float4 nv = *reinterpret_cast<const float4 *>(at + 2 * g.tile_px);
          t[0] = __fmul_rn(__fmul_rn(gv.x, xv.x), Power::Map(nv.x, neg_beta_1));
          t[1] = __fmul_rn(__fmul_rn(gv.y, xv.y), Power::Map(nv.y, neg_beta_1));
          t[2] = __fmul_rn(__fmul_rn(gv.z, xv.z), Power::Map(nv.z, neg_beta_1));
          t[3] = __fmul_rn(__fmul_rn(gv.w, xv.w), Power::Map(nv.w, neg_beta_1));
        }
        win[j][0] = t[0], win[j][1] = t[1], win[j][2] = t[2], win[j][3] = t[3];
        if (s >= 2 * kPad && mine) {
          // output channel ch - kPad; its own three values still sit in the slot of step s - kPad
          const float *at = my_centre;
          const float4 gv = *reinterpret_cast<const float4 *>(at);
          const float4 xv = *reinterpret_cast<const float4 *>(at + g.tile_px);
          const float4 nv = *reinterpret_cast<const float4 *>(at + 2 * g.tile_px);
          const float gc[4] = {gv.x, gv.y, gv.z, gv.w}, xc[4] = {xv.x, xv.y, xv.z, xv.w}, nc[4] = {nv.x, nv.y, nv.z, nv.w};
          float o[4];
#pragma unroll
          for (int l = 0; l < 4; ++l) {
            float sum = 0.0f;
#pragma unroll
            for (int u = 1; u <= NSIZE; ++u) sum = __fadd_rn(sum, win[(j + u) % NSIZE][l]);
            const float first = __fmul_rn(gc[l], Power::Map(nc[l], neg_beta));
            o[l] = __fadd_rn(first, __fmul_rn(__fmul_rn(scale, sum), xc[l]));
          }
          __stcs(reinterpret_cast<float4 *>(my_out), make_float4(o[0], o[1], o[2], o[3]));
          my_out += g.plane;
        }
        // the slot of step s - kPad has now been read for the last time
        __syncwarp();
        if (s >= static_cast<uint32_t>(kPad)) {
          if (lane == 0) tma::BarrierArrive(&empty[centre]);
          my_centre += slot_floats;
          if (++centre == g.ring) {
            centre = 0;
            my_centre = slots + threadIdx.x * 4;
          }
        }
        ++ch;
        my_slot += slot_floats;
        if (++slot == g.ring) {
          slot = 0;
          ++lap;
          my_slot = slots + threadIdx.x * 4;
        }
      }
    }
  }
}

namespace lrndetail {
/*! \brief window sizes the kernels are instantiated for, and the layout they need */
inline bool Supported(int nsize, int64_t c, int64_t plane, const void *a, const void *b, const void *d, const void *e) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                         reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(e);
  return (nsize == 3 || nsize == 5 || nsize == 7) && c >= 2 * nsize && plane % 4 == 0 && plane >= 4 && bits % 16 == 0;
}

/*! \brief tile, ring and channel segments; `planes_per_slot` is 1 (forward) or 3 (backward) */
template <typename Kernel>
inline Geometry Plan(Kernel kernel, int64_t n, int64_t c, int64_t plane, int nsize, uint32_t planes_per_slot,
                     uint32_t budget_bytes, uint32_t *threads, size_t *smem, dim3 *grid) {
  Geometry g;
  g.channels = static_cast<uint32_t>(c);
  g.plane = static_cast<uint32_t>(plane);
  g.tiles_per_plane = (g.plane + kMaxTilePx - 1) / kMaxTilePx;
  g.tile_px = ((g.plane + g.tiles_per_plane - 1) / g.tiles_per_plane + 3) & ~3u;
  *threads = (((g.tile_px / 4) + 31) & ~31u) + 32;
  const uint32_t slot_bytes = planes_per_slot * g.tile_px * 4;
  uint32_t ring = budget_bytes / slot_bytes;
  const uint32_t least = static_cast<uint32_t>(nsize) / 2 + 3;  // the backward kernel holds nsize/2 slots back
  if (ring < least) ring = least;
  if (ring > kMaxRing) ring = kMaxRing;
  g.ring = ring;
  *smem = static_cast<size_t>(ring) * slot_bytes;
  MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  int per_sm = 0;
  MSHADOW_CUDA_CALL(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, static_cast<int>(*threads), *smem));
  const uint32_t slots = static_cast<uint32_t>(per_sm < 1 ? 1 : per_sm) * gpu_rt::CurrentDevice().sm_count;
  const uint32_t fixed = static_cast<uint32_t>(n) * g.tiles_per_plane;
  // channel segments: whole waves of resident CTAs, weighed against the nsize-1 halo channels each re-reads
  uint32_t segs = 1;
  double best = 0.0;
  for (uint32_t k = 1; k <= 16 && k * 2 * nsize <= g.channels; ++k) {
    const uint64_t ctas = static_cast<uint64_t>(fixed) * k;
    const uint64_t waves = (ctas + slots - 1) / slots;
    const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots) /
                       (1.0 + static_cast<double>((nsize - 1) * k) / static_cast<double>(g.channels));
    if (eff > best + 1e-9) {
      best = eff;
      segs = k;
    }
  }
  g.seg_len = (g.channels + segs - 1) / segs;
  *grid = dim3(fixed, (g.channels + g.seg_len - 1) / g.seg_len);
  return g;
}
}  // namespace lrndetail

/*! \brief dense (n, c, h, w) tensors; requires lrndetail::Supported; `norm` may be null */
template <typename Power>
inline void LrnForwardLaunch(float *dst, float *norm, const float *src, int64_t n, int64_t c, int64_t plane, int nsize,
                             float salpha, float beta, float knorm, cudaStream_t stream) {
  if (n == 0 || c == 0 || plane == 0) return;
  CHECK_LT(n * ((plane + lrndetail::kMaxTilePx - 1) / lrndetail::kMaxTilePx), int64_t(1) << 31) << "LRNForward: too many tiles";
  uint32_t threads = 0;
  size_t smem = 0;
  dim3 grid;
#define MSHADOW_B200_LRN_FWD_(NS)                                                                                 \
  {                                                                                                               \
    auto kernel = LrnForwardKernel<Power, NS>;                                                                    \
    const lrndetail::Geometry g = lrndetail::Plan(kernel, n, c, plane, NS, 1, MSHADOW_B200_CHPOOL_RING_KB * 1024, \
                                                  &threads, &smem, &grid);                                       \
    kernel<<<grid, threads, smem, stream>>>(dst, norm, src, g, salpha, beta, knorm, gpu_rt::StatusWord());        \
  }
  if (nsize == 3) MSHADOW_B200_LRN_FWD_(3) else if (nsize == 5) MSHADOW_B200_LRN_FWD_(5) else MSHADOW_B200_LRN_FWD_(7)
#undef MSHADOW_B200_LRN_FWD_
  MSHADOW_CUDA_POST_KERNEL_CHECK(LrnForwardKernel);
}

/*! \brief dense (n, c, h, w) tensors; requires lrndetail::Supported */
template <typename Power>
inline void LrnBackwardLaunch(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n, int64_t c,
                              int64_t plane, int nsize, float salpha, float beta, cudaStream_t stream) {
  if (n == 0 || c == 0 || plane == 0) return;
  CHECK_LT(n * ((plane + lrndetail::kMaxTilePx - 1) / lrndetail::kMaxTilePx), int64_t(1) << 31) << "LRNBackward: too many tiles";
  uint32_t threads = 0;
  size_t smem = 0;
  dim3 grid;
  const float scale = -2.0f * beta * salpha;  // as the layer's expression computes it, in binary32
#define MSHADOW_B200_LRN_BWD_(NS)                                                                                 \
  {                                                                                                               \
    auto kernel = LrnBackwardKernel<Power, NS>;                                                                   \
    const lrndetail::Geometry g = lrndetail::Plan(kernel, n, c, plane, NS, 3, 190 * 1024, &threads, &smem, &grid); \
    kernel<<<grid, threads, smem, stream>>>(gsrc, gout, src, norm, g, scale, beta, gpu_rt::StatusWord());         \
  }
  if (nsize == 3) MSHADOW_B200_LRN_BWD_(3) else if (nsize == 5) MSHADOW_B200_LRN_BWD_(5) else MSHADOW_B200_LRN_BWD_(7)
#undef MSHADOW_B200_LRN_BWD_
  MSHADOW_CUDA_POST_KERNEL_CHECK(LrnBackwardKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_LRN_CUH_
