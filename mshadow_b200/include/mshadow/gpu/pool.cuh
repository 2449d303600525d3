/*
 * Dedicated kernels for the pooling expressions over plain tensors:
 *   PoolPlanes     out = pool<Reducer>(src, ky, kx, sy, sx)
 *   UnpoolPlanes   out = unpool<Reducer>(src, pooled, grad_pooled, ky, kx, sy, sx)
 *   ChannelPool    out = chpool<Reducer>(src, nsize)            (stride 1, pad nsize/2)
 * In the reference these have no kernels of their own: the window loop sits inside
 * Plan::Eval (mshadow/extension/spatial_pool.h:125-142, spatial_unpool.h:102-125,
 * channel_pool.h:85-99) and runs in the generic one-thread-per-output map kernel, so each
 * output re-reads its window from global memory with stride-2, 4-byte accesses.
 *
 * Spatial kernels: a CTA takes a group of consecutive image planes, brings them into shared
 * memory with one bulk asynchronous copy per operand (plain 128-bit loads when the group is
 * not 16-byte sized/aligned or rows are pitched), evaluates the windows out of shared
 * memory and writes the result coalesced.  HBM traffic is one read of every input and one
 * write of the output.
 *
 * Arithmetic is the reference's, operation for operation: windows are walked y-outer /
 * x-inner from Reducer::SetInitValue; unpool adds PartialGrad(src, pooled) * grad for the
 * covering windows in py-outer / px-inner order starting from zero, so tied maxima all
 * receive the gradient; chpool adds its channels in ascending order starting from zero.
 * Results are therefore bit-identical to the CPU evaluation.
 */
#ifndef MSHADOW_GPU_POOL_CUH_
#define MSHADOW_GPU_POOL_CUH_

#include "./runtime.h"
#include "./tma.cuh"

namespace mshadow {
namespace cuda {

const int kPoolThreads = 256;

/*! \brief window geometry; a template value of 0 means "read the run-time field" */
struct PoolGeom {
  int ky, kx, sy, sx;
};

namespace pooldetail {

/*! \brief floor(a / b) for b > 0, also for negative a */
__host__ __device__ constexpr int FloorDiv(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }

/*!
 * \brief bring `count` floats that start at `src` into shared memory.  Uses the bulk copy
 *  when the byte range is 16-byte aligned and sized, otherwise plain loads by all threads.
 *  Must be called by every thread of the CTA.  Returns false after a copy timeout.
 */
__device__ __forceinline__ bool StageDense(float *smem, const float *src, uint32_t count, uint64_t *bar,
                                           bool *used_bulk) {
  const bool bulk = (reinterpret_cast<uintptr_t>(src) % 16 == 0) && (count % 4 == 0);
  *used_bulk = bulk;
  if (bulk) {
    if (threadIdx.x == 0) {
      tma::BarrierExpect(bar, count * 4u);
      tma::BulkLoad(smem, src, count * 4u, bar);
    }
    return true;
  }
  for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) smem[i] = src[i];
  return true;
}

/*! \brief rows of `w` floats, `ld` apart in global memory, packed densely into shared memory */
__device__ __forceinline__ void StagePitched(float *smem, const float *src, uint32_t nrows, uint32_t w, int64_t ld) {
  const uint32_t count = nrows * w;
  for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
    const uint32_t r = i / w;
    smem[i] = src[r * ld + (i - r * w)];
  }
}

}  // namespace pooldetail

/*!
 * \brief spatial pooling of groups of `gplanes` planes.  Shared memory: gplanes*h*w floats.
 *  KY/KX/SY/SX > 0 fix the window at compile time.
 */
template <typename Reducer, int KY, int KX, int SY, int SX>
__global__ void __launch_bounds__(kPoolThreads)
PoolPlanesKernel(float *dst, const float *src, uint32_t planes, uint32_t h, uint32_t w, uint32_t ph, uint32_t pw,
                 PoolGeom g, int64_t ld_src, int64_t ld_dst, uint32_t gplanes, gpu_rt::FastDiv div_pw,
                 gpu_rt::FastDiv div_ph, gpu_rt::FastDiv div_pairs, int *status) {
  gpu_rt::GridDependencySync();
  extern __shared__ __align__(16) float tile[];
  __shared__ uint64_t bar;
  const int ky = KY > 0 ? KY : g.ky, kx = KX > 0 ? KX : g.kx;
  const int sy = SY > 0 ? SY : g.sy, sx = SX > 0 ? SX : g.sx;
  if (threadIdx.x == 0) tma::BarrierInit(&bar, 1);
  __syncthreads();
  uint32_t phase = 0;
  const bool dense_in = ld_src == static_cast<int64_t>(w);
  for (uint32_t first = blockIdx.x * gplanes; first < planes; first += gridDim.x * gplanes) {
    const uint32_t np = min(gplanes, planes - first);
    bool bulk = false;
    if (dense_in) {
      pooldetail::StageDense(tile, src + static_cast<int64_t>(first) * h * w, np * h * w, &bar, &bulk);
    } else {
      pooldetail::StagePitched(tile, src + static_cast<int64_t>(first) * h * ld_src, np * h, w, ld_src);
    }
    if (bulk) {
      if (!tma::WaitBounded(&bar, phase)) {
        if (threadIdx.x == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
        tma::WaitBounded(&bar, phase);
        return;
      }
      phase ^= 1;
    } else {
      __syncthreads();
    }
    const uint32_t nout = np * ph * pw;
    if ((KX == 3 || KX == 2) && SX == 2 && KY > 0 && MSHADOW_B200_POOL_PAIRS && (w & 3u) == 0) {
      // two adjacent outputs per thread: their windows span columns x0 .. x0+4 (x0+3 for 2-wide windows)
      // with x0 a multiple of four, so each window row is one 16-byte and at most one 4-byte
      // shared-memory load instead of six 4-byte loads, and the index split is paid once per pair: the
      // one-output loop below keeps the issue slots 70 % busy, i.e. it is bound by instructions.  (The
      // launcher only takes shapes in which no window is clipped.)  Values enter each output's
      // reduction in the same order as below.
      const uint32_t pairs_per_row = (pw + 1) >> 1;
      const uint32_t npairs = np * ph * pairs_per_row;
      for (uint32_t o = threadIdx.x; o < npairs; o += kPoolThreads) {
        const uint32_t row = div_pairs.Quot(o);
        const uint32_t px = (o - row * pairs_per_row) * 2;
        const uint32_t p = div_ph.Quot(row);
        const uint32_t py = row - p * ph;
        const float *at = tile + p * h * w + py * SY * w + px * 2;
        const bool second = px + 1 < pw;
        float r0, r1;
        Reducer::SetInitValue(r0);
        Reducer::SetInitValue(r1);
#pragma unroll
        for (int dy = 0; dy < (KY > 0 ? KY : 1); ++dy) {
          const float4 v = *reinterpret_cast<const float4 *>(at + dy * w);
          Reducer::Reduce(r0, v.x);
          Reducer::Reduce(r0, v.y);
          if (KX == 3) {
            const float e = second ? at[dy * w + 4] : 0.0f;
            Reducer::Reduce(r0, v.z);
            Reducer::Reduce(r1, v.z);
            Reducer::Reduce(r1, v.w);
            Reducer::Reduce(r1, e);
          } else {
            Reducer::Reduce(r1, v.z);
            Reducer::Reduce(r1, v.w);
          }
        }
        float *out = dst + (static_cast<int64_t>(first) * ph + row) * ld_dst + px;
        out[0] = r0;
        if (second) out[1] = r1;
      }
      tma::FenceAsyncShared();
      __syncthreads();
      continue;
    }
    for (uint32_t o = threadIdx.x; o < nout; o += kPoolThreads) {
      const uint32_t row = div_pw.Quot(o);  // plane-local output row index: p * ph + py
      const uint32_t px = o - row * pw;
      const uint32_t p = div_ph.Quot(row);
      const uint32_t py = row - p * ph;
      const uint32_t y0 = py * sy, x0 = px * sx;
      const uint32_t y1 = min(y0 + ky, h), x1 = min(x0 + kx, w);
      const float *plane = tile + p * h * w;
      float res;
      Reducer::SetInitValue(res);
      if (KY > 0 && y0 + KY <= h && x0 + KX <= w) {
#pragma unroll
        for (int dy = 0; dy < (KY > 0 ? KY : 1); ++dy)
#pragma unroll
          for (int dx = 0; dx < (KX > 0 ? KX : 1); ++dx) Reducer::Reduce(res, plane[(y0 + dy) * w + x0 + dx]);
      } else {
        for (uint32_t y = y0; y < y1; ++y)
          for (uint32_t x = x0; x < x1; ++x) Reducer::Reduce(res, plane[y * w + x]);
      }
      dst[(static_cast<int64_t>(first) * ph + row) * ld_dst + px] = res;
    }
    // all reads of the tile are done before the next group overwrites it
    tma::FenceAsyncShared();
    __syncthreads();
  }
}

/*!
 * \brief backward of spatial pooling for groups of `gplanes` planes.
 *  Shared memory: gplanes * (h*w + 2*ph*pw) floats (source, pooled, pooled gradient).
 */
template <typename Reducer, int KY, int KX, int SY, int SX>
__global__ void __launch_bounds__(kPoolThreads)
UnpoolPlanesKernel(float *dst, const float *src, const float *pooled, const float *gpooled, uint32_t planes,
                   uint32_t h, uint32_t w, uint32_t ph, uint32_t pw, PoolGeom g, int64_t ld_src, int64_t ld_pooled,
                   int64_t ld_dst, uint32_t gplanes, gpu_rt::FastDiv div_w, gpu_rt::FastDiv div_h,
                   gpu_rt::FastDiv div_sy, gpu_rt::FastDiv div_sx, gpu_rt::FastDiv div_wq, int *status) {
  gpu_rt::GridDependencySync();
  extern __shared__ __align__(16) float tile[];
  __shared__ uint64_t bar;
  const uint32_t ky = KY > 0 ? KY : g.ky, kx = KX > 0 ? KX : g.kx;
  const uint32_t sy = SY > 0 ? SY : g.sy, sx = SX > 0 ? SX : g.sx;
  // group sizes are padded to multiples of 4 floats so that every region starts 16-byte aligned
  const uint32_t src_cap = (gplanes * h * w + 3) & ~3u, pool_cap = (gplanes * ph * pw + 3) & ~3u;
  float *s_src = tile, *s_pool = tile + src_cap, *s_grad = s_pool + pool_cap;
  if (threadIdx.x == 0) tma::BarrierInit(&bar, 1);
  __syncthreads();
  uint32_t phase = 0;
  const bool dense = ld_src == static_cast<int64_t>(w) && ld_pooled == static_cast<int64_t>(pw);
  // the four-pixels-per-thread path needs a compile-time window, a stride dividing 4 and rows
  // that are whole groups of four
  constexpr bool kQuad = KY > 0 && KX > 0 && SY > 0 && SX > 0 && (4 % (SX > 0 ? SX : 1) == 0);
  const bool quad_ok = (w & 3u) == 0;
  const bool vec_out = (ld_dst & 3) == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  for (uint32_t first = blockIdx.x * gplanes; first < planes; first += gridDim.x * gplanes) {
    const uint32_t np = min(gplanes, planes - first);
    const uint32_t n_src = np * h * w, n_pool = np * ph * pw;
    const float *g_src = src + static_cast<int64_t>(first) * h * ld_src;
    const float *g_pool = pooled + static_cast<int64_t>(first) * ph * ld_pooled;
    const float *g_grad = gpooled + static_cast<int64_t>(first) * ph * ld_pooled;
    const bool bulk = dense && n_src % 4 == 0 && n_pool % 4 == 0 && reinterpret_cast<uintptr_t>(g_src) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(g_pool) % 16 == 0 && reinterpret_cast<uintptr_t>(g_grad) % 16 == 0;
    if (bulk) {
      if (threadIdx.x == 0) {
        tma::BarrierExpect(&bar, (n_src + 2 * n_pool) * 4u);
        tma::BulkLoad(s_src, g_src, n_src * 4u, &bar);
        tma::BulkLoad(s_pool, g_pool, n_pool * 4u, &bar);
        tma::BulkLoad(s_grad, g_grad, n_pool * 4u, &bar);
      }
      if (!tma::WaitBounded(&bar, phase)) {
        if (threadIdx.x == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
        tma::WaitBounded(&bar, phase);
        return;
      }
      phase ^= 1;
    } else {
      pooldetail::StagePitched(s_src, g_src, np * h, w, ld_src);
      pooldetail::StagePitched(s_pool, g_pool, np * ph, pw, ld_pooled);
      pooldetail::StagePitched(s_grad, g_grad, np * ph, pw, ld_pooled);
      __syncthreads();
    }
    if (kQuad && quad_ok) {
      // Four adjacent outputs per thread.  With the window fixed at compile time and a stride
      // that divides 4, which pooled columns cover which of the four pixels is a compile-time
      // pattern relative to the first candidate column pxb; only the image borders need
      // run-time checks.  Windows are visited row-major, as the reference does.
      constexpr int kSXs = SX > 0 ? SX : 1, kSYs = SY > 0 ? SY : 1;
      constexpr int kOff = pooldetail::FloorDiv(kSXs - KX, kSXs);
      constexpr int kCols = (3 / kSXs + 1) - kOff;
      constexpr int kRows = (KY - 1) / kSYs + 1;
      const uint32_t wq = w >> 2;
      const uint32_t nq = np * h * wq;
      for (uint32_t it = threadIdx.x; it < nq; it += kPoolThreads) {
        const uint32_t row = div_wq.Quot(it);  // p * h + y
        const uint32_t xq = it - row * wq;
        const uint32_t p = div_h.Quot(row);
        const uint32_t y = row - p * h;
        const float4 sv4 = *reinterpret_cast<const float4 *>(s_src + row * w + 4 * xq);
        const float sv[4] = {sv4.x, sv4.y, sv4.z, sv4.w};
        constexpr uint32_t kKYs = KY > 0 ? KY : 1;
        const int py_lo = y < kKYs ? 0 : static_cast<int>((y - kKYs + kSYs) / kSYs);
        const int py_hi = min(static_cast<int>((y + kSYs) / kSYs), static_cast<int>(ph));
        const int pxb = static_cast<int>(xq) * (4 / kSXs) + kOff;
        const float *pp = s_pool + p * ph * pw;
        const float *gp = s_grad + p * ph * pw;
        float val[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int py = py_lo + r;
          if (py < py_hi) {
#pragma unroll
            for (int cc = 0; cc < kCols; ++cc) {
              const int px = pxb + cc;
              if (px >= 0 && px < static_cast<int>(pw)) {
                const float pv = pp[py * pw + px];
                const float gv = gp[py * pw + px];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  // pixel 4*xq+i is covered by pooled columns [lo, hi) relative to pxb
                  const int lo = pooldetail::FloorDiv(i - KX + kSXs, kSXs) - kOff;
                  const int hi = i / kSXs + 1 - kOff;
                  if (cc >= lo && cc < hi) {
                    val[i] = __fadd_rn(val[i], __fmul_rn(Reducer::PartialGrad(sv[i], pv), gv));
                  }
                }
              }
            }
          }
        }
        float *out = dst + (static_cast<int64_t>(first) * h + row) * ld_dst + 4 * xq;
        if (vec_out) {
          __stcs(reinterpret_cast<float4 *>(out), make_float4(val[0], val[1], val[2], val[3]));
        } else {
          out[0] = val[0];
          out[1] = val[1];
          out[2] = val[2];
          out[3] = val[3];
        }
      }
    } else {
      for (uint32_t o = threadIdx.x; o < n_src; o += kPoolThreads) {
        const uint32_t row = div_w.Quot(o);  // p * h + y
        const uint32_t x = o - row * w;
        const uint32_t p = div_h.Quot(row);
        const uint32_t y = row - p * h;
        const float vsrc = s_src[o];
        const uint32_t py_min = y < ky ? 0 : (SY > 0 ? (y - ky + sy) / sy : div_sy.Quot(y - ky + sy));
        const uint32_t px_min = x < kx ? 0 : (SX > 0 ? (x - kx + sx) / sx : div_sx.Quot(x - kx + sx));
        const uint32_t py_max = min(SY > 0 ? (y + sy) / sy : div_sy.Quot(y + sy), ph);
        const uint32_t px_max = min(SX > 0 ? (x + sx) / sx : div_sx.Quot(x + sx), pw);
        const float *pp = s_pool + p * ph * pw;
        const float *gp = s_grad + p * ph * pw;
        float val = 0.0f;
        for (uint32_t py = py_min; py < py_max; ++py)
          for (uint32_t px = px_min; px < px_max; ++px) {
            const float pg = Reducer::PartialGrad(vsrc, pp[py * pw + px]);
            val = __fadd_rn(val, __fmul_rn(pg, gp[py * pw + px]));
          }
        dst[(static_cast<int64_t>(first) * h + row) * ld_dst + x] = val;
      }
    }
    tma::FenceAsyncShared();
    __syncthreads();
  }
}

namespace pooldetail {
/*!
 * \brief bring the `count` floats that start at `first` into shared memory at tile + *off.
 *  The bulk copy needs 16-byte aligned ends, so it fetches the 16-byte aligned window around the
 *  range and *off tells where the range starts inside it (0..3); that is only done when the
 *  window stays inside [lo_limit, hi_limit), the storage the caller vouches for.  Otherwise
 *  all threads copy with plain loads and *off is 0.  Returns whether a bulk copy was issued (the
 *  caller then waits on `bar`); `expect` accumulates the bytes announced to the barrier.
 */
__device__ __forceinline__ bool StageAround(float *tile, const float *first, uint32_t count, const float *lo_limit,
                                            const float *hi_limit, bool allow_bulk, uint64_t *bar, uint32_t *off) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(first);
  const uintptr_t lo = a & ~static_cast<uintptr_t>(15);
  const uintptr_t hi = (a + static_cast<uintptr_t>(count) * 4 + 15) & ~static_cast<uintptr_t>(15);
  const bool bulk = allow_bulk && count > 0 && lo >= reinterpret_cast<uintptr_t>(lo_limit) &&
                    hi <= reinterpret_cast<uintptr_t>(hi_limit);
  if (bulk) {
    *off = static_cast<uint32_t>((a - lo) >> 2);
    if (threadIdx.x == 0) tma::BulkLoad(tile, reinterpret_cast<const float *>(lo), static_cast<uint32_t>(hi - lo), bar);
    return true;
  }
  *off = 0;
  for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) tile[i] = first[i];
  return false;
}
/*! \brief bytes StageAround's bulk copy moves for this range */
__device__ __forceinline__ uint32_t AroundBytes(const float *first, uint32_t count) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(first);
  return static_cast<uint32_t>(((a + static_cast<uintptr_t>(count) * 4 + 15) & ~static_cast<uintptr_t>(15)) -
                               (a & ~static_cast<uintptr_t>(15)));
}
/*! \brief whether StageAround would issue a bulk copy for this range */
__device__ __forceinline__ bool AroundFits(const float *first, uint32_t count, const float *lo_limit,
                                           const float *hi_limit) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(first);
  return count > 0 && (a & ~static_cast<uintptr_t>(15)) >= reinterpret_cast<uintptr_t>(lo_limit) &&
         ((a + static_cast<uintptr_t>(count) * 4 + 15) & ~static_cast<uintptr_t>(15)) <=
             reinterpret_cast<uintptr_t>(hi_limit);
}
}  // namespace pooldetail

/*!
 * \brief spatial pooling of planes that do not fit shared memory.  The rows of a plane are
 *  contiguous, so a band of whole rows is one contiguous range: work item = (plane, band of
 *  `band_rows` output rows); the (band_rows - 1) * sy + ky input rows it reads are staged by one
 *  bulk copy (the 16-byte aligned window around them; plain loads for pitched rows or at the
 *  very ends of the tensor), windows are evaluated out of shared memory in the reference's
 *  order, results leave coalesced.  Neighbouring bands re-read ky - sy rows.
 *  Shared memory: ((band_rows - 1) * sy + ky) * w + 8 floats.
 */
template <typename Reducer, int KY, int KX, int SY, int SX>
__global__ void __launch_bounds__(kPoolThreads)
PoolBandsKernel(float *dst, const float *src, uint32_t planes, uint32_t h, uint32_t w, uint32_t ph, uint32_t pw,
                PoolGeom g, int64_t ld_src, int64_t ld_dst, uint32_t band_rows, uint32_t bands,
                gpu_rt::FastDiv div_bands, gpu_rt::FastDiv div_pw, gpu_rt::FastDiv div_pairs, int *status) {
  gpu_rt::GridDependencySync();
  extern __shared__ __align__(16) float tile[];
  __shared__ uint64_t bar;
  const int ky = KY > 0 ? KY : g.ky, kx = KX > 0 ? KX : g.kx;
  const int sy = SY > 0 ? SY : g.sy, sx = SX > 0 ? SX : g.sx;
  if (threadIdx.x == 0) tma::BarrierInit(&bar, 1);
  __syncthreads();
  uint32_t phase = 0;
  const bool dense_in = ld_src == static_cast<int64_t>(w);
  const float *src_end = src + static_cast<int64_t>(planes) * h * w;  // dense case only
  const uint32_t items = planes * bands;
  for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
    const uint32_t p = div_bands.Quot(item);
    const uint32_t py0 = (item - p * bands) * band_rows;
    const uint32_t npy = min(band_rows, ph - py0);
    const uint32_t nrows = (npy - 1) * sy + ky;
    const float *first = src + (static_cast<int64_t>(p) * h + py0 * sy) * ld_src;
    uint32_t off = 0;
    bool bulk = false;
    if (dense_in) {
      const bool fits = pooldetail::AroundFits(first, nrows * w, src, src_end);
      if (fits && threadIdx.x == 0) tma::BarrierExpect(&bar, pooldetail::AroundBytes(first, nrows * w));
      bulk = pooldetail::StageAround(tile, first, nrows * w, src, src_end, fits, &bar, &off);
    } else {
      pooldetail::StagePitched(tile, first, nrows, w, ld_src);
    }
    if (bulk) {
      if (!tma::WaitBounded(&bar, phase)) {
        if (threadIdx.x == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
        tma::WaitBounded(&bar, phase);
        return;
      }
      phase ^= 1;
    } else {
      __syncthreads();
    }
    const float *band = tile + off;
    float *out_band = dst + (static_cast<int64_t>(p) * ph + py0) * ld_dst;
    if ((KX == 3 || KX == 2) && SX == 2 && KY > 0 && MSHADOW_B200_POOL_PAIRS && (w & 3u) == 0 && (off & 3u) == 0) {
      // two adjacent outputs per thread from 16-byte shared-memory loads, as in PoolPlanesKernel
      const uint32_t pairs_per_row = (pw + 1) >> 1;
      const uint32_t npairs = npy * pairs_per_row;
      for (uint32_t o = threadIdx.x; o < npairs; o += kPoolThreads) {
        const uint32_t lpy = div_pairs.Quot(o);
        const uint32_t px = (o - lpy * pairs_per_row) * 2;
        const float *at = band + lpy * SY * w + px * 2;
        const bool second = px + 1 < pw;
        float r0, r1;
        Reducer::SetInitValue(r0);
        Reducer::SetInitValue(r1);
#pragma unroll
        for (int dy = 0; dy < (KY > 0 ? KY : 1); ++dy) {
          const float4 v = *reinterpret_cast<const float4 *>(at + dy * w);
          Reducer::Reduce(r0, v.x);
          Reducer::Reduce(r0, v.y);
          if (KX == 3) {
            const float e = second ? at[dy * w + 4] : 0.0f;
            Reducer::Reduce(r0, v.z);
            Reducer::Reduce(r1, v.z);
            Reducer::Reduce(r1, v.w);
            Reducer::Reduce(r1, e);
          } else {
            Reducer::Reduce(r1, v.z);
            Reducer::Reduce(r1, v.w);
          }
        }
        float *out = out_band + static_cast<int64_t>(lpy) * ld_dst + px;
        out[0] = r0;
        if (second) out[1] = r1;
      }
    } else {
      const uint32_t nout = npy * pw;
      for (uint32_t o = threadIdx.x; o < nout; o += kPoolThreads) {
        const uint32_t lpy = div_pw.Quot(o);
        const uint32_t px = o - lpy * pw;
        const float *at = band + lpy * sy * w + px * sx;
        float res;
        Reducer::SetInitValue(res);
        if (KY > 0) {
#pragma unroll
          for (int dy = 0; dy < (KY > 0 ? KY : 1); ++dy)
#pragma unroll
            for (int dx = 0; dx < (KX > 0 ? KX : 1); ++dx) Reducer::Reduce(res, at[dy * w + dx]);
        } else {
          for (int dy = 0; dy < ky; ++dy)
            for (int dx = 0; dx < kx; ++dx) Reducer::Reduce(res, at[dy * w + dx]);
        }
        out_band[static_cast<int64_t>(lpy) * ld_dst + px] = res;
      }
    }
    // all reads of the tile are done before the next band overwrites it
    tma::FenceAsyncShared();
    __syncthreads();
  }
}

/*!
 * \brief backward of spatial pooling for planes that do not fit shared memory: work item =
 *  (plane, band of `band_rows` source rows).  The band of the source, and the rows of the pooled
 *  plane and of its gradient whose windows reach into the band, are three contiguous ranges,
 *  staged like the forward kernel's.  Sums run over the covering windows in py-outer / px-inner
 *  order from zero with one rounding per product and per sum, as in UnpoolPlanesKernel.
 *  Shared memory: band_rows * w + 2 * pooled_rows * pw + 24 floats, pooled_rows being the most
 *  pooled rows any band needs.
 */
template <typename Reducer, int KY, int KX, int SY, int SX>
__global__ void __launch_bounds__(kPoolThreads)
UnpoolBandsKernel(float *dst, const float *src, const float *pooled, const float *gpooled, uint32_t planes,
                  uint32_t h, uint32_t w, uint32_t ph, uint32_t pw, PoolGeom g, int64_t ld_src, int64_t ld_pooled,
                  int64_t ld_dst, uint32_t band_rows, uint32_t bands, uint32_t pooled_rows_cap,
                  gpu_rt::FastDiv div_bands, gpu_rt::FastDiv div_w, gpu_rt::FastDiv div_wq, gpu_rt::FastDiv div_sy,
                  gpu_rt::FastDiv div_sx, int *status) {
  gpu_rt::GridDependencySync();
  extern __shared__ __align__(16) float tile[];
  __shared__ uint64_t bar;
  const uint32_t ky = KY > 0 ? KY : g.ky, kx = KX > 0 ? KX : g.kx;
  const uint32_t sy = SY > 0 ? SY : g.sy, sx = SX > 0 ? SX : g.sx;
  // three regions, each with room for the aligned window around its range
  const uint32_t src_cap = ((band_rows * w + 3) & ~3u) + 8, pool_cap = ((pooled_rows_cap * pw + 3) & ~3u) + 8;
  float *r_src = tile, *r_pool = tile + src_cap, *r_grad = r_pool + pool_cap;
  if (threadIdx.x == 0) tma::BarrierInit(&bar, 1);
  __syncthreads();
  uint32_t phase = 0;
  const bool dense = ld_src == static_cast<int64_t>(w) && ld_pooled == static_cast<int64_t>(pw);
  const float *src_end = src + static_cast<int64_t>(planes) * h * w;
  const float *pool_end = pooled + static_cast<int64_t>(planes) * ph * pw;
  const float *grad_end = gpooled + static_cast<int64_t>(planes) * ph * pw;
  constexpr bool kQuad = KY > 0 && KX > 0 && SY > 0 && SX > 0 && (4 % (SX > 0 ? SX : 1) == 0);
  const bool vec_out = (ld_dst & 3) == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  const uint32_t items = planes * bands;
  for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
    const uint32_t p = div_bands.Quot(item);
    const uint32_t y0 = (item - p * bands) * band_rows;
    const uint32_t nrows = min(band_rows, h - y0);
    // pooled rows whose windows reach rows y0 .. y0 + nrows - 1
    const uint32_t py_lo = y0 < ky ? 0 : (SY > 0 ? (y0 - ky + sy) / sy : div_sy.Quot(y0 - ky + sy));
    const uint32_t py_top = min(SY > 0 ? (y0 + nrows - 1 + sy) / sy : div_sy.Quot(y0 + nrows - 1 + sy), ph);
    const uint32_t npr = py_top > py_lo ? py_top - py_lo : 0;
    const float *g_src = src + (static_cast<int64_t>(p) * h + y0) * ld_src;
    const float *g_pool = pooled + (static_cast<int64_t>(p) * ph + py_lo) * ld_pooled;
    const float *g_grad = gpooled + (static_cast<int64_t>(p) * ph + py_lo) * ld_pooled;
    uint32_t off_s = 0, off_p = 0, off_g = 0;
    bool bulk = false;
    if (dense) {
      bulk = pooldetail::AroundFits(g_src, nrows * w, src, src_end) &&
             (npr == 0 || (pooldetail::AroundFits(g_pool, npr * pw, pooled, pool_end) &&
                           pooldetail::AroundFits(g_grad, npr * pw, gpooled, grad_end)));
      if (bulk && threadIdx.x == 0) {
        tma::BarrierExpect(&bar, pooldetail::AroundBytes(g_src, nrows * w) +
                                     (npr == 0 ? 0u : pooldetail::AroundBytes(g_pool, npr * pw) +
                                                          pooldetail::AroundBytes(g_grad, npr * pw)));
      }
      pooldetail::StageAround(r_src, g_src, nrows * w, src, src_end, bulk, &bar, &off_s);
      if (npr > 0) {
        pooldetail::StageAround(r_pool, g_pool, npr * pw, pooled, pool_end, bulk, &bar, &off_p);
        pooldetail::StageAround(r_grad, g_grad, npr * pw, gpooled, grad_end, bulk, &bar, &off_g);
      }
    } else {
      pooldetail::StagePitched(r_src, g_src, nrows, w, ld_src);
      pooldetail::StagePitched(r_pool, g_pool, npr, pw, ld_pooled);
      pooldetail::StagePitched(r_grad, g_grad, npr, pw, ld_pooled);
    }
    if (bulk) {
      if (!tma::WaitBounded(&bar, phase)) {
        if (threadIdx.x == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
        tma::WaitBounded(&bar, phase);
        return;
      }
      phase ^= 1;
    } else {
      __syncthreads();
    }
    const float *s_src = r_src + off_s;
    // pooled row py of the plane sits at pp + (py - py_lo) * pw; fold the offset into the base
    const float *pp = r_pool + off_p - static_cast<int64_t>(py_lo) * pw;
    const float *gp = r_grad + off_g - static_cast<int64_t>(py_lo) * pw;
    float *out_band = dst + (static_cast<int64_t>(p) * h + y0) * ld_dst;
    if (kQuad && (w & 3u) == 0 && (off_s & 3u) == 0) {
      constexpr int kSXs = SX > 0 ? SX : 1, kSYs = SY > 0 ? SY : 1;
      constexpr int kOff = pooldetail::FloorDiv(kSXs - KX, kSXs);
      constexpr int kCols = (3 / kSXs + 1) - kOff;
      constexpr int kRows = (KY - 1) / kSYs + 1;
      constexpr uint32_t kKYs = KY > 0 ? KY : 1;
      const uint32_t wq = w >> 2;
      const uint32_t nq = nrows * wq;
      for (uint32_t it = threadIdx.x; it < nq; it += kPoolThreads) {
        const uint32_t ly = div_wq.Quot(it);
        const uint32_t xq = it - ly * wq;
        const uint32_t y = y0 + ly;
        const float4 sv4 = *reinterpret_cast<const float4 *>(s_src + ly * w + 4 * xq);
        const float sv[4] = {sv4.x, sv4.y, sv4.z, sv4.w};
        const int py_first = y < kKYs ? 0 : static_cast<int>((y - kKYs + kSYs) / kSYs);
        const int py_hi = min(static_cast<int>((y + kSYs) / kSYs), static_cast<int>(ph));
        const int pxb = static_cast<int>(xq) * (4 / kSXs) + kOff;
        float val[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int py = py_first + r;
          if (py < py_hi) {
#pragma unroll
            for (int cc = 0; cc < kCols; ++cc) {
              const int px = pxb + cc;
              if (px >= 0 && px < static_cast<int>(pw)) {
                const float pv = pp[py * static_cast<int>(pw) + px];
                const float gv = gp[py * static_cast<int>(pw) + px];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int lo = pooldetail::FloorDiv(i - KX + kSXs, kSXs) - kOff;
                  const int hi = i / kSXs + 1 - kOff;
                  if (cc >= lo && cc < hi) {
                    val[i] = __fadd_rn(val[i], __fmul_rn(Reducer::PartialGrad(sv[i], pv), gv));
                  }
                }
              }
            }
          }
        }
        float *out = out_band + static_cast<int64_t>(ly) * ld_dst + 4 * xq;
        if (vec_out) {
          __stcs(reinterpret_cast<float4 *>(out), make_float4(val[0], val[1], val[2], val[3]));
        } else {
          out[0] = val[0];
          out[1] = val[1];
          out[2] = val[2];
          out[3] = val[3];
        }
      }
    } else {
      const uint32_t n = nrows * w;
      for (uint32_t o = threadIdx.x; o < n; o += kPoolThreads) {
        const uint32_t ly = div_w.Quot(o);
        const uint32_t x = o - ly * w;
        const uint32_t y = y0 + ly;
        const float vsrc = s_src[o];
        const uint32_t py_min = y < ky ? 0 : (SY > 0 ? (y - ky + sy) / sy : div_sy.Quot(y - ky + sy));
        const uint32_t px_min = x < kx ? 0 : (SX > 0 ? (x - kx + sx) / sx : div_sx.Quot(x - kx + sx));
        const uint32_t py_max = min(SY > 0 ? (y + sy) / sy : div_sy.Quot(y + sy), ph);
        const uint32_t px_max = min(SX > 0 ? (x + sx) / sx : div_sx.Quot(x + sx), pw);
        float val = 0.0f;
        for (uint32_t py = py_min; py < py_max; ++py)
          for (uint32_t px = px_min; px < px_max; ++px) {
            const float pg = Reducer::PartialGrad(vsrc, pp[py * pw + px]);
            val = __fadd_rn(val, __fmul_rn(pg, gp[py * pw + px]));
          }
        out_band[static_cast<int64_t>(ly) * ld_dst + x] = val;
      }
    }
    tma::FenceAsyncShared();
    __syncthreads();
  }
}

/*!
 * \brief channel-window pooling with stride 1 and pad NSIZE/2 (the chpool(src, nsize) form).
 *  A thread owns kLanes adjacent pixels of one image and marches over the channels with the
 *  last NSIZE values in registers, so every input element is read from HBM once.
 *  Work item = (image, pixel group), numbered across all images so that no lane idles at
 *  image borders; blockIdx.y selects a segment of `seg_len` output channels, which lets the
 *  host cut the march into as many equal pieces as fill whole waves of resident CTAs (a
 *  segment re-reads NSIZE-1 halo channels).  `plane` = h*w elements per channel, dense.
 */
template <typename Reducer, int NSIZE, int kLanes>
__global__ void __launch_bounds__(kPoolThreads, MSHADOW_B200_CHPOOL_MIN_CTAS)
ChannelPoolKernel(float *dst, const float *src, uint32_t channels, uint32_t plane, uint32_t groups_per_image,
                  uint32_t total_items, gpu_rt::FastDiv image_of_item, uint32_t seg_len) {
  gpu_rt::GridDependencySync();
  constexpr int kPad = NSIZE / 2;
  constexpr int kAhead = MSHADOW_B200_CHPOOL_AHEAD;  // loads issued this many channels before they are needed
  constexpr int kRing = NSIZE + kAhead;
  const uint32_t item = blockIdx.x * kPoolThreads + threadIdx.x;
  if (item >= total_items) return;
  const uint32_t image_idx = image_of_item.Quot(item);
  const uint32_t pix = (item - image_idx * groups_per_image) * kLanes;
  const uint32_t c_begin = blockIdx.y * seg_len;
  const uint32_t c_end = min(channels, c_begin + seg_len);
  const int64_t image = static_cast<int64_t>(image_idx) * channels * plane;
  const float *in = src + image + pix;
  float *out = dst + image + pix;
  float ring[kRing][kLanes];
  float init;
  Reducer::SetInitValue(init);
  // channels a segment may touch: its own plus the halo, clipped to the tensor
  const int64_t load_end = min(static_cast<int64_t>(channels), static_cast<int64_t>(c_end) + kPad);
  auto load = [&](int slot, int64_t c) {
    if (c >= 0 && c < load_end) {
      if (kLanes == 4) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(in + c * plane));
        ring[slot][0] = p.x;
        ring[slot][1 % kLanes] = p.y;
        ring[slot][2 % kLanes] = p.z;
        ring[slot][3 % kLanes] = p.w;
      } else {
        ring[slot][0] = __ldcs(in + c * plane);
      }
    } else {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) ring[slot][l] = init;
    }
  };
  // ring slot of channel c is (c - c_begin + kPad) mod kRing; preload the first window and
  // kAhead channels beyond it
#pragma unroll
  for (int s = 0; s < kRing; ++s) load(s, static_cast<int64_t>(c_begin) + s - kPad);
  for (uint32_t c0 = c_begin; c0 < c_end; c0 += kRing) {
#pragma unroll
    for (int j = 0; j < kRing; ++j) {
      const uint32_t c = c0 + j;
      if (c < c_end) {
        // window of channel c: slots j .. j + NSIZE - 1 (mod kRing), ascending channel order
        float res[kLanes];
#pragma unroll
        for (int l = 0; l < kLanes; ++l) res[l] = init;
#pragma unroll
        for (int t = 0; t < NSIZE; ++t)
#pragma unroll
          for (int l = 0; l < kLanes; ++l) Reducer::Reduce(res[l], ring[(j + t) % kRing][l]);
        if (kLanes == 4) {
          float4 p;
          p.x = res[0];
          p.y = res[1 % kLanes];
          p.z = res[2 % kLanes];
          p.w = res[3 % kLanes];
          __stcs(reinterpret_cast<float4 *>(out + static_cast<int64_t>(c) * plane), p);
        } else {
          __stcs(out + static_cast<int64_t>(c) * plane, res[0]);
        }
        // slot j held channel c - kPad, which no later window needs: refill it with the
        // channel kRing further on
        load(j, static_cast<int64_t>(c) - kPad + kRing);
      }
    }
  }
}

/*!
 * \brief gradient of the channel-window pooling above (ch_unpool(src, pooled, grad, nsize): stride
 *  1, pad NSIZE/2, pooled tensor with as many channels as src).  Source channel c collects
 *  PartialGrad(src(c), pooled(cc)) * grad(cc) over cc = c - pad .. c + pad inside the tensor, in
 *  ascending cc from zero, with one rounding per product and per sum, as the window loop of
 *  mshadow/extension/channel_unpool.h:102-133 does.  Same march as ChannelPoolKernel: a thread
 *  owns kLanes adjacent pixels, keeps the last NSIZE pooled and gradient values (and the source
 *  values on their way) in registers, and reads every element from HBM once apart from the
 *  NSIZE-1 halo channels per segment.  Channels outside the tensor enter as gradient +0, which
 *  adds nothing.
 */
template <typename Reducer, int NSIZE, int kLanes>
__global__ void __launch_bounds__(kPoolThreads, 2)
ChannelUnpoolKernel(float *dst, const float *src, const float *pooled, const float *gpooled, uint32_t channels,
                    uint32_t plane, uint32_t groups_per_image, uint32_t total_items, gpu_rt::FastDiv image_of_item,
                    uint32_t seg_len) {
  gpu_rt::GridDependencySync();
  constexpr int kPad = NSIZE / 2;
  // loads are issued this many channels before they are needed (for red::sum PartialGrad is the
  // constant 1, so the compiler drops the source and pooled rings and only the gradient is read)
  constexpr int kAhead = MSHADOW_B200_CHPOOL_AHEAD;
  constexpr int kRing = NSIZE + kAhead;
  const uint32_t item = blockIdx.x * kPoolThreads + threadIdx.x;
  if (item >= total_items) return;
  const uint32_t image_idx = image_of_item.Quot(item);
  const uint32_t pix = (item - image_idx * groups_per_image) * kLanes;
  const uint32_t c_begin = blockIdx.y * seg_len;
  const uint32_t c_end = min(channels, c_begin + seg_len);
  const int64_t image = static_cast<int64_t>(image_idx) * channels * plane + pix;
  const float *in = src + image, *pin = pooled + image, *gin = gpooled + image;
  float *out = dst + image;
  float rs[kRing][kLanes], rp[kRing][kLanes], rg[kRing][kLanes];
  const int64_t load_end = min(static_cast<int64_t>(channels), static_cast<int64_t>(c_end) + kPad);
  auto load = [&](int slot, int64_t c) {
    if (c >= 0 && c < load_end) {
      // a halo channel contributes its pooled value and gradient only: its source value is not read
      const bool own = c >= static_cast<int64_t>(c_begin) && c < static_cast<int64_t>(c_end);
      if (kLanes == 4) {
        const float4 s = own ? __ldcs(reinterpret_cast<const float4 *>(in + c * plane)) : make_float4(0, 0, 0, 0);
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(pin + c * plane));
        const float4 g = __ldcs(reinterpret_cast<const float4 *>(gin + c * plane));
        rs[slot][0] = s.x, rs[slot][1 % kLanes] = s.y, rs[slot][2 % kLanes] = s.z, rs[slot][3 % kLanes] = s.w;
        rp[slot][0] = p.x, rp[slot][1 % kLanes] = p.y, rp[slot][2 % kLanes] = p.z, rp[slot][3 % kLanes] = p.w;
        rg[slot][0] = g.x, rg[slot][1 % kLanes] = g.y, rg[slot][2 % kLanes] = g.z, rg[slot][3 % kLanes] = g.w;
      } else {
        rs[slot][0] = own ? __ldcs(in + c * plane) : 0.0f;
        rp[slot][0] = __ldcs(pin + c * plane);
        rg[slot][0] = __ldcs(gin + c * plane);
      }
    } else {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) rs[slot][l] = 0.0f, rp[slot][l] = 0.0f, rg[slot][l] = 0.0f;
    }
  };
  // ring slot of channel c is (c - c_begin + kPad) mod kRing
#pragma unroll
  for (int s = 0; s < kRing; ++s) load(s, static_cast<int64_t>(c_begin) + s - kPad);
  for (uint32_t c0 = c_begin; c0 < c_end; c0 += kRing) {
#pragma unroll
    for (int j = 0; j < kRing; ++j) {
      const uint32_t c = c0 + j;
      if (c < c_end) {
        float val[kLanes];
#pragma unroll
        for (int l = 0; l < kLanes; ++l) val[l] = 0.0f;
#pragma unroll
        for (int t = 0; t < NSIZE; ++t)
#pragma unroll
          for (int l = 0; l < kLanes; ++l) {
            const float pg = Reducer::PartialGrad(rs[(j + kPad) % kRing][l], rp[(j + t) % kRing][l]);
            val[l] = __fadd_rn(val[l], __fmul_rn(pg, rg[(j + t) % kRing][l]));
          }
        if (kLanes == 4) {
          __stcs(reinterpret_cast<float4 *>(out + static_cast<int64_t>(c) * plane),
                 make_float4(val[0], val[1 % kLanes], val[2 % kLanes], val[3 % kLanes]));
        } else {
          __stcs(out + static_cast<int64_t>(c) * plane, val[0]);
        }
        load(j, static_cast<int64_t>(c) - kPad + kRing);
      }
    }
  }
}

/*!
 * \brief channel-window pooling with the channel planes staged through shared memory.
 *  Same arithmetic as ChannelPoolKernel (window kept in registers, channels added in
 *  ascending order), but no thread waits on its own global loads: a producer thread issues
 *  one bulk asynchronous copy per channel plane (or plane tile) into a ring of `ring`
 *  shared-memory slots, up to `ring` channels ahead of the march, so a CTA keeps
 *  ring * tile bytes in flight at no register cost and reads memory in long contiguous pieces.
 *  Every slot has two transaction barriers: `full` completes when the copy has landed,
 *  `empty` when every consumer warp has read the slot (one arrival per warp).  Warps therefore
 *  drift apart freely; nothing in the march synchronises the whole CTA.
 *  CTA = (image, pixel tile) x channel segment; warps 0 .. n-2 consume, 4 adjacent pixels per
 *  thread, the last warp produces.  Dynamic shared memory: ring * tile_px floats.
 *  (A variant with one persistent CTA per SM walking an equal share of all output planes --
 *  no idle SMs in the last wave, a halo only where a share starts inside an image -- was built
 *  and measured: its consumer loop has to carry the piece state, the compiler then wants 128
 *  registers for the unrolled window, and the form that fits 64 registers shifts the window every
 *  step: 0.85 of the copy bandwidth against 0.92 for this kernel.)
 */
template <typename Reducer, int NSIZE>
__global__ void __launch_bounds__(1024, 1)
ChannelPoolStagedKernel(float *dst, const float *src, uint32_t channels, uint32_t plane, uint32_t tile_px,
                        uint32_t tiles_per_plane, uint32_t seg_len, uint32_t ring, int *status) {
  gpu_rt::GridDependencySync();
  constexpr int kPad = NSIZE / 2;
  constexpr uint32_t kMaxRing = 16;
  extern __shared__ __align__(16) float slots[];
  __shared__ uint64_t full[kMaxRing], empty[kMaxRing];
  const uint32_t image_idx = blockIdx.x / tiles_per_plane;
  const uint32_t tile_idx = blockIdx.x - image_idx * tiles_per_plane;
  const uint32_t px0 = tile_idx * tile_px;
  const uint32_t len = min(tile_px, plane - px0);  // pixels of this tile, a multiple of 4
  const uint32_t c_begin = blockIdx.y * seg_len;
  const uint32_t c_end = min(channels, c_begin + seg_len);
  const int64_t base = static_cast<int64_t>(image_idx) * channels * plane + px0;
  const float *in = src + base;
  float *out = dst + base;
  const uint32_t nsteps = (c_end - c_begin) + 2 * kPad;  // channels c_begin-kPad .. c_end-1+kPad
  const uint32_t consumer_warps = (blockDim.x >> 5) - 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (uint32_t j = 0; j < ring; ++j) {
      tma::BarrierInit(&full[j], 1);
      tma::BarrierInit(&empty[j], consumer_warps);
    }
  }
  __syncthreads();
  if (warp == consumer_warps) {
    // producer: step s uses slot s % ring for the (s / ring)-th time, once the consumers have
    // released its previous use
    if (lane != 0) return;
    // (slot and lap are counted, not computed as s % ring and s / ring: with a run-time ring the two
    // divisions per step were a third of the consumers' instructions)
    uint32_t slot = 0, use = 0;
    for (uint32_t s = 0; s < nsteps; ++s) {
      if (use > 0 && !tma::WaitBounded(&empty[slot], (use - 1) & 1u)) {
        atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      const int64_t ch = static_cast<int64_t>(c_begin) - kPad + s;
      if (ch >= 0 && ch < static_cast<int64_t>(channels)) {
        tma::BarrierExpect(&full[slot], len * 4u);
        tma::BulkLoad(slots + static_cast<size_t>(slot) * tile_px, in + ch * plane, len * 4u, &full[slot]);
      } else {
        // a channel outside the tensor still takes its turn on the slot: the consumers wait for
        // `full` at every step, so they can never release a slot twice before this thread has
        // seen the first release
        tma::BarrierArrive(&full[slot]);
      }
      if (++slot == ring) {
        slot = 0;
        ++use;
      }
    }
    return;
  }
  const bool mine = threadIdx.x * 4 < len;
  float init;
  Reducer::SetInitValue(init);
  float win[NSIZE][4];
#pragma unroll
  for (int j = 0; j < NSIZE; ++j) win[j][0] = win[j][1] = win[j][2] = win[j][3] = init;
  uint32_t slot = 0, lap = 0;
  // 32-bit bookkeeping in the march: the channel of step s as an unsigned number (a channel before
  // the tensor wraps to a huge one and fails the one comparison), slot and output addresses advanced
  // by additions
  uint32_t ch = c_begin - kPad;
  const float *my_slot = slots + threadIdx.x * 4;
  float *my_out = out + static_cast<int64_t>(c_begin) * plane + threadIdx.x * 4;
  for (uint32_t s0 = 0; s0 < nsteps; s0 += NSIZE) {
#pragma unroll
    for (int j = 0; j < NSIZE; ++j) {
      const uint32_t s = s0 + j;
      if (s < nsteps) {
        float4 v = make_float4(init, init, init, init);
        if (!tma::WaitBounded(&full[slot], lap & 1u)) {
          if (lane == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
          return;
        }
        if (ch < channels && mine) {
          v = *reinterpret_cast<const float4 *>(my_slot);
        }
        // this warp is done with the slot (the producer counts one release per warp and step)
        __syncwarp();
        if (lane == 0) tma::BarrierArrive(&empty[slot]);
        win[j][0] = v.x;
        win[j][1] = v.y;
        win[j][2] = v.z;
        win[j][3] = v.w;
        if (s + 1 > 2 * kPad && mine) {
          // window of output channel ch - kPad: the last NSIZE loaded channels, oldest first
          float res[4] = {init, init, init, init};
#pragma unroll
          for (int t = 1; t <= NSIZE; ++t)
#pragma unroll
            for (int l = 0; l < 4; ++l) Reducer::Reduce(res[l], win[(j + t) % NSIZE][l]);
          __stcs(reinterpret_cast<float4 *>(my_out), make_float4(res[0], res[1], res[2], res[3]));
          my_out += plane;
        }
        ++ch;
        my_slot += tile_px;
        if (++slot == ring) {
          slot = 0;
          ++lap;
          my_slot = slots + threadIdx.x * 4;
        }
      }
    }
  }
}

/*!
 * \brief backward pass of channel-window pooling for reducers whose gradient depends on the values
 *  (maximum, minimum), with the planes staged through shared memory like ChannelPoolStagedKernel.
 *  A ring slot holds the three planes of one channel (source, pooled, pooled gradient; the source
 *  plane is left out for the halo channels of a segment).  Consumers keep the last NSIZE pooled
 *  values and gradients of their four pixels in registers; the source value of the output channel,
 *  loaded NSIZE / 2 steps earlier, is read from its slot, which is released that much later.
 *  Arithmetic as in ChannelUnpoolKernel: val = 0, then val += PartialGrad(src, pooled) * gradient
 *  over the window in ascending channel order, product and sum rounded one by one.
 *  CTA = (image, pixel tile of at most kChUnpoolTilePx pixels) x channel segment; block = tile / 4
 *  consumer threads + one producer warp; dynamic shared memory ring * 3 * tile_px floats.
 */
const uint32_t kChUnpoolTilePx = 3200;                       // 800 consumer threads: 78 registers each
const int kChUnpoolMaxThreads = kChUnpoolTilePx / 4 + 32;

template <typename Reducer, int NSIZE>
__global__ void __launch_bounds__(kChUnpoolMaxThreads, 1)
ChannelUnpoolStagedKernel(float *dst, const float *src, const float *pooled, const float *gpooled, uint32_t channels,
                          uint32_t plane, uint32_t tile_px, uint32_t tiles_per_plane, uint32_t seg_len, uint32_t ring,
                          int *status) {
  gpu_rt::GridDependencySync();
  constexpr int kPad = NSIZE / 2;
  constexpr uint32_t kMaxRing = 16;
  extern __shared__ __align__(16) float slots[];
  __shared__ uint64_t full[kMaxRing], empty[kMaxRing];
  const uint32_t image_idx = blockIdx.x / tiles_per_plane;
  const uint32_t px0 = (blockIdx.x - image_idx * tiles_per_plane) * tile_px;
  const uint32_t len = min(tile_px, plane - px0);
  const uint32_t c_begin = blockIdx.y * seg_len;
  const uint32_t c_end = min(channels, c_begin + seg_len);
  const int64_t base = static_cast<int64_t>(image_idx) * channels * plane + px0;
  const uint32_t nsteps = (c_end - c_begin) + 2 * kPad;
  const uint32_t consumer_warps = (blockDim.x >> 5) - 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t slot_floats = static_cast<size_t>(3) * tile_px;
  if (threadIdx.x == 0) {
    for (uint32_t j = 0; j < ring; ++j) {
      tma::BarrierInit(&full[j], 1);
      tma::BarrierInit(&empty[j], consumer_warps);
    }
  }
  __syncthreads();
  if (warp == consumer_warps) {
    if (lane != 0) return;
    uint32_t slot = 0, use = 0;  // counted, not s % ring and s / ring
    for (uint32_t s = 0; s < nsteps; ++s) {
      if (use > 0 && !tma::WaitBounded(&empty[slot], (use - 1) & 1u)) {
        atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      const int64_t ch = static_cast<int64_t>(c_begin) - kPad + s;
      if (ch >= 0 && ch < static_cast<int64_t>(channels)) {
        float *at = slots + slot * slot_floats;
        const int64_t from = base + ch * plane;
        // the source plane is needed only where this segment produces an output
        const bool own = ch >= static_cast<int64_t>(c_begin) && ch < static_cast<int64_t>(c_end);
        tma::BarrierExpect(&full[slot], (own ? 3u : 2u) * len * 4u);
        if (own) tma::BulkLoad(at, src + from, len * 4u, &full[slot]);
        tma::BulkLoad(at + tile_px, pooled + from, len * 4u, &full[slot]);
        tma::BulkLoad(at + 2 * tile_px, gpooled + from, len * 4u, &full[slot]);
      } else {
        tma::BarrierArrive(&full[slot]);
      }
      if (++slot == ring) {
        slot = 0;
        ++use;
      }
    }
    return;
  }
  const bool mine = threadIdx.x * 4 < len;
  float wp[NSIZE][4], wg[NSIZE][4];
#pragma unroll
  for (int j = 0; j < NSIZE; ++j) {
#pragma unroll
    for (int l = 0; l < 4; ++l) wp[j][l] = 0.0f, wg[j][l] = 0.0f;
  }
  uint32_t slot = 0, lap = 0, centre = 0;  // ring position of step s, and of step s - kPad
  // 32-bit bookkeeping: the channel of a step as an unsigned number (one before the tensor wraps and
  // fails the one comparison), slot and output addresses advanced by additions
  uint32_t ch = c_begin - kPad;
  const float *my_slot = slots + threadIdx.x * 4, *my_centre = my_slot;
  float *my_out = dst + base + static_cast<int64_t>(c_begin) * plane + threadIdx.x * 4;
  for (uint32_t s0 = 0; s0 < nsteps; s0 += NSIZE) {
#pragma unroll
    for (int j = 0; j < NSIZE; ++j) {
      const uint32_t s = s0 + j;
      if (s < nsteps) {
        if (!tma::WaitBounded(&full[slot], lap & 1u)) {
          if (lane == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
          return;
        }
        // a channel outside the tensor enters as gradient +0, which adds nothing
        float4 pv = make_float4(0.0f, 0.0f, 0.0f, 0.0f), gv = pv;
        if (ch < channels && mine) {
          const float *at = my_slot;
          pv = *reinterpret_cast<const float4 *>(at + tile_px);
          gv = *reinterpret_cast<const float4 *>(at + 2 * tile_px);
        }
        wp[j][0] = pv.x, wp[j][1] = pv.y, wp[j][2] = pv.z, wp[j][3] = pv.w;
        wg[j][0] = gv.x, wg[j][1] = gv.y, wg[j][2] = gv.z, wg[j][3] = gv.w;
        if (s >= 2 * kPad && mine) {
          // output channel ch - kPad; its source values still sit in the slot of step s - kPad
          const float4 xv = *reinterpret_cast<const float4 *>(my_centre);
          const float xc[4] = {xv.x, xv.y, xv.z, xv.w};
          float val[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
          for (int u = 1; u <= NSIZE; ++u)
#pragma unroll
            for (int l = 0; l < 4; ++l) {
              const float pg = Reducer::PartialGrad(xc[l], wp[(j + u) % NSIZE][l]);
              val[l] = __fadd_rn(val[l], __fmul_rn(pg, wg[(j + u) % NSIZE][l]));
            }
          __stcs(reinterpret_cast<float4 *>(my_out), make_float4(val[0], val[1], val[2], val[3]));
          my_out += plane;
        }
        // the slot of step s - kPad has now been read for the last time
        __syncwarp();
        if (s >= static_cast<uint32_t>(kPad)) {
          if (lane == 0) tma::BarrierArrive(&empty[centre]);
          my_centre += slot_floats;
          if (++centre == ring) {
            centre = 0;
            my_centre = slots + threadIdx.x * 4;
          }
        }
        ++ch;
        my_slot += slot_floats;
        if (++slot == ring) {
          slot = 0;
          ++lap;
          my_slot = slots + threadIdx.x * 4;
        }
      }
    }
  }
}

// ------------------------------- host side ----------------------------------------------

namespace pooldetail {
/*! \brief device status word (see tma.cuh); lives as long as the process */
inline int *StatusWord() { return gpu_rt::StatusWord(); }

/*! \brief planes per CTA: as many as fit `budget` bytes, in multiples of `quantum` */
inline uint32_t GroupSize(uint64_t bytes_per_plane, uint32_t quantum, uint64_t budget, uint32_t planes) {
  uint64_t g = budget / bytes_per_plane;
  if (g >= quantum) g -= g % quantum;
  if (g < 1) g = 1;
  if (g > planes) g = planes;
  if (g > 64) g = 64;
  return static_cast<uint32_t>(g);
}

inline uint32_t Gcd(uint32_t a, uint32_t b) { return b == 0 ? a : Gcd(b, a % b); }

/*!
 * \brief how many equal segments (1..kmax) to cut each of `fixed` CTA columns into so that the
 *  grid of fixed*k CTAs fills whole waves of `slots` resident CTAs; the smallest k reaching
 *  95 %, else the best one
 */
inline uint32_t WaveFriendlySegments(uint32_t fixed, uint32_t kmax, uint32_t slots) {
  uint32_t best = 1;
  double best_eff = 0.0;
  for (uint32_t k = 1; k <= kmax; ++k) {
    const uint64_t ctas = static_cast<uint64_t>(fixed) * k;
    const uint64_t waves = (ctas + slots - 1) / slots;
    const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = k;
    }
    if (eff >= 0.95) return k;
  }
  return best;
}
}  // namespace pooldetail

/*! \brief dynamic shared memory per CTA: forward leaves room for 4 CTAs per SM, backward for 3 */
const uint64_t kPoolSmemBudget = MSHADOW_B200_POOL_SMEM_KB * 1024;
const uint64_t kUnpoolSmemBudget = MSHADOW_B200_UNPOOL_SMEM_KB * 1024;

/*! \brief true when the plane kernels can run: at least one plane has to fit the budget */
inline bool PoolPlanesFit(int64_t h, int64_t w, int64_t ph, int64_t pw, bool backward) {
  const uint64_t per_plane = static_cast<uint64_t>(h) * w * 4 + (backward ? 2ull * ph * pw * 4 : 0ull);
  return per_plane + 32 <= (backward ? kUnpoolSmemBudget : kPoolSmemBudget) && static_cast<int64_t>(h) * w < (1 << 24);
}

template <typename Reducer>
inline void PoolPlanesLaunch(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky, int kx,
                             int sy, int sx, int64_t ld_src, int64_t ld_dst, cudaStream_t stream) {
  const uint32_t ph = static_cast<uint32_t>((h - ky) / sy + 1), pw = static_cast<uint32_t>((w - kx) / sx + 1);
  if (planes == 0) return;
  const uint32_t hw = static_cast<uint32_t>(h * w);
  // groups start 16-byte aligned when their plane count is a multiple of 4 / gcd(h*w, 4)
  const uint32_t quantum = 4 / pooldetail::Gcd(hw, 4);
  const uint32_t gp = pooldetail::GroupSize(hw * 4ull, quantum, kPoolSmemBudget, static_cast<uint32_t>(planes));
  const size_t smem = static_cast<size_t>(gp) * hw * 4;
  const int groups = gpu_rt::CeilDiv(planes, gp);
  const int cap = gpu_rt::CurrentDevice().sm_count * 16;
  const int grid = groups < cap ? groups : cap;
  const PoolGeom g = {ky, kx, sy, sx};
  int *status = pooldetail::StatusWord();
#define MSHADOW_B200_POOL_LAUNCH_(KY, KX, SY, SX)                                                                 \
  {                                                                                                               \
    auto kernel = PoolPlanesKernel<Reducer, KY, KX, SY, SX>;                                                      \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                                           static_cast<int>(kPoolSmemBudget)));                                   \
    gpu_rt::LaunchAfterDrain(kernel, dim3(grid), dim3(kPoolThreads), smem, stream, dst, src, static_cast<uint32_t>(planes), static_cast<uint32_t>(h), \
                                                static_cast<uint32_t>(w), ph, pw, g, ld_src, ld_dst, gp,          \
                                                gpu_rt::FastDiv(pw), gpu_rt::FastDiv(ph),                         \
                                                gpu_rt::FastDiv((pw + 1) / 2), status);                           \
  }
  if (ky == 3 && kx == 3 && sy == 2 && sx == 2) MSHADOW_B200_POOL_LAUNCH_(3, 3, 2, 2)
  else if (ky == 2 && kx == 2 && sy == 2 && sx == 2) MSHADOW_B200_POOL_LAUNCH_(2, 2, 2, 2)
  else MSHADOW_B200_POOL_LAUNCH_(0, 0, 0, 0)
#undef MSHADOW_B200_POOL_LAUNCH_
  MSHADOW_CUDA_POST_KERNEL_CHECK(PoolPlanesKernel);
}

template <typename Reducer>
inline void UnpoolPlanesLaunch(float *dst, const float *src, const float *pooled, const float *gpooled,
                               int64_t planes, int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx, int sy,
                               int sx, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst, cudaStream_t stream) {
  if (planes == 0) return;
  const uint32_t hw = static_cast<uint32_t>(h * w), phw = static_cast<uint32_t>(ph * pw);
  const uint32_t q1 = 4 / pooldetail::Gcd(hw, 4), q2 = 4 / pooldetail::Gcd(phw, 4);
  const uint32_t quantum = q1 > q2 ? q1 : q2;
  const uint32_t gp = pooldetail::GroupSize((hw + 2ull * phw) * 4, quantum, kUnpoolSmemBudget - 32,
                                            static_cast<uint32_t>(planes));
  const size_t smem = (((static_cast<size_t>(gp) * hw + 3) & ~size_t(3)) +
                       2 * ((static_cast<size_t>(gp) * phw + 3) & ~size_t(3))) * 4;
  const int groups = gpu_rt::CeilDiv(planes, gp);
  const int cap = gpu_rt::CurrentDevice().sm_count * 16;
  const int grid = groups < cap ? groups : cap;
  const PoolGeom g = {ky, kx, sy, sx};
  int *status = pooldetail::StatusWord();
#define MSHADOW_B200_UNPOOL_LAUNCH_(KY, KX, SY, SX)                                                               \
  {                                                                                                               \
    auto kernel = UnpoolPlanesKernel<Reducer, KY, KX, SY, SX>;                                                    \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                                           static_cast<int>(kUnpoolSmemBudget)));                                 \
    gpu_rt::LaunchAfterDrain(kernel, dim3(grid), dim3(kPoolThreads), smem, stream,                                                                  \
        dst, src, pooled, gpooled, static_cast<uint32_t>(planes), static_cast<uint32_t>(h),                       \
        static_cast<uint32_t>(w), static_cast<uint32_t>(ph), static_cast<uint32_t>(pw), g, ld_src, ld_pooled,     \
        ld_dst, gp, gpu_rt::FastDiv(static_cast<uint32_t>(w)), gpu_rt::FastDiv(static_cast<uint32_t>(h)),         \
        gpu_rt::FastDiv(static_cast<uint32_t>(sy)), gpu_rt::FastDiv(static_cast<uint32_t>(sx)),                   \
        gpu_rt::FastDiv(static_cast<uint32_t>(w / 4 > 0 ? w / 4 : 1)), status);                                   \
  }
  if (ky == 3 && kx == 3 && sy == 2 && sx == 2) MSHADOW_B200_UNPOOL_LAUNCH_(3, 3, 2, 2)
  else if (ky == 2 && kx == 2 && sy == 2 && sx == 2) MSHADOW_B200_UNPOOL_LAUNCH_(2, 2, 2, 2)
  else MSHADOW_B200_UNPOOL_LAUNCH_(0, 0, 0, 0)
#undef MSHADOW_B200_UNPOOL_LAUNCH_
  MSHADOW_CUDA_POST_KERNEL_CHECK(UnpoolPlanesKernel);
}

/*! \brief launch shape of the band kernels for planes beyond shared memory; ok == false: not applicable */
struct BandPlan {
  uint32_t band_rows, bands, pooled_rows;
  size_t smem;
  bool ok;
};

/*! \brief forward: as many output rows per band as the budget allows, bands of equal height */
inline BandPlan PlanPoolBands(int64_t h, int64_t w, int64_t ph, int ky, int sy) {
  BandPlan bp = {0, 0, 0, 0, false};
  const uint64_t budget = static_cast<uint64_t>(MSHADOW_B200_POOL_BAND_SMEM_KB) * 1024;
  if (h * w >= (int64_t(1) << 31) || ph < 1) return bp;
  const uint64_t rows_cap = (budget - 64) / (static_cast<uint64_t>(w) * 4);
  if (rows_cap < static_cast<uint64_t>(ky)) return bp;
  const uint64_t out_cap = (rows_cap - ky) / sy + 1;
  bp.bands = static_cast<uint32_t>((ph + out_cap - 1) / out_cap);
  bp.band_rows = static_cast<uint32_t>((ph + bp.bands - 1) / bp.bands);
  bp.bands = static_cast<uint32_t>((ph + bp.band_rows - 1) / bp.band_rows);
  bp.smem = ((static_cast<size_t>(bp.band_rows - 1) * sy + ky) * w + 8) * 4;
  bp.ok = true;
  return bp;
}

/*! \brief backward: the fewest bands of source rows whose staged ranges fit the budget */
inline BandPlan PlanUnpoolBands(int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int sy) {
  BandPlan bp = {0, 0, 0, 0, false};
  if (h * w >= (int64_t(1) << 31) || h < 1) return bp;
  for (uint32_t bands = 1; bands <= static_cast<uint32_t>(h); ++bands) {
    const uint32_t br = static_cast<uint32_t>((h + bands - 1) / bands);
    uint32_t prc = 0;
    for (uint32_t y0 = 0; y0 < static_cast<uint32_t>(h); y0 += br) {
      const uint32_t nrows = static_cast<uint32_t>(h) - y0 < br ? static_cast<uint32_t>(h) - y0 : br;
      const uint32_t lo = y0 < static_cast<uint32_t>(ky) ? 0 : (y0 - ky + sy) / sy;
      uint32_t top = (y0 + nrows - 1 + sy) / sy;
      if (top > static_cast<uint32_t>(ph)) top = static_cast<uint32_t>(ph);
      if (top > lo && top - lo > prc) prc = top - lo;
    }
    const size_t smem = ((((static_cast<size_t>(br) * w + 3) & ~size_t(3)) + 8) +
                         2 * (((static_cast<size_t>(prc) * pw + 3) & ~size_t(3)) + 8)) * 4;
    if (smem <= kUnpoolSmemBudget) {
      bp.band_rows = br;
      bp.bands = static_cast<uint32_t>((h + br - 1) / br);
      bp.pooled_rows = prc;
      bp.smem = smem;
      bp.ok = true;
      return bp;
    }
    if (br == 1) break;
  }
  return bp;
}

template <typename Reducer>
inline void PoolBandsLaunch(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky, int kx, int sy,
                            int sx, int64_t ld_src, int64_t ld_dst, const BandPlan &bp, cudaStream_t stream) {
  const uint32_t ph = static_cast<uint32_t>((h - ky) / sy + 1), pw = static_cast<uint32_t>((w - kx) / sx + 1);
  if (planes == 0) return;
  CHECK_LT(planes * static_cast<int64_t>(bp.bands), int64_t(1) << 31) << "pool: too many bands";
  const uint32_t items = static_cast<uint32_t>(planes) * bp.bands;
  const uint32_t cap = static_cast<uint32_t>(gpu_rt::CurrentDevice().sm_count) * 16;
  const uint32_t grid = items < cap ? items : cap;
  const PoolGeom g = {ky, kx, sy, sx};
  int *status = pooldetail::StatusWord();
#define MSHADOW_B200_POOL_BANDS_(KY, KX, SY, SX)                                                                  \
  {                                                                                                               \
    auto kernel = PoolBandsKernel<Reducer, KY, KX, SY, SX>;                                                       \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                                           MSHADOW_B200_POOL_BAND_SMEM_KB * 1024));                               \
    gpu_rt::LaunchAfterDrain(kernel, dim3(grid), dim3(kPoolThreads), bp.smem, stream, dst, src, static_cast<uint32_t>(planes),                     \
                                                   static_cast<uint32_t>(h), static_cast<uint32_t>(w), ph, pw, g, \
                                                   ld_src, ld_dst, bp.band_rows, bp.bands,                        \
                                                   gpu_rt::FastDiv(bp.bands), gpu_rt::FastDiv(pw),                \
                                                   gpu_rt::FastDiv((pw + 1) / 2), status);                        \
  }
  if (ky == 3 && kx == 3 && sy == 2 && sx == 2) MSHADOW_B200_POOL_BANDS_(3, 3, 2, 2)
  else if (ky == 2 && kx == 2 && sy == 2 && sx == 2) MSHADOW_B200_POOL_BANDS_(2, 2, 2, 2)
  else MSHADOW_B200_POOL_BANDS_(0, 0, 0, 0)
#undef MSHADOW_B200_POOL_BANDS_
  MSHADOW_CUDA_POST_KERNEL_CHECK(PoolBandsKernel);
}

template <typename Reducer>
inline void UnpoolBandsLaunch(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t planes,
                              int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx, int sy, int sx,
                              int64_t ld_src, int64_t ld_pooled, int64_t ld_dst, const BandPlan &bp,
                              cudaStream_t stream) {
  if (planes == 0) return;
  CHECK_LT(planes * static_cast<int64_t>(bp.bands), int64_t(1) << 31) << "unpool: too many bands";
  const uint32_t items = static_cast<uint32_t>(planes) * bp.bands;
  const uint32_t cap = static_cast<uint32_t>(gpu_rt::CurrentDevice().sm_count) * 16;
  const uint32_t grid = items < cap ? items : cap;
  const PoolGeom g = {ky, kx, sy, sx};
  int *status = pooldetail::StatusWord();
  const uint32_t uw = static_cast<uint32_t>(w);
#define MSHADOW_B200_UNPOOL_BANDS_(KY, KX, SY, SX)                                                                \
  {                                                                                                               \
    auto kernel = UnpoolBandsKernel<Reducer, KY, KX, SY, SX>;                                                     \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                                           static_cast<int>(kUnpoolSmemBudget)));                                 \
    gpu_rt::LaunchAfterDrain(kernel, dim3(grid), dim3(kPoolThreads), bp.smem, stream,                                                               \
        dst, src, pooled, gpooled, static_cast<uint32_t>(planes), static_cast<uint32_t>(h), uw,                   \
        static_cast<uint32_t>(ph), static_cast<uint32_t>(pw), g, ld_src, ld_pooled, ld_dst, bp.band_rows,         \
        bp.bands, bp.pooled_rows, gpu_rt::FastDiv(bp.bands), gpu_rt::FastDiv(uw),                                 \
        gpu_rt::FastDiv(uw / 4 > 0 ? uw / 4 : 1), gpu_rt::FastDiv(static_cast<uint32_t>(sy)),                     \
        gpu_rt::FastDiv(static_cast<uint32_t>(sx)), status);                                                      \
  }
  if (ky == 3 && kx == 3 && sy == 2 && sx == 2) MSHADOW_B200_UNPOOL_BANDS_(3, 3, 2, 2)
  else if (ky == 2 && kx == 2 && sy == 2 && sx == 2) MSHADOW_B200_UNPOOL_BANDS_(2, 2, 2, 2)
  else MSHADOW_B200_UNPOOL_BANDS_(0, 0, 0, 0)
#undef MSHADOW_B200_UNPOOL_BANDS_
  MSHADOW_CUDA_POST_KERNEL_CHECK(UnpoolBandsKernel);
}

/*! \brief window sizes the register-ring channel kernel is instantiated for */
inline bool ChannelPoolSupported(int nsize, int stride, int pad) {
  return stride == 1 && pad == nsize / 2 && (nsize == 1 || nsize == 3 || nsize == 5 || nsize == 7 || nsize == 9);
}

/*! \brief dense (n, c, h, w) in and out; requires ChannelPoolSupported */
template <typename Reducer>
inline void ChannelPoolLaunch(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int nsize,
                              cudaStream_t stream) {
  if (n == 0 || c == 0 || h * w == 0) return;
  const uint32_t plane = static_cast<uint32_t>(h * w);
  const bool vec = plane % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0;
  const int lanes = vec ? 4 : 1;
  const uint32_t groups = plane / lanes;
  const int64_t items64 = n * static_cast<int64_t>(groups);
  CHECK_LT(items64, (int64_t(1) << 31)) << "chpool: tensor too large for 32-bit indexing";
  const uint32_t items = static_cast<uint32_t>(items64);
  const uint32_t tiles = static_cast<uint32_t>(gpu_rt::CeilDiv(items, kPoolThreads));
#define MSHADOW_B200_CHPOOL_LAUNCH_(NS, LANES)                                                                 \
  {                                                                                                            \
    auto kernel = ChannelPoolKernel<Reducer, NS, LANES>;                                                       \
    /* cut the channel march into the number of segments that fills whole waves of resident CTAs; every      \
       segment costs NS-1 halo channels, so segments stay at least 8 windows long */                          \
    const uint32_t slots = static_cast<uint32_t>(gpu_rt::ResidentPerSM(kernel, kPoolThreads)) *               \
                           gpu_rt::CurrentDevice().sm_count;                                                   \
    uint32_t max_seg = static_cast<uint32_t>(c) / (8 * NS);                                                    \
    if (max_seg < 1) max_seg = 1;                                                                              \
    if (max_seg > 16) max_seg = 16;                                                                            \
    const uint32_t segs = pooldetail::WaveFriendlySegments(tiles, max_seg, slots);                            \
    const uint32_t seg_len = (static_cast<uint32_t>(c) + segs - 1) / segs;                                     \
    const uint32_t nseg = (static_cast<uint32_t>(c) + seg_len - 1) / seg_len;                                  \
    gpu_rt::LaunchAfterDrain(kernel, dim3(tiles, nseg), dim3(kPoolThreads), 0, stream, dst, src, static_cast<uint32_t>(c), plane, groups,  \
                                                            items, gpu_rt::FastDiv(groups), seg_len);          \
  }
  // staged variant: planes (or plane tiles of at most 3968 pixels: 31 consumer warps of 128 pixels and one
  // producer warp make a 1024-thread CTA) ride through a shared-memory ring
  const uint32_t tiles_per_plane = (plane + 3967) / 3968;
  const uint32_t tile_px = ((plane + tiles_per_plane - 1) / tiles_per_plane + 3) & ~3u;
  const uint32_t st_threads = (((tile_px / 4) + 31) & ~31u) + 32;
  const bool staged = vec && MSHADOW_B200_CHPOOL_STAGED && c >= 2 * nsize &&
                      n * static_cast<int64_t>(tiles_per_plane) < (int64_t(1) << 31);
#define MSHADOW_B200_CHPOOL_STAGED_LAUNCH_(NS)                                                                 \
  {                                                                                                            \
    auto kernel = ChannelPoolStagedKernel<Reducer, NS>;                                                        \
    uint32_t ring = static_cast<uint32_t>((MSHADOW_B200_CHPOOL_RING_KB * 1024) / (tile_px * 4));               \
    if (ring < NS + 2) ring = NS + 2;                                                                          \
    if (ring > 16) ring = 16;                                                                                  \
    const size_t smem = static_cast<size_t>(ring) * tile_px * 4;                                               \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));  \
    int per_sm = 0;                                                                                            \
    MSHADOW_CUDA_CALL(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, st_threads, smem));       \
    const uint32_t slots = static_cast<uint32_t>(per_sm < 1 ? 1 : per_sm) * gpu_rt::CurrentDevice().sm_count;  \
    const uint32_t fixed = static_cast<uint32_t>(n) * tiles_per_plane;                                         \
    /* segments: whole waves of resident CTAs, weighed against the NS-1 halo channels each one re-reads */    \
    uint32_t segs = 1;                                                                                         \
    double best = 0.0;                                                                                         \
    for (uint32_t k = 1; k <= 16 && k * 2 * NS <= static_cast<uint32_t>(c); ++k) {                             \
      const uint64_t ctas = static_cast<uint64_t>(fixed) * k;                                                  \
      const uint64_t waves = (ctas + slots - 1) / slots;                                                       \
      const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots) /                     \
                         (1.0 + static_cast<double>((NS - 1) * k) / static_cast<double>(c));                   \
      if (eff > best + 1e-9) {                                                                                 \
        best = eff;                                                                                            \
        segs = k;                                                                                              \
      }                                                                                                        \
    }                                                                                                          \
    const uint32_t seg_len = (static_cast<uint32_t>(c) + segs - 1) / segs;                                     \
    const uint32_t nseg = (static_cast<uint32_t>(c) + seg_len - 1) / seg_len;                                  \
    gpu_rt::LaunchAfterDrain(kernel, dim3(fixed, nseg), dim3(st_threads), smem, stream, dst, src, static_cast<uint32_t>(c), plane, tile_px, \
                                                             tiles_per_plane, seg_len, ring,                   \
                                                             gpu_rt::StatusWord());                            \
  }
#define MSHADOW_B200_CHPOOL_PICK_(NS)                \
  if (staged) MSHADOW_B200_CHPOOL_STAGED_LAUNCH_(NS) \
  else if (vec) MSHADOW_B200_CHPOOL_LAUNCH_(NS, 4) else MSHADOW_B200_CHPOOL_LAUNCH_(NS, 1)
  switch (nsize) {
    case 1: MSHADOW_B200_CHPOOL_PICK_(1) break;
    case 3: MSHADOW_B200_CHPOOL_PICK_(3) break;
    case 5: MSHADOW_B200_CHPOOL_PICK_(5) break;
    case 7: MSHADOW_B200_CHPOOL_PICK_(7) break;
    default: MSHADOW_B200_CHPOOL_PICK_(9) break;
  }
#undef MSHADOW_B200_CHPOOL_PICK_
#undef MSHADOW_B200_CHPOOL_STAGED_LAUNCH_
#undef MSHADOW_B200_CHPOOL_LAUNCH_
  MSHADOW_CUDA_POST_KERNEL_CHECK(ChannelPoolKernel);
}

/*! \brief window sizes ChannelUnpoolKernel is instantiated for (stride 1, pad nsize/2) */
inline bool ChannelUnpoolSupported(int nsize, int stride, int pad) {
  return stride == 1 && pad == nsize / 2 && (nsize == 1 || nsize == 3 || nsize == 5 || nsize == 7);
}

/*! \brief dense (n, c, h, w) src, pooled, pooled gradient and dst; requires ChannelUnpoolSupported */
template <typename Reducer>
inline void ChannelUnpoolLaunch(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t n,
                                int64_t c, int64_t h, int64_t w, int nsize, cudaStream_t stream) {
  if (n == 0 || c == 0 || h * w == 0) return;
  if (std::is_same<Reducer, red::sum>::value) {
    // The gradient of a sum does not depend on the values: red::sum::PartialGrad is the constant 1, so
    // the reference's loop (mshadow/extension/channel_unpool.h:118-125) adds 1 * g over the pooled
    // channels c - pad .. c + pad in ascending order from 0 -- which is chpool<red::sum> of the pooled
    // gradient, term for term.  The staged pooling kernel serves it (0.77 -> 0.92 of copy bandwidth).
    ChannelPoolLaunch<red::sum>(dst, gpooled, n, c, h, w, nsize, stream);
    return;
  }
  const uint32_t plane = static_cast<uint32_t>(h * w);
  const bool vec = plane % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(pooled) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(gpooled) % 16 == 0;
  // staged variant: three planes per ring slot; the ring has to hold the nsize / 2 slots kept back
  // for the source values plus a few in flight inside 200 KB, so plane tiles shrink with the window
  if (vec && MSHADOW_B200_CHUNPOOL_STAGED && nsize >= 3 && c >= 2 * nsize) {
    const uint32_t least = static_cast<uint32_t>(nsize) / 2 + 3;
    uint32_t max_tile = (200u * 1024u / (least * 12u)) & ~3u;
    if (max_tile > kChUnpoolTilePx) max_tile = kChUnpoolTilePx;
    const uint32_t tiles_per_plane = (plane + max_tile - 1) / max_tile;
    const uint32_t tile_px = ((plane + tiles_per_plane - 1) / tiles_per_plane + 3) & ~3u;
    const uint32_t st_threads = (((tile_px / 4) + 31) & ~31u) + 32;
    const int64_t fixed64 = n * static_cast<int64_t>(tiles_per_plane);
    if (tile_px >= 128 && fixed64 < (int64_t(1) << 31)) {
      uint32_t ring = (200u * 1024u) / (tile_px * 12u);
      if (ring > 16) ring = 16;
      const size_t smem = static_cast<size_t>(ring) * tile_px * 12;
      const uint32_t fixed = static_cast<uint32_t>(fixed64);
#define MSHADOW_B200_CHUNPOOL_STAGED_LAUNCH_(NS)                                                               \
  {                                                                                                            \
    auto kernel = ChannelUnpoolStagedKernel<Reducer, NS>;                                                      \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));  \
    const uint32_t slots = static_cast<uint32_t>(gpu_rt::ResidentPerSM(kernel, st_threads, smem)) *            \
                           gpu_rt::CurrentDevice().sm_count;                                                   \
    /* segments: whole waves of resident CTAs, weighed against the NS-1 halo channels each one re-reads */    \
    uint32_t segs = 1;                                                                                         \
    double best = 0.0;                                                                                         \
    for (uint32_t k = 1; k <= 16 && k * 2 * NS <= static_cast<uint32_t>(c); ++k) {                             \
      const uint64_t ctas = static_cast<uint64_t>(fixed) * k;                                                  \
      const uint64_t waves = (ctas + slots - 1) / slots;                                                       \
      const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots) /                     \
                         (1.0 + static_cast<double>((NS - 1) * k) / static_cast<double>(c));                   \
      if (eff > best + 1e-9) {                                                                                 \
        best = eff;                                                                                            \
        segs = k;                                                                                              \
      }                                                                                                        \
    }                                                                                                          \
    const uint32_t seg_len = (static_cast<uint32_t>(c) + segs - 1) / segs;                                     \
    const uint32_t nseg = (static_cast<uint32_t>(c) + seg_len - 1) / seg_len;                                  \
    gpu_rt::LaunchAfterDrain(kernel, dim3(fixed, nseg), dim3(st_threads), smem, stream, dst, src, pooled, gpooled, \
                             static_cast<uint32_t>(c), plane, tile_px, tiles_per_plane, seg_len, ring,         \
                             gpu_rt::StatusWord());                                                            \
  }
      switch (nsize) {
        case 3: MSHADOW_B200_CHUNPOOL_STAGED_LAUNCH_(3) break;
        case 5: MSHADOW_B200_CHUNPOOL_STAGED_LAUNCH_(5) break;
        default: MSHADOW_B200_CHUNPOOL_STAGED_LAUNCH_(7) break;
      }
#undef MSHADOW_B200_CHUNPOOL_STAGED_LAUNCH_
      MSHADOW_CUDA_POST_KERNEL_CHECK(ChannelUnpoolStagedKernel);
      return;
    }
  }
  const uint32_t groups = plane / (vec ? 4 : 1);
  const int64_t items64 = n * static_cast<int64_t>(groups);
  CHECK_LT(items64, (int64_t(1) << 31)) << "ch_unpool: tensor too large for 32-bit indexing";
  const uint32_t items = static_cast<uint32_t>(items64);
  const uint32_t tiles = static_cast<uint32_t>(gpu_rt::CeilDiv(items, kPoolThreads));
#define MSHADOW_B200_CHUNPOOL_LAUNCH_(NS, LANES)                                                               \
  {                                                                                                            \
    auto kernel = ChannelUnpoolKernel<Reducer, NS, LANES>;                                                     \
    const uint32_t slots = static_cast<uint32_t>(gpu_rt::ResidentPerSM(kernel, kPoolThreads)) *               \
                           gpu_rt::CurrentDevice().sm_count;                                                   \
    /* channel segments that fill whole waves; each re-reads NS-1 halo channels of two tensors */            \
    uint32_t max_seg = static_cast<uint32_t>(c) / (8 * NS);                                                    \
    if (max_seg < 1) max_seg = 1;                                                                              \
    if (max_seg > 16) max_seg = 16;                                                                            \
    const uint32_t segs = pooldetail::WaveFriendlySegments(tiles, max_seg, slots);                            \
    const uint32_t seg_len = (static_cast<uint32_t>(c) + segs - 1) / segs;                                     \
    const uint32_t nseg = (static_cast<uint32_t>(c) + seg_len - 1) / seg_len;                                  \
    gpu_rt::LaunchAfterDrain(kernel, dim3(tiles, nseg), dim3(kPoolThreads), 0, stream, dst, src, pooled, gpooled, static_cast<uint32_t>(c), \
                                                            plane, groups, items, gpu_rt::FastDiv(groups),     \
                                                            seg_len);                                          \
  }
#define MSHADOW_B200_CHUNPOOL_PICK_(NS) \
  if (vec) MSHADOW_B200_CHUNPOOL_LAUNCH_(NS, 4) else MSHADOW_B200_CHUNPOOL_LAUNCH_(NS, 1)
  switch (nsize) {
    case 1: MSHADOW_B200_CHUNPOOL_PICK_(1) break;
    case 3: MSHADOW_B200_CHUNPOOL_PICK_(3) break;
    case 5: MSHADOW_B200_CHUNPOOL_PICK_(5) break;
    default: MSHADOW_B200_CHUNPOOL_PICK_(7) break;
  }
#undef MSHADOW_B200_CHUNPOOL_PICK_
#undef MSHADOW_B200_CHUNPOOL_LAUNCH_
  MSHADOW_CUDA_POST_KERNEL_CHECK(ChannelUnpoolKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_POOL_CUH_
