/*
 * The fused element-wise kernel: dst(y,x) <Saver>= plan(y,x) over a matrix view of the
 * destination.  Replaces the reference's MapPlanKernel / MapPlanLargeKernel
 * (mshadow/cuda/tensor_gpu-inl.cuh:67-120), which evaluate one element per thread with a
 * 4-byte access and an integer divide per element.
 *
 * Two kernels:
 *   MapPackKernel    every operand is read and the destination written in 16-byte groups.
 *                    Each thread owns kUnroll groups per sweep, issues all of their loads
 *                    first (so that several 128-bit requests per operand are in flight per
 *                    thread) and stores afterwards.  Rows whose length is not a multiple of
 *                    the group width finish with a scalar tail.  Dense operands are walked
 *                    as one long row, which removes the (y,x) split altogether.
 *                    With kSrcPack = false the same kernel serves expressions that only know
 *                    Eval(y,x) but are cheap per element (expr::LaneInfo): a thread puts its
 *                    group together from kLanes element evaluations, so the index split and
 *                    the store are still paid once per 16 bytes.
 *   MapScalarKernel  the general fallback: plans that only know Eval(y,x) and walk other
 *                    elements per result (axis reductions), user-defined expressions,
 *                    misaligned or odd-pitched destinations.
 * Both are grid-stride loops over a grid sized to the number of SMs; (y,x) is recovered
 * from the linear work index by multiplication with a precomputed reciprocal.
 *
 * The kernels are HBM-bandwidth bound: config "A*B + 0.5*C through a sigmoid plus bias"
 * moves 16 bytes per element and does ~40 flops on it.
 */
#ifndef MSHADOW_GPU_MAP_CUH_
#define MSHADOW_GPU_MAP_CUH_

#include "./runtime.h"

namespace mshadow {
namespace cuda {

const int kMapThreads = MSHADOW_B200_MAP_THREADS;
const int kMapUnroll = MSHADOW_B200_MAP_UNROLL;
const int kMapScalarUnroll = MSHADOW_B200_MAP_SCALAR_UNROLL;
/*! \brief resident CTAs per SM that the grid is sized for */
const int kMapCtasPerSM = 8;

/*!
 * \tparam kSrcPack the source plan serves 16-byte groups (EvalPack); if false the group is put
 *  together from kLanes element evaluations and only the destination is accessed 128 bits wide
 */
template <typename Saver, typename DPlan, typename SPlan, typename DType, bool kSrcPack = true>
__global__ void __launch_bounds__(kMapThreads)
MapPackKernel(DPlan dst, const SPlan src, uint32_t rows, uint32_t cols, uint32_t packs_per_row,
              gpu_rt::FastDiv row_of_pack) {
  constexpr int kLanes = expr::Pack<DType>::kLanes;
  gpu_rt::GridDependencySync();
  const uint32_t total = rows * packs_per_row;
  const uint32_t step = gridDim.x * kMapThreads;
  for (uint32_t base = blockIdx.x * kMapThreads + threadIdx.x; base < total;
       base += step * kMapUnroll) {
    expr::Pack<DType> val[kMapUnroll];
    uint32_t ys[kMapUnroll], xs[kMapUnroll];
#pragma unroll
    for (int u = 0; u < kMapUnroll; ++u) {
      const uint32_t i = base + u * step;
      if (i < total) {
        const uint32_t y = rows == 1 ? 0 : row_of_pack.Quot(i);
        const uint32_t x = (i - y * packs_per_row) * kLanes;
        ys[u] = y;
        xs[u] = x;
        expr::Pack<DType> v;
        if constexpr (kSrcPack) {
          v = src.EvalPack(y, x);
        } else {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) v.v[l] = src.Eval(y, x + l);
        }
        if (!std::is_same<Saver, sv::saveto>::value) {
          expr::Pack<DType> d = dst.EvalPack(y, x);
#pragma unroll
          for (int l = 0; l < kLanes; ++l) Saver::Save(d.v[l], v.v[l]);
          v = d;
        }
        val[u] = v;
      }
    }
#pragma unroll
    for (int u = 0; u < kMapUnroll; ++u) {
      if (base + u * step < total) dst.StorePack(ys[u], xs[u], val[u]);
    }
  }
  // columns past the last full group of each row
  const uint32_t tail = cols - packs_per_row * kLanes;
  if (tail != 0) {
    const uint32_t ntail = rows * tail;
    for (uint32_t i = blockIdx.x * kMapThreads + threadIdx.x; i < ntail; i += step) {
      const uint32_t y = i / tail;
      const uint32_t x = packs_per_row * kLanes + (i - y * tail);
      Saver::Save(dst.REval(y, x), src.Eval(y, x));
    }
  }
}

template <typename Saver, typename DPlan, typename SPlan, typename DType>
__global__ void __launch_bounds__(kMapThreads)
MapScalarKernel(DPlan dst, const SPlan src, uint32_t rows, uint32_t cols, gpu_rt::FastDiv row_of_elem) {
  gpu_rt::GridDependencySync();
  const uint32_t total = rows * cols;
  const uint32_t step = gridDim.x * kMapThreads;
  for (uint32_t base = blockIdx.x * kMapThreads + threadIdx.x; base < total;
       base += step * kMapScalarUnroll) {
    DType val[kMapScalarUnroll];
    uint32_t ys[kMapScalarUnroll], xs[kMapScalarUnroll];
#pragma unroll
    for (int u = 0; u < kMapScalarUnroll; ++u) {
      const uint32_t i = base + u * step;
      if (i < total) {
        const uint32_t y = row_of_elem.Quot(i);
        const uint32_t x = i - y * cols;
        ys[u] = y;
        xs[u] = x;
        val[u] = src.Eval(y, x);
      }
    }
#pragma unroll
    for (int u = 0; u < kMapScalarUnroll; ++u) {
      if (base + u * step < total) Saver::Save(dst.REval(ys[u], xs[u]), val[u]);
    }
  }
}

/*!
 * \brief grid for a grid-stride kernel: enough CTAs for the work, but never more than the
 *  device keeps resident at once for this kernel (registers decide), so that no partly
 *  filled second wave trails behind
 */
template <typename Kernel>
inline int MapGridSize(int64_t work_items, Kernel kernel) {
  int per_sm = gpu_rt::ResidentPerSM(kernel, kMapThreads);
  if (per_sm > kMapCtasPerSM) per_sm = kMapCtasPerSM;
  const int resident = per_sm * gpu_rt::CurrentDevice().sm_count;
  const int want = gpu_rt::CeilDiv(work_items, static_cast<int64_t>(kMapThreads) * kMapUnroll);
  return want < 1 ? 1 : (want < resident ? want : resident);
}

/*!
 * \brief launch the 128-bit path.  `flat` says that all operands are dense and the
 *  expression is position-independent, so the matrix is walked as a single row.
 */
template <typename Saver, typename DType, bool kSrcPack = true, typename DPlan, typename SPlan>
inline void MapPlanPacked(DPlan dplan, const SPlan &splan, Shape<2> dshape, bool flat,
                          cudaStream_t stream) {
  constexpr int kLanes = expr::Pack<DType>::kLanes;
  const int64_t count = static_cast<int64_t>(dshape[0]) * dshape[1];
  if (count == 0) return;
  CHECK_LT(count, (int64_t(1) << 31)) << "MapExp: tensor too large for 32-bit indexing";
  uint32_t rows = dshape[0], cols = dshape[1];
  if (flat) {
    rows = 1;
    cols = static_cast<uint32_t>(count);
  }
  const uint32_t ppr = cols / kLanes;
  const int64_t work = static_cast<int64_t>(rows) * (ppr == 0 ? 1 : ppr);
  auto kernel = MapPackKernel<Saver, DPlan, SPlan, DType, kSrcPack>;
  gpu_rt::LaunchAfterDrain(kernel, dim3(MapGridSize(work, kernel)), dim3(kMapThreads), 0, stream, dplan, splan, rows,
                           cols, ppr, gpu_rt::FastDiv(ppr == 0 ? 1 : ppr));
  MSHADOW_CUDA_POST_KERNEL_CHECK(MapPackKernel);
}

/*! \brief launch the general element-at-a-time path */
template <typename Saver, typename DType, typename DPlan, typename SPlan>
inline void MapPlanScalar(DPlan dplan, const SPlan &splan, Shape<2> dshape, cudaStream_t stream) {
  const int64_t count = static_cast<int64_t>(dshape[0]) * dshape[1];
  if (count == 0) return;
  CHECK_LT(count, (int64_t(1) << 31)) << "MapExp: tensor too large for 32-bit indexing";
  auto kernel = MapScalarKernel<Saver, DPlan, SPlan, DType>;
  gpu_rt::LaunchAfterDrain(kernel, dim3(MapGridSize(count, kernel)), dim3(kMapThreads), 0, stream, dplan, splan,
                           static_cast<uint32_t>(dshape[0]), static_cast<uint32_t>(dshape[1]),
                           gpu_rt::FastDiv(static_cast<uint32_t>(dshape[1])));
  MSHADOW_CUDA_POST_KERNEL_CHECK(MapScalarKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_MAP_CUH_
