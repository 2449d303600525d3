/*
 * Permutations of a dense tensor's axes that move the LAST axis: `dst = transpose(src, axes)`
 * with axes[last] != last, and `dst = swapaxis<last, a2>(src)`.
 *
 * Through the generic map kernel such an assignment reads the source with a large stride
 * (one 4-byte element per 32-byte sector); the reference does the same
 * (mshadow/extension/transpose.h:64-72 and swapaxis.h:97-103 inside MapPlanKernel).  Here the
 * work is cut into 64 x 64 tiles spanned by the two axes that matter: the source's last axis
 * (contiguous on the way in) and the axis that becomes the result's last axis (contiguous on
 * the way out).  A CTA reads its tile row by row along the source's last axis, turns it round
 * in shared memory (65-element rows, so neither direction has bank conflicts) and writes it row
 * by row along the result's last axis: both sides move whole 128-byte lines.  All other axes
 * only select which tile a CTA works on.
 */
#ifndef MSHADOW_GPU_TRANSPOSE_CUH_
#define MSHADOW_GPU_TRANSPOSE_CUH_

#include "./runtime.h"

namespace mshadow {
namespace cuda {

const int kTransposeTile = MSHADOW_B200_TRANSPOSE_TILE;
const int kTransposeRows = 8;  // CTA = 32 x 8 threads: each thread moves 64 * 64 / 256 = 16 elements
const int kTransposeMaxOuter = 3;

/*! \brief how a permutation decomposes: two tile axes and up to three outer axes (in result order) */
struct TransposeGeom {
  uint32_t ext_in;     // extent of the source's last axis
  uint32_t ext_out;    // extent of the axis that becomes the result's last axis
  int64_t src_stride;  // source elements between neighbours along the `out` axis
  int64_t dst_stride;  // result elements between neighbours along the `in` axis
  int nouter;
  gpu_rt::FastDiv outer_div[kTransposeMaxOuter];  // extents of the outer axes, innermost first
  int64_t outer_src[kTransposeMaxOuter];          // their strides in the source
  int64_t outer_dst[kTransposeMaxOuter];          // ... and in the result
  gpu_rt::FastDiv tiles_in, tiles_out;            // tiles along the two tile axes
};

template <typename DType>
__global__ void __launch_bounds__(32 * kTransposeRows)
TiledPermuteKernel(DType *dst, const DType *src, TransposeGeom g) {
  __shared__ DType tile[kTransposeTile][kTransposeTile + 1];
  constexpr int kHalves = kTransposeTile / 32;  // a warp covers the tile's width in this many steps
  // blockIdx.x = ((outer index) * tiles_out + tile_out) * tiles_in + tile_in
  uint32_t t = blockIdx.x;
  uint32_t q = g.tiles_in.Quot(t);
  const uint32_t tile_in = t - q * g.tiles_in.div;
  t = q;
  q = g.tiles_out.Quot(t);
  const uint32_t tile_out = t - q * g.tiles_out.div;
  t = q;
  int64_t src_base = 0, dst_base = 0;
#pragma unroll
  for (int k = 0; k < kTransposeMaxOuter; ++k) {
    if (k < g.nouter) {
      q = g.outer_div[k].Quot(t);
      const uint32_t coord = t - q * g.outer_div[k].div;
      src_base += coord * g.outer_src[k];
      dst_base += coord * g.outer_dst[k];
      t = q;
    }
  }
  const uint32_t in0 = tile_in * kTransposeTile, out0 = tile_out * kTransposeTile;
  // read: threadIdx.x runs along the source's last axis; all of a thread's loads are issued
  // before the first is stored to shared memory
  DType held[kTransposeTile / kTransposeRows][kHalves];
#pragma unroll
  for (int k = 0; k < kTransposeTile / kTransposeRows; ++k) {
#pragma unroll
    for (int hf = 0; hf < kHalves; ++hf) {
      const uint32_t o = out0 + threadIdx.y + k * kTransposeRows, i = in0 + threadIdx.x + hf * 32;
      held[k][hf] = (o < g.ext_out && i < g.ext_in) ? __ldcs(src + src_base + o * g.src_stride + i) : DType();
    }
  }
#pragma unroll
  for (int k = 0; k < kTransposeTile / kTransposeRows; ++k) {
#pragma unroll
    for (int hf = 0; hf < kHalves; ++hf) tile[threadIdx.y + k * kTransposeRows][threadIdx.x + hf * 32] = held[k][hf];
  }
  __syncthreads();
  // write: threadIdx.x runs along the result's last axis
#pragma unroll
  for (int k = 0; k < kTransposeTile / kTransposeRows; ++k) {
#pragma unroll
    for (int hf = 0; hf < kHalves; ++hf) {
      const uint32_t i = in0 + threadIdx.y + k * kTransposeRows, o = out0 + threadIdx.x + hf * 32;
      if (o < g.ext_out && i < g.ext_in) {
        __stcs(dst + dst_base + i * g.dst_stride + o, tile[threadIdx.x + hf * 32][threadIdx.y + k * kTransposeRows]);
      }
    }
  }
}

/*!
 * \brief dst = src with result axis k taken from source axis axes[k]; both dense, `dim` <= 5,
 *  axes[dim-1] != dim-1.  Returns false (and launches nothing) when the shape does not fit the
 *  kernel's 32-bit tile counter; the caller then uses the generic kernel.
 */
template <typename DType, int dim>
inline bool TiledPermuteLaunch(DType *dst, const DType *src, const Shape<dim> &src_shape, const Shape<dim> &axes,
                               cudaStream_t stream) {
  static_assert(dim >= 2 && dim <= kTransposeMaxOuter + 2, "TiledPermute: 2 to 5 dimensions");
  int64_t src_stride[dim], dst_stride[dim];
  Shape<dim> dst_shape;
  for (int k = 0; k < dim; ++k) dst_shape[k] = src_shape[axes[k]];
  src_stride[dim - 1] = dst_stride[dim - 1] = 1;
  for (int k = dim - 2; k >= 0; --k) {
    src_stride[k] = src_stride[k + 1] * src_shape[k + 1];
    dst_stride[k] = dst_stride[k + 1] * dst_shape[k + 1];
  }
  const int a_out = axes[dim - 1];  // source axis that becomes the result's last axis
  int pos_in = 0;                   // where the source's last axis lands in the result
  for (int k = 0; k < dim; ++k) {
    if (static_cast<int>(axes[k]) == dim - 1) pos_in = k;
  }
  TransposeGeom g;
  g.ext_in = src_shape[dim - 1];
  g.ext_out = src_shape[a_out];
  g.src_stride = src_stride[a_out];
  g.dst_stride = dst_stride[pos_in];
  g.nouter = 0;
  int64_t outer_count = 1;
  for (int k = dim - 2; k >= 0; --k) {  // result axes other than the two tile axes, innermost first
    if (k == pos_in) continue;
    g.outer_div[g.nouter] = gpu_rt::FastDiv(dst_shape[k]);
    g.outer_src[g.nouter] = src_stride[axes[k]];
    g.outer_dst[g.nouter] = dst_stride[k];
    outer_count *= dst_shape[k];
    ++g.nouter;
  }
  const uint32_t tiles_in = (g.ext_in + kTransposeTile - 1) / kTransposeTile;
  const uint32_t tiles_out = (g.ext_out + kTransposeTile - 1) / kTransposeTile;
  const int64_t ctas = outer_count * tiles_in * tiles_out;
  if (ctas == 0) return true;
  if (ctas >= (int64_t(1) << 31)) return false;
  g.tiles_in = gpu_rt::FastDiv(tiles_in);
  g.tiles_out = gpu_rt::FastDiv(tiles_out);
  TiledPermuteKernel<DType><<<static_cast<unsigned>(ctas), dim3(32, kTransposeRows), 0, stream>>>(dst, src, g);
  MSHADOW_CUDA_POST_KERNEL_CHECK(TiledPermuteKernel);
  return true;
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_TRANSPOSE_CUH_
