/*
 * Patch <-> column conversion ("im2col" and its transpose) as dedicated kernels.
 *
 * In the matrix of unpack_patch2col, row (c, ky, kx) restricted to the columns of image n is
 * one contiguous run of o_height * o_width values, all taken from plane (n, c) shifted by
 * (ky, kx).
 *
 *   unpack_patch2col  a CTA stages one plane in shared memory and writes its psize_y * psize_x
 *                     runs with fully coalesced stores: the plane is read from HBM once instead
 *                     of once per patch position, with one index split per element instead of
 *                     four.
 *   pack_col2patch    every matrix entry belongs to exactly one image element, so nothing is
 *                     staged: one thread per image element gathers the element's covering
 *                     patches in the reference's order (patch rows ascending, then patch columns
 *                     ascending: mshadow/extension/pack_col2patch.h:126-136), which makes the
 *                     sums bit-identical.  The kernel is bound by instruction issue, not by
 *                     memory, so the work per tap is cut to a predicate, a load and an add: the
 *                     plane is fixed per CTA (its offsets live in uniform registers), the tap
 *                     loops unroll for compile-time patch sizes, and unit stride, the common
 *                     case, needs no division.  Measured alternatives, 3 x 3 patches on
 *                     (64, 64, 56, 56): adding the runs into a staged plane pass by pass 29 %,
 *                     staging the runs of a band of rows and summing out of shared memory
 *                     23-49 % (best with the smallest bands), the generic path 47 % of copy
 *                     bandwidth.
 *
 * The generic expression path (mshadow/cuda/tensor_gpu-inl.cuh:67-120 with the plans of
 * mshadow/extension/unpack_patch2col.h:115-133 and pack_col2patch.h:108-140 in the reference)
 * remains the route for unpack_patch2col of planes that do not fit shared memory or are tiny,
 * and for pack_col2patch with dilation.
 */
#ifndef MSHADOW_GPU_PATCH_CUH_
#define MSHADOW_GPU_PATCH_CUH_

#include "../engine/fastdiv.h"
#include "./runtime.h"

namespace mshadow {
namespace cuda {

const int kPatchThreads = 256;
/*! \brief planes smaller than this many elements leave most of a CTA idle: generic path */
const uint32_t kPatchMinPlane = 512;

struct PatchGeom {
  uint32_t channels, h, w, oh, ow, psy, psx, sy, sx, dy, dx;
};

/*! \brief whether a plane of h x w elements of `elem_bytes` can be staged */
inline bool PatchPlaneFits(uint32_t h, uint32_t w, size_t elem_bytes) {
  const uint64_t elems = static_cast<uint64_t>(h) * w;
  return elems >= kPatchMinPlane && elems * elem_bytes + 1024 <= static_cast<uint64_t>(gpu_rt::CurrentDevice().max_smem_optin);
}

template <typename Saver, typename DType>
__global__ void __launch_bounds__(kPatchThreads)
UnpackPatchPlaneKernel(DType *__restrict__ mat, int64_t ld_mat, const DType *__restrict__ img, int64_t ld_img,
                       PatchGeom g, gpu_rt::FastDiv by_w, gpu_rt::FastDiv by_ow, gpu_rt::FastDiv by_channels) {
  extern __shared__ __align__(16) unsigned char patch_smem[];
  DType *plane = reinterpret_cast<DType *>(patch_smem);
  const uint32_t p = blockIdx.x;  // plane (n, c)
  const uint32_t n = by_channels.Quot(p), c = p - n * g.channels;
  const uint32_t hw = g.h * g.w, seg = g.oh * g.ow;
  const DType *src = img + static_cast<int64_t>(p) * g.h * ld_img;
  for (uint32_t i = threadIdx.x; i < hw; i += kPatchThreads) {
    const uint32_t y = by_w.Quot(i);
    plane[i] = gpu_rt::LoadCg(src + static_cast<int64_t>(y) * ld_img + (i - y * g.w));
  }
  __syncthreads();
  const uint32_t row_step = g.sy * g.w;
  constexpr uint32_t kGroup = 16 / sizeof(DType);
  struct alignas(16) Group {
    DType v[kGroup];
  };
  // runs that start and end on 16-byte boundaries leave in 16-byte groups: one index split and one
  // store per group (with 4-byte stores the kernel was bound by instruction issue, not by memory).
  // Thread t then reads shared-memory words 4t .. 4t+3, four to a bank across the warp; a
  // conflict-free rotated read order was measured and changed nothing.
  const bool wide = MSHADOW_B200_UNPACK_WIDE && seg % kGroup == 0 && ld_mat % kGroup == 0 && g.ow >= kGroup &&
                    reinterpret_cast<uintptr_t>(mat) % 16 == 0;
  const uint32_t next_row = row_step - g.ow * g.sx;  // added to a plane index that passed the end of a patch row
  for (uint32_t ky = 0, k = 0; ky < g.psy; ++ky) {
    for (uint32_t kx = 0; kx < g.psx; ++kx, ++k) {
      DType *out = mat + (static_cast<int64_t>(c) * g.psy * g.psx + k) * ld_mat + static_cast<int64_t>(n) * seg;
      const uint32_t off = ky * g.dy * g.w + kx * g.dx;
      if (wide) {
#pragma unroll 2
        for (uint32_t e = threadIdx.x * kGroup; e < seg; e += kPatchThreads * kGroup) {
          const uint32_t oy = by_ow.Quot(e);
          const uint32_t ox = e - oy * g.ow, at = off + oy * row_step + ox * g.sx;
          Group grp;
          // a group may run over the end of its patch row (at most once: ow >= kGroup); no branch, since
          // nearly every warp holds such a group and would execute both sides
#pragma unroll
          for (uint32_t l = 0; l < kGroup; ++l) {
            grp.v[l] = plane[at + l * g.sx + (ox + l >= g.ow ? next_row : 0u)];
          }
          Group *dst = reinterpret_cast<Group *>(out + e);
          if (!std::is_same<Saver, sv::saveto>::value) {
            Group old = *dst;
#pragma unroll
            for (uint32_t l = 0; l < kGroup; ++l) Saver::Save(old.v[l], grp.v[l]);
            grp = old;
          }
          *dst = grp;
        }
      } else {
#pragma unroll 4
        for (uint32_t e = threadIdx.x; e < seg; e += kPatchThreads) {
          const uint32_t oy = by_ow.Quot(e);
          Saver::Save(out[e], plane[off + oy * row_step + (e - oy * g.ow) * g.sx]);
        }
      }
    }
  }
}

/*!
 * \brief pack_col2patch without dilation, one thread per image element; blockIdx.x is the plane,
 *  blockIdx.y the block of kPatchThreads elements within it.
 * \tparam PSY, PSX patch size known at compile time (the tap loops unroll), or 0 for a size read from `g`
 * \tparam kUnit both strides are 1: patch (py, px) = (y - ky, x - kx), valid when inside the patch grid
 */
template <typename Saver, typename DType, int PSY, int PSX, bool kUnit>
__global__ void __launch_bounds__(kPatchThreads)
PackPatchKernel(DType *__restrict__ img, int64_t ld_img, const DType *__restrict__ mat, int64_t ld_mat, PatchGeom g,
                gpu_rt::FastDiv by_w, gpu_rt::FastDiv by_channels, expr::FastDiv by_sy, expr::FastDiv by_sx) {
  const uint32_t i = blockIdx.y * kPatchThreads + threadIdx.x;
  if (i >= g.h * g.w) return;
  const uint32_t psy = PSY ? PSY : g.psy, psx = PSX ? PSX : g.psx;
  const uint32_t p = blockIdx.x;
  const uint32_t n = by_channels.Quot(p), c = p - n * g.channels;
  const uint32_t y = by_w.Quot(i), x = i - y * g.w;
  // the matrix has fewer than 2^31 elements (the launcher checks), so element offsets from its base
  // fit 32 bits; `first` is the plane's first run at the columns of image n
  const uint32_t ld = static_cast<uint32_t>(ld_mat);
  const uint32_t first = c * psy * psx * ld + n * g.oh * g.ow;
  DType res = static_cast<DType>(0);
  if constexpr (kUnit) {
    const uint32_t at = first + y * g.ow + x;  // tap (ky, kx) lies k * ld - ky * ow - kx, a launch constant, further on
    if constexpr (PSY > 0 && PSX > 0) {
      // all loads of the element first (predicated, independent), then the adds in the reference's order
      DType v[PSY * PSX];
      bool ok[PSY * PSX];
#pragma unroll
      for (uint32_t ky = 0; ky < PSY; ++ky) {
        const bool row_ok = y - ky < g.oh;  // unsigned: also false for y < ky
#pragma unroll
        for (uint32_t kx = 0; kx < PSX; ++kx) {
          const uint32_t k = ky * PSX + kx;
          ok[k] = row_ok && x - kx < g.ow;
          v[k] = ok[k] ? gpu_rt::LoadCg(mat + (at + (k * ld - (ky * g.ow + kx)))) : static_cast<DType>(0);
        }
      }
#pragma unroll
      for (int k = PSY * PSX - 1; k >= 0; --k) {
        if (ok[k]) res = detail::AddRN<DType>(res, v[k]);
      }
    } else {
      for (uint32_t ky = psy; ky-- > 0;) {
        const bool row_ok = y - ky < g.oh;
        for (uint32_t kx = psx; kx-- > 0;) {
          if (row_ok && x - kx < g.ow) {
            res = detail::AddRN<DType>(res, gpu_rt::LoadCg(mat + (at + ((ky * psx + kx) * ld - (ky * g.ow + kx)))));
          }
        }
      }
    }
  } else {
#pragma unroll
    for (uint32_t ky = psy; ky-- > 0;) {
      uint32_t py;
      const bool row_ok = y >= ky && by_sy.DivMod(y - ky, &py) == 0 && py < g.oh;
#pragma unroll
      for (uint32_t kx = psx; kx-- > 0;) {
        uint32_t px;
        if (row_ok && x >= kx && by_sx.DivMod(x - kx, &px) == 0 && px < g.ow) {
          res = detail::AddRN<DType>(res, gpu_rt::LoadCg(mat + (first + (ky * psx + kx) * ld + py * g.ow + px)));
        }
      }
    }
  }
  Saver::Save(img[(static_cast<int64_t>(p) * g.h + y) * ld_img + x], res);
}

namespace patchdetail {
template <typename Kernel>
inline void AllowSmem(Kernel kernel, size_t smem) {
  if (smem > 48 * 1024) {
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           gpu_rt::CurrentDevice().max_smem_optin));
  }
}
}  // namespace patchdetail

/*! \brief mat <Saver>= unpack_patch2col(img): `planes` = images * channels planes of g.h x g.w */
template <typename Saver, typename DType>
inline void UnpackPatchLaunch(DType *mat, int64_t ld_mat, const DType *img, int64_t ld_img, int64_t planes,
                              const PatchGeom &g, cudaStream_t stream) {
  if (planes == 0) return;
  const size_t smem = static_cast<size_t>(g.h) * g.w * sizeof(DType);
  auto kernel = UnpackPatchPlaneKernel<Saver, DType>;
  patchdetail::AllowSmem(kernel, smem);
  kernel<<<static_cast<unsigned>(planes), kPatchThreads, smem, stream>>>(mat, ld_mat, img, ld_img, g, gpu_rt::FastDiv(g.w),
                                                                         gpu_rt::FastDiv(g.ow), gpu_rt::FastDiv(g.channels));
  MSHADOW_CUDA_POST_KERNEL_CHECK(UnpackPatchPlaneKernel);
}

/*! \brief whether PackPatchLaunch can take the shape (the grid's second dimension holds the blocks of a plane) */
inline bool PackPatchSupported(uint32_t h, uint32_t w) {
  return (static_cast<uint64_t>(h) * w + kPatchThreads - 1) / kPatchThreads <= 65535;
}

/*! \brief img <Saver>= pack_col2patch(mat), no dilation */
template <typename Saver, typename DType>
inline void PackPatchLaunch(DType *img, int64_t ld_img, const DType *mat, int64_t ld_mat, int64_t planes,
                            const PatchGeom &g, cudaStream_t stream) {
  if (planes == 0 || g.h * g.w == 0) return;
  const dim3 grid(static_cast<unsigned>(planes), (g.h * g.w + kPatchThreads - 1) / kPatchThreads);
  const bool unit = g.sy == 1 && g.sx == 1;
#define MSHADOW_B200_PACK_PATCH_LAUNCH_(PSY, PSX)                                                             \
  {                                                                                                           \
    if (unit) {                                                                                               \
      PackPatchKernel<Saver, DType, PSY, PSX, true><<<grid, kPatchThreads, 0, stream>>>(                      \
          img, ld_img, mat, ld_mat, g, gpu_rt::FastDiv(g.w), gpu_rt::FastDiv(g.channels), expr::FastDiv(1),   \
          expr::FastDiv(1));                                                                                  \
    } else {                                                                                                  \
      PackPatchKernel<Saver, DType, PSY, PSX, false><<<grid, kPatchThreads, 0, stream>>>(                     \
          img, ld_img, mat, ld_mat, g, gpu_rt::FastDiv(g.w), gpu_rt::FastDiv(g.channels), expr::FastDiv(g.sy), \
          expr::FastDiv(g.sx));                                                                               \
    }                                                                                                         \
  }
  if (g.psy == 3 && g.psx == 3) MSHADOW_B200_PACK_PATCH_LAUNCH_(3, 3)
  else if (g.psy == 5 && g.psx == 5) MSHADOW_B200_PACK_PATCH_LAUNCH_(5, 5)
  else if (g.psy == 2 && g.psx == 2) MSHADOW_B200_PACK_PATCH_LAUNCH_(2, 2)
  else if (g.psy == 1 && g.psx == 1) MSHADOW_B200_PACK_PATCH_LAUNCH_(1, 1)
  else MSHADOW_B200_PACK_PATCH_LAUNCH_(0, 0)
#undef MSHADOW_B200_PACK_PATCH_LAUNCH_
  MSHADOW_CUDA_POST_KERNEL_CHECK(PackPatchKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_PATCH_CUH_
