/*
 * Patch <-> column conversion for convolutions ("im2col" and its transpose):
 *
 *   unpack_patch2col(img, psize_y, psize_x, pstride[_y, _x], pdilate[_y, _x])
 *       img (.., c, h, w)  ->  matrix (psize_y * psize_x * c,  o_height * o_width * n)
 *       row (c, ky, kx), column (n, oy, ox) holds img(n, c, oy * stride_y + ky * dilate_y,
 *       ox * stride_x + kx * dilate_x)
 *   pack_col2patch(mat, imshape, psize_y, psize_x, pstride[_y, _x], pdilate[_y, _x])
 *       the transpose: every image element collects the matrix entries of all patches that
 *       cover it, summed patch row by patch row
 *
 * Signatures, shapes, checks and the order of the additions follow dmlc/mshadow's
 * mshadow/extension/unpack_patch2col.h (:15-148) and pack_col2patch.h (:15-151).  The plans split
 * their row and column indices by multiplication with precomputed reciprocals instead of the
 * six to ten integer divisions per element that the reference's Eval performs.
 */
#ifndef MSHADOW_EXTENSION_PATCH_H_
#define MSHADOW_EXTENSION_PATCH_H_

#include "../engine/check.h"
#include "../engine/fastdiv.h"
#if MSHADOW_USE_CUDA && defined(__CUDACC__)
#include "../gpu/patch.cuh"
#endif

namespace mshadow {
namespace expr {

// ------------------------------------------------------------------------------------------
// unpack_patch2col
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int srcdim>
struct UnpackPatchToColXExp : public MakeTensorExp<UnpackPatchToColXExp<SrcExp, DType, srcdim>, SrcExp, 2, DType> {
  const SrcExp &img_;
  index_t psize_y_, psize_x_, pstride_y_, pstride_x_, pdilate_y_, pdilate_x_;
  index_t i_channel_, i_height_, i_width_;
  UnpackPatchToColXExp(const SrcExp &img, index_t psize_y, index_t psize_x, index_t pstride_y, index_t pstride_x,
                       index_t pdilate_y, index_t pdilate_x)
      : img_(img), psize_y_(psize_y), psize_x_(psize_x), pstride_y_(pstride_y), pstride_x_(pstride_x),
        pdilate_y_(pdilate_y), pdilate_x_(pdilate_x) {
    const Shape<srcdim> imshape = ShapeCheck<srcdim, SrcExp>::Check(img_);
    CHECK(imshape[srcdim - 1] >= psize_x && imshape[srcdim - 2] >= psize_y)
        << "UnpackPatchToCol:image shape smaller than patch size";
    CHECK(psize_y > 0 && psize_x > 0 && pstride_y > 0 && pstride_x > 0 && pdilate_y > 0 && pdilate_x > 0)
        << "UnpackPatchToCol: patch size, stride and dilation must be positive";
    i_channel_ = imshape[srcdim - 3];
    i_height_ = imshape[srcdim - 2];
    i_width_ = imshape[srcdim - 1];
    const index_t num = imshape.ProdShape(0, srcdim - 3);
    const index_t o_height = (i_height_ - (pdilate_y * (psize_y - 1) + 1)) / pstride_y + 1;
    const index_t o_width = (i_width_ - (pdilate_x * (psize_x - 1) + 1)) / pstride_x + 1;
    this->shape_[1] = o_height * o_width * num;
    this->shape_[0] = psize_y * psize_x * i_channel_;
    const uint64_t total = static_cast<uint64_t>(this->shape_[0]) * this->shape_[1];
    CHECK_LT(total, (uint64_t(1) << 31)) << "UnpackPatchToCol: result too large for 32-bit indexing";
  }
};

template <typename SrcExp, typename DType, int etype>
inline UnpackPatchToColXExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> unpack_patch2col(
    const Exp<SrcExp, DType, etype> &img, index_t psize_y, index_t psize_x, index_t pstride_y, index_t pstride_x,
    index_t pdilate_y, index_t pdilate_x) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim >= 3>::Error_Expression_Does_Not_Meet_Dimension_Req();
  return UnpackPatchToColXExp<SrcExp, DType, ExpInfo<SrcExp>::kDim>(img.self(), psize_y, psize_x, pstride_y, pstride_x,
                                                                    pdilate_y, pdilate_x);
}
template <typename SrcExp, typename DType, int etype>
inline UnpackPatchToColXExp<SrcExp, DType, ExpInfo<SrcExp>::kDim> unpack_patch2col(
    const Exp<SrcExp, DType, etype> &img, index_t psize_y, index_t psize_x, index_t pstride, index_t pdilate) {
  return unpack_patch2col(img, psize_y, psize_x, pstride, pstride, pdilate, pdilate);
}

template <typename SrcExp, typename DType, int srcdim>
class Plan<UnpackPatchToColXExp<SrcExp, DType, srcdim>, DType> {
 public:
  explicit Plan(const UnpackPatchToColXExp<SrcExp, DType, srcdim> &e)
      : src_(MakePlan(e.img_)), by_psize_x_(e.psize_x_), by_psize_y_(e.psize_y_), pstride_y_(e.pstride_y_),
        pstride_x_(e.pstride_x_), pdilate_y_(e.pdilate_y_), pdilate_x_(e.pdilate_x_), i_channel_(e.i_channel_),
        i_height_(e.i_height_), i_width_(e.i_width_),
        by_o_height_((e.i_height_ - (e.pdilate_y_ * (e.psize_y_ - 1) + 1)) / e.pstride_y_ + 1),
        by_o_width_((e.i_width_ - (e.pdilate_x_ * (e.psize_x_ - 1) + 1)) / e.pstride_x_ + 1) {}
  /*! \brief row i = (c, ky, kx), column j = (n, oy, ox) */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t idivp, c, jdivw, n;
    const uint32_t x_offset = by_psize_x_.DivMod(i, &idivp) * pdilate_x_;
    const uint32_t y_offset = by_psize_y_.DivMod(idivp, &c) * pdilate_y_;
    const uint32_t x = by_o_width_.DivMod(j, &jdivw) * pstride_x_ + x_offset;
    const uint32_t y = by_o_height_.DivMod(jdivw, &n) * pstride_y_ + y_offset;
    if (x < static_cast<uint32_t>(i_width_) && y < static_cast<uint32_t>(i_height_)) {
      return src_.Eval((n * i_channel_ + c) * i_height_ + y, x);
    }
    return DType(0.0f);
  }
#ifdef __CUDACC__
  /*!
   * \brief a 16-byte group of one matrix row: row and first column are split once, the following
   *  columns step (ox, oy, n) forward; the image needs no alignment since it is read by element
   */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    uint32_t idivp, c, jdivw, n;
    const uint32_t x_offset = by_psize_x_.DivMod(i, &idivp) * pdilate_x_;
    const uint32_t y_offset = by_psize_y_.DivMod(idivp, &c) * pdilate_y_;
    uint32_t ox = by_o_width_.DivMod(j, &jdivw);
    uint32_t oy = by_o_height_.DivMod(jdivw, &n);
    Pack<DType> r;
#pragma unroll
    for (int l = 0; l < Pack<DType>::kLanes; ++l) {
      const uint32_t x = ox * pstride_x_ + x_offset, y = oy * pstride_y_ + y_offset;
      r.v[l] = (x < static_cast<uint32_t>(i_width_) && y < static_cast<uint32_t>(i_height_))
                   ? src_.Eval((n * i_channel_ + c) * i_height_ + y, x)
                   : DType(0.0f);
      if (++ox == by_o_width_.div) {
        ox = 0;
        if (++oy == by_o_height_.div) {
          oy = 0;
          ++n;
        }
      }
    }
    return r;
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const FastDiv by_psize_x_, by_psize_y_;
  const index_t pstride_y_, pstride_x_, pdilate_y_, pdilate_x_, i_channel_, i_height_, i_width_;
  const FastDiv by_o_height_, by_o_width_;
};

// served in 16-byte groups whatever the image's alignment (the image is read by element)
template <typename SrcExp, typename DType, int srcdim>
struct PackInfo<UnpackPatchToColXExp<SrcExp, DType, srcdim> > {
  static const bool kPass = true;
};
template <typename SrcExp, typename DType, int srcdim>
struct PackAlign<UnpackPatchToColXExp<SrcExp, DType, srcdim> > {
  inline static bool Check(const UnpackPatchToColXExp<SrcExp, DType, srcdim> &) { return true; }
};

// ------------------------------------------------------------------------------------------
// pack_col2patch
// ------------------------------------------------------------------------------------------
template <typename SrcExp, typename DType, int dstdim>
struct PackColToPatchXExp : public MakeTensorExp<PackColToPatchXExp<SrcExp, DType, dstdim>, SrcExp, dstdim, DType> {
  const SrcExp &src_;
  index_t psize_y_, psize_x_, pstride_y_, pstride_x_, pdilate_y_, pdilate_x_;
  PackColToPatchXExp(const SrcExp &src, Shape<dstdim> imshape, index_t psize_y, index_t psize_x, index_t pstride_y,
                     index_t pstride_x, index_t pdilate_y, index_t pdilate_x)
      : src_(src), psize_y_(psize_y), psize_x_(psize_x), pstride_y_(pstride_y), pstride_x_(pstride_x),
        pdilate_y_(pdilate_y), pdilate_x_(pdilate_x) {
    CHECK(psize_y > 0 && psize_x > 0 && pstride_y > 0 && pstride_x > 0 && pdilate_y > 0 && pdilate_x > 0)
        << "PackColToPatch: patch size, stride and dilation must be positive";
    this->shape_ = imshape;
    const index_t o_height = (imshape[dstdim - 2] - (pdilate_y * (psize_y - 1) + 1)) / pstride_y + 1;
    const index_t o_width = (imshape[dstdim - 1] - (pdilate_x * (psize_x - 1) + 1)) / pstride_x + 1;
    const Shape<2> sshape = ShapeCheck<2, SrcExp>::Check(src_);
    CHECK_EQ(sshape[1], o_height * o_width * imshape.ProdShape(0, dstdim - 3)) << "PackColToPatchExp: src.size(1) mismatch";
    CHECK_EQ(sshape[0], psize_y * psize_x * imshape[dstdim - 3]) << "PackColToPatchExp: src.size(0) mismatch";
    const uint64_t total = static_cast<uint64_t>(sshape[0]) * sshape[1];
    CHECK_LT(total, (uint64_t(1) << 31)) << "PackColToPatch: source too large for 32-bit indexing";
  }
};

template <typename SrcExp, typename DType, int dstdim, int etype>
inline PackColToPatchXExp<SrcExp, DType, dstdim> pack_col2patch(const expr::Exp<SrcExp, DType, etype> &src,
                                                                Shape<dstdim> imshape, index_t psize_y, index_t psize_x,
                                                                index_t pstride_y, index_t pstride_x, index_t pdilate_y,
                                                                index_t pdilate_x) {
  TypeCheckPass<ExpInfo<SrcExp>::kDim == 2>::Error_Expression_Does_Not_Meet_Dimension_Req();
  CHECK(imshape[dstdim - 1] >= psize_x && imshape[dstdim - 2] >= psize_y)
      << "PackColToPatch:image shape smaller than patch size";
  return PackColToPatchXExp<SrcExp, DType, dstdim>(src.self(), imshape, psize_y, psize_x, pstride_y, pstride_x,
                                                   pdilate_y, pdilate_x);
}
template <typename SrcExp, typename DType, int dstdim, int etype>
inline PackColToPatchXExp<SrcExp, DType, dstdim> pack_col2patch(const expr::Exp<SrcExp, DType, etype> &src,
                                                                Shape<dstdim> imshape, index_t psize_y, index_t psize_x,
                                                                index_t pstride, index_t pdilate) {
  return pack_col2patch(src, imshape, psize_y, psize_x, pstride, pstride, pdilate, pdilate);
}

template <typename SrcExp, typename DType, int dstdim>
class Plan<PackColToPatchXExp<SrcExp, DType, dstdim>, DType> {
 public:
  explicit Plan(const PackColToPatchXExp<SrcExp, DType, dstdim> &e)
      : src_(MakePlan(e.src_)), psize_y_(e.psize_y_), psize_x_(e.psize_x_), by_stride_y_(e.pstride_y_),
        by_stride_x_(e.pstride_x_), by_channel_(e.shape_[dstdim - 3]), by_dilate_y_(e.pdilate_y_),
        by_dilate_x_(e.pdilate_x_), by_height_(e.shape_[dstdim - 2]),
        o_height_((e.shape_[dstdim - 2] - (e.pdilate_y_ * (e.psize_y_ - 1) + 1)) / e.pstride_y_ + 1),
        o_width_((e.shape_[dstdim - 1] - (e.pdilate_x_ * (e.psize_x_ - 1) + 1)) / e.pstride_x_ + 1) {}
  /*!
   * \brief image element (n, c, y, x): sum over the patches (py, px) that cover it, py outer and px
   *  inner, of the matrix entry in row (c, ky, kx) and column (n, py, px); the patch ranges and
   *  their dilation steps are the reference's (pack_col2patch.h:117-139)
   */
  MSHADOW_XINLINE DType Eval(index_t i, index_t j) const {
    uint32_t idivh, n;
    const uint32_t y = by_height_.DivMod(i, &idivh);
    const uint32_t c = by_channel_.DivMod(idivh, &n);
    const uint32_t x = j;
    const uint32_t sy = by_stride_y_.div, sx = by_stride_x_.div, dy = by_dilate_y_.div, dx = by_dilate_x_.div;
    const uint32_t psize_y_dilate = dy * (psize_y_ - 1) + 1, psize_x_dilate = dx * (psize_x_ - 1) + 1;
    uint32_t q;
    const uint32_t py_min = y < psize_y_dilate ? by_dilate_y_.DivMod(y, &q) : by_stride_y_.Quot(y - psize_y_dilate + sy);
    const uint32_t px_min = x < psize_x_dilate ? by_dilate_x_.DivMod(x, &q) : by_stride_x_.Quot(x - psize_x_dilate + sx);
    uint32_t py_max = by_stride_y_.Quot(y + sy), px_max = by_stride_x_.Quot(x + sx);
    if (py_max > static_cast<uint32_t>(o_height_)) py_max = o_height_;
    if (px_max > static_cast<uint32_t>(o_width_)) px_max = o_width_;
    DType res = static_cast<DType>(0);
    for (uint32_t py = py_min; py < py_max; py += dy) {
      for (uint32_t px = px_min; px < px_max; px += dx) {
        res = detail::AddRN<DType>(
            res, src_.Eval((c * psize_y_ + by_dilate_y_.Quot(y - py * sy)) * psize_x_ + by_dilate_x_.Quot(x - px * sx),
                           (n * o_height_ + py) * o_width_ + px));
      }
    }
    return res;
  }
#ifdef __CUDACC__
  /*!
   * \brief a 16-byte group of one image row: the row index and the range of patch rows are worked
   *  out once; every lane keeps the addition order of Eval
   */
  __device__ __forceinline__ Pack<DType> EvalPack(index_t i, index_t j) const {
    uint32_t idivh, n, q;
    const uint32_t y = by_height_.DivMod(i, &idivh);
    const uint32_t c = by_channel_.DivMod(idivh, &n);
    const uint32_t sy = by_stride_y_.div, sx = by_stride_x_.div, dy = by_dilate_y_.div, dx = by_dilate_x_.div;
    const uint32_t psize_y_dilate = dy * (psize_y_ - 1) + 1, psize_x_dilate = dx * (psize_x_ - 1) + 1;
    const uint32_t py_min = y < psize_y_dilate ? by_dilate_y_.DivMod(y, &q) : by_stride_y_.Quot(y - psize_y_dilate + sy);
    uint32_t py_max = by_stride_y_.Quot(y + sy);
    if (py_max > static_cast<uint32_t>(o_height_)) py_max = o_height_;
    uint32_t px_min[Pack<DType>::kLanes], px_max[Pack<DType>::kLanes];
    Pack<DType> r;
#pragma unroll
    for (int l = 0; l < Pack<DType>::kLanes; ++l) {
      const uint32_t x = j + l;
      px_min[l] = x < psize_x_dilate ? by_dilate_x_.DivMod(x, &q) : by_stride_x_.Quot(x - psize_x_dilate + sx);
      px_max[l] = by_stride_x_.Quot(x + sx);
      if (px_max[l] > static_cast<uint32_t>(o_width_)) px_max[l] = o_width_;
      r.v[l] = static_cast<DType>(0);
    }
    for (uint32_t py = py_min; py < py_max; py += dy) {
      const uint32_t krow = (c * psize_y_ + by_dilate_y_.Quot(y - py * sy)) * psize_x_;
      const uint32_t col = (n * o_height_ + py) * o_width_;
#pragma unroll
      for (int l = 0; l < Pack<DType>::kLanes; ++l) {
        const uint32_t x = j + l;
        for (uint32_t px = px_min[l]; px < px_max[l]; px += dx) {
          r.v[l] = detail::AddRN<DType>(r.v[l], src_.Eval(krow + by_dilate_x_.Quot(x - px * sx), col + px));
        }
      }
    }
    return r;
  }
#endif

 private:
  Plan<SrcExp, DType> src_;
  const index_t psize_y_, psize_x_;
  const FastDiv by_stride_y_, by_stride_x_, by_channel_, by_dilate_y_, by_dilate_x_, by_height_;
  const index_t o_height_, o_width_;
};

template <typename SrcExp, typename DType, int dstdim>
struct PackInfo<PackColToPatchXExp<SrcExp, DType, dstdim> > {
  static const bool kPass = true;
};
template <typename SrcExp, typename DType, int dstdim>
struct PackAlign<PackColToPatchXExp<SrcExp, DType, dstdim> > {
  inline static bool Check(const PackColToPatchXExp<SrcExp, DType, dstdim> &) { return true; }
};

}  // namespace expr

#if MSHADOW_USE_CUDA && defined(__CUDACC__)
namespace cuda {

// `mat <Saver>= unpack_patch2col(tensor, ...)`: planes staged in shared memory where they fit
template <typename Saver, typename DType, int srcdim>
struct MapDispatch<Saver, Tensor<gpu, 2, DType>, expr::UnpackPatchToColXExp<Tensor<gpu, srcdim, DType>, DType, srcdim>,
                   DType, 2> {
  typedef expr::UnpackPatchToColXExp<Tensor<gpu, srcdim, DType>, DType, srcdim> E;
  inline static void Run(Tensor<gpu, 2, DType> *dst, const E &e, Shape<2> dshape, cudaStream_t stream) {
    const Tensor<gpu, srcdim, DType> &img = e.img_;
    if (PatchPlaneFits(e.i_height_, e.i_width_, sizeof(DType))) {
      PatchGeom g;
      g.channels = e.i_channel_; g.h = e.i_height_; g.w = e.i_width_;
      g.psy = e.psize_y_; g.psx = e.psize_x_; g.sy = e.pstride_y_; g.sx = e.pstride_x_;
      g.dy = e.pdilate_y_; g.dx = e.pdilate_x_;
      g.oh = (g.h - (g.dy * (g.psy - 1) + 1)) / g.sy + 1;
      g.ow = (g.w - (g.dx * (g.psx - 1) + 1)) / g.sx + 1;
      UnpackPatchLaunch<Saver, DType>(dst->dptr_, dst->stride_, img.dptr_, img.stride_,
                                      img.shape_.ProdShape(0, srcdim - 2), g, stream);
    } else {
      MapGeneric<Saver, DType>(dst, e, dshape, stream);
    }
  }
};

// `img <Saver>= pack_col2patch(matrix, ...)` without dilation
template <typename Saver, typename DType, int dstdim>
struct MapDispatch<Saver, Tensor<gpu, dstdim, DType>, expr::PackColToPatchXExp<Tensor<gpu, 2, DType>, DType, dstdim>,
                   DType, dstdim> {
  typedef expr::PackColToPatchXExp<Tensor<gpu, 2, DType>, DType, dstdim> E;
  inline static void Run(Tensor<gpu, dstdim, DType> *dst, const E &e, Shape<dstdim> dshape, cudaStream_t stream) {
    const Tensor<gpu, 2, DType> &mat = e.src_;
    const bool offsets_fit = static_cast<int64_t>(mat.size(0)) * mat.stride_ < (int64_t(1) << 31);
    if (e.pdilate_y_ == 1 && e.pdilate_x_ == 1 && offsets_fit &&
        PackPatchSupported(dshape[dstdim - 2], dshape[dstdim - 1])) {
      PatchGeom g;
      g.channels = dshape[dstdim - 3]; g.h = dshape[dstdim - 2]; g.w = dshape[dstdim - 1];
      g.psy = e.psize_y_; g.psx = e.psize_x_; g.sy = e.pstride_y_; g.sx = e.pstride_x_;
      g.dy = 1; g.dx = 1;
      g.oh = (g.h - g.psy) / g.sy + 1;
      g.ow = (g.w - g.psx) / g.sx + 1;
      PackPatchLaunch<Saver, DType>(dst->dptr_, dst->stride_, mat.dptr_, mat.stride_, dshape.ProdShape(0, dstdim - 2), g,
                                    stream);
    } else {
      MapGeneric<Saver, DType>(dst, e, dshape, stream);
    }
  }
};

}  // namespace cuda
#endif  // MSHADOW_USE_CUDA && __CUDACC__

}  // namespace mshadow
#endif  // MSHADOW_EXTENSION_PATCH_H_
