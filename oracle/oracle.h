/*
 * CPU oracle for the mshadow lazy-evaluation hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of what mshadow's CPU evaluator (mshadow/tensor_cpu-inl.h and
 * the extension Plan::Eval bodies) computes for the operators that the CUDA library
 * accelerates.  It exists so that parity tests have something to compare against on a
 * machine that has no copy of the reference tree.  It is never linked into, loaded by,
 * or called from the product library; only the test-suite, the smoke check and the
 * benchmark's cpu_baseline leg may use it.
 *
 * Parity pinning: every function below is checked bit-for-bit against the unmodified
 * reference headers compiled into oracle/_ref/libmshadow_ref.so (see ref_shim.cc and
 * the Makefile) and against the fixtures in tests/golden/ that were produced by that
 * reference build.
 *
 * Conventions shared with ref_shim.cc (which exports the same entry points with a
 * ref_ prefix):  all matrices are row-major fp32 with an explicit leading dimension
 * `ld` counted in elements (mshadow's Tensor::stride_);  `saver` picks mshadow's
 * sv::saveto/plusto/minusto/multo/divto as 0..4;  `reducer` picks red::sum (0),
 * red::maximum (1) or red::minimum (2).
 */
#ifndef MSHADOW_B200_ORACLE_H_
#define MSHADOW_B200_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef ORC_PREFIX
#define ORC_PREFIX orc_
#endif
#define ORC_CAT2(a, b) a##b
#define ORC_CAT(a, b) ORC_CAT2(a, b)
#define ORC(name) ORC_CAT(ORC_PREFIX, name)

/* Number of elementwise expression cases understood by expr_case(). */
#define ORC_NUM_EXPR_CASES 10

/*
 * Elementwise expression cases evaluated through MapExp (tensor_cpu-inl.h:143-201).
 *   0  dst  = F<sigmoid>(A*B + 0.5f*C) + repmat(bias, rows)     sigmoid(a)=1.0f/(1.0f+expf(-a))
 *   1  dst += A*2.0f - B/C
 *   2  dst  = F<clip_mul>(A, B) * C          clip_mul(a,b) = a > b ? a*b : b
 *   3  dst *= A + 1.5f
 *   4  dst -= A * B
 *   5  dst /= C*C + 1.0f
 *   6  dst  = 3.25f                          (scalar broadcast, all-zero shape sentinel)
 *   7  dst  = F<fma3>(A, B, C)               fma3(a,b,c) = a*b + c   (ternary map)
 *   8  dst  = broadcast<0>(bias_rows, shape) * A + B   bias_rows has `rows` entries
 *   9  dst  = F<square>(A - 1.0f) / (B*B + 2.0f) + C   square(a) = a*a
 * `bias` holds max(rows, cols) floats.
 */
void ORC(expr_case)(int id, float *dst, const float *A, const float *B, const float *C,
                    const float *bias, int64_t rows, int64_t cols, int64_t ld_dst,
                    int64_t ld_a, int64_t ld_b, int64_t ld_c);

/* dst[x] <saver>= scale * Reduce_y src(y,x)     (tensor_cpu-inl.h:203-228) */
void ORC(reduce_keep_lowest)(float *dst, const float *src, int64_t rows, int64_t cols,
                             int64_t ld, float scale, int saver, int reducer);

/* dst[c] <saver>= scale * Reduce_{n,y,x} src((n*C+c)*H+y, x)   (tensor_cpu-inl.h:230-268) */
void ORC(reduce_keep_highdim)(float *dst, const float *src, int64_t n, int64_t c, int64_t h,
                              int64_t w, int64_t ld, float scale, int saver, int reducer);

/* row softmax (tensor_cpu-inl.h:270-285, 464-472) */
void ORC(softmax)(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst,
                  int64_t ld_src);

/*
 * SoftmaxGrad family (tensor_cpu-inl.h:287-368).  mode bit0 = label smoothing with
 * `alpha`, bit1 = rows whose label equals `ignore_label` are zero-filled.
 */
void ORC(softmax_grad)(float *dst, const float *src, const float *label, int64_t rows,
                       int64_t cols, int64_t ld_dst, int64_t ld_src, int mode,
                       float ignore_label, float alpha);

/* pool<Reducer>(src, ky, kx, sy, sx) on `planes` images of h x w (extension/spatial_pool.h:116-149) */
void ORC(pool)(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky,
               int kx, int sy, int sx, int64_t ld_src, int64_t ld_dst, int reducer);

/* unpool<Reducer>(src, pooled, grad_pooled, ...) (extension/spatial_unpool.h:93-132) */
void ORC(unpool)(float *dst, const float *src, const float *pooled, const float *gpooled,
                 int64_t planes, int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx,
                 int sy, int sx, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst,
                 int reducer);

/* chpool<Reducer>(src, nsize, stride, pad) on (n, c, h, w) (extension/channel_pool.h:21-104) */
void ORC(chpool)(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                 int nsize, int stride, int pad, int64_t ld_src, int64_t ld_dst, int reducer);

/* ch_unpool<Reducer>(src, pooled, grad_pooled, nsize, stride, pad): gradient of chpool;
   src is (n, c, h, w), pooled and grad_pooled are (n, pc, h, w) (extension/channel_unpool.h:102-133) */
void ORC(ch_unpool)(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t n,
                    int64_t c, int64_t pc, int64_t h, int64_t w, int nsize, int stride, int pad,
                    int64_t ld_src, int64_t ld_pooled, int64_t ld_dst, int reducer);

/* dst[clip(index[y])] += src[y]  (tensor_cpu-inl.h:497-508) */
void ORC(addtakegrad)(float *dst, const int32_t *index, const float *src, int64_t k,
                      int64_t d, int64_t nidx, int64_t ld_dst, int64_t ld_src);

/* dst[sorted[y]] += src[index[y]]  (tensor_cpu-inl.h:510-518) */
void ORC(addtakegrad_largebatch)(float *dst, const int32_t *sorted, const int32_t *index,
                                 const float *src, int64_t k, int64_t d, int64_t nidx);

/* stable key/value sort, ascending or descending (tensor_cpu-inl.h:531-560) */
void ORC(sort_by_key)(int32_t *keys, int32_t *values, int64_t n, int ascend);

/*
 * Softmax over the middle axis of a (batch, classes, positions) tensor
 * (tensor_cpu-inl.h:474-495): for every (y, n) the column src[y][.][n] is normalised.
 * `ld_*` is the pitch of the last axis.
 */
void ORC(softmax3d)(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos,
                    int64_t ld_dst, int64_t ld_src);

/*
 * SoftmaxGrad family on (batch, classes, positions) with label (batch, positions)
 * (tensor_cpu-inl.h:370-462); mode bits as for softmax_grad.
 */
void ORC(softmax_grad3d)(float *dst, const float *src, const float *label, int64_t batch,
                         int64_t classes, int64_t npos, int64_t ld_dst, int64_t ld_src,
                         int64_t ld_label, int mode, float ignore_label, float alpha);

/* dst[index[y]][j] = src[y][j] for y ascending: the last writer of a row wins
   (tensor_cpu-inl.h:520-529) */
void ORC(index_fill)(float *dst, const int32_t *index, const float *src, int64_t d, int64_t nidx,
                     int64_t ld_dst, int64_t ld_src);

/* sort `values` ascending inside each run of equal `segments` (segments ascending on entry):
   two stable pair sorts (tensor_cpu-inl.h:562-567) */
void ORC(vectorized_sort)(float *values, int32_t *segments, int64_t n);

/*
 * Index-remapping expressions evaluated through MapExp, on dense fp32 tensors A and B of shape
 * (n, c, h, w); p0, p1 are per-case parameters.  `dst` is dense with the case's result shape,
 * which remap_shape() reports.
 *    0  dst = reshape(A, Shape4(n, h, c, w))                    extension/reshape.h
 *    1  dst = slice<1>(A, p0, p1)                               extension/slice.h
 *    2  dst = slice<3>(A, p0, p1)
 *    3  dst = concat<1>(A, B)                                   extension/concat.h
 *    4  dst = concat<3>(A, B)
 *    5  dst = swapaxis<2, 1>(A)                                 extension/swapaxis.h
 *    6  dst = swapaxis<3, 1>(A)
 *    7  dst = transpose(A, Shape4(0, 2, 1, 3))                  extension/transpose.h
 *    8  dst = transpose(A, Shape4(3, 1, 0, 2))
 *    9  dst = pad(A, p0, p1)                                    extension/pad.h
 *   10  dst = crop(A, Shape2(p0, p1))                           extension/crop.h (centred)
 *   11  dst = crop(A, Shape2(p0, p1), h - p0, w - p1)
 *   12  dst = mirror(A)                                         extension/mirror.h
 *   13  dst = flip(A, 1)                                        extension/flip.h
 *   14  dst = B;  slice<1>(dst, p0, p1) = slice<1>(A, p0, p1) + 1.0f      (slice as l-value)
 *   15  concat<1>(dst[0:n], dst[n:2n]) = F<op::identity>(concat<1>(B, A))   dst is (2n, c, h, w) (concat as l-value)
 *   16  dst = crop(pad(A, p0, p1), Shape2(h, w)) + mirror(A)    (nesting)
 */
#define ORC_NUM_REMAP_CASES 17
void ORC(remap_shape)(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                      int64_t out_shape[4]);
void ORC(remap_case)(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c,
                     int64_t h, int64_t w, int64_t p0, int64_t p1);

/*
 * Index-selecting expressions evaluated through MapExp on dense fp32 matrices A and B
 * (rows x cols).  idx_r holds `rows` integers in [0, rows) stored as floats, idx_c `rows`
 * integers in [0, cols); p0 is a per-case parameter.  Result shape: (rows, cols) unless noted.
 *    0  dst = take(idx_r, A)                                   extension/take.h
 *    1  dst = one_hot_encode(idx_c, cols)                      extension/one_hot.h
 *    2  dst = mat_choose_row_element(A, idx_c)      (rows)     extension/choose.h
 *    3  dst = mat_fill_row_element(A, B[0:rows], idx_c)        extension/fill.h (B flat, first `rows` values)
 *    4  dst = mask(idx_c, A)                                   extension/mask.h (row y scaled by idx_c[y])
 *    5  dst = upsampling_nearest(A, p0)    (rows*p0, cols*p0)  extension/spatial_upsampling_nearest.h
 *    6  dst = take_grad(idx_r, A, rows)                        extension/take_grad.h
 *    7  dst = take(idx_r, A) * B + one_hot_encode(idx_c, cols)
 */
#define ORC_NUM_SELECT_CASES 8
void ORC(select_case)(int id, float *dst, const float *A, const float *B, const float *idx_r,
                      const float *idx_c, int64_t rows, int64_t cols, int64_t p0);

/*
 * Patch <-> column conversion on a dense (n, c, h, w) image (extension/unpack_patch2col.h:115-133,
 * extension/pack_col2patch.h:108-140).  With oh = (h - (dy*(psy-1)+1))/sy + 1 and ow likewise, the
 * matrix is (psy*psx*c) x (oh*ow*n), dense.
 */
void ORC(unpack_patch2col)(float *mat, const float *img, int64_t n, int64_t c, int64_t h, int64_t w,
                           int psy, int psx, int sy, int sx, int dy, int dx);
void ORC(pack_col2patch)(float *img, const float *mat, int64_t n, int64_t c, int64_t h, int64_t w,
                         int psy, int psx, int sy, int sx, int dy, int dx);

/*
 * Expressions addressed by an axis number or a begin/end box, evaluated through MapExp on a dense
 * fp32 tensor A of shape (n, c, h, w); p0, p1 are per-case parameters.  `dst` is dense with the
 * case's result shape; axis_shape() writes its extents to out_shape (unused entries 1) and
 * returns their number.
 *    0  dst = range(p0, p0 + p1, 0.5f, 2)              (1-d)       extension/range.h
 *    1  dst = range(p0 + p1, p0, -1.5f, 1)             (1-d)
 *    2  dst = slice(A, begin, end)                                 extension/slice_ex.h
 *         begin = (p0 % n, p1 % c, p0 % h, p1 % w), end = (n, c, begin_h + (h - begin_h + 1) / 2, w)
 *    3  dst = A * 2;  slice(dst, begin, end) = slice(A, begin, end) + 1    (the box as l-value)
 *    4  dst = reduce_with_axis<red::sum, false>(A, p0)  (3-d)      extension/reduce_with_axis.h
 *    5  dst = reduce_with_axis<red::maximum, true>(A, p0)   (position of the maximum along the axis)
 *    6  dst = reduce_keepdim<red::minimum, false>(A, p0)  (4-d, extent 1 at p0)
 *    7  dst = broadcast_with_axis(A3, p0 - 1, p1), A3 = A seen as (n*c, h, w)   extension/broadcast_with_axis.h
 *    8  dst = broadcast_keepdim(slice<1>(A, 0, 1), 1, p1)  -> (n, p1, h, w)
 *    9  dst = broadcast_to(S, (n, p0, h, p1)), S = the first n*h elements of A seen as (n, 1, h, 1)
 *   10  dst = broadcast_multi_axes(S, axes (0, 2), sizes (p0, p1)), S = the first c*w elements of A
 *         seen as (1, c, 1, w)  -> (p0, c, p1, w)
 */
#define ORC_NUM_AXIS_CASES 11
int ORC(axis_shape)(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                    int64_t out_shape[4]);
void ORC(axis_case)(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w,
                    int64_t p0, int64_t p1);

/*
 * Complex arithmetic (extension/complex.h) evaluated through MapExp.  A and B are dense fp32
 * matrices of rows x cols floats, read as rows x cols/2 complex numbers (re, im interleaved);
 * Ah and Bh are the first rows*cols/2 floats of the same buffers read as real rows x cols/2
 * matrices.  cols must be a multiple of 4.  Result rows x cols unless noted:
 *    0  complex_mul_cc(A, B)      1  complex_mul_cr(A, Bh)     2  complex_mul_rc(Ah, B)
 *    3  complex_div_cc(A, B)      4  complex_div_cr(A, Bh)     5  complex_div_rc(Ah, B)
 *    6  conj(A)                   7  complex_exchange(A)       8  complex_pad_imag(Ah)
 *    9  complex_toreal(A)        10  complex_abs_square(A)    11  complex_sum_real_imag(A)   (rows x cols/2)
 *   12  complex_mul_cc(conj(A), B) + complex_pad_imag(complex_abs_square(B)) * 0.5f
 */
#define ORC_NUM_COMPLEX_CASES 13
void ORC(complex_case)(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols);

/*
 * Local response normalisation as a layer composes it from chpool<red::sum> and user functors
 * (extension/channel_pool.h:77-104 through MapExp, tensor_cpu-inl.h:143-201):
 *   lrn_forward    norm = chpool<red::sum>(F<square>(src), nsize) * salpha + knorm;
 *                  out  = src * F<power>(norm, -beta);
 *   lrn_backward   gsrc  = gout * F<power>(norm, -beta);
 *                  gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<power>(norm, -beta - 1.0f), nsize) * src;
 * square(a) = a * a.  power_kind 0: power(a, b) = powf(a, b); 1: for b = -0.75 / -1.75,
 * 1 / (sqrtf(a) * sqrtf(sqrtf(a)) [* a]), else powf; 2: powf.  Dense (n, c, h, w) tensors.
 */
void ORC(lrn_forward)(float *out, float *norm, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                      int nsize, float salpha, float beta, float knorm, int power_kind);
void ORC(lrn_backward)(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n, int64_t c,
                       int64_t h, int64_t w, int nsize, float salpha, float beta, int power_kind);

/* number of OpenMP threads the library will use (for cpu_baseline.cores) */
int ORC(num_threads)(void);
/* sets the number of OpenMP threads of later calls (n < 1: leave unchanged); a launcher may have
 * exported OMP_NUM_THREADS=1 into the environment before this library was loaded */
void ORC(set_num_threads)(int n);

#ifdef __cplusplus
}
#endif
#endif  /* MSHADOW_B200_ORACLE_H_ */
