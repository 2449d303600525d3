/*
 * C entry points around the UNMODIFIED reference GPU evaluator -- TEST / BASELINE INFRASTRUCTURE ONLY.
 *
 * Like ref_shim.cc, this file holds no arithmetic and no kernels of its own: every function
 * wraps caller DEVICE memory in mshadow::Tensor<gpu,...> handles and calls the reference's
 * public API, so what runs on the GPU are dmlc/mshadow's own kernels
 * (mshadow/cuda/tensor_gpu-inl.cuh), recompiled for sm_100a.  The benchmark's reference arm
 * uses it to time "the reference as it ships, on this GPU" next to the reference's CPU path.
 * It is compiled against the reference headers where they lie (include path only; see the
 * Makefile) into oracle/_ref/libmshadow_ref_gpu.so and is never linked into the product library.
 *
 * Every entry returns 0, or 1 when the reference refused the call (its CHECKs throw because
 * the file is built with DMLC_LOG_FATAL_THROW=1); refgpu_last_error() then holds the message.
 * All pointers are device pointers; matrices are dense.
 */
#include <cstdint>
#include <string>

#include "mshadow/tensor.h"

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

namespace {

std::string g_error;

typedef Tensor<gpu, 1, float> G1;
typedef Tensor<gpu, 2, float> G2;
typedef Tensor<gpu, 4, float> G4;

/* a Stream<gpu> object around a caller's cudaStream_t; the reference only reads stream_ on these paths */
struct Borrowed {
  Stream<gpu> s;
  explicit Borrowed(void *stream) { s.stream_ = static_cast<cudaStream_t>(stream); }
  Stream<gpu> *get() { return &s; }
};

inline G2 mat(const float *p, int64_t rows, int64_t cols, Stream<gpu> *s) {
  return G2(const_cast<float *>(p), Shape2(rows, cols), static_cast<index_t>(cols), s);
}
inline G1 vec(const float *p, int64_t n, Stream<gpu> *s) {
  return G1(const_cast<float *>(p), Shape1(n), static_cast<index_t>(n), s);
}
inline G4 img(const float *p, int64_t n, int64_t c, int64_t h, int64_t w, Stream<gpu> *s) {
  return G4(const_cast<float *>(p), Shape4(n, c, h, w), static_cast<index_t>(w), s);
}

/* the benchmark's element-wise functor, as in guide/README.md:152-157 */
struct sigmoid {
  MSHADOW_XINLINE static float Map(float a) { return 1.0f / (1.0f + expf(-a)); }
};

}  // namespace

#define REFGPU_BEGIN try {
#define REFGPU_END                 \
  }                                \
  catch (const std::exception &e) { \
    g_error = e.what();            \
    return 1;                      \
  }                                \
  return 0;

extern "C" {

const char *refgpu_last_error(void) { return g_error.c_str(); }

int refgpu_expr_case0(float *dst, const float *A, const float *B, const float *C, const float *bias, int64_t rows,
                      int64_t cols, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  G2 d = mat(dst, rows, cols, st.get());
  d = F<sigmoid>(mat(A, rows, cols, st.get()) * mat(B, rows, cols, st.get()) + 0.5f * mat(C, rows, cols, st.get())) +
      repmat(vec(bias, cols, st.get()), rows);
  REFGPU_END
}

int refgpu_sum_rows(float *dst, const float *src, int64_t rows, int64_t cols, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  G1 d = vec(dst, cols, st.get());
  d = sum_rows(mat(src, rows, cols, st.get()));
  REFGPU_END
}

int refgpu_sumall_except_dim1(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                              void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  G1 d = vec(dst, c, st.get());
  d = sumall_except_dim<1>(img(src, n, c, h, w, st.get()));
  REFGPU_END
}

int refgpu_softmax(float *dst, const float *src, int64_t rows, int64_t cols, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  Softmax(mat(dst, rows, cols, st.get()), mat(src, rows, cols, st.get()));
  REFGPU_END
}

int refgpu_softmax_grad(float *dst, const float *src, const float *label, int64_t rows, int64_t cols,
                        void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  SoftmaxGrad(mat(dst, rows, cols, st.get()), mat(src, rows, cols, st.get()), vec(label, rows, st.get()));
  REFGPU_END
}

int refgpu_pool_max(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky, int kx, int sy,
                    int sx, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  const int64_t ph = (h - ky) / sy + 1, pw = (w - kx) / sx + 1;
  G4 d = img(dst, 1, planes, ph, pw, st.get());
  d = pool<red::maximum>(img(src, 1, planes, h, w, st.get()), ky, kx, sy, sx);
  REFGPU_END
}

int refgpu_unpool_max(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t planes,
                      int64_t h, int64_t w, int ky, int kx, int sy, int sx, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  const int64_t ph = (h - ky) / sy + 1, pw = (w - kx) / sx + 1;
  G4 d = img(dst, 1, planes, h, w, st.get());
  d = unpool<red::maximum>(img(src, 1, planes, h, w, st.get()), img(pooled, 1, planes, ph, pw, st.get()),
                           img(gpooled, 1, planes, ph, pw, st.get()), ky, kx, sy, sx);
  REFGPU_END
}

int refgpu_chpool_sum(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w, int nsize,
                      void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  G4 d = img(dst, n, c, h, w, st.get());
  d = chpool<red::sum>(img(src, n, c, h, w, st.get()), nsize);
  REFGPU_END
}

int refgpu_addtakegrad_largebatch(float *dst, const int32_t *sorted, const int32_t *index, const float *src,
                                  int64_t k, int64_t d, int64_t nidx, void *stream) {
  REFGPU_BEGIN
  Borrowed st(stream);
  Tensor<gpu, 1, int32_t> s(const_cast<int32_t *>(sorted), Shape1(nidx), nidx, st.get());
  Tensor<gpu, 1, int32_t> i(const_cast<int32_t *>(index), Shape1(nidx), nidx, st.get());
  AddTakeGradLargeBatch(mat(dst, k, d, st.get()), s, i, mat(src, nidx, d, st.get()));
  REFGPU_END
}

}  // extern "C"
