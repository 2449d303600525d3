/*
 * CPU oracle for the mshadow lazy-evaluation hot path -- TEST INFRASTRUCTURE ONLY.
 * See oracle.h for the role of this file and for how it is pinned to the reference.
 *
 * Build: gcc -O2 -std=c11 -fopenmp -ffp-contract=off -fPIC -shared oracle.c -lm
 * (-ffp-contract=off is mandatory: a fused multiply-add changes result bits, and the
 *  reference CPU build uses plain SSE arithmetic.)
 *
 * Each function names the reference lines it restates.  Loops run in the reference's
 * order wherever order affects floating-point results; OpenMP is only ever applied to
 * loops whose iterations produce disjoint outputs, exactly as the reference does.
 */
#define _GNU_SOURCE
#include "oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* sv::saveto / plusto / minusto / multo / divto  (mshadow/base.h:539-602) */
static inline void save(float *a, float b, int saver) {
  switch (saver) {
    case 0: *a = b; break;
    case 1: *a += b; break;
    case 2: *a -= b; break;
    case 3: *a *= b; break;
    default: *a /= b; break;
  }
}

/* red::sum / maximum / minimum ::Reduce  (mshadow/base.h:692-862) */
static inline float reduce(float acc, float v, int reducer) {
  switch (reducer) {
    case 0: return acc + v;
    case 1: return acc < v ? v : acc;  /* std::max(acc, v) */
    default: return v < acc ? v : acc; /* std::min(acc, v) */
  }
}

/* Reducer::SetInitValue  (mshadow/base.h:742-749, 795-797, 857-860) */
static inline float reduce_init(int reducer) {
  switch (reducer) {
    case 0: return 0.0f;
    case 1: return -FLT_MAX;
    default: return FLT_MAX;
  }
}

/* Reducer::PartialGrad  (mshadow/base.h:736-739, 787-790) */
static inline float partial_grad(float redres, float redsrc, int reducer) {
  if (reducer == 0) return 1.0f;
  return redres == redsrc ? 1.0f : 0.0f;
}

/* ---- elementwise: scalar MapPlan, y outer / x inner (tensor_cpu-inl.h:143-159) ---- */

static inline float sigmoid(float a) { return 1.0f / (1.0f + expf(-a)); }

void ORC(expr_case)(int id, float *dst, const float *A, const float *B, const float *C,
                    const float *bias, int64_t rows, int64_t cols, int64_t ld_dst,
                    int64_t ld_a, int64_t ld_b, int64_t ld_c) {
#pragma omp parallel for
  for (int64_t y = 0; y < rows; ++y) {
    float *d = dst + y * ld_dst;
    const float *a = A + y * ld_a, *b = B + y * ld_b, *c = C + y * ld_c;
    for (int64_t x = 0; x < cols; ++x) {
      switch (id) {
        case 0: {
          /* repmat plan reads src(0, x): extension/broadcast.h:137-148 */
          float t = a[x] * b[x];
          float u = 0.5f * c[x];
          d[x] = sigmoid(t + u) + bias[x];
          break;
        }
        case 1: {
          float t = a[x] * 2.0f;
          float u = b[x] / c[x];
          d[x] += t - u;
          break;
        }
        case 2: {
          float m = a[x] > b[x] ? a[x] * b[x] : b[x];
          d[x] = m * c[x];
          break;
        }
        case 3: d[x] *= a[x] + 1.5f; break;
        case 4: d[x] -= a[x] * b[x]; break;
        case 5: {
          float t = c[x] * c[x];
          d[x] /= t + 1.0f;
          break;
        }
        case 6: d[x] = 3.25f; break;
        case 7: {
          float t = a[x] * b[x];
          d[x] = t + c[x];
          break;
        }
        case 8: {
          /* general broadcast plan reads src(0, (y / ystride) % length), with
             ystride = 1 and length = rows for dimcast 0 of a matrix:
             extension/broadcast.h:116-135 */
          float t = bias[y] * a[x];
          d[x] = t + b[x];
          break;
        }
        default: {
          float s = a[x] - 1.0f;
          float num = s * s;
          float t = b[x] * b[x];
          float q = num / (t + 2.0f);
          d[x] = q + c[x];
          break;
        }
      }
    }
  }
}

/* ---- reductions ---- */

/* tensor_cpu-inl.h:221-227: seed from row 0, fold rows 1.. in order, scale, save */
void ORC(reduce_keep_lowest)(float *dst, const float *src, int64_t rows, int64_t cols,
                             int64_t ld, float scale, int saver, int reducer) {
#pragma omp parallel for
  for (int64_t x = 0; x < cols; ++x) {
    float res = src[x];
    for (int64_t y = 1; y < rows; ++y) res = reduce(res, src[y * ld + x], reducer);
    save(dst + x, res * scale, saver);
  }
}

/* tensor_cpu-inl.h:254-267: per-n partial from the init value, then folded into res */
void ORC(reduce_keep_highdim)(float *dst, const float *src, int64_t n, int64_t c, int64_t h,
                              int64_t w, int64_t ld, float scale, int saver, int reducer) {
#pragma omp parallel for
  for (int64_t ci = 0; ci < c; ++ci) {
    float res = reduce_init(reducer);
    for (int64_t ni = 0; ni < n; ++ni) {
      float tres = reduce_init(reducer);
      for (int64_t y = 0; y < h; ++y) {
        const float *row = src + ((ni * c + ci) * h + y) * ld;
        for (int64_t x = 0; x < w; ++x) tres = reduce(tres, row[x], reducer);
      }
      res = reduce(res, tres, reducer);
    }
    save(dst + ci, res * scale, saver);
  }
}

/* ---- softmax ---- */

/* tensor_cpu-inl.h:270-285 applied per row by :464-472 */
void ORC(softmax)(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst,
                  int64_t ld_src) {
#pragma omp parallel for
  for (int64_t y = 0; y < rows; ++y) {
    const float *e = src + y * ld_src;
    float *d = dst + y * ld_dst;
    float mmax = e[0];
    for (int64_t x = 1; x < cols; ++x)
      if (mmax < e[x]) mmax = e[x];
    float sum = 0.0f;
    for (int64_t x = 0; x < cols; ++x) {
      d[x] = expf(e[x] - mmax);
      sum += d[x];
    }
    for (int64_t x = 0; x < cols; ++x) d[x] /= sum;
  }
}

/* tensor_cpu-inl.h:287-302 (plain), :304-321 (smooth), :324-344 (ignore), :346-368 (both) */
void ORC(softmax_grad)(float *dst, const float *src, const float *label, int64_t rows,
                       int64_t cols, int64_t ld_dst, int64_t ld_src, int mode,
                       float ignore_label, float alpha) {
  const int smooth = mode & 1, ignore = mode & 2;
  const float smooth_grad = alpha / (float)(cols - 1);
#pragma omp parallel for
  for (int64_t y = 0; y < rows; ++y) {
    const int k = (int)label[y];
    const float *s = src + y * ld_src;
    float *d = dst + y * ld_dst;
    for (int64_t x = 0; x < cols; ++x) {
      if (ignore && (int)ignore_label == k) {
        d[x] = 0.0f;
      } else if (x == k) {
        d[x] = smooth ? s[x] - 1.0f + alpha : s[x] - 1.0f;
      } else {
        d[x] = smooth ? s[x] - smooth_grad : s[x];
      }
    }
  }
}

/* ---- pooling ---- */

static inline int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }

/* extension/spatial_pool.h:39-51 (output size) and :125-142 (window walk) */
void ORC(pool)(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky,
               int kx, int sy, int sx, int64_t ld_src, int64_t ld_dst, int reducer) {
  const int64_t ph = (h - ky) / sy + 1, pw = (w - kx) / sx + 1;
#pragma omp parallel for
  for (int64_t i = 0; i < planes * ph; ++i) {
    const int64_t py = i % ph, c = i / ph;
    const int64_t y0 = py * sy, y1 = imin(y0 + ky, h);
    for (int64_t px = 0; px < pw; ++px) {
      const int64_t x0 = px * sx, x1 = imin(x0 + kx, w);
      float res = reduce_init(reducer);
      for (int64_t y = y0; y < y1; ++y)
        for (int64_t x = x0; x < x1; ++x)
          res = reduce(res, src[(c * h + y) * ld_src + x], reducer);
      dst[i * ld_dst + px] = res;
    }
  }
}

/* extension/spatial_unpool.h:102-125 */
void ORC(unpool)(float *dst, const float *src, const float *pooled, const float *gpooled,
                 int64_t planes, int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx,
                 int sy, int sx, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst,
                 int reducer) {
#pragma omp parallel for
  for (int64_t i = 0; i < planes * h; ++i) {
    const int64_t y = i % h, c = i / h;
    const int64_t py_min = y < ky ? 0 : (y - ky + sy) / sy;
    const int64_t py_max = imin((y + sy) / sy, ph);
    for (int64_t x = 0; x < w; ++x) {
      const float vsrc = src[i * ld_src + x];
      const int64_t px_min = x < kx ? 0 : (x - kx + sx) / sx;
      const int64_t px_max = imin((x + sx) / sx, pw);
      float val = 0.0f;
      for (int64_t py = py_min; py < py_max; ++py)
        for (int64_t px = px_min; px < px_max; ++px) {
          const int64_t o = (c * ph + py) * ld_pooled + px;
          val += partial_grad(vsrc, pooled[o], reducer) * gpooled[o];
        }
      dst[i * ld_dst + x] = val;
    }
  }
}

/* extension/channel_pool.h:35-42 (output channels) and :85-99 (window walk; note that
   the upper clamp uses the OUTPUT channel count, as the reference does) */
void ORC(chpool)(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                 int nsize, int stride, int pad, int64_t ld_src, int64_t ld_dst, int reducer) {
  const int64_t co = (c - nsize + pad * 2 + 1) / stride;
#pragma omp parallel for
  for (int64_t i = 0; i < n * co * h; ++i) {
    const int64_t y = i % h, oc = (i / h) % co, ni = i / h / co;
    const int64_t cstart = oc * stride < pad ? 0 : oc * stride - pad;
    const int64_t cend = imin(oc * stride - pad + nsize, co);
    for (int64_t x = 0; x < w; ++x) {
      float res = reduce_init(reducer);
      for (int64_t cc = cstart; cc < cend; ++cc)
        res = reduce(res, src[((ni * c + cc) * h + y) * ld_src + x], reducer);
      dst[i * ld_dst + x] = res;
    }
  }
}

/* extension/channel_unpool.h:108-126: pooled channels [cstart, cend) cover source channel c;
   the upper clamp uses the SOURCE channel count, as the reference does */
void ORC(ch_unpool)(float *dst, const float *src, const float *pooled, const float *gpooled, int64_t n,
                    int64_t c, int64_t pc, int64_t h, int64_t w, int nsize, int stride, int pad,
                    int64_t ld_src, int64_t ld_pooled, int64_t ld_dst, int reducer) {
#pragma omp parallel for
  for (int64_t i = 0; i < n * c * h; ++i) {
    const int64_t y = i % h, ci = (i / h) % c, ni = i / h / c;
    const int64_t cstart = ci < nsize - pad ? 0 : (ci - (nsize - pad) + stride) / stride;
    const int64_t cend = imin((ci + pad + stride) / stride, c);
    for (int64_t x = 0; x < w; ++x) {
      const float vsrc = src[i * ld_src + x];
      float val = 0.0f;
      for (int64_t cc = cstart; cc < cend; ++cc) {
        const int64_t o = ((ni * pc + cc) * h + y) * ld_pooled + x;
        val += partial_grad(vsrc, pooled[o], reducer) * gpooled[o];
      }
      dst[i * ld_dst + x] = val;
    }
  }
}

/* ---- local response normalisation composed from chpool<red::sum> ----
   The expressions of a layer written against the reference, evaluated element by element as
   MapExp does (tensor_cpu-inl.h:143-201) with the window loop of extension/channel_pool.h:85-99
   (stride 1, pad nsize / 2, channels [max(c - pad, 0), min(c - pad + nsize, C)) in ascending order
   from zero). */
static float lrn_power(float a, float b, int kind) {
  if (kind == 1 && (b == -0.75f || b == -1.75f)) {
    const float r = sqrtf(a);
    float t = r * sqrtf(r);
    if (b == -1.75f) t = t * a;
    return 1.0f / t;
  }
  return powf(a, b);
}

void ORC(lrn_forward)(float *out, float *norm, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                      int nsize, float salpha, float beta, float knorm, int power_kind) {
  const int64_t plane = h * w, pad = nsize / 2;
#pragma omp parallel for
  for (int64_t i = 0; i < n * c; ++i) {
    const int64_t ci = i % c, ni = i / c;
    const int64_t cstart = ci < pad ? 0 : ci - pad;
    const int64_t cend = imin(ci - pad + nsize, c);
    for (int64_t p = 0; p < plane; ++p) {
      float sum = 0.0f;
      for (int64_t cc = cstart; cc < cend; ++cc) {
        const float a = src[(ni * c + cc) * plane + p];
        sum = sum + a * a;
      }
      const float nrm = sum * salpha + knorm;
      norm[i * plane + p] = nrm;
      out[i * plane + p] = src[i * plane + p] * lrn_power(nrm, -beta, power_kind);
    }
  }
}

void ORC(lrn_backward)(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n, int64_t c,
                       int64_t h, int64_t w, int nsize, float salpha, float beta, int power_kind) {
  const int64_t plane = h * w, pad = nsize / 2;
  const float scale = -2.0f * beta * salpha;
  const float e1 = -beta - 1.0f;
#pragma omp parallel for
  for (int64_t i = 0; i < n * c; ++i) {
    const int64_t ci = i % c, ni = i / c;
    const int64_t cstart = ci < pad ? 0 : ci - pad;
    const int64_t cend = imin(ci - pad + nsize, c);
    for (int64_t p = 0; p < plane; ++p) {
      float sum = 0.0f;
      for (int64_t cc = cstart; cc < cend; ++cc) {
        const int64_t o = (ni * c + cc) * plane + p;
        sum = sum + (gout[o] * src[o]) * lrn_power(norm[o], e1, power_kind);
      }
      const float first = gout[i * plane + p] * lrn_power(norm[i * plane + p], -beta, power_kind);
      gsrc[i * plane + p] = first + (scale * sum) * src[i * plane + p];
    }
  }
}

/* ---- embedding backward ---- */

/* tensor_cpu-inl.h:497-508: serial over the batch, index clipped into [0, K-1] */
void ORC(addtakegrad)(float *dst, const int32_t *index, const float *src, int64_t k,
                      int64_t d, int64_t nidx, int64_t ld_dst, int64_t ld_src) {
  for (int64_t y = 0; y < nidx; ++y) {
    int64_t j = index[y];
    if (j <= 0) j = 0;
    else if (j >= k) j = k - 1;
    float *row = dst + j * ld_dst;
    const float *s = src + y * ld_src;
    for (int64_t x = 0; x < d; ++x) row[x] += s[x];
  }
}

/* tensor_cpu-inl.h:510-518: serial over the sorted list, no clipping */
void ORC(addtakegrad_largebatch)(float *dst, const int32_t *sorted, const int32_t *index,
                                 const float *src, int64_t k, int64_t d, int64_t nidx) {
  (void)k;
  for (int64_t y = 0; y < nidx; ++y) {
    float *row = dst + (int64_t)sorted[y] * d;
    const float *s = src + (int64_t)index[y] * d;
    for (int64_t x = 0; x < d; ++x) row[x] += s[x];
  }
}

/* ---- SortByKey: stable permutation sort, then gather (tensor_cpu-inl.h:531-560) ---- */

static void merge_sort_perm(int64_t *perm, int64_t *tmp, const int32_t *keys, int64_t lo,
                            int64_t hi, int ascend) {
  if (hi - lo < 2) return;
  const int64_t mid = lo + (hi - lo) / 2;
  merge_sort_perm(perm, tmp, keys, lo, mid, ascend);
  merge_sort_perm(perm, tmp, keys, mid, hi, ascend);
  int64_t i = lo, j = mid, o = lo;
  while (i < mid && j < hi) {
    /* take from the right run only when it is strictly "before" the left head */
    const int right_first =
        ascend ? keys[perm[j]] < keys[perm[i]] : keys[perm[j]] > keys[perm[i]];
    tmp[o++] = right_first ? perm[j++] : perm[i++];
  }
  while (i < mid) tmp[o++] = perm[i++];
  while (j < hi) tmp[o++] = perm[j++];
  memcpy(perm + lo, tmp + lo, (size_t)(hi - lo) * sizeof(int64_t));
}

void ORC(sort_by_key)(int32_t *keys, int32_t *values, int64_t n, int ascend) {
  if (n <= 0) return;
  int64_t *perm = (int64_t *)malloc((size_t)n * sizeof(int64_t));
  int64_t *tmp = (int64_t *)malloc((size_t)n * sizeof(int64_t));
  int32_t *k2 = (int32_t *)malloc((size_t)n * sizeof(int32_t));
  int32_t *v2 = (int32_t *)malloc((size_t)n * sizeof(int32_t));
  for (int64_t i = 0; i < n; ++i) perm[i] = i;
  merge_sort_perm(perm, tmp, keys, 0, n, ascend);
  for (int64_t i = 0; i < n; ++i) {
    k2[i] = keys[perm[i]];
    v2[i] = values[perm[i]];
  }
  memcpy(keys, k2, (size_t)n * sizeof(int32_t));
  memcpy(values, v2, (size_t)n * sizeof(int32_t));
  free(perm); free(tmp); free(k2); free(v2);
}

/* ---- softmax over the middle axis (tensor_cpu-inl.h:474-495) ---- */

void ORC(softmax3d)(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos,
                    int64_t ld_dst, int64_t ld_src) {
#pragma omp parallel for
  for (int64_t y = 0; y < batch; ++y) {
    for (int64_t n = 0; n < npos; ++n) {
      const float *e = src + y * classes * ld_src + n;
      float *d = dst + y * classes * ld_dst + n;
      float mmax = e[0];
      for (int64_t x = 1; x < classes; ++x)
        if (mmax < e[x * ld_src]) mmax = e[x * ld_src];
      float sum = 0.0f;
      for (int64_t x = 0; x < classes; ++x) {
        d[x * ld_dst] = expf(e[x * ld_src] - mmax);
        sum += d[x * ld_dst];
      }
      for (int64_t x = 0; x < classes; ++x) d[x * ld_dst] /= sum;
    }
  }
}

/* tensor_cpu-inl.h:370-387 (plain), :389-408 (smooth), :410-434 (ignore), :436-462 (both) */
void ORC(softmax_grad3d)(float *dst, const float *src, const float *label, int64_t batch,
                         int64_t classes, int64_t npos, int64_t ld_dst, int64_t ld_src,
                         int64_t ld_label, int mode, float ignore_label, float alpha) {
  const int smooth = mode & 1, ignore = mode & 2;
  const float smooth_grad = alpha / (float)(classes - 1);
#pragma omp parallel for
  for (int64_t n = 0; n < npos; ++n) {
    for (int64_t y = 0; y < batch; ++y) {
      const int k = (int)label[y * ld_label + n];
      for (int64_t x = 0; x < classes; ++x) {
        const float s = src[(y * classes + x) * ld_src + n];
        float *d = dst + (y * classes + x) * ld_dst + n;
        if (ignore && k == (int)ignore_label) {
          *d = 0.0f;
        } else if (x == k) {
          *d = smooth ? s - 1.0f + alpha : s - 1.0f;
        } else {
          *d = smooth ? s - smooth_grad : s;
        }
      }
    }
  }
}

/* ---- IndexFill (tensor_cpu-inl.h:520-529): serial, so a row named twice keeps the later source ---- */

void ORC(index_fill)(float *dst, const int32_t *index, const float *src, int64_t d, int64_t nidx,
                     int64_t ld_dst, int64_t ld_src) {
  for (int64_t y = 0; y < nidx; ++y) {
    float *row = dst + (int64_t)index[y] * ld_dst;
    const float *s = src + y * ld_src;
    for (int64_t j = 0; j < d; ++j) row[j] = s[j];
  }
}

/* ---- VectorizedSort (tensor_cpu-inl.h:562-567): SortByKey(values, segments), then
        SortByKey(segments, values), both stable and ascending ---- */

static void merge_sort_perm_f32(int64_t *perm, int64_t *tmp, const float *keys, int64_t lo, int64_t hi) {
  if (hi - lo < 2) return;
  const int64_t mid = lo + (hi - lo) / 2;
  merge_sort_perm_f32(perm, tmp, keys, lo, mid);
  merge_sort_perm_f32(perm, tmp, keys, mid, hi);
  int64_t i = lo, j = mid, o = lo;
  while (i < mid && j < hi) tmp[o++] = keys[perm[j]] < keys[perm[i]] ? perm[j++] : perm[i++];
  while (i < mid) tmp[o++] = perm[i++];
  while (j < hi) tmp[o++] = perm[j++];
  memcpy(perm + lo, tmp + lo, (size_t)(hi - lo) * sizeof(int64_t));
}

void ORC(vectorized_sort)(float *values, int32_t *segments, int64_t n) {
  if (n <= 0) return;
  int64_t *perm = (int64_t *)malloc((size_t)n * sizeof(int64_t));
  int64_t *tmp = (int64_t *)malloc((size_t)n * sizeof(int64_t));
  float *v2 = (float *)malloc((size_t)n * sizeof(float));
  int32_t *s2 = (int32_t *)malloc((size_t)n * sizeof(int32_t));
  for (int pass = 0; pass < 2; ++pass) {
    for (int64_t i = 0; i < n; ++i) perm[i] = i;
    if (pass == 0) merge_sort_perm_f32(perm, tmp, values, 0, n);
    else merge_sort_perm(perm, tmp, segments, 0, n, 1);
    for (int64_t i = 0; i < n; ++i) {
      v2[i] = values[perm[i]];
      s2[i] = segments[perm[i]];
    }
    memcpy(values, v2, (size_t)n * sizeof(float));
    memcpy(segments, s2, (size_t)n * sizeof(int32_t));
  }
  free(perm); free(tmp); free(v2); free(s2);
}

/* ---- index-remapping expressions: every Plan::Eval(i, j) of the reference restated on the
        flattened (rows, last extent) view that MapExp walks (tensor_cpu-inl.h:143-201) ---- */

void ORC(remap_shape)(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                      int64_t o[4]) {
  o[0] = n; o[1] = c; o[2] = h; o[3] = w;
  switch (id) {
    case 0: case 5: case 7: o[1] = h; o[2] = c; break;
    case 1: o[1] = p1 - p0; break;
    case 2: o[3] = p1 - p0; break;
    case 3: o[1] = 2 * c; break;
    case 4: o[3] = 2 * w; break;
    case 6: o[1] = w; o[3] = c; break;
    case 8: o[0] = w; o[1] = c; o[2] = n; o[3] = h; break;
    case 9: o[2] = h + 2 * p0; o[3] = w + 2 * p1; break;
    case 10: case 11: o[2] = p0; o[3] = p1; break;
    case 15: o[0] = 2 * n; break;
    default: break;
  }
}

/* A(row, col) of a dense tensor whose last extent is `w` */
#define AT(p, w, row, col) ((p)[(int64_t)(row) * (w) + (col)])

/* extension/pad.h:84-95 on a source of `sh` x `sw` planes */
static float pad_eval(const float *A, int64_t sh, int64_t sw, int64_t py, int64_t px, int64_t i, int64_t j) {
  const int64_t nh = sh + 2 * py;
  const int64_t y = i % nh, cc = i / nh;
  if (y < py || j < px) return 0.0f;
  const int64_t hh = y - py, ww = j - px;
  return (hh < sh && ww < sw) ? AT(A, sw, cc * sh + hh, ww) : 0.0f;
}

void ORC(remap_case)(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c,
                     int64_t h, int64_t w, int64_t p0, int64_t p1) {
  int64_t o[4];
  ORC(remap_shape)(id, n, c, h, w, p0, p1, o);
  const int64_t rows = o[0] * o[1] * o[2], cols = o[3];
  if (id == 14) memcpy(dst, B, (size_t)(n * c * h * w) * sizeof(float));
#pragma omp parallel for
  for (int64_t i = 0; i < rows; ++i) {
    for (int64_t j = 0; j < cols; ++j) {
      float v = 0.0f;
      int store = 1;
      switch (id) {
        case 0: {  /* reshape.h:58-61: linear offset re-split by the source's last extent */
          const int64_t idx = i * cols + j;
          v = AT(A, w, idx / w, idx % w);
        } break;
        case 1: {  /* slice.h:101-109, dimslice = 1: height = h */
          const int64_t y = i % h, t = i / h, ch = p1 - p0;
          const int64_t cc = t % ch + p0, b = t / ch;
          v = AT(A, w, (b * c + cc) * h + y, j);
        } break;
        case 2:  /* slice.h:132-134: last dimension */
          v = AT(A, w, i, j + p0);
          break;
        case 3: {  /* concat.h:120-132, dimcat = 1 */
          const int64_t y = i % h, t = i / h;
          const int64_t cc = t % (2 * c), b = t / (2 * c);
          v = cc < c ? AT(A, w, (b * c + cc) * h + y, j) : AT(B, w, (b * c + cc - c) * h + y, j);
        } break;
        case 4:  /* concat.h:163-169: last dimension */
          v = j < w ? AT(A, w, i, j) : AT(B, w, i, j - w);
          break;
        case 5: {  /* swapaxis.h:72-84, a1 = 2, a2 = 1: shapey = 1, shapez = c(out axis 2), shapec = 1, shapen = h */
          const int64_t z = i % c, t = i / c;
          const int64_t nn = t % h, b = t / h;
          v = AT(A, w, (b * c + z) * h + nn, j);
        } break;
        case 6: {  /* swapaxis.h:97-103, a1 = 3, a2 = 1: out (n, w, h, c); shapex = c, shapey = h, shapez = w */
          const int64_t y = i % h, t = i / h;
          const int64_t z = t % w, b = t / w;
          v = AT(A, w, (b * c + j) * h + y, z);
        } break;
        case 7: case 8: {  /* transpose.h:64-72 */
          const int64_t ss[4] = {c * h * w, h * w, w, 1};  /* dense strides of the source */
          const int ax[2][4] = {{0, 2, 1, 3}, {3, 1, 0, 2}};
          const int *a = ax[id - 7];
          int64_t idx = j * ss[a[3]], r = i;
          for (int k = 2; k >= 0; --k) {
            idx += (r % o[k]) * ss[a[k]];
            r /= o[k];
          }
          v = AT(A, w, idx / w, idx % w);
        } break;
        case 9:
          v = pad_eval(A, h, w, p0, p1, i, j);
          break;
        case 10: case 11: {  /* crop.h:96-103 */
          const int64_t ph = id == 10 ? (h - p0) / 2 : h - p0, pw = id == 10 ? (w - p1) / 2 : w - p1;
          const int64_t y = i % p0, cc = i / p0;
          v = AT(A, w, cc * h + y + ph, j + pw);
        } break;
        case 12:  /* mirror.h:51-53 */
          v = AT(A, w, i, w - j - 1);
          break;
        case 13: {  /* flip.h:99-107, dim = 1: trailing = h*w, stride = c */
          int64_t idx = i * w + j;
          const int64_t low = idx % (h * w);
          int64_t high = idx / (h * w);
          const int64_t x = high % c;
          high /= c;
          idx = (high * c + c - 1 - x) * (h * w) + low;
          v = AT(A, w, idx / w, idx % w);
        } break;
        case 14: {  /* destination rows (b, cc, y) with cc in [p0, p1) are overwritten */
          const int64_t cc = (i / h) % c;
          if (cc >= p0 && cc < p1) v = AT(A, w, i, j) + 1.0f;
          else store = 0;
        } break;
        case 15: {  /* first n images receive B, the following n receive A */
          v = i < n * c * h ? AT(B, w, i, j) : AT(A, w, i - n * c * h, j);
        } break;
        default: {  /* 16: centred crop of the padded tensor gives A back */
          const int64_t nh = h + 2 * p0;
          const int64_t y = i % h, cc = i / h;
          v = pad_eval(A, h, w, p0, p1, cc * nh + y + p0, j + p1) + AT(A, w, i, w - j - 1);
        } break;
      }
      if (store) dst[i * cols + j] = v;
    }
  }
}

/* ---- index-selecting expressions: the Plan::Eval bodies of extension/{take, one_hot, choose, fill,
        mask, spatial_upsampling_nearest, take_grad}.h ---- */

void ORC(select_case)(int id, float *dst, const float *A, const float *B, const float *idx_r,
                      const float *idx_c, int64_t rows, int64_t cols, int64_t p0) {
  if (id == 2) {  /* choose.h:50-53: a vector result, element y = A(y, idx_c[y]) */
    for (int64_t y = 0; y < rows; ++y) dst[y] = AT(A, cols, y, (int64_t)idx_c[y]);
    return;
  }
  const int64_t orows = id == 5 ? rows * p0 : rows, ocols = id == 5 ? cols * p0 : cols;
#pragma omp parallel for
  for (int64_t y = 0; y < orows; ++y) {
    for (int64_t x = 0; x < ocols; ++x) {
      float v;
      switch (id) {
        case 0:  /* take.h:48-51 */
          v = AT(A, cols, (int64_t)idx_r[y], x);
          break;
        case 1:  /* one_hot.h:47-50 */
          v = (float)(x == (int64_t)idx_c[y]);
          break;
        case 3:  /* fill.h:55-62 */
          v = (int64_t)idx_c[y] == x ? B[y] : AT(A, cols, y, x);
          break;
        case 4:  /* mask.h:47-49 */
          v = AT(A, cols, y, x) * idx_c[y];
          break;
        case 5:  /* spatial_upsampling_nearest.h:50-57 with one plane */
          v = AT(A, cols, y / p0, x / p0);
          break;
        case 6: {  /* take_grad.h:52-60: the whole batch is walked for every element, in order */
          v = 0.0f;
          for (int64_t i = 0; i < rows; ++i)
            if ((int64_t)idx_r[i] == y) v += AT(A, cols, i, x);
        } break;
        default:  /* 7 */
          v = AT(A, cols, (int64_t)idx_r[y], x) * AT(B, cols, y, x) + (float)(x == (int64_t)idx_c[y]);
          break;
      }
      dst[y * ocols + x] = v;
    }
  }
}

/* ---- patch <-> column (extension/unpack_patch2col.h:115-133, pack_col2patch.h:108-140) ---- */

void ORC(unpack_patch2col)(float *mat, const float *img, int64_t n, int64_t c, int64_t h, int64_t w,
                           int psy, int psx, int sy, int sx, int dy, int dx) {
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  const int64_t rows = (int64_t)psy * psx * c, cols = oh * ow * n;
#pragma omp parallel for
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t x_offset = i % psx * dx, idivp = i / psx;
    const int64_t y_offset = idivp % psy * dy, ch = idivp / psy;
    for (int64_t j = 0; j < cols; ++j) {
      const int64_t x = (j % ow) * sx + x_offset, jdivw = j / ow;
      const int64_t y = (jdivw % oh) * sy + y_offset, ni = jdivw / oh;
      mat[i * cols + j] = (x < w && y < h) ? img[((ni * c + ch) * h + y) * w + x] : 0.0f;
    }
  }
}

void ORC(pack_col2patch)(float *img, const float *mat, int64_t n, int64_t c, int64_t h, int64_t w,
                         int psy, int psx, int sy, int sx, int dy, int dx) {
  const int64_t oh = (h - (dy * (psy - 1) + 1)) / sy + 1, ow = (w - (dx * (psx - 1) + 1)) / sx + 1;
  const int64_t cols = oh * ow * n;
  const int64_t psy_d = dy * (psy - 1) + 1, psx_d = dx * (psx - 1) + 1;
#pragma omp parallel for
  for (int64_t i = 0; i < n * c * h; ++i) {
    const int64_t y = i % h, idivh = i / h;
    const int64_t ch = idivh % c, ni = idivh / c;
    for (int64_t x = 0; x < w; ++x) {
      const int64_t py_min = y < psy_d ? y % dy : (y - psy_d + sy) / sy;
      const int64_t px_min = x < psx_d ? x % dx : (x - psx_d + sx) / sx;
      const int64_t py_max = imin((y + sy) / sy, oh), px_max = imin((x + sx) / sx, ow);
      float res = 0.0f;
      for (int64_t py = py_min; py < py_max; py += dy)
        for (int64_t px = px_min; px < px_max; px += dx)
          res += mat[((ch * psy + (y - py * sy) / dy) * psx + (x - px * sx) / dx) * cols +
                     (ni * oh + py) * ow + px];
      img[i * w + x] = res;
    }
  }
}

/* ---- expressions addressed by axis or box ---- */

/* begin and end of the box of cases 2 and 3 */
static void axis_box(int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t b[4], int64_t e[4]) {
  b[0] = p0 % n; b[1] = p1 % c; b[2] = p0 % h; b[3] = p1 % w;
  e[0] = n; e[1] = c; e[2] = b[2] + (h - b[2] + 1) / 2; e[3] = w;
}

int ORC(axis_shape)(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1, int64_t o[4]) {
  const int64_t s[4] = {n, c, h, w};
  int64_t b[4], e[4];
  o[0] = o[1] = o[2] = o[3] = 1;
  switch (id) {
    case 0:  /* range.h:79-83: repeat * ceil((stop - start) / step) in double */
      o[0] = 2 * (int64_t)ceil(((double)(float)(p0 + p1) - (double)(float)p0) / 0.5);
      return 1;
    case 1:
      o[0] = (int64_t)ceil(((double)(float)p0 - (double)(float)(p0 + p1)) / -1.5);
      return 1;
    case 2:
      axis_box(n, c, h, w, p0, p1, b, e);
      for (int k = 0; k < 4; ++k) o[k] = e[k] - b[k];
      return 4;
    case 3:
      for (int k = 0; k < 4; ++k) o[k] = s[k];
      return 4;
    case 4: case 5:  /* reduce_with_axis.h:39-48: the axis is dropped */
      for (int k = 0, m = 0; k < 4; ++k) if (k != p0) o[m++] = s[k];
      return 3;
    case 6:  /* reduce_with_axis.h:49-55: the axis keeps extent 1 */
      for (int k = 0; k < 4; ++k) o[k] = k == p0 ? 1 : s[k];
      return 4;
    case 7: {  /* broadcast_with_axis.h:46-53: a new axis of extent p1 behind axis p0 - 1 of (n*c, h, w) */
      const int64_t s3[3] = {n * c, h, w};
      for (int k = 0, m = 0; k < 4; ++k) o[k] = k == p0 ? p1 : s3[m++];
      return 4;
    }
    case 8: o[0] = n; o[1] = p1; o[2] = h; o[3] = w; return 4;
    case 9: o[0] = n; o[1] = p0; o[2] = h; o[3] = p1; return 4;
    default: o[0] = p0; o[1] = c; o[2] = p1; o[3] = w; return 4;
  }
}

void ORC(axis_case)(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0,
                    int64_t p1) {
  int64_t o[4], b[4], e[4];
  const int ndim = ORC(axis_shape)(id, n, c, h, w, p0, p1, o);
  const int64_t s[4] = {n, c, h, w};
  const int64_t cols = o[ndim - 1];
  int64_t rows = 1;
  for (int k = 0; k + 1 < ndim; ++k) rows *= o[k];
  axis_box(n, c, h, w, p0, p1, b, e);
  if (id == 3) {
    for (int64_t i = 0; i < n * c * h * w; ++i) dst[i] = A[i] * 2.0f;
    /* slice_ex.h:112-121: the same row/column mapping, written through */
    const int64_t bs[4] = {e[0] - b[0], e[1] - b[1], e[2] - b[2], e[3] - b[3]};
    for (int64_t i = 0; i < bs[0] * bs[1] * bs[2]; ++i) {
      int64_t idx = 0, stride = 1, r = i;
      for (int k = 2; k >= 0; --k) {
        idx += stride * (r % bs[k] + b[k]);
        r /= bs[k];
        stride *= s[k];
      }
      for (int64_t j = 0; j < bs[3]; ++j) AT(dst, w, idx, j + b[3]) = AT(A, w, idx, j + b[3]) + 1.0f;
    }
    return;
  }
  /* reductions (cases 4-6): trailing = product of the extents behind the axis, size = the axis' extent */
  int64_t trailing = 1, size = 1;
  if (id >= 4 && id <= 6) {
    size = s[p0];
    for (int64_t k = p0 + 1; k < 4; ++k) trailing *= s[k];
  }
#pragma omp parallel for
  for (int64_t i = 0; i < rows; ++i) {
    for (int64_t j = 0; j < cols; ++j) {
      const int64_t lin = i * cols + j;
      float v = 0.0f;
      switch (id) {
        case 0:  /* range.h:53-55 */
          v = (float)p0 + (float)((int)j / 2) * 0.5f;
          break;
        case 1:
          v = (float)(p0 + p1) + (float)((int)j / 1) * -1.5f;
          break;
        case 2: {  /* slice_ex.h:101-111 */
          int64_t idx = 0, stride = 1, r = i;
          for (int k = 2; k >= 0; --k) {
            idx += stride * (r % o[k] + b[k]);
            r /= o[k];
            stride *= s[k];
          }
          v = AT(A, w, idx, j + b[3]);
        } break;
        case 4: case 5: case 6: {  /* reduce_with_axis.h:103-127 */
          const int64_t x = lin / trailing, y = lin % trailing;
          float res = id == 4 ? 0.0f : (id == 5 ? -FLT_MAX : FLT_MAX);
          int64_t pos = 0;
          for (int64_t k = 0; k < size; ++k) {
            const int64_t z = (x * size + k) * trailing + y;
            const float a = AT(A, w, z / w, z % w), before = res;
            if (id == 4) res += a;
            else if (id == 5) res = res < a ? a : res;
            else res = a < res ? a : res;
            if (before != res) pos = k;
          }
          v = id == 5 ? (float)(int)pos : res;
        } break;
        case 7: {  /* broadcast_with_axis.h:205-210: source (n*c, h, w), last extent w */
          int64_t tr = 1;
          const int64_t s3[3] = {n * c, h, w};
          for (int64_t k = p0; k < 3; ++k) tr *= s3[k];
          const int64_t x = lin / tr / p1, y = lin % tr, z = x * tr + y;
          v = AT(A, w, z / w, z % w);
        } break;
        case 8: {  /* source slice<1>(A, 0, 1) = (n, 1, h, w): trailing h*w, last extent w; slice.h:101-109 */
          const int64_t tr = h * w, x = lin / tr / p1, y = lin % tr, z = x * tr + y;
          const int64_t srow = z / w, scol = z % w;  /* row (b, 0, yy) of the slice is row (b*c + 0)*h + yy of A */
          v = AT(A, w, (srow / h) * c * h + srow % h, scol);
        } break;
        case 9: {  /* broadcast_with_axis.h:229-238: axes (1, 3) of (n, 1, h, 1), trailings (h*p1, 1), last extent 1 */
          int64_t idx = lin;
          idx = (idx / (h * p1) / p0) * (h * p1) + idx % (h * p1);
          idx = (idx / 1 / p1) * 1 + idx % 1;
          v = A[idx];
        } break;
        default: {  /* axes (0, 2) of (1, c, 1, w): trailings (c*p1*w, w), last extent w */
          int64_t idx = lin;
          idx = (idx / (c * p1 * w) / p0) * (c * p1 * w) + idx % (c * p1 * w);
          idx = (idx / w / p1) * w + idx % w;
          v = A[idx];
        } break;
      }
      dst[lin] = v;
    }
  }
}

/* ---- complex arithmetic: extension/complex.h:17-112 (operators), :370-489 (which operand elements feed
        column x: the pair (x & ~1, x | 1) of a complex operand, element x / 2 of a real one) ---- */

static float cmul_part(int imag, float ar, float ai, float br, float bi) {
  return imag ? ar * bi + br * ai : ar * br - ai * bi;
}
static float cdiv_part(int imag, float ar, float ai, float br, float bi) {
  return imag ? (br * ai - ar * bi) / (br * br + bi * bi) : (ar * br + ai * bi) / (br * br + bi * bi);
}

void ORC(complex_case)(int id, float *dst, const float *A, const float *B, int64_t rows, int64_t cols) {
  const int64_t half = cols / 2, ocols = (id >= 9 && id <= 11) ? half : cols;
#pragma omp parallel for
  for (int64_t y = 0; y < rows; ++y) {
    const float *a = A + y * cols, *b = B + y * cols;  /* complex rows */
    const float *ah = A + y * half, *bh = B + y * half; /* real rows */
    for (int64_t x = 0; x < ocols; ++x) {
      const int64_t re = x & ~(int64_t)1, im = re + 1, h = x / 2;
      const int imag = (int)(x & 1);
      float v;
      switch (id) {
        case 0: v = cmul_part(imag, a[re], a[im], b[re], b[im]); break;
        case 1: v = cmul_part(imag, a[re], a[im], bh[h], 0.0f); break;
        case 2: v = cmul_part(imag, ah[h], 0.0f, b[re], b[im]); break;
        case 3: v = cdiv_part(imag, a[re], a[im], b[re], b[im]); break;
        case 4: v = cdiv_part(imag, a[re], a[im], bh[h], 0.0f); break;
        case 5: v = cdiv_part(imag, ah[h], 0.0f, b[re], b[im]); break;
        case 6: v = imag ? -a[im] : a[re]; break;
        case 7: v = imag ? a[re] : a[im]; break;
        case 8: v = imag ? 0.0f : ah[h]; break;
        case 9: v = a[2 * x]; break;
        case 10: v = a[2 * x] * a[2 * x] + a[2 * x + 1] * a[2 * x + 1]; break;
        case 11: v = a[2 * x] + a[2 * x + 1]; break;
        default: {
          const float prod = cmul_part(imag, a[re], -a[im], b[re], b[im]);
          const float pad = imag ? 0.0f : b[2 * h] * b[2 * h] + b[2 * h + 1] * b[2 * h + 1];
          v = prod + pad * 0.5f;
        } break;
      }
      dst[y * ocols + x] = v;
    }
  }
}

int ORC(num_threads)(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void ORC(set_num_threads)(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
