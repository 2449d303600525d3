/*
 * C ABI of the B200 evaluation engine for the mshadow lazy-evaluation path.
 *
 * dmlc/mshadow has no FFI of its own: its public interface is a C++ template header API
 * (mshadow/tensor.h).  The template part of that interface (expression plans) cannot cross
 * a C boundary and stays in headers (mshadow_b200/include/mshadow/); everything that is not
 * a template -- the function-form operators, memory, streams, and fp32 instantiations of
 * the reductions and pooling expressions -- is exported here with plain pointers and
 * sizes.  Each entry names the reference interface it stands for (file:line within
 * dmlc/mshadow).
 *
 * Conventions
 *   - every function returns an msb_status; 0 is success.  Nothing throws or aborts.
 *     msb_last_error() returns a thread-local, human-readable description of the last
 *     failure on the calling thread.
 *   - device pointers are raw CUDA device addresses; `ld_*` are leading dimensions counted
 *     in elements (mshadow's Tensor::stride_); sizes are int64_t.
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 *     default stream) and is asynchronous, like every mshadow GPU operation
 *     (mshadow/tensor_gpu-inl.h:101-156).  The caller synchronises.
 *   - `saver` selects mshadow's sv::saveto/plusto/minusto/multo/divto as 0..4
 *     (mshadow/base.h:539-602); `reducer` selects red::sum / maximum / minimum as 0..2
 *     (mshadow/base.h:604-862).
 *   - operators may use a library-owned scratch buffer that is cached per (device, stream)
 *     and released by msb_shutdown(); callers never see it, in keeping with mshadow's
 *     "no temporary allocation" contract (README.md:19-20 of the reference).
 */
#ifndef MSHADOW_B200_C_API_H_
#define MSHADOW_B200_C_API_H_

#include <stdint.h>

#include "mshadow_b200_peer_sink.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  MSB_OK = 0,
  MSB_ERR_ARGUMENT = 1,  /* null pointer, negative size, unknown selector */
  MSB_ERR_SHAPE = 2,     /* shapes of the operands do not agree */
  MSB_ERR_LAYOUT = 3,    /* operand must be contiguous / sufficiently aligned */
  MSB_ERR_CUDA = 4,      /* a CUDA runtime call or kernel launch failed */
  MSB_ERR_MEMORY = 5,    /* allocation failed */
  MSB_ERR_TIMEOUT = 6    /* a bounded device-side wait gave up */
} msb_status;

typedef void *msb_stream_t; /* cudaStream_t */

const char *msb_last_error(void);
int msb_version(void);
/* Number of kernels the library has launched so far in this process (its own kernels only;
   library sorts and memory copies are not counted).  No counterpart in the reference;
   benchmarks use the difference across a timed region. */
int64_t msb_launch_count(void);

/* ---- engine life cycle and streams ------------------------------------------------- */

/* InitTensorEngine<gpu>(dev) / SetDevice<gpu>(dev): mshadow/tensor_gpu-inl.h:14-36 */
int msb_init(int device);
int msb_set_device(int device);
/* ShutdownTensorEngine<gpu>(): additionally frees every cached scratch buffer */
int msb_shutdown(void);
/* NewStream<gpu> / DeleteStream / Stream<gpu>::Wait / CheckIdle: mshadow/stream_gpu-inl.h:18-211 */
int msb_stream_create(msb_stream_t *out);
int msb_stream_destroy(msb_stream_t stream);
int msb_stream_wait(msb_stream_t stream);
int msb_stream_idle(msb_stream_t stream, int *idle);
/* Self-test of the failure path that every kernel with a device-side wait relies on (no counterpart
   in the reference, whose kernels do not wait): one thread waits, bounded by limit_ms (1..1000), on a
   barrier that nothing signals, gives up, and marks the device status word.  The next msb_stream_wait
   on the stream must then return MSB_ERR_TIMEOUT, and the device stays usable. */
int msb_selftest_bounded_wait(int limit_ms, msb_stream_t stream);

/* ---- memory ------------------------------------------------------------------------ */

/* AllocSpace(Tensor<gpu,...>*, pad) / FreeSpace: mshadow/tensor_gpu-inl.h:37-56.
   rows = product of all but the last extent, cols = last extent.  With pad != 0 and
   cols >= 64 the rows are pitched; *ld_out receives the resulting stride in elements. */
int msb_alloc_space(void **dptr_out, int64_t *ld_out, int64_t rows, int64_t cols,
                    int64_t elem_size, int pad);
int msb_free_space(void *dptr);
/* AllocHost<gpu> / FreeHost<gpu> (page-locked host memory): mshadow/tensor_cpu-inl.h:60-92 */
int msb_alloc_host(void **ptr_out, int64_t bytes);
int msb_free_host(void *ptr);
/* Copy(dst, src, stream) in its host->device (1), device->host (2) and device->device (3)
   forms: mshadow/tensor_gpu-inl.h:57-92.  Honours both strides. */
int msb_copy_2d(void *dst, int64_t ld_dst, const void *src, int64_t ld_src, int64_t rows,
                int64_t cols, int64_t elem_size, int kind, msb_stream_t stream);
/* Scratch buffer of at least `bytes` for the caller's own work on `stream`; owned by the library
   (one per device and stream, grown on demand, released by msb_stream_destroy / msb_shutdown).
   It is not the buffer the operators use internally, so calls to them leave its contents alone.
   The pointer stays valid until the next msb_workspace call on the same stream that asks for
   more (the buffer is then replaced after the stream has drained). */
int msb_workspace(msb_stream_t stream, int64_t bytes, void **out);
/* No counterpart in the reference: bytes of device memory the library currently holds for `stream`
   on the current device, as the operators' internal scratch and as the caller's workspace.  Lets
   an integrator see when (and that) the library allocated on its behalf. */
int msb_scratch_bytes(msb_stream_t stream, int64_t *engine_bytes, int64_t *caller_bytes);

/* ---- element-wise expressions (MapExp): mshadow/tensor_gpu-inl.h:101-116 -------------
   Expression plans are C++ templates; these are fixed fp32 instantiations compiled from the
   header API, exported so that non-C++ callers and the parity tests can reach the fused
   map kernel.  `id`:
     0  dst  = F<sigmoid>(A*B + 0.5f*C) + repmat(bias, rows)   sigmoid(a) = 1/(1+exp(-a))
     1  dst += A*2.0f - B/C
     2  dst  = F<clip_mul>(A, B) * C          clip_mul(a,b) = a > b ? a*b : b
     3  dst *= A + 1.5f
     4  dst -= A * B
     5  dst /= C*C + 1.0f
     6  dst  = 3.25f
     7  dst  = F<fma3>(A, B, C)               fma3(a,b,c) = a*b + c, two roundings
     8  dst  = broadcast<0>(bias, shape) * A + B      (bias has `rows` entries)
     9  dst  = F<square>(A - 1.0f) / (B*B + 2.0f) + C
   `bias` must hold max(rows, cols) floats. */
int msb_expr_case_f32(int id, float *dst, const float *A, const float *B, const float *C,
                      const float *bias, int64_t rows, int64_t cols, int64_t ld_dst,
                      int64_t ld_a, int64_t ld_b, int64_t ld_c, msb_stream_t stream);

/* ---- reductions --------------------------------------------------------------------- */

/* MapReduceKeepLowest<Saver,Reducer>(dst, src, scale) -- e.g. dst = sum_rows(src):
   mshadow/tensor_gpu-inl.h:118-133, mshadow/extension/reduceto1d.h:77-101 */
int msb_reduce_keep_lowest_f32(float *dst, const float *src, int64_t rows, int64_t cols,
                               int64_t ld, float scale, int saver, int reducer,
                               msb_stream_t stream);
/* dst[x] = scale * sum over rows of src(y, x), computed exactly as by
   msb_reduce_keep_lowest_f32 with saver 0 / reducer 0, but WITHOUT allocating anything.
   This entry point has no counterpart in the reference.  It is for callers that must not
   cause a cudaMalloc at call time (frozen memory pools, real-time paths that cannot take
   cudaMalloc's implicit device synchronisation, processes whose device memory is already
   fully assigned).  Its cross-cluster scratch is a fixed 1 MiB array inside the library's
   device image, resident on every GPU that loads the library.  Limits and rules:
     - inputs whose partial rows (clusters x cols floats) exceed 1 MiB are rejected with
       MSB_ERR_SHAPE and nothing is launched;
     - the first call on a device resolves the array's address; make that call before any
       stream capture begins;
     - all calls share the array, so calls that can overlap on the GPU (different streams
       without ordering) race and must be serialised by the caller. */
int msb_reduce_keep_lowest_sum_f32_noalloc(float *dst, const float *src, int64_t rows,
                                           int64_t cols, int64_t ld, float scale,
                                           msb_stream_t stream);
/* MapReduceKeepHighDim<Saver,Reducer,1>(dst, src(n,c,h,w), scale) -- e.g.
   dst = sumall_except_dim<1>(src): mshadow/tensor_gpu-inl.h:135-156 */
int msb_reduce_keep_highdim_f32(float *dst, const float *src, int64_t n, int64_t c, int64_t h,
                                int64_t w, int64_t ld, float scale, int saver, int reducer,
                                msb_stream_t stream);
/* The same two reductions with their results also delivered to the other GPUs of an exchange
   group, from the threads that compute them (no second kernel): see mshadow_b200_peer_sink.h.
   No counterpart in the reference.  `sink` may be NULL (then they are the calls above); it must
   expect exactly cols (c) results.  The value delivered is scale * Reduce(...), i.e. what the
   saver receives, whatever the saver does with dst. */
int msb_reduce_keep_lowest_f32_sink(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld,
                                    float scale, int saver, int reducer, const msb_peer_sink_t *sink,
                                    msb_stream_t stream);
int msb_reduce_keep_highdim_f32_sink(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                                     int64_t ld, float scale, int saver, int reducer, const msb_peer_sink_t *sink,
                                     msb_stream_t stream);


/* ---- softmax family ----------------------------------------------------------------- */

/* Softmax(Tensor<gpu,2>, Tensor<gpu,2>): mshadow/tensor_gpu-inl.h:157-161 */
int msb_softmax_f32(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst,
                    int64_t ld_src, msb_stream_t stream);
/* SoftmaxGrad / SmoothSoftmaxGrad, with and without ignore_label:
   mshadow/tensor_gpu-inl.h:169-214.  mode bit0 = smoothing by `alpha`, bit1 = rows whose
   label equals `ignore_label` become zero.  Labels are floats holding integers. */
int msb_softmax_grad_f32(float *dst, const float *src, const float *label, int64_t rows,
                         int64_t cols, int64_t ld_dst, int64_t ld_src, int mode,
                         float ignore_label, float alpha, msb_stream_t stream);

/* dst = Softmax(logits) - onehot(label) in ONE pass: the result of msb_softmax_f32 followed
   by msb_softmax_grad_f32 (mode 0) without storing the probabilities.  No counterpart in the
   reference; for loss layers that need only the gradient (8 instead of 16 bytes per element). */
int msb_softmax_grad_fused_f32(float *dst, const float *logits, const float *label, int64_t rows,
                               int64_t cols, int64_t ld_dst, int64_t ld_src, msb_stream_t stream);

/* ---- pooling expressions (fp32 instantiations over plain tensors) -------------------- */

/* dst = pool<Reducer>(src, ky, kx, sy, sx) on `planes` images of h x w; output
   ((h-ky)/sy+1) x ((w-kx)/sx+1): mshadow/extension/spatial_pool.h:20-149 */
int msb_pool_f32(float *dst, const float *src, int64_t planes, int64_t h, int64_t w, int ky,
                 int kx, int sy, int sx, int64_t ld_src, int64_t ld_dst, int reducer,
                 msb_stream_t stream);
/* dst = unpool<Reducer>(src, pooled, grad_pooled, ky, kx, sy, sx):
   mshadow/extension/spatial_unpool.h:20-132 */
int msb_unpool_f32(float *dst, const float *src, const float *pooled, const float *gpooled,
                   int64_t planes, int64_t h, int64_t w, int64_t ph, int64_t pw, int ky, int kx,
                   int sy, int sx, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst,
                   int reducer, msb_stream_t stream);
/* dst = chpool<Reducer>(src, nsize, stride, pad) on (n, c, h, w):
   mshadow/extension/channel_pool.h:21-104 */
int msb_chpool_f32(float *dst, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                   int nsize, int stride, int pad, int64_t ld_src, int64_t ld_dst, int reducer,
                   msb_stream_t stream);

/* dst = ch_unpool<Reducer>(src, pooled, grad_pooled, nsize, stride, pad), the gradient of
   chpool; src and dst are (n, c, h, w), pooled and grad_pooled (n, pc, h, w):
   mshadow/extension/channel_unpool.h:20-133.  Shapes for which the reference's window would
   run past the pooled channels (it clamps with c, not pc) are refused with MSB_ERR_SHAPE. */
int msb_ch_unpool_f32(float *dst, const float *src, const float *pooled, const float *gpooled,
                      int64_t n, int64_t c, int64_t pc, int64_t h, int64_t w, int nsize, int stride,
                      int pad, int64_t ld_src, int64_t ld_pooled, int64_t ld_dst, int reducer,
                      msb_stream_t stream);
/* Local response normalisation across channels as single passes (no single reference call: a layer
   written against the reference composes it from chpool<red::sum> and its own square / power
   functors, mshadow/extension/channel_pool.h:77-104, channel_unpool.h:102-133):
     forward    norm = chpool<red::sum>(F<square>(src), nsize) * salpha + knorm;
                out  = src * F<power>(norm, -beta);                       (norm may be NULL: not kept)
     backward   gsrc  = gout * F<power>(norm, -beta);
                gsrc += (-2.0f * beta * salpha) * chpool<red::sum>(gout * src * F<power>(norm, -beta - 1.0f), nsize) * src;
   Dense (n, c, h, w) tensors.  power_kind 0: powf; 1: exponents -0.75 and -1.75 from square roots
   (bit-identical on every device); 2: the GPU's fast exp2 / log2 units (about 2^-21 relative).
   Products and sums are rounded one by one in the order of the expressions. */
int msb_lrn_forward_f32(float *out, float *norm, const float *src, int64_t n, int64_t c, int64_t h, int64_t w,
                        int nsize, float salpha, float beta, float knorm, int power_kind, msb_stream_t stream);
int msb_lrn_backward_f32(float *gsrc, const float *gout, const float *src, const float *norm, int64_t n,
                         int64_t c, int64_t h, int64_t w, int nsize, float salpha, float beta, int power_kind,
                         msb_stream_t stream);


/* ---- embedding backward --------------------------------------------------------------- */

/* AddTakeGrad(dst, index, src): dst[clip(index[y])] += src[y]:
   mshadow/tensor_gpu-inl.h:216-221 */
int msb_addtakegrad_f32_i32(float *dst, const int32_t *index, const float *src, int64_t k,
                            int64_t d, int64_t nidx, int64_t ld_dst, int64_t ld_src,
                            msb_stream_t stream);
/* AddTakeGradLargeBatch(dst, sorted, index, src): dst[sorted[y]] += src[index[y]], all
   operands contiguous, `sorted` ascending: mshadow/tensor_gpu-inl.h:223-229 */
int msb_addtakegrad_largebatch_f32_i32(float *dst, const int32_t *sorted, const int32_t *index,
                                       const float *src, int64_t k, int64_t d, int64_t nidx,
                                       msb_stream_t stream);
/* SortByKey(keys, values, is_ascend), stable: mshadow/tensor_gpu-inl.h:231-235 */
int msb_sort_by_key_i32(int32_t *keys, int32_t *values, int64_t n, int ascend,
                        msb_stream_t stream);
/* The `count` most frequent keys of an ascending key list, most frequent first, equal counts in
   ascending key order: rows_out[count], counts_out[count] (device memory).  Fewer distinct keys
   than `count` leave trailing entries with counts_out == 0.  Host-side helper of the row-sharded
   AddTakeGradLargeBatch (mshadow/tensor_gpu-inl.h:223-229 on one slice of the table per GPU);
   the reference has no multi-GPU form of it. */
int msb_frequent_rows_i32(int32_t *rows_out, int32_t *counts_out, const int32_t *sorted,
                          int64_t n, int64_t count, msb_stream_t stream);
/* Numbers the runs of equal keys of an ascending list: run_of[i] = 0, 1, ... for every entry,
   run_keys[j] = the key of run j (room for n entries), total[0] (a device word) = number of
   runs.  msb_addtakegrad_largebatch_f32_i32 with run_of in place of `sorted` sums into a compact
   matrix of one row per distinct key: what a GPU hands to the owners of the table rows when
   the source rows are spread over the GPUs by batch position. */
int msb_run_index_i32(int32_t *run_of, int32_t *run_keys, uint32_t *total, const int32_t *sorted,
                      int64_t n, msb_stream_t stream);
/* The three calls below serve AddTakeGradLargeBatch when the SOURCE rows are spread over the GPUs
   by batch position and table row t lives on GPU t % world as local row t / world.  A GPU sorts
   its entries by the key (t % world) * per_owner + t / world, numbers the runs
   (msb_run_index_i32), and then:
   msb_run_bounds_i32: first[q] (device, world + 1 entries) = number of runs whose key is below
     q * per_owner: the runs of owner q are first[q] .. first[q + 1] - 1.
   msb_take_sum_to_owners_f32_i32: the sum of the source rows of run j is STORED into row
     j - first[q] of row_blocks[q] (host array of `world` device addresses, 16-byte aligned, row
     pitch d; an address may belong to another GPU's memory mapped into this process, see
     msb_ps_peer_window: the kernel only stores there, 16 bytes at a time, each row once).
   msb_run_keys_to_owners_i32: key_blocks[q][j - first[q]] = run key - q * per_owner, the owner's
     own row number, beside the rows.
   The owner then sorts what it received by row and adds it with
   msb_addtakegrad_largebatch_f32_i32, its receive block as `src`.  The reference has no
   multi-GPU form of this operator (mshadow/tensor_gpu-inl.h:223-229 serves one device). */
int msb_run_bounds_i32(int32_t *first, const int32_t *run_keys, const uint32_t *total, int world,
                       int64_t per_owner, msb_stream_t stream);
int msb_run_keys_to_owners_i32(int32_t *const *key_blocks, const int32_t *first,
                               const int32_t *run_keys, int64_t n, int world, int64_t per_owner,
                               msb_stream_t stream);
int msb_take_sum_to_owners_f32_i32(float *const *row_blocks, const int32_t *first,
                                   const int32_t *run_of, const int32_t *index, const float *src,
                                   int64_t d, int64_t nidx, int world, msb_stream_t stream);
/* This GPU's part of AddTakeGradLargeBatch's (sorted, index) lists when table row r lives on
   GPU r % world as local row r / world and the rows listed in `hot` (ascending, <= 1024) are
   summed by every GPU over the source rows [src_begin, src_end) it holds.  Writes, in list order,
   first the entries of this GPU's rows with keys rewritten to local rows, then its hot entries
   with keys hot_base + position in `hot`; totals[0], totals[1] (device words) receive the two
   counts.  keys_out / rows_out need room for n entries.  With hot_base = number of local rows the
   output is one ascending list for a single msb_addtakegrad_largebatch_f32_i32 call. */
int msb_route_cyclic_hot_i32(int32_t *keys_out, int32_t *rows_out, uint32_t *totals,
                             const int32_t *sorted, const int32_t *index, int64_t n,
                             const int32_t *hot, int64_t hot_count, int world, int rank,
                             int64_t src_begin, int64_t src_end, int64_t hot_base,
                             msb_stream_t stream);
/* SortByKey (ascending, stable) for keys known to lie in [0, 2^bits): only those bits are
   sorted, in an even number of passes of at most nine bits (row numbers of a 2^18-row table:
   two passes instead of the four of msb_sort_by_key_i32).  Keys outside the range give an
   order by their low bits only. */
int msb_sort_by_key_lowbits_i32(int32_t *keys, int32_t *values, int64_t n, int bits,
                                msb_stream_t stream);
/* VectorizedSort(values, segments): values sorted ascending inside each run of equal
   `segments` (ascending on entry), two stable pair sorts: mshadow/tensor.h:905-915,
   mshadow/tensor_cpu-inl.h:562-567 */
int msb_vectorized_sort_f32_i32(float *values, int32_t *segments, int64_t n, msb_stream_t stream);
/* IndexFill(dst, index, src): dst[index[y]] = src[y], dst is k x d and src nidx x d, both
   contiguous: mshadow/tensor_gpu-inl.h:237-242.  A row named by several entries keeps the last
   one (the CPU evaluator's outcome, mshadow/tensor_cpu-inl.h:520-529); entries outside [0, k)
   are skipped. */
int msb_index_fill_f32_i32(float *dst, const int32_t *index, const float *src, int64_t k,
                           int64_t d, int64_t nidx, msb_stream_t stream);

/*
 * Index-remapping expressions (pure data movement) evaluated by MapExp on dense fp32 tensors A
 * and B of shape (n, c, h, w); p0 and p1 are per-case parameters.  Expression plans cannot
 * cross a C ABI, so a fixed set is exported, as for msb_expr_case_f32:
 *    0  dst = reshape(A, Shape4(n, h, c, w))                 mshadow/extension/reshape.h
 *    1  dst = slice<1>(A, p0, p1)                            mshadow/extension/slice.h
 *    2  dst = slice<3>(A, p0, p1)
 *    3  dst = concat<1>(A, B)                                mshadow/extension/concat.h
 *    4  dst = concat<3>(A, B)
 *    5  dst = swapaxis<2, 1>(A)                              mshadow/extension/swapaxis.h
 *    6  dst = swapaxis<3, 1>(A)
 *    7  dst = transpose(A, Shape4(0, 2, 1, 3))               mshadow/extension/transpose.h
 *    8  dst = transpose(A, Shape4(3, 1, 0, 2))
 *    9  dst = pad(A, p0, p1)                                 mshadow/extension/pad.h
 *   10  dst = crop(A, Shape2(p0, p1))                        mshadow/extension/crop.h
 *   11  dst = crop(A, Shape2(p0, p1), h - p0, w - p1)
 *   12  dst = mirror(A)                                      mshadow/extension/mirror.h
 *   13  dst = flip(A, 1)                                     mshadow/extension/flip.h
 *   14  dst = B; slice<1>(dst, p0, p1) = slice<1>(A, p0, p1) + 1.0f
 *   15  concat<1>(dst[0:n], dst[n:2n]) = F<op::identity>(concat<1>(B, A)), dst is (2n, c, h, w)
 *   16  dst = crop(pad(A, p0, p1), Shape2(h, w)) + mirror(A)
 * msb_remap_shape reports the (dense) shape dst must have.  Arguments the expressions' own
 * checks reject (a slice out of range, a crop larger than the image) return MSB_ERR_SHAPE.
 */
int msb_remap_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                    int64_t *out_shape);
int msb_remap_case_f32(int id, float *dst, const float *A, const float *B, int64_t n, int64_t c,
                       int64_t h, int64_t w, int64_t p0, int64_t p1, msb_stream_t stream);

/*
 * Index-selecting expressions evaluated by MapExp on dense fp32 matrices A and B (rows x cols);
 * idx_r: `rows` integers in [0, rows) stored as floats, idx_c: `rows` integers in [0, cols).
 * Result (rows x cols) unless noted:
 *    0  dst = take(idx_r, A)                                  mshadow/extension/take.h
 *    1  dst = one_hot_encode(idx_c, cols)                     mshadow/extension/one_hot.h
 *    2  dst = mat_choose_row_element(A, idx_c)     (rows)     mshadow/extension/choose.h
 *    3  dst = mat_fill_row_element(A, B[0:rows], idx_c)       mshadow/extension/fill.h
 *    4  dst = mask(idx_c, A)                                  mshadow/extension/mask.h
 *    5  dst = upsampling_nearest(A, p0)   (rows*p0, cols*p0)  mshadow/extension/spatial_upsampling_nearest.h
 *    6  dst = take_grad(idx_r, A, rows)                       mshadow/extension/take_grad.h
 *    7  dst = take(idx_r, A) * B + one_hot_encode(idx_c, cols)
 * Index values outside their range are not checked (they are not in the reference either).
 */
int msb_select_case_f32(int id, float *dst, const float *A, const float *B, const float *idx_r,
                        const float *idx_c, int64_t rows, int64_t cols, int64_t p0,
                        msb_stream_t stream);

/*
 * Patch <-> column conversion for convolutions on a dense (n, c, h, w) image:
 *   mat = unpack_patch2col(img, psy, psx, sy, sx, dy, dx)      mshadow/extension/unpack_patch2col.h
 *   img = pack_col2patch(mat, imshape, psy, psx, sy, sx, dy, dx)   mshadow/extension/pack_col2patch.h
 * with patch size (psy, psx), stride (sy, sx) and dilation (dy, dx).  The matrix is dense,
 * (psy*psx*c) x (oh*ow*n) with oh = (h - (dy*(psy-1)+1))/sy + 1 and ow likewise.
 */
int msb_unpack_patch2col_f32(float *mat, const float *img, int64_t n, int64_t c, int64_t h,
                             int64_t w, int psy, int psx, int sy, int sx, int dy, int dx,
                             msb_stream_t stream);
int msb_pack_col2patch_f32(float *img, const float *mat, int64_t n, int64_t c, int64_t h,
                           int64_t w, int psy, int psx, int sy, int sx, int dy, int dx,
                           msb_stream_t stream);

/*
 * Expressions addressed by an axis number or a begin/end box, evaluated by MapExp on a dense fp32
 * tensor A of shape (n, c, h, w); p0 and p1 are per-case parameters:
 *    0  dst = range(p0, p0 + p1, 0.5f, 2)            (1-d)        mshadow/extension/range.h
 *    1  dst = range(p0 + p1, p0, -1.5f, 1)           (1-d)
 *    2  dst = slice(A, begin, end)                                mshadow/extension/slice_ex.h
 *         begin = (p0 % n, p1 % c, p0 % h, p1 % w), end = (n, c, begin_h + (h - begin_h + 1) / 2, w)
 *    3  dst = A * 2;  slice(dst, begin, end) = slice(A, begin, end) + 1
 *    4  dst = reduce_with_axis<red::sum, false>(A, p0)   (3-d)    mshadow/extension/reduce_with_axis.h
 *    5  dst = reduce_with_axis<red::maximum, true>(A, p0)     (position of the maximum along axis p0)
 *    6  dst = reduce_keepdim<red::minimum, false>(A, p0)
 *    7  dst = broadcast_with_axis(A3, p0 - 1, p1), A3 = A seen as (n*c, h, w)   mshadow/extension/broadcast_with_axis.h
 *    8  dst = broadcast_keepdim(slice<1>(A, 0, 1), 1, p1)         -> (n, p1, h, w)
 *    9  dst = broadcast_to(S, (n, p0, h, p1)), S = the first n*h elements of A seen as (n, 1, h, 1)
 *   10  dst = broadcast_multi_axes(S, axes (0, 2), sizes (p0, p1)), S = the first c*w elements of A
 *         seen as (1, c, 1, w)                                    -> (p0, c, p1, w)
 * msb_axis_shape reports the extents of the (dense) result: *out_ndim of them in out_shape[0..3],
 * the rest 1.  Parameters outside a case's domain return MSB_ERR_SHAPE.
 */
int msb_axis_shape(int id, int64_t n, int64_t c, int64_t h, int64_t w, int64_t p0, int64_t p1,
                   int64_t *out_shape, int *out_ndim);
int msb_axis_case_f32(int id, float *dst, const float *A, int64_t n, int64_t c, int64_t h, int64_t w,
                      int64_t p0, int64_t p1, msb_stream_t stream);

/*
 * Complex arithmetic (mshadow/extension/complex.h) evaluated by MapExp.  A and B are dense fp32
 * matrices of rows x cols floats read as rows x cols/2 complex numbers (re, im interleaved); Ah and
 * Bh are the first rows*cols/2 floats of the same buffers read as real rows x cols/2 matrices.
 * cols must be a multiple of 4.  dst is dense, rows x cols unless noted:
 *    0  complex_mul_cc(A, B)      1  complex_mul_cr(A, Bh)     2  complex_mul_rc(Ah, B)
 *    3  complex_div_cc(A, B)      4  complex_div_cr(A, Bh)     5  complex_div_rc(Ah, B)
 *    6  conj(A)                   7  complex_exchange(A)       8  complex_pad_imag(Ah)
 *    9  complex_toreal(A)        10  complex_abs_square(A)    11  complex_sum_real_imag(A)   (rows x cols/2)
 *   12  complex_mul_cc(conj(A), B) + complex_pad_imag(complex_abs_square(B)) * 0.5f
 */
int msb_complex_case_f32(int id, float *dst, const float *A, const float *B, int64_t rows,
                         int64_t cols, msb_stream_t stream);

/* Softmax(Tensor<gpu,3>): softmax over the middle axis of (batch, classes, positions);
   ld_* = pitch of the last axis: mshadow/tensor_gpu-inl.h:163-167 */
int msb_softmax3d_f32(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos,
                      int64_t ld_dst, int64_t ld_src, msb_stream_t stream);
/* SoftmaxGrad / SmoothSoftmaxGrad on (batch, classes, positions) with label (batch, positions);
   mode as for msb_softmax_grad_f32: mshadow/tensor_gpu-inl.h:201-214,
   mshadow/tensor_cpu-inl.h:370-462 */
int msb_softmax_grad3d_f32(float *dst, const float *src, const float *label, int64_t batch,
                           int64_t classes, int64_t npos, int64_t ld_dst, int64_t ld_src,
                           int64_t ld_label, int mode, float ignore_label, float alpha,
                           msb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MSHADOW_B200_C_API_H_ */
