/*
 * C ABI of the multi-GPU synchronisation model (libmshadow_b200_ps.so): the ISharedModel
 * interface of dmlc/mshadow's mshadow-ps (mshadow-ps/mshadow_ps.h:37-258: Init, InitKey, Push,
 * PullReq, PullWait, SetWeight, CheckWeight) for fp32 tensors, implemented by NCCL all-reduce
 * between one process per GPU (C++ class: mshadow::ps::NcclModel in mshadow-ps/mshadow_ps.h of
 * this package).  It replaces mshadow::ps::CreateSharedModel<gpu, float>("local") and the
 * LocalModel behind it (mshadow-ps/ps_local-inl.h), which stages every tensor through host
 * memory inside one multi-threaded process.
 *
 * All functions return 0 on success and a non-zero status otherwise; msb_ps_last_error() then
 * describes the failure.  Pointers are device pointers of the GPU the model was created on;
 * matrices are row-major with a leading dimension `ld` in elements.
 */
#ifndef MSHADOW_B200_PS_C_API_H_
#define MSHADOW_B200_PS_C_API_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *msb_ps_t;

const char *msb_ps_last_error(void);

/* Writes a new group identifier (256 hexadecimal digits and a terminating zero) into `hex`;
   `capacity` must be at least 257.  Call on ONE process and hand the text to the others. */
int msb_ps_new_unique_id(char *hex, int64_t capacity);

/* ISharedModel::SetParam("rank" / "world_size" / "nccl_id") + Init({device}): collective over
   all `world` processes.  `id_hex` may be NULL when world is 1. */
int msb_ps_create(int rank, int world, const char *id_hex, int device, msb_ps_t *out);
int msb_ps_destroy(msb_ps_t model);

/* ISharedModel::InitKey(Shape2(rows, cols), key, device) */
int msb_ps_init_key(msb_ps_t model, int key, int64_t rows, int64_t cols);
/* ISharedModel::Push: contribute `data` to the sum under `key`; ordered after the work already
   enqueued on `stream` (the stream the tensor is produced on; NULL = the default stream) */
int msb_ps_push(msb_ps_t model, const float *data, int64_t rows, int64_t cols, int64_t ld, int key,
                void *stream);
/* ISharedModel::PullReq without callback: write the sum under `key` into `data` */
int msb_ps_pull_req(msb_ps_t model, float *data, int64_t rows, int64_t cols, int64_t ld, int key,
                    void *stream);
/* ISharedModel::PullWait: block the host until the last pull of `key` has completed */
int msb_ps_pull_wait(msb_ps_t model, int key);
/* ISharedModel::SetWeight_: every process's `data` becomes that of rank 0 (synchronous) */
int msb_ps_set_weight(msb_ps_t model, float *data, int64_t rows, int64_t cols, int64_t ld, int key,
                      void *stream);
/* ISharedModel::CheckWeight_: fails unless `data` equals rank 0's bit for bit (synchronous) */
int msb_ps_check_weight(msb_ps_t model, const float *data, int64_t rows, int64_t cols, int64_t ld,
                        int key, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MSHADOW_B200_PS_C_API_H_ */
