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

#include "mshadow_b200_peer_sink.h"

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

/* A second model behind the same interface, for small fp32 tensors whose exchange is bound by
   latency (a few thousand partial sums per step): mshadow::ps::PeerModel.  Push stores every
   element, tagged with its step, straight into a window of every GPU's memory over NVLink;
   PullReq reads the contributions of all ranks as they arrive (waiting at most wait_limit_ms,
   then msb_ps_pull_wait fails) and adds them in rank order, so that every rank receives the same
   bits.  It replaces the same LocalModel path (mshadow-ps/ps_local-inl.h:443-461, 625-662,
   700-736: device -> host copy, sum on a CPU thread, host -> device copy).
   window_bytes, depth, wait_limit_ms: 0 selects the defaults (64 MiB, 4 slots, 2000 ms); a key of
   n floats takes depth * world * n * 8 bytes of the window.  With depth d a rank may push at most
   d/2 - 1 steps of a key ahead of pulling them.  own_stream 0: push and pull kernels run on the
   stream given with the call; 1: on a stream of the model, ordered behind the given stream by an
   event at every call, so that the exchange runs beside the caller's next kernels (the caller
   then leaves a pushed tensor alone until its step has been pulled, and uses msb_ps_pull_wait or
   msb_ps_pull_fence before touching a result).
   Set-up: every rank creates its model, obtains its handle (128 hexadecimal digits and a
   terminating zero; capacity at least 129), the application gathers the handles of all ranks in
   rank order into one string and gives it to msb_ps_peer_connect on every rank.  world 1 needs no
   connect.  The tensor calls below (init_key, push, pull_req, pull_wait, set_weight, check_weight,
   destroy) serve both models; the application lets all ranks reach a barrier of its own before
   it destroys a peer model.
   msb_ps_peer_next_sink takes the place of msb_ps_push when a reduction kernel delivers the
   step's data itself: it returns the sink for `count` results starting at element `offset` of
   the key's row.  The segment at offset 0 opens the step; the segments of a step must cover the
   whole row before msb_ps_pull_req is called for it. */
int msb_ps_peer_create(int rank, int world, int device, int64_t window_bytes, int depth, int wait_limit_ms,
                       int own_stream, msb_ps_t *out);
int msb_ps_peer_handle(msb_ps_t model, char *hex, int64_t capacity);
int msb_ps_peer_connect(msb_ps_t model, const char *all_handles_hex);
int msb_ps_peer_next_sink(msb_ps_t model, int key, int64_t offset, int64_t count, msb_peer_sink_t *out);
/* Regions of the windows for the caller's own kernels (bulk data that a kernel stores straight
   into another GPU's memory, e.g. msb_addtakegrad_largebatch_store_f32_i32 with a destination in
   the owner's window).  msb_ps_peer_reserve sets `bytes` of every rank's window aside and returns
   their offset; all ranks make the same calls in the same order.  msb_ps_peer_window gives the
   address, in this process, of byte `offset` of rank `rank`'s window (after connect); only plain
   loads and stores of the caller's own kernels may use an address of another rank.  A key pushed
   after the writing kernels, on the same stream, is the completion signal: whoever has pulled
   that step finds the data in place.  The window (msb_ps_peer_create's window_bytes) must be
   sized for keys and regions together. */
int msb_ps_peer_reserve(msb_ps_t model, int64_t bytes, int64_t *offset);
int msb_ps_peer_window(msb_ps_t model, int rank, int64_t offset, void **ptr);

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
/* No counterpart in the reference: the device-side form of PullWait.  Work enqueued on `stream`
   after this call runs after the last pull of `key`; the host does not block. */
int msb_ps_pull_fence(msb_ps_t model, int key, void *stream);
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
