/*
 * msb_peer_sink_t: where a reduction delivers its results on other GPUs (plain data, shared by
 * libmshadow_b200.so and libmshadow_b200_ps.so).  It has no counterpart in dmlc/mshadow, whose
 * reductions end on the GPU that ran them and whose exchange between GPUs goes through the host
 * (mshadow-ps/ps_local-inl.h:443-461, 625-662).  Obtain one per step and row segment from
 * msb_ps_peer_next_sink (mshadow_b200_ps.h) and pass it to msb_reduce_keep_lowest_f32_sink or
 * msb_reduce_keep_highdim_f32_sink (mshadow_b200.h): the thread that stores result i then also
 * stores the 64-bit word (tag << 32 | bits of the value) at row[p] + i for every rank p < world.
 * The layout is that of mshadow::gpu_rt::PeerSink.
 */
#ifndef MSHADOW_B200_PEER_SINK_C_API_H_
#define MSHADOW_B200_PEER_SINK_C_API_H_

#include <stdint.h>

#define MSB_PEER_MAX_WORLD 16

typedef struct msb_peer_sink {
  unsigned long long *row[MSB_PEER_MAX_WORLD]; /* mapped addresses in every rank's window */
  uint32_t tag;                                /* step + 1 */
  uint32_t count;                              /* results the segment expects */
  int world;                                   /* number of ranks; 0 disables the sink */
} msb_peer_sink_t;

#endif /* MSHADOW_B200_PEER_SINK_C_API_H_ */
