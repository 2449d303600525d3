/*
 * Launch-shape constants of the kernels, chosen by measurement on B200 (148 SMs, 64 K
 * registers and 227 KB shared memory per SM).  Each can be overridden on the compiler command
 * line for experiments; the defaults are what ships.
 */
#ifndef MSHADOW_GPU_TUNING_H_
#define MSHADOW_GPU_TUNING_H_

#ifndef MSHADOW_B200_EARLY_LAUNCH
#define MSHADOW_B200_EARLY_LAUNCH 1  // programmatic dependent launch for the kernels that support it
#endif
#ifndef MSHADOW_B200_MAP_THREADS
#define MSHADOW_B200_MAP_THREADS 256  // threads per CTA of the element-wise kernels
#endif
#ifndef MSHADOW_B200_MAP_UNROLL
#define MSHADOW_B200_MAP_UNROLL 1  // 16-byte groups per thread and sweep; 1 keeps the sweep linear in memory
                                   // (measured: 1 -> 94 %, 2 or 4 -> 87 %, 8 -> 60 % of copy bandwidth)
#endif
#ifndef MSHADOW_B200_MAP_SCALAR_UNROLL
#define MSHADOW_B200_MAP_SCALAR_UNROLL 1  // elements per thread and sweep of the element-at-a-time kernel
#endif
#ifndef MSHADOW_B200_MAP_HYBRID
#define MSHADOW_B200_MAP_HYBRID 1  // cheap expressions without EvalPack: 16-byte groups from element evaluations
                                   // (pad 53 -> 89 %, flip 49 -> 82 %, upsampling 41 -> 76 % of copy bandwidth;
                                   // reductions along an axis lose a factor of three, hence expr::LaneInfo)
#endif
#ifndef MSHADOW_B200_SEG_CHUNK
#define MSHADOW_B200_SEG_CHUNK 64  // sorted entries per CTA of the segmented sum (32: 81 %, 64: 87 %, 128: 81 %)
#endif
#ifndef MSHADOW_B200_SEG_DEPTH
#define MSHADOW_B200_SEG_DEPTH 4  // source rows in flight per thread
#endif
#ifndef MSHADOW_B200_LRN_TILE_PX
#define MSHADOW_B200_LRN_TILE_PX 3968  // pixels per CTA of the LRN kernels (a multiple of 128)
#endif
#ifndef MSHADOW_B200_SEG_STAGED
#define MSHADOW_B200_SEG_STAGED 1  // segmented sum: source rows through a shared-memory ring filled by bulk copies
#endif
#ifndef MSHADOW_B200_SEG_STAGED_MIN_CHUNKS
#define MSHADOW_B200_SEG_STAGED_MIN_CHUNKS 296  // first-level chunks (two per SM) from which the staged form is used
#endif
#ifndef MSHADOW_B200_SEG_CHUNK_UPPER
#define MSHADOW_B200_SEG_CHUNK_UPPER 16  // entries per CTA on the levels above the first, and on every level of a short list
#endif
#ifndef MSHADOW_B200_SEG_RING
#define MSHADOW_B200_SEG_RING 8  // rows (of up to 4 KB) in flight per CTA of the staged segmented sum
#endif
#ifndef MSHADOW_B200_SEG_MIN_CTAS
#define MSHADOW_B200_SEG_MIN_CTAS 4  // resident CTAs per SM the register allocation must allow
#endif
#ifndef MSHADOW_B200_CHPOOL_AHEAD
#define MSHADOW_B200_CHPOOL_AHEAD 4  // channels loaded ahead of the window
#endif
#ifndef MSHADOW_B200_CHPOOL_MIN_CTAS
#define MSHADOW_B200_CHPOOL_MIN_CTAS 1
#endif
#ifndef MSHADOW_B200_CHPOOL_STAGED
#define MSHADOW_B200_CHPOOL_STAGED 1  // route dense 16-byte-aligned inputs through the shared-memory ring kernel
#endif
#ifndef MSHADOW_B200_CHUNPOOL_STAGED
#define MSHADOW_B200_CHUNPOOL_STAGED 1  // ch_unpool of maximum / minimum: planes through a shared-memory ring (0.79 -> see pool.cuh)
#endif
#ifndef MSHADOW_B200_CHPOOL_RING_KB
#define MSHADOW_B200_CHPOOL_RING_KB 100  // shared memory of the ring per CTA (two CTAs per SM)
#endif
#ifndef MSHADOW_B200_POOL_SMEM_KB
#define MSHADOW_B200_POOL_SMEM_KB 28  // staged planes per CTA, forward pooling (14: 78 %, 28: 86 %, 56: 83 %)
#endif
#ifndef MSHADOW_B200_POOL_BAND_SMEM_KB
#define MSHADOW_B200_POOL_BAND_SMEM_KB 48  // staged row band per CTA, forward pooling of planes beyond shared memory
#endif
#ifndef MSHADOW_B200_POOL_PAIRS
#define MSHADOW_B200_POOL_PAIRS 1  // forward pooling 3 x 3 / 2: two adjacent outputs per thread from 16-byte loads
#endif
#ifndef MSHADOW_B200_UNPOOL_SMEM_KB
#define MSHADOW_B200_UNPOOL_SMEM_KB 74  // staged planes per CTA, backward pooling
#endif
#ifndef MSHADOW_B200_UNPACK_WIDE
#define MSHADOW_B200_UNPACK_WIDE 1  // unpack_patch2col: 16-byte stores where the runs are aligned
#endif
#ifndef MSHADOW_B200_SMGRAD_UNROLL
#define MSHADOW_B200_SMGRAD_UNROLL 1  // as for the map kernel: 1 -> 102 %, 2 -> 95-97 %, 4 -> 94 % of copy bandwidth
#endif

#ifndef MSHADOW_B200_SM3D_THREADS
#define MSHADOW_B200_SM3D_THREADS 128  // softmax over the middle axis: threads per CTA, 4 positions each
                                       // (64: 78.5 %, 128: 77.3 %, 256: 71.0 % of copy bandwidth, 21 classes)
#endif
#ifndef MSHADOW_B200_SM3D_DEPTH
#define MSHADOW_B200_SM3D_DEPTH 4  // classes loaded ahead per thread in the first pass (4: 77.3 %, 8: 71.0 %, 21: 78.5 %)
#endif

#ifndef MSHADOW_B200_REDLOW_THREADS
#define MSHADOW_B200_REDLOW_THREADS 128  // column reduce: threads per CTA (4 columns each)
#endif
#ifndef MSHADOW_B200_REDLOW_DEPTH
#define MSHADOW_B200_REDLOW_DEPTH 8  // column reduce: rows in flight per thread
#endif
#ifndef MSHADOW_B200_REDHIGH_THREADS
#define MSHADOW_B200_REDHIGH_THREADS 256  // channel reduce: threads per CTA
#endif
#ifndef MSHADOW_B200_REDHIGH_DEPTH
#define MSHADOW_B200_REDHIGH_DEPTH 4  // channel reduce: 16-byte groups in flight per thread
#endif

#ifndef MSHADOW_B200_REDLOW_CTAS_PER_SM
#define MSHADOW_B200_REDLOW_CTAS_PER_SM 7  // column reduce: CTAs (= DRAM streams) per SM aimed for on large inputs
#endif
#ifndef MSHADOW_B200_REDLOW_CHUNKS
#define MSHADOW_B200_REDLOW_CHUNKS 0  // column reduce: row chunks per column tile; 0 = chosen per shape
#endif
#ifndef MSHADOW_B200_REDHIGH_CHUNKS
#define MSHADOW_B200_REDHIGH_CHUNKS 0  // channel reduce: chunks of the outer axis per channel; 0 = fill whole waves
#endif

#ifndef MSHADOW_B200_TRANSPOSE_TILE
#define MSHADOW_B200_TRANSPOSE_TILE 64  // edge of the shared-memory tile of axis permutations (32: 62 %, 64: 90 %)
#endif

#endif  // MSHADOW_GPU_TUNING_H_
