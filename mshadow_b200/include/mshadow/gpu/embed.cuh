/*
 * Embedding backward: AddTakeGradLargeBatch (dst[sorted[y]] += src[index[y]]), AddTakeGrad
 * (dst[clip(index[y])] += src[y]) and SortByKey.
 *
 * The reference's large-batch kernel (mshadow/cuda/tensor_gpu-inl.cuh:619-672) lets the
 * warp that sits on the first entry of a run of equal indices walk the whole run while all
 * other warps exit, so a frequent index (a Zipf head holds an eighth of a million-entry
 * batch) is accumulated serially by one warp per 128 features; its small-batch kernel
 * (:599-617) is serial over the entire batch.
 *
 * Here the sorted list is cut into fixed chunks of kSegChunk entries, one CTA per chunk and
 * per 1024-feature slab.  A thread owns four adjacent features and streams the source rows
 * of its chunk with 128-bit loads, eight rows in flight, accumulating in registers while
 * the key stays the same.  A run that lies wholly inside one chunk is added to its table
 * row directly.  A run that crosses a chunk boundary leaves one partial row per chunk in a
 * scratch matrix; those partial rows, keyed by table row and still in sorted order, are the
 * input of the same kernel one level up.  The first level of a long list uses chunks of
 * kSegChunk entries and is bound by bandwidth; the levels above it are a few CTAs each and bound
 * by latency, so they use short chunks (kSegChunkUpper entries, shrinking a level by half that
 * factor), all their rows in flight at once, and add to the table rows in batches.  A million
 * entries take six launches, the last five a few microseconds each.  No atomics are used and
 * every addition order is fixed by the chunk geometry, so results are reproducible.
 *
 * Traffic: each source row is read once (4*N*D bytes), each touched table row is read and
 * written once, partial rows add a few percent.  The kernel is bound by HBM bandwidth.
 */
#ifndef MSHADOW_GPU_EMBED_CUH_
#define MSHADOW_GPU_EMBED_CUH_

#include <cub/device/device_radix_sort.cuh>

#include "./radix_sort.cuh"
#include "./route.cuh"
#include "./runtime.h"
#include "./tma.cuh"

namespace mshadow {
namespace cuda {

const uint32_t kSegChunk = MSHADOW_B200_SEG_CHUNK;
const int kSegDepth = MSHADOW_B200_SEG_DEPTH;
const uint32_t kSegRing = MSHADOW_B200_SEG_RING;       // source rows in flight per CTA of the staged kernel
const uint32_t kSegSlab = 1024;                        // features per CTA: 256 threads x 4
const int kSegDepthUpper = 8;                          // rows in flight per thread above the first level
const uint32_t kSegChunkUpper = MSHADOW_B200_SEG_CHUNK_UPPER;  // entries per CTA above the first level
const uint32_t kSegStagedMinChunks = MSHADOW_B200_SEG_STAGED_MIN_CHUNKS;

/*!
 * \brief one level of the chunked segmented sum.
 *  keys[n] ascending; rows[n] (or identity when null) names the source row of each entry, a
 *  negative row contributes nothing.  part_keys / part_rows / partials receive two slots per
 *  chunk for the next level.  grid = (chunks, feature slabs).  kDepth source rows are in flight
 *  per thread: kSegDepth on the first level, which is bound by bandwidth and wants many CTAs per
 *  SM, kSegDepthUpper on the levels above it, which are a few CTAs each walking a list of partial
 *  rows and are bound by the latency of those loads.
 */
template <int kLanes, int kDepth>
__global__ void __launch_bounds__(256, kDepth > 4 ? 2 : MSHADOW_B200_SEG_MIN_CTAS)
SegmentSumKernel(float *dst, int64_t ld_dst, const int32_t *keys, const int32_t *rows, const float *src,
                 int64_t ld_src, uint32_t n, uint32_t width, uint32_t chunk_len, int32_t *part_keys,
                 int32_t *part_rows, float *partials, int store, const routedetail::RowRoute route) {
  gpu_rt::GridDependencySync();
  // store != 0: a finished run's sum is stored into its table row instead of added to it (the
  // row is not read; it may then live in another GPU's memory).
  // With kDepth > 4 (the upper levels) the additions to table rows are batched: a run that ends
  // inside a batch of kDepth entries is parked, and once the batch has been walked the table rows
  // of all parked runs are loaded together, added to and stored.  Done one by one -- load, add,
  // store at the moment the run ends -- a CTA walking 64 entries of 64 different rows spent 44 us
  // on the 64 dependent round trips.
  constexpr bool kBatched = kDepth > 4;
  const uint32_t chunk = blockIdx.x;
  const uint32_t begin = chunk * chunk_len;
  const uint32_t end = min(n, begin + chunk_len);
  const uint32_t col = (blockIdx.y * blockDim.x + threadIdx.x) * kLanes;
  const bool active = col < width;
  const bool lead = blockIdx.y == 0 && threadIdx.x == 0;
  const bool joins_prev = chunk > 0 && keys[begin - 1] == keys[begin];
  const bool joins_next = end < n && keys[end] == keys[end - 1];
  if (lead && part_rows != nullptr) {
    part_keys[2 * chunk] = keys[begin];
    part_keys[2 * chunk + 1] = keys[end - 1];
    part_rows[2 * chunk] = -1;
    part_rows[2 * chunk + 1] = -1;
  }
  int32_t cur = keys[begin];
  bool first_run = true, any = false;
  float acc[kLanes];
#pragma unroll
  for (int l = 0; l < kLanes; ++l) acc[l] = 0.0f;

  routedetail::OwnerHint hint = {0, 0, 0};
  auto add_to_row = [&](float *row, const float (&a)[kLanes]) {
    if (store) {
      if (kLanes == 4) {
        *reinterpret_cast<float4 *>(row) = make_float4(a[0], a[1 % kLanes], a[2 % kLanes], a[3 % kLanes]);
      } else {
        row[0] = a[0];
      }
    } else if (kLanes == 4) {
      float4 d = *reinterpret_cast<float4 *>(row);
      d.x = __fadd_rn(d.x, a[0]);
      d.y = __fadd_rn(d.y, a[1 % kLanes]);
      d.z = __fadd_rn(d.z, a[2 % kLanes]);
      d.w = __fadd_rn(d.w, a[3 % kLanes]);
      *reinterpret_cast<float4 *>(row) = d;
    } else {
      row[0] = __fadd_rn(row[0], a[0]);
    }
  };
  // a finished run: parked in the scratch matrix if it continues in a neighbouring chunk, else
  // added to its table row -- at once, or (park != nullptr) handed back to be added with its batch
  auto flush = [&](bool last_run, float **park, float (*park_acc)[kLanes]) {
    const bool spans = (first_run && joins_prev) || (last_run && joins_next);
    if (!spans) {
      if (any && active) {
        float *row = routedetail::RowOf(route, dst, ld_dst, cur, &hint) + col;
        if (park != nullptr) {
          *park = row;
#pragma unroll
          for (int l = 0; l < kLanes; ++l) (*park_acc)[l] = acc[l];
        } else {
          add_to_row(row, acc);
        }
      }
    } else if (any) {
      const uint32_t slot = 2 * chunk + (first_run ? 0 : 1);
      if (active) {
        float *row = partials + static_cast<int64_t>(slot) * width + col;
        if (kLanes == 4) {
          *reinterpret_cast<float4 *>(row) = make_float4(acc[0], acc[1 % kLanes], acc[2 % kLanes], acc[3 % kLanes]);
        } else {
          row[0] = acc[0];
        }
      }
      if (lead) part_rows[slot] = static_cast<int32_t>(slot);
    }
  };

  for (uint32_t i = begin; i < end; i += kDepth) {
    int32_t k[kDepth], r[kDepth];
    float v[kDepth][kLanes];
#pragma unroll
    for (int u = 0; u < kDepth; ++u) {
      const uint32_t e = i + u;
      const bool in = e < end;
      k[u] = in ? keys[e] : 0;
      r[u] = in ? (rows != nullptr ? rows[e] : static_cast<int32_t>(e)) : -1;
    }
#pragma unroll
    for (int u = 0; u < kDepth; ++u) {
      if (r[u] >= 0 && active) {
        const float *p = src + static_cast<int64_t>(r[u]) * ld_src + col;
        if (kLanes == 4) {
          const float4 q = __ldcs(reinterpret_cast<const float4 *>(p));
          v[u][0] = q.x;
          v[u][1 % kLanes] = q.y;
          v[u][2 % kLanes] = q.z;
          v[u][3 % kLanes] = q.w;
        } else {
          v[u][0] = __ldcs(p);
        }
      } else {
#pragma unroll
        for (int l = 0; l < kLanes; ++l) v[u][l] = 0.0f;
      }
    }
    float *parked[kBatched ? kDepth : 1];
    float parked_acc[kBatched ? kDepth : 1][kLanes];
#pragma unroll
    for (int u = 0; u < (kBatched ? kDepth : 1); ++u) parked[u] = nullptr;
#pragma unroll
    for (int u = 0; u < kDepth; ++u) {
      if (i + u < end) {
        if (k[u] != cur) {
          if (kBatched) flush(false, &parked[kBatched ? u : 0], &parked_acc[kBatched ? u : 0]); else flush(false, nullptr, nullptr);
          cur = k[u];
          first_run = false;
          any = false;
#pragma unroll
          for (int l = 0; l < kLanes; ++l) acc[l] = 0.0f;
        }
        if (r[u] >= 0) {
          any = true;
#pragma unroll
          for (int l = 0; l < kLanes; ++l) acc[l] = __fadd_rn(acc[l], v[u][l]);
        }
      }
    }
    if (kBatched) {
      // table rows of the runs that ended in this batch: all loads first, then the additions
      float d[kDepth][kLanes];
#pragma unroll
      for (int u = 0; u < kDepth; ++u) {
#pragma unroll
        for (int l = 0; l < kLanes; ++l) d[u][l] = 0.0f;
        if (parked[u] != nullptr && !store) {
          if (kLanes == 4) {
            const float4 q = *reinterpret_cast<const float4 *>(parked[u]);
            d[u][0] = q.x;
            d[u][1 % kLanes] = q.y;
            d[u][2 % kLanes] = q.z;
            d[u][3 % kLanes] = q.w;
          } else {
            d[u][0] = parked[u][0];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kDepth; ++u) {
        if (parked[u] != nullptr) {
          if (kLanes == 4) {
            *reinterpret_cast<float4 *>(parked[u]) =
                store ? make_float4(parked_acc[u][0], parked_acc[u][1 % kLanes], parked_acc[u][2 % kLanes],
                                    parked_acc[u][3 % kLanes])
                      : make_float4(__fadd_rn(d[u][0], parked_acc[u][0]),
                                    __fadd_rn(d[u][1 % kLanes], parked_acc[u][1 % kLanes]),
                                    __fadd_rn(d[u][2 % kLanes], parked_acc[u][2 % kLanes]),
                                    __fadd_rn(d[u][3 % kLanes], parked_acc[u][3 % kLanes]));
          } else {
            parked[u][0] = store ? parked_acc[u][0] : __fadd_rn(d[u][0], parked_acc[u][0]);
          }
        }
      }
    }
  }
  flush(true, nullptr, nullptr);
}

/*!
 * \brief the same level of the segmented sum with the source rows staged through shared memory.
 *  SegmentSumKernel keeps kSegDepth 16-byte loads in flight per thread and then waits for them:
 *  measured, its warps spend most of their time on those loads.  Here a producer warp issues
 *  one bulk asynchronous copy per source row (a row's slab of up to 1024 features is contiguous
 *  and 16-byte aligned) into a ring of kSegRing shared-memory slots, up to kSegRing rows ahead;
 *  the eight consumer warps take the rows from shared memory in list order.  Each slot has a
 *  `full` barrier (the copy has landed) and an `empty` barrier (every consumer warp has read
 *  it), so no step synchronises the whole CTA.  Keys and row numbers of the chunk are brought
 *  into shared memory once.  Arithmetic, run handling and results are SegmentSumKernel<4>'s.
 *  Block: 256 consumer threads + one producer warp.  Dynamic shared memory: kSegRing * 4 KB.
 *  (A template only so that the header can be included from several translation units.)
 */
template <int kRingSlots>
__global__ void __launch_bounds__(288, MSHADOW_B200_SEG_MIN_CTAS)
SegmentSumStagedKernel(float *dst, int64_t ld_dst, const int32_t *keys, const int32_t *rows, const float *src,
                       int64_t ld_src, uint32_t n, uint32_t width, int32_t *part_keys, int32_t *part_rows,
                       float *partials, int *status, int store, const routedetail::RowRoute route) {
  gpu_rt::GridDependencySync();
  extern __shared__ __align__(16) float ring[];
  __shared__ uint64_t full[kSegRing], empty[kSegRing];
  __shared__ int32_t s_keys[kSegChunk], s_rows[kSegChunk];
  const uint32_t chunk = blockIdx.x;
  const uint32_t begin = chunk * kSegChunk;
  const uint32_t end = min(n, begin + kSegChunk);
  const uint32_t cnt = end - begin;
  const uint32_t col0 = blockIdx.y * kSegSlab;
  const uint32_t slab_w = min(kSegSlab, width - col0);  // a multiple of 4
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kSegChunk) {
    const uint32_t e = begin + threadIdx.x;
    s_keys[threadIdx.x] = e < end ? keys[e] : 0;
    s_rows[threadIdx.x] = e < end ? (rows != nullptr ? rows[e] : static_cast<int32_t>(e)) : -1;
  }
  if (threadIdx.x == 0) {
    for (uint32_t j = 0; j < kSegRing; ++j) {
      tma::BarrierInit(&full[j], 1);
      tma::BarrierInit(&empty[j], 8);
    }
  }
  __syncthreads();
  if (warp == 8) {
    // producer: one thread issues the copies in list order; a slot is refilled once the consumers
    // have released the row it held (slots are released in the order they were filled)
    if (lane != 0) return;
    for (uint32_t e = 0; e < cnt; ++e) {
      const uint32_t slot = e % kSegRing, use = e / kSegRing;
      if (use > 0 && !tma::WaitBounded(&empty[slot], (use - 1) & 1u)) {
        atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      const int32_t r = s_rows[e];
      if (r >= 0) {
        tma::BarrierExpect(&full[slot], slab_w * 4u);
        tma::BulkLoad(ring + static_cast<size_t>(slot) * kSegSlab, src + static_cast<int64_t>(r) * ld_src + col0,
                      slab_w * 4u, &full[slot]);
      } else {
        // an entry without a source row still takes its turn on the slot: the consumers wait for
        // `full` on every entry, so they can never release a slot twice before this thread has
        // seen the first release
        tma::BarrierArrive(&full[slot]);
      }
    }
    return;
  }
  const uint32_t col = col0 + threadIdx.x * 4;
  const bool active = threadIdx.x * 4 < slab_w;
  const bool lead = blockIdx.y == 0 && threadIdx.x == 0;
  const bool joins_prev = chunk > 0 && keys[begin - 1] == s_keys[0];
  const bool joins_next = end < n && keys[end] == s_keys[cnt - 1];
  if (lead && part_rows != nullptr) {
    part_keys[2 * chunk] = s_keys[0];
    part_keys[2 * chunk + 1] = s_keys[cnt - 1];
    part_rows[2 * chunk] = -1;
    part_rows[2 * chunk + 1] = -1;
  }
  int32_t cur = s_keys[0];
  bool first_run = true, any = false;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // (Loading the table row when a run ends and adding to it when the next one ends would hide the
  // round trip, but the 16 registers it takes leave four CTAs per SM instead of five: measured
  // 0.87 against 0.93 of the copy bandwidth.)
  auto flush = [&](bool last_run) {
    const bool spans = (first_run && joins_prev) || (last_run && joins_next);
    if (!spans) {
      if (any && active) {
        // (no cached owner block here: its three registers would cost this kernel its fifth CTA per SM)
        routedetail::OwnerHint look = {0, 0, 0};
        float *row = routedetail::RowOf(route, dst, ld_dst, cur, &look) + col;
        if (store) {
          *reinterpret_cast<float4 *>(row) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        } else {
          float4 d = *reinterpret_cast<float4 *>(row);
          d.x = __fadd_rn(d.x, acc[0]);
          d.y = __fadd_rn(d.y, acc[1]);
          d.z = __fadd_rn(d.z, acc[2]);
          d.w = __fadd_rn(d.w, acc[3]);
          *reinterpret_cast<float4 *>(row) = d;
        }
      }
    } else if (any) {
      const uint32_t slot = 2 * chunk + (first_run ? 0 : 1);
      if (active) {
        *reinterpret_cast<float4 *>(partials + static_cast<int64_t>(slot) * width + col) =
            make_float4(acc[0], acc[1], acc[2], acc[3]);
      }
      if (lead) part_rows[slot] = static_cast<int32_t>(slot);
    }
  };
  for (uint32_t e = 0; e < cnt; ++e) {
    const uint32_t slot = e % kSegRing;
    const int32_t k = s_keys[e], r = s_rows[e];
    if (k != cur) {
      flush(false);
      cur = k;
      first_run = false;
      any = false;
      acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    }
    if (!tma::WaitBounded(&full[slot], (e / kSegRing) & 1u)) {
      if (lane == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
      return;
    }
    if (r >= 0) {
      if (active) {
        const float4 v = *reinterpret_cast<const float4 *>(ring + static_cast<size_t>(slot) * kSegSlab + threadIdx.x * 4);
        acc[0] = __fadd_rn(acc[0], v.x);
        acc[1] = __fadd_rn(acc[1], v.y);
        acc[2] = __fadd_rn(acc[2], v.z);
        acc[3] = __fadd_rn(acc[3], v.w);
      }
      any = true;
    }
    __syncwarp();
    if (lane == 0) tma::BarrierArrive(&empty[slot]);
  }
  flush(true);
}

/*! \brief keys[i] = clip(index[i], 0, k-1), vals[i] = i */
template <typename IndexType>
__global__ void ClipIotaKernel(IndexType *keys, IndexType *vals, const IndexType *index, uint32_t n, IndexType k) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  IndexType j = index[i];
  j = j <= 0 ? 0 : (j >= k ? k - 1 : j);
  keys[i] = j;
  vals[i] = static_cast<int32_t>(i);
}

namespace embeddetail {
inline size_t Align256(size_t b) { return (b + 255) / 256 * 256; }

const int kMaxLevels = 16;

/*!
 * \brief entries, chunk length and chunk count of every level until one chunk remains.
 *  The first level of a long list uses chunks of kSegChunk entries (bandwidth: few, long CTAs);
 *  the levels above it, and every level of a short list, use chunks of kSegChunkUpper entries:
 *  they are bound by latency, and shorter chunks spread their rows over more CTAs.
 */
inline int Levels(uint32_t n, uint32_t (&entries)[kMaxLevels], uint32_t (&chunks)[kMaxLevels],
                  uint32_t (&len)[kMaxLevels]) {
  int levels = 0;
  uint32_t cur = n;
  const bool long_list = (n + kSegChunk - 1) / kSegChunk >= kSegStagedMinChunks;
  while (levels < kMaxLevels) {
    entries[levels] = cur;
    len[levels] = (levels == 0 && long_list) ? kSegChunk : kSegChunkUpper;
    chunks[levels] = (cur + len[levels] - 1) / len[levels];
    ++levels;
    if (chunks[levels - 1] <= 1) break;
    cur = 2 * chunks[levels - 1];
  }
  return levels;
}

/*! \brief bytes of scratch the levels below need (partial rows + their keys and row ids) */
inline size_t SegmentScratchBytes(uint32_t n, uint32_t width) {
  uint32_t entries[kMaxLevels], chunks[kMaxLevels], len[kMaxLevels];
  const int levels = Levels(n, entries, chunks, len);
  size_t bytes = 0;
  for (int l = 0; l + 1 < levels; ++l) {
    bytes += Align256(2ull * chunks[l] * width * sizeof(float));
    bytes += 2 * Align256(2ull * chunks[l] * sizeof(int32_t));
  }
  return bytes;
}

/*! \brief run all levels; `scratch` must hold SegmentScratchBytes(n, width) */
inline void SegmentSumRun(float *dst, int64_t ld_dst, const int32_t *keys, const int32_t *rows, const float *src,
                          int64_t ld_src, uint32_t n, uint32_t width, char *scratch, cudaStream_t stream,
                          bool store = false, const routedetail::RowRoute *route = nullptr) {
  const int st = store ? 1 : 0;
  routedetail::RowRoute rt;
  if (route != nullptr) {
    rt = *route;
  } else {
    for (int q = 0; q < routedetail::kMaxOwners; ++q) rt.base[q] = nullptr;
    rt.first = nullptr;
    rt.world = 0;
  }
  if (n == 0 || width == 0) return;
  uint32_t entries[kMaxLevels], chunks[kMaxLevels], len[kMaxLevels];
  const int levels = Levels(n, entries, chunks, len);
  const int32_t *lkeys = keys, *lrows = rows;
  const float *lsrc = src;
  int64_t lld = ld_src;
  for (int l = 0; l < levels; ++l) {
    int32_t *pk = nullptr, *pr = nullptr;
    float *pp = nullptr;
    if (l + 1 < levels) {
      pp = reinterpret_cast<float *>(scratch);
      scratch += Align256(2ull * chunks[l] * width * sizeof(float));
      pk = reinterpret_cast<int32_t *>(scratch);
      scratch += Align256(2ull * chunks[l] * sizeof(int32_t));
      pr = reinterpret_cast<int32_t *>(scratch);
      scratch += Align256(2ull * chunks[l] * sizeof(int32_t));
    }
    const bool vec = width % 4 == 0 && lld % 4 == 0 && ld_dst % 4 == 0 &&
                     reinterpret_cast<uintptr_t>(lsrc) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
    // (a routed call passes dst == nullptr; its owners' blocks are checked for alignment by the caller)
    const uint32_t items = vec ? width / 4 : width;
    uint32_t threads = (items + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    const dim3 grid(chunks[l], (items + threads - 1) / threads);
    const bool long_chunks = len[l] == kSegChunk && kSegChunk != kSegChunkUpper;
    if (vec && MSHADOW_B200_SEG_STAGED && width >= 256 && long_chunks) {
      // rows of a kilobyte and more, enough chunks to fill the GPU: staged through shared memory by
      // bulk copies.  (Measured on a list of 2039 chunks: the staged kernel took 32, 28 and 4.5 us
      // for the three upper levels of 64, 2 and 1 chunks -- its in-order ring serves a lone CTA one
      // row per 0.44 us -- which is why those levels use the register form.)
      auto kernel = SegmentSumStagedKernel<static_cast<int>(kSegRing)>;
      const size_t smem = static_cast<size_t>(kSegRing) * kSegSlab * sizeof(float);
      MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      gpu_rt::LaunchAfterDrain(kernel, dim3(chunks[l], (width + kSegSlab - 1) / kSegSlab), dim3(288), smem, stream, 
          dst, ld_dst, lkeys, lrows, lsrc, lld, entries[l], width, pk, pr, pp, gpu_rt::StatusWord(), st, rt);
    } else if (vec && long_chunks) {
      gpu_rt::LaunchAfterDrain(SegmentSumKernel<4, kSegDepth>, dim3(grid), dim3(threads), 0, stream, dst, ld_dst, lkeys, lrows, lsrc, lld, entries[l],
                                                                   width, len[l], pk, pr, pp, st, rt);
    } else if (vec) {
      gpu_rt::LaunchAfterDrain(SegmentSumKernel<4, kSegDepthUpper>, dim3(grid), dim3(threads), 0, stream, dst, ld_dst, lkeys, lrows, lsrc, lld,
                                                                        entries[l], width, len[l], pk, pr, pp, st, rt);
    } else if (long_chunks) {
      gpu_rt::LaunchAfterDrain(SegmentSumKernel<1, kSegDepth>, dim3(grid), dim3(threads), 0, stream, dst, ld_dst, lkeys, lrows, lsrc, lld, entries[l],
                                                                   width, len[l], pk, pr, pp, st, rt);
    } else {
      gpu_rt::LaunchAfterDrain(SegmentSumKernel<1, kSegDepthUpper>, dim3(grid), dim3(threads), 0, stream, dst, ld_dst, lkeys, lrows, lsrc, lld,
                                                                        entries[l], width, len[l], pk, pr, pp, st, rt);
    }
    MSHADOW_CUDA_POST_KERNEL_CHECK(SegmentSumKernel);
    lkeys = pk;
    lrows = pr;
    lsrc = pp;
    lld = width;
  }
}
}  // namespace embeddetail

/*!
 * \brief dst[sorted[y]] += src[index[y]]; `sorted` ascending.  With store, the rows named by `sorted`
 *  receive the sum itself (dst[r] = sum; rows not named stay as they are): every named row is
 *  written exactly once and never read, so dst may be memory of another GPU.
 */
inline void AddTakeGradLargeBatchLaunch(float *dst, int64_t ld_dst, const int32_t *sorted, const int32_t *index,
                                        const float *src, int64_t ld_src, int64_t n, int64_t width,
                                        cudaStream_t stream, bool store = false,
                                        const routedetail::RowRoute *route = nullptr) {
  if (n == 0 || width == 0) return;
  CHECK_LT(n, (int64_t(1) << 31));
  const size_t bytes = embeddetail::SegmentScratchBytes(static_cast<uint32_t>(n), static_cast<uint32_t>(width));
  char *scratch = bytes == 0 ? nullptr : static_cast<char *>(gpu_rt::Scratch::Get(stream, bytes));
  embeddetail::SegmentSumRun(dst, ld_dst, sorted, index, src, ld_src, static_cast<uint32_t>(n),
                             static_cast<uint32_t>(width), scratch, stream, store, route);
}

namespace embeddetail {
/*! \brief 4-byte arithmetic keys with 4-byte values: this engine's own radix sort (radix_sort.cuh) */
template <typename KDType, typename VDType>
inline void SortPairs4(KDType *keys, VDType *values, int64_t n, bool ascend, cudaStream_t stream, std::true_type) {
  char *scratch = static_cast<char *>(gpu_rt::Scratch::Get(stream, sortdetail::ScratchBytes(n)));
  const sortdetail::Source as_given = {0};
  sortdetail::SortPairs<KDType, VDType>(keys, values, keys, n, 32, ascend, as_given, scratch, stream);
}
template <typename KDType, typename VDType>
inline void SortPairs4(KDType *, VDType *, int64_t, bool, cudaStream_t, std::false_type) {}
}  // namespace embeddetail

/*! \brief stable key/value sort, in place from the caller's point of view */
template <typename KDType, typename VDType>
inline void SortPairsLaunch(KDType *keys, VDType *values, int64_t n, bool ascend, cudaStream_t stream) {
  if (n <= 1) return;
  CHECK_LT(n, (int64_t(1) << 31));
  constexpr bool kOwn = sizeof(KDType) == 4 && sizeof(VDType) == 4 && std::is_arithmetic<KDType>::value;
  if (kOwn) {
    embeddetail::SortPairs4(keys, values, n, ascend, stream, std::integral_constant<bool, kOwn>());
    return;
  }
  // other element sizes: the CUDA toolkit's device-wide radix sort
  size_t temp = 0;
  if (ascend) {
    MSHADOW_CUDA_CALL((cub::DeviceRadixSort::SortPairs<KDType, VDType>(nullptr, temp, keys, keys, values, values,
                                                                       static_cast<int>(n), 0, sizeof(KDType) * 8,
                                                                       stream)));
  } else {
    MSHADOW_CUDA_CALL((cub::DeviceRadixSort::SortPairsDescending<KDType, VDType>(
        nullptr, temp, keys, keys, values, values, static_cast<int>(n), 0, sizeof(KDType) * 8, stream)));
  }
  const size_t kb = embeddetail::Align256(n * sizeof(KDType)), vb = embeddetail::Align256(n * sizeof(VDType));
  char *base = static_cast<char *>(gpu_rt::Scratch::Get(stream, kb + vb + temp));
  KDType *k2 = reinterpret_cast<KDType *>(base);
  VDType *v2 = reinterpret_cast<VDType *>(base + kb);
  void *work = base + kb + vb;
  if (ascend) {
    MSHADOW_CUDA_CALL((cub::DeviceRadixSort::SortPairs<KDType, VDType>(work, temp, keys, k2, values, v2,
                                                                       static_cast<int>(n), 0, sizeof(KDType) * 8,
                                                                       stream)));
  } else {
    MSHADOW_CUDA_CALL((cub::DeviceRadixSort::SortPairsDescending<KDType, VDType>(
        work, temp, keys, k2, values, v2, static_cast<int>(n), 0, sizeof(KDType) * 8, stream)));
  }
  MSHADOW_CUDA_CALL(cudaMemcpyAsync(keys, k2, n * sizeof(KDType), cudaMemcpyDeviceToDevice, stream));
  MSHADOW_CUDA_CALL(cudaMemcpyAsync(values, v2, n * sizeof(VDType), cudaMemcpyDeviceToDevice, stream));
}

/*! \brief dst[clip(index[y], 0, k-1)] += src[y], contributions to a row added in batch order */
inline void AddTakeGradLaunch(float *dst, int64_t ld_dst, const int32_t *index, const float *src, int64_t ld_src,
                              int64_t k, int64_t n, int64_t width, cudaStream_t stream) {
  if (n == 0 || width == 0) return;
  CHECK_LT(n, (int64_t(1) << 31));
  using embeddetail::Align256;
  const uint32_t un = static_cast<uint32_t>(n);
  // clip + stable sort of (index, position) + segmented sum.  Only the bits a row number can have
  // are sorted (two passes for up to 2^18 rows); the first pass clips the raw indices and
  // generates the positions itself.
  int bits = 1;
  while (bits < 31 && (int64_t(1) << bits) < k) ++bits;
  const size_t ib = Align256(n * sizeof(int32_t));
  const size_t sort_bytes = sortdetail::ScratchBytes(n);
  const size_t seg = embeddetail::SegmentScratchBytes(un, static_cast<uint32_t>(width));
  char *base = static_cast<char *>(gpu_rt::Scratch::Get(stream, 2 * ib + Align256(sort_bytes) + seg));
  int32_t *k_sorted = reinterpret_cast<int32_t *>(base), *v_sorted = reinterpret_cast<int32_t *>(base + ib);
  char *sort_scratch = base + 2 * ib;
  char *seg_scratch = base + 2 * ib + Align256(sort_bytes);
  const sortdetail::Source clipped = {static_cast<int>(k)};
  sortdetail::SortPairs<int32_t, int32_t>(k_sorted, v_sorted, index, n, bits, true, clipped, sort_scratch, stream);
  embeddetail::SegmentSumRun(dst, ld_dst, k_sorted, v_sorted, src, ld_src, un, static_cast<uint32_t>(width), seg_scratch,
                             stream);
}

// ----------------------------------------------------------------------------------------
// IndexFill: dst[index[y]] = src[y].  The reference's kernel (mshadow/cuda/tensor_gpu-inl.cuh:
// 736-782) lets all batch entries write at once, so a row named twice ends up with either
// source.  Here the CPU's outcome (mshadow/tensor_cpu-inl.h:520-529: entries in batch order,
// the later one stays) is reproduced: a first pass records, per table row, the last batch entry
// that names it; the second pass copies only those entries.
// ----------------------------------------------------------------------------------------

/*! \brief last[index[y]] = max(last[index[y]], y); `last` starts at -1; rows outside the table are skipped */
template <typename IndexType>
__global__ void __launch_bounds__(256)
IndexFillOwnerKernel(int32_t *last, const IndexType *index, uint32_t n, int32_t k) {
  const uint32_t y = blockIdx.x * 256 + threadIdx.x;
  if (y >= n) return;
  const int32_t j = static_cast<int32_t>(index[y]);
  if (j >= 0 && j < k) atomicMax(last + j, static_cast<int32_t>(y));
}

/*! \brief a CTA takes four batch entries per grid-stride sweep; an entry copies its source row if it is the last one
 *  naming that table row */
template <int kLanes>
__global__ void __launch_bounds__(256)
IndexFillCopyKernel(float *dst, int64_t ld_dst, const int32_t *last, const int32_t *index, const float *src,
                    int64_t ld_src, uint32_t n, uint32_t items, int32_t k) {
  constexpr int kRows = 4;  // batch entries per sweep: their index look-ups and row loads overlap
  for (uint32_t y0 = blockIdx.x * kRows; y0 < n; y0 += gridDim.x * kRows) {
    int32_t j[kRows];
    bool live[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) j[r] = y0 + r < n ? index[y0 + r] : -1;
#pragma unroll
    for (int r = 0; r < kRows; ++r) live[r] = j[r] >= 0 && j[r] < k && last[j[r]] == static_cast<int32_t>(y0 + r);
    for (uint32_t i = threadIdx.x; i < items; i += 256) {
      float v[kRows][kLanes];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (!live[r]) continue;
        const float *in = src + (y0 + r) * ld_src;
        if (kLanes == 4) {
          const float4 p = __ldcs(reinterpret_cast<const float4 *>(in) + i);
          v[r][0] = p.x, v[r][1 % kLanes] = p.y, v[r][2 % kLanes] = p.z, v[r][3 % kLanes] = p.w;
        } else {
          v[r][0] = __ldcs(in + i);
        }
      }
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (!live[r]) continue;
        float *out = dst + j[r] * ld_dst;
        if (kLanes == 4) {
          __stcs(reinterpret_cast<float4 *>(out) + i,
                 make_float4(v[r][0], v[r][1 % kLanes], v[r][2 % kLanes], v[r][3 % kLanes]));
        } else {
          __stcs(out + i, v[r][0]);
        }
      }
    }
  }
}

/*! \brief dst[index[y]] = src[y] with the outcome of a serial walk over y; indices outside [0, k) are ignored */
inline void IndexFillLaunch(float *dst, int64_t ld_dst, const int32_t *index, const float *src, int64_t ld_src,
                            int64_t k, int64_t n, int64_t width, cudaStream_t stream) {
  if (n == 0 || width == 0 || k == 0) return;
  CHECK_LT(n, (int64_t(1) << 31));
  CHECK_LT(k, (int64_t(1) << 31));
  int32_t *last = static_cast<int32_t *>(gpu_rt::Scratch::Get(stream, k * sizeof(int32_t)));
  MSHADOW_CUDA_CALL(cudaMemsetAsync(last, 0xff, k * sizeof(int32_t), stream));  // every entry -1
  const uint32_t un = static_cast<uint32_t>(n);
  IndexFillOwnerKernel<int32_t><<<gpu_rt::CeilDiv(n, 256), 256, 0, stream>>>(last, index, un, static_cast<int32_t>(k));
  MSHADOW_CUDA_POST_KERNEL_CHECK(IndexFillOwnerKernel);
  const bool vec = width % 4 == 0 && ld_src % 4 == 0 && ld_dst % 4 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  const int cap = gpu_rt::CurrentDevice().sm_count * 8;
  const int64_t sweeps = (n + 3) / 4;  // IndexFillCopyKernel takes four batch entries per sweep
  const int grid = sweeps < cap ? static_cast<int>(sweeps) : cap;
  if (vec) {
    IndexFillCopyKernel<4><<<grid, 256, 0, stream>>>(dst, ld_dst, last, index, src, ld_src, un,
                                                    static_cast<uint32_t>(width / 4), static_cast<int32_t>(k));
  } else {
    IndexFillCopyKernel<1><<<grid, 256, 0, stream>>>(dst, ld_dst, last, index, src, ld_src, un,
                                                    static_cast<uint32_t>(width), static_cast<int32_t>(k));
  }
  MSHADOW_CUDA_POST_KERNEL_CHECK(IndexFillCopyKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_EMBED_CUH_
