/*
 * Routing of a sorted (table row, source row) list to the GPU that owns the table rows, on the
 * device.  Used when the table of AddTakeGradLargeBatch (mshadow/cuda/tensor_gpu-inl.cuh:619-672:
 * dst[sorted[y]] += src[index[y]]) is spread over several GPUs with row r owned by GPU r % world
 * and a short list of frequent ("hot") rows summed by every GPU over its slice of the batch.
 *
 *   RunLengthKernel      for every list entry that starts a run of equal keys: the run's length
 *                        (0 for the other entries).  Sorting these lengths in descending order
 *                        with the engine's stable radix sort puts the most frequent rows first,
 *                        equal counts in ascending row order.
 *   RouteCountKernel     per tile of the list, how many entries belong to this GPU's "tail" part
 *                        (key not hot, key % world == rank) and to its "hot" part (key hot, source
 *                        row inside [src_begin, src_end)).
 *   RouteScanKernel      exclusive scan of the per-tile counts (one CTA), totals to `totals`.
 *   RouteScatterKernel   writes the selected entries in list order: first the tail part with keys
 *                        rewritten to local rows (key / world), then the hot part with keys
 *                        rewritten to hot_base + position in the hot list.  Both parts are sorted,
 *                        and every hot key is larger than every tail key when hot_base is the
 *                        number of local rows, so the output is again one sorted list.
 *
 *   RunHeadCountKernel / RunHeadScanKernel / RunIndexKernel
 *                        number the runs of equal keys (run_of[i], run_keys[j]): the key list of
 *                        a segmented sum into a compact matrix with one row per distinct key, which
 *                        is what a GPU sends to the owners when the SOURCE rows are spread over
 *                        the GPUs by batch position.
 *
 *   RunBoundsKernel / RunKeysToOwnersKernel, RowRoute
 *                        with keys of the form owner * per_owner + local row the runs of one owner
 *                        form a block; RowRoute tells the segmented sum (embed.cuh) to store the
 *                        sum of run j into row j - first[owner] of a matrix in the OWNER's memory,
 *                        and RunKeysToOwnersKernel stores the local row numbers beside them.
 *
 * The selection is stable, so each table row keeps its accumulation order.  All arithmetic is on
 * 32-bit integers; results are exact.
 */
#ifndef MSHADOW_GPU_ROUTE_CUH_
#define MSHADOW_GPU_ROUTE_CUH_

#include "./runtime.h"

namespace mshadow {
namespace cuda {
namespace routedetail {
const int kThreads = 256;
const int kItems = 8;                       // consecutive entries per thread
const int kTile = kThreads * kItems;
const int kMaxHot = 1024;                   // hot list length the kernels keep in shared memory

struct Geometry {
  int32_t world, rank;
  int32_t src_begin, src_end;               // source rows held by this GPU (for the hot part)
  int32_t hot_count, hot_base;
};

const int kMaxOwners = 16;

/*!
 * \brief where the rows of a compact run numbering live when consecutive blocks of runs belong to
 *  different owners: run j with first[q] <= j < first[q + 1] is row j - first[q] of the matrix at
 *  base[q] (an address in owner q's memory as mapped into this process).  world == 0: not routed.
 */
template <typename T>
struct OwnerBlocks {
  T *base[kMaxOwners];
  const int32_t *first;   // device array of world + 1 entries
  int32_t world;
};
typedef OwnerBlocks<float> RowRoute;

/*! \brief the owner of run j: the last q with first[q] <= j */
__device__ __forceinline__ int OwnerOf(const int32_t *first, int world, int32_t j) {
  int lo = 0, hi = world;               // first[lo] <= j < first[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (first[mid] <= j) lo = mid; else hi = mid;
  }
  return lo;
}

/*! \brief the owner block a thread looked up last: consecutive runs mostly share it */
struct OwnerHint {
  int32_t lo, hi;   // runs lo .. hi - 1 belong to owner q (lo == hi: nothing cached)
  int q;
};

/*! \brief address of row `run`: in the routed case inside its owner's block, else dst + run * ld */
__device__ __forceinline__ float *RowOf(const RowRoute &r, float *dst, int64_t ld, int32_t run, OwnerHint *hint) {
  if (r.world == 0) return dst + static_cast<int64_t>(run) * ld;
  if (run < hint->lo || run >= hint->hi) {
    hint->q = OwnerOf(r.first, r.world, run);
    hint->lo = r.first[hint->q];
    hint->hi = r.first[hint->q + 1];
  }
  return r.base[hint->q] + static_cast<int64_t>(run - hint->lo) * ld;
}

/*! \brief 0: tail entry of this GPU, 1: hot entry of this GPU, 2: not ours; `pos` = position in the hot list */
__device__ __forceinline__ int Classify(int32_t key, int32_t row, const Geometry &g, const int32_t *s_hot, int32_t *pos) {
  // lower bound of key in the ascending hot list
  int lo = 0, hi = g.hot_count;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (s_hot[mid] < key) lo = mid + 1; else hi = mid;
  }
  if (lo < g.hot_count && s_hot[lo] == key) {
    *pos = lo;
    return (row >= g.src_begin && row < g.src_end) ? 1 : 2;
  }
  return (key % g.world == g.rank) ? 0 : 2;
}

/*! \brief inclusive scan of one value per thread over a CTA of kThreads; returns this thread's exclusive prefix, total in *total */
__device__ __forceinline__ uint32_t CtaExclusiveScan(uint32_t v, uint32_t *s_warp, uint32_t *total) {
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= static_cast<uint32_t>(d)) inc += o;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  uint32_t base = 0, sum = 0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) {
    if (static_cast<uint32_t>(w) < warp) base += s_warp[w];
    sum += s_warp[w];
  }
  *total = sum;
  __syncthreads();
  return base + inc - v;
}
}  // namespace routedetail

/*! \brief lens[i] = length of the run of equal keys starting at i, 0 if i does not start one; rows[i] = keys[i] */
template <int kDummy>
__global__ void __launch_bounds__(256)
RunLengthKernel(int32_t *lens, int32_t *rows, const int32_t *keys, uint32_t n) {
  gpu_rt::GridDependencySync();
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int32_t k = keys[i];
  rows[i] = k;
  if (i > 0 && keys[i - 1] == k) {
    lens[i] = 0;
    return;
  }
  // first position after i whose key differs: doubling steps, then bisection
  uint32_t lo = i, step = 1;            // keys[lo] == k
  uint32_t hi = n;                      // keys[hi] != k (or hi == n)
  while (lo + step < n) {
    if (keys[lo + step] != k) {
      hi = lo + step;
      break;
    }
    lo += step;
    step <<= 1;
  }
  while (hi - lo > 1) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (keys[mid] == k) lo = mid; else hi = mid;
  }
  lens[i] = static_cast<int32_t>(hi - i);
}

/*! \brief counts[tile] = tail entries, counts[tiles + tile] = hot entries of this GPU in the tile */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RouteCountKernel(uint32_t *counts, const int32_t *keys, const int32_t *rows, uint32_t n, const int32_t *hot,
                 const routedetail::Geometry g) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ int32_t s_hot[kMaxHot];
  __shared__ uint32_t s_warp[kThreads / 32];
  for (int j = threadIdx.x; j < g.hot_count; j += kThreads) s_hot[j] = hot[j];
  __syncthreads();
  const uint32_t first = blockIdx.x * kTile + threadIdx.x * kItems;
  uint32_t mine = 0;                    // tail count in the low half, hot count in the high half
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const uint32_t e = first + u;
    if (e < n) {
      int32_t pos;
      const int c = Classify(keys[e], rows[e], g, s_hot, &pos);
      mine += c == 0 ? 1u : (c == 1 ? 65536u : 0u);
    }
  }
  uint32_t total;
  CtaExclusiveScan(mine, s_warp, &total);
  if (threadIdx.x == 0) {
    counts[blockIdx.x] = total & 0xffffu;
    counts[gridDim.x + blockIdx.x] = total >> 16;
  }
}

/*! \brief in-place exclusive scan of counts[0 .. 2*tiles) as two arrays of `tiles`; totals[0] = tail entries, totals[1] = hot entries */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RouteScanKernel(uint32_t *counts, uint32_t tiles, uint32_t *totals) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ uint32_t s_warp[kThreads / 32];
  for (int part = 0; part < 2; ++part) {
    uint32_t *c = counts + part * tiles;
    uint32_t running = 0;
    for (uint32_t t0 = 0; t0 < tiles; t0 += kThreads) {
      const uint32_t t = t0 + threadIdx.x;
      const uint32_t v = t < tiles ? c[t] : 0u;
      uint32_t total;
      const uint32_t ex = CtaExclusiveScan(v, s_warp, &total);
      if (t < tiles) c[t] = running + ex;
      running += total;
    }
    if (threadIdx.x == 0) totals[part] = running;
  }
}

/*! \brief writes this GPU's entries: tail part at [0, totals[0]), hot part behind it */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RouteScatterKernel(int32_t *out_keys, int32_t *out_rows, const uint32_t *bases, const uint32_t *totals,
                   const int32_t *keys, const int32_t *rows, uint32_t n, const int32_t *hot,
                   const routedetail::Geometry g) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ int32_t s_hot[kMaxHot];
  __shared__ uint32_t s_warp[kThreads / 32];
  for (int j = threadIdx.x; j < g.hot_count; j += kThreads) s_hot[j] = hot[j];
  __syncthreads();
  const uint32_t first = blockIdx.x * kTile + threadIdx.x * kItems;
  int32_t k[kItems], r[kItems], pos[kItems];
  int cls[kItems];
  uint32_t mine = 0;
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const uint32_t e = first + u;
    cls[u] = 2;
    pos[u] = 0;
    if (e < n) {
      k[u] = keys[e];
      r[u] = rows[e];
      cls[u] = Classify(k[u], r[u], g, s_hot, &pos[u]);
      mine += cls[u] == 0 ? 1u : (cls[u] == 1 ? 65536u : 0u);
    }
  }
  uint32_t total;
  const uint32_t ex = CtaExclusiveScan(mine, s_warp, &total);
  uint32_t at_tail = bases[blockIdx.x] + (ex & 0xffffu);
  uint32_t at_hot = totals[0] + bases[gridDim.x + blockIdx.x] + (ex >> 16);
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    if (cls[u] == 0) {
      out_keys[at_tail] = k[u] / g.world;
      out_rows[at_tail] = r[u];
      ++at_tail;
    } else if (cls[u] == 1) {
      out_keys[at_hot] = g.hot_base + pos[u];
      out_rows[at_hot] = r[u];
      ++at_hot;
    }
  }
}

/*! \brief counts[tile] = entries of the tile that start a run of equal keys */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RunHeadCountKernel(uint32_t *counts, const int32_t *keys, uint32_t n) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ uint32_t s_warp[kThreads / 32];
  const uint32_t first = blockIdx.x * kTile + threadIdx.x * kItems;
  uint32_t mine = 0;
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const uint32_t e = first + u;
    if (e < n && (e == 0 || keys[e - 1] != keys[e])) ++mine;
  }
  uint32_t total;
  CtaExclusiveScan(mine, s_warp, &total);
  if (threadIdx.x == 0) counts[blockIdx.x] = total;
}

/*! \brief in-place exclusive scan of counts[0 .. tiles); total[0] = sum */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RunHeadScanKernel(uint32_t *counts, uint32_t tiles, uint32_t *total_out) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ uint32_t s_warp[kThreads / 32];
  uint32_t running = 0;
  for (uint32_t t0 = 0; t0 < tiles; t0 += kThreads) {
    const uint32_t t = t0 + threadIdx.x;
    const uint32_t v = t < tiles ? counts[t] : 0u;
    uint32_t total;
    const uint32_t ex = CtaExclusiveScan(v, s_warp, &total);
    if (t < tiles) counts[t] = running + ex;
    running += total;
  }
  if (threadIdx.x == 0) total_out[0] = running;
}

/*! \brief run_of[i] = number of the run entry i belongs to (0, 1, ...); run_keys[j] = key of run j */
template <int kDummy>
__global__ void __launch_bounds__(routedetail::kThreads)
RunIndexKernel(int32_t *run_of, int32_t *run_keys, const uint32_t *bases, const int32_t *keys, uint32_t n) {
  gpu_rt::GridDependencySync();
  using namespace routedetail;
  __shared__ uint32_t s_warp[kThreads / 32];
  const uint32_t first = blockIdx.x * kTile + threadIdx.x * kItems;
  int32_t k[kItems];
  bool head[kItems];
  uint32_t mine = 0;
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const uint32_t e = first + u;
    head[u] = false;
    if (e < n) {
      k[u] = keys[e];
      head[u] = e == 0 || keys[e - 1] != k[u];
      mine += head[u] ? 1u : 0u;
    }
  }
  uint32_t total;
  // runs that start before this thread's first entry, minus one: the run its first entry continues
  uint32_t at = bases[blockIdx.x] + CtaExclusiveScan(mine, s_warp, &total);
#pragma unroll
  for (int u = 0; u < kItems; ++u) {
    const uint32_t e = first + u;
    if (e < n) {
      if (head[u]) {
        run_keys[at] = k[u];
        ++at;
      }
      run_of[e] = static_cast<int32_t>(at - 1);
    }
  }
}

/*!
 * \brief first[q] = number of runs whose key is below q * per_owner, for q = 0 .. world: with keys
 *  of the form owner * per_owner + local row, the block of runs of every owner.  One warp.
 */
template <int kDummy>
__global__ void RunBoundsKernel(int32_t *first, const int32_t *run_keys, const uint32_t *total, int world,
                                int32_t per_owner) {
  gpu_rt::GridDependencySync();
  const int q = threadIdx.x;
  if (q > world) return;
  const uint32_t runs = total[0];
  const int64_t want = static_cast<int64_t>(q) * per_owner;
  uint32_t lo = 0, hi = runs;           // lower bound of `want` in run_keys[0 .. runs)
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    if (run_keys[mid] < want) lo = mid + 1; else hi = mid;
  }
  first[q] = static_cast<int32_t>(lo);
}

/*! \brief hands every owner the local row numbers of its runs: to.base[q][j - first[q]] = run_keys[j] - q * per_owner */
template <int kDummy>
__global__ void __launch_bounds__(256)
RunKeysToOwnersKernel(const routedetail::OwnerBlocks<int32_t> to, const int32_t *run_keys, int32_t per_owner) {
  gpu_rt::GridDependencySync();
  const int32_t runs = to.first[to.world];
  for (int32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < runs; j += gridDim.x * blockDim.x) {
    const int q = routedetail::OwnerOf(to.first, to.world, j);
    to.base[q][j - to.first[q]] = run_keys[j] - q * per_owner;
  }
}

namespace routedetail {
inline size_t Align256(size_t b) { return (b + 255) / 256 * 256; }
inline uint32_t Tiles(int64_t n) { return static_cast<uint32_t>((n + kTile - 1) / kTile); }
/*! \brief bytes of scratch RouteCyclicHotLaunch needs */
inline size_t RouteScratchBytes(int64_t n) { return Align256(2ull * Tiles(n) * sizeof(uint32_t)); }
}  // namespace routedetail

/*!
 * \brief this GPU's part of a sorted (key, source row) list under cyclic row ownership with hot rows.
 *  out_keys / out_rows need room for n entries; totals (two device words) receives the number of
 *  tail and of hot entries written.  `hot` is ascending, at most routedetail::kMaxHot long.
 */
inline void RouteCyclicHotLaunch(int32_t *out_keys, int32_t *out_rows, uint32_t *totals, const int32_t *keys,
                                 const int32_t *rows, int64_t n, const int32_t *hot, int hot_count, int world, int rank,
                                 int32_t src_begin, int32_t src_end, int32_t hot_base, cudaStream_t stream) {
  using namespace routedetail;
  CHECK_LT(n, (int64_t(1) << 31));
  CHECK(hot_count >= 0 && hot_count <= kMaxHot) << "RouteCyclicHot: at most " << kMaxHot << " hot rows";
  CHECK(world >= 1 && rank >= 0 && rank < world) << "RouteCyclicHot: rank outside the group";
  if (n == 0) {
    MSHADOW_CUDA_CALL(cudaMemsetAsync(totals, 0, 2 * sizeof(uint32_t), stream));
    return;
  }
  const uint32_t tiles = Tiles(n);
  uint32_t *counts = static_cast<uint32_t *>(gpu_rt::Scratch::Get(stream, RouteScratchBytes(n)));
  const Geometry g = {world, rank, src_begin, src_end, hot_count, hot_base};
  const uint32_t un = static_cast<uint32_t>(n);
  gpu_rt::LaunchAfterDrain(RouteCountKernel<0>, dim3(tiles), dim3(kThreads), 0, stream, counts, keys, rows, un, hot, g);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RouteCountKernel);
  gpu_rt::LaunchAfterDrain(RouteScanKernel<0>, dim3(1), dim3(kThreads), 0, stream, counts, tiles, totals);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RouteScanKernel);
  gpu_rt::LaunchAfterDrain(RouteScatterKernel<0>, dim3(tiles), dim3(kThreads), 0, stream, out_keys, out_rows, counts, totals, keys, rows, un, hot, g);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RouteScatterKernel);
}

/*!
 * \brief numbers the runs of equal keys of an ascending list: run_of[i] in 0 .. runs-1 for every
 *  entry, run_keys[j] the key of run j (room for n), total[0] (device word) the number of runs.
 *  With run_of as the key list, a segmented sum lands in a compact matrix of one row per
 *  distinct key instead of a table of all possible keys.
 */
inline void RunIndexLaunch(int32_t *run_of, int32_t *run_keys, uint32_t *total, const int32_t *keys, int64_t n,
                           cudaStream_t stream) {
  using namespace routedetail;
  CHECK_LT(n, (int64_t(1) << 31));
  if (n == 0) {
    MSHADOW_CUDA_CALL(cudaMemsetAsync(total, 0, sizeof(uint32_t), stream));
    return;
  }
  const uint32_t tiles = Tiles(n);
  uint32_t *counts = static_cast<uint32_t *>(gpu_rt::Scratch::Get(stream, RouteScratchBytes(n)));
  const uint32_t un = static_cast<uint32_t>(n);
  gpu_rt::LaunchAfterDrain(RunHeadCountKernel<0>, dim3(tiles), dim3(kThreads), 0, stream, counts, keys, un);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunHeadCountKernel);
  gpu_rt::LaunchAfterDrain(RunHeadScanKernel<0>, dim3(1), dim3(kThreads), 0, stream, counts, tiles, total);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunHeadScanKernel);
  gpu_rt::LaunchAfterDrain(RunIndexKernel<0>, dim3(tiles), dim3(kThreads), 0, stream, run_of, run_keys, counts, keys, un);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunIndexKernel);
}

/*! \brief first[0 .. world] (device): the block of runs of every owner, for run keys owner * per_owner + local row */
inline void RunBoundsLaunch(int32_t *first, const int32_t *run_keys, const uint32_t *total, int world,
                            int32_t per_owner, cudaStream_t stream) {
  CHECK(world >= 1 && world <= routedetail::kMaxOwners) << "RunBounds: at most " << routedetail::kMaxOwners << " owners";
  gpu_rt::LaunchAfterDrain(RunBoundsKernel<0>, dim3(1), dim3(32), 0, stream, first, run_keys, total, world, per_owner);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunBoundsKernel);
}

/*! \brief the owners' row numbers of all runs, stored into the owners' blocks (`n` bounds the number of runs) */
inline void RunKeysToOwnersLaunch(const routedetail::OwnerBlocks<int32_t> &to, const int32_t *run_keys, int64_t n,
                                  int32_t per_owner, cudaStream_t stream) {
  if (n == 0) return;
  unsigned grid = gpu_rt::CeilDiv(static_cast<uint32_t>(n), 256u);
  if (grid > 1184u) grid = 1184u;
  gpu_rt::LaunchAfterDrain(RunKeysToOwnersKernel<0>, dim3(grid), dim3(256), 0, stream, to, run_keys, per_owner);
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunKeysToOwnersKernel);
}

/*! \brief lens[i] = run length at run heads of the sorted list, 0 elsewhere; rows[i] = keys[i] */
inline void RunLengthLaunch(int32_t *lens, int32_t *rows, const int32_t *keys, int64_t n, cudaStream_t stream) {
  if (n == 0) return;
  CHECK_LT(n, (int64_t(1) << 31));
  gpu_rt::LaunchAfterDrain(RunLengthKernel<0>, dim3(gpu_rt::CeilDiv(static_cast<uint32_t>(n), 256u)), dim3(256), 0, stream, lens, rows, keys,
                                                                                        static_cast<uint32_t>(n));
  MSHADOW_CUDA_POST_KERNEL_CHECK(RunLengthKernel);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_ROUTE_CUH_
