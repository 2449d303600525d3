/*
 * Reductions of a matrix-viewed expression to a vector:
 *   KeepLowest   dst[x] <Saver>= scale * Reduce_y plan(y, x)               (column reduce)
 *   KeepHighDim  dst[c] <Saver>= scale * Reduce_{n,y,x} plan((n*C+c)*H+y, x) (channel reduce)
 * They replace MapRedKeepLowestKernel / MapReduceKeepDim1Kernel and the shared-memory tree
 * of the reference (mshadow/cuda/tensor_gpu-inl.cuh:122-215, mshadow/cuda/reduce.cuh:42-116),
 * which give each output column strip / channel to a single CTA -- 128 CTAs for a 4096-wide
 * matrix, each walking all 65536 rows -- and so cannot fill a 148-SM device.
 *
 * Here the reduced extent is split over many CTAs.  Each thread accumulates 16-byte groups
 * in registers; inside a CTA values meet through warp shuffles and a small shared buffer;
 * the CTAs of a thread-block cluster (up to 8, laid along the reduced extent) meet through
 * distributed shared memory, read by the cluster's first CTA in rank order; and if more
 * than one cluster covers an output, cluster results go to a scratch matrix that a small
 * second kernel folds in a fixed order.  Every combine order is fixed by the launch
 * geometry, so results are reproducible run to run.  Both kernels are bound by HBM
 * bandwidth: 4 bytes read per input element, nothing else of size.
 *
 * The thread that stores a final result can also hand it to the other GPUs of an exchange
 * group (gpu_rt::PeerSink, see peer_sink.h): the value scale * Reduce(...) -- what the saver
 * receives -- goes into every rank's exchange window by one 64-bit store per rank.
 */
#ifndef MSHADOW_GPU_REDUCE_CUH_
#define MSHADOW_GPU_REDUCE_CUH_

#include <cooperative_groups.h>

#include "./peer_sink.h"
#include "./runtime.h"

namespace mshadow {
namespace cuda {

namespace cg = cooperative_groups;

const int kRedLowThreads = MSHADOW_B200_REDLOW_THREADS;
const int kRedHighThreads = MSHADOW_B200_REDHIGH_THREADS;
const int kRedMaxCluster = 8;

namespace reddetail {

/*! \brief kLanes consecutive elements of a plan row, by one 128-bit access when kLanes > 1 */
template <int kLanes, typename DType, typename SPlan>
__device__ __forceinline__ void LoadLanes(const SPlan &plan, index_t y, index_t x, DType (&out)[kLanes]) {
  if constexpr (kLanes == 1) {
    out[0] = plan.Eval(y, x);
  } else {
    const expr::Pack<DType> p = plan.EvalPack(y, x);
#pragma unroll
    for (int l = 0; l < kLanes; ++l) out[l] = p.v[l];
  }
}

/*!
 * \brief folds first[0], first[stride], ..., first[(count-1)*stride] (values parked by other CTAs of
 *  the launch) in that order.  The loads go out in batches of eight before any is used: one
 *  dependent L2 round trip per value would cost more than the fold is allowed to.
 */
template <typename Reducer, typename DType>
__device__ __forceinline__ DType FoldParked(const DType *first, size_t stride, unsigned count) {
  constexpr int kBatch = 8;
  DType sum = gpu_rt::LoadCg(first);
  for (unsigned k = 1; k < count; k += kBatch) {
    DType v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k + j < count) v[j] = gpu_rt::LoadCg(first + static_cast<size_t>(k + j) * stride);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k + j < count) Reducer::Reduce(sum, v[j]);
    }
  }
  return sum;
}

template <typename DType>
__device__ __forceinline__ DType ShflDown(DType v, int delta) {
  if constexpr (sizeof(DType) == 8) {
    const unsigned long long b = __shfl_down_sync(0xffffffffu, *reinterpret_cast<unsigned long long *>(&v), delta);
    return *reinterpret_cast<const DType *>(&b);
  } else {
    static_assert(sizeof(DType) <= 4, "unsupported element size");
    unsigned int raw = 0;
    memcpy(&raw, &v, sizeof(DType));
    raw = __shfl_down_sync(0xffffffffu, raw, delta);
    DType r;
    memcpy(&r, &raw, sizeof(DType));
    return r;
  }
}

/*! \brief fold the values of a CTA into thread 0; `buf` holds one element per warp */
template <typename Reducer, typename DType, int kThreads>
__device__ __forceinline__ DType BlockReduce(DType v, DType *buf) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    DType o = ShflDown(v, d);
    Reducer::Reduce(v, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  if (warp == 0) {
    DType init;
    Reducer::SetInitValue(init);
    v = lane < kThreads / 32 ? buf[lane] : init;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      DType o = ShflDown(v, d);
      Reducer::Reduce(v, o);
    }
  }
  return v;
}

}  // namespace reddetail

/*!
 * \brief column reduce.  grid = (column tiles, row chunks); a cluster spans row chunks.
 *  Each thread owns kLanes adjacent columns and the rows of its chunk.
 *  If `partial` is null the grid has a single cluster per column tile and results go
 *  straight to `dst`; otherwise cluster c writes row c of the `partial` matrix.
 */
template <typename Saver, typename Reducer, int kLanes, typename DType, typename DPlan, typename SPlan>
__global__ void __launch_bounds__(kRedLowThreads)
ReduceKeepLowestKernel(DPlan dst, const SPlan src, uint32_t rows, uint32_t cols, uint32_t rows_per_chunk,
                       DType scale, DType *partial, const gpu_rt::PeerSink sink) {
  gpu_rt::GridDependencySync();
  __shared__ __align__(16) DType stage[kRedLowThreads * kLanes];
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t x = (blockIdx.x * kRedLowThreads + threadIdx.x) * kLanes;
  const uint32_t y0 = blockIdx.y * rows_per_chunk;
  uint32_t y1 = y0 + rows_per_chunk;
  if (y1 > rows) y1 = rows;
  const bool live = x < cols && y0 < y1;
  DType acc[kLanes];
  if (live) {
    reddetail::LoadLanes<kLanes>(src, y0, x, acc);
    uint32_t y = y0 + 1;
    constexpr int kDepth = MSHADOW_B200_REDLOW_DEPTH;
    for (; y + kDepth <= y1; y += kDepth) {
      DType v[kDepth][kLanes];
#pragma unroll
      for (int k = 0; k < kDepth; ++k) reddetail::LoadLanes<kLanes>(src, y + k, x, v[k]);
#pragma unroll
      for (int k = 0; k < kDepth; ++k)
#pragma unroll
        for (int l = 0; l < kLanes; ++l) Reducer::Reduce(acc[l], v[k][l]);
    }
    for (; y < y1; ++y) {
      DType v[kLanes];
      reddetail::LoadLanes<kLanes>(src, y, x, v);
#pragma unroll
      for (int l = 0; l < kLanes; ++l) Reducer::Reduce(acc[l], v[l]);
    }
  }
  const unsigned csize = cluster.num_blocks();
  if (csize > 1) {
    // meet the other row chunks of this cluster through distributed shared memory
    const unsigned crank = cluster.block_rank();
    if (crank != 0 && live) {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) stage[threadIdx.x * kLanes + l] = acc[l];
    }
    cluster.sync();
    if (crank == 0 && live) {
      for (unsigned r = 1; r < csize; ++r) {
        // a later chunk may lie wholly past the last row; it then holds nothing
        if ((blockIdx.y + r) * rows_per_chunk >= rows) break;
        const DType *remote = cluster.map_shared_rank(stage, r);
#pragma unroll
        for (int l = 0; l < kLanes; ++l) Reducer::Reduce(acc[l], remote[threadIdx.x * kLanes + l]);
      }
    }
    cluster.sync();  // keep every CTA's shared memory alive until the first CTA has read it
    if (crank != 0) return;
  }
  if (partial == nullptr) {
    if (!live) return;
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      if (x + l < cols) {
        Saver::Save(dst.REval(0, x + l), DType(acc[l] * scale));
        if (sink.world > 0) sink.Put(x + l, DType(acc[l] * scale));
      }
    }
    return;
  }
  // several clusters share these columns: park this cluster's row for ReduceFinishKernel
  if (!live) return;
  DType *row = partial + static_cast<size_t>(blockIdx.y / csize) * cols;
#pragma unroll
  for (int l = 0; l < kLanes; ++l) {
    if (x + l < cols) row[x + l] = acc[l];
  }
}

/*!
 * \brief fold the `nparts` rows that the clusters of a reduction parked in `partial`, in row
 *  order, into dst.  A second launch rather than a fold by the last-arriving cluster of the
 *  first: the ticket counter, fences and barriers which that needs at the end of every
 *  cluster cost more (measured: about 1.5 % of the 65536 x 4096 column sum) than this
 *  launch, which only exists for inputs large enough to need several clusters per output.
 */
template <typename Saver, typename Reducer, typename DType, typename DPlan>
__global__ void ReduceFinishKernel(DPlan dst, const DType *partial, uint32_t nparts, uint32_t cols, DType scale,
                                   const gpu_rt::PeerSink sink) {
  gpu_rt::GridDependencySync();
  const uint32_t x = blockIdx.x * blockDim.x + threadIdx.x;
  if (x >= cols) return;
  const DType sum = reddetail::FoldParked<Reducer>(partial + x, cols, nparts);
  Saver::Save(dst.REval(0, x), DType(sum * scale));
  if (sink.world > 0) sink.Put(x, DType(sum * scale));
}

/*!
 * \brief channel reduce.  grid = (channels, n chunks); a cluster spans n chunks.
 *  The (inner_rows x width) plane of every (n, c) is walked as packs_per_row groups per
 *  row; `width` must be a multiple of kLanes.
 */
template <typename Saver, typename Reducer, int kLanes, typename DType, typename DPlan, typename SPlan>
__global__ void __launch_bounds__(kRedHighThreads)
ReduceKeepHighDimKernel(DPlan dst, const SPlan src, uint32_t outer, uint32_t channels, uint32_t inner_rows,
                        uint32_t packs_per_row, gpu_rt::FastDiv row_of_pack, gpu_rt::FastDiv plane_of_pack,
                        uint32_t outer_per_chunk, DType scale, DType *partial, const gpu_rt::PeerSink sink) {
  gpu_rt::GridDependencySync();
  __shared__ DType warp_buf[kRedHighThreads / 32];
  __shared__ DType cta_val;
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t c = blockIdx.x;
  const uint32_t n0 = blockIdx.y * outer_per_chunk;
  uint32_t n1 = n0 + outer_per_chunk;
  if (n1 > outer) n1 = outer;
  const uint32_t per_plane = inner_rows * packs_per_row;
  DType acc[kLanes];
#pragma unroll
  for (int l = 0; l < kLanes; ++l) Reducer::SetInitValue(acc[l]);
  // the chunk's planes are walked as one list of 16-byte groups, so that every thread always
  // has kDepth independent loads in flight whatever the plane size
  constexpr int kDepth = MSHADOW_B200_REDHIGH_DEPTH;
  const uint32_t npacks = (n1 > n0 ? n1 - n0 : 0) * per_plane;
  for (uint32_t base = threadIdx.x; base < npacks; base += kRedHighThreads * kDepth) {
    DType v[kDepth][kLanes];
#pragma unroll
    for (int k = 0; k < kDepth; ++k) {
      const uint32_t i = base + k * kRedHighThreads;
      if (i < npacks) {
        const uint32_t dn = plane_of_pack.Quot(i);
        const uint32_t r = i - dn * per_plane;
        const uint32_t y = inner_rows == 1 ? 0 : row_of_pack.Quot(r);
        reddetail::LoadLanes<kLanes>(src, ((n0 + dn) * channels + c) * inner_rows + y,
                                     (r - y * packs_per_row) * kLanes, v[k]);
      } else {
#pragma unroll
        for (int l = 0; l < kLanes; ++l) Reducer::SetInitValue(v[k][l]);
      }
    }
#pragma unroll
    for (int k = 0; k < kDepth; ++k)
#pragma unroll
      for (int l = 0; l < kLanes; ++l) Reducer::Reduce(acc[l], v[k][l]);
  }
#pragma unroll
  for (int l = 1; l < kLanes; ++l) Reducer::Reduce(acc[0], acc[l]);
  DType total = reddetail::BlockReduce<Reducer, DType, kRedHighThreads>(acc[0], warp_buf);
  const unsigned csize = cluster.num_blocks();
  if (csize > 1) {
    const unsigned crank = cluster.block_rank();
    if (threadIdx.x == 0) cta_val = total;
    cluster.sync();
    if (crank == 0 && threadIdx.x == 0) {
      for (unsigned r = 1; r < csize; ++r) {
        const DType *remote = cluster.map_shared_rank(&cta_val, r);
        Reducer::Reduce(total, *remote);
      }
    }
    cluster.sync();
    if (crank != 0) return;
  }
  if (threadIdx.x != 0) return;
  if (partial == nullptr) {
    Saver::Save(dst.REval(0, c), DType(total * scale));
    if (sink.world > 0) sink.Put(c, DType(total * scale));
    return;
  }
  // several clusters per channel: park the cluster's value for ReduceFinishKernel
  partial[static_cast<size_t>(blockIdx.y / csize) * channels + c] = total;
}

namespace reddetail {
/*! \brief launch with a (1, cluster_y, 1) thread-block cluster */
template <typename Kernel, typename... Args>
inline void LaunchClustered(Kernel kernel, dim3 grid, dim3 block, unsigned cluster_y, cudaStream_t stream,
                            Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cluster_y;
  attr[0].val.clusterDim.z = 1;
  // the kernels begin with GridDependencySync(): see gpu_rt::LaunchAfterDrain
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = MSHADOW_B200_EARLY_LAUNCH ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, kernel, args...));
}

/*! \brief split `extent` into chunks: about `want` of them, a multiple of the cluster size */
struct Split {
  uint32_t per_chunk, chunks, cluster, clusters;
};
inline Split PlanSplit(uint32_t extent, uint32_t want, uint32_t min_per_chunk) {
  Split s;
  uint32_t chunks = want < 1 ? 1 : want;
  const uint32_t max_chunks = (extent + min_per_chunk - 1) / min_per_chunk;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  s.per_chunk = (extent + chunks - 1) / chunks;
  chunks = (extent + s.per_chunk - 1) / s.per_chunk;  // drop chunks that would be empty
  s.cluster = chunks < static_cast<uint32_t>(kRedMaxCluster) ? chunks : kRedMaxCluster;
  s.clusters = (chunks + s.cluster - 1) / s.cluster;
  s.chunks = s.clusters * s.cluster;  // trailing chunks of the last cluster may be empty
  return s;
}

/*!
 * \brief number of chunks k (1..kmax) for a grid of fixed*k CTAs on a device that keeps
 *  `slots` CTAs resident: the smallest k that fills whole waves to at least 95 %, or the
 *  best-filling k if none does.  A partly filled last wave is pure loss for kernels whose
 *  CTAs all run equally long.
 */
inline uint32_t WaveFriendlyChunks(uint32_t fixed, uint32_t kmax, uint32_t slots) {
  if (kmax < 1) kmax = 1;
  if (static_cast<uint64_t>(fixed) * kmax <= slots) return kmax;  // cannot even fill one wave
  uint32_t best = 1;
  double best_eff = 0.0;
  for (uint32_t k = 1; k <= kmax; ++k) {
    const uint64_t ctas = static_cast<uint64_t>(fixed) * k;
    if (ctas < slots) continue;
    const uint64_t waves = (ctas + slots - 1) / slots;
    const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = k;
    }
    if (eff >= 0.95) return k;
  }
  return best;
}

/*! \brief split `extent` into exactly-planned chunks; the cluster size is the largest divisor <= 8 */
inline Split PlanSplitWaves(uint32_t extent, uint32_t fixed, uint32_t slots, uint32_t max_chunks) {
  Split s;
  if (extent == 0) {  // nothing to walk: one CTA per output stores the reducer's initial value
    s.per_chunk = s.chunks = s.cluster = s.clusters = 1;
    return s;
  }
  if (max_chunks > extent) max_chunks = extent;
  // Few, long CTAs first: with at most kRedMaxCluster chunks one cluster covers an output, so no
  // partial rows are parked and no finishing launch follows.  Measured on (256,512,28,28) with 1184
  // resident CTAs: 2 or 4 chunks 93 %, 6 chunks 90 %, 8 chunks 88 %, 9 chunks (three clusters and a
  // finishing launch, 97 % wave fill) 82-86 %, 16 chunks 78 % of copy bandwidth.  So: the best wave
  // fill among 1..kRedMaxCluster chunks, the fewest chunks on a tie, if that fills 80 % of its waves;
  // otherwise the search over any number of chunks.
  uint32_t chunks = 0;
  double best_fill = 0.0;
  for (uint32_t k = 1; k <= static_cast<uint32_t>(kRedMaxCluster) && k <= max_chunks; ++k) {
    const uint64_t ctas = static_cast<uint64_t>(fixed) * k;
    const uint64_t waves = (ctas + slots - 1) / slots;
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    if (fill > best_fill + 1e-9) {
      best_fill = fill;
      chunks = k;
    }
  }
  if (best_fill < 0.80) chunks = WaveFriendlyChunks(fixed, max_chunks, slots);
  if (MSHADOW_B200_REDHIGH_CHUNKS > 0 && MSHADOW_B200_REDHIGH_CHUNKS <= max_chunks) chunks = MSHADOW_B200_REDHIGH_CHUNKS;
  s.per_chunk = (extent + chunks - 1) / chunks;
  chunks = (extent + s.per_chunk - 1) / s.per_chunk;
  s.cluster = 1;
  for (uint32_t d = kRedMaxCluster; d >= 1; --d) {
    if (chunks % d == 0) {
      s.cluster = d;
      break;
    }
  }
  s.clusters = chunks / s.cluster;
  s.chunks = chunks;
  return s;
}

/*!
 * \brief row split of the column reduce: `col_tiles` CTA columns times k row chunks, at least
 *  32 rows per chunk.  Prefers the smallest k that is a multiple of the cluster size and fills
 *  whole waves of `slots` resident CTAs to 95 %; otherwise the best-filling k of any kind.
 *  Shared by the allocating and the allocation-free entry points, which must agree.
 */
inline Split PlanKeepLowest(uint32_t rows, uint32_t col_tiles, uint32_t slots) {
  uint32_t kmax = rows / 32;
  if (kmax < 1) kmax = 1;
  if (kmax > 4096) kmax = 4096;
  uint32_t pick = 0;
  // Few, long CTAs first.  Every CTA streams its own band of rows, so the number of CTAs in flight is
  // the number of DRAM streams; measured on 65536 x 4096 (8 column tiles, 148 SMs, 16 CTAs resident
  // per SM): 128 chunks = 1024 CTAs, seven per SM, 98 % of copy bandwidth; 256 chunks 96 %; 288 chunks
  // (what filling one wave of resident CTAs to 95 % picks) 93 %; 296 chunks = every slot taken 86 %;
  // 64 chunks (3.5 per SM, unbalanced) 84 %.  So: about MSHADOW_B200_REDLOW_CTAS_PER_SM CTAs per SM,
  // a multiple of the cluster size, nudged downwards until the SMs carry equal numbers of CTAs.
  const uint32_t sms = static_cast<uint32_t>(gpu_rt::CurrentDevice().sm_count);
  const uint64_t target = static_cast<uint64_t>(MSHADOW_B200_REDLOW_CTAS_PER_SM) * sms;
  if (static_cast<uint64_t>(col_tiles) * kmax >= target && target / col_tiles >= static_cast<uint64_t>(kRedMaxCluster)) {
    uint32_t k0 = static_cast<uint32_t>(target / col_tiles);
    k0 -= k0 % kRedMaxCluster;
    double best_balance = 0.0;
    for (uint32_t k = k0; k >= static_cast<uint32_t>(kRedMaxCluster) && 2 * k >= k0; k -= kRedMaxCluster) {
      const uint64_t ctas = static_cast<uint64_t>(col_tiles) * k;
      const uint64_t per_sm = (ctas + sms - 1) / sms;
      const double balance = static_cast<double>(ctas) / static_cast<double>(per_sm * sms);
      if (balance > best_balance + 1e-9) {
        best_balance = balance;
        pick = k;
      }
      if (balance >= 0.97) break;
    }
  }
  if (pick == 0 && static_cast<uint64_t>(col_tiles) * kmax > slots) {
    for (uint32_t k = kRedMaxCluster; k <= kmax && pick == 0; k += kRedMaxCluster) {
      const uint64_t ctas = static_cast<uint64_t>(col_tiles) * k;
      if (ctas * 20 < static_cast<uint64_t>(slots) * 19) continue;  // under 95 % of one wave
      const uint64_t waves = (ctas + slots - 1) / slots;
      if (ctas * 20 >= waves * slots * 19) pick = k;
    }
  }
  if (pick == 0) pick = WaveFriendlyChunks(col_tiles, kmax, slots);
  if (MSHADOW_B200_REDLOW_CHUNKS > 0 && MSHADOW_B200_REDLOW_CHUNKS <= kmax) pick = MSHADOW_B200_REDLOW_CHUNKS;
  Split s;
  s.per_chunk = (rows + pick - 1) / pick;
  uint32_t chunks = (rows + s.per_chunk - 1) / s.per_chunk;
  s.cluster = 1;
  for (uint32_t d = kRedMaxCluster; d >= 1; --d) {
    if (chunks % d == 0) {
      s.cluster = d;
      break;
    }
  }
  s.clusters = chunks / s.cluster;
  s.chunks = chunks;
  return s;
}

/*! \brief the sink armed for this host thread's next reduction (peer_sink.h), checked against the launch */
template <typename DType>
inline gpu_rt::PeerSink TakePeerSink(uint32_t results) {
  const gpu_rt::PeerSink *pending = gpu_rt::PendingPeerSink();
  if (pending == nullptr || pending->world == 0) return gpu_rt::PeerSink();
  gpu_rt::PendingPeerSink() = nullptr;  // one reduction per arming
  CHECK_EQ(sizeof(DType), 4U) << "a peer sink carries 4-byte elements";
  CHECK_EQ(pending->count, results) << "the peer sink expects " << pending->count << " results, the reduction gives "
                                    << results;
  return *pending;
}

/*! \brief CTAs of `kernel` that the current device keeps resident at once */
template <typename Kernel>
inline uint32_t ResidentCtas(Kernel kernel, int threads) {
  return static_cast<uint32_t>(gpu_rt::ResidentPerSM(kernel, threads)) *
         static_cast<uint32_t>(gpu_rt::CurrentDevice().sm_count);
}
}  // namespace reddetail

/*! \brief host side of the column reduce */
template <typename Saver, typename Reducer, int kLanes, typename DType, typename DPlan, typename SPlan>
inline void ReduceKeepLowestLaunch(DPlan dplan, const SPlan &splan, Shape<2> eshape, DType scale,
                                   cudaStream_t stream) {
  const uint32_t rows = eshape[0], cols = eshape[1];
  const uint32_t col_tiles = gpu_rt::CeilDiv(cols, kRedLowThreads * kLanes);
  auto kernel = ReduceKeepLowestKernel<Saver, Reducer, kLanes, DType, DPlan, SPlan>;
  const uint32_t slots = reddetail::ResidentCtas(kernel, kRedLowThreads);
  const reddetail::Split sp = reddetail::PlanKeepLowest(rows, col_tiles, slots);
  const gpu_rt::PeerSink sink = reddetail::TakePeerSink<DType>(cols);
  const gpu_rt::PeerSink none;
  DType *partial = nullptr;
  if (sp.clusters > 1) {
    partial = static_cast<DType *>(
        gpu_rt::Scratch::Get(stream, static_cast<size_t>(sp.clusters) * cols * sizeof(DType)));
  }
  reddetail::LaunchClustered(kernel, dim3(col_tiles, sp.chunks), dim3(kRedLowThreads), sp.cluster, stream,
                             dplan, splan, rows, cols, sp.per_chunk, scale, partial, partial == nullptr ? sink : none);
  MSHADOW_CUDA_POST_KERNEL_CHECK(ReduceKeepLowestKernel);
  if (partial != nullptr) {
    gpu_rt::LaunchAfterDrain(ReduceFinishKernel<Saver, Reducer, DType, DPlan>, dim3(gpu_rt::CeilDiv(cols, 256)), dim3(256),
                             0, stream, dplan, partial, sp.clusters, cols, scale, sink);
    MSHADOW_CUDA_POST_KERNEL_CHECK(ReduceFinishKernel);
  }
}

/*! \brief host side of the channel reduce; pshape = (outer, channels, inner rows, width) */
template <typename Saver, typename Reducer, int kLanes, typename DType, typename DPlan, typename SPlan>
inline void ReduceKeepHighDimLaunch(DPlan dplan, const SPlan &splan, Shape<4> pshape, DType scale,
                                    cudaStream_t stream) {
  const uint32_t outer = pshape[0], channels = pshape[1], inner_rows = pshape[2], width = pshape[3];
  CHECK_EQ(width % kLanes, 0U);
  const uint32_t ppr = width / kLanes;
  auto kernel = ReduceKeepHighDimKernel<Saver, Reducer, kLanes, DType, DPlan, SPlan>;
  // whole waves of resident CTAs; at most 64 chunks, each at least one outer index
  const uint32_t slots = reddetail::ResidentCtas(kernel, kRedHighThreads);
  const reddetail::Split sp = reddetail::PlanSplitWaves(outer, channels, slots, 64);
  const gpu_rt::PeerSink sink = reddetail::TakePeerSink<DType>(channels);
  const gpu_rt::PeerSink none;
  DType *partial = nullptr;
  if (sp.clusters > 1) {
    partial = static_cast<DType *>(
        gpu_rt::Scratch::Get(stream, static_cast<size_t>(sp.clusters) * channels * sizeof(DType)));
  }
  const uint32_t per_plane = inner_rows * ppr;
  reddetail::LaunchClustered(kernel, dim3(channels, sp.chunks), dim3(kRedHighThreads), sp.cluster, stream,
                             dplan, splan, outer, channels, inner_rows, ppr, gpu_rt::FastDiv(ppr),
                             gpu_rt::FastDiv(per_plane == 0 ? 1 : per_plane), sp.per_chunk, scale, partial,
                             partial == nullptr ? sink : none);
  MSHADOW_CUDA_POST_KERNEL_CHECK(ReduceKeepHighDimKernel);
  if (partial != nullptr) {
    gpu_rt::LaunchAfterDrain(ReduceFinishKernel<Saver, Reducer, DType, DPlan>, dim3(gpu_rt::CeilDiv(channels, 256)),
                             dim3(256), 0, stream, dplan, partial, sp.clusters, channels, scale, sink);
    MSHADOW_CUDA_POST_KERNEL_CHECK(ReduceFinishKernel);
  }
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_REDUCE_CUH_
