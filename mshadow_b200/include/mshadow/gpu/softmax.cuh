/*
 * Row softmax and the SoftmaxGrad family on the GPU.
 *
 * Softmax replaces the reference's SoftmaxKernel (mshadow/cuda/tensor_gpu-inl.cuh:330-393),
 * which walks each row three times through global memory (20 bytes of traffic per element)
 * with 256 threads.  Here a CTA loads its row once into registers (up to 32 floats per
 * thread), finds the maximum, exponentiates and sums in registers, and writes the
 * normalised row once: 8 bytes per element, the algorithmic minimum.  Rows of more than 32768
 * columns are held in the registers of a thread-block cluster (up to 8 x 32768 columns); rows
 * beyond that are read once from HBM with a running (maximum, sum) pair per thread and a
 * second time from the L2 for the normalisation.
 *
 * The arithmetic follows the reference's CPU definition (mshadow/tensor_cpu-inl.h:270-285):
 * exp(x - max) with true division by the sum.  The sum is formed pairwise (registers, warp
 * shuffles, shared memory) instead of left to right, which changes results by rounding only.
 *
 * SoftmaxGrad and its smooth / ignore-label variants (reference kernels :239-328) are
 * element-wise copies with a per-row fix-up; they run as a 128-bit grid-stride sweep.
 */
#ifndef MSHADOW_GPU_SOFTMAX_CUH_
#define MSHADOW_GPU_SOFTMAX_CUH_

#include "./reduce.cuh"
#include "./tma.cuh"

namespace mshadow {
namespace cuda {

namespace smdetail {
struct MaxOp {
  __device__ __forceinline__ static void Reduce(float &a, float b) { a = a < b ? b : a; }  // NOLINT(*)
  __device__ __forceinline__ static void SetInitValue(float &a) { a = -FLT_MAX; }          // NOLINT(*)
};
struct SumOp {
  __device__ __forceinline__ static void Reduce(float &a, float b) { a = __fadd_rn(a, b); }  // NOLINT(*)
  __device__ __forceinline__ static void SetInitValue(float &a) { a = 0.0f; }                // NOLINT(*)
};

/*!
 * \brief v / s given r = 1/s (rounded): the product v*r refined by one fused correction step.
 *  Equals IEEE division except for rare last-bit cases, at two instructions per element instead
 *  of a division routine of twenty.
 */
__device__ __forceinline__ float DivByReciprocal(float v, float s, float r) {
  const float q0 = __fmul_rn(v, r);
  return __fmaf_rn(__fmaf_rn(-q0, s, v), r, q0);
}

/*! \brief value of a CTA-wide reduction, broadcast to every thread */
template <typename Op, int kThreads>
__device__ __forceinline__ float BlockAll(float v, float *buf) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) Op::Reduce(v, __shfl_xor_sync(0xffffffffu, v, d));
  if (kThreads == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // buf may still be read from a previous call
  if (lane == 0) buf[warp] = v;
  __syncthreads();
  float init;
  Op::SetInitValue(init);
  v = lane < kThreads / 32 ? buf[lane] : init;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) Op::Reduce(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
}  // namespace smdetail

/*!
 * \brief one CTA per row, row resident in registers.  Thread t owns items t, t+kThreads, ...
 *  (kItems of them), an item being kLanes adjacent floats.
 */
template <int kThreads, int kItems, int kLanes>
__global__ void __launch_bounds__(kThreads)
SoftmaxRowKernel(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols, int64_t ld_dst,
                 int64_t ld_src) {
  gpu_rt::GridDependencySync();
  __shared__ float buf[32];
  const uint32_t nitems = (cols + kLanes - 1) / kLanes;
  for (uint32_t y = blockIdx.x; y < rows; y += gridDim.x) {
    const float *in = src + y * ld_src;
    float *out = dst + y * ld_dst;
    float v[kItems][kLanes];
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        if (kLanes == 4) {
          const float4 p = __ldcs(reinterpret_cast<const float4 *>(in) + item);
          v[k][0] = p.x;
          v[k][1 % kLanes] = p.y;
          v[k][2 % kLanes] = p.z;
          v[k][3 % kLanes] = p.w;
        } else {
          v[k][0] = __ldcs(in + item);
        }
      } else {
#pragma unroll
        for (int l = 0; l < kLanes; ++l) v[k][l] = -FLT_MAX;
      }
    }
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < kItems; ++k)
#pragma unroll
      for (int l = 0; l < kLanes; ++l) m = m < v[k][l] ? v[k][l] : m;
    m = smdetail::BlockAll<smdetail::MaxOp, kThreads>(m, buf);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const bool in_row = threadIdx.x + k * kThreads < nitems;
#pragma unroll
      for (int l = 0; l < kLanes; ++l) {
        v[k][l] = in_row ? expf(__fsub_rn(v[k][l], m)) : 0.0f;
        s = __fadd_rn(s, v[k][l]);
      }
    }
    s = smdetail::BlockAll<smdetail::SumOp, kThreads>(s, buf);
    // fused gradient: subtract one at the label's column (label == nullptr: plain softmax)
    const int hot = label != nullptr ? static_cast<int>(label[y]) : -1;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        float q[kLanes];
#pragma unroll
        for (int l = 0; l < kLanes; ++l) {
          q[l] = __fdiv_rn(v[k][l], s);
          if (static_cast<int>(item * kLanes + l) == hot) q[l] = __fsub_rn(q[l], 1.0f);
        }
        if (kLanes == 4) {
          __stcs(reinterpret_cast<float4 *>(out) + item, make_float4(q[0], q[1 % kLanes], q[2 % kLanes], q[3 % kLanes]));
        } else {
          __stcs(out + item, q[0]);
        }
      }
    }
  }
}

/*!
 * \brief long rows: one persistent CTA of 1024 threads per SM.  While the CTA works on row y
 *  out of registers (max, exp, sum, normalise, store), a bulk asynchronous copy already
 *  brings row y + gridDim.x into shared memory, so the read of the next row overlaps the
 *  arithmetic and the write of the current one; with a whole row per CTA and the register
 *  file full, no second CTA could provide that overlap.  Dynamic shared memory: one row.
 *  The quotient v / s is formed as v * (1/s) with one fused correction step, which equals
 *  IEEE division except for rare last-bit cases.
 */
template <int kItems>
__global__ void __launch_bounds__(1024, 1)
SoftmaxStagedKernel(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols, int64_t ld_dst,
                    int64_t ld_src, int *status) {
  gpu_rt::GridDependencySync();
  constexpr int kThreads = 1024;
  extern __shared__ __align__(16) float4 staged_row[];
  __shared__ uint64_t bar;
  __shared__ float buf[32];
  const uint32_t nitems = cols >> 2;
  const uint32_t row_bytes = cols * 4u;
  uint32_t y = blockIdx.x;
  if (y >= rows) return;
  if (threadIdx.x == 0) {
    tma::BarrierInit(&bar, 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    tma::BarrierExpect(&bar, row_bytes);
    tma::BulkLoad(staged_row, src + y * ld_src, row_bytes, &bar);
  }
  uint32_t phase = 0;
  for (; y < rows; y += gridDim.x) {
    if (!tma::WaitBounded(&bar, phase)) {
      if (threadIdx.x == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
      tma::WaitBounded(&bar, phase);
      return;
    }
    phase ^= 1;
    // the row's label is fetched now, so that its round trip overlaps the two reductions
    const float hot_f = label != nullptr ? __ldg(label + y) : -1.0f;
    float v[kItems][4];
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        const float4 p = staged_row[item];
        v[k][0] = p.x;
        v[k][1] = p.y;
        v[k][2] = p.z;
        v[k][3] = p.w;
      } else {
        v[k][0] = v[k][1] = v[k][2] = v[k][3] = -FLT_MAX;
      }
    }
    __syncthreads();  // every thread holds its part of the row: the buffer may be refilled
    const uint32_t ynext = y + gridDim.x;
    if (threadIdx.x == 0 && ynext < rows) {
      tma::FenceAsyncShared();
      tma::BarrierExpect(&bar, row_bytes);
      tma::BulkLoad(staged_row, src + ynext * ld_src, row_bytes, &bar);
    }
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < kItems; ++k)
#pragma unroll
      for (int l = 0; l < 4; ++l) m = m < v[k][l] ? v[k][l] : m;
    m = smdetail::BlockAll<smdetail::MaxOp, kThreads>(m, buf);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const bool in_row = threadIdx.x + k * kThreads < nitems;
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        v[k][l] = in_row ? expf(__fsub_rn(v[k][l], m)) : 0.0f;
        s = __fadd_rn(s, v[k][l]);
      }
    }
    s = smdetail::BlockAll<smdetail::SumOp, kThreads>(s, buf);
    const float r = __frcp_rn(s);
    const int hot = label != nullptr ? static_cast<int>(hot_f) : -1;
    const int hot_item = hot >= 0 ? hot >> 2 : -1, hot_lane = hot & 3;
    float4 *out = reinterpret_cast<float4 *>(dst + y * ld_dst);
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        float q[4];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
          const float q0 = __fmul_rn(v[k][l], r);
          q[l] = __fmaf_rn(__fmaf_rn(-q0, s, v[k][l]), r, q0);
        }
        if (static_cast<int>(item) == hot_item) {  // one group per row holds the label's column
          q[0] = hot_lane == 0 ? __fsub_rn(q[0], 1.0f) : q[0];
          q[1] = hot_lane == 1 ? __fsub_rn(q[1], 1.0f) : q[1];
          q[2] = hot_lane == 2 ? __fsub_rn(q[2], 1.0f) : q[2];
          q[3] = hot_lane == 3 ? __fsub_rn(q[3], 1.0f) : q[3];
        }
        __stcs(out + item, make_float4(q[0], q[1], q[2], q[3]));
      }
    }
  }
}

/*!
 * \brief rows of up to 8 x 32768 columns: the row is resident in the registers of a thread-block
 *  CLUSTER.  grid.x = cluster size; CTA `rank` holds columns [rank * seg, (rank + 1) * seg), kItems
 *  16-byte items per thread.  The CTAs agree on the row maximum and on the sum through distributed
 *  shared memory (each publishes its value, all read all, in rank order), everything else is
 *  SoftmaxRowKernel: one read of the row from HBM, one exp per element, one write.
 *  A CTA loads, computes and stores in turn, so the launcher prefers 512-thread CTAs (two or
 *  three per SM, whose phases overlap) whenever a cluster of eight of them covers the row.
 */
template <int kThreads, int kItems>
__global__ void __launch_bounds__(kThreads)
SoftmaxClusterRowKernel(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols,
                        int64_t ld_dst, int64_t ld_src, uint32_t seg) {
  __shared__ float buf[32];
  // published values alternate between two places from row to row: a CTA may still be reading
  // row y's values when a faster one publishes row y + 1's, and by the time row y + 2 reuses the
  // place every CTA has passed a cluster barrier of row y + 1
  __shared__ float cta_max_buf[2], cta_sum_buf[2];
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned csize = cluster.num_blocks(), crank = cluster.block_rank();
  const uint32_t x0 = crank * seg;
  const uint32_t x1 = min(cols, x0 + seg);
  const uint32_t nitems = x1 > x0 ? (x1 - x0) / 4 : 0;  // cols and seg are multiples of 4
  uint32_t flip = 0;
  for (uint32_t y = blockIdx.y; y < rows; y += gridDim.y, flip ^= 1u) {
    float &cta_max = cta_max_buf[flip];
    float &cta_sum = cta_sum_buf[flip];
    const float4 *in = reinterpret_cast<const float4 *>(src + y * ld_src + x0);
    float4 *out = reinterpret_cast<float4 *>(dst + y * ld_dst + x0);
    float v[kItems][4];
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        const float4 p = __ldcs(in + item);
        v[k][0] = p.x, v[k][1] = p.y, v[k][2] = p.z, v[k][3] = p.w;
      } else {
        v[k][0] = v[k][1] = v[k][2] = v[k][3] = -FLT_MAX;
      }
    }
    float m = -FLT_MAX;
#pragma unroll
    for (int k = 0; k < kItems; ++k)
#pragma unroll
      for (int l = 0; l < 4; ++l) m = m < v[k][l] ? v[k][l] : m;
    m = smdetail::BlockAll<smdetail::MaxOp, kThreads>(m, buf);
    if (threadIdx.x == 0) cta_max = m;
    cluster.sync();
    for (unsigned r = 0; r < csize; ++r) {
      const float o = *cluster.map_shared_rank(&cta_max, r);
      m = m < o ? o : m;
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const bool in_row = threadIdx.x + k * kThreads < nitems;
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        v[k][l] = in_row ? expf(__fsub_rn(v[k][l], m)) : 0.0f;
        s = __fadd_rn(s, v[k][l]);
      }
    }
    s = smdetail::BlockAll<smdetail::SumOp, kThreads>(s, buf);
    if (threadIdx.x == 0) cta_sum = s;
    cluster.sync();
    s = *cluster.map_shared_rank(&cta_sum, 0);
    for (unsigned r = 1; r < csize; ++r) s = __fadd_rn(s, *cluster.map_shared_rank(&cta_sum, r));
    const int hot = label != nullptr ? static_cast<int>(label[y]) - static_cast<int>(x0) : -1;
    const float rcp = __frcp_rn(s);
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const uint32_t item = threadIdx.x + k * kThreads;
      if (item < nitems) {
        float q[4];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
          q[l] = smdetail::DivByReciprocal(v[k][l], s, rcp);
          if (static_cast<int>(item * 4 + l) == hot) q[l] = __fsub_rn(q[l], 1.0f);
        }
        __stcs(out + item, make_float4(q[0], q[1], q[2], q[3]));
      }
    }
  }
  cluster.sync();  // no CTA leaves while others may still read its shared memory
}

namespace smdetail {
/*! \brief running (maximum, sum of exp(x - maximum)) of a stream of values */
struct MaxSum {
  float m, s;
};
/*! \brief both streams as one: the sums are brought to the common maximum before they are added */
__device__ __forceinline__ MaxSum Merge(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = a.m < b.m ? b.m : a.m;
  r.s = __fadd_rn(__fmul_rn(a.s, expf(__fsub_rn(a.m, r.m))), __fmul_rn(b.s, expf(__fsub_rn(b.m, r.m))));
  return r;
}
}  // namespace smdetail

/*!
 * \brief rows of any length, in particular those beyond the register budget of the kernels
 *  above: ONE pass over HBM that keeps a running (maximum, sum) pair per thread -- when a new
 *  maximum appears the sum so far is rescaled by exp(old - new) -- followed by a second read of
 *  the row, which the L2 still holds (a row of 100 000 floats is 400 KB), to write
 *  exp(x - max) / sum.  DRAM traffic is therefore the 8 bytes per element of the register
 *  kernels, not the 20 of a max / exp-sum / normalise triple sweep.
 *  A row is shared by the CTAs of a thread-block cluster (grid.x = cluster size, each CTA takes
 *  a contiguous segment of the columns): few long rows would otherwise leave most SMs idle.
 *  The CTAs exchange their pairs through distributed shared memory and every CTA merges them in
 *  rank order, so all arrive at the same (max, sum).  exp(x - max) is evaluated with the row's
 *  true maximum, exactly as the CPU evaluator does (mshadow/tensor_cpu-inl.h:270-285); only the
 *  order of the additions in the sum differs.
 */
template <int kThreads, int kLanes>
__global__ void __launch_bounds__(kThreads)
SoftmaxOnlineKernel(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols, int64_t ld_dst,
                    int64_t ld_src, uint32_t seg) {
  __shared__ smdetail::MaxSum warp_pair[kThreads / 32];
  __shared__ smdetail::MaxSum cta_pair;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned csize = cluster.num_blocks(), crank = cluster.block_rank();
  const uint32_t x0 = crank * seg;
  const uint32_t x1 = min(cols, x0 + seg);
  for (uint32_t y = blockIdx.y; y < rows; y += gridDim.y) {
    const float *in = src + y * ld_src;
    float *out = dst + y * ld_dst;
    smdetail::MaxSum acc = {-FLT_MAX, 0.0f};
    constexpr int kDepth = 4;  // loads in flight per thread: 64 KB per CTA with 16-byte loads
    for (uint32_t xb = x0 + threadIdx.x * kLanes; xb < x1; xb += kThreads * kLanes * kDepth) {
      float v[kDepth][kLanes];
#pragma unroll
      for (int k = 0; k < kDepth; ++k) {
        const uint32_t x = xb + k * kThreads * kLanes;
        if (x < x1) {
          if (kLanes == 4) {
            const float4 p = __ldcg(reinterpret_cast<const float4 *>(in + x));  // the L2 keeps the row for the second read
            v[k][0] = p.x, v[k][1 % kLanes] = p.y, v[k][2 % kLanes] = p.z, v[k][3 % kLanes] = p.w;
          } else {
            v[k][0] = __ldcg(in + x);
          }
        } else {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) v[k][l] = -FLT_MAX;  // adds exp(-huge) = 0
        }
      }
      float top = v[0][0];
#pragma unroll
      for (int k = 0; k < kDepth; ++k)
#pragma unroll
        for (int l = 0; l < kLanes; ++l) top = top < v[k][l] ? v[k][l] : top;
      if (top > acc.m) {
        acc.s = __fmul_rn(acc.s, expf(__fsub_rn(acc.m, top)));
        acc.m = top;
      }
#pragma unroll
      for (int k = 0; k < kDepth; ++k)
#pragma unroll
        for (int l = 0; l < kLanes; ++l) acc.s = __fadd_rn(acc.s, expf(__fsub_rn(v[k][l], acc.m)));
    }
    // warp, CTA, cluster
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      smdetail::MaxSum o;
      o.m = __shfl_xor_sync(0xffffffffu, acc.m, d);
      o.s = __shfl_xor_sync(0xffffffffu, acc.s, d);
      // lower lane first, so that both partners compute the same bits
      acc = (threadIdx.x & d) ? smdetail::Merge(o, acc) : smdetail::Merge(acc, o);
    }
    if ((threadIdx.x & 31) == 0) warp_pair[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      smdetail::MaxSum t = warp_pair[0];
      for (int wi = 1; wi < kThreads / 32; ++wi) t = smdetail::Merge(t, warp_pair[wi]);
      cta_pair = t;
    }
    if (csize > 1) {
      cluster.sync();
    } else {
      __syncthreads();
    }
    smdetail::MaxSum row = *cluster.map_shared_rank(&cta_pair, 0);
    for (unsigned r = 1; r < csize; ++r) row = smdetail::Merge(row, *cluster.map_shared_rank(&cta_pair, r));
    if (csize > 1) {
      cluster.sync();  // every CTA has read the pairs before any of them is overwritten
    } else {
      __syncthreads();
    }
    const int hot = label != nullptr ? static_cast<int>(label[y]) : -1;
    const float rcp = __frcp_rn(row.s);
    for (uint32_t xb = x0 + threadIdx.x * kLanes; xb < x1; xb += kThreads * kLanes * kDepth) {
      float v[kDepth][kLanes];
#pragma unroll
      for (int k = 0; k < kDepth; ++k) {
        const uint32_t x = xb + k * kThreads * kLanes;
        if (x < x1) {
          if (kLanes == 4) {
            const float4 p = __ldcs(reinterpret_cast<const float4 *>(in + x));  // last use of the row
            v[k][0] = p.x, v[k][1 % kLanes] = p.y, v[k][2 % kLanes] = p.z, v[k][3 % kLanes] = p.w;
          } else {
            v[k][0] = __ldcs(in + x);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < kDepth; ++k) {
        const uint32_t x = xb + k * kThreads * kLanes;
        if (x < x1) {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) {
            const float q = smdetail::DivByReciprocal(expf(__fsub_rn(v[k][l], row.m)), row.s, rcp);
            v[k][l] = static_cast<int>(x + l) == hot ? __fsub_rn(q, 1.0f) : q;
          }
          if (kLanes == 4) {
            __stcs(reinterpret_cast<float4 *>(out + x),
                   make_float4(v[k][0], v[k][1 % kLanes], v[k][2 % kLanes], v[k][3 % kLanes]));
          } else {
            __stcs(out + x, v[k][0]);
          }
        }
      }
    }
  }
}

namespace smdetail {
template <int kThreads, int kItems, int kLanes>
inline void LaunchRow(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols, int64_t ld_dst,
                      int64_t ld_src, cudaStream_t stream) {
  // persistent over rows only when there are more rows than a generous grid
  const uint32_t cap = static_cast<uint32_t>(gpu_rt::CurrentDevice().sm_count) * 64u;
  const uint32_t grid = rows < cap ? rows : cap;
  gpu_rt::LaunchAfterDrain(SoftmaxRowKernel<kThreads, kItems, kLanes>, dim3(grid), dim3(kThreads), 0, stream, dst, src,
                           label, rows, cols, ld_dst, ld_src);
}
}  // namespace smdetail

/*!
 * \brief dst = softmax(src) row by row, fp32.  With `label` (one float per row holding a column
 *  index) the gradient of the cross-entropy loss is produced in the same pass instead:
 *  dst = softmax(src) - onehot(label), i.e. SoftmaxGrad(Softmax(src)) without writing and
 *  re-reading the probabilities.
 */
inline void SoftmaxLaunch(float *dst, const float *src, int64_t rows, int64_t cols, int64_t ld_dst, int64_t ld_src,
                          cudaStream_t stream, const float *label = nullptr) {
  if (rows == 0 || cols == 0) return;
  CHECK_LT(rows, (int64_t(1) << 31));
  CHECK_LT(cols, (int64_t(1) << 31));
  const uint32_t r = static_cast<uint32_t>(rows), c = static_cast<uint32_t>(cols);
  const bool vec = cols % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0 && (rows == 1 || (ld_dst % 4 == 0 && ld_src % 4 == 0));
  using smdetail::LaunchRow;
  const int sms = gpu_rt::CurrentDevice().sm_count;
  if (vec && cols >= 4096 && cols <= 32768 && rows >= sms) {
    // long rows, enough of them to keep one persistent CTA per SM busy
    const uint32_t n = c / 4;
    const size_t smem = static_cast<size_t>(c) * 4;
    int *status = gpu_rt::StatusWord();
#define MSHADOW_B200_SOFTMAX_STAGED_(ITEMS)                                                                       \
  {                                                                                                               \
    auto kernel = SoftmaxStagedKernel<ITEMS>;                                                                     \
    MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));     \
    gpu_rt::LaunchAfterDrain(kernel, dim3(sms), dim3(1024), smem, stream, dst, src, label, r, c, ld_dst, ld_src, status); \
  }
    if (n <= 1024) MSHADOW_B200_SOFTMAX_STAGED_(1)
    else if (n <= 2048) MSHADOW_B200_SOFTMAX_STAGED_(2)
    else if (n <= 4096) MSHADOW_B200_SOFTMAX_STAGED_(4)
    else MSHADOW_B200_SOFTMAX_STAGED_(8)
#undef MSHADOW_B200_SOFTMAX_STAGED_
  } else if (vec && cols <= 32768) {
    const uint32_t n = c / 4;  // 16-byte items per row
    if (n <= 32) LaunchRow<32, 1, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 128) LaunchRow<128, 1, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 256) LaunchRow<256, 1, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 512) LaunchRow<256, 2, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 1024) LaunchRow<256, 4, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 2048) LaunchRow<512, 4, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (n <= 4096) LaunchRow<1024, 4, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else LaunchRow<1024, 8, 4>(dst, src, label, r, c, ld_dst, ld_src, stream);
  } else if (cols <= 8192) {
    if (c <= 32) LaunchRow<32, 1, 1>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (c <= 128) LaunchRow<128, 1, 1>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (c <= 512) LaunchRow<256, 2, 1>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else if (c <= 2048) LaunchRow<256, 8, 1>(dst, src, label, r, c, ld_dst, ld_src, stream);
    else LaunchRow<512, 16, 1>(dst, src, label, r, c, ld_dst, ld_src, stream);
  } else if (vec && cols <= 8 * 32768) {
    // the row lives in the registers of a cluster of 2, 4 or 8 CTAs
    const bool narrow = c <= 8 * 16384;  // eight CTAs of 512 threads x 8 items x 4 floats hold the row
    const uint32_t threads = narrow ? 512 : 1024;
    const uint32_t per_cta = threads * 32;
    uint32_t csize = 2;
    while (csize < 8 && static_cast<uint64_t>(csize) * per_cta < c) csize *= 2;
    // few rows: more CTAs per row keep more SMs busy
    while (csize < 8 && static_cast<uint64_t>(r) * csize < static_cast<uint64_t>(sms) && c / (csize * 2) >= 4096) csize *= 2;
    uint32_t seg = ((c + csize - 1) / csize + 3) & ~3u;
    const uint32_t items = (seg / 4 + threads - 1) / threads;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, r < 65535u ? r : 65535u);
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define MSHADOW_B200_SOFTMAX_CLUSTER_(ITEMS)                                                                      \
  {                                                                                                               \
    if (narrow) {                                                                                                 \
      MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, SoftmaxClusterRowKernel<512, ITEMS>, dst, src, label, r, c,      \
                                           ld_dst, ld_src, seg));                                                 \
    } else {                                                                                                      \
      MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, SoftmaxClusterRowKernel<1024, ITEMS>, dst, src, label, r, c,     \
                                           ld_dst, ld_src, seg));                                                 \
    }                                                                                                             \
  }
    if (items <= 1) MSHADOW_B200_SOFTMAX_CLUSTER_(1)
    else if (items <= 2) MSHADOW_B200_SOFTMAX_CLUSTER_(2)
    else if (items <= 4) MSHADOW_B200_SOFTMAX_CLUSTER_(4)
    else MSHADOW_B200_SOFTMAX_CLUSTER_(8)
#undef MSHADOW_B200_SOFTMAX_CLUSTER_
  } else {
    // longer (or unaligned) rows: one pass with a running (max, sum), rows split over clusters
    // A row goes to a cluster of 1, 2, 4 or 8 CTAs: more while there are fewer CTAs than SMs, and
    // more while the rows in flight at once (about two CTAs per SM) would not fit the L2 together,
    // because the second read of a row is meant to come from there.
    uint32_t csize = 1;
    const uint64_t l2_share = static_cast<uint64_t>(gpu_rt::CurrentDevice().l2_bytes) * 3 / 4;
    while (csize < 8 && c / (csize * 2) >= 4096) {
      const bool few_ctas = static_cast<uint64_t>(r) * csize < static_cast<uint64_t>(sms);
      const uint64_t rows_in_flight = static_cast<uint64_t>(sms) * 2 / csize < r ? static_cast<uint64_t>(sms) * 2 / csize : r;
      const bool spills = rows_in_flight * c * 4 > l2_share;
      if (!few_ctas && !spills) break;
      csize *= 2;
    }
    const uint32_t lanes = vec ? 4 : 1;
    uint32_t seg = (c + csize - 1) / csize;
    seg = (seg + 3) & ~3u;  // segments start on 16-byte boundaries
    const uint32_t row_grid = r < 65535u ? r : 65535u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, row_grid);
    cfg.blockDim = dim3(1024);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (lanes == 4) {
      MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, SoftmaxOnlineKernel<1024, 4>, dst, src, label, r, c, ld_dst, ld_src, seg));
    } else {
      MSHADOW_CUDA_CALL(cudaLaunchKernelEx(&cfg, SoftmaxOnlineKernel<1024, 1>, dst, src, label, r, c, ld_dst, ld_src, seg));
    }
  }
  MSHADOW_CUDA_POST_KERNEL_CHECK(Softmax);
}

/*!
 * \brief dst = src - onehot(label) with optional label smoothing (mode bit 0) and row
 *  zeroing for ignored labels (mode bit 1); arithmetic as mshadow/tensor_cpu-inl.h:287-368.
 */
template <int kLanes>
__global__ void __launch_bounds__(256)
SoftmaxGradKernel(float *dst, const float *src, const float *label, uint32_t rows, uint32_t cols,
                  uint32_t items_per_row, gpu_rt::FastDiv row_of_item, int64_t ld_dst, int64_t ld_src, int mode,
                  int ignore_label, float alpha, float smooth_grad) {
  gpu_rt::GridDependencySync();
  const uint32_t total = rows * items_per_row;
  const uint32_t step = gridDim.x * 256;
  constexpr int kUnroll = MSHADOW_B200_SMGRAD_UNROLL;
  for (uint32_t base = blockIdx.x * 256 + threadIdx.x; base < total; base += step * kUnroll) {
    float v[kUnroll][kLanes];
    int kk[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * step;
      if (i < total) {
        const uint32_t y = row_of_item.Quot(i);
        const uint32_t x = (i - y * items_per_row) * kLanes;
        const int k = static_cast<int>(label[y]);
        kk[u] = k;
        const bool zero_row = (mode & 2) && k == ignore_label;
        if (zero_row) {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) v[u][l] = 0.0f;
        } else if (kLanes == 4) {
          const float4 p = __ldcs(reinterpret_cast<const float4 *>(src + y * ld_src + x));
          v[u][0] = p.x;
          v[u][1 % kLanes] = p.y;
          v[u][2 % kLanes] = p.z;
          v[u][3 % kLanes] = p.w;
        } else {
          v[u][0] = __ldcs(src + y * ld_src + x);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t i = base + u * step;
      if (i < total) {
        const uint32_t y = row_of_item.Quot(i);
        const uint32_t x = (i - y * items_per_row) * kLanes;
        const bool zero_row = (mode & 2) && kk[u] == ignore_label;
        if (!zero_row) {
#pragma unroll
          for (int l = 0; l < kLanes; ++l) {
            const bool hit = static_cast<int>(x) + l == kk[u];
            if (mode & 1) {
              v[u][l] = hit ? __fadd_rn(__fsub_rn(v[u][l], 1.0f), alpha) : __fsub_rn(v[u][l], smooth_grad);
            } else if (hit) {
              v[u][l] = __fsub_rn(v[u][l], 1.0f);
            }
          }
        }
        if (kLanes == 4) {
          float4 p;
          p.x = v[u][0];
          p.y = v[u][1 % kLanes];
          p.z = v[u][2 % kLanes];
          p.w = v[u][3 % kLanes];
          __stcs(reinterpret_cast<float4 *>(dst + y * ld_dst + x), p);
        } else {
          __stcs(dst + y * ld_dst + x, v[u][0]);
        }
      }
    }
  }
}

inline void SoftmaxGradLaunch(float *dst, const float *src, const float *label, int64_t rows, int64_t cols,
                              int64_t ld_dst, int64_t ld_src, int mode, float ignore_label, float alpha,
                              cudaStream_t stream) {
  if (rows == 0 || cols == 0) return;
  CHECK_LT(rows * cols, (int64_t(1) << 31)) << "SoftmaxGrad: tensor too large for 32-bit indexing";
  const float smooth_grad = alpha / static_cast<float>(static_cast<index_t>(cols) - 1);
  const bool vec = cols % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0 && (rows == 1 || (ld_dst % 4 == 0 && ld_src % 4 == 0));
  const uint32_t r = static_cast<uint32_t>(rows), c = static_cast<uint32_t>(cols);
  const uint32_t ipr = vec ? c / 4 : c;
  const int64_t work = static_cast<int64_t>(r) * ipr;
  int grid = gpu_rt::CeilDiv(work, 256 * MSHADOW_B200_SMGRAD_UNROLL);
  const int cap = gpu_rt::CurrentDevice().sm_count * 8;
  if (grid > cap) grid = cap;
  if (vec) {
    // (launched the ordinary way: placed on the SMs while the previous kernel drains, this kernel was
    // measured 2.3 % slower back to back -- 1.290 against 1.259 ms on 32768 x 32000 -- while the map and
    // pooling kernels gain 2 - 7 % from gpu_rt::LaunchAfterDrain)
    SoftmaxGradKernel<4><<<grid, 256, 0, stream>>>(dst, src, label, r, c, ipr, gpu_rt::FastDiv(ipr), ld_dst, ld_src,
                                                  mode, static_cast<int>(ignore_label), alpha, smooth_grad);
  } else {
    SoftmaxGradKernel<1><<<grid, 256, 0, stream>>>(dst, src, label, r, c, ipr, gpu_rt::FastDiv(ipr), ld_dst, ld_src,
                                                  mode, static_cast<int>(ignore_label), alpha, smooth_grad);
  }
  MSHADOW_CUDA_POST_KERNEL_CHECK(SoftmaxGrad);
}

// ----------------------------------------------------------------------------------------
// (batch, classes, positions) tensors: softmax over the middle axis.  Element (y, x, n) lives
// at (y * classes + x) * ld + n, so the classes of one position are `ld` floats apart and
// neighbouring threads take neighbouring positions.
// ----------------------------------------------------------------------------------------

const int kSoftmax3DThreads = MSHADOW_B200_SM3D_THREADS;
constexpr int kSoftmax3DDepth = MSHADOW_B200_SM3D_DEPTH;

/*!
 * \brief one CTA = one image y and a tile of kThreads * kLanes positions; thread t owns kLanes
 *  adjacent positions and walks the classes.  With kStaged the tile (classes x positions) is
 *  parked in shared memory between the three passes, so global memory sees one read and one
 *  write per element; without it (more classes than shared memory holds) the exponentials are
 *  parked in dst and read back, mostly from L2.  Each column is summed by one thread in class
 *  order, as mshadow/tensor_cpu-inl.h:474-495 does.
 */
template <int kLanes, bool kStaged, bool kBulk = false>
__global__ void __launch_bounds__(kSoftmax3DThreads)
Softmax3DKernel(float *dst, const float *src, uint32_t classes, uint32_t npos, uint32_t tiles, int64_t ld_dst,
                int64_t ld_src, int *status) {
  extern __shared__ __align__(16) float tile[];  // [classes][kThreads * kLanes]
  constexpr int kWidth = kSoftmax3DThreads * kLanes;
  const uint32_t y = blockIdx.x / tiles;
  const uint32_t n0 = (blockIdx.x - y * tiles) * kWidth;
  const uint32_t n = n0 + threadIdx.x * kLanes;
  // kBulk (16-byte aligned rows, four positions per thread): a tile that lies wholly inside the
  // position axis is brought in by one bulk asynchronous copy per class row (kWidth contiguous
  // floats each), all of them in flight at once on one barrier, instead of kSoftmax3DDepth loads
  // per thread: 43 KB per CTA against 8 KB for 21 classes (0.77 -> see the launch site).
  bool from_tile = false;
  if (kBulk && kStaged && kLanes == 4) {
    __shared__ uint64_t landed;
    if (n0 + kWidth <= npos) {   // the same for all threads of the CTA
      if (threadIdx.x == 0) tma::BarrierInit(&landed, 1);
      __syncthreads();
      if (threadIdx.x == 0) {
        tma::BarrierExpect(&landed, classes * static_cast<uint32_t>(kWidth) * 4u);
        const float *row = src + static_cast<int64_t>(y) * classes * ld_src + n0;
        for (uint32_t x = 0; x < classes; ++x)
          tma::BulkLoad(tile + static_cast<size_t>(x) * kWidth, row + x * ld_src, kWidth * 4u, &landed);
      }
      if (!tma::WaitBounded(&landed, 0u)) {
        if ((threadIdx.x & 31) == 0) atomicExch(status, tma::kStatusBulkCopyTimeout);
        return;
      }
      from_tile = true;
    }
  }
  if (n >= npos) return;  // no CTA-wide barrier below: every thread works on its own columns
  const float *in = src + static_cast<int64_t>(y) * classes * ld_src + n;
  float *out = dst + static_cast<int64_t>(y) * classes * ld_dst + n;
  float *mine = tile + threadIdx.x * kLanes;
  float m[kLanes], s[kLanes];
#pragma unroll
  for (int l = 0; l < kLanes; ++l) m[l] = -FLT_MAX, s[l] = 0.0f;
  if (from_tile) {
#pragma unroll 4
    for (uint32_t x = 0; x < classes; ++x) {
      const float4 p = *reinterpret_cast<const float4 *>(mine + x * kWidth);
      const float v[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int l = 0; l < kLanes; ++l) m[l] = m[l] < v[l % 4] ? v[l % 4] : m[l];
    }
  }
#pragma unroll kSoftmax3DDepth
  for (uint32_t x = from_tile ? classes : 0; x < classes; ++x) {
    float v[kLanes];
    if (kLanes == 4) {
      const float4 p = __ldcs(reinterpret_cast<const float4 *>(in + x * ld_src));
      v[0] = p.x, v[1 % kLanes] = p.y, v[2 % kLanes] = p.z, v[3 % kLanes] = p.w;
      if (kStaged) *reinterpret_cast<float4 *>(mine + x * kWidth) = p;
    } else {
      v[0] = __ldcs(in + x * ld_src);
      if (kStaged) mine[x * kWidth] = v[0];
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) m[l] = m[l] < v[l] ? v[l] : m[l];
  }
#pragma unroll 4
  for (uint32_t x = 0; x < classes; ++x) {
    float v[kLanes];
    if (kLanes == 4) {
      const float4 p = kStaged ? *reinterpret_cast<const float4 *>(mine + x * kWidth)
                               : __ldcg(reinterpret_cast<const float4 *>(in + x * ld_src));
      v[0] = p.x, v[1 % kLanes] = p.y, v[2 % kLanes] = p.z, v[3 % kLanes] = p.w;
    } else {
      v[0] = kStaged ? mine[x * kWidth] : __ldcg(in + x * ld_src);
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      v[l] = expf(__fsub_rn(v[l], m[l]));
      s[l] = __fadd_rn(s[l], v[l]);
    }
    if (kLanes == 4) {
      const float4 p = make_float4(v[0], v[1 % kLanes], v[2 % kLanes], v[3 % kLanes]);
      if (kStaged) *reinterpret_cast<float4 *>(mine + x * kWidth) = p;
      else *reinterpret_cast<float4 *>(out + x * ld_dst) = p;
    } else {
      if (kStaged) mine[x * kWidth] = v[0];
      else out[x * ld_dst] = v[0];
    }
  }
  float r[kLanes];
#pragma unroll
  for (int l = 0; l < kLanes; ++l) r[l] = __frcp_rn(s[l]);
#pragma unroll 4
  for (uint32_t x = 0; x < classes; ++x) {
    if (kLanes == 4) {
      float4 p = kStaged ? *reinterpret_cast<const float4 *>(mine + x * kWidth)
                         : *reinterpret_cast<const float4 *>(out + x * ld_dst);
      p.x = smdetail::DivByReciprocal(p.x, s[0], r[0]);
      p.y = smdetail::DivByReciprocal(p.y, s[1 % kLanes], r[1 % kLanes]);
      p.z = smdetail::DivByReciprocal(p.z, s[2 % kLanes], r[2 % kLanes]);
      p.w = smdetail::DivByReciprocal(p.w, s[3 % kLanes], r[3 % kLanes]);
      __stcs(reinterpret_cast<float4 *>(out + x * ld_dst), p);
    } else {
      const float e = kStaged ? mine[x * kWidth] : out[x * ld_dst];
      __stcs(out + x * ld_dst, smdetail::DivByReciprocal(e, s[0], r[0]));
    }
  }
}

namespace smdetail {
template <int kLanes>
inline void LaunchSoftmax3D(float *dst, const float *src, uint32_t batch, uint32_t classes, uint32_t npos,
                            int64_t ld_dst, int64_t ld_src, cudaStream_t stream) {
  const uint32_t width = kSoftmax3DThreads * kLanes;
  const uint32_t tiles = (npos + width - 1) / width;
  const size_t smem = static_cast<size_t>(classes) * width * sizeof(float);
  const size_t limit = static_cast<size_t>(gpu_rt::CurrentDevice().max_smem_optin);
  const int64_t ctas = static_cast<int64_t>(batch) * tiles;
  CHECK_LT(ctas, (int64_t(1) << 31)) << "Softmax: too many tiles for one launch";
  int *status = gpu_rt::StatusWord();
  if (smem + 64 <= limit) {  // (the bulk variant has a few bytes of static shared memory beside the tile)
    // bulk-copy staging where the class rows of a tile are 16-byte aligned pieces of at most 1 MB in all
    const bool bulk = kLanes == 4 && ld_src % 4 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                      smem < (size_t(1) << 20) && npos >= width;
    auto kernel = bulk ? Softmax3DKernel<kLanes, true, true> : Softmax3DKernel<kLanes, true, false>;
    if (smem > 48 * 1024) {
      MSHADOW_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(limit - 64)));
    }
    kernel<<<static_cast<unsigned>(ctas), kSoftmax3DThreads, smem, stream>>>(dst, src, classes, npos, tiles, ld_dst,
                                                                            ld_src, status);
  } else {
    Softmax3DKernel<kLanes, false><<<static_cast<unsigned>(ctas), kSoftmax3DThreads, 0, stream>>>(
        dst, src, classes, npos, tiles, ld_dst, ld_src, status);
  }
  MSHADOW_CUDA_POST_KERNEL_CHECK(Softmax3D);
}
}  // namespace smdetail

/*! \brief softmax over the middle axis; dst may alias src */
inline void Softmax3DLaunch(float *dst, const float *src, int64_t batch, int64_t classes, int64_t npos,
                            int64_t ld_dst, int64_t ld_src, cudaStream_t stream) {
  if (batch == 0 || classes == 0 || npos == 0) return;
  CHECK_LT(batch * classes * std::max(ld_dst, ld_src), (int64_t(1) << 40)) << "Softmax: tensor too large";
  const uint32_t b = static_cast<uint32_t>(batch), c = static_cast<uint32_t>(classes), p = static_cast<uint32_t>(npos);
  const bool vec = npos % 4 == 0 && ld_dst % 4 == 0 && ld_src % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0;
  // narrow position axes keep one position per thread so that a tile is not mostly idle threads;
  // the same when only the one-lane tile of all classes fits shared memory
  const size_t limit = static_cast<size_t>(gpu_rt::CurrentDevice().max_smem_optin);
  const bool wide_fits = static_cast<size_t>(classes) * kSoftmax3DThreads * 4 * sizeof(float) + 64 <= limit;
  const bool narrow_fits = static_cast<size_t>(classes) * kSoftmax3DThreads * sizeof(float) + 64 <= limit;
  if (vec && npos >= 4 * kSoftmax3DThreads && (wide_fits || !narrow_fits)) {
    smdetail::LaunchSoftmax3D<4>(dst, src, b, c, p, ld_dst, ld_src, stream);
  } else {
    smdetail::LaunchSoftmax3D<1>(dst, src, b, c, p, ld_dst, ld_src, stream);
  }
}

/*!
 * \brief dst(y,x,n) = src(y,x,n) - [x == label(y,n)], with the smoothing / ignore-label modes
 *  of SoftmaxGradKernel; arithmetic as mshadow/tensor_cpu-inl.h:370-462
 */
template <int kLanes>
__global__ void __launch_bounds__(256)
SoftmaxGrad3DKernel(float *dst, const float *src, const float *label, uint32_t total, uint32_t items_per_row,
                    gpu_rt::FastDiv row_of_item, gpu_rt::FastDiv image_of_row, int64_t ld_dst, int64_t ld_src,
                    int64_t ld_label, int mode, int ignore_label, float alpha, float smooth_grad) {
  const uint32_t step = gridDim.x * 256;
  for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
    const uint32_t row = row_of_item.Quot(i);  // row = y * classes + x
    const uint32_t n = (i - row * items_per_row) * kLanes;
    const uint32_t y = image_of_row.Quot(row);
    const int x = static_cast<int>(row - y * image_of_row.div);
    int k[kLanes];
    float v[kLanes];
#pragma unroll
    for (int l = 0; l < kLanes; ++l) v[l] = 0.0f;
    // without an ignore label every position is live: the source is requested before the labels, so
    // that the two round trips overlap instead of following one another
    const bool may_skip = (mode & 2) != 0;
    if (!may_skip) {
      if (kLanes == 4) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(src + row * ld_src + n));
        v[0] = p.x, v[1 % kLanes] = p.y, v[2 % kLanes] = p.z, v[3 % kLanes] = p.w;
      } else {
        v[0] = __ldcs(src + row * ld_src + n);
      }
    }
    bool any_live = false;
    if (kLanes == 4 && ld_label % 4 == 0 && reinterpret_cast<uintptr_t>(label) % 16 == 0) {
      const float4 q = __ldg(reinterpret_cast<const float4 *>(label + y * ld_label + n));
      k[0] = static_cast<int>(q.x), k[1 % kLanes] = static_cast<int>(q.y), k[2 % kLanes] = static_cast<int>(q.z),
      k[3 % kLanes] = static_cast<int>(q.w);
    } else {
#pragma unroll
      for (int l = 0; l < kLanes; ++l) k[l] = static_cast<int>(__ldg(label + y * ld_label + n + l));
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) any_live |= !(may_skip && k[l] == ignore_label);
    if (any_live && may_skip) {
      if (kLanes == 4) {
        const float4 p = __ldcs(reinterpret_cast<const float4 *>(src + row * ld_src + n));
        v[0] = p.x, v[1 % kLanes] = p.y, v[2 % kLanes] = p.z, v[3 % kLanes] = p.w;
      } else {
        v[0] = __ldcs(src + row * ld_src + n);
      }
    }
#pragma unroll
    for (int l = 0; l < kLanes; ++l) {
      if ((mode & 2) && k[l] == ignore_label) {
        v[l] = 0.0f;
      } else if (mode & 1) {
        v[l] = x == k[l] ? __fadd_rn(__fsub_rn(v[l], 1.0f), alpha) : __fsub_rn(v[l], smooth_grad);
      } else if (x == k[l]) {
        v[l] = __fsub_rn(v[l], 1.0f);
      }
    }
    if (kLanes == 4) {
      __stcs(reinterpret_cast<float4 *>(dst + row * ld_dst + n),
             make_float4(v[0], v[1 % kLanes], v[2 % kLanes], v[3 % kLanes]));
    } else {
      __stcs(dst + row * ld_dst + n, v[0]);
    }
  }
}

inline void SoftmaxGrad3DLaunch(float *dst, const float *src, const float *label, int64_t batch, int64_t classes,
                                int64_t npos, int64_t ld_dst, int64_t ld_src, int64_t ld_label, int mode,
                                float ignore_label, float alpha, cudaStream_t stream) {
  if (batch == 0 || classes == 0 || npos == 0) return;
  CHECK_LT(batch * classes * npos, (int64_t(1) << 31)) << "SoftmaxGrad: tensor too large for 32-bit indexing";
  const float smooth_grad = alpha / static_cast<float>(static_cast<index_t>(classes) - 1);
  const bool vec = npos % 4 == 0 && ld_dst % 4 == 0 && ld_src % 4 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(src) % 16 == 0;
  const uint32_t rows = static_cast<uint32_t>(batch * classes);
  const uint32_t ipr = static_cast<uint32_t>(vec ? npos / 4 : npos);
  const uint32_t total = rows * ipr;
  int grid = gpu_rt::CeilDiv(total, 256);
  const int cap = gpu_rt::CurrentDevice().sm_count * 8;
  if (grid > cap) grid = cap;
  const gpu_rt::FastDiv by_items(ipr), by_classes(static_cast<uint32_t>(classes));
  if (vec) {
    SoftmaxGrad3DKernel<4><<<grid, 256, 0, stream>>>(dst, src, label, total, ipr, by_items, by_classes, ld_dst, ld_src,
                                                    ld_label, mode, static_cast<int>(ignore_label), alpha, smooth_grad);
  } else {
    SoftmaxGrad3DKernel<1><<<grid, 256, 0, stream>>>(dst, src, label, total, ipr, by_items, by_classes, ld_dst, ld_src,
                                                    ld_label, mode, static_cast<int>(ignore_label), alpha, smooth_grad);
  }
  MSHADOW_CUDA_POST_KERNEL_CHECK(SoftmaxGrad3D);
}

}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_SOFTMAX_CUH_
