/*
 * Stable radix sort of (key, value) pairs of 4-byte types, least significant digit first.
 *
 * It takes the place of the thrust::stable_sort_by_key call behind the reference's GPU SortByKey
 * (mshadow/cuda/tensor_gpu-inl.cuh:784-806; CPU definition: mshadow/tensor_cpu-inl.h:531-560,
 * std::stable_sort on the keys with the values carried along) and of the sort inside AddTakeGrad.
 * What the callers of this engine need from a sort is narrow, and the kernels are built for it:
 *
 *   - only as many key bits are sorted as the caller says matter: the indices of an embedding
 *     table with K rows have ceil(log2 K) of them, which is two passes of at most nine bits
 *     instead of the four 8-bit passes of a full 32-bit sort;
 *   - the number of passes is even, so that the result lands in the caller's arrays without a
 *     copy back;
 *   - the first pass can produce its input on the fly: keys clipped to [0, K) from the raw index
 *     array and values 0, 1, 2, ... (what AddTakeGrad starts from), so that no clip / iota kernel
 *     and no extra 8 bytes per entry are needed;
 *   - keys compare as the CPU's operator< does: signed integers by value, floats by value with
 *     -0 == +0 (a bit-pattern sort would put -0 first and break the stable order of ties).
 *
 * A pass is three launches: per-tile digit counts, a scan with one warp per digit, the stable scatter.  Order
 * inside a tile is (warp, round, lane), ranks inside a round come from __match_any_sync, so equal
 * digits keep their order and the whole sort is stable.  All of it is integer work on a few
 * megabytes; for a million pairs the passes cost a few microseconds each and launch latency is
 * what is left.
 */
#ifndef MSHADOW_GPU_RADIX_SORT_CUH_
#define MSHADOW_GPU_RADIX_SORT_CUH_

#include <type_traits>

#include "./runtime.h"

namespace mshadow {
namespace cuda {
namespace sortdetail {

const int kThreads = 512;            // 16 warps
const int kItems = 8;                // rounds per warp: a tile is 512 * 8 = 4096 elements
const uint32_t kTile = kThreads * kItems;
const int kMaxDigitBits = 9;

/*! \brief how the first pass obtains its input */
struct Source {
  int clip_rows;  // > 0: keys are raw indices to be clipped to [0, clip_rows), values are 0, 1, 2, ...
};

/*! \brief 32 bits whose unsigned order is the key order (ascending), or its reverse */
template <typename K>
__device__ __forceinline__ uint32_t OrderedBits(K key, bool ascend) {
  static_assert(sizeof(K) == 4, "4-byte keys");
  uint32_t b;
  memcpy(&b, &key, 4);
  if (std::is_floating_point<K>::value) {
    if (b == 0x80000000u) b = 0u;  // -0 and +0 are equal keys
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  } else if (std::is_signed<K>::value) {
    b ^= 0x80000000u;
  }
  return ascend ? b : ~b;
}

template <typename K>
__device__ __forceinline__ K LoadKey(const K *keys, uint32_t i, const Source &src) {
  K k = keys[i];
  if (src.clip_rows > 0) {
    int32_t j;
    memcpy(&j, &k, 4);
    j = j <= 0 ? 0 : (j >= src.clip_rows ? src.clip_rows - 1 : j);
    memcpy(&k, &j, 4);
  }
  return k;
}

/*! \brief counts[d * tiles + tile] = number of elements of the tile whose digit is d */
template <typename K>
__global__ void __launch_bounds__(kThreads)
RadixCountKernel(const K *keys, uint32_t n, int shift, uint32_t mask, bool ascend, Source src, uint32_t *counts,
                 uint32_t tiles) {
  gpu_rt::GridDependencySync();
  extern __shared__ uint32_t hist[];
  for (uint32_t d = threadIdx.x; d <= mask; d += kThreads) hist[d] = 0;
  __syncthreads();
  const uint32_t base = blockIdx.x * kTile;
  const uint32_t lane = threadIdx.x & 31;
  uint32_t digit[kItems];
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const uint32_t i = base + r * kThreads + threadIdx.x;
    digit[r] = i < n ? (OrderedBits(LoadKey(keys, i, src), ascend) >> shift) & mask : mask + 1;
  }
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    // one atomic per distinct digit of the warp: sorted or skewed keys put whole warps on one bin
    const uint32_t peers = __match_any_sync(0xffffffffu, digit[r]);
    if (digit[r] <= mask && (peers & ((1u << lane) - 1u)) == 0) atomicAdd(&hist[digit[r]], __popc(peers));
  }
  __syncthreads();
  for (uint32_t d = threadIdx.x; d <= mask; d += kThreads) counts[d * tiles + blockIdx.x] = hist[d];
}

/*!
 * \brief counts[d][tile] becomes the number of elements with digit d in earlier tiles, total[d]
 *  the number of elements with digit d.  One warp per digit (grid = digits / 8 CTAs of 8 warps); a
 *  warp takes the digit's tiles 256 at a time: eight independent coalesced loads per lane first,
 *  then the warp scans, so that the kernel costs a few memory round trips, not one per tile.
 */
template <int kWarps>  // a template only so that the header can be included from several translation units
__global__ void __launch_bounds__(kWarps * 32) RadixScanKernel(uint32_t *counts, uint32_t *total, uint32_t digits,
                                                                uint32_t tiles) {
  gpu_rt::GridDependencySync();
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t d = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (d >= digits) return;
  uint32_t *row = counts + static_cast<size_t>(d) * tiles;
  uint32_t carry = 0;
  for (uint32_t t0 = 0; t0 < tiles; t0 += 256) {
    uint32_t c[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t t = t0 + k * 32 + lane;
      c[k] = t < tiles ? row[t] : 0u;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint32_t incl = c[k];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= static_cast<uint32_t>(o)) incl += up;
      }
      const uint32_t t = t0 + k * 32 + lane;
      if (t < tiles) row[t] = carry + incl - c[k];
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (lane == 0) total[d] = carry;
}

/*!
 * \brief stable scatter of one tile.  Warp w owns rounds of 32 consecutive elements; an
 *  element's place is digit_base[d] + counts[d][tile] + (elements with digit d earlier in the tile).
 */
template <typename K, typename V>
__global__ void __launch_bounds__(kThreads)
RadixScatterKernel(const K *keys_in, const V *vals_in, K *keys_out, V *vals_out, uint32_t n, int shift, uint32_t mask,
                   bool ascend, Source src, const uint32_t *counts, const uint32_t *total, uint32_t tiles) {
  gpu_rt::GridDependencySync();
  extern __shared__ uint32_t warp_count[];  // [16][digits], then digit_base[digits]
  __shared__ uint32_t warp_sum[16];
  const uint32_t digits = mask + 1;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t *digit_base = warp_count + 16 * digits;
  for (uint32_t i = threadIdx.x; i < 16 * digits; i += kThreads) warp_count[i] = 0;
  {
    // digit_base[d] = number of elements with a smaller digit: exclusive scan of the digit totals
    // (at most 512, one per thread)
    const uint32_t mine_total = threadIdx.x < digits ? total[threadIdx.x] : 0u;
    uint32_t incl = mine_total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= static_cast<uint32_t>(o)) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    uint32_t before = 0;
    for (uint32_t w = 0; w < warp; ++w) before += warp_sum[w];
    if (threadIdx.x < digits) digit_base[threadIdx.x] = before + incl - mine_total;
  }
  __syncthreads();
  const uint32_t base = blockIdx.x * kTile + warp * (kItems * 32);
  K key[kItems];
  V val[kItems];
  uint32_t digit[kItems], rank[kItems];
  uint32_t *mine = warp_count + warp * digits;
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    const uint32_t i = base + r * 32 + lane;
    const bool valid = i < n;
    if (valid) {
      key[r] = LoadKey(keys_in, i, src);
      if (src.clip_rows > 0) {
        const uint32_t iota = i;
        memcpy(&val[r], &iota, 4);
      } else {
        val[r] = vals_in[i];
      }
      digit[r] = (OrderedBits(key[r], ascend) >> shift) & mask;
    } else {
      digit[r] = digits;  // matches only other elements past the end
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, digit[r]);
    const uint32_t before = __popc(peers & ((1u << lane) - 1u));
    const uint32_t seen = valid ? mine[digit[r]] : 0u;
    __syncwarp();
    if (valid && before == 0) mine[digit[r]] = seen + __popc(peers);
    __syncwarp();
    rank[r] = seen + before;
  }
  __syncthreads();
  // per digit: counts of the warps become the place of the warp's first element with that digit
  for (uint32_t d = threadIdx.x; d < digits; d += kThreads) {
    uint32_t run = digit_base[d] + counts[d * tiles + blockIdx.x];
    for (uint32_t w = 0; w < 16; ++w) {
      const uint32_t c = warp_count[w * digits + d];
      warp_count[w * digits + d] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kItems; ++r) {
    if (base + r * 32 + lane < n) {
      const uint32_t at = mine[digit[r]] + rank[r];
      keys_out[at] = key[r];
      vals_out[at] = val[r];
    }
  }
}

inline size_t Align256(size_t b) { return (b + 255) / 256 * 256; }

/*! \brief passes and bits per pass for `bits` significant key bits: an even number of passes of at most nine bits */
inline void PlanPasses(int bits, int *passes, int *per_pass) {
  if (bits < 1) bits = 1;
  *passes = 2 * ((bits + 2 * kMaxDigitBits - 1) / (2 * kMaxDigitBits));
  *per_pass = (bits + *passes - 1) / *passes;
}

/*! \brief bytes of scratch SortPairs needs for n pairs */
inline size_t ScratchBytes(int64_t n) {
  const size_t tiles = static_cast<size_t>((n + kTile - 1) / kTile);
  return 2 * Align256(static_cast<size_t>(n) * 4) + Align256((tiles << kMaxDigitBits) * 4) + Align256(4u << kMaxDigitBits);
}

/*!
 * \brief sorts n pairs by the low `bits` bits of the ordered key, stably; the result ends in
 *  keys / vals.  With src.clip_rows > 0 the input keys are taken from `raw` (clipped) instead of
 *  `keys`, and the values are generated.  `scratch` holds ScratchBytes(n).
 */
template <typename K, typename V>
inline void SortPairs(K *keys, V *vals, const K *raw, int64_t n, int bits, bool ascend, Source src, char *scratch,
                      cudaStream_t stream) {
  static_assert(sizeof(K) == 4 && sizeof(V) == 4, "4-byte keys and values");
  if (n <= 0) return;
  const uint32_t un = static_cast<uint32_t>(n);
  const uint32_t tiles = (un + kTile - 1) / kTile;
  K *k2 = reinterpret_cast<K *>(scratch);
  V *v2 = reinterpret_cast<V *>(scratch + Align256(n * 4));
  uint32_t *counts = reinterpret_cast<uint32_t *>(scratch + 2 * Align256(n * 4));
  uint32_t *totals = counts + Align256((static_cast<size_t>(tiles) << kMaxDigitBits) * 4) / 4;
  int passes = 0, per_pass = 0;
  PlanPasses(bits, &passes, &per_pass);
  const K *kin = src.clip_rows > 0 ? raw : keys;
  const V *vin = vals;
  K *kout = k2;
  V *vout = v2;
  Source from = src;
  for (int p = 0; p < passes; ++p) {
    const int shift = p * per_pass;
    int width = bits - shift < per_pass ? bits - shift : per_pass;
    if (width < 1) width = 1;  // a pass over no remaining bits still moves the data to the other buffer
    const uint32_t mask = (1u << width) - 1u;
    const uint32_t digits = mask + 1;
    gpu_rt::LaunchAfterDrain(RadixCountKernel<K>, dim3(tiles), dim3(kThreads), digits * 4, stream, kin, un, shift, mask, ascend, from, counts, tiles);
    MSHADOW_CUDA_POST_KERNEL_CHECK(RadixCountKernel);
    gpu_rt::LaunchAfterDrain(RadixScanKernel<8>, dim3((digits + 7) / 8), dim3(256), 0, stream, counts, totals, digits, tiles);
    MSHADOW_CUDA_POST_KERNEL_CHECK(RadixScanKernel);
    gpu_rt::LaunchAfterDrain(RadixScatterKernel<K, V>, dim3(tiles), dim3(kThreads), 17 * digits * 4, stream, kin, vin, kout, vout, un, shift, mask,
                                                                           ascend, from, counts, totals, tiles);
    MSHADOW_CUDA_POST_KERNEL_CHECK(RadixScatterKernel);
    // the next pass reads what this one wrote; only the first pass clips and generates
    kin = kout;
    vin = vout;
    kout = kout == k2 ? keys : k2;
    vout = vout == v2 ? vals : v2;
    from.clip_rows = 0;
  }
}

}  // namespace sortdetail
}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_RADIX_SORT_CUH_
