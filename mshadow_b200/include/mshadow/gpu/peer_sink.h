/*
 * PeerSink: lets the last stage of a reduction deliver its results to other GPUs as well.
 *
 * A reduction that is followed by an exchange between GPUs (per-GPU partial sums combined
 * over NVLink, as in `sumall_except_dim` sharded on the batch dimension) normally costs a second
 * kernel that reads the results back and sends them.  With a sink the thread that stores result
 * element i into the destination also stores it into row `rank` of a slot in every rank's
 * exchange window (mshadow-ps/peer_model.h), as one 64-bit word: the 32 bits of the value and the
 * 32-bit tag of the step.  The word is written by one naturally aligned 64-bit store, which the
 * memory system does not tear, so a reader that sees the tag has the value: no fence, no flag and
 * no "everybody is done" detection are needed, and the reduction kernel is not slowed by them.
 *
 * The sink is plain data (pointers into mapped peer memory, a tag, a count).  Only ordinary
 * stores are issued to peer memory.
 *
 * Use: obtain the sink of the next step from the exchange model, then
 *     { gpu_rt::PeerSinkScope scope(&sink); MapReduceKeepLowest<sv::saveto, red::sum>(&dst, src, 1.0f); }
 * The next reduction launched by this host thread inside the scope carries the sink; it applies to
 * 4-byte element types and must cover exactly `count` results.
 */
#ifndef MSHADOW_GPU_PEER_SINK_H_
#define MSHADOW_GPU_PEER_SINK_H_

#include <cstdint>
#include <cstring>

namespace mshadow {
namespace gpu_rt {

const int kPeerMaxWorld = 16;

struct PeerSink {
  unsigned long long *row[kPeerMaxWorld];  // where result 0 of this rank goes in each rank's window
  uint32_t tag;                            // step + 1; what the readers wait for
  uint32_t count;                          // results the row segment expects
  int world;                               // 0: no sink
  PeerSink() : tag(0), count(0), world(0) {
    for (int p = 0; p < kPeerMaxWorld; ++p) row[p] = nullptr;
  }
#ifdef __CUDACC__
  /*! \brief (value, tag) as the 64-bit word of the exchange protocol */
  template <typename DType>
  __device__ __forceinline__ static unsigned long long Word(DType v, uint32_t tag) {
    static_assert(sizeof(DType) == 4, "the exchange carries 4-byte elements");
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return (static_cast<unsigned long long>(tag) << 32) | bits;
  }
  /*! \brief deliver result i to every rank */
  template <typename DType>
  __device__ __forceinline__ void Put(uint32_t i, DType v) const {
    if constexpr (sizeof(DType) == 4) {
      const unsigned long long w = Word(v, tag);
#pragma unroll
      for (int p = 0; p < kPeerMaxWorld; ++p) {
        if (p < world) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(row[p] + i), "l"(w) : "memory");
      }
    }
  }
#endif
};

/*! \brief the sink that the next reduction launched by this host thread will carry, if any */
inline const PeerSink *&PendingPeerSink() {
  thread_local const PeerSink *pending = nullptr;
  return pending;
}

/*! \brief arms a sink for the next reduction of this host thread; disarms it on leaving the scope */
class PeerSinkScope {
 public:
  explicit PeerSinkScope(const PeerSink *sink) { PendingPeerSink() = sink; }
  ~PeerSinkScope() { PendingPeerSink() = nullptr; }
  PeerSinkScope(const PeerSinkScope &) = delete;
  PeerSinkScope &operator=(const PeerSinkScope &) = delete;
};

}  // namespace gpu_rt
}  // namespace mshadow
#endif  // MSHADOW_GPU_PEER_SINK_H_
