// Row rings in shared memory: mbarrier, TMA (cp.async.bulk.tensor) and cp.async helpers of the
// producer / consumer kernels in dk_local_ring.cu.
//
// A block streams the rows of its part of the tensors through rings of row slots.  One producer
// warp fills slots (a tiled TMA copy per row of all the block's channels, with the hardware's zero
// fill supplying the convolution padding; cp.async for the narrow offset rows; where a row is not a
// multiple of 16 bytes and TMA cannot fetch it, up to four producer warps share its cp.async
// pieces); the other warps consume them.  Per slot there is a "full" mbarrier (the copy's bytes have landed) and an "empty"
// mbarrier (every consumer item that reads the slot is done).  No block-wide barrier is executed
// after the set-up, so filling and computing overlap.
//
// Every wait is bounded: when it runs out the waiting warp records an error code in global memory
// and leaves its loop, so a mistake in the hand-over logic ends the kernel instead of hanging it.
#pragma once

#include <cuda.h>

#include "dk_mma_common.cuh"

namespace dk {
namespace ring {

constexpr unsigned kMaxPolls = 1u << 17;  // try_wait suspends for a while by itself; this bounds a wait to a fraction of a second

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// makes the initialised barriers visible to the async proxy (the TMA unit) as well
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// orders this thread's ordinary shared-memory writes before later async-proxy accesses
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(unsigned bar, unsigned count) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete.  false = gave up after kMaxPolls polls.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  if (mbar_try_wait(bar, parity)) return true;
  for (unsigned i = 0; i < kMaxPolls; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// The barrier receives one arrival (already counted in its initial count) once all cp.async
// copies this thread issued before have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(unsigned bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(sa), "l"(gmem));
}

// One box of a rank-3 tensor map into this block's shared memory; completion is counted in bytes on
// `bar`.  Coordinates are (innermost, row, plane); x * element size must be a multiple of 16 bytes.
// Only this GPU's memory, only this block's shared memory.
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* tm, int x, int y, int z, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
      "l"(tm), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(tm) : "memory");
}

// Bookkeeping of one ring of n slots (any n from 2 up, not only powers of two: shared memory decides the depth).
// Fill number k goes to slot k mod n and is phase k / n ("turn") of that slot's two barriers.  A phase can only
// be told from its parity, so a consumer may wait on the "full" barrier of fill k only once the slot has been
// reclaimed for that fill (all users of fill k - n are done); the producer publishes that in `issued`, a counter
// in shared memory that only grows.
struct Ring {
  unsigned full, empty;  // shared-memory addresses of the two barrier arrays
  unsigned issued;       // shared-memory address of the counter
  int n;                 // slots
  unsigned magic;        // ceil(2^32 / n): k / n = high word of k * magic as long as k * n < 2^32

  __device__ __forceinline__ void set_slots(int slots) {
    n = slots;
    magic = (unsigned)((0x100000000ull + (unsigned)slots - 1) / (unsigned)slots);
  }
  __device__ __forceinline__ int turn(int k) const { return (int)__umulhi((unsigned)k, magic); }
  __device__ __forceinline__ int slot(int k) const { return k - turn(k) * n; }

  // producer, whole warp: wait until the slot of fill k may be overwritten, then publish that.  Where several producer
  // warps share the copies of a fill, all of them wait and the first publishes: a consumer that then waits on the "full"
  // barrier cannot be released early, because that barrier also counts the arrivals of the producers still on their way.
  __device__ __forceinline__ bool reclaim(int k, int lane, bool publish = true) const {
    bool ok = true;
    if (k >= n) ok = mbar_wait(empty + 8 * slot(k), (turn(k) - 1) & 1);
    if (lane == 0 && publish) asm volatile("st.release.cta.shared::cta.b32 [%0], %1;\n" ::"r"(issued), "r"(k + 1) : "memory");
    return ok;
  }
  // consumer: wait until fill k has landed
  __device__ __forceinline__ bool wait_full(int k) const {
    int seen;
    unsigned polls = 0;
    for (;;) {
      asm volatile("ld.acquire.cta.shared::cta.b32 %0, [%1];\n" : "=r"(seen) : "r"(issued) : "memory");
      if (seen > k) break;
      if (++polls > (kMaxPolls << 4)) return false;
      __nanosleep(64);
    }
    return mbar_wait(full + 8 * slot(k), turn(k) & 1);
  }
  // consumer, one lane: m users of fill k are done with it
  __device__ __forceinline__ void release(int k, int m) const { mbar_arrive_n(empty + 8 * slot(k), m); }
};

// Row layout of a ring slot holding rows of width Wd (halves): 8 zero halves in front (left padding; the
// next channel's front doubles as this channel's right padding), then the row; the pitch is = 8 (mod 16)
// halves so that the eight channels of an mma fragment start in distinct banks.
template <int Wd>
struct RowLayout {
  static constexpr int kLeft = 8;
  static constexpr int kInner = ((Wd + 8 + 7) / 16) * 16 + 8;  // halves per channel row
  static constexpr bool kTma = (Wd % 8 == 0);                   // rows are multiples of 16 bytes: a tiled TMA copy can fetch them
  static constexpr int kPiece = (Wd % 8 == 0) ? 16 : ((Wd % 4 == 0) ? 8 : ((Wd % 2 == 0) ? 4 : 0));  // cp.async piece otherwise
};

}  // namespace ring
}  // namespace dk
