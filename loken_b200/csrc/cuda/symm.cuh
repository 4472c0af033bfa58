// Device view of the symmetric heaps and the signal primitives built on them.
//
// Heap layout (identical on every rank):
//   [0, 64)                 control words: epoch, finished-CTA counter
//   flags_off               flags[2 halves][MAX_RANKS sources][max_chunks] : unsigned epoch values
//   recv_off                recv[2 halves][MAX_RANKS sources][slot_bytes]  : payload slots
//   ll_off                  ll[2 halves][ll_half_bytes] : flag-in-data areas (tp_fused.cu, ep_moe.cu), zero at
//                           allocation; inside a half, [0, ll_hop2_off) takes the first hop of a collective and
//                           [ll_hop2_off, ll_half_bytes) the second
// A collective takes the next epoch number; the half in use is epoch & 1.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "tc100.cuh"

namespace lk {

constexpr int MAX_RANKS = 8;

struct SymmView {
  void* base[MAX_RANKS];     // every rank's heap as mapped into this process (base[rank] is local)
  int world, rank;
  long long flags_off, recv_off, slot_bytes;
  int max_chunks;
  int pad;
  long long ll_off, ll_half_bytes, ll_hop2_off;
};

#ifndef LK_PEER_WAIT_CYCLES
#define LK_PEER_WAIT_CYCLES (4000000000ll)   // about two seconds of SM clock
#endif

__device__ __forceinline__ unsigned* symm_ctrl(const SymmView& sv) {
  return reinterpret_cast<unsigned*>(sv.base[sv.rank]);
}
// Epoch of the collective now running: every CTA reads the word before any CTA can bump it
// (the bump happens after the last CTA has finished).
__device__ __forceinline__ unsigned symm_epoch_begin(const SymmView& sv) {
  return *reinterpret_cast<volatile unsigned*>(symm_ctrl(sv)) + 1u;
}
__device__ __forceinline__ void symm_epoch_end(const SymmView& sv) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* ctrl = symm_ctrl(sv);
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    __threadfence();
    if (atomicAdd(ctrl + 1, 1u) == total - 1) {
      ctrl[1] = 0;
      __threadfence();
      atomicAdd(ctrl, 1u);
    }
  }
}
__device__ __forceinline__ char* symm_recv(const SymmView& sv, int on_rank, int half, int src) {
  return reinterpret_cast<char*>(sv.base[on_rank]) + sv.recv_off + ((long long)half * MAX_RANKS + src) * sv.slot_bytes;
}
__device__ __forceinline__ unsigned* symm_flag(const SymmView& sv, int on_rank, int half, int src, int chunk) {
  return reinterpret_cast<unsigned*>(reinterpret_cast<char*>(sv.base[on_rank]) + sv.flags_off) +
         ((long long)half * MAX_RANKS + src) * sv.max_chunks + chunk;
}
// Tell rank `dst` that chunk `chunk` of source `src` (this rank) has landed there.  The caller
// has passed a CTA barrier after the data stores: the release store orders them before the flag.
__device__ __forceinline__ void symm_signal(const SymmView& sv, int dst, int half, int src, int chunk,
                                            unsigned epoch) {
  unsigned* f = symm_flag(sv, dst, half, src, chunk);
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
}
// Wait until source `src` has signalled chunk `chunk` for this epoch.  Bounded: returns false
// and records LK_ERR_PEER_TIMEOUT when the peer never shows up.
__device__ __forceinline__ bool symm_wait(const SymmView& sv, int half, int src, int chunk, unsigned epoch,
                                          int* status) {
  const unsigned* f = symm_flag(sv, sv.rank, half, src, chunk);
  const long long t0 = clock64();
  // (measured: acquire polls are faster here than relaxed polls followed by one fence)
  for (unsigned it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int)(v - epoch) >= 0) return true;
    if ((it & 63u) == 63u) {
      if (clock64() - t0 > LK_PEER_WAIT_CYCLES) break;
      __nanosleep(32);
    }
  }
  if (status) atomicCAS(status, 0, LK_ERR_PEER_TIMEOUT | (src << 8));
  return false;
}

}  // namespace lk
