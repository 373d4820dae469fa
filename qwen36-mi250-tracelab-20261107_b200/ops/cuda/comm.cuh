// Device-side pieces of the NVLink collectives: the symmetric-memory context every fused
// compute+collective kernel receives, system-scope flag stores/loads and the bounded peer wait.
//
// Memory model of a rank group of R ranks (R <= 8), all buffers allocated with cudaMalloc on their
// own GPU and mapped into every peer process through CUDA IPC (parallel/symm.py):
//   recv[r]  : rank r's receive area, float [2 parities][R sources][slot_elems]
//   flags[r] : rank r's arrival counters, uint32 [R sources][max_blocks]
//   epoch    : this rank's per-block call counter, uint32 [max_blocks] (device-resident so that a
//              captured CUDA graph needs no host input to tell calls apart; the reference keeps
//              per-CTA epochs in device memory for the same reason, engine/fast/tp.py:132-162)
// A block (CTA or output tile) of call e writes its partial into slot [e & 1][my rank] of every
// rank, then releases flag[my rank][block] = e on every rank; it reads only after all R flags of
// that block reached e. Every rank adds the R partials in rank order, so results are bitwise equal
// on all ranks. Peer traffic is plain st.global / ld.global over NVLink: no multimem, no TMA.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int MAX_RANKS = 8;

struct CommCtx {
  float* recv[MAX_RANKS];
  uint32_t* flags[MAX_RANKS];
  uint32_t* epoch;
  int* err;
  int rank;
  int world;
  int max_blocks;
  unsigned long long slot_elems;  // floats per (parity, source) slot
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p reaches `want` (wrap-safe). Gives up after WAIT_CYCLES, records ERR_WAIT_PEER. Once the error word
// is set (by this wait or any earlier one of the step) every further wait gives up at once, so a step whose peer is
// gone costs one timeout, not one per collective.
// `limit`: clock ticks before giving up. A second is right for kernels whose peers were launched by the same host
// thread or in the same captured graph; replicas that launch their passes from separate processes (each under its own
// interpreter lock, with its own request threads) give their peer waits a limit set by the host (EpCtx::wait_cycles).
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, int* err, long long limit = WAIT_CYCLES) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(p) - want) < 0) {
    if (err && *reinterpret_cast<volatile int*>(err) != 0) return false;
    if (clock64() - t0 > limit) {
      if (err) atomicCAS(err, 0, ERR_WAIT_PEER);
      return false;
    }
    __nanosleep(20);
  }
  return true;
}

__device__ __forceinline__ float* comm_slot(const CommCtx& c, int dst_rank, uint32_t epoch, int src_rank) {
  return c.recv[dst_rank] + (static_cast<size_t>(epoch & 1) * c.world + src_rank) * c.slot_elems;
}

}  // namespace b200
