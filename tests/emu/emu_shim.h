// Host shim that lets a CUDA kernel source compile and run as plain C++20: every CUDA thread of one CTA is a
// std::thread, __syncthreads() is a std::barrier, __shared__ variables become function statics (one CTA runs at a
// time), warp shuffles go through a per-CTA exchange array. Bulk copies are memcpy and mbarrier waits succeed at
// once, so only the kernel's arithmetic, indexing and barrier placement are under test: a missing barrier shows up
// as a wrong result (or a data race under -fsanitize=thread), without a GPU.
// (The reference checks its HIP kernel the same way: tools/emu/gdn_hip_emu.cpp, tools/emu/gdn_hip_emu_shim.h.)
#pragma once

#include <algorithm>
#include <atomic>
#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <thread>
#include <vector>

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static
#define __align__(n) alignas(n)
#define __launch_bounds__(...)

namespace b200 {

struct Dim3 { unsigned x = 1, y = 1, z = 1; };
struct alignas(16) uint4 { unsigned x, y, z, w; };
struct alignas(16) float4 { float x, y, z, w; };
struct alignas(16) int4 { int x, y, z, w; };
inline int4 make_int4(int x, int y, int z, int w) { return int4{x, y, z, w}; }
inline thread_local Dim3 threadIdx, blockIdx;
inline Dim3 blockDim, gridDim;
inline std::barrier<>* cta_barrier = nullptr;
inline float* shfl_buf = nullptr;            // one float per thread of the CTA
inline std::vector<std::unique_ptr<std::barrier<>>>* warp_barriers = nullptr;  // one per warp of the CTA
alignas(128) inline float sS_storage[128 * 128];  // dynamic shared memory of the CTA under test
#define EMU_DYNAMIC_SMEM sS_storage

inline void __syncthreads() { cta_barrier->arrive_and_wait(); }

// bf16 with round-to-nearest-even conversion, as the device intrinsics do
struct bf16 { uint16_t bits; };
inline bf16 __float2bfloat16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return bf16{static_cast<uint16_t>((u >> 16) | 0x40)};
  u += 0x7fffu + ((u >> 16) & 1u);
  return bf16{static_cast<uint16_t>(u >> 16)};
}
inline float __bfloat162float(bf16 b) {
  const uint32_t u = static_cast<uint32_t>(b.bits) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline float __expf(float x) { return std::exp(x); }
inline float rsqrtf(float x) { return 1.0f / std::sqrt(x); }
inline float silu_f(float x) { return x / (1.0f + __expf(-x)); }
inline float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }
inline float softplus_f(float x) { return x > 20.0f ? x : std::log1p(__expf(x)); }

// Shuffles exchange through a per-CTA array under a barrier of the calling warp only, so a warp may shuffle while
// the others do something else (the plan kernels scan per-warp totals in warp 0). All lanes of a warp that exist
// must take part, as with a full mask on the GPU.
inline void warp_sync() { (*warp_barriers)[threadIdx.x >> 5]->arrive_and_wait(); }
inline float shfl_xor(float v, int mask) {
  shfl_buf[threadIdx.x] = v;
  warp_sync();
  const float o = shfl_buf[threadIdx.x ^ static_cast<unsigned>(mask)];
  warp_sync();
  return o;
}
inline float shfl_up(float v, int delta) {
  shfl_buf[threadIdx.x] = v;
  warp_sync();
  const float o = (threadIdx.x & 31u) >= static_cast<unsigned>(delta) ? shfl_buf[threadIdx.x - delta] : v;
  warp_sync();
  return o;
}
inline float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += shfl_xor(v, o);
  return v;
}
inline float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = std::fmax(v, shfl_xor(v, o));
  return v;
}
// The CUDA spelling of the shuffle, for 4-byte values (the routing kernel exchanges a float and an int per round).
template <typename T>
inline T __shfl_xor_sync(unsigned, T v, int mask) {
  static_assert(sizeof(T) == sizeof(float), "4-byte values only");
  float f;
  std::memcpy(&f, &v, sizeof f);
  f = shfl_xor(f, mask);
  std::memcpy(&v, &f, sizeof f);
  return v;
}
template <typename T>
inline T __shfl_up_sync(unsigned, T v, int delta) {
  static_assert(sizeof(T) == sizeof(float), "4-byte values only");
  float f;
  std::memcpy(&f, &v, sizeof f);
  f = shfl_up(f, delta);
  std::memcpy(&v, &f, sizeof f);
  return v;
}
inline int atomicAdd(int* p, int v) { return std::atomic_ref<int>(*p).fetch_add(v); }
inline unsigned atomicAdd(unsigned* p, unsigned v) { return std::atomic_ref<unsigned>(*p).fetch_add(v); }
inline int atomicCAS(int* p, int expect, int v) {
  std::atomic_ref<int>(*p).compare_exchange_strong(expect, v);
  return expect;
}
template <typename T>
inline T __ldcg(const T* p) { return *p; }
inline void __threadfence() { std::atomic_thread_fence(std::memory_order_seq_cst); }
using std::max;
using std::min;

enum ErrCode : int { ERR_NONE = 0, ERR_WAIT_FULL = 1, ERR_BAD_INDEX = 5 };
inline void mbar_init(uint64_t*, uint32_t) {}
inline void mbar_fence_init() {}
inline void mbar_expect_tx(uint64_t*, uint32_t) {}
inline bool mbar_wait(uint64_t*, uint32_t, int*, int, volatile int*) { return true; }
inline void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t*) { std::memcpy(dst, src, bytes); }
inline void bulk_store(void* dst, const void* src, uint32_t bytes) { std::memcpy(dst, src, bytes); }
inline void bulk_store_wait_read() {}
inline void proxy_fence() {}
inline void pdl_wait() {}
inline void pdl_launch() {}

// Run `body` as one CTA of `threads` threads at block index (bx, by).
inline void run_cta(unsigned threads, unsigned bx, unsigned by, const std::function<void()>& body) {
  std::barrier<> bar(static_cast<std::ptrdiff_t>(threads));
  std::vector<float> buf(threads);
  std::vector<std::unique_ptr<std::barrier<>>> warps;
  for (unsigned w = 0; w * 32 < threads; ++w)
    warps.push_back(std::make_unique<std::barrier<>>(static_cast<std::ptrdiff_t>(std::min(32u, threads - 32 * w))));
  cta_barrier = &bar;
  shfl_buf = buf.data();
  warp_barriers = &warps;
  blockDim.x = threads;
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (unsigned t = 0; t < threads; ++t)
    pool.emplace_back([&, t] {
      threadIdx = Dim3{t, 0, 0};
      blockIdx = Dim3{bx, by, 0};
      body();
      bar.arrive_and_drop();
      warps[t >> 5]->arrive_and_drop();
    });
  for (auto& th : pool) th.join();
}

}  // namespace b200
