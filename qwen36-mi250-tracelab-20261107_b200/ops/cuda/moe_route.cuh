// Router softmax / top-k of one row by one warp, shared by the local MoE glue (elementwise.cu) and the
// expert-parallel dispatch (ep_moe.cu).
#pragma once

#ifdef B200_EMU  // host build of the routing body for tests/emu (shuffles and atomics come from the shim)
#include "emu_shim.h"
#else
#include "common.cuh"
#endif

namespace b200 {

constexpr int MAX_PER_LANE = 16;  // E <= 512

// One warp per row: fp32 softmax over E router logits, iterative top-k with ties to the lower
// expert id, renormalise, round weights to bf16; pair k (the last) is the shared expert with
// weight sigmoid(logit[E]) when `shared` is set. PER_LANE * 32 >= E.
template <int PER_LANE>
__device__ __forceinline__ void route_row(const float* row, int E, int top_k, int shared, float* wts, int* idx,
                                          const int* expert_map, int* counts, int lane) {
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    v[i] = (i * 32 + lane) < E ? expf(v[i] - mx) : -1.0f;
    sum += v[i] > 0.f ? v[i] : 0.f;
  }
  sum = warp_sum(sum);
  float sel_w = 0.f;  // lane j keeps the j-th selected probability
  int sel_e = 0;
  float tot = 0.f;
  for (int k = 0; k < top_k; ++k) {
    float bm = -1.0f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bm) { bm = v[i]; be = e; }  // ascending e within a lane: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, bm, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (om > bm || (om == bm && oe < be)) { bm = om; be = oe; }
    }
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i)
      if (i * 32 + lane == be) v[i] = -1.0f;  // remove the winner (static indexing keeps v in registers)
    const float pr = bm / sum;
    tot += pr;
    if (lane == k) { sel_w = pr; sel_e = be; }
  }
  if (lane < top_k) {
    const float wv = __bfloat162float(__float2bfloat16(sel_w / tot));
    // expert parallelism: experts hosted elsewhere map to -1 and are skipped by the later stages
    const int le = expert_map ? expert_map[sel_e] : sel_e;
    wts[lane] = wv;
    idx[lane] = le;
    if (counts && le >= 0) atomicAdd(&counts[le], 1);
  }
  if (shared && lane == 0) {
    const float sg = sigmoid_f(row[E]);
    const int le = expert_map ? expert_map[E] : E;
    wts[top_k] = __bfloat162float(__float2bfloat16(sg));
    idx[top_k] = le;
    if (counts && le >= 0) atomicAdd(&counts[le], 1);
  }
}


}  // namespace b200
