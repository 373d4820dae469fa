// The expert plan of the MoE block: (row, pair) -> expert table in, expert-sorted layout out (rows per expert,
// offsets, token-tile table, positions of the pairs), as one CTA, as the tail of the routing launch, or split into
// a grid-wide histogram + a scan by the last CTA + a grid-wide scatter. Used by elementwise.cu; kept in a header of
// its own so that the same source also compiles as host C++ for tests/emu (threads, barriers, shuffles and atomics
// then come from the shim).
#pragma once

#ifdef B200_EMU
#include "emu_shim.h"
#else
#include "common.cuh"
#endif
#include "moe_route.cuh"

namespace b200 {

// One CTA of 1024 threads turns the (row, pair) -> expert table into everything the grouped GEMMs need, without
// global atomics or a zeroed workspace: rows per expert (shared-memory histogram), exclusive offsets (experts laid
// out in id order, rows of one expert contiguous), the token-tile table (expert, row0, nrows) and its length, and
// the position of every pair in the expert-sorted order (perm / inv). The order inside an expert does not influence
// any output value: every sorted row is computed on its own.
__device__ void plan_scatter(const int* idx, int n_pairs, int Et, int bt, int* offsets, int4* tiles, int* n_tiles,
                             int max_tiles, int* perm, int* inv, int* err, int P, int* src_rows) {
  __shared__ int s_count[1024], s_off[1024], s_cur[1024];
  __shared__ int w_rows[32], w_tiles[32];
  const int e = threadIdx.x, lane = e & 31, w = e >> 5;
  s_count[e] = 0;
  s_cur[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int x = __ldcg(idx + i);  // through L2: other CTAs of the same launch may have written it
    if (x >= 0 && x < Et) atomicAdd(&s_count[x], 1);
  }
  __syncthreads();
  const int c = e < Et ? s_count[e] : 0;
  const int t = (c + bt - 1) / bt;
  int sc = c, stl = t;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, sc, o), b2 = __shfl_up_sync(0xffffffffu, stl, o);
    if (lane >= o) { sc += a; stl += b2; }
  }
  if (lane == 31) { w_rows[w] = sc; w_tiles[w] = stl; }
  __syncthreads();
  if (w == 0) {
    int a = w_rows[lane], b2 = w_tiles[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b2, o);
      if (lane >= o) { a += x; b2 += y; }
    }
    w_rows[lane] = a; w_tiles[lane] = b2;
  }
  __syncthreads();
  const int row0 = sc - c + (w ? w_rows[w - 1] : 0);    // exclusive prefix
  const int tile0 = stl - t + (w ? w_tiles[w - 1] : 0);
  s_off[e] = row0;
  if (e < Et) {
    offsets[e] = row0;
    for (int i = 0, ti = tile0; i * bt < c && ti < max_tiles; ++i, ++ti)
      tiles[ti] = make_int4(e, row0 + i * bt, min(bt, c - i * bt), 0);
  }
  if (e == Et - 1) {
    offsets[Et] = row0 + c;
    const int total = tile0 + t;
    *n_tiles = total < max_tiles ? total : max_tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int x = __ldcg(idx + i);
    if (x < 0) { inv[i] = -1; continue; }  // pair served by another rank
    if (x >= Et) { atomicCAS(err, 0, ERR_BAD_INDEX); inv[i] = -1; continue; }
    const int pos = s_off[x] + atomicAdd(&s_cur[x], 1);
    perm[pos] = i;
    inv[i] = pos;
    if (src_rows) src_rows[pos] = i / P;  // the activation row behind sorted position pos (for a gathering GEMM)
  }
}

__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* idx, int n_pairs, int Et, int bt, int* offsets, int4* tiles, int* n_tiles, int max_tiles,
                int* perm, int* inv, int* err, int P, int* src_rows) {
  pdl_wait();
  pdl_launch();
  plan_scatter(idx, n_pairs, Et, bt, offsets, tiles, n_tiles, max_tiles, perm, inv, err, P, src_rows);
}

// Decode-size batches: routing of every row (one warp each, 32 warps) and the plan in ONE launch.
template <int PER_LANE>
__global__ void __launch_bounds__(1024)
moe_route_plan_kernel(const float* logits, int ldl, int T, int E, int top_k, int shared, float* wts, int* idx,
                      const int* expert_map, int Et, int bt, int* offsets, int4* tiles, int* n_tiles, int max_tiles,
                      int* perm, int* inv, int* err, int* src_rows) {
  pdl_wait();
  pdl_launch();
  const int P = top_k + (shared ? 1 : 0);
  const int lane = threadIdx.x & 31;
  for (int r = threadIdx.x >> 5; r < T; r += 32)
    route_row<PER_LANE>(logits + static_cast<size_t>(r) * ldl, E, top_k, shared, wts + static_cast<size_t>(r) * P,
                        idx + static_cast<size_t>(r) * P, expert_map, nullptr, lane);
  __syncthreads();  // this CTA wrote idx: visible to all its threads after the barrier
  plan_scatter(idx, T * P, Et, bt, offsets, tiles, n_tiles, max_tiles, perm, inv, err, P, src_rows);
}

// Any number of rows, still one launch: a grid of 1024-thread CTAs routes 32 rows each; the CTA that finishes last
// (a ticket counter in global memory, which it puts back to zero for the next launch) builds the plan from the whole
// index table. Everything the other CTAs wrote is visible to it: they fence before taking their ticket.
// `work` (optional): 2 * 1024 ints kept zero between launches (per-expert counts, per-expert cursors). With it the
// CTAs add their rows' expert counts to the global histogram and the last CTA only turns the counts into offsets and
// the tile table (a scan over the experts); the positions of the pairs are then handed out by a second, grid-wide
// launch (moe_scatter_kernel). Without it the last CTA does everything, which is right up to a few hundred rows: at
// 8192 rows the single CTA's histogram and scatter of 73,728 pairs took 87 us per layer.
template <int PER_LANE>
__global__ void __launch_bounds__(1024)
moe_route_plan_grid_kernel(const float* logits, int ldl, int T, int E, int top_k, int shared, float* wts, int* idx,
                           const int* expert_map, int Et, int bt, int* offsets, int4* tiles, int* n_tiles,
                           int max_tiles, int* perm, int* inv, int* err, int* src_rows, unsigned int* ticket, int* work) {
  pdl_wait();
  pdl_launch();
  __shared__ int s_last;
  __shared__ int s_hist[1024];
  const int P = top_k + (shared ? 1 : 0);
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 32 + (threadIdx.x >> 5);
  if (work) s_hist[threadIdx.x] = 0;
  if (r < T)
    route_row<PER_LANE>(logits + static_cast<size_t>(r) * ldl, E, top_k, shared, wts + static_cast<size_t>(r) * P,
                        idx + static_cast<size_t>(r) * P, expert_map, nullptr, lane);
  if (work) {
    __syncthreads();  // this CTA's 32 rows of idx are written (and visible to the CTA)
    const int row0 = blockIdx.x * 32;
    const int n_here = min(32, T - row0) * P;
    for (int i = threadIdx.x; i < n_here; i += blockDim.x) {
      const int x = idx[static_cast<size_t>(row0) * P + i];
      if (x >= 0 && x < Et) atomicAdd(&s_hist[x], 1);
    }
    __syncthreads();
    if (threadIdx.x < Et && s_hist[threadIdx.x]) atomicAdd(&work[threadIdx.x], s_hist[threadIdx.x]);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(ticket, 1u);
    s_last = t == gridDim.x - 1;
    if (s_last) *ticket = 0;  // every CTA has taken its ticket: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (work == nullptr) {
    plan_scatter(idx, T * P, Et, bt, offsets, tiles, n_tiles, max_tiles, perm, inv, err, P, src_rows);
    return;
  }
  // counts -> offsets and tile table (one thread per expert), counts and cursors back to zero
  __shared__ int w_rows[32], w_tiles[32];
  const int e = threadIdx.x, w = e >> 5;
  const int c = e < Et ? __ldcg(work + e) : 0;
  if (e < Et) { work[e] = 0; work[1024 + e] = 0; }
  const int t = (c + bt - 1) / bt;
  int sc = c, stl = t;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, sc, o), b2 = __shfl_up_sync(0xffffffffu, stl, o);
    if (lane >= o) { sc += a; stl += b2; }
  }
  if (lane == 31) { w_rows[w] = sc; w_tiles[w] = stl; }
  __syncthreads();
  if (w == 0) {
    int a = w_rows[lane], b2 = w_tiles[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b2, o);
      if (lane >= o) { a += x; b2 += y; }
    }
    w_rows[lane] = a; w_tiles[lane] = b2;
  }
  __syncthreads();
  const int row0 = sc - c + (w ? w_rows[w - 1] : 0);
  const int tile0 = stl - t + (w ? w_tiles[w - 1] : 0);
  if (e < Et) {
    offsets[e] = row0;
    for (int i = 0, ti = tile0; i * bt < c && ti < max_tiles; ++i, ++ti)
      tiles[ti] = make_int4(e, row0 + i * bt, min(bt, c - i * bt), 0);
  }
  if (e == Et - 1) {
    offsets[Et] = row0 + c;
    const int total = tile0 + t;
    *n_tiles = total < max_tiles ? total : max_tiles;
  }
}

// Second half of the plan at prefill sizes: every pair takes the next free position of its expert's run
// (a global cursor per expert, zero before the launch; the order inside an expert does not influence any output).
__global__ void moe_scatter_kernel(const int* idx, int n_pairs, int Et, const int* offsets, int* cursors, int* perm,
                                   int* inv, int* err, int P, int* src_rows) {
  pdl_wait();
  pdl_launch();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int x = idx[i];
    if (x < 0) { inv[i] = -1; continue; }  // pair served by another rank
    if (x >= Et) { atomicCAS(err, 0, ERR_BAD_INDEX); inv[i] = -1; continue; }
    const int pos = offsets[x] + atomicAdd(&cursors[x], 1);
    perm[pos] = i;
    inv[i] = pos;
    if (src_rows) src_rows[pos] = i / P;
  }
}

}  // namespace b200
