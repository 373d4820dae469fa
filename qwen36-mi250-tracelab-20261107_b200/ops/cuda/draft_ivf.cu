// Shortlist scoring for speculative drafts: the draft token of a row is the best LM-head row among the members of
// the few vocabulary clusters whose centroids score highest for that row, instead of the best of all 248320 rows.
// A draft only has to be a good guess (the verify pass decides), and at small batches the full LM head is most of
// a draft link: 1 GB of weights per link against ~16 MB for 64 clusters of ~60 rows each.
// (Reference: the IVF draft of engine/fast/draft_ivf.py:159, 362-499 - centroid GEMV, top clusters, gathered GEMV,
// argmax; its predicated full-vocabulary fallback is left out: a weak draft costs one rejected token.)
//
// The centroid scores come from the dense GEMM and the cluster choice from a top-k over them; this file is the
// gathered GEMV: one CTA per (row, probed cluster), one warp per member row of the LM head (plain or tile-packed
// layout), fp32 dot products, first maximum with ties to the lower token id. The per-(cluster, row) partials have the
// layout of the LM-head argmax partials, so argmax_finish_kernel reduces them.
#include "common.cuh"

namespace b200 {

__global__ void __launch_bounds__(256)
ivf_pick_kernel(const bf16* hidden, int ldh, const bf16* W, int ldw, int packed, int H, const int* probes, int P,
                const int* offsets, const int* order, int n_clusters, int V, float* part_max, int* part_idx, int R,
                int* err) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float s_h[];  // the row's hidden state in fp32
  __shared__ float w_max[8];
  __shared__ int w_idx[8];
  const int r = blockIdx.x, p = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s_h[i] = __bfloat162float(hidden[static_cast<size_t>(r) * ldh + i]);
  __syncthreads();
  int c = probes[r * P + p];
  float best = -INFINITY;
  int best_id = 0x7fffffff;
  if (c < 0 || c >= n_clusters) {
    if (threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_INDEX);
  } else {
    const int m0 = offsets[c], m1 = offsets[c + 1];
    const int nk = H / 64;
    for (int m = m0 + warp; m < m1; m += 8) {
      const int id = order[m];
      if (id < 0 || id >= V) { if (lane == 0) atomicCAS(err, 0, ERR_BAD_INDEX); continue; }
      float acc = 0.f;
      for (int k0 = lane * 8; k0 < H; k0 += 256) {
        const size_t off = packed ? ((static_cast<size_t>(id >> 7) * nk + (k0 >> 6)) * 128 + (id & 127)) * 64 + (k0 & 63)
                                  : static_cast<size_t>(id) * ldw + k0;
        const uint4 v = *reinterpret_cast<const uint4*>(W + off);
        const bf16* e = reinterpret_cast<const bf16*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += s_h[k0 + j] * __bfloat162float(e[j]);
      }
      acc = warp_sum(acc);
      if (acc > best || (acc == best && id < best_id)) { best = acc; best_id = id; }
    }
  }
  if (lane == 0) { w_max[warp] = best; w_idx[warp] = best_id; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (w_max[w] > best || (w_max[w] == best && w_idx[w] < best_id)) { best = w_max[w]; best_id = w_idx[w]; }
    part_max[static_cast<size_t>(p) * R + r] = best;
    part_idx[static_cast<size_t>(p) * R + r] = best_id;
  }
}

}  // namespace b200

using namespace b200;

// hidden [R, ldh] bf16; W: the LM head [V, H] (plain, row stride ldw) or tile-packed; probes [R, P] cluster ids;
// offsets [n_clusters + 1] / order [V]: members of each cluster; part_max / part_idx [P, R] receive the best member
// of every probed cluster (reduce with b200_argmax_finish(part_max, part_idx, P, R, ...)). H a multiple of 8 (of 64 when packed).
extern "C" int b200_ivf_pick(const void* hidden, int ldh, const void* W, int ldw, int packed, int H, const int* probes,
                             int P, const int* offsets, const int* order, int n_clusters, int V, float* part_max,
                             int* part_idx, int R, int* err, cudaStream_t st) {
  if (R <= 0 || P <= 0) return 0;
  if (H % 8 || H > 8192 || (packed && H % 64)) return -7;
  return launch_pdl(ivf_pick_kernel, dim3(R, P), dim3(256), H * sizeof(float), st, static_cast<const bf16*>(hidden), ldh,
                    static_cast<const bf16*>(W), ldw, packed, H, probes, P, offsets, order, n_clusters, V, part_max,
                    part_idx, R, err) == cudaSuccess ? 0 : -4;
}
