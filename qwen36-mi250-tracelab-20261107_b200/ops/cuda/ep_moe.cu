// Expert-parallel MoE over NVLink peer memory for token-sharded activations: every rank holds its own
// rows and E / R of the routed experts (plus a replica of the shared expert).
//
//   ep_counts   : publish this rank's per-expert pair counts to every rank and wait for everyone's
//   ep_plan     : from all counts, the row layout of every host's buffer (expert-major, source-major inside
//                 an expert) -> where this rank's pairs go, and the local tile table of the grouped GEMMs
//   ep_dispatch : the all-to-all. One CTA per (row, pair): the activation row is stored straight into the
//                 hosting rank's expert-sorted buffer (peer store), with (source rank, pair slot) beside it
//   ep_signal / ep_wait : release / acquire flags around the peer stores (bounded waits)
//   grouped GEMMs (gemm_tcgen05.cu): gate/up + SiLU-mul on the received rows, then the down projection whose
//                 epilogue scatters each output row back to the token's owner (the combine all-to-all)
//   ep_combine  : after all hosts have signalled, the top-k weighted sum in pair order
//
// The reference has no expert parallelism (its TP halves every expert, engine/fast/tp.py:19-21, 716-736).
// All buffers are symmetric CUDA IPC mappings; flags carry a device-resident epoch so that the sequence can
// be captured in a CUDA graph. No multimem, no TMA on peer memory.
#include "comm.cuh"

namespace b200 {

struct EpCtx {
  bf16* xs[MAX_RANKS];          // [cap_rows, H] expert-sorted incoming rows of each rank
  int2* meta[MAX_RANKS];        // [cap_rows] (source rank, pair slot)
  bf16* pair_out[MAX_RANKS];    // [max_pairs, H] expert outputs returned to each rank
  int* counts_all[MAX_RANKS];   // [R, Etot] per-expert pair counts of every source
  uint32_t* flags[MAX_RANKS];   // [3, R]: counts / dispatch / combine arrival epochs per source
  uint32_t* epoch;              // this rank's call counter (device resident)
  int* err;
  int rank, world;
  int E;                        // routed experts (global); expert id E is the shared expert, hosted by everyone
  int per;                      // routed experts per rank
  int cap_rows, max_pairs;
};

// counts[Etot] -> counts_all[me] on every rank; then wait for all sources. One CTA. Also advances the epoch.
__device__ __forceinline__ void ep_counts_body(const EpCtx& c, const int* counts) {
  const int Etot = c.E + 1;
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) { s_e = c.epoch[0] + 1; c.epoch[0] = s_e; }
  __syncthreads();
  const uint32_t e = s_e;
  for (int i = threadIdx.x; i < Etot; i += blockDim.x) {
    const int v = counts[i];
    for (int r = 0; r < c.world; ++r) c.counts_all[r][c.rank * Etot + i] = v;
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + 0 * MAX_RANKS + c.rank, e);
    wait_flag(c.flags[c.rank] + 0 * MAX_RANKS + threadIdx.x, e, c.err);
  }
}
__global__ void ep_counts_kernel(EpCtx c, const int* counts) { ep_counts_body(c, counts); }

// One CTA of 1024 threads, Etot <= 1024. Outputs: send_base[Etot] (first position of my rows of expert e in
// its host's buffer), cursors[Etot] = 0, local tile table, n_tiles, n_rows (rows this rank receives).
__global__ void __launch_bounds__(1024)
ep_plan_kernel(EpCtx c, int bt, int* send_base, int* cursors, int4* tiles, int* n_tiles, int max_tiles, int* n_rows,
               const int* counts) {
  if (counts != nullptr) {  // fused form: the count exchange and its wait run in this CTA first
    ep_counts_body(c, counts);
    __syncthreads();
  }
  const int Etot = c.E + 1, E = c.E, R = c.world, me = c.rank;
  const int* ca = c.counts_all[me];
  __shared__ int G[1025];   // exclusive prefix of routed totals in global expert order
  __shared__ int wsum[32];
  const int e = threadIdx.x, lane = e & 31, w = e >> 5;
  int tot = 0, before_me = 0;
  if (e < E) {
    for (int s = 0; s < R; ++s) { const int v = ca[s * Etot + e]; tot += v; if (s < me) before_me += v; }
  }
  int sc = tot;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, sc, o); if (lane >= o) sc += a; }
  if (lane == 31) wsum[w] = sc;
  __syncthreads();
  if (w == 0) {
    int a = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int x = __shfl_up_sync(0xffffffffu, a, o); if (lane >= o) a += x; }
    wsum[lane] = a;
  }
  __syncthreads();
  const int excl = sc - tot + (w ? wsum[w - 1] : 0);
  if (e <= E) G[e] = excl;  // thread E has tot = 0, so G[E] is the number of routed pairs
  __syncthreads();
  if (e < E) {
    const int host = e / c.per;
    send_base[e] = (G[e] - G[host * c.per]) + before_me;
    cursors[e] = 0;
  }
  if (e == E) {  // shared expert: my own rows, after my routed rows
    send_base[E] = G[(me + 1) * c.per] - G[me * c.per];
    cursors[E] = 0;
  }
  // local tile table: my routed experts in id order, then the shared expert
  const bool mine = e < E && e / c.per == me;
  const int rows_e = mine ? tot : (e == E ? ca[me * Etot + E] : 0);
  const int nt = (rows_e + bt - 1) / bt;
  int st = nt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, st, o); if (lane >= o) st += a; }
  __syncthreads();
  if (lane == 31) wsum[w] = st;
  __syncthreads();
  if (w == 0) {
    int a = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int x = __shfl_up_sync(0xffffffffu, a, o); if (lane >= o) a += x; }
    wsum[lane] = a;
  }
  __syncthreads();
  const int tile0 = st - nt + (w ? wsum[w - 1] : 0);
  if (rows_e > 0) {
    const int local = e == E ? c.per : e - me * c.per;
    const int row0 = e == E ? G[(me + 1) * c.per] - G[me * c.per] : G[e] - G[me * c.per];
    for (int i = 0, ti = tile0; i * bt < rows_e && ti < max_tiles; ++i, ++ti)
      tiles[ti] = make_int4(local, row0 + i * bt, min(bt, rows_e - i * bt), 0);
  }
  if (e == E) {
    const int total_tiles = tile0 + nt;
    *n_tiles = total_tiles < max_tiles ? total_tiles : max_tiles;
    const int rows = G[(me + 1) * c.per] - G[me * c.per] + ca[me * Etot + E];
    *n_rows = rows;
    if (rows > c.cap_rows) atomicCAS(c.err, 0, ERR_BAD_INDEX);
  }
}

// One CTA per (row, pair) of this rank: copy the activation row into its host's sorted buffer.
__global__ void ep_dispatch_kernel(EpCtx c, const bf16* x, const int* idx, const int* send_base, int* cursors, int P,
                                   int H) {
  const int pair = blockIdx.x;
  const int e = idx[pair];
  if (e < 0 || e > c.E) return;
  const int host = e == c.E ? c.rank : e / c.per;
  __shared__ int s_pos;
  if (threadIdx.x == 0) s_pos = send_base[e] + atomicAdd(&cursors[e], 1);
  __syncthreads();
  const int pos = s_pos;
  if (pos >= c.cap_rows) { if (threadIdx.x == 0) atomicCAS(c.err, 0, ERR_BAD_INDEX); return; }
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(pair / P) * H);
  uint4* dst = reinterpret_cast<uint4*>(c.xs[host] + static_cast<size_t>(pos) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
  if (threadIdx.x == 0) c.meta[host][pos] = make_int2(c.rank, pair);
}

// Release flag `which` (1 = dispatch done, 2 = combine done) towards every rank, for the current epoch.
__global__ void ep_signal_kernel(EpCtx c, int which) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + which * MAX_RANKS + c.rank, c.epoch[0]);
  }
}
// Wait until every source has released flag `which` for the current epoch.
__global__ void ep_wait_kernel(EpCtx c, int which) {
  if (threadIdx.x < c.world) wait_flag(c.flags[c.rank] + which * MAX_RANKS + threadIdx.x, c.epoch[0], c.err);
}
// Both in one launch: thread r releases towards rank r, then waits for rank r's release.
__global__ void ep_signal_wait_kernel(EpCtx c, int which) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + which * MAX_RANKS + c.rank, c.epoch[0]);
    wait_flag(c.flags[c.rank] + which * MAX_RANKS + threadIdx.x, c.epoch[0], c.err);
  }
}

// out[t] = bf16(sum_j w[t, j] * pair_out[t * P + j]) in pair order, fp32 accumulation.
__global__ void ep_combine_kernel(const bf16* pair_out, const float* wts, int P, int H, bf16* out) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < P; ++j) {
      const float wv = wts[static_cast<size_t>(t) * P + j];
      uint4 pv = *reinterpret_cast<const uint4*>(pair_out + (static_cast<size_t>(t) * P + j) * H + i);
      const bf16* pe = reinterpret_cast<const bf16*>(&pv);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += wv * __bfloat162float(pe[k]);
    }
    uint4 ov;
    bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int k = 0; k < 8; ++k) oe[k] = __float2bfloat16(acc[k]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + i) = ov;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_ep_ctx_size() { return static_cast<int>(sizeof(EpCtx)); }

extern "C" int b200_ep_counts(const EpCtx* c, const int* counts, cudaStream_t st) {
  ep_counts_kernel<<<1, 256, 0, st>>>(*c, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_ep_plan(const EpCtx* c, int bt, int* send_base, int* cursors, void* tiles, int* n_tiles,
                            int max_tiles, int* n_rows, cudaStream_t st) {
  if (c->E + 1 > 1024) return -7;
  ep_plan_kernel<<<1, 1024, 0, st>>>(*c, bt, send_base, cursors, static_cast<int4*>(tiles), n_tiles, max_tiles, n_rows,
                                     nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
// Count exchange + plan in one launch (one CTA either way; saves a launch per MoE block).
extern "C" int b200_ep_counts_plan(const EpCtx* c, const int* counts, int bt, int* send_base, int* cursors, void* tiles,
                                   int* n_tiles, int max_tiles, int* n_rows, cudaStream_t st) {
  if (c->E + 1 > 1024) return -7;
  ep_plan_kernel<<<1, 1024, 0, st>>>(*c, bt, send_base, cursors, static_cast<int4*>(tiles), n_tiles, max_tiles, n_rows,
                                     counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_ep_dispatch(const EpCtx* c, const void* x, const int* idx, const int* send_base, int* cursors,
                                int n_pairs, int P, int H, cudaStream_t st) {
  if (n_pairs > 0)
    ep_dispatch_kernel<<<n_pairs, 128, 0, st>>>(*c, static_cast<const bf16*>(x), idx, send_base, cursors, P, H);
  ep_signal_wait_kernel<<<1, 32, 0, st>>>(*c, 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
extern "C" int b200_ep_combine(const EpCtx* c, const float* wts, int T, int P, int H, void* out, cudaStream_t st) {
  ep_signal_wait_kernel<<<1, 32, 0, st>>>(*c, 2);
  if (T > 0)
    ep_combine_kernel<<<T, 256, 0, st>>>(c->pair_out[c->rank], wts, P, H, static_cast<bf16*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
