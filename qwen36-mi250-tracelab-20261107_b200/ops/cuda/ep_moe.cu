// Expert-parallel MoE over NVLink peer memory for token-sharded activations: every rank holds its own
// rows and E / R of the routed experts (plus a replica of the shared expert).
//
//   ep_route_send : routing and the dispatch all-to-all in one launch. One CTA per row: its first warp turns the
//                 row's router logits into (expert, weight) pairs, then one warp per pair stores the activation
//                 row straight into the hosting rank's receive buffer, in the region reserved for this source rank,
//                 in arrival order, with (local expert, pair index) beside it. Nothing has to be agreed beforehand:
//                 the last CTA to finish publishes how many rows each host got and releases this source's arrival
//                 flag there.
//   ep_plan     : on the host, waits for every source's flag (the one rendezvous of the dispatch), then sorts the
//                 received rows by expert WITHOUT moving them: the token-tile table of the grouped GEMMs plus, for
//                 every sorted position, the row of the receive buffer behind it (the gate/up GEMM's producer
//                 fetches rows by that index) and where its result goes (source rank, pair index).
//   grouped GEMMs (gemm_tcgen05.cu): gate/up + SiLU-mul over the received rows, then the down projection whose
//                 epilogue stores each output row into the pair slot of the token's owner (the combine
//                 all-to-all, peer stores from the epilogue).
//   ep_combine  : releases "my results are out" towards every rank, waits for every host's release (the one
//                 rendezvous of the combine), then the top-k weighted sum in pair order, optionally with the
//                 residual add and the next RMSNorm.
//
// Two waits per MoE block, both inside kernels that do other work, no count exchange, no separate signal launches.
// The reference has no expert parallelism (its TP halves every expert, engine/fast/tp.py:19-21, 716-736).
// All buffers are symmetric CUDA IPC mappings; flags carry a device-resident epoch so that the sequence can
// be captured in a CUDA graph. No multimem, no TMA on peer memory. Every wait is bounded (comm.cuh).
//
// Buffer reuse between consecutive calls needs no extra synchronisation: a source can only start the next call's
// sends after its own combine, which waited for every host's release, which a host issues after its down GEMM (and
// so after its gate/up GEMM has read the receive buffer); a host can only overwrite a rank's pair slots after its
// next plan, which waited for that rank's next send, which follows that rank's combine.
#include "comm.cuh"
#include "moe_route.cuh"

namespace b200 {

struct EpCtx {
  bf16* xs[MAX_RANKS];          // receive buffer of each rank: [R source regions][cap_src rows][H]
  int2* meta[MAX_RANKS];        // per received row: (local expert, pair index at the source)
  bf16* pair_out[MAX_RANKS];    // [max_pairs, H] expert outputs returned to each rank
  unsigned long long* arrive[MAX_RANKS];  // [R] per source: (call epoch << 32) | rows that source sent to this rank
                                // in that call: count and arrival flag travel in ONE release store
  uint32_t* flags[MAX_RANKS];   // [2][MAX_RANKS]: row 1 = combine arrival epochs per source (row 0 unused)
  uint32_t* epoch;              // this rank's call counter (device resident)
  int* cursors;                 // this rank's send cursors [R] and the CTA ticket [1]; zero between calls
  int* err;
  int rank, world;
  int E;                        // routed experts (global); expert id E is the shared expert, hosted by everyone
  int per;                      // routed experts per rank
  int cap_src, max_pairs;
  long long wait_cycles;        // clock ticks a peer wait may take before it gives up with ERR_WAIT_PEER
};

// Last CTA out: release (epoch, rows sent) of this source on every host. The CTA's peer stores
// are ordered before the ticket by the barrier followed by ONE system-scope fence of the thread that takes the
// ticket (a fence per thread cost 3x the kernel's time: the profile showed every warp stalled on it).
__device__ __forceinline__ void ep_send_finish(const EpCtx& c) {
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&c.cursors[MAX_RANKS], 1) == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  const uint32_t e = c.epoch[0] + 1;
  if (threadIdx.x < c.world) {
    const int r = threadIdx.x;
    const int n = atomicAdd(&c.cursors[r], 0);
    const unsigned long long word = (static_cast<unsigned long long>(e) << 32) | static_cast<unsigned>(n < c.cap_src ? n : c.cap_src);
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(c.arrive[r] + c.rank), "l"(word) : "memory");
    c.cursors[r] = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) { c.cursors[MAX_RANKS] = 0; c.epoch[0] = e; }
}

// One pair of one row by the calling warp: take the next slot of this source's region on the expert's host, store the
// row and its (local expert, pair index) there.
__device__ __forceinline__ void ep_send_pair(const EpCtx& c, const bf16* xrow, int e, int pair, int H, int lane) {
  if (e < 0 || e > c.E) {
    if (lane == 0) atomicCAS(c.err, 0, ERR_BAD_INDEX);
    return;
  }
  const int host = e == c.E ? c.rank : e / c.per;
  const int local = e == c.E ? c.per : e - host * c.per;
  int pos = lane == 0 ? atomicAdd(&c.cursors[host], 1) : 0;
  pos = __shfl_sync(0xffffffffu, pos, 0);
  if (pos < c.cap_src) {
    const size_t slot = static_cast<size_t>(c.rank) * c.cap_src + pos;
    const uint4* src = reinterpret_cast<const uint4*>(xrow);
    uint4* dst = reinterpret_cast<uint4*>(c.xs[host] + slot * H);
    for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
    if (lane == 0) c.meta[host][slot] = make_int2(local, pair);
  } else if (lane == 0) {
    atomicCAS(c.err, 0, ERR_BAD_INDEX);  // more rows for one host than its region holds
  }
}

// Routing fused with the dispatch: one CTA of 32 * P threads per row (at least one CTA). Warp 0 routes the row
// (softmax, top-k, ties to the lower id, bf16-rounded weights; the shared expert as pair P - 1) into `wts` / `idx`,
// then warp p sends pair p.
template <int PER_LANE>
__global__ void ep_route_send_kernel(EpCtx c, const bf16* x, const float* logits, int ldl, int T, int top_k, int P,
                                     int H, float* wts, int* idx) {
  pdl_wait();
  pdl_launch();
  __shared__ int s_idx[32];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (row < T) {
    if (warp == 0) {
      route_row<PER_LANE>(logits + static_cast<size_t>(row) * ldl, c.E, top_k, P > top_k ? 1 : 0,
                          wts + static_cast<size_t>(row) * P, s_idx, nullptr, nullptr, lane);
      __syncwarp();
      if (lane < P) idx[static_cast<size_t>(row) * P + lane] = s_idx[lane];
    }
    __syncthreads();
    if (warp < P)
      ep_send_pair(c, x + static_cast<size_t>(row) * H, s_idx[warp], row * P + warp, H, lane);
  }
  ep_send_finish(c);
}

// One CTA of 1024 threads on the host side: wait for every source, then lay the received rows out by expert
// (local experts in id order, the shared expert last) without moving them.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(EpCtx c, int bt, int4* tiles, int* n_tiles, int max_tiles, int* gather_rows, int2* ret_meta,
               int* n_rows) {
  const int R = c.world, me = c.rank, El = c.per + 1;
  __shared__ int s_cnt[MAX_RANKS];
  __shared__ int s_count[1024], s_off[1024], s_cur[1024];
  __shared__ int w_rows[32], w_tiles[32];
  __shared__ int s_ok;
  const int e = threadIdx.x, lane = e & 31, w = e >> 5;
  if (e == 0) s_ok = 1;
  s_count[e] = 0;
  s_cur[e] = 0;
  pdl_wait();  // this rank's send kernel advanced the epoch
  pdl_launch();
  __syncthreads();
  if (e < R) {
    // bounded wait for source e's (epoch, count) word of this call
    const uint32_t want = c.epoch[0];
    const unsigned long long* p = c.arrive[me] + e;
    unsigned long long word;
    const long long t0 = clock64();
    bool ok = true;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(p) : "memory");
      if (static_cast<int32_t>(static_cast<uint32_t>(word >> 32) - want) >= 0) break;
      if (*reinterpret_cast<volatile int*>(c.err) != 0) { ok = false; break; }
      if (clock64() - t0 > c.wait_cycles) { atomicCAS(c.err, 0, ERR_WAIT_PEER); ok = false; break; }
      __nanosleep(20);
    }
    if (!ok) s_ok = 0;
    const int n = ok ? static_cast<int>(static_cast<uint32_t>(word)) : 0;
    s_cnt[e] = (n >= 0 && n <= c.cap_src) ? n : 0;
    if (n < 0 || n > c.cap_src) atomicCAS(c.err, 0, ERR_BAD_INDEX);
  }
  __syncthreads();
  if (!s_ok) {  // a source never arrived: publish an empty plan so that the GEMMs behind run zero tiles
    if (e == 0) { *n_tiles = 0; *n_rows = 0; }
    return;
  }
  const int2* meta = c.meta[me];
  for (int r = 0; r < R; ++r)
    for (int i = threadIdx.x; i < s_cnt[r]; i += blockDim.x) {
      const int le = meta[static_cast<size_t>(r) * c.cap_src + i].x;
      if (le >= 0 && le < El) atomicAdd(&s_count[le], 1);
    }
  __syncthreads();
  const int cn = e < El ? s_count[e] : 0;
  const int t = (cn + bt - 1) / bt;
  int sc = cn, stl = t;
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
  const int row0 = sc - cn + (w ? w_rows[w - 1] : 0);
  const int tile0 = stl - t + (w ? w_tiles[w - 1] : 0);
  s_off[e] = row0;
  if (e < El)
    for (int i = 0, ti = tile0; i * bt < cn && ti < max_tiles; ++i, ++ti)
      tiles[ti] = make_int4(e, row0 + i * bt, min(bt, cn - i * bt), 0);
  if (e == El - 1) {
    const int total = tile0 + t;
    *n_tiles = total < max_tiles ? total : max_tiles;
    *n_rows = row0 + cn;
  }
  __syncthreads();
  for (int r = 0; r < R; ++r)
    for (int i = threadIdx.x; i < s_cnt[r]; i += blockDim.x) {
      const int slot = r * c.cap_src + i;
      const int2 m = meta[slot];
      if (m.x < 0 || m.x >= El) { atomicCAS(c.err, 0, ERR_BAD_INDEX); continue; }
      const int pos = s_off[m.x] + atomicAdd(&s_cur[m.x], 1);
      gather_rows[pos] = slot;
      ret_meta[pos] = make_int2(r, m.y);
    }
}

// sorted[pos] = xs[rows[pos]] for the first *n_valid positions: the expert-sorted copy that token tiles wider than
// the gathering GEMM's limit (prefill sizes) read through their tensor map.
__global__ void ep_compact_kernel(const bf16* xs, const int* rows, const int* n_valid, int H, bf16* sorted) {
  pdl_wait();
  pdl_launch();
  // grid-stride over the rows that arrived: their number is known on the device only and may be far above what this
  // rank sent itself (a peer with a long prefill pass), so the grid is sized for the machine, not for a row count
  const int n = *n_valid;
  for (int pos = blockIdx.x; pos < n; pos += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(xs + static_cast<size_t>(rows[pos]) * H);
    uint4* dst = reinterpret_cast<uint4*>(sorted + static_cast<size_t>(pos) * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
  }
}

// Release "my expert outputs are out" towards every rank, wait for every host's release, then
// out[t] = bf16(sum_j w[t, j] * pair_out[t * P + j]) in pair order, fp32 accumulation. With NORM the launch also adds
// the residual and applies the next zero-centred RMSNorm with the rounding points of add_rmsnorm_kernel.
template <bool NORM>
__global__ void ep_combine_kernel(EpCtx c, const float* wts, int T, int P, int H, bf16* out, const bf16* res,
                                  const bf16* norm_w, bf16* res_out, bf16* y, float eps) {
  extern __shared__ float vals[];  // NORM: H floats
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  pdl_wait();  // the down projection's peer stores of this rank are complete
  pdl_launch();
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + 1 * MAX_RANKS + c.rank, c.epoch[0]);
  }
  if (threadIdx.x < c.world && !wait_flag(c.flags[c.rank] + 1 * MAX_RANKS + threadIdx.x, c.epoch[0], c.err, c.wait_cycles)) s_ok = 0;
  __syncthreads();
  const int t = blockIdx.x;
  if (!s_ok || t >= T) return;
  const bf16* pair_out = c.pair_out[c.rank];
  float ss = 0.f;
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
    if (NORM) {
      if (res) {
        uint4 rv = *reinterpret_cast<const uint4*>(res + static_cast<size_t>(t) * H + i);
        const bf16* re = reinterpret_cast<const bf16*>(&rv);
#pragma unroll
        for (int k = 0; k < 8; ++k) oe[k] = __float2bfloat16(__bfloat162float(oe[k]) + __bfloat162float(re[k]));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float f = __bfloat162float(oe[k]);
        vals[i + k] = f;
        ss += f * f;
      }
      *reinterpret_cast<uint4*>(res_out + static_cast<size_t>(t) * H + i) = ov;
    } else {
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + i) = ov;
    }
  }
  if (NORM) {
    __shared__ float part[32];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += part[i];
    const float inv_rms = rsqrtf(tot / H + eps);
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 wv = *reinterpret_cast<const uint4*>(norm_w + i);
      const bf16* we = reinterpret_cast<const bf16*>(&wv);
      uint4 ov;
      bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
      for (int k = 0; k < 8; ++k) oe[k] = __float2bfloat16(vals[i + k] * inv_rms * (1.0f + __bfloat162float(we[k])));
      *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + i) = ov;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_ep_ctx_size() { return static_cast<int>(sizeof(EpCtx)); }

// Routing of logits [T, ldl] (E routed experts + the shared expert's gate when P = top_k + 1) and the dispatch of
// x [T, H] in one launch; writes wts / idx [T, P] for the combine.
extern "C" int b200_ep_route_send(const EpCtx* c, const void* x, const float* logits, int ldl, int T, int top_k, int P,
                                  int H, float* wts, int* idx, cudaStream_t st) {
  if (H % 8 || P <= 0 || P > 32 || top_k > P || c->E > 32 * MAX_PER_LANE) return -7;
  auto k = c->E <= 256 ? ep_route_send_kernel<8> : ep_route_send_kernel<MAX_PER_LANE>;
  return launch_pdl(k, dim3(T > 0 ? T : 1), dim3(32 * P), 0, st, *c, static_cast<const bf16*>(x), logits, ldl, T, top_k,
                    P, H, wts, idx) == cudaSuccess ? 0 : -4;
}
extern "C" int b200_ep_plan(const EpCtx* c, int bt, void* tiles, int* n_tiles, int max_tiles, int* gather_rows,
                            void* ret_meta, int* n_rows, cudaStream_t st) {
  if (c->per + 1 > 1024) return -7;
  return launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, st, *c, bt, static_cast<int4*>(tiles), n_tiles, max_tiles,
                    gather_rows, static_cast<int2*>(ret_meta), n_rows) == cudaSuccess ? 0 : -4;
}
extern "C" int b200_ep_compact(const void* xs, const int* rows, const int* n_valid, int max_rows, int H, void* sorted,
                               cudaStream_t st) {
  if (max_rows <= 0) return 0;
  return launch_pdl(ep_compact_kernel, dim3(max_rows < 4096 ? max_rows : 4096), dim3(128), 0, st,
                    static_cast<const bf16*>(xs), rows, n_valid, H, static_cast<bf16*>(sorted)) == cudaSuccess ? 0 : -4;
}
// out [T, H] = weighted sum; or, with norm_w: res_out = bf16(res + sum), y = norm(res_out) * (1 + norm_w).
extern "C" int b200_ep_combine(const EpCtx* c, const float* wts, int T, int P, int H, void* out, const void* res,
                               const void* norm_w, void* res_out, void* y, float eps, cudaStream_t st) {
  if (H % 8) return -7;
  const int grid = T > 0 ? T : 1;
  if (norm_w != nullptr)
    return launch_pdl(ep_combine_kernel<true>, dim3(grid), dim3(256), H * sizeof(float), st, *c, wts, T, P, H,
                      static_cast<bf16*>(nullptr), static_cast<const bf16*>(res), static_cast<const bf16*>(norm_w),
                      static_cast<bf16*>(res_out), static_cast<bf16*>(y), eps) == cudaSuccess ? 0 : -4;
  return launch_pdl(ep_combine_kernel<false>, dim3(grid), dim3(256), 0, st, *c, wts, T, P, H, static_cast<bf16*>(out),
                    static_cast<const bf16*>(nullptr), static_cast<const bf16*>(nullptr), static_cast<bf16*>(nullptr),
                    static_cast<bf16*>(nullptr), 0.f) == cudaSuccess ? 0 : -4;
}
