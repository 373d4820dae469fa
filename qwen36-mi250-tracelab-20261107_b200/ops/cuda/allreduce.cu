// One-shot all-reduce over NVLink peer memory for decode-sized activations, with the residual add
// folded in: out = bf16(residual + sum_r partial_r), every rank pushing its partial into all
// peers' receive slots and adding the R partials in rank order (reference: the in-graph
// "LL" all-reduce, engine/fast/tp.py:121-184, which does the same between two ranks with the flag
// packed into each data word; here a block-level release/acquire flag covers 16 KB of payload).
//
// A loopback mode (world == 1, or every pointer of the context naming this rank's own buffers)
// exercises the whole protocol on a single GPU inside ONE kernel; ranks are never emulated as
// separate launches that wait on one another.
#include "comm.cuh"

namespace b200 {

constexpr int AR_THREADS = 256;
constexpr int AR_ELEMS = 4096;  // floats per block

template <typename TIn>
__device__ __forceinline__ float to_f(TIn v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

// With `norm_w` (rows of H elements, H dividing the block's 4096 elements, so a block owns whole rows) the kernel also
// applies the zero-centred RMSNorm that follows the residual add: y = norm(out) * (1 + norm_w), with the rounding
// points of add_rmsnorm_kernel (the sum is rounded to bf16, the residual added, rounded again; the norm reads those
// bf16 values). One launch replaces all-reduce + add + norm (reference: engine/fast/tp.py:220-257).
template <typename TIn>
__global__ void __launch_bounds__(AR_THREADS)
allreduce_push_kernel(CommCtx c, const TIn* in, const bf16* residual, bf16* out, float* out_f32, size_t n,
                      const bf16* norm_w, bf16* y, int H, float eps) {
  __shared__ float s_row[AR_ELEMS];   // norm: the block's new residual rows as the bf16 values just stored
  __shared__ float s_ss[AR_ELEMS / 64];
  const int blk = blockIdx.x;
  const size_t base = static_cast<size_t>(blk) * AR_ELEMS;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = c.epoch[blk] + 1;
    c.epoch[blk] = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  // push my partial into every rank's slot [e & 1][my rank]
  for (int i = threadIdx.x * 4; i < AR_ELEMS; i += AR_THREADS * 4) {
    const size_t g = base + i;
    if (g >= n) break;
    float4 v;
    v.x = to_f<TIn>(in[g]);
    v.y = g + 1 < n ? to_f<TIn>(in[g + 1]) : 0.f;
    v.z = g + 2 < n ? to_f<TIn>(in[g + 2]) : 0.f;
    v.w = g + 3 < n ? to_f<TIn>(in[g + 3]) : 0.f;
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<float4*>(comm_slot(c, r, e, c.rank) + g) = v;
  }
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + static_cast<size_t>(c.rank) * c.max_blocks + blk, e);
  }
  if (threadIdx.x < c.world) {
    if (!wait_flag(c.flags[c.rank] + static_cast<size_t>(threadIdx.x) * c.max_blocks + blk, e, c.err)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;  // status word set; output left untouched
  for (int i = threadIdx.x * 4; i < AR_ELEMS; i += AR_THREADS * 4) {
    const size_t g = base + i;
    if (g >= n) break;
    float4 acc = *reinterpret_cast<const float4*>(comm_slot(c, c.rank, e, 0) + g);
    for (int r = 1; r < c.world; ++r) {
      const float4 v = *reinterpret_cast<const float4*>(comm_slot(c, c.rank, e, r) + g);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (g + k >= n) break;
      float v = a[k];
      if (out_f32) out_f32[g + k] = v;
      if (out) {
        if (residual) v = __bfloat162float(__float2bfloat16(v)) + __bfloat162float(residual[g + k]);
        const bf16 o = __float2bfloat16(v);
        out[g + k] = o;
        if (norm_w) s_row[i + k] = __bfloat162float(o);
      }
    }
  }
  if (norm_w == nullptr) return;
  __syncthreads();
  // rows of this block: r = 0 .. AR_ELEMS / H - 1; one warp per row at a time
  const int rows_here = AR_ELEMS / H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < rows_here; r += AR_THREADS / 32) {
    if (base + static_cast<size_t>(r) * H >= n) break;
    float ss = 0.f;
    for (int i = lane; i < H; i += 32) { const float f = s_row[r * H + i]; ss += f * f; }
    ss = warp_sum(ss);
    if (lane == 0) s_ss[r] = rsqrtf(ss / H + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < AR_ELEMS; i += AR_THREADS) {
    const size_t g = base + i;
    if (g >= n) break;
    const int r = i / H, col = i - r * H;
    y[g] = __float2bfloat16(s_row[i] * s_ss[r] * (1.0f + __bfloat162float(norm_w[col])));
  }
}

}  // namespace b200

using namespace b200;

// `n` elements (a multiple of 4, at most slot_elems); in_is_f32 selects the partial's dtype.
// out (bf16, optional residual added) and/or out_f32 receive the sum.
extern "C" int b200_allreduce_push(const CommCtx* ctx, const void* in, int in_is_f32, const void* residual, void* out,
                                   float* out_f32, unsigned long long n, cudaStream_t st) {
  if (n == 0) return 0;
  if (n % 4 || n > ctx->slot_elems) return -7;
  const int blocks = static_cast<int>((n + AR_ELEMS - 1) / AR_ELEMS);
  if (blocks > ctx->max_blocks) return -7;
  if (in_is_f32)
    allreduce_push_kernel<float><<<blocks, AR_THREADS, 0, st>>>(*ctx, static_cast<const float*>(in),
                                                               static_cast<const bf16*>(residual),
                                                               static_cast<bf16*>(out), out_f32, n, nullptr, nullptr, 0, 0.f);
  else
    allreduce_push_kernel<bf16><<<blocks, AR_THREADS, 0, st>>>(*ctx, static_cast<const bf16*>(in),
                                                              static_cast<const bf16*>(residual),
                                                              static_cast<bf16*>(out), out_f32, n, nullptr, nullptr, 0, 0.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// All-reduce of rows [T, H] + residual add + the RMSNorm that follows, in one launch: out = bf16(bf16(sum) + residual)
// (residual optional), y = norm(out) * (1 + norm_w). H must divide 4096 (a block of the all-reduce owns whole rows).
extern "C" int b200_allreduce_push_norm(const CommCtx* ctx, const void* in, int in_is_f32, const void* residual,
                                        void* out, const void* norm_w, void* y, int T, int H, float eps,
                                        cudaStream_t st) {
  const unsigned long long n = static_cast<unsigned long long>(T) * H;
  if (n == 0) return 0;
  if (H < 64 || AR_ELEMS % H || n > ctx->slot_elems) return -7;
  const int blocks = static_cast<int>((n + AR_ELEMS - 1) / AR_ELEMS);
  if (blocks > ctx->max_blocks) return -7;
  if (in_is_f32)
    allreduce_push_kernel<float><<<blocks, AR_THREADS, 0, st>>>(
        *ctx, static_cast<const float*>(in), static_cast<const bf16*>(residual), static_cast<bf16*>(out), nullptr, n,
        static_cast<const bf16*>(norm_w), static_cast<bf16*>(y), H, eps);
  else
    allreduce_push_kernel<bf16><<<blocks, AR_THREADS, 0, st>>>(
        *ctx, static_cast<const bf16*>(in), static_cast<const bf16*>(residual), static_cast<bf16*>(out), nullptr, n,
        static_cast<const bf16*>(norm_w), static_cast<bf16*>(y), H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ------------------------------------------------------------------ symmetric memory (CUDA IPC)
// ------------------------------------------------------------------ RMSNorm + all-gather push
// Sequence-parallel half of a tensor-parallel layer: after a GEMM -> reduce-scatter each rank owns `rows` token
// rows of the residual stream. This kernel normalises the rank's rows and stores every normalised row straight
// into the full activation buffer of EVERY rank (peer stores over NVLink; `xfull[r]` is rank r's [R * rows, H]
// buffer), so the all-gather needs no separate pass. The last CTA to finish publishes the arrival epoch of this
// rank's shard on every rank; the consuming GEMM (b200_gemm_gathered) waits for exactly the shards its tile reads.
struct AgCtx {
  bf16* xfull[MAX_RANKS];
  uint32_t* flags[MAX_RANKS];  // rank r's arrival epochs, uint32 [R sources]
  uint32_t* epoch;             // this rank's call counter (device-resident: graph-capturable)
  uint32_t* counter;           // CTAs of the current call that have finished
  int rank, world;
};

// REDUCE: the rows come from a GEMM -> reduce-scatter (gemm_tcgen05.cu, EPI_REDUCE_SCATTER): wait for the arrival
// flags of the row's tiles (gx tiles of 128 columns x R sources), add the R fp32 partials in rank order, round to
// bf16, add the residual, store the new residual row, then normalise. Otherwise x is the row itself.
template <bool ZERO_CENTRED, bool REDUCE>
__global__ void reduce_norm_allgather_kernel(AgCtx c, CommCtx cc, const bf16* x, const bf16* res, bf16* res_out,
                                             const bf16* w, int rows, int H, float eps, int bt) {
  extern __shared__ float vals[];  // H floats
  const size_t row = static_cast<size_t>(blockIdx.x) * H;
  __shared__ int s_ok;
  if (REDUCE) {
    const int gx = (H + 127) / 128;
    const int by = (cc.rank * rows + blockIdx.x) / bt;  // token tile of this row in the GEMM's grid
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    for (int i = threadIdx.x; i < gx * cc.world; i += blockDim.x) {
      const int nx = i % gx, src = i / gx;
      const int blk = by * gx + nx;
      if (!wait_flag(cc.flags[cc.rank] + static_cast<size_t>(src) * cc.max_blocks + blk, cc.epoch[blk], cc.err)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;  // the error word is set; the shard's epoch is never published, consumers time out the same way
  }
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8];
    if (REDUCE) {
      const uint32_t ei = cc.epoch[((cc.rank * rows + blockIdx.x) / bt) * ((H + 127) / 128) + i / 128];
      const float4* s0 = reinterpret_cast<const float4*>(comm_slot(cc, cc.rank, ei, 0) + row + i);
      float4 a = s0[0], b = s0[1];
      for (int r = 1; r < cc.world; ++r) {
        const float4* sr = reinterpret_cast<const float4*>(comm_slot(cc, cc.rank, ei, r) + row + i);
        const float4 a2 = sr[0], b2 = sr[1];
        a.x += a2.x; a.y += a2.y; a.z += a2.z; a.w += a2.w;
        b.x += b2.x; b.y += b2.y; b.z += b2.z; b.w += b2.w;
      }
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      uint4 rv;
      const bf16* re = reinterpret_cast<const bf16*>(&rv);
      if (res) rv = *reinterpret_cast<const uint4*>(res + row + i);
      uint4 ov;
      bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        bf16 s = __float2bfloat16(f[j]);
        if (res) s = __float2bfloat16(__bfloat162float(s) + __bfloat162float(re[j]));
        oe[j] = s;
        f[j] = __bfloat162float(s);
      }
      if (res_out) *reinterpret_cast<uint4*>(res_out + row + i) = ov;
    } else {
      uint4 xv = *reinterpret_cast<const uint4*>(x + row + i);
      const bf16* xe = reinterpret_cast<const bf16*>(&xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(xe[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      vals[i + j] = f[j];
      ss += f[j] * f[j];
    }
  }
  __shared__ float part[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += part[i];  // fixed order
  const float inv = rsqrtf(tot / H + eps);
  const size_t grow = (static_cast<size_t>(c.rank) * rows + blockIdx.x) * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const bf16* we = reinterpret_cast<const bf16*>(&wv);
    uint4 ov;
    bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = ZERO_CENTRED ? 1.0f + __bfloat162float(we[j]) : __bfloat162float(we[j]);
      oe[j] = __float2bfloat16(vals[i + j] * inv * g);
    }
    for (int r = 0; r < c.world; ++r) *reinterpret_cast<uint4*>(c.xfull[r] + grow + i) = ov;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(c.counter, 1u);
    if (done == gridDim.x - 1) {
      __threadfence_system();
      *c.counter = 0;
      const uint32_t en = *c.epoch + 1;
      *c.epoch = en;
      for (int r = 0; r < c.world; ++r) st_release_sys(c.flags[r] + c.rank, en);
    }
  }
}

// comm == nullptr: plain rows `x` [rows, H]. Otherwise the rows are reduced from the receive slots that a preceding
// b200_gemm_reduce_scatter with token tile `bt` filled; `res` (may be null) is added, `res_out` (may be null, may
// alias `res`) receives the new residual rows.
extern "C" int b200_reduce_norm_allgather(const AgCtx* ctx, const CommCtx* comm, const void* x, const void* res,
                                          void* res_out, const void* w, int rows, int H, float eps, int zero_centred,
                                          int bt, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (H % 8) return -7;
  const int threads = H >= 2048 ? 256 : 128;
  const size_t sm = H * sizeof(float);
  const bf16 *xb = static_cast<const bf16*>(x), *rb = static_cast<const bf16*>(res), *wb = static_cast<const bf16*>(w);
  bf16* ro = static_cast<bf16*>(res_out);
  if (comm) {
    if (bt <= 0 || rows % bt || static_cast<unsigned long long>(rows) * H > comm->slot_elems) return -7;
    if (zero_centred) reduce_norm_allgather_kernel<true, true><<<rows, threads, sm, st>>>(*ctx, *comm, xb, rb, ro, wb, rows, H, eps, bt);
    else reduce_norm_allgather_kernel<false, true><<<rows, threads, sm, st>>>(*ctx, *comm, xb, rb, ro, wb, rows, H, eps, bt);
  } else {
    if (zero_centred) reduce_norm_allgather_kernel<true, false><<<rows, threads, sm, st>>>(*ctx, CommCtx{}, xb, rb, ro, wb, rows, H, eps, bt);
    else reduce_norm_allgather_kernel<false, false><<<rows, threads, sm, st>>>(*ctx, CommCtx{}, xb, rb, ro, wb, rows, H, eps, bt);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
// Reduce-scatter push of an fp32 partial [T, N] that no GEMM epilogue produced (the expert-parallel MoE block's
// partial sums): tile (by, nx) of bt rows x 128 columns goes to the receive slot of the rank that owns its rows,
// with the same flags and epochs as the EPI_REDUCE_SCATTER epilogue, so b200_reduce_norm_allgather consumes
// either. T must be a multiple of world * bt.
__global__ void __launch_bounds__(256)
rs_push_kernel(CommCtx cc, const float* part, int N, int bt, int rows_per_rank) {
  const int nx = blockIdx.x, by = blockIdx.y;
  const int blk = by * gridDim.x + nx;
  const int row0 = by * bt, owner = row0 / rows_per_rank, lrow0 = row0 - owner * rows_per_rank;
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) { s_e = cc.epoch[blk] + 1; cc.epoch[blk] = s_e; }
  __syncthreads();
  const uint32_t e = s_e;
  float* dst = comm_slot(cc, owner, e, cc.rank);
  const int cols = min(128, N - nx * 128);  // N is a multiple of 4
  for (int idx = threadIdx.x; idx < bt * 32; idx += blockDim.x) {
    const int r = idx >> 5, c4 = (idx & 31) * 4;
    if (c4 < cols)
      *reinterpret_cast<float4*>(dst + static_cast<size_t>(lrow0 + r) * N + nx * 128 + c4) =
          *reinterpret_cast<const float4*>(part + static_cast<size_t>(row0 + r) * N + nx * 128 + c4);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(cc.flags[owner] + static_cast<size_t>(cc.rank) * cc.max_blocks + blk, e);
}

extern "C" int b200_rs_push(const CommCtx* ctx, const float* part, int T, int N, int bt, cudaStream_t st) {
  if (T <= 0) return 0;
  if (bt <= 0 || T % (ctx->world * bt) || N % 4) return -7;
  const int rpr = T / ctx->world, gx = (N + 127) / 128, gy = T / bt;
  if (static_cast<unsigned long long>(rpr) * N > ctx->slot_elems || gx * gy > ctx->max_blocks) return -7;
  rs_push_kernel<<<dim3(gx, gy), 256, 0, st>>>(*ctx, part, N, bt, rpr);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Wait until every rank's shard of the current all-gather has arrived (for a consumer that is not a gathered GEMM).
__global__ void ag_wait_kernel(const uint32_t* flags, const uint32_t* epoch, int world, int* err) {
  if (static_cast<int>(threadIdx.x) < world) wait_flag(flags + threadIdx.x, *epoch, err);
}
extern "C" int b200_ag_wait(const AgCtx* ctx, int* err, cudaStream_t st) {
  ag_wait_kernel<<<1, 32, 0, st>>>(ctx->flags[ctx->rank], ctx->epoch, ctx->world, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int b200_ag_ctx_size() { return static_cast<int>(sizeof(AgCtx)); }

extern "C" int b200_symm_alloc(void** ptr, unsigned long long bytes) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -1;
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? 0 : -2;
}
extern "C" int b200_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int b200_symm_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int b200_symm_import(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
extern "C" int b200_symm_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int b200_comm_ctx_size() { return static_cast<int>(sizeof(CommCtx)); }
