// Row-wise glue kernels: embedding gather, zero-centred RMSNorm with residual add, the MoE
// routing / ordering / gather / combine steps around the grouped GEMMs.
//
// Reference counterparts: engine/fast/kernels.py:506-522 (add + RMSNorm), engine/fast/fused.py:553-579
// and engine/fast/prefill_kernels.py:194-230 (softmax/top-k, per-expert counts, expert order),
// engine/fast/moe_prefill.py:92-154 (device-side tile table), engine/fast/prefill_kernels.py:253-272
// (top-k weighted combine). Everything stays on the device: no host synchronisation between the
// router and the expert GEMMs.
#include "common.cuh"
#include "moe_route.cuh"
#include "moe_plan.cuh"

namespace b200 {

// ------------------------------------------------------------------ embedding
__global__ void embed_kernel(const int64_t* tokens, const bf16* table, bf16* out, int H, int vocab) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  int64_t tok = tokens[t];
  if (tok < 0 || tok >= vocab) tok = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + tok * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------ (add +) RMSNorm
// res' = bf16(res + x) (or x when res == nullptr); y = bf16(res' * rsqrt(mean(res'^2)+eps) * (1 + w)).
// One CTA per row, 8 elements per thread per step. `res_out` may alias `res` or `x`.
template <bool ZERO_CENTRED>
__global__ void add_rmsnorm_kernel(const bf16* x, const bf16* res, const bf16* w, bf16* res_out, bf16* y, int H,
                                   float eps) {
  pdl_wait();
  pdl_launch();
  const size_t row = static_cast<size_t>(blockIdx.x) * H;
  extern __shared__ float vals[];  // H floats
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + row + i);
    const bf16* xe = reinterpret_cast<const bf16*>(&xv);
    uint4 rv;
    const bf16* re = reinterpret_cast<const bf16*>(&rv);
    if (res) rv = *reinterpret_cast<const uint4*>(res + row + i);
    uint4 ov;
    bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      bf16 s = res ? __float2bfloat16(__bfloat162float(xe[j]) + __bfloat162float(re[j])) : xe[j];
      oe[j] = s;
      const float f = __bfloat162float(s);
      vals[i + j] = f;
      ss += f * f;
    }
    if (res_out) *reinterpret_cast<uint4*>(res_out + row + i) = ov;
  }
  __shared__ float part[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += part[i];  // fixed order
  const float inv = rsqrtf(tot / H + eps);
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
    *reinterpret_cast<uint4*>(y + row + i) = ov;
  }
}

// ------------------------------------------------------------------ MoE routing (route_row: moe_route.cuh)

// Grid of warps, one row each. `counts` (optional, zeroed by the caller) receives the rows per expert.
template <int PER_LANE>
__global__ void route_kernel(const float* logits, int ldl, int T, int E, int top_k, int shared, float* wts, int* idx,
                             int* counts, const int* expert_map) {
  pdl_wait();
  pdl_launch();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= T) return;
  const int P = top_k + (shared ? 1 : 0);
  route_row<PER_LANE>(logits + static_cast<size_t>(warp_global) * ldl, E, top_k, shared,
                      wts + static_cast<size_t>(warp_global) * P, idx + static_cast<size_t>(warp_global) * P, expert_map,
                      counts, lane);
}

// The expert plan (plan_scatter, moe_plan_kernel, moe_route_plan_kernel, moe_route_plan_grid_kernel,
// moe_scatter_kernel) lives in moe_plan.cuh.

// x_sorted[pos] = x[perm[pos] / P]
__global__ void moe_gather_kernel(const bf16* x, const int* perm, const int* n_valid, int T, int P, int H, bf16* xs) {
  pdl_wait();
  pdl_launch();
  const int pos = blockIdx.x;
  if (pos >= *n_valid) return;  // with expert parallelism only the locally served pairs are laid out
  const int t = perm[pos] / P;
  if (t < 0 || t >= T) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(pos) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t] = bf16( sum_j w[t,j] * pair_out[inv[t,j]] ) in pair order, fp32 accumulation, rounded once.
// With NORM the same launch also does what add_rmsnorm would do next: res' = bf16(res + out[t]) and
// y = bf16(res' * rsqrt(mean(res'^2) + eps) * (1 + w)) (zero-centred weight), with the same rounding points.
template <bool NORM>
__global__ void moe_combine_kernel(const bf16* pair_out, const float* wts, const int* inv, int P, int H, bf16* out,
                                   float* out_f32, const bf16* res, const bf16* norm_w, bf16* res_out, bf16* y,
                                   float eps) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float vals[];  // NORM: H floats
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < P; ++j) {
      const float wv = wts[static_cast<size_t>(t) * P + j];
      const int pos = inv[static_cast<size_t>(t) * P + j];
      if (pos < 0) continue;
      uint4 pv = *reinterpret_cast<const uint4*>(pair_out + static_cast<size_t>(pos) * H + i);
      const bf16* pe = reinterpret_cast<const bf16*>(&pv);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += wv * __bfloat162float(pe[k]);
    }
    if (!NORM && out_f32) {  // a partial sum that still has to be added across ranks
#pragma unroll
      for (int k = 0; k < 8; ++k) out_f32[static_cast<size_t>(t) * H + i + k] = acc[k];
      continue;
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
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += part[i];  // fixed order, as add_rmsnorm_kernel
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

// ------------------------------------------------------------------ MTP / speculative-chain glue
// Input of the MTP block for packed rows: out[t] = [ rmsnorm(embed[tok[t]]) * (1 + w_e) | rmsnorm(hidden[t]) * (1 + w_h) ]
// (zero-centred norms, fp32 math, bf16 out), one CTA per row (reference: _mtp_in_kernel, engine/fast/kernels.py:524-542).
__global__ void mtp_in_kernel(const int64_t* tokens, const bf16* embed, const bf16* hidden, const bf16* w_e,
                              const bf16* w_h, bf16* out, int H, int vocab, float eps) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  int64_t tok = tokens[t];
  if (tok < 0 || tok >= vocab) tok = 0;
  extern __shared__ float vals[];  // H floats
  __shared__ float part[32];
  for (int half = 0; half < 2; ++half) {
    const bf16* src = half == 0 ? embed + tok * H : hidden + static_cast<size_t>(t) * H;
    const bf16* w = half == 0 ? w_e : w_h;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 xv = *reinterpret_cast<const uint4*>(src + i);
      const bf16* xe = reinterpret_cast<const bf16*>(&xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = __bfloat162float(xe[j]);
        vals[i + j] = f;
        ss += f * f;
      }
    }
    ss = warp_sum(ss);
    __syncthreads();  // part[] of the first half has been read by everyone
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += part[i];
    const float inv = rsqrtf(tot / H + eps);
    bf16* dst = out + static_cast<size_t>(t) * 2 * H + half * H;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 wv = *reinterpret_cast<const uint4*>(w + i);
      const bf16* we = reinterpret_cast<const bf16*>(&wv);
      uint4 ov;
      bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
      for (int j = 0; j < 8; ++j) oe[j] = __float2bfloat16(vals[i + j] * inv * (1.0f + __bfloat162float(we[j])));
      *reinterpret_cast<uint4*>(dst + i) = ov;
    }
  }
}

// After a verify pass over G = k + 1 rows per sequence: the number of leading drafts that equal the model's pick of
// the row before them (acc), the MTP hidden of the last accepted row (the chain's first link starts from it), and
// the positions of the chain's later links. One CTA per sequence (reference: _chain_accept_kernel,
// engine/fast/kernels.py:544-571; _chain_next_kernel, engine/fast/tp.py:296-318).
__global__ void chain_accept_kernel(const int64_t* tokens, const int64_t* picks, const int* n_valid,
                                    const int64_t* positions, const bf16* y, int G, int H, int links, int B,
                                    int64_t* acc_out, bf16* h_sel, int64_t* link_pos) {
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.x;
  __shared__ int s_acc;
  if (threadIdx.x == 0) {
    int a = 0;
    const int nv = n_valid[b] < G - 1 ? n_valid[b] : G - 1;
    while (a < nv && tokens[static_cast<size_t>(b) * G + a + 1] == picks[static_cast<size_t>(b) * G + a]) ++a;
    s_acc = a;
    acc_out[b] = a;
    const int64_t base = positions[static_cast<size_t>(b) * G] + a + 1;
    for (int j = 0; j < links; ++j) link_pos[static_cast<size_t>(j) * B + b] = base + j;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(y + (static_cast<size_t>(b) * G + s_acc) * H);
  uint4* dst = reinterpret_cast<uint4*>(h_sel + static_cast<size_t>(b) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

}  // namespace b200

using namespace b200;

#define CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? 0 : -4
#define LAUNCHED(expr) return (expr) == cudaSuccess ? 0 : -4

extern "C" int b200_embed(const int64_t* tokens, const void* table, void* out, int T, int H, int vocab, cudaStream_t st) {
  if (T <= 0) return 0;
  LAUNCHED(launch_pdl(embed_kernel, dim3(T), dim3(128), 0, st, tokens, static_cast<const bf16*>(table),
                      static_cast<bf16*>(out), H, vocab));
}

extern "C" int b200_add_rmsnorm(const void* x, const void* res, const void* w, void* res_out, void* y, int T, int H,
                                float eps, int zero_centred, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -7;
  const int threads = H >= 2048 ? 256 : 128;
  auto k = zero_centred ? add_rmsnorm_kernel<true> : add_rmsnorm_kernel<false>;
  LAUNCHED(launch_pdl(k, dim3(T), dim3(threads), H * sizeof(float), st, static_cast<const bf16*>(x),
                      static_cast<const bf16*>(res), static_cast<const bf16*>(w), static_cast<bf16*>(res_out),
                      static_cast<bf16*>(y), H, eps));
}

// Routing only (any number of rows). `counts` may be null; when given it is zeroed here and receives rows per expert.
extern "C" int b200_moe_route(const float* logits, int ldl, int T, int E, int top_k, int shared, float* wts, int* idx,
                              int* counts, int n_counts, const int* expert_map, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_PER_LANE || top_k > 32) return -7;
  if (counts) cudaMemsetAsync(counts, 0, sizeof(int) * n_counts, st);
  auto k = E <= 256 ? route_kernel<8> : route_kernel<MAX_PER_LANE>;
  LAUNCHED(launch_pdl(k, dim3((T + 3) / 4), dim3(128), 0, st, logits, ldl, T, E, top_k, shared, wts, idx, counts,
                      expert_map));
}

// Expert-sorted layout of the (row, pair) table `idx` [n_pairs]: offsets [Et + 1], tile table, perm / inv [n_pairs].
// `src_rows` (optional, [n_pairs]) receives row = pair / P of every sorted position.
extern "C" int b200_moe_plan(const int* idx, int n_pairs, int Et, int bt, int* offsets, void* tiles, int* n_tiles,
                             int max_tiles, int* perm, int* inv, int* err, int P, int* src_rows, cudaStream_t st) {
  if (Et > 1024 || P <= 0) return -7;
  LAUNCHED(launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, st, idx, n_pairs, Et, bt, offsets,
                      static_cast<int4*>(tiles), n_tiles, max_tiles, perm, inv, err, P, src_rows));
}

// Routing and plan in one launch (two above 512 rows). `ticket`: a zero-initialised area of 1 + 2 * 1024 words that the
// kernels leave zero (the ticket, then per-expert counts and cursors for the large sizes); with at most 32 rows a
// single CTA does everything and the area is not touched.
extern "C" int b200_moe_route_plan(const float* logits, int ldl, int T, int E, int top_k, int shared, float* wts,
                                   int* idx, const int* expert_map, int Et, int bt, int* offsets, void* tiles,
                                   int* n_tiles, int max_tiles, int* perm, int* inv, int* err, int* src_rows,
                                   unsigned int* ticket, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 32 * MAX_PER_LANE || top_k > 32 || Et > 1024) return -7;
  if (T <= 32 || ticket == nullptr) {
    auto k = E <= 256 ? moe_route_plan_kernel<8> : moe_route_plan_kernel<MAX_PER_LANE>;
    LAUNCHED(launch_pdl(k, dim3(1), dim3(1024), 0, st, logits, ldl, T, E, top_k, shared, wts, idx, expert_map, Et, bt,
                        offsets, static_cast<int4*>(tiles), n_tiles, max_tiles, perm, inv, err, src_rows));
  }
  auto k = E <= 256 ? moe_route_plan_grid_kernel<8> : moe_route_plan_grid_kernel<MAX_PER_LANE>;
  // prefill sizes with a work area: histogram by all CTAs, scan by the last one, positions by a second launch
  int* work = (T > 512 && ticket != nullptr) ? reinterpret_cast<int*>(ticket + 1) : nullptr;
  if (launch_pdl(k, dim3((T + 31) / 32), dim3(1024), 0, st, logits, ldl, T, E, top_k, shared, wts, idx, expert_map, Et,
                 bt, offsets, static_cast<int4*>(tiles), n_tiles, max_tiles, perm, inv, err, src_rows, ticket,
                 work) != cudaSuccess)
    return -4;
  if (work == nullptr) return 0;
  const int n_pairs = T * (top_k + (shared ? 1 : 0));
  LAUNCHED(launch_pdl(moe_scatter_kernel, dim3(min((n_pairs + 255) / 256, 592)), dim3(256), 0, st,
                      static_cast<const int*>(idx), n_pairs, Et, static_cast<const int*>(offsets), work + 1024, perm, inv,
                      err, top_k + (shared ? 1 : 0), src_rows));
}

extern "C" int b200_moe_gather(const void* x, const int* perm, const int* n_valid, int n_pairs, int T, int P, int H,
                               void* xs, cudaStream_t st) {
  if (n_pairs <= 0) return 0;
  LAUNCHED(launch_pdl(moe_gather_kernel, dim3(n_pairs), dim3(128), 0, st, static_cast<const bf16*>(x), perm, n_valid, T,
                      P, H, static_cast<bf16*>(xs)));
}

extern "C" int b200_moe_combine(const void* pair_out, const float* wts, const int* inv, int T, int P, int H, void* out,
                                float* out_f32, cudaStream_t st) {
  if (T <= 0) return 0;
  LAUNCHED(launch_pdl(moe_combine_kernel<false>, dim3(T), dim3(256), 0, st, static_cast<const bf16*>(pair_out), wts,
                      inv, P, H, static_cast<bf16*>(out), out_f32, static_cast<const bf16*>(nullptr),
                      static_cast<const bf16*>(nullptr), static_cast<bf16*>(nullptr), static_cast<bf16*>(nullptr), 0.f));
}

// Combine, residual add and the next (zero-centred) RMSNorm in one launch: res_out = bf16(res + combine),
// y = norm(res_out) * (1 + norm_w). `res` may be null (res_out = combine).
extern "C" int b200_moe_combine_norm(const void* pair_out, const float* wts, const int* inv, int T, int P, int H,
                                     const void* res, const void* norm_w, void* res_out, void* y, float eps,
                                     cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -7;
  LAUNCHED(launch_pdl(moe_combine_kernel<true>, dim3(T), dim3(256), H * sizeof(float), st,
                      static_cast<const bf16*>(pair_out), wts, inv, P, H, static_cast<bf16*>(nullptr),
                      static_cast<float*>(nullptr), static_cast<const bf16*>(res), static_cast<const bf16*>(norm_w),
                      static_cast<bf16*>(res_out), static_cast<bf16*>(y), eps));
}

extern "C" int b200_mtp_in(const int64_t* tokens, const void* embed, const void* hidden, const void* w_e,
                           const void* w_h, void* out, int T, int H, int vocab, float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -7;
  LAUNCHED(launch_pdl(mtp_in_kernel, dim3(T), dim3(H >= 2048 ? 256 : 128), H * sizeof(float), st, tokens,
                      static_cast<const bf16*>(embed), static_cast<const bf16*>(hidden), static_cast<const bf16*>(w_e),
                      static_cast<const bf16*>(w_h), static_cast<bf16*>(out), H, vocab, eps));
}

// tokens / picks / positions [B * G] int64, n_valid [B] int32, y [B * G, H]; acc [B] int64, h_sel [B, H],
// link_pos [links, B] int64 (positions of chain links 2 .. links + 1).
extern "C" int b200_chain_accept(const int64_t* tokens, const int64_t* picks, const int* n_valid,
                                 const int64_t* positions, const void* y, int B, int G, int H, int links, int64_t* acc,
                                 void* h_sel, int64_t* link_pos, cudaStream_t st) {
  if (B <= 0) return 0;
  if (H % 8 || G < 1) return -7;
  LAUNCHED(launch_pdl(chain_accept_kernel, dim3(B), dim3(128), 0, st, tokens, picks, n_valid, positions,
                      static_cast<const bf16*>(y), G, H, links, B, acc, static_cast<bf16*>(h_sel), link_pos));
}

// Kernels launched through this library so far (see launch_counter in common.cuh).
extern "C" unsigned long long b200_launch_count() { return launch_counter(); }
