// Gated full-attention decode path over the paged KV pool.
//
//  attn_prep:    split the merged q|gate|k|v projection row, zero-centred RMSNorm of q and k per
//                head, partial RoPE on the first `rot` dims, write k and v into the sequence's page
//                (reference: engine/fast/fused.py:476-528).
//  paged_attn:   flash-decoding of G query rows per sequence against its pages. One CTA per
//                (sequence, kv head, lane z of Z); warp w serves query head w of the GQA group.
//                CTA z walks pages z, z+Z, z+2Z, ... with one running online softmax, so the
//                reduction order of a sequence depends only on its own length, never on the batch
//                (reference: engine/fast/kernels.py:377-443 splits the context the same way).
//  attn_combine: merge the Z partials in order, multiply by sigmoid(gate), store bf16
//                (reference: engine/fast/fused.py:530-551).
//
// KV layout: kv[page][2][n_kv][PAGE][D] bf16; page tables int32 [B, max_pages]; page 0 is scratch.
#include "common.cuh"

namespace b200 {

constexpr int PAGE = 64;

// PER consecutive bf16 (PER = 1, 2, 4 or 8) as floats with one vector load.
template <int PER>
__device__ __forceinline__ void load_bf16_vec(const bf16* p, float* out) {
  if constexpr (PER == 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __bfloat162float(e[i]);
  } else if constexpr (PER == 4) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __bfloat162float(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) out[i] = __bfloat162float(p[i]);
  }
}

// PER consecutive floats rounded to bf16 with one vector store; copy_bf16_vec moves PER bf16 as they are.
template <int PER>
__device__ __forceinline__ void store_bf16_vec(bf16* p, const float* v) {
  bf16 e[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) e[i] = __float2bfloat16(v[i]);
  if constexpr (PER == 8) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(e);
  else if constexpr (PER == 4) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(e);
  else {
#pragma unroll
    for (int i = 0; i < PER; ++i) p[i] = e[i];
  }
}
template <int PER>
__device__ __forceinline__ void copy_bf16_vec(bf16* dst, const bf16* src) {
  if constexpr (PER == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  else if constexpr (PER == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
  else {
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[i] = src[i];
  }
}

template <int D>
__global__ void attn_prep_kernel(const bf16* qkv, int ld, const int64_t* positions, const int* tables, int max_pages,
                                 const int* seq_of_row, const bf16* q_norm, const bf16* k_norm, bf16* q_out,
                                 bf16* gate_out, bf16* kv, int n_q, int n_kv, int rot, float theta, float eps,
                                 int num_pages, int* err) {
  // one warp per (row, head); heads: [0,n_q) query, [n_q, n_q+n_kv) key, then value
  pdl_wait();
  pdl_launch();
  const int row = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (head >= n_q + 2 * n_kv) return;
  constexpr int PER = D / 32;
  const int64_t pos = positions[row];
  const bf16* src;
  const bf16* nw = nullptr;
  if (head < n_q) { src = qkv + static_cast<size_t>(row) * ld + head * 2 * D; nw = q_norm; }
  else if (head < n_q + n_kv) { src = qkv + static_cast<size_t>(row) * ld + n_q * 2 * D + (head - n_q) * D; nw = k_norm; }
  else src = qkv + static_cast<size_t>(row) * ld + n_q * 2 * D + n_kv * D + (head - n_q - n_kv) * D;

  // lane owns the PER consecutive dims [lane * PER, +PER): one vector load / store per tensor; the rotary partner
  // (d, d + rot/2) of a dim lives in another lane and is read through shared memory
  const int d0 = lane * PER;
  float v[PER];
  load_bf16_vec<PER>(src + d0, v);
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss += v[i] * v[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / D + eps);
    float g[PER];
    load_bf16_vec<PER>(nw + d0, g);
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = __bfloat162float(__float2bfloat16(v[i] * inv * (1.0f + g[i])));
    // partial RoPE, half-split pairing: (d, d + rot/2) for d < rot/2
    const int half = rot / 2;
    __shared__ float tmp[8][D];
    float* t = tmp[threadIdx.x >> 5];
#pragma unroll
    for (int i = 0; i < PER; ++i) t[d0 + i] = v[i];
    __syncwarp();
    // the rotation itself is spread over all lanes (dim lane + 32 i), two transcendental evaluations per lane instead
    // of PER of them on the few lanes that own the rotary dims, and goes back through shared memory
    float rotated[(D / 32)];
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int d = lane + 32 * i;
      rotated[i] = 0.f;
      if (d < rot) {
        const int fi = d < half ? d : d - half;
        const float inv_freq = powf(theta, -2.0f * fi / rot);
        float sn, c;
        sincosf(static_cast<float>(pos) * inv_freq, &sn, &c);
        const float cb = __bfloat162float(__float2bfloat16(c)), sb = __bfloat162float(__float2bfloat16(sn));
        const float other = d < half ? -t[d + half] : t[d - half];
        rotated[i] = __bfloat162float(__float2bfloat16(t[d] * cb)) + __bfloat162float(__float2bfloat16(other * sb));
      }
    }
    __syncwarp();  // every lane has read its partners before anyone overwrites them
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < rot) t[d] = rotated[i];
    }
    __syncwarp();
    if (d0 < rot) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (d0 + i < rot) v[i] = t[d0 + i];
    }
  }
  if (head < n_q) {
    store_bf16_vec<PER>(q_out + (static_cast<size_t>(row) * n_q + head) * D + d0, v);
    copy_bf16_vec<PER>(gate_out + (static_cast<size_t>(row) * n_q + head) * D + d0, src + D + d0);
  } else {
    const int seq = seq_of_row[row];
    const int page = tables[static_cast<size_t>(seq) * max_pages + pos / PAGE];
    if (page < 0 || page >= num_pages) { if (lane == 0) atomicCAS(err, 0, ERR_BAD_INDEX); return; }
    const int which = head < n_q + n_kv ? 0 : 1;
    const int kh = which ? head - n_q - n_kv : head - n_q;
    bf16* dst = kv + ((((static_cast<size_t>(page) * 2 + which) * n_kv + kh) * PAGE) + pos % PAGE) * D;
    store_bf16_vec<PER>(dst + d0, v);
  }
}

// Partials: part_acc [B*G, n_q, Z, D] fp32, part_ml [B*G, n_q, Z, 2] (running max, running sum).
//
// One CTA per (sequence, kv head, lane z); warp w serves query head w of the GQA group. A page's
// K and V tiles (64 tokens x D) are staged in shared memory once with coalesced 16-byte loads
// and shared by all heads of the group, so HBM sees every KV byte once per layer. K rows are
// padded by 16 bytes: lane t reads row t, and the pad spreads rows over the banks. Scores: lane
// owns tokens `lane` and `lane + 32`; softmax statistics by warp reductions once per page;
// P.V: lane owns D/32 consecutive output dims.
template <int D>
struct AttnSmem {
  static constexpr int KSTRIDE = D + 8;  // bf16 elements per padded K row
  static constexpr size_t bytes(int group) {
    return static_cast<size_t>(PAGE) * KSTRIDE * 2 + static_cast<size_t>(PAGE) * D * 2 +
           static_cast<size_t>(group) * D * 4 + static_cast<size_t>(group) * PAGE * 4;
  }
};

template <int D, int GROUP>
__global__ void __launch_bounds__(32 * GROUP)
paged_attn_kernel(const bf16* q, const bf16* kv, const int* tables, int max_pages, const int64_t* positions,
                  float* part_acc, float* part_ml, int n_q, int n_kv, int G, int Z, float scale, int num_pages) {
  constexpr int KS = AttnSmem<D>::KSTRIDE;
  constexpr int PER = D / 32;
  constexpr int NT = 32 * GROUP;
  constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t smem_attn[];
  bf16* sK = reinterpret_cast<bf16*>(smem_attn);
  bf16* sV = sK + PAGE * KS;
  float* sQ = reinterpret_cast<float*>(sV + PAGE * D);
  float* sP = sQ + GROUP * D;
  const int b = blockIdx.x, kh = blockIdx.y, z = blockIdx.z;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qh = kh * GROUP + w;
  for (int g = 0; g < G; ++g) {
    const int row = b * G + g;
    const int len = static_cast<int>(positions[row]) + 1;  // keys 0..pos inclusive
    {
      const bf16* qp = q + (static_cast<size_t>(row) * n_q + qh) * D;
#pragma unroll
      for (int i = 0; i < PER; ++i) sQ[w * D + lane + 32 * i] = __bfloat162float(qp[lane + 32 * i]) * scale;
    }
    float m = -INFINITY, l = 0.f;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    const int n_pages = (len + PAGE - 1) / PAGE;
    for (int pg = z; pg < n_pages; pg += Z) {
      int page = tables[static_cast<size_t>(b) * max_pages + pg];
      if (page < 0 || page >= num_pages) page = 0;
      const bf16* kp = kv + ((static_cast<size_t>(page) * 2 + 0) * n_kv + kh) * PAGE * D;
      const bf16* vp = kv + ((static_cast<size_t>(page) * 2 + 1) * n_kv + kh) * PAGE * D;
      const int n_tok = min(PAGE, len - pg * PAGE);
      __syncthreads();  // previous page (and the q of a previous row) fully consumed
      for (int c = threadIdx.x; c < n_tok * CHUNKS; c += NT) {
        const int t = c / CHUNKS, j = c % CHUNKS;
        *reinterpret_cast<uint4*>(sK + t * KS + j * 8) = *reinterpret_cast<const uint4*>(kp + static_cast<size_t>(t) * D + j * 8);
        *reinterpret_cast<uint4*>(sV + t * D + j * 8) = *reinterpret_cast<const uint4*>(vp + static_cast<size_t>(t) * D + j * 8);
      }
      __syncthreads();
      // scores of this head against tokens lane and lane + 32
      float s0 = 0.f, s1 = 0.f;
      const bool v0 = lane < n_tok, v1 = lane + 32 < n_tok;
      const bf16* k0 = sK + lane * KS;
      const bf16* k1 = sK + (lane + 32) * KS;
      const float* qv = sQ + w * D;
#pragma unroll 4
      for (int j = 0; j < CHUNKS; ++j) {
        const float4 qa = *reinterpret_cast<const float4*>(qv + j * 8);
        const float4 qb = *reinterpret_cast<const float4*>(qv + j * 8 + 4);
        if (v0) {
          uint4 raw = *reinterpret_cast<const uint4*>(k0 + j * 8);
          const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
          const float2 a = __bfloat1622float2(e[0]), bb = __bfloat1622float2(e[1]), c2 = __bfloat1622float2(e[2]), d2 = __bfloat1622float2(e[3]);
          s0 += qa.x * a.x + qa.y * a.y + qa.z * bb.x + qa.w * bb.y + qb.x * c2.x + qb.y * c2.y + qb.z * d2.x + qb.w * d2.y;
        }
        if (v1) {
          uint4 raw = *reinterpret_cast<const uint4*>(k1 + j * 8);
          const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
          const float2 a = __bfloat1622float2(e[0]), bb = __bfloat1622float2(e[1]), c2 = __bfloat1622float2(e[2]), d2 = __bfloat1622float2(e[3]);
          s1 += qa.x * a.x + qa.y * a.y + qa.z * bb.x + qa.w * bb.y + qb.x * c2.x + qb.y * c2.y + qb.z * d2.x + qb.w * d2.y;
        }
      }
      if (!v0) s0 = -INFINITY;
      if (!v1) s1 = -INFINITY;
      const float mn = fmaxf(m, warp_max(fmaxf(s0, s1)));
      const float corr = __expf(m - mn);
      const float p0 = v0 ? __expf(s0 - mn) : 0.f, p1 = v1 ? __expf(s1 - mn) : 0.f;
      sP[w * PAGE + lane] = p0;
      sP[w * PAGE + lane + 32] = p1;
      l = l * corr + warp_sum(p0 + p1);
      m = mn;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] *= corr;
      __syncwarp();
      const float* pw = sP + w * PAGE;
      for (int t = 0; t < n_tok; ++t) {
        const float pt = pw[t];
        float ve[PER];
        load_bf16_vec<PER>(sV + t * D + lane * PER, ve);
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += pt * ve[i];
      }
      __syncwarp();
    }
    float* pa = part_acc + ((static_cast<size_t>(row) * n_q + qh) * Z + z) * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) pa[i] = acc[i];
    if (lane == 0) {
      float* pm = part_ml + ((static_cast<size_t>(row) * n_q + qh) * Z + z) * 2;
      pm[0] = m; pm[1] = l;
    }
    __syncthreads();  // sQ is rewritten for the next row
  }
}

template <int D>
__global__ void attn_combine_kernel(const float* part_acc, const float* part_ml, const bf16* gate, bf16* out, int n_q,
                                    int Z) {
  pdl_wait();
  pdl_launch();
  const int row = blockIdx.x, qh = blockIdx.y;
  const int d = threadIdx.x;  // D threads
  const float* pm = part_ml + (static_cast<size_t>(row) * n_q + qh) * Z * 2;
  float m = -INFINITY;
  for (int z = 0; z < Z; ++z) m = fmaxf(m, pm[2 * z]);
  float l = 0.f, acc = 0.f;
  for (int z = 0; z < Z; ++z) {
    const float mz = pm[2 * z];
    if (mz == -INFINITY) continue;
    const float sc = __expf(mz - m);
    l += pm[2 * z + 1] * sc;
    acc += part_acc[((static_cast<size_t>(row) * n_q + qh) * Z + z) * D + d] * sc;
  }
  const float o = __bfloat162float(__float2bfloat16(acc / l));
  const float g = __bfloat162float(gate[(static_cast<size_t>(row) * n_q + qh) * D + d]);
  out[(static_cast<size_t>(row) * n_q + qh) * D + d] = __float2bfloat16(o * sigmoid_f(g));
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_prep(const void* qkv, int ld, const int64_t* positions, const int* tables, int max_pages,
                              const int* seq_of_row, const void* q_norm, const void* k_norm, void* q_out, void* gate_out,
                              void* kv, int rows, int n_q, int n_kv, int D, int rot, float theta, float eps,
                              int num_pages, int* err, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int heads = n_q + 2 * n_kv;
  dim3 grid(rows, (heads + 7) / 8);
#define PREP(DD)                                                                                                      \
  launch_pdl(attn_prep_kernel<DD>, grid, dim3(256), 0, st, static_cast<const bf16*>(qkv), ld, positions, tables,    \
             max_pages, seq_of_row, static_cast<const bf16*>(q_norm), static_cast<const bf16*>(k_norm),              \
             static_cast<bf16*>(q_out), static_cast<bf16*>(gate_out), static_cast<bf16*>(kv), n_q, n_kv, rot, theta, \
             eps, num_pages, err)
  if (D == 256) PREP(256);
  else if (D == 128) PREP(128);
  else if (D == 64) PREP(64);
  else if (D == 32) PREP(32);
  else return -7;
#undef PREP
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_paged_attn(const void* q, const void* gate, const void* kv, const int* tables, int max_pages,
                               const int64_t* positions, float* part_acc, float* part_ml, void* out, int B, int G,
                               int n_q, int n_kv, int D, int Z, int num_pages, cudaStream_t st) {
  if (B <= 0) return 0;
  const int group = n_q / n_kv;
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  dim3 grid(B, n_kv, Z);
#define ATT(DD, GG)                                                                                                  \
  do {                                                                                                                \
    auto kern = paged_attn_kernel<DD, GG>;                                                                           \
    const size_t smem = AttnSmem<DD>::bytes(GG);                                                                     \
    static bool configured = false;                                                                                  \
    if (!configured) {                                                                                               \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) return -3; \
      configured = true;                                                                                             \
    }                                                                                                                \
    kern<<<grid, 32 * GG, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(kv), tables, max_pages, \
                                      positions, part_acc, part_ml, n_q, n_kv, G, Z, scale, num_pages);              \
  } while (0)
#define ATT_GROUPS(DD)                         \
  if (group == 8) ATT(DD, 8);                  \
  else if (group == 4) ATT(DD, 4);             \
  else if (group == 2) ATT(DD, 2);             \
  else if (group == 1) ATT(DD, 1);             \
  else return -7
  if (D == 256) { ATT_GROUPS(256); }
  else if (D == 128) { ATT_GROUPS(128); }
  else if (D == 64) { ATT_GROUPS(64); }
  else if (D == 32) { ATT_GROUPS(32); }
  else return -7;
#undef ATT_GROUPS
#undef ATT
  dim3 cgrid(B * G, n_q);
  if (D == 256) attn_combine_kernel<256><<<cgrid, 256, 0, st>>>(part_acc, part_ml, static_cast<const bf16*>(gate), static_cast<bf16*>(out), n_q, Z);
  else if (D == 128) attn_combine_kernel<128><<<cgrid, 128, 0, st>>>(part_acc, part_ml, static_cast<const bf16*>(gate), static_cast<bf16*>(out), n_q, Z);
  else if (D == 64) attn_combine_kernel<64><<<cgrid, 64, 0, st>>>(part_acc, part_ml, static_cast<const bf16*>(gate), static_cast<bf16*>(out), n_q, Z);
  else if (D == 32) attn_combine_kernel<32><<<cgrid, 32, 0, st>>>(part_acc, part_ml, static_cast<const bf16*>(gate), static_cast<bf16*>(out), n_q, Z);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Merge split partials [rows, n_q, Z, D] / [rows, n_q, Z, 2] in split order, apply sigmoid(gate), store bf16.
extern "C" int b200_attn_combine(const float* part_acc, const float* part_ml, const void* gate, void* out, int rows,
                                 int n_q, int D, int Z, cudaStream_t st) {
  if (rows <= 0) return 0;
  dim3 cgrid(rows, n_q);
  const bf16* g = static_cast<const bf16*>(gate);
  bf16* o = static_cast<bf16*>(out);
  cudaError_t rc;
  if (D == 256) rc = launch_pdl(attn_combine_kernel<256>, cgrid, dim3(256), 0, st, part_acc, part_ml, g, o, n_q, Z);
  else if (D == 128) rc = launch_pdl(attn_combine_kernel<128>, cgrid, dim3(128), 0, st, part_acc, part_ml, g, o, n_q, Z);
  else if (D == 64) rc = launch_pdl(attn_combine_kernel<64>, cgrid, dim3(64), 0, st, part_acc, part_ml, g, o, n_q, Z);
  else return -7;
  return rc == cudaSuccess ? 0 : -4;
}
