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

template <int D>
__global__ void attn_prep_kernel(const bf16* qkv, int ld, const int64_t* positions, const int* tables, int max_pages,
                                 const int* seq_of_row, const bf16* q_norm, const bf16* k_norm, bf16* q_out,
                                 bf16* gate_out, bf16* kv, int n_q, int n_kv, int rot, float theta, float eps,
                                 int num_pages, int* err) {
  // one warp per (row, head); heads: [0,n_q) query, [n_q, n_q+n_kv) key, then value
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

  // lane owns dims lane + 32*i (pairs (d, d + rot/2) of the rotary part fall in the same lane when rot/2 % 32 == 0;
  // otherwise fetched by shuffle-free direct reads below)
  float v[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) v[i] = __bfloat162float(src[lane + 32 * i]);
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss += v[i] * v[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / D + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i)
      v[i] = __bfloat162float(__float2bfloat16(v[i] * inv * (1.0f + __bfloat162float(nw[lane + 32 * i]))));
    // partial RoPE, half-split pairing: (d, d + rot/2) for d < rot/2
    const int half = rot / 2;
    __shared__ float tmp[8][D];
    float* t = tmp[threadIdx.x >> 5];
#pragma unroll
    for (int i = 0; i < PER; ++i) t[lane + 32 * i] = v[i];
    __syncwarp();
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < rot) {
        const int fi = d < half ? d : d - half;
        const float inv_freq = powf(theta, -2.0f * fi / rot);
        float s, c;
        sincosf(static_cast<float>(pos) * inv_freq, &s, &c);
        const float cb = __bfloat162float(__float2bfloat16(c)), sb = __bfloat162float(__float2bfloat16(s));
        const float other = d < half ? -t[d + half] : t[d - half];
        v[i] = __bfloat162float(__float2bfloat16(t[d] * cb)) + __bfloat162float(__float2bfloat16(other * sb));
      }
    }
  }
  if (head < n_q) {
    bf16* dq = q_out + (static_cast<size_t>(row) * n_q + head) * D;
    bf16* dg = gate_out + (static_cast<size_t>(row) * n_q + head) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      dq[lane + 32 * i] = __float2bfloat16(v[i]);
      dg[lane + 32 * i] = src[D + lane + 32 * i];
    }
  } else {
    const int seq = seq_of_row[row];
    const int page = tables[static_cast<size_t>(seq) * max_pages + pos / PAGE];
    if (page < 0 || page >= num_pages) { if (lane == 0) atomicCAS(err, 0, ERR_BAD_INDEX); return; }
    const int which = head < n_q + n_kv ? 0 : 1;
    const int kh = which ? head - n_q - n_kv : head - n_q;
    bf16* dst = kv + ((((static_cast<size_t>(page) * 2 + which) * n_kv + kh) * PAGE) + pos % PAGE) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[lane + 32 * i] = __float2bfloat16(v[i]);
  }
}

// Partials: part_acc [B*G, n_q, Z, D] fp32, part_ml [B*G, n_q, Z, 2] (running max, running sum).
template <int D, int GROUP>
__global__ void __launch_bounds__(32 * GROUP)
paged_attn_kernel(const bf16* q, const bf16* kv, const int* tables, int max_pages, const int64_t* positions,
                  float* part_acc, float* part_ml, int n_q, int n_kv, int G, int Z, float scale, int num_pages) {
  const int b = blockIdx.x, kh = blockIdx.y, z = blockIdx.z;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qh = kh * GROUP + w;
  constexpr int PER = D / 32;  // dims per lane, contiguous: lane*PER .. lane*PER+PER-1
  for (int g = 0; g < G; ++g) {
    const int row = b * G + g;
    const int len = static_cast<int>(positions[row]) + 1;  // keys 0..pos inclusive
    float qv[PER];
    {
      const bf16* qp = q + (static_cast<size_t>(row) * n_q + qh) * D + lane * PER;
#pragma unroll
      for (int i = 0; i < PER; ++i) qv[i] = __bfloat162float(qp[i]) * scale;
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
      for (int t = 0; t < n_tok; ++t) {
        float ke[PER], ve[PER];
        load_bf16_vec<PER>(kp + static_cast<size_t>(t) * D + lane * PER, ke);
        load_bf16_vec<PER>(vp + static_cast<size_t>(t) * D + lane * PER, ve);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) s += qv[i] * ke[i];
        s = warp_sum(s);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn);
        const float pexp = __expf(s - mn);
        l = l * corr + pexp;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = acc[i] * corr + pexp * ve[i];
        m = mn;
      }
    }
    float* pa = part_acc + ((static_cast<size_t>(row) * n_q + qh) * Z + z) * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) pa[i] = acc[i];
    if (lane == 0) {
      float* pm = part_ml + ((static_cast<size_t>(row) * n_q + qh) * Z + z) * 2;
      pm[0] = m; pm[1] = l;
    }
  }
}

template <int D>
__global__ void attn_combine_kernel(const float* part_acc, const float* part_ml, const bf16* gate, bf16* out, int n_q,
                                    int Z) {
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
  attn_prep_kernel<DD><<<grid, 256, 0, st>>>(static_cast<const bf16*>(qkv), ld, positions, tables, max_pages,        \
                                             seq_of_row, static_cast<const bf16*>(q_norm),                           \
                                             static_cast<const bf16*>(k_norm), static_cast<bf16*>(q_out),            \
                                             static_cast<bf16*>(gate_out), static_cast<bf16*>(kv), n_q, n_kv, rot,   \
                                             theta, eps, num_pages, err)
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
  paged_attn_kernel<DD, GG><<<grid, 32 * GG, 0, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(kv),    \
                                                      tables, max_pages, positions, part_acc, part_ml, n_q, n_kv, G, \
                                                      Z, scale, num_pages)
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
