// Gated DeltaNet chunked prefill (64-row chunks), fp32 on the CUDA cores.
//
//  gdn_conv_prefill  : causal depthwise conv (kernel 4) + SiLU over packed spans, reading each span's first
//                      inputs from its slot's conv state; gdn_conv_state_update then stores the last 3 inputs
//                      (reference: engine/fast/prefill_kernels.py:279-317).
//  gdn_chunk_wy      : per (chunk, value head), all chunks in parallel: gates and their cumulative sum,
//                      L2-normalised q/k, A = (k beta) k^T * exp(g_i - g_j) strictly lower, T = (I + A)^-1
//                      by forward substitution, w = T (k beta e^g), u = T (v beta), masked q k^T scores, and
//                      the decayed copies of q and k that the state pass consumes
//                      (reference: engine/fast/gdn_chunk.py:203-471, the WY / UT transform).
//  gdn_chunk_scan    : per (sequence, value head, 32-column block of the state), chunks in order:
//                      v_new = u - w S; o = (q e^g) S + scores v_new; S = S e^{g_last} + (k e^{g_last-g})^T v_new
//                      with the fp32 state block resident in shared memory
//                      (reference: engine/fast/gdn_chunk.py:494-628). Padding rows are identity.
//  gdn_gated_norm    : per-head RMSNorm of o times silu(z) (reference: engine/fast/prefill_kernels.py:319-354).
//
// A row's result depends only on its own sequence: chunk boundaries are multiples of 64 rows from the span
// start, and no reduction ever mixes rows of different sequences.
#include "common.cuh"

namespace b200 {

constexpr int CH = 64;  // rows per chunk

struct ChunkInfo {  // one per (sequence chunk)
  int seg;          // sequence index in the pass
  int row0;         // first packed row of the chunk
  int nrows;        // valid rows (<= 64)
  int first;        // 1 when this is the first chunk of its span
};

// ------------------------------------------------------------------ conv
// x: [T, ld] (conv input at columns [0, C)); seg_start[seg] = first row of the span; out: [T, C] bf16.
// A thread owns 8 consecutive channels (16-byte loads) over CONV_ROWS rows and slides a 3-row window down them, so each
// input element is read once; the window is rebuilt from the three rows above at the start of a run, or from the slot's
// conv state where a span starts. (Measured at 8192 rows x 8192 channels: 131 us with runs of 32 rows, 136 us with
// runs of 8, 143 us with eight rows' loads issued together: the kernel is not bound by the latency of its row loads.)
constexpr int CONV_ROWS = 32;
__global__ void __launch_bounds__(128)
gdn_conv_prefill_kernel(const bf16* x, int ld, const int* seq_of_row, const int* seg_start, const int* slots,
                        const bf16* conv_state, const bf16* conv_w, bf16* out, int T, int C) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const int r0 = blockIdx.y * CONV_ROWS;
  if (c >= C) return;
  float w[8][4];
  {
    uint4 wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wv[i] = reinterpret_cast<const uint4*>(conv_w + static_cast<size_t>(c) * 4)[i];
    const bf16* we = reinterpret_cast<const bf16*>(wv);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
      for (int k = 0; k < 4; ++k) w[ch][k] = __bfloat162float(we[ch * 4 + k]);
  }
  float win[3][8];  // inputs of rows r-3, r-2, r-1
  const int r1 = min(T, r0 + CONV_ROWS);
  for (int r = r0; r < r1; ++r) {
    const int seg = seq_of_row[r];
    const int s0 = seg_start[seg];
    if (r == r0 || r == s0) {
      uint4 sv[3];
      const uint4* sp = reinterpret_cast<const uint4*>(conv_state + (static_cast<size_t>(slots[seg]) * C + c) * 3);
      if (r - 3 < s0) { sv[0] = sp[0]; sv[1] = sp[1]; sv[2] = sp[2]; }
      const bf16* se = reinterpret_cast<const bf16*>(sv);
#pragma unroll
      for (int back = 3; back >= 1; --back) {
        const int rr = r - back;
        if (rr >= s0) {
          const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(rr) * ld + c);
          const bf16* xe = reinterpret_cast<const bf16*>(&xv);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) win[3 - back][ch] = __bfloat162float(xe[ch]);
        } else {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) win[3 - back][ch] = __bfloat162float(se[ch * 3 + 3 - (s0 - rr)]);  // s0 - rr in 1..3
        }
      }
    }
    const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ld + c);
    const bf16* xe = reinterpret_cast<const bf16*>(&xv);
    uint4 ov;
    bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const float cur = __bfloat162float(xe[ch]);
      const float acc = w[ch][0] * win[0][ch] + w[ch][1] * win[1][ch] + w[ch][2] * win[2][ch] + w[ch][3] * cur;
      oe[ch] = __float2bfloat16(silu_f(acc));
      win[0][ch] = win[1][ch];
      win[1][ch] = win[2][ch];
      win[2][ch] = cur;
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * C + c) = ov;
  }
}

// New conv state of each span's slot: its last 3 inputs (older state entries shift in when the span is shorter).
__global__ void gdn_conv_state_update_kernel(const bf16* x, int ld, const int* seg_start, const int* slots,
                                             bf16* conv_state, int C) {
  const int seg = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s0 = seg_start[seg], s1 = seg_start[seg + 1], n = s1 - s0;
  bf16* st = conv_state + (static_cast<size_t>(slots[seg]) * C + c) * 3;
  bf16 old[3] = {st[0], st[1], st[2]};
  bf16 nw[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    const int back = 3 - k;  // this entry is the input `back` rows before the end
    nw[k] = back <= n ? x[static_cast<size_t>(s1 - back) * ld + c] : old[k + n];  // k + n < 3 here
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) st[k] = nw[k];
}

// ------------------------------------------------------------------ WY / UT transform of one chunk
// Workspace of one (chunk, head), fp32: W[64][DK] | U[64][DV] | QG[64][DK] | KG[64][DK] | QK[64][64] | glast.
template <int DK, int DV>
struct WyLayout {
  static constexpr int W = 0, U = W + CH * DK, QG = U + CH * DV, KG = QG + CH * DK, QK = KG + CH * DK,
                       GLAST = QK + CH * CH, STRIDE = GLAST + 64;
};

template <int DK, int DV>
__global__ void __launch_bounds__(256)
gdn_chunk_wy_kernel(const bf16* conv_out, const bf16* mixed, int ld, int b_off, int a_off, const ChunkInfo* chunks,
                    const float* A_log, const float* dt_bias, float* work, int HK, int HV) {
  using L = WyLayout<DK, DV>;
  constexpr int KS = DK + 1, VS = DV + 1, AS = CH + 1;  // padded strides: consecutive rows land in different banks
  extern __shared__ float sm[];
  float* kn = sm;                 // [64][KS]
  float* qn = kn + CH * KS;       // [64][KS]
  float* vb = qn + CH * KS;       // [64][VS]  v * beta
  float* A = vb + CH * VS;        // [64][AS]
  float* Tm = A + CH * AS;        // [64][AS]
  float* gc = Tm + CH * AS;       // [64]
  float* beta = gc + CH;          // [64]
  float* rn = beta + CH;          // [64][2] inverse norms
  const ChunkInfo ci = chunks[blockIdx.x];
  const int h = blockIdx.y, hk = h / (HV / HK);
  const int key_dim = HK * DK, C = 2 * key_dim + HV * DV;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* out = work + (static_cast<size_t>(blockIdx.x) * HV + h) * L::STRIDE;

  // gates of the chunk's rows; padding rows are identity (beta = 0, g = 0)
  if (tid < CH) {
    float g = 0.f, b = 0.f;
    if (tid < ci.nrows) {
      const size_t row = static_cast<size_t>(ci.row0 + tid);
      const float av = __bfloat162float(mixed[row * ld + a_off + h]);
      const float bv = __bfloat162float(mixed[row * ld + b_off + h]);
      g = -__expf(A_log[h]) * softplus_f(av + dt_bias[h]);
      b = sigmoid_f(bv);
    }
    gc[tid] = g;
    beta[tid] = b;
  }
  for (int idx = tid; idx < CH * DK; idx += 256) {
    const int r = idx / DK, d = idx % DK;
    float qv = 0.f, kv = 0.f;
    if (r < ci.nrows) {
      const bf16* co = conv_out + static_cast<size_t>(ci.row0 + r) * C;
      qv = __bfloat162float(co[hk * DK + d]);
      kv = __bfloat162float(co[key_dim + hk * DK + d]);
    }
    qn[r * KS + d] = qv;
    kn[r * KS + d] = kv;
  }
  __syncthreads();
  if (warp == 0) {  // inclusive scan of the 64 log-decays
    float a = gc[lane], b2 = gc[lane + 32];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float x = __shfl_up_sync(0xffffffffu, a, o), y = __shfl_up_sync(0xffffffffu, b2, o);
      if (lane >= o) { a += x; b2 += y; }
    }
    const float tot = __shfl_sync(0xffffffffu, a, 31);
    gc[lane] = a;
    gc[lane + 32] = b2 + tot;
  }
  for (int r = warp; r < CH; r += 8) {  // L2 norms, one warp per row
    float sq = 0.f, sk = 0.f;
    for (int d = lane; d < DK; d += 32) { const float a = qn[r * KS + d], b2 = kn[r * KS + d]; sq += a * a; sk += b2 * b2; }
    sq = warp_sum(sq); sk = warp_sum(sk);
    if (lane == 0) { rn[2 * r] = rsqrtf(sq + 1e-6f) * rsqrtf(static_cast<float>(DK)); rn[2 * r + 1] = rsqrtf(sk + 1e-6f); }
  }
  __syncthreads();
  for (int idx = tid; idx < CH * DK; idx += 256) {
    const int r = idx / DK, d = idx % DK;
    qn[r * KS + d] *= rn[2 * r];
    kn[r * KS + d] *= rn[2 * r + 1];
  }
  for (int idx = tid; idx < CH * DV; idx += 256) {
    const int r = idx / DV, d = idx % DV;
    float vv = 0.f;
    if (r < ci.nrows) vv = __bfloat162float(conv_out[static_cast<size_t>(ci.row0 + r) * C + 2 * key_dim + h * DV + d]);
    vb[r * VS + d] = vv * beta[r];
  }
  __syncthreads();
  // A = (k beta) k^T decay (strictly lower) and the causal q k^T scores; thread (ty, tx) owns rows ty + 16 ii,
  // columns tx + 16 jj
  const int ty = tid >> 4, tx = tid & 15;
  {
    float akk[4][4], aqk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) { akk[a][b2] = 0.f; aqk[a][b2] = 0.f; }
    for (int d = 0; d < DK; ++d) {
      float ki[4], qi[4], kj[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) { ki[a] = kn[(ty + 16 * a) * KS + d]; qi[a] = qn[(ty + 16 * a) * KS + d]; kj[a] = kn[(tx + 16 * a) * KS + d]; }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b2 = 0; b2 < 4; ++b2) { akk[a][b2] += ki[a] * kj[b2]; aqk[a][b2] += qi[a] * kj[b2]; }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) {
        const int i = ty + 16 * a, j = tx + 16 * b2;
        const float dec = j <= i ? __expf(gc[i] - gc[j]) : 0.f;
        A[i * AS + j] = j < i ? akk[a][b2] * beta[i] * dec : 0.f;
        out[L::QK + i * CH + j] = aqk[a][b2] * dec;
      }
  }
  // decayed copies for the state pass, then k <- k beta e^g in place
  const float glast = gc[CH - 1];
  for (int idx = tid; idx < CH * DK; idx += 256) {
    const int r = idx / DK, d = idx % DK;
    const float kv = kn[r * KS + d];
    out[L::QG + idx] = qn[r * KS + d] * __expf(gc[r]);
    out[L::KG + idx] = kv * __expf(glast - gc[r]);
  }
  if (tid == 0) out[L::GLAST] = glast;
  __syncthreads();
  for (int idx = tid; idx < CH * DK; idx += 256) {
    const int r = idx / DK, d = idx % DK;
    kn[r * KS + d] *= beta[r] * __expf(gc[r]);
  }
  // T = (I + A)^-1 by forward substitution, one row per step; thread c < 64 owns column c
  if (tid < CH) {
    for (int j = 0; j < CH; ++j) Tm[j * AS + tid] = j == tid ? 1.f : 0.f;
  }
  __syncthreads();
  for (int i = 1; i < CH; ++i) {
    if (tid < i) {
      float acc = A[i * AS + tid];
      for (int j = tid + 1; j < i; ++j) acc += A[i * AS + j] * Tm[j * AS + tid];
      Tm[i * AS + tid] = -acc;
    }
    __syncthreads();
  }
  // w = T (k beta e^g), u = T (v beta)
  {
    constexpr int NK = DK / 16, NV = DV / 16;
    float aw[4][NK], au[4][NV];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
      for (int b2 = 0; b2 < NK; ++b2) aw[a][b2] = 0.f;
#pragma unroll
      for (int b2 = 0; b2 < NV; ++b2) au[a][b2] = 0.f;
    }
    for (int j = 0; j < CH; ++j) {
      float t4[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) t4[a] = Tm[(ty + 16 * a) * AS + j];
#pragma unroll
      for (int b2 = 0; b2 < NK; ++b2) {
        const float kv = kn[j * KS + tx + 16 * b2];
#pragma unroll
        for (int a = 0; a < 4; ++a) aw[a][b2] += t4[a] * kv;
      }
#pragma unroll
      for (int b2 = 0; b2 < NV; ++b2) {
        const float vv = vb[j * VS + tx + 16 * b2];
#pragma unroll
        for (int a = 0; a < 4; ++a) au[a][b2] += t4[a] * vv;
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
#pragma unroll
      for (int b2 = 0; b2 < NK; ++b2) out[L::W + i * DK + tx + 16 * b2] = aw[a][b2];
#pragma unroll
      for (int b2 = 0; b2 < NV; ++b2) out[L::U + i * DV + tx + 16 * b2] = au[a][b2];
    }
  }
}

// ------------------------------------------------------------------ sequential state pass
// grid (sequences, value heads, DV / 32). seg_chunks[seg] = (first chunk, number of chunks).
template <int DK, int DV>
__global__ void __launch_bounds__(256)
gdn_chunk_scan_kernel(const float* work, const ChunkInfo* chunks, const int2* seg_chunks, const int* slots,
                      float* rec_state, bf16* o_out, int HV) {
  using L = WyLayout<DK, DV>;
  constexpr int KS = DK + 1, CB = 32, CS = CB + 1, AS = CH + 1;
  extern __shared__ float sm[];
  float* S = sm;                  // [DK][CB]
  float* Wc = S + DK * CB;        // [64][KS]
  float* QGc = Wc + CH * KS;      // [64][KS]
  float* KGc = QGc + CH * KS;     // [64][KS]
  float* Uc = KGc + CH * KS;      // [64][CS]  u, then v_new in place
  float* QKc = Uc + CH * CS;      // [64][AS]
  const int seg = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * CB;
  const int tid = threadIdx.x;
  const int2 sc = seg_chunks[seg];
  float* Sg = rec_state + ((static_cast<size_t>(slots[seg]) * HV + h) * DK) * DV;
  for (int idx = tid; idx < DK * CB; idx += 256) S[idx] = Sg[static_cast<size_t>(idx / CB) * DV + c0 + idx % CB];
  for (int cc = 0; cc < sc.y; ++cc) {
    const int cidx = sc.x + cc;
    const ChunkInfo ci = chunks[cidx];
    const float* in = work + (static_cast<size_t>(cidx) * HV + h) * L::STRIDE;
    __syncthreads();  // previous chunk done with every buffer
    for (int idx = tid; idx < CH * DK; idx += 256) {
      const int r = idx / DK, d = idx % DK;
      Wc[r * KS + d] = in[L::W + idx];
      QGc[r * KS + d] = in[L::QG + idx];
      KGc[r * KS + d] = in[L::KG + idx];
    }
    for (int idx = tid; idx < CH * CB; idx += 256) Uc[(idx / CB) * CS + idx % CB] = in[L::U + (idx / CB) * DV + c0 + idx % CB];
    for (int idx = tid; idx < CH * CH; idx += 256) QKc[(idx / CH) * AS + idx % CH] = in[L::QK + idx];
    const float eg = __expf(in[L::GLAST]);
    __syncthreads();
    // v_new = u - w S and the state part of the output; thread owns row r, 8 columns
    const int r = tid >> 2, cb = (tid & 3) * 8;
    float vn[8], oo[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { vn[j] = 0.f; oo[j] = 0.f; }
    for (int k = 0; k < DK; ++k) {
      const float wv = Wc[r * KS + k], qv = QGc[r * KS + k];
      const float* srow = S + k * CB + cb;
#pragma unroll
      for (int j = 0; j < 8; ++j) { vn[j] += wv * srow[j]; oo[j] += qv * srow[j]; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) vn[j] = Uc[r * CS + cb + j] - vn[j];
    __syncthreads();  // everyone has read u (and S for this chunk's outputs)
#pragma unroll
    for (int j = 0; j < 8; ++j) Uc[r * CS + cb + j] = vn[j];
    __syncthreads();
    for (int jj = 0; jj <= r; ++jj) {  // causal scores: columns beyond the row are zero
      const float a = QKc[r * AS + jj];
      const float* vrow = Uc + jj * CS + cb;
#pragma unroll
      for (int j = 0; j < 8; ++j) oo[j] += a * vrow[j];
    }
    if (r < ci.nrows) {
      bf16* dst = o_out + (static_cast<size_t>(ci.row0 + r) * HV + h) * DV + c0 + cb;
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = __float2bfloat16(oo[j]);
    }
    // S = S e^{g_last} + (k e^{g_last - g})^T v_new; thread owns key row k2, 16 columns
    const int k2 = tid >> 1, hb = (tid & 1) * 16;
    if (k2 < DK) {  // each thread reads and writes only its own 16 state elements
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = S[k2 * CB + hb + j] * eg;
      for (int rr = 0; rr < CH; ++rr) {
        const float kv = KGc[rr * KS + k2];
        const float* vrow = Uc + rr * CS + hb;
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] += kv * vrow[j];
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) S[k2 * CB + hb + j] = acc[j];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < DK * CB; idx += 256) Sg[static_cast<size_t>(idx / CB) * DV + c0 + idx % CB] = S[idx];
}

// out[row, h, :] = bf16(w * bf16(o * rsqrt(mean(o^2) + eps)) * silu(z)); one warp per (row, head).
template <int DV>
__global__ void gdn_gated_norm_kernel(const bf16* o, const bf16* mixed, int ld, int z_off, const bf16* w, bf16* out,
                                      int rows, int HV, float eps) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= rows * HV) return;
  const int row = gw / HV, h = gw % HV;
  constexpr int PER = DV / 32;  // consecutive elements per lane: one vector load each of o, z and w
  static_assert(PER == 1 || PER == 2 || PER == 4, "head dim 32, 64 or 128");
  const size_t o_at = (static_cast<size_t>(row) * HV + h) * DV + lane * PER;
  const size_t z_at = static_cast<size_t>(row) * ld + z_off + h * DV + lane * PER;
  bf16 ov[PER], zv[PER], wv[PER], rv[PER];
  if constexpr (PER == 4) {
    *reinterpret_cast<uint2*>(ov) = *reinterpret_cast<const uint2*>(o + o_at);
    *reinterpret_cast<uint2*>(zv) = *reinterpret_cast<const uint2*>(mixed + z_at);
    *reinterpret_cast<uint2*>(wv) = *reinterpret_cast<const uint2*>(w + lane * PER);
  } else if constexpr (PER == 2) {
    *reinterpret_cast<uint32_t*>(ov) = *reinterpret_cast<const uint32_t*>(o + o_at);
    *reinterpret_cast<uint32_t*>(zv) = *reinterpret_cast<const uint32_t*>(mixed + z_at);
    *reinterpret_cast<uint32_t*>(wv) = *reinterpret_cast<const uint32_t*>(w + lane * PER);
  } else {
    ov[0] = o[o_at]; zv[0] = mixed[z_at]; wv[0] = w[lane];
  }
  float v[PER], ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) { v[i] = __bfloat162float(ov[i]); ss += v[i] * v[i]; }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / DV + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const float nb = __bfloat162float(__float2bfloat16(v[i] * inv));
    rv[i] = __float2bfloat16(__bfloat162float(wv[i]) * nb * silu_f(__bfloat162float(zv[i])));
  }
  if constexpr (PER == 4) *reinterpret_cast<uint2*>(out + o_at) = *reinterpret_cast<const uint2*>(rv);
  else if constexpr (PER == 2) *reinterpret_cast<uint32_t*>(out + o_at) = *reinterpret_cast<const uint32_t*>(rv);
  else out[o_at] = rv[0];
}

}  // namespace b200

using namespace b200;

namespace {
template <int DKV>
int gdn_prefill_launch(const bf16* mixed, int ld, const bf16* conv_out, const ChunkInfo* chunks, int n_chunks,
                       const int2* seg_chunks, int n_seg, const int* slots, float* rec_state, const float* A_log,
                       const float* dt_bias, const bf16* gnorm_w, float* work, bf16* o_tmp, bf16* out, int T, int HK,
                       int HV, float eps, cudaStream_t st) {
  const int key_dim = HK * DKV, value_dim = HV * DKV, C = 2 * key_dim + value_dim;
  const int z_off = C, b_off = C + value_dim, a_off = C + value_dim + HV;
  auto wy = gdn_chunk_wy_kernel<DKV, DKV>;
  auto scan = gdn_chunk_scan_kernel<DKV, DKV>;
  constexpr int wy_smem = (2 * CH * (DKV + 1) + CH * (DKV + 1) + 2 * CH * (CH + 1) + 4 * CH) * 4;
  constexpr int scan_smem = (DKV * 32 + 3 * CH * (DKV + 1) + CH * 33 + CH * (CH + 1)) * 4;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(wy, cudaFuncAttributeMaxDynamicSharedMemorySize, wy_smem) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(scan, cudaFuncAttributeMaxDynamicSharedMemorySize, scan_smem) != cudaSuccess) return -3;
    configured = true;
  }
  wy<<<dim3(n_chunks, HV), 256, wy_smem, st>>>(conv_out, mixed, ld, b_off, a_off, chunks, A_log, dt_bias, work, HK, HV);
  scan<<<dim3(n_seg, HV, DKV / 32), 256, scan_smem, st>>>(work, chunks, seg_chunks, slots, rec_state, o_tmp, HV);
  const int warps = T * HV;
  gdn_gated_norm_kernel<DKV><<<(warps + 7) / 8, 256, 0, st>>>(o_tmp, mixed, ld, z_off, gnorm_w, out, T, HV, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
}  // namespace

extern "C" int b200_gdn_prefill_tc(const void* mixed, int ld, const void* conv_out, const void* chunks, int n_chunks,
                                   const void* seg_chunks, int n_seg, const int* slots, float* rec_state,
                                   const float* A_log, const float* dt_bias, void* work, void* o_tmp, int T, int HK,
                                   int HV, int* err, cudaStream_t st);

// Workspace floats needed per (chunk, head).
extern "C" int b200_gdn_prefill_work_stride(int DK) { return 64 * (4 * DK + 64) + 64; }

// mixed: [T, ld] in_proj output (qkv | z | b | a); conv_out: [T, C] scratch; chunks: ChunkInfo[n_chunks] in sequence
// order; seg_chunks: int2[n_seg]; seq_of_row / seg_start: row -> sequence, sequence -> first row (n_seg + 1 entries);
// work: fp32 [n_chunks * HV * stride]; o_tmp: bf16 [T, HV * DV]; out: bf16 [T, HV * DV]. use_tc: head dims of 128
// take the tcgen05 kernels of gdn_prefill_tc.cu (other head dims always run the fp32 kernels).
extern "C" int b200_gdn_prefill(const void* mixed, int ld, const int* seq_of_row, const int* seg_start, const int* slots,
                                void* conv_state, float* rec_state, const void* conv_w, const float* A_log,
                                const float* dt_bias, const void* gnorm_w, void* conv_out, const void* chunks,
                                int n_chunks, const void* seg_chunks, int n_seg, float* work, void* o_tmp, void* out,
                                int T, int HK, int HV, int DK, int DV, float eps, int use_tc, int* err,
                                cudaStream_t st) {
  if (T <= 0) return 0;
  if (DK != DV) return -7;
  const int C = 2 * HK * DK + HV * DV;
  if (C % 8 || ld % 8) return -7;
  gdn_conv_prefill_kernel<<<dim3((C / 8 + 127) / 128, (T + CONV_ROWS - 1) / CONV_ROWS), 128, 0, st>>>(
      static_cast<const bf16*>(mixed), ld, seq_of_row, seg_start, slots, static_cast<const bf16*>(conv_state),
      static_cast<const bf16*>(conv_w), static_cast<bf16*>(conv_out), T, C);
  gdn_conv_state_update_kernel<<<dim3((C + 127) / 128, n_seg), 128, 0, st>>>(
      static_cast<const bf16*>(mixed), ld, seg_start, slots, static_cast<bf16*>(conv_state), C);
#define GP(DKV)                                                                                                      \
  return gdn_prefill_launch<DKV>(static_cast<const bf16*>(mixed), ld, static_cast<const bf16*>(conv_out),            \
                                 static_cast<const ChunkInfo*>(chunks), n_chunks, static_cast<const int2*>(seg_chunks), \
                                 n_seg, slots, rec_state, A_log, dt_bias, static_cast<const bf16*>(gnorm_w), work,   \
                                 static_cast<bf16*>(o_tmp), static_cast<bf16*>(out), T, HK, HV, eps, st)
  if (DK == 128 && use_tc) {
    // tensor-core WY transform and state pass (gdn_prefill_tc.cu), then the same gated norm
    const int rc = b200_gdn_prefill_tc(mixed, ld, conv_out, chunks, n_chunks, seg_chunks, n_seg, slots, rec_state, A_log,
                                       dt_bias, work, o_tmp, T, HK, HV, err, st);
    if (rc) return rc;
    const int warps = T * HV;
    gdn_gated_norm_kernel<128><<<(warps + 7) / 8, 256, 0, st>>>(static_cast<const bf16*>(o_tmp), static_cast<const bf16*>(mixed),
                                                                ld, C, static_cast<const bf16*>(gnorm_w),
                                                                static_cast<bf16*>(out), T, HV, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  if (DK == 128) GP(128);
  if (DK == 64) GP(64);
  if (DK == 32) GP(32);
#undef GP
  return -7;
}
