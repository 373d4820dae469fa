// Gated DeltaNet decode: short-conv step, gated delta rule on the fp32 recurrent state, gated
// RMSNorm. One (row, value head) per CTA; the 128 x 128 fp32 state tile is read once into
// registers (32 values per thread), updated and written back once, so the kernel moves the
// state-streaming minimum (reference: engine/fast/hip/gdn_chain.hip:132-386 keeps the tile in
// registers the same way; engine/fast/kernels.py:573-633 are its unfused Triton forms).
//
// Work split inside a CTA of 4*DV threads: thread (p, c) owns state column c for key rows
// [p*DK/4, (p+1)*DK/4). The four partial sums of a column are always combined as
// ((p0 + p1) + (p2 + p3)), and the layout never depends on the number of rows in the launch,
// so a sequence's state and outputs are bit-identical for any batch size.
//
// G rows per sequence (speculative verify) are processed in order on the same register tile;
// the state after row j can be stored to `ring` so that the host can commit the accepted prefix.
#ifdef B200_EMU  // host build of the kernel bodies for tests/emu (threads, barriers and copies come from the shim)
#include "emu_shim.h"
#else
#include "common.cuh"
#endif

namespace b200 {

// ------------------------------------------------------------------ conv step
// mixed: [B*G, ld] rows (row b*G + j), conv input at columns [0, C). conv_state: [slots, C, KW-1].
// out: [B*G, C] = silu(sum_k w[c,k] * window[k]). The slot's state ends as the last KW-1 inputs;
// with G > 1 the state after each row is also kept in ring_conv [B, G, C, KW-1] when given.
template <int KW>
__global__ void gdn_conv_step_kernel(const bf16* mixed, int ld, const int* slots, bf16* conv_state, const bf16* conv_w,
                                     bf16* out, bf16* ring_conv, int C, int G) {
  // a thread owns 8 consecutive channels: 16-byte loads of the inputs, 48 / 64 contiguous bytes of state / weights
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int slot = slots[b];
  bf16* st = conv_state + (static_cast<size_t>(slot) * C + c) * (KW - 1);
  float win[8][KW];
  float w[8][KW];
  {
    bf16 sv[8 * (KW - 1)], wv[8 * KW];
#pragma unroll
    for (int i = 0; i < (KW - 1); ++i) reinterpret_cast<uint4*>(sv)[i] = reinterpret_cast<const uint4*>(st)[i];
#pragma unroll
    for (int i = 0; i < KW; ++i) reinterpret_cast<uint4*>(wv)[i] = reinterpret_cast<const uint4*>(conv_w + static_cast<size_t>(c) * KW)[i];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
#pragma unroll
      for (int k = 0; k < KW - 1; ++k) win[ch][k] = __bfloat162float(sv[ch * (KW - 1) + k]);
#pragma unroll
      for (int k = 0; k < KW; ++k) w[ch][k] = __bfloat162float(wv[ch * KW + k]);
    }
  }
  for (int j = 0; j < G; ++j) {
    const size_t row = static_cast<size_t>(b) * G + j;
    bf16 xv[8], ov[8];
    *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(mixed + row * ld + c);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      win[ch][KW - 1] = __bfloat162float(xv[ch]);
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < KW; ++k) acc += win[ch][k] * w[ch][k];
      ov[ch] = __float2bfloat16(silu_f(acc));
#pragma unroll
      for (int k = 0; k < KW - 1; ++k) win[ch][k] = win[ch][k + 1];
    }
    *reinterpret_cast<uint4*>(out + row * C + c) = *reinterpret_cast<const uint4*>(ov);
    if (ring_conv) {
      bf16 rv[8 * (KW - 1)];
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
#pragma unroll
        for (int k = 0; k < KW - 1; ++k) rv[ch * (KW - 1) + k] = __float2bfloat16(win[ch][k]);
      uint4* r = reinterpret_cast<uint4*>(ring_conv + ((static_cast<size_t>(b) * G + j) * C + c) * (KW - 1));
#pragma unroll
      for (int i = 0; i < (KW - 1); ++i) r[i] = reinterpret_cast<const uint4*>(rv)[i];
    }
  }
  bf16 sv[8 * (KW - 1)];
#pragma unroll
  for (int ch = 0; ch < 8; ++ch)
#pragma unroll
    for (int k = 0; k < KW - 1; ++k) sv[ch * (KW - 1) + k] = __float2bfloat16(win[ch][k]);
#pragma unroll
  for (int i = 0; i < (KW - 1); ++i) reinterpret_cast<uint4*>(st)[i] = reinterpret_cast<const uint4*>(sv)[i];
}

// One channel per thread: for channel counts or row strides that are not multiples of 8 (odd tensor-parallel shards).
template <int KW>
__global__ void gdn_conv_step_scalar_kernel(const bf16* mixed, int ld, const int* slots, bf16* conv_state, const bf16* conv_w,
                                     bf16* out, bf16* ring_conv, int C, int G) {
  pdl_wait();
  pdl_launch();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slots[b];
  bf16* st = conv_state + (static_cast<size_t>(slot) * C + c) * (KW - 1);
  float win[KW];
  float w[KW];
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) win[k] = __bfloat162float(st[k]);
#pragma unroll
  for (int k = 0; k < KW; ++k) w[k] = __bfloat162float(conv_w[c * KW + k]);
  for (int j = 0; j < G; ++j) {
    const size_t row = static_cast<size_t>(b) * G + j;
    win[KW - 1] = __bfloat162float(mixed[row * ld + c]);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < KW; ++k) acc += win[k] * w[k];
    out[row * C + c] = __float2bfloat16(silu_f(acc));
#pragma unroll
    for (int k = 0; k < KW - 1; ++k) win[k] = win[k + 1];
    if (ring_conv) {
      bf16* r = ring_conv + ((static_cast<size_t>(b) * G + j) * C + c) * (KW - 1);
#pragma unroll
      for (int k = 0; k < KW - 1; ++k) r[k] = __float2bfloat16(win[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) st[k] = __float2bfloat16(win[k]);
}

// ------------------------------------------------------------------ delta-rule step
// The DK x DV fp32 state tile of one (sequence, value head) is brought into shared memory by one bulk
// async copy (TMA, no registers held while it is in flight), updated in place for the G rows of the step,
// and written back by one bulk store; with 64 KB per CTA three CTAs fit an SM, so loads, updates and
// stores of different tiles overlap. Thread (p, c) owns column c for key rows [p*DK/4, (p+1)*DK/4).
#ifndef B200_EMU
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
#endif

template <int DK, int DV>
__global__ void __launch_bounds__(4 * DV, 3)
gdn_step_kernel(const bf16* conv_out,   // [B*G, C]  q | k | v after conv+silu
                const bf16* mixed,      // [B*G, ld] z at column z_off, b at b_off, a at a_off
                int ld, int z_off, int b_off, int a_off,
                const int* slots, float* rec_state,  // [slots, HV, DK, DV]
                const float* A_log, const float* dt_bias, const bf16* gnorm_w,
                bf16* out,              // [B*G, HV*DV]
                float* ring_rec,        // optional [B, G, HV, DK, DV]
                int HK, int HV, int G, float eps, int* err) {
  constexpr int KP = DK / 4;  // key rows per partition
  constexpr uint32_t TILE_BYTES = DK * DV * sizeof(float);
#ifdef B200_EMU
  float* sS = EMU_DYNAMIC_SMEM;
#else
  extern __shared__ __align__(128) float sS[];
#endif
  const int b = blockIdx.y, h = blockIdx.x;
  const int c = threadIdx.x % DV, p = threadIdx.x / DV;
  const int hk = h / (HV / HK);
  const int key_dim = HK * DK;
  const int C = 2 * key_dim + HV * DV;

  __align__(16) __shared__ float sq[DK], sk[DK];
  __shared__ float red[4][DV][2];
  __shared__ float nred[4][3];
  __shared__ float wred[4 * DV / 32];
  __shared__ uint64_t bar;
  __shared__ int s_abort;

  // The recurrent state was last written by an earlier decode step or prefill pass, never by the kernel just before
  // this one (the conv step), and the slot table is an input of the whole pass: the tile is requested before the
  // dependency wait, so its latency overlaps the tail of the conv kernel and this CTA's own row set-up.
  const int slot = slots[b];
  float* S = rec_state + ((static_cast<size_t>(slot) * HV + h) * DK) * DV;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    s_abort = 0;
    mbar_fence_init();
    mbar_expect_tx(&bar, TILE_BYTES);
    bulk_load(sS, S, TILE_BYTES, &bar);
  }
  pdl_wait();
  pdl_launch();
  __syncthreads();
  const float gw = __bfloat162float(gnorm_w[c]);
  const float a_log = A_log[h], dtb = dt_bias[h];

  for (int j = 0; j < G; ++j) {
    const size_t row = static_cast<size_t>(b) * G + j;
    const bf16* co = conv_out + row * C;
    // q and k of the key head: L2 normalise (q also scaled by DK^-0.5). Threads beyond DK contribute zeros; the
    // shuffles stay unconditional (every thread of the CTA takes part, which the host build of this file needs)
    float qv = 0.f, kv = 0.f;
    if (threadIdx.x < DK) {
      qv = __bfloat162float(co[hk * DK + threadIdx.x]);
      kv = __bfloat162float(co[key_dim + hk * DK + threadIdx.x]);
      sq[threadIdx.x] = qv; sk[threadIdx.x] = kv;
    }
    const float a = __bfloat162float(mixed[row * ld + a_off + h]);
    const float bb = __bfloat162float(mixed[row * ld + b_off + h]);
    const float v = __bfloat162float(co[2 * key_dim + h * DV + c]);
    const float z = (p == 0) ? __bfloat162float(mixed[row * ld + z_off + h * DV + c]) : 0.f;
    const float ssq = warp_sum(qv * qv), ssk = warp_sum(kv * kv), sqk = warp_sum(qv * kv);
    if ((threadIdx.x & 31) == 0 && threadIdx.x < DK) {
      nred[threadIdx.x >> 5][0] = ssq; nred[threadIdx.x >> 5][1] = ssk; nred[threadIdx.x >> 5][2] = sqk;
    }
    const float decay = __expf(-__expf(a_log) * softplus_f(a + dtb));
    const float beta = sigmoid_f(bb);
    __syncthreads();
    float tq = 0.f, tk = 0.f, tqk = 0.f;
#pragma unroll
    for (int i = 0; i < DK / 32; ++i) { tq += nred[i][0]; tk += nred[i][1]; tqk += nred[i][2]; }
    const float qs = rsqrtf(tq + 1e-6f) * rsqrtf(static_cast<float>(DK));
    const float ks = rsqrtf(tk + 1e-6f);
    const float kq = tqk * qs * ks;  // k . q of the normalised vectors

    // the first row's inputs are in registers: only now wait for the state tile
    if (j == 0 && !mbar_wait(&bar, 0, err, ERR_WAIT_FULL, &s_abort)) return;  // status recorded; the state is left as it was

    // pass 1: partial S^T k and S^T q over this thread's key rows, on the raw tile and the raw k / q: the decay and
    // the two normalisation factors are common to the whole sum and are applied once to its result. The column
    // segment stays in registers for pass 2; k and q come as 16-byte broadcast reads.
    float pk = 0.f, pq = 0.f;
    float colv[KP];
    float* col = sS + static_cast<size_t>(p * KP) * DV + c;
    const float4* k4 = reinterpret_cast<const float4*>(sk + p * KP);
    const float4* q4 = reinterpret_cast<const float4*>(sq + p * KP);
#pragma unroll
    for (int i4 = 0; i4 < KP / 4; ++i4) {
      const float4 kk = k4[i4], qq = q4[i4];
      const float ke[4] = {kk.x, kk.y, kk.z, kk.w}, qe[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float sv = col[(i4 * 4 + u) * DV];
        colv[i4 * 4 + u] = sv;
        pk += sv * ke[u];
        pq += sv * qe[u];
      }
    }
    red[p][c][0] = pk; red[p][c][1] = pq;
    __syncthreads();
    const float kv_mem = ((red[0][c][0] + red[1][c][0]) + (red[2][c][0] + red[3][c][0])) * (decay * ks);
    const float sq_mem = ((red[0][c][1] + red[1][c][1]) + (red[2][c][1] + red[3][c][1])) * (decay * qs);
    const float delta = (v - kv_mem) * beta;
    // pass 2: S = decay * S + k delta^T, in place
    const float kd = ks * delta;
#pragma unroll
    for (int i4 = 0; i4 < KP / 4; ++i4) {
      const float4 kk = k4[i4];
      const float ke[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) col[(i4 * 4 + u) * DV] = colv[i4 * 4 + u] * decay + ke[u] * kd;
    }
    const float o = sq_mem + delta * kq;  // = S_new^T q

    // gated RMSNorm over the head's DV outputs
    const bf16 ob = __float2bfloat16(o);
    const float of = __bfloat162float(ob);
    const float ss = warp_sum((p == 0) ? of * of : 0.f);
    if ((threadIdx.x & 31) == 0) wred[threadIdx.x >> 5] = ss;
    proxy_fence();  // the tile as updated by this thread, for the bulk stores issued after the barrier
    __syncthreads();
    if (j + 1 == G) {
      // last row: the slot (and the ring entry of this row) get the tile while the outputs are still being formed
      if (threadIdx.x == 0) {
        if (ring_rec) bulk_store(ring_rec + (((static_cast<size_t>(b) * G + j) * HV + h) * DK) * DV, sS, TILE_BYTES);
        bulk_store(S, sS, TILE_BYTES);
      }
    }
    if (p == 0) {
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < DV / 32; ++i) tot += wred[i];  // partition 0's warps only
      const float inv = rsqrtf(tot / DV + eps);
      const float nb = __bfloat162float(__float2bfloat16(of * inv));
      out[row * (HV * DV) + h * DV + c] = __float2bfloat16(gw * nb * silu_f(z));
    }
    if (ring_rec && j + 1 < G) {  // keep the state after this row; the tile may only change again once the store has read it
      if (threadIdx.x == 0) {
        bulk_store(ring_rec + (((static_cast<size_t>(b) * G + j) * HV + h) * DK) * DV, sS, TILE_BYTES);
        bulk_store_wait_read();
      }
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) bulk_store_wait_read();  // shared memory must outlive the stores that read it
}

}  // namespace b200

#ifndef B200_EMU
namespace b200 {
// After a verify pass: slot state <- state after row keep[b] of sequence b, for every GDN layer. The step kernel
// leaves the state after the LAST row in the slot, so sequences that keep every row need no copy; the others copy
// one contiguous row of the ring (conv: C x 3 bf16, recurrent: HV x DK x DV fp32). Grid (chunks, B, layers).
__global__ void ring_commit_kernel(uint4* conv_state, uint4* rec_state, const uint4* ring_conv, const uint4* ring_rec,
                                   const int* slots, const int64_t* keep, int B, int G, int n_slots, size_t conv_row,
                                   size_t rec_row) {
  const int b = blockIdx.y, layer = blockIdx.z;
  const int k = static_cast<int>(keep[b]);
  if (k >= G - 1 || k < 0) return;
  const size_t slot = static_cast<size_t>(slots[b]);
  const uint4* src_r = ring_rec + ((static_cast<size_t>(layer) * B + b) * G + k) * rec_row;
  uint4* dst_r = rec_state + (static_cast<size_t>(layer) * n_slots + slot) * rec_row;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < rec_row; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst_r[i] = src_r[i];
  const uint4* src_c = ring_conv + ((static_cast<size_t>(layer) * B + b) * G + k) * conv_row;
  uint4* dst_c = conv_state + (static_cast<size_t>(layer) * n_slots + slot) * conv_row;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < conv_row; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst_c[i] = src_c[i];
}
}  // namespace b200

using namespace b200;

// conv_state [layers, n_slots, conv_bytes], rec_state [layers, n_slots, rec_bytes], rings [layers, B, G, row bytes];
// the first n <= B sequences are committed; row sizes in bytes, multiples of 16.
extern "C" int b200_ring_commit(void* conv_state, void* rec_state, const void* ring_conv, const void* ring_rec,
                                const int* slots, const int64_t* keep, int layers, int B, int n, int G, int n_slots,
                                unsigned long long conv_bytes, unsigned long long rec_bytes, cudaStream_t st) {
  if (n <= 0 || layers <= 0) return 0;
  if (n > B) return -7;
  if (conv_bytes % 16 || rec_bytes % 16) return -7;
  ring_commit_kernel<<<dim3(32, n, layers), 256, 0, st>>>(
      static_cast<uint4*>(conv_state), static_cast<uint4*>(rec_state), static_cast<const uint4*>(ring_conv),
      static_cast<const uint4*>(ring_rec), slots, keep, B, G, n_slots, conv_bytes / 16, rec_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int b200_gdn_decode(const void* mixed, int ld, const int* slots, void* conv_state, void* rec_state,
                               const void* conv_w, const float* A_log, const float* dt_bias, const void* gnorm_w,
                               void* conv_out, void* out, void* ring_conv, float* ring_rec, int B, int G, int HK, int HV,
                               int DK, int DV, int KW, float eps, int* err, cudaStream_t st) {
  if (B <= 0) return 0;
  const int key_dim = HK * DK, value_dim = HV * DV, C = 2 * key_dim + value_dim;
  if (KW != 4) return -7;
  if (C % 8 || ld % 8) {
    if (launch_pdl(gdn_conv_step_scalar_kernel<4>, dim3((C + 127) / 128, B), dim3(128), 0, st,
                   static_cast<const bf16*>(mixed), ld, slots, static_cast<bf16*>(conv_state),
                   static_cast<const bf16*>(conv_w), static_cast<bf16*>(conv_out), static_cast<bf16*>(ring_conv), C,
                   G) != cudaSuccess) return -4;
  } else {
    if (launch_pdl(gdn_conv_step_kernel<4>, dim3((C / 8 + 63) / 64, B), dim3(64), 0, st,
                   static_cast<const bf16*>(mixed), ld, slots, static_cast<bf16*>(conv_state),
                   static_cast<const bf16*>(conv_w), static_cast<bf16*>(conv_out), static_cast<bf16*>(ring_conv), C,
                   G) != cudaSuccess) return -4;
  }
  dim3 grid(HV, B);
  const int z_off = C, b_off = C + value_dim, a_off = C + value_dim + HV;
#define LAUNCH_STEP(DKV)                                                                                           \
  do {                                                                                                             \
    auto kern = gdn_step_kernel<DKV, DKV>;                                                                         \
    constexpr int smem = DKV * DKV * 4;                                                                            \
    static bool configured[64] = {};                                                                               \
    int dev = 0;                                                                                                   \
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;                                     \
    if (!configured[dev]) {                                                                                        \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3; \
      configured[dev] = true;                                                                                      \
    }                                                                                                              \
    if (launch_pdl(kern, grid, dim3(4 * DKV), smem, st, static_cast<const bf16*>(conv_out),                        \
                   static_cast<const bf16*>(mixed), ld, z_off, b_off, a_off, slots, static_cast<float*>(rec_state), \
                   A_log, dt_bias, static_cast<const bf16*>(gnorm_w), static_cast<bf16*>(out), ring_rec, HK, HV, G, \
                   eps, err) != cudaSuccess) return -4;                                                            \
  } while (0)
  if (DK == 128 && DV == 128) LAUNCH_STEP(128);
  else if (DK == 32 && DV == 32) LAUNCH_STEP(32);
  else if (DK == 64 && DV == 64) LAUNCH_STEP(64);
  else return -7;
#undef LAUNCH_STEP
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
#endif  // B200_EMU
