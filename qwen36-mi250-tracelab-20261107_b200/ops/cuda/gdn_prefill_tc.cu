// Gated DeltaNet chunked prefill on the sm_100a tensor cores (head dims 128 x 128, 64-row chunks).
//
// Two kernels replace the fp32 CUDA-core WY transform and state pass of gdn_prefill.cu for the full-size model:
//
//  gdn_wy_tc   : one CTA per (pair of chunks, value head); thread i owns token row i of the 128 rows = TMEM lane i.
//                TMA brings the raw q / k / v rows of both chunks into 128B-swizzled tiles. tcgen05.mma forms the
//                128 x 128 Gram matrices K K^T and Q K^T (only the two 64 x 64 diagonal blocks are used), threads
//                turn them into A = (k beta) k^T decay (strictly lower) and the causal scores, each thread then
//                solves its own column of T = (I + A)^-1 by forward substitution, and a second pair of MMAs with
//                the block-diagonal T diag(beta) forms w = T (k beta e^g) and u = T (v beta). Everything the state
//                pass needs is written as bf16: w, u, q e^g, k e^{g_last - g}, scores, and g_last in fp32
//                (reference: engine/fast/gdn_chunk.py:203-471).
//  gdn_scan_tc : one CTA per (sequence, value head), chunks in order. The transposed fp32 state S^T [dv, dk] lives
//                in TMEM for the whole sequence, with a bf16 copy in shared memory as the MMA operand. Per chunk:
//                v_new^T = u^T - S^T w^T and o^T = S^T (q e^g)^T (tcgen05, N = 64 tokens), v_new goes to shared memory
//                as bf16, then o^T += v_new^T scores^T and S^T = S^T e^{g_last} + v_new^T (k e^{g_last-g})
//                (reference: engine/fast/gdn_chunk.py:494-628). A TMA producer warp runs two chunks ahead.
//
// Operands are rounded to bf16 where the reference's chunk kernels round them too (w, u, the decayed q / k, the
// state as an MMA operand); accumulation and the resident state are fp32. Padding rows of a partial chunk have
// beta = 0 and g = 0, which makes them identity rows of T and keeps them out of the state.
#include "common.cuh"

namespace b200 {

struct ChunkInfoTc {  // same layout as gdn_prefill.cu's ChunkInfo
  int seg, row0, nrows, first;
};

// Workspace (bytes) for NCH = chunks * heads: A-region [NCH * 256 rows][128] bf16 (w | u | qg | kg, 64 rows each),
// then the scores [NCH * 64 rows][64] bf16, then g_last fp32 [NCH].
__host__ __device__ inline size_t tc_region_b(size_t nch) { return nch * 65536; }
__host__ __device__ inline size_t tc_region_g(size_t nch) { return nch * 65536 + nch * 8192; }

// byte offset of the 16-byte chunk `c16` (0..7) of row `row` inside a 128B-swizzled tile atom
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t c16) { return row * 128 + ((c16 ^ (row & 7)) << 4); }

struct WyParams {
  const bf16* mixed;
  int ld, b_off, a_off;
  const ChunkInfoTc* chunks;
  int n_chunks;
  const float* A_log;
  const float* dt_bias;
  uint8_t* work;
  int HK, HV;
  int* err;
};

constexpr int WY_SMEM = 3 * 32768 + 1024 /*align*/ + 5120 /*small arrays + barriers*/;

// In-kernel phase clocks: thread 0 of CTA (0, 0) stamps clock64() at the phase boundaries of the WY kernel; the host
// reads the last launch's stamps with b200_gdn_wy_phase_clocks (the reference's HIP kernel has the same kind of
// phase clocks behind its PROF template argument, engine/fast/hip/gdn_chain.hip:163-165, 367-385).
__device__ long long g_wy_clocks[12];
#define WY_STAMP(k) do { if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) g_wy_clocks[k] = clock64(); } while (0)

// 256 threads. Row phases: thread (i = tid & 127, half = tid >> 7) works on token row i = TMEM lane i and on one
// 64-column half of it. Substitution phase: thread (col = tid >> 1, part = tid & 1) owns column col of T together with
// its neighbour lane; the pair splits every dot product and meets in one shuffle.
__global__ void __launch_bounds__(256, 2)
gdn_wy_tc_kernel(const __grid_constant__ CUtensorMap tmConv, WyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;            // raw q, later the fp32 A blocks, later the bf16 block-diagonal T diag(beta)
  uint8_t* sK = smem + 32768;    // raw k, later k e^g / |k|
  uint8_t* sV = smem + 65536;    // the substitution's columns (fp32), later raw v
  float* sG = reinterpret_cast<float*>(smem + 98304);  // [128] cumulative log decay
  float* sRk = sG + 128;                               // [128] 1 / |k|
  float* sBeta = sRk + 128;                            // [128]
  float* sPart = sBeta + 128;                          // [2][128][2] partial squared norms of the two row halves
  float* sFq = sPart + 512;                            // [128] row factors of the decayed q copy
  float* sFk = sFq + 128;                              // [128] row factors of the decayed k copy
  float* sTot = sFk + 128;                             // [4] warp totals of the scan
  uint64_t* bars = reinterpret_cast<uint64_t*>(sTot + 8);
  uint64_t* tma_bar = bars;
  uint64_t* mma_bar = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int i = tid & 127, half = tid >> 7;
  const int c = i >> 6, r = i & 63;  // chunk of the pair, row inside it
  const int h = blockIdx.y, hk = h / (p.HV / p.HK);
  const int key_dim = p.HK * 128;
  const int chunk_idx = 2 * blockIdx.x + c;
  const bool present = chunk_idx < p.n_chunks;
  const ChunkInfoTc ci = p.chunks[present ? chunk_idx : 2 * blockIdx.x];
  const bool valid = present && r < ci.nrows;

  if (tid == 0) {
    mbar_init(tma_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmConv);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;

  if (tid == 0) {
    // q and k rows of both chunks (a missing second chunk re-reads the first: finite data, never written out);
    // v arrives later: its region is scratch for the substitution first
    mbar_expect_tx(tma_bar, 2 * 32768);
    for (int cc = 0; cc < 2; ++cc) {
      const int idx = 2 * blockIdx.x + cc;
      const int row0 = p.chunks[idx < p.n_chunks ? idx : 2 * blockIdx.x].row0;
      for (int a = 0; a < 2; ++a) {
        tma_load_2d(sQ + a * 16384 + cc * 8192, &tmConv, tma_bar, hk * 128 + a * 64, row0);
        tma_load_2d(sK + a * 16384 + cc * 8192, &tmConv, tma_bar, key_dim + hk * 128 + a * 64, row0);
      }
    }
  }
  WY_STAMP(0);
  // gates and their inclusive scan inside each chunk (two warps per chunk; both halves compute the same values)
  float g = 0.f, beta = 0.f;
  if (valid) {
    const size_t row = static_cast<size_t>(ci.row0 + r);
    g = -__expf(p.A_log[h]) * softplus_f(__bfloat162float(p.mixed[row * p.ld + p.a_off + h]) + p.dt_bias[h]);
    beta = sigmoid_f(__bfloat162float(p.mixed[row * p.ld + p.b_off + h]));
  }
  float gs = g;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float x = __shfl_up_sync(0xffffffffu, gs, o);
    if (lane >= o) gs += x;
  }
  if (half == 0 && lane == 31) sTot[warp] = gs;
  __syncthreads();
  if (warp & 1) gs += sTot[(warp & 3) - 1];
  if (half == 0) { sG[i] = gs; sBeta[i] = beta; }
  __syncthreads();
  const float glast = sG[c * 64 + 63];

  WY_STAMP(1);  // gates done
  bool ok = mbar_wait(tma_bar, 0, p.err, ERR_WAIT_FULL, abort_flag);
  tc_fence_after();
  __syncthreads();
  if (tid == 0 && ok) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem, umma_smem_desc(ka + off), umma_smem_desc(ka + off), idesc, kk != 0);          // K K^T
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem + 128, umma_smem_desc(qa + off), umma_smem_desc(ka + off), idesc, kk != 0);    // Q K^T
    }
    umma_commit(mma_bar);
  }
  WY_STAMP(2);  // q / k tiles arrived, Gram MMAs issued
  // squared norms: each half sums its 64 columns of the q and k rows
  const uint32_t tile_row = i;  // row inside each 128-row atom
  {
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int c16 = 0; c16 < 8; ++c16) {
      const uint4 qv = *reinterpret_cast<const uint4*>(sQ + half * 16384 + swz(tile_row, c16));
      const uint4 kv = *reinterpret_cast<const uint4*>(sK + half * 16384 + swz(tile_row, c16));
      const bf16* qe = reinterpret_cast<const bf16*>(&qv);
      const bf16* ke = reinterpret_cast<const bf16*>(&kv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = __bfloat162float(qe[j]), y = __bfloat162float(ke[j]);
        sq += x * x;
        sk += y * y;
      }
    }
    sPart[(half * 128 + i) * 2] = sq;
    sPart[(half * 128 + i) * 2 + 1] = sk;
  }
  __syncthreads();
  const float rq = rsqrtf(sPart[i * 2] + sPart[(128 + i) * 2] + 1e-6f) * 0.08838834764831845f;  // 1 / |q| / sqrt(128)
  const float rk = rsqrtf(sPart[i * 2 + 1] + sPart[(128 + i) * 2 + 1] + 1e-6f);
  if (half == 0) {
    sRk[i] = rk;
    sFq[i] = rq * __expf(gs);
    sFk[i] = rk * __expf(glast - gs);
  }
  const size_t ch = static_cast<size_t>(present ? chunk_idx : 0) * p.HV + h;
  bf16* regA = reinterpret_cast<bf16*>(p.work) + ch * 256 * 128;
  if (present && r == 63 && half == 0)
    *reinterpret_cast<float*>(p.work + tc_region_g(static_cast<size_t>(p.n_chunks) * p.HV) + ch * 4) = glast;
  __syncthreads();
  // the decayed copies the state pass consumes, q e^g / |q| / sqrt(dk) and k e^{g_last - g} / |k|: warp w copies rows
  // [16 w, 16 w + 16); 16 lanes cover the 256 bytes of one row, so every store instruction writes two whole rows
#pragma unroll 2
  for (int it = 0; it < 8; ++it) {
    const int row = warp * 16 + it * 2 + (lane >> 4), chunk = lane & 15;
    const int cpr = row >> 6, rrow = row & 63;
    const int cidx = 2 * blockIdx.x + cpr;
    const uint32_t off = (chunk >> 3) * 16384 + swz(row, chunk & 7);
    const uint4 qv = *reinterpret_cast<const uint4*>(sQ + off);
    const uint4 kv = *reinterpret_cast<const uint4*>(sK + off);
    const float fq = sFq[row], fk = sFk[row];
    const bf16* qe = reinterpret_cast<const bf16*>(&qv);
    const bf16* ke = reinterpret_cast<const bf16*>(&kv);
    uint4 qo, ko;
    bf16* qoe = reinterpret_cast<bf16*>(&qo);
    bf16* koe = reinterpret_cast<bf16*>(&ko);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      qoe[j] = __float2bfloat16(__bfloat162float(qe[j]) * fq);
      koe[j] = __float2bfloat16(__bfloat162float(ke[j]) * fk);
    }
    if (cidx < p.n_chunks) {
      bf16* base = reinterpret_cast<bf16*>(p.work) + (static_cast<size_t>(cidx) * p.HV + h) * 256 * 128;
      reinterpret_cast<uint4*>(base + (128 + rrow) * 128)[chunk] = qo;
      reinterpret_cast<uint4*>(base + (192 + rrow) * 128)[chunk] = ko;
    }
  }
  WY_STAMP(3);  // norms + decayed copies written
  __syncthreads();  // sRk complete; every thread is done with the raw q tile
  ok = mbar_wait(mma_bar, 0, p.err, ERR_WAIT_TMEM, abort_flag) && !*abort_flag;
  tc_fence_after();

  WY_STAMP(4);  // Gram matrices in TMEM
  // A = (k beta) k^T decay, strictly lower, fp32 into the q region: element (r, j) of chunk c at
  // c * 16384 + r * 256 + (((j >> 2) + r) & 15) * 16 + (j & 3) * 4 bytes (row-rotated float4 groups).
  // Each half builds 32 of the row's 64 columns.
  float* sA = reinterpret_cast<float*>(sQ + c * 16384);
  bf16* regB = reinterpret_cast<bf16*>(p.work + tc_region_b(static_cast<size_t>(p.n_chunks) * p.HV)) + ch * 64 * 64;
#pragma unroll
  for (int jj0 = 0; jj0 < 32; jj0 += 16) {
    const int j0 = half * 32 + jj0;
    float kk[16], qk[16];
    tmem_ld16(tmem + lane_base + c * 64 + j0, kk);
    tmem_ld16(tmem + lane_base + 128 + c * 64 + j0, qk);
    uint4 so[2];
    bf16* soe = reinterpret_cast<bf16*>(so);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int jj = j0 + j;
      const float dec = jj <= r ? __expf(gs - sG[c * 64 + jj]) * sRk[c * 64 + jj] : 0.f;
      kk[j] = jj < r ? kk[j] * rk * beta * dec : 0.f;
      soe[j] = __float2bfloat16(qk[j] * rq * dec);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4)
      *reinterpret_cast<float4*>(sA + r * 64 + ((((j0 >> 2) + q4 + r) & 15) << 2)) =
          make_float4(kk[4 * q4], kk[4 * q4 + 1], kk[4 * q4 + 2], kk[4 * q4 + 3]);
    if (present) {
      reinterpret_cast<uint4*>(regB + r * 64 + j0)[0] = so[0];
      reinterpret_cast<uint4*>(regB + r * 64 + j0)[1] = so[1];
    }
  }
  // k <- k e^g / |k| in place (the first pair of MMAs has finished reading it); beta is folded into T below
  {
    const float fk = rk * __expf(gs);
#pragma unroll
    for (int c16 = 0; c16 < 8; ++c16) {
      uint4* kp = reinterpret_cast<uint4*>(sK + half * 16384 + swz(tile_row, c16));
      uint4 kv = *kp;
      bf16* ke = reinterpret_cast<bf16*>(&kv);
#pragma unroll
      for (int j = 0; j < 8; ++j) ke[j] = __float2bfloat16(__bfloat162float(ke[j]) * fk);
      *kp = kv;
    }
  }
  __syncthreads();
  WY_STAMP(5);  // A built, k scaled
  // T = (I + A)^-1 by forward substitution. Lanes (2m, 2m + 1) of a warp own column col = tid >> 1 of T: entry j of
  // the column lives at sC[(j >> 2) * 512 + col * 4 + (j & 3)] (the v region, free until v is loaded); the pair
  // splits the groups of four entries of every dot product by parity and adds the halves with one shuffle. A column
  // is private to its pair and the reads of A are the same addresses across the warp, so only __syncwarp is needed.
  {
    const int col = tid >> 1, part = tid & 1;
    const int cc = col >> 6, rr = col & 63;
    const float* sAc = reinterpret_cast<const float*>(sQ + cc * 16384);
    float* sC = reinterpret_cast<float*>(sV);
    // Blocked by 16 rows so that a column entry is read from shared memory once per BLOCK, not once per row: for
    // block b, first the panel acc[i] = sum over earlier blocks' entries j of A[16 b + i][j] T[j] (the pair splits
    // the groups of four j by parity and meets in 16 shuffles), then the 16 x 16 triangle with the block's own
    // entries in registers, then one store of the block's 16 entries. Blocks that lie entirely above every diagonal
    // of the warp's columns are zero and skipped.
    const int lo = (warp & 3) * 16;  // smallest column of this warp inside its chunk
#pragma unroll 1
    for (int blk = 0; blk < 4; ++blk) {
      float t[16];
      if (16 * blk + 15 < lo) {  // warp-uniform
        if (part == 0) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) *reinterpret_cast<float4*>(sC + (4 * blk + q4) * 512 + col * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        continue;
      }
      float acc[16];
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) acc[ii] = 0.f;
#pragma unroll 1
      for (int j4 = (lo >> 2) + part; j4 < 4 * blk; j4 += 2) {
        const float4 c4 = *reinterpret_cast<const float4*>(sC + j4 * 512 + col * 4);
#pragma unroll
        for (int ii = 0; ii < 16; ++ii) {
          const int row = 16 * blk + ii;
          const float4 a4 = *reinterpret_cast<const float4*>(sAc + row * 64 + (((j4 + row) & 15) << 2));
          acc[ii] += (a4.x * c4.x + a4.y * c4.y) + (a4.z * c4.z + a4.w * c4.w);
        }
      }
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) acc[ii] += __shfl_xor_sync(0xffffffffu, acc[ii], 1);
      // the block's own triangle: both lanes of the pair compute it (entries in registers, static indices)
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) {
        const int row = 16 * blk + ii;
        float a = acc[ii];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          if (4 * q4 < ii) {
            const float4 a4 = *reinterpret_cast<const float4*>(sAc + row * 64 + (((4 * blk + q4 + row) & 15) << 2));
            if (4 * q4 + 0 < ii) a += a4.x * t[4 * q4 + 0];
            if (4 * q4 + 1 < ii) a += a4.y * t[4 * q4 + 1];
            if (4 * q4 + 2 < ii) a += a4.z * t[4 * q4 + 2];
            if (4 * q4 + 3 < ii) a += a4.w * t[4 * q4 + 3];
          }
        }
        t[ii] = row > rr ? -a : (row == rr ? 1.f : 0.f);
      }
      if (part == 0) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          *reinterpret_cast<float4*>(sC + (4 * blk + q4) * 512 + col * 4) = make_float4(t[4 * q4], t[4 * q4 + 1], t[4 * q4 + 2], t[4 * q4 + 3]);
      }
      __syncwarp();
    }
    WY_STAMP(6);  // substitution done (this warp)
    __syncthreads();  // every thread has finished reading A: the region becomes the bf16 operand tile
    // T diag(beta), block-diagonal, as a K-major A operand: row (cc * 64 + ii), K index (cc * 64 + rr) -> atom cc;
    // the pair writes alternate rows
    uint8_t* tile = sQ + cc * 16384;
    const float bcol = sBeta[col];
#pragma unroll 8
    for (int ii = part; ii < 64; ii += 2)
      *reinterpret_cast<bf16*>(tile + swz(cc * 64 + ii, rr >> 3) + (rr & 7) * 2) =
          __float2bfloat16(sC[(ii >> 2) * 512 + col * 4 + (ii & 3)] * bcol);
  }
  {  // the other atom's rows of this chunk are zero: w = (T diag(beta)) (k e^g), u = (T diag(beta)) v
    uint8_t* other = sQ + (1 - c) * 16384;
#pragma unroll
    for (int c16 = 0; c16 < 4; ++c16) *reinterpret_cast<uint4*>(other + swz(tile_row, half * 4 + c16)) = make_uint4(0, 0, 0, 0);
  }
  WY_STAMP(7);  // T tile written
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && ok) {
    tc_fence_after();
    // the v rows of both chunks replace the scratch columns while the first MMA runs
    mbar_expect_tx(tma_bar, 32768);
    for (int cc = 0; cc < 2; ++cc) {
      const int idx = 2 * blockIdx.x + cc;
      const int row0 = p.chunks[idx < p.n_chunks ? idx : 2 * blockIdx.x].row0;
      for (int a = 0; a < 2; ++a)
        tma_load_2d(sV + a * 16384 + cc * 8192, &tmConv, tma_bar, 2 * key_dim + h * 128 + a * 64, row0);
    }
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128) | (1u << 16);  // B operand MN-major: [token][feature]
    const uint32_t ta = smem_u32(sQ), ka = smem_u32(sK), va = smem_u32(sV);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
      umma_bf16(tmem, umma_smem_desc(ta + aoff), umma_smem_desc_mn(ka + kk * 2048, 16384), idesc, kk != 0);        // w
    }
    if (!mbar_wait(tma_bar, 1, p.err, ERR_WAIT_FULL, abort_flag)) ok = false;
    tc_fence_after();
    if (ok) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
        umma_bf16(tmem + 128, umma_smem_desc(ta + aoff), umma_smem_desc_mn(va + kk * 2048, 16384), idesc, kk != 0);  // u
      }
    }
    umma_commit(mma_bar);
  }
  WY_STAMP(8);  // second pair of MMAs issued
  ok = mbar_wait(mma_bar, 1, p.err, ERR_WAIT_TMEM, abort_flag) && !*abort_flag;
  tc_fence_after();
  WY_STAMP(9);  // w / u in TMEM
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {  // 0: w -> rows [0, 64), 1: u -> rows [64, 128) of the chunk's A-region
    uint4* dst = reinterpret_cast<uint4*>(regA + (which * 64 + r) * 128) + half * 8;
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 16) {
      float v[16];
      tmem_ld16(tmem + lane_base + which * 128 + half * 64 + c0, v);  // warp-collective: never predicated
      uint4 o[2];
      bf16* oe = reinterpret_cast<bf16*>(o);
#pragma unroll
      for (int j = 0; j < 16; ++j) oe[j] = __float2bfloat16(v[j]);
      if (present && ok) { dst[c0 / 8] = o[0]; dst[c0 / 8 + 1] = o[1]; }
    }
  }
  WY_STAMP(10);  // w / u written
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

}  // namespace b200

namespace b200 {

// ------------------------------------------------------------------ state pass
struct ScanParams {
  const ChunkInfoTc* chunks;
  const int2* seg_chunks;  // (first chunk, number of chunks) per sequence
  const int* slots;
  float* rec_state;        // [slots, HV, 128 (dk), 128 (dv)] fp32
  const float* glast;      // [n_chunks * HV]
  bf16* o_out;             // [T, HV * 128]
  int HV;
  int* err;
};

constexpr int SC_STAGE = 4 * 16384 + 8192;  // w | u | qg | kg | scores
constexpr int SC_SMEM = 32768 + 16384 + 2 * SC_STAGE + 1024 /*align*/ + 256 /*barriers*/;

__global__ void __launch_bounds__(192, 1)
gdn_scan_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sS = smem;                 // bf16 S^T [128 dv][128 dk], two K atoms
  uint8_t* sVN = smem + 32768;        // bf16 v_new^T [128 dv][64 tokens]
  uint8_t* stages = smem + 49152;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stages + 2 * SC_STAGE);
  uint64_t* full = bars;              // [2]
  uint64_t* empty = bars + 2;         // [2]
  uint64_t* vn_done = bars + 4;       // MMA -> threads: v_new and the state part of o are in TMEM
  uint64_t* vn_ready = bars + 5;      // threads -> MMA: bf16 v_new in shared memory, state scaled (128 arrivals)
  uint64_t* o_done = bars + 6;        // MMA -> threads: o complete, state updated
  uint64_t* s_ready = bars + 7;       // threads -> MMA: bf16 state copy refreshed (128 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = blockIdx.x, h = blockIdx.y;
  const int2 sc = p.seg_chunks[seg];
  const int nc = sc.y;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(vn_done, 1);
    mbar_init(vn_ready, 128);
    mbar_init(o_done, 1);
    mbar_init(s_ready, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_S = tmem, tmem_VN = tmem + 128, tmem_O = tmem + 192;

  if (warp == 0) {
    if (elect_one()) {
      for (int i = 0; i < nc; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&empty[s], ((i >> 1) & 1) ^ 1, p.err, ERR_WAIT_EMPTY, abort_flag)) break;
        uint8_t* st = stages + s * SC_STAGE;
        const int ch = (sc.x + i) * p.HV + h;
        mbar_expect_tx(&full[s], SC_STAGE);
        for (int part = 0; part < 4; ++part)
          for (int a = 0; a < 2; ++a)
            tma_load_2d(st + part * 16384 + a * 8192, &tmA, &full[s], a * 64, ch * 256 + part * 64);
        tma_load_2d(st + 65536, &tmB, &full[s], 0, ch * 64);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc64 = umma_idesc_bf16(128, 64);
      constexpr uint32_t idesc_kg = umma_idesc_bf16(128, 128) | (1u << 16);  // B MN-major: [token][dk]
      const uint32_t sa = smem_u32(sS), vna = smem_u32(sVN);
      for (int i = 0; i < nc; ++i) {
        const int s = i & 1;
        const uint32_t st = smem_u32(stages + s * SC_STAGE);
        if (!mbar_wait(&full[s], (i >> 1) & 1, p.err, ERR_WAIT_FULL, abort_flag)) break;
        if (!mbar_wait(s_ready, i & 1, p.err, ERR_WAIT_FULL, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // v_new^T partial: S^T w^T, contraction over dk
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32, boff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_VN, umma_smem_desc(sa + aoff), umma_smem_desc(st + boff), idesc64, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // o^T = S^T (q e^g)^T
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32, boff = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_O, umma_smem_desc(sa + aoff), umma_smem_desc(st + 32768 + boff), idesc64, kk != 0);
        }
        umma_commit(vn_done);
        if (!mbar_wait(vn_ready, i & 1, p.err, ERR_WAIT_FULL, abort_flag)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)    // o^T += v_new^T scores^T, contraction over the chunk's tokens
          umma_bf16(tmem_O, umma_smem_desc(vna + kk * 32), umma_smem_desc(st + 65536 + kk * 32), idesc64, 1);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)    // S^T += v_new^T (k e^{g_last - g})
          umma_bf16(tmem_S, umma_smem_desc(vna + kk * 32), umma_smem_desc_mn(st + 49152 + kk * 2048, 8192), idesc_kg, 1);
        umma_commit(&empty[s]);
        umma_commit(o_done);
      }
    }
  } else {
    // ---------------- thread dv owns TMEM lane dv: one row of S^T, v_new^T and o^T
    const int q = warp & 3;
    const int dv = q * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    float* Sg = p.rec_state + (static_cast<size_t>(p.slots[seg]) * p.HV + h) * 128 * 128;
    // initial state: S[k][dv] -> TMEM row dv and the bf16 copy
#pragma unroll 1
    for (int k0 = 0; k0 < 128; k0 += 16) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = Sg[static_cast<size_t>(k0 + j) * 128 + dv];
      tmem_st16(tmem_S + lane_base + k0, v);
      uint4 o[2];
      bf16* oe = reinterpret_cast<bf16*>(o);
#pragma unroll
      for (int j = 0; j < 16; ++j) oe[j] = __float2bfloat16(v[j]);
      uint8_t* atom = sS + (k0 >> 6) * 16384;
      *reinterpret_cast<uint4*>(atom + swz(dv, (k0 & 63) >> 3)) = o[0];
      *reinterpret_cast<uint4*>(atom + swz(dv, ((k0 & 63) >> 3) + 1)) = o[1];
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    mbar_arrive(s_ready);
    bool ok = true;
    for (int i = 0; i < nc && ok; ++i) {
      const int s = i & 1;
      const uint8_t* st = stages + s * SC_STAGE;
      const int cidx = sc.x + i;
      const ChunkInfoTc ci = p.chunks[cidx];
      const float eg = __expf(p.glast[static_cast<size_t>(cidx) * p.HV + h]);
      ok = mbar_wait(vn_done, i & 1, p.err, ERR_WAIT_TMEM, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // v_new^T[dv][t] = u[t][dv] - (S^T w^T)[dv][t], as bf16 into the K-major operand tile (row dv, 64 tokens)
      const uint8_t* su = st + 16384 + (dv >> 6) * 8192;
      const uint32_t ucol = ((dv & 63) >> 3), ubyte = (dv & 7) * 2;
#pragma unroll
      for (int t0 = 0; t0 < 64; t0 += 16) {
        float v[16];
        tmem_ld16(tmem_VN + lane_base + t0, v);
        uint4 o[2];
        bf16* oe = reinterpret_cast<bf16*>(o);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float u = __bfloat162float(*reinterpret_cast<const bf16*>(su + swz(t0 + j, ucol) + ubyte));
          oe[j] = __float2bfloat16(u - v[j]);
        }
        *reinterpret_cast<uint4*>(sVN + swz(dv, t0 >> 3)) = o[0];
        *reinterpret_cast<uint4*>(sVN + swz(dv, (t0 >> 3) + 1)) = o[1];
      }
      // S^T *= e^{g_last} before the MMA adds this chunk's update
#pragma unroll 1
      for (int k0 = 0; k0 < 128; k0 += 16) {
        float v[16];
        tmem_ld16(tmem_S + lane_base + k0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= eg;
        tmem_st16(tmem_S + lane_base + k0, v);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(vn_ready);
      ok = mbar_wait(o_done, i & 1, p.err, ERR_WAIT_TMEM, abort_flag);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int t0 = 0; t0 < 64; t0 += 16) {
        float v[16];
        tmem_ld16(tmem_O + lane_base + t0, v);  // warp-collective: never predicated
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (t0 + j < ci.nrows)
            p.o_out[(static_cast<size_t>(ci.row0 + t0 + j) * p.HV + h) * 128 + dv] = __float2bfloat16(v[j]);
      }
      const bool last = i + 1 == nc;
#pragma unroll 1
      for (int k0 = 0; k0 < 128; k0 += 16) {
        float v[16];
        tmem_ld16(tmem_S + lane_base + k0, v);
        if (last) {
#pragma unroll
          for (int j = 0; j < 16; ++j) Sg[static_cast<size_t>(k0 + j) * 128 + dv] = v[j];
        } else {
          uint4 o[2];
          bf16* oe = reinterpret_cast<bf16*>(o);
#pragma unroll
          for (int j = 0; j < 16; ++j) oe[j] = __float2bfloat16(v[j]);
          uint8_t* atom = sS + (k0 >> 6) * 16384;
          *reinterpret_cast<uint4*>(atom + swz(dv, (k0 & 63) >> 3)) = o[0];
          *reinterpret_cast<uint4*>(atom + swz(dv, ((k0 & 63) >> 3) + 1)) = o[1];
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(s_ready);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

}  // namespace b200

using namespace b200;

namespace {
typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TcEncodeFn tc_encode_fn() {
  static TcEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess)
      fn = reinterpret_cast<TcEncodeFn>(ptr);
  }
  return fn;
}
// bf16 [rows, cols] row-major with row stride `ld` elements; box 64 columns x 64 rows, 128-byte swizzle, zero fill
int tc_map_2d(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t ld) {
  TcEncodeFn fn = tc_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, 64};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -2;
}
}  // namespace

// Phase clocks of CTA (0, 0) of the last WY launch on the current device: 11 clock64() stamps (see WY_STAMP).
extern "C" int b200_gdn_wy_phase_clocks(long long* out11) {
  return cudaMemcpyFromSymbol(out11, g_wy_clocks, 11 * sizeof(long long)) == cudaSuccess ? 0 : -1;
}

// Workspace bytes per (chunk, head) of the tensor-core path (fits inside the fp32 path's workspace).
extern "C" int b200_gdn_prefill_tc_work_bytes() { return 65536 + 8192 + 4; }

// Tensor-core WY transform + state pass for DK = DV = 128. Arguments as b200_gdn_prefill's second half: conv_out
// [T, C] bf16 holds the convolved q | k | v, `work` holds at least n_chunks * HV * b200_gdn_prefill_tc_work_bytes()
// bytes (256-byte aligned), o_tmp receives the un-normalised outputs [T, HV * 128].
extern "C" int b200_gdn_prefill_tc(const void* mixed, int ld, const void* conv_out, const void* chunks, int n_chunks,
                                   const void* seg_chunks, int n_seg, const int* slots, float* rec_state,
                                   const float* A_log, const float* dt_bias, void* work, void* o_tmp, int T, int HK,
                                   int HV, int* err, cudaStream_t st) {
  if (n_chunks <= 0) return 0;
  const int key_dim = HK * 128, value_dim = HV * 128, C = 2 * key_dim + value_dim;
  const size_t nch = static_cast<size_t>(n_chunks) * HV;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gdn_wy_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WY_SMEM) != cudaSuccess) return -3;
    if (cudaFuncSetAttribute(gdn_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_SMEM) != cudaSuccess) return -3;
    configured = true;
  }
  CUtensorMap tc, ta, tb;
  if (tc_map_2d(&tc, conv_out, C, T, C)) return -1;
  if (tc_map_2d(&ta, work, 128, nch * 256, 128)) return -1;
  if (tc_map_2d(&tb, static_cast<uint8_t*>(work) + tc_region_b(nch), 64, nch * 64, 64)) return -1;
  WyParams wp{static_cast<const bf16*>(mixed), ld, C + value_dim, C + value_dim + HV,
              static_cast<const ChunkInfoTc*>(chunks), n_chunks, A_log, dt_bias, static_cast<uint8_t*>(work), HK, HV, err};
  gdn_wy_tc_kernel<<<dim3((n_chunks + 1) / 2, HV), 256, WY_SMEM, st>>>(tc, wp);
  ScanParams sp{static_cast<const ChunkInfoTc*>(chunks), static_cast<const int2*>(seg_chunks), slots, rec_state,
                reinterpret_cast<const float*>(static_cast<uint8_t*>(work) + tc_region_g(nch)),
                static_cast<bf16*>(o_tmp), HV, err};
  gdn_scan_tc_kernel<<<dim3(n_seg, HV), 192, SC_SMEM, st>>>(ta, tb, sp);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
