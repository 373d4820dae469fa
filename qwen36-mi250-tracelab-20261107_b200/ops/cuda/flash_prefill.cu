// Causal gated flash attention for prefill spans over the paged KV cache, on tcgen05.
//
// One CTA per (query tile, kv head). A tile is 128 MMA rows = (128 / GROUP) consecutive query
// positions x the GROUP query heads that share the kv head, so every K/V page fetched by TMA is
// used by all heads of the group (reference: engine/fast/flash_prefill.py:97-186 tiles
// M = BLOCK_R x GROUP rows the same way on MFMA). Per 64-key page:
//
//   S[128 x 64]  = Q[128 x D] K[64 x D]^T      tcgen05.mma, both operands K-major, S in TMEM
//   softmax      : each of 128 threads owns one TMEM lane = one row, so row max / sum need no
//                  shuffles; P = exp2(S - m) goes to shared memory as bf16 in the swizzled K-major
//                  layout the next MMA reads; the O accumulator in TMEM is rescaled only when a
//                  row maximum grew by more than 2^8 (exact: the final division uses the same m)
//   O[128 x D]  += P[128 x 64] V[64 x D]       V is read straight from its page layout as an
//                                              MN-major B operand (no transpose)
//
// Warp 4 lane 0 drives TMA (Q once, K/V pages double-buffered) and issues all MMAs; warps 0..3
// do the softmax and the epilogue (divide by the row sum, multiply by sigmoid(gate), store bf16).
// Chunked prefill: queries sit at positions pos0.. of their sequence, keys are 0..pos.
// All waits are bounded (common.cuh). No cluster multicast.
#include "common.cuh"

namespace b200 {

constexpr int FP_PAGE = 64;

struct FlashParams {
  const int4* tiles;      // (segment, first local position, segment start row, segment length)
  const int* seg_pos0;    // position of each segment's first row
  const int* tables;      // [segments, max_pages]
  int max_pages;
  int num_pages;
  const bf16* gate;       // [T, n_q * D]
  bf16* out;              // [T, n_q * D]
  int n_q, n_kv;
  float scale_log2;       // D^-0.5 * log2(e)
  int* err;
  int split_pages;        // > 0: blockIdx.z handles pages [z*split, (z+1)*split) and writes partials
  float* part_acc;        // [T, n_q, gridDim.z, D] unnormalised partial outputs
  float* part_ml;         // [T, n_q, gridDim.z, 2] (row maximum in natural-log units, row sum)
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
// DEC (decode: one query position per tile, so GROUP <= 8 real rows): the Q and P operands keep only their first
// 8-row swizzle atom per 128-byte block (1 KB instead of 16 KB); the MMA still reads 128 rows from those bases, the
// other 120 come from whatever shared memory follows (the K/V stages) and land in accumulator rows nobody reads: an
// output row of an MMA depends on its own A row only. The 106 KB this frees hold a third K/V stage, so two pages
// are on their way while one is being used.
template <int D, bool DEC = false>
struct FlashCfg {
  static constexpr int DB = D / 64;             // 64-element (128-byte) blocks along the head dim
  static constexpr int Q_BLOCK = DEC ? 1024 : 128 * 128;  // bytes between the 64-element blocks of the Q tile
  static constexpr int Q_BYTES = DB * Q_BLOCK;
  static constexpr int KV_BYTES = DB * FP_PAGE * 128;  // one of K or V, one stage
  static constexpr int P_BYTES = DEC ? 1024 : 128 * 128;  // one probability tile; two are kept
  static constexpr int ST = DEC ? 3 : 2;        // K/V stages
  // dynamic shared memory is declared 1024-byte aligned (checked at run time), so no alignment slack is budgeted:
  // with D = 256 the tiles, the barriers and the 2 KB of static exchange arrays fill the 227 KB of an SM
  static constexpr int SMEM = Q_BYTES + 2 * ST * KV_BYTES + 2 * P_BYTES + 256;
  static constexpr int TMEM_COLS = (128 + D) <= 256 ? 256 : 512;  // two score tiles of 64 columns + the output
};

template <int D, int GROUP, bool DEC = false>
__global__ void __launch_bounds__(288, 1)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, FlashParams p) {
  using C = FlashCfg<D, DEC>;
  constexpr int DB = C::DB;
  constexpr int ST = C::ST;
  constexpr int R = DEC ? 1 : 128 / GROUP;  // query positions per tile
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need this alignment; leave with a status rather than compute garbage
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_INDEX);
    return;
  }
  // Q and P first: in the decode form the MMAs read past their real rows into the K/V stages that follow
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + C::Q_BYTES;               // [2][128 x 128 B] (decode: [2][8 x 128 B]): page i uses tile i & 1
  uint8_t* sK = sP + 2 * C::P_BYTES;           // [ST stages][DB][64 x 128 B]
  uint8_t* sV = sK + ST * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + ST * C::KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                // [ST]
  uint64_t* kv_empty = bars + 4;               // [ST]: completes when P.V of the page in that stage has finished
  uint64_t* s_full = bars + 7;                 // [2]: one per score tile
  uint64_t* p_full = bars + 9;
  uint64_t* acc_done = bars + 10;
  uint64_t* x_bar = bars + 11;                 // exchange point of the 256 softmax threads (bounded wait, unlike bar.sync)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  pdl_wait();  // the tile table, positions and Q / K / V all come from kernels earlier in the stream
  const int4 tile = p.tiles[blockIdx.x];
  const int seg = tile.x, p0 = tile.y, seg_row0 = tile.z, seg_len = tile.w;
  const int kh = blockIdx.y;
  const int pos0 = p.seg_pos0[seg];
  const int n_pos = min(R, seg_len - p0);
  if (n_pos <= 0) return;  // filler entry: a captured prefill pass keeps its tile table at a fixed length
  const int np_all = (pos0 + p0 + n_pos - 1) / FP_PAGE + 1;  // pages that hold visible keys
  // split mode: a fixed number of consecutive pages per CTA, so the partition of a sequence's context
  // depends on its own length only, never on what else is in the batch
  const int first = p.split_pages > 0 ? static_cast<int>(blockIdx.z) * p.split_pages : 0;
  const int np = p.split_pages > 0 ? max(0, min(np_all, first + p.split_pages) - first) : np_all;
  if (np == 0) {  // nothing for this split: publish an empty partial and leave before any barrier / TMEM use
    const int r = threadIdx.x;
    if (r < 128 && r / GROUP < n_pos) {
      const size_t row = static_cast<size_t>(seg_row0 + p0 + r / GROUP);
      float* pm = p.part_ml + ((row * p.n_q + kh * GROUP + r % GROUP) * gridDim.z + blockIdx.z) * 2;
      pm[0] = -INFINITY; pm[1] = 0.f;
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ST; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_full, 256);
    mbar_init(acc_done, 1);
    mbar_init(x_bar, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
  }
  if (warp == 8) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_launch();  // this CTA holds its TMEM columns: the next kernel's CTAs may queue behind it
  const uint32_t tmem_S = tmem, tmem_O = tmem + 128;  // score tile of page i at tmem_S + (i & 1) * 64

  if (warp == 8) {
    if (elect_one()) {
      auto load_page = [&](int i) {
        const int s = i % ST;
        int page = p.tables[static_cast<size_t>(seg) * p.max_pages + first + i];
        if (page < 0 || page >= p.num_pages) { atomicCAS(p.err, 0, ERR_BAD_INDEX); page = 0; }
        const int krow = ((page * 2 + 0) * p.n_kv + kh) * FP_PAGE;
        const int vrow = ((page * 2 + 1) * p.n_kv + kh) * FP_PAGE;
        mbar_expect_tx(&kv_full[s], 2 * C::KV_BYTES);
        for (int a = 0; a < DB; ++a) {
          tma_load_2d(sK + s * C::KV_BYTES + a * FP_PAGE * 128, &tmKV, &kv_full[s], a * 64, krow);
          tma_load_2d(sV + s * C::KV_BYTES + a * FP_PAGE * 128, &tmKV, &kv_full[s], a * 64, vrow);
        }
      };
      mbar_expect_tx(q_full, DEC ? DB * GROUP * 128 : C::Q_BYTES);  // decode: GROUP rows of 128 bytes per block
      for (int a = 0; a < DB; ++a) tma_load_4d(sQ + a * C::Q_BLOCK, &tmQ, q_full, a * 64, 0, kh, seg_row0 + p0);
      for (int i = 0; i < ST && i < np; ++i) load_page(i);
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 64);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, D) | (1u << 16);  // B operand MN-major
      // Software pipeline: Q K^T of page i + 1 is issued before the wait for the probabilities of page i, into the
      // other score tile, so the tensor pipe works on the next scores while the softmax threads are busy.
      bool ok = mbar_wait(q_full, 0, p.err, ERR_WAIT_FULL, abort_flag);
      const uint32_t qa = smem_u32(sQ);
      auto issue_qk = [&](int i) {
        const int s = i % ST;
        if (!mbar_wait(&kv_full[s], (i / ST) & 1, p.err, ERR_WAIT_FULL, abort_flag)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(sK + s * C::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t blk = kk >> 2, koff = (kk & 3) * 32;
          umma_bf16(tmem_S + (i & 1) * 64, umma_smem_desc(qa + blk * C::Q_BLOCK + koff),
                    umma_smem_desc(ka + blk * FP_PAGE * 128 + koff), idesc_qk, kk != 0);
        }
        umma_commit(&s_full[i & 1]);
        return true;
      };
      ok = ok && issue_qk(0);
      // The stage of page i - 1 is free once its P.V has finished; it takes page i - 1 + ST. With two stages that is
      // page i + 1, which Q K^T needs in this very iteration, so the refill comes first (and waits for the P.V just
      // issued). With three stages page i + 1 is already there and the refill waits until the softmax of page i has
      // run, by when P.V of page i - 1 is long done: two pages are loaded or on their way while page i is used.
      auto refill = [&](int i) {
        if (i < 1 || i - 1 + ST >= np) return true;
        if (!mbar_wait(&kv_empty[(i - 1) % ST], ((i - 1) / ST) & 1, p.err, ERR_WAIT_EMPTY, abort_flag)) return false;
        load_page(i - 1 + ST);
        return true;
      };
      for (int i = 0; i < np && ok; ++i) {
        const int s = i % ST;
        if (ST == 2) { ok = refill(i); if (!ok) break; }
        if (i + 1 < np) {
          ok = issue_qk(i + 1);  // its score tile was last read by the softmax of page i - 1, which has arrived at p_full
          if (!ok) break;
        }
        ok = mbar_wait(p_full, i & 1, p.err, ERR_WAIT_FULL, abort_flag);
        if (!ok) break;
        if (ST > 2) { ok = refill(i); if (!ok) break; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP + (i & 1) * C::P_BYTES), va = smem_u32(sV + s * C::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < FP_PAGE / 16; ++kk)
          umma_bf16(tmem_O, umma_smem_desc(pa + kk * 32), umma_smem_desc_mn(va + kk * 2048, FP_PAGE * 128), idesc_pv,
                    (i | kk) != 0);
        umma_commit(&kv_empty[s]);
      }
      umma_commit(acc_done);
    }
  } else {
    // ---------------- softmax + epilogue: 256 threads, two per TMEM lane. Thread (r = tid & 127, hf = tid >> 7) owns
    // row r = one (position, head) and the half hf of everything indexed by a column: 32 of the page's 64 scores,
    // half of the output columns. The two halves of a row agree on the row maximum through shared memory, so both
    // take the same rescale decision; their partial row sums are added (half 0 + half 1) at the end.
    __shared__ float s_mx[2][2][128];  // [page parity][half][row]; reused for the row sums at the end
    const int r = threadIdx.x & 127, hf = threadIdx.x >> 7;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int lp = r / GROUP, head = r % GROUP;
    const int qpos = pos0 + p0 + lp;
    const bool row_valid = lp < n_pos;
    constexpr int DH = D / 2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < np && ok; ++i) {
      ok = mbar_wait(&s_full[i & 1], (i >> 1) & 1, p.err, ERR_WAIT_TMEM, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float sc[32];
#pragma unroll
      for (int c = 0; c < 32; c += 16) tmem_ld16(tmem_S + (i & 1) * 64 + hf * 32 + lane_base + c, sc + c);
      float mx = -INFINITY;
      const int kbase = (first + i) * FP_PAGE + hf * 32;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        // decode: rows past the real ones hold whatever the MMA read behind the Q atom; masked, so that they never
        // ask for a rescale of the output tile
        sc[j] = (kbase + j <= qpos && (!DEC || row_valid)) ? sc[j] * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, sc[j]);
      }
      s_mx[i & 1][hf][r] = mx;
      mbar_arrive(x_bar);
      ok = mbar_wait(x_bar, i & 1, p.err, ERR_WAIT_FULL, abort_flag);
      if (!ok) break;
      mx = fmaxf(mx, s_mx[i & 1][hf ^ 1][r]);
      const bool need = mx > m_used + 8.0f;
      // The scores of this page were computed while P.V of the previous page may still be running. This page's
      // probability tile was last read by P.V of page i - 2; the output tile may only be rescaled once P.V of page
      // i - 1 has finished, which is waited for only in the (rare, after the first pages) case of a rescale.
      if (i >= 2) {
        ok = mbar_wait(&kv_empty[(i - 2) % ST], ((i - 2) / ST) & 1, p.err, ERR_WAIT_EMPTY, abort_flag);
        if (!ok) break;
      }
      const bool any_need = __any_sync(0xffffffffu, need);
      if (any_need && i > 0) {
        ok = mbar_wait(&kv_empty[(i - 1) % ST], ((i - 1) / ST) & 1, p.err, ERR_WAIT_EMPTY, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      if (any_need) {  // warp-uniform: TMEM loads/stores are warp-collective
        const float factor = need ? exp2f(m_used - mx) : 1.0f;  // exp2(-inf) = 0 on the first page
        if (need) { m_used = mx; l *= factor; }
        if (i > 0) {
#pragma unroll 1
          for (int c = 0; c < DH; c += 16) {
            float o[16];
            tmem_ld16(tmem_O + lane_base + hf * DH + c, o);
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] *= factor;
            tmem_st16(tmem_O + lane_base + hf * DH + c, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      float sum = 0.f;
      uint8_t* prow = sP + (i & 1) * C::P_BYTES + r * 128;
      if (!DEC || r < 8)  // decode: the probability tile holds one 8-row atom; the other rows' scores are not kept
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 packed;
        __nv_bfloat162* pe = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = exp2f(sc[c * 8 + 2 * j] - m_used), b2 = exp2f(sc[c * 8 + 2 * j + 1] - m_used);
          sum += a + b2;
          pe[j] = __floats2bfloat162_rn(a, b2);
        }
        *reinterpret_cast<uint4*>(prow + (((hf * 4 + c) ^ (r & 7)) * 16)) = packed;  // 128-byte swizzle of the K-major tile
      }
      l += sum;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(p_full);
    }
    ok = ok && mbar_wait(acc_done, 0, p.err, ERR_WAIT_TMEM, abort_flag) && !*abort_flag;
    tc_fence_after();
    if (ok) {
      // every thread has read its partner's last maximum (it arrived at p_full afterwards, and acc_done follows that)
      s_mx[0][hf][r] = l;
      mbar_arrive(x_bar);
      ok = mbar_wait(x_bar, np & 1, p.err, ERR_WAIT_FULL, abort_flag);
      l = s_mx[0][0][r] + s_mx[0][1][r];
    }
    if (ok && p.split_pages > 0) {
      const size_t row = static_cast<size_t>(seg_row0 + p0 + lp);
      const size_t slot = (row * p.n_q + kh * GROUP + head) * gridDim.z + blockIdx.z;
#pragma unroll 1
      for (int c = hf * DH; c < hf * DH + DH; c += 16) {
        float o[16];
        tmem_ld16(tmem_O + lane_base + c, o);  // warp-collective: never predicated
        if (row_valid) {
          float4* dst = reinterpret_cast<float4*>(p.part_acc + slot * D + c);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
      }
      if (row_valid && hf == 0) {
        p.part_ml[slot * 2] = m_used * 0.6931471805599453f;  // log2 units -> natural log, as the combine expects
        p.part_ml[slot * 2 + 1] = l;
      }
    } else
    if (ok) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      const size_t row = static_cast<size_t>(seg_row0 + p0 + lp);
      const size_t base = row * (static_cast<size_t>(p.n_q) * D) + static_cast<size_t>(kh * GROUP + head) * D;
#pragma unroll 1
      for (int c = hf * DH; c < hf * DH + DH; c += 16) {
        float o[16];
        tmem_ld16(tmem_O + lane_base + c, o);  // warp-collective: never predicated
        if (row_valid) {
          uint4 g0 = *reinterpret_cast<const uint4*>(p.gate + base + c), g1 = *reinterpret_cast<const uint4*>(p.gate + base + c + 8);
          const bf16* ge0 = reinterpret_cast<const bf16*>(&g0);
          const bf16* ge1 = reinterpret_cast<const bf16*>(&g1);
          uint4 o0, o1;
          bf16* oe0 = reinterpret_cast<bf16*>(&o0);
          bf16* oe1 = reinterpret_cast<bf16*>(&o1);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            oe0[j] = __float2bfloat16(__bfloat162float(__float2bfloat16(o[j] * inv)) * sigmoid_f(__bfloat162float(ge0[j])));
            oe1[j] = __float2bfloat16(__bfloat162float(__float2bfloat16(o[8 + j] * inv)) * sigmoid_f(__bfloat162float(ge1[j])));
          }
          *reinterpret_cast<uint4*>(p.out + base + c) = o0;
          *reinterpret_cast<uint4*>(p.out + base + c + 8) = o1;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

}  // namespace b200

using namespace b200;

namespace {
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn fp_encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}
int fp_make_map(CUtensorMap* m, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                const cuuint32_t* box) {
  EncodeFn fn = fp_encode_fn();
  if (!fn) return -1;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides_bytes, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

template <int D, int GROUP, bool DEC>
int fp_launch(const CUtensorMap& tq, const CUtensorMap& tkv, const FlashParams& p, int n_tiles, int gz, cudaStream_t st) {
  auto kern = flash_prefill_kernel<D, GROUP, DEC>;
  static bool configured[64] = {};  // a function attribute is set per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashCfg<D, DEC>::SMEM) != cudaSuccess) return -3;
    configured[dev] = true;
  }
  return launch_pdl(kern, dim3(n_tiles, p.n_kv, gz), dim3(288), FlashCfg<D, DEC>::SMEM, st, tq, tkv, p) == cudaSuccess ? 0 : -4;
}
}  // namespace

// q: [T, n_q, D] bf16 (already normed and rotated), gate/out: [T, n_q * D], kv: one layer of the paged pool
// [num_pages, 2, n_kv, 64, D]; tiles: int4 (segment, first local position, segment start row, segment length) with
// 128 / (n_q / n_kv) positions per tile; seg_pos0 / tables per segment. The span's K/V must already be in the pages.
extern "C" int b200_flash_prefill(const void* q, const void* gate, const void* kv, void* out, const void* tiles,
                                  int n_tiles, const int* seg_pos0, const int* tables, int max_pages, int num_pages,
                                  int T, int n_q, int n_kv, int D, int split_pages, int n_splits, float* part_acc,
                                  float* part_ml, int one_position, int* err, cudaStream_t st) {
  // one_position != 0: every tile holds a single query position (plain decode): the form with small Q / P tiles
  // and three K/V stages is used
  if (n_tiles <= 0) return 0;
  const int group = n_q / n_kv;
  if (group * n_kv != n_q || (D != 64 && D != 128 && D != 256) || 128 % group) return -7;
  CUtensorMap tq, tkv;
  {
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(group), static_cast<cuuint64_t>(n_kv),
                          static_cast<cuuint64_t>(T)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(group) * D * 2,
                             static_cast<cuuint64_t>(n_q) * D * 2};
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(group), 1, static_cast<cuuint32_t>(one_position ? 1 : 128 / group)};
    if (fp_make_map(&tq, q, 4, dims, strides, box)) return -1;
  }
  {
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(num_pages) * 2 * n_kv * FP_PAGE};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 2};
    cuuint32_t box[2] = {64, FP_PAGE};
    if (fp_make_map(&tkv, kv, 2, dims, strides, box)) return -1;
  }
  FlashParams p{static_cast<const int4*>(tiles), seg_pos0, tables, max_pages, num_pages, static_cast<const bf16*>(gate),
                static_cast<bf16*>(out), n_q, n_kv, 1.4426950408889634f / sqrtf(static_cast<float>(D)), err,
                split_pages, part_acc, part_ml};
  const int gz = split_pages > 0 ? n_splits : 1;
#define FP_GROUPS(DD)                                                         \
  if (one_position) switch (group) {                                          \
    case 1: return fp_launch<DD, 1, true>(tq, tkv, p, n_tiles, gz, st);           \
    case 2: return fp_launch<DD, 2, true>(tq, tkv, p, n_tiles, gz, st);           \
    case 4: return fp_launch<DD, 4, true>(tq, tkv, p, n_tiles, gz, st);           \
    case 8: return fp_launch<DD, 8, true>(tq, tkv, p, n_tiles, gz, st);           \
    default: return -7;                                                       \
  }                                                                           \
  switch (group) {                                                            \
    case 1: return fp_launch<DD, 1, false>(tq, tkv, p, n_tiles, gz, st);          \
    case 2: return fp_launch<DD, 2, false>(tq, tkv, p, n_tiles, gz, st);          \
    case 4: return fp_launch<DD, 4, false>(tq, tkv, p, n_tiles, gz, st);          \
    case 8: return fp_launch<DD, 8, false>(tq, tkv, p, n_tiles, gz, st);          \
    default: return -7;                                                       \
  }
  if (D == 256) { FP_GROUPS(256) }
  if (D == 128) { FP_GROUPS(128) }
  FP_GROUPS(64)
#undef FP_GROUPS
}
