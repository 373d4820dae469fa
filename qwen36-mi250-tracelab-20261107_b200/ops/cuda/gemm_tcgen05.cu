// Weight-stationary ("swap-AB") bf16 GEMM on the sm_100a tensor cores.
//
//   out[t, n] = sum_k X[t, k] * W[n, k]          X: [T, K] activations, W: [N, K] weights
//
// The MMA's M dimension (128 TMEM lanes) runs over *weight rows*, its N dimension over
// *token rows* (16..256 per tile). A decode step with a handful of rows and a prefill pass
// with thousands therefore use the same instruction shape along K; the accumulation order of
// one output element never depends on how many other rows share the launch, which is what
// keeps a request's greedy tokens identical whether it is served alone or in a batch (the
// reference gets the same property from fixed GEMV tiles, engine/fast/mfma.py:6-11, 60-71).
//
// Pipeline per CTA (192 threads): warp 0 = TMA producer, warp 1 = tcgen05.mma issuer and TMEM
// owner, warps 2..5 = epilogue (one TMEM lane quarter each). Operand tiles are 64 bf16 wide
// (128 bytes, TMA 128B swizzle), STAGES deep, guarded by full/empty mbarriers; tcgen05.commit
// releases a stage when the MMAs that read it have finished. No cluster multicast is used.
//
// Variants (template): plain store (bf16 or fp32), SiLU(gate)*up over two accumulators,
// per-tile argmax partials for the LM head, and a grouped mode where a device-side tile table
// names (expert, first row, row count) for each token tile of an expert-sorted activation
// buffer (replaces the reference's Triton GEMV / grouped GEMM family: engine/fast/mfma.py:90-179,
// engine/fast/moe_prefill.py:156-319, engine/fast/fused.py:581-692).
#include "comm.cuh"

namespace b200 {

constexpr int BM = 128;  // weight rows per tile (TMEM lanes)
constexpr int BK = 64;   // bf16 per operand row per stage (128 bytes)
constexpr int GATHER_BT_MAX = 64;  // widest token tile whose rows the grouped GEMM's producer warp can fetch by index
constexpr int UMMA_K = 16;
constexpr int MAX_DEVICES = 64;  // per-device launch state (function attributes, SM counts)

enum Epilogue : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU_MUL = 2, EPI_ARGMAX = 3, EPI_ALLREDUCE = 4, EPI_SCATTER = 5, EPI_REDUCE_SCATTER = 6 };

struct GemmParams {
  int N;             // weight rows (per expert when grouped)
  int K;
  int T;             // activation rows (dense) or capacity of the sorted buffer (grouped)
  int ldo;           // output row stride in elements
  void* out;         // bf16 or fp32 [T, ldo]
  const int4* tiles; // grouped: (expert, row0, nrows, 0) per token tile
  const int* n_tiles;// grouped: number of valid entries in `tiles`
  int up_offset;     // EPI_SILU_MUL: row offset of the "up" half inside W
  float* part_max;   // EPI_ARGMAX: [n_tiles_n, T]
  int* part_idx;     // EPI_ARGMAX: [n_tiles_n, T]
  int* err;          // error word (0 = ok)
  const bf16* residual; // EPI_ALLREDUCE: optional [T, ldo] added after the cross-rank sum
  CommCtx comm;      // EPI_ALLREDUCE: the rank group's symmetric buffers
  int rows_per_rank; // EPI_REDUCE_SCATTER / gathered X: token rows owned by each rank (a multiple of the token tile)
  const uint32_t* x_flags;  // gathered X: per-owner arrival epochs of this rank's full activation buffer (or null)
  const uint32_t* x_epoch;  // gathered X: the epoch the current call waits for
  int splits;        // split-K: CTAs of one cluster share an output tile, each taking 1/splits of the k-blocks
  const int2* meta;  // EPI_SCATTER: (source rank, pair slot) of every sorted row
  bf16* pair_out[MAX_RANKS];  // EPI_SCATTER: every rank's pair-output buffer [pairs, ldo] as mapped here
  int y_rot;         // dense sequence-parallel GEMMs: token tile = (blockIdx.y + y_rot) % gridDim.y, so that each rank
                     // starts with the tiles whose data (or whose consumer) is furthest from being the bottleneck
  int grid_y;        // dense: number of token tiles (set by the launcher)
  const int* gather_rows;  // grouped, token tiles <= 64 rows: sorted position -> row of `gx`; the producer warp then
                     // fetches each activation row by index (16-byte async copies into the swizzled operand layout)
                     // instead of reading an expert-sorted copy through the tensor map
  const bf16* gx;    // gather source [rows, ldgx]
  int ldgx;
  int packed;        // W is stored tile by tile: [expert][weight tile][k-block][128 * A_TILES rows][64], each (tile,
                     // k-block) one contiguous 16 KB (32 KB with the up half) run, so a stage is one sequential DRAM read
  int w_tiles;       // packed: weight tiles per expert
};

template <int BT, int EPI>
struct Cfg {
  static constexpr int A_TILES = (EPI == EPI_SILU_MUL) ? 2 : 1;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BT * BK * 2;
  static constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
  // small token tiles (decode) leave room for two CTAs per SM: one CTA's pipeline fill and epilogue
  // overlap the other's main loop, which matters when K is short (the MoE down projection has 8 k-blocks)
  // The fused gate/up GEMM at 16-row token tiles runs three CTAs per SM with two deep stages each: the same bytes in
  // flight per SM, but a decode step's ~1300 tiles then fill 2.9 waves of 444 CTAs instead of 4.4 waves of 296, and
  // the partial last wave is what the weight-streaming time loses.
  static constexpr int CTAS_PER_SM = (BT <= 16 && EPI == EPI_SILU_MUL) ? 3 : BT <= 64 ? 2 : 1;
  static constexpr int BUDGET = CTAS_PER_SM == 3 ? 72 * 1024 : BT <= 64 ? 108 * 1024 : 200 * 1024;
  static constexpr int STAGES_RAW = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int ACC_COLS = A_TILES * BT;  // one accumulator stage
  // two accumulator stages whenever they fit (512 columns per SM shared by the resident CTAs): the epilogue of
  // one tile then overlaps the main loop of the CTA's next tile
  static constexpr int ACC_STAGES = (2 * ACC_COLS * CTAS_PER_SM <= 512) ? 2 : 1;
  static constexpr int TMEM_COLS_RAW = ACC_COLS * ACC_STAGES;
  static constexpr int TMEM_COLS = TMEM_COLS_RAW <= 32 ? 32 : TMEM_COLS_RAW <= 64 ? 64 : TMEM_COLS_RAW <= 128 ? 128 : TMEM_COLS_RAW <= 256 ? 256 : 512;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BT, int EPI, bool GROUPED, bool SPLIT = false>
__global__ void __launch_bounds__(192, Cfg<BT, EPI>::CTAS_PER_SM)
gemm_swapab_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmParams p) {
  using C = Cfg<BT, EPI>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* acc_full = bars + 2 * C::STAGES;   // [2]
  uint64_t* acc_empty = bars + 2 * C::STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float red_max[4][BT > 0 ? BT : 1];
  __shared__ int red_idx[4][BT > 0 ? BT : 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The grouped tile table is written by the kernel just before this one: wait for it before the first read.
  // Dense launches wait later (the producer streams the first weight stages before it waits).
  if (GROUPED) pdl_wait();
  // Persistent tile loop: CTA b takes output tiles b, b + gridDim.x, ... (weight tile fastest, so CTAs that run
  // together share the activation tile). A split-K cluster takes the single tile its grid position names.
  const int tiles_n = (p.N + BM - 1) / BM;
  const int tiles_y = GROUPED ? *p.n_tiles : p.grid_y;
  const int total = tiles_n * tiles_y;
  const int tile0 = SPLIT ? static_cast<int>(blockIdx.y) * tiles_n + static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int tstep = SPLIT ? (1 << 30) : static_cast<int>(gridDim.x);
  constexpr int ACC = SPLIT ? 1 : C::ACC_STAGES;
  if (SPLIT && tile0 >= total) return;  // the whole cluster leaves together, before any barrier or TMEM use
  const int num_k_all = (p.K + BK - 1) / BK;
  // split-K: the cluster's CTAs (blockIdx.z = rank in the cluster) take consecutive runs of k-blocks; their fp32
  // partial tiles meet in the leader through distributed shared memory, added in rank order
  const int k_per = SPLIT ? (num_k_all + p.splits - 1) / p.splits : num_k_all;
  const int kb0 = SPLIT ? static_cast<int>(blockIdx.z) * k_per : 0;
  const int num_k = SPLIT ? max(0, min(num_k_all, kb0 + k_per) - kb0) : num_k_all;

  if (threadIdx.x == 0) {
    // a gathering producer: lane 0's expect_tx arrival for the weight tile plus one arrival per lane when that
    // lane's row copies have landed
    const uint32_t full_count = (GROUPED && BT <= GATHER_BT_MAX && p.gather_rows != nullptr) ? 33 : 1;
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], full_count); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // geometry of output tile `tile`
  auto tile_geom = [&](int tile, int& n0, int& by, int& expert, int& row0, int& nrows) {
    const int nx = tile % tiles_n, byr = tile / tiles_n;
    n0 = nx * BM;
    by = (!GROUPED && p.y_rot) ? (byr + p.y_rot) % tiles_y : byr;
    expert = 0;
    if (GROUPED) {
      const int4 t = p.tiles[by];
      expert = t.x; row0 = t.y; nrows = t.z;
    } else {
      row0 = by * BT;
      nrows = min(BT, p.T - row0);
    }
  };

  if (warp == 0 && GROUPED && BT <= GATHER_BT_MAX && p.gather_rows != nullptr) {
    // ---------------- gathering producer (all 32 lanes): weights by TMA from lane 0, activation rows by index.
    // Chunk q = lane + 32 i of a k-block is bytes [16 (q & 7), +16) of tile row q >> 3; it lands where the 128-byte
    // swizzle of the K-major operand layout puts it: row r at (r >> 3) * 1024 + (r & 7) * 128, chunk j at
    // ((j ^ (r & 7)) * 16). Rows beyond the tile's row count are left as they are: an MMA column depends on its own
    // row only, and the epilogue never stores those columns.
    constexpr int PER_LANE = BT / 4 > 0 ? BT / 4 : 1;
    int it = 0;
    bool live = true;
    const int j = lane & 7;
    for (int tile = tile0; tile < total && live; tile += tstep) {
      int n0, by, expert, row0, nrows;
      tile_geom(tile, n0, by, expert, row0, nrows);
      const bf16* src[PER_LANE];
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int r = (lane >> 3) + 4 * i;
        const int g = r < nrows ? p.gather_rows[row0 + r] : -1;
        src[i] = g >= 0 ? p.gx + static_cast<size_t>(g) * p.ldgx + j * 8 : nullptr;
      }
      for (int kb = 0; kb < num_k; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY, abort_flag)) { live = false; break; }
        uint8_t* st = smem + s * C::STAGE_BYTES;
        if (lane == 0) {
          mbar_expect_tx(&full[s], C::A_TILES * C::A_BYTES);
          if (p.packed) {
            tma_load_2d(st, &tmW, &full[s], 0,
                        ((expert * p.w_tiles + n0 / BM) * num_k_all + kb0 + kb) * (BM * C::A_TILES));
          } else {
            tma_load_3d(st, &tmW, &full[s], (kb0 + kb) * BK, n0, expert);
            if (EPI == EPI_SILU_MUL) tma_load_3d(st + C::A_BYTES, &tmW, &full[s], (kb0 + kb) * BK, p.up_offset + n0, expert);
          }
        }
        const uint32_t xb = smem_u32(st + C::A_TILES * C::A_BYTES);
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
          const int r = (lane >> 3) + 4 * i;
          if (src[i] != nullptr) {
            const uint32_t dst = xb + (r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src[i] + (kb0 + kb) * BK) : "memory");
          }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[s])) : "memory");
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // no copy of this lane may outlive the CTA's shared memory
  } else if (warp == 0) {
    if (elect_one()) {
      int it = 0;  // k-blocks issued so far, over all tiles of this CTA
      bool live = true;
      // Dense weights are written by nobody in the stream: fill the first stages of this CTA's first tile with weight
      // tiles before waiting for the previous kernel (whose output is X), so that their latency hides behind its tail.
      int pre = 0;
      if (!GROUPED && !SPLIT && tile0 < total) {
        int n0, by, expert, row0, nrows;
        tile_geom(tile0, n0, by, expert, row0, nrows);
        pre = num_k < C::STAGES ? num_k : C::STAGES;
        for (int kb = 0; kb < pre; ++kb) {
          uint8_t* st = smem + kb * C::STAGE_BYTES;
          mbar_expect_tx(&full[kb], C::STAGE_BYTES);
          if (p.packed) {
            tma_load_2d(st, &tmW, &full[kb], 0, ((n0 / BM) * num_k_all + kb) * (BM * C::A_TILES));
          } else {
            tma_load_2d(st, &tmW, &full[kb], kb * BK, n0);
            if (EPI == EPI_SILU_MUL) tma_load_2d(st + C::A_BYTES, &tmW, &full[kb], kb * BK, p.up_offset + n0);
          }
        }
      }
      pdl_wait();
      pdl_launch();
      for (int tile = tile0; tile < total && live; tile += tstep) {
      int n0, by, expert, row0, nrows;
      tile_geom(tile, n0, by, expert, row0, nrows);
      // all-gather -> GEMM: the activation rows of this tile were pushed here by their owner rank; wait for that
      // shard only, so tiles of shards that have already arrived run while the others are still in flight
      if (p.x_flags != nullptr && !wait_flag(p.x_flags + row0 / p.rows_per_rank, *p.x_epoch, p.err)) *abort_flag = 1;
      for (int kb = 0; kb < num_k; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        if (it >= pre) {
        if (!mbar_wait(&empty[s], ph ^ 1, p.err, ERR_WAIT_EMPTY, abort_flag)) { live = false; break; }
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        if (p.packed) {
          tma_load_2d(st, &tmW, &full[s], 0,
                      ((expert * p.w_tiles + n0 / BM) * num_k_all + kb0 + kb) * (BM * C::A_TILES));
        } else if (GROUPED) {
          tma_load_3d(st, &tmW, &full[s], (kb0 + kb) * BK, n0, expert);
          if (EPI == EPI_SILU_MUL) tma_load_3d(st + C::A_BYTES, &tmW, &full[s], (kb0 + kb) * BK, p.up_offset + n0, expert);
        } else {
          tma_load_2d(st, &tmW, &full[s], (kb0 + kb) * BK, n0);
          if (EPI == EPI_SILU_MUL) tma_load_2d(st + C::A_BYTES, &tmW, &full[s], (kb0 + kb) * BK, p.up_offset + n0);
        }
        }
        tma_load_2d(st + C::A_TILES * C::A_BYTES, &tmX, &full[s], (kb0 + kb) * BK, row0);
      }
      }
    }
    if (SPLIT) { __syncwarp(); cluster_sync(); }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BT);
      bool ok = true;
      int it = 0, lt = 0;  // k-blocks and tiles consumed so far
      for (int tile = tile0; tile < total && ok; tile += tstep, ++lt) {
      const int acc = lt % ACC;
      const uint32_t tmem = tmem_base + acc * C::ACC_COLS;
      // the epilogue must have drained this accumulator stage (two tiles ago) before it is overwritten
      ok = mbar_wait(&acc_empty[acc], ((lt / ACC) & 1) ^ 1, p.err, ERR_WAIT_TMEM, abort_flag);
      if (ok) tc_fence_after();
      for (int kb = 0; kb < num_k && ok; ++kb, ++it) {
        const int s = it % C::STAGES;
        const uint32_t ph = (it / C::STAGES) & 1;
        ok = mbar_wait(&full[s], ph, p.err, ERR_WAIT_FULL, abort_flag);
        if (!ok) break;
        // rows that the gathering producer wrote through the generic proxy must be visible to the tensor core's reads
        if (GROUPED && BT <= GATHER_BT_MAX && p.gather_rows != nullptr) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
        const uint32_t b_addr = a_addr + C::A_TILES * C::A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t koff = k * UMMA_K * 2;  // bytes inside the 128-byte swizzled row
          const uint64_t db = umma_smem_desc(b_addr + koff);
          umma_bf16(tmem, umma_smem_desc(a_addr + koff), db, idesc, (kb | k) != 0);
          if (EPI == EPI_SILU_MUL)
            umma_bf16(tmem + BT, umma_smem_desc(a_addr + C::A_BYTES + koff), db, idesc, (kb | k) != 0);
        }
        umma_commit(&empty[s]);  // stage reusable once these MMAs have read it
      }
      umma_commit(&acc_full[acc]);  // always arrive so that the epilogue is released
      }
    }
    if (SPLIT) { __syncwarp(); cluster_sync(); }
  } else {
    // ---------------- epilogue: warp q owns TMEM lanes [32q, 32q+32)
    pdl_wait();  // first global write of the CTA comes from here
    const int q = warp & 3;
    int lt = 0;
    for (int tile = tile0; tile < total; tile += tstep, ++lt) {
    int n0, by, expert, row0, nrows;
    tile_geom(tile, n0, by, expert, row0, nrows);
    (void)expert;
    const int nx = n0 / BM;
    const int acc = lt % ACC;
    const uint32_t tmem = tmem_base + acc * C::ACC_COLS;
    const bool ok = mbar_wait(&acc_full[acc], (lt / ACC) & 1, p.err, ERR_WAIT_TMEM, abort_flag) && !*abort_flag;
    tc_fence_after();
    const int n = n0 + q * 32 + lane;
    const bool n_ok = n < p.N;
    if (EPI == EPI_ALLREDUCE) {
      // Fused GEMM -> one-shot all-reduce: this tile's fp32 partial goes straight from TMEM into every
      // rank's receive slot over NVLink; when all R partials of the tile have arrived they are added in
      // rank order (+ residual) and stored as bf16. No partial ever touches this rank's output buffer.
      const CommCtx& cc = p.comm;
      const int blk = by * tiles_n + nx;
      __shared__ uint32_t s_epoch;
      __shared__ int s_peer_ok;
      const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
      if (et == 0) { s_epoch = cc.epoch[blk] + 1; cc.epoch[blk] = s_epoch; s_peer_ok = 1; }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t e = s_epoch;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < nrows; c += 16) {
          float v[16];
          tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c, v);  // warp-collective: never predicated
          if (n_ok) {
            for (int r = 0; r < cc.world; ++r) {
              float* dst = comm_slot(cc, r, e, cc.rank);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (c + j < nrows) dst[static_cast<size_t>(row0 + c + j) * p.ldo + n] = v[j];
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et < cc.world) {
        __threadfence_system();
        st_release_sys(cc.flags[et] + static_cast<size_t>(cc.rank) * cc.max_blocks + blk, e);
        if (!wait_flag(cc.flags[cc.rank] + static_cast<size_t>(et) * cc.max_blocks + blk, e, cc.err)) s_peer_ok = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok && n_ok && s_peer_ok) {
        for (int t = 0; t < nrows; ++t) {
          const size_t o = static_cast<size_t>(row0 + t) * p.ldo + n;
          float acc = comm_slot(cc, cc.rank, e, 0)[o];
          for (int r = 1; r < cc.world; ++r) acc += comm_slot(cc, cc.rank, e, r)[o];
          if (p.residual) acc = __bfloat162float(__float2bfloat16(acc)) + __bfloat162float(p.residual[o]);
          reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(acc);
        }
      }
    } else if (EPI == EPI_REDUCE_SCATTER) {
      // Fused GEMM -> reduce-scatter: the tile's token rows belong to one owner rank. Every rank stores its fp32
      // partial straight from TMEM into the owner's receive slot (a peer store over NVLink unless it is the
      // owner) and releases the tile's arrival flag there. Nothing waits here: the owner adds the R partials in
      // rank order inside the following norm kernel (allreduce.cu, reduce_norm_allgather_kernel), at full occupancy.
      const CommCtx& cc = p.comm;
      const int blk = by * tiles_n + nx;
      const int owner = row0 / p.rows_per_rank;
      const int lrow0 = row0 - owner * p.rows_per_rank;
      __shared__ uint32_t s_epoch_rs;
      const int et = threadIdx.x - 64;
      if (et == 0) { s_epoch_rs = cc.epoch[blk] + 1; cc.epoch[blk] = s_epoch_rs; }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t e = s_epoch_rs;
      if (ok) {
        float* dst = comm_slot(cc, owner, e, cc.rank);
#pragma unroll 1
        for (int c = 0; c < nrows; c += 16) {
          float v[16];
          tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c, v);  // warp-collective: never predicated
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < nrows) dst[static_cast<size_t>(lrow0 + c + j) * p.ldo + n] = v[j];
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) {
        __threadfence_system();
        st_release_sys(cc.flags[owner] + static_cast<size_t>(cc.rank) * cc.max_blocks + blk, e);
      }
    } else
    if (SPLIT && blockIdx.z != 0) {
      // split-K follower: park the partial tile in shared memory (the pipeline stages are idle now) as
      // red[column][weight row]; a CTA without k-blocks contributes zeros
      float* red = reinterpret_cast<float*>(smem);
#pragma unroll 1
      for (int c = 0; c < nrows; c += 16) {
        float v[16];
        if (num_k > 0 && ok) tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c, v);
        else { for (int j = 0; j < 16; ++j) v[j] = 0.f; }
#pragma unroll
        for (int j = 0; j < 16; ++j) red[(c + j) * BM + q * 32 + lane] = v[j];
        if (EPI == EPI_SILU_MUL) {
          if (num_k > 0 && ok) tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + BT + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) red[(BT + c + j) * BM + q * 32 + lane] = v[j];
        }
      }
      cluster_sync();  // first cluster barrier (every thread of the cluster takes part exactly once)
    } else {
    if (SPLIT) cluster_sync();  // first cluster barrier: the followers' partial tiles are in place
    if (ok) {
      const uint32_t red_local = smem_u32(smem);
#pragma unroll 1
      for (int c = 0; c < BT; c += 16) {
        if (c >= nrows && EPI != EPI_ARGMAX) break;  // warp-uniform
        float v[16];
        tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + c, v);
        if (SPLIT) {
          for (int r = 1; r < p.splits; ++r) {
            const uint32_t remote = dsmem_addr(red_local, r);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += ld_dsmem_f32(remote + ((c + j) * BM + q * 32 + lane) * 4);
          }
        }
        if (EPI == EPI_SILU_MUL) {
          float u[16];
          tmem_ld16(tmem + (static_cast<uint32_t>(q * 32) << 16) + BT + c, u);
          if (SPLIT) {
            for (int r = 1; r < p.splits; ++r) {
              const uint32_t remote = dsmem_addr(red_local, r);
#pragma unroll
              for (int j = 0; j < 16; ++j) u[j] += ld_dsmem_f32(remote + ((BT + c + j) * BM + q * 32 + lane) * 4);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // round gate and up to bf16 first, as the unfused sequence of ops does
            const float g = __bfloat162float(__float2bfloat16(v[j]));
            const float uu = __bfloat162float(__float2bfloat16(u[j]));
            v[j] = __bfloat162float(__float2bfloat16(silu_f(g))) * uu;
          }
        }
        if (EPI == EPI_ARGMAX) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float m = n_ok ? v[j] : -INFINITY;
            int idx = n;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
              const float om = __shfl_xor_sync(0xffffffffu, m, o);
              const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
              if (om > m || (om == m && oi < idx)) { m = om; idx = oi; }
            }
            if (lane == 0) { red_max[q][c + j] = m; red_idx[q][c + j] = idx; }
          }
        } else if (EPI == EPI_SCATTER) {
          // expert-parallel combine: each output row goes straight to the rank that owns the token,
          // into the slot of its (token, pair) - a peer store over NVLink when that rank is not this one
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < nrows) {
                const int2 m = p.meta[row0 + c + j];
                p.pair_out[m.x][static_cast<size_t>(m.y) * p.ldo + n] = __float2bfloat16(v[j]);
              }
            }
          }
        } else if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c + j < nrows) {
              const size_t o = static_cast<size_t>(row0 + c + j) * p.ldo + n;
              if (EPI == EPI_F32) reinterpret_cast<float*>(p.out)[o] = v[j];
              else reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(v[j]);
            }
          }
        }
      }
    }
    }
    if (EPI == EPI_ARGMAX) {
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
      const int t = (warp - 2) * 32 + lane;
      for (int c = t; c < BT; c += 128) {
        if (c < nrows && ok) {
          float m = red_max[0][c]; int idx = red_idx[0][c];
#pragma unroll
          for (int w = 1; w < 4; ++w) {
            const float om = red_max[w][c]; const int oi = red_idx[w][c];
            if (om > m || (om == m && oi < idx)) { m = om; idx = oi; }
          }
          const size_t o = static_cast<size_t>(nx) * p.T + row0 + c;
          p.part_max[o] = m; p.part_idx[o] = idx;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // red_max / red_idx are reused by the next tile
    }
    // this accumulator stage may be overwritten: every tcgen05.ld of the warp has completed (wait::ld)
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&acc_empty[acc]);
    if (!ok) break;
    }
  }
  if (SPLIT) cluster_sync();  // second cluster barrier: the leader has read every partial tile
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, C::TMEM_COLS); }
}

// Reduce the LM-head partials of each row over the vocabulary tiles, first maximum wins.
__global__ void argmax_finish_kernel(const float* part_max, const int* part_idx, int n_tiles, int T, int64_t* out,
                                     float* out_val) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  float m = -INFINITY; int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
    const float om = part_max[static_cast<size_t>(i) * T + t]; const int oi = part_idx[static_cast<size_t>(i) * T + t];
    if (om > m || (om == m && oi < idx)) { m = om; idx = oi; }
  }
  __shared__ float sm[32]; __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o); const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (om > m || (om == m && oi < idx)) { m = om; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; si[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w)
      if (sm[w] > m || (sm[w] == m && si[w] < idx)) { m = sm[w]; idx = si[w]; }
    out[t] = idx;
    if (out_val) out_val[t] = m;
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

// bf16 tensor [d2, d1, d0] (d0 contiguous), box {BK, box1, 1}, 128-byte swizzle, zero fill.
static int make_map(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2,
                    uint32_t box1) {
  EncodeFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1 * 2, ld2 * 2};
  cuuint32_t box[3] = {BK, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const int rank = d2 > 0 ? 3 : 2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Tile-packed weights: a 2-D view [tiles * box_rows, 64] whose boxes of `box_rows` rows are contiguous runs.
static int make_map_packed(CUtensorMap* m, const void* base, uint64_t total_rows, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {BK, total_rows};
  cuuint64_t strides[1] = {BK * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -2;
}

// Weight map of a launch: `packed` selects the tile-packed layout (N padded to a multiple of 128 per expert, K a
// multiple of 64; with the SiLU-mul epilogue the gate and up tiles of a k-block are stored back to back).
static int weight_map(CUtensorMap* m, const void* W, int E, int N, int w_rows, int K, int ldw, bool silu, int packed,
                      GemmParams* p) {
  if (!packed) return E > 0 ? make_map(m, W, K, w_rows, E, K, static_cast<uint64_t>(w_rows) * K, BM)
                            : make_map(m, W, K, w_rows, 0, ldw, 0, BM);
  if (K % BK) return -7;
  const uint64_t tiles = (N + BM - 1) / BM, nk = K / BK, a = silu ? 2 : 1;
  p->packed = 1;
  p->w_tiles = static_cast<int>(tiles);
  return make_map_packed(m, W, static_cast<uint64_t>(E > 0 ? E : 1) * tiles * nk * BM * a, static_cast<uint32_t>(BM * a));
}

template <int BT, int EPI, bool GROUPED>
static int launch_split(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int grid_y, cudaStream_t st) {
  using C = Cfg<BT, EPI>;
  auto kern = gemm_swapab_kernel<BT, EPI, GROUPED, true>;
  static bool configured[MAX_DEVICES] = {};  // a function attribute is set per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -3;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess) return -3;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + BM - 1) / BM, grid_y, p.splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GemmParams q = p;
  q.grid_y = grid_y;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, q) == cudaSuccess ? 0 : -4;
}

template <int BT, int EPI, bool GROUPED>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int grid_y, cudaStream_t st) {
  using C = Cfg<BT, EPI>;
  if constexpr (EPI == EPI_BF16 || EPI == EPI_F32 || EPI == EPI_SILU_MUL) {
    if (p.splits > 1) return launch_split<BT, EPI, GROUPED>(tw, tx, p, grid_y, st);
  }
  auto kern = gemm_swapab_kernel<BT, EPI, GROUPED, false>;
  // per device: the shared-memory attribute is set on the device that is current, and the persistent grid is sized
  // from that device's SM count (a process may drive several GPUs)
  static bool configured[MAX_DEVICES] = {};
  static int resident_of[MAX_DEVICES] = {};  // CTAs the device holds at once: the persistent grid is never larger
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -3;
  if (!configured[dev]) {
    int sms = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess) return -3;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -3;
    resident_of[dev] = sms * C::CTAS_PER_SM;
    configured[dev] = true;
  }
  const int resident = resident_of[dev];
  GemmParams q = p;
  q.grid_y = grid_y;
  const long long tiles = static_cast<long long>((p.N + BM - 1) / BM) * grid_y;
  return launch_pdl(kern, dim3(static_cast<unsigned>(tiles < resident ? tiles : resident)), dim3(192), C::SMEM, st, tw,
                    tx, q) == cudaSuccess ? 0 : -4;
}

template <int EPI, bool GROUPED>
static int dispatch_bt(int bt, const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int grid_y, cudaStream_t st) {
  switch (bt) {
    case 16: return launch<16, EPI, GROUPED>(tw, tx, p, grid_y, st);
    case 32: return launch<32, EPI, GROUPED>(tw, tx, p, grid_y, st);
    case 64: return launch<64, EPI, GROUPED>(tw, tx, p, grid_y, st);
    case 128: return launch<128, EPI, GROUPED>(tw, tx, p, grid_y, st);
    case 256:
      if (EPI != EPI_SILU_MUL) return launch<(EPI != EPI_SILU_MUL ? 256 : 128), EPI, GROUPED>(tw, tx, p, grid_y, st);
      return -5;  // the gate/up epilogue has no 256-row form
    default: return -5;
  }
}

}  // namespace b200

using namespace b200;

// Token-tile width for a dense GEMM over T rows: a function of T only through the tile
// count, never through the per-element arithmetic.
extern "C" int b200_pick_bt(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  return 256;
}

// Dense: out[T, N] = X[T, K] W[N, K]^T.   epi: 0 bf16, 1 fp32, 2 silu(gate)*up (N = rows of each half, W has 2N rows
// with the up half at row `up_offset`), 3 argmax partials (part_max/part_idx sized [ceil(N/128), T]).
extern "C" int b200_gemm_dense(const void* X, const void* W, void* out, int T, int N, int K, int ldx, int ldw, int ldo,
                               int epi, int up_offset, int bt, float* part_max, int* part_idx, int* err,
                               int splits, int packed, cudaStream_t st) {
  if (T <= 0) return 0;
  if (splits < 1 || splits > 8 || splits > (K + BK - 1) / BK) splits = 1;
  if (bt <= 0) bt = b200_pick_bt(T);
  if (epi == EPI_SILU_MUL && bt > 128) bt = 128;
  CUtensorMap tw, tx;
  const int w_rows = (epi == EPI_SILU_MUL) ? up_offset + N : N;
  GemmParams p{N, K, T, ldo, out, nullptr, nullptr, up_offset, part_max, part_idx, err, nullptr, CommCtx{}, 0, nullptr, nullptr, splits, nullptr, {}};
  if (weight_map(&tw, W, 0, N, w_rows, K, ldw, epi == EPI_SILU_MUL, packed, &p)) return -1;
  if (make_map(&tx, X, K, T, 0, ldx, 0, bt)) return -1;
  const int gy = (T + bt - 1) / bt;
  switch (epi) {
    case EPI_BF16: return dispatch_bt<EPI_BF16, false>(bt, tw, tx, p, gy, st);
    case EPI_F32: return dispatch_bt<EPI_F32, false>(bt, tw, tx, p, gy, st);
    case EPI_SILU_MUL: return dispatch_bt<EPI_SILU_MUL, false>(bt, tw, tx, p, gy, st);
    case EPI_ARGMAX: return dispatch_bt<EPI_ARGMAX, false>(bt, tw, tx, p, gy, st);
  }
  return -6;
}

// Grouped: X is the expert-sorted activation buffer [cap, K]; tile i covers rows
// [tiles[i].y, +tiles[i].z) of expert tiles[i].x; W is [E, rows, K]. `max_tiles` bounds the grid.
extern "C" int b200_gemm_grouped(const void* X, const void* W, void* out, int cap, int E, int N, int w_rows, int K,
                                 int ldo, int epi, int up_offset, int bt, const void* tiles, const int* n_tiles,
                                 int max_tiles, int* err, int splits, int packed, const int* gather_rows, int ldx,
                                 cudaStream_t st) {
  // gather_rows != null (token tiles of at most 64 rows): X is [any rows, ldx] and sorted position i reads row
  // gather_rows[i] of it; otherwise X is the expert-sorted buffer [cap, K] itself.
  if (max_tiles <= 0) return 0;
  if (gather_rows != nullptr && (bt > GATHER_BT_MAX || splits > 1 || ldx % 8)) return -7;
  if (splits < 1 || splits > 8 || splits > (K + BK - 1) / BK) splits = 1;
  CUtensorMap tw, tx;
  GemmParams p{N, K, cap, ldo, out, reinterpret_cast<const int4*>(tiles), n_tiles, up_offset, nullptr, nullptr, err, nullptr, CommCtx{}, 0, nullptr, nullptr, splits, nullptr, {}};
  if (weight_map(&tw, W, E, N, w_rows, K, K, epi == EPI_SILU_MUL, packed, &p)) return -1;
  if (gather_rows != nullptr) {
    p.gather_rows = gather_rows;
    p.gx = static_cast<const bf16*>(X);
    p.ldgx = ldx;
    if (make_map(&tx, X, K, bt, 0, ldx, 0, bt)) return -1;  // unused by the gathering producer, but a valid map
  } else if (make_map(&tx, X, K, cap, 0, K, 0, bt)) return -1;
  switch (epi) {
    case EPI_BF16: return dispatch_bt<EPI_BF16, true>(bt, tw, tx, p, max_tiles, st);
    case EPI_SILU_MUL: return dispatch_bt<EPI_SILU_MUL, true>(bt, tw, tx, p, max_tiles, st);
  }
  return -6;
}

// Tensor-parallel output projection: out[T, N] = bf16(residual + sum over ranks of X_r[T, K_r] W_r[N, K_r]^T).
// Every rank calls this with its K-shard; the all-reduce happens inside the GEMM epilogue over peer memory.
// Needs T * N <= ctx->slot_elems and ceil(N/128) * ceil(T/bt) <= ctx->max_blocks.
extern "C" int b200_gemm_allreduce(const CommCtx* ctx, const void* X, const void* W, const void* residual, void* out,
                                   int T, int N, int K, int ldx, int ldw, int bt, cudaStream_t st) {
  if (T <= 0) return 0;
  if (bt <= 0) bt = b200_pick_bt(T);
  const int gy = (T + bt - 1) / bt;
  if (static_cast<unsigned long long>(T) * N > ctx->slot_elems || ((N + BM - 1) / BM) * gy > ctx->max_blocks) return -7;
  CUtensorMap tw, tx;
  if (make_map(&tw, W, K, N, 0, ldw, 0, BM)) return -1;
  if (make_map(&tx, X, K, T, 0, ldx, 0, bt)) return -1;
  GemmParams p{N, K, T, N, out, nullptr, nullptr, 0, nullptr, nullptr, ctx->err, static_cast<const bf16*>(residual), *ctx, 0, nullptr, nullptr, 1, nullptr, {}};
  return dispatch_bt<EPI_ALLREDUCE, false>(bt, tw, tx, p, gy, st);
}

// Expert-parallel down projection: grouped GEMM whose epilogue scatters every output row to the owner of its
// token (`meta[row] = (rank, pair slot)`, `pair_out[rank]` = that rank's [pairs, N] buffer as mapped in this process).
extern "C" int b200_gemm_grouped_scatter(const void* X, const void* W, int cap, int E, int N, int K, int bt,
                                         const void* tiles, const int* n_tiles, int max_tiles, const void* meta,
                                         void* const* pair_out, int world, int* err, int packed, cudaStream_t st) {
  if (max_tiles <= 0) return 0;
  CUtensorMap tw, tx;
  GemmParams p{N, K, cap, N, nullptr, reinterpret_cast<const int4*>(tiles), n_tiles, 0, nullptr, nullptr, err, nullptr,
               CommCtx{}, 0, nullptr, nullptr, 1, static_cast<const int2*>(meta), {}};
  if (weight_map(&tw, W, E, N, N, K, K, false, packed, &p)) return -1;
  if (make_map(&tx, X, K, cap, 0, K, 0, bt)) return -1;
  for (int r = 0; r < world && r < MAX_RANKS; ++r) p.pair_out[r] = static_cast<bf16*>(pair_out[r]);
  return dispatch_bt<EPI_SCATTER, true>(bt, tw, tx, p, max_tiles, st);
}

// Tensor-parallel output projection with a reduce-scatter epilogue: every rank calls it with its K-shard of X and
// W [N, K]; afterwards the fp32 partials of rank r's rows [r * T / R, (r + 1) * T / R) sit in rank r's receive
// slots, one per source rank, with one arrival flag per (source, tile). b200_reduce_norm_allgather consumes them.
// T must be a multiple of world * bt. Needs (T / R) * N <= ctx->slot_elems and the tile count <= ctx->max_blocks.
extern "C" int b200_gemm_reduce_scatter(const CommCtx* ctx, const void* X, const void* W, int T, int N, int K, int ldx,
                                        int ldw, int bt, cudaStream_t st) {
  if (T <= 0) return 0;
  if (bt <= 0) bt = b200_pick_bt(T / ctx->world);
  if (T % (ctx->world * bt)) return -7;
  const int rpr = T / ctx->world, gy = T / bt;
  if (static_cast<unsigned long long>(rpr) * N > ctx->slot_elems || ((N + BM - 1) / BM) * gy > ctx->max_blocks) return -7;
  CUtensorMap tw, tx;
  if (make_map(&tw, W, K, N, 0, ldw, 0, BM)) return -1;
  if (make_map(&tx, X, K, T, 0, ldx, 0, bt)) return -1;
  GemmParams p{N, K, T, N, nullptr, nullptr, nullptr, 0, nullptr, nullptr, ctx->err, nullptr, *ctx,
               rpr, nullptr, nullptr, 1, nullptr, {}};
  // each rank runs the tiles of the next rank first and its own last: partials reach their owners early, and an
  // owner's waits fall at the end of its grid, on tiles every peer has already pushed
  p.y_rot = ((ctx->rank + 1) % ctx->world) * (rpr / bt);
  return dispatch_bt<EPI_REDUCE_SCATTER, false>(bt, tw, tx, p, gy, st);
}

// All-gather -> GEMM: X [T, K] is this rank's full activation buffer into which every owner rank pushes its row
// shard (allreduce.cu: norm_allgather); a tile starts as soon as its owner's shard has arrived (x_flags[owner] >=
// *x_epoch). out[T, N] = X W^T, bf16 or fp32. `y_rot` = rank * (rows_per_rank / bt) makes each rank start with its
// own shard, which is already there.
extern "C" int b200_gemm_gathered(const void* X, const void* W, void* out, int T, int N, int K, int ldx, int ldw,
                                  int out_f32, int bt, int rows_per_rank, int y_rot, const uint32_t* x_flags,
                                  const uint32_t* x_epoch, int* err, cudaStream_t st) {
  if (T <= 0) return 0;
  if (bt <= 0) bt = b200_pick_bt(rows_per_rank);
  if (rows_per_rank % bt) return -7;
  CUtensorMap tw, tx;
  if (make_map(&tw, W, K, N, 0, ldw, 0, BM)) return -1;
  if (make_map(&tx, X, K, T, 0, ldx, 0, bt)) return -1;
  GemmParams p{N, K, T, N, out, nullptr, nullptr, 0, nullptr, nullptr, err, nullptr, CommCtx{}, rows_per_rank, x_flags,
               x_epoch, 1, nullptr, {}};
  p.y_rot = y_rot;
  const int gy = (T + bt - 1) / bt;
  return out_f32 ? dispatch_bt<EPI_F32, false>(bt, tw, tx, p, gy, st) : dispatch_bt<EPI_BF16, false>(bt, tw, tx, p, gy, st);
}

extern "C" int b200_argmax_finish(const float* part_max, const int* part_idx, int n_tiles, int T, int64_t* out,
                                  float* out_val, cudaStream_t st) {
  if (T <= 0) return 0;
  return launch_pdl(argmax_finish_kernel, dim3(T), dim3(256), 0, st, part_max, part_idx, n_tiles, T, out, out_val) ==
                 cudaSuccess ? 0 : -4;
}

// ------------------------------------------------------------------ allocation-free greedy head
// See b200serve_noalloc.h. The per-tile (max, index) partials of the LM-head argmax live in a
// fixed device array instead of caller-provided workspace.
#include <stdio.h>

#include "b200serve_noalloc.h"

namespace {
constexpr size_t NOALLOC_PART_ELEMS = static_cast<size_t>(B200_NOALLOC_MAX_ROWS) * B200_NOALLOC_MAX_TILES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_PART_ELEMS * (sizeof(float) + sizeof(int))];
constexpr int NOALLOC_MAX_DEVICES = MAX_DEVICES;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" int b200_lm_head_argmax_noalloc(const void* X, const void* W, int64_t* out_idx, float* out_val, int T, int V,
                                           int K, int ldx, int ldw, int* err, cudaStream_t st) {
  if (T <= 0) return 0;
  const int n_tiles = (V + BM - 1) / BM;
  if (T > B200_NOALLOC_MAX_ROWS || n_tiles > B200_NOALLOC_MAX_TILES) {
    fprintf(stderr,
            "b200_lm_head_argmax_noalloc: %d rows x %d vocabulary entries exceed the built-in scratch "
            "(at most %d rows and %d entries)\n",
            T, V, B200_NOALLOC_MAX_ROWS, B200_NOALLOC_MAX_TILES * BM);
    return B200_NOALLOC_TOO_LARGE;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return B200_NOALLOC_BAD_DEVICE;
  if (g_noalloc_ptr[dev] == nullptr) {
    // The array's name is only a host-side handle; the device address of this device's copy has to be
    // asked for, once, with the device current. Not a stream operation: do the first call outside capture.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return B200_NOALLOC_NO_SYMBOL;
    g_noalloc_ptr[dev] = p;
  }
  float* part_max = static_cast<float*>(g_noalloc_ptr[dev]);
  int* part_idx = reinterpret_cast<int*>(part_max + NOALLOC_PART_ELEMS);
  const int bt = b200_pick_bt(T);
  CUtensorMap tw, tx;
  if (make_map(&tw, W, K, V, 0, ldw, 0, BM)) return -1;
  if (make_map(&tx, X, K, T, 0, ldx, 0, bt)) return -1;
  GemmParams p{V, K, T, 0, nullptr, nullptr, nullptr, 0, part_max, part_idx, err, nullptr, CommCtx{}, 0, nullptr, nullptr, 1, nullptr, {}};
  const int rc = dispatch_bt<EPI_ARGMAX, false>(bt, tw, tx, p, (T + bt - 1) / bt, st);
  if (rc) return rc;
  argmax_finish_kernel<<<T, 256, 0, st>>>(part_max, part_idx, n_tiles, T, out_idx, out_val);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
