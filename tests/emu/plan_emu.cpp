// Runs the expert-plan kernels of the MoE block (ops/cuda/moe_plan.cuh: 1024-thread CTAs with a shared-memory
// histogram, two-level scans over warp shuffles, a scatter through per-expert cursors, and the "last CTA builds the
// plan" ticket), compiled as host C++ through emu_shim.h, against a plain restatement of what a plan must satisfy.
// Under -fsanitize=thread every barrier these kernels rely on is checked. Exit code 0 and a line "OK ..." on success.
//   g++ -std=c++20 -O1 -pthread -DB200_EMU -I tests/emu -x c++ tests/emu/plan_emu.cpp -o plan_emu
#include "emu_shim.h"

#include "../../qwen36-mi250-tracelab-20261107_b200/ops/cuda/moe_plan.cuh"

#include <cstdio>
#include <random>

using namespace b200;

struct Plan {
  std::vector<int> offsets, perm, inv, src_rows;
  std::vector<int4> tiles;
  int n_tiles = -1, err = 0;
  Plan(int Et, int n_pairs, int max_tiles) : offsets(Et + 1, -1), perm(n_pairs, -1), inv(n_pairs, -2), src_rows(n_pairs, -1), tiles(max_tiles) {}
};

// What every form of the plan must produce from idx (values in [0, Et) are local experts, -1 = served elsewhere).
static int check(const char* what, const std::vector<int>& idx, int Et, int bt, int P, const Plan& p, int max_tiles, bool want_err) {
  int bad = 0;
  auto fail = [&](const char* msg, int a, int b) { std::printf("%s: %s (%d, %d)\n", what, msg, a, b); ++bad; };
  std::vector<int> count(Et, 0);
  for (int x : idx) if (x >= 0 && x < Et) ++count[x];
  int run = 0, tiles = 0;
  for (int e = 0; e < Et; ++e) {
    if (p.offsets[e] != run) fail("offset of expert", e, p.offsets[e]);
    for (int i = 0; i * bt < count[e]; ++i, ++tiles) {
      if (tiles >= max_tiles) break;
      const int4 t = p.tiles[tiles];
      if (t.x != e || t.y != run + i * bt || t.z != std::min(bt, count[e] - i * bt)) fail("tile", tiles, t.x);
    }
    run += count[e];
  }
  if (p.offsets[Et] != run) fail("total rows", run, p.offsets[Et]);
  if (p.n_tiles != std::min(tiles, max_tiles)) fail("tile count", tiles, p.n_tiles);
  std::vector<char> taken(idx.size(), 0);
  for (size_t i = 0; i < idx.size(); ++i) {
    const int x = idx[i];
    if (x < 0 || x >= Et) { if (p.inv[i] != -1) fail("pair of no local expert must have inv -1", static_cast<int>(i), p.inv[i]); continue; }
    const int pos = p.inv[i];
    if (pos < p.offsets[x] || pos >= p.offsets[x] + count[x]) { fail("position outside its expert's run", static_cast<int>(i), pos); continue; }
    if (taken[pos]++) fail("position handed out twice", pos, 0);
    if (p.perm[pos] != static_cast<int>(i)) fail("perm is not the inverse of inv", pos, p.perm[pos]);
    if (p.src_rows[pos] != static_cast<int>(i) / P) fail("source row", pos, p.src_rows[pos]);
  }
  if ((p.err != 0) != want_err) fail("error word", p.err, want_err);
  return bad;
}

int main() {
  constexpr int E = 256, K = 8, P = K + 1, Et = E + 1, PER_LANE = 8;
  std::mt19937 rng(5);
  std::normal_distribution<float> nd(0.f, 1.f);
  int bad = 0;

  // 1. plan of a given index table by one CTA, more pairs than threads, some pairs served elsewhere, one bad index
  {
    const int n_pairs = 3000, bt = 16, max_tiles = 600;
    std::vector<int> idx(n_pairs);
    for (auto& x : idx) x = static_cast<int>(rng() % (Et + 40)) - 40;  // about an eighth are -1..-40 -> clamp to -1
    for (auto& x : idx) if (x < 0) x = -1;
    for (int pass = 0; pass < 2; ++pass) {
      if (pass == 1) idx[1234] = Et + 3;  // out of range: reported in the error word, treated as not local
      Plan p(Et, n_pairs, max_tiles);
      run_cta(1024, 0, 0, [&] {
        moe_plan_kernel(idx.data(), n_pairs, Et, bt, p.offsets.data(), p.tiles.data(), &p.n_tiles, max_tiles, p.perm.data(),
                        p.inv.data(), &p.err, P, p.src_rows.data());
      });
      bad += check(pass ? "plan (bad index)" : "plan", idx, Et, bt, P, p, max_tiles, pass == 1);
    }
  }

  // 2. routing + plan in one CTA (decode sizes), and 3. the grid forms whose last CTA builds the plan
  for (int T : {20, 100}) {
    std::vector<float> logits(T * (E + 1));
    for (auto& v : logits) v = nd(rng) * 2.f;
    const int bt = 16, n_pairs = T * P, max_tiles = std::min(Et, n_pairs) + n_pairs / bt + 1;
    std::vector<float> wts(n_pairs);
    std::vector<int> idx(n_pairs, -5);
    if (T <= 32) {
      Plan p(Et, n_pairs, max_tiles);
      run_cta(1024, 0, 0, [&] {
        moe_route_plan_kernel<PER_LANE>(logits.data(), E + 1, T, E, K, 1, wts.data(), idx.data(), nullptr, Et, bt, p.offsets.data(),
                                        p.tiles.data(), &p.n_tiles, max_tiles, p.perm.data(), p.inv.data(), &p.err, p.src_rows.data());
      });
      bad += check("route + plan, one CTA", idx, Et, bt, P, p, max_tiles, false);
    }
    for (int with_work = 0; with_work < 2; ++with_work) {
      std::vector<int> idx2(n_pairs, -5), work(2 * 1024, 0);
      unsigned ticket = 0;
      Plan p(Et, n_pairs, max_tiles);
      gridDim.x = (T + 31) / 32;
      for (unsigned bx = 0; bx < gridDim.x; ++bx)
        run_cta(1024, bx, 0, [&] {
          moe_route_plan_grid_kernel<PER_LANE>(logits.data(), E + 1, T, E, K, 1, wts.data(), idx2.data(), nullptr, Et, bt,
                                               p.offsets.data(), p.tiles.data(), &p.n_tiles, max_tiles, p.perm.data(), p.inv.data(),
                                               &p.err, p.src_rows.data(), &ticket, with_work ? work.data() : nullptr);
        });
      if (with_work) {  // the positions of the pairs come from a second, grid-wide launch
        gridDim.x = 3;
        for (unsigned bx = 0; bx < gridDim.x; ++bx)
          run_cta(256, bx, 0, [&] {
            moe_scatter_kernel(idx2.data(), n_pairs, Et, p.offsets.data(), work.data() + 1024, p.perm.data(), p.inv.data(), &p.err, P,
                               p.src_rows.data());
          });
      }
      bad += check(with_work ? "grid route + scan, then scatter" : "grid route, last CTA plans", idx2, Et, bt, P, p, max_tiles, false);
      if (ticket != 0) { std::printf("the ticket word was not put back to zero\n"); ++bad; }
      for (int e = 0; e < Et; ++e) if (work[e] != 0) { std::printf("count of expert %d was not put back to zero\n", e); ++bad; break; }
      if (T <= 32 && idx2 != idx) { std::printf("the grid form routed differently from the single CTA\n"); ++bad; }
    }
  }
  if (bad) return 1;
  std::printf("OK expert plan: single CTA, routing + plan, grid forms with and without the split scatter\n");
  return 0;
}
