// Runs the router's per-row body (ops/cuda/moe_route.cuh: softmax, iterative top-k with ties to the lower expert id,
// renormalised bf16 weights, shared-expert gate, local expert map and per-expert counts), compiled as host C++
// through emu_shim.h, one warp of 32 std::threads per row, against a float64 restatement. Exit code 0 and a line
// "OK ..." on success.
//   g++ -std=c++20 -O1 -pthread -DB200_EMU -I tests/emu -x c++ tests/emu/route_emu.cpp -o route_emu
#include "emu_shim.h"

#include "../../qwen36-mi250-tracelab-20261107_b200/ops/cuda/moe_route.cuh"

#include <algorithm>
#include <cstdio>
#include <numeric>
#include <random>

using namespace b200;

int main() {
  constexpr int E = 256, K = 8, PER_LANE = 8, ROWS = 6;
  std::mt19937 rng(11);
  std::normal_distribution<float> nd(0.f, 1.f);
  std::vector<float> logits(ROWS * (E + 1));
  for (auto& v : logits) v = nd(rng) * 2.f;
  for (int e = 0; e < E; ++e) logits[1 * (E + 1) + e] = 0.25f;                 // row 1: every expert tied
  for (int e = 0; e < E; ++e) logits[2 * (E + 1) + e] = (e % 50 == 49) ? 3.f : -1.f;  // row 2: 5 tied leaders, then ties
  for (int e = 0; e < E; ++e) logits[3 * (E + 1) + e] = static_cast<float>(e) * 0.01f;  // row 3: strictly increasing
  logits[4 * (E + 1) + 200] = 40.f;                                              // row 4: one dominant expert
  // local expert map of a rank that hosts the even experts and the shared one
  std::vector<int> map(E + 1);
  for (int e = 0; e < E; ++e) map[e] = e % 2 == 0 ? e / 2 : -1;
  map[E] = E / 2;

  int bad = 0;
  for (int use_map = 0; use_map < 2; ++use_map) {
    std::vector<float> wts(ROWS * (K + 1), -1.f);
    std::vector<int> idx(ROWS * (K + 1), -7), counts(E + 1, 0), want_counts(E + 1, 0);
    for (int r = 0; r < ROWS; ++r)
      run_cta(32, r, 0, [&] {
        route_row<PER_LANE>(logits.data() + r * (E + 1), E, K, 1, wts.data() + r * (K + 1), idx.data() + r * (K + 1),
                            use_map ? map.data() : nullptr, counts.data(), static_cast<int>(threadIdx.x));
      });
    for (int r = 0; r < ROWS; ++r) {
      const float* row = logits.data() + r * (E + 1);
      // float64 restatement: probabilities, order by (probability descending, id ascending), renormalise
      const double mx = *std::max_element(row, row + E);
      std::vector<double> pr(E);
      double sum = 0;
      for (int e = 0; e < E; ++e) sum += pr[e] = std::exp(static_cast<double>(row[e]) - mx);
      std::vector<int> order(E);
      std::iota(order.begin(), order.end(), 0);
      // the kernel compares float exponentials: equal floats are ties even where the doubles differ in the last bits
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
        const float fa = std::exp(row[a] - static_cast<float>(mx)), fb = std::exp(row[b] - static_cast<float>(mx));
        return fa > fb;
      });
      double tot = 0;
      for (int k = 0; k < K; ++k) tot += pr[order[k]] / sum;
      for (int k = 0; k < K; ++k) {
        const int e = order[k];
        const int want_idx = use_map ? map[e] : e;
        const double want_w = pr[e] / sum / tot;
        const float got_w = wts[r * (K + 1) + k];
        if (idx[r * (K + 1) + k] != want_idx || std::fabs(got_w - want_w) > want_w / 128 + 1e-6) {
          std::printf("row %d pick %d: got (%d, %f), want (%d, %f)\n", r, k, idx[r * (K + 1) + k], got_w, want_idx, want_w);
          ++bad;
        }
        if (__bfloat162float(__float2bfloat16(got_w)) != got_w) { std::printf("row %d pick %d: weight is not a bf16 value\n", r, k); ++bad; }
        if (want_idx >= 0) ++want_counts[want_idx];
      }
      const double gate = 1.0 / (1.0 + std::exp(-static_cast<double>(row[E])));
      const int want_shared = use_map ? map[E] : E;
      if (idx[r * (K + 1) + K] != want_shared || std::fabs(wts[r * (K + 1) + K] - gate) > gate / 128 + 1e-6) {
        std::printf("row %d shared expert: got (%d, %f), want (%d, %f)\n", r, idx[r * (K + 1) + K], wts[r * (K + 1) + K], want_shared, gate);
        ++bad;
      }
      ++want_counts[want_shared];
    }
    if (counts != want_counts) { std::printf("per-expert counts differ (map %d)\n", use_map); ++bad; }
    // the tie rule, spelled out: all-equal logits pick experts 0..7 with equal weights
    for (int k = 0; k < K; ++k)
      if (idx[1 * (K + 1) + k] != (use_map ? map[k] : k)) { std::printf("tied row picked %d at %d\n", idx[1 * (K + 1) + k], k); ++bad; }
  }
  if (bad) return 1;
  std::printf("OK route_row: %d rows x top-%d of %d experts, with and without a local expert map\n", ROWS, K, E);
  return 0;
}
