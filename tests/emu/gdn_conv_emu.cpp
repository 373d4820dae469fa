// Runs the short-convolution decode step (ops/cuda/gdn_decode.cu: gdn_conv_step_kernel<4>, compiled as host C++
// through emu_shim.h) for B sequences x G rows and checks outputs, the state left in the slots and the per-row
// state ring against a float64 restatement. Exit code 0 and a line "OK ..." on success.
//   g++ -std=c++20 -O1 -pthread -DB200_EMU -I tests/emu -x c++ tests/emu/gdn_conv_emu.cpp -o gdn_conv_emu
#include "emu_shim.h"

#include "../../qwen36-mi250-tracelab-20261107_b200/ops/cuda/gdn_decode.cu"

#include <cstdio>
#include <random>

using namespace b200;

int main() {
  constexpr int KW = 4, C = 48, B = 3, G = 3, SLOTS = 5, THREADS = 4;
  constexpr int ld = C + 24;  // the conv input is the first C columns of a wider row
  std::mt19937 rng(3);
  std::normal_distribution<float> nd(0.f, 1.f);
  auto rb = [&](float s) { return __float2bfloat16(nd(rng) * s); };
  std::vector<bf16> mixed(B * G * ld), state(SLOTS * C * (KW - 1)), w(C * KW), out(B * G * C), ring(B * G * C * (KW - 1));
  for (auto& v : mixed) v = rb(1.f);
  for (auto& v : state) v = rb(1.f);
  for (auto& v : w) v = rb(0.5f);
  const std::vector<int> slots = {4, 1, 2};
  const std::vector<bf16> state0 = state;

  gridDim.x = (C / 8 + THREADS - 1) / THREADS;
  for (int b = 0; b < B; ++b)
    for (unsigned bx = 0; bx < gridDim.x; ++bx)
      run_cta(THREADS, bx, b, [&] {
        gdn_conv_step_kernel<KW>(mixed.data(), ld, slots.data(), state.data(), w.data(), out.data(), ring.data(), C, G);
      });

  int bad = 0;
  double worst = 0;
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < C; ++c) {
      double win[KW];
      for (int k = 0; k < KW - 1; ++k) win[k] = __bfloat162float(state0[(slots[b] * C + c) * (KW - 1) + k]);
      for (int j = 0; j < G; ++j) {
        win[KW - 1] = __bfloat162float(mixed[(b * G + j) * ld + c]);
        double acc = 0;
        for (int k = 0; k < KW; ++k) acc += win[k] * __bfloat162float(w[c * KW + k]);
        const double want = acc / (1.0 + std::exp(-acc));
        const double got = __bfloat162float(out[(b * G + j) * C + c]);
        worst = std::max(worst, std::fabs(got - want));
        if (std::fabs(got - want) > std::fabs(want) / 100 + 1e-2) { std::printf("out[%d,%d,%d] = %f, want %f\n", b, j, c, got, want); ++bad; }
        for (int k = 0; k < KW - 1; ++k) win[k] = win[k + 1];
        for (int k = 0; k < KW - 1; ++k)  // the window after row j, exactly (inputs are bf16 values already)
          if (__bfloat162float(ring[((b * G + j) * C + c) * (KW - 1) + k]) != static_cast<float>(win[k])) { std::printf("ring[%d,%d,%d,%d]\n", b, j, c, k); ++bad; }
      }
      for (int k = 0; k < KW - 1; ++k)
        if (__bfloat162float(state[(slots[b] * C + c) * (KW - 1) + k]) != static_cast<float>(win[k])) { std::printf("state[%d,%d,%d]\n", b, c, k); ++bad; }
    }
  // slots that no sequence used are untouched
  for (int s : {0, 3})
    for (int i = 0; i < C * (KW - 1); ++i)
      if (state[s * C * (KW - 1) + i].bits != state0[s * C * (KW - 1) + i].bits) { std::printf("slot %d changed\n", s); ++bad; break; }
  if (bad) return 1;
  std::printf("OK gdn_conv_step emu: %d sequences x %d rows x %d channels, max |output err| %.3g\n", B, G, C, worst);
  return 0;
}
