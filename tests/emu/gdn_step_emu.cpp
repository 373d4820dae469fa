// Runs the Gated DeltaNet decode-step kernel body (ops/cuda/gdn_decode.cu, compiled as host C++ through
// emu_shim.h) for a few (sequence, head) CTAs with G rows each and checks state and outputs against a float64
// restatement of the gated delta rule. Exit code 0 and a line "OK ..." on success.
//   g++ -std=c++20 -O1 -pthread -DB200_EMU -I tests/emu -x c++ tests/emu/gdn_step_emu.cpp -o gdn_step_emu
#include "emu_shim.h"

#include "../../qwen36-mi250-tracelab-20261107_b200/ops/cuda/gdn_decode.cu"

#include <cstdio>
#include <random>

using namespace b200;

int main() {
  constexpr int DK = 32, DV = 32, HK = 1, HV = 2, B = 2, G = 3;
  constexpr int key_dim = HK * DK, C = 2 * key_dim + HV * DV;
  constexpr int ld = C + HV * DV + 2 * HV, z_off = C, b_off = C + HV * DV, a_off = b_off + HV;
  const float eps = 1e-6f;
  std::mt19937 rng(7);
  std::normal_distribution<float> nd(0.f, 1.f);
  auto rb = [&](float s) { return __float2bfloat16(nd(rng) * s); };

  std::vector<bf16> conv_out(B * G * C), mixed(B * G * ld), gnorm(DV), out(B * G * HV * DV);
  for (auto& v : conv_out) v = rb(1.f);
  for (auto& v : mixed) v = rb(1.f);
  for (auto& v : gnorm) v = rb(0.5f);
  std::vector<float> A_log(HV), dt_bias(HV), state((B + 1) * HV * DK * DV), ring(B * G * HV * DK * DV);
  for (auto& v : A_log) v = nd(rng) * 0.5f;
  for (auto& v : dt_bias) v = nd(rng) * 0.5f;
  for (auto& v : state) v = nd(rng) * 0.1f;
  std::vector<int> slots = {2, 1};
  std::vector<double> ref_state(state.begin(), state.end());
  int err = 0;

  for (int b = 0; b < B; ++b)
    for (int h = 0; h < HV; ++h)
      run_cta(4 * DV, h, b, [&] {
        gdn_step_kernel<DK, DV>(conv_out.data(), mixed.data(), ld, z_off, b_off, a_off, slots.data(), state.data(),
                                A_log.data(), dt_bias.data(), gnorm.data(), out.data(), ring.data(), HK, HV, G, eps, &err);
      });

  // float64 reference of the same rule, row by row
  double max_out = 0, max_state = 0, max_ring = 0;
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < HV; ++h) {
      double* S = ref_state.data() + (static_cast<size_t>(slots[b]) * HV + h) * DK * DV;
      const int hk = h / (HV / HK);
      for (int j = 0; j < G; ++j) {
        const size_t row = static_cast<size_t>(b) * G + j;
        const bf16* co = conv_out.data() + row * C;
        double q[DK], k[DK], nq = 0, nk = 0;
        for (int i = 0; i < DK; ++i) {
          q[i] = __bfloat162float(co[hk * DK + i]);
          k[i] = __bfloat162float(co[key_dim + hk * DK + i]);
          nq += q[i] * q[i];
          nk += k[i] * k[i];
        }
        for (int i = 0; i < DK; ++i) { q[i] *= 1.0 / std::sqrt(nq + 1e-6) / std::sqrt(double(DK)); k[i] *= 1.0 / std::sqrt(nk + 1e-6); }
        const double a = __bfloat162float(mixed[row * ld + a_off + h]), bb = __bfloat162float(mixed[row * ld + b_off + h]);
        const double x = a + dt_bias[h];
        const double decay = std::exp(-std::exp(double(A_log[h])) * (x > 20 ? x : std::log1p(std::exp(x))));
        const double beta = 1.0 / (1.0 + std::exp(-bb));
        double o[DV], ss = 0;
        for (int c = 0; c < DV; ++c) {
          double kv = 0;
          for (int i = 0; i < DK; ++i) { S[i * DV + c] *= decay; kv += S[i * DV + c] * k[i]; }
          const double delta = (__bfloat162float(co[2 * key_dim + h * DV + c]) - kv) * beta;
          o[c] = 0;
          for (int i = 0; i < DK; ++i) { S[i * DV + c] += k[i] * delta; o[c] += S[i * DV + c] * q[i]; }
          ss += o[c] * o[c];
        }
        const double inv = 1.0 / std::sqrt(ss / DV + eps);
        for (int c = 0; c < DV; ++c) {
          const double z = __bfloat162float(mixed[row * ld + z_off + h * DV + c]);
          const double want = __bfloat162float(gnorm[c]) * o[c] * inv * (z / (1.0 + std::exp(-z)));
          max_out = std::fmax(max_out, std::fabs(want - __bfloat162float(out[row * (HV * DV) + h * DV + c])));
        }
        const float* rr = ring.data() + ((static_cast<size_t>(b) * G + j) * HV + h) * DK * DV;
        for (int i = 0; i < DK * DV; ++i) max_ring = std::fmax(max_ring, std::fabs(S[i] - rr[i]));
      }
      const float* got = state.data() + (static_cast<size_t>(slots[b]) * HV + h) * DK * DV;
      for (int i = 0; i < DK * DV; ++i) max_state = std::fmax(max_state, std::fabs(S[i] - got[i]));
    }
  // the untouched slot 0 must still hold its initial values
  double untouched = 0;
  for (int i = 0; i < HV * DK * DV; ++i) untouched = std::fmax(untouched, std::fabs(ref_state[i] - state[i]));
  const bool ok = err == 0 && max_state < 1e-4 && max_ring < 1e-4 && max_out < 0.06 && untouched == 0;
  std::printf("%s gdn_step emu: max |state err| %.3g, ring %.3g, output %.3g (bf16 outputs), err word %d\n",
              ok ? "OK" : "FAIL", max_state, max_ring, max_out, err);
  return ok ? 0 : 1;
}
