// Control for the race check of the emulated kernels: a "kernel" in which every thread of a CTA reads its neighbour's
// slot of a shared array, once with the barrier between the write and the read and once without it. Under
// -fsanitize=thread the second form must be reported as a data race and the first must not: this shows that a
// missing __syncthreads() in a kernel compiled through emu_shim.h would be seen. Host code only.
//   g++ -std=c++20 -O1 -g -pthread -fsanitize=thread -I tests/emu -x c++ tests/emu/race_control.cpp -o race_control
//   ./race_control with-barrier ; ./race_control without-barrier
#include "emu_shim.h"

#include <cstdio>
#include <cstring>

using namespace b200;

static float slots[64];

static void neighbour_sum(float* out, bool barrier) {
  const unsigned t = threadIdx.x;
  slots[t] = static_cast<float>(t);
  if (barrier) __syncthreads();
  out[t] = slots[t] + slots[(t + 1) % blockDim.x];
}

int main(int argc, char** argv) {
  const bool barrier = argc > 1 && std::strcmp(argv[1], "with-barrier") == 0;
  std::vector<float> out(64, 0.f);
  run_cta(64, 0, 0, [&] { neighbour_sum(out.data(), barrier); });
  std::printf("done %s\n", barrier ? "with-barrier" : "without-barrier");
  return 0;
}
