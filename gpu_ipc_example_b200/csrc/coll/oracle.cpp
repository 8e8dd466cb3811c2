#include "oracle.h"

#include <cmath>

#include "../common/half_host.h"

namespace b200ipc {

void fill_pattern(DType t, uint16_t* dst, int rank, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = from_float(t, float((i % 32) * size_t(rank + 1)));
}

namespace {
// splitmix64: counter based, so any element can be regenerated independently
uint64_t mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
double unit(uint64_t x) { return double(x >> 11) * (1.0 / 9007199254740992.0); }
}  // namespace

void fill_random(DType t, uint16_t* dst, int rank, size_t n, bool uniform) {
  const uint64_t seed = mix(uint64_t(rank) * 0x100000001b3ull + 12345);
  for (size_t i = 0; i < n; ++i) {
    const uint64_t a = mix(seed ^ (2 * i));
    const uint64_t b = mix(seed ^ (2 * i + 1));
    float v;
    if (uniform) {
      v = float(2.0 * unit(a) - 1.0);
    } else {
      double u1 = unit(a);
      if (u1 < 1e-300) u1 = 1e-300;
      v = float(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * unit(b)));
    }
    dst[i] = from_float(t, v);
  }
}

void cpu_all_reduce(DType t, const std::vector<const uint16_t*>& inputs, uint16_t* result, size_t n, bool round_each) {
  const size_t N = inputs.size();
  for (size_t i = 0; i < n; ++i) {
    float acc = to_float(t, inputs[0][i]);
    for (size_t r = 1; r < N; ++r) {
      acc += to_float(t, inputs[r][i]);
      if (round_each) acc = to_float(t, from_float(t, acc));
    }
    result[i] = from_float(t, acc);
  }
}

void cpu_all_gather(const std::vector<const uint16_t*>& inputs, uint16_t* result, size_t n_per_rank) {
  for (size_t r = 0; r < inputs.size(); ++r)
    for (size_t i = 0; i < n_per_rank; ++i) result[r * n_per_rank + i] = inputs[r][i];
}

VerifyReport verify_buffer(DType t, const uint16_t* got, const uint16_t* want, size_t n, bool exact, float atol,
                           float rtol) {
  VerifyReport rep;
  for (size_t i = 0; i < n; ++i) {
    bool bad;
    const float g = to_float(t, got[i]);
    const float w = to_float(t, want[i]);
    if (exact) {
      bad = got[i] != want[i];
    } else {
      const float err = std::fabs(g - w);
      bad = !(err <= atol + rtol * std::fabs(w));
      if (double(err) > rep.max_abs_err) rep.max_abs_err = err;
    }
    if (bad) {
      if (rep.mismatches == 0) {
        rep.first_index = i;
        rep.first_expected = w;
        rep.first_got = g;
      }
      ++rep.mismatches;
    }
  }
  return rep;
}

}  // namespace b200ipc
