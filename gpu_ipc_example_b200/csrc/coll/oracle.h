// CPU oracles for verification.
//
// Capability parity: fill_pattern (utils.hpp:15-19), the CPU allreduce/allgather
// and the verify functions (allreduce.cpp:5-35, 519-585).  Unlike the reference,
// whose verify prints mismatches but reports success (allreduce.cpp:543-550), the
// verifiers here return the number of mismatches so that callers can fail.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include "../common/types.h"

namespace b200ipc {

// input[i] = T((i % 32) * (rank + 1)).  Every partial sum of these over up to 8
// ranks is an integer <= 31 * 36 = 1116, exact in fp16 (not in bf16, so bf16
// verification uses a tolerance).
void fill_pattern(DType t, uint16_t* dst, int rank, size_t n);
// Reproducible pseudo-random values: normal(0,1) (all-reduce) or uniform(-1,1)
// (all-gather) from a counter-based generator seeded by the rank.
void fill_random(DType t, uint16_t* dst, int rank, size_t n, bool uniform);

// Expected all-reduce of explicit inputs, summed in rank order 0..N-1.
//   round_each=true sums in T like the reference; otherwise fp32 accumulate, one rounding.
// (The two-phase schedules add in owner rotation y, y+1, ...; for the integer pattern every order
// gives the same bits, for random data the comparison uses a tolerance.)
void cpu_all_reduce(DType t, const std::vector<const uint16_t*>& inputs, uint16_t* result, size_t n, bool round_each);
void cpu_all_gather(const std::vector<const uint16_t*>& inputs, uint16_t* result, size_t n_per_rank);

struct VerifyReport {
  size_t mismatches = 0;
  size_t first_index = 0;
  float first_expected = 0, first_got = 0;
  double max_abs_err = 0;
};
// exact: bit-for-bit (fp16 pattern).  Otherwise |got - want| <= atol + rtol * |want|.
VerifyReport verify_buffer(DType t, const uint16_t* got, const uint16_t* want, size_t n, bool exact, float atol,
                           float rtol);

}  // namespace b200ipc
