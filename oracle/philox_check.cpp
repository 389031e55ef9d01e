// philox_check.cpp — prints Philox4x32-10 outputs of PyTorch's own host engine
// (ATen/core/PhiloxRNGEngine.h, header only) for counters read from stdin, so that the numpy
// and C restatements under oracle/ can be pinned against an independent implementation.
// TEST INFRASTRUCTURE: built by oracle/Makefile, run by tests/golden/make_golden.py.
//
// stdin : lines "seed c0 c1 c2 c3" (decimal, seed 64-bit, counters 32-bit)
// stdout: lines "w0 w1 w2 w3"
// at::philox_engine(seed, subsequence, offset) places offset in counter words 0-1 and
// subsequence in words 2-3, so counter (c0,c1,c2,c3) is offset = c0 | c1<<32,
// subsequence = c2 | c3<<32.
#include <ATen/core/PhiloxRNGEngine.h>

#include <cinttypes>
#include <cstdio>

int main() {
  uint64_t seed;
  uint32_t c[4];
  while (std::scanf("%" SCNu64 " %" SCNu32 " %" SCNu32 " %" SCNu32 " %" SCNu32, &seed, &c[0], &c[1], &c[2], &c[3]) == 5) {
    at::philox_engine eng(seed, static_cast<uint64_t>(c[2]) | (static_cast<uint64_t>(c[3]) << 32),
                          static_cast<uint64_t>(c[0]) | (static_cast<uint64_t>(c[1]) << 32));
    const uint32_t w0 = eng(), w1 = eng(), w2 = eng(), w3 = eng();
    std::printf("%" PRIu32 " %" PRIu32 " %" PRIu32 " %" PRIu32 "\n", w0, w1, w2, w3);
  }
  return 0;
}
