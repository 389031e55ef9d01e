// philox.cuh — Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3",
// SC'11) and the dropout rule built on it.  Host and device compile the same functions, so
// the mask a test regenerates on the CPU is the mask the kernels applied.
//
// Dropout definition (shared by forward, backward and the mask generators):
//   draw   = philox4x32_10(key = (seed_lo, seed_hi),
//                          counter = (q_row, key_col / 16, b*H + h, offset))
//   byte i = (draw.word[i / 4] >> (8 * (i % 4))) & 0xff        for key_col % 16 == i
//   keep   = (byte & 0x7f) >= T,   T = round(128 * p_drop) in [0, 127]
//   kept probabilities are multiplied by 128 / (128 - T).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FMHA_HD __host__ __device__ __forceinline__
#else
#define FMHA_HD inline
#endif

namespace fmha {

struct U4 {
  uint32_t x, y, z, w;
};

FMHA_HD void mulhilo32(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
#if defined(__CUDA_ARCH__)
  // one 32x32->64 multiply instead of separate low and high halves
  asm("{\n\t"
      ".reg .b64 p;\n\t"
      "mul.wide.u32 p, %2, %3;\n\t"
      "mov.b64 {%0, %1}, p;\n\t"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(a), "r"(b));
#else
  const uint64_t p = static_cast<uint64_t>(a) * static_cast<uint64_t>(b);
  lo = static_cast<uint32_t>(p);
  hi = static_cast<uint32_t>(p >> 32);
#endif
}

FMHA_HD U4 philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  constexpr uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo32(M0, c0, hi0, lo0);
    mulhilo32(M1, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n1 = lo1;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    const uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += W0;
    k1 += W1;
  }
  U4 out;
  out.x = c0; out.y = c1; out.z = c2; out.w = c3;
  return out;
}

// Same generator with the ten round keys supplied by the caller (key r = seed word + r * Weyl
// constant).  The kernels receive them as launch parameters, so the per-round key update costs
// no instruction: the key is a constant-bank operand of the XOR.
struct PhiloxKeys {
  uint32_t k[20];  // k[2r], k[2r+1] = keys of round r
};
FMHA_HD PhiloxKeys philox_round_keys(uint64_t seed) {
  PhiloxKeys ks;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    ks.k[2 * r] = k0;
    ks.k[2 * r + 1] = k1;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return ks;
}
FMHA_HD U4 philox4x32_10_keys(const PhiloxKeys& ks, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    mulhilo32(M0, c0, hi0, lo0);
    mulhilo32(M1, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ ks.k[2 * r];
    const uint32_t n2 = hi0 ^ c3 ^ ks.k[2 * r + 1];
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
  }
  U4 out;
  out.x = c0; out.y = c1; out.z = c2; out.w = c3;
  return out;
}
// The 16 random bytes that decide keys [16*kb, 16*kb+16) of query row `row` in head `bh`.
FMHA_HD U4 dropout_draw_keys(const PhiloxKeys& ks, uint32_t offset, uint32_t bh, uint32_t row, uint32_t kb) {
  return philox4x32_10_keys(ks, row, kb, bh, offset);
}

// T = round(128 p), clamped so that at least 1/128 of the entries survive.
FMHA_HD int dropout_threshold(float p_drop) {
  int t = static_cast<int>(p_drop * 128.0f + 0.5f);
  if (t < 0) t = 0;
  if (t > 127) t = 127;
  return t;
}

// The 16 random bytes that decide keys [16*kb, 16*kb+16) of query row `row` in head `bh`.
FMHA_HD U4 dropout_draw(uint64_t seed, uint32_t offset, uint32_t bh, uint32_t row, uint32_t kb) {
  return philox4x32_10(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), row, kb, bh, offset);
}

// Bit 7 of each byte of the result is the keep decision of that byte of `w`.
FMHA_HD uint32_t dropout_keep_bits(uint32_t w, uint32_t thr) {
  return ((w & 0x7F7F7F7Fu) + (0x80u - thr) * 0x01010101u) & 0x80808080u;
}

}  // namespace fmha
