/* philox_ref.c — plain-C restatement of Philox4x32-10 and of the dropout keep-mask rule.
 * TEST INFRASTRUCTURE: compiled by oracle/Makefile into oracle/_build/libphilox_ref.so and
 * loaded only by tests and the smoke check.  The reference project (shmsong/NvFuserExamples)
 * contains no random-number code (its train operators take a dense dropout mask,
 * fmha/fmha_manual.cpp:433-449); this follows the published algorithm (Salmon et al., SC'11).
 */
#include <stdint.h>
#include <stddef.h>

static void philox_round(uint32_t c[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void philox4x32_10_c(uint32_t k0, uint32_t k1, const uint32_t ctr[4], uint32_t out[4]) {
  uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

int dropout_threshold_c(float p_drop) {
  int t = (int)(p_drop * 128.0f + 0.5f);
  if (t < 0) t = 0;
  if (t > 127) t = 127;
  return t;
}

/* out: [n_bh][S_q][S_k] bytes, 1 = kept */
void dropout_keep_mask_c(uint64_t seed, uint32_t offset, int32_t bh_offset, int32_t n_bh, int32_t S_q, int32_t S_k,
                         float p_drop, uint8_t* out) {
  const uint32_t thr = (uint32_t)dropout_threshold_c(p_drop);
  for (int32_t bh = 0; bh < n_bh; ++bh)
    for (int32_t r = 0; r < S_q; ++r)
      for (int32_t kb = 0; kb * 16 < S_k; ++kb) {
        const uint32_t ctr[4] = {(uint32_t)r, (uint32_t)kb, (uint32_t)(bh_offset + bh), offset};
        uint32_t w[4];
        philox4x32_10_c((uint32_t)seed, (uint32_t)(seed >> 32), ctr, w);
        for (int i = 0; i < 16 && kb * 16 + i < S_k; ++i) {
          const uint32_t byte = (w[i / 4] >> (8 * (i % 4))) & 0xffu;
          out[((size_t)bh * S_q + r) * S_k + kb * 16 + i] = (uint8_t)(((byte & 0x7fu) >= thr) ? 1 : 0);
        }
      }
}
