// fmha_fwd_sm100.cu — fused multi-head-attention forward for B200 (sm_100a).
//
// The general kernel: everything the three reference operators need that the production kernel
// (fmha_fwd_fast_sm100.cu) leaves out -- dense [B*H,S,S] masks, a dense dropout mask, saved
// intermediates, debug outputs.  One CTA owns a 128-row query tile of one (batch, head) and walks
// the keys in 128-wide tiles with an online softmax:
//
//   warp 0      TMA producer : Q once, then K and V tiles (and the dense padding-mask tile of
//                              the step) into shared memory (128-byte swizzle, zero fill past
//                              the tensor edge)
//   warp 1      MMA issuer   : S = Q K^T and O += P V as tcgen05.mma with fp32 accumulators
//                              in tensor memory; also owns the tensor-memory allocation
//   warps 2-5   softmax      : thread r owns row r of the tile: reads S from tensor memory,
//                              applies scale / mask, keeps the running max and sum, applies
//                              dropout, writes P (16-bit) back into the columns S occupied,
//                              rescales O when the running max moved, and at the end
//                              normalises O and stores it through shared memory with TMA.
//
// Tensor memory (256 columns per CTA, so two CTAs share an SM and overlap each other's
// softmax with tensor-core work): columns [0,128) hold S (fp32) and are overwritten by P
// (two 16-bit values per column, columns [0,64)); columns [128,128+D) hold O (fp32).
//
// What the math follows: the reference's fused forward definition
// (fmha/fmha_manual.cpp:55-97 inference, :457-492 train, :891-897 saved intermediates of
// shmsong/NvFuserExamples): fp16/bf16 operands, fp32 scores and softmax statistics, one
// rounding of P to 16 bits after the dropout factor, fp32 accumulation of O, one rounding of O.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "../../include/fmha_sm100.h"
#include "fmha_device_utils.cuh"
#include "fmha_kernel_args.h"
#include "philox.cuh"
#include "sm100_ptx.cuh"

namespace fmha {

namespace {

constexpr int kFwdThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMaskedKeep = -10000.0f;  // (1 - amask) * -10000, fmha_manual.cpp:64-65

enum WaitSite {
  kSiteQFull = 101, kSiteKEmpty = 102, kSiteVEmpty = 103, kSiteKFull = 104, kSiteVFull = 105,
  kSitePFull = 106, kSiteSFull = 107, kSiteOFull = 108, kSiteMFull = 109, kSiteMEmpty = 110
};

template <int D, bool PSMEM>
struct FwdSmem {
  static constexpr int kStages = 1;                  // K / V stages (CTAs sharing the SM overlap each other instead)
  static constexpr int kTileBytes = kTileM * D * 2;  // one Q / K / V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kTileBytes;
  static constexpr int kOffV = kOffK + kStages * kTileBytes;
  static constexpr int kOffP = kOffV + kStages * kTileBytes;
  static constexpr int kPBytes = PSMEM ? kTileM * kTileN * 2 : 0;
  static constexpr int kOffMask = kOffP + kPBytes;       // 2 x 128 floats
  static constexpr int kOffBar = kOffMask + 2 * kTileN * 4;
  static constexpr int kNumBars = 6 + 4 * kStages;       // q_full, s_full, p_full, o_full, m_full, m_empty + 4 per stage
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;  // tmem base, abort flag
  static constexpr int kBytes = kOffMisc + 16;
  // the dense mask tile (present or not, chosen per launch) follows: 128 x 128 16-bit = two swizzled 16 KB halves
  static constexpr int kOffMaskTiles = (kBytes + 1023) / 1024 * 1024;
  static constexpr int kMaskTileBytes = kTileM * kTileN * 2;
  static constexpr int dyn_bytes(int mask_tiles) { return kOffMaskTiles + mask_tiles * kMaskTileBytes + 1024; }  // + alignment slack
};

}  // namespace

template <int D, bool BF16, bool LEGACY, bool PSMEM>
__global__ void __launch_bounds__(kFwdThreads, 1) fmha_fwd_kernel(const __grid_constant__ FwdArgs a) {
  griddep_wait();
  using L = FwdSmem<D, PSMEM>;
  constexpr int ST = L::kStages;
  constexpr int kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColO = 128;
  constexpr int kFmt = BF16 ? 1 : 0;
  constexpr uint32_t kIdescQK = make_idesc_f16(128, 128, kFmt, false, false);
  constexpr uint32_t kIdescPV = make_idesc_f16(128, D, kFmt, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint8_t* sP = smem + L::kOffP;
  float* sMask = reinterpret_cast<float*>(smem + L::kOffMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;
  uint64_t* s_full = bars + 1;
  uint64_t* p_full = bars + 2;
  uint64_t* o_full = bars + 3;
  uint64_t* m_full = bars + 4;    // dense mask tiles of a step have landed
  uint64_t* m_empty = bars + 5;   // ... and have been consumed (all softmax threads arrive)
  uint64_t* k_full = bars + 6;
  uint64_t* k_empty = k_full + ST;
  uint64_t* v_full = k_empty + ST;
  uint64_t* v_empty = v_full + ST;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);
  uint8_t* sMaskT = smem + L::kOffMaskTiles;   // present when a.mask_tiles > 0

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q_tile = blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int q0 = q_tile * kTileM;
  const int bh = b * a.H + h;

  // ---- work list -------------------------------------------------------------------
  int k_limit = a.S_k;  // keys [0, k_limit) take part; the rest of the last tile is excluded
  int len_valid = a.S_k;  // FMHA_MASK_SEQLEN: keys >= len_valid are masked
  if (a.mask_kind == FMHA_MASK_SEQLEN) {
    const int len = reinterpret_cast<const int*>(a.mask)[b];
    if (len > 0 && len < a.S_k) { len_valid = len; k_limit = len; }
  }
  const int n_kv = (k_limit + kTileN - 1) / kTileN;
  const bool save_mode = LEGACY && (a.save_softmax != nullptr || a.save_dropout != nullptr);
  const int n_pre = save_mode ? n_kv : 0;  // statistics-only sweeps before the real one
  const int n_steps = n_pre + n_kv;

  // ---- set-up ----------------------------------------------------------------------
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(m_full, 1);
    mbar_init(m_empty, 128);
    for (int s = 0; s < ST; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&a.tm_q);
    tma_prefetch_desc(&a.tm_k);
    tma_prefetch_desc(&a.tm_v);
    tma_prefetch_desc(&a.tm_o);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  const WaitCtx wctx{abort_flag, a.status};

  if (warp == 0) {
    // ============================ TMA producer ======================================
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, L::kTileBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_4d(sQ + c * 16384, &a.tm_q, q_full, c * 64, q0, h, b);
      int kcnt = 0, vcnt = 0;
      for (int i = 0; i < n_steps; ++i) {
        const bool stats_only = i < n_pre;
        const int j = stats_only ? i : i - n_pre;
        if constexpr (LEGACY) {
          if (a.mask_tiles > 0) {
            // the mask tile of this step: rows of this query tile, key columns [j*128, +128) in two 64-column boxes
            if (i > 0) mbar_wait(m_empty, (i - 1) & 1, wctx, kSiteMEmpty);
            mbar_arrive_expect_tx(m_full, L::kMaskTileBytes);
            const int mrow = bh * a.S_q + q0;
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d(sMaskT + c * 16384, &a.tm_mask, m_full, j * kTileN + c * 64, mrow);
          }
        }
        {
          const int s = kcnt % ST;
          if (kcnt >= ST) mbar_wait(k_empty + s, ((kcnt / ST) - 1) & 1, wctx, kSiteKEmpty);
          mbar_arrive_expect_tx(k_full + s, L::kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(sK + s * L::kTileBytes + c * 16384, &a.tm_k, k_full + s, c * 64, j * kTileN, h, b);
          ++kcnt;
        }
        if (!stats_only) {
          const int s = vcnt % ST;
          if (vcnt >= ST) mbar_wait(v_empty + s, ((vcnt / ST) - 1) & 1, wctx, kSiteVEmpty);
          mbar_arrive_expect_tx(v_full + s, L::kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c)
            tma_load_4d(sV + s * L::kTileBytes + c * 16384, &a.tm_v, v_full + s, c * 64, j * kTileN, h, b);
          ++vcnt;
        }
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ========================================
    // The warp runs the loop convergently and issues the MMAs in bursts from one elected lane with
    // descriptors prepared beforehand (see umma_ss_x4): a single lane that computes each descriptor
    // and then issues is starved of issue slots by the softmax warps.
    {
      constexpr int KQ = D / 16;
      const uint32_t tS = tmem_base + kColS;
      const uint32_t tO = tmem_base + kColO;
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      uint64_t aq[KQ];
#pragma unroll
      for (int kk = 0; kk < KQ; ++kk) aq[kk] = dq + kmajor_step(kk, 16384);
      mbar_wait(q_full, 0, wctx, kSiteQFull);
      int kcnt = 0, vcnt = 0;
      for (int i = 0; i < n_steps; ++i) {
        const bool stats_only = i < n_pre;
        {
          const int s = kcnt % ST;
          const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + s * L::kTileBytes), 16, 1024);
          uint64_t bk[KQ];
#pragma unroll
          for (int kk = 0; kk < KQ; ++kk) bk[kk] = dk + kmajor_step(kk, 16384);
          mbar_wait(k_full + s, (kcnt / ST) & 1, wctx, kSiteKFull);
          tc_fence_after_sync();
          if constexpr (KQ == 4) umma_ss_x4(tS, aq, bk, kIdescQK, 0u);
          else umma_ss_x8(tS, aq, bk, kIdescQK, 0u);
          umma_commit_elect(k_empty + s);
          umma_commit_elect(s_full);
          ++kcnt;
        }
        mbar_wait(p_full, i & 1, wctx, kSitePFull);
        tc_fence_after_sync();
        if (!stats_only) {
          const int s = vcnt % ST;
          // B = V tile, MN-major: 16 key rows per step (2048 B), 64-wide d chunks 16 KB apart
          const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + s * L::kTileBytes), 16384, 1024);
          uint64_t bv[8];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) bv[kk] = dv + mnmajor_step(kk);
          mbar_wait(v_full + s, (vcnt / ST) & 1, wctx, kSiteVFull);
          tc_fence_after_sync();
          const uint32_t acc0 = (vcnt > 0) ? 1u : 0u;
          if constexpr (PSMEM) {
            const uint64_t dp = make_smem_desc_sw128(smem_u32(sP), 16, 1024);
            uint64_t ap[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) ap[kk] = dp + kmajor_step(kk, 16384);
            umma_ss_x8(tO, ap, bv, kIdescPV, acc0);
          } else {
            const uint64_t (&b0)[4] = *reinterpret_cast<const uint64_t (*)[4]>(&bv[0]);
            const uint64_t (&b1)[4] = *reinterpret_cast<const uint64_t (*)[4]>(&bv[4]);
            umma_ts_x4(tO, tS, 8u, b0, kIdescPV, acc0);
            umma_ts_x4(tO, tS + 32u, 8u, b1, kIdescPV, 1u);
          }
          umma_commit_elect(v_empty + s);
          ++vcnt;
        }
      }
      umma_commit_elect(o_full);
    }
  } else {
    // ============================ softmax / epilogue ================================
    const int quad = warp & 3;            // tensor-memory lane quarter this warp may touch
    const int row = quad * 32 + lane;     // row of the tile owned by this thread
    const int tid = threadIdx.x - 64;     // 0..127 within the softmax group
    const int q_row = q0 + row;
    const bool row_ok = q_row < a.S_q;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + kColS;
    const uint32_t tO = tmem_base + lane_addr + kColO;
    const size_t dense_row = (static_cast<size_t>(bh) * a.S_q + (row_ok ? q_row : 0)) * a.S_k;
    const float sl2 = a.scale_log2;
    const uint32_t gbh = static_cast<uint32_t>(a.philox_bh_offset + bh);

    float m_ref = -INFINITY;  // reference max (log2 domain) the stored exponentials use
    float l_sum = 0.f;        // running sum of exp2(t - m_ref)
    float inv_l = 1.f;        // save mode: 1 / final sum
    int pv_done = 0;

    for (int i = 0; i < n_steps; ++i) {
      const bool stats_only = i < n_pre;
      const int j = stats_only ? i : i - n_pre;
      const int col0 = j * kTileN;
      const int n_cols = min(kTileN, k_limit - col0);  // valid columns of this tile (>= 1)
      float* mask_stage = sMask + (i & 1) * kTileN;
      if (a.mask_kind == FMHA_MASK_KEY_ADDITIVE) {
        const int c = col0 + tid;
        mask_stage[tid] = (c < a.S_k) ? reinterpret_cast<const float*>(a.mask)[static_cast<size_t>(b) * a.S_k + c] * kLog2e : 0.f;
        named_bar_sync(1, 128);
      }
      mbar_wait(s_full, i & 1, wctx, kSiteSFull);
      tc_fence_after_sync();
      [[maybe_unused]] const bool mask_staged = LEGACY && a.mask_tiles > 0;
      if constexpr (LEGACY) {
        if (mask_staged) mbar_wait(m_full, i & 1, wctx, kSiteMFull);
      }
      // 32 staged 16-bit values of this thread's row: chunk c of the mask tile
      [[maybe_unused]] auto staged_row32 = [&](int c, float (&out)[32]) {
        const uint32_t tile = smem_u32(sMaskT + (c / 2) * 16384);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 w = lds128(tile + sw128_offset(row, (c % 2) * 4 + q));
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            out[q * 8 + 2 * k] = unpack_lo<BF16>(ws[k]);
            out[q * 8 + 2 * k + 1] = unpack_hi<BF16>(ws[k]);
          }
        }
      };

      // Produces chunk c (32 columns) of this row in the log2 domain: t = s*scale*log2e + mask*log2e,
      // -inf for excluded columns.
      auto load_t = [&](int c, float (&t)[32]) {
        uint32_t r[32];
        tmem_ld32(tS + c * 32, r);
        tmem_wait_ld();
        const int cbase = c * 32;
        if constexpr (LEGACY) {
          if (a.debug_scores != nullptr && row_ok && !stats_only) {
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (cbase + k < n_cols) a.debug_scores[dense_row + col0 + cbase + k] = __uint_as_float(r[k]);
          }
          if (a.mask_kind == FMHA_MASK_DENSE_KEEP || a.mask_kind == FMHA_MASK_DENSE_ADDITIVE) {
            float mv[32];
            const int nv = row_ok ? max(0, min(32, n_cols - cbase)) : 0;
            if (mask_staged) staged_row32(c, mv);   // columns past n_cols are excluded below, rows past S_q are never stored
            else load_row32<BF16>(a.mask, dense_row + col0 + cbase, nv, a.mask_kind == FMHA_MASK_DENSE_KEEP ? 1.f : 0.f, mv);
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float add = (a.mask_kind == FMHA_MASK_DENSE_KEEP) ? (1.0f - mv[k]) * kMaskedKeep : mv[k];
              t[k] = fmaf(__uint_as_float(r[k]), sl2, add * kLog2e);
            }
          } else if (a.mask_kind == FMHA_MASK_KEY_ADDITIVE) {
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = fmaf(__uint_as_float(r[k]), sl2, mask_stage[cbase + k]);
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = __uint_as_float(r[k]) * sl2;
          }
        } else {
          if (a.mask_kind == FMHA_MASK_KEY_ADDITIVE) {
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = fmaf(__uint_as_float(r[k]), sl2, mask_stage[cbase + k]);
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k) t[k] = __uint_as_float(r[k]) * sl2;
          }
        }
        if (cbase + 32 > n_cols) {
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (cbase + k >= n_cols) t[k] = -INFINITY;
        }
      };

      // ---- pass 1: row maximum ------------------------------------------------------
      float tile_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kTileN / 32; ++c) {
        if (c * 32 >= n_cols) break;
        float t[32];
        load_t(c, t);
        float mx0 = fmaxf(t[0], t[1]), mx1 = fmaxf(t[2], t[3]);
#pragma unroll
        for (int k = 4; k < 32; k += 2) {
          mx0 = fmaxf(mx0, t[k]);
          mx1 = fmaxf(mx1, t[k + 1]);
        }
        tile_max = fmaxf(tile_max, fmaxf(mx0, mx1));
      }

      const bool fixed_stats = save_mode && !stats_only;  // m_ref and l_sum are final already
      if (!fixed_stats) {
        float m_new = fmaxf(m_ref, tile_max);
        // Keep the old reference while the maximum moved by less than 2^8: the stored
        // exponentials stay below 256 and no rescale of O is needed.
        if (m_ref != -INFINITY && m_new - m_ref <= 8.0f) m_new = m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        const bool moved = (m_new != m_ref) && (m_ref != -INFINITY);
        if (pv_done > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * alpha);
            tmem_st32(tO + c * 32, r);
          }
        }
        l_sum *= alpha;
        m_ref = m_new;
      }

      // ---- pass 2: exponentials, dropout, P ----------------------------------------
      float psum = 0.f;
#pragma unroll 1
      for (int c = 0; c < kTileN / 32; ++c) {
        uint32_t packed[16];
        if (c * 32 < n_cols) {
          float t[32];
          load_t(c, t);
#pragma unroll
          for (int k = 0; k < 32; ++k) t[k] = fast_exp2(t[k] - m_ref);
          if (!fixed_stats) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int k = 0; k < 32; k += 2) { s0 += t[k]; s1 += t[k + 1]; }
            psum += s0 + s1;
          }
          if (stats_only) continue;
          const int cbase = c * 32;
          const int nv = row_ok ? max(0, min(32, n_cols - cbase)) : 0;
          if constexpr (LEGACY) {
            if (save_mode) {
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] *= inv_l;
              if (a.save_softmax != nullptr && nv > 0) store_row32<BF16>(a.save_softmax, dense_row + col0 + cbase, nv, t);
            }
            if (a.dropout_kind == FMHA_DROPOUT_DENSE) {
              float dm[32];
              load_row32<BF16>(a.dropout_mask, dense_row + col0 + cbase, nv, 0.f, dm);
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] *= dm[k] * (save_mode ? a.dropout_scale : 1.0f);
            }
          }
#pragma unroll
          for (int k = 0; k < 16; ++k) packed[k] = pack2<BF16>(t[2 * k], t[2 * k + 1]);
          if (a.dropout_kind == FMHA_DROPOUT_PHILOX) {
#pragma unroll
            for (int d = 0; d < 2; ++d) {
              const U4 draw = dropout_draw(a.philox_seed, a.philox_offset, gbh, static_cast<uint32_t>(q_row),
                                           static_cast<uint32_t>((col0 + cbase) / 16 + d));
              const uint32_t w[4] = {draw.x, draw.y, draw.z, draw.w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t keep = dropout_keep_bits(w[k], a.philox_thr);
                packed[d * 8 + 2 * k] &= prmt(keep, 0u, 0x9988u);
                packed[d * 8 + 2 * k + 1] &= prmt(keep, 0u, 0xBBAAu);
                if constexpr (LEGACY) {
                  if (a.keep_mask_out != nullptr && row_ok) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      const int col = cbase + d * 16 + k * 4 + e;
                      if (col < n_cols) a.keep_mask_out[dense_row + col0 + col] = (keep >> (8 * e + 7)) & 1u;
                    }
                  }
                }
              }
            }
            if constexpr (LEGACY) {
              if (save_mode) {
                // saved tensors carry the scale explicitly: P <- P * keep * scale
#pragma unroll
                for (int k = 0; k < 16; ++k)
                  packed[k] = pack2<BF16>(unpack_lo<BF16>(packed[k]) * a.dropout_scale,
                                          unpack_hi<BF16>(packed[k]) * a.dropout_scale);
              }
            }
          }
          if constexpr (LEGACY) {
            if (save_mode && a.save_dropout != nullptr && nv > 0) {
              float dv[32];
#pragma unroll
              for (int k = 0; k < 16; ++k) { dv[2 * k] = unpack_lo<BF16>(packed[k]); dv[2 * k + 1] = unpack_hi<BF16>(packed[k]); }
              store_row32<BF16>(a.save_dropout, dense_row + col0 + cbase, nv, dv);
            }
          }
        } else {
          if (stats_only) continue;
#pragma unroll
          for (int k = 0; k < 16; ++k) packed[k] = 0u;
        }
        if constexpr (PSMEM) {
          uint8_t* tile = sP + (c / 2) * 16384;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 w = make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
            *reinterpret_cast<uint4*>(tile + sw128_offset(row, (c % 2) * 4 + q)) = w;
          }
        } else {
          tmem_st16(tS + c * 16, packed);
        }
      }
      if (!fixed_stats) l_sum += psum;
      if (stats_only && i == n_pre - 1) inv_l = 1.0f / l_sum;

      if (!stats_only) {
        if constexpr (PSMEM) fence_proxy_async_smem();
        ++pv_done;
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(p_full);
      if constexpr (LEGACY) {
        if (mask_staged) mbar_arrive(m_empty);
      }
    }

    // ---- epilogue: normalise O, store O and the logsumexp --------------------------
    mbar_wait(o_full, 0, wctx, kSiteOFull);
    tc_fence_after_sync();
    float out_scale;
    if (save_mode) out_scale = 1.0f;  // P was normalised (and dropout-scaled) before the second GEMM
    else out_scale = ((a.dropout_kind != FMHA_DROPOUT_NONE) ? a.dropout_scale : 1.0f) / l_sum;
    if (a.lse != nullptr && row_ok)
      a.lse[static_cast<size_t>(bh) * a.S_q + q_row] = (m_ref + fast_log2(l_sum)) * kLn2;
    // sQ is free: every QK^T finished before o_full fired.
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + c * 32, r);
      tmem_wait_ld();
      uint8_t* tile = sQ + (c / 2) * 16384;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 w;
        w.x = pack2<BF16>(__uint_as_float(r[q * 8 + 0]) * out_scale, __uint_as_float(r[q * 8 + 1]) * out_scale);
        w.y = pack2<BF16>(__uint_as_float(r[q * 8 + 2]) * out_scale, __uint_as_float(r[q * 8 + 3]) * out_scale);
        w.z = pack2<BF16>(__uint_as_float(r[q * 8 + 4]) * out_scale, __uint_as_float(r[q * 8 + 5]) * out_scale);
        w.w = pack2<BF16>(__uint_as_float(r[q * 8 + 6]) * out_scale, __uint_as_float(r[q * 8 + 7]) * out_scale);
        *reinterpret_cast<uint4*>(tile + sw128_offset(row, (c % 2) * 4 + q)) = w;
      }
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (tid == 0) {
      if (*abort_flag == 0) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_store_4d(&a.tm_o, sQ + c * 16384, c * 64, q0, h, b);
        tma_store_commit();
      }
      tma_store_wait_all();
    }
  }

  // ---- teardown ----------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // A wait was abandoned: give copies that may still be in flight time to land before
    // the shared memory of this CTA is released.
    for (int k = 0; k < 20; ++k) __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------------
// launcher
// --------------------------------------------------------------------------------------
template <int D, bool BF16, bool LEGACY, bool PSMEM>
static int launch_fwd_impl(const FwdArgs& a, cudaStream_t stream) {
  using L = FwdSmem<D, PSMEM>;
  auto kfn = fmha_fwd_kernel<D, BF16, LEGACY, PSMEM>;
  static std::atomic<bool> configured[64] = {};   // per device; set after the attribute call succeeded
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::dyn_bytes(1));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid((a.S_q + kTileM - 1) / kTileM, a.H, a.B);
  const cudaError_t e = launch_overlapped(kfn, grid, dim3(kFwdThreads), L::dyn_bytes(a.mask_tiles), stream, a);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_fwd(const FwdArgs& a, int D, int dtype, bool legacy, bool p_via_smem, cudaStream_t stream) {
  if (!legacy) return launch_fwd_fast(a, D, dtype, stream);  // compact masks, Philox dropout: the production kernel
  // the reference's dense-mask operators with nothing saved: the persistent, double-buffered kernel
  if (!p_via_smem && fwd_dense_applies(a, D)) return launch_fwd_dense(a, dtype, stream);
#define FMHA_FWD_CASE(DD, BF, LG, PS) \
  if (D == DD && (dtype == FMHA_DTYPE_BF16) == BF && legacy == LG && p_via_smem == PS) \
    return launch_fwd_impl<DD, BF, LG, PS>(a, stream);
  FMHA_FWD_CASE(64, false, true, false)
  FMHA_FWD_CASE(64, true, true, false)
  FMHA_FWD_CASE(128, false, true, false)
  FMHA_FWD_CASE(128, true, true, false)
  FMHA_FWD_CASE(64, false, true, true)
  FMHA_FWD_CASE(64, true, true, true)
  FMHA_FWD_CASE(128, false, true, true)
  FMHA_FWD_CASE(128, true, true, true)
#undef FMHA_FWD_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // namespace fmha
