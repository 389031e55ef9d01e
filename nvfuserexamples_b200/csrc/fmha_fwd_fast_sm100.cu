// fmha_fwd_fast_sm100.cu — the production forward kernel: compact masks only (none, valid
// lengths, additive [B,S_k] row, or a packed variable-length batch), optional Philox dropout,
// writes O and the row logsumexp.
//
// CTA organisation as in the general kernel in fmha_fwd_sm100.cu (TMA producer, tcgen05.mma
// issuer, four softmax warps with one thread per query row; S in tensor memory, P written back
// over it, O beside it).  Head dimension 64 walks the keys in 64-key steps (S 64 + O 64 = 128
// tensor-memory columns); there the producer and the MMA issuer are ONE warp, so a CTA has five
// warps and four CTAs share an SM at 96 registers per thread.  Head dimension 128 uses 128-key
// steps, separate producer and MMA warps and two CTAs per SM.  The softmax is written for instruction count and
// latency, because at head dimension 64 the softmax warps, not the tensor core, set the pace:
//   * mask kind, dropout and the packed-batch bookkeeping are template parameters: no
//     per-chunk branches and no registers spent on modes that are off;
//   * the row maximum is taken over the raw accumulators with 3-input max (the scale is
//     positive), the exponent argument is one packed fma.rn.f32x2 per two elements, the row
//     sum one packed add;
//   * S is read twice from tensor memory (max, then exponentials) instead of being held in
//     registers; in the second sweep the load of the next 32 columns is in flight while the
//     current 32 are processed;
//   * Philox uses one 32x32->64 multiply per product, its keep words for a key step are
//     computed before the step's scores are awaited (they do not depend on them), and the
//     keep decision is applied to the packed 16-bit pairs with two byte permutes and two ANDs
//     per four elements;
//   * the MMA warp issues in bursts from a converged warp (see umma_ss_x4 in sm100_ptx.cuh).
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

// D = 128: 192 threads (TMA producer warp, MMA warp, four softmax warps).  D = 64: 160 threads, one warp issues both
// the TMA loads and the MMAs.  Registers are allocated per SM sub-partition (16 384 each, warps dealt round-robin):
// four CTAs of six warps put six warps on a sub-partition (80 registers per thread), four CTAs of five warps put
// five (96), which is what the dropout and additive-mask variants need to stay out of local memory.
constexpr int kThreadsSplit = 192, kThreadsMerged = 160;
template <int D> constexpr int fast_threads() { return D == 64 ? kThreadsMerged : kThreadsSplit; }
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

enum FastWaitSite {
  kFQFull = 111, kFKEmpty = 112, kFVEmpty = 113, kFKFull = 114, kFVFull = 115, kFPFull = 116, kFSFull = 117,
  kFOFull = 118
};

// TN = keys per step.  D = 64 uses 64-key steps: S (64 columns) + O (64 columns) = 128 tensor-memory
// columns and 48 KB of shared memory per CTA, so FOUR CTAs share an SM and their softmax and
// tensor-core phases interleave; D = 128 uses 128-key steps and two CTAs per SM.
template <int D, bool DROP = false>
struct FastSmem {
  static constexpr int TN = (D == 64) ? 64 : 128;
  // Four CTAs per SM at D = 64 (five warps each: 96 registers per thread), two at D = 128.
  static constexpr int kCtasPerSm = (D == 64) ? 4 : 2;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kQBytes = kTileM * D * 2;
  static constexpr int kTileBytes = TN * D * 2;    // one K or V tile
  static constexpr int kSubTile = TN * 128;        // one 64-column sub-tile of a K/V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQBytes;
  static constexpr int kOffV = kOffK + kStages * kTileBytes;
  static constexpr int kOffMask = kOffV + kStages * kTileBytes;  // 2 x TN floats
  static constexpr int kOffBar = kOffMask + 2 * TN * 4;
  static constexpr int kNumBars = 4 + 4 * kStages;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kBytes = kOffMisc + 16;
  static constexpr int kDynBytes = kBytes + 1024;
};

// One 32-column chunk of the second sweep: r holds raw accumulators of columns
// [cbase, cbase+32); produces 16 packed 16-bit pairs of exp2(t - m_ref) (dropout applied) and
// adds the undropped values to sum2.
template <bool BF16, bool KEYADD, bool DROP, bool BOUNDARY>
__device__ __forceinline__ void softmax_chunk(const uint32_t (&r)[32], int cbase, int n_cols, float sl2, float neg_m,
                                              const float* mask_stage, float2& sum2, uint32_t (&packed)[16],
                                              const uint32_t* keepw) {
  const float2 sl22 = make_float2(sl2, sl2);
  const float2 negm2 = make_float2(neg_m, neg_m);
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    float2 x = make_float2(__uint_as_float(r[2 * k]), __uint_as_float(r[2 * k + 1]));
    if constexpr (KEYADD) {
      const float2 mk = *reinterpret_cast<const float2*>(mask_stage + cbase + 2 * k);
      x = __fadd2_rn(__ffma2_rn(x, sl22, mk), negm2);
    } else {
      x = __ffma2_rn(x, sl22, negm2);
    }
    if constexpr (BOUNDARY) {
      if (cbase + 2 * k >= n_cols) x.x = -INFINITY;
      if (cbase + 2 * k + 1 >= n_cols) x.y = -INFINITY;
    }
    float2 p;
    p.x = fast_exp2(x.x);
    p.y = fast_exp2(x.y);
    sum2 = __fadd2_rn(sum2, p);
    packed[k] = pack2<BF16>(p.x, p.y);
  }
  if constexpr (DROP) {
    // keepw[i]: bit 7 of byte e = keep decision of column cbase + 4*i + e; the permutes replicate it over a 16-bit lane
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      packed[2 * i] &= prmt(keepw[i], 0u, 0x9988u);
      packed[2 * i + 1] &= prmt(keepw[i], 0u, 0xBBAAu);
    }
  }
}

}  // namespace

// PACKED: the batch is one [total_rows, H, D] tensor per operand with row offsets (FMHA_MASK_CU_SEQLENS); a
// template parameter so that the padded kernels carry none of its bookkeeping in registers.
template <int D, bool BF16, bool KEYADD, bool DROP, bool PACKED = false>
__global__ void __launch_bounds__(fast_threads<D>(), FastSmem<D, DROP>::kCtasPerSm) fmha_fwd_fast_kernel(const __grid_constant__ FwdArgs a) {
  griddep_wait();
  constexpr bool MERGED = (D == 64);          // one warp issues the loads and the MMAs
  constexpr int kMmaWarp = MERGED ? 0 : 1;    // it also owns the tensor-memory allocation
  constexpr int kFirstSoftmaxThread = MERGED ? 32 : 64;
  using L = FastSmem<D>;
  constexpr int ST = L::kStages;
  constexpr int TN = L::TN;
  constexpr int kTmemCols = (TN + D <= 128) ? 128 : 256;
  constexpr uint32_t kColS = 0, kColO = TN;
  constexpr int kFmt = BF16 ? 1 : 0;
  constexpr uint32_t kIdescQK = make_idesc_f16(128, TN, kFmt, false, false);
  constexpr uint32_t kIdescPV = make_idesc_f16(128, D, kFmt, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  float* sMask = reinterpret_cast<float*>(smem + L::kOffMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;
  uint64_t* s_full = bars + 1;
  uint64_t* p_full = bars + 2;
  uint64_t* o_full = bars + 3;
  uint64_t* k_full = bars + 4;
  uint64_t* k_empty = k_full + ST;
  uint64_t* v_full = k_empty + ST;
  uint64_t* v_empty = v_full + ST;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);
  // Philox offset of this launch: the launch parameter plus the optional device-resident value.  Kept in shared
  // memory and read where a draw starts, so that it holds no register in between.
  volatile uint32_t* philox_off = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int q0 = blockIdx.x * kTileM;
  const int bh = b * a.H + h;

  int k_limit = a.S_k;
  int q_limit = a.S_q;     // query rows [0, q_limit) of this (b, h) exist
  int row_base = 0;        // packed batch: first row of sequence b in the [total_rows, H, D] tensors
  int tb = b;              // batch coordinate of the tensor maps (0 for a packed batch)
  constexpr bool packed = PACKED;
  if (!packed && a.mask_kind == FMHA_MASK_SEQLEN) {
    const int len = reinterpret_cast<const int*>(a.mask)[b];
    if (len > 0 && len < a.S_k) k_limit = len;
  } else if (packed) {
    const int* cu = reinterpret_cast<const int*>(a.mask);
    row_base = cu[b];
    const int len = min(cu[b + 1] - row_base, a.S_q);   // a sequence longer than the stated maximum is cut there
    k_limit = len;
    q_limit = len;
    tb = 0;
    if (q0 >= len) return;   // this sequence has no such query tile (whole CTA, before any barrier)
  }
  const int n_kv = (k_limit + TN - 1) / TN;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *philox_off = a.philox_offset + (a.philox_offset_dev != nullptr ? static_cast<uint32_t>(*a.philox_offset_dev) : 0u);
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
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
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  const WaitCtx wctx{abort_flag, a.status};

  if (warp == 0 && !MERGED) {
    // ============================ TMA producer ======================================
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, L::kQBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_4d(sQ + c * 16384, &a.tm_q, q_full, c * 64, row_base + q0, h, tb);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % ST;
        if (j >= ST) mbar_wait(k_empty + s, ((j / ST) - 1) & 1, wctx, kFKEmpty);
        mbar_arrive_expect_tx(k_full + s, L::kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(sK + s * L::kTileBytes + c * L::kSubTile, &a.tm_k, k_full + s, c * 64, row_base + j * TN, h, tb);
        if (j >= ST) mbar_wait(v_empty + s, ((j / ST) - 1) & 1, wctx, kFVEmpty);
        mbar_arrive_expect_tx(v_full + s, L::kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(sV + s * L::kTileBytes + c * L::kSubTile, &a.tm_v, v_full + s, c * 64, row_base + j * TN, h, tb);
      }
    }
  } else if (warp == 0 && MERGED) {
    // ============================ TMA producer + MMA issuer in one warp (D = 64) =====
    // The warp runs convergently; one elected lane issues the loads, MMA bursts go out as in the split version.
    // Order per key step j: Q K^T(j); then, while the softmax warps work on S(j), wait for that MMA to complete
    // (a few hundred cycles) and refill what it and the previous P V have released: K of step j+ST and V of step
    // j-1+ST (the tensor core works in order, so P V(j-1), issued before Q K^T(j), has completed too); then wait
    // for P(j) and issue P V(j).  No refill ever stands between P V(j) and Q K^T(j+1), the chain the step time
    // hangs on.
    if constexpr (MERGED) {
      constexpr int KQ = D / 16;     // k-steps of S = Q K^T
      constexpr int KP = TN / 16;    // k-steps of O += P V
      static_assert(KQ == 4 && KP == 4, "merged warp: D = 64 with 64-key steps");
      const uint32_t tS = tmem_base + kColS;
      const uint32_t tO = tmem_base + kColO;
      auto load_k = [&](int j) {
        const int s = j % ST;
        mbar_arrive_expect_tx(k_full + s, L::kTileBytes);
        tma_load_4d(sK + s * L::kTileBytes, &a.tm_k, k_full + s, 0, row_base + j * TN, h, tb);
      };
      auto load_v = [&](int j) {
        const int s = j % ST;
        mbar_arrive_expect_tx(v_full + s, L::kTileBytes);
        tma_load_4d(sV + s * L::kTileBytes, &a.tm_v, v_full + s, 0, row_base + j * TN, h, tb);
      };
      if (elect_one()) {
        mbar_arrive_expect_tx(q_full, L::kQBytes);
        tma_load_4d(sQ, &a.tm_q, q_full, 0, row_base + q0, h, tb);
        for (int j = 0; j < ST && j < n_kv; ++j) {
          load_k(j);
          load_v(j);
        }
      }
      __syncwarp();
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      uint64_t aq[KQ];
#pragma unroll
      for (int kk = 0; kk < KQ; ++kk) aq[kk] = dq + kmajor_step(kk, 16384);
      mbar_wait(q_full, 0, wctx, kFQFull);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % ST;
        const uint32_t ph = (j / ST) & 1;
        const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + s * L::kTileBytes), 16, 1024);
        const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + s * L::kTileBytes), L::kSubTile, 1024);
        uint64_t bk[KQ], bv[KP];
#pragma unroll
        for (int kk = 0; kk < KQ; ++kk) bk[kk] = dk + kmajor_step(kk, L::kSubTile);
#pragma unroll
        for (int kk = 0; kk < KP; ++kk) bv[kk] = dv + mnmajor_step(kk);
        mbar_wait(k_full + s, ph, wctx, kFKFull);
        tc_fence_after_sync();
        umma_ss_x4(tS, aq, bk, kIdescQK, 0u);
        umma_commit_elect(k_empty + s);
        umma_commit_elect(s_full);
        // refills, under the softmax of this step
        const bool more_k = j + ST < n_kv, more_v = j >= 1 && j - 1 + ST < n_kv;
        if (more_k || more_v) {
          mbar_wait(k_empty + s, ph, wctx, kFKEmpty);       // Q K^T(j) has completed, and P V(j-1) before it
          if (more_v) mbar_wait(v_empty + ((j - 1) % ST), ((j - 1) / ST) & 1, wctx, kFVEmpty);
          if (elect_one()) {
            if (more_k) load_k(j + ST);
            if (more_v) load_v(j - 1 + ST);
          }
          __syncwarp();
        }
        mbar_wait(p_full, j & 1, wctx, kFPFull);
        mbar_wait(v_full + s, ph, wctx, kFVFull);
        tc_fence_after_sync();
        umma_ts_x4(tO, tS, 8u, bv, kIdescPV, (j > 0) ? 1u : 0u);
        umma_commit_elect(v_empty + s);
      }
      umma_commit_elect(o_full);
    }
  } else if (warp == 1 && !MERGED) {
    // ============================ MMA issuer ========================================
    // The warp runs the loop convergently and issues the MMAs in bursts from one elected lane
    // with descriptors prepared beforehand (see umma_ss_x4): a single lane that computes each
    // descriptor and then issues is starved of issue slots by the softmax warps.
    {
      constexpr int KQ = D / 16;     // k-steps of S = Q K^T
      constexpr int KP = TN / 16;    // k-steps of O += P V
      const uint32_t tS = tmem_base + kColS;
      const uint32_t tO = tmem_base + kColO;
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ), 16, 1024);
      uint64_t aq[KQ];
#pragma unroll
      for (int kk = 0; kk < KQ; ++kk) aq[kk] = dq + kmajor_step(kk, 16384);
      mbar_wait(q_full, 0, wctx, kFQFull);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % ST;
        const uint32_t ph = (j / ST) & 1;
        const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + s * L::kTileBytes), 16, 1024);
        const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + s * L::kTileBytes), L::kSubTile, 1024);
        uint64_t bk[KQ], bv[KP];
#pragma unroll
        for (int kk = 0; kk < KQ; ++kk) bk[kk] = dk + kmajor_step(kk, L::kSubTile);
#pragma unroll
        for (int kk = 0; kk < KP; ++kk) bv[kk] = dv + mnmajor_step(kk);
        mbar_wait(k_full + s, ph, wctx, kFKFull);
        tc_fence_after_sync();
        if constexpr (KQ == 4) umma_ss_x4(tS, aq, bk, kIdescQK, 0u);
        else umma_ss_x8(tS, aq, bk, kIdescQK, 0u);
        umma_commit_elect(k_empty + s);
        umma_commit_elect(s_full);
        mbar_wait(p_full, j & 1, wctx, kFPFull);
        mbar_wait(v_full + s, ph, wctx, kFVFull);
        tc_fence_after_sync();
        const uint32_t acc0 = (j > 0) ? 1u : 0u;
        {
          const uint64_t (&b0)[4] = *reinterpret_cast<const uint64_t (*)[4]>(&bv[0]);
          umma_ts_x4(tO, tS, 8u, b0, kIdescPV, acc0);
        }
        if constexpr (KP == 8) {
          const uint64_t (&b1)[4] = *reinterpret_cast<const uint64_t (*)[4]>(&bv[4]);
          umma_ts_x4(tO, tS + 32u, 8u, b1, kIdescPV, 1u);
        }
        umma_commit_elect(v_empty + s);
      }
      umma_commit_elect(o_full);
    }
  } else {
    // ============================ softmax / epilogue ================================
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int tid = threadIdx.x - kFirstSoftmaxThread;
    const int q_row = q0 + row;
    const bool row_ok = q_row < q_limit;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + kColS;
    const uint32_t tO = tmem_base + lane_addr + kColO;
    const float sl2 = a.scale_log2;
    const uint32_t gbh = static_cast<uint32_t>(a.philox_bh_offset + bh);

    float m_ref = -INFINITY;
    float2 sum2 = make_float2(0.f, 0.f);  // running sum of exp2(t - m_ref), two interleaved partial sums

    for (int j = 0; j < n_kv; ++j) {
      const int col0 = j * TN;
      const int n_cols = min(TN, k_limit - col0);
      const float* mask_stage = sMask + (j & 1) * TN;
      if constexpr (KEYADD) {
        const int c = col0 + tid;
        if (tid < TN)
          sMask[(j & 1) * TN + tid] =
              (c < a.S_k) ? reinterpret_cast<const float*>(a.mask)[static_cast<size_t>(b) * a.S_k + c] * kLog2eF : 0.f;
        named_bar_sync(1, 128);
      }
      // Keep decisions of this step's TN columns: Philox does not depend on the scores, so it runs
      // before they are awaited, while the tensor core is still busy with Q K^T.
      [[maybe_unused]] uint32_t keepw[DROP ? TN / 4 : 1];
      if constexpr (DROP) {
        const uint32_t kb0 = static_cast<uint32_t>(col0 / 16);
        const uint32_t poff = *philox_off;
#pragma unroll
        for (int d = 0; d < TN / 16; ++d) {
          const U4 draw = dropout_draw_keys(a.philox_keys, poff, gbh, static_cast<uint32_t>(q_row), kb0 + d);
          keepw[d * 4 + 0] = (draw.x & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
          keepw[d * 4 + 1] = (draw.y & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
          keepw[d * 4 + 2] = (draw.z & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
          keepw[d * 4 + 3] = (draw.w & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
        }
      }
      mbar_wait(s_full, j & 1, wctx, kFSFull, 32);
      tc_fence_after_sync();

      // ---- sweep 1: row maximum --------------------------------------------------------
      float tile_max = -INFINITY;
      {
        uint32_t sv[TN / 32][32];
#pragma unroll
        for (int c = 0; c < TN / 32; ++c) tmem_ld32(tS + c * 32, sv[c]);
#pragma unroll
        for (int c = 0; c < TN / 32; ++c) tmem_wait_ld_dep(sv[c]);
#pragma unroll
        for (int c = 0; c < TN / 32; ++c) {
          const int cbase = c * 32;
          float v[32];
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            v[k] = __uint_as_float(sv[c][k]);
            if constexpr (KEYADD) v[k] = fmaf(v[k], sl2, mask_stage[cbase + k]);
          }
          if (n_cols < TN) {
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (cbase + k >= n_cols) v[k] = -INFINITY;
          }
          float m0 = fmax3(v[0], v[1], v[2]);
          float m1 = fmax3(v[3], v[4], v[5]);
#pragma unroll
          for (int k = 6; k + 3 < 32; k += 4) {
            m0 = fmax3(m0, v[k], v[k + 1]);
            m1 = fmax3(m1, v[k + 2], v[k + 3]);
          }
          tile_max = fmax3(tile_max, fmax3(m0, m1, v[30]), v[31]);
        }
        if constexpr (!KEYADD) tile_max *= sl2;  // scale > 0: the maximum commutes with it
      }
      // ---- running reference maximum, lazy rescale of O ------------------------------------
      {
        float m_new = fmaxf(m_ref, tile_max);
        if (m_ref != -INFINITY && m_new - m_ref <= 8.0f) m_new = m_ref;  // exponentials stay below 2^8
        const bool moved = (m_new != m_ref) && (m_ref != -INFINITY);
        const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        if (j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + c * 32, r);
            tmem_wait_ld_dep(r);
#pragma unroll
            for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * alpha);
            tmem_st32(tO + c * 32, r);
          }
        }
        sum2.x *= alpha;
        sum2.y *= alpha;
        m_ref = m_new;
      }
      // ---- sweep 2: exponentials, dropout, P (next chunk's load in flight) ----------------------
      {
        const float neg_m = -m_ref;
        uint32_t ra[32], rb[32], packed[16];
        tmem_ld32(tS + 0, ra);
        auto run = [&](const uint32_t (&r)[32], int c) {
          if (n_cols >= TN)
            softmax_chunk<BF16, KEYADD, DROP, false>(r, c * 32, n_cols, sl2, neg_m, mask_stage, sum2, packed, keepw + (DROP ? c * 8 : 0));
          else
            softmax_chunk<BF16, KEYADD, DROP, true>(r, c * 32, n_cols, sl2, neg_m, mask_stage, sum2, packed, keepw + (DROP ? c * 8 : 0));
          tmem_st16(tS + c * 16, packed);
        };
#pragma unroll
        for (int c = 0; c < TN / 32; c += 2) {   // chunk c+1 (then c+2) is in flight while chunk c (c+1) is processed
          tmem_wait_ld_dep(ra);
          tmem_ld32(tS + (c + 1) * 32, rb);
          run(ra, c);
          tmem_wait_ld_dep(rb);
          if (c + 2 < TN / 32) tmem_ld32(tS + (c + 2) * 32, ra);
          run(rb, c + 1);
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(p_full);
    }

    // ---- epilogue ------------------------------------------------------------------------
    mbar_wait(o_full, 0, wctx, kFOFull, 32);
    tc_fence_after_sync();
    const float l_sum = sum2.x + sum2.y;
    const float out_scale = (DROP ? a.dropout_scale : 1.0f) / l_sum;
    if (a.lse != nullptr && row_ok) {
      const size_t li = packed ? static_cast<size_t>(h) * a.total_rows + row_base + q_row   // [H, total_rows]
                               : static_cast<size_t>(bh) * a.S_q + q_row;                   // [B*H, S_q]
      a.lse[li] = (m_ref + fast_log2(l_sum)) * kLn2F;
    }
    // A packed batch's last query tile of a sequence holds rows of the NEXT sequence past q_limit: its rows
    // are written one by one from registers instead of through the tile store.
    const bool partial_rows = packed && (q0 + kTileM > q_limit);
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + c * 32, r);
      tmem_wait_ld_dep(r);
      uint8_t* tile = sQ + (c / 2) * 16384;  // Q is no longer needed: every QK^T has completed
      unsigned short* grow = reinterpret_cast<unsigned short*>(a.o_ptr) + static_cast<int64_t>(row_base + q_row) * a.o_ss +
                             static_cast<int64_t>(h) * a.o_sh + c * 32;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 w;
        w.x = pack2<BF16>(__uint_as_float(r[q * 8 + 0]) * out_scale, __uint_as_float(r[q * 8 + 1]) * out_scale);
        w.y = pack2<BF16>(__uint_as_float(r[q * 8 + 2]) * out_scale, __uint_as_float(r[q * 8 + 3]) * out_scale);
        w.z = pack2<BF16>(__uint_as_float(r[q * 8 + 4]) * out_scale, __uint_as_float(r[q * 8 + 5]) * out_scale);
        w.w = pack2<BF16>(__uint_as_float(r[q * 8 + 6]) * out_scale, __uint_as_float(r[q * 8 + 7]) * out_scale);
        if (partial_rows) {
          if (row_ok) *reinterpret_cast<uint4*>(grow + q * 8) = w;
        } else {
          *reinterpret_cast<uint4*>(tile + sw128_offset(row, (c % 2) * 4 + q)) = w;
        }
      }
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (tid == 0) {
      if (*abort_flag == 0 && !partial_rows) {
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_store_4d(&a.tm_o, sQ + c * 16384, c * 64, row_base + q0, h, tb);
        tma_store_commit();
      }
      tma_store_wait_read();  // the shared-memory source must outlive the copy; the writes finish on their own
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 20; ++k) __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, bool BF16, bool KEYADD, bool DROP, bool PACKED = false>
static int launch_fast_impl(const FwdArgs& a, cudaStream_t stream) {
  using L = FastSmem<D>;
  auto kfn = fmha_fwd_fast_kernel<D, BF16, KEYADD, DROP, PACKED>;
  static std::atomic<bool> configured[64] = {};   // per device; set after the attribute call succeeded
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  dim3 grid((a.S_q + kTileM - 1) / kTileM, a.H, a.B);
  const cudaError_t e = launch_overlapped(kfn, grid, dim3(fast_threads<D>()), L::kDynBytes, stream, a);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_fwd_fast(const FwdArgs& a, int D, int dtype, cudaStream_t stream) {
  const bool bf = dtype == FMHA_DTYPE_BF16;
  const bool keyadd = a.mask_kind == FMHA_MASK_KEY_ADDITIVE;
  const bool drop = a.dropout_kind == FMHA_DROPOUT_PHILOX;
  if (a.mask_kind == FMHA_MASK_CU_SEQLENS) {
#define FMHA_FAST_PACKED(DD, BF, DR) \
  if (D == DD && bf == BF && drop == DR) return launch_fast_impl<DD, BF, false, DR, true>(a, stream);
    FMHA_FAST_PACKED(64, false, false)
    FMHA_FAST_PACKED(64, false, true)
    FMHA_FAST_PACKED(64, true, false)
    FMHA_FAST_PACKED(64, true, true)
    FMHA_FAST_PACKED(128, false, false)
    FMHA_FAST_PACKED(128, false, true)
    FMHA_FAST_PACKED(128, true, false)
    FMHA_FAST_PACKED(128, true, true)
#undef FMHA_FAST_PACKED
    return static_cast<int>(cudaErrorInvalidValue);
  }
#define FMHA_FAST_CASE(DD, BF, KA, DR) \
  if (D == DD && bf == BF && keyadd == KA && drop == DR) return launch_fast_impl<DD, BF, KA, DR>(a, stream);
  FMHA_FAST_CASE(64, false, false, false)
  FMHA_FAST_CASE(64, false, false, true)
  FMHA_FAST_CASE(64, false, true, false)
  FMHA_FAST_CASE(64, false, true, true)
  FMHA_FAST_CASE(64, true, false, false)
  FMHA_FAST_CASE(64, true, false, true)
  FMHA_FAST_CASE(64, true, true, false)
  FMHA_FAST_CASE(64, true, true, true)
  FMHA_FAST_CASE(128, false, false, false)
  FMHA_FAST_CASE(128, false, false, true)
  FMHA_FAST_CASE(128, false, true, false)
  FMHA_FAST_CASE(128, false, true, true)
  FMHA_FAST_CASE(128, true, false, false)
  FMHA_FAST_CASE(128, true, false, true)
  FMHA_FAST_CASE(128, true, true, false)
  FMHA_FAST_CASE(128, true, true, true)
#undef FMHA_FAST_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // namespace fmha
