// fmha_fwd_dense_sm100.cu — the forward kernel behind the reference's operators `fmha_nvfuser` and
// `fmha_train_nvfuser` (shmsong/NvFuserExamples fmha/fmha_manual.cpp:1218-1229) at head dimension 64: a dense
// [B*H, S_q, S_k] keep mask (1 = keep, converted as (1 - m) * -10000, fmha_manual.cpp:64-65) or additive mask
// (:463), and optionally a dense 0/1 dropout mask whose factor is applied once to O (:478-480).
//
// These operators move 1.5 to 2 times more mask bytes than Q, K, V and O together and do little arithmetic per
// byte: they are bound by HBM, and what the kernel has to do is keep loads in flight and keep the per-item chain of
// dependent phases short.  One persistent CTA per SM walks its share of the (head, 128-row query tile) items:
//   * a producer thread streams Q, K, V and the mask tiles through TMA, every operand in its own ring with its own
//     barriers, so that each load goes out as soon as ITS buffer is free and runs one to two key steps ahead;
//   * sixteen softmax warps (thread = query row x 32 key columns; the four parts of a row meet through shared
//     memory) do the exponentials; the dense masks reach them through shared memory, never by row-wise global
//     loads: a warp instruction that touches 32 different rows costs 32 cycles of the load/store unit, which
//     measured as 1.3 us per item when the dropout mask and O went that way;
//   * S and O are double-buffered in tensor memory: the tensor core forms the next S while the current one is
//     exponentiated (also across an item boundary), and an item's O is read out after the NEXT item's softmax,
//     when its last P V has long completed.
//
// Numerics as in the general kernel (fmha_fwd_sm100.cu) and the reference's fused definition
// (fmha_manual.cpp:60-97, 457-492): fp32 scores and row statistics, one rounding of P to 16 bits, the 0/1 dropout
// mask applied to the rounded P, fp32 accumulation of O, one rounding of O.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "../../include/fmha_sm100.h"
#include "fmha_device_utils.cuh"
#include "fmha_kernel_args.h"
#include "sm100_ptx.cuh"

namespace fmha {

namespace {

constexpr int kDnSoftmaxThreads = 512;              // 16 warps
constexpr int kDnThreads = 64 + kDnSoftmaxThreads + 32;  // + producer warp + MMA warp + store warp
constexpr float kDnLog2e = 1.4426950408889634f;
constexpr float kDnLn2 = 0.6931471805599453f;
constexpr uint32_t kDnSleepNs = 32;

enum DnWaitSite {
  kDQFull = 141, kDQEmpty = 142, kDStFull = 143, kDStEmpty = 144, kDSFull = 145, kDPFull = 146, kDPvDone = 147,
  kDOFull = 148, kDOFree = 149
};

// Shared memory of one CTA.  With a dropout mask every key step stages two 32 KB mask tiles, and Q, V and the output
// staging tile give up their second (third) buffer for it: their loads then start one step later, which the
// larger step (twice the mask bytes) covers.
template <bool DROPMASK>
struct DnSmem {
  static constexpr int kTile = kTileM * 64 * 2;          // a Q, K, V or O tile: 16 KB
  static constexpr int kMaskTile = kTileM * kTileN * 2;  // a mask tile: 32 KB (two swizzled 64-column halves)
  static constexpr int kQSlots = DROPMASK ? 1 : 2;
  static constexpr int kVSlots = DROPMASK ? 1 : 3;
  static constexpr int kOSlots = DROPMASK ? 1 : 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + kQSlots * kTile;  // [2] by key-step parity
  static constexpr int kOffV = kOffK + 2 * kTile;
  static constexpr int kOffM = kOffV + kVSlots * kTile;  // [2] by key-step parity
  static constexpr int kOffDM = kOffM + 2 * kMaskTile;   // [2] dropout mask tiles
  static constexpr int kOffO = kOffDM + (DROPMASK ? 2 * kMaskTile : 0);
  static constexpr int kOffX = kOffO + kOSlots * kTile;  // [2 slots][4 column quarters][128 rows] floats
  static constexpr int kOffBar = kOffX + 2 * 4 * kTileM * 4;
  static constexpr int kNumBars = 34;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kBytes = kOffMisc + 16;
  static constexpr int kDynBytes = kBytes + 1024;
  static_assert(kDynBytes <= 232448, "shared memory budget of one CTA exceeded");
};

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

template <bool BF16>
__device__ __forceinline__ uint32_t mul2_16bit(uint32_t a, uint32_t b) {
  if constexpr (BF16) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  } else {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

// The bounded wait, inlined: an out-of-line slow path would make the code a fifth smaller, but its call made the
// compiler spill loop-carried values to local memory, and each reload sat on the per-item critical path.
__device__ __forceinline__ bool dn_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where, uint32_t sleep_ns = 0) {
  return mbar_wait(bar, parity, ctx, where, sleep_ns);
}

}  // namespace

// KEEP: the dense mask is a keep mask (1 = keep), else additive.  DROPMASK: a dense 0/1 dropout mask is applied.
// SAVE (`fmha_train_saveim_nvfuser`, fmha_manual.cpp:1231-1238; one key step, i.e. S_k <= 128): the normalised softmax
// and softmax * mask * scale are also written as 16-bit [B*H, S_q, S_k] tensors, and the ROUNDED second tensor is what
// the second GEMM consumes (fmha_manual.cpp:891-897).  Both tiles are staged in the shared-memory slots their mask
// tiles came in (every thread overwrites exactly the 64 bytes it read) and leave through the store warp.
template <bool BF16, bool KEEP, bool DROPMASK, bool SAVE>
__global__ void __launch_bounds__(kDnThreads, 1) fmha_fwd_dense_kernel(const __grid_constant__ FwdArgs a) {
  static_assert(!SAVE || DROPMASK, "the save mode is the train operator's: it has a dropout mask");
  // The kernel is launched with programmatic stream serialization: everything up to the first access to global
  // memory (barrier set-up, tensor-memory allocation) may run while the previous kernel of the stream drains; each
  // thread calls griddep_wait() before its own first access.
  using L = DnSmem<DROPMASK>;
  constexpr int D = 64;
  constexpr int QS = L::kQSlots, VS = L::kVSlots, OS = L::kOSlots;
  constexpr int kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 2 * kTileN;   // S0 S1 | O0 O1
  constexpr int kFmt = BF16 ? 1 : 0;
  constexpr uint32_t kIdescQK = make_idesc_f16(128, kTileN, kFmt, false, false);
  constexpr uint32_t kIdescPV = make_idesc_f16(128, D, kFmt, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint8_t* sM = smem + L::kOffM;
  [[maybe_unused]] uint8_t* sDM = smem + L::kOffDM;
  uint8_t* sO = smem + L::kOffO;
  float* sX = reinterpret_cast<float*>(smem + L::kOffX);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars + 0;     // [QS] Q of an item has landed
  uint64_t* q_empty = bars + 2;    // [QS] ... and every Q K^T of the item has completed
  uint64_t* k_full = bars + 4;     // [2] K of a key step has landed
  uint64_t* k_empty = bars + 6;    // [2] ... and its Q K^T has completed
  uint64_t* m_full = bars + 8;     // [2] the mask tile(s) of a key step have landed
  uint64_t* m_empty = bars + 10;   // [2] ... and the 16 softmax warps have taken them into registers
  uint64_t* s_full = bars + 12;    // [2] S of a key step is in tensor memory
  uint64_t* p_full = bars + 14;    // [2] P of a key step is in tensor memory (over its S)
  uint64_t* pv_done = bars + 16;   // [2] O += P V of a key step has completed
  uint64_t* o_full = bars + 18;    // [2] the last P V of an item has completed
  uint64_t* o_free = bars + 20;    // [2] ... and O has been read out
  uint64_t* v_full = bars + 22;    // [VS] V of a key step has landed
  uint64_t* v_empty = bars + 25;   // [VS] ... and its P V has completed
  uint64_t* o_staged = bars + 28;  // [OS] the rounded O tile of an item is in its staging tile
  uint64_t* o_stage_free = bars + 30;  // [OS] ... and the TMA store has read it
  [[maybe_unused]] uint64_t* save_staged = bars + 32;  // [2] SAVE: the two saved tiles of a key step are in their mask slots
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_q = (a.S_q + kTileM - 1) / kTileM;
  const int n_kv = (a.S_k + kTileN - 1) / kTileN;
  const int num_items = n_q * a.H * a.B;   // item = (b*H + h) * n_q + q_tile; this CTA takes blockIdx.x, + gridDim.x, ...
  const WaitCtx wctx{abort_flag, a.status};

  // Loads of one item (Q) and of one key step (K, the mask tiles, V), by the producer thread.
  auto load_q = [&](int n, int q0, int h, int b) {
    const int qs = n % QS;
    if (n >= QS) dn_wait(q_empty + qs, ((n / QS) - 1) & 1, wctx, kDQEmpty);
    mbar_arrive_expect_tx(q_full + qs, L::kTile);
    tma_load_4d(sQ + qs * L::kTile, &a.tm_q, q_full + qs, 0, q0, h, b);
  };
  auto load_km = [&](int g, int j, int bh, int q0, int h, int b) {
    const int st = g & 1;
    if (g >= 2) dn_wait(k_empty + st, ((g >> 1) - 1) & 1, wctx, kDStEmpty);
    mbar_arrive_expect_tx(k_full + st, L::kTile);
    tma_load_4d(sK + st * L::kTile, &a.tm_k, k_full + st, 0, j * kTileN, h, b);
    // the mask tiles of this step: rows of this query tile, key columns [j*128, +128) in two 64-column boxes each
    if (g >= 2) dn_wait(m_empty + st, ((g >> 1) - 1) & 1, wctx, kDStEmpty);
    mbar_arrive_expect_tx(m_full + st, (DROPMASK ? 2 : 1) * L::kMaskTile);
    const int mrow = bh * a.S_q + q0;
#pragma unroll
    for (int c = 0; c < 2; ++c)
      tma_load_2d(sM + st * L::kMaskTile + c * 16384, &a.tm_mask, m_full + st, j * kTileN + c * 64, mrow);
    if constexpr (DROPMASK) {
#pragma unroll
      for (int c = 0; c < 2; ++c)
        tma_load_2d(sDM + st * L::kMaskTile + c * 16384, &a.tm_dmask, m_full + st, j * kTileN + c * 64, mrow);
    }
  };
  auto load_v = [&](int g, int j, int h, int b) {
    const int vs = g % VS;
    if (g >= VS) dn_wait(v_empty + vs, ((g / VS) - 1) & 1, wctx, kDStEmpty);
    mbar_arrive_expect_tx(v_full + vs, L::kTile);
    tma_load_4d(sV + vs * L::kTile, &a.tm_v, v_full + vs, 0, j * kTileN, h, b);
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(q_full + i, 1);
      mbar_init(q_empty + i, 1);
      mbar_init(k_full + i, 1);
      mbar_init(k_empty + i, 1);
      mbar_init(m_full + i, 1);
      mbar_init(m_empty + i, SAVE ? 1 : kDnSoftmaxThreads / 32);   // SAVE: released by the store warp
      mbar_init(save_staged + i, kDnSoftmaxThreads / 32);
      mbar_init(s_full + i, 1);
      mbar_init(p_full + i, kDnSoftmaxThreads);
      mbar_init(pv_done + i, 1);
      mbar_init(o_full + i, 1);
      mbar_init(o_free + i, kDnSoftmaxThreads);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(o_staged + i, kDnSoftmaxThreads / 32);
      mbar_init(o_stage_free + i, 1);
    }
    mbar_fence_init();
    griddep_wait();
    // The first item's loads go out at once: the rest of the set-up (tensor-memory allocation, the CTA-wide
    // synchronisation) runs under their latency.
    if (static_cast<int>(blockIdx.x) < num_items) {
      const int bh = blockIdx.x / n_q, q0 = (blockIdx.x % n_q) * kTileM;
      load_q(0, q0, bh % a.H, bh / a.H);
      load_km(0, 0, bh, q0, bh % a.H, bh / a.H);
      load_v(0, 0, bh % a.H, bh / a.H);
    }
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
  griddep_wait();

  if (warp == 0) {
    // ============================ TMA producer ======================================
    if (lane == 0) {
      // Order: K and the masks of step g, then V of step g-1.  V's buffer is the last of a step to come free (after
      // P V), and waiting for it first would hold back the K and mask loads of the next step, which can go earlier.
      int n = 0, g = 0;   // items and key steps loaded so far
      int pj = 0, ph = 0, pb = 0;   // the step whose V is still to be loaded
      for (int item = blockIdx.x; item < num_items && *abort_flag == 0; item += gridDim.x, ++n) {
        const int bh = item / n_q, q0 = (item % n_q) * kTileM;
        const int h = bh % a.H, b = bh / a.H;
        if (n > 0) load_q(n, q0, h, b);
        for (int j = 0; j < n_kv; ++j, ++g) {
          if (g > 0) {   // step 0 went out before the set-up
            load_km(g, j, bh, q0, h, b);
            if (g > 1) load_v(g - 1, pj, ph, pb);
          }
          pj = j; ph = h; pb = b;
        }
      }
      if (g > 1 && *abort_flag == 0) load_v(g - 1, pj, ph, pb);
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ========================================
    // Convergent warp, bursts from one elected lane (see umma_ss_x4).  S of key step g+1 is issued before O += P V
    // of step g, also across an item boundary, so the softmax warps find their next scores ready.
    const uint32_t tS = tmem_base + kColS, tO = tmem_base + kColO;
    auto issue_qk = [&](int g, int qs) {
      const int st = g & 1;
      dn_wait(k_full + st, (g >> 1) & 1, wctx, kDStFull);
      tc_fence_after_sync();
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ + qs * L::kTile), 16, 1024);
      const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + st * L::kTile), 16, 1024);
      uint64_t aq[4], bk[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        aq[kk] = dq + kmajor_step(kk, 16384);
        bk[kk] = dk + kmajor_step(kk, 16384);
      }
      umma_ss_x4(tS + st * kTileN, aq, bk, kIdescQK, 0u);
      umma_commit_elect(s_full + st);
      umma_commit_elect(k_empty + st);
    };
    const int my_items = (num_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    int g = 0;
    if (my_items > 0) {
      dn_wait(q_full + 0, 0, wctx, kDQFull);
      issue_qk(0, 0);
      if (n_kv == 1) umma_commit_elect(q_empty + 0);
    }
    for (int n = 0; n < my_items; ++n) {
      const int qs = n % QS, ob = n & 1;
      for (int j = 0; j < n_kv; ++j, ++g) {
        const int st = g & 1, vs = g % VS;
        // the next S: of this item's next step, or of the next item's first step
        if (j + 1 < n_kv) {
          issue_qk(g + 1, qs);
          if (j + 2 == n_kv) umma_commit_elect(q_empty + qs);
        } else if (n + 1 < my_items) {
          const int qn = (n + 1) % QS;
          dn_wait(q_full + qn, ((n + 1) / QS) & 1, wctx, kDQFull);
          issue_qk(g + 1, qn);
          if (n_kv == 1) umma_commit_elect(q_empty + qn);
        }
        // O of this item overwrites the accumulator the item before last used: its epilogue must have read it
        if (j == 0 && n >= 2) dn_wait(o_free + ob, ((n >> 1) - 1) & 1, wctx, kDOFree);
        dn_wait(v_full + vs, (g / VS) & 1, wctx, kDStFull);
        dn_wait(p_full + st, (g >> 1) & 1, wctx, kDPFull);
        tc_fence_after_sync();
        const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + vs * L::kTile), 16384, 1024);
        uint64_t b0[4], b1[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          b0[kk] = dv + mnmajor_step(kk);
          b1[kk] = dv + mnmajor_step(4 + kk);
        }
        const uint32_t tP = tS + st * kTileN;
        umma_ts_x4(tO + ob * D, tP, 8u, b0, kIdescPV, j > 0 ? 1u : 0u);
        umma_ts_x4(tO + ob * D, tP + 32u, 8u, b1, kIdescPV, 1u);
        umma_commit_elect(v_empty + vs);
        umma_commit_elect(pv_done + st);
        if (j == n_kv - 1) umma_commit_elect(o_full + ob);
      }
    }
  } else if (warp == 18) {
    // ============================ store warp =========================================
    // One thread: as each item's O tile is staged, hands it to TMA and releases the staging tile once it is read.
    if (lane == 0) {
      const int my_items = (num_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
      auto store_o = [&](int n) {   // O of this CTA's item number n
        const int os = n % OS;
        if (!dn_wait(o_staged + os, (n / OS) & 1, wctx, kDOFull, kDnSleepNs)) return;
        const int item = blockIdx.x + n * gridDim.x;
        const int bh = item / n_q, q0 = (item % n_q) * kTileM;
        tma_store_4d(&a.tm_o, sO + os * L::kTile, 0, q0, bh % a.H, bh / a.H);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(o_stage_free + os);
      };
      for (int n = 0; n < my_items && *abort_flag == 0; ++n) {
        if constexpr (SAVE) {
          // the saved tiles of item n are staged right after its softmax, O of item n-1 right after that
          const int st = n & 1;   // one key step per item
          if (!dn_wait(save_staged + st, (n >> 1) & 1, wctx, kDOFull, kDnSleepNs)) break;
          const int item = blockIdx.x + n * gridDim.x;
          const int bh = item / n_q, q0 = (item % n_q) * kTileM;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tma_store_3d(&a.tm_save_sm, sM + st * L::kMaskTile + c * 16384, c * 64, q0, bh);
            tma_store_3d(&a.tm_save_dr, sDM + st * L::kMaskTile + c * 16384, c * 64, q0, bh);
          }
          tma_store_commit();
          tma_store_wait_read();
          mbar_arrive(m_empty + st);   // the slots may take the masks of the step after next
          if (n > 0) store_o(n - 1);
        } else {
          store_o(n);
        }
      }
      if (SAVE && my_items > 0 && *abort_flag == 0) store_o(my_items - 1);
      tma_store_wait_read();   // the shared-memory sources must outlive the copies
    }
  } else {
    // ============================ softmax / epilogue: 16 warps ======================
    // warp (quad, cq) owns rows [32*quad, +32) (its tensor-memory lane quarter) and the 32 key columns [32*cq, +32)
    // of every 128-key step, and the 16 columns [16*cq, +16) of O.
    const int quad = warp & 3;
    const int cq = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float2 sc2 = make_float2(a.scale, a.scale);

    int g = 0;
    int n = 0;
    bool stop = false;   // "a wait of this CTA was given up": agreed on by all softmax threads at the end of each item
    // O of item number n_ep of this CTA (accumulator n_ep & 1): scale, round, stage in shared memory for the store
    // warp.  No CTA-wide barrier and no TMA instruction here: issuing a TMA store behind the producer's queued loads
    // took the issuing thread some 600 cycles, with every other softmax warp waiting for it at the next barrier.
    auto epilogue = [&](int n_ep, float out_scale) {
      const int ob = n_ep & 1;
      const int os = n_ep % OS;
      // both polls go out before either answer is looked at (each is a round trip of about a hundred cycles, and both
      // barriers have completed long ago as a rule)
      const bool o_ok = mbar_try_wait(o_full + ob, (n_ep >> 1) & 1);
      const bool st_ok = n_ep < OS || mbar_try_wait(o_stage_free + os, ((n_ep / OS) - 1) & 1);
      if (!o_ok) dn_wait(o_full + ob, (n_ep >> 1) & 1, wctx, kDOFull, kDnSleepNs);
      if (!st_ok) dn_wait(o_stage_free + os, ((n_ep / OS) - 1) & 1, wctx, kDOFree, kDnSleepNs);
      tc_fence_after_sync();
      uint32_t r[16];
      tmem_ld16(tmem_base + lane_addr + kColO + ob * D + cq * 16, r);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(o_free + ob);
      uint8_t* stage = sO + os * L::kTile;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint4 w;
        w.x = pack2<BF16>(__uint_as_float(r[q * 8 + 0]) * out_scale, __uint_as_float(r[q * 8 + 1]) * out_scale);
        w.y = pack2<BF16>(__uint_as_float(r[q * 8 + 2]) * out_scale, __uint_as_float(r[q * 8 + 3]) * out_scale);
        w.z = pack2<BF16>(__uint_as_float(r[q * 8 + 4]) * out_scale, __uint_as_float(r[q * 8 + 5]) * out_scale);
        w.w = pack2<BF16>(__uint_as_float(r[q * 8 + 6]) * out_scale, __uint_as_float(r[q * 8 + 7]) * out_scale);
        *reinterpret_cast<uint4*>(stage + sw128_offset(row, cq * 2 + q)) = w;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_staged + os);   // the store warp takes it from here
    };
    // (head, query tile) of the current item, advanced without divisions: the item number grows by gridDim.x
    int bh = blockIdx.x / n_q, qt = blockIdx.x % n_q;
    const int d_bh = gridDim.x / n_q, d_qt = gridDim.x % n_q;
    float pend_scale = 0.f;
    for (int item = blockIdx.x;; item += gridDim.x, ++n) {
      const bool have = item < num_items && !stop;   // the same for all softmax threads
      float out_scale_item = 0.f;
      const int q0 = qt * kTileM;
      if (have) {
        const int ob = n & 1;
        const int q_row = q0 + row;
        const bool row_ok = q_row < a.S_q;
        float m_ref = -INFINITY;
        float2 sum2 = make_float2(0.f, 0.f);
        [[maybe_unused]] float l_row = 1.0f;

        for (int j = 0; j < n_kv; ++j, ++g) {
          const int st = g & 1;
          const int col0 = j * kTileN + cq * 32;                 // first key column of this thread in this step
          const int n_cols = min(32, a.S_k - col0);              // valid ones among its 32 (may be <= 0)

          // S and the mask tile(s): both polls are issued before either answer is looked at, their latencies overlap.
          // (Nothing but straight-line code may stand between a tensor-memory load and its wait: the destination
          // registers are written until then, and a wait loop in between lets the compiler move them.)
          const bool s_ok = mbar_try_wait(s_full + st, (g >> 1) & 1);
          const bool m_ok = mbar_try_wait(m_full + st, (g >> 1) & 1);
          if (!s_ok) dn_wait(s_full + st, (g >> 1) & 1, wctx, kDSFull, kDnSleepNs);
          if (!m_ok) dn_wait(m_full + st, (g >> 1) & 1, wctx, kDStFull, kDnSleepNs);
          tc_fence_after_sync();
          uint32_t sv[32];
          tmem_ld32(tmem_base + lane_addr + kColS + st * kTileN + cq * 32, sv);
          tmem_wait_ld_dep(sv);
          // this row's 32 mask values: 64 bytes = four 16-byte chunks of one swizzled half tile; and
          // t = s * scale + additive mask (natural-log domain, two scores per packed instruction)
          {
            const uint32_t tile = smem_u32(sM + st * L::kMaskTile + (cq >> 1) * 16384);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 w = lds128(tile + sw128_offset(row, (cq & 1) * 4 + q));
              const uint32_t mw[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int k = q * 4 + e;
                float2 add = unpack2<BF16>(mw[e]);
                if constexpr (KEEP) {   // (1 - m) * -10000, the constants as immediates
                  add.x = fmaf(add.x, 10000.0f, -10000.0f);
                  add.y = fmaf(add.y, 10000.0f, -10000.0f);
                }
                const float2 t = __ffma2_rn(make_float2(__uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1])), sc2, add);
                sv[2 * k] = __float_as_uint(t.x);
                sv[2 * k + 1] = __float_as_uint(t.y);
              }
            }
          }
          if constexpr (!DROPMASK) {
            __syncwarp();
            if (lane == 0) mbar_arrive(m_empty + st);   // this warp has read its part of the mask tile
          }
          [[maybe_unused]] const uint32_t mtile = smem_u32(sM + st * L::kMaskTile + (cq >> 1) * 16384);
          if (n_cols < 32) {   // the same for the whole warp
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (k >= n_cols) sv[k] = __float_as_uint(-INFINITY);
          }
          float cmax = -INFINITY;
#pragma unroll
          for (int k = 0; k < 16; ++k) cmax = fmax3(cmax, __uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1]));
          // the row maximum over the four column quarters
          const int xs = (g + n) & 1;   // exchanges so far: one per key step and one per finished item
          sX[(xs * 4 + cq) * kTileM + row] = cmax;
          named_bar_sync(1, kDnSoftmaxThreads);   // also: every thread holds its scores, P may overwrite S
          const float* xr = sX + xs * 4 * kTileM + row;
          const float tile_max = fmaxf(fmaxf(xr[0], xr[kTileM]), fmaxf(xr[2 * kTileM], xr[3 * kTileM]));

          float m_new = fmaxf(m_ref, tile_max);
          if (m_ref != -INFINITY && m_new - m_ref <= 5.5f) m_new = m_ref;   // exponentials stay below e^5.5 < 2^8
          const bool moved = (m_new != m_ref) && (m_ref != -INFINITY);
          const float alpha = (m_ref == -INFINITY) ? 0.f : (moved ? fast_exp2((m_ref - m_new) * kDnLog2e) : 1.0f);
          if (j > 0 && __any_sync(0xffffffffu, moved)) {
            // rescale this thread's 16 columns of O; O += P V of the previous step must be complete
            dn_wait(pv_done + ((g - 1) & 1), ((g - 1) >> 1) & 1, wctx, kDPvDone, kDnSleepNs);
            tc_fence_after_sync();
            uint32_t r[16];
            tmem_ld16(tmem_base + lane_addr + kColO + ob * D + cq * 16, r);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 16; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * alpha);
            tmem_st16(tmem_base + lane_addr + kColO + ob * D + cq * 16, r);
          }
          sum2.x *= alpha;
          sum2.y *= alpha;
          m_ref = m_new;

          // the dropout mask of this thread's 32 scores, taken from its tile only now: sixteen registers less while the
          // scores and the padding mask are live (columns past the end of a mask row arrive as zeros, like P there)
          [[maybe_unused]] uint32_t dmw[DROPMASK ? 16 : 1];
          if constexpr (DROPMASK) {
            const uint32_t dtile = smem_u32(sDM + st * L::kMaskTile + (cq >> 1) * 16384);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 w = lds128(dtile + sw128_offset(row, (cq & 1) * 4 + q));
              dmw[q * 4 + 0] = w.x; dmw[q * 4 + 1] = w.y; dmw[q * 4 + 2] = w.z; dmw[q * 4 + 3] = w.w;
            }
            if constexpr (!SAVE) {
              __syncwarp();
              if (lane == 0) mbar_arrive(m_empty + st);   // this warp has read its part of both mask tiles
            }
          }
          uint32_t packed[16];
          const float2 negm2 = make_float2(-m_ref * kDnLog2e, -m_ref * kDnLog2e);
          const float2 l2e2 = make_float2(kDnLog2e, kDnLog2e);
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1])), l2e2, negm2);
            float2 p;
            p.x = fast_exp2(x.x);
            p.y = fast_exp2(x.y);
            sum2 = __fadd2_rn(sum2, p);
            if constexpr (SAVE) {
              sv[2 * k] = __float_as_uint(p.x);
              sv[2 * k + 1] = __float_as_uint(p.y);
            } else {
              packed[k] = pack2<BF16>(p.x, p.y);
              if constexpr (DROPMASK) packed[k] = mul2_16bit<BF16>(packed[k], dmw[k]);
            }
          }
          if constexpr (SAVE) {
            // One key step per item: the row sum is final.  Normalise, write the softmax tile and the dropout tile
            // (fp32 product, one rounding each, as fmha_manual.cpp:880-897) over the mask tiles, and hand the rounded
            // dropout tile to the second GEMM.
            const int xs2 = (g + n + 1) & 1;
            sX[(xs2 * 4 + cq) * kTileM + row] = sum2.x + sum2.y;
            stop = named_bar_or(1, kDnSoftmaxThreads, *abort_flag != 0);
            const float* xr2 = sX + xs2 * 4 * kTileM + row;
            l_row = (xr2[0] + xr2[kTileM]) + (xr2[2 * kTileM] + xr2[3 * kTileM]);
            const float inv_l = __fdividef(1.0f, l_row);
            const float2 il2 = make_float2(inv_l, inv_l);
            const float2 ds2 = make_float2(a.dropout_scale, a.dropout_scale);
            const uint32_t dtile = smem_u32(sDM + st * L::kMaskTile + (cq >> 1) * 16384);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t smw[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int k = q * 4 + e;
                const float2 sm = __fmul2_rn(make_float2(__uint_as_float(sv[2 * k]), __uint_as_float(sv[2 * k + 1])), il2);
                smw[e] = pack2<BF16>(sm.x, sm.y);
                const float2 dr = __fmul2_rn(sm, __fmul2_rn(unpack2<BF16>(dmw[k]), ds2));
                packed[k] = pack2<BF16>(dr.x, dr.y);
              }
              const uint32_t off = sw128_offset(row, (cq & 1) * 4 + q);
              sts128(mtile + off, smw[0], smw[1], smw[2], smw[3]);
              sts128(dtile + off, packed[q * 4 + 0], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(save_staged + st);
          }
          // P over S: 128 16-bit values in 64 columns; this thread's 32 values are columns [16*cq, +16)
          tmem_st16(tmem_base + lane_addr + kColS + st * kTileN + cq * 16, packed);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(p_full + st);
        }

        // ---- end of the item: row sum over the four quarters, logsumexp -----------------------------------------
        float l_sum;
        if constexpr (SAVE) {
          l_sum = l_row;              // exchanged inside the (only) key step; P is normalised already
          out_scale_item = 1.0f;
        } else {
          const int xs = (g + n) & 1;   // exchanges so far: one per key step and one per finished item
          sX[(xs * 4 + cq) * kTileM + row] = sum2.x + sum2.y;
          stop = named_bar_or(1, kDnSoftmaxThreads, *abort_flag != 0);
          const float* xr = sX + xs * 4 * kTileM + row;
          l_sum = (xr[0] + xr[kTileM]) + (xr[2 * kTileM] + xr[3 * kTileM]);
          out_scale_item = __fdividef(DROPMASK ? a.dropout_scale : 1.0f, l_sum);
        }
        if (cq == 0 && a.lse != nullptr && row_ok) a.lse[static_cast<size_t>(bh) * a.S_q + q_row] = m_ref + fast_log2(l_sum) * kDnLn2;
        bh += d_bh;
        qt += d_qt;
        if (qt >= n_q) { qt -= n_q; ++bh; }
      }
      // The read-out of an item's O waits for its last P V, which has only just been handed to the tensor core: it is
      // done after the softmax of the NEXT item (whose S is ready already), when that wait costs nothing.
      if (n > 0) epilogue(n - 1, pend_scale);
      if (!have) break;
      pend_scale = out_scale_item;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int k = 0; k < 20; ++k) __nanosleep(1000000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool BF16, bool KEEP, bool DROPMASK, bool SAVE>
static int launch_dense_impl(const FwdArgs& a, cudaStream_t stream) {
  auto kfn = fmha_fwd_dense_kernel<BF16, KEEP, DROPMASK, SAVE>;
  static std::atomic<bool> configured[64] = {};   // per device; set after the attribute call succeeded
  static std::atomic<int> sm_count[64] = {};
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, DnSmem<DROPMASK>::kDynBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev >= 0 && dev < 64) {
      sm_count[dev] = sms;
      configured[dev] = true;
    }
  } else {
    sms = sm_count[dev];
  }
  const int64_t items = static_cast<int64_t>((a.S_q + kTileM - 1) / kTileM) * a.H * a.B;
  const int grid = static_cast<int>(items < sms ? items : sms);   // one persistent CTA per SM
  const cudaError_t e = launch_overlapped(kfn, dim3(grid), dim3(kDnThreads), DnSmem<DROPMASK>::kDynBytes, stream, a);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// The dense-mask operators this kernel serves: head dimension 64, a dense keep or additive mask and (if any) a dense
// dropout mask that TMA can address (rows of 16-byte multiples), nothing saved.  Everything else stays with the
// general kernel.
bool fwd_dense_applies(const FwdArgs& a, int D) {
  const bool dense_mask = a.mask_kind == FMHA_MASK_DENSE_KEEP || a.mask_kind == FMHA_MASK_DENSE_ADDITIVE;
  const bool drop_dense = a.dropout_kind == FMHA_DROPOUT_DENSE && a.dmask_tiles > 0;
  if (D != 64 || !dense_mask || a.mask_tiles <= 0 || a.keep_mask_out != nullptr || a.debug_scores != nullptr) return false;
  if (a.save_softmax == nullptr && a.save_dropout == nullptr) return a.dropout_kind == FMHA_DROPOUT_NONE || drop_dense;
  // the save-intermediates operator: both tensors, an additive mask, a dropout mask, one key step
  return a.save_tiles > 0 && a.mask_kind == FMHA_MASK_DENSE_ADDITIVE && drop_dense && a.S_k <= kTileN;
}

int launch_fwd_dense(const FwdArgs& a, int dtype, cudaStream_t stream) {
  const bool bf = dtype == FMHA_DTYPE_BF16;
  const bool keep = a.mask_kind == FMHA_MASK_DENSE_KEEP;
  const bool dm = a.dropout_kind == FMHA_DROPOUT_DENSE;
  if (a.save_softmax != nullptr)
    return bf ? launch_dense_impl<true, false, true, true>(a, stream) : launch_dense_impl<false, false, true, true>(a, stream);
#define FMHA_DENSE_CASE(BF, KP, DM) \
  if (bf == BF && keep == KP && dm == DM) return launch_dense_impl<BF, KP, DM, false>(a, stream);
  FMHA_DENSE_CASE(false, false, false)
  FMHA_DENSE_CASE(false, false, true)
  FMHA_DENSE_CASE(false, true, false)
  FMHA_DENSE_CASE(false, true, true)
  FMHA_DENSE_CASE(true, false, false)
  FMHA_DENSE_CASE(true, false, true)
  FMHA_DENSE_CASE(true, true, false)
  FMHA_DENSE_CASE(true, true, true)
#undef FMHA_DENSE_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

}  // namespace fmha
