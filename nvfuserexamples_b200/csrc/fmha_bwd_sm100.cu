// fmha_bwd_sm100.cu — fused multi-head-attention backward for B200 (sm_100a).
//
// The reference project has no backward pass (shmsong/NvFuserExamples README.md:1); its
// provision for one is the pair of S x S tensors saved by FMHATrainKernelSaveIntermediate
// (fmha/fmha_manual.cpp:891-897).  This backward needs neither: it recomputes the
// probabilities from Q, K and the per-row logsumexp the forward kernel wrote.
//
// Three kernels per call:
//   1. bwd_prepare : delta[row] = sum_d dO[row,d] * O[row,d]  and zero the fp32 dQ accumulator
//   2. bwd_main    : persistent CTAs (one per SM) draw (128-key tile, head, batch) work items from a
//                    counter and loop over the 128-row query tiles of each
//                      S  = Q K^T            dP = dO V^T              (tcgen05.mma, fp32 in TMEM)
//                      P  = exp2(S*scale*log2e + mask - lse*log2e)   (16 warps, thread = row, a quarter of the columns)
//                      dS = P * (keep*c*dP - delta)                   c = 1/(1-p_drop)
//                      dV += (keep*P)^T dO     dK += dS^T Q     dQ_tile = dS K
//                    P and dS go through shared memory (16-bit, 128-byte swizzle) and are read
//                    by the tensor core both as K-major (dQ) and as MN-major (dV, dK) operands;
//                    dQ tiles are staged in shared memory and added to the fp32 accumulator by TMA
//                    reduce-add (cp.reduce.async.bulk.tensor ... .add);
//                    dK and dV leave through per-warp staging tiles and TMA stores when the next item is
//                    already under way.
//   3. bwd_finish  : dQ = (scale * accumulator) rounded to the 16-bit dtype
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include <cstring>
#include <type_traits>

#include "../../include/fmha_sm100.h"
#include "fmha_device_utils.cuh"
#include "fmha_kernel_args.h"
#include "philox.cuh"
#include "sm100_ptx.cuh"

namespace fmha {

namespace {

#ifndef FMHA_BWD_POLL_SLEEP_NS
#define FMHA_BWD_POLL_SLEEP_NS 48
#endif
constexpr uint32_t kComputeSleepNs = FMHA_BWD_POLL_SLEEP_NS;  // pause between barrier polls of the compute warps
constexpr int kComputeThreads = 512;               // 16 compute warps
constexpr int kBwdThreads = 64 + kComputeThreads;   // + producer warp + MMA warp
constexpr float kLog2eB = 1.4426950408889634f;

enum BwdWaitSite {
  kSiteKvFull = 201, kSiteQdoFull = 202, kSiteQdoEmpty = 203, kSiteSdpFull = 204, kSitePdsFull = 205,
  kSiteDqFull = 206, kSiteDqFree = 207, kSiteAccFull = 208, kSiteSdpFree = 209, kSiteKvEmpty = 210,
  kSiteItemFull = 211, kSiteItemEmpty = 212
};

template <int D>
struct BwdSmem {
  // D = 64: two K/V buffers (the next work item's K and V arrive while this one finishes) and two
  // Q/dO stages.  D = 128 fills shared memory with one of each.
  static constexpr int kKvBufs = (D == 64) ? 2 : 1;
  static constexpr int kStages = (D == 64) ? 2 : 1;   // Q / dO stages
  static constexpr int kPdsBufs = 1;                  // P / dS buffers
  // dQ tiles leave through shared memory + TMA reduce-add.  D = 64 has a dedicated 32 KB staging area
  // (2 KB per compute warp); at D = 128 the 64 KB fp32 tile is staged in the P/dS buffers (4 KB per
  // compute warp), which are idle between the completion of a tile's MMAs and the next tile's P/dS write.
  static constexpr bool kDqStageOwn = (D == 64);
  static constexpr int kTileBytes = kTileM * D * 2;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kOffK + kKvBufs * kTileBytes;
  static constexpr int kOffQ = kOffV + kKvBufs * kTileBytes;
  static constexpr int kOffdO = kOffQ + kStages * kTileBytes;
  static constexpr int kOffP = kOffdO + kStages * kTileBytes;
  static constexpr int kOffdS = kOffP + kPdsBufs * kTileM * kTileN * 2;
  static constexpr int kOffDQ = kOffdS + kPdsBufs * kTileM * kTileN * 2;    // fp32 staging of dQ
  static constexpr int kOffMask = kOffDQ + (kDqStageOwn ? kTileM * D * 4 : 0);   // 2 x 128 floats
  static constexpr int kOffBar = kOffMask + 2 * kTileN * 4;
  static constexpr int kNumBars = 6 + 2 * kKvBufs + 2 * kStages + 4;
  static constexpr int kOffMisc = kOffBar + kNumBars * 8;
  static constexpr int kBytes = kOffMisc + 32;
  static constexpr int kDynBytes = kBytes + 1024;
  static_assert(kDynBytes <= 232448, "shared memory budget of one CTA exceeded");
};

}  // namespace

// ---------------------------------------------------------------------------------------
// 1. delta and accumulator clearing
// ---------------------------------------------------------------------------------------
struct PrepArgs {
  const void* o;
  const void* d_o;
  int64_t o_sb, o_sh, o_ss, do_sb, do_sh, do_ss;
  int B, H, S_q, S_q_pad, D;
  float* delta;     // [B*H, S_q]
  float* dq_accum;  // [B*H, S_q_pad, D]
  int* work_counter;  // the main kernel's work-item counter, cleared here
  const int* cu_seqlens;  // packed batch: row offsets into the [total_rows, H, D] tensors (o_sb / do_sb unused), else null
};

template <bool BF16>
__global__ void __launch_bounds__(256) bwd_prepare_kernel(const PrepArgs a) {
  griddep_wait();
  // grid = (B*H, blocks of 32 rows); 8 threads per row (D = 64: 8 elements each; D = 128: 16 each).
  // The head index comes from the grid, so no thread divides 64-bit indices.
  const int per = a.D / 8;
  const int part = threadIdx.x & 7;
  const int bh = blockIdx.x;
  const int h = bh % a.H;
  const int b = bh / a.H;
  const int r = blockIdx.y * 32 + (threadIdx.x >> 3);
  const bool in_range = r < a.S_q_pad;  // no early exit: the shuffles below need every lane
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && a.work_counter != nullptr) *a.work_counter = 0;
  if (in_range) {
    float4* acc = reinterpret_cast<float4*>(a.dq_accum + (static_cast<int64_t>(bh) * a.S_q_pad + r) * a.D + part * per);
    for (int i = 0; i < per / 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // packed batch: row r of sequence b is row cu[b] + r of the tensors, and exists for r < cu[b+1] - cu[b]
  int64_t row_o = static_cast<int64_t>(b) * a.o_sb + static_cast<int64_t>(r) * a.o_ss;
  int64_t row_do = static_cast<int64_t>(b) * a.do_sb + static_cast<int64_t>(r) * a.do_ss;
  int q_limit = a.S_q;
  if (a.cu_seqlens != nullptr) {
    const int base = a.cu_seqlens[b];
    q_limit = min(a.cu_seqlens[b + 1] - base, a.S_q);   // rows past the stated maximum length take no part
    row_o = static_cast<int64_t>(base + r) * a.o_ss;
    row_do = static_cast<int64_t>(base + r) * a.do_ss;
  }
  float sum = 0.f;
  if (in_range && r < q_limit) {
    const unsigned short* po = reinterpret_cast<const unsigned short*>(a.o) + row_o + h * a.o_sh + part * per;
    const unsigned short* pd = reinterpret_cast<const unsigned short*>(a.d_o) + row_do + h * a.do_sh + part * per;
    for (int i = 0; i < per / 8; ++i) {
      const uint4 wo = __ldg(reinterpret_cast<const uint4*>(po) + i);
      const uint4 wd = __ldg(reinterpret_cast<const uint4*>(pd) + i);
      const uint32_t xo[4] = {wo.x, wo.y, wo.z, wo.w};
      const uint32_t xd[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        sum = fmaf(unpack_lo<BF16>(xo[k]), unpack_lo<BF16>(xd[k]), sum);
        sum = fmaf(unpack_hi<BF16>(xo[k]), unpack_hi<BF16>(xd[k]), sum);
      }
    }
  }
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  sum += __shfl_xor_sync(0xffffffffu, sum, 4);
  if (part == 0 && in_range && r < q_limit) a.delta[static_cast<int64_t>(bh) * a.S_q + r] = sum;
}

// ---------------------------------------------------------------------------------------
// 3. dQ = scale * accumulator
// ---------------------------------------------------------------------------------------
struct FinishArgs {
  const float* dq_accum;
  void* dq;
  int64_t sb, sh, ss;
  int B, H, S_q, S_q_pad, D;
  float scale;
  const int* cu_seqlens;  // packed batch: row offsets into the [total_rows, H, D] dQ (sb unused), else null
};

template <bool BF16>
__global__ void __launch_bounds__(256) bwd_finish_kernel(const FinishArgs a) {
  griddep_wait();
  // grid = (B*H, row blocks); one thread converts 8 consecutive elements, D/8 threads per row
  const int per_row = a.D / 8;
  const int part = threadIdx.x % per_row;
  const int r = blockIdx.y * (256 / per_row) + threadIdx.x / per_row;
  if (r >= a.S_q) return;
  const int bh = blockIdx.x;
  const int h = bh % a.H;
  const int b = bh / a.H;
  int64_t row_dq = static_cast<int64_t>(b) * a.sb + static_cast<int64_t>(r) * a.ss;
  if (a.cu_seqlens != nullptr) {
    const int base = a.cu_seqlens[b];
    if (r >= min(a.cu_seqlens[b + 1] - base, a.S_q)) return;   // rows past the stated maximum length take no part
    row_dq = static_cast<int64_t>(base + r) * a.ss;
  }
  const float4* src = reinterpret_cast<const float4*>(a.dq_accum + (static_cast<int64_t>(bh) * a.S_q_pad + r) * a.D + part * 8);
  const float4 x = src[0], y = src[1];
  uint4 w;
  w.x = pack2<BF16>(x.x * a.scale, x.y * a.scale);
  w.y = pack2<BF16>(x.z * a.scale, x.w * a.scale);
  w.z = pack2<BF16>(y.x * a.scale, y.y * a.scale);
  w.w = pack2<BF16>(y.z * a.scale, y.w * a.scale);
  unsigned short* dst = reinterpret_cast<unsigned short*>(a.dq) + row_dq + h * a.sh + part * 8;
  *reinterpret_cast<uint4*>(dst) = w;
}

// ---------------------------------------------------------------------------------------
// 2. main kernel
// ---------------------------------------------------------------------------------------
// Work.  An item is one (128-key tile, head, batch); kv tile is the fastest index.  One CTA per SM
// draws items from a global counter (the first item is blockIdx.x), so the fixed cost of an item --
// loading K and V, the first S/dP, the last tile's dV/dK/dQ, the dQ reduce and the dK/dV write-out --
// overlaps the neighbouring items instead of leaving the SM idle (it was ~30 % of a CTA's life when
// every item was its own CTA).  Items whose key tile lies wholly past the valid length write zeros.
//
// Schedule inside the stream of (item, query tile) pairs, numbered t = 0, 1, ...:
//   compute warps:  S,dP(t) -> registers, release the columns (sdp_free) -> P, dS in registers ->
//                   [first tile of an item: dK, dV of the previous item -> global memory] ->
//                   P,dS(t) -> shared memory (pds_full) -> dQ(t-1) -> staging -> TMA reduce-add
//   MMA warp:       S,dP(t+1) as soon as sdp_free(t), also across an item boundary (D = 64: the next
//                   item's K and V are already in the second buffer) -> dV,dK(t) -> dQ(t)
// At D = 128 shared and tensor memory are full: one K/V buffer, dQ shares the dP columns and is read
// out at the end of its own iteration, S/dP(t+1) follow dQ(t).
struct BwdItem {
  int id;      // < 0: no more work
  int b, h, bh, k0, n_cols;   // n_cols <= 0: key tile wholly masked out
  int n_q;     // query tiles of this item
  int q_limit; // query rows [0, q_limit) exist
  int row_base;  // packed batch: first row of the sequence in the [total_rows, H, D] tensors (else 0)
  int tb;        // batch coordinate of the tensor maps (0 for a packed batch)
};

// PACKED: FMHA_MASK_CU_SEQLENS; a template parameter so that the padded kernels carry none of its bookkeeping.
template <int D, bool BF16, bool KEYADD, bool DROP, bool PACKED = false>
__global__ void __launch_bounds__(kBwdThreads, 1) fmha_bwd_kernel(const __grid_constant__ BwdArgs a) {
  griddep_wait();
  using L = BwdSmem<D>;
  constexpr int ST = L::kStages;
  constexpr int KV = L::kKvBufs;
  constexpr bool OWNSTAGE = L::kDqStageOwn;
  constexpr bool EARLY = (D == 64);  // S/dP of the next tile are issued before dV/dK/dQ of this one
  constexpr int kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColdP = 128, kColdV = 256, kColdK = 256 + D;
  constexpr uint32_t kColdQ = (D == 64) ? 384 : kColdP;
  constexpr int kFmt = BF16 ? 1 : 0;
  constexpr uint32_t kIdescS = make_idesc_f16(128, 128, kFmt, false, false);
  constexpr uint32_t kIdescT = make_idesc_f16(128, D, kFmt, true, true);    // dV, dK: A and B MN-major
  constexpr uint32_t kIdescQ = make_idesc_f16(128, D, kFmt, false, true);   // dQ: A K-major, B MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::kOffK;
  uint8_t* sV = smem + L::kOffV;
  uint8_t* sQ = smem + L::kOffQ;
  uint8_t* sdO = smem + L::kOffdO;
  uint8_t* sP = smem + L::kOffP;
  uint8_t* sdS = smem + L::kOffdS;
  uint8_t* sDQ = OWNSTAGE ? smem + L::kOffDQ : smem + L::kOffP;   // fp32 dQ staging
  float* sMask = reinterpret_cast<float*>(smem + L::kOffMask);     // [2][128], by work-item parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* sdp_full = bars + 0;   // S and dP of a tile are in tensor memory
  uint64_t* sdp_free = bars + 1;   // ... and have been copied to registers (all compute threads arrive)
  uint64_t* pds_full = bars + 2;   // P and dS are in shared memory (all compute threads arrive)
  uint64_t* dq_full = bars + 3;    // dQ tile is in tensor memory; dV/dK/dQ of that tile are complete
  uint64_t* dq_free = bars + 4;    // dQ tile has been read out (all compute threads arrive)
  uint64_t* acc_full = bars + 5;   // dK / dV of a work item are complete
  uint64_t* kv_full = bars + 6;
  uint64_t* kv_empty = kv_full + KV;
  uint64_t* qdo_full = kv_empty + KV;
  uint64_t* qdo_empty = qdo_full + ST;
  uint64_t* item_full = qdo_empty + ST;   // [2] ring of work-item ids
  uint64_t* item_empty = item_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 4);
  volatile int* ring = reinterpret_cast<volatile int*>(smem + L::kOffMisc + 8);   // [2]
  // Philox offset of this launch (launch parameter + optional device-resident value), read where a draw starts
  volatile uint32_t* philox_off = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc + 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_tiles = (a.S_k + kTileN - 1) / kTileN;
  const int n_q_all = (a.S_q + kTileM - 1) / kTileM;
  const int num_items = kv_tiles * a.H * a.B;
  constexpr bool packed = PACKED;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *philox_off = a.philox_offset + (a.philox_offset_dev != nullptr ? static_cast<uint32_t>(*a.philox_offset_dev) : 0u);
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, kComputeThreads);
    mbar_init(pds_full, kComputeThreads);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, kComputeThreads);
    mbar_init(acc_full, 1);
    for (int s = 0; s < KV; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    for (int s = 0; s < ST; ++s) {
      mbar_init(qdo_full + s, 1);
      mbar_init(qdo_empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(item_full + s, 1);
      mbar_init(item_empty + s, 1 + kComputeThreads / 32);   // the MMA warp and every compute warp
    }
    mbar_fence_init();
    tma_prefetch_desc(&a.tm_q);
    tma_prefetch_desc(&a.tm_k);
    tma_prefetch_desc(&a.tm_v);
    tma_prefetch_desc(&a.tm_do);
    tma_prefetch_desc(&a.tm_dk);
    tma_prefetch_desc(&a.tm_dv);
    tma_prefetch_desc(&a.tm_dq);
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

  auto decode = [&](int id) {
    BwdItem it;
    it.id = id;
    it.b = it.h = it.bh = it.k0 = 0;
    it.n_cols = 0;
    it.n_q = n_q_all;
    it.q_limit = a.S_q;
    it.row_base = 0;
    it.tb = 0;
    if (id >= 0) {
      const int kv_tile = id % kv_tiles;
      it.bh = id / kv_tiles;
      it.h = it.bh % a.H;
      it.b = it.bh / a.H;
      it.tb = it.b;
      it.k0 = kv_tile * kTileN;
      int k_limit = a.S_k;
      if (!packed && a.mask_kind == FMHA_MASK_SEQLEN) {
        const int len = reinterpret_cast<const int*>(a.mask)[it.b];
        if (len > 0 && len < a.S_k) k_limit = len;
      } else if (packed) {
        const int* cu = reinterpret_cast<const int*>(a.mask);
        it.row_base = cu[it.b];
        // a sequence longer than the stated maximum is cut there: its tiles would otherwise run into the next
        // head's rows of the dQ accumulator and of delta
        const int len = min(cu[it.b + 1] - it.row_base, a.S_q);
        k_limit = len;
        it.q_limit = len;
        it.n_q = (len + kTileM - 1) / kTileM;
        it.tb = 0;
      }
      it.n_cols = min(kTileN, k_limit - it.k0);
    }
    return it;
  };
  // Consumer side of the work-item ring (whole warp): item number `n` of this CTA.
  auto fetch_item = [&](int n, uint32_t sleep_ns) {
    const int slot = n & 1;
    mbar_wait(item_full + slot, (n >> 1) & 1, wctx, kSiteItemFull, sleep_ns);
    int id = ring[slot];
    if (*abort_flag) id = -1;
    __syncwarp();
    if (lane == 0) mbar_arrive(item_empty + slot);
    return decode(id);
  };

  if (warp == 0) {
    // ============================ TMA producer ======================================
    if (lane == 0) {
      int w = 0, g = 0;   // work items with keys / query tiles loaded so far
      for (int n = 0;; ++n) {
        const int slot = n & 1;
        if (n >= 2) mbar_wait(item_empty + slot, ((n >> 1) - 1) & 1, wctx, kSiteItemEmpty);
        int id = (n == 0) ? static_cast<int>(blockIdx.x) : atomicAdd(a.work_counter, 1) + static_cast<int>(gridDim.x);
        if (id >= num_items || *abort_flag) id = -1;
        ring[slot] = id;
        mbar_arrive(item_full + slot);
        if (id < 0) break;
        const BwdItem it = decode(id);
        if (it.n_cols <= 0) continue;
        const int kvb = w % KV;
        if (w >= KV) mbar_wait(kv_empty + kvb, ((w / KV) - 1) & 1, wctx, kSiteKvEmpty);
        mbar_arrive_expect_tx(kv_full + kvb, 2 * L::kTileBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(sK + kvb * L::kTileBytes + c * 16384, &a.tm_k, kv_full + kvb, c * 64, it.row_base + it.k0, it.h, it.tb);
          tma_load_4d(sV + kvb * L::kTileBytes + c * 16384, &a.tm_v, kv_full + kvb, c * 64, it.row_base + it.k0, it.h, it.tb);
        }
        for (int i = 0; i < it.n_q; ++i, ++g) {
          const int s = g % ST;
          if (g >= ST) mbar_wait(qdo_empty + s, ((g / ST) - 1) & 1, wctx, kSiteQdoEmpty);
          mbar_arrive_expect_tx(qdo_full + s, 2 * L::kTileBytes);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            tma_load_4d(sQ + s * L::kTileBytes + c * 16384, &a.tm_q, qdo_full + s, c * 64, it.row_base + i * kTileM, it.h, it.tb);
            tma_load_4d(sdO + s * L::kTileBytes + c * 16384, &a.tm_do, qdo_full + s, c * 64, it.row_base + i * kTileM, it.h, it.tb);
          }
        }
        ++w;
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ========================================
    // The whole warp runs this loop convergently; the MMAs go out in bursts of 4 or 8 from one
    // elected lane with descriptors prepared beforehand as warp-uniform values (see umma_ss_x4).
    // A loop in which a single lane computes each descriptor and then issues was starved by the
    // compute warps' arithmetic: ~150 cycles per MMA during their exp/Philox phase, which put the
    // tensor core's work on the critical path of every tile.
    constexpr int KS = D / 16;      // k-steps of S and dP
    const uint32_t tS = tmem_base + kColS, tdP = tmem_base + kColdP, tdV = tmem_base + kColdV,
                   tdK = tmem_base + kColdK, tdQ = tmem_base + kColdQ;
    auto issue_s = [&](int stage, int kvb) {
      const uint64_t dq = make_smem_desc_sw128(smem_u32(sQ + stage * L::kTileBytes), 16, 1024);
      const uint64_t dk = make_smem_desc_sw128(smem_u32(sK + kvb * L::kTileBytes), 16, 1024);   // K as K-major B
      uint64_t aq[KS], bk[KS];
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        aq[kk] = dq + kmajor_step(kk, 16384);
        bk[kk] = dk + kmajor_step(kk, 16384);
      }
      if constexpr (KS == 4) umma_ss_x4(tS, aq, bk, kIdescS, 0u);
      else umma_ss_x8(tS, aq, bk, kIdescS, 0u);
    };
    auto issue_dp = [&](int stage, int kvb) {
      const uint64_t dd = make_smem_desc_sw128(smem_u32(sdO + stage * L::kTileBytes), 16, 1024);
      const uint64_t dv = make_smem_desc_sw128(smem_u32(sV + kvb * L::kTileBytes), 16, 1024);   // V as K-major B
      uint64_t ad[KS], bv[KS];
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        ad[kk] = dd + kmajor_step(kk, 16384);
        bv[kk] = dv + kmajor_step(kk, 16384);
      }
      if constexpr (KS == 4) umma_ss_x4(tdP, ad, bv, kIdescS, 0u);
      else umma_ss_x8(tdP, ad, bv, kIdescS, 0u);
      umma_commit_elect(sdp_full);
    };

    int n = 0, w = 0, t = 0;   // items fetched, items with work, query tiles so far
    bool ahead = false;         // S and dP of the current item's first tile were issued during the previous item
    BwdItem cur = fetch_item(n++, 0);
    while (cur.id >= 0) {
      if (cur.n_cols <= 0) {
        cur = fetch_item(n++, 0);
        continue;
      }
      const int kvb = w % KV;
      if (!ahead) {
        mbar_wait(kv_full + kvb, (w / KV) & 1, wctx, kSiteKvFull);
        if (t > 0) {
          mbar_wait(sdp_free, (t - 1) & 1, wctx, kSiteSdpFree);
          if constexpr (!EARLY) mbar_wait(dq_free, (t - 1) & 1, wctx, kSiteDqFree);   // dQ shares the dP columns
        }
        mbar_wait(qdo_full + (t % ST), (t / ST) & 1, wctx, kSiteQdoFull);
        tc_fence_after_sync();
        issue_s(t % ST, kvb);
        issue_dp(t % ST, kvb);
      }
      ahead = false;
      BwdItem nxt = cur;
      bool have_nxt = false;
      const uint64_t dK_m = make_smem_desc_sw128(smem_u32(sK + kvb * L::kTileBytes), 16384, 1024);   // K as MN-major B (dQ)
      const int n_q = cur.n_q;
      for (int i = 0; i < n_q; ++i, ++t) {
        const int s = t % ST;
        if constexpr (EARLY) {
          if (i + 1 < n_q) {
            mbar_wait(sdp_free, t & 1, wctx, kSiteSdpFree);
            mbar_wait(qdo_full + ((t + 1) % ST), ((t + 1) / ST) & 1, wctx, kSiteQdoFull);
            tc_fence_after_sync();
            issue_s((t + 1) % ST, kvb);
            issue_dp((t + 1) % ST, kvb);
          } else {
            // last tile of this item: look at the next item and start its first tile now
            nxt = fetch_item(n++, 0);
            have_nxt = true;
            if (nxt.id >= 0 && nxt.n_cols > 0) {
              const int nkvb = (w + 1) % KV;
              mbar_wait(kv_full + nkvb, ((w + 1) / KV) & 1, wctx, kSiteKvFull);
              mbar_wait(sdp_free, t & 1, wctx, kSiteSdpFree);
              mbar_wait(qdo_full + ((t + 1) % ST), ((t + 1) / ST) & 1, wctx, kSiteQdoFull);
              tc_fence_after_sync();
              issue_s((t + 1) % ST, nkvb);
              issue_dp((t + 1) % ST, nkvb);
              ahead = true;
            }
          }
        }
        // MN-major views of this tile's operands (16 rows = 2048 B per k-step, 64-wide halves 16 KB apart)
        const uint64_t dQ_m = make_smem_desc_sw128(smem_u32(sQ + s * L::kTileBytes), 16384, 1024);
        const uint64_t ddO_m = make_smem_desc_sw128(smem_u32(sdO + s * L::kTileBytes), 16384, 1024);
        const uint64_t dP_m = make_smem_desc_sw128(smem_u32(sP), 16384, 1024);
        const uint64_t ddS_m = make_smem_desc_sw128(smem_u32(sdS), 16384, 1024);
        const uint64_t ddS_k = make_smem_desc_sw128(smem_u32(sdS), 16, 1024);
        mbar_wait(pds_full, t & 1, wctx, kSitePdsFull);
        tc_fence_after_sync();
        // dV += P^T dO ; dK += dS^T Q : A is the [q x keys] tile read MN-major (keys contiguous),
        // 16 query rows (2048 B) per k-step, the two 64-key halves 16 KB apart.
        const uint32_t acc0 = (i > 0) ? 1u : 0u;
        {
          uint64_t x[8], y[8];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            x[kk] = dP_m + mnmajor_step(kk);
            y[kk] = ddO_m + mnmajor_step(kk);
          }
          umma_ss_x8(tdV, x, y, kIdescT, acc0);
        }
        {
          uint64_t x[8], y[8];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            x[kk] = ddS_m + mnmajor_step(kk);
            y[kk] = dQ_m + mnmajor_step(kk);
          }
          umma_ss_x8(tdK, x, y, kIdescT, acc0);
        }
        umma_commit_elect(qdo_empty + s);  // Q and dO of this stage are not read again (dQ needs dS and K only)
        if (i == n_q - 1) umma_commit_elect(acc_full);
        if (t > 0) {
          mbar_wait(dq_free, (t - 1) & 1, wctx, kSiteDqFree);
          tc_fence_after_sync();
        }
        // dQ tile = dS K : A K-major (keys along the row), B = K tile read MN-major
        {
          uint64_t x[8], y[8];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            x[kk] = ddS_k + kmajor_step(kk, 16384);
            y[kk] = dK_m + mnmajor_step(kk);
          }
          umma_ss_x8(tdQ, x, y, kIdescQ, 0u);
        }
        umma_commit_elect(dq_full);
        if (i == n_q - 1) umma_commit_elect(kv_empty + kvb);   // K and V of this item are not read again
        if constexpr (!EARLY) {
          if (i + 1 < n_q) {
            mbar_wait(qdo_full + ((t + 1) % ST), ((t + 1) / ST) & 1, wctx, kSiteQdoFull);
            tc_fence_after_sync();
            issue_s((t + 1) % ST, kvb);                          // S columns were released before pds_full(t)
            mbar_wait(dq_free, t & 1, wctx, kSiteDqFree);        // dQ shares the dP columns
            tc_fence_after_sync();
            issue_dp((t + 1) % ST, kvb);
          }
        }
      }
      ++w;
      cur = have_nxt ? nxt : fetch_item(n++, 0);
    }
  } else {
    // ============================ compute warps =====================================
    // 16 warps: warp (quad, cq) owns rows [32*quad, +32) (its tensor-memory lane quarter) and the
    // 32 columns [32*cq, +32) of every 128 x 128 tile.
    const int cw = warp - 2;             // 0..15
    const int quad = warp & 3;           // tensor-memory lane quarter of this warp
    const int cq = cw >> 2;              // which 32 columns of the tile
    const int row = quad * 32 + lane;
    const int tid = threadIdx.x - 64;    // 0..511
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = a.scale_log2;
    // With dropout dS is formed as keep*P*dP - P*delta/c and the factor c = 1/(1-p) moves into the
    // final scaling of dQ and dK (and of dV, whose P operand is unscaled as well).
    const float inv_c = DROP ? 1.0f / a.dropout_scale : 1.0f;
    const float dscale = DROP ? a.dropout_scale : 1.0f;
    const int cbase = cq * 32;           // first column of this thread within the tile
    constexpr int DQ = D / 4;            // columns of a [128 x D] accumulator handled by one thread

    // Every warp polls the mbarrier itself: funnelling the wait through one warp and a named barrier
    // was measured 8 % slower (it removes the skew between warps that lets their phases overlap).
    auto wait_all = [&](uint64_t* bar, uint32_t parity, int site) {
      mbar_wait(bar, parity, wctx, site, kComputeSleepNs);
      tc_fence_after_sync();
    };

    // D = 128: every warp stages its own 32 rows x 32 columns of dQ tile `tt` (4 KB, 128-byte swizzle)
    // in the idle P/dS buffers and its lane 0 issues one TMA reduce-add for it.  The additions are
    // performed line by line by the TMA unit instead of 2048 scattered 16-byte atomics per tile, which
    // occupied the compute warps for ~1500 cycles per tile, and no warp waits for another one here.
    auto dq_readout_tma = [&](int tt, int row0) {
      wait_all(dq_full, tt & 1, kSiteDqFull);
      uint32_t r[DQ];
#pragma unroll
      for (int c = 0; c < DQ / 16; ++c)
        tmem_ld16(tmem_base + lane_addr + kColdQ + cq * DQ + c * 16, *reinterpret_cast<uint32_t(*)[16]>(r + c * 16));
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(dq_free);                          // the dQ columns may be overwritten
      uint8_t* stage = sDQ + cw * 4096;
      const uint32_t rowaddr = smem_u32(stage) + lane * 128;
      const uint32_t sw = lane & 7;                  // 128-byte swizzle: 16-byte chunk ^= row mod 8
#pragma unroll
      for (int q = 0; q < DQ / 4; ++q)
        sts128(rowaddr + ((q ^ sw) << 4), r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && *abort_flag == 0) {
        tma_reduce_add_2d(&a.tm_dq, stage, cq * DQ, row0 + quad * 32);
        tma_store_commit();
      }
    };
    // D = 64: every warp stages its own 32 rows x 16 columns (2 KB, 64-byte swizzle) and its lane 0
    // issues the reduce, so the warps never wait for one another here.
    auto dq_readout_warp = [&](int tt, int row0) {
      wait_all(dq_full, tt & 1, kSiteDqFull);
      uint32_t t16[16];
      tmem_ld16(tmem_base + lane_addr + kColdQ + cq * 16, t16);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(dq_free);                          // the dQ columns may be overwritten
      if (lane == 0) tma_store_wait_read();          // this warp's previous reduce has read its staging tile
      __syncwarp();
      uint8_t* stage = sDQ + cw * 2048;
      const uint32_t rowaddr = smem_u32(stage) + lane * 64;
      const uint32_t sw = (lane >> 1) & 3;           // 64-byte swizzle: 16-byte chunk ^= bits 7..8 of the offset
#pragma unroll
      for (int q = 0; q < 4; ++q)
        sts128(rowaddr + ((q ^ sw) << 4), t16[q * 4], t16[q * 4 + 1], t16[q * 4 + 2], t16[q * 4 + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && *abort_flag == 0) {
        tma_reduce_add_2d(&a.tm_dq, stage, cq * 16, row0 + quad * 32);
        tma_store_commit();
      }
    };
    // dK and dV of a finished item: tensor memory -> registers -> this warp's staging tile -> two TMA
    // stores issued by its lane 0.  Warp (quad, cq) holds key rows [32*quad, +32) x columns [cq*DQ, +DQ)
    // of both accumulators: 32 rows of DQ*2 bytes each, dV first, dK behind it.  The staging tile is the
    // warp's dQ staging slot (D = 64) or its 4 KB share of the idle P/dS buffers (D = 128).  Rows past
    // S_k are clipped by the TMA unit.  The caller orders this against other users of the tile.
    constexpr int kDkvRowBytes = DQ * 2;
    auto store_dkdv = [&](int item_id, bool from_tmem) {
      const BwdItem it = decode(item_id);
      uint8_t* stage = OWNSTAGE ? sDQ + cw * 2048 : sP + cw * 4096;
      // Packed batch: a slice that reaches past the end of the sequence would overwrite the next sequence's
      // rows, so its rows are written one by one from registers.
      const int key = it.k0 + quad * 32 + lane;
      const bool edge = packed && (it.k0 + quad * 32 + 32 > it.q_limit);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const float mul = (which == 0) ? dscale : a.scale * dscale;
        const uint32_t rowaddr = smem_u32(stage) + which * 32 * kDkvRowBytes + lane * kDkvRowBytes;
        unsigned short* grow = reinterpret_cast<unsigned short*>(which == 0 ? a.dv_ptr : a.dk_ptr) +
                               static_cast<int64_t>(it.row_base + key) * (which == 0 ? a.dv_ss : a.dk_ss) +
                               static_cast<int64_t>(it.h) * (which == 0 ? a.dv_sh : a.dk_sh) + cq * DQ;
#pragma unroll
        for (int c = 0; c < DQ / 16; ++c) {
          uint32_t r[16];
          if (from_tmem) {
            tmem_ld16(tmem_base + lane_addr + (which == 0 ? kColdV : kColdK) + cq * DQ + c * 16, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) r[k] = 0u;
          }
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul);
            w.y = pack2<BF16>(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul);
            w.z = pack2<BF16>(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul);
            w.w = pack2<BF16>(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul);
            if (edge) {
              if (key < it.q_limit) *reinterpret_cast<uint4*>(grow + c * 16 + q * 8) = w;
            } else {
              sts128(rowaddr + c * 32 + q * 16, w.x, w.y, w.z, w.w);
            }
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && *abort_flag == 0 && !edge) {
        tma_store_4d(&a.tm_dv, stage, cq * DQ, it.row_base + it.k0 + quad * 32, it.h, it.tb);
        tma_store_4d(&a.tm_dk, stage + 32 * kDkvRowBytes, cq * DQ, it.row_base + it.k0 + quad * 32, it.h, it.tb);
        tma_store_commit();
      }
    };
    // Frees the warp's staging tile for store_dkdv / the next dQ tile (D = 64 only: at D = 128 the
    // tile lies in the P/dS buffers, whose users are ordered by the CTA-wide barrier 2).
    auto own_stage_free = [&]() {
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
    };

    int n = 0, w = 0, t = 0;      // items fetched, items with work, query tiles so far
    int prev_id = -1;             // >= 0: dK/dV of that item are still in tensor memory
    int prev_row0 = 0;            // accumulator row of the tile whose dQ is still in tensor memory (D = 64)

    while (true) {
      const BwdItem cur = fetch_item(n++, kComputeSleepNs);
      if (cur.id < 0) break;
      if (cur.n_cols <= 0) {
        if (packed) continue;   // a packed sequence has no rows past its length
        // key tile wholly past the valid length: its gradients are zero
        if constexpr (OWNSTAGE) {
          own_stage_free();
          store_dkdv(cur.id, false);
        } else {
          // the P/dS buffers may still be read by the previous tile's MMAs and dQ reduce
          if (t > 0) {
            if (lane == 0) tma_store_wait_read();
            named_bar_sync(2, kComputeThreads);
          }
          store_dkdv(cur.id, false);
          if (lane == 0) tma_store_wait_read();
          named_bar_sync(2, kComputeThreads);
        }
        continue;
      }
      const int k0 = cur.k0, n_cols = cur.n_cols, bh = cur.bh, n_q = cur.n_q, q_limit = cur.q_limit;
      const uint32_t gbh = static_cast<uint32_t>(a.philox_bh_offset + bh);
      // logsumexp rows: [B*H, S_q], or [H, total_rows] for a packed batch; delta is always [B*H, S_q]
      const int64_t lse_base = packed ? static_cast<int64_t>(cur.h) * a.total_rows + cur.row_base : static_cast<int64_t>(bh) * a.S_q;
      const int64_t delta_base = static_cast<int64_t>(bh) * a.S_q;
      const float* mask_row = sMask + (w & 1) * kTileN;
      if constexpr (KEYADD) {
        // both barriers are needed: a slower warp may still read the other item's values (first),
        // and every warp reads what the first four wrote (second)
        named_bar_sync(1, kComputeThreads);
        if (tid < kTileN) {
          const int c = k0 + tid;
          sMask[(w & 1) * kTileN + tid] =
              (c < a.S_k) ? reinterpret_cast<const float*>(a.mask)[static_cast<size_t>(cur.b) * a.S_k + c] * kLog2eB : 0.f;
        }
        named_bar_sync(1, kComputeThreads);
      }

      // Row statistics of the next tile are fetched one iteration ahead and kept RAW: any arithmetic
      // on the loaded value here would make the warp wait for the load at once (~1000 cycles per tile).
      float lse_next = INFINITY, delta_next = 0.f;
      if (row < q_limit) {
        lse_next = a.lse[lse_base + row];
        delta_next = a.delta[delta_base + row];
      }

      for (int i = 0; i < n_q; ++i, ++t) {
        const int q_row = i * kTileM + row;
        // lse in the log2 domain; +inf for rows past the end makes their probabilities zero
        const float neg_lse2 = -lse_next * kLog2eB;
        const float delta = delta_next * inv_c;
        {
          const int nr = q_row + kTileM;  // prefetch the statistics of the next tile's row
          const bool ok = (i + 1 < n_q) && nr < q_limit;
          lse_next = INFINITY;
          delta_next = 0.f;
          if (ok) {
            lse_next = a.lse[lse_base + nr];
            delta_next = a.delta[delta_base + nr];
          }
        }

        // keep decisions of the 32 columns: two Philox draws, computed together (their rounds
        // interleave) and before S and dP are needed
        [[maybe_unused]] uint32_t kw8[8];
        if constexpr (DROP) {
          const uint32_t poff = *philox_off;
#pragma unroll
          for (int d = 0; d < 2; ++d) {
            const U4 draw = dropout_draw_keys(a.philox_keys, poff, gbh, static_cast<uint32_t>(q_row),
                                         static_cast<uint32_t>((k0 + cbase) / 16 + d));
            kw8[d * 4 + 0] = (draw.x & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
            kw8[d * 4 + 1] = (draw.y & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
            kw8[d * 4 + 2] = (draw.z & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
            kw8[d * 4 + 3] = (draw.w & 0x7F7F7F7Fu) + (0x80u - a.philox_thr) * 0x01010101u;
          }
        }
        wait_all(sdp_full, t & 1, kSiteSdpFull);
        // The 32 columns are processed as two halves of 16: the second half of S and dP is fetched
        // from tensor memory only after the first has been turned into packed P and dS, which keeps
        // 32 fewer values live (the kernel is bound by the ALU pipe, and with all 64 values in
        // registers the compiler spilled and shuffled registers in this loop).
        uint32_t pk_p[16], pk_ds[16];  // 32 columns: 16 packed pairs each
        auto half_chunk = [&](auto edge_tag, auto half_tag, const uint32_t (&rs)[16], const uint32_t (&rp)[16]) {
          constexpr bool EDGE = decltype(edge_tag)::value;
          constexpr int HALF = decltype(half_tag)::value;
          const float2 sl22 = make_float2(sl2, sl2);
          const float2 nl2 = make_float2(neg_lse2, neg_lse2);
          const float2 nd2 = make_float2(-delta, -delta);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int col = cbase + HALF * 16 + 2 * k;       // column of the pair within the tile
            float2 x = make_float2(__uint_as_float(rs[2 * k]), __uint_as_float(rs[2 * k + 1]));
            if constexpr (KEYADD) {
              const float2 mk = *reinterpret_cast<const float2*>(mask_row + col);
              x = __fadd2_rn(__ffma2_rn(x, sl22, mk), nl2);
            } else {
              x = __ffma2_rn(x, sl22, nl2);
            }
            float2 p;
            p.x = fast_exp2(x.x);
            p.y = fast_exp2(x.y);
            if constexpr (EDGE) {                            // keys past the valid length / tensor edge
              if (col >= n_cols) p.x = 0.f;
              if (col + 1 >= n_cols) p.y = 0.f;
            }
            const float2 dp = make_float2(__uint_as_float(rp[2 * k]), __uint_as_float(rp[2 * k + 1]));
            float2 pkeep = p;
            if constexpr (DROP) {
              // bit 7 of byte e of the keep word decides element e; the permute smears it over 32 bits
              const uint32_t kw = kw8[HALF * 4 + (k >> 1)];
              const uint32_t m0 = prmt(kw, 0u, (k & 1) ? 0xAAAAu : 0x8888u);
              const uint32_t m1 = prmt(kw, 0u, (k & 1) ? 0xBBBBu : 0x9999u);
              pkeep.x = __uint_as_float(__float_as_uint(p.x) & m0);
              pkeep.y = __uint_as_float(__float_as_uint(p.y) & m1);
            }
            const float2 ds = __ffma2_rn(pkeep, dp, __fmul2_rn(p, nd2));
            pk_p[HALF * 8 + k] = pack2<BF16>(pkeep.x, pkeep.y);
            pk_ds[HALF * 8 + k] = pack2<BF16>(ds.x, ds.y);
          }
        };
        {
          uint32_t rs[16], rp[16];
          tmem_ld16(tmem_base + lane_addr + kColS + cbase, rs);
          tmem_ld16(tmem_base + lane_addr + kColdP + cbase, rp);
          tmem_wait_ld_dep16(rs, rp);
          if (n_cols >= kTileN) half_chunk(std::false_type{}, std::integral_constant<int, 0>{}, rs, rp);
          else half_chunk(std::true_type{}, std::integral_constant<int, 0>{}, rs, rp);
        }
        {
          uint32_t rs[16], rp[16];
          tmem_ld16(tmem_base + lane_addr + kColS + cbase + 16, rs);
          tmem_ld16(tmem_base + lane_addr + kColdP + cbase + 16, rp);
          tmem_wait_ld_dep16(rs, rp);
          tc_fence_before_sync();
          mbar_arrive(sdp_free);   // the tensor core may overwrite S and dP now
          if (n_cols >= kTileN) half_chunk(std::false_type{}, std::integral_constant<int, 1>{}, rs, rp);
          else half_chunk(std::true_type{}, std::integral_constant<int, 1>{}, rs, rp);
        }

        if constexpr (EARLY) {
          // dQ of the previous tile is complete <=> the MMAs which read the single P/dS buffer have
          // completed, so it can be overwritten below (the dQ tile itself is read out afterwards).
          if (t > 0) wait_all(dq_full, (t - 1) & 1, kSiteDqFull);
        } else {
          // D = 128: the previous tile's dQ was staged in the P/dS buffers; the reduce must have read them.
          if (t > 0) {
            if (lane == 0) tma_store_wait_read();
            named_bar_sync(2, kComputeThreads);
          }
        }
        if (i == 0 && prev_id >= 0) {
          // dK and dV of the previous item: complete since its last dV/dK MMAs, and they must be out
          // of tensor memory before this tile's P and dS let the tensor core overwrite them.
          wait_all(acc_full, (w - 1) & 1, kSiteAccFull);
          if constexpr (OWNSTAGE) {
            own_stage_free();
            store_dkdv(prev_id, true);
          } else {
            store_dkdv(prev_id, true);
            if (lane == 0) tma_store_wait_read();   // every warp's slice must be read before P and dS land there
            named_bar_sync(2, kComputeThreads);
          }
          tc_fence_before_sync();
          prev_id = -1;
        }
        {
          // columns [32*cq, +32) of row `row`: 64 bytes = 16-byte chunks (cq%2)*4 .. +3 of sub-tile cq/2
          const uint32_t bufP = smem_u32(sP + (cq >> 1) * 16384);
          const uint32_t bufS = smem_u32(sdS + (cq >> 1) * 16384);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t off = sw128_offset(row, (cq & 1) * 4 + q);
            sts128(bufP + off, pk_p[q * 4], pk_p[q * 4 + 1], pk_p[q * 4 + 2], pk_p[q * 4 + 3]);
            sts128(bufS + off, pk_ds[q * 4], pk_ds[q * 4 + 1], pk_ds[q * 4 + 2], pk_ds[q * 4 + 3]);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(pds_full);
        const int row0 = bh * a.S_q_pad + i * kTileM;
        if constexpr (EARLY) {
          if (t > 0) dq_readout_warp(t - 1, prev_row0);
          prev_row0 = row0;
        } else {
          dq_readout_tma(t, row0);   // D = 128: dQ shares columns with dP, it must be out before dP of tile t+1
        }
      }
      prev_id = cur.id;
      ++w;
    }
    // ---- drain: the last tile's dQ and the last item's dK, dV ------------------------------
    if constexpr (EARLY) {
      if (t > 0) dq_readout_warp(t - 1, prev_row0);
    }
    if (prev_id >= 0) {
      wait_all(acc_full, (w - 1) & 1, kSiteAccFull);
      if constexpr (OWNSTAGE) {
        own_stage_free();
      } else {
        if (lane == 0) tma_store_wait_read();  // the last dQ reduces have read the P/dS buffers
        named_bar_sync(2, kComputeThreads);
      }
      store_dkdv(prev_id, true);
    }
    if (lane == 0) tma_store_wait_read();   // shared memory stays valid until the TMA unit has read it
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

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
template <int D, bool BF16, bool KEYADD, bool DROP, bool PACKED = false>
static int launch_bwd_impl(const BwdArgs& a, cudaStream_t stream) {
  using L = BwdSmem<D>;
  auto kfn = fmha_bwd_kernel<D, BF16, KEYADD, DROP, PACKED>;
  static std::atomic<bool> configured[64] = {};   // per device; set after the attribute call succeeded
  static std::atomic<int> sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = 0;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes);
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
  const int64_t items = static_cast<int64_t>((a.S_k + kTileN - 1) / kTileN) * a.H * a.B;
  const int grid = static_cast<int>(items < sms ? items : sms);   // one persistent CTA per SM
  const cudaError_t e = launch_overlapped(kfn, dim3(grid), dim3(kBwdThreads), L::kDynBytes, stream, a);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_bwd(const BwdArgs& a, int D, int dtype, cudaStream_t stream) {
  const bool bf = dtype == FMHA_DTYPE_BF16;
  const bool keyadd = a.mask_kind == FMHA_MASK_KEY_ADDITIVE;
  const bool drop = a.dropout_kind == FMHA_DROPOUT_PHILOX;
  if (a.mask_kind == FMHA_MASK_CU_SEQLENS) {
#define FMHA_BWD_PACKED(DD, BF, DR) \
  if (D == DD && bf == BF && drop == DR) return launch_bwd_impl<DD, BF, false, DR, true>(a, stream);
    FMHA_BWD_PACKED(64, false, false)
    FMHA_BWD_PACKED(64, false, true)
    FMHA_BWD_PACKED(64, true, false)
    FMHA_BWD_PACKED(64, true, true)
    FMHA_BWD_PACKED(128, false, false)
    FMHA_BWD_PACKED(128, false, true)
    FMHA_BWD_PACKED(128, true, false)
    FMHA_BWD_PACKED(128, true, true)
#undef FMHA_BWD_PACKED
    return static_cast<int>(cudaErrorInvalidValue);
  }
#define FMHA_BWD_CASE(DD, BF, KA, DR) \
  if (D == DD && bf == BF && keyadd == KA && drop == DR) return launch_bwd_impl<DD, BF, KA, DR>(a, stream);
  FMHA_BWD_CASE(64, false, false, false)
  FMHA_BWD_CASE(64, false, false, true)
  FMHA_BWD_CASE(64, false, true, false)
  FMHA_BWD_CASE(64, false, true, true)
  FMHA_BWD_CASE(64, true, false, false)
  FMHA_BWD_CASE(64, true, false, true)
  FMHA_BWD_CASE(64, true, true, false)
  FMHA_BWD_CASE(64, true, true, true)
  FMHA_BWD_CASE(128, false, false, false)
  FMHA_BWD_CASE(128, false, false, true)
  FMHA_BWD_CASE(128, false, true, false)
  FMHA_BWD_CASE(128, false, true, true)
  FMHA_BWD_CASE(128, true, false, false)
  FMHA_BWD_CASE(128, true, false, true)
  FMHA_BWD_CASE(128, true, true, false)
  FMHA_BWD_CASE(128, true, true, true)
#undef FMHA_BWD_CASE
  return static_cast<int>(cudaErrorInvalidValue);
}

int launch_bwd_prepare(const void* o, const fmha_tensor4& ot, const fmha_tensor4& dot, int B, int H, int S_q, int S_q_pad,
                       int D, int dtype, float* delta, float* dq_accum, int* work_counter, const int* cu_seqlens, cudaStream_t stream) {
  PrepArgs p;
  p.o = ot.ptr; p.d_o = dot.ptr;
  (void)o;
  p.o_sb = ot.stride_b; p.o_sh = ot.stride_h; p.o_ss = ot.stride_s;
  p.do_sb = dot.stride_b; p.do_sh = dot.stride_h; p.do_ss = dot.stride_s;
  p.B = B; p.H = H; p.S_q = S_q; p.S_q_pad = S_q_pad; p.D = D;
  p.delta = delta; p.dq_accum = dq_accum; p.work_counter = work_counter; p.cu_seqlens = cu_seqlens;
  const dim3 grid(static_cast<unsigned>(B) * H, static_cast<unsigned>((S_q_pad + 31) / 32));
  const cudaError_t e = launch_overlapped(dtype == FMHA_DTYPE_BF16 ? bwd_prepare_kernel<true> : bwd_prepare_kernel<false>, grid,
                                          dim3(256), 0, stream, p);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_bwd_finish(const float* dq_accum, const fmha_tensor4& dq, int B, int H, int S_q, int S_q_pad, int D, int dtype,
                      float scale, const int* cu_seqlens, cudaStream_t stream) {
  FinishArgs f;
  f.dq_accum = dq_accum; f.dq = dq.ptr;
  f.sb = dq.stride_b; f.sh = dq.stride_h; f.ss = dq.stride_s;
  f.B = B; f.H = H; f.S_q = S_q; f.S_q_pad = S_q_pad; f.D = D; f.scale = scale; f.cu_seqlens = cu_seqlens;
  const int rows_per_block = 256 / (D / 8);
  const dim3 grid(static_cast<unsigned>(B) * H, static_cast<unsigned>((S_q + rows_per_block - 1) / rows_per_block));
  const cudaError_t e = launch_overlapped(dtype == FMHA_DTYPE_BF16 ? bwd_finish_kernel<true> : bwd_finish_kernel<false>, grid,
                                          dim3(256), 0, stream, f);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace fmha
