// sm100_ptx.cuh — thin inline-PTX wrappers for the Blackwell (sm_100a) features the
// attention kernels are built from: mbarrier, TMA (cp.async.bulk.tensor), tensor memory
// (tcgen05.alloc/ld/st) and the 5th-generation tensor core (tcgen05.mma / commit).
//
// Every wait in here is bounded: after `kWaitLimitNs` of wall time a waiter records an
// error code in the kernel's status block, raises the CTA-wide abort flag and returns, so
// a broken pipeline ends as an error status instead of a hung GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmha {

// ------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint: the thread may sleep in hardware up to `hint_ns` before the
// instruction returns, which keeps waiting warps out of the issue slots of working ones.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Wall-time limit of one wait.  Legitimate waits inside a CTA last microseconds.
constexpr uint64_t kWaitLimitNs = 400ull * 1000ull * 1000ull;

// Block of state every bounded wait needs: the CTA's abort flag (shared memory) and the
// kernel's status words (global memory, may be null).
struct WaitCtx {
  volatile int* abort_flag;  // shared
  int* status;               // global int32[4] or nullptr
};

// Waits for `parity` of `bar`.  Returns false if the wait was given up (either because
// this wait ran out of time, or because another thread of the CTA already did).
// `sleep_ns` > 0 makes the waiter sleep between polls: for the many compute threads, whose polling
// would otherwise take issue slots from the warps that are still working.  The single MMA and
// TMA threads poll without sleeping (their wake-up latency is on the critical path).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where,
                                          uint32_t sleep_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*ctx.abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitNs) {
        *ctx.abort_flag = 1;
        if (ctx.status) {
          atomicCAS(ctx.status, 0, where);          // first failing site
          atomicAdd(ctx.status + 1, 1);              // how many waiters gave up
          ctx.status[2] = static_cast<int>(blockIdx.x);
          ctx.status[3] = static_cast<int>(blockIdx.y);
        }
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// proxies and fences
// ------------------------------------------------------------------------------------
// Generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Barrier that also ORs a predicate over its participants: every one of them gets the same answer, which a
// flag read by each thread on its own cannot promise (used for "has any wait of this CTA been given up?",
// where threads that disagree would leave each other alone at the next barrier).
__device__ __forceinline__ bool named_bar_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %3, 0;\n\t"
      "bar.red.or.pred q, %1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

// ------------------------------------------------------------------------------------
// TMA: 4-D tiled loads and stores. coordinates are (c0 innermost .. c3 outermost)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const void* tmap, const void* smem_src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* smem_src, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Bulk reduction shared -> global: every element of the 2-D box is ADDED to the tensor in global
// memory by the TMA unit (asynchronous, tracked by the same bulk groups as stores).
__device__ __forceinline__ void tma_reduce_add_2d(const void* tmap, const void* smem_src, int c0, int c1) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
      : "memory");
}
// First statement of every kernel that is launched with programmatic stream serialization (see
// launch_overlapped): returns once the preceding kernels of the stream have completed and their
// writes are visible.  A no-op for a launch without that attribute.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// (An explicit griddepcontrol.launch_dependents at the top of the kernels was measured 2 % slower: the next
// grid's CTAs then take multiprocessors while this grid's last wave still needs them.)
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the shared-memory source of every committed store has been read.
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Waits until every committed store is complete (writes visible).
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------------------------
// tensor memory allocation (one full warp executes these)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ------------------------------------------------------------------------------------
// tcgen05.mma descriptors
// ------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  `lbo`/`sbo` in bytes.
//   K-major operand  (rows of 64 16-bit elements = 128 B): sbo = 1024 (8 rows), lbo unused (1).
//   MN-major operand (rows of 64 MN elements, one row per k): sbo = 1024 (8 k rows),
//                     lbo = distance between 64-element MN chunks.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of sm_100
  d |= 2ull << 61;  // layout type: 128-byte swizzle
  return d;
}

// Instruction descriptor of kind::f16 with fp32 accumulation.
//   fmt: 0 = fp16 operands, 1 = bf16 operands;  *_mn_major: operand is MN-major in smem.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, int fmt, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) |                                  // accumulator format: f32
         (static_cast<uint32_t>(fmt) << 7) |          // A format
         (static_cast<uint32_t>(fmt) << 10) |         // B format
         ((a_mn_major ? 1u : 0u) << 15) |             // A major
         ((b_mn_major ? 1u : 0u) << 16) |             // B major
         (static_cast<uint32_t>(n >> 3) << 17) |      // N / 8
         (static_cast<uint32_t>(m >> 4) << 24);       // M / 16
}

// D[tmem] (+)= A[smem] * B[smem].  One thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem].
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The issuing thread is a single lane, so every instruction between two tcgen05.mma counts
// (a 128x64x16 MMA occupies the tensor core for only ~48 cycles).  These variants take the
// descriptor as (low word, high word): the caller builds the descriptor of a tile once and per
// k-step only adds a constant to the low word (the 16-byte-unit start address lives in its low
// 14 bits and a tile never crosses the 256 KB field).
struct DescWords {
  uint32_t lo, hi;
};
__device__ __forceinline__ DescWords desc_words(uint64_t d) {
  DescWords w;
  w.lo = static_cast<uint32_t>(d);
  w.hi = static_cast<uint32_t>(d >> 32);
  return w;
}
__device__ __forceinline__ void umma_ss_w(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- burst issue from a converged warp ---------------------------------------------------
// The warp scheduler gives a warp whose next instruction is not ready no slot, and a warp that
// competes with arithmetic-heavy warps waits tens of cycles for each slot it asks for.  An MMA loop
// written as "one lane computes a descriptor, then issues" therefore degrades from ~50 to ~150
// cycles per MMA next to busy softmax warps (measured: 147 cycles against a backward-like
// instruction mix, 1600 against pure Philox).  These helpers are executed by ALL 32 lanes of a
// converged warp: the descriptors are warp-uniform values prepared beforehand, one lane is elected
// inside the block and the MMAs follow each other without branches or dependent arithmetic
// (measured under the same load: 62 cycles per MMA).
//   acc_first: accumulate flag of the first MMA; the others always accumulate.
__device__ __forceinline__ void umma_ss_x4(uint32_t d_tmem, const uint64_t (&a)[4], const uint64_t (&b)[4], uint32_t idesc,
                                           uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q, pe;\n\t"
      "setp.ne.b32 p, %10, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %9, p;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %4, %9, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %9, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %9, q;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a[0]), "l"(b[0]), "l"(a[1]), "l"(b[1]), "l"(a[2]), "l"(b[2]), "l"(a[3]), "l"(b[3]), "r"(idesc),
        "r"(acc_first)
      : "memory");
}
__device__ __forceinline__ void umma_ss_x8(uint32_t d_tmem, const uint64_t (&a)[8], const uint64_t (&b)[8], uint32_t idesc,
                                           uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q, pe;\n\t"
      "setp.ne.b32 p, %18, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %17, p;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %4, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %10, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %11, %12, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %13, %14, %17, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %15, %16, %17, q;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a[0]), "l"(b[0]), "l"(a[1]), "l"(b[1]), "l"(a[2]), "l"(b[2]), "l"(a[3]), "l"(b[3]), "l"(a[4]), "l"(b[4]),
        "l"(a[5]), "l"(b[5]), "l"(a[6]), "l"(b[6]), "l"(a[7]), "l"(b[7]), "r"(idesc), "r"(acc_first)
      : "memory");
}
// A from tensor memory: a_tmem + k * a_step is the A address of MMA k.
__device__ __forceinline__ void umma_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t a_step, const uint64_t (&b)[4],
                                           uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q, pe;\n\t"
      ".reg .b32 a1, a2, a3;\n\t"
      "setp.ne.b32 p, %8, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "add.u32 a1, %1, %2;\n\t"
      "add.u32 a2, a1, %2;\n\t"
      "add.u32 a3, a2, %2;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %3, %7, p;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %4, %7, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %5, %7, q;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %6, %7, q;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(a_step), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "r"(idesc), "r"(acc_first)
      : "memory");
}
// tcgen05.commit by the elected lane of a converged warp.  elect.sync picks the same lane every
// time for a full mask, so the commit tracks the MMAs issued by the helpers above.
__device__ __forceinline__ void umma_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n"
      ::"r"(smem_u32(bar))
      : "memory");
}

// Low-word increments: k-step kk of a K-major operand (16 elements = 32 bytes, 64-column
// sub-tiles `sub` bytes apart) and of an MN-major operand (16 rows = 2048 bytes).
__host__ __device__ constexpr uint32_t kmajor_step(int kk, int sub) { return static_cast<uint32_t>(((kk / 4) * sub + (kk % 4) * 32) >> 4); }
__host__ __device__ constexpr uint32_t mnmajor_step(int kk) { return static_cast<uint32_t>((kk * 2048) >> 4); }

// Arrive on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ------------------------------------------------------------------------------------
// tensor memory loads / stores, shape 32x32b: thread i of the warp owns lane
// (lane_base + i); register k holds column (col + k).
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Same wait, but the 32 destination registers of an earlier tcgen05.ld are listed as read-write
// operands, so the compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tmem_wait_ld_dep(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// The wait for two 16-register loads at once.
__device__ __forceinline__ void tmem_wait_ld_dep16(uint32_t (&r)[16], uint32_t (&q)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(q[0]), "+r"(q[1]), "+r"(q[2]), "+r"(q[3]), "+r"(q[4]), "+r"(q[5]), "+r"(q[6]), "+r"(q[7]),
                 "+r"(q[8]), "+r"(q[9]), "+r"(q[10]), "+r"(q[11]), "+r"(q[12]), "+r"(q[13]), "+r"(q[14]), "+r"(q[15])
               :
               : "memory");
}

// ------------------------------------------------------------------------------------
// math
// ------------------------------------------------------------------------------------
// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16-byte store to shared memory through a 32-bit shared address (one STS.128, no generic address).
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t saddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 128 B] tile
// laid out with the 128-byte swizzle TMA and tcgen05 use (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
  return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

}  // namespace fmha
