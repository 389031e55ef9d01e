/*
 * fmha_sm100.h — C ABI of the B200 (sm_100a) fused multi-head-attention library.
 *
 * This is the boundary a foreign-function binding attaches to.  Every entry point
 * takes plain pointers, sizes and POD structs, never throws, and returns an int
 * status (FMHA_OK == 0).  The torch operator layer (`torch.ops.mha_manual.*`) and the
 * ctypes tests are the two callers shipped with this repository.
 *
 * Which reference interface each entry point stands in for (paths are inside the
 * shmsong/NvFuserExamples project):
 *   fmha_sm100_fwd       — the three fused forward generators and their runner:
 *                          FMHAKernel::fusedKernel               fmha/fmha_manual.cpp:22-408
 *                          FMHATrainKernel::fusedKernel          fmha/fmha_manual.cpp:413-806
 *                          FMHATrainKernelSaveIntermediate::...  fmha/fmha_manual.cpp:812-1213
 *                          NVFuserOpBase<T>::run                 common/manual_scheduled_kernel.h:13-19
 *                          reached from fmha_nvfuser / fmha_train_nvfuser /
 *                          fmha_train_saveim_nvfuser             fmha/fmha_manual.cpp:1218-1238
 *   fmha_sm100_bwd       — no counterpart: the reference is forward only (README.md:1);
 *                          its oracle is autograd through the eager composite
 *                          (test_train_mha.py:14-21).
 *   fmha_sm100_philox_*  — no counterpart: the reference takes a dense dropout mask
 *                          tensor (fmha/fmha_manual.cpp:433-449); these regenerate that
 *                          mask from (seed, offset) so that it never has to be stored.
 */
#ifndef FMHA_SM100_H_
#define FMHA_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------------- */
enum {
  FMHA_OK = 0,
  FMHA_ERR_BAD_ARG = 1,        /* null pointer, negative size, misaligned pointer/stride   */
  FMHA_ERR_UNSUPPORTED = 2,    /* head dim, dtype or mode the kernels do not implement      */
  FMHA_ERR_LAUNCH = 3,         /* CUDA runtime / driver call failed (see fmha_sm100_last_cuda_error) */
  FMHA_ERR_DEVICE_TIMEOUT = 4, /* a bounded in-kernel wait ran out (read back by fmha_sm100_check_status) */
  FMHA_ERR_NO_DEVICE = 5,      /* no sm_100 device is current                               */
  FMHA_ERR_TOO_LARGE = 6       /* size exceeds a documented maximum: B, H <= 65535, B*H < 2^31,
                                  S_q, S_k <= 2^20 (or the static scratch, where that is used)  */
};

/* ---- enums ---------------------------------------------------------------------- */
enum { FMHA_DTYPE_F16 = 0, FMHA_DTYPE_BF16 = 1 };

/* How scores are masked before the softmax. */
enum {
  FMHA_MASK_NONE = 0,
  /* dense [B*H, S_q, S_k] tensor of the Q/K/V dtype, 1 = keep, 0 = masked; converted as
     (1 - m) * -10000 exactly like fmha/fmha_manual.cpp:64-65 and test.py:15. */
  FMHA_MASK_DENSE_KEEP = 1,
  /* dense [B*H, S_q, S_k] tensor of the Q/K/V dtype, added to the scaled scores
     (fmha/fmha_manual.cpp:463, test_train_mha.py:17). */
  FMHA_MASK_DENSE_ADDITIVE = 2,
  /* float32 [B, S_k] additive row (0 / -1e4 padding mask broadcast over heads and queries). */
  FMHA_MASK_KEY_ADDITIVE = 3,
  /* int32 [B] valid key length: keys j >= len[b] get -10000 added (and whole key tiles past
     len[b] are skipped, which is exact in fp32 whenever len[b] >= 1; len[b] == 0 is
     treated as "nothing masked", the value the uniform shift of the composite converges to). */
  FMHA_MASK_SEQLEN = 4,
  /* Packed variable-length batch (self-attention): int32 [B+1] cumulative row offsets, cu[0] = 0,
     cu[B] = total_rows.  q, k, v, o (and d_o, dq, dk, dv) are [total_rows, H, D] views -- stride_s and
     stride_h are used, stride_b is ignored -- and sequence b owns rows [cu[b], cu[b+1]).  S_q = S_k =
     an upper bound of the sequence lengths (it sizes the grid).  lse is [H, total_rows].  Rows of a
     tile past the end of its sequence are read (they belong to the next sequence) but never take
     part: keys are masked, queries are not written.  The Philox counter uses positions inside the
     sequence, so a packed batch draws the same bits as the padded batch. */
  FMHA_MASK_CU_SEQLENS = 5
};

/* How dropout is applied to the softmax probabilities. */
enum {
  FMHA_DROPOUT_NONE = 0,
  /* dense [B*H, S_q, S_k] 0/1 tensor of the Q/K/V dtype, P <- P * mask * dropout_scale
     (fmha/fmha_manual.cpp:478-480 with dropout_scale = 1/0.5). */
  FMHA_DROPOUT_DENSE = 1,
  /* Philox4x32-10 keyed by (seed), counter (q_row, key/16, b*H+h, offset): one 128-bit draw
     covers 16 consecutive keys, one byte each; a key is kept iff (byte & 0x7f) >= T with
     T = fmha_sm100_dropout_threshold(p); kept probabilities are scaled by 128/(128-T). */
  FMHA_DROPOUT_PHILOX = 2
};

/* A [B, H, S, D] view: element strides for b, h, s; the D axis is contiguous.  A
   [B*H, S, D] tensor is the case stride_b = H*stride_h.  Pointers must be 16-byte aligned
   and every stride a multiple of 8 elements (TMA global-address rules). */
typedef struct {
  void* ptr;
  int64_t stride_b, stride_h, stride_s;
} fmha_tensor4;

typedef struct {
  int32_t struct_bytes; /* sizeof(fmha_fwd_params): ABI check */
  int32_t dtype;        /* FMHA_DTYPE_* of q, k, v, o and of dense masks */
  int32_t B, H, S_q, S_k, D; /* D in {64, 128} */
  float scale;          /* softmax scale, typically 1/sqrt(D) */
  fmha_tensor4 q, k, v; /* inputs, borrowed, never written */
  fmha_tensor4 o;       /* output [B,H,S_q,D] */
  float* lse;           /* optional [B*H, S_q] natural-log logsumexp of the scaled+masked scores */
  int32_t mask_kind;    /* FMHA_MASK_* */
  const void* mask;     /* see FMHA_MASK_* */
  int32_t dropout_kind; /* FMHA_DROPOUT_* */
  const void* dropout_mask; /* FMHA_DROPOUT_DENSE */
  float dropout_scale;      /* FMHA_DROPOUT_DENSE: multiplier of kept entries */
  float p_drop;             /* FMHA_DROPOUT_PHILOX: drop probability in [0, 1) */
  uint64_t philox_seed;
  uint64_t philox_offset;   /* < 2^32; one value per launch */
  int32_t philox_bh_offset; /* global index of this call's (b=0,h=0): lets a B*H shard draw
                               the same bits as the unsharded call */
  /* optional dense [B*H,S_q,S_k] outputs of the Q/K/V dtype: softmax before dropout, and
     softmax*mask*scale (fmha/fmha_manual.cpp:891-897) */
  void* save_softmax;
  void* save_dropout;
  uint8_t* keep_mask_out;   /* optional [B*H,S_q,S_k] bytes: the keep decisions the kernel took */
  float* debug_scores;      /* optional [B*H,S_q,S_k] raw Q.K^T accumulators (testing aid) */
  int32_t flags;            /* FMHA_FLAG_* */
  int32_t* status;          /* optional device int32[4]: nonzero word 0 = in-kernel wait ran out */
  int32_t total_rows;       /* FMHA_MASK_CU_SEQLENS: rows of the packed tensors (= cu[B]) */
  const int64_t* philox_offset_dev; /* optional device int64: its value (mod 2^32) is added to philox_offset by the
                               kernel.  A call captured in a CUDA graph can then draw new bits on every replay:
                               advance the device value between replays (and give forward and backward the
                               same pointer).  Not supported together with dense masks / saved intermediates. */
} fmha_fwd_params;

enum {
  FMHA_FLAG_P_VIA_SMEM = 1, /* forward: stage the probability tile through shared memory instead
                               of tensor memory for the second GEMM (slower; diagnostic) */
  /* backward, measurement aids: launch only part of the three-kernel sequence so that the main
     kernel can be timed alone.  The workspace must have been prepared by an earlier full call;
     results of such partial calls are not meaningful. */
  FMHA_FLAG_BWD_SKIP_PREPARE = 2,
  FMHA_FLAG_BWD_SKIP_FINISH = 4
};

typedef struct {
  int32_t struct_bytes; /* sizeof(fmha_bwd_params) */
  int32_t dtype;
  int32_t B, H, S_q, S_k, D;
  float scale;
  fmha_tensor4 q, k, v, o, d_o; /* inputs */
  const float* lse;           /* [B*H, S_q] from the forward call */
  fmha_tensor4 dq, dk, dv;    /* outputs */
  int32_t mask_kind;          /* NONE, KEY_ADDITIVE, SEQLEN or CU_SEQLENS */
  const void* mask;
  int32_t dropout_kind;       /* NONE or PHILOX */
  float p_drop;
  uint64_t philox_seed, philox_offset;
  int32_t philox_bh_offset;
  void* workspace;            /* device scratch of fmha_sm100_bwd_workspace_bytes() bytes */
  size_t workspace_bytes;
  int32_t flags;
  int32_t* status;
  int32_t total_rows;         /* FMHA_MASK_CU_SEQLENS: rows of the packed tensors (= cu[B]) */
  const int64_t* philox_offset_dev; /* optional device int64 added to philox_offset, see fmha_fwd_params */
} fmha_bwd_params;

/* ---- entry points --------------------------------------------------------------- */

/* Forward: O = dropout(softmax(scale * Q K^T + mask)) V, plus the row logsumexp.
   `stream` is a cudaStream_t passed as void*. Asynchronous. */
int fmha_sm100_fwd(const fmha_fwd_params* p, void* stream);

/* Backward: dQ, dK, dV from (Q, K, V, O, dO, LSE).  P is recomputed from LSE. */
int fmha_sm100_bwd(const fmha_bwd_params* p, void* stream);

/* Bytes of device scratch fmha_sm100_bwd needs for these sizes (fp32 dQ accumulator and
   the row term delta = rowsum(dO * O)). */
int fmha_sm100_bwd_workspace_bytes(const fmha_bwd_params* p, size_t* bytes);

/* Backward for callers that cannot hand over a workspace (this entry point has no counterpart
   in the reference, which has no backward pass and lets its JIT runner allocate).
   Some hosts of this library cannot allocate device memory at call time: a serving process that
   gave every free byte to its own pool at start-up, a foreign runtime whose calling thread may
   not enter the CUDA allocator, a latency-critical loop for which the implicit device
   synchronisation of cudaMalloc/cudaFree is unacceptable.  For them this variant of
   fmha_sm100_bwd takes its scratch (fp32 dQ accumulator + delta) from an array that is part of
   the library image instead of p->workspace, which is ignored.  It calls no cudaMalloc, cudaFree
   or other allocating routine.
     - The array is FMHA_STATIC_SCRATCH_BYTES large on EVERY GPU that loads the library, from load
       to process exit.  Sizes whose fmha_sm100_bwd_workspace_bytes() exceeds it are refused with
       FMHA_ERR_TOO_LARGE and nothing is launched.
     - The first call on each device looks up the array's device address (once per device, with
       that device current); make that first call before any stream capture begins.
     - All calls share the one array and it keeps what the previous call left; the kernels clear
       the part that must start at zero themselves.  Two calls that overlap on the same GPU
       (different streams, or several host threads) race on it: serialise them.
   Inputs, outputs, status codes and numerics are those of fmha_sm100_bwd. */
#define FMHA_STATIC_SCRATCH_BYTES (32u << 20)
int fmha_sm100_bwd_static_scratch(const fmha_bwd_params* p, void* stream);

/* 7-bit dropout threshold T for a drop probability: T = round(128 p) clamped to [0,127]. */
int32_t fmha_sm100_dropout_threshold(float p_drop);

/* Dense keep mask (1 = kept) for [n_bh, S_q, S_k], regenerated on the HOST from the same
   Philox definition the kernels use.  `out` is host memory of n_bh*S_q*S_k bytes. */
int fmha_sm100_philox_mask_host(uint64_t seed, uint64_t offset, int32_t bh_offset,
                                int32_t n_bh, int32_t S_q, int32_t S_k, float p_drop,
                                uint8_t* out);

/* Same mask generated on the device (out is device memory). */
int fmha_sm100_philox_mask_device(uint64_t seed, uint64_t offset, int32_t bh_offset,
                                  int32_t n_bh, int32_t S_q, int32_t S_k, float p_drop,
                                  uint8_t* out, void* stream);

/* Synchronises `stream`, reads the 4-word device status block and clears it.
   Returns FMHA_OK or FMHA_ERR_DEVICE_TIMEOUT; host_copy (optional int32[4]) receives the words. */
int fmha_sm100_check_status(int32_t* status, void* stream, int32_t* host_copy);

/* Failure-detection self test (no counterpart in the reference): launches one CTA that waits
   on a barrier nothing ever signals, so the bounded wait every kernel uses runs out (about
   0.4 s), records wait site 900 in `status` and returns normally; the context stays usable.
   Follow with fmha_sm100_check_status, which then reports FMHA_ERR_DEVICE_TIMEOUT. */
int fmha_sm100_selftest_wait_timeout(int32_t* status, void* stream);

/* Text for a status code. Never NULL. */
const char* fmha_sm100_strerror(int code);

/* cudaError_t (as int) of the last failing CUDA call made by this library on this thread. */
int fmha_sm100_last_cuda_error(void);

/* Library ABI version (bumped when a struct changes). */
int fmha_sm100_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FMHA_SM100_H_ */
