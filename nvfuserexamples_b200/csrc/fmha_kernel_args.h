// fmha_kernel_args.h — parameter blocks passed (by value, __grid_constant__) to the kernels,
// and the launch functions the C ABI layer calls.  Internal to the library.
#pragma once
#include <cuda.h>  // CUtensorMap (type only; the encode entry point is looked up at run time)
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fmha_sm100.h"
#include "philox.cuh"

namespace fmha {

constexpr int kTileM = 128;  // query rows per CTA tile
constexpr int kTileN = 128;  // keys per step (general forward kernel, backward kernel)
// Keys per step of the forward kernel that will run: the production kernel walks the keys in
// 64-key steps at head dimension 64 (see fmha_fwd_fast_sm100.cu); the TMA box of K and V follows.
constexpr int fwd_key_tile(int D, bool legacy) { return (!legacy && D == 64) ? 64 : 128; }

struct FwdArgs {
  alignas(64) CUtensorMap tm_q;
  alignas(64) CUtensorMap tm_k;
  alignas(64) CUtensorMap tm_v;
  alignas(64) CUtensorMap tm_o;
  // general kernel only: the dense [B*H*S_q, S_k] 16-bit padding mask as a 2-D map with {64 x 128} boxes
  alignas(64) CUtensorMap tm_mask;
  // dense-mask kernel only: the dense dropout mask, same shape and boxes as tm_mask (valid when dmask_tiles is 1)
  alignas(64) CUtensorMap tm_dmask;
  int dmask_tiles;
  // dense-mask kernel only: the two saved [B*H, S_q, S_k] tensors as 3-D maps {S_k, S_q, B*H} with {64 x 128 x 1}
  // boxes, so that a tile stored at the end of a head's rows is clipped there (valid when save_tiles is 1)
  alignas(64) CUtensorMap tm_save_sm;
  alignas(64) CUtensorMap tm_save_dr;
  int save_tiles;
  int mask_tiles;   // 0: the mask is read with plain loads; 1: staged tile by tile through TMA
  // FMHA_MASK_CU_SEQLENS (production kernel): mask = int32 [B+1] row offsets into the packed [total_rows, H, D]
  // tensors; o_ptr / strides serve the row-wise stores of a sequence's last, partial query tile
  int total_rows;
  void* o_ptr;
  int64_t o_ss, o_sh, o_sb;   // strides in elements (o_sb: dense-mask kernel, which stores O row by row)
  int B, H, S_q, S_k;
  float scale_log2;  // softmax scale * log2(e)
  float scale;       // softmax scale
  float* lse;
  int mask_kind;
  const void* mask;
  int dropout_kind;
  const void* dropout_mask;
  float dropout_scale;   // multiplier applied to kept probabilities
  uint32_t philox_thr;   // 7-bit threshold
  uint64_t philox_seed;
  PhiloxKeys philox_keys;  // round keys of philox_seed
  uint32_t philox_offset;
  const long long* philox_offset_dev;   // optional device value added to philox_offset (production kernel)
  int philox_bh_offset;
  void* save_softmax;
  void* save_dropout;
  uint8_t* keep_mask_out;
  float* debug_scores;
  int* status;
};

struct BwdArgs {
  alignas(64) CUtensorMap tm_q;
  alignas(64) CUtensorMap tm_k;
  alignas(64) CUtensorMap tm_v;
  alignas(64) CUtensorMap tm_do;
  alignas(64) CUtensorMap tm_dk;  // 16-bit outputs, {D/4 x 32} boxes (one per compute warp), no swizzle
  alignas(64) CUtensorMap tm_dv;
  alignas(64) CUtensorMap tm_dq;  // fp32 dQ accumulator as [B*H*S_q_pad, D], 32-column boxes (TMA reduce-add)
  int B, H, S_q, S_k;
  float scale;       // softmax scale
  float scale_log2;  // softmax scale * log2(e)
  const float* lse;  // [B*H, S_q] natural log
  const float* delta;  // [B*H, S_q] rowsum(dO * O)
  float* dq_accum;     // [B*H, S_q_pad, D] fp32, zero on entry
  int* work_counter;   // zero on entry; the persistent CTAs draw their work items from it
  // FMHA_MASK_CU_SEQLENS: mask = int32 [B+1] row offsets into the packed [total_rows, H, D] tensors; the raw
  // dK / dV pointers serve the row-wise stores of a sequence's last, partial key tile
  int total_rows;
  void* dk_ptr;
  void* dv_ptr;
  int64_t dk_ss, dk_sh, dv_ss, dv_sh;
  int S_q_pad;         // S_q rounded up to the tile
  int mask_kind;
  const void* mask;
  int dropout_kind;
  float dropout_scale;
  uint32_t philox_thr;
  uint64_t philox_seed;
  PhiloxKeys philox_keys;  // round keys of philox_seed
  uint32_t philox_offset;
  const long long* philox_offset_dev;   // optional device value added to philox_offset
  int philox_bh_offset;
  int* status;
};

// Launchers (defined in the .cu files).  Return a cudaError_t as int.
int launch_fwd(const FwdArgs& a, int D, int dtype, bool legacy, bool p_via_smem, cudaStream_t stream);
int launch_fwd_fast(const FwdArgs& a, int D, int dtype, cudaStream_t stream);
// the persistent kernel of the dense-mask operators at head dimension 64 (fmha_fwd_dense_sm100.cu)
bool fwd_dense_applies(const FwdArgs& a, int D);
int launch_fwd_dense(const FwdArgs& a, int dtype, cudaStream_t stream);
int launch_bwd(const BwdArgs& a, int D, int dtype, cudaStream_t stream);
int launch_bwd_prepare(const void* o, const fmha_tensor4& ot, const fmha_tensor4& dot, int B, int H, int S_q, int S_q_pad,
                       int D, int dtype, float* delta, float* dq_accum, int* work_counter, const int* cu_seqlens, cudaStream_t stream);
int launch_bwd_finish(const float* dq_accum, const fmha_tensor4& dq, int B, int H, int S_q, int S_q_pad, int D, int dtype,
                      float scale, const int* cu_seqlens, cudaStream_t stream);

// Launches `kernel` with programmatic stream serialization: its CTAs may be scheduled while the previous
// kernel of the stream drains (which hides the launch latency between the kernels of a training step); the
// kernel itself calls griddep_wait() before it touches global memory, so stream order is preserved.
template <typename Arg>
inline cudaError_t launch_overlapped(void (*kernel)(Arg), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream,
                                     const Arg& arg) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, arg);
}

}  // namespace fmha
