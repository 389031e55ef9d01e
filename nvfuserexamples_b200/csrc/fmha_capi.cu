// fmha_capi.cu — the extern "C" boundary of libfmha_sm100.so: argument validation, TMA
// tensor-map construction and kernel launches.  Nothing here allocates device memory and
// nothing throws; every failure is an int status (see include/fmha_sm100.h).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/fmha_sm100.h"
#include "fmha_kernel_args.h"
#include "philox.cuh"
#include "sm100_ptx.cuh"

namespace fmha {

static thread_local int g_last_cuda_error = 0;

static int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return FMHA_ERR_LAUNCH;
}

// cuTensorMapEncodeTiled, fetched through the runtime so that the library does not link
// against libcuda directly.
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// Tensor map of a [B,H,S,D] view.  Default: {64 x box_rows x 1 x 1} boxes with 128-byte swizzle (operand
// tiles).  box_cols > 0: {box_cols x box_rows x 1 x 1} boxes without swizzle (the per-warp slices in which
// the backward kernel writes dK and dV).
static int make_tmap(CUtensorMap* out, const fmha_tensor4& t, int dtype, int B, int H, int S, int D, int box_rows,
                     int box_cols = 0) {
  auto enc = get_encode_fn();
  if (enc == nullptr) return FMHA_ERR_LAUNCH;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(t.stride_s) * 2, static_cast<cuuint64_t>(t.stride_h) * 2,
                                 static_cast<cuuint64_t>(t.stride_b) * 2};
  const cuuint32_t box[4] = {box_cols > 0 ? static_cast<cuuint32_t>(box_cols) : 64u, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = (dtype == FMHA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 4, t.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_cols > 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

// Tensor map of the fp32 dQ accumulator [rows, D].  One box per compute warp, so that no CTA-wide barrier is
// needed around the staging buffer: its 32 rows x 16 columns with 64-byte swizzle at D = 64, its 32 rows x
// 32 columns with 128-byte swizzle at D = 128.
static int make_tmap_accum(CUtensorMap* out, float* ptr, uint64_t rows, int D) {
  auto enc = get_encode_fn();
  if (enc == nullptr) return FMHA_ERR_LAUNCH;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * 4};
  const bool per_warp = (D == 64);   // box = one warp's slice: 32 rows x 16 columns (D = 64) or x 32 (D = 128)
  const cuuint32_t box[2] = {per_warp ? 16u : 32u, 32u};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   per_warp ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

// Tensor map of a dense 16-bit [rows, cols] mask with {64 x 128} boxes and 128-byte swizzle.
static int make_tmap_dense(CUtensorMap* out, const void* ptr, int dtype, uint64_t rows, uint64_t cols) {
  auto enc = get_encode_fn();
  if (enc == nullptr) return FMHA_ERR_LAUNCH;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(kTileM)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = (dtype == FMHA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

// Tensor map of a dense 16-bit [heads, rows, cols] output with {64 x 128 x 1} boxes and 128-byte swizzle (stores of a
// tile that reaches past a head's last row are clipped at that row).
static int make_tmap_dense3(CUtensorMap* out, void* ptr, int dtype, uint64_t heads, uint64_t rows, uint64_t cols) {
  auto enc = get_encode_fn();
  if (enc == nullptr) return FMHA_ERR_LAUNCH;
  const cuuint64_t dims[3] = {cols, rows, heads};
  const cuuint64_t strides[2] = {cols * 2, rows * cols * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(kTileM), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = (dtype == FMHA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = enc(out, dt, 3, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

static bool tensor_ok(const fmha_tensor4& t, int B, int H) {
  if (t.ptr == nullptr) return false;
  if (reinterpret_cast<uintptr_t>(t.ptr) & 15) return false;
  if (t.stride_s <= 0 || (t.stride_s % 8) != 0) return false;
  if (H > 1 && (t.stride_h <= 0 || (t.stride_h % 8) != 0)) return false;
  if (B > 1 && (t.stride_b <= 0 || (t.stride_b % 8) != 0)) return false;
  return true;
}

// Strides of size-1 axes are irrelevant to addressing but must still satisfy the encoder.
static fmha_tensor4 sanitized(const fmha_tensor4& t, int B, int H, int S, int D) {
  fmha_tensor4 r = t;
  if (H <= 1 || r.stride_h <= 0) r.stride_h = static_cast<int64_t>(S) * r.stride_s;
  if (B <= 1 || r.stride_b <= 0) r.stride_b = static_cast<int64_t>(H) * r.stride_h;
  (void)D;
  return r;
}

static int check_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FMHA_ERR_NO_DEVICE; }
  // Bind the device's primary context to this thread: a thread that has made no CUDA call yet
  // (an autograd worker, a fresh FFI thread) has no current context, and launches from it fail.
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FMHA_ERR_NO_DEVICE; }
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FMHA_ERR_NO_DEVICE; }
  if (major != 10) return FMHA_ERR_NO_DEVICE;
  return FMHA_OK;
}

static int validate_common(int struct_bytes, size_t expect, int dtype, int B, int H, int S_q, int S_k, int D, float scale) {
  if (struct_bytes != static_cast<int>(expect)) return FMHA_ERR_BAD_ARG;
  if (dtype != FMHA_DTYPE_F16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_UNSUPPORTED;
  if (D != 64 && D != 128) return FMHA_ERR_UNSUPPORTED;
  if (B < 0 || H < 0 || S_q < 0 || S_k < 0) return FMHA_ERR_BAD_ARG;
  if (B > 65535 || H > 65535) return FMHA_ERR_TOO_LARGE;
  // grids: B*H heads along x (< 2^31), blocks of query / key rows along y (<= 65535 blocks of >= 16 rows)
  if (static_cast<int64_t>(B) * H > 0x7fffffffll || S_q > (1 << 20) || S_k > (1 << 20)) return FMHA_ERR_TOO_LARGE;
  if (!(scale > 0.f) || !std::isfinite(scale)) return FMHA_ERR_BAD_ARG;
  return FMHA_OK;
}

}  // namespace fmha

using namespace fmha;

extern "C" {

int fmha_sm100_abi_version(void) { return 3; }

int fmha_sm100_last_cuda_error(void) { return g_last_cuda_error; }

const char* fmha_sm100_strerror(int code) {
  switch (code) {
    case FMHA_OK: return "ok";
    case FMHA_ERR_BAD_ARG: return "bad argument (null/misaligned pointer, bad stride, size or struct_bytes)";
    case FMHA_ERR_UNSUPPORTED: return "unsupported head dimension, dtype or mode";
    case FMHA_ERR_LAUNCH: return "CUDA call failed (see fmha_sm100_last_cuda_error)";
    case FMHA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside the kernel ran out";
    case FMHA_ERR_NO_DEVICE: return "current device is not an sm_100 GPU";
    case FMHA_ERR_TOO_LARGE: return "size exceeds the documented maximum";
    default: return "unknown status";
  }
}

int32_t fmha_sm100_dropout_threshold(float p_drop) { return dropout_threshold(p_drop); }

int fmha_sm100_fwd(const fmha_fwd_params* p, void* stream) {
  if (p == nullptr) return FMHA_ERR_BAD_ARG;
  int rc = validate_common(p->struct_bytes, sizeof(fmha_fwd_params), p->dtype, p->B, p->H, p->S_q, p->S_k, p->D, p->scale);
  if (rc != FMHA_OK) return rc;
  if (p->mask_kind < FMHA_MASK_NONE || p->mask_kind > FMHA_MASK_CU_SEQLENS) return FMHA_ERR_UNSUPPORTED;
  if (p->dropout_kind < FMHA_DROPOUT_NONE || p->dropout_kind > FMHA_DROPOUT_PHILOX) return FMHA_ERR_UNSUPPORTED;
  if (p->mask_kind != FMHA_MASK_NONE && p->mask == nullptr) return FMHA_ERR_BAD_ARG;
  if (p->dropout_kind == FMHA_DROPOUT_DENSE && p->dropout_mask == nullptr) return FMHA_ERR_BAD_ARG;
  const bool packed = p->mask_kind == FMHA_MASK_CU_SEQLENS;
  if (packed && (p->total_rows <= 0 || p->S_q != p->S_k)) return FMHA_ERR_BAD_ARG;
  if (p->dropout_kind == FMHA_DROPOUT_PHILOX) {
    if (!(p->p_drop >= 0.f && p->p_drop < 1.f)) return FMHA_ERR_BAD_ARG;
    if (p->philox_offset >> 32) return FMHA_ERR_BAD_ARG;
  }
  if (p->B == 0 || p->H == 0 || p->S_q == 0) return FMHA_OK;  // nothing to write
  if (p->S_k == 0) return FMHA_ERR_BAD_ARG;                    // softmax over no keys is undefined
  const int cB = packed ? 1 : p->B;   // the batch stride of packed tensors is not used
  if (!tensor_ok(p->q, cB, p->H) || !tensor_ok(p->k, cB, p->H) || !tensor_ok(p->v, cB, p->H) || !tensor_ok(p->o, cB, p->H))
    return FMHA_ERR_BAD_ARG;
  rc = check_device();
  if (rc != FMHA_OK) return rc;

  FwdArgs a;
  std::memset(&a, 0, sizeof(a));
  const bool p_via_smem = (p->flags & FMHA_FLAG_P_VIA_SMEM) != 0;
  const bool legacy = p_via_smem || p->mask_kind == FMHA_MASK_DENSE_KEEP || p->mask_kind == FMHA_MASK_DENSE_ADDITIVE ||
                      p->dropout_kind == FMHA_DROPOUT_DENSE || p->save_softmax || p->save_dropout ||
                      p->keep_mask_out || p->debug_scores;
  if (packed && legacy) return FMHA_ERR_UNSUPPORTED;   // packed batches: production kernel only
  if (p->philox_offset_dev != nullptr && legacy) return FMHA_ERR_UNSUPPORTED;   // likewise the device-resident offset
  // tensor-map extents: [B, H, S, D], or one "batch" of total_rows rows for a packed batch
  const int mB = packed ? 1 : p->B, mSq = packed ? p->total_rows : p->S_q, mSk = packed ? p->total_rows : p->S_k;
  if ((rc = make_tmap(&a.tm_q, sanitized(p->q, mB, p->H, mSq, p->D), p->dtype, mB, p->H, mSq, p->D, kTileM))) return rc;
  const int kv_rows = fwd_key_tile(p->D, legacy);
  if ((rc = make_tmap(&a.tm_k, sanitized(p->k, mB, p->H, mSk, p->D), p->dtype, mB, p->H, mSk, p->D, kv_rows))) return rc;
  if ((rc = make_tmap(&a.tm_v, sanitized(p->v, mB, p->H, mSk, p->D), p->dtype, mB, p->H, mSk, p->D, kv_rows))) return rc;
  if ((rc = make_tmap(&a.tm_o, sanitized(p->o, mB, p->H, mSq, p->D), p->dtype, mB, p->H, mSq, p->D, kTileM))) return rc;
  a.total_rows = p->total_rows;
  a.o_ptr = p->o.ptr; a.o_ss = p->o.stride_s; a.o_sh = p->o.stride_h;
  a.o_sb = sanitized(p->o, mB, p->H, mSq, p->D).stride_b;
  a.o_sh = sanitized(p->o, mB, p->H, mSq, p->D).stride_h;
  a.B = p->B; a.H = p->H; a.S_q = p->S_q; a.S_k = p->S_k;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.scale = p->scale;
  a.lse = p->lse;
  a.mask_kind = p->mask_kind;
  a.mask = p->mask;
  a.dropout_kind = p->dropout_kind;
  a.dropout_mask = p->dropout_mask;
  a.dropout_scale = 1.0f;
  if (p->dropout_kind == FMHA_DROPOUT_DENSE) a.dropout_scale = p->dropout_scale;
  if (p->dropout_kind == FMHA_DROPOUT_PHILOX) {
    const int thr = dropout_threshold(p->p_drop);
    a.philox_thr = static_cast<uint32_t>(thr);
    a.dropout_scale = 128.0f / static_cast<float>(128 - thr);
    if (thr == 0) a.dropout_kind = FMHA_DROPOUT_NONE;  // nothing is ever dropped
  }
  a.philox_seed = p->philox_seed;
  a.philox_keys = philox_round_keys(p->philox_seed);
  a.philox_offset = static_cast<uint32_t>(p->philox_offset);
  a.philox_offset_dev = reinterpret_cast<const long long*>(p->philox_offset_dev);
  a.philox_bh_offset = p->philox_bh_offset;
  a.save_softmax = p->save_softmax;
  a.save_dropout = p->save_dropout;
  a.keep_mask_out = p->keep_mask_out;
  a.debug_scores = p->debug_scores;
  a.status = p->status;
  // A dense padding mask whose rows are 16-byte multiples is staged tile by tile through TMA (coalesced, read
  // once for both softmax passes); otherwise the softmax threads read it directly.  The dense dropout mask is
  // always read directly: a second 32 KB tile would leave room for one CTA per SM only, which measured slower
  // (35.6 us against 22.9 us for the train operator at B*H = 512, S = 128, D = 64).
  a.mask_tiles = 0;
  const bool dense_mask = p->mask_kind == FMHA_MASK_DENSE_KEEP || p->mask_kind == FMHA_MASK_DENSE_ADDITIVE;
  if (dense_mask && (p->S_k % 8) == 0 && (reinterpret_cast<uintptr_t>(p->mask) & 15) == 0) {
    if ((rc = make_tmap_dense(&a.tm_mask, p->mask, p->dtype, static_cast<uint64_t>(p->B) * p->H * p->S_q, p->S_k))) return rc;
    a.mask_tiles = 1;
  }
  a.save_tiles = 0;
  if (p->save_softmax != nullptr && p->save_dropout != nullptr && (p->S_k % 8) == 0 &&
      (reinterpret_cast<uintptr_t>(p->save_softmax) & 15) == 0 && (reinterpret_cast<uintptr_t>(p->save_dropout) & 15) == 0) {
    const uint64_t heads = static_cast<uint64_t>(p->B) * p->H;
    if ((rc = make_tmap_dense3(&a.tm_save_sm, p->save_softmax, p->dtype, heads, p->S_q, p->S_k))) return rc;
    if ((rc = make_tmap_dense3(&a.tm_save_dr, p->save_dropout, p->dtype, heads, p->S_q, p->S_k))) return rc;
    a.save_tiles = 1;
  }
  a.dmask_tiles = 0;
  if (p->dropout_kind == FMHA_DROPOUT_DENSE && p->dropout_mask != nullptr && (p->S_k % 8) == 0 &&
      (reinterpret_cast<uintptr_t>(p->dropout_mask) & 15) == 0) {
    if ((rc = make_tmap_dense(&a.tm_dmask, p->dropout_mask, p->dtype, static_cast<uint64_t>(p->B) * p->H * p->S_q, p->S_k))) return rc;
    a.dmask_tiles = 1;
  }

  const int e = launch_fwd(a, p->D, p->dtype, legacy, p_via_smem, static_cast<cudaStream_t>(stream));
  if (e != 0) return cuda_fail(static_cast<cudaError_t>(e));
  return FMHA_OK;
}

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

int fmha_sm100_bwd_workspace_bytes(const fmha_bwd_params* p, size_t* bytes) {
  if (p == nullptr || bytes == nullptr) return FMHA_ERR_BAD_ARG;
  int rc = validate_common(p->struct_bytes, sizeof(fmha_bwd_params), p->dtype, p->B, p->H, p->S_q, p->S_k, p->D, p->scale);
  if (rc != FMHA_OK) return rc;
  const size_t bh = static_cast<size_t>(p->B) * p->H;
  const size_t s_q_pad = (static_cast<size_t>(p->S_q) + kTileM - 1) / kTileM * kTileM;
  // fp32 dQ accumulator, delta, and the work-item counter of the persistent main kernel
  *bytes = align256(bh * s_q_pad * p->D * sizeof(float)) + align256(bh * p->S_q * sizeof(float)) + 256;
  return FMHA_OK;
}

int fmha_sm100_bwd(const fmha_bwd_params* p, void* stream_) {
  if (p == nullptr) return FMHA_ERR_BAD_ARG;
  int rc = validate_common(p->struct_bytes, sizeof(fmha_bwd_params), p->dtype, p->B, p->H, p->S_q, p->S_k, p->D, p->scale);
  if (rc != FMHA_OK) return rc;
  if (p->mask_kind != FMHA_MASK_NONE && p->mask_kind != FMHA_MASK_KEY_ADDITIVE && p->mask_kind != FMHA_MASK_SEQLEN &&
      p->mask_kind != FMHA_MASK_CU_SEQLENS)
    return FMHA_ERR_UNSUPPORTED;
  const bool packed = p->mask_kind == FMHA_MASK_CU_SEQLENS;
  if (packed && (p->total_rows <= 0 || p->S_q != p->S_k)) return FMHA_ERR_BAD_ARG;
  if (p->dropout_kind != FMHA_DROPOUT_NONE && p->dropout_kind != FMHA_DROPOUT_PHILOX) return FMHA_ERR_UNSUPPORTED;
  if (p->mask_kind != FMHA_MASK_NONE && p->mask == nullptr) return FMHA_ERR_BAD_ARG;
  if (p->dropout_kind == FMHA_DROPOUT_PHILOX) {
    if (!(p->p_drop >= 0.f && p->p_drop < 1.f)) return FMHA_ERR_BAD_ARG;
    if (p->philox_offset >> 32) return FMHA_ERR_BAD_ARG;
  }
  if (p->B == 0 || p->H == 0) return FMHA_OK;
  if (p->S_q == 0 && p->S_k == 0) return FMHA_OK;
  if (p->S_k == 0 || p->S_q == 0) return FMHA_ERR_BAD_ARG;
  const int cB = packed ? 1 : p->B;   // the batch stride of packed tensors is not used
  if (!tensor_ok(p->q, cB, p->H) || !tensor_ok(p->k, cB, p->H) || !tensor_ok(p->v, cB, p->H) || !tensor_ok(p->o, cB, p->H) ||
      !tensor_ok(p->d_o, cB, p->H) || !tensor_ok(p->dq, cB, p->H) || !tensor_ok(p->dk, cB, p->H) || !tensor_ok(p->dv, cB, p->H) ||
      p->lse == nullptr)
    return FMHA_ERR_BAD_ARG;
  size_t need = 0;
  rc = fmha_sm100_bwd_workspace_bytes(p, &need);
  if (rc != FMHA_OK) return rc;
  if (p->workspace == nullptr || p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255))
    return FMHA_ERR_BAD_ARG;
  rc = check_device();
  if (rc != FMHA_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  const int s_q_pad = (p->S_q + kTileM - 1) / kTileM * kTileM;
  const size_t bh = static_cast<size_t>(p->B) * p->H;
  float* dq_accum = reinterpret_cast<float*>(p->workspace);
  float* delta = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(p->workspace) + align256(bh * s_q_pad * p->D * sizeof(float)));
  int* work_counter = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(delta) + align256(bh * p->S_q * sizeof(float)));

  BwdArgs a;
  std::memset(&a, 0, sizeof(a));
  // tensor-map extents: [B, H, S, D], or one "batch" of total_rows rows for a packed batch
  const int mB = packed ? 1 : p->B, mSq = packed ? p->total_rows : p->S_q, mSk = packed ? p->total_rows : p->S_k;
  const fmha_tensor4 tq = sanitized(p->q, mB, p->H, mSq, p->D), tk = sanitized(p->k, mB, p->H, mSk, p->D),
                     tv = sanitized(p->v, mB, p->H, mSk, p->D), to = sanitized(p->o, mB, p->H, mSq, p->D),
                     tdo = sanitized(p->d_o, mB, p->H, mSq, p->D), tdq = sanitized(p->dq, mB, p->H, mSq, p->D),
                     tdk = sanitized(p->dk, mB, p->H, mSk, p->D), tdv = sanitized(p->dv, mB, p->H, mSk, p->D);
  if ((rc = make_tmap(&a.tm_q, tq, p->dtype, mB, p->H, mSq, p->D, kTileM))) return rc;
  if ((rc = make_tmap(&a.tm_k, tk, p->dtype, mB, p->H, mSk, p->D, kTileN))) return rc;
  if ((rc = make_tmap(&a.tm_v, tv, p->dtype, mB, p->H, mSk, p->D, kTileN))) return rc;
  if ((rc = make_tmap(&a.tm_do, tdo, p->dtype, mB, p->H, mSq, p->D, kTileM))) return rc;
  // dK and dV leave in per-warp slices of 32 key rows x D/4 columns
  if ((rc = make_tmap(&a.tm_dk, tdk, p->dtype, mB, p->H, mSk, p->D, 32, p->D / 4))) return rc;
  if ((rc = make_tmap(&a.tm_dv, tdv, p->dtype, mB, p->H, mSk, p->D, 32, p->D / 4))) return rc;
  a.work_counter = work_counter;
  a.total_rows = p->total_rows;
  a.dk_ptr = tdk.ptr; a.dk_ss = tdk.stride_s; a.dk_sh = tdk.stride_h;
  a.dv_ptr = tdv.ptr; a.dv_ss = tdv.stride_s; a.dv_sh = tdv.stride_h;
  const int* cu_seqlens = packed ? reinterpret_cast<const int*>(p->mask) : nullptr;
  if ((rc = make_tmap_accum(&a.tm_dq, dq_accum, static_cast<uint64_t>(bh) * s_q_pad, p->D))) return rc;
  a.B = p->B; a.H = p->H; a.S_q = p->S_q; a.S_k = p->S_k;
  a.scale = p->scale;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.lse = p->lse;
  a.delta = delta;
  a.dq_accum = dq_accum;
  a.S_q_pad = s_q_pad;
  a.mask_kind = p->mask_kind;
  a.mask = p->mask;
  a.dropout_kind = p->dropout_kind;
  a.dropout_scale = 1.0f;
  if (p->dropout_kind == FMHA_DROPOUT_PHILOX) {
    const int thr = dropout_threshold(p->p_drop);
    a.philox_thr = static_cast<uint32_t>(thr);
    a.dropout_scale = 128.0f / static_cast<float>(128 - thr);
    if (thr == 0) a.dropout_kind = FMHA_DROPOUT_NONE;
  }
  a.philox_seed = p->philox_seed;
  a.philox_keys = philox_round_keys(p->philox_seed);
  a.philox_offset = static_cast<uint32_t>(p->philox_offset);
  a.philox_offset_dev = reinterpret_cast<const long long*>(p->philox_offset_dev);
  a.philox_bh_offset = p->philox_bh_offset;
  a.status = p->status;

  int e = 0;
  if (!(p->flags & FMHA_FLAG_BWD_SKIP_PREPARE)) {
    e = launch_bwd_prepare(nullptr, to, tdo, p->B, p->H, p->S_q, s_q_pad, p->D, p->dtype, delta, dq_accum, work_counter, cu_seqlens,
                           stream);
    if (e != 0) return cuda_fail(static_cast<cudaError_t>(e));
  } else {
    // the caller prepared delta and the accumulator itself; the work counter is still ours to clear
    cudaError_t ce = cudaMemsetAsync(work_counter, 0, sizeof(int), stream);
    if (ce != cudaSuccess) return cuda_fail(ce);
  }
  e = launch_bwd(a, p->D, p->dtype, stream);
  if (e != 0) return cuda_fail(static_cast<cudaError_t>(e));
  if (!(p->flags & FMHA_FLAG_BWD_SKIP_FINISH)) {
    // the main kernel leaves the dropout factor 1/(1-p) out of dS; it is applied here (and to dK, dV in its epilogue)
    e = launch_bwd_finish(dq_accum, tdq, p->B, p->H, p->S_q, s_q_pad, p->D, p->dtype, p->scale * a.dropout_scale, cu_seqlens,
                          stream);
    if (e != 0) return cuda_fail(static_cast<cudaError_t>(e));
  }
  return FMHA_OK;
}

int fmha_sm100_check_status(int32_t* status, void* stream, int32_t* host_copy) {
  if (status == nullptr) return FMHA_ERR_BAD_ARG;
  int32_t h[4] = {0, 0, 0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(h, status, sizeof(h), cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e);
  if (host_copy) std::memcpy(host_copy, h, sizeof(h));
  if (h[0] != 0) {
    e = cudaMemsetAsync(status, 0, sizeof(h), s);
    if (e != cudaSuccess) return cuda_fail(e);
    return FMHA_ERR_DEVICE_TIMEOUT;
  }
  return FMHA_OK;
}

int fmha_sm100_philox_mask_host(uint64_t seed, uint64_t offset, int32_t bh_offset, int32_t n_bh, int32_t S_q,
                                int32_t S_k, float p_drop, uint8_t* out) {
  if (out == nullptr || n_bh < 0 || S_q < 0 || S_k < 0) return FMHA_ERR_BAD_ARG;
  if (!(p_drop >= 0.f && p_drop < 1.f) || (offset >> 32)) return FMHA_ERR_BAD_ARG;
  const uint32_t thr = static_cast<uint32_t>(dropout_threshold(p_drop));
  for (int bh = 0; bh < n_bh; ++bh)
    for (int r = 0; r < S_q; ++r) {
      uint8_t* row = out + (static_cast<size_t>(bh) * S_q + r) * S_k;
      for (int kb = 0; kb * 16 < S_k; ++kb) {
        const U4 d = dropout_draw(seed, static_cast<uint32_t>(offset), static_cast<uint32_t>(bh_offset + bh),
                                  static_cast<uint32_t>(r), static_cast<uint32_t>(kb));
        const uint32_t w[4] = {d.x, d.y, d.z, d.w};
        for (int i = 0; i < 16 && kb * 16 + i < S_k; ++i) {
          const uint32_t byte = (w[i / 4] >> (8 * (i % 4))) & 0xffu;
          row[kb * 16 + i] = ((byte & 0x7fu) >= thr) ? 1 : 0;
        }
      }
    }
  return FMHA_OK;
}

}  // extern "C"

namespace fmha {
__global__ void philox_mask_kernel(uint64_t seed, uint32_t offset, int bh_offset, int n_bh, int S_q, int S_k,
                                   uint32_t thr, uint8_t* out) {
  const int n_kb = (S_k + 15) / 16;
  const size_t total = static_cast<size_t>(n_bh) * S_q * n_kb;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int kb = static_cast<int>(idx % n_kb);
    const size_t rr = idx / n_kb;
    const int r = static_cast<int>(rr % S_q);
    const int bh = static_cast<int>(rr / S_q);
    const U4 d = dropout_draw(seed, offset, static_cast<uint32_t>(bh_offset + bh), static_cast<uint32_t>(r),
                              static_cast<uint32_t>(kb));
    const uint32_t w[4] = {d.x, d.y, d.z, d.w};
    uint8_t* row = out + (static_cast<size_t>(bh) * S_q + r) * S_k;
    for (int k = 0; k < 4; ++k) {
      const uint32_t keep = dropout_keep_bits(w[k], thr);
      for (int e = 0; e < 4; ++e) {
        const int col = kb * 16 + k * 4 + e;
        if (col < S_k) row[col] = (keep >> (8 * e + 7)) & 1u;
      }
    }
  }
}
}  // namespace fmha

extern "C" int fmha_sm100_philox_mask_device(uint64_t seed, uint64_t offset, int32_t bh_offset, int32_t n_bh,
                                              int32_t S_q, int32_t S_k, float p_drop, uint8_t* out, void* stream) {
  if (out == nullptr || n_bh < 0 || S_q < 0 || S_k < 0) return FMHA_ERR_BAD_ARG;
  if (!(p_drop >= 0.f && p_drop < 1.f) || (offset >> 32)) return FMHA_ERR_BAD_ARG;
  const size_t total = static_cast<size_t>(n_bh) * S_q * ((S_k + 15) / 16);
  if (total == 0) return FMHA_OK;
  const uint32_t thr = static_cast<uint32_t>(dropout_threshold(p_drop));
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
  fmha::philox_mask_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      seed, static_cast<uint32_t>(offset), bh_offset, n_bh, S_q, S_k, thr, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FMHA_OK;
}

namespace fmha {
// One thread waits on an mbarrier that has no other participant: exercises the bounded wait.
__global__ void selftest_wait_kernel(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  abort_flag = 0;
  mbar_init(&bar, 1);
  mbar_fence_init();
  const WaitCtx ctx{&abort_flag, status};
  mbar_wait(&bar, 0, ctx, 900);
}
}  // namespace fmha

extern "C" int fmha_sm100_selftest_wait_timeout(int32_t* status, void* stream) {
  if (status == nullptr) return FMHA_ERR_BAD_ARG;
  const int rc = check_device();
  if (rc != FMHA_OK) return rc;
  fmha::selftest_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return FMHA_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward without a caller workspace: scratch lives in the library image.
// ---------------------------------------------------------------------------------------------
// In host code `g_bwd_static_scratch` is only a handle for the runtime's symbol table, never a
// device address; the address each device gave the array is fetched below with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_bwd_static_scratch[FMHA_STATIC_SCRATCH_BYTES];

namespace fmha {
constexpr int kMaxScratchDevices = 64;
static std::mutex g_scratch_mu;
static void* g_scratch_addr[kMaxScratchDevices] = {};

// Device address of the static scratch on the CURRENT device (looked up once per device).
static int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { g_last_cuda_error = static_cast<int>(e); return FMHA_ERR_NO_DEVICE; }
  if (dev < 0 || dev >= kMaxScratchDevices) return FMHA_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_bwd_static_scratch);  // needs `dev` current: it is
    if (e != cudaSuccess) return cuda_fail(e);
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255)) return FMHA_ERR_LAUNCH;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return FMHA_OK;
}
}  // namespace fmha

extern "C" int fmha_sm100_bwd_static_scratch(const fmha_bwd_params* p, void* stream) {
  if (p == nullptr) return FMHA_ERR_BAD_ARG;
  size_t need = 0;
  int rc = fmha_sm100_bwd_workspace_bytes(p, &need);  // also validates struct size, dtype, D, sizes
  if (rc != FMHA_OK) return rc;
  if (need > FMHA_STATIC_SCRATCH_BYTES) return FMHA_ERR_TOO_LARGE;
  rc = check_device();
  if (rc != FMHA_OK) return rc;
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != FMHA_OK) return rc;
  fmha_bwd_params q = *p;            // same call, scratch pointer swapped in; the caller's struct is untouched
  q.workspace = scratch;
  q.workspace_bytes = FMHA_STATIC_SCRATCH_BYTES;
  return fmha_sm100_bwd(&q, stream);
}
