// fmha_device_utils.cuh — small device helpers shared by the forward and backward kernels:
// 16-bit packing for fp16 / bf16, byte permutes, and row-segment loads/stores of the dense
// [B*H, S_q, S_k] tensors the legacy operators use.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace fmha {

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
template <bool BF16>
__device__ __forceinline__ float unpack_lo(uint32_t v) {
  if constexpr (BF16) return __uint_as_float(v << 16);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xffff)));
}
template <bool BF16>
__device__ __forceinline__ float unpack_hi(uint32_t v) {
  if constexpr (BF16) return __uint_as_float(v & 0xffff0000u);
  else return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16)));
}
template <bool BF16>
__device__ __forceinline__ float load_elem(const void* base, size_t idx) {
  const unsigned short raw = reinterpret_cast<const unsigned short*>(base)[idx];
  if constexpr (BF16) return __uint_as_float(static_cast<uint32_t>(raw) << 16);
  else return __half2float(__ushort_as_half(raw));
}
template <bool BF16>
__device__ __forceinline__ unsigned short to_elem(float x) {
  if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  else return __half_as_ushort(__float2half_rn(x));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// Loads 32 consecutive elements of a dense [.., S_k] row (16-bit dtype) as floats; entries
// past `n_valid` read as `fill`.  Uses 16-byte loads when the row segment is aligned.
template <bool BF16>
__device__ __forceinline__ void load_row32(const void* base, size_t elem_off, int n_valid, float fill,
                                           float (&out)[32]) {
  const unsigned short* p = reinterpret_cast<const unsigned short*>(base) + elem_off;
  if (n_valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(p) + v);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        out[v * 8 + 2 * k] = unpack_lo<BF16>(ws[k]);
        out[v * 8 + 2 * k + 1] = unpack_hi<BF16>(ws[k]);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 32; ++k) out[k] = (k < n_valid) ? load_elem<BF16>(p, k) : fill;
  }
}

template <bool BF16>
__device__ __forceinline__ void store_row32(void* base, size_t elem_off, int n_valid, const float (&v)[32]) {
  unsigned short* p = reinterpret_cast<unsigned short*>(base) + elem_off;
  if (n_valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 w;
      w.x = pack2<BF16>(v[q * 8 + 0], v[q * 8 + 1]);
      w.y = pack2<BF16>(v[q * 8 + 2], v[q * 8 + 3]);
      w.z = pack2<BF16>(v[q * 8 + 4], v[q * 8 + 5]);
      w.w = pack2<BF16>(v[q * 8 + 6], v[q * 8 + 7]);
      reinterpret_cast<uint4*>(p)[q] = w;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 32; ++k)
      if (k < n_valid) p[k] = to_elem<BF16>(v[k]);
  }
}

}  // namespace fmha
