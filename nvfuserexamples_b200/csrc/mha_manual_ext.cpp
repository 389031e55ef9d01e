// mha_manual_ext.cpp — the torch operator layer: `import mha_manual` registers
// torch.ops.mha_manual.* and forwards every call to the C ABI of libfmha_sm100.so.
//
// The three legacy operators keep the names, arity and positional order of the reference's
// (shmsong/NvFuserExamples fmha/fmha_manual.cpp:1218-1250), so its test.py, test_train_mha.py
// and perf_measurement*.py run against this module unchanged:
//     fmha_nvfuser(q, k, v, amask)                              -> ctx
//     fmha_train_nvfuser(q, k, v, pad_mask, dropout_mask)       -> ctx
//     fmha_train_saveim_nvfuser(q, k, v, pad_mask, dropout_mask)-> [ctx, softmax, dropout_out]
// Unlike the reference they accept any [B*H, S, D] (D in {64,128}, fp16/bf16) and validate
// their arguments.  The softmax scale is 1/sqrt(D) (the reference hard-wires 1/8 for D=64,
// fmha_manual.cpp:68) and the dropout factor is the reference's 1/0.5 (fmha_manual.cpp:478-480).
//
// New operators (no reference counterpart): fmha_fwd / fmha_bwd / fmha (autograd) take a
// compact padding mask or valid lengths and Philox (seed, offset) dropout, and
// philox_dropout_mask regenerates the dense keep mask for checking.
//
// There is no CPU implementation: the operators are registered for the CUDA key only and
// every failure of the kernel library surfaces as a RuntimeError.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cmath>
#include <ATen/cuda/CUDAGraphsUtils.cuh>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "fmha_sm100.h"

namespace {

constexpr int kMaxDevices = 64;

// One int32[4] status block per device, allocated on first use and kept for the process.
at::Tensor& status_block(int device) {
  static std::mutex mu;
  static at::Tensor blocks[kMaxDevices];
  std::lock_guard<std::mutex> g(mu);
  TORCH_CHECK(device >= 0 && device < kMaxDevices, "mha_manual: device index out of range");
  if (!blocks[device].defined()) {
    // A tensor allocated during a stream capture lives in the graph's private pool: the block must exist before.
    TORCH_CHECK(at::cuda::currentStreamCaptureStatus() == at::cuda::CaptureStatus::None,
                "mha_manual: the first operator call on a device allocates its status block; make one call before "
                "capturing a CUDA graph");
    blocks[device] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  }
  return blocks[device];
}

bool checked_mode() {
  static const bool on = [] {
    const char* e = std::getenv("MHA_MANUAL_CHECKED");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}

void raise_if(int rc, const char* what) {
  TORCH_CHECK(rc == FMHA_OK, "mha_manual::", what, " failed: ", fmha_sm100_strerror(rc), " (status ", rc,
              ", cuda error ", fmha_sm100_last_cuda_error(), ")");
}

void finish_call(int rc, const char* what, int device) {
  raise_if(rc, what);
  if (checked_mode()) {
    int32_t words[4];
    const int s = fmha_sm100_check_status(status_block(device).data_ptr<int32_t>(),
                                          at::cuda::getCurrentCUDAStream(device).stream(), words);
    TORCH_CHECK(s == FMHA_OK, "mha_manual::", what, ": ", fmha_sm100_strerror(s), " at wait site ", words[0],
                " (CTA ", words[2], ",", words[3], ")");
  }
}

struct View4 {
  fmha_tensor4 t;
  int64_t B, H, S, D;
};

// Accepts [B,H,S,D] or [B*H,S,D] (then B := B*H, H := 1) with a contiguous last axis.
View4 view4(const at::Tensor& x, const char* name) {
  TORCH_CHECK(x.is_cuda(), "mha_manual: ", name, " must be a CUDA tensor");
  TORCH_CHECK(x.dim() == 3 || x.dim() == 4, "mha_manual: ", name, " must be [B,H,S,D] or [B*H,S,D]");
  TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "mha_manual: ", name,
              " must be float16 or bfloat16");
  TORCH_CHECK(x.stride(-1) == 1, "mha_manual: ", name, " must be contiguous along the head dimension");
  View4 v;
  v.t.ptr = x.data_ptr();
  if (x.dim() == 4) {
    v.B = x.size(0); v.H = x.size(1); v.S = x.size(2); v.D = x.size(3);
    v.t.stride_b = x.stride(0); v.t.stride_h = x.stride(1); v.t.stride_s = x.stride(2);
  } else {
    v.B = x.size(0); v.H = 1; v.S = x.size(1); v.D = x.size(2);
    v.t.stride_b = x.stride(0); v.t.stride_h = x.stride(0); v.t.stride_s = x.stride(1);
  }
  TORCH_CHECK((reinterpret_cast<uintptr_t>(v.t.ptr) & 15) == 0, "mha_manual: ", name, " must be 16-byte aligned");
  TORCH_CHECK(v.t.stride_s % 8 == 0 && (v.H == 1 || v.t.stride_h % 8 == 0) && (v.B == 1 || v.t.stride_b % 8 == 0),
              "mha_manual: strides of ", name, " must be multiples of 8 elements");
  return v;
}

int dtype_code(const at::Tensor& x) { return x.scalar_type() == at::kBFloat16 ? FMHA_DTYPE_BF16 : FMHA_DTYPE_F16; }

void check_same(const at::Tensor& ref, const at::Tensor& x, const char* name) {
  TORCH_CHECK(x.device() == ref.device(), "mha_manual: ", name, " is on a different device");
  TORCH_CHECK(x.scalar_type() == ref.scalar_type(), "mha_manual: ", name, " has a different dtype");
}

void check_qkv(const View4& q, const View4& k, const View4& v) {
  TORCH_CHECK(q.D == 64 || q.D == 128, "mha_manual: head dimension must be 64 or 128, got ", q.D);
  TORCH_CHECK(k.D == q.D && v.D == q.D, "mha_manual: q, k, v head dimensions differ");
  TORCH_CHECK(k.B == q.B && v.B == q.B && k.H == q.H && v.H == q.H, "mha_manual: q, k, v batch/head sizes differ");
  TORCH_CHECK(k.S == v.S, "mha_manual: k and v sequence lengths differ");
  TORCH_CHECK(q.S == 0 || k.S > 0, "mha_manual: key length must be positive");
}

at::Tensor dense_3d(const at::Tensor& m, const at::Tensor& q, int64_t bh, int64_t sq, int64_t sk, const char* name) {
  check_same(q, m, name);
  TORCH_CHECK(m.numel() == bh * sq * sk, "mha_manual: ", name, " must have B*H*S_q*S_k elements");
  return m.contiguous();
}

// ---------------------------------------------------------------------------------------
// legacy operators
// ---------------------------------------------------------------------------------------
std::vector<at::Tensor> legacy_forward(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                       const at::Tensor& mask, int mask_kind, const at::Tensor* dropout_mask,
                                       bool save, const char* what) {
  const View4 vq = view4(q, "q"), vk = view4(k, "k"), vv = view4(v, "v");
  check_same(q, k, "k");
  check_same(q, v, "v");
  check_qkv(vq, vk, vv);
  const c10::cuda::CUDAGuard guard(q.device());
  const int dev = q.get_device();
  const int64_t bh = vq.B * vq.H;
  at::Tensor mask_c = dense_3d(mask, q, bh, vq.S, vk.S, "mask");
  at::Tensor dm_c;
  if (dropout_mask) dm_c = dense_3d(*dropout_mask, q, bh, vq.S, vk.S, "dropout_mask");
  at::Tensor o = at::empty(q.sizes(), q.options());
  const View4 vo = view4(o, "o");
  std::vector<at::Tensor> outs{o};
  fmha_fwd_params p{};
  p.struct_bytes = sizeof(p);
  p.dtype = dtype_code(q);
  p.B = static_cast<int32_t>(vq.B); p.H = static_cast<int32_t>(vq.H);
  p.S_q = static_cast<int32_t>(vq.S); p.S_k = static_cast<int32_t>(vk.S); p.D = static_cast<int32_t>(vq.D);
  p.scale = 1.0f / std::sqrt(static_cast<float>(vq.D));
  p.q = vq.t; p.k = vk.t; p.v = vv.t; p.o = vo.t;
  p.mask_kind = mask_kind;
  p.mask = mask_c.data_ptr();
  if (dropout_mask) {
    p.dropout_kind = FMHA_DROPOUT_DENSE;
    p.dropout_mask = dm_c.data_ptr();
    p.dropout_scale = 2.0f;  // 1 / dropout_prob with dropout_prob = 0.5, fmha_manual.cpp:421,478-479
  }
  if (save) {
    at::Tensor sm = at::empty({bh, vq.S, vk.S}, q.options());
    at::Tensor dr = at::empty({bh, vq.S, vk.S}, q.options());
    p.save_softmax = sm.data_ptr();
    p.save_dropout = dr.data_ptr();
    outs.push_back(sm);
    outs.push_back(dr);
  }
  p.status = status_block(dev).data_ptr<int32_t>();
  finish_call(fmha_sm100_fwd(&p, at::cuda::getCurrentCUDAStream(dev).stream()), what, dev);
  return outs;
}

at::Tensor fmha_nvfuser(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v, const at::Tensor& amask) {
  return legacy_forward(input, qk, v, amask, FMHA_MASK_DENSE_KEEP, nullptr, false, "fmha_nvfuser")[0];
}

at::Tensor fmha_train_nvfuser(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v,
                              const at::Tensor& pad_mask, const at::Tensor& dropout_mask) {
  return legacy_forward(input, qk, v, pad_mask, FMHA_MASK_DENSE_ADDITIVE, &dropout_mask, false, "fmha_train_nvfuser")[0];
}

std::vector<at::Tensor> fmha_train_saveim_nvfuser(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v,
                                                  const at::Tensor& pad_mask, const at::Tensor& dropout_mask) {
  return legacy_forward(input, qk, v, pad_mask, FMHA_MASK_DENSE_ADDITIVE, &dropout_mask, true,
                        "fmha_train_saveim_nvfuser");
}

// ---------------------------------------------------------------------------------------
// new operators
// ---------------------------------------------------------------------------------------
struct MaskArg {
  int kind = FMHA_MASK_NONE;
  at::Tensor holder;
  const void* ptr = nullptr;
};

MaskArg resolve_mask(const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, int64_t B,
                     int64_t S_k, const at::Tensor& q) {
  MaskArg m;
  TORCH_CHECK(!(mask.has_value() && seqlens.has_value()), "mha_manual: give either mask or seqlens, not both");
  if (mask.has_value()) {
    const at::Tensor& t = *mask;
    TORCH_CHECK(t.device() == q.device(), "mha_manual: mask is on a different device");
    TORCH_CHECK(t.numel() == B * S_k, "mha_manual: mask must be [B,S_k] (or [B,1,1,S_k]) additive");
    m.holder = t.reshape({B, S_k}).to(at::kFloat).contiguous();
    m.kind = FMHA_MASK_KEY_ADDITIVE;
    m.ptr = m.holder.data_ptr();
  } else if (seqlens.has_value()) {
    const at::Tensor& t = *seqlens;
    TORCH_CHECK(t.device() == q.device(), "mha_manual: seqlens is on a different device");
    TORCH_CHECK(t.numel() == B, "mha_manual: seqlens must be [B]");
    m.holder = t.reshape({B}).to(at::kInt).contiguous();
    m.kind = FMHA_MASK_SEQLEN;
    m.ptr = m.holder.data_ptr();
  }
  return m;
}

// Optional device-resident Philox offset: a one-element int64 CUDA tensor whose value the kernels add to
// `offset`, so that a captured CUDA graph draws new bits whenever the tensor is advanced between replays.
const int64_t* offset_tensor_ptr(const c10::optional<at::Tensor>& t, const at::Tensor& q) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->device() == q.device(), "mha_manual: offset_tensor is on a different device");
  TORCH_CHECK(t->scalar_type() == at::kLong && t->numel() == 1, "mha_manual: offset_tensor must hold one int64");
  return t->data_ptr<int64_t>();
}

// Forward into a caller-allocated `o` (any strides with a contiguous last axis); returns lse.
at::Tensor fwd_into(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                    const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double p_drop,
                    int64_t seed, int64_t offset, c10::optional<double> scale, int64_t bh_offset,
                    const c10::optional<at::Tensor>& offset_tensor, const char* what) {
  const View4 vq = view4(q, "q"), vk = view4(k, "k"), vv = view4(v, "v");
  check_same(q, k, "k");
  check_same(q, v, "v");
  check_qkv(vq, vk, vv);
  const c10::cuda::CUDAGuard guard(q.device());
  const int dev = q.get_device();
  const MaskArg m = resolve_mask(mask, seqlens, vq.B, vk.S, q);
  std::vector<int64_t> lse_shape{vq.B, vq.S};
  if (q.dim() == 4) lse_shape = {vq.B, vq.H, vq.S};
  at::Tensor lse = at::empty(lse_shape, q.options().dtype(at::kFloat));
  const View4 vo = view4(o, "o");
  fmha_fwd_params p{};
  p.struct_bytes = sizeof(p);
  p.dtype = dtype_code(q);
  p.B = static_cast<int32_t>(vq.B); p.H = static_cast<int32_t>(vq.H);
  p.S_q = static_cast<int32_t>(vq.S); p.S_k = static_cast<int32_t>(vk.S); p.D = static_cast<int32_t>(vq.D);
  p.scale = scale.has_value() ? static_cast<float>(*scale) : 1.0f / std::sqrt(static_cast<float>(vq.D));
  p.q = vq.t; p.k = vk.t; p.v = vv.t; p.o = vo.t;
  p.lse = lse.data_ptr<float>();
  p.mask_kind = m.kind;
  p.mask = m.ptr;
  if (p_drop > 0.0) {
    p.dropout_kind = FMHA_DROPOUT_PHILOX;
    p.p_drop = static_cast<float>(p_drop);
    p.philox_seed = static_cast<uint64_t>(seed);
    p.philox_offset = static_cast<uint64_t>(offset);
    p.philox_offset_dev = offset_tensor_ptr(offset_tensor, q);
  }
  p.philox_bh_offset = static_cast<int32_t>(bh_offset);
  p.status = status_block(dev).data_ptr<int32_t>();
  finish_call(fmha_sm100_fwd(&p, at::cuda::getCurrentCUDAStream(dev).stream()), what, dev);
  return lse;
}

std::tuple<at::Tensor, at::Tensor> fmha_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                            const c10::optional<at::Tensor>& mask,
                                            const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed,
                                            int64_t offset, c10::optional<double> scale, int64_t bh_offset,
                                            const c10::optional<at::Tensor>& offset_tensor) {
  TORCH_CHECK(q.is_cuda(), "mha_manual: q must be a CUDA tensor");
  at::Tensor o = at::empty(q.sizes(), q.options());
  at::Tensor lse = fwd_into(q, k, v, o, mask, seqlens, p_drop, seed, offset, scale, bh_offset, offset_tensor, "fmha_fwd");
  return {o, lse};
}


// An incoming gradient may be any view (autograd hands out expanded, i.e. stride-0, tensors for a broadcast loss):
// what the tensor maps cannot describe - a non-contiguous last axis, a zero, negative or non-multiple-of-8 outer
// stride, a misaligned base - is copied to a dense tensor first.
at::Tensor dense_if_needed(const at::Tensor& t) {
  bool ok = t.stride(-1) == 1 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0;
  for (int64_t d = 0; ok && d + 1 < t.dim(); ++d)
    if (t.size(d) > 1 && (t.stride(d) <= 0 || t.stride(d) % 8 != 0)) ok = false;
  return ok ? t : t.contiguous();
}

// Backward into caller-allocated dq, dk, dv (any strides with a contiguous last axis).
void bwd_into(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
              const at::Tensor& lse, const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv,
              const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed,
              int64_t offset, c10::optional<double> scale, int64_t bh_offset,
              const c10::optional<at::Tensor>& offset_tensor, const char* what) {
  const View4 vq = view4(q, "q"), vk = view4(k, "k"), vv = view4(v, "v"), vo = view4(o, "o");
  at::Tensor d_o_c = dense_if_needed(d_o);
  const View4 vdo = view4(d_o_c, "d_o");
  check_same(q, k, "k"); check_same(q, v, "v"); check_same(q, o, "o"); check_same(q, d_o_c, "d_o");
  check_qkv(vq, vk, vv);
  TORCH_CHECK(vo.B == vq.B && vo.H == vq.H && vo.S == vq.S && vo.D == vq.D, "mha_manual: o must have the shape of q");
  TORCH_CHECK(vdo.B == vq.B && vdo.H == vq.H && vdo.S == vq.S && vdo.D == vq.D, "mha_manual: d_o must have the shape of q");
  TORCH_CHECK(lse.device() == q.device() && lse.scalar_type() == at::kFloat && lse.numel() == vq.B * vq.H * vq.S,
              "mha_manual: lse must be float32 [B,H,S_q] on the device of q");
  const c10::cuda::CUDAGuard guard(q.device());
  const int dev = q.get_device();
  const MaskArg m = resolve_mask(mask, seqlens, vq.B, vk.S, q);
  at::Tensor lse_c = lse.contiguous();
  const View4 vdq = view4(dq, "dq"), vdk = view4(dk, "dk"), vdv = view4(dv, "dv");
  fmha_bwd_params p{};
  p.struct_bytes = sizeof(p);
  p.dtype = dtype_code(q);
  p.B = static_cast<int32_t>(vq.B); p.H = static_cast<int32_t>(vq.H);
  p.S_q = static_cast<int32_t>(vq.S); p.S_k = static_cast<int32_t>(vk.S); p.D = static_cast<int32_t>(vq.D);
  p.scale = scale.has_value() ? static_cast<float>(*scale) : 1.0f / std::sqrt(static_cast<float>(vq.D));
  p.q = vq.t; p.k = vk.t; p.v = vv.t; p.o = vo.t; p.d_o = vdo.t;
  p.lse = lse_c.data_ptr<float>();
  p.dq = vdq.t; p.dk = vdk.t; p.dv = vdv.t;
  p.mask_kind = m.kind;
  p.mask = m.ptr;
  if (p_drop > 0.0) {
    p.dropout_kind = FMHA_DROPOUT_PHILOX;
    p.p_drop = static_cast<float>(p_drop);
    p.philox_seed = static_cast<uint64_t>(seed);
    p.philox_offset = static_cast<uint64_t>(offset);
    p.philox_offset_dev = offset_tensor_ptr(offset_tensor, q);
  }
  p.philox_bh_offset = static_cast<int32_t>(bh_offset);
  size_t ws = 0;
  raise_if(fmha_sm100_bwd_workspace_bytes(&p, &ws), "fmha_bwd_workspace_bytes");
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, q.options().dtype(at::kByte));
  p.workspace = workspace.data_ptr();
  p.workspace_bytes = ws;
  p.status = status_block(dev).data_ptr<int32_t>();
  finish_call(fmha_sm100_bwd(&p, at::cuda::getCurrentCUDAStream(dev).stream()), what, dev);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_bwd(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                        const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                        const c10::optional<at::Tensor>& mask,
                                                        const c10::optional<at::Tensor>& seqlens, double p_drop,
                                                        int64_t seed, int64_t offset, c10::optional<double> scale,
                                                        int64_t bh_offset, const c10::optional<at::Tensor>& offset_tensor) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "mha_manual: q, k, v must be CUDA tensors");
  at::Tensor dq = at::empty(q.sizes(), q.options());
  at::Tensor dk = at::empty(k.sizes(), k.options());
  at::Tensor dv = at::empty(v.sizes(), v.options());
  bwd_into(d_o, q, k, v, o, lse, dq, dk, dv, mask, seqlens, p_drop, seed, offset, scale, bh_offset, offset_tensor, "fmha_bwd");
  return {dq, dk, dv};
}

// ---------------------------------------------------------------------------------------
// fused QKV projection layout: qkv [B,S,3,H,D] in, o [B,S,H,D] out, gradients in one [B,S,3,H,D] tensor.
// The kernels read and write these layouts through their tensor-map strides: the permutes and copies
// that the reference leaves to the caller ("no permute" in its perf scripts) do not exist here.
// ---------------------------------------------------------------------------------------
void check_qkvpacked(const at::Tensor& qkv) {
  TORCH_CHECK(qkv.is_cuda(), "mha_manual: qkv must be a CUDA tensor");
  TORCH_CHECK(qkv.dim() == 5 && qkv.size(2) == 3, "mha_manual: qkv must be [B,S,3,H,D]");
  TORCH_CHECK(qkv.is_contiguous(), "mha_manual: qkv must be contiguous");
}
// [B,S,3,H,D] -> the [B,H,S,D] view of slice i
at::Tensor qkv_slice(const at::Tensor& qkv, int64_t i) { return qkv.select(2, i).permute({0, 2, 1, 3}); }

std::tuple<at::Tensor, at::Tensor> fmha_qkvpacked_fwd(const at::Tensor& qkv, const c10::optional<at::Tensor>& mask,
                                                      const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed,
                                                      int64_t offset, c10::optional<double> scale, int64_t bh_offset,
                                                      const c10::optional<at::Tensor>& offset_tensor) {
  check_qkvpacked(qkv);
  at::Tensor o = at::empty({qkv.size(0), qkv.size(1), qkv.size(3), qkv.size(4)}, qkv.options());   // [B,S,H,D]
  at::Tensor lse = fwd_into(qkv_slice(qkv, 0), qkv_slice(qkv, 1), qkv_slice(qkv, 2), o.permute({0, 2, 1, 3}), mask, seqlens,
                            p_drop, seed, offset, scale, bh_offset, offset_tensor, "fmha_qkvpacked_fwd");
  return {o, lse};
}

at::Tensor fmha_qkvpacked_bwd(const at::Tensor& d_o, const at::Tensor& qkv, const at::Tensor& o, const at::Tensor& lse,
                              const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double p_drop,
                              int64_t seed, int64_t offset, c10::optional<double> scale, int64_t bh_offset,
                              const c10::optional<at::Tensor>& offset_tensor) {
  check_qkvpacked(qkv);
  TORCH_CHECK(d_o.dim() == 4 && o.dim() == 4 && d_o.sizes() == o.sizes() && o.size(0) == qkv.size(0) &&
                  o.size(1) == qkv.size(1) && o.size(2) == qkv.size(3) && o.size(3) == qkv.size(4),
              "mha_manual: o and d_o must be [B,S,H,D]");
  at::Tensor dqkv = at::empty(qkv.sizes(), qkv.options());
  bwd_into(d_o.permute({0, 2, 1, 3}), qkv_slice(qkv, 0), qkv_slice(qkv, 1), qkv_slice(qkv, 2), o.permute({0, 2, 1, 3}), lse,
           qkv_slice(dqkv, 0), qkv_slice(dqkv, 1), qkv_slice(dqkv, 2), mask, seqlens, p_drop, seed, offset, scale, bh_offset,
           offset_tensor, "fmha_qkvpacked_bwd");
  return dqkv;
}

// ---------------------------------------------------------------------------------------
// packed variable-length batches: q, k, v [total, H, D]; cu_seqlens int32 [B+1] on the device
// ---------------------------------------------------------------------------------------
struct Packed {
  fmha_tensor4 t;
  int64_t total, H, D;
};
Packed packed3(const at::Tensor& x, const char* name) {
  TORCH_CHECK(x.is_cuda(), "mha_manual: ", name, " must be a CUDA tensor");
  TORCH_CHECK(x.dim() == 3, "mha_manual: ", name, " must be [total_rows, H, D]");
  TORCH_CHECK(x.scalar_type() == at::kHalf || x.scalar_type() == at::kBFloat16, "mha_manual: ", name,
              " must be float16 or bfloat16");
  TORCH_CHECK(x.stride(-1) == 1, "mha_manual: ", name, " must be contiguous along the head dimension");
  Packed v;
  v.total = x.size(0); v.H = x.size(1); v.D = x.size(2);
  v.t.ptr = x.data_ptr();
  v.t.stride_b = 0; v.t.stride_h = x.stride(1); v.t.stride_s = x.stride(0);
  TORCH_CHECK((reinterpret_cast<uintptr_t>(v.t.ptr) & 15) == 0, "mha_manual: ", name, " must be 16-byte aligned");
  TORCH_CHECK(v.t.stride_s % 8 == 0 && (v.H == 1 || v.t.stride_h % 8 == 0), "mha_manual: strides of ", name,
              " must be multiples of 8 elements");
  return v;
}
at::Tensor check_cu_seqlens(const at::Tensor& cu, const at::Tensor& q) {
  TORCH_CHECK(cu.device() == q.device(), "mha_manual: cu_seqlens is on a different device");
  TORCH_CHECK(cu.dim() == 1 && cu.numel() >= 2, "mha_manual: cu_seqlens must be [B+1]");
  return cu.to(at::kInt).contiguous();
}
void check_packed_qkv(const Packed& q, const Packed& k, const Packed& v, int64_t max_seqlen) {
  TORCH_CHECK(q.D == 64 || q.D == 128, "mha_manual: head dimension must be 64 or 128, got ", q.D);
  TORCH_CHECK(k.D == q.D && v.D == q.D && k.H == q.H && v.H == q.H && k.total == q.total && v.total == q.total,
              "mha_manual: packed q, k, v must have the same [total_rows, H, D] shape");
  TORCH_CHECK(max_seqlen > 0, "mha_manual: max_seqlen must be positive");
}

// Packed forward into a caller-allocated `o` ([total_rows, H, D] with any row / head strides); returns lse.
at::Tensor varlen_fwd_into(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                           const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset,
                           c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor, const char* what) {
  const Packed vq = packed3(q, "q"), vk = packed3(k, "k"), vv = packed3(v, "v");
  check_same(q, k, "k");
  check_same(q, v, "v");
  check_packed_qkv(vq, vk, vv, max_seqlen);
  const c10::cuda::CUDAGuard guard(q.device());
  const int dev = q.get_device();
  const at::Tensor cu = check_cu_seqlens(cu_seqlens, q);
  at::Tensor lse = at::empty({vq.H, vq.total}, q.options().dtype(at::kFloat));
  if (vq.total == 0) return lse;
  fmha_fwd_params p{};
  p.struct_bytes = sizeof(p);
  p.dtype = dtype_code(q);
  p.B = static_cast<int32_t>(cu.numel() - 1); p.H = static_cast<int32_t>(vq.H);
  p.S_q = p.S_k = static_cast<int32_t>(max_seqlen); p.D = static_cast<int32_t>(vq.D);
  p.scale = scale.has_value() ? static_cast<float>(*scale) : 1.0f / std::sqrt(static_cast<float>(vq.D));
  p.q = vq.t; p.k = vk.t; p.v = vv.t; p.o = packed3(o, "o").t;
  p.lse = lse.data_ptr<float>();
  p.mask_kind = FMHA_MASK_CU_SEQLENS;
  p.mask = cu.data_ptr();
  p.total_rows = static_cast<int32_t>(vq.total);
  if (p_drop > 0.0) {
    p.dropout_kind = FMHA_DROPOUT_PHILOX;
    p.p_drop = static_cast<float>(p_drop);
    p.philox_seed = static_cast<uint64_t>(seed);
    p.philox_offset = static_cast<uint64_t>(offset);
    p.philox_offset_dev = offset_tensor_ptr(offset_tensor, q);
  }
  p.status = status_block(dev).data_ptr<int32_t>();
  finish_call(fmha_sm100_fwd(&p, at::cuda::getCurrentCUDAStream(dev).stream()), what, dev);
  return lse;
}

std::tuple<at::Tensor, at::Tensor> fmha_varlen_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                   const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop,
                                                   int64_t seed, int64_t offset, c10::optional<double> scale,
                                                   const c10::optional<at::Tensor>& offset_tensor) {
  TORCH_CHECK(q.is_cuda(), "mha_manual: q must be a CUDA tensor");
  // zero-filled: rows of a sequence beyond max_seqlen (where the kernels cut it) are never written
  at::Tensor o = at::zeros(q.sizes(), q.options());
  at::Tensor lse = varlen_fwd_into(q, k, v, o, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor, "fmha_varlen_fwd");
  return {o, lse};
}

// Packed backward into caller-allocated dq, dk, dv ([total_rows, H, D] with any row / head strides).
void varlen_bwd_into(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                     const at::Tensor& lse, const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv,
                     const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset,
                     c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor, const char* what) {
  const Packed vq = packed3(q, "q"), vk = packed3(k, "k"), vv = packed3(v, "v"), vo = packed3(o, "o");
  at::Tensor d_o_c = dense_if_needed(d_o);
  const Packed vdo = packed3(d_o_c, "d_o");
  check_same(q, k, "k"); check_same(q, v, "v"); check_same(q, o, "o"); check_same(q, d_o_c, "d_o");
  check_packed_qkv(vq, vk, vv, max_seqlen);
  TORCH_CHECK(o.sizes() == q.sizes() && d_o_c.sizes() == q.sizes(), "mha_manual: o and d_o must have the shape of q");
  TORCH_CHECK(lse.device() == q.device() && lse.scalar_type() == at::kFloat && lse.numel() == vq.H * vq.total,
              "mha_manual: lse must be float32 [H, total_rows] on the device of q");
  const c10::cuda::CUDAGuard guard(q.device());
  const int dev = q.get_device();
  const at::Tensor cu = check_cu_seqlens(cu_seqlens, q);
  at::Tensor lse_c = lse.contiguous();
  if (vq.total == 0) return;
  fmha_bwd_params p{};
  p.struct_bytes = sizeof(p);
  p.dtype = dtype_code(q);
  p.B = static_cast<int32_t>(cu.numel() - 1); p.H = static_cast<int32_t>(vq.H);
  p.S_q = p.S_k = static_cast<int32_t>(max_seqlen); p.D = static_cast<int32_t>(vq.D);
  p.scale = scale.has_value() ? static_cast<float>(*scale) : 1.0f / std::sqrt(static_cast<float>(vq.D));
  p.q = vq.t; p.k = vk.t; p.v = vv.t; p.o = vo.t; p.d_o = vdo.t;
  p.lse = lse_c.data_ptr<float>();
  p.dq = packed3(dq, "dq").t; p.dk = packed3(dk, "dk").t; p.dv = packed3(dv, "dv").t;
  p.mask_kind = FMHA_MASK_CU_SEQLENS;
  p.mask = cu.data_ptr();
  p.total_rows = static_cast<int32_t>(vq.total);
  if (p_drop > 0.0) {
    p.dropout_kind = FMHA_DROPOUT_PHILOX;
    p.p_drop = static_cast<float>(p_drop);
    p.philox_seed = static_cast<uint64_t>(seed);
    p.philox_offset = static_cast<uint64_t>(offset);
    p.philox_offset_dev = offset_tensor_ptr(offset_tensor, q);
  }
  size_t ws = 0;
  raise_if(fmha_sm100_bwd_workspace_bytes(&p, &ws), "fmha_bwd_workspace_bytes");
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, q.options().dtype(at::kByte));
  p.workspace = workspace.data_ptr();
  p.workspace_bytes = ws;
  p.status = status_block(dev).data_ptr<int32_t>();
  finish_call(fmha_sm100_bwd(&p, at::cuda::getCurrentCUDAStream(dev).stream()), what, dev);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_varlen_bwd(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                               const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                               const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop,
                                                               int64_t seed, int64_t offset, c10::optional<double> scale,
                                                               const c10::optional<at::Tensor>& offset_tensor) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "mha_manual: q, k, v must be CUDA tensors");
  // zero-filled: rows of a sequence beyond max_seqlen (where the kernels cut it) are never written
  at::Tensor dq = at::zeros(q.sizes(), q.options());
  at::Tensor dk = at::zeros(k.sizes(), k.options());
  at::Tensor dv = at::zeros(v.sizes(), v.options());
  varlen_bwd_into(d_o, q, k, v, o, lse, dq, dk, dv, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor,
                  "fmha_varlen_bwd");
  return {dq, dk, dv};
}

// Packed batch AND fused projection layout: qkv [total_rows, 3, H, D] in, o [total_rows, H, D] out, one
// [total_rows, 3, H, D] gradient back (the form an unpadded BERT layer keeps its activations in).
void check_varlen_qkvpacked(const at::Tensor& qkv) {
  TORCH_CHECK(qkv.is_cuda(), "mha_manual: qkv must be a CUDA tensor");
  TORCH_CHECK(qkv.dim() == 4 && qkv.size(1) == 3, "mha_manual: qkv must be [total_rows, 3, H, D]");
  TORCH_CHECK(qkv.is_contiguous(), "mha_manual: qkv must be contiguous");
}
std::tuple<at::Tensor, at::Tensor> fmha_varlen_qkvpacked_fwd(const at::Tensor& qkv, const at::Tensor& cu_seqlens,
                                                             int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset,
                                                             c10::optional<double> scale,
                                                             const c10::optional<at::Tensor>& offset_tensor) {
  check_varlen_qkvpacked(qkv);
  at::Tensor o = at::zeros({qkv.size(0), qkv.size(2), qkv.size(3)}, qkv.options());
  at::Tensor lse = varlen_fwd_into(qkv.select(1, 0), qkv.select(1, 1), qkv.select(1, 2), o, cu_seqlens, max_seqlen, p_drop, seed,
                                   offset, scale, offset_tensor, "fmha_varlen_qkvpacked_fwd");
  return {o, lse};
}
at::Tensor fmha_varlen_qkvpacked_bwd(const at::Tensor& d_o, const at::Tensor& qkv, const at::Tensor& o, const at::Tensor& lse,
                                     const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop, int64_t seed,
                                     int64_t offset, c10::optional<double> scale,
                                     const c10::optional<at::Tensor>& offset_tensor) {
  check_varlen_qkvpacked(qkv);
  at::Tensor dqkv = at::zeros(qkv.sizes(), qkv.options());
  varlen_bwd_into(d_o, qkv.select(1, 0), qkv.select(1, 1), qkv.select(1, 2), o, lse, dqkv.select(1, 0), dqkv.select(1, 1),
                  dqkv.select(1, 2), cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor,
                  "fmha_varlen_qkvpacked_bwd");
  return dqkv;
}

at::Tensor philox_dropout_mask(int64_t B, int64_t H, int64_t S_q, int64_t S_k, double p, int64_t seed, int64_t offset,
                               int64_t bh_offset, bool on_device) {
  TORCH_CHECK(B >= 0 && H >= 0 && S_q >= 0 && S_k >= 0, "mha_manual: negative size");
  if (on_device) {
    at::Tensor out = at::empty({B, H, S_q, S_k}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA));
    raise_if(fmha_sm100_philox_mask_device(static_cast<uint64_t>(seed), static_cast<uint64_t>(offset),
                                           static_cast<int32_t>(bh_offset), static_cast<int32_t>(B * H),
                                           static_cast<int32_t>(S_q), static_cast<int32_t>(S_k), static_cast<float>(p),
                                           out.data_ptr<uint8_t>(), at::cuda::getCurrentCUDAStream().stream()),
             "philox_dropout_mask");
    return out;
  }
  at::Tensor out = at::empty({B, H, S_q, S_k}, at::TensorOptions().dtype(at::kByte));
  raise_if(fmha_sm100_philox_mask_host(static_cast<uint64_t>(seed), static_cast<uint64_t>(offset),
                                       static_cast<int32_t>(bh_offset), static_cast<int32_t>(B * H),
                                       static_cast<int32_t>(S_q), static_cast<int32_t>(S_k), static_cast<float>(p),
                                       out.data_ptr<uint8_t>()),
           "philox_dropout_mask");
  return out;
}

void check_status() {
  const int dev = at::cuda::current_device();
  int32_t words[4];
  const int s = fmha_sm100_check_status(status_block(dev).data_ptr<int32_t>(),
                                        at::cuda::getCurrentCUDAStream(dev).stream(), words);
  TORCH_CHECK(s == FMHA_OK, "mha_manual: ", fmha_sm100_strerror(s), " at wait site ", words[0], " (CTA ", words[2], ",",
              words[3], ")");
}

// ---------------------------------------------------------------------------------------
// autograd: fmha = fmha_fwd + fmha_bwd
// ---------------------------------------------------------------------------------------
class FmhaFunction : public torch::autograd::Function<FmhaFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& q, const at::Tensor& k,
                            const at::Tensor& v, const c10::optional<at::Tensor>& mask,
                            const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed, int64_t offset,
                            c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor) {
    at::AutoDispatchBelowADInplaceOrView guard;
    // through the dispatcher, so that fake / meta tensors reach the shape-only kernels
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_fwd", "")
                         .typed<std::tuple<at::Tensor, at::Tensor>(const at::Tensor&, const at::Tensor&, const at::Tensor&,
                                                                   const c10::optional<at::Tensor>&,
                                                                   const c10::optional<at::Tensor>&, double, int64_t, int64_t,
                                                                   c10::optional<double>, int64_t,
                                                                   const c10::optional<at::Tensor>&)>();
    auto [o, lse] = op.call(q, k, v, mask, seqlens, p_drop, seed, offset, scale, 0, offset_tensor);
    // The backward pass must see the value the forward pass saw, even if the caller advances the tensor in
    // between: it gets a private copy.
    ctx->save_for_backward({q, k, v, o, lse, mask.has_value() ? *mask : at::Tensor(),
                            seqlens.has_value() ? *seqlens : at::Tensor(),
                            offset_tensor.has_value() ? offset_tensor->clone() : at::Tensor()});
    ctx->saved_data["p_drop"] = p_drop;
    ctx->saved_data["seed"] = seed;
    ctx->saved_data["offset"] = offset;
    ctx->saved_data["has_scale"] = scale.has_value();
    ctx->saved_data["scale"] = scale.has_value() ? *scale : 0.0;
    return o;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grads) {
    const auto saved = ctx->get_saved_variables();
    c10::optional<at::Tensor> mask, seqlens;
    if (saved[5].defined()) mask = saved[5];
    if (saved[6].defined()) seqlens = saved[6];
    c10::optional<at::Tensor> offset_tensor;
    if (saved[7].defined()) offset_tensor = saved[7];
    c10::optional<double> scale;
    if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
    static auto op =
        c10::Dispatcher::singleton()
            .findSchemaOrThrow("mha_manual::fmha_bwd", "")
            .typed<std::tuple<at::Tensor, at::Tensor, at::Tensor>(
                const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, double, int64_t, int64_t,
                c10::optional<double>, int64_t, const c10::optional<at::Tensor>&)>();
    auto [dq, dk, dv] = op.call(grads[0], saved[0], saved[1], saved[2], saved[3], saved[4], mask, seqlens,
                                ctx->saved_data["p_drop"].toDouble(), ctx->saved_data["seed"].toInt(),
                                ctx->saved_data["offset"].toInt(), scale, 0, offset_tensor);
    return {dq, dk, dv, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

class FmhaVarlenFunction : public torch::autograd::Function<FmhaVarlenFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& q, const at::Tensor& k,
                            const at::Tensor& v, const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop,
                            int64_t seed, int64_t offset, c10::optional<double> scale,
                            const c10::optional<at::Tensor>& offset_tensor) {
    at::AutoDispatchBelowADInplaceOrView guard;
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_varlen_fwd", "")
                         .typed<std::tuple<at::Tensor, at::Tensor>(const at::Tensor&, const at::Tensor&, const at::Tensor&,
                                                                   const at::Tensor&, int64_t, double, int64_t, int64_t,
                                                                   c10::optional<double>, const c10::optional<at::Tensor>&)>();
    auto [o, lse] = op.call(q, k, v, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor);
    ctx->save_for_backward({q, k, v, o, lse, cu_seqlens, offset_tensor.has_value() ? offset_tensor->clone() : at::Tensor()});
    ctx->saved_data["max_seqlen"] = max_seqlen;
    ctx->saved_data["p_drop"] = p_drop;
    ctx->saved_data["seed"] = seed;
    ctx->saved_data["offset"] = offset;
    ctx->saved_data["has_scale"] = scale.has_value();
    ctx->saved_data["scale"] = scale.has_value() ? *scale : 0.0;
    return o;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grads) {
    const auto saved = ctx->get_saved_variables();
    c10::optional<double> scale;
    if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_varlen_bwd", "")
                         .typed<std::tuple<at::Tensor, at::Tensor, at::Tensor>(
                             const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                             const at::Tensor&, const at::Tensor&, int64_t, double, int64_t, int64_t, c10::optional<double>,
                             const c10::optional<at::Tensor>&)>();
    c10::optional<at::Tensor> offset_tensor;
    if (saved[6].defined()) offset_tensor = saved[6];
    auto [dq, dk, dv] = op.call(grads[0], saved[0], saved[1], saved[2], saved[3], saved[4], saved[5],
                                ctx->saved_data["max_seqlen"].toInt(), ctx->saved_data["p_drop"].toDouble(),
                                ctx->saved_data["seed"].toInt(), ctx->saved_data["offset"].toInt(), scale, offset_tensor);
    return {dq, dk, dv, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

class FmhaVarlenQkvPackedFunction : public torch::autograd::Function<FmhaVarlenQkvPackedFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& qkv, const at::Tensor& cu_seqlens,
                            int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset, c10::optional<double> scale,
                            const c10::optional<at::Tensor>& offset_tensor) {
    at::AutoDispatchBelowADInplaceOrView guard;
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_varlen_qkvpacked_fwd", "")
                         .typed<std::tuple<at::Tensor, at::Tensor>(const at::Tensor&, const at::Tensor&, int64_t, double, int64_t,
                                                                   int64_t, c10::optional<double>,
                                                                   const c10::optional<at::Tensor>&)>();
    auto [o, lse] = op.call(qkv, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor);
    ctx->save_for_backward({qkv, o, lse, cu_seqlens, offset_tensor.has_value() ? offset_tensor->clone() : at::Tensor()});
    ctx->saved_data["max_seqlen"] = max_seqlen;
    ctx->saved_data["p_drop"] = p_drop;
    ctx->saved_data["seed"] = seed;
    ctx->saved_data["offset"] = offset;
    ctx->saved_data["has_scale"] = scale.has_value();
    ctx->saved_data["scale"] = scale.has_value() ? *scale : 0.0;
    return o;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grads) {
    const auto saved = ctx->get_saved_variables();
    c10::optional<double> scale;
    if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
    c10::optional<at::Tensor> offset_tensor;
    if (saved[4].defined()) offset_tensor = saved[4];
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_varlen_qkvpacked_bwd", "")
                         .typed<at::Tensor(const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                                           const at::Tensor&, int64_t, double, int64_t, int64_t, c10::optional<double>,
                                           const c10::optional<at::Tensor>&)>();
    at::Tensor dqkv = op.call(grads[0].contiguous(), saved[0], saved[1], saved[2], saved[3],
                              ctx->saved_data["max_seqlen"].toInt(), ctx->saved_data["p_drop"].toDouble(),
                              ctx->saved_data["seed"].toInt(), ctx->saved_data["offset"].toInt(), scale, offset_tensor);
    return {dqkv, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

at::Tensor fmha_varlen_qkvpacked_autograd(const at::Tensor& qkv, const at::Tensor& cu_seqlens, int64_t max_seqlen,
                                          double p_drop, int64_t seed, int64_t offset, c10::optional<double> scale,
                                          const c10::optional<at::Tensor>& offset_tensor) {
  return FmhaVarlenQkvPackedFunction::apply(qkv, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor);
}

at::Tensor fmha_varlen_autograd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu_seqlens,
                                int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset, c10::optional<double> scale,
                                const c10::optional<at::Tensor>& offset_tensor) {
  return FmhaVarlenFunction::apply(q, k, v, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor);
}

class FmhaQkvPackedFunction : public torch::autograd::Function<FmhaQkvPackedFunction> {
 public:
  static at::Tensor forward(torch::autograd::AutogradContext* ctx, const at::Tensor& qkv,
                            const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double p_drop,
                            int64_t seed, int64_t offset, c10::optional<double> scale,
                            const c10::optional<at::Tensor>& offset_tensor) {
    at::AutoDispatchBelowADInplaceOrView guard;
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_qkvpacked_fwd", "")
                         .typed<std::tuple<at::Tensor, at::Tensor>(const at::Tensor&, const c10::optional<at::Tensor>&,
                                                                   const c10::optional<at::Tensor>&, double, int64_t, int64_t,
                                                                   c10::optional<double>, int64_t,
                                                                   const c10::optional<at::Tensor>&)>();
    auto [o, lse] = op.call(qkv, mask, seqlens, p_drop, seed, offset, scale, 0, offset_tensor);
    ctx->save_for_backward({qkv, o, lse, mask.has_value() ? *mask : at::Tensor(),
                            seqlens.has_value() ? *seqlens : at::Tensor(),
                            offset_tensor.has_value() ? offset_tensor->clone() : at::Tensor()});
    ctx->saved_data["p_drop"] = p_drop;
    ctx->saved_data["seed"] = seed;
    ctx->saved_data["offset"] = offset;
    ctx->saved_data["has_scale"] = scale.has_value();
    ctx->saved_data["scale"] = scale.has_value() ? *scale : 0.0;
    return o;
  }
  static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx,
                                                 torch::autograd::variable_list grads) {
    const auto saved = ctx->get_saved_variables();
    c10::optional<at::Tensor> mask, seqlens, offset_tensor;
    if (saved[3].defined()) mask = saved[3];
    if (saved[4].defined()) seqlens = saved[4];
    if (saved[5].defined()) offset_tensor = saved[5];
    c10::optional<double> scale;
    if (ctx->saved_data["has_scale"].toBool()) scale = ctx->saved_data["scale"].toDouble();
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("mha_manual::fmha_qkvpacked_bwd", "")
                         .typed<at::Tensor(const at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                                           const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, double, int64_t,
                                           int64_t, c10::optional<double>, int64_t, const c10::optional<at::Tensor>&)>();
    at::Tensor dqkv = op.call(grads[0].contiguous(), saved[0], saved[1], saved[2], mask, seqlens,
                              ctx->saved_data["p_drop"].toDouble(), ctx->saved_data["seed"].toInt(),
                              ctx->saved_data["offset"].toInt(), scale, 0, offset_tensor);
    return {dqkv, at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor(), at::Tensor()};
  }
};

at::Tensor fmha_qkvpacked_autograd(const at::Tensor& qkv, const c10::optional<at::Tensor>& mask,
                                   const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed, int64_t offset,
                                   c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor) {
  return FmhaQkvPackedFunction::apply(qkv, mask, seqlens, p_drop, seed, offset, scale, offset_tensor);
}

at::Tensor fmha_autograd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                         const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double p_drop,
                         int64_t seed, int64_t offset, c10::optional<double> scale,
                         const c10::optional<at::Tensor>& offset_tensor) {
  return FmhaFunction::apply(q, k, v, mask, seqlens, p_drop, seed, offset, scale, offset_tensor);
}

// The same four operators below the autograd keys (torch.inference_mode(), a redispatch from another autograd
// layer): forward only, no graph is recorded.  Registered for the CUDA and Meta keys; they go through the dispatcher,
// so a Meta call lands in the shape-only kernels.
template <typename Ret, typename... Args>
Ret call_op(const char* name, Args... args) {
  return c10::Dispatcher::singleton().findSchemaOrThrow(name, "").typed<Ret(Args...)>().call(args...);
}
at::Tensor fmha_noautograd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const c10::optional<at::Tensor>& mask,
                           const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed, int64_t offset,
                           c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor) {
  return std::get<0>(call_op<std::tuple<at::Tensor, at::Tensor>, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                             const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&, double, int64_t, int64_t,
                             c10::optional<double>, int64_t, const c10::optional<at::Tensor>&>(
      "mha_manual::fmha_fwd", q, k, v, mask, seqlens, p_drop, seed, offset, scale, 0, offset_tensor));
}
at::Tensor fmha_qkvpacked_noautograd(const at::Tensor& qkv, const c10::optional<at::Tensor>& mask,
                                     const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t seed, int64_t offset,
                                     c10::optional<double> scale, const c10::optional<at::Tensor>& offset_tensor) {
  return std::get<0>(call_op<std::tuple<at::Tensor, at::Tensor>, const at::Tensor&, const c10::optional<at::Tensor>&,
                             const c10::optional<at::Tensor>&, double, int64_t, int64_t, c10::optional<double>, int64_t,
                             const c10::optional<at::Tensor>&>("mha_manual::fmha_qkvpacked_fwd", qkv, mask, seqlens, p_drop, seed,
                                                               offset, scale, 0, offset_tensor));
}
at::Tensor fmha_varlen_noautograd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu_seqlens,
                                  int64_t max_seqlen, double p_drop, int64_t seed, int64_t offset, c10::optional<double> scale,
                                  const c10::optional<at::Tensor>& offset_tensor) {
  return std::get<0>(call_op<std::tuple<at::Tensor, at::Tensor>, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                             const at::Tensor&, int64_t, double, int64_t, int64_t, c10::optional<double>,
                             const c10::optional<at::Tensor>&>("mha_manual::fmha_varlen_fwd", q, k, v, cu_seqlens, max_seqlen,
                                                               p_drop, seed, offset, scale, offset_tensor));
}
at::Tensor fmha_varlen_qkvpacked_noautograd(const at::Tensor& qkv, const at::Tensor& cu_seqlens, int64_t max_seqlen, double p_drop,
                                            int64_t seed, int64_t offset, c10::optional<double> scale,
                                            const c10::optional<at::Tensor>& offset_tensor) {
  return std::get<0>(call_op<std::tuple<at::Tensor, at::Tensor>, const at::Tensor&, const at::Tensor&, int64_t, double, int64_t,
                             int64_t, c10::optional<double>, const c10::optional<at::Tensor>&>(
      "mha_manual::fmha_varlen_qkvpacked_fwd", qkv, cu_seqlens, max_seqlen, p_drop, seed, offset, scale, offset_tensor));
}

// ---------------------------------------------------------------------------------------
// shape-only kernels (Meta key): what fake-tensor tracing and torch.compile need.  They check the
// same shape rules as the CUDA kernels' wrappers and allocate outputs of the same shapes.
// ---------------------------------------------------------------------------------------
struct MetaDims {
  int64_t B, H, S, D;
};
MetaDims meta_dims(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 3 || t.dim() == 4, "mha_manual: ", name, " must be [B*H,S,D] or [B,H,S,D]");
  if (t.dim() == 3) return {t.size(0), 1, t.size(1), t.size(2)};
  return {t.size(0), t.size(1), t.size(2), t.size(3)};
}
void meta_check_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  const MetaDims dq = meta_dims(q, "q"), dk = meta_dims(k, "k"), dv = meta_dims(v, "v");
  TORCH_CHECK(q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16, "mha_manual: q must be float16 or bfloat16");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "mha_manual: q, k, v dtypes differ");
  TORCH_CHECK(dq.D == 64 || dq.D == 128, "mha_manual: head dimension must be 64 or 128, got ", dq.D);
  TORCH_CHECK(dk.D == dq.D && dv.D == dq.D, "mha_manual: q, k, v head dimensions differ");
  TORCH_CHECK(dk.B == dq.B && dv.B == dq.B && dk.H == dq.H && dv.H == dq.H, "mha_manual: q, k, v batch/head sizes differ");
  TORCH_CHECK(dk.S == dv.S, "mha_manual: k and v sequence lengths differ");
}
std::vector<at::Tensor> legacy_meta(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& mask,
                                    const at::Tensor* dropout_mask, bool save) {
  meta_check_qkv(q, k, v);
  const MetaDims dq = meta_dims(q, "q"), dk = meta_dims(k, "k");
  const int64_t bh = dq.B * dq.H;
  TORCH_CHECK(mask.numel() == bh * dq.S * dk.S, "mha_manual: mask must have B*H*S_q*S_k elements");
  if (dropout_mask) TORCH_CHECK(dropout_mask->numel() == bh * dq.S * dk.S, "mha_manual: dropout_mask must have B*H*S_q*S_k elements");
  std::vector<at::Tensor> outs{at::empty(q.sizes(), q.options())};
  if (save) {
    outs.push_back(at::empty({bh, dq.S, dk.S}, q.options()));
    outs.push_back(at::empty({bh, dq.S, dk.S}, q.options()));
  }
  return outs;
}
at::Tensor fmha_nvfuser_meta(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v, const at::Tensor& amask) {
  return legacy_meta(input, qk, v, amask, nullptr, false)[0];
}
at::Tensor fmha_train_nvfuser_meta(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v,
                                   const at::Tensor& pad_mask, const at::Tensor& dropout_mask) {
  return legacy_meta(input, qk, v, pad_mask, &dropout_mask, false)[0];
}
std::vector<at::Tensor> fmha_train_saveim_nvfuser_meta(const at::Tensor& input, const at::Tensor& qk, const at::Tensor& v,
                                                       const at::Tensor& pad_mask, const at::Tensor& dropout_mask) {
  return legacy_meta(input, qk, v, pad_mask, &dropout_mask, true);
}
std::tuple<at::Tensor, at::Tensor> fmha_fwd_meta(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                 const c10::optional<at::Tensor>& mask,
                                                 const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t, int64_t offset,
                                                 c10::optional<double>, int64_t, const c10::optional<at::Tensor>&) {
  meta_check_qkv(q, k, v);
  const MetaDims dq = meta_dims(q, "q"), dk = meta_dims(k, "k");
  TORCH_CHECK(!(mask.has_value() && seqlens.has_value()), "mha_manual: pass either mask or seqlens, not both");
  if (mask.has_value()) TORCH_CHECK(mask->numel() == dq.B * dk.S, "mha_manual: mask must hold B*S_k additive values");
  if (seqlens.has_value()) TORCH_CHECK(seqlens->numel() == dq.B, "mha_manual: seqlens must be [B]");
  TORCH_CHECK(p_drop >= 0.0 && p_drop < 1.0, "mha_manual: p_drop must be in [0, 1)");
  TORCH_CHECK(offset >= 0 && offset < (int64_t(1) << 32), "mha_manual: offset must be in [0, 2^32)");
  std::vector<int64_t> lse_shape{dq.B, dq.S};
  if (q.dim() == 4) lse_shape = {dq.B, dq.H, dq.S};
  return {at::empty(q.sizes(), q.options()), at::empty(lse_shape, q.options().dtype(at::kFloat))};
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_bwd_meta(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                             const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                             const c10::optional<at::Tensor>&, const c10::optional<at::Tensor>&,
                                                             double, int64_t, int64_t, c10::optional<double>, int64_t,
                                                             const c10::optional<at::Tensor>&) {
  meta_check_qkv(q, k, v);
  const MetaDims dq = meta_dims(q, "q");
  TORCH_CHECK(o.sizes() == q.sizes(), "mha_manual: o must have the shape of q");
  TORCH_CHECK(d_o.sizes() == q.sizes(), "mha_manual: d_o must have the shape of q");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == dq.B * dq.H * dq.S, "mha_manual: lse must be float32 [B,H,S_q]");
  return {at::empty(q.sizes(), q.options()), at::empty(k.sizes(), k.options()), at::empty(v.sizes(), v.options())};
}

void meta_check_qkvpacked(const at::Tensor& qkv, const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens) {
  TORCH_CHECK(qkv.dim() == 5 && qkv.size(2) == 3, "mha_manual: qkv must be [B,S,3,H,D]");
  TORCH_CHECK(qkv.scalar_type() == at::kHalf || qkv.scalar_type() == at::kBFloat16, "mha_manual: qkv must be float16 or bfloat16");
  TORCH_CHECK(qkv.size(4) == 64 || qkv.size(4) == 128, "mha_manual: head dimension must be 64 or 128, got ", qkv.size(4));
  TORCH_CHECK(!(mask.has_value() && seqlens.has_value()), "mha_manual: pass either mask or seqlens, not both");
  if (mask.has_value()) TORCH_CHECK(mask->numel() == qkv.size(0) * qkv.size(1), "mha_manual: mask must hold B*S_k additive values");
  if (seqlens.has_value()) TORCH_CHECK(seqlens->numel() == qkv.size(0), "mha_manual: seqlens must be [B]");
}
std::tuple<at::Tensor, at::Tensor> fmha_qkvpacked_fwd_meta(const at::Tensor& qkv, const c10::optional<at::Tensor>& mask,
                                                           const c10::optional<at::Tensor>& seqlens, double p_drop, int64_t,
                                                           int64_t offset, c10::optional<double>, int64_t,
                                                           const c10::optional<at::Tensor>&) {
  meta_check_qkvpacked(qkv, mask, seqlens);
  TORCH_CHECK(p_drop >= 0.0 && p_drop < 1.0, "mha_manual: p_drop must be in [0, 1)");
  TORCH_CHECK(offset >= 0 && offset < (int64_t(1) << 32), "mha_manual: offset must be in [0, 2^32)");
  return {at::empty({qkv.size(0), qkv.size(1), qkv.size(3), qkv.size(4)}, qkv.options()),
          at::empty({qkv.size(0), qkv.size(3), qkv.size(1)}, qkv.options().dtype(at::kFloat))};
}
at::Tensor fmha_qkvpacked_bwd_meta(const at::Tensor& d_o, const at::Tensor& qkv, const at::Tensor& o, const at::Tensor& lse,
                                   const c10::optional<at::Tensor>& mask, const c10::optional<at::Tensor>& seqlens, double,
                                   int64_t, int64_t, c10::optional<double>, int64_t, const c10::optional<at::Tensor>&) {
  meta_check_qkvpacked(qkv, mask, seqlens);
  TORCH_CHECK(o.dim() == 4 && d_o.sizes() == o.sizes() && o.size(0) == qkv.size(0) && o.size(1) == qkv.size(1) &&
                  o.size(2) == qkv.size(3) && o.size(3) == qkv.size(4),
              "mha_manual: o and d_o must be [B,S,H,D]");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == qkv.size(0) * qkv.size(3) * qkv.size(1),
              "mha_manual: lse must be float32 [B,H,S]");
  return at::empty(qkv.sizes(), qkv.options());
}

void meta_check_packed(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& cu, int64_t max_seqlen) {
  TORCH_CHECK(q.dim() == 3, "mha_manual: q must be [total_rows, H, D]");
  TORCH_CHECK(q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16, "mha_manual: q must be float16 or bfloat16");
  TORCH_CHECK(k.sizes() == q.sizes() && v.sizes() == q.sizes() && k.scalar_type() == q.scalar_type() &&
                  v.scalar_type() == q.scalar_type(),
              "mha_manual: packed q, k, v must have the same [total_rows, H, D] shape and dtype");
  TORCH_CHECK(q.size(2) == 64 || q.size(2) == 128, "mha_manual: head dimension must be 64 or 128, got ", q.size(2));
  TORCH_CHECK(cu.dim() == 1 && cu.numel() >= 2, "mha_manual: cu_seqlens must be [B+1]");
  TORCH_CHECK(max_seqlen > 0, "mha_manual: max_seqlen must be positive");
}
std::tuple<at::Tensor, at::Tensor> fmha_varlen_fwd_meta(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                        const at::Tensor& cu_seqlens, int64_t max_seqlen, double, int64_t, int64_t,
                                                        c10::optional<double>, const c10::optional<at::Tensor>&) {
  meta_check_packed(q, k, v, cu_seqlens, max_seqlen);
  return {at::empty(q.sizes(), q.options()), at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat))};
}
std::tuple<at::Tensor, at::Tensor, at::Tensor> fmha_varlen_bwd_meta(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                                    const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                                    const at::Tensor& cu_seqlens, int64_t max_seqlen, double, int64_t,
                                                                    int64_t, c10::optional<double>, const c10::optional<at::Tensor>&) {
  meta_check_packed(q, k, v, cu_seqlens, max_seqlen);
  TORCH_CHECK(o.sizes() == q.sizes() && d_o.sizes() == q.sizes(), "mha_manual: o and d_o must have the shape of q");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == q.size(0) * q.size(1), "mha_manual: lse must be float32 [H, total_rows]");
  return {at::empty(q.sizes(), q.options()), at::empty(k.sizes(), k.options()), at::empty(v.sizes(), v.options())};
}

void meta_check_varlen_qkvpacked(const at::Tensor& qkv, const at::Tensor& cu, int64_t max_seqlen) {
  TORCH_CHECK(qkv.dim() == 4 && qkv.size(1) == 3, "mha_manual: qkv must be [total_rows, 3, H, D]");
  TORCH_CHECK(qkv.scalar_type() == at::kHalf || qkv.scalar_type() == at::kBFloat16, "mha_manual: qkv must be float16 or bfloat16");
  TORCH_CHECK(qkv.size(3) == 64 || qkv.size(3) == 128, "mha_manual: head dimension must be 64 or 128, got ", qkv.size(3));
  TORCH_CHECK(cu.dim() == 1 && cu.numel() >= 2, "mha_manual: cu_seqlens must be [B+1]");
  TORCH_CHECK(max_seqlen > 0, "mha_manual: max_seqlen must be positive");
}
std::tuple<at::Tensor, at::Tensor> fmha_varlen_qkvpacked_fwd_meta(const at::Tensor& qkv, const at::Tensor& cu_seqlens,
                                                                  int64_t max_seqlen, double, int64_t, int64_t,
                                                                  c10::optional<double>, const c10::optional<at::Tensor>&) {
  meta_check_varlen_qkvpacked(qkv, cu_seqlens, max_seqlen);
  return {at::empty({qkv.size(0), qkv.size(2), qkv.size(3)}, qkv.options()),
          at::empty({qkv.size(2), qkv.size(0)}, qkv.options().dtype(at::kFloat))};
}
at::Tensor fmha_varlen_qkvpacked_bwd_meta(const at::Tensor& d_o, const at::Tensor& qkv, const at::Tensor& o, const at::Tensor& lse,
                                          const at::Tensor& cu_seqlens, int64_t max_seqlen, double, int64_t, int64_t,
                                          c10::optional<double>, const c10::optional<at::Tensor>&) {
  meta_check_varlen_qkvpacked(qkv, cu_seqlens, max_seqlen);
  TORCH_CHECK(o.dim() == 3 && d_o.sizes() == o.sizes() && o.size(0) == qkv.size(0) && o.size(1) == qkv.size(2) &&
                  o.size(2) == qkv.size(3),
              "mha_manual: o and d_o must be [total_rows, H, D]");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == qkv.size(0) * qkv.size(2),
              "mha_manual: lse must be float32 [H, total_rows]");
  return at::empty(qkv.sizes(), qkv.options());
}

}  // namespace

TORCH_LIBRARY(mha_manual, m) {
  m.def("fmha_nvfuser(Tensor input, Tensor qk, Tensor v, Tensor amask) -> Tensor");
  m.def("fmha_train_nvfuser(Tensor input, Tensor qk, Tensor v, Tensor pad_mask, Tensor dropout_mask) -> Tensor");
  m.def("fmha_train_saveim_nvfuser(Tensor input, Tensor qk, Tensor v, Tensor pad_mask, Tensor dropout_mask) -> Tensor[]");
  m.def("fmha_fwd(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? seqlens=None, float p_drop=0.0, "
        "int seed=0, int offset=0, float? scale=None, int bh_offset=0, Tensor? offset_tensor=None) -> (Tensor, Tensor)");
  m.def("fmha_bwd(Tensor d_o, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, Tensor? mask=None, "
        "Tensor? seqlens=None, float p_drop=0.0, int seed=0, int offset=0, float? scale=None, int bh_offset=0, "
        "Tensor? offset_tensor=None) -> (Tensor, Tensor, Tensor)");
  m.def("fmha(Tensor q, Tensor k, Tensor v, Tensor? mask=None, Tensor? seqlens=None, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> Tensor");
  m.def("fmha_varlen_fwd(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens, int max_seqlen, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> (Tensor, Tensor)");
  m.def("fmha_varlen_bwd(Tensor d_o, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, Tensor cu_seqlens, int max_seqlen, "
        "float p_drop=0.0, int seed=0, int offset=0, float? scale=None, Tensor? offset_tensor=None) -> (Tensor, Tensor, Tensor)");
  m.def("fmha_varlen(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens, int max_seqlen, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> Tensor");
  m.def("fmha_qkvpacked_fwd(Tensor qkv, Tensor? mask=None, Tensor? seqlens=None, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, int bh_offset=0, Tensor? offset_tensor=None) -> (Tensor, Tensor)");
  m.def("fmha_qkvpacked_bwd(Tensor d_o, Tensor qkv, Tensor o, Tensor lse, Tensor? mask=None, Tensor? seqlens=None, "
        "float p_drop=0.0, int seed=0, int offset=0, float? scale=None, int bh_offset=0, Tensor? offset_tensor=None) -> Tensor");
  m.def("fmha_qkvpacked(Tensor qkv, Tensor? mask=None, Tensor? seqlens=None, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> Tensor");
  m.def("fmha_varlen_qkvpacked_fwd(Tensor qkv, Tensor cu_seqlens, int max_seqlen, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> (Tensor, Tensor)");
  m.def("fmha_varlen_qkvpacked_bwd(Tensor d_o, Tensor qkv, Tensor o, Tensor lse, Tensor cu_seqlens, int max_seqlen, "
        "float p_drop=0.0, int seed=0, int offset=0, float? scale=None, Tensor? offset_tensor=None) -> Tensor");
  m.def("fmha_varlen_qkvpacked(Tensor qkv, Tensor cu_seqlens, int max_seqlen, float p_drop=0.0, int seed=0, "
        "int offset=0, float? scale=None, Tensor? offset_tensor=None) -> Tensor");
  m.def("philox_dropout_mask(int B, int H, int S_q, int S_k, float p, int seed, int offset, int bh_offset=0, "
        "bool on_device=False) -> Tensor", philox_dropout_mask);
  m.def("check_status() -> ()", check_status);
}

TORCH_LIBRARY_IMPL(mha_manual, CUDA, m) {
  m.impl("fmha_nvfuser", fmha_nvfuser);
  m.impl("fmha_train_nvfuser", fmha_train_nvfuser);
  m.impl("fmha_train_saveim_nvfuser", fmha_train_saveim_nvfuser);
  m.impl("fmha_fwd", fmha_fwd);
  m.impl("fmha_bwd", fmha_bwd);
  m.impl("fmha_varlen_fwd", fmha_varlen_fwd);
  m.impl("fmha_varlen_bwd", fmha_varlen_bwd);
  m.impl("fmha_qkvpacked_fwd", fmha_qkvpacked_fwd);
  m.impl("fmha_qkvpacked_bwd", fmha_qkvpacked_bwd);
  m.impl("fmha_varlen_qkvpacked_fwd", fmha_varlen_qkvpacked_fwd);
  m.impl("fmha_varlen_qkvpacked_bwd", fmha_varlen_qkvpacked_bwd);
  m.impl("fmha", fmha_noautograd);
  m.impl("fmha_varlen", fmha_varlen_noautograd);
  m.impl("fmha_qkvpacked", fmha_qkvpacked_noautograd);
  m.impl("fmha_varlen_qkvpacked", fmha_varlen_qkvpacked_noautograd);
}

TORCH_LIBRARY_IMPL(mha_manual, Meta, m) {
  m.impl("fmha_nvfuser", fmha_nvfuser_meta);
  m.impl("fmha_train_nvfuser", fmha_train_nvfuser_meta);
  m.impl("fmha_train_saveim_nvfuser", fmha_train_saveim_nvfuser_meta);
  m.impl("fmha_fwd", fmha_fwd_meta);
  m.impl("fmha_bwd", fmha_bwd_meta);
  m.impl("fmha_varlen_fwd", fmha_varlen_fwd_meta);
  m.impl("fmha_varlen_bwd", fmha_varlen_bwd_meta);
  m.impl("fmha_qkvpacked_fwd", fmha_qkvpacked_fwd_meta);
  m.impl("fmha_qkvpacked_bwd", fmha_qkvpacked_bwd_meta);
  m.impl("fmha_varlen_qkvpacked_fwd", fmha_varlen_qkvpacked_fwd_meta);
  m.impl("fmha_varlen_qkvpacked_bwd", fmha_varlen_qkvpacked_bwd_meta);
  m.impl("fmha", fmha_noautograd);
  m.impl("fmha_varlen", fmha_varlen_noautograd);
  m.impl("fmha_qkvpacked", fmha_qkvpacked_noautograd);
  m.impl("fmha_varlen_qkvpacked", fmha_varlen_qkvpacked_noautograd);
}

TORCH_LIBRARY_IMPL(mha_manual, Autograd, m) {
  m.impl("fmha", fmha_autograd);
  m.impl("fmha_varlen", fmha_varlen_autograd);
  m.impl("fmha_qkvpacked", fmha_qkvpacked_autograd);
  m.impl("fmha_varlen_qkvpacked", fmha_varlen_qkvpacked_autograd);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "B200 fused multi-head attention operators (torch.ops.mha_manual.*)";
}
