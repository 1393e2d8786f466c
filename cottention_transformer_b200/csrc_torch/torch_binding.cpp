// Compiled torch binding over the C ABI of libcottention_b200.so (include/cottention_b200.h).
//
// 1. The reference's extension module: four functions with the signature its pybind block registers
//    (Cuda_Kernel/combined_kernel_general.cu:353,444-454),
//        float32 / float64 / float16 / bfloat16 (Tensor Q, Tensor K, Tensor V, int block_size,
//                                                bool inplace = false, bool reversed = false) -> Tensor
//    with the checks, messages, autocast dtype rule and in-place behaviour of forward_<dtype> (:355-407).
// 2. The fused operators as torch.library ops (namespace cottention_b200), so that the autograd functions of the
//    package make one dispatcher call per direction instead of a dozen Python-level tensor calls -- at BERT shapes
//    the step is otherwise bound by the host, not by its kernels.
//
// Nothing here computes: every function validates, allocates its outputs and calls one extern "C" entry point on
// torch's current stream.  The ctypes route (cottention_transformer_b200/_lib.py) stays for non-torch hosts.
#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include "../../include/cottention_b200.h"

namespace {

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return COTT_F32;
    case at::kDouble: return COTT_F64;
    case at::kHalf: return COTT_F16;
    case at::kBFloat16: return COTT_BF16;
    default: TORCH_CHECK(false, "Only float32, float64, float16, and bfloat16 are supported");
  }
}

void check(int status, const char* what) {
  TORCH_CHECK(status == COTT_OK, what, ": ", cott_status_string(status), " (", status, "): ", cott_last_error());
}

void* stream_of(const at::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

const void* ptr_or_null(const c10::optional<at::Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// ---- 1. FastAttention2.kernel.<dtype> ------------------------------------------------------------------------
// AUTOCAST: the dtype the entry point runs in when autocast is on and Q is float32 (:377-389)
template <at::ScalarType AUTOCAST>
at::Tensor forward_(at::Tensor& Q, at::Tensor& K, at::Tensor& V, const int8_t block_size, bool inplace, bool reversed) {
  (void)block_size;  // accepted and ignored, as in the reference (:353)
  TORCH_CHECK(Q.device().is_cuda(), "Q must be a CUDA tensor");
  TORCH_CHECK(K.device().is_cuda(), "K must be a CUDA tensor");
  TORCH_CHECK(V.device().is_cuda(), "V must be a CUDA tensor");
  TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4, "Q, K and V must be 4-dimensional [N, H, S, D]");
  TORCH_CHECK(Q.size(3) == K.size(3), "Q and K must have the same dimension");
  const int64_t D_attn = Q.size(3);
  TORCH_CHECK(D_attn % 16 == 0, "D_attn must be divisible by 16");
  TORCH_CHECK(D_attn >= 16 * 2, "D_attn must be greater than or equal to 16*2");
  for (int i = 0; i < 3; ++i)
    TORCH_CHECK(K.size(i) == Q.size(i) && V.size(i) == Q.size(i), "Q, K and V must agree in their first three dimensions");
  const at::ScalarType data_type =
      (at::autocast::is_autocast_enabled(at::kCUDA) && Q.scalar_type() == at::kFloat) ? AUTOCAST : Q.scalar_type();
  const int code = dtype_code(data_type);
  Q = Q.contiguous().to(data_type);  // :397-399 (rebinding the caller's handles, like the reference's Tensor&)
  K = K.contiguous().to(data_type);
  V = V.contiguous().to(data_type);
  at::Tensor out = inplace ? V : at::empty({Q.size(0), Q.size(1), Q.size(2), V.size(3)}, Q.options());  // :402-407
  const c10::cuda::CUDAGuard guard(Q.device());  // :412
  check(cott_scan(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), (int)Q.size(0), (int)Q.size(1), (int)Q.size(2),
                  (int)D_attn, (int)V.size(3), code, reversed ? 1 : 0, stream_of(Q)),
        "cott_scan");
  return out;
}

// ---- 2. fused operators ---------------------------------------------------------------------------------------
at::Tensor nc_f32(const at::Tensor& norm_const, const at::Tensor& like, int64_t H) {
  at::Tensor nc = norm_const.detach().reshape({-1}).to(like.device(), at::kFloat).contiguous();
  TORCH_CHECK(nc.numel() == H, "norm_const must have one entry per head (", H, "), got ", nc.numel());
  return nc;
}

// causal forward: returns (out, workspace, saved); workspace / saved are empty tensors when not needed
std::tuple<at::Tensor, at::Tensor, at::Tensor> causal_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                          const at::Tensor& norm_const, const c10::optional<at::Tensor>& keep,
                                                          int64_t nseg, bool save_states) {
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous(), "contiguous CUDA tensors expected");
  const int B = (int)q.size(0), H = (int)q.size(1), N = (int)q.size(2), D = (int)q.size(3);
  const int code = dtype_code(q.scalar_type());
  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor nc = nc_f32(norm_const, q, H);
  at::Tensor out = at::empty_like(v);
  const auto bytes = q.options().dtype(at::kByte);
  if (nseg <= 0) nseg = cott_cos_attn_seg_count(B, H, N);
  const bool general = nseg > 1 || (keep.has_value() && keep->defined());
  at::Tensor ws = at::empty({general ? (int64_t)std::max<size_t>(cott_cos_attn_seg_workspace_bytes(B, H, N, (int)nseg), 16) : 0}, bytes);
  at::Tensor saved = at::empty({save_states ? (int64_t)std::max<size_t>(cott_cos_attn_saved_bytes(B, H, N), 16) : 0}, bytes);
  const unsigned char* kp = static_cast<const unsigned char*>(ptr_or_null(keep));
  if (save_states)
    check(cott_cos_attn_fwd_train(q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, nc.data_ptr<float>(), out.data_ptr(), saved.data_ptr(),
                                  general ? ws.data_ptr() : nullptr, (int)nseg, nullptr, B, H, N, D, D, code, stream_of(q)),
          "cott_cos_attn_fwd_train");
  else if (general)
    check(cott_cos_attn_fwd_seg(q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, nc.data_ptr<float>(), out.data_ptr(), ws.data_ptr(),
                                (int)nseg, nullptr, B, H, N, D, D, code, stream_of(q)),
          "cott_cos_attn_fwd_seg");
  else
    check(cott_cos_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), nc.data_ptr<float>(), out.data_ptr(), B, H, N, D, D, code,
                            stream_of(q)),
          "cott_cos_attn_fwd");
  return {out, ws, saved};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> causal_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                                      const at::Tensor& norm_const,
                                                                      const c10::optional<at::Tensor>& keep, const at::Tensor& dout_,
                                                                      const at::Tensor& ws, const at::Tensor& saved, int64_t nseg) {
  const int B = (int)q.size(0), H = (int)q.size(1), N = (int)q.size(2), D = (int)q.size(3);
  const int code = dtype_code(q.scalar_type());
  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor nc = nc_f32(norm_const, q, H);
  at::Tensor dout = dout_.contiguous().to(q.scalar_type());
  at::Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  at::Tensor dnc = at::empty({H}, q.options().dtype(at::kFloat));
  const unsigned char* kp = static_cast<const unsigned char*>(ptr_or_null(keep));
  void* wsp = ws.numel() ? ws.data_ptr() : nullptr;
  if (nseg <= 0) nseg = cott_cos_attn_seg_count(B, H, N);  // the forward's choice for the same sizes on the same device
  if (saved.numel())
    check(cott_cos_attn_bwd_train(q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, nc.data_ptr<float>(), dout.data_ptr(), saved.data_ptr(), wsp,
                                  (int)nseg, nullptr, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dnc.data_ptr<float>(), B, H, N, D, D,
                                  code, stream_of(q)),
          "cott_cos_attn_bwd_train");
  else if (ws.numel())
    check(cott_cos_attn_bwd_seg(q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, nc.data_ptr<float>(), dout.data_ptr(), wsp, (int)nseg, nullptr,
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dnc.data_ptr<float>(), B, H, N, D, D, code, stream_of(q)),
          "cott_cos_attn_bwd_seg");
  else
    check(cott_cos_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), nc.data_ptr<float>(), dout.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                            dv.data_ptr(), dnc.data_ptr<float>(), B, H, N, D, D, code, stream_of(q)),
          "cott_cos_attn_bwd");
  return {dq, dk, dv, dnc};
}

// bidirectional forward: returns (out, scratch)
std::tuple<at::Tensor, at::Tensor> bidir_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& norm_const,
                                             const c10::optional<at::Tensor>& keep) {
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous(), "contiguous CUDA tensors expected");
  const int B = (int)q.size(0), H = (int)q.size(1), N = (int)q.size(2), Dk = (int)q.size(3), Dv = (int)v.size(3);
  const int code = dtype_code(q.scalar_type());
  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor nc = nc_f32(norm_const, q, H);
  at::Tensor out = at::empty({B, H, N, Dv}, q.options());
  at::Tensor scratch = at::empty({(int64_t)std::max<size_t>(cott_bidir_scratch_bytes(B, H, N, Dk, Dv, code), 1)}, q.options().dtype(at::kByte));
  check(cott_bidir_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), static_cast<const unsigned char*>(ptr_or_null(keep)), nc.data_ptr<float>(),
                       out.data_ptr(), scratch.data_ptr(), B, H, N, Dk, Dv, code, stream_of(q)),
        "cott_bidir_fwd");
  return {out, scratch};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bidir_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                                                     const at::Tensor& norm_const, const c10::optional<at::Tensor>& keep,
                                                                     const at::Tensor& dout_, const at::Tensor& scratch) {
  const int B = (int)q.size(0), H = (int)q.size(1), N = (int)q.size(2), Dk = (int)q.size(3), Dv = (int)v.size(3);
  const int code = dtype_code(q.scalar_type());
  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor nc = nc_f32(norm_const, q, H);
  at::Tensor dout = dout_.contiguous().to(q.scalar_type());
  at::Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  at::Tensor dnc = at::empty({H}, q.options().dtype(at::kFloat));
  at::Tensor scratch2 = at::empty_like(scratch);
  check(cott_bidir_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), static_cast<const unsigned char*>(ptr_or_null(keep)), nc.data_ptr<float>(),
                       dout.data_ptr(), scratch.data_ptr(), scratch2.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                       dnc.data_ptr<float>(), B, H, N, Dk, Dv, code, stream_of(q)),
        "cott_bidir_bwd");
  return {dq, dk, dv, dnc};
}

}  // namespace

TORCH_LIBRARY(cottention_b200, m) {
  m.def("causal_fwd(Tensor q, Tensor k, Tensor v, Tensor norm_const, Tensor? keep, int nseg, bool save_states) -> (Tensor, Tensor, Tensor)");
  m.def("causal_bwd(Tensor q, Tensor k, Tensor v, Tensor norm_const, Tensor? keep, Tensor dout, Tensor ws, Tensor saved, int nseg) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("bidir_fwd(Tensor q, Tensor k, Tensor v, Tensor norm_const, Tensor? keep) -> (Tensor, Tensor)");
  m.def("bidir_bwd(Tensor q, Tensor k, Tensor v, Tensor norm_const, Tensor? keep, Tensor dout, Tensor scratch) -> (Tensor, Tensor, Tensor, Tensor)");
}
TORCH_LIBRARY_IMPL(cottention_b200, CUDA, m) {
  m.impl("causal_fwd", &causal_fwd);
  m.impl("causal_bwd", &causal_bwd);
  m.impl("bidir_fwd", &bidir_fwd);
  m.impl("bidir_bwd", &bidir_bwd);
}

// The reference registers its four functions with pybind (combined_kernel_general.cu:444-454); the argument names and
// defaults are its own.
PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  // how a non-zero status of the C ABI surfaces in Python: RuntimeError carrying the status text and the library's message
  m.def("_raise_for_status", [](int status) { check(status, "cottention_b200"); }, py::arg("status"));
  m.def("float32", &forward_<at::kBFloat16>, "FastAttention forward (float32 entry point)", py::arg("Q"), py::arg("K"), py::arg("V"),
        py::arg("block_size"), py::arg("inplace") = false, py::arg("reversed") = false);
  m.def("float64", &forward_<at::kBFloat16>, "FastAttention forward (float64 entry point)", py::arg("Q"), py::arg("K"), py::arg("V"),
        py::arg("block_size"), py::arg("inplace") = false, py::arg("reversed") = false);
  m.def("float16", &forward_<at::kHalf>, "FastAttention forward (float16 entry point)", py::arg("Q"), py::arg("K"), py::arg("V"),
        py::arg("block_size"), py::arg("inplace") = false, py::arg("reversed") = false);
  m.def("bfloat16", &forward_<at::kBFloat16>, "FastAttention forward (bfloat16 entry point)", py::arg("Q"), py::arg("K"), py::arg("V"),
        py::arg("block_size"), py::arg("inplace") = false, py::arg("reversed") = false);
}
