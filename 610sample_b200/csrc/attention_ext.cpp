// Python module `attention_cuda`: the three functions the reference's pybind shim
// exports (reference csrc/attention_ext.cpp:19-35) with the same names, keyword
// names, argument order and list-of-tensors results, backed by libattn_b200.so.
//
// Differences, all additive: a trailing `mask_mode` keyword (0 = the reference's
// causal + sliding-window + validity mask, 1 = no mask) and an `impl` keyword
// (0 auto, 1 fp32 SIMT kernels, 2 tensor-core kernels); float32 inputs and head
// dimensions up to 128 are accepted.  Kernels run on the current PyTorch stream
// of the tensors' device.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstdio>
#include <mutex>
#include <vector>

#include "attn_b200.h"

namespace {

int dtype_code(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kHalf: return ATTN_F16;
    case at::kBFloat16: return ATTN_BF16;
    case at::kFloat: return ATTN_F32;
    default: TORCH_CHECK(false, "V7 requires fp16, bf16 or fp32, got ", t.scalar_type());
  }
  return -1;
}

// Contiguous, and re-materialised if a view starts at an address TMA cannot use.
torch::Tensor dense(const torch::Tensor& t) {
  torch::Tensor c = t.contiguous();
  if (reinterpret_cast<uintptr_t>(c.data_ptr()) % 16 != 0) c = c.clone();
  return c;
}

void check_qkv(const torch::Tensor& Q, const torch::Tensor& K, const torch::Tensor& V) {
  TORCH_CHECK(Q.is_cuda(), "Q must be a CUDA tensor");
  TORCH_CHECK(K.is_cuda() && V.is_cuda(), "K and V must be CUDA tensors");
  TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4, "Q, K, V must be [B, H, N, D]");
  TORCH_CHECK(K.sizes() == V.sizes(), "K and V must have the same shape");
  TORCH_CHECK(Q.size(0) == K.size(0) && Q.size(1) == K.size(1) && Q.size(3) == K.size(3),
              "Q and K must agree in B, H and D");
  TORCH_CHECK(Q.scalar_type() == K.scalar_type() && Q.scalar_type() == V.scalar_type(),
              "Q, K, V must have the same dtype");
  TORCH_CHECK(Q.device() == K.device() && Q.device() == V.device(), "Q, K, V must be on one device");
}

void check_like(const torch::Tensor& x, const torch::Tensor& ref, const char* name) {
  TORCH_CHECK(x.is_cuda() && x.device() == ref.device(), name, " must be on the same device as Q");
  TORCH_CHECK(x.sizes() == ref.sizes(), name, " has the wrong shape");
  TORCH_CHECK(x.scalar_type() == ref.scalar_type(), name, " has the wrong dtype");
}

attn_shape_t make_shape(const torch::Tensor& Q, const torch::Tensor& K, int window_size, int chunk_id,
                        int mask_mode, int impl) {
  attn_shape_t s;
  s.B = (int32_t)Q.size(0);
  s.H = (int32_t)Q.size(1);
  s.N_q = (int32_t)Q.size(2);
  s.N_kv = (int32_t)K.size(2);
  s.D = (int32_t)Q.size(3);
  s.window_size = window_size;
  s.chunk_id = chunk_id;
  s.mask_mode = mask_mode;
  s.dtype = dtype_code(Q);
  s.impl = impl;
  return s;
}

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == ATTN_OK, what, " failed (", rc, "): ", attn_b200_last_error());
}

// A kernel that gives up on a bounded wait stores a code in the device's status word and returns;
// its outputs are then meaningless.  This module registers one page-locked host word per device
// as a mirror of that status word (the failing kernel writes its code there too) and looks at it
// at the start of every call: a time-out of an earlier call is reported as an exception of the
// first call that starts after it, and the good path costs one read of host memory.
uint32_t* status_mirror(int device) {
  static torch::Tensor words[64];
  static std::mutex mu;
  TORCH_CHECK(device >= 0 && device < 64, "device index out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!words[device].defined()) {
    words[device] = torch::zeros({1}, torch::dtype(torch::kInt32).pinned_memory(true));
    check_rc(attn_b200_set_status_mirror(reinterpret_cast<uint32_t*>(words[device].data_ptr<int32_t>())),
             "attn_b200_set_status_mirror");
  }
  return reinterpret_cast<uint32_t*>(words[device].data_ptr<int32_t>());
}

void raise_if_earlier_call_timed_out(int device) {
  volatile uint32_t* w = status_mirror(device);
  if (*w == 0u) return;
  *w = 0u;
  uint32_t code = 0;
  int rc = attn_b200_device_status(&code);     // synchronises, reads and clears the device word
  char hex[16];
  snprintf(hex, sizeof(hex), "0x%x", code);
  TORCH_CHECK(rc == ATTN_OK && code == 0u, "an earlier attention kernel on this device gave up on a bounded wait (status ",
              hex, "); its outputs are invalid");
}

}  // namespace

std::vector<torch::Tensor> v7_forward_cuda(torch::Tensor Q, torch::Tensor K, torch::Tensor V, int window_size,
                                           int chunk_id, int mask_mode, int impl) {
  check_qkv(Q, K, V);
  c10::cuda::CUDAGuard guard(Q.device());
  raise_if_earlier_call_timed_out(Q.device().index());
  Q = dense(Q); K = dense(K); V = dense(V);
  attn_shape_t s = make_shape(Q, K, window_size, chunk_id, mask_mode, impl);
  auto O = torch::empty_like(Q);
  auto L = torch::empty({Q.size(0), Q.size(1), Q.size(2)}, Q.options().dtype(torch::kFloat32));
  check_rc(attn_b200_forward(&s, Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), L.data_ptr<float>(),
                             at::cuda::getCurrentCUDAStream().stream()),
           "v7_forward");
  return {O, L};
}

std::vector<torch::Tensor> v7_backward_cuda(torch::Tensor dO, torch::Tensor Q, torch::Tensor K, torch::Tensor V,
                                            torch::Tensor O, torch::Tensor L, int window_size, int chunk_id,
                                            int mask_mode, int impl) {
  check_qkv(Q, K, V);
  check_like(dO, Q, "dO");
  check_like(O, Q, "O");
  TORCH_CHECK(L.is_cuda() && L.scalar_type() == at::kFloat && L.numel() == Q.size(0) * Q.size(1) * Q.size(2),
              "L must be a float32 CUDA tensor of shape [B, H, N_q]");
  c10::cuda::CUDAGuard guard(Q.device());
  raise_if_earlier_call_timed_out(Q.device().index());
  dO = dense(dO); Q = dense(Q); K = dense(K); V = dense(V); O = dense(O); L = L.contiguous();
  attn_shape_t s = make_shape(Q, K, window_size, chunk_id, mask_mode, impl);
  auto dQ = torch::empty_like(Q);
  auto dK = torch::empty_like(K);
  auto dV = torch::empty_like(V);
  auto scratch = torch::empty({(int64_t)(attn_b200_backward_scratch_bytes(&s) / sizeof(float)) + 4},
                              Q.options().dtype(torch::kFloat32));
  check_rc(attn_b200_backward(&s, dO.data_ptr(), Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                              L.data_ptr<float>(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(),
                              scratch.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()),
           "v7_backward");
  return {dQ, dK, dV};
}

std::vector<torch::Tensor> v7_double_backward_cuda(torch::Tensor g_dQ, torch::Tensor g_dK, torch::Tensor g_dV,
                                                   torch::Tensor dO, torch::Tensor Q, torch::Tensor K,
                                                   torch::Tensor V, torch::Tensor O, torch::Tensor L,
                                                   int window_size, int chunk_id, int mask_mode, int impl) {
  check_qkv(Q, K, V);
  check_like(dO, Q, "dO");
  check_like(g_dQ, Q, "g_dQ");
  check_like(g_dK, K, "g_dK");
  check_like(g_dV, V, "g_dV");
  TORCH_CHECK(L.is_cuda() && L.scalar_type() == at::kFloat && L.numel() == Q.size(0) * Q.size(1) * Q.size(2),
              "L must be a float32 CUDA tensor of shape [B, H, N_q]");
  c10::cuda::CUDAGuard guard(Q.device());
  raise_if_earlier_call_timed_out(Q.device().index());
  g_dQ = dense(g_dQ); g_dK = dense(g_dK); g_dV = dense(g_dV);
  dO = dense(dO); Q = dense(Q); K = dense(K); V = dense(V); L = L.contiguous();
  attn_shape_t s = make_shape(Q, K, window_size, chunk_id, mask_mode, impl);
  auto g_dO = torch::empty_like(Q);
  auto g_Q = torch::empty_like(Q);
  auto g_K = torch::empty_like(K);
  auto g_V = torch::empty_like(V);
  auto scratch = torch::empty({(int64_t)(attn_b200_double_backward_scratch_bytes(&s) / sizeof(float)) + 4},
                              Q.options().dtype(torch::kFloat32));
  check_like(O, Q, "O");
  O = dense(O);
  check_rc(attn_b200_double_backward(&s, g_dQ.data_ptr(), g_dK.data_ptr(), g_dV.data_ptr(), dO.data_ptr(),
                                     Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), L.data_ptr<float>(),
                                     g_dO.data_ptr(), g_Q.data_ptr(), g_K.data_ptr(), g_V.data_ptr(),
                                     scratch.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()),
           "v7_double_backward");
  return {g_dO, g_Q, g_K, g_V};
}

// x [n_tok, H, d] -> [1, H, n_tok, d]: RMS normalisation (rows >= norm_from, when a weight is given),
// rotary embedding with freqs [positions, d/2, 2] (float32 cos, sin), layout change; one kernel.
torch::Tensor qk_norm_rope_cuda(torch::Tensor x, c10::optional<torch::Tensor> weight, torch::Tensor freqs, int pos0,
                                double eps, int norm_from) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3, "x must be a CUDA tensor [n_tok, H, d]");
  TORCH_CHECK(freqs.is_cuda() && freqs.scalar_type() == at::kFloat && freqs.dim() == 3 && freqs.size(2) == 2 &&
              freqs.size(1) * 2 == x.size(2), "freqs must be float32 [positions, d/2, 2]");
  TORCH_CHECK(pos0 >= 0 && pos0 + x.size(0) <= freqs.size(0), "positions out of the range of freqs");
  c10::cuda::CUDAGuard guard(x.device());
  x = x.contiguous();
  freqs = freqs.contiguous();
  torch::Tensor w;
  if (weight.has_value() && weight->defined()) {
    TORCH_CHECK(weight->is_cuda() && weight->numel() == x.size(2), "weight must be a CUDA tensor [d]");
    w = weight->to(x.scalar_type()).contiguous();
  }
  auto out = torch::empty({1, x.size(1), x.size(0), x.size(2)}, x.options());
  check_rc(attn_b200_qk_norm_rope(x.data_ptr(), w.defined() ? w.data_ptr() : nullptr, freqs.data_ptr<float>(), out.data_ptr(),
                                  (int32_t)x.size(0), (int32_t)x.size(1), (int32_t)x.size(2), pos0, norm_from, (float)eps,
                                  dtype_code(x), at::cuda::getCurrentCUDAStream().stream()),
           "qk_norm_rope");
  return out;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("qk_norm_rope", &qk_norm_rope_cuda, "fused RMS norm + rotary embedding + [n_tok,H,d] -> [1,H,n_tok,d]",
        py::arg("x"), py::arg("weight"), py::arg("freqs"), py::arg("pos0") = 0, py::arg("eps") = 1e-6, py::arg("norm_from") = 0);
  m.def("v7_forward", &v7_forward_cuda, "Rectangular sliding-window flash attention forward -> [O, L]",
        py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("window_size"), py::arg("chunk_id"),
        py::arg("mask_mode") = 0, py::arg("impl") = 0);
  m.def("v7_backward", &v7_backward_cuda, "Rectangular sliding-window flash attention backward -> [dQ, dK, dV]",
        py::arg("dO"), py::arg("Q"), py::arg("K"), py::arg("V"), py::arg("O"), py::arg("L"),
        py::arg("window_size"), py::arg("chunk_id"), py::arg("mask_mode") = 0, py::arg("impl") = 0);
  m.def("v7_double_backward", &v7_double_backward_cuda,
        "Rectangular sliding-window flash attention double backward -> [g_dO, g_Q, g_K, g_V]",
        py::arg("g_dQ"), py::arg("g_dK"), py::arg("g_dV"), py::arg("dO"), py::arg("Q"), py::arg("K"),
        py::arg("V"), py::arg("O"), py::arg("L"), py::arg("window_size"), py::arg("chunk_id"),
        py::arg("mask_mode") = 0, py::arg("impl") = 0);
  m.def("last_launch_count", &attn_b200_last_launch_count, "kernels launched by the last call of this thread");
  m.def("device_status", []() {
    uint32_t code = 0;
    int rc = attn_b200_device_status(&code);
    return py::make_tuple(rc, code);
  }, "(return code, status word) of the current device; synchronises");
}
