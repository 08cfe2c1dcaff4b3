// Native symbols of the WKV7 training operator: names, argument order and checks of the reference's
// pretrain_tmix_wkv7_recurrent_forward / _backward (rwkv-rs/FlashRWKV2
// csrc/sm120/tmix/wkv7/pretrain_recurrent_bf16_forward.cpp), over the C ABI of libfrwkv_sm100.so.  D = 64 only.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "bindings.h"
#include "frwkv_sm100.h"

namespace {

void check_dense(const torch::Tensor& t, const torch::Tensor& like, const char* name, c10::ScalarType dtype) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, " must be contiguous CUDA");
  TORCH_CHECK(t.scalar_type() == dtype, name, " has the wrong dtype");
  TORCH_CHECK(t.device() == like.device(), name, " must share r's device");
}

struct Shape {
  int batch, tokens, heads;
};

Shape check_inputs(const torch::Tensor& r, const std::initializer_list<std::pair<const torch::Tensor*, const char*>>& same,
                   int64_t head_size) {
  TORCH_CHECK(head_size == 64, "this backend builds the WKV7 training operator for head_size 64 only");
  TORCH_CHECK(r.dim() == 4 && r.size(3) == 64 && r.numel() > 0, "r must have shape [B,T,H,64]");
  check_dense(r, r, "r", torch::kBFloat16);
  for (const auto& item : same) {
    check_dense(*item.first, r, item.second, torch::kBFloat16);
    TORCH_CHECK(item.first->sizes() == r.sizes(), item.second, " must match r's shape");
  }
  TORCH_CHECK(r.size(1) % 16 == 0, "T must be divisible by the chunk length 16");
  return Shape{static_cast<int>(r.size(0)), static_cast<int>(r.size(1)), static_cast<int>(r.size(2))};
}

void check_saved(const torch::Tensor& boundary, const torch::Tensor& state_dot_a, const torch::Tensor& r, const Shape& s) {
  check_dense(boundary, r, "boundary", torch::kFloat32);
  check_dense(state_dot_a, r, "state_dot_a", torch::kFloat32);
  TORCH_CHECK(boundary.dim() == 5 && boundary.size(0) == s.batch && boundary.size(1) == s.heads &&
                  boundary.size(2) == s.tokens / 16 && boundary.size(3) == 64 && boundary.size(4) == 64,
              "boundary must have shape [B,H,T/16,64,64]");
  TORCH_CHECK(state_dot_a.sizes() == r.sizes(), "state_dot_a must have shape [B,T,H,64]");
}

void check_abi(int rc) { TORCH_CHECK(rc == 0, frwkv_sm100_last_error()); }

void pretrain_forward(torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a,
                      torch::Tensor b, torch::Tensor output, torch::Tensor boundary, torch::Tensor state_dot_a,
                      int64_t head_size) {
  const Shape s = check_inputs(r, {{&w, "w"}, {&k, "k"}, {&v, "v"}, {&a, "a"}, {&b, "b"}, {&output, "output"}}, head_size);
  check_saved(boundary, state_dot_a, r, s);
  const c10::cuda::CUDAGuard guard(r.device());
  check_abi(frwkv_sm100_wkv7_pretrain_forward(r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                              b.data_ptr(), output.data_ptr(), boundary.data_ptr<float>(),
                                              state_dot_a.data_ptr<float>(), s.batch, s.tokens, s.heads,
                                              at::cuda::getCurrentCUDAStream(r.device().index()).stream()));
}

void pretrain_backward(torch::Tensor r, torch::Tensor w, torch::Tensor k, torch::Tensor v, torch::Tensor a,
                       torch::Tensor b, torch::Tensor grad_output, torch::Tensor boundary, torch::Tensor state_dot_a,
                       torch::Tensor grad_r, torch::Tensor grad_w, torch::Tensor grad_k, torch::Tensor grad_v,
                       torch::Tensor grad_a, torch::Tensor grad_b, int64_t head_size) {
  const Shape s = check_inputs(r,
                               {{&w, "w"}, {&k, "k"}, {&v, "v"}, {&a, "a"}, {&b, "b"}, {&grad_output, "grad_output"},
                                {&grad_r, "grad_r"}, {&grad_w, "grad_w"}, {&grad_k, "grad_k"}, {&grad_v, "grad_v"},
                                {&grad_a, "grad_a"}, {&grad_b, "grad_b"}},
                               head_size);
  check_saved(boundary, state_dot_a, r, s);
  const c10::cuda::CUDAGuard guard(r.device());
  check_abi(frwkv_sm100_wkv7_pretrain_backward(
      r.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(), grad_output.data_ptr(),
      boundary.data_ptr<float>(), state_dot_a.data_ptr<float>(), grad_r.data_ptr(), grad_w.data_ptr(), grad_k.data_ptr(),
      grad_v.data_ptr(), grad_a.data_ptr(), grad_b.data_ptr(), s.batch, s.tokens, s.heads,
      at::cuda::getCurrentCUDAStream(r.device().index()).stream()));
}

}  // namespace

void register_pretrain_tmix_wkv7_recurrent_bindings(py::module_& module) {
  module.def("pretrain_tmix_wkv7_recurrent_forward", &pretrain_forward, "WKV7 training forward with state checkpoints",
             py::arg("r"), py::arg("w"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"),
             py::arg("boundary"), py::arg("state_dot_a"), py::arg("head_size"));
  module.def("pretrain_tmix_wkv7_recurrent_backward", &pretrain_backward, "WKV7 training backward",
             py::arg("r"), py::arg("w"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("grad_output"),
             py::arg("boundary"), py::arg("state_dot_a"), py::arg("grad_r"), py::arg("grad_w"), py::arg("grad_k"),
             py::arg("grad_v"), py::arg("grad_a"), py::arg("grad_b"), py::arg("head_size"));
}
