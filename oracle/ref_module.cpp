// Test infrastructure, not product code.
//
// Module entry for a build of the reference project's own WKV7 CUDA sources (arch-neutral CUDA C++, compiled for
// sm_100 where they lie in a reference checkout by oracle/build_ref.py).  The two registration functions are the
// reference's (csrc/bindings.h: register_infer_tmix_wkv7_recurrent_fp32io16_bindings and
// register_rl_infctx_tmix_wkv7_chunk_forward_bindings); the resulting module exposes the same pybind symbols as the
// product's _C_sm100, so tests and the bench can run both on identical device tensors.
#include <torch/extension.h>

void register_infer_tmix_wkv7_recurrent_fp32io16_bindings(py::module_&);
void register_rl_infctx_tmix_wkv7_chunk_forward_bindings(py::module_&);
void register_infer_tmix_wkv7_recurrent_fp16_bindings(py::module_&);
void register_pretrain_tmix_wkv7_recurrent_bindings(py::module_&);  // the training operator (forward + backward)
// host launcher of the reference's kk/a-gate kernels
// (csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/infer_fp16_forward_varlen.cu:209-260); its own binding lives in the
// wkv_prepare operator, which is not built here
void tmix_kk_a_gate_forward_varlen_cuda(int batch_size, int max_seqlen, int total_tokens, int channels, int heads,
                                        int head_size, torch::Tensor k, torch::Tensor k_k, torch::Tensor a0,
                                        torch::Tensor a12, torch::Tensor k_a, torch::Tensor new_k, torch::Tensor neg_kk,
                                        torch::Tensor kka);
// host launcher of the reference's elementwise readout kernels (head norm, r.k residual, gate;
// csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:306-386); its own binding adds the output projection
void tmix_lnx_rkvres_xg_forward_varlen_cuda(int batch_size, int max_seqlen, int total_tokens, int channels, int heads,
                                            int head_size, torch::Tensor x, torch::Tensor r, torch::Tensor k,
                                            torch::Tensor v, torch::Tensor r_k, torch::Tensor weight,
                                            torch::Tensor bias, torch::Tensor g, torch::Tensor output);

PYBIND11_MODULE(_C_ref, module) {
  module.doc() = "reference FlashRWKV2 WKV7 kernels, built unmodified for comparison";
  register_infer_tmix_wkv7_recurrent_fp32io16_bindings(module);
  register_rl_infctx_tmix_wkv7_chunk_forward_bindings(module);
  register_infer_tmix_wkv7_recurrent_fp16_bindings(module);
  register_pretrain_tmix_wkv7_recurrent_bindings(module);
  module.def("tmix_kk_a_gate_forward_varlen", &tmix_kk_a_gate_forward_varlen_cuda, py::arg("batch_size"),
             py::arg("max_seqlen"), py::arg("total_tokens"), py::arg("channels"), py::arg("heads"), py::arg("head_size"),
             py::arg("k"), py::arg("k_k"), py::arg("a0"), py::arg("a12"), py::arg("k_a"), py::arg("new_k"),
             py::arg("neg_kk"), py::arg("kka"));
  module.def("tmix_lnx_rkvres_xg_forward_varlen", &tmix_lnx_rkvres_xg_forward_varlen_cuda, py::arg("batch_size"),
             py::arg("max_seqlen"), py::arg("total_tokens"), py::arg("channels"), py::arg("heads"), py::arg("head_size"),
             py::arg("x"), py::arg("r"), py::arg("k"), py::arg("v"), py::arg("r_k"), py::arg("weight"), py::arg("bias"),
             py::arg("g"), py::arg("output"));
}
