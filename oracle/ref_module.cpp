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

PYBIND11_MODULE(_C_ref, module) {
  module.doc() = "reference FlashRWKV2 WKV7 kernels, built unmodified for comparison";
  register_infer_tmix_wkv7_recurrent_fp32io16_bindings(module);
  register_rl_infctx_tmix_wkv7_chunk_forward_bindings(module);
}
