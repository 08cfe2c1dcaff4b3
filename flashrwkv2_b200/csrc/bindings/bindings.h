// pybind registration points of the private native module (_C_sm100).
// Shape follows rwkv-rs/FlashRWKV2 csrc/bindings.h:8-43, csrc/bindings.cpp:6-49: one register_*
// function per operator family, selected per backend by a preprocessor ladder.
#pragma once

#include <torch/extension.h>

void register_flashrwkv2_bindings(py::module_& module);
void register_infer_tmix_wkv7_recurrent_fp32io16_bindings(py::module_& module);
void register_rl_infctx_tmix_wkv7_chunk_forward_bindings(py::module_& module);
void register_pretrain_tmix_wkv7_recurrent_bindings(py::module_& module);
