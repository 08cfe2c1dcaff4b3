// Per-backend list of registered operator families (rwkv-rs/FlashRWKV2 csrc/bindings.cpp:6-49 has the
// same ladder for its SM90 and SM120 backends; this build adds the SM100 branch, WKV7 only).
#include "bindings.h"

void register_flashrwkv2_bindings(py::module_& module) {
#if defined(FLASHRWKV_BACKEND_SM100)
  register_infer_tmix_wkv7_recurrent_fp32io16_bindings(module);
  register_rl_infctx_tmix_wkv7_chunk_forward_bindings(module);
  register_pretrain_tmix_wkv7_recurrent_bindings(module);
#else
#error "this tree builds the SM100 backend only: define FLASHRWKV_BACKEND_SM100"
#endif
}
