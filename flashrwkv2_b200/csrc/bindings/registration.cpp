// Module entry of the private native module; same shape as rwkv-rs/FlashRWKV2 csrc/registration.cpp:6-8.
#include "bindings.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) {
  register_flashrwkv2_bindings(module);
}
