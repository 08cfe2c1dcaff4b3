// Entry point of the private native module _C_sm100 (the counterpart of the reference's
// csrc/registration.cpp): everything the module exports is registered by register_flashrwkv2_bindings.
#include "bindings.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, native_module) { register_flashrwkv2_bindings(native_module); }
