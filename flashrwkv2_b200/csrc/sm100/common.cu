// Error reporting of the C ABI.
#include "common.cuh"

namespace frwkv {

char* last_error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, args);
  va_end(args);
  return code;
}

int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  return FRWKV_OK;
}

}  // namespace frwkv

extern "C" int frwkv_sm100_abi_version(void) { return FRWKV_SM100_ABI_VERSION; }
extern "C" const char* frwkv_sm100_last_error(void) { return frwkv::last_error_buffer(); }
