// Shared host/device helpers of the sm_100a WKV7 backend.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../../include/frwkv_sm100.h"

namespace frwkv {

// Thread-local text of the last rejected call; read through frwkv_sm100_last_error().
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
// Returns FRWKV_OK or records the CUDA error of the launch that just happened.
int check_launch(const char* what);

constexpr int kHeadDim = 64;
// exp(-1/2) * log2(e) and log2(e): rho = exp2(-kRateLog2e / (1 + exp2(-kLog2e * x)))
constexpr float kRateLog2e = 0.8750387749145276f;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRate = 0.6065306597126334f;

__device__ __forceinline__ float retention_from_logit(float x) {
  return exp2f(-kRateLog2e / (1.0f + exp2f(-kLog2e * x)));
}
// The same with the SFU approximations (ex2.approx, rcp.approx: relative error about 2^-22 each), for 16-bit tokens.
__device__ __forceinline__ float retention_from_logit_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-kLog2e * x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fdividef(-kRateLog2e, 1.0f + e)));
  return r;
}
// log(rho) for a raw logit: -exp(-1/2) * sigmoid(x)
__device__ __forceinline__ float log_retention_from_logit(float x) {
  return -kRate / (1.0f + exp2f(-kLog2e * x));
}

__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(float x) { return x; }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }

// NaN fill of the whole output when the metadata status is nonzero (fail-closed).
template <typename io_t>
__device__ __forceinline__ void fill_output_nan(io_t* y, float* y_f32, long long elements,
                                                long long thread, long long threads) {
  const float qnan = __int_as_float(0x7fffffff);
  for (long long i = thread; i < elements; i += threads) {
    y[i] = from_f32<io_t>(qnan);
    if (y_f32 != nullptr) y_f32[i] = qnan;
  }
}

}  // namespace frwkv
