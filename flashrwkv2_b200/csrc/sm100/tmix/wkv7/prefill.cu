// Prefill entry of the C ABI: strategy selection between the tensor-core chunk kernel
// and the register-streaming recurrence.
#include "../../common.cuh"

#include <cstdlib>

namespace frwkv {

int check_wkv7_arguments(const char* who, const int32_t* cu, const int32_t* slots, float* pool,
                         const void* r, const void* w, const void* k, const void* v, const void* a,
                         const void* b, const void* bias, void* y, int n_seq, int total_tokens, int heads,
                         int io_dtype, int decay_mode, float scale);
int launch_recurrent_stream(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool,
                            const void* r, const void* w, const void* k, const void* v, const void* a,
                            const void* b, const void* bias, void* y, float* y_f32, int n_seq,
                            int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
                            int max_seqlen, int parts_override, cudaStream_t stream);
int launch_chunk64_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                      float scale, int max_seqlen, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                      cudaStream_t stream);
int launch_chunk32_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                      float scale, int32_t* error_flag, cudaStream_t stream);

size_t chunk_tc_workspace_bytes(int, int, int) { return 0; }

// Chunk length of the tensor-core kernel: 32-row chunks keep two CTAs resident per SM, 64-row chunks
// do more work per barrier.  FRWKV_PREFILL_CHUNK=32|64 overrides the default (tuning / test hook).
int launch_chunk_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                    const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                    float scale, int max_seqlen, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                    cudaStream_t stream) {
  int chunk = 32;
  if (const char* e = std::getenv("FRWKV_PREFILL_CHUNK")) chunk = std::atoi(e);
  if (chunk == 32)
    return launch_chunk32_tc(cu, slots, status, pool, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads,
                             io_dtype, decay_mode, scale, error_flag, stream);
  return launch_chunk64_tc(cu, slots, status, pool, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads,
                           io_dtype, decay_mode, scale, max_seqlen, workspace, workspace_bytes, error_flag, stream);
}

}  // namespace frwkv

extern "C" size_t frwkv_sm100_wkv7_prefill_workspace_bytes(int n_seq, int total_tokens, int heads) {
  return frwkv::chunk_tc_workspace_bytes(n_seq, total_tokens, heads);
}

extern "C" int frwkv_sm100_wkv7_prefill(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
    int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy, void* workspace,
    size_t workspace_bytes, int32_t* error_flag, void* stream) {
  using namespace frwkv;
  int rc = check_wkv7_arguments("wkv7_prefill", cu_seqlens, slots, state_pool, r, w, k, v, a, b, decay_bias, y,
                                n_seq, total_tokens, heads, io_dtype, decay_mode, scale);
  if (rc != FRWKV_OK) return rc;
  if (strategy != FRWKV_PREFILL_AUTO && strategy != FRWKV_PREFILL_RECURRENT && strategy != FRWKV_PREFILL_CHUNK_TC)
    return fail(FRWKV_ERR_ARGUMENT, "wkv7_prefill: unknown strategy %d", strategy);
  if (strategy == FRWKV_PREFILL_AUTO) {
    // fp32 tokens ask for 1e-5 agreement: that is the CUDA-core recurrence.  Rows of a
    // few tokens gain nothing from 64-row chunks.
    const bool tc = io_dtype != FRWKV_IO_FP32 && (max_seqlen <= 0 || max_seqlen >= 16);
    strategy = tc ? FRWKV_PREFILL_CHUNK_TC : FRWKV_PREFILL_RECURRENT;
  }
  if (strategy == FRWKV_PREFILL_CHUNK_TC) {
    if (io_dtype == FRWKV_IO_FP32)
      return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_prefill: the tensor-core chunk kernel takes float16 or bfloat16 tokens");
    return launch_chunk_tc(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32, n_seq,
                           total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, workspace,
                           workspace_bytes, error_flag, static_cast<cudaStream_t>(stream));
  }
  return launch_recurrent_stream(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32,
                                 n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0,
                                 static_cast<cudaStream_t>(stream));
}
