// Prefill entry of the C ABI: strategy selection between the tensor-core chunk kernel
// and the register-streaming recurrence.
#include "../../common.cuh"


namespace frwkv {

int check_wkv7_arguments(const char* who, const int32_t* cu, const int32_t* slots, float* pool,
                         const void* r, const void* w, const void* k, const void* v, const void* a,
                         const void* b, const void* bias, void* y, const float* y_f32, int n_seq, int total_tokens,
                         int heads, int io_dtype, int decay_mode, float scale);
int launch_recurrent_stream(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool,
                            const void* r, const void* w, const void* k, const void* v, const void* a,
                            const void* b, const void* bias, void* y, float* y_f32, int n_seq,
                            int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
                            int max_seqlen, int parts_override, int len_below, const void* const* gate,
                            cudaStream_t stream);
int launch_chunk32_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                      float scale, const int32_t* order, int len_from, int32_t* error_flag, const void* const* gate,
                      cudaStream_t stream);

namespace {

// Ragged batches: CTAs are handed to SMs in grid order, and a CTA's run time is proportional to its
// sequence length, so the tail of the launch is as long as whichever long sequence happens to start
// last.  With the sequences ranked longest-first the tail shrinks to the shortest ones.  The ranking is
// one small kernel (rank of i = number of sequences that are longer, ties by index) writing
// order[rank] = i into caller-provided scratch; batches above kMaxOrdered sequences keep their natural
// order (their tail is negligible and an all-pairs ranking would not be).
constexpr int kShortRow = 16;  // rows shorter than this go to the recurrence kernel under AUTO
constexpr int kMaxOrdered = 2048;
constexpr int kOrderThreads = 1024;

__global__ void __launch_bounds__(kOrderThreads) sequence_order_kernel(const int* __restrict__ cu,
                                                                       const int* __restrict__ status, int n_seq,
                                                                       int* __restrict__ order) {
  __shared__ int len[kMaxOrdered];
  const bool valid = status == nullptr || status[0] == 0;
  const int active = status == nullptr ? n_seq : status[2];
  for (int i = threadIdx.x; i < n_seq; i += kOrderThreads)
    len[i] = (valid && i < active) ? max(cu[i + 1] - cu[i], 0) : 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_seq; i += kOrderThreads) {
    const int mine = len[i];
    int rank = 0;
    for (int j = 0; j < n_seq; ++j) rank += (len[j] > mine) || (len[j] == mine && j < i);
    order[rank] = i;
  }
}

}  // namespace

size_t chunk_tc_workspace_bytes(int n_seq, int, int) {
  return n_seq > 1 && n_seq <= kMaxOrdered ? static_cast<size_t>(n_seq) * sizeof(int) : 0;
}

// The tensor-core path: optional longest-first ranking, then the 32-row chunk kernel.
int launch_chunk_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                    const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                    float scale, int max_seqlen, int len_from, void* workspace, size_t workspace_bytes,
                    int32_t* error_flag, const void* const* gate, cudaStream_t stream) {
  (void)max_seqlen;
  const int32_t* order = nullptr;
  const size_t need = chunk_tc_workspace_bytes(n_seq, total_tokens, heads);
  if (need > 0 && workspace != nullptr) {  // no scratch given: natural order
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 3) != 0)
      return fail(FRWKV_ERR_WORKSPACE, "wkv7_prefill: workspace of %zu bytes (4-byte aligned) needed, got %zu", need,
                  workspace_bytes);
    sequence_order_kernel<<<1, kOrderThreads, 0, stream>>>(cu, status, n_seq, static_cast<int*>(workspace));
    const int rc = check_launch("sequence_order_kernel");
    if (rc != FRWKV_OK) return rc;
    order = static_cast<const int32_t*>(workspace);
  }
  return launch_chunk32_tc(cu, slots, status, pool, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads,
                           io_dtype, decay_mode, scale, order, len_from, error_flag, gate, stream);
}

}  // namespace frwkv

extern "C" size_t frwkv_sm100_wkv7_prefill_workspace_bytes(int n_seq, int total_tokens, int heads) {
  return frwkv::chunk_tc_workspace_bytes(n_seq, total_tokens, heads);
}

namespace frwkv {
namespace {

// Shared body of the two prefill entries.  `gate` = {k_k, a0, k_a} of the fused kk / a-gate producer (then k is the
// raw key projection, a the gate logits a12 and b is not read), or nullptr.
int prefill_impl(const char* who, const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status,
                 float* state_pool, const void* r, const void* w, const void* k, const void* v, const void* a,
                 const void* b, const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
                 int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy, void* workspace,
                 size_t workspace_bytes, int32_t* error_flag, const void* const* gate, cudaStream_t s) {
  int rc = check_wkv7_arguments(who, cu_seqlens, slots, state_pool, r, w, k, v, a, gate != nullptr ? a : b,
                                decay_bias, y, y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale);
  if (rc != FRWKV_OK) return rc;
  if (strategy != FRWKV_PREFILL_AUTO && strategy != FRWKV_PREFILL_RECURRENT && strategy != FRWKV_PREFILL_CHUNK_TC)
    return fail(FRWKV_ERR_ARGUMENT, "%s: unknown strategy %d", who, strategy);
  if (gate != nullptr) {
    for (int i = 0; i < 3; ++i)
      if (gate[i] == nullptr || (reinterpret_cast<uintptr_t>(gate[i]) & 15) != 0)
        return fail(FRWKV_ERR_ARGUMENT, "%s: k_k, a0 and k_a must be non-null and 16-byte aligned", who);
    if (io_dtype == FRWKV_IO_FP32)
      return fail(FRWKV_ERR_UNSUPPORTED, "%s: the fused kk/a-gate input form takes float16 or bfloat16 tokens", who);
  }
  if (strategy == FRWKV_PREFILL_AUTO) {
    // fp32 tokens ask for 1e-5 agreement: that is the CUDA-core recurrence.  Rows of a few tokens gain
    // nothing from 32-row chunks either.  A batch that may hold both kinds (continuous batching: decode
    // rows next to a prompt) is split by length: two launches, each kernel skipping the other's rows.
    if (io_dtype == FRWKV_IO_FP32 || (max_seqlen > 0 && max_seqlen < kShortRow))
      strategy = FRWKV_PREFILL_RECURRENT;
    else {
      rc = launch_recurrent_stream(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32,
                                   n_seq, total_tokens, heads, io_dtype, decay_mode, scale, kShortRow - 1, 0,
                                   kShortRow, gate, s);
      if (rc != FRWKV_OK) return rc;
      return launch_chunk_tc(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32, n_seq,
                             total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, kShortRow, workspace,
                             workspace_bytes, error_flag, gate, s);
    }
  }
  if (strategy == FRWKV_PREFILL_CHUNK_TC) {
    if (io_dtype == FRWKV_IO_FP32)
      return fail(FRWKV_ERR_UNSUPPORTED, "%s: the tensor-core chunk kernel takes float16 or bfloat16 tokens", who);
    return launch_chunk_tc(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32, n_seq,
                           total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0, workspace,
                           workspace_bytes, error_flag, gate, s);
  }
  return launch_recurrent_stream(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32,
                                 n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0, 0, gate, s);
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_prefill(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
    int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy, void* workspace,
    size_t workspace_bytes, int32_t* error_flag, void* stream) {
  return frwkv::prefill_impl("wkv7_prefill", cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y,
                             y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, strategy,
                             workspace, workspace_bytes, error_flag, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int frwkv_sm100_wkv7_prefill_fused_gate(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k_raw, const void* v, const void* a12, const void* gate_k_k,
    const void* gate_a0, const void* gate_k_a, const void* decay_bias, void* y, float* y_f32, int n_seq,
    int total_tokens, int heads, int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy,
    void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream) {
  const void* gate[3] = {gate_k_k, gate_a0, gate_k_a};
  return frwkv::prefill_impl("wkv7_prefill_fused_gate", cu_seqlens, slots, status, state_pool, r, w, k_raw, v, a12,
                             nullptr, decay_bias, y, y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale,
                             max_seqlen, strategy, workspace, workspace_bytes, error_flag, gate,
                             static_cast<cudaStream_t>(stream));
}
