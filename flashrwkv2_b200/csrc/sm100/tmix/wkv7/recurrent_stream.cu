// WKV7 recurrence with the fp32 state streamed through registers (decode / short rows).
//
// One warp owns a (sequence, head, value-column part).  The pool layout is the
// reference's [slot, H, key, value] fp32 (rwkv-rs/FlashRWKV2
// csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:86-89,135-143), so a
// key row is 256 contiguous bytes.  With the 64 value columns split over P warps, a
// lane holds a float4 of COLS/4-th of a row and a warp instruction covers 32/LPR full
// row segments: every 128-bit access touches whole 32-byte sectors, each state element
// is read once and written once per call (the reference's T=1 kernel at :197-281 reads
// its column twice with 4-byte accesses at a 256-byte stride).  Both reductions over
// the key index (a^T S from the old state, r^T S' from the new one) are in-thread sums
// over the lane's rows followed by log2(32/LPR) xor-shuffles; nothing goes through
// shared memory and there is no block-level barrier.
//
// Per token (tests/tmix/wkv7/test.py:66-83 of the reference):
//   sa = a^T S;  S = diag(rho) S + b sa + k v^T;  y = scale * r^T S.
//
// The same kernel serves the reference's fp16-state decode contract (state pool in fp16, fp16 tokens;
// csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:244-340, oracle tests/tmix/wkv7/test.py:88-149):
//   delta = fp16(rho - 1 + dither(phase)),  phase = elapsed[slot] + head*64 + key + token offset,
//   S = fp16(S + S*delta + b sa + k v^T) evaluated in fp32,  y = fp16(scale * r^T S) from the rounded state.
// A key row is then 128 contiguous bytes and a lane moves 8 bytes of it per access; everything else is shared.
//
// One-token steps of large batches take the pipelined launch of the same kernel (recurrent_stream.cuh): a warp keeps
// its head and column part, walks several sequences, and has the cp.async of its next state (8 KB into shared
// memory, each lane copying what it reads back) in flight while it computes the current one.
#include "recurrent_stream.cuh"

namespace frwkv {

#ifdef FRWKV_TEST_HOOKS
int& test_recurrent_parts() {
  static int parts = 0;
  return parts;
}
int& test_pipeline_min_rounds() {
  static int rounds = 0;
  return rounds;
}
#endif

namespace {
// fp16-state contract: after the recurrence every active sequence's phase counter moves on by its token count
// (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:57-75 of the reference).  A separate launch: the
// recurrence's CTAs of all heads read the counter, so nobody may change it while they run.  Fail-closed like the
// recurrence: invalid metadata leaves every counter untouched.
__global__ void advance_elapsed_kernel(const int* __restrict__ cu, const int* __restrict__ slots,
                                       const int* __restrict__ status, int* __restrict__ elapsed, int n_seq) {
  // scheduled early under the recurrence kernel's tail (programmatic dependent launch), it waits here for that
  // kernel to complete: only then may a counter change
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (status != nullptr && status[0] != 0) return;
  const int active = status != nullptr ? status[2] : n_seq;
  const int seq = blockIdx.x * blockDim.x + threadIdx.x;
  if (seq >= n_seq || seq >= active) return;
  elapsed[slots[seq]] += cu[seq + 1] - cu[seq];
}
}  // namespace

// FRWKV_PDL=0 (read once) turns programmatic dependent launch off everywhere.
bool programmatic_launch_enabled() { return pdl_enabled(); }

// Shared argument checks of the recurrent and prefill entries.
int check_wkv7_arguments(const char* who, const int32_t* cu, const int32_t* slots, float* pool,
                         const void* r, const void* w, const void* k, const void* v, const void* a,
                         const void* b, const void* bias, void* y, const float* y_f32, int n_seq, int total_tokens,
                         int heads, int io_dtype, int decay_mode, float scale) {
  if (!cu || !slots || !pool || !r || !w || !k || !v || !a || !b || !y)
    return fail(FRWKV_ERR_ARGUMENT, "%s: cu_seqlens, slots, state_pool, r, w, k, v, a, b and y must be non-null", who);
  if (n_seq <= 0 || n_seq > 65535)
    return fail(FRWKV_ERR_ARGUMENT, "%s: sequence count must be in 1..65535, got %d", who, n_seq);
  if (total_tokens <= 0 || heads <= 0)
    return fail(FRWKV_ERR_ARGUMENT, "%s: total_tokens and heads must be positive", who);
  if (io_dtype != FRWKV_IO_BF16 && io_dtype != FRWKV_IO_FP16 && io_dtype != FRWKV_IO_FP32)
    return fail(FRWKV_ERR_ARGUMENT, "%s: unknown token dtype %d", who, io_dtype);
  if (decay_mode != FRWKV_DECAY_LOGITS && decay_mode != FRWKV_DECAY_RETENTION)
    return fail(FRWKV_ERR_ARGUMENT, "%s: unknown decay mode %d", who, decay_mode);
  if (bias != nullptr && decay_mode != FRWKV_DECAY_LOGITS)
    return fail(FRWKV_ERR_ARGUMENT, "%s: decay_bias only applies to decay logits", who);
  if (!(scale == scale) || scale - scale != 0.0f)
    return fail(FRWKV_ERR_ARGUMENT, "%s: scale must be finite", who);
  // every tensor is accessed with 16-byte vectors (decay_bias and y_f32 too, when given): a misaligned view
  // is rejected here instead of faulting on the device
  const void* ptrs[] = {r, w, k, v, a, b, y, pool, bias, y_f32};
  for (const void* q : ptrs)
    if ((reinterpret_cast<uintptr_t>(q) & 15) != 0)
      return fail(FRWKV_ERR_ARGUMENT, "%s: tensors must be 16-byte aligned", who);
  return FRWKV_OK;
}

int launch_recurrent_stream(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool,
                            const void* r, const void* w, const void* k, const void* v, const void* a,
                            const void* b, const void* bias, void* y, float* y_f32, int n_seq,
                            int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
                            int max_seqlen, int parts_override, int len_below, const void* const* gate,
                            cudaStream_t stream) {
  RecurrentParams p{cu, slots, status, pool, nullptr, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads,
                    scale, len_below, nullptr, nullptr, nullptr};
  if (gate != nullptr) {
    p.gate_kk = gate[0];
    p.gate_a0 = gate[1];
    p.gate_ka = gate[2];
  }
  // Launch shape.  Decode (one token per row): the state is loaded, used once and stored,
  // so all that matters is bytes in flight; two column parts per pair keep every access a
  // full 128-byte line.  Long rows are a latency-bound token loop: thinner warps (more of
  // them, fewer rows per lane, next token prefetched) shorten the per-token chain.
  const int parts = choose_parts(n_seq, heads, max_seqlen, parts_override);
  const bool prefetch = max_seqlen <= 0 || max_seqlen > 1;
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  if (gate != nullptr) {
    switch (io_dtype) {
      case FRWKV_IO_BF16: return dispatch_parts<__nv_bfloat16, float, true>(p, logits, parts, prefetch, stream);
      case FRWKV_IO_FP16: return dispatch_parts<__half, float, true>(p, logits, parts, prefetch, stream);
      default: return fail(FRWKV_ERR_UNSUPPORTED, "the fused kk/a-gate input form takes float16 or bfloat16 tokens");
    }
  }
  switch (io_dtype) {
    case FRWKV_IO_BF16: return dispatch_parts<__nv_bfloat16>(p, logits, parts, prefetch, stream);
    case FRWKV_IO_FP16: return dispatch_parts<__half>(p, logits, parts, prefetch, stream);
    default: return dispatch_parts<float>(p, logits, parts, prefetch, stream);
  }
}

int launch_decode_fp16_state(const int32_t* cu, const int32_t* slots, const int32_t* status, const int32_t* elapsed,
                             void* pool, int pool_slots, const void* r, const void* w, const void* k, const void* v,
                             const void* a, const void* b, const void* bias, void* y, int n_seq, int total_tokens,
                             int heads, int decay_mode, float scale, int32_t* error_flag, cudaStream_t stream);

// One-token steps (max_seqlen == 1) go to the TMA-fed ring kernel, everything else to the register-streaming
// kernel; FRWKV_FP16_STATE_KERNEL=stream forces the latter (tuning hook, read once).
int launch_recurrent_fp16_state(const int32_t* cu, const int32_t* slots, const int32_t* status, int32_t* elapsed,
                                void* pool, int pool_slots, const void* r, const void* w, const void* k,
                                const void* v, const void* a, const void* b, const void* bias, void* y, int n_seq,
                                int total_tokens, int heads, int decay_mode, float scale, int max_seqlen,
                                int32_t* error_flag, cudaStream_t stream) {
  static const bool force_stream = [] {
    const char* e = std::getenv("FRWKV_FP16_STATE_KERNEL");
    return e != nullptr && e[0] == 's';
  }();
  int rc;
  if (max_seqlen == 1 && !force_stream) {
    rc = launch_decode_fp16_state(cu, slots, status, elapsed, pool, pool_slots, r, w, k, v, a, b, bias, y, n_seq,
                                  total_tokens, heads, decay_mode, scale, error_flag, stream);
  } else {
    RecurrentParams p{cu, slots, status, pool, elapsed, r, w, k, v, a, b, bias, y, nullptr, n_seq, total_tokens,
                      heads, scale, 0, nullptr, nullptr, nullptr};
    const int parts = choose_parts(n_seq, heads, max_seqlen, 0);
    const bool prefetch = max_seqlen <= 0 || max_seqlen > 1;
    rc = dispatch_parts<__half, __half>(p, decay_mode == FRWKV_DECAY_LOGITS, parts, prefetch, stream);
  }
  if (rc != FRWKV_OK) return rc;
  // launched so that it is scheduled under the recurrence kernel's tail; it waits for that kernel's completion
  // (griddepcontrol.wait) before it touches a counter
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((n_seq + 255) / 256);
  config.blockDim = dim3(256);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, advance_elapsed_kernel, static_cast<const int*>(cu),
                                             static_cast<const int*>(slots), static_cast<const int*>(status), elapsed,
                                             n_seq);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "advance_elapsed_kernel: %s", cudaGetErrorString(err));
  return check_launch("advance_elapsed_kernel");
}

}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_recurrent_fp16_state(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, int32_t* elapsed_pool,
    void* state_pool_f16, int pool_slots, const void* r, const void* w, const void* k, const void* v, const void* a,
    const void* b, const void* decay_bias, void* y, int n_seq, int total_tokens, int heads, int decay_mode,
    float scale, int max_seqlen, int32_t* error_flag, void* stream) {
  using namespace frwkv;
  if (elapsed_pool == nullptr) return fail(FRWKV_ERR_ARGUMENT, "wkv7_recurrent_fp16_state: elapsed_pool must be non-null");
  if (pool_slots <= 0) return fail(FRWKV_ERR_ARGUMENT, "wkv7_recurrent_fp16_state: pool_slots must be positive");
  if ((reinterpret_cast<uintptr_t>(state_pool_f16) & 1023) != 0 && max_seqlen == 1)
    max_seqlen = 0;  // the TMA-fed kernel wants the pool 1024-byte aligned; any other pool takes the streaming kernel
  int rc = check_wkv7_arguments("wkv7_recurrent_fp16_state", cu_seqlens, slots, static_cast<float*>(state_pool_f16), r, w,
                                k, v, a, b, decay_bias, y, nullptr, n_seq, total_tokens, heads, FRWKV_IO_FP16,
                                decay_mode, scale);
  if (rc != FRWKV_OK) return rc;
  return launch_recurrent_fp16_state(cu_seqlens, slots, status, elapsed_pool, state_pool_f16, pool_slots, r, w, k, v,
                                     a, b, decay_bias, y, n_seq, total_tokens, heads, decay_mode, scale, max_seqlen,
                                     error_flag, static_cast<cudaStream_t>(stream));
}

extern "C" int frwkv_sm100_wkv7_recurrent(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
    int io_dtype, int decay_mode, float scale, int max_seqlen, void* stream) {
  using namespace frwkv;
  int rc = check_wkv7_arguments("wkv7_recurrent", cu_seqlens, slots, state_pool, r, w, k, v, a, b, decay_bias,
                                y, y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale);
  if (rc != FRWKV_OK) return rc;
  return launch_recurrent_stream(cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32,
                                 n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0, 0, nullptr,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int frwkv_sm100_wkv7_recurrent_fused_gate(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k_raw, const void* v, const void* a12, const void* gate_k_k,
    const void* gate_a0, const void* gate_k_a, const void* decay_bias, void* y, float* y_f32, int n_seq,
    int total_tokens, int heads, int io_dtype, int decay_mode, float scale, int max_seqlen, void* stream) {
  using namespace frwkv;
  if (!gate_k_k || !gate_a0 || !gate_k_a)
    return fail(FRWKV_ERR_ARGUMENT, "wkv7_recurrent_fused_gate: k_k, a0 and k_a must be non-null");
  int rc = check_wkv7_arguments("wkv7_recurrent_fused_gate", cu_seqlens, slots, state_pool, r, w, k_raw, v, a12, a12,
                                decay_bias, y, y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale);
  if (rc != FRWKV_OK) return rc;
  const void* gate[3] = {gate_k_k, gate_a0, gate_k_a};
  for (const void* q : gate)
    if ((reinterpret_cast<uintptr_t>(q) & 15) != 0)
      return fail(FRWKV_ERR_ARGUMENT, "wkv7_recurrent_fused_gate: tensors must be 16-byte aligned");
  return launch_recurrent_stream(cu_seqlens, slots, status, state_pool, r, w, k_raw, v, a12, nullptr, decay_bias, y,
                                 y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0, 0,
                                 gate, static_cast<cudaStream_t>(stream));
}

#ifdef FRWKV_TEST_HOOKS
// Test build only: force the column split (2, 4 or 8; 0 = automatic) of the recurrence kernel's next launches.
extern "C" void frwkv_sm100_test_recurrent_parts(int parts) { frwkv::test_recurrent_parts() = parts; }
// Test build only: sequences per resident warp from which one-token steps take the pipelined launch (0 = default).
extern "C" void frwkv_sm100_test_pipeline_min_rounds(int rounds) { frwkv::test_pipeline_min_rounds() = rounds; }
#endif
