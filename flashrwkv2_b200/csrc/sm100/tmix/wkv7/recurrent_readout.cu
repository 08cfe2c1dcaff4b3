// WKV7 recurrence with the readout's elementwise stage as its epilogue (decode / short rows).
//
// The reference runs `wkv7 -> readout` as two operators: the recurrence stores y, and the readout's first kernel
// (rwkv-rs/FlashRWKV2 csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:135-196; oracle
// tests/tmix/readout/test.py:43-66) reads y, r, k, v and the output gate again to form, per (token, head),
//   x = (headnorm(y) * ln_w + ln_b + (sum_c r_c k_c r_k_c) * v) * gate
// which then feeds the output projection.  Here that stage runs on the y row while it is still in registers:
// r, k and v are already on chip, the gate row is the only extra read, and x replaces y as the stored result
// (y itself is stored only when the caller asks for it).  The normalisation sees y rounded to the token dtype,
// exactly what the two-operator pipeline stores and reads back.
//
// The 64 value columns of a (sequence, head) are split over 2 or 4 warps of one CTA; each reduces its columns to
// (mean, sum of squared deviations) and the warps exchange those two numbers through shared memory with one named
// barrier per token.  The key used in the residual is the key the recurrence consumes (the gated key of the fused
// kk / a-gate form).  One-token steps of large batches take the pipelined launch (recurrent_stream.cuh): the extra
// instructions of the epilogue then run under the flight of the warp's next state, and the step costs what the
// plain recurrence costs.
#include "recurrent_stream.cuh"

namespace frwkv {

int check_wkv7_arguments(const char* who, const int32_t* cu, const int32_t* slots, float* pool,
                         const void* r, const void* w, const void* k, const void* v, const void* a,
                         const void* b, const void* bias, void* y, const float* y_f32, int n_seq, int total_tokens,
                         int heads, int io_dtype, int decay_mode, float scale);

namespace {

template <typename io_t, bool FUSED>
int dispatch_readout(const RecurrentParams& p, bool logits, int parts, bool prefetch, cudaStream_t stream) {
  if (!prefetch) {
    if (parts == 2) {
      const int rc = launch_pipelined<io_t, FUSED, true>(p, logits, stream);
      if (rc >= 0) return rc;
    }
    if (parts == 2) return launch<io_t, float, 2, false, FUSED, true>(p, logits, stream);
    return launch<io_t, float, 4, false, FUSED, true>(p, logits, stream);
  }
  if (parts == 2) return launch<io_t, float, 2, true, FUSED, true>(p, logits, stream);
  return launch<io_t, float, 4, true, FUSED, true>(p, logits, stream);
}

}  // namespace

int launch_recurrent_readout(const RecurrentParams& params, int io_dtype, int decay_mode, int max_seqlen,
                             cudaStream_t stream) {
  // all column parts of a pair must sit in one CTA: at most 4 (the kernel without epilogue goes to 8 for long rows)
  int parts = choose_parts(params.n_seq, params.heads, max_seqlen, 0);
  if (parts > 4) parts = 4;
  const bool prefetch = max_seqlen <= 0 || max_seqlen > 1;
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  const bool fused = params.gate_kk != nullptr;
  if (io_dtype == FRWKV_IO_BF16)
    return fused ? dispatch_readout<__nv_bfloat16, true>(params, logits, parts, prefetch, stream)
                 : dispatch_readout<__nv_bfloat16, false>(params, logits, parts, prefetch, stream);
  if (io_dtype == FRWKV_IO_FP16)
    return fused ? dispatch_readout<__half, true>(params, logits, parts, prefetch, stream)
                 : dispatch_readout<__half, false>(params, logits, parts, prefetch, stream);
  return fail(FRWKV_ERR_UNSUPPORTED, "the readout epilogue takes float16 or bfloat16 tokens");
}

}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_recurrent_readout(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* gate_k_k, const void* gate_a0, const void* gate_k_a, const void* decay_bias,
    const void* out_gate, const void* r_k, const void* ln_weight, const void* ln_bias, void* out,
    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
    int max_seqlen, void* stream) {
  using namespace frwkv;
  const char* who = "wkv7_recurrent_readout";
  const int given = (gate_k_k != nullptr) + (gate_a0 != nullptr) + (gate_k_a != nullptr);
  if (given != 0 && given != 3)
    return fail(FRWKV_ERR_ARGUMENT, "%s: k_k, a0 and k_a must be given together or not at all", who);
  const bool fused = given == 3;
  if (!out_gate || !r_k || !ln_weight || !ln_bias || !out)
    return fail(FRWKV_ERR_ARGUMENT, "%s: out_gate, r_k, ln_weight, ln_bias and out must be non-null", who);
  int rc = check_wkv7_arguments(who, cu_seqlens, slots, state_pool, r, w, k, v, a, fused ? a : b, decay_bias,
                                y != nullptr ? y : out, y_f32, n_seq, total_tokens, heads, io_dtype, decay_mode,
                                scale);
  if (rc != FRWKV_OK) return rc;
  const void* more[] = {gate_k_k, gate_a0, gate_k_a, out_gate, r_k, ln_weight, ln_bias, out};
  for (const void* q : more)
    if ((reinterpret_cast<uintptr_t>(q) & 15) != 0)
      return fail(FRWKV_ERR_ARGUMENT, "%s: tensors must be 16-byte aligned", who);
  RecurrentParams p{cu_seqlens, slots, status, state_pool, nullptr, r, w, k, v, a, fused ? nullptr : b, decay_bias, y,
                    y_f32, n_seq, total_tokens, heads, scale, 0, gate_k_k, gate_a0, gate_k_a, out_gate, r_k,
                    ln_weight, ln_bias, out};
  return launch_recurrent_readout(p, io_dtype, decay_mode, max_seqlen, static_cast<cudaStream_t>(stream));
}
