/* C ABI of the sm_100a (B200) WKV7 backend: libfrwkv_sm100.so.
 *
 * Every entry takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream and returns an int: 0 = launched, nonzero = the
 * arguments were rejected and nothing was launched (frwkv_sm100_last_error()
 * gives the reason).  Unless an entry's comment says otherwise the library
 * owns nothing, allocates nothing and never synchronises; no entry throws.
 *
 * Each entry cites the interface of rwkv-rs/FlashRWKV2 it stands in for
 * (paths inside that project).
 *
 * Layouts (identical to the reference):
 *   token tensors r, w, k, v, a, b, y : [total_tokens, H, 64], contiguous,
 *       bf16 / fp16 (the reference's contract) or fp32 (verification mode);
 *   state pool                       : [slots, H, 64(key), 64(value)] fp32,
 *       element (k, v) at k*64+v, updated in place at `slots[seq]` only;
 *   cu_seqlens [n_seq+1], slots [n_seq], status [3] : int32.
 *   status = {error bitmask, active tokens, active sequences}.
 */
#ifndef FRWKV_SM100_H_
#define FRWKV_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FRWKV_SM100_ABI_VERSION 2 /* 2: fp16-state, fused-gate, readout and training entries added; the entries of 1 unchanged */

/* token dtype of r,w,k,v,a,b,y */
enum { FRWKV_IO_BF16 = 0, FRWKV_IO_FP16 = 1, FRWKV_IO_FP32 = 2 };
/* meaning of w: raw decay logits (the reference's contract:
 * rho = exp(-exp(-1/2) * sigmoid(w + bias)), csrc/sm120/tmix/wkv7/recurrent_decay.cuh:18-23)
 * or the retention rho itself (how the benchmark workloads are specified).
 * RWKV-7 retentions lie in [exp(-exp(-1/2)), 1] = [0.545, 1], which is what the logits form can produce.  The chunked
 * prefill kernel divides by the running product of rho over one 32-row chunk, so in retention mode that product
 * must stay above 1e-36 (rho >= 0.08 on every row is enough); a chunk that violates it sets bit 1 of the prefill
 * entry's error_flag instead of passing inf/NaN on silently.  The recurrent entry and FRWKV_PREFILL_RECURRENT take
 * any rho in [0, 1]. */
enum { FRWKV_DECAY_LOGITS = 0, FRWKV_DECAY_RETENTION = 1 };
/* metadata error bits written to status[0]; same values as
 * csrc/validation/recurrent_metadata.cu:15-22 */
enum {
  FRWKV_META_BAD_ENDPOINT = 1 << 0,
  FRWKV_META_BAD_RANGE = 1 << 1,
  FRWKV_META_BAD_SLOT = 1 << 2,
  FRWKV_META_DUPLICATE_SLOT = 1 << 3,
  FRWKV_META_BAD_ACTIVE_COUNT = 1 << 4,
  FRWKV_META_SEQUENCE_TOO_LONG = 1 << 5,
};
/* prefill strategy */
enum { FRWKV_PREFILL_AUTO = 0, FRWKV_PREFILL_RECURRENT = 1, FRWKV_PREFILL_CHUNK_TC = 2 };
/* return codes */
enum {
  FRWKV_OK = 0,
  FRWKV_ERR_ARGUMENT = 1,
  FRWKV_ERR_UNSUPPORTED = 2,
  FRWKV_ERR_WORKSPACE = 3,
  FRWKV_ERR_CUDA = 4,
};

int frwkv_sm100_abi_version(void);
/* Message for the last nonzero return on the calling thread ("" if none). */
const char* frwkv_sm100_last_error(void);

/* Device-side metadata validation; stands in for validate_recurrent_metadata_kernel
 * and its launchers (csrc/validation/recurrent_metadata.cu:24-132,196-225).
 * One launch.  Checks the end points, strictly increasing non-empty ranges,
 * slot bounds, duplicate slots and the active counts; writes status[3].
 *   n_active_tokens / n_active_sequences : device scalars or NULL (= capacities);
 *   seen_slots   : scratch of pool_size int32;
 *   cu_snapshot / slots_snapshot : both NULL, or buffers of n_seq_capacity+1 /
 *       n_seq_capacity int32 that receive a copy which is then what is validated. */
int frwkv_sm100_wkv7_validate_metadata(
    const int32_t* cu_seqlens, const int32_t* slots, int n_seq_capacity, int token_capacity,
    int pool_size, int max_seqlen, const int32_t* n_active_tokens,
    const int32_t* n_active_sequences, int32_t* status, int32_t* seen_slots,
    int32_t* cu_snapshot, int32_t* slots_snapshot, void* stream);

/* The same validation for hosts that cannot provide device scratch (a binding from another
 * language that owns no device allocator; a serving loop where cudaMalloc is off limits because
 * it may synchronise the device).  No counterpart in the reference.  The duplicate-slot scratch
 * is a fixed array inside the library (FRWKV_SM100_STATIC_POOL_SLOTS int32, 256 KiB, held by
 * every GPU that loads the library until the process exits), so the call takes no seen_slots
 * and neither it nor anything it calls allocates or frees memory.
 *   - pool_size above FRWKV_SM100_STATIC_POOL_SLOTS is rejected (FRWKV_ERR_UNSUPPORTED);
 *   - the first call on each device looks up the array's device address (a cheap runtime
 *     query made with that device current); make that first call outside any stream capture.
 *     The per-device address cache is written without synchronisation: two host threads that make
 *     their first call on one device at the same time both store the same value, which is harmless;
 *   - all calls on a device share the one array: the kernel re-initialises the part it uses
 *     at the start of every call, but two such calls that overlap in time on the GPU
 *     (different streams) would race, so keep them on one stream or otherwise ordered. */
#define FRWKV_SM100_STATIC_POOL_SLOTS 65536
int frwkv_sm100_wkv7_validate_metadata_static(
    const int32_t* cu_seqlens, const int32_t* slots, int n_seq_capacity, int token_capacity,
    int pool_size, int max_seqlen, const int32_t* n_active_tokens,
    const int32_t* n_active_sequences, int32_t* status, int32_t* cu_snapshot,
    int32_t* slots_snapshot, void* stream);

/* Register-streaming recurrence (decode and short rows); stands in for
 * tmix_wkv7_recurrent_fp32_from_decay_logits_cuda and the kernels it selects
 * (csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:90-281,457-517).
 * Fail-closed like the reference (:116-123): status[0] != 0 fills y with NaN and
 * leaves the pool untouched; sequences at or beyond status[2] are skipped.
 *   status     : device int32[3], or NULL to trust the metadata (all n_seq active);
 *   decay_bias : [H*64] in the token dtype or NULL (logits mode only);
 *   y_f32      : optional fp32 copy of y before rounding (verification), or NULL;
 *   max_seqlen : largest sequence length (a launch-shape hint; <= 0 if unknown). */
int frwkv_sm100_wkv7_recurrent(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
    int io_dtype, int decay_mode, float scale, int max_seqlen, void* stream);

/* The fp16-state decode contract ("Albatross" family): fp16 tokens, fp16 state pool [slots, H, 64, 64] (half the
 * state traffic of the fp32 contract), decay applied as S + S*delta with
 * delta = fp16(rho - 1 + dither(phase)), phase = elapsed_pool[slot] + head*64 + key + token offset, the new state
 * rounded to fp16 after every token and y = fp16(scale * r^T S) read from the rounded state; afterwards
 * elapsed_pool[slot] advances by the sequence's token count (a second small launch).  Stands in for
 * tmix_wkv7_recurrent_fp16_from_decay_logits and the kernels behind it
 * (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:57-75,244-380,459-583,1204-1286; arithmetic as in
 * its exact kernel :244-340 and the oracle tests/tmix/wkv7/test.py:88-149).  Same fail-closed rules: invalid
 * metadata fills y with NaN and leaves state and elapsed counters untouched.
 *   elapsed_pool : device int32 [pool_slots];  state_pool_f16 : device fp16 [pool_slots, H, 64, 64];
 *   tokens, decay_bias, y : fp16;  max_seqlen : 1 for a decode step (every row one token: the TMA-fed kernel,
 *   which wants the pool 1024-byte aligned), the largest row length otherwise (<= 0 if unknown);
 *   error_flag : optional device int32, bit 0 set if a bounded wait of the decode kernel gave up. */
int frwkv_sm100_wkv7_recurrent_fp16_state(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, int32_t* elapsed_pool,
    void* state_pool_f16, int pool_slots, const void* r, const void* w, const void* k, const void* v, const void* a,
    const void* b, const void* decay_bias, void* y, int n_seq, int total_tokens, int heads, int decay_mode,
    float scale, int max_seqlen, int32_t* error_flag, void* stream);

/* Chunked prefill (32-row chunks, WY/UT transform on tcgen05 tensor cores, fp32 state
 * carry), in place on the pool; stands in for the kernels behind
 * rl_infctx_tmix_wkv7_chunk_fp32io16_forward
 * (csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cu:41-135,318-539 and
 * rl_infctx_chunk_fp32io16_backward.cu:47-128), taking cu_seqlens directly
 * instead of host-built per-chunk metadata.  Same fail-closed rules as above.
 *   strategy   : FRWKV_PREFILL_AUTO picks the tensor-core kernel for 16-bit
 *                tokens and long rows, else the register-streaming recurrence;
 *   workspace  : device scratch of at least frwkv_sm100_wkv7_prefill_workspace_bytes() bytes, 16-byte aligned.
 *                For batches of 2..2048 sequences it holds the length ranking (4 bytes per sequence), used to
 *                hand the sequences to the SMs longest first, and, when the batch has more (sequence, head)
 *                streams than the GPU has CTA slots, the header and per-stream flags of the chunk kernel's
 *                work queue (persistent CTAs that take (stream, segment) tasks; a segment's state passes to the
 *                next through the pool slot).  NULL is accepted and keeps the natural order with one CTA per
 *                stream (same results, a longer tail on ragged batches and partly filled last waves);
 *   error_flag : optional device int32; the tensor-core kernel ORs in bit 0 if one of its bounded waits gave up
 *                (that (sequence, head)'s rows of y are then NaN and its state slot keeps its old value) and bit 1
 *                if a chunk's decay product left the fp32 range (retention mode only; the output is then invalid).
 * The kernel's 16-bit operands are fp16 where they are bounded by the data: |state|, |r.k| sums and V beyond
 * 65504 overflow to inf and show as NaN in y.  Tensor maps for the six token tensors are encoded on the host at
 * the first call with a given (address, shape) and cached, so repeated calls on the same buffers make no driver
 * call. */
int frwkv_sm100_wkv7_prefill(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* decay_bias, void* y, float* y_f32, int n_seq, int total_tokens, int heads,
    int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy, void* workspace,
    size_t workspace_bytes, int32_t* error_flag, void* stream);

size_t frwkv_sm100_wkv7_prefill_workspace_bytes(int n_seq, int total_tokens, int heads);

/* The two entries above with the kk / a-gate producer fused into their operand-preparation stage.  The reference
 * materialises a = -kk, b = kk * sigmoid(a0 + a12) and the gated key k' = k * (1 + (sigmoid(a0 + a12) - 1) * k_a) as
 * three [total_tokens, H, 64] tensors before WKV7 (tmix_kk_a_gate kernels,
 * csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/infer_fp16_forward_varlen.cu:52-106,131-156; oracle
 * tests/tmix/wkv_prepare/test.py:103-126), kk = normalize(k * k_k) over the 64 channels of a head.  Here the caller
 * passes what that kernel reads and the kernels form a, b and k' in registers, rounded to the token dtype where the
 * reference stores them: five token tensors are read per (token, head) instead of six (640 B instead of 768 B
 * besides y), and the producer's own pass over k and a12 with its three stores disappears.
 *   k_raw : raw key projection;  a12 : per-token gate logits;  both [total_tokens, H, 64];
 *   gate_k_k, gate_a0, gate_k_a : per-channel parameters [H*64];  all in the token dtype (bf16 or fp16).
 * Everything else as in frwkv_sm100_wkv7_recurrent / frwkv_sm100_wkv7_prefill. */
int frwkv_sm100_wkv7_recurrent_fused_gate(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k_raw, const void* v, const void* a12, const void* gate_k_k,
    const void* gate_a0, const void* gate_k_a, const void* decay_bias, void* y, float* y_f32, int n_seq,
    int total_tokens, int heads, int io_dtype, int decay_mode, float scale, int max_seqlen, void* stream);
int frwkv_sm100_wkv7_prefill_fused_gate(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k_raw, const void* v, const void* a12, const void* gate_k_k,
    const void* gate_a0, const void* gate_k_a, const void* decay_bias, void* y, float* y_f32, int n_seq,
    int total_tokens, int heads, int io_dtype, int decay_mode, float scale, int max_seqlen, int strategy,
    void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream);

/* WKV7 recurrence with the readout's elementwise stage as epilogue (decode and short rows; the register-streaming
 * kernel serves every row length).  Replaces the pair of reference operators `wkv7 recurrent` + the first kernel of
 * `readout` (flashrwkv2/tmix/readout/__init__.py:10-77; csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:135-196;
 * oracle tests/tmix/readout/test.py:43-66): per (token, head)
 *   out = (headnorm(y) * ln_weight + ln_bias + (sum_c r_c k_c r_k_c) * v) * out_gate,   eps = 64e-5,
 * with y rounded to the token dtype before the normalisation (what the two-operator pipeline stores and reads back) and
 * k the key the recurrence consumes.  The output projection stays with the caller.
 *   out_gate : [total_tokens, H, 64];  r_k, ln_weight, ln_bias : [H*64];  out : [total_tokens, H, 64]; token dtype
 *              (bf16 or fp16);
 *   y, y_f32 : optional stores of the recurrence's own output, or NULL;
 *   gate_k_k, gate_a0, gate_k_a : all NULL, or all given: then k is the raw key, a the gate logits a12 and b is not
 *              read (the input form of frwkv_sm100_wkv7_recurrent_fused_gate).
 * Everything else as in frwkv_sm100_wkv7_recurrent.  Invalid metadata: `out` (and y when given) NaN-filled. */
int frwkv_sm100_wkv7_recurrent_readout(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* gate_k_k, const void* gate_a0, const void* gate_k_a, const void* decay_bias,
    const void* out_gate, const void* r_k, const void* ln_weight, const void* ln_bias, void* out,
    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
    int max_seqlen, void* stream);

/* Prefill with the same readout stage.  The chunk kernel is bound by its CUDA-core instruction count, so here the stage
 * is a second, HBM-bound launch over the rows the prefill stored (768 bytes per (token, head); with the fused producer
 * the gated key is recomputed from the raw key and the gate logits): y is required as the intermediate.  Arguments as
 * in frwkv_sm100_wkv7_recurrent_readout and frwkv_sm100_wkv7_prefill. */
int frwkv_sm100_wkv7_prefill_readout(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* gate_k_k, const void* gate_a0, const void* gate_k_a, const void* decay_bias,
    const void* out_gate, const void* r_k, const void* ln_weight, const void* ln_bias, void* out,
    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
    int max_seqlen, int strategy, void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream);

/* WKV7 training operator (dense [B, T, H, 64] bf16 tensors, T a multiple of 16, zero initial state, decay logits):
 * the forward and backward passes behind the reference's pretrain_tmix_wkv7_recurrent_bf16
 * (flashrwkv2/tmix/wkv7/pretrain.py:52-116; csrc/sm120/tmix/wkv7/pretrain_recurrent_bf16_forward.cu; oracle
 * tests/tmix/wkv7/pretrain/test.py:44-65).  Stand in for its native symbols pretrain_tmix_wkv7_recurrent_forward /
 * _backward with the same saved tensors:
 *   boundary     : fp32 [B, H, T/16, 64, 64], the state after every 16th token;
 *   state_dot_a  : fp32 [B, T, H, 64], a^T S_{t-1} of every token;
 *   dy, dr .. db : bf16 [B, T, H, 64]. */
int frwkv_sm100_wkv7_pretrain_forward(const void* r, const void* w, const void* k, const void* v, const void* a,
                                      const void* b, void* y, float* boundary, float* state_dot_a, int batch,
                                      int tokens, int heads, void* stream);
int frwkv_sm100_wkv7_pretrain_backward(const void* r, const void* w, const void* k, const void* v, const void* a,
                                       const void* b, const void* dy, const float* boundary,
                                       const float* state_dot_a, void* dr, void* dw, void* dk, void* dv, void* da,
                                       void* db, int batch, int tokens, int heads, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FRWKV_SM100_H_ */
