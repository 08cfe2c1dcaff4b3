// Prefill entry of the C ABI: strategy selection between the tensor-core chunk kernel
// and the register-streaming recurrence.
#include "../../common.cuh"
#include "chunk_common.cuh"


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
                      void* queue, cudaStream_t stream);

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

// Segments per stream that minimise ceil(N S / slots) / S * (1 + 1.5 S / chunks) for N streams of `chunks` chunks
// (see sequence_order_kernel); shared by the kernel and by the host's choice of launch mode.
__host__ __device__ inline int pick_segments(long long streams, int chunks_longest, int cta_slots) {
  int best = 1;
  float best_cost = 1e30f;
  for (int S = 1; S <= chunk::kQueueLevels && S * 8 <= chunks_longest; ++S) {
    const float rounds = static_cast<float>((streams * S + cta_slots - 1) / cta_slots) / S;
    const float cost = rounds * (1.0f + 1.5f * S / chunks_longest);
    if (cost < best_cost * 0.995f) {
      best_cost = cost;
      best = S;
    }
  }
  return best;
}

// Host-side choice between the two launch modes for N equal streams, in units of one stream's time at two CTAs per
// SM.  Whole streams: the full rounds, plus a last partial round that costs 0.6 when at most half the slots are
// taken (a CTA alone on its SM runs a quarter faster, and rounds overlap) and a whole round otherwise.  Queue: the
// cost model's best segmentation plus 3 % for the persistent loop.  Measured on 148 SMs, 64 heads, 8192-token rows:
// 512 streams 2.60 ms whole, 2.36 ms queued; 1024 streams 4.58 ms whole, 4.64 ms queued.
inline bool queue_beats_whole_streams(long long streams, int chunks, int cta_slots) {
  const int segments = pick_segments(streams, chunks, cta_slots);
  if (segments <= 1) return false;
  const long long full = streams / cta_slots, rest = streams % cta_slots;
  const double whole = static_cast<double>(full) + (rest == 0 ? 0.0 : 2 * rest <= cta_slots ? 0.6 : 1.0);
  const double rounds = static_cast<double>((streams * segments + cta_slots - 1) / cta_slots) / segments;
  const double queued = 1.03 * rounds * (1.0 + 1.5 * segments / chunks);
  return queued < whole;
}

__global__ void __launch_bounds__(kOrderThreads) sequence_order_kernel(const int* __restrict__ cu,
                                                                       const int* __restrict__ status, int n_seq,
                                                                       int* __restrict__ order, int heads, int len_from,
                                                                       chunk::QueueHeader* queue, int cta_slots) {
  __shared__ int len[kMaxOrdered];
  __shared__ int level_count[chunk::kQueueLevels];
  __shared__ int longest, shortest, live, segment_chunks_shared;
  const bool valid = status == nullptr || status[0] == 0;
  const int active = status == nullptr ? n_seq : status[2];
  if (threadIdx.x < chunk::kQueueLevels) level_count[threadIdx.x] = 0;
  if (threadIdx.x == 0) {
    longest = 0;
    shortest = 0x7fffffff;
    live = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_seq; i += kOrderThreads) {
    len[i] = (valid && i < active) ? max(cu[i + 1] - cu[i], 0) : 0;
    if (queue != nullptr && len[i] >= max(len_from, 1)) {  // the sequences the chunk kernel works on
      atomicMax(&longest, len[i]);
      atomicMin(&shortest, len[i]);
      atomicAdd(&live, 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_seq; i += kOrderThreads) {
    const int mine = len[i];
    int rank = 0;
    for (int j = 0; j < n_seq; ++j) rank += (len[j] > mine) || (len[j] == mine && j < i);
    order[rank] = i;
  }
  if (queue == nullptr) return;
  // Work queue.  How many segments S to cut the longest sequence into: with N streams of about equal length on
  // `cta_slots` persistent CTAs the launch takes ceil(N S / slots) / S stream times, and every segment costs about
  // one and a half chunk times of start-up (first load, first operand preparation, state through the pool slot).
  // S = 1 is the plain longest-first order; ragged batches keep it, it balances them by itself.
  if (threadIdx.x == 0) {
    const int chunks_longest = max(1, (longest + 31) / 32);
    int best = 1;
    if (live > 0 && shortest >= longest - longest / 10)
      best = pick_segments(static_cast<long long>(live) * heads, chunks_longest, cta_slots);
    segment_chunks_shared = (chunks_longest + best - 1) / best;
  }
  __syncthreads();
  const int segment_chunks = segment_chunks_shared;
  for (int i = threadIdx.x; i < n_seq; i += kOrderThreads) {
    const int chunks = (len[i] + 31) / 32;
    const int segments = len[i] >= max(len_from, 1) ? (chunks + segment_chunks - 1) / segment_chunks : 0;
    for (int g = 0; g < segments; ++g) atomicAdd(&level_count[g], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int end = 0;
    for (int g = 0; g < chunk::kQueueLevels; ++g) {
      end += level_count[g] * heads;
      queue->level_end[g] = end;
    }
    queue->total_tasks = end;
    queue->segment_chunks = segment_chunks;
    queue->next_task = 0;
  }
}

}  // namespace

// Layout of the scratch: order[n_seq] (padded to 16 bytes), then, for batches with more streams than the GPU has
// CTA slots, the work-queue header and one flag per (sequence, head).
size_t order_bytes(int n_seq) { return (static_cast<size_t>(n_seq) * sizeof(int) + 15) & ~size_t(15); }
int cta_slots() {  // two resident CTAs of the chunk kernel per SM
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return 2 * sms;
}
bool wants_queue(int n_seq, int heads) { return static_cast<long long>(n_seq) * heads > 2LL * 148; }

size_t chunk_tc_workspace_bytes(int n_seq, int, int heads) {
  if (n_seq > kMaxOrdered) return 0;
  if (wants_queue(n_seq, heads))
    return order_bytes(n_seq) + sizeof(chunk::QueueHeader) + static_cast<size_t>(n_seq) * heads * sizeof(int);
  return n_seq > 1 ? static_cast<size_t>(n_seq) * sizeof(int) : 0;
}

// The tensor-core path: optional longest-first ranking, then the 32-row chunk kernel.
int launch_chunk_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                    const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                    float scale, int max_seqlen, int len_from, void* workspace, size_t workspace_bytes,
                    int32_t* error_flag, const void* const* gate, cudaStream_t stream) {
  const int32_t* order = nullptr;
  void* queue = nullptr;
  const size_t need = chunk_tc_workspace_bytes(n_seq, total_tokens, heads);
  if (need > 0 && workspace != nullptr) {  // no scratch given: natural order, one CTA per stream
    if (workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15) != 0)
      return fail(FRWKV_ERR_WORKSPACE, "wkv7_prefill: workspace of %zu bytes (16-byte aligned) needed, got %zu", need,
                  workspace_bytes);
    // Persistent CTAs with the work queue pay about 3 % against one CTA per stream (task hand-out, no overlap of a
    // CTA's tail with the next CTA's start), so they are used only where cutting streams into segments wins:
    // uniform batches (every row max_seqlen long) for which the queue's estimate beats the estimate for whole
    // streams.  Ragged batches are balanced by the longest-first order alone.
    const bool uniform = max_seqlen > 0 && static_cast<long long>(n_seq) * max_seqlen == total_tokens;
    if (wants_queue(n_seq, heads) && uniform &&
        queue_beats_whole_streams(static_cast<long long>(n_seq) * heads, (max_seqlen + 31) / 32, cta_slots())) {
      queue = static_cast<char*>(workspace) + order_bytes(n_seq);
      const size_t queue_bytes = sizeof(chunk::QueueHeader) + static_cast<size_t>(n_seq) * heads * sizeof(int);
      if (cudaMemsetAsync(queue, 0, queue_bytes, stream) != cudaSuccess) return check_launch("work-queue memset");
    }
    sequence_order_kernel<<<1, kOrderThreads, 0, stream>>>(cu, status, n_seq, static_cast<int*>(workspace), heads,
                                                           len_from, static_cast<chunk::QueueHeader*>(queue),
                                                           cta_slots());
    const int rc = check_launch("sequence_order_kernel");
    if (rc != FRWKV_OK) return rc;
    order = static_cast<const int32_t*>(workspace);
  }
  return launch_chunk32_tc(cu, slots, status, pool, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads,
                           io_dtype, decay_mode, scale, order, len_from, error_flag, gate, queue, stream);
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

namespace frwkv {
int launch_readout_rows(const void* y, const void* r, const void* k, const void* v, const void* out_gate,
                        const void* r_k, const void* ln_w, const void* ln_b, const void* const* gate, void* out,
                        int total_tokens, int heads, int io_dtype, cudaStream_t stream);
}

extern "C" int frwkv_sm100_wkv7_prefill_readout(
    const int32_t* cu_seqlens, const int32_t* slots, const int32_t* status, float* state_pool,
    const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
    const void* gate_k_k, const void* gate_a0, const void* gate_k_a, const void* decay_bias,
    const void* out_gate, const void* r_k, const void* ln_weight, const void* ln_bias, void* out,
    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode, float scale,
    int max_seqlen, int strategy, void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream) {
  using namespace frwkv;
  const char* who = "wkv7_prefill_readout";
  const int given = (gate_k_k != nullptr) + (gate_a0 != nullptr) + (gate_k_a != nullptr);
  if (given != 0 && given != 3)
    return fail(FRWKV_ERR_ARGUMENT, "%s: k_k, a0 and k_a must be given together or not at all", who);
  if (!out_gate || !r_k || !ln_weight || !ln_bias || !out || !y)
    return fail(FRWKV_ERR_ARGUMENT, "%s: out_gate, r_k, ln_weight, ln_bias, out and y must be non-null", who);
  const void* more[] = {out_gate, r_k, ln_weight, ln_bias, out};
  for (const void* q : more)
    if ((reinterpret_cast<uintptr_t>(q) & 15) != 0)
      return fail(FRWKV_ERR_ARGUMENT, "%s: tensors must be 16-byte aligned", who);
  if (io_dtype == FRWKV_IO_FP32)
    return fail(FRWKV_ERR_UNSUPPORTED, "%s: the readout stage takes float16 or bfloat16 tokens", who);
  const void* gate[3] = {gate_k_k, gate_a0, gate_k_a};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = prefill_impl(who, cu_seqlens, slots, status, state_pool, r, w, k, v, a, b, decay_bias, y, y_f32, n_seq,
                        total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, strategy, workspace,
                        workspace_bytes, error_flag, given == 3 ? gate : nullptr, s);
  if (rc != FRWKV_OK) return rc;
  const void* producer[3] = {a, gate_a0, gate_k_a};  // the gate logits a12 travel in the a argument
  return launch_readout_rows(y, r, k, v, out_gate, r_k, ln_weight, ln_bias, given == 3 ? producer : nullptr, out,
                             total_tokens, heads, io_dtype, s);
}
