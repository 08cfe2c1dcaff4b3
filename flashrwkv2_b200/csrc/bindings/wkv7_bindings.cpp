// Torch-facing shim of the WKV7 path: validates tensors, owns the metadata ticket and passes raw
// device pointers plus the current CUDA stream to the C ABI in libfrwkv_sm100.so.  No arithmetic here.
//
// Surface (names, argument order, defaults, error text) follows the reference's pybind module:
//   rwkv-rs/FlashRWKV2 csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cpp:89-458
//   rwkv-rs/FlashRWKV2 csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cpp:158-241
//   rwkv-rs/FlashRWKV2 csrc/validation.cpp:27-129 (host argument contract)
// Additions: `decay_mode` ("logits" | "retention"), an optional fp32 `output_f32`, and
// `tmix_wkv7_prefill_fp32`, which takes cu_seqlens directly.
#include "bindings.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <memory>
#include <optional>
#include <string>
#include <unordered_set>
#include <vector>

#include "frwkv_sm100.h"

namespace {

constexpr int64_t kHeadSize = 64;

void check_abi(int rc) { TORCH_CHECK(rc == 0, frwkv_sm100_last_error()); }

void check_cuda_contiguous(const torch::Tensor& tensor, const char* name) {
  TORCH_CHECK(tensor.is_cuda(), name, " must be CUDA");
  TORCH_CHECK(tensor.is_contiguous(), name, " must be contiguous");
}

void check_same_device(const torch::Tensor& reference, const torch::Tensor& tensor, const char* name) {
  TORCH_CHECK(tensor.device() == reference.device(), name, " must be on the same device as state");
}

int io_code(const torch::Tensor& tokens) {
  switch (tokens.scalar_type()) {
    case torch::kBFloat16: return FRWKV_IO_BF16;
    case torch::kFloat16: return FRWKV_IO_FP16;
    default: return FRWKV_IO_FP32;
  }
}

int decay_code(const std::string& decay_mode) {
  TORCH_CHECK(decay_mode == "logits" || decay_mode == "retention", "decay_mode must be 'logits' or 'retention'");
  return decay_mode == "logits" ? FRWKV_DECAY_LOGITS : FRWKV_DECAY_RETENTION;
}

struct Dimensions {
  int64_t sequences, heads;
};

// csrc/validation.cpp:27-129 of the reference; head size 64 only here.
Dimensions check_recurrent_layout(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices,
                                  const torch::Tensor& state, const torch::Tensor& r, const torch::Tensor& w,
                                  const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& a,
                                  const torch::Tensor& b, const torch::Tensor& output, double scale,
                                  bool allow_fp32_tokens) {
  const std::pair<const torch::Tensor*, const char*> named[] = {
      {&query_start_loc, "query_start_loc"}, {&state_indices, "state_indices"}, {&state, "state"}, {&r, "r"},
      {&w, "decay_logits"}, {&k, "k"}, {&v, "v"}, {&a, "a"}, {&b, "b"}, {&output, "output"}};
  for (const auto& item : named) check_cuda_contiguous(*item.first, item.second);
  TORCH_CHECK(query_start_loc.scalar_type() == torch::kInt32, "query_start_loc must be int32");
  TORCH_CHECK(state_indices.scalar_type() == torch::kInt32, "state_indices must be int32");
  TORCH_CHECK(std::isfinite(scale), "scale must be finite");
  const int64_t n = state_indices.numel();
  TORCH_CHECK(n > 0 && n <= 65535, "state_indices must contain 1..65535 sequences");
  TORCH_CHECK(state_indices.dim() == 1, "state_indices must have shape [N]");
  TORCH_CHECK(query_start_loc.dim() == 1 && query_start_loc.size(0) == n + 1, "query_start_loc must have shape [N+1]");
  TORCH_CHECK(state.dim() == 4 && state.size(0) > 0 && state.size(1) > 0 && state.size(2) == state.size(3),
              "state must have square shape [slots,H,D,D]");
  TORCH_CHECK(state.scalar_type() == torch::kFloat32, "state must be float32");
  const int64_t d = state.size(2);
  TORCH_CHECK(d == 64 || d == 128 || d == 256, "recurrent head size must be 64, 128, or 256, got ", d);
  TORCH_CHECK(d == kHeadSize, "the sm_100a backend implements head size 64 only, got ", d);
  TORCH_CHECK(state.size(0) <= std::numeric_limits<int>::max(), "state slot count must fit in int32");
  const int64_t h = state.size(1);
  TORCH_CHECK(r.dim() == 3 && r.size(0) > 0 && r.size(1) == h && r.size(2) == d,
              "r must have shape [total_tokens,H,D] matching state");
  TORCH_CHECK(r.size(0) <= std::numeric_limits<int>::max(), "token count must fit in int32");
  TORCH_CHECK(r.sizes() == w.sizes() && r.sizes() == k.sizes() && r.sizes() == v.sizes() && r.sizes() == a.sizes() &&
                  r.sizes() == b.sizes() && r.sizes() == output.sizes(),
              "r,decay_logits,k,v,a,b,output shape mismatch");
  const auto dtype = r.scalar_type();
  TORCH_CHECK(dtype == torch::kFloat16 || dtype == torch::kBFloat16 || (allow_fp32_tokens && dtype == torch::kFloat32),
              "token tensors must be float16 or bfloat16");
  TORCH_CHECK(dtype == w.scalar_type() && dtype == k.scalar_type() && dtype == v.scalar_type() &&
                  dtype == a.scalar_type() && dtype == b.scalar_type() && dtype == output.scalar_type(),
              "r,decay_logits,k,v,a,b,output dtype mismatch");
  for (const auto& item : named) check_same_device(state, *item.first, item.second);
  return Dimensions{n, h};
}

void check_decay_bias(const std::optional<torch::Tensor>& decay_bias, const torch::Tensor& state,
                      const torch::Tensor& r, int decay_mode) {
  if (!decay_bias.has_value()) return;
  check_cuda_contiguous(*decay_bias, "decay_bias");
  check_same_device(state, *decay_bias, "decay_bias");
  TORCH_CHECK(decay_bias->scalar_type() == r.scalar_type(), "decay_bias must match the token tensor dtype");
  const int64_t h = state.size(1), d = state.size(2);
  TORCH_CHECK((decay_bias->dim() == 1 && decay_bias->numel() == h * d) ||
                  (decay_bias->dim() == 2 && decay_bias->size(0) == h && decay_bias->size(1) == d),
              "decay_bias must have shape [H*D] or [H,D]");
  TORCH_CHECK(decay_mode == FRWKV_DECAY_LOGITS, "decay_bias only applies to decay logits");
}

void check_output_f32(const std::optional<torch::Tensor>& output_f32, const torch::Tensor& output) {
  if (!output_f32.has_value()) return;
  check_cuda_contiguous(*output_f32, "output_f32");
  TORCH_CHECK(output_f32->scalar_type() == torch::kFloat32 && output_f32->sizes() == output.sizes() &&
                  output_f32->device() == output.device(),
              "output_f32 must be a float32 tensor shaped like output");
}

std::optional<uint32_t> tensor_version(const torch::Tensor& tensor) {
  if (tensor.unsafeGetTensorImpl()->is_inference()) return std::nullopt;
  return tensor.unsafeGetTensorImpl()->version_counter().current_version();
}

struct Prepared {
  torch::Tensor cu, slots, status, workspace;
};

// One launch of the validation kernel on the current stream of the metadata's device.
Prepared launch_validation(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices,
                           const torch::Tensor& num_active_tokens, const torch::Tensor& num_active_sequences,
                           int64_t token_capacity, int64_t sequence_capacity, int64_t state_pool_size,
                           int64_t max_seqlen, bool snapshot) {
  const c10::cuda::CUDAGuard guard(query_start_loc.device());
  auto status = torch::empty({3}, query_start_loc.options());
  auto seen = torch::empty({state_pool_size}, query_start_loc.options());
  auto cu_snap = snapshot ? torch::empty_like(query_start_loc) : query_start_loc;
  auto slots_snap = snapshot ? torch::empty_like(state_indices) : state_indices;
  check_abi(frwkv_sm100_wkv7_validate_metadata(
      query_start_loc.data_ptr<int>(), state_indices.data_ptr<int>(), static_cast<int>(sequence_capacity),
      static_cast<int>(token_capacity), static_cast<int>(state_pool_size), static_cast<int>(max_seqlen),
      num_active_tokens.defined() ? num_active_tokens.data_ptr<int>() : nullptr,
      num_active_sequences.defined() ? num_active_sequences.data_ptr<int>() : nullptr, status.data_ptr<int>(),
      seen.data_ptr<int>(), snapshot ? cu_snap.data_ptr<int>() : nullptr,
      snapshot ? slots_snap.data_ptr<int>() : nullptr,
      at::cuda::getCurrentCUDAStream(query_start_loc.device().index()).stream()));
  return Prepared{std::move(cu_snap), std::move(slots_snap), std::move(status), std::move(seen)};
}

// Static tickets validate on the host as well and raise, as the reference does (one D2H copy).
int64_t host_check_metadata(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices,
                            int64_t total_tokens, int64_t state_pool_size) {
  auto cu_cpu = query_start_loc.to(torch::kCPU).contiguous();
  auto slots_cpu = state_indices.to(torch::kCPU).contiguous();
  const int32_t* cu = cu_cpu.data_ptr<int32_t>();
  const int32_t* slots = slots_cpu.data_ptr<int32_t>();
  const int64_t n = state_indices.numel();
  TORCH_CHECK(cu[0] == 0, "query_start_loc must start at 0");
  TORCH_CHECK(cu[n] == total_tokens, "the final query_start_loc offset must equal total_tokens");
  std::unordered_set<int32_t> seen;
  int64_t longest = 0;
  for (int64_t i = 0; i < n; ++i) {
    TORCH_CHECK(cu[i] >= 0 && cu[i + 1] > cu[i] && cu[i + 1] <= total_tokens,
                "query_start_loc must be strictly increasing with non-empty sequences");
    TORCH_CHECK(slots[i] >= 0 && slots[i] < state_pool_size, "state_indices entries must be within the state pool");
    TORCH_CHECK(seen.insert(slots[i]).second, "state_indices must be unique within one call");
    longest = std::max<int64_t>(longest, cu[i + 1] - cu[i]);
  }
  return longest;
}

// Validated packed-sequence metadata bound to one stream (counterpart of the reference's
// RecurrentMetadataTicket, infer_recurrent_fp32io16_forward_varlen.cpp:89-225).
class RecurrentMetadataTicket final {
 public:
  RecurrentMetadataTicket(torch::Tensor query_start_loc, torch::Tensor state_indices, Prepared prepared,
                          torch::Tensor num_active_tokens, torch::Tensor num_active_sequences, int64_t total_tokens,
                          int64_t state_pool_size, int64_t max_seqlen, bool graph_mode, cudaStream_t stream)
      : cu_(std::move(query_start_loc)), slots_(std::move(state_indices)), prepared_(std::move(prepared)),
        n_tok_(std::move(num_active_tokens)), n_seq_(std::move(num_active_sequences)),
        cu_version_(tensor_version(cu_)), slots_version_(tensor_version(slots_)), cu_data_(cu_.data_ptr()),
        slots_data_(slots_.data_ptr()), cu_sizes_(cu_.sizes().vec()), slots_sizes_(slots_.sizes().vec()),
        cu_strides_(cu_.strides().vec()), slots_strides_(slots_.strides().vec()), total_tokens_(total_tokens),
        state_pool_size_(state_pool_size), max_seqlen_(max_seqlen), graph_mode_(graph_mode), device_(cu_.device()),
        stream_(stream) {}

  void check_compatible(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices,
                        int64_t total_tokens, int64_t state_pool_size, int64_t max_seqlen) const {
    TORCH_CHECK(query_start_loc.is_same(cu_), "validated_metadata query_start_loc identity mismatch");
    TORCH_CHECK(state_indices.is_same(slots_), "validated_metadata state_indices identity mismatch");
    TORCH_CHECK(query_start_loc.data_ptr() == cu_data_ && state_indices.data_ptr() == slots_data_,
                "validated_metadata metadata data_ptr mismatch");
    TORCH_CHECK(query_start_loc.sizes().vec() == cu_sizes_ && state_indices.sizes().vec() == slots_sizes_ &&
                    query_start_loc.strides().vec() == cu_strides_ && state_indices.strides().vec() == slots_strides_,
                "validated_metadata metadata shape or stride mismatch");
    if (!graph_mode_ && cu_version_.has_value())
      TORCH_CHECK(tensor_version(query_start_loc) == cu_version_, "validated_metadata query_start_loc version mismatch");
    if (!graph_mode_ && slots_version_.has_value())
      TORCH_CHECK(tensor_version(state_indices) == slots_version_, "validated_metadata state_indices version mismatch");
    TORCH_CHECK(query_start_loc.device() == device_ && state_indices.device() == device_,
                "validated_metadata device mismatch");
    TORCH_CHECK(total_tokens == total_tokens_, "validated_metadata total_tokens mismatch");
    TORCH_CHECK(state_pool_size == state_pool_size_, "validated_metadata state_pool_size mismatch");
    if (max_seqlen > 0) TORCH_CHECK(max_seqlen == max_seqlen_, "validated_metadata max_seqlen mismatch");
    TORCH_CHECK(at::cuda::getCurrentCUDAStream(device_.index()).stream() == stream_,
                "validated_metadata stream mismatch; prepare and consume the ticket on the same CUDA stream");
  }

  const torch::Tensor& cu_snapshot() const { return prepared_.cu; }
  const torch::Tensor& slots_snapshot() const { return prepared_.slots; }
  const torch::Tensor& status() const { return prepared_.status; }
  int64_t max_seqlen() const { return max_seqlen_; }
  bool graph_mode() const { return graph_mode_; }
  const torch::Tensor& num_active_tokens() const { return n_tok_; }
  const torch::Tensor& num_active_sequences() const { return n_seq_; }

 private:
  torch::Tensor cu_, slots_;
  Prepared prepared_;
  torch::Tensor n_tok_, n_seq_;
  std::optional<uint32_t> cu_version_, slots_version_;
  void* cu_data_;
  void* slots_data_;
  std::vector<int64_t> cu_sizes_, slots_sizes_, cu_strides_, slots_strides_;
  int64_t total_tokens_, state_pool_size_, max_seqlen_;
  bool graph_mode_;
  c10::Device device_;
  cudaStream_t stream_;
};

using TicketPtr = std::shared_ptr<RecurrentMetadataTicket>;

void check_metadata_tensors(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices) {
  check_cuda_contiguous(query_start_loc, "query_start_loc");
  check_cuda_contiguous(state_indices, "state_indices");
  check_same_device(query_start_loc, state_indices, "state_indices");
  TORCH_CHECK(query_start_loc.scalar_type() == torch::kInt32 && state_indices.scalar_type() == torch::kInt32,
              "recurrent metadata must be int32");
}

TicketPtr prepare_tmix_wkv7_recurrent_metadata(torch::Tensor query_start_loc, torch::Tensor state_indices,
                                               int64_t total_tokens, int64_t state_pool_size, int64_t max_seqlen) {
  check_metadata_tensors(query_start_loc, state_indices);
  TORCH_CHECK(query_start_loc.dim() == 1 && state_indices.dim() == 1 && state_indices.numel() > 0 &&
                  query_start_loc.numel() == state_indices.numel() + 1,
              "query_start_loc must have shape [B+1] and state_indices shape [B]");
  TORCH_CHECK(state_indices.numel() <= 65535, "state_indices must contain at most 65535 sequences");
  TORCH_CHECK(total_tokens > 0 && total_tokens <= std::numeric_limits<int>::max(),
              "total_tokens must be positive and fit in int32");
  TORCH_CHECK(state_pool_size > 0 && state_pool_size <= std::numeric_limits<int>::max(),
              "state_pool_size must be positive and fit in int32");
  const int64_t inferred = host_check_metadata(query_start_loc, state_indices, total_tokens, state_pool_size);
  if (max_seqlen <= 0) {
    max_seqlen = inferred;
  } else {
    TORCH_CHECK(max_seqlen == inferred, "max_seqlen must equal the largest packed sequence length");
  }
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(query_start_loc.device().index()).stream();
  auto prepared = launch_validation(query_start_loc, state_indices, torch::Tensor(), torch::Tensor(), total_tokens,
                                    state_indices.numel(), state_pool_size, total_tokens, true);
  return std::make_shared<RecurrentMetadataTicket>(std::move(query_start_loc), std::move(state_indices),
                                                   std::move(prepared), torch::Tensor(), torch::Tensor(),
                                                   total_tokens, state_pool_size, max_seqlen, false, stream);
}

void check_graph_scalar(const torch::Tensor& tensor, const torch::Tensor& reference, const char* name) {
  TORCH_CHECK(tensor.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(tensor.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(tensor.device() == reference.device(), name, " must share the metadata CUDA device");
  TORCH_CHECK(tensor.scalar_type() == torch::kInt32, name, " must have dtype int32");
  TORCH_CHECK(tensor.numel() == 1, name, " must contain one element");
}

TicketPtr prepare_tmix_wkv7_recurrent_graph_metadata(torch::Tensor query_start_loc, torch::Tensor state_indices,
                                                     torch::Tensor num_active_tokens,
                                                     torch::Tensor num_active_sequences, int64_t token_capacity,
                                                     int64_t sequence_capacity, int64_t state_pool_size,
                                                     int64_t max_seqlen_capacity) {
  check_metadata_tensors(query_start_loc, state_indices);
  TORCH_CHECK(sequence_capacity > 0 && sequence_capacity <= 65535 && state_indices.dim() == 1 &&
                  state_indices.numel() == sequence_capacity && query_start_loc.dim() == 1 &&
                  query_start_loc.numel() == sequence_capacity + 1,
              "graph metadata shapes must match sequence_capacity");
  TORCH_CHECK(token_capacity > 0 && token_capacity <= std::numeric_limits<int>::max(),
              "token_capacity must be positive and fit in int32");
  TORCH_CHECK(state_pool_size > 0 && state_pool_size <= std::numeric_limits<int>::max(),
              "state_pool_size must be positive and fit in int32");
  TORCH_CHECK(max_seqlen_capacity > 0 && max_seqlen_capacity <= token_capacity,
              "max_seqlen_capacity must be positive and not exceed token_capacity");
  check_graph_scalar(num_active_tokens, query_start_loc, "num_active_tokens");
  check_graph_scalar(num_active_sequences, query_start_loc, "num_active_sequences");
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(query_start_loc.device().index()).stream();
  auto prepared = launch_validation(query_start_loc, state_indices, num_active_tokens, num_active_sequences,
                                    token_capacity, sequence_capacity, state_pool_size, max_seqlen_capacity, false);
  return std::make_shared<RecurrentMetadataTicket>(std::move(query_start_loc), std::move(state_indices),
                                                   std::move(prepared), std::move(num_active_tokens),
                                                   std::move(num_active_sequences), token_capacity, state_pool_size,
                                                   max_seqlen_capacity, true, stream);
}

struct Resolved {
  torch::Tensor cu, slots, status;
  int64_t max_seqlen;
  torch::Tensor keep;  // scratch of an un-ticketed validation, kept alive until the launch is enqueued
};

Resolved resolve_metadata(const torch::Tensor& query_start_loc, const torch::Tensor& state_indices,
                          const torch::Tensor& state, const torch::Tensor& r, const TicketPtr& ticket,
                          int64_t max_seqlen) {
  if (ticket) {
    ticket->check_compatible(query_start_loc, state_indices, r.size(0), state.size(0), max_seqlen);
    return Resolved{ticket->cu_snapshot(), ticket->slots_snapshot(), ticket->status(), ticket->max_seqlen(),
                    torch::Tensor()};
  }
  // un-ticketed native call: device validation only (the raising host check belongs to the static
  // prepare entry, as in the reference binding :375-381)
  auto prepared = launch_validation(query_start_loc, state_indices, torch::Tensor(), torch::Tensor(), r.size(0),
                                    state_indices.numel(), state.size(0), r.size(0), true);
  return Resolved{prepared.cu, prepared.slots, prepared.status, max_seqlen, prepared.workspace};
}

void tmix_wkv7_recurrent_fp32_from_decay_logits(torch::Tensor query_start_loc, torch::Tensor state_indices,
                                                torch::Tensor state, torch::Tensor r, torch::Tensor decay_logits,
                                                torch::Tensor k, torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                torch::Tensor output, double scale,
                                                std::optional<torch::Tensor> decay_bias, TicketPtr validated_metadata,
                                                int64_t max_seqlen, const std::string& decay_mode,
                                                std::optional<torch::Tensor> output_f32) {
  const int mode = decay_code(decay_mode);
  const auto dims = check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b, output,
                                           scale, true);
  check_decay_bias(decay_bias, state, r, mode);
  check_output_f32(output_f32, output);
  const auto meta = resolve_metadata(query_start_loc, state_indices, state, r, validated_metadata, max_seqlen);
  const c10::cuda::CUDAGuard guard(state.device());
  check_abi(frwkv_sm100_wkv7_recurrent(
      meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
      output_f32.has_value() ? output_f32->data_ptr<float>() : nullptr, static_cast<int>(dims.sequences),
      static_cast<int>(r.size(0)), static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale),
      static_cast<int>(meta.max_seqlen), at::cuda::getCurrentCUDAStream(state.device().index()).stream()));
}

// fp16-state contract; argument order and checks of the reference binding
// (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cpp:44-190).
void tmix_wkv7_recurrent_fp16_from_decay_logits(torch::Tensor query_start_loc, torch::Tensor state_indices,
                                                torch::Tensor elapsed_state, torch::Tensor state, torch::Tensor r,
                                                torch::Tensor decay_logits, torch::Tensor k, torch::Tensor v,
                                                torch::Tensor a, torch::Tensor b, torch::Tensor output, double scale,
                                                std::optional<torch::Tensor> decay_bias, TicketPtr validated_metadata,
                                                int64_t max_seqlen) {
  const std::pair<const torch::Tensor*, const char*> named[] = {
      {&query_start_loc, "query_start_loc"}, {&state_indices, "state_indices"}, {&elapsed_state, "elapsed_state_pool"},
      {&state, "state"}, {&r, "r"}, {&decay_logits, "decay_logits"}, {&k, "k"}, {&v, "v"}, {&a, "a"}, {&b, "b"},
      {&output, "output"}};
  for (const auto& item : named) check_cuda_contiguous(*item.first, item.second);
  for (const auto& item : named) check_same_device(state, *item.first, item.second);
  TORCH_CHECK(query_start_loc.scalar_type() == torch::kInt32 && state_indices.scalar_type() == torch::kInt32,
              "query_start_loc and state_indices must be int32");
  TORCH_CHECK(std::isfinite(scale), "scale must be finite");
  const int64_t n = state_indices.numel();
  TORCH_CHECK(state_indices.dim() == 1 && n > 0 && n <= 65535, "state_indices must contain 1..65535 sequences");
  TORCH_CHECK(query_start_loc.dim() == 1 && query_start_loc.size(0) == n + 1, "query_start_loc must have shape [N+1]");
  TORCH_CHECK(state.dim() == 4 && state.size(0) > 0 && state.size(1) > 0 && state.size(2) == state.size(3),
              "state must have square shape [slots,H,D,D]");
  TORCH_CHECK(state.scalar_type() == torch::kFloat16, "FP16-state state must be float16");
  TORCH_CHECK(state.size(2) == kHeadSize, "the sm_100a backend implements head size 64 only, got ", state.size(2));
  TORCH_CHECK(elapsed_state.scalar_type() == torch::kInt32, "elapsed_state_pool must be int32");
  TORCH_CHECK(elapsed_state.dim() == 1 && elapsed_state.size(0) == state.size(0),
              "elapsed_state_pool must have shape [state_pool_slots]");
  const int64_t h = state.size(1);
  TORCH_CHECK(r.dim() == 3 && r.size(0) > 0 && r.size(1) == h && r.size(2) == kHeadSize,
              "r must have shape [total_tokens,H,D] matching state");
  TORCH_CHECK(r.size(0) <= std::numeric_limits<int>::max(), "token count must fit in int32");
  TORCH_CHECK(r.sizes() == decay_logits.sizes() && r.sizes() == k.sizes() && r.sizes() == v.sizes() &&
                  r.sizes() == a.sizes() && r.sizes() == b.sizes() && r.sizes() == output.sizes(),
              "r,decay_logits,k,v,a,b,output shape mismatch");
  for (const torch::Tensor* t : {&r, &decay_logits, &k, &v, &a, &b, &output})
    TORCH_CHECK(t->scalar_type() == torch::kFloat16, "FP16-state token tensors must be float16");
  if (decay_bias.has_value()) {
    check_cuda_contiguous(*decay_bias, "decay_bias");
    check_same_device(state, *decay_bias, "decay_bias");
    TORCH_CHECK(decay_bias->scalar_type() == torch::kFloat16 &&
                    ((decay_bias->dim() == 1 && decay_bias->numel() == h * kHeadSize) ||
                     (decay_bias->dim() == 2 && decay_bias->size(0) == h && decay_bias->size(1) == kHeadSize)),
                "decay_bias must be float16 with shape [H*D] or [H,D]");
  }
  Resolved meta;
  if (validated_metadata) {
    validated_metadata->check_compatible(query_start_loc, state_indices, r.size(0), state.size(0), max_seqlen);
    meta = Resolved{validated_metadata->cu_snapshot(), validated_metadata->slots_snapshot(),
                    validated_metadata->status(), validated_metadata->max_seqlen(), torch::Tensor()};
  } else {
    auto prepared = launch_validation(query_start_loc, state_indices, torch::Tensor(), torch::Tensor(), r.size(0),
                                      state_indices.numel(), state.size(0), r.size(0), true);
    meta = Resolved{prepared.cu, prepared.slots, prepared.status, max_seqlen, prepared.workspace};
  }
  const c10::cuda::CUDAGuard guard(state.device());
  check_abi(frwkv_sm100_wkv7_recurrent_fp16_state(
      meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), elapsed_state.data_ptr<int>(),
      state.data_ptr(), static_cast<int>(state.size(0)), r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(),
      v.data_ptr(), a.data_ptr(), b.data_ptr(), decay_bias.has_value() ? decay_bias->data_ptr() : nullptr,
      output.data_ptr(), static_cast<int>(n), static_cast<int>(r.size(0)), static_cast<int>(h), FRWKV_DECAY_LOGITS,
      static_cast<float>(scale), static_cast<int>(meta.max_seqlen), nullptr,
      at::cuda::getCurrentCUDAStream(state.device().index()).stream()));
}

void tmix_wkv7_prefill_fp32(torch::Tensor query_start_loc, torch::Tensor state_indices, torch::Tensor state,
                            torch::Tensor r, torch::Tensor decay_logits, torch::Tensor k, torch::Tensor v,
                            torch::Tensor a, torch::Tensor b, torch::Tensor output, double scale,
                            std::optional<torch::Tensor> decay_bias, TicketPtr validated_metadata, int64_t max_seqlen,
                            const std::string& decay_mode, const std::string& strategy,
                            std::optional<torch::Tensor> output_f32, std::optional<torch::Tensor> error_flag) {
  const int mode = decay_code(decay_mode);
  TORCH_CHECK(strategy == "auto" || strategy == "recurrent" || strategy == "chunk_tc",
              "strategy must be 'auto', 'recurrent' or 'chunk_tc'");
  const int strategy_code = strategy == "auto" ? FRWKV_PREFILL_AUTO
                            : strategy == "recurrent" ? FRWKV_PREFILL_RECURRENT : FRWKV_PREFILL_CHUNK_TC;
  const auto dims = check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b, output,
                                           scale, true);
  check_decay_bias(decay_bias, state, r, mode);
  check_output_f32(output_f32, output);
  if (error_flag.has_value())
    TORCH_CHECK(error_flag->is_cuda() && error_flag->scalar_type() == torch::kInt32 && error_flag->numel() >= 1,
                "error_flag must be a CUDA int32 tensor");
  const auto meta = resolve_metadata(query_start_loc, state_indices, state, r, validated_metadata, max_seqlen);
  const c10::cuda::CUDAGuard guard(state.device());
  const size_t need = frwkv_sm100_wkv7_prefill_workspace_bytes(static_cast<int>(dims.sequences),
                                                               static_cast<int>(r.size(0)),
                                                               static_cast<int>(dims.heads));
  torch::Tensor workspace;
  if (need > 0) workspace = torch::empty({static_cast<int64_t>(need)}, state.options().dtype(torch::kUInt8));
  check_abi(frwkv_sm100_wkv7_prefill(
      meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(),
      decay_bias.has_value() ? decay_bias->data_ptr() : nullptr, output.data_ptr(),
      output_f32.has_value() ? output_f32->data_ptr<float>() : nullptr, static_cast<int>(dims.sequences),
      static_cast<int>(r.size(0)), static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale),
      static_cast<int>(meta.max_seqlen), strategy_code, need > 0 ? workspace.data_ptr() : nullptr, need,
      error_flag.has_value() ? error_flag->data_ptr<int>() : nullptr,
      at::cuda::getCurrentCUDAStream(state.device().index()).stream()));
}

// The two in-place operators with the kk / a-gate producer fused in (see include/frwkv_sm100.h): `k` is the raw key
// projection, `a12` the per-token gate logits, k_k / a0 / k_a the per-channel parameters [H*D] or [H,D].
void check_gate_parameter(const torch::Tensor& parameter, const torch::Tensor& state, const torch::Tensor& r,
                          const char* name) {
  check_cuda_contiguous(parameter, name);
  check_same_device(state, parameter, name);
  TORCH_CHECK(parameter.scalar_type() == r.scalar_type(), name, " must match the token tensor dtype");
  const int64_t h = state.size(1), d = state.size(2);
  TORCH_CHECK((parameter.dim() == 1 && parameter.numel() == h * d) ||
                  (parameter.dim() == 2 && parameter.size(0) == h && parameter.size(1) == d),
              name, " must have shape [H*D] or [H,D]");
}

void tmix_wkv7_fused_gate_fp32(torch::Tensor query_start_loc, torch::Tensor state_indices, torch::Tensor state,
                               torch::Tensor r, torch::Tensor decay_logits, torch::Tensor k, torch::Tensor v,
                               torch::Tensor a12, torch::Tensor k_k, torch::Tensor a0, torch::Tensor k_a,
                               torch::Tensor output, double scale, std::optional<torch::Tensor> decay_bias,
                               TicketPtr validated_metadata, int64_t max_seqlen, const std::string& decay_mode,
                               const std::string& strategy, std::optional<torch::Tensor> output_f32,
                               std::optional<torch::Tensor> error_flag) {
  const int mode = decay_code(decay_mode);
  TORCH_CHECK(strategy == "decode" || strategy == "auto" || strategy == "recurrent" || strategy == "chunk_tc",
              "strategy must be 'decode', 'auto', 'recurrent' or 'chunk_tc'");
  const auto dims = check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a12, a12,
                                           output, scale, false);
  check_decay_bias(decay_bias, state, r, mode);
  check_output_f32(output_f32, output);
  check_gate_parameter(k_k, state, r, "k_k");
  check_gate_parameter(a0, state, r, "a0");
  check_gate_parameter(k_a, state, r, "k_a");
  if (error_flag.has_value())
    TORCH_CHECK(error_flag->is_cuda() && error_flag->scalar_type() == torch::kInt32 && error_flag->numel() >= 1,
                "error_flag must be a CUDA int32 tensor");
  const auto meta = resolve_metadata(query_start_loc, state_indices, state, r, validated_metadata, max_seqlen);
  const c10::cuda::CUDAGuard guard(state.device());
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(state.device().index()).stream();
  const void* bias = decay_bias.has_value() ? decay_bias->data_ptr() : nullptr;
  float* y32 = output_f32.has_value() ? output_f32->data_ptr<float>() : nullptr;
  if (strategy == "decode") {
    check_abi(frwkv_sm100_wkv7_recurrent_fused_gate(
        meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
        r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a12.data_ptr(), k_k.data_ptr(), a0.data_ptr(),
        k_a.data_ptr(), bias, output.data_ptr(), y32, static_cast<int>(dims.sequences), static_cast<int>(r.size(0)),
        static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale), static_cast<int>(meta.max_seqlen),
        stream));
    return;
  }
  const int strategy_code = strategy == "auto" ? FRWKV_PREFILL_AUTO
                            : strategy == "recurrent" ? FRWKV_PREFILL_RECURRENT : FRWKV_PREFILL_CHUNK_TC;
  const size_t need = frwkv_sm100_wkv7_prefill_workspace_bytes(static_cast<int>(dims.sequences),
                                                               static_cast<int>(r.size(0)),
                                                               static_cast<int>(dims.heads));
  torch::Tensor workspace;
  if (need > 0) workspace = torch::empty({static_cast<int64_t>(need)}, state.options().dtype(torch::kUInt8));
  check_abi(frwkv_sm100_wkv7_prefill_fused_gate(
      meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a12.data_ptr(), k_k.data_ptr(), a0.data_ptr(),
      k_a.data_ptr(), bias, output.data_ptr(), y32, static_cast<int>(dims.sequences), static_cast<int>(r.size(0)),
      static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale), static_cast<int>(meta.max_seqlen),
      strategy_code, need > 0 ? workspace.data_ptr() : nullptr, need,
      error_flag.has_value() ? error_flag->data_ptr<int>() : nullptr, stream));
}

// WKV7 with the readout's elementwise stage (head norm, r.k residual, output gate): epilogue of the decode /
// short-row kernel (strategy "decode"), or a second launch behind the prefill strategies.  `output` receives the
// gated result that feeds the output projection; `wkv_output` (y itself) is stored only when given ("decode").  With
// k_k, a0 and k_a the kk / a-gate producer is fused in as well: k is then the raw key, a the gate logits a12, and b
// is not read.
void tmix_wkv7_readout_fp32(torch::Tensor query_start_loc, torch::Tensor state_indices, torch::Tensor state,
                            torch::Tensor r, torch::Tensor decay_logits, torch::Tensor k, torch::Tensor v,
                            torch::Tensor a, std::optional<torch::Tensor> b, torch::Tensor out_gate,
                            torch::Tensor r_k, torch::Tensor ln_weight, torch::Tensor ln_bias, torch::Tensor output,
                            double scale, std::optional<torch::Tensor> k_k, std::optional<torch::Tensor> a0,
                            std::optional<torch::Tensor> k_a, std::optional<torch::Tensor> decay_bias,
                            TicketPtr validated_metadata, int64_t max_seqlen, const std::string& decay_mode,
                            std::optional<torch::Tensor> wkv_output, std::optional<torch::Tensor> output_f32,
                            const std::string& strategy, std::optional<torch::Tensor> error_flag) {
  const int mode = decay_code(decay_mode);
  TORCH_CHECK(strategy == "decode" || strategy == "auto" || strategy == "recurrent" || strategy == "chunk_tc",
              "strategy must be 'decode', 'auto', 'recurrent' or 'chunk_tc'");
  if (error_flag.has_value())
    TORCH_CHECK(error_flag->is_cuda() && error_flag->scalar_type() == torch::kInt32 && error_flag->numel() >= 1,
                "error_flag must be a CUDA int32 tensor");
  const bool fused = k_k.has_value() || a0.has_value() || k_a.has_value();
  TORCH_CHECK(!fused || (k_k.has_value() && a0.has_value() && k_a.has_value()),
              "k_k, a0 and k_a must be given together");
  TORCH_CHECK(fused || b.has_value(), "b is required unless the kk / a-gate parameters are given");
  const torch::Tensor& b_checked = fused ? a : *b;
  const auto dims = check_recurrent_layout(query_start_loc, state_indices, state, r, decay_logits, k, v, a, b_checked,
                                           output, scale, false);
  TORCH_CHECK(r.scalar_type() != torch::kFloat32, "the readout epilogue takes float16 or bfloat16 tokens");
  check_decay_bias(decay_bias, state, r, mode);
  check_output_f32(output_f32, output);
  TORCH_CHECK(out_gate.is_cuda() && out_gate.is_contiguous() && out_gate.device() == r.device() &&
                  out_gate.scalar_type() == r.scalar_type() && out_gate.sizes() == r.sizes(),
              "out_gate must match r's packed shape, dtype and device");
  if (wkv_output.has_value())
    TORCH_CHECK(wkv_output->is_cuda() && wkv_output->is_contiguous() && wkv_output->device() == r.device() &&
                    wkv_output->scalar_type() == r.scalar_type() && wkv_output->sizes() == r.sizes(),
                "wkv_output must match r's packed shape, dtype and device");
  check_gate_parameter(r_k, state, r, "r_k");
  check_gate_parameter(ln_weight, state, r, "ln_weight");
  check_gate_parameter(ln_bias, state, r, "ln_bias");
  if (fused) {
    check_gate_parameter(*k_k, state, r, "k_k");
    check_gate_parameter(*a0, state, r, "a0");
    check_gate_parameter(*k_a, state, r, "k_a");
  }
  const auto meta = resolve_metadata(query_start_loc, state_indices, state, r, validated_metadata, max_seqlen);
  const c10::cuda::CUDAGuard guard(state.device());
  const cudaStream_t stream = at::cuda::getCurrentCUDAStream(state.device().index()).stream();
  if (strategy != "decode") {
    // prefill strategies: the recurrence stores y, a second launch applies the readout stage to those rows
    torch::Tensor y = wkv_output.has_value() ? *wkv_output : torch::empty_like(output);
    const int strategy_code = strategy == "auto" ? FRWKV_PREFILL_AUTO
                              : strategy == "recurrent" ? FRWKV_PREFILL_RECURRENT : FRWKV_PREFILL_CHUNK_TC;
    const size_t need = frwkv_sm100_wkv7_prefill_workspace_bytes(static_cast<int>(dims.sequences),
                                                                 static_cast<int>(r.size(0)),
                                                                 static_cast<int>(dims.heads));
    torch::Tensor workspace;
    if (need > 0) workspace = torch::empty({static_cast<int64_t>(need)}, state.options().dtype(torch::kUInt8));
    check_abi(frwkv_sm100_wkv7_prefill_readout(
        meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
        r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
        fused ? nullptr : b->data_ptr(), fused ? k_k->data_ptr() : nullptr, fused ? a0->data_ptr() : nullptr,
        fused ? k_a->data_ptr() : nullptr, decay_bias.has_value() ? decay_bias->data_ptr() : nullptr,
        out_gate.data_ptr(), r_k.data_ptr(), ln_weight.data_ptr(), ln_bias.data_ptr(), output.data_ptr(), y.data_ptr(),
        output_f32.has_value() ? output_f32->data_ptr<float>() : nullptr, static_cast<int>(dims.sequences),
        static_cast<int>(r.size(0)), static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale),
        static_cast<int>(meta.max_seqlen), strategy_code, need > 0 ? workspace.data_ptr() : nullptr, need,
        error_flag.has_value() ? error_flag->data_ptr<int>() : nullptr, stream));
    return;
  }
  check_abi(frwkv_sm100_wkv7_recurrent_readout(
      meta.cu.data_ptr<int>(), meta.slots.data_ptr<int>(), meta.status.data_ptr<int>(), state.data_ptr<float>(),
      r.data_ptr(), decay_logits.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
      fused ? nullptr : b->data_ptr(), fused ? k_k->data_ptr() : nullptr, fused ? a0->data_ptr() : nullptr,
      fused ? k_a->data_ptr() : nullptr, decay_bias.has_value() ? decay_bias->data_ptr() : nullptr,
      out_gate.data_ptr(), r_k.data_ptr(), ln_weight.data_ptr(), ln_bias.data_ptr(), output.data_ptr(),
      wkv_output.has_value() ? wkv_output->data_ptr() : nullptr,
      output_f32.has_value() ? output_f32->data_ptr<float>() : nullptr, static_cast<int>(dims.sequences),
      static_cast<int>(r.size(0)), static_cast<int>(dims.heads), io_code(r), mode, static_cast<float>(scale),
      static_cast<int>(meta.max_seqlen), stream));
}

// Reference-shaped chunk forward: `state` is the gathered working state [B,H,D,D]; returns
// (output, final_state) and leaves `state` untouched.  The reference's per-chunk host metadata is
// accepted for signature compatibility; only the sequence boundaries it encodes are used (recovered
// on the device, without a sync).  Both `strategy` values map to the one fused kernel.
py::tuple rl_infctx_tmix_wkv7_chunk_fp32io16_forward(torch::Tensor sequence_chunk_offsets,
                                                     torch::Tensor chunk_token_starts,
                                                     torch::Tensor chunk_token_ends, torch::Tensor state,
                                                     torch::Tensor r, torch::Tensor decay_logits, torch::Tensor k,
                                                     torch::Tensor v, torch::Tensor a, torch::Tensor b,
                                                     int64_t strategy, double scale,
                                                     std::optional<torch::Tensor> decay_bias,
                                                     const std::string& decay_mode) {
  TORCH_CHECK(strategy == 0 || strategy == 1, "strategy must be 0 (materialized) or 1 (recompute)");
  TORCH_CHECK(state.is_cuda() && state.is_contiguous() && state.scalar_type() == torch::kFloat32,
              "RL/Infctx state must be contiguous CUDA float32");
  TORCH_CHECK(state.dim() == 4 && state.size(0) > 0 && state.size(1) > 0 && state.size(2) == state.size(3) &&
                  (state.size(2) == 64 || state.size(2) == 128 || state.size(2) == 256),
              "RL/Infctx state must have shape [B,H,D,D], D in {64,128,256}");
  const std::pair<const torch::Tensor*, const char*> meta[] = {{&sequence_chunk_offsets, "sequence_chunk_offsets"},
                                                               {&chunk_token_starts, "chunk_token_starts"},
                                                               {&chunk_token_ends, "chunk_token_ends"}};
  for (const auto& item : meta) {
    check_cuda_contiguous(*item.first, item.second);
    TORCH_CHECK(item.first->scalar_type() == torch::kInt32 && item.first->dim() == 1, item.second,
                " must be a one-dimensional int32 tensor");
  }
  TORCH_CHECK(chunk_token_starts.sizes() == chunk_token_ends.sizes() && chunk_token_starts.numel() > 0,
              "chunk token metadata must have matching shape [C]");
  TORCH_CHECK(sequence_chunk_offsets.numel() == state.size(0) + 1, "query_start_loc must have shape [N+1]");
  const c10::cuda::CUDAGuard guard(state.device());
  auto working = state.clone();
  auto output = torch::empty_like(v);
  auto slots = torch::arange(state.size(0), torch::TensorOptions().device(state.device()).dtype(torch::kInt32));
  auto starts_ext = torch::cat({chunk_token_starts, chunk_token_ends.slice(0, chunk_token_ends.numel() - 1)});
  auto cu = starts_ext.index_select(0, sequence_chunk_offsets.to(torch::kInt64)).contiguous();
  tmix_wkv7_prefill_fp32(cu, slots, working, r, decay_logits, k, v, a, b, output, scale, decay_bias, nullptr, -1,
                         decay_mode, "auto", std::nullopt, std::nullopt);
  return py::make_tuple(output, working);
}

}  // namespace

void register_infer_tmix_wkv7_recurrent_fp32io16_bindings(py::module_& module) {
  py::class_<RecurrentMetadataTicket, TicketPtr>(module, "_RecurrentMetadataTicket")
      .def("_check_compatible", &RecurrentMetadataTicket::check_compatible, py::arg("query_start_loc"),
           py::arg("state_indices"), py::arg("total_tokens"), py::arg("state_pool_size"), py::arg("max_seqlen"))
      .def("_query_start_loc_snapshot", [](const TicketPtr& t) { return t->cu_snapshot(); })
      .def("_state_indices_snapshot", [](const TicketPtr& t) { return t->slots_snapshot(); })
      .def("_status", [](const TicketPtr& t) { return t->status(); })
      .def("_max_seqlen", [](const TicketPtr& t) { return t->max_seqlen(); })
      .def("_is_graph", [](const TicketPtr& t) { return t->graph_mode(); })
      .def("_num_active_tokens", [](const TicketPtr& t) { return t->num_active_tokens(); })
      .def("_num_active_sequences", [](const TicketPtr& t) { return t->num_active_sequences(); });
  module.def("prepare_tmix_wkv7_recurrent_metadata", &prepare_tmix_wkv7_recurrent_metadata,
             "Prepare packed recurrent metadata for same-stream reuse", py::arg("query_start_loc"),
             py::arg("state_indices"), py::arg("total_tokens"), py::arg("state_pool_size"),
             py::arg("max_seqlen") = -1);
  module.def("prepare_tmix_wkv7_recurrent_graph_metadata", &prepare_tmix_wkv7_recurrent_graph_metadata,
             "Prepare live packed recurrent metadata for warm-up or CUDA Graph capture", py::arg("query_start_loc"),
             py::arg("state_indices"), py::arg("num_active_tokens"), py::arg("num_active_sequences"),
             py::arg("token_capacity"), py::arg("sequence_capacity"), py::arg("state_pool_size"),
             py::arg("max_seqlen_capacity"));
  module.def("tmix_wkv7_recurrent_fp32_from_decay_logits", &tmix_wkv7_recurrent_fp32_from_decay_logits,
             "WKV7 recurrence with fused raw decay logits and fp32 state, in place", py::arg("query_start_loc"),
             py::arg("state_indices"), py::arg("state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"),
             py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"), py::arg("scale"),
             py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
             py::arg("max_seqlen") = -1, py::arg("decay_mode") = "logits", py::arg("output_f32") = py::none());
  module.def("tmix_wkv7_recurrent_fp16_from_decay_logits", &tmix_wkv7_recurrent_fp16_from_decay_logits,
             "WKV7 recurrence with an fp16 state pool, delta decay and elapsed-phase dither, in place",
             py::arg("query_start_loc"), py::arg("state_indices"), py::arg("elapsed_state_pool"), py::arg("state"),
             py::arg("r"), py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"),
             py::arg("output"), py::arg("scale"), py::arg("decay_bias") = py::none(),
             py::arg("validated_metadata") = py::none(), py::arg("max_seqlen") = -1);
  module.def("tmix_wkv7_fused_gate_fp32", &tmix_wkv7_fused_gate_fp32,
             "WKV7 with the kk / a-gate producer fused in (decode kernel or prefill strategies), fp32 state in place",
             py::arg("query_start_loc"), py::arg("state_indices"), py::arg("state"), py::arg("r"),
             py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a12"), py::arg("k_k"), py::arg("a0"),
             py::arg("k_a"), py::arg("output"), py::arg("scale"), py::arg("decay_bias") = py::none(),
             py::arg("validated_metadata") = py::none(), py::arg("max_seqlen") = -1, py::arg("decay_mode") = "logits",
             py::arg("strategy") = "auto", py::arg("output_f32") = py::none(), py::arg("error_flag") = py::none());
  module.def("tmix_wkv7_readout_fp32", &tmix_wkv7_readout_fp32,
             "WKV7 recurrence with the readout's head norm, r.k residual and output gate as epilogue",
             py::arg("query_start_loc"), py::arg("state_indices"), py::arg("state"), py::arg("r"),
             py::arg("decay_logits"), py::arg("k"), py::arg("v"), py::arg("a"), py::arg("b"), py::arg("out_gate"),
             py::arg("r_k"), py::arg("ln_weight"), py::arg("ln_bias"), py::arg("output"), py::arg("scale"),
             py::arg("k_k") = py::none(), py::arg("a0") = py::none(), py::arg("k_a") = py::none(),
             py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
             py::arg("max_seqlen") = -1, py::arg("decay_mode") = "logits", py::arg("wkv_output") = py::none(),
             py::arg("output_f32") = py::none(), py::arg("strategy") = "decode", py::arg("error_flag") = py::none());
  module.def("tmix_wkv7_prefill_fp32", &tmix_wkv7_prefill_fp32,
             "WKV7 chunked prefill taking cu_seqlens directly, fp32 state in place", py::arg("query_start_loc"),
             py::arg("state_indices"), py::arg("state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"),
             py::arg("v"), py::arg("a"), py::arg("b"), py::arg("output"), py::arg("scale"),
             py::arg("decay_bias") = py::none(), py::arg("validated_metadata") = py::none(),
             py::arg("max_seqlen") = -1, py::arg("decay_mode") = "logits", py::arg("strategy") = "auto",
             py::arg("output_f32") = py::none(), py::arg("error_flag") = py::none());
}

void register_rl_infctx_tmix_wkv7_chunk_forward_bindings(py::module_& module) {
  module.def("rl_infctx_tmix_wkv7_chunk_fp32io16_forward", &rl_infctx_tmix_wkv7_chunk_fp32io16_forward,
             "RL/Infctx raw-decay chunk forward", py::arg("sequence_chunk_offsets"), py::arg("chunk_token_starts"),
             py::arg("chunk_token_ends"), py::arg("state"), py::arg("r"), py::arg("decay_logits"), py::arg("k"),
             py::arg("v"), py::arg("a"), py::arg("b"), py::arg("strategy") = 1, py::arg("scale") = 1.0,
             py::arg("decay_bias") = py::none(), py::arg("decay_mode") = "logits");
}
