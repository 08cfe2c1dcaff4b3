// Device-side validation of packed-sequence metadata for the WKV7 state pool.
//
// Behaviour follows rwkv-rs/FlashRWKV2 csrc/validation/recurrent_metadata.cu:24-132:
// the same six error bits, the same status word {error, active tokens, active
// sequences} with the counts zeroed on error, optional snapshots that are what gets
// validated, and optional live active counts (the CUDA-graph form).  One CTA of 1024
// threads; the slot scratch is cleared with 128-bit stores.
#include "../../common.cuh"

namespace frwkv {
namespace {

constexpr int kThreads = 1024;

__global__ void __launch_bounds__(kThreads) validate_metadata_kernel(
    const int* __restrict__ cu, const int* __restrict__ slots, int n_seq_cap, int tok_cap,
    int pool_size, int max_seqlen, const int* __restrict__ n_active_tok,
    const int* __restrict__ n_active_seq, int* __restrict__ status, int* __restrict__ seen,
    int* __restrict__ cu_snap, int* __restrict__ slots_snap) {
  __shared__ int s_err, s_tok, s_seq;
  const int tid = threadIdx.x;
  if (tid == 0) {
    int tok = n_active_tok ? n_active_tok[0] : tok_cap;
    int seq = n_active_seq ? n_active_seq[0] : n_seq_cap;
    int err = 0;
    if (tok < 0 || tok > tok_cap || seq < 0 || seq > n_seq_cap || ((tok == 0) != (seq == 0))) {
      err = FRWKV_META_BAD_ACTIVE_COUNT;
      tok = 0;
      seq = 0;
    }
    s_err = err;
    s_tok = tok;
    s_seq = seq;
  }
  // clear the duplicate-detection scratch
  {
    const int vec = ((reinterpret_cast<uintptr_t>(seen) & 15) == 0) ? pool_size / 4 : 0;
    int4* seen4 = reinterpret_cast<int4*>(seen);
    for (int i = tid; i < vec; i += kThreads) seen4[i] = make_int4(-1, -1, -1, -1);
    for (int i = vec * 4 + tid; i < pool_size; i += kThreads) seen[i] = -1;
  }
  if (cu_snap != nullptr) {
    for (int i = tid; i <= n_seq_cap; i += kThreads) cu_snap[i] = cu[i];
    for (int i = tid; i < n_seq_cap; i += kThreads) slots_snap[i] = slots[i];
  }
  __syncthreads();
  const int* vcu = cu_snap ? cu_snap : cu;
  const int* vslots = cu_snap ? slots_snap : slots;
  const int tok = s_tok, seq = s_seq;
  // The end-point test looks at the error word, so it is finished (barrier) before any thread can add a range or
  // slot error to it: whether the end-point bit appears beside those never depends on timing.
  if (tid == 0 && s_err == 0 && (vcu[0] != 0 || vcu[seq] != tok)) s_err = FRWKV_META_BAD_ENDPOINT;
  __syncthreads();
  int err = 0;
  for (int i = tid; i < seq; i += kThreads) {
    const int lo = vcu[i], hi = vcu[i + 1];
    if (lo < 0 || hi <= lo || hi > tok) {
      err |= FRWKV_META_BAD_RANGE;
    } else if (hi - lo > max_seqlen) {
      err |= FRWKV_META_SEQUENCE_TOO_LONG;
    }
    const int slot = vslots[i];
    if (slot < 0 || slot >= pool_size) {
      err |= FRWKV_META_BAD_SLOT;
    } else if (atomicCAS(seen + slot, -1, i) != -1) {
      err |= FRWKV_META_DUPLICATE_SLOT;
    }
  }
  if (err != 0) atomicOr(&s_err, err);
  __syncthreads();
  if (tid == 0) {
    status[0] = s_err;
    status[1] = s_err == 0 ? tok : 0;
    status[2] = s_err == 0 ? seq : 0;
  }
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_validate_metadata(
    const int32_t* cu_seqlens, const int32_t* slots, int n_seq_capacity, int token_capacity,
    int pool_size, int max_seqlen, const int32_t* n_active_tokens,
    const int32_t* n_active_sequences, int32_t* status, int32_t* seen_slots,
    int32_t* cu_snapshot, int32_t* slots_snapshot, void* stream) {
  using namespace frwkv;
  if (!cu_seqlens || !slots || !status || !seen_slots)
    return fail(FRWKV_ERR_ARGUMENT, "validate_metadata: cu_seqlens, slots, status and seen_slots must be non-null");
  if ((cu_snapshot == nullptr) != (slots_snapshot == nullptr))
    return fail(FRWKV_ERR_ARGUMENT, "validate_metadata: pass both snapshots or neither");
  if (n_seq_capacity <= 0 || n_seq_capacity > 65535)
    return fail(FRWKV_ERR_ARGUMENT, "validate_metadata: sequence count must be in 1..65535, got %d", n_seq_capacity);
  if (token_capacity <= 0 || pool_size <= 0 || max_seqlen <= 0)
    return fail(FRWKV_ERR_ARGUMENT, "validate_metadata: token_capacity, pool_size and max_seqlen must be positive");
  validate_metadata_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      cu_seqlens, slots, n_seq_capacity, token_capacity, pool_size, max_seqlen, n_active_tokens,
      n_active_sequences, status, seen_slots, cu_snapshot, slots_snapshot);
  return check_launch("validate_metadata");
}

// ---- the same validation with built-in scratch: nothing is allocated by anyone ----------------
//
// Some hosts that bind this library have no way to hand over device scratch: a foreign-language
// runtime that wraps only the launch calls and owns no device allocator, or a serving loop that
// must not call cudaMalloc on its hot path because that call can synchronise the whole device.
// For them the duplicate-slot scratch lives in this module's own global memory: a fixed array
// that every GPU loading the library keeps until the process exits (256 KiB).
namespace frwkv {
namespace {

constexpr int kStaticSeenSlots = FRWKV_SM100_STATIC_POOL_SLOTS;
static __device__ __align__(256) int g_static_seen_slots[kStaticSeenSlots];

constexpr int kMaxDevices = 64;
int* g_static_seen_ptr[kMaxDevices] = {nullptr};  // device address of the array, per device

// In host code the array's name is only a handle; the device address must be asked for, once per
// device and with that device current.
int static_scratch(int** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "validate_metadata_static: cudaGetDevice: %s", cudaGetErrorString(err));
  if (device < 0 || device >= kMaxDevices)
    return fail(FRWKV_ERR_UNSUPPORTED, "validate_metadata_static: device index %d out of range", device);
  if (g_static_seen_ptr[device] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_seen_slots);
    if (err != cudaSuccess || ptr == nullptr)
      return fail(FRWKV_ERR_CUDA, "validate_metadata_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
    g_static_seen_ptr[device] = static_cast<int*>(ptr);
  }
  *out = g_static_seen_ptr[device];
  return FRWKV_OK;
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_validate_metadata_static(
    const int32_t* cu_seqlens, const int32_t* slots, int n_seq_capacity, int token_capacity,
    int pool_size, int max_seqlen, const int32_t* n_active_tokens,
    const int32_t* n_active_sequences, int32_t* status, int32_t* cu_snapshot,
    int32_t* slots_snapshot, void* stream) {
  using namespace frwkv;
  if (pool_size > kStaticSeenSlots)
    return fail(FRWKV_ERR_UNSUPPORTED,
                "validate_metadata_static: state pool of %d slots exceeds the built-in scratch of %d slots; "
                "use frwkv_sm100_wkv7_validate_metadata with caller-provided scratch",
                pool_size, kStaticSeenSlots);
  int* seen = nullptr;
  const int rc = static_scratch(&seen);
  if (rc != FRWKV_OK) return rc;
  // the kernel itself resets the first pool_size entries to "unseen" before using them, so
  // whatever the previous call left behind cannot leak into this one
  return frwkv_sm100_wkv7_validate_metadata(cu_seqlens, slots, n_seq_capacity, token_capacity, pool_size,
                                            max_seqlen, n_active_tokens, n_active_sequences, status, seen,
                                            cu_snapshot, slots_snapshot, stream);
}
