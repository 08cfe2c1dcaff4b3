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
#include "../../common.cuh"

#include <cstdlib>
#include <type_traits>

namespace frwkv {
namespace {

#ifndef FRWKV_WARPS_PER_CTA
#define FRWKV_WARPS_PER_CTA 4
#endif
constexpr int kWarpsPerCta = FRWKV_WARPS_PER_CTA;

template <typename io_t, int N> struct RowVals {  // N consecutive token-dtype values, kept packed
  static constexpr int kBytes = N * sizeof(io_t);
  static_assert(kBytes % 8 == 0, "row slice must be a multiple of 8 bytes");
  static constexpr int kWords = kBytes / 4;
  uint32_t raw[kWords];
  __device__ __forceinline__ void load(const io_t* p) {
    if constexpr (kBytes % 16 == 0) {
#pragma unroll
      for (int i = 0; i < kBytes / 16; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(p) + i);
        raw[4 * i] = q.x; raw[4 * i + 1] = q.y; raw[4 * i + 2] = q.z; raw[4 * i + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < kBytes / 8; ++i) {
        const uint2 q = __ldg(reinterpret_cast<const uint2*>(p) + i);
        raw[2 * i] = q.x; raw[2 * i + 1] = q.y;
      }
    }
  }
  __device__ __forceinline__ float get(int i) const {
    if constexpr (sizeof(io_t) == 4) {
      return __uint_as_float(raw[i]);
    } else {
      const uint32_t word = raw[i >> 1];
      const unsigned short bits = static_cast<unsigned short>((i & 1) ? (word >> 16) : (word & 0xffffu));
      if constexpr (std::is_same<io_t, __nv_bfloat16>::value) {
        return __uint_as_float(static_cast<uint32_t>(bits) << 16);
      } else {
        return __half2float(__ushort_as_half(bits));
      }
    }
  }
};

template <typename io_t> struct Quad {  // 4 consecutive token-dtype values (value columns)
  io_t vals[4];
  __device__ __forceinline__ void load(const io_t* p) {
    if constexpr (sizeof(io_t) == 2) {
      *reinterpret_cast<uint2*>(vals) = __ldg(reinterpret_cast<const uint2*>(p));
    } else {
      *reinterpret_cast<uint4*>(vals) = __ldg(reinterpret_cast<const uint4*>(p));
    }
  }
  __device__ __forceinline__ void store(io_t* p) const {
    if constexpr (sizeof(io_t) == 2) {
      *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(vals);
    } else {
      *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(vals);
    }
  }
};

template <typename io_t, int RPL> struct TokenRows {  // one token's operands for this lane
  RowVals<io_t, RPL> r, w, k, a, b;
  Quad<io_t> v;
};

struct RecurrentParams {
  const int* cu;
  const int* slots;
  const int* status;
  float* pool;
  const void *r, *w, *k, *v, *a, *b, *bias;
  void* y;
  float* y_f32;
  int n_seq, total_tokens, heads;
  float scale;
  int len_below;  // > 0: only sequences shorter than this (the rest belongs to another kernel of the same call)
};

template <typename io_t, int PARTS, bool LOGITS, bool PREFETCH>
__global__ void __launch_bounds__(kWarpsPerCta * 32) wkv7_recurrent_stream_kernel(const RecurrentParams p) {
  constexpr int COLS = kHeadDim / PARTS;   // value columns of this warp
  constexpr int LPR = COLS / 4;            // lanes per key row
  constexpr int GROUPS = 32 / LPR;         // key-row groups in a warp
  constexpr int RPL = kHeadDim / GROUPS;   // key rows per lane
  const int lane = threadIdx.x & 31;
  const long long warp = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);

  // Programmatic dependent launch: this grid may be scheduled while the previous kernel of the stream
  // drains (its launch latency and ramp are hidden), but nothing is read before that kernel has
  // completed and its writes are visible -- the state pool is updated in place from step to step.
  // Without the launch attribute both instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (p.status != nullptr && p.status[0] != 0) {
    fill_output_nan(static_cast<io_t*>(p.y), p.y_f32,
                    static_cast<long long>(p.total_tokens) * p.heads * kHeadDim,
                    static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x,
                    static_cast<long long>(gridDim.x) * blockDim.x);
    return;
  }
  const int active = p.status != nullptr ? p.status[2] : p.n_seq;
  const long long pair = warp / PARTS;
  const int part = static_cast<int>(warp % PARTS);
  const int seq = static_cast<int>(pair / p.heads);
  const int head = static_cast<int>(pair % p.heads);
  if (seq >= active || seq >= p.n_seq) return;

  const int t_lo = p.cu[seq], t_hi = p.cu[seq + 1];
  if (p.len_below > 0 && t_hi - t_lo >= p.len_below) return;
  const int slot = p.slots[seq];
  const int group = lane / LPR;
  const int col = part * COLS + (lane % LPR) * 4;
  const int row0 = group * RPL;

  float* sbase = p.pool + (static_cast<size_t>(slot) * p.heads + head) * (kHeadDim * kHeadDim) +
                 static_cast<size_t>(row0) * kHeadDim + col;
  float4 S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) S[i] = __ldcs(reinterpret_cast<const float4*>(sbase + i * kHeadDim));

  const io_t* rp = static_cast<const io_t*>(p.r);
  const io_t* wp = static_cast<const io_t*>(p.w);
  const io_t* kp = static_cast<const io_t*>(p.k);
  const io_t* vp = static_cast<const io_t*>(p.v);
  const io_t* ap = static_cast<const io_t*>(p.a);
  const io_t* bp = static_cast<const io_t*>(p.b);
  io_t* yp = static_cast<io_t*>(p.y);

  RowVals<io_t, RPL> bias;
  const bool has_bias = LOGITS && p.bias != nullptr;
  if (has_bias) bias.load(static_cast<const io_t*>(p.bias) + head * kHeadDim + row0);

  auto fetch = [&](TokenRows<io_t, RPL>& dst, int t) {
    const size_t row = (static_cast<size_t>(t) * p.heads + head) * kHeadDim;
    dst.a.load(ap + row + row0);
    dst.w.load(wp + row + row0);
    dst.b.load(bp + row + row0);
    dst.k.load(kp + row + row0);
    dst.r.load(rp + row + row0);
    dst.v.load(vp + row + col);
  };
  TokenRows<io_t, RPL> cur, nxt;
  if (PREFETCH && t_lo < t_hi) fetch(nxt, t_lo);

  for (int t = t_lo; t < t_hi; ++t) {
    if constexpr (PREFETCH) {
      cur = nxt;
      if (t + 1 < t_hi) fetch(nxt, t + 1);  // next token's rows are in flight during the math
    } else {
      fetch(cur, t);
    }
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const float fa = cur.a.get(i);
      sa.x = fmaf(fa, S[i].x, sa.x);
      sa.y = fmaf(fa, S[i].y, sa.y);
      sa.z = fmaf(fa, S[i].z, sa.z);
      sa.w = fmaf(fa, S[i].w, sa.w);
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1) {
      sa.x += __shfl_xor_sync(0xffffffffu, sa.x, m);
      sa.y += __shfl_xor_sync(0xffffffffu, sa.y, m);
      sa.z += __shfl_xor_sync(0xffffffffu, sa.z, m);
      sa.w += __shfl_xor_sync(0xffffffffu, sa.w, m);
    }
    const float4 v4 = make_float4(to_f32(cur.v.vals[0]), to_f32(cur.v.vals[1]), to_f32(cur.v.vals[2]),
                                  to_f32(cur.v.vals[3]));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      float fw = cur.w.get(i);
      if constexpr (LOGITS) fw = retention_from_logit(has_bias ? fw + bias.get(i) : fw);
      const float fb = cur.b.get(i), fk = cur.k.get(i), fr = cur.r.get(i);
      S[i].x = fmaf(fw, S[i].x, fmaf(fb, sa.x, fk * v4.x));
      S[i].y = fmaf(fw, S[i].y, fmaf(fb, sa.y, fk * v4.y));
      S[i].z = fmaf(fw, S[i].z, fmaf(fb, sa.z, fk * v4.z));
      S[i].w = fmaf(fw, S[i].w, fmaf(fb, sa.w, fk * v4.w));
      acc.x = fmaf(fr, S[i].x, acc.x);
      acc.y = fmaf(fr, S[i].y, acc.y);
      acc.z = fmaf(fr, S[i].z, acc.z);
      acc.w = fmaf(fr, S[i].w, acc.w);
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1) {
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, m);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, m);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, m);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, m);
    }
    if (group == 0) {
      const size_t out = (static_cast<size_t>(t) * p.heads + head) * kHeadDim + col;
      acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
      Quad<io_t> q;
      q.vals[0] = from_f32<io_t>(acc.x);
      q.vals[1] = from_f32<io_t>(acc.y);
      q.vals[2] = from_f32<io_t>(acc.z);
      q.vals[3] = from_f32<io_t>(acc.w);
      q.store(yp + out);
      if (p.y_f32 != nullptr) *reinterpret_cast<float4*>(p.y_f32 + out) = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < RPL; ++i) __stcs(reinterpret_cast<float4*>(sbase + i * kHeadDim), S[i]);
}

// Tuning hooks, read from the environment once per process (not on every launch):
// FRWKV_PDL=0 turns programmatic dependent launch off; FRWKV_RECURRENT_PARTS=2|4|8 forces the column split.
inline bool pdl_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("FRWKV_PDL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return enabled;
}
inline int parts_from_environment() {
  static const int parts = [] {
    const char* e = std::getenv("FRWKV_RECURRENT_PARTS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  return parts;
}
#ifdef FRWKV_TEST_HOOKS
int& test_recurrent_parts() {  // test build only: column split forced by the next launches (0 = none)
  static int parts = 0;
  return parts;
}
#endif

template <typename io_t, int PARTS, bool PREFETCH>
int launch(const RecurrentParams& p, bool logits, cudaStream_t stream) {
  const long long warps = static_cast<long long>(p.n_seq) * p.heads * PARTS;
  const long long ctas = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
  if (ctas > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "recurrent: too many (sequence, head) pairs");
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(ctas));
  config.blockDim = dim3(kWarpsPerCta * 32);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  // one-token steps only (PREFETCH is off exactly there): the next step's CTAs then ramp up under this step's tail.
  // Multi-token rows run for milliseconds; measured on the dense 8 x 4096 prefill, dependent CTAs that take their
  // slots early make back-to-back calls 59 % slower (4.36 ms against 2.75 ms).
  attribute[0].val.programmaticStreamSerializationAllowed = (!PREFETCH && pdl_enabled()) ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  auto kernel = logits ? wkv7_recurrent_stream_kernel<io_t, PARTS, true, PREFETCH>
                       : wkv7_recurrent_stream_kernel<io_t, PARTS, false, PREFETCH>;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, p);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_stream_kernel: %s", cudaGetErrorString(err));
  return check_launch("wkv7_recurrent_stream_kernel");
}

template <typename io_t>
int dispatch_parts(const RecurrentParams& p, bool logits, int parts, bool prefetch, cudaStream_t stream) {
  if (!prefetch) {
    if (parts == 2) return launch<io_t, 2, false>(p, logits, stream);
    if (parts == 4) return launch<io_t, 4, false>(p, logits, stream);
    return launch<io_t, 8, false>(p, logits, stream);
  }
  if (parts == 2) return launch<io_t, 2, true>(p, logits, stream);
  if (parts == 4) return launch<io_t, 4, true>(p, logits, stream);
  return launch<io_t, 8, true>(p, logits, stream);
}

}  // namespace

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
                            int max_seqlen, int parts_override, int len_below, cudaStream_t stream) {
  RecurrentParams p{cu, slots, status, pool, r, w, k, v, a, b, bias, y, y_f32, n_seq, total_tokens, heads, scale,
                    len_below};
  // Launch shape.  Decode (one token per row): the state is loaded, used once and stored,
  // so all that matters is bytes in flight; two column parts per pair keep every access a
  // full 128-byte line.  Long rows are a latency-bound token loop: thinner warps (more of
  // them, fewer rows per lane, next token prefetched) shorten the per-token chain.
  int parts = 2;
  const long long pairs = static_cast<long long>(n_seq) * heads;
  if (max_seqlen <= 0 || max_seqlen > 2) parts = 4;
  if (max_seqlen <= 0 || max_seqlen > 64 || pairs < 148LL * 4) parts = 8;
  if (parts_override == 0) parts_override = parts_from_environment();
#ifdef FRWKV_TEST_HOOKS
  if (test_recurrent_parts() != 0) parts_override = test_recurrent_parts();
#endif
  if (parts_override == 2 || parts_override == 4 || parts_override == 8) parts = parts_override;
  const bool prefetch = max_seqlen <= 0 || max_seqlen > 1;
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  switch (io_dtype) {
    case FRWKV_IO_BF16: return dispatch_parts<__nv_bfloat16>(p, logits, parts, prefetch, stream);
    case FRWKV_IO_FP16: return dispatch_parts<__half>(p, logits, parts, prefetch, stream);
    default: return dispatch_parts<float>(p, logits, parts, prefetch, stream);
  }
}

}  // namespace frwkv

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
                                 n_seq, total_tokens, heads, io_dtype, decay_mode, scale, max_seqlen, 0, 0,
                                 static_cast<cudaStream_t>(stream));
}

#ifdef FRWKV_TEST_HOOKS
// Test build only: force the column split (2, 4 or 8; 0 = automatic) of the recurrence kernel's next launches.
extern "C" void frwkv_sm100_test_recurrent_parts(int parts) { frwkv::test_recurrent_parts() = parts; }
#endif
