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

template <typename io_t> struct Pair {  // 2 consecutive token-dtype values
  io_t vals[2];
  __device__ __forceinline__ void load(const io_t* p) {
    if constexpr (sizeof(io_t) == 2) {
      *reinterpret_cast<uint32_t*>(vals) = __ldg(reinterpret_cast<const uint32_t*>(p));
    } else {
      *reinterpret_cast<uint2*>(vals) = __ldg(reinterpret_cast<const uint2*>(p));
    }
  }
};

template <typename io_t, int RPL> struct TokenRows {  // one token's operands for this lane
  RowVals<io_t, RPL> r, w, k, a, b;
  Pair<io_t> w2;  // the two key rows whose decay this lane evaluates for its row group (see the kernel)
  Pair<io_t> g2, k2;  // fused producer: gate logits a12 and raw key of the same two rows
  Quad<io_t> v;
};

// Dither of the fp16-state update (csrc/sm120/tmix/wkv7/recurrent_decay.cuh:32-46 of the reference): a
// multiplicative hash of the phase, scaled to +-2^-10, added to rho - 1 before it is rounded to fp16.
__device__ __forceinline__ float fp16_state_dither(int phase) {
  const uint32_t bits = 2654435769u * static_cast<uint32_t>(phase);
  return 4.547473508864641e-13f * static_cast<float>(static_cast<int32_t>(bits));
}
__device__ __forceinline__ float round_to_half(float x) { return __half2float(__float2half_rn(x)); }

// four consecutive state values of one key row
template <typename state_t> __device__ __forceinline__ float4 load_state4(const state_t* p);
template <> __device__ __forceinline__ float4 load_state4<float>(const float* p) {
  return __ldcs(reinterpret_cast<const float4*>(p));
}
template <> __device__ __forceinline__ float4 load_state4<__half>(const __half* p) {
  const uint2 q = __ldcs(reinterpret_cast<const uint2*>(p));
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store_state4(float* p, const float4& v) { __stcs(reinterpret_cast<float4*>(p), v); }
__device__ __forceinline__ void store_state4(__half* p, const float4& v) {
  const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  uint2 q;
  q.x = *reinterpret_cast<const uint32_t*>(&lo);
  q.y = *reinterpret_cast<const uint32_t*>(&hi);
  __stcs(reinterpret_cast<uint2*>(p), q);
}

struct RecurrentParams {
  const int* cu;
  const int* slots;
  const int* status;
  void* pool;           // fp32 pool, or fp16 pool of the fp16-state contract
  const int* elapsed;   // fp16-state contract: per-slot phase counter (read here, advanced by advance_elapsed_kernel)
  const void *r, *w, *k, *v, *a, *b, *bias;
  void* y;
  float* y_f32;
  int n_seq, total_tokens, heads;
  float scale;
  int len_below;  // > 0: only sequences shorter than this (the rest belongs to another kernel of the same call)
  // fused producer (all three non-null or all null): per-channel [H*64] parameters of the kk / a-gate.  With them
  // k is the raw key projection and a is the per-token gate logit a12; b is not read.
  const void *gate_kk, *gate_a0, *gate_ka;
};

// The gate of the reference's producer kernel (csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/
// infer_fp16_forward_varlen.cu:52-106,131-156): sigmoid as 1 / (1 + exp(-x)) with the fast exponential.
__device__ __forceinline__ float gate_sigmoid(float x) { return 1.0f / (1.0f + __expf(-x)); }
// The producer stores its three outputs in the token dtype; the fused path rounds at the same point so that it
// reproduces the two-kernel pipeline.
template <typename io_t> __device__ __forceinline__ float round_io(float x) { return to_f32(from_f32<io_t>(x)); }

// Resident CTAs per SM asked of the compiler.  The one-token kernels are sized by bytes in flight: with an fp32
// state 4 CTAs (128 registers) already saturate HBM; a warp of the fp16-state kernel carries half the bytes, so it
// runs with 5 (96 registers, a few spilled words).  0 = no request (multi-token variants).  A request of 1 is not
// the same as none: it makes the compiler spend 190 registers and costs a third of the bandwidth.
#ifndef FRWKV_HALF_STATE_MIN_CTAS
#define FRWKV_HALF_STATE_MIN_CTAS 5
#endif
template <typename io_t, typename state_t, int PARTS, bool LOGITS, bool PREFETCH, bool FUSED = false>
__global__ void __launch_bounds__(kWarpsPerCta * 32,
                                  (PREFETCH || sizeof(io_t) == 4)
                                      ? 0 : (std::is_same<state_t, __half>::value ? FRWKV_HALF_STATE_MIN_CTAS : 4))
wkv7_recurrent_stream_kernel(const RecurrentParams p) {
  constexpr bool kHalfState = std::is_same<state_t, __half>::value;
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

  state_t* sbase = static_cast<state_t*>(p.pool) + (static_cast<size_t>(slot) * p.heads + head) * (kHeadDim * kHeadDim) +
                   static_cast<size_t>(row0) * kHeadDim + col;
  float4 S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) S[i] = load_state4<state_t>(sbase + i * kHeadDim);

  const io_t* rp = static_cast<const io_t*>(p.r);
  const io_t* wp = static_cast<const io_t*>(p.w);
  const io_t* kp = static_cast<const io_t*>(p.k);
  const io_t* vp = static_cast<const io_t*>(p.v);
  const io_t* ap = static_cast<const io_t*>(p.a);
  const io_t* bp = static_cast<const io_t*>(p.b);
  io_t* yp = static_cast<io_t*>(p.y);

  // Decay per key row.  In retention mode with an fp32 state the lane simply reads w for its rows.  Otherwise the
  // decay is work per row (two exp2 and a divide for logits; dither, delta and a rounding for the fp16 state) that
  // the LPR lanes of a row group would repeat: every lane does it for two of the group's rows (RPL = 2 * LPR for
  // every column split) and the values are handed round with shuffles.
  constexpr bool kSharedDecay = LOGITS || kHalfState;
  static_assert(RPL == 2 * LPR, "two decay rows per lane");
  const int my_rows = row0 + 2 * (lane % LPR);
  Pair<io_t> bias2;
  const bool has_bias = LOGITS && p.bias != nullptr;
  if (has_bias) bias2.load(static_cast<const io_t*>(p.bias) + head * kHeadDim + my_rows);
  int phase0 = 0;  // fp16 state: dither phase of this lane's first decay row at the sequence's first token
  if constexpr (kHalfState) phase0 = p.elapsed[slot] + head * kHeadDim + my_rows - t_lo;

  // fused producer: every lane evaluates the gate for the same two key rows whose decay it evaluates (the 32 lanes
  // of the warp cover the 64 rows exactly once), so it needs the per-channel parameters of those two rows only
  Pair<io_t> gate_kk, gate_ka, gate_a0;
  if constexpr (FUSED) {
    gate_kk.load(static_cast<const io_t*>(p.gate_kk) + head * kHeadDim + my_rows);
    gate_ka.load(static_cast<const io_t*>(p.gate_ka) + head * kHeadDim + my_rows);
    gate_a0.load(static_cast<const io_t*>(p.gate_a0) + head * kHeadDim + my_rows);
  }

  auto fetch = [&](TokenRows<io_t, RPL>& dst, int t) {
    const size_t row = (static_cast<size_t>(t) * p.heads + head) * kHeadDim;
    if constexpr (FUSED) {  // raw key and gate logits a12 of this lane's two gate rows only; b is not read
      dst.g2.load(ap + row + my_rows);
      dst.k2.load(kp + row + my_rows);
      dst.r.load(rp + row + row0);
      dst.v.load(vp + row + col);
      if constexpr (kSharedDecay) {
        dst.w2.load(wp + row + my_rows);
      } else {
        dst.w.load(wp + row + row0);
      }
      return;
    }
    dst.a.load(ap + row + row0);
    if constexpr (kSharedDecay) {
      dst.w2.load(wp + row + my_rows);
    } else {
      dst.w.load(wp + row + row0);
    }
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
    // fused producer, for this lane's two rows: kk = normalize(k * kk_scale) over the 64 channels (a full-warp sum:
    // the lanes hold two rows each), a = -kk, b = kk * g, k' = k * (1 + (g - 1) * k_a), g = sigmoid(a0 + a12);
    // rounded to the token dtype and handed to the lanes of the row group with shuffles
    float own_a[2] = {0.f, 0.f}, own_b[2] = {0.f, 0.f}, own_k[2] = {0.f, 0.f};
    if constexpr (FUSED) {
      float u[2], ss = 0.f;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        u[e] = to_f32(cur.k2.vals[e]) * to_f32(gate_kk.vals[e]);
        ss = fmaf(u[e], u[e], ss);
      }
      // each of the 64 rows belongs to exactly one lane of this warp: a sum over all 32 lanes is the whole norm
#pragma unroll
      for (int m = 1; m < 32; m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float inv_norm = 1.0f / fmaxf(sqrtf(ss), 1.0e-12f);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float g = gate_sigmoid(to_f32(gate_a0.vals[e]) + to_f32(cur.g2.vals[e]));
        const float kk = u[e] * inv_norm, ka = to_f32(gate_ka.vals[e]);
        own_a[e] = round_io<io_t>(-kk);
        own_b[e] = round_io<io_t>(kk * g);
        own_k[e] = round_io<io_t>(to_f32(cur.k2.vals[e]) * fmaf(g, ka, 1.0f - ka));
      }
    }
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      float fa;
      if constexpr (FUSED) {
        fa = __shfl_sync(0xffffffffu, own_a[i & 1], group * LPR + (i >> 1));
      } else {
        fa = cur.a.get(i);
      }
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
    float mine[2] = {0.f, 0.f};  // rho (fp32 state) or delta (fp16 state) of this lane's two decay rows
    if constexpr (kSharedDecay) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = to_f32(cur.w2.vals[e]);
        if constexpr (LOGITS) {
          if (has_bias) x += to_f32(bias2.vals[e]);
#if defined(FRWKV_EXP_IDENTITY)
          x = 0.9f;
#elif defined(FRWKV_FAST_DECAY)
          x = sizeof(io_t) == 2 ? retention_from_logit_fast(x) : retention_from_logit(x);
#else
          x = retention_from_logit(x);
#endif
        }
        if constexpr (kHalfState) x = round_to_half(x - 1.0f + fp16_state_dither(phase0 + e + t));
        mine[e] = x;
      }
    }
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      float fw;
      if constexpr (kSharedDecay) {
        fw = __shfl_sync(0xffffffffu, mine[i & 1], group * LPR + (i >> 1));
      } else {
        fw = cur.w.get(i);
      }
      float fb, fk;
      const float fr = cur.r.get(i);
      if constexpr (FUSED) {
        fb = __shfl_sync(0xffffffffu, own_b[i & 1], group * LPR + (i >> 1));
        fk = __shfl_sync(0xffffffffu, own_k[i & 1], group * LPR + (i >> 1));
      } else {
        fb = cur.b.get(i);
        fk = cur.k.get(i);
      }
      if constexpr (kHalfState) {
        // S + S*delta + b*sa + k*v in fp32, then rounded to the stored precision; y reads the rounded state
        const float delta = fw;
        S[i].x = round_to_half(fmaf(fk, v4.x, fmaf(fb, sa.x, fmaf(S[i].x, delta, S[i].x))));
        S[i].y = round_to_half(fmaf(fk, v4.y, fmaf(fb, sa.y, fmaf(S[i].y, delta, S[i].y))));
        S[i].z = round_to_half(fmaf(fk, v4.z, fmaf(fb, sa.z, fmaf(S[i].z, delta, S[i].z))));
        S[i].w = round_to_half(fmaf(fk, v4.w, fmaf(fb, sa.w, fmaf(S[i].w, delta, S[i].w))));
      } else {
        S[i].x = fmaf(fw, S[i].x, fmaf(fb, sa.x, fk * v4.x));
        S[i].y = fmaf(fw, S[i].y, fmaf(fb, sa.y, fk * v4.y));
        S[i].z = fmaf(fw, S[i].z, fmaf(fb, sa.z, fk * v4.z));
        S[i].w = fmaf(fw, S[i].w, fmaf(fb, sa.w, fk * v4.w));
      }
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
  for (int i = 0; i < RPL; ++i) store_state4(sbase + i * kHeadDim, S[i]);
}

// fp16-state contract: after the recurrence every active sequence's phase counter moves on by its token count
// (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:57-75 of the reference).  A separate launch: the
// recurrence's CTAs of all heads read the counter, so nobody may change it while they run.  Fail-closed like the
// recurrence: invalid metadata leaves every counter untouched.
__global__ void advance_elapsed_kernel(const int* __restrict__ cu, const int* __restrict__ slots,
                                       const int* __restrict__ status, int* __restrict__ elapsed, int n_seq) {
  if (status != nullptr && status[0] != 0) return;
  const int active = status != nullptr ? status[2] : n_seq;
  const int seq = blockIdx.x * blockDim.x + threadIdx.x;
  if (seq >= n_seq || seq >= active) return;
  elapsed[slots[seq]] += cu[seq + 1] - cu[seq];
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

template <typename io_t, typename state_t, int PARTS, bool PREFETCH, bool FUSED = false>
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
  auto kernel = logits ? wkv7_recurrent_stream_kernel<io_t, state_t, PARTS, true, PREFETCH, FUSED>
                       : wkv7_recurrent_stream_kernel<io_t, state_t, PARTS, false, PREFETCH, FUSED>;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, p);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_stream_kernel: %s", cudaGetErrorString(err));
  return check_launch("wkv7_recurrent_stream_kernel");
}

template <typename io_t, typename state_t = float, bool FUSED = false>
int dispatch_parts(const RecurrentParams& p, bool logits, int parts, bool prefetch, cudaStream_t stream) {
  if (!prefetch) {
    if (parts == 2) return launch<io_t, state_t, 2, false, FUSED>(p, logits, stream);
    if (parts == 4) return launch<io_t, state_t, 4, false, FUSED>(p, logits, stream);
    return launch<io_t, state_t, 8, false, FUSED>(p, logits, stream);
  }
  if (parts == 2) return launch<io_t, state_t, 2, true, FUSED>(p, logits, stream);
  if (parts == 4) return launch<io_t, state_t, 4, true, FUSED>(p, logits, stream);
  return launch<io_t, state_t, 8, true, FUSED>(p, logits, stream);
}

// column split: see launch_recurrent_stream
int choose_parts(int n_seq, int heads, int max_seqlen, int parts_override) {
  int parts = 2;
  const long long pairs = static_cast<long long>(n_seq) * heads;
  if (max_seqlen <= 0 || max_seqlen > 2) parts = 4;
  if (max_seqlen <= 0 || max_seqlen > 64 || pairs < 148LL * 4) parts = 8;
  if (parts_override == 0) parts_override = parts_from_environment();
#ifdef FRWKV_TEST_HOOKS
  if (test_recurrent_parts() != 0) parts_override = test_recurrent_parts();
#endif
  if (parts_override == 2 || parts_override == 4 || parts_override == 8) parts = parts_override;
  return parts;
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
  advance_elapsed_kernel<<<(n_seq + 255) / 256, 256, 0, stream>>>(cu, slots, status, elapsed, n_seq);
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
#endif
