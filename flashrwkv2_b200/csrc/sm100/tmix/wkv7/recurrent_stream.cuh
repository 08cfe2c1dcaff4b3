// Kernel and launch templates of the register-streaming WKV7 recurrence, shared by the translation units that
// instantiate them (recurrent_stream.cu: the fp32- and fp16-state contracts and the fused kk/a-gate input form;
// recurrent_readout.cu: the forms with the readout epilogue).  See recurrent_stream.cu for the design.
#pragma once
// Compile-time tuning: sequences per warp of the pipelined one-token launch (the grid is that much deeper than the
// resident CTAs), and whether the plain recurrence takes that launch too (the fused forms always may).
#ifndef FRWKV_PIPELINE_DEPTH
#define FRWKV_PIPELINE_DEPTH 3
#endif
#ifndef FRWKV_PIPELINE_PLAIN
#define FRWKV_PIPELINE_PLAIN 1
#endif
#include "../../common.cuh"

#include <algorithm>
#include <cstdlib>
#include <type_traits>

namespace frwkv {
#ifdef FRWKV_TEST_HOOKS
int& test_recurrent_parts();  // test build only: column split forced by the next launches (0 = none)
int& test_pipeline_min_rounds();  // test build only: threshold of the pipelined one-token launch (0 = default)
#endif
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
  // compact form (fused producer, readout epilogue): the same two rows of a (fused: gate logits a12), b, k (fused:
  // raw key) and r
  Pair<io_t> g2, b2, k2, r2;
  Quad<io_t> v;
  Quad<io_t> g;       // readout epilogue: output gate of this lane's value columns
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
  // readout epilogue (READOUT kernels): per-token output gate [T, H, 64], per-channel [H*64] residual weight r_k and
  // head-norm weight and bias, and the destination of the gated result.  y and y_f32 may then be null.
  const void *ro_gate, *ro_rk, *ro_lnw, *ro_lnb;
  void* ro_out;
};

// Epsilon of the reference's per-head normalisation (csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:25).
constexpr float kHeadNormEps = 64.0e-5f;

// The gate of the reference's producer kernel (csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/
// infer_fp16_forward_varlen.cu:52-106,131-156): sigmoid as 1 / (1 + exp(-x)) with the fast exponential.
__device__ __forceinline__ float gate_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
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
template <typename io_t, typename state_t, int PARTS, bool LOGITS, bool PREFETCH, bool FUSED = false,
          bool READOUT = false, bool PIPELINED = false>
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
    const long long n_out = static_cast<long long>(p.total_tokens) * p.heads * kHeadDim;
    const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    if (!READOUT || p.y != nullptr) fill_output_nan(static_cast<io_t*>(p.y), p.y_f32, n_out, first, stride);
    if constexpr (READOUT) fill_output_nan(static_cast<io_t*>(p.ro_out), nullptr, n_out, first, stride);
    return;
  }
  const int active = min(p.status != nullptr ? p.status[2] : p.n_seq, p.n_seq);
  // Work items.  Plain launch: one (sequence, head, column part) per warp.  PIPELINED launch (one-token steps of
  // large batches): the grid is a whole number of "sequence lanes" of
  // heads * PARTS warps; a warp keeps its head and part and walks the sequences lane by lane, and the state of its
  // next sequence travels to shared memory (cp.async, 16 bytes per lane and row: each lane copies exactly what it
  // reads back) while the current one is computed, so that the warp always has a state in flight.
  static_assert(!PIPELINED || (!PREFETCH && !kHalfState), "pipelined items: one-token steps on the fp32 state");
  int seq, head, part, seq_stride = 0;
  if constexpr (PIPELINED) {
    const int per_seq = p.heads * PARTS;
    seq = static_cast<int>(warp / per_seq);
    const int rem = static_cast<int>(warp % per_seq);
    head = rem / PARTS;
    part = rem % PARTS;
    seq_stride = static_cast<int>(static_cast<long long>(gridDim.x) * kWarpsPerCta / per_seq);
  } else {
    const long long pair = warp / PARTS;
    part = static_cast<int>(warp % PARTS);
    seq = static_cast<int>(pair / p.heads);
    head = static_cast<int>(pair % p.heads);
  }
  if (seq >= active) return;
  const int group = lane / LPR;
  const int col = part * COLS + (lane % LPR) * 4;
  const int row0 = group * RPL;
  float4 S[RPL];

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

  // fused producer: every lane evaluates the gate for the same two key rows whose decay it evaluates (the 32 lanes
  // of the warp cover the 64 rows exactly once), so it needs the per-channel parameters of those two rows only
  Pair<io_t> gate_kk, gate_ka, gate_a0;
  if constexpr (FUSED) {
    gate_kk.load(static_cast<const io_t*>(p.gate_kk) + head * kHeadDim + my_rows);
    gate_ka.load(static_cast<const io_t*>(p.gate_ka) + head * kHeadDim + my_rows);
    gate_a0.load(static_cast<const io_t*>(p.gate_a0) + head * kHeadDim + my_rows);
  }

  // readout epilogue: the warps of a (sequence, head) exchange their y columns through shared memory (two buffers,
  // alternating by token, so that one barrier per token is enough); per-channel parameters of this lane's value
  // columns and of its two residual rows stay in registers
  static_assert(!READOUT || (kWarpsPerCta % PARTS == 0 && sizeof(io_t) == 2 && !kHalfState),
                "readout epilogue: 16-bit tokens, fp32 state, all column parts of a pair in one CTA");
  Quad<io_t> ro_w, ro_b;
  Pair<io_t> ro_rk;
  const int pair_in_cta = (threadIdx.x >> 5) / PARTS;
  if constexpr (READOUT) {
    ro_w.load(static_cast<const io_t*>(p.ro_lnw) + head * kHeadDim + col);
    ro_b.load(static_cast<const io_t*>(p.ro_lnb) + head * kHeadDim + col);
    ro_rk.load(static_cast<const io_t*>(p.ro_rk) + head * kHeadDim + my_rows);
  }

  // Token rows.  The plain kernels keep the RPL rows of r, w, k, a, b that a lane needs in registers (every lane
  // of a row group holds the same copy).  The kernels with the fused producer or the readout epilogue carry more
  // per-token state than the register budget of four CTAs per SM allows, so there a lane keeps only its own two
  // rows of each tensor as one packed word and the row group hands them round: one shuffle per tensor and pair of
  // rows (COMPACT).
  constexpr bool COMPACT = FUSED || READOUT || PIPELINED;
  static_assert(!COMPACT || sizeof(io_t) == 2, "packed pair words need 16-bit tokens");
  auto word_of = [](const Pair<io_t>& x) { return *reinterpret_cast<const uint32_t*>(x.vals); };
  auto half_of = [](uint32_t word, int e) -> float {
    const unsigned short bits = static_cast<unsigned short>(e ? (word >> 16) : (word & 0xffffu));
    if constexpr (std::is_same<io_t, __nv_bfloat16>::value) {
      return __uint_as_float(static_cast<uint32_t>(bits) << 16);
    } else {
      return __half2float(__ushort_as_half(bits));
    }
  };
  auto pack_io = [](float lo, float hi) -> uint32_t {
    alignas(4) io_t two[2] = {from_f32<io_t>(lo), from_f32<io_t>(hi)};
    return *reinterpret_cast<const uint32_t*>(two);
  };

  auto fetch = [&](TokenRows<io_t, RPL>& dst, int t) {
    const size_t row = (static_cast<size_t>(t) * p.heads + head) * kHeadDim;
    if constexpr (READOUT) dst.g.load(static_cast<const io_t*>(p.ro_gate) + row + col);
    if constexpr (COMPACT) {  // this lane's two rows of every tensor (FUSED: raw key, gate logits a12, no b)
      dst.g2.load(ap + row + my_rows);
      dst.w2.load(wp + row + my_rows);
      if constexpr (!FUSED) dst.b2.load(bp + row + my_rows);
      dst.k2.load(kp + row + my_rows);
      dst.r2.load(rp + row + my_rows);
      dst.v.load(vp + row + col);
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
  int phase_base = 0;  // fp16 state: dither phase of this lane's first decay row at token 0 (set per item)
  // Everything of a token that needs no state: the packed row words of the compact form (with the fused producer:
  // the gate), the per-row decay and the readout's residual weight.  In the pipelined launch it runs before the
  // staged state is taken.  (Doing it one item ahead, at the end of the previous item, was measured slower: the
  // values carried across the item boundary cost more registers than the four-CTA budget has.)
  struct Prepared {
    uint32_t word_a, word_b, word_k, word_r, word_w;  // COMPACT: rows my_rows, my_rows + 1 of a, b, k, r, w
    float own_k[2];                                   // the key the recurrence consumes, this lane's two rows
    float mine[2];                                    // rho (fp32 state) or delta (fp16 state) of the same rows
    float dot;                                        // readout: sum_c r_c k_c r_k_c
  };
  auto prepare = [&](const TokenRows<io_t, RPL>& rows, int t) {
    Prepared pr;
    pr.word_a = pr.word_b = pr.word_k = pr.word_r = pr.word_w = 0;
    pr.own_k[0] = pr.own_k[1] = pr.mine[0] = pr.mine[1] = pr.dot = 0.f;
    if constexpr (FUSED) {
      // fused producer, for this lane's two rows: kk = normalize(k * kk_scale) over the 64 channels (a full-warp
      // sum: the lanes hold two rows each), a = -kk, b = kk * g, k' = k * (1 + (g - 1) * k_a), g = sigmoid(a0 + a12);
      // rounded to the token dtype, as the reference's producer stores them
      float u[2], ss = 0.f;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        u[e] = to_f32(rows.k2.vals[e]) * to_f32(gate_kk.vals[e]);
        ss = fmaf(u[e], u[e], ss);
      }
      // each of the 64 rows belongs to exactly one lane of this warp: a sum over all 32 lanes is the whole norm
#pragma unroll
      for (int m = 1; m < 32; m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
      const float inv_norm = rsqrtf(fmaxf(ss, 1.0e-24f));  // = 1 / max(|k * k_k|, 1e-12), two units in the last place
      float own_a[2], own_b[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float g = gate_sigmoid(to_f32(gate_a0.vals[e]) + to_f32(rows.g2.vals[e]));
        const float kk = u[e] * inv_norm, ka = to_f32(gate_ka.vals[e]);
        own_a[e] = -kk;
        own_b[e] = kk * g;
        pr.own_k[e] = round_io<io_t>(to_f32(rows.k2.vals[e]) * fmaf(g, ka, 1.0f - ka));
      }
      pr.word_a = pack_io(own_a[0], own_a[1]);
      pr.word_b = pack_io(own_b[0], own_b[1]);
      pr.word_k = pack_io(pr.own_k[0], pr.own_k[1]);
    } else if constexpr (COMPACT) {
      pr.word_a = word_of(rows.g2);
      pr.word_b = word_of(rows.b2);
      pr.word_k = word_of(rows.k2);
      pr.own_k[0] = to_f32(rows.k2.vals[0]);
      pr.own_k[1] = to_f32(rows.k2.vals[1]);
    }
    if constexpr (COMPACT) {
      pr.word_r = word_of(rows.r2);
      if constexpr (!kSharedDecay) pr.word_w = word_of(rows.w2);
    }
    if constexpr (kSharedDecay) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = to_f32(rows.w2.vals[e]);
        if constexpr (LOGITS) {
          if (has_bias) x += to_f32(bias2.vals[e]);
#if defined(FRWKV_FAST_DECAY)
          x = sizeof(io_t) == 2 ? retention_from_logit_fast(x) : retention_from_logit(x);
#else
          x = retention_from_logit(x);
#endif
        }
        if constexpr (kHalfState) x = round_to_half(x - 1.0f + fp16_state_dither(phase_base + e + t));
        pr.mine[e] = x;
      }
    }
    if constexpr (READOUT) {
      // every key row belongs to exactly one lane: a full-warp sum is the whole dot product
#pragma unroll
      for (int e = 0; e < 2; ++e)
        pr.dot = fmaf(to_f32(rows.r2.vals[e]) * pr.own_k[e], to_f32(ro_rk.vals[e]), pr.dot);
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) pr.dot += __shfl_xor_sync(0xffffffffu, pr.dot, m);
    }
    return pr;
  };
  TokenRows<io_t, RPL> cur, nxt;

  // PIPELINED: staging area of this warp (row i of lane l at [i][l]: conflict-free by construction)
  __shared__ float4 stage[PIPELINED ? kWarpsPerCta * RPL * 32 : 1];
  float4* const my_stage = stage + (PIPELINED ? (threadIdx.x >> 5) * RPL * 32 + lane : 0);
  auto state_of = [&](int slot_of_item) {
    return static_cast<state_t*>(p.pool) + (static_cast<size_t>(slot_of_item) * p.heads + head) * (kHeadDim * kHeadDim) +
           static_cast<size_t>(row0) * kHeadDim + col;
  };
  auto issue_state_copy = [&](int slot_of_item) {
    const state_t* src = state_of(slot_of_item);
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(my_stage));
#pragma unroll
    for (int i = 0; i < RPL; ++i)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 32 * 16), "l"(src + i * kHeadDim)
                   : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int t_lo_next = 0, t_hi_next = 0, slot_next = 0;
  if constexpr (PIPELINED) {
    t_lo_next = p.cu[seq];
    t_hi_next = p.cu[seq + 1];
    slot_next = p.slots[seq];
    issue_state_copy(slot_next);
    if (t_lo_next < t_hi_next) fetch(nxt, t_lo_next);
  }
  unsigned tokens_done = 0;  // readout epilogue: selects the exchange buffer (the warps of a pair count alike)

  for (;;) {  // items of this warp (a plain launch has exactly one)
  int t_lo, t_hi, slot;
  if constexpr (PIPELINED) {
    t_lo = t_lo_next;
    t_hi = t_hi_next;
    slot = slot_next;
  } else {
    t_lo = p.cu[seq];
    t_hi = p.cu[seq + 1];
    if (p.len_below > 0 && t_hi - t_lo >= p.len_below) return;
    slot = p.slots[seq];
  }
  state_t* const sbase = state_of(slot);
  // the item after this one: its metadata is requested now and used after the first reduction below
  const int seq_after = seq + seq_stride;
  const bool more = PIPELINED && seq_after < active;
  if (more) {
    t_lo_next = p.cu[seq_after];
    t_hi_next = p.cu[seq_after + 1];
    slot_next = p.slots[seq_after];
  }
  bool next_issued = false;
  // PIPELINED: the staged state is taken into registers as late as possible (after the token-only work of the
  // first token), because the staging area is refilled right after its first use
  bool state_ready = !PIPELINED;
  auto take_staged_state = [&]() {
    asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
    for (int i = 0; i < RPL; ++i) S[i] = my_stage[i * 32];
    state_ready = true;
  };
  if constexpr (!PIPELINED) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) S[i] = load_state4<state_t>(sbase + i * kHeadDim);
  }
  if constexpr (kHalfState) phase_base = p.elapsed[slot] + head * kHeadDim + my_rows - t_lo;
  if (PREFETCH && t_lo < t_hi) fetch(nxt, t_lo);

  for (int t = t_lo; t < t_hi; ++t) {
    if constexpr (PREFETCH) {
      cur = nxt;
      if (t + 1 < t_hi) fetch(nxt, t + 1);  // next token's rows are in flight during the math
    } else if constexpr (PIPELINED) {
      if (t == t_lo) {
        cur = nxt;  // requested while the previous item was computed
      } else {
        fetch(cur, t);
      }
    } else {
      fetch(cur, t);
    }
    const Prepared pr = prepare(cur, t);
    if constexpr (PIPELINED) {
      if (!state_ready) take_staged_state();
    }
    float4 sa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < RPL / 2; ++j) {
      float fa[2];
      if constexpr (COMPACT) {
        const uint32_t x = __shfl_sync(0xffffffffu, pr.word_a, group * LPR + j);
        fa[0] = half_of(x, 0);
        fa[1] = half_of(x, 1);
      } else {
        fa[0] = cur.a.get(2 * j);
        fa[1] = cur.a.get(2 * j + 1);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = 2 * j + e;
        sa.x = fmaf(fa[e], S[i].x, sa.x);
        sa.y = fmaf(fa[e], S[i].y, sa.y);
        sa.z = fmaf(fa[e], S[i].z, sa.z);
        sa.w = fmaf(fa[e], S[i].w, sa.w);
      }
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1) {
      sa.x += __shfl_xor_sync(0xffffffffu, sa.x, m);
      sa.y += __shfl_xor_sync(0xffffffffu, sa.y, m);
      sa.z += __shfl_xor_sync(0xffffffffu, sa.z, m);
      sa.w += __shfl_xor_sync(0xffffffffu, sa.w, m);
    }
    if constexpr (PIPELINED) {
      // every staged value has been consumed by the reduction above, so the staging area is free: the next item's
      // state and token rows start their way now and arrive under the rest of this item
      if (!next_issued && more) {
        issue_state_copy(slot_next);
        if (t_lo_next < t_hi_next) fetch(nxt, t_lo_next);
      }
      next_issued = true;
    }
    const float4 v4 = make_float4(to_f32(cur.v.vals[0]), to_f32(cur.v.vals[1]), to_f32(cur.v.vals[2]),
                                  to_f32(cur.v.vals[3]));
    const float dot = pr.dot;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < RPL / 2; ++j) {
      const int src = group * LPR + j;  // the lane of this row group that owns rows 2j and 2j + 1
      float fw[2], fb[2], fk[2], fr[2];
      if constexpr (kSharedDecay) {
        fw[0] = __shfl_sync(0xffffffffu, pr.mine[0], src);
        fw[1] = __shfl_sync(0xffffffffu, pr.mine[1], src);
      } else if constexpr (COMPACT) {
        const uint32_t x = __shfl_sync(0xffffffffu, pr.word_w, src);
        fw[0] = half_of(x, 0);
        fw[1] = half_of(x, 1);
      } else {
        fw[0] = cur.w.get(2 * j);
        fw[1] = cur.w.get(2 * j + 1);
      }
      if constexpr (COMPACT) {
        const uint32_t xb = __shfl_sync(0xffffffffu, pr.word_b, src);
        const uint32_t xk = __shfl_sync(0xffffffffu, pr.word_k, src);
        const uint32_t xr = __shfl_sync(0xffffffffu, pr.word_r, src);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          fb[e] = half_of(xb, e);
          fk[e] = half_of(xk, e);
          fr[e] = half_of(xr, e);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          fb[e] = cur.b.get(2 * j + e);
          fk[e] = cur.k.get(2 * j + e);
          fr[e] = cur.r.get(2 * j + e);
        }
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = 2 * j + e;
        if constexpr (kHalfState) {
          // S + S*delta + b*sa + k*v in fp32, then rounded to the stored precision; y reads the rounded state
          const float delta = fw[e];
          S[i].x = round_to_half(fmaf(fk[e], v4.x, fmaf(fb[e], sa.x, fmaf(S[i].x, delta, S[i].x))));
          S[i].y = round_to_half(fmaf(fk[e], v4.y, fmaf(fb[e], sa.y, fmaf(S[i].y, delta, S[i].y))));
          S[i].z = round_to_half(fmaf(fk[e], v4.z, fmaf(fb[e], sa.z, fmaf(S[i].z, delta, S[i].z))));
          S[i].w = round_to_half(fmaf(fk[e], v4.w, fmaf(fb[e], sa.w, fmaf(S[i].w, delta, S[i].w))));
        } else {
          S[i].x = fmaf(fw[e], S[i].x, fmaf(fb[e], sa.x, fk[e] * v4.x));
          S[i].y = fmaf(fw[e], S[i].y, fmaf(fb[e], sa.y, fk[e] * v4.y));
          S[i].z = fmaf(fw[e], S[i].z, fmaf(fb[e], sa.z, fk[e] * v4.z));
          S[i].w = fmaf(fw[e], S[i].w, fmaf(fb[e], sa.w, fk[e] * v4.w));
        }
        acc.x = fmaf(fr[e], S[i].x, acc.x);
        acc.y = fmaf(fr[e], S[i].y, acc.y);
        acc.z = fmaf(fr[e], S[i].z, acc.z);
        acc.w = fmaf(fr[e], S[i].w, acc.w);
      }
    }
#pragma unroll
    for (int m = LPR; m < 32; m <<= 1) {
      acc.x += __shfl_xor_sync(0xffffffffu, acc.x, m);
      acc.y += __shfl_xor_sync(0xffffffffu, acc.y, m);
      acc.z += __shfl_xor_sync(0xffffffffu, acc.z, m);
      acc.w += __shfl_xor_sync(0xffffffffu, acc.w, m);
    }
    const size_t out = (static_cast<size_t>(t) * p.heads + head) * kHeadDim + col;
    acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
    Quad<io_t> q;
    q.vals[0] = from_f32<io_t>(acc.x);
    q.vals[1] = from_f32<io_t>(acc.y);
    q.vals[2] = from_f32<io_t>(acc.z);
    q.vals[3] = from_f32<io_t>(acc.w);
    if (group == 0 && (!READOUT || p.y != nullptr)) q.store(yp + out);
    if (group == 0 && p.y_f32 != nullptr) *reinterpret_cast<float4*>(p.y_f32 + out) = acc;
    if constexpr (READOUT) {
      // Consumer of y (csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:135-196 of the reference; oracle
      // tests/tmix/readout/test.py:43-66): per-head normalisation of the rounded y, residual (sum_c r k r_k) v,
      // output gate.  The epilogue is a latency chain at the end of a warp that otherwise only waits for HBM, so it
      // is kept short: the state goes out first, each warp reduces its own columns to (mean, sum of squared
      // deviations) with log2(LPR) shuffle steps, and the warps of the pair exchange just those two numbers through
      // shared memory (two buffers alternating by token: one named barrier per token) and merge them in part order,
      // so that every warp of the pair holds bit-identical statistics.
      if (t + 1 == t_hi) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) store_state4(sbase + i * kHeadDim, S[i]);
      }
      __shared__ float2 stats_exchange[2 * kWarpsPerCta];
      const float y4[4] = {to_f32(q.vals[0]), to_f32(q.vals[1]), to_f32(q.vals[2]), to_f32(q.vals[3])};
      float mean = 0.25f * ((y4[0] + y4[1]) + (y4[2] + y4[3]));
      float m2 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) m2 = fmaf(y4[c] - mean, y4[c] - mean, m2);
      float count = 4.f;
#pragma unroll
      for (int m = 1; m < LPR; m <<= 1) {  // equal-sized halves: mean of means, M2 += delta^2 * n / 2
        const float other_mean = __shfl_xor_sync(0xffffffffu, mean, m);
        const float other_m2 = __shfl_xor_sync(0xffffffffu, m2, m);
        const float delta = other_mean - mean;
        mean = 0.5f * (mean + other_mean);
        m2 = (m2 + other_m2) + delta * delta * (0.5f * count);
        count *= 2.f;
      }
      float2* ex = stats_exchange + (tokens_done++ & 1u) * kWarpsPerCta + pair_in_cta * PARTS;
      if (lane == 0) ex[part] = make_float2(mean, m2);
      asm volatile("bar.sync %0, %1;" ::"r"(1 + pair_in_cta), "r"(PARTS * 32) : "memory");
      mean = ex[0].x;
      m2 = ex[0].y;
#pragma unroll
      for (int q2 = 1; q2 < PARTS; ++q2) {  // part q2 (COLS values) joins the first q2 parts
        const float2 other = ex[q2];
        const float delta = other.x - mean;
        mean = fmaf(delta, 1.0f / (q2 + 1), mean);
        m2 = (m2 + other.y) + delta * delta * (static_cast<float>(COLS) * q2 / (q2 + 1));
      }
      const float rstd = rsqrtf(m2 * (1.0f / kHeadDim) + kHeadNormEps);
      if (group == 0) {
        const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
        Quad<io_t> o;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          o.vals[c] = from_f32<io_t>(((y4[c] - mean) * rstd * to_f32(ro_w.vals[c]) + to_f32(ro_b.vals[c]) +
                                      dot * vv[c]) * to_f32(cur.g.vals[c]));
        o.store(static_cast<io_t*>(p.ro_out) + out);
      }
    }
  }
  if constexpr (PIPELINED) {
    if (!state_ready) take_staged_state();  // a row without tokens
  }
  if (!(READOUT && t_lo < t_hi)) {  // with the readout epilogue the state went out before the last token's epilogue
#pragma unroll
    for (int i = 0; i < RPL; ++i) store_state4(sbase + i * kHeadDim, S[i]);
  }
  if constexpr (PIPELINED) {
    if (!more) break;
    if (!next_issued) {  // a row without tokens: the state registers have just been consumed by the stores
      issue_state_copy(slot_next);
      if (t_lo_next < t_hi_next) fetch(nxt, t_lo_next);
    }
    seq = seq_after;
  } else {
    break;
  }
  }  // items
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
// FRWKV_PIPELINE_MIN_ROUNDS: the pipelined one-token launch is taken from this many sequences per resident warp
// upwards (a large value turns it off).  Defaults, measured at H = 64 on 148 SMs: the plain recurrence gains from
// 1024 sequences (57 rounds: 352 -> 334 us; 2048: 683 -> 657 us) and loses below (512: 169 -> 171 us, 256: 84 -> 89 us),
// so it switches at 40; the kernels with the fused producer or the readout epilogue have more to hide and switch at 8.
inline int pipeline_min_rounds(bool more_than_the_recurrence) {
  static const int forced = [] {
    const char* e = std::getenv("FRWKV_PIPELINE_MIN_ROUNDS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced > 0) return forced;
#ifdef FRWKV_TEST_HOOKS
  if (test_pipeline_min_rounds() > 0) return test_pipeline_min_rounds();
#endif
  return more_than_the_recurrence ? 8 : 40;
}
inline int parts_from_environment() {
  static const int parts = [] {
    const char* e = std::getenv("FRWKV_RECURRENT_PARTS");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  return parts;
}

template <typename io_t, typename state_t, int PARTS, bool PREFETCH, bool FUSED = false, bool READOUT = false>
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
  auto kernel = logits ? wkv7_recurrent_stream_kernel<io_t, state_t, PARTS, true, PREFETCH, FUSED, READOUT>
                       : wkv7_recurrent_stream_kernel<io_t, state_t, PARTS, false, PREFETCH, FUSED, READOUT>;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, p);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_stream_kernel: %s", cudaGetErrorString(err));
  return check_launch("wkv7_recurrent_stream_kernel");
}

// Pipelined one-token launch (two column parts per pair) of the kernels with the fused producer and / or the readout
// epilogue: a persistent grid of whole sequence lanes, four CTAs per SM.  Returns -1 when the batch does not give
// every warp at least two sequences (the plain launch is then the same thing) or no whole lane fits.
inline int resident_warp_slots() {
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cached[device] = sms * 4 * kWarpsPerCta;
  }
  return cached[device];
}
template <typename io_t, bool FUSED, bool READOUT>
int launch_pipelined(const RecurrentParams& p, bool logits, cudaStream_t stream) {
  constexpr int PARTS = 2;
  const long long per_seq = static_cast<long long>(p.heads) * PARTS;
  long long lanes = resident_warp_slots() / per_seq;
  while (lanes > 0 && (lanes * per_seq) % kWarpsPerCta != 0) --lanes;
  if (lanes < 1 || p.n_seq < pipeline_min_rounds(FUSED || READOUT) * lanes || p.len_below > 0) return -1;
  // Several resident grids' worth of CTAs, about a dozen sequences per warp: a grid of exactly the resident CTAs
  // would fix every SM's share in advance, and SMs do not run equally fast (measured: the slowest SM needed 14 %
  // more cycles than the average); with more CTAs than slots the hardware scheduler evens that out.
  lanes *= std::max<long long>(1, p.n_seq / (lanes * FRWKV_PIPELINE_DEPTH));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(lanes * per_seq / kWarpsPerCta));
  config.blockDim = dim3(kWarpsPerCta * 32);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  auto kernel = logits ? wkv7_recurrent_stream_kernel<io_t, float, PARTS, true, false, FUSED, READOUT, true>
                       : wkv7_recurrent_stream_kernel<io_t, float, PARTS, false, false, FUSED, READOUT, true>;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, p);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_stream_kernel: %s", cudaGetErrorString(err));
  return check_launch("wkv7_recurrent_stream_kernel");
}

template <typename io_t, typename state_t = float, bool FUSED = false>
int dispatch_parts(const RecurrentParams& p, bool logits, int parts, bool prefetch, cudaStream_t stream) {
  if (!prefetch) {
    if constexpr (sizeof(io_t) == 2 && std::is_same<state_t, float>::value) {
      if (parts == 2 && FRWKV_PIPELINE_PLAIN + FUSED > 0) {
        const int rc = launch_pipelined<io_t, FUSED, false>(p, logits, stream);
        if (rc >= 0) return rc;
      }
    }
    if (parts == 2) return launch<io_t, state_t, 2, false, FUSED>(p, logits, stream);
    if (parts == 4) return launch<io_t, state_t, 4, false, FUSED>(p, logits, stream);
    return launch<io_t, state_t, 8, false, FUSED>(p, logits, stream);
  }
  if (parts == 2) return launch<io_t, state_t, 2, true, FUSED>(p, logits, stream);
  if (parts == 4) return launch<io_t, state_t, 4, true, FUSED>(p, logits, stream);
  return launch<io_t, state_t, 8, true, FUSED>(p, logits, stream);
}

// column split: see launch_recurrent_stream
inline int choose_parts(int n_seq, int heads, int max_seqlen, int parts_override) {
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

}  // namespace frwkv
