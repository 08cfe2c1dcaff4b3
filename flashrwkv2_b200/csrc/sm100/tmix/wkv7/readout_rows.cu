// The readout's elementwise stage as a kernel of its own, for the rows the chunk kernel produced.
//
// Per (token, head) row of 64 channels (rwkv-rs/FlashRWKV2 csrc/sm120/tmix/readout/infer_fp16_forward_varlen.cu:135-196;
// oracle tests/tmix/readout/test.py:43-66):
//   out = (headnorm(y) * ln_w + ln_b + (sum_c r_c k_c r_k_c) * v) * gate,   eps = 64e-5, two-pass variance.
// The decode / short-row kernel has this as its epilogue (recurrent_readout.cu).  The tensor-core chunk kernel is bound
// by its CUDA-core instruction count, so there the stage stays a second, HBM-bound pass: 768 bytes per row (y, r, k,
// v, gate in, the result out; 896 with the fused producer, whose gated key is recomputed from the raw key and the
// gate logits instead of being stored).  Half a warp owns a row: a lane holds four consecutive channels (8-byte
// accesses), the three reductions are four xor-shuffle steps each, and a warp keeps 1.3 KB of loads in flight.
#include "../../common.cuh"

#include <type_traits>

namespace frwkv {
namespace {

constexpr int kRowsPerCta = 16;  // 8 warps, two rows each
constexpr float kHeadNormEpsilon = 64.0e-5f;

template <typename io_t> struct Four {
  io_t vals[4];
  __device__ __forceinline__ void load(const io_t* p) {
    *reinterpret_cast<uint2*>(vals) = __ldg(reinterpret_cast<const uint2*>(p));
  }
  __device__ __forceinline__ void load_streaming(const io_t* p) {
    *reinterpret_cast<uint2*>(vals) = __ldcs(reinterpret_cast<const uint2*>(p));
  }
  __device__ __forceinline__ float get(int i) const { return to_f32(vals[i]); }
};

__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int m = 8; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}

struct ReadoutRowsParams {
  const void *y, *r, *k, *v, *gate, *r_k, *ln_w, *ln_b;
  const void *a12, *gate_a0, *gate_ka;  // fused producer: k is the raw key; all three null otherwise
  void* out;
  long long rows;  // total_tokens * heads
  int heads;
};

template <typename io_t, bool FUSED>
__global__ void __launch_bounds__(kRowsPerCta * 16) wkv7_readout_rows_kernel(const ReadoutRowsParams p) {
  const long long row = static_cast<long long>(blockIdx.x) * kRowsPerCta + (threadIdx.x >> 4);
  const bool live = row < p.rows;  // a dead half-warp still takes part in its warp's shuffles
  const long long at = (live ? row : 0) * kHeadDim + (threadIdx.x & 15) * 4;
  const int channel = static_cast<int>((live ? row : 0) % p.heads) * kHeadDim + (threadIdx.x & 15) * 4;
  Four<io_t> y, r, k, v, g, rk, lw, lb;
  y.load_streaming(static_cast<const io_t*>(p.y) + at);
  r.load_streaming(static_cast<const io_t*>(p.r) + at);
  k.load_streaming(static_cast<const io_t*>(p.k) + at);
  v.load_streaming(static_cast<const io_t*>(p.v) + at);
  g.load_streaming(static_cast<const io_t*>(p.gate) + at);
  rk.load(static_cast<const io_t*>(p.r_k) + channel);
  lw.load(static_cast<const io_t*>(p.ln_w) + channel);
  lb.load(static_cast<const io_t*>(p.ln_b) + channel);
  float key[4];
  if constexpr (FUSED) {
    // the key the recurrence consumed: k * (1 + (sigmoid(a0 + a12) - 1) * k_a), rounded to the token dtype as the
    // reference's producer stores it
    Four<io_t> a12, a0, ka;
    a12.load_streaming(static_cast<const io_t*>(p.a12) + at);
    a0.load(static_cast<const io_t*>(p.gate_a0) + channel);
    ka.load(static_cast<const io_t*>(p.gate_ka) + channel);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float gate = __fdividef(1.0f, 1.0f + __expf(-(a0.get(c) + a12.get(c))));
      key[c] = to_f32(from_f32<io_t>(k.get(c) * fmaf(gate, ka.get(c), 1.0f - ka.get(c))));
    }
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) key[c] = k.get(c);
  }
  const float mean = half_warp_sum((y.get(0) + y.get(1)) + (y.get(2) + y.get(3))) * (1.0f / kHeadDim);
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float d = y.get(c) - mean;
    ss = fmaf(d, d, ss);
    dot = fmaf(r.get(c) * key[c], rk.get(c), dot);
  }
  ss = half_warp_sum(ss);
  dot = half_warp_sum(dot);
  const float rstd = rsqrtf(ss * (1.0f / kHeadDim) + kHeadNormEpsilon);
  if (!live) return;
  alignas(8) io_t result[4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
    result[c] = from_f32<io_t>(((y.get(c) - mean) * rstd * lw.get(c) + lb.get(c) + dot * v.get(c)) * g.get(c));
  __stcs(reinterpret_cast<uint2*>(static_cast<io_t*>(p.out) + at), *reinterpret_cast<const uint2*>(result));
}

}  // namespace

// gate: {a12, a0, k_a} of the fused producer or nullptr.
int launch_readout_rows(const void* y, const void* r, const void* k, const void* v, const void* out_gate,
                        const void* r_k, const void* ln_w, const void* ln_b, const void* const* gate, void* out,
                        int total_tokens, int heads, int io_dtype, cudaStream_t stream) {
  ReadoutRowsParams p{y, r, k, v, out_gate, r_k, ln_w, ln_b, nullptr, nullptr, nullptr, out,
                      static_cast<long long>(total_tokens) * heads, heads};
  if (gate != nullptr) {
    p.a12 = gate[0];
    p.gate_a0 = gate[1];
    p.gate_ka = gate[2];
  }
  const long long ctas = (p.rows + kRowsPerCta - 1) / kRowsPerCta;
  if (ctas > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "readout rows: too many (token, head) rows");
  const dim3 grid(static_cast<unsigned>(ctas)), block(kRowsPerCta * 16);
  const bool fused = gate != nullptr;
  if (io_dtype == FRWKV_IO_BF16) {
    if (fused) wkv7_readout_rows_kernel<__nv_bfloat16, true><<<grid, block, 0, stream>>>(p);
    else wkv7_readout_rows_kernel<__nv_bfloat16, false><<<grid, block, 0, stream>>>(p);
  } else if (io_dtype == FRWKV_IO_FP16) {
    if (fused) wkv7_readout_rows_kernel<__half, true><<<grid, block, 0, stream>>>(p);
    else wkv7_readout_rows_kernel<__half, false><<<grid, block, 0, stream>>>(p);
  } else {
    return fail(FRWKV_ERR_UNSUPPORTED, "the readout stage takes float16 or bfloat16 tokens");
  }
  return check_launch("wkv7_readout_rows_kernel");
}

}  // namespace frwkv
