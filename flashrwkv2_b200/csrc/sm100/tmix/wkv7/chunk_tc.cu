// WKV7 chunked prefill on tcgen05 tensor cores (sm_100a): 64-row chunks, WY/UT transform,
// fp32 state carried in TMEM.
//
// One CTA (256 threads) walks one (sequence, head) chunk by chunk.  Per chunk of L <= 64 rows,
// with g_t = prod_{s<=t} rho_s (per key channel; g_{t-1} is the exclusive product):
//     At = a * g_{t-1}   Bt = b / g_t   Kt = k / g_t   Rt = r * g_t                    [L, K]
//     P  = [At; Rt] [Bt; Kt]^T  -> A_ab, A_ak (strictly lower), A_rb, A_rk (lower)      [2L, 2L]
//     Q  = [At; Rt] S0 + [A_ak; A_rk] V     (rows 0..63 = W, rows 64..127 = part of Y)
//     U  = (I - A_ab)^-1 W                  (U[t] = a_t^T S_{t-1})
//     Y  = scale * (Q[64..] + A_rb U)
//     S  = diag(g_L) (S0 + Bt^T U + Kt^T V)
// which is the token recurrence of rwkv-rs/FlashRWKV2 tests/tmix/wkv7/test.py:66-83 regrouped;
// the reference computes the same quantities on CUDA cores in
// csrc/sm120/tmix/wkv7/rl_infctx_chunk_fp32io16_forward.cu:318-539.
//
// Precision: every dense contraction is a tcgen05.mma kind::f16 on bf16 operands with fp32
// accumulation in TMEM.  A single bf16 rounding of the decay-scaled operands is not accurate
// enough, so each fp32 operand x is split into hi = bf16(x), lo = bf16(x - hi) and a product
// is issued as hi*hi + hi*lo + lo*hi (about 16 significant bits); V is exact in bf16 and
// needs no lo part.  The triangular inverse is computed in fp32 on CUDA cores (16x16
// diagonal blocks by substitution, merged to 32x32 and then 64x64 by block products).
//
// Data movement: the six token tiles of a chunk arrive by TMA (cp.async.bulk.tensor.3d over
// the [64, H, T] view of each tensor) into one staging area; operands are written into
// un-swizzled core-matrix tiles (see tcgen05.cuh) so that the same tile can be read K-major
// or MN-major; accumulators P (128 columns), Q, U and the state S (64 columns each) live in
// TMEM.  Rows past the end of a sequence are masked to rho = 1, r = k = a = b = 0.
// Every wait on an mbarrier is bounded; on a timeout the CTA raises *error_flag, waits
// (bounded) for its TMA load, frees its TMEM and returns.
#include "chunk_common.cuh"

namespace frwkv {
namespace {

using namespace tc;
using namespace chunk;

constexpr int kThreads = 256;
constexpr int kChunk = 64;

// ---- shared-memory map (bytes) -------------------------------------------------------------
// K-major 128-row tiles (also read MN-major with the strides swapped)
constexpr uint32_t kChunkStride128 = 16 * 128 + 16;  // stride between 16-byte k-chunks, 128-row tile (padded)
constexpr uint32_t kTile128 = 8 * kChunkStride128;   // 16512: one bf16 part (hi or lo)
// MN-major 64-row operand tiles (rows = contraction index, 64 contiguous columns)
constexpr uint32_t kChunkStride64 = 8 * 128 + 16;    // stride between 16-byte column chunks
constexpr uint32_t kTile64 = 8 * kChunkStride64;     // 8320

constexpr uint32_t kRawTile = 64 * 128;              // one [64][64] 16-bit tile as TMA writes it
constexpr uint32_t kOffRaw = 0;                      // r, w, k, v, a, b
constexpr uint32_t kOffX1 = kOffRaw + 6 * kRawTile;  // [At; Rt] hi, lo  -> later [T; A_rb]
constexpr uint32_t kOffX2 = kOffX1 + 2 * kTile128;   // [Bt; Kt] hi, lo
constexpr uint32_t kOffX3 = kOffX2 + 2 * kTile128;   // [A_ak; A_rk] hi, lo
constexpr uint32_t kOffOp = kOffX3 + 2 * kTile128;   // S0 / W / U operand hi, lo
constexpr uint32_t kOffV = kOffOp + 2 * kTile64;     // V operand hi, lo
constexpr uint32_t kOffMisc = kOffV + 2 * kTile64;   // gamma_L[64], partial sums[8][64], barriers
constexpr uint32_t kMiscBytes = 64 * 4 + 8 * 64 * 4 + 64;
constexpr uint32_t kSmemBytes = kOffMisc + kMiscBytes + 128;  // + alignment slack
// fp32 scratch of the triangular inverse, aliased onto the TMA staging area (free after stage A)
constexpr int kInvLd = 68;                                      // padded row length (floats)
constexpr uint32_t kOffAb = kOffRaw;                            // A_ab   [64][68]
constexpr uint32_t kOffTi = kOffAb + 64 * kInvLd * 4;           // T      [64][68]
constexpr int kMbLd = 34;                                       // padded row length of the product scratch
constexpr uint32_t kOffMb = kOffTi + 64 * kInvLd * 4;           // intermediate block product [32][34]
static_assert(kOffMb + 32 * kMbLd * 4 <= kOffX1, "inverse scratch must fit in the staging area");

// ---- TMEM map (columns) --------------------------------------------------------------------
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColP = 0, kColQ = 128, kColU = 192, kColS = 256;

template <typename io_t, bool LOGITS>
__global__ void __launch_bounds__(kThreads, 1)
wkv7_chunk_tc_kernel(const ChunkParams p, const __grid_constant__ Maps maps) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte aligned base (TMA destination and descriptor addresses)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3;   // TMEM lane quadrant this warp may access
  const int half = warp >> 2;  // which half of the columns this warp handles

  if (p.status != nullptr && p.status[0] != 0) {
    if constexpr (std::is_same<io_t, __nv_bfloat16>::value || std::is_same<io_t, __half>::value) {
      fill_output_nan(static_cast<io_t*>(p.y), p.y_f32, static_cast<long long>(p.total_tokens) * p.heads * kHeadDim,
                      static_cast<long long>(blockIdx.x) * kThreads + tid, static_cast<long long>(gridDim.x) * kThreads);
    }
    return;
  }
  const int active = p.status != nullptr ? p.status[2] : p.n_seq;
  const int rank = blockIdx.x / p.heads, head = blockIdx.x % p.heads;
  if (rank >= p.n_seq) return;
  const int seq = p.order != nullptr ? p.order[rank] : rank;
  if (seq >= active || seq < 0 || seq >= p.n_seq) return;
  const int t_begin = p.cu[seq], len = p.cu[seq + 1] - t_begin;
  if (len <= 0 || len < p.len_from) return;
  const int n_chunks = (len + kChunk - 1) / kChunk;
  const int slot = p.slots[seq];

  float* gamma_l = reinterpret_cast<float*>(smem + kOffMisc);
  float* part = gamma_l + 64;                       // [8][64] log2-decay sums of each 8-row group
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(part + 8 * 64);
  uint64_t* bar_mma = bar_tma + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mma + 1);
  const uint32_t sbase = smem_u32(smem);

  if (tid == 0) {
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
    tma_prefetch_descriptor(&maps.r);
    tma_prefetch_descriptor(&maps.w);
    tma_prefetch_descriptor(&maps.k);
    tma_prefetch_descriptor(&maps.v);
    tma_prefetch_descriptor(&maps.a);
    tma_prefetch_descriptor(&maps.b);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_lane = tmem + (static_cast<uint32_t>(quad * 32) << 16);

  auto issue_tma = [&](int chunk) {  // thread 0 only
    const int row = t_begin + chunk * kChunk;
    mbar_expect_tx(bar_tma, 6 * kRawTile);
    tma_load_3d(smem + kOffRaw + 0 * kRawTile, &maps.r, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 1 * kRawTile, &maps.w, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 2 * kRawTile, &maps.k, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 3 * kRawTile, &maps.v, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 4 * kRawTile, &maps.a, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 5 * kRawTile, &maps.b, bar_tma, 0, head, row);
  };
  if (tid == 0) issue_tma(0);
  bool tma_in_flight = true;
  uint32_t tma_parity = 0;  // parity of the load in flight

  // ---- initial state: global -> TMEM (fp32) and -> S0 operand tile (hi/lo, MN-major) ----------
  float* state_g = p.pool + (static_cast<size_t>(slot) * p.heads + head) * (kHeadDim * kHeadDim);
  if (quad < 2) {
    const int krow = quad * 32 + lane;
    uint32_t regs[32];
    const float4* src = reinterpret_cast<const float4*>(state_g + krow * kHeadDim + half * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 f = __ldcs(src + i);
      regs[4 * i] = __float_as_uint(f.x);
      regs[4 * i + 1] = __float_as_uint(f.y);
      regs[4 * i + 2] = __float_as_uint(f.z);
      regs[4 * i + 3] = __float_as_uint(f.w);
    }
    tmem_st32(tmem_lane + kColS + half * 32, regs);
    uint8_t* op = smem + kOffOp + (krow & 7) * 16 + (krow >> 3) * kRowGroup;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 hi, lo;
      split8(reinterpret_cast<const float*>(regs) + 8 * j, hi, lo);
      *reinterpret_cast<uint4*>(op + (half * 4 + j) * kChunkStride64) = hi;
      *reinterpret_cast<uint4*>(op + kTile64 + (half * 4 + j) * kChunkStride64) = lo;
    }
    tmem_st_wait();
  }

  constexpr uint32_t idesc_kk128 = instr_desc_f16(128, 128, kMajorK, kMajorK);
  constexpr uint32_t idesc_kmn64 = instr_desc_f16(128, 64, kMajorK, kMajorMN);
  constexpr uint32_t idesc_mnmn64 = instr_desc_f16(128, 64, kMajorMN, kMajorMN);
  constexpr bool kVExact = std::is_same<io_t, __nv_bfloat16>::value;
  constexpr uint32_t v_lo_off = kVExact ? 0u : kTile64;

  // operand descriptors (fixed for the whole kernel)
  const Operand op_x1 = make_operand(sbase + kOffX1, kTile128, 2 * kChunkStride128, kChunkStride128, kRowGroup);
  const Operand op_x2 = make_operand(sbase + kOffX2, kTile128, 2 * kChunkStride128, kChunkStride128, kRowGroup);
  const Operand op_x3 = make_operand(sbase + kOffX3, kTile128, 2 * kChunkStride128, kChunkStride128, kRowGroup);
  const Operand op_rows = make_operand(sbase + kOffOp, kTile64, 2 * kRowGroup, kRowGroup, kChunkStride64);
  const Operand op_v = make_operand(sbase + kOffV, v_lo_off, 2 * kRowGroup, kRowGroup, kChunkStride64);
  // [Bt; Kt] read MN-major: M = key channel (16-byte chunks at kChunkStride128), contraction = tile row
  const Operand op_bt = make_operand(sbase + kOffX2, kTile128, 2 * kRowGroup, kRowGroup, kChunkStride128);
  const Operand op_kt = make_operand(sbase + kOffX2 + 8 * kRowGroup, kTile128, 2 * kRowGroup, kRowGroup,
                                     kChunkStride128);

  uint32_t mma_uses = 0;
  bool failed = false;
#ifdef FRWKV_CHUNK_TIMING
  long long phase_t0 = clock64();
#endif
  const io_t* bias_g = LOGITS && p.bias != nullptr ? static_cast<const io_t*>(p.bias) + head * kHeadDim : nullptr;

  for (int c = 0; c < n_chunks; ++c) {
    const int rows = min(kChunk, len - c * kChunk);
    const int row0 = t_begin + c * kChunk;

    // ================= stage A: decay products and scaled operands =================
    {
      const bool ok = mbar_wait(bar_tma, tma_parity);
      if (__syncthreads_or(!ok)) { failed = true; break; }
      tma_in_flight = false;
      tma_parity ^= 1u;
    }
    FRWKV_PHASE(0)
    {
      const int kp = lane;       // key channels 2*kp, 2*kp+1
      const int tg = warp;       // rows 8*tg .. 8*tg+7
      const uint32_t* raw_r = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 0 * kRawTile);
      const uint32_t* raw_w = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 1 * kRawTile);
      const uint32_t* raw_k = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 2 * kRawTile);
      const uint32_t* raw_a = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 4 * kRawTile);
      const uint32_t* raw_b = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 5 * kRawTile);
      float2 bias2 = make_float2(0.f, 0.f);
      if (bias_g != nullptr) bias2 = make_float2(to_f32(bias_g[2 * kp]), to_f32(bias_g[2 * kp + 1]));
      float2 lw[8];   // log2(rho) per row
      float2 run = make_float2(0.f, 0.f);
      float2 cum[8];  // inclusive sums within this 8-row group
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = tg * 8 + i;
        const float2 w2 = unpack2<io_t>(raw_w[t * 32 + kp]);
        float2 l;
        if constexpr (LOGITS) {
          l.x = __fdividef(-kRateLog2e, 1.0f + fast_exp2(-kLog2e * (w2.x + bias2.x)));
          l.y = __fdividef(-kRateLog2e, 1.0f + fast_exp2(-kLog2e * (w2.y + bias2.y)));
        } else {
          l.x = fast_log2(w2.x);
          l.y = fast_log2(w2.y);
        }
        if (t >= rows) l = make_float2(0.f, 0.f);
        lw[i] = l;
        run.x += l.x;
        run.y += l.y;
        cum[i] = run;
      }
      reinterpret_cast<float2*>(part + tg * 64)[kp] = run;
      __syncthreads();
      float2 off = make_float2(0.f, 0.f);
      for (int g = 0; g < tg; ++g) {
        const float2 s = reinterpret_cast<const float2*>(part + g * 64)[kp];
        off.x += s.x;
        off.y += s.y;
      }
      float2 g_prev = make_float2(fast_exp2(off.x), fast_exp2(off.y));
      uint8_t* x1 = smem + kOffX1 + (kp >> 2) * kChunkStride128 + (kp & 3) * 4;
      uint8_t* x2 = smem + kOffX2 + (kp >> 2) * kChunkStride128 + (kp & 3) * 4;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = tg * 8 + i;
        const bool live = t < rows;
        const float2 lg = make_float2(off.x + cum[i].x, off.y + cum[i].y);
        const float2 g = make_float2(fast_exp2(lg.x), fast_exp2(lg.y));
        const float2 gi = make_float2(fast_exp2(-lg.x), fast_exp2(-lg.y));
        const float2 gx = g_prev;  // exclusive product = inclusive product of the previous row
        g_prev = g;
        float2 r2 = unpack2<io_t>(raw_r[t * 32 + kp]);
        float2 k2 = unpack2<io_t>(raw_k[t * 32 + kp]);
        float2 a2 = unpack2<io_t>(raw_a[t * 32 + kp]);
        float2 b2 = unpack2<io_t>(raw_b[t * 32 + kp]);
        if (!live) {
          r2 = k2 = a2 = b2 = make_float2(0.f, 0.f);
        }
        const float at[2] = {a2.x * gx.x, a2.y * gx.y};
        const float rt[2] = {r2.x * g.x, r2.y * g.y};
        const float bt[2] = {b2.x * gi.x, b2.y * gi.y};
        const float kt[2] = {k2.x * gi.x, k2.y * gi.y};
        const uint32_t row_off = (t >> 3) * kRowGroup + (t & 7) * 16;          // rows 0..63
        const uint32_t row_off_hi = ((t + 64) >> 3) * kRowGroup + (t & 7) * 16;  // rows 64..127
        uint32_t h;
        h = pack_bf16x2(at[0], at[1]);
        *reinterpret_cast<uint32_t*>(x1 + row_off) = h;
        *reinterpret_cast<uint32_t*>(x1 + kTile128 + row_off) = pack_bf16x2(at[0] - bf16_lo_as_f32(h), at[1] - bf16_hi_as_f32(h));
        h = pack_bf16x2(rt[0], rt[1]);
        *reinterpret_cast<uint32_t*>(x1 + row_off_hi) = h;
        *reinterpret_cast<uint32_t*>(x1 + kTile128 + row_off_hi) = pack_bf16x2(rt[0] - bf16_lo_as_f32(h), rt[1] - bf16_hi_as_f32(h));
        h = pack_bf16x2(bt[0], bt[1]);
        *reinterpret_cast<uint32_t*>(x2 + row_off) = h;
        *reinterpret_cast<uint32_t*>(x2 + kTile128 + row_off) = pack_bf16x2(bt[0] - bf16_lo_as_f32(h), bt[1] - bf16_hi_as_f32(h));
        h = pack_bf16x2(kt[0], kt[1]);
        *reinterpret_cast<uint32_t*>(x2 + row_off_hi) = h;
        *reinterpret_cast<uint32_t*>(x2 + kTile128 + row_off_hi) = pack_bf16x2(kt[0] - bf16_lo_as_f32(h), kt[1] - bf16_hi_as_f32(h));
        if (t == kChunk - 1) reinterpret_cast<float2*>(gamma_l)[kp] = g;
      }
      // V operand: rows = token, 64 contiguous value columns (MN-major); bf16 is copied, fp16 is split
      const uint8_t* raw_v = smem + kOffRaw + 3 * kRawTile;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int id = tid + j * kThreads;  // 512 chunks of 8 values
        const int s = id >> 3, vc = id & 7;
        uint4 q = *reinterpret_cast<const uint4*>(raw_v + s * 128 + vc * 16);
        uint8_t* dst = smem + kOffV + vc * kChunkStride64 + (s & 7) * 16 + (s >> 3) * kRowGroup;
        if (s >= rows) q = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (kVExact) {
          *reinterpret_cast<uint4*>(dst) = q;
        } else {
          float x[8];
          const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2<io_t>(words[e]);
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
          }
          uint4 hi, lo;
          split8(x, hi, lo);
          *reinterpret_cast<uint4*>(dst) = hi;
          *reinterpret_cast<uint4*>(dst + kTile64) = lo;
        }
      }
    }
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();

    FRWKV_PHASE(1)
    // ================= P = X1 X2^T ; Q = X1 S0 =================
    if (tid == 0) {
      tcgen05_fence_after_sync();
      issue_gemm<true, true>(tmem + kColP, op_x1, op_x2, idesc_kk128, false);
      issue_gemm<true, true>(tmem + kColQ, op_x1, op_rows, idesc_kmn64, false);
      mma_commit(bar_mma);
    }
    {
      const bool ok = mbar_wait(bar_mma, mma_uses & 1);
      ++mma_uses;
      if (__syncthreads_or(!ok)) { failed = true; break; }
      tcgen05_fence_after_sync();
    }

    FRWKV_PHASE(2)
    // ================= read P: masks, A_ab -> fp32 scratch, others -> operand tiles =================
    {
      const int t = (quad & 1) * 32 + lane;  // chunk row of this thread
      float vals[64];
      {
        uint32_t regs[32];
        tmem_ld32(tmem_lane + kColP + half * 64, regs);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) vals[i] = __uint_as_float(regs[i]);
        tmem_ld32(tmem_lane + kColP + half * 64 + 32, regs);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) vals[32 + i] = __uint_as_float(regs[i]);
      }
      const int limit = quad < 2 ? t : t + 1;  // keep columns s < limit
#pragma unroll
      for (int s = 0; s < 64; ++s)
        if (s >= limit) vals[s] = 0.0f;
      if (quad < 2 && half == 0) {  // A_ab -> fp32 scratch for the inverse
        float4* dst = reinterpret_cast<float4*>(smem + kOffAb + t * kInvLd * 4);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j] = make_float4(vals[4 * j], vals[4 * j + 1], vals[4 * j + 2], vals[4 * j + 3]);
      } else {
        // quad<2, half=1: A_ak -> X3 row t;   quad>=2, half=1: A_rk -> X3 row 64+t;
        // quad>=2, half=0: A_rb -> X1 area (now [T; A_rb]) row 64+t
        const int row = quad < 2 ? t : 64 + t;
        uint8_t* dst = smem + (half == 1 ? kOffX3 : kOffX1) + (row >> 3) * kRowGroup + (row & 7) * 16;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 hi, lo;
          split8(vals + 8 * j, hi, lo);
          *reinterpret_cast<uint4*>(dst + j * kChunkStride128) = hi;
          *reinterpret_cast<uint4*>(dst + kTile128 + j * kChunkStride128) = lo;
        }
      }
    }
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();

    FRWKV_PHASE(3)
    // ================= Q += [A_ak; A_rk] V (async) while the inverse runs on CUDA cores =================
    if (tid == 0) {
      tcgen05_fence_after_sync();
      issue_gemm<true, !kVExact>(tmem + kColQ, op_x3, op_v, idesc_kmn64, true);
      mma_commit(bar_mma);
    }
    {
      float* ab = reinterpret_cast<float*>(smem + kOffAb);
      float* ti = reinterpret_cast<float*>(smem + kOffTi);
      float* mb = reinterpret_cast<float*>(smem + kOffMb);
      // level 0: the four 16x16 diagonal blocks by forward substitution, one column per thread
      if (tid < 64) {
        const int d = tid >> 4, j = tid & 15;
        const float* blk = ab + (16 * d) * kInvLd + 16 * d;
        float part[16];  // right-looking substitution: part[t] collects the row sums as columns finish
#pragma unroll
        for (int t = 0; t < 16; ++t) part[t] = t == j ? 1.0f : 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < 16; ++s2) {
          const float xs = part[s2];  // x[s2] is final: every earlier column has been folded in
          ti[(16 * d + s2) * kInvLd + 16 * d + j] = xs;
#pragma unroll
          for (int t = s2 + 1; t < 16; ++t) part[t] = fmaf(blk[t * kInvLd + s2], xs, part[t]);
        }
      } else {  // zero everything above the block diagonal: 16-blocks (0,1), (2,3) and the 32-block (0,1)
        for (int e = tid - 64; e < 512 + 1024; e += kThreads - 64) {
          int rr, cc;
          if (e < 512) {
            const int blk = e >> 8;
            rr = 32 * blk + ((e >> 4) & 15);
            cc = 32 * blk + 16 + (e & 15);
          } else {
            rr = (e - 512) >> 5;
            cc = 32 + ((e - 512) & 31);
          }
          ti[rr * kInvLd + cc] = 0.0f;
        }
      }
      __syncthreads();
      // level 1: the two 32x32 diagonal blocks: T[hi,lo] = D_hi * (A[hi,lo] * D_lo), 16x16 each
      {
        const int b = tid >> 7, rr = (tid >> 3) & 15, c0 = (tid & 7) * 2;
        const int lo = 32 * b, hi = 32 * b + 16;
        float acc[2] = {0.0f, 0.0f};
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const float4 av = *reinterpret_cast<const float4*>(ab + (hi + rr) * kInvLd + lo + 4 * s4);
          const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 tv = *reinterpret_cast<const float2*>(ti + (lo + 4 * s4 + e) * kInvLd + lo + c0);
            acc[0] = fmaf(a4[e], tv.x, acc[0]);
            acc[1] = fmaf(a4[e], tv.y, acc[1]);
          }
        }
        *reinterpret_cast<float2*>(mb + (b * 16 + rr) * kMbLd + c0) = make_float2(acc[0], acc[1]);
        __syncthreads();
        acc[0] = acc[1] = 0.0f;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const float4 dv = *reinterpret_cast<const float4*>(ti + (hi + rr) * kInvLd + hi + 4 * s4);
          const float d4[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xv = *reinterpret_cast<const float2*>(mb + (b * 16 + 4 * s4 + e) * kMbLd + c0);
            acc[0] = fmaf(d4[e], xv.x, acc[0]);
            acc[1] = fmaf(d4[e], xv.y, acc[1]);
          }
        }
        *reinterpret_cast<float2*>(ti + (hi + rr) * kInvLd + lo + c0) = make_float2(acc[0], acc[1]);
      }
      __syncthreads();
      // level 2: T[32..63, 0..31] = T_hi * (A[32..63, 0..31] * T_lo), 32x32, a 2x2 tile per thread
      {
        const int r0 = (tid >> 4) * 2, c0 = (tid & 15) * 2;
        float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
        for (int s4 = 0; s4 < 8; ++s4) {
          const float4 a0 = *reinterpret_cast<const float4*>(ab + (32 + r0) * kInvLd + 4 * s4);
          const float4 a1 = *reinterpret_cast<const float4*>(ab + (33 + r0) * kInvLd + 4 * s4);
          const float a0v[4] = {a0.x, a0.y, a0.z, a0.w}, a1v[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 tv = *reinterpret_cast<const float2*>(ti + (4 * s4 + e) * kInvLd + c0);
            acc[0][0] = fmaf(a0v[e], tv.x, acc[0][0]);
            acc[0][1] = fmaf(a0v[e], tv.y, acc[0][1]);
            acc[1][0] = fmaf(a1v[e], tv.x, acc[1][0]);
            acc[1][1] = fmaf(a1v[e], tv.y, acc[1][1]);
          }
        }
        *reinterpret_cast<float2*>(mb + r0 * kMbLd + c0) = make_float2(acc[0][0], acc[0][1]);
        *reinterpret_cast<float2*>(mb + (r0 + 1) * kMbLd + c0) = make_float2(acc[1][0], acc[1][1]);
        __syncthreads();
        acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = 0.0f;
#pragma unroll
        for (int s4 = 0; s4 < 8; ++s4) {
          const float4 d0 = *reinterpret_cast<const float4*>(ti + (32 + r0) * kInvLd + 32 + 4 * s4);
          const float4 d1 = *reinterpret_cast<const float4*>(ti + (33 + r0) * kInvLd + 32 + 4 * s4);
          const float d0v[4] = {d0.x, d0.y, d0.z, d0.w}, d1v[4] = {d1.x, d1.y, d1.z, d1.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 xv = *reinterpret_cast<const float2*>(mb + (4 * s4 + e) * kMbLd + c0);
            acc[0][0] = fmaf(d0v[e], xv.x, acc[0][0]);
            acc[0][1] = fmaf(d0v[e], xv.y, acc[0][1]);
            acc[1][0] = fmaf(d1v[e], xv.x, acc[1][0]);
            acc[1][1] = fmaf(d1v[e], xv.y, acc[1][1]);
          }
        }
        *reinterpret_cast<float2*>(ti + (32 + r0) * kInvLd + c0) = make_float2(acc[0][0], acc[0][1]);
        *reinterpret_cast<float2*>(ti + (33 + r0) * kInvLd + c0) = make_float2(acc[1][0], acc[1][1]);
      }
      __syncthreads();
      // step 3: T -> rows 0..63 of the X1 area (hi/lo, K-major)
      {
        const int t = tid >> 2, cg = tid & 3;
        const float* src = ti + t * kInvLd + cg * 16;
        uint8_t* dst = smem + kOffX1 + (t >> 3) * kRowGroup + (t & 7) * 16;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = src[8 * j + e];
          uint4 hi, lo;
          split8(x, hi, lo);
          *reinterpret_cast<uint4*>(dst + (cg * 2 + j) * kChunkStride128) = hi;
          *reinterpret_cast<uint4*>(dst + kTile128 + (cg * 2 + j) * kChunkStride128) = lo;
        }
      }
    }
    FRWKV_PHASE(4)
    // wait for Q, then W = Q[0..63] -> operand tile (rows = token, MN-major)
    {
      const bool ok = mbar_wait(bar_mma, mma_uses & 1);
      ++mma_uses;
      if (__syncthreads_or(!ok)) { failed = true; break; }
      tcgen05_fence_after_sync();
    }
    auto rows_to_operand = [&](uint32_t col) {  // lanes 0..63 x 64 columns at `col` -> kOffOp (hi/lo)
      if (quad < 2) {
        const int t = quad * 32 + lane;
        uint32_t regs[32];
        tmem_ld32(tmem_lane + col + half * 32, regs);
        tmem_ld_wait();
        uint8_t* op = smem + kOffOp + (t & 7) * 16 + (t >> 3) * kRowGroup;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 hi, lo;
          split8(reinterpret_cast<const float*>(regs) + 8 * j, hi, lo);
          *reinterpret_cast<uint4*>(op + (half * 4 + j) * kChunkStride64) = hi;
          *reinterpret_cast<uint4*>(op + kTile64 + (half * 4 + j) * kChunkStride64) = lo;
        }
      }
    };
    rows_to_operand(kColQ);
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();

    FRWKV_PHASE(5)
    // ================= U = T W  (rows 64..127 of this product are unused) =================
    if (tid == 0) {
      tcgen05_fence_after_sync();
      if (c + 1 < n_chunks) issue_tma(c + 1);  // the staging area (and the inverse scratch in it) is free
      issue_gemm<true, true>(tmem + kColU, op_x1, op_rows, idesc_kmn64, false);
      mma_commit(bar_mma);
    }
    if (c + 1 < n_chunks) tma_in_flight = true;
    {
      const bool ok = mbar_wait(bar_mma, mma_uses & 1);
      ++mma_uses;
      if (__syncthreads_or(!ok)) { failed = true; break; }
      tcgen05_fence_after_sync();
    }
    FRWKV_PHASE(6)
    rows_to_operand(kColU);
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();

    FRWKV_PHASE(7)
    // ================= Q[64..] += A_rb U ;  S += Bt^T U + Kt^T V =================
    if (tid == 0) {
      tcgen05_fence_after_sync();
      issue_gemm<true, true>(tmem + kColQ, op_x1, op_rows, idesc_kmn64, true);
      issue_gemm<true, true>(tmem + kColS, op_bt, op_rows, idesc_mnmn64, true);
      issue_gemm<true, !kVExact>(tmem + kColS, op_kt, op_v, idesc_mnmn64, true);
      mma_commit(bar_mma);
    }
    {
      const bool ok = mbar_wait(bar_mma, mma_uses & 1);
      ++mma_uses;
      if (__syncthreads_or(!ok)) { failed = true; break; }
      tcgen05_fence_after_sync();
    }
    FRWKV_PHASE(8)
    if (quad >= 2) {
      // ---- y rows: lanes 64..127 of Q ----
      const int t = (quad - 2) * 32 + lane;
      uint32_t regs[32];
      tmem_ld32(tmem_lane + kColQ + half * 32, regs);
      tmem_ld_wait();
      if (t < rows) {
        const size_t out = (static_cast<size_t>(row0 + t) * p.heads + head) * kHeadDim + half * 32;
        float yv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) yv[i] = __uint_as_float(regs[i]) * p.scale;
        io_t* yp = static_cast<io_t*>(p.y) + out;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          alignas(16) io_t packed[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) packed[e] = from_f32<io_t>(yv[8 * j + e]);
          *reinterpret_cast<uint4*>(yp + 8 * j) = *reinterpret_cast<const uint4*>(packed);
        }
        if (p.y_f32 != nullptr) {
          float4* yf = reinterpret_cast<float4*>(p.y_f32 + out);
#pragma unroll
          for (int j = 0; j < 8; ++j) yf[j] = make_float4(yv[4 * j], yv[4 * j + 1], yv[4 * j + 2], yv[4 * j + 3]);
        }
      }
    } else {
      // ---- state rows: S <- diag(g_L) S; keep in TMEM, refresh the S0 operand (or store at the end) ----
      const int krow = quad * 32 + lane;
      uint32_t regs[32];
      tmem_ld32(tmem_lane + kColS + half * 32, regs);
      tmem_ld_wait();
      const float gl = gamma_l[krow];
#pragma unroll
      for (int i = 0; i < 32; ++i) regs[i] = __float_as_uint(__uint_as_float(regs[i]) * gl);
      if (c + 1 < n_chunks) {
        tmem_st32(tmem_lane + kColS + half * 32, regs);
        uint8_t* op = smem + kOffOp + (krow & 7) * 16 + (krow >> 3) * kRowGroup;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 hi, lo;
          split8(reinterpret_cast<const float*>(regs) + 8 * j, hi, lo);
          *reinterpret_cast<uint4*>(op + (half * 4 + j) * kChunkStride64) = hi;
          *reinterpret_cast<uint4*>(op + kTile64 + (half * 4 + j) * kChunkStride64) = lo;
        }
        tmem_st_wait();
      } else {
        float4* dst = reinterpret_cast<float4*>(state_g + krow * kHeadDim + half * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          __stcs(dst + i, make_float4(__uint_as_float(regs[4 * i]), __uint_as_float(regs[4 * i + 1]),
                                      __uint_as_float(regs[4 * i + 2]), __uint_as_float(regs[4 * i + 3])));
      }
    }
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    FRWKV_PHASE(9)
  }

  if (failed) {
    if (tid == 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 1);
    if (tma_in_flight) mbar_wait(bar_tma, tma_parity, 200000u);  // bounded drain of the load in flight
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

template <typename io_t>
int launch_typed(const ChunkParams& p, const Maps& maps, bool logits, cudaStream_t stream) {
  auto kernel = logits ? wkv7_chunk_tc_kernel<io_t, true> : wkv7_chunk_tc_kernel<io_t, false>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return check_launch("wkv7_chunk_tc_kernel shared-memory attribute");
  const long long ctas = static_cast<long long>(p.n_seq) * p.heads;
  if (ctas > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "wkv7_prefill: too many (sequence, head) pairs");
  kernel<<<static_cast<unsigned>(ctas), kThreads, kSmemBytes, stream>>>(p, maps);
  return check_launch("wkv7_chunk_tc_kernel");
}

}  // namespace

int launch_chunk64_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                    const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                    void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                    float scale, const int32_t* order, int len_from, int32_t* error_flag, cudaStream_t stream) {
  const bool bf16 = io_dtype == FRWKV_IO_BF16;
  Maps maps;
  const int map_rc = make_maps(&maps, r, w, k, v, a, b, total_tokens, heads, bf16, kChunk);
  if (map_rc != FRWKV_OK) return map_rc;
  ChunkParams p{cu, slots, status, pool, bias, y, y_f32, error_flag, n_seq, total_tokens, heads, scale, order, len_from, -1};
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  if (bf16) return launch_typed<__nv_bfloat16>(p, maps, logits, stream);
  return launch_typed<__half>(p, maps, logits, stream);
}

}  // namespace frwkv
