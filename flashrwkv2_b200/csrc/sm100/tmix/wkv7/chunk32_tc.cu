// WKV7 chunked prefill on tcgen05 tensor cores, 32-row chunks, two CTAs resident per SM.
//
// One CTA walks one (sequence, head) chunk by chunk with the fp32 state resident in TMEM.  With 32-row chunks
// the stacked operands [At; Rt], [Bt; Kt], [A_ak; A_rk] and [T; A_rb] have 64 rows, so every product is a
// natural M=64 MMA, one CTA needs about 111 KB of shared memory and 256 TMEM columns, and two CTAs of 288
// threads (96 registers) share an SM: while one waits for its MMAs or a barrier the other one's CUDA-core
// phases run.  A 64-row accumulator of an M=64 MMA puts row i in TMEM lane 32*(i/16) + i%16, i.e. every warp
// quadrant holds 16 rows in its lanes 0..15; the read-backs use the 16x256b fragment shape, which spreads
// those 16 rows over all 32 threads.  Eight warps compute; a ninth issues every MMA and TMA load.  Inside the
// stacked operands the two kinds of rows alternate in groups of eight (token t: 16*(t/8) + t%8 and eight
// further), so that every thread's fragment holds one row of each kind and all eight warps share every
// read-back.
//
// Per chunk of L <= 32 rows (g_t = inclusive product of the retentions inside the chunk, g_L its last value):
//     At = a g_{t-1}   Rt = r g_t   Bt = b / g_t   Kt = k / g_t   Bl = b g_L / g_t   Kl = k g_L / g_t
//     P  = [At; Rt] [Bt; Kt]^T  (64x64) -> A_ab, A_ak (strictly lower), A_rb, A_rk (lower), 32x32 each
//     Q  = [At; Rt] S0 + [A_ak; A_rk] V      (rows of the At kind = W, rows of the Rt kind = part of Y)
//     U  = (I - A_ab)^-1 W ;  Y = scale (Q[Rt rows] + A_rb U) ;  S <- diag(g_L) S0 + Bl^T U + Kl^T V
//
// Precision.  The 5e-3 gate on max|error|/RMS needs about 13 significant bits in the operands of the
// products that see the decay-scaled tokens twice (P) and 11 elsewhere; the cost of a product is the number
// of 16-bit terms it is issued as.  P is the only product whose operands are unbounded (1/g_t reaches 2^28
// over 32 rows), so it stays in bf16 with three terms (hi*hi + hi*lo + lo*hi, 16 bits).  Every other product
// uses operands that are bounded by the data (At, Rt, Bl, Kl carry factors <= 1; the masked blocks of P, T,
// W, U, V and the state are data-sized) and runs in fp16: one term (11 bits) for T W, A_rb U and Bl^T U, two
// terms for [At; Rt] S0 (hi + lo of the state), [A_ak; A_rk] V and Kl^T V (hi + lo of the left operand; V is
// exact).  34 MMAs per chunk instead of the 50 of an all-three-term scheme; emulated and measured error
// 1.1e-3 .. 2.4e-3 on the benchmark distributions, the reference's test distributions and on channels that
// always decay at the fastest rate.
#include "chunk_common.cuh"

namespace frwkv {
namespace {

using namespace tc;
using namespace chunk;

constexpr int kWarps = 8;                       // compute warps
constexpr int kComputeThreads = kWarps * 32;    // 256
constexpr int kThreads = kComputeThreads + 32;  // + one warp that issues every MMA and TMA load
// named barriers (0 is __syncthreads): the compute warps' own barrier, and five hand-offs on which the compute
// threads arrive (without waiting) and the issuer warp waits
constexpr int kBarCompute = 1, kBarOperands = 2, kBarState = 3, kBarMasks = 4, kBarInverse = 5, kBarU = 6;
constexpr int kBarDiag = 7, kBarMerge = 8;  // inside the inverse: warp 2 -> warps 4..7, and among warps 4..7
constexpr int kChunk = 32;

// ---- shared-memory map (bytes) -------------------------------------------------------------
constexpr uint32_t kStride64 = 8 * 128 + 16;  // stride between 16-byte chunks of a 64-row tile (padded)
constexpr uint32_t kTileK64 = 8 * kStride64;  // 64 rows x 64 columns, one 16-bit part: 8320
constexpr uint32_t kTileK32 = 4 * kStride64;  // 64 rows x 32 columns, one 16-bit part: 4160
constexpr uint32_t kStride32 = 4 * 128 + 16;  // stride between 16-byte chunks of a 32-row tile (padded)
constexpr uint32_t kTile32 = 8 * kStride32;   // 32 rows x 64 columns, one 16-bit part: 4224

constexpr uint32_t kRawTile = kChunk * 128;           // one [32][64] 16-bit tile as TMA writes it
constexpr uint32_t kOffRaw = 0;                       // r, w, k, v, a, b
constexpr uint32_t kOffX1 = kOffRaw + 6 * kRawTile;   // [At; Rt] bf16 hi, lo (64 x 64): left operand of P
constexpr uint32_t kOffX2 = kOffX1 + 2 * kTileK64;    // [Bt; Kt] bf16 hi, lo (64 x 64): right operand of P  (*)
constexpr uint32_t kOffX1h = kOffX2 + 2 * kTileK64;   // [At; Rt] fp16 (64 x 64): left operand of Q
constexpr uint32_t kOffBl = kOffX1h + kTileK64;       // Bl fp16 (32 rows = tokens, 64 key channels)
constexpr uint32_t kOffKl = kOffBl + kTile32;         // Kl fp16 hi, lo
constexpr uint32_t kOffX4 = kOffKl + 2 * kTile32;     // [T; A_rb] fp16 (64 x 32)
constexpr uint32_t kOffOp = kOffX4 + kTileK32;        // S0 hi, lo (64 rows) / W / U (32 rows, hi only) fp16, right operand
constexpr uint32_t kOffV = kOffOp + 2 * kTileK64;     // V fp16 (32 rows x 64)
constexpr uint32_t kOffMisc = kOffV + kTile32;        // group products [8][64], barriers
constexpr uint32_t kMiscBytes = kWarps * 64 * 4 + 64;
// (*) The operands of P are written during the previous chunk's last products and are dead as soon as P has
// completed, which is when the masked blocks of P and the scratch of the inverse come to life (and those are dead
// again before the next chunk's operands are written): [A_ak; A_rk] and the A_ab scratch share the area of [Bt; Kt].
constexpr uint32_t kOffX3 = kOffX2;                   // [A_ak; A_rk] fp16 hi, lo (64 x 32)
// fp32 scratch of the 32x32 inverse.  The 16x16 block product of level 1 lives in T's upper-right block, which is
// zero and never stored.
constexpr int kInvLd = 36;
constexpr uint32_t kOffAb = kOffX3 + 2 * kTileK32;     // A_ab [32][36]
static_assert(kOffAb + 32 * kInvLd * 4 <= kOffX1h, "masked blocks and A_ab scratch must fit in the area of [Bt; Kt]");
constexpr uint32_t kOffTi = kOffMisc + kMiscBytes;     // T    [32][36]
constexpr int kMbLd = kInvLd;
constexpr uint32_t kOffMb = kOffTi + 16 * 4;           // block product [16][16] at T[0..15][16..31]
constexpr uint32_t kSmemBytes = kOffTi + 32 * kInvLd * 4 + 128;
static_assert(2 * (kSmemBytes + 1024) <= 227 * 1024, "two CTAs must fit in one SM's shared memory");

// ---- TMEM map (columns) --------------------------------------------------------------------
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColP = 0, kColQ = 64, kColU = 128, kColS = 192;

template <typename io_t, bool LOGITS, bool FUSED, bool QUEUE>
__global__ void __launch_bounds__(kThreads, 2)
wkv7_chunk32_tc_kernel(const ChunkParams p, const __grid_constant__ Maps maps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3;       // TMEM lane quadrant this warp may access
  const int half = warp >> 2;      // which 32 of an accumulator's 64 columns this warp handles
  const bool row_lane = lane < 16; // lanes 0..15 of a quadrant hold accumulator rows 16*quad + lane
  const int arow = quad * 16 + (lane & 15);

  if (p.status != nullptr && p.status[0] != 0) {
    fill_output_nan(static_cast<io_t*>(p.y), p.y_f32, static_cast<long long>(p.total_tokens) * p.heads * kHeadDim,
                    static_cast<long long>(blockIdx.x) * kThreads + tid, static_cast<long long>(gridDim.x) * kThreads);
    return;
  }
  const int active = p.status != nullptr ? p.status[2] : p.n_seq;
  // The stream (sequence, head) and the range of its rows this CTA works on.  Direct mode: one stream per CTA, all of
  // its rows.  Queue mode (QUEUE): CTAs are persistent and take (stream, segment) tasks from a counter;
  // a segment is a run of `segment chunks` 32-row chunks, the state travels from a segment to the next through the
  // pool slot, and a per-stream flag says how many segments are complete (see QueueHeader in chunk_common.cuh).
  int head = 0, t_begin = 0, len = 0, n_chunks = 0, slot = 0, segment = 0;
  bool last_segment = true;
  int* segments_done = nullptr;  // queue mode: this stream's flag

  float* group_prod = reinterpret_cast<float*>(smem + kOffMisc);  // [8][64] retention products of each 4-row group
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(group_prod + kWarps * 64);
  uint64_t* bar_mma = bar_tma + 1;    // Q, U, Y of every chunk, in this order
  uint64_t* bar_state = bar_tma + 2;  // its own barrier: two commits may not complete two phases of one
  uint64_t* bar_drain = bar_tma + 3;  // the issuer warp's last commit: every MMA has retired before TMEM is freed
  uint64_t* bar_p = bar_tma + 4;      // P of the next chunk is issued while this chunk's Y is still outstanding
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 5);
  volatile uint32_t* abort_flag = tmem_slot + 1;  // set by the compute warps when a bounded wait gave up
  volatile uint32_t* decay_flag = tmem_slot + 2;  // a chunk's decay product left the representable range
  const uint32_t sbase = smem_u32(smem);

  if (tid == 0) {
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_state, 1);
    mbar_init(bar_drain, 1);
    mbar_init(bar_p, 1);
    mbar_fence_init();
    *abort_flag = 0u;
    *decay_flag = 0u;
    tma_prefetch_descriptor(&maps.r);
    tma_prefetch_descriptor(&maps.w);
    tma_prefetch_descriptor(&maps.k);
    tma_prefetch_descriptor(&maps.v);
    tma_prefetch_descriptor(&maps.a);
    if constexpr (!FUSED) tma_prefetch_descriptor(&maps.b);
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

  auto issue_tma = [&](int chunk_index) {  // one thread
    const int row = t_begin + chunk_index * kChunk;
    mbar_expect_tx(bar_tma, (FUSED ? 5 : 6) * kRawTile);  // the fused producer form has no b tensor
    tma_load_3d(smem + kOffRaw + 0 * kRawTile, &maps.r, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 1 * kRawTile, &maps.w, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 2 * kRawTile, &maps.k, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 3 * kRawTile, &maps.v, bar_tma, 0, head, row);
    tma_load_3d(smem + kOffRaw + 4 * kRawTile, &maps.a, bar_tma, 0, head, row);
    if constexpr (!FUSED) tma_load_3d(smem + kOffRaw + 5 * kRawTile, &maps.b, bar_tma, 0, head, row);
  };
  bool tma_in_flight = false;
  uint32_t tma_parity = 0;
  uint32_t chunks_done = 0;  // chunks of earlier tasks: bar_p and bar_state complete one phase per chunk

  // Fragment view of an accumulator block (tmem_ld_frag16): this thread holds rows frow0 and frow0 + 8 of its
  // quadrant and, of the 32 columns at 32*half, the pairs 8n + 2*fq + {0,1}, n = 0..3.
  const int fq = lane & 3;
  const int frow0 = quad * 16 + (lane >> 2);
  // fragment -> fp16 operand tile at `tile` (rows = accumulator rows, 16-byte column chunks from `chunk0` on):
  // one 4-byte store per pair; the 32 lanes of a store cover 128 contiguous bytes
  auto store_frag_f16_split = [&](uint32_t tile, uint32_t lo_off, int chunk0, const float (&x)[16]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = frow0 + 8 * h;
      uint8_t* dst = smem + tile + (row >> 3) * kRowGroup + (row & 7) * 16 + fq * 4;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        uint32_t hi, lo;
        split2_f16(x[4 * n + 2 * h], x[4 * n + 2 * h + 1], hi, lo);
        *reinterpret_cast<uint32_t*>(dst + (chunk0 + n) * kStride64) = hi;
        *reinterpret_cast<uint32_t*>(dst + lo_off + (chunk0 + n) * kStride64) = lo;
      }
    }
  };

  float* state_g = nullptr;
  const bool compute_warp = warp < kWarps;

  constexpr uint32_t idesc_p = instr_desc_f16(64, 64, kMajorK, kMajorK, true);        // bf16 x bf16
  constexpr uint32_t idesc_kmn = instr_desc_f16(64, 64, kMajorK, kMajorMN, false);    // fp16, A K-major, B MN-major
  constexpr uint32_t idesc_mnmn = instr_desc_f16(64, 64, kMajorMN, kMajorMN, false);  // fp16, both MN-major

  // operand descriptors (fixed for the whole kernel); K-major tiles: chunk stride kStride64, row groups 128 B
  const Operand op_x1 = make_operand(sbase + kOffX1, kTileK64, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x2 = make_operand(sbase + kOffX2, kTileK64, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x1h = make_operand(sbase + kOffX1h, 0, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x3 = make_operand(sbase + kOffX3, kTileK32, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x4 = make_operand(sbase + kOffX4, 0, 2 * kStride64, kStride64, kRowGroup);
  // MN-major tiles (rows = contraction index): row groups 128 B apart, 16-byte column chunks at the tile's stride
  const Operand op_rows = make_operand(sbase + kOffOp, kTileK64, 2 * kRowGroup, kRowGroup, kStride64);
  const Operand op_v = make_operand(sbase + kOffV, 0, 2 * kRowGroup, kRowGroup, kStride32);
  // Bl, Kl read MN-major as left operands: M = key channel, contraction = token row
  const Operand op_bl = make_operand(sbase + kOffBl, 0, 2 * kRowGroup, kRowGroup, kStride32);
  const Operand op_kl = make_operand(sbase + kOffKl, kTile32, 2 * kRowGroup, kRowGroup, kStride32);

  // Row order of the stacked 64-row operands [At; Rt], [A_ak; A_rk], [T; A_rb] and of their accumulators: the two
  // kinds alternate in groups of eight, token t's At-kind row at 16*(t/8) + t%8 and its Rt-kind row eight further.
  // A quadrant then holds eight rows of each kind, and in the fragment view every thread has one of each (rows
  // frow0 and frow0 + 8, both of token ftok): W, U and y read-backs are spread over all eight compute warps.
  const int ftok = quad * 8 + (lane >> 2);
  auto rows_to_operand = [&](uint32_t col) {  // the 32 At-kind accumulator rows x 64 columns at `col` -> kOffOp (row = token)
    uint32_t regs[16];
    tmem_ld_frag16(tmem_lane + col + half * 32, regs);
    tmem_ld_wait();
    uint8_t* dst = smem + kOffOp + (ftok >> 3) * kRowGroup + (ftok & 7) * 16 + fq * 4;
#pragma unroll
    for (int n = 0; n < 4; ++n)
      *reinterpret_cast<uint32_t*>(dst + (half * 4 + n) * kStride64) =
          pack_f16x2(__uint_as_float(regs[4 * n]), __uint_as_float(regs[4 * n + 1]));
  };

  bool failed = false;
  bool bad = false;  // this thread saw a bounded wait give up; turned into `failed` at the next CTA barrier
#ifdef FRWKV_CHUNK_TIMING
  long long phase_t0 = clock64();
#endif
  const io_t* bias_g = nullptr;
  // fused kk / a-gate producer (csrc/sm120/tmix/wkv_prepare/internal/kk_a_gate/infer_fp16_forward_varlen.cu:131-156
  // of the reference): this thread's two key channels of the per-head parameters (set per task)
  float2 gate_kk = make_float2(0.f, 0.f), gate_a0 = gate_kk, gate_ka = gate_kk;

  // ---- operand preparation of one chunk (decay products, scaled operands) -----------------------------------
  // It depends on the tokens only, so it runs for chunk c+1 while the tensor pipe works on chunk c's last
  // products.  The operands of P and Q go straight to their tiles (P and Q of chunk c are long finished), and so
  // does Kl (Kl^T V of chunk c has retired once U has); V and Bl, whose tiles chunk c's products may still read,
  // wait in registers until release_v() / release_bl().
  uint32_t held_bl[kChunk / kWarps];  // per row of this thread: Bl, two key channels
  uint4 held_v;
  float2 held_g[kChunk / kWarps];  // inclusive retention product g_t of this thread's rows, scan -> scaling
  float2 held_off = make_float2(1.f, 1.f);  // ... of the rows before them
  float2 held_tot = make_float2(1.f, 1.f);  // ... and of the whole chunk (g_L)
  auto scan_decay = [&](int chunk) -> bool {  // first half (all compute threads; one compute barrier inside)
    const int rows = min(kChunk, len - chunk * kChunk);
    const bool ok = mbar_wait(bar_tma, tma_parity);
    tma_in_flight = false;
    tma_parity ^= 1u;
    constexpr int kRowsPerWarp = kChunk / kWarps;  // 4
    const int kp = lane;                           // key channels 2*kp, 2*kp+1
    const int tg = warp;                           // rows 4*tg .. 4*tg+3
    const uint32_t* raw_w = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 1 * kRawTile);
    float2 bias2 = make_float2(0.f, 0.f);
    if (bias_g != nullptr) bias2 = make_float2(to_f32(bias_g[2 * kp]), to_f32(bias_g[2 * kp + 1]));
    float2 run = make_float2(1.f, 1.f);
    float2 cum[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int t = tg * kRowsPerWarp + i;
      float2 rho = unpack2<io_t>(raw_w[t * 32 + kp]);
      if constexpr (LOGITS) {
        rho.x = fast_exp2(__fdividef(-kRateLog2e, 1.0f + fast_exp2(-kLog2e * (rho.x + bias2.x))));
        rho.y = fast_exp2(__fdividef(-kRateLog2e, 1.0f + fast_exp2(-kLog2e * (rho.y + bias2.y))));
      }
      if (t >= rows) rho = make_float2(1.f, 1.f);
      run.x *= rho.x;
      run.y *= rho.y;
      cum[i] = run;
    }
    reinterpret_cast<float2*>(group_prod + tg * 64)[kp] = run;
    // V operand: rows = token, 64 contiguous value columns (MN-major), converted to fp16 (exact for bf16 values
    // inside the fp16 range)
    {
      const uint8_t* raw_v = smem + kOffRaw + 3 * kRawTile;
      const int sr = tid >> 3, vc = tid & 7;  // 256 chunks of 8 values
      uint4 q = *reinterpret_cast<const uint4*>(raw_v + sr * 128 + vc * 16);
      if (sr >= rows) q = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (std::is_same<io_t, __half>::value) {
        held_v = q;
      } else {
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        uint32_t out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack2<io_t>(words[e]);
          out[e] = pack_f16x2(f.x, f.y);
        }
        held_v = make_uint4(out[0], out[1], out[2], out[3]);
      }
    }
    named_sync(kBarCompute, kComputeThreads);
    float2 off = make_float2(1.f, 1.f), tot = make_float2(1.f, 1.f);
#pragma unroll
    for (int g = 0; g < kWarps; ++g) {  // loads issued together; only the products are a chain
      const float2 pgrp = reinterpret_cast<const float2*>(group_prod + g * 64)[kp];
      if (g < tg) {
        off.x *= pgrp.x;
        off.y *= pgrp.y;
      }
      tot.x *= pgrp.x;
      tot.y *= pgrp.y;
    }
    held_off = off;
    held_tot = tot;
    if constexpr (!LOGITS) {
      // 1/g_t must stay inside the fp32 range (the logits form cannot produce less than 2^-28 over a chunk)
      if (!(tot.x > 1e-36f) || !(tot.y > 1e-36f)) *decay_flag = 1u;
    }
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) held_g[i] = make_float2(off.x * cum[i].x, off.y * cum[i].y);
    return ok;
  };
  // g_L of the chunk scan_decay() ran for last, for key channel `channel`: every warp holds all 64 values (lane l has
  // channels 2l and 2l+1), so a shuffle delivers it without shared memory or a barrier.  All lanes must call it.
  auto chunk_decay_of = [&](int channel) -> float {
    const float x = __shfl_sync(0xffffffffu, held_tot.x, channel >> 1);
    const float y = __shfl_sync(0xffffffffu, held_tot.y, channel >> 1);
    return (channel & 1) ? y : x;
  };
  auto scale_operands = [&](int chunk) {  // second half: no barrier inside
    const int rows = min(kChunk, len - chunk * kChunk);
    constexpr int kRowsPerWarp = kChunk / kWarps;
    const int kp = lane, tg = warp;
    const uint32_t* raw_r = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 0 * kRawTile);
    const uint32_t* raw_k = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 2 * kRawTile);
    const uint32_t* raw_a = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 4 * kRawTile);
    const uint32_t* raw_b = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 5 * kRawTile);
    float2 g_prev = held_off;
    const float2 gl = held_tot;
    const uint32_t col64 = (kp >> 2) * kStride64 + (kp & 3) * 4;  // this thread's two channels in a 64-row tile
    const uint32_t col32 = (kp >> 2) * kStride32 + (kp & 3) * 4;  // ... in a 32-row tile
    uint8_t* x1 = smem + kOffX1 + col64;
    uint8_t* x2 = smem + kOffX2 + col64;
    uint8_t* x1h = smem + kOffX1h + col64;
    uint8_t* kl = smem + kOffKl + col32;
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int t = tg * kRowsPerWarp + i;
      const float2 g = held_g[i];
      float2 gi;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(gi.x) : "f"(g.x));
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(gi.y) : "f"(g.y));
      const float2 gx = g_prev;  // exclusive product = inclusive product of the previous row
      g_prev = g;
      float2 r2 = unpack2<io_t>(raw_r[t * 32 + kp]);
      float2 k2 = unpack2<io_t>(raw_k[t * 32 + kp]);
      float2 a2 = unpack2<io_t>(raw_a[t * 32 + kp]);
      float2 b2 = make_float2(0.f, 0.f);
      if constexpr (!FUSED) b2 = unpack2<io_t>(raw_b[t * 32 + kp]);
      if (t >= rows) {  // rows past the end of the sequence belong to somebody else (or are the loader's zero fill)
        r2 = k2 = a2 = b2 = make_float2(0.f, 0.f);
      }
      if constexpr (FUSED) {
        // k2 is the raw key and a2 the gate logit a12: kk = normalize(k * k_k) over the 64 channels of the row (the
        // 32 lanes hold two each), a = -kk, b = kk * g, k' = k * (1 + (g - 1) * k_a), g = sigmoid(a0 + a12); the three
        // results are rounded to the token dtype where the reference's producer kernel stores them
        const float2 u = make_float2(k2.x * gate_kk.x, k2.y * gate_kk.y);
        float ss = fmaf(u.x, u.x, u.y * u.y);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        // SFU forms (rsqrt, ex2, rcp; 2^-22 relative): the values are rounded to 16 bits right below
        float inv;
        asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(fmaxf(ss, 1.0e-24f)));
        float2 g2;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g2.x) : "f"(1.0f + fast_exp2(-kLog2e * (gate_a0.x + a2.x))));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g2.y) : "f"(1.0f + fast_exp2(-kLog2e * (gate_a0.y + a2.y))));
        const float2 kk = make_float2(u.x * inv, u.y * inv);
        auto rnd = [](float x) { return to_f32(from_f32<io_t>(x)); };
        a2 = make_float2(rnd(-kk.x), rnd(-kk.y));
        b2 = make_float2(rnd(kk.x * g2.x), rnd(kk.y * g2.y));
        k2 = make_float2(rnd(k2.x * fmaf(g2.x, gate_ka.x, 1.0f - gate_ka.x)), rnd(k2.y * fmaf(g2.y, gate_ka.y, 1.0f - gate_ka.y)));
        if (t >= rows) a2 = b2 = k2 = make_float2(0.f, 0.f);
      }
      const uint32_t row_a = 2 * (t >> 3) * kRowGroup + (t & 7) * 16;  // At row of token t: 16*(t/8) + t%8
      const uint32_t row_r = row_a + kRowGroup;                        // Rt row: eight further
      const uint32_t row_b = (t >> 3) * kRowGroup + (t & 7) * 16;      // Bt row t, Kt row 32 + t; Bl / Kl row t
      uint32_t h, l;
      const float2 at = make_float2(a2.x * gx.x, a2.y * gx.y), rt = make_float2(r2.x * g.x, r2.y * g.y);
      const float2 bt = make_float2(b2.x * gi.x, b2.y * gi.y), kt = make_float2(k2.x * gi.x, k2.y * gi.y);
      split2(at.x, at.y, h, l);
      *reinterpret_cast<uint32_t*>(x1 + row_a) = h;
      *reinterpret_cast<uint32_t*>(x1 + kTileK64 + row_a) = l;
      *reinterpret_cast<uint32_t*>(x1h + row_a) = pack_f16x2(at.x, at.y);
      split2(rt.x, rt.y, h, l);
      *reinterpret_cast<uint32_t*>(x1 + row_r) = h;
      *reinterpret_cast<uint32_t*>(x1 + kTileK64 + row_r) = l;
      *reinterpret_cast<uint32_t*>(x1h + row_r) = pack_f16x2(rt.x, rt.y);
      split2(bt.x, bt.y, h, l);
      *reinterpret_cast<uint32_t*>(x2 + row_b) = h;
      *reinterpret_cast<uint32_t*>(x2 + kTileK64 + row_b) = l;
      split2(kt.x, kt.y, h, l);
      *reinterpret_cast<uint32_t*>(x2 + row_b + 4 * kRowGroup) = h;
      *reinterpret_cast<uint32_t*>(x2 + kTileK64 + row_b + 4 * kRowGroup) = l;
      held_bl[i] = pack_f16x2(bt.x * gl.x, bt.y * gl.y);  // Bl = b g_L / g_t: a factor <= 1
      split2_f16(kt.x * gl.x, kt.y * gl.y, h, l);
      *reinterpret_cast<uint32_t*>(kl + row_b) = h;
      *reinterpret_cast<uint32_t*>(kl + kTile32 + row_b) = l;
    }
  };
  auto release_v = [&]() {  // V of the prepared chunk: registers -> tile
    const int sr = tid >> 3, vc = tid & 7;
    *reinterpret_cast<uint4*>(smem + kOffV + vc * kStride32 + (sr & 7) * 16 + (sr >> 3) * kRowGroup) = held_v;
  };
  auto release_bl = [&]() {  // Bl of the prepared chunk: registers -> tile
    const int kp = lane, tg = warp;
    uint8_t* bl = smem + kOffBl + (kp >> 2) * kStride32 + (kp & 3) * 4;
#pragma unroll
    for (int i = 0; i < kChunk / kWarps; ++i) {
      const int t = tg * (kChunk / kWarps) + i;
      *reinterpret_cast<uint32_t*>(bl + (t >> 3) * kRowGroup + (t & 7) * 16) = held_bl[i];
    }
  };

  uint32_t mma_phase = 0;  // completed phases of bar_mma, counted the same way by every compute thread
  volatile int* task_word = reinterpret_cast<volatile int*>(tmem_slot + 3);

  for (bool first_task = true;; first_task = false) {
  // ---- next task ------------------------------------------------------------------------------------------
  // every warp has left the previous task; if that one was aborted (the compute warps carry `failed`), everybody
  // leaves the loop together
  int task;
  if constexpr (QUEUE) {
    if (__syncthreads_or(failed ? 1 : 0) != 0) break;
    if (tid == 0) {
      int next = atomicAdd(&p.queue->next_task, 1);
      if (next >= p.queue->total_tasks) next = -1;
      *task_word = next;
    }
    __syncthreads();
    task = *task_word;
    if (task < 0) break;
  } else {  // one CTA per (sequence, head): a single pass
    if (!first_task) break;
    task = static_cast<int>(blockIdx.x);
  }
  {
    int rank;
    if (QUEUE) {
      // tasks are numbered segment by segment; the streams that have a segment g are the first level_end[g] -
      // level_end[g-1] ranks of the longest-first order, all heads of a rank next to each other
      int g = 0;
      while (g + 1 < kQueueLevels && task >= p.queue->level_end[g]) ++g;
      const int in_level = task - (g > 0 ? p.queue->level_end[g - 1] : 0);
      rank = in_level / p.heads;
      head = in_level % p.heads;
      segment = g;
    } else {
      rank = task / p.heads;
      head = task % p.heads;
      segment = 0;
    }
    if (rank >= p.n_seq) continue;
    const int seq = p.order != nullptr ? p.order[rank] : rank;
    if (seq >= active || seq < 0 || seq >= p.n_seq) continue;
    const int seq_begin = p.cu[seq], seq_len = p.cu[seq + 1] - seq_begin;
    if (seq_len <= 0 || seq_len < p.len_from) continue;
    const int seg_rows = QUEUE ? p.queue->segment_chunks * kChunk : seq_len;
    t_begin = seq_begin + segment * seg_rows;
    len = min(seq_len - segment * seg_rows, seg_rows);
    if (len <= 0) continue;
    last_segment = segment * seg_rows + len >= seq_len;
    n_chunks = (len + kChunk - 1) / kChunk;
    slot = p.slots[seq];
    state_g = p.pool + (static_cast<size_t>(slot) * p.heads + head) * (kHeadDim * kHeadDim);
    segments_done = QUEUE ? p.queue_flags + static_cast<size_t>(seq) * p.heads + head : nullptr;
    bias_g = LOGITS && p.bias != nullptr ? static_cast<const io_t*>(p.bias) + head * kHeadDim : nullptr;
    if constexpr (FUSED) {
      const int at = head * kHeadDim + 2 * lane;
      gate_kk = unpack2<io_t>(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.gate_kk) + at));
      gate_a0 = unpack2<io_t>(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.gate_a0) + at));
      gate_ka = unpack2<io_t>(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.gate_ka) + at));
    }
  }
  if (tid == 0) issue_tma(0);
  tma_in_flight = true;

  if (compute_warp) {
    // =====================================================================================================
    // Compute warps.  They never wait for the issuer warp except through the MMA mbarriers (bounded waits);
    // at each hand-off they arrive on a named barrier and go on.  A wait that gave up sets `bad`; the compute
    // warps agree on it at their next own barrier (`failed`), set `abort_flag`, make the one arrival the issuer
    // warp may still be waiting for, and leave.  The issuer warp reads `abort_flag` after every hand-off, so it
    // is never left waiting.
    // =====================================================================================================
    // chunk 0 is prepared up front; afterwards every chunk prepares its successor
    bad |= !scan_decay(0);
    scale_operands(0);
    release_v();
    release_bl();
    // ---- queue mode, later segment: the previous segment of this stream must have stored its state.  Its task
    // was handed out before this one, so the CTA that took it is running or done: the wait ends, and is bounded
    // anyway.  The flag is read with acquire semantics by one thread; the barrier passes the ordering on.
    if (QUEUE && segment > 0) {
      if (tid == 0) {
        int seen = 0;
        for (int poll = 0; poll < (1 << 22); ++poll) {
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(segments_done) : "memory");
          if (seen >= segment) break;
          __nanosleep(200);
        }
        if (seen < segment) bad = true;
      }
      named_sync(kBarCompute, kComputeThreads);
      __threadfence();
    }
    // ---- initial state: global -> S0 operand tile (fp16) and -> TMEM (fp32, already times g_L of chunk 0) ----
    {
      uint32_t regs[32];
      const float g0 = chunk_decay_of(arow);
      if (row_lane) {
        const float4* src = reinterpret_cast<const float4*>(state_g + arow * kHeadDim + half * 32);
        uint8_t* op = smem + kOffOp + (arow & 7) * 16 + (arow >> 3) * kRowGroup;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 f0 = __ldcg(src + 2 * j), f1 = __ldcg(src + 2 * j + 1);  // L2: another SM may have written it
          uint32_t hi[4], lo[4];
          split2_f16(f0.x, f0.y, hi[0], lo[0]);
          split2_f16(f0.z, f0.w, hi[1], lo[1]);
          split2_f16(f1.x, f1.y, hi[2], lo[2]);
          split2_f16(f1.z, f1.w, hi[3], lo[3]);
          *reinterpret_cast<uint4*>(op + (half * 4 + j) * kStride64) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(op + kTileK64 + (half * 4 + j) * kStride64) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          regs[8 * j + 0] = __float_as_uint(f0.x * g0);
          regs[8 * j + 1] = __float_as_uint(f0.y * g0);
          regs[8 * j + 2] = __float_as_uint(f0.z * g0);
          regs[8 * j + 3] = __float_as_uint(f0.w * g0);
          regs[8 * j + 4] = __float_as_uint(f1.x * g0);
          regs[8 * j + 5] = __float_as_uint(f1.y * g0);
          regs[8 * j + 6] = __float_as_uint(f1.z * g0);
          regs[8 * j + 7] = __float_as_uint(f1.w * g0);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) regs[i] = 0u;
      }
      tmem_st32(tmem_lane + kColS + half * 32, regs);
      tmem_st_wait();
    }
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    failed = named_sync_or(kBarCompute, kComputeThreads, bad);
    if (failed && tid == 0) *abort_flag = 1u;
    named_arrive(kBarOperands, kThreads);  // the operands of P for chunk 0 are in place -> P
    if (!failed) {
      named_arrive(kBarState, kThreads);   // ... and so are S0 and the scaled state -> Q, then the next chunk's load
      if (n_chunks > 1) tma_in_flight = true;
    }

    for (int c = 0; c < n_chunks && !failed; ++c) {
      const int rows = min(kChunk, len - c * kChunk);
      const int row0 = t_begin + c * kChunk;
      const bool more = c + 1 < n_chunks;
      FRWKV_PHASE(0)

      // ================= P = X1 X2^T (issued during the previous chunk; Q = X1 S0 runs under the read-back) ====
      bad |= !mbar_wait(bar_p, (chunks_done + c) & 1);
      tcgen05_fence_after_sync();
      FRWKV_PHASE(2)
      // ================= read P: masks, A_ab -> fp32 scratch, others -> operand tiles =================
      {
        // this thread's rows: h = 0 the At row of token ftok (products with Bt: A_ab, with Kt: A_ak; strictly lower),
        // h = 1 its Rt row (A_rb, A_rk; lower); columns 32*half..: half 0 = products with Bt, half 1 = with Kt
        uint32_t regs[16];
        tmem_ld_frag16(tmem_lane + kColP + half * 32, regs);
        tmem_ld_wait();
        // Column block n (columns 8n..8n+7) against this quadrant's tokens 8*quad..8*quad+7: blocks left of the
        // diagonal are kept whole, blocks right of it are zero, only block n == quad needs the per-element test.
        float vals[16];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int limit = ftok + h;  // keep columns s < limit
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float x = __uint_as_float(regs[4 * n + 2 * h + e]);
              vals[4 * n + 2 * h + e] = n < quad ? x : (n == quad && 8 * n + 2 * fq + e < limit ? x : 0.0f);
            }
          }
        }
        if (half == 0) {
          // A_ab row -> fp32 scratch of the inverse; A_rb row -> [T; A_rb] at its accumulator position
          float* ab_row = reinterpret_cast<float*>(smem + kOffAb) + ftok * kInvLd + 2 * fq;
          const int row = frow0 + 8;
          uint8_t* rb = smem + kOffX4 + (row >> 3) * kRowGroup + (row & 7) * 16 + fq * 4;
#pragma unroll
          for (int n = 0; n < 4; ++n) {
            *reinterpret_cast<float2*>(ab_row + 8 * n) = make_float2(vals[4 * n], vals[4 * n + 1]);
            *reinterpret_cast<uint32_t*>(rb + n * kStride64) = pack_f16x2(vals[4 * n + 2], vals[4 * n + 3]);
          }
        } else {
          // A_ak and A_rk rows, in accumulator order (hi/lo; a block right of the diagonal is stored as zeros)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = frow0 + 8 * h;
            uint8_t* dst = smem + kOffX3 + (row >> 3) * kRowGroup + (row & 7) * 16 + fq * 4;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
              uint32_t hi = 0u, lo = 0u;
              if (n <= quad) split2_f16(vals[4 * n + 2 * h], vals[4 * n + 2 * h + 1], hi, lo);
              *reinterpret_cast<uint32_t*>(dst + n * kStride64) = hi;
              *reinterpret_cast<uint32_t*>(dst + kTileK32 + n * kStride64) = lo;
            }
          }
        }
      }
      fence_proxy_async_smem();
      tcgen05_fence_before_sync();
      named_arrive(kBarMasks, kThreads);  // -> Q += [A_ak; A_rk] V
      failed = named_sync_or(kBarCompute, kComputeThreads, bad);  // A_ab scratch visible to the inverse
      if (failed) {
        if (tid == 0) *abort_flag = 1u;
        named_arrive(kBarInverse, kThreads);  // the issuer warp's next hand-off
        break;
      }
      FRWKV_PHASE(3)

      // ================= 32x32 inverse on CUDA cores while Q is finished by the tensor pipe =================
      {
        float* ab = reinterpret_cast<float*>(smem + kOffAb);
        float* ti = reinterpret_cast<float*>(smem + kOffTi);
        float* mb = reinterpret_cast<float*>(smem + kOffMb);
        bool w_ready = true;
        // Levels 0 and 1 of the inverse run on five warps while the others only wait for Q:
        // level 0 (warp 2): the four 8x8 diagonal blocks of (I - A_ab)^-1 by right-looking forward substitution, one
        // column per lane, 8 steps; level 1 (warps 4..7, after clearing the 8x8 blocks above the diagonal): inside each
        // 16x16 diagonal block T[8..15, 0..7] = D_1 * (A[8..15, 0..7] * D_0), 64 outputs per block.
        if (warp == 2) {
          const int o = 8 * (lane >> 3), j = lane & 7;
          const float* blk = ab + o * kInvLd + o;
          float part[8];  // part[t] collects the row sums as columns finish
#pragma unroll
          for (int t = 0; t < 8; ++t) part[t] = t == j ? 1.0f : 0.0f;
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2) {
            const float xs = part[s2];  // x[s2] is final: every earlier column has been folded in
            ti[(o + s2) * kInvLd + o + j] = xs;
#pragma unroll
            for (int t = s2 + 1; t < 8; ++t) part[t] = fmaf(blk[t * kInvLd + s2], xs, part[t]);
          }
          named_arrive(kBarDiag, 32 + 128);
        } else if (warp >= 4) {
          const int u = tid - 128;
          const int o = 16 * (u >> 6), r8 = (u >> 3) & 7, c8 = u & 7;
          float* m8 = mb + 8 * (u >> 6);  // 8x8 scratch of this block inside T's (zero) upper-right block
          ti[(o + r8) * kInvLd + o + 8 + c8] = 0.0f;
          named_sync(kBarDiag, 32 + 128);  // warp 2's diagonal blocks are in place
          float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
          for (int s4 = 0; s4 < 2; ++s4) {
            const float4 av = *reinterpret_cast<const float4*>(ab + (o + 8 + r8) * kInvLd + o + 4 * s4);
            acc0 = fmaf(av.x, ti[(o + 4 * s4 + 0) * kInvLd + o + c8], acc0);
            acc1 = fmaf(av.y, ti[(o + 4 * s4 + 1) * kInvLd + o + c8], acc1);
            acc0 = fmaf(av.z, ti[(o + 4 * s4 + 2) * kInvLd + o + c8], acc0);
            acc1 = fmaf(av.w, ti[(o + 4 * s4 + 3) * kInvLd + o + c8], acc1);
          }
          m8[r8 * kMbLd + c8] = acc0 + acc1;
          named_sync(kBarMerge, 128);
          acc0 = acc1 = 0.0f;
#pragma unroll
          for (int s4 = 0; s4 < 2; ++s4) {
            const float4 dv = *reinterpret_cast<const float4*>(ti + (o + 8 + r8) * kInvLd + o + 8 + 4 * s4);
            acc0 = fmaf(dv.x, m8[(4 * s4 + 0) * kMbLd + c8], acc0);
            acc1 = fmaf(dv.y, m8[(4 * s4 + 1) * kMbLd + c8], acc1);
            acc0 = fmaf(dv.z, m8[(4 * s4 + 2) * kMbLd + c8], acc0);
            acc1 = fmaf(dv.w, m8[(4 * s4 + 3) * kMbLd + c8], acc1);
          }
          ti[(o + 8 + r8) * kInvLd + o + c8] = acc0 + acc1;
        }
        // meanwhile Q has been finished by the tensor pipe: its At-kind rows (W) become the operand tile
        w_ready = __all_sync(0xffffffffu, mbar_wait(bar_mma, mma_phase & 1));
        tcgen05_fence_after_sync();
        if (w_ready) rows_to_operand(kColQ);
        ++mma_phase;
        bad |= !w_ready;
        named_sync(kBarCompute, kComputeThreads);
        FRWKV_PHASE(10)
        // level 2: T[16..31, 0..15] = D_1 * (A[16..31, 0..15] * D_0) with the 16x16 blocks, one output per thread
        {
          const int rr = tid >> 4, cc = tid & 15;
          float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // four independent partial sums: no 16-deep FMA chain
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const float4 av = *reinterpret_cast<const float4*>(ab + (16 + rr) * kInvLd + 4 * s4);
            acc[0] = fmaf(av.x, ti[(4 * s4 + 0) * kInvLd + cc], acc[0]);
            acc[1] = fmaf(av.y, ti[(4 * s4 + 1) * kInvLd + cc], acc[1]);
            acc[2] = fmaf(av.z, ti[(4 * s4 + 2) * kInvLd + cc], acc[2]);
            acc[3] = fmaf(av.w, ti[(4 * s4 + 3) * kInvLd + cc], acc[3]);
          }
          mb[rr * kMbLd + cc] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
          named_sync(kBarCompute, kComputeThreads);
          acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const float4 dv = *reinterpret_cast<const float4*>(ti + (16 + rr) * kInvLd + 16 + 4 * s4);
            acc[0] = fmaf(dv.x, mb[(4 * s4 + 0) * kMbLd + cc], acc[0]);
            acc[1] = fmaf(dv.y, mb[(4 * s4 + 1) * kMbLd + cc], acc[1]);
            acc[2] = fmaf(dv.z, mb[(4 * s4 + 2) * kMbLd + cc], acc[2]);
            acc[3] = fmaf(dv.w, mb[(4 * s4 + 3) * kMbLd + cc], acc[3]);
          }
          ti[(16 + rr) * kInvLd + cc] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        named_sync(kBarCompute, kComputeThreads);
        FRWKV_PHASE(11)
        // T -> the At-kind rows of X4 (fp16, K-major): one 16-byte chunk per thread (128 threads)
        if (tid < 128) {
          const int t = tid & 31, cj = tid >> 5;  // a quarter-warp stores eight consecutive rows: 128 contiguous bytes
          float4 f0 = *reinterpret_cast<const float4*>(ti + t * kInvLd + cj * 8);
          float4 f1 = *reinterpret_cast<const float4*>(ti + t * kInvLd + cj * 8 + 4);
          if (t < 16 && cj >= 2) f0 = f1 = make_float4(0.f, 0.f, 0.f, 0.f);  // block above the diagonal (holds scratch)
          *reinterpret_cast<uint4*>(smem + kOffX4 + 2 * (t >> 3) * kRowGroup + (t & 7) * 16 + cj * kStride64) =
              make_uint4(pack_f16x2(f0.x, f0.y), pack_f16x2(f0.z, f0.w), pack_f16x2(f1.x, f1.y), pack_f16x2(f1.z, f1.w));
        }
      }
      FRWKV_PHASE(4)
      fence_proxy_async_smem();
      tcgen05_fence_before_sync();
      named_arrive(kBarInverse, kThreads);  // -> U = T W (the Rt-kind rows of this product are unused)
      FRWKV_PHASE(5)

      // while U is computed: first half of the next chunk's operand preparation (decay scan)
      if (more) bad |= !scan_decay(c + 1);
      bad |= !mbar_wait(bar_mma, mma_phase & 1);
      ++mma_phase;
      tcgen05_fence_after_sync();
      FRWKV_PHASE(6)
      rows_to_operand(kColU);
      // U has retired, and with it Q += [A_ak; A_rk] V and S += Kl^T V, the last readers of this chunk's V and Kl
      if (more) release_v();
      fence_proxy_async_smem();
      tcgen05_fence_before_sync();
      named_arrive(kBarU, kThreads);  // -> Q[Rt rows] += A_rb U ;  S += Bl^T U
      FRWKV_PHASE(7)

      // the tensor pipe is busy with Y and S: second half of the next chunk's operand preparation meanwhile, and the
      // next chunk's P = X1 X2^T right behind them
      if (more) {
        scale_operands(c + 1);
        fence_proxy_async_smem();
        named_arrive(kBarOperands, kThreads);
      }
      FRWKV_PHASE(1)
      bad |= !mbar_wait(bar_mma, mma_phase & 1);
      ++mma_phase;
      tcgen05_fence_after_sync();
      FRWKV_PHASE(8)
      // ---- y rows: the Rt-kind rows of Q (h = 1 of every thread) ----
      {
        uint32_t regs[16];
        tmem_ld_frag16(tmem_lane + kColQ + half * 32, regs);
        tmem_ld_wait();
        if (ftok < rows) {
          const size_t out = (static_cast<size_t>(row0 + ftok) * p.heads + head) * kHeadDim + half * 32 + 2 * fq;
          io_t* yp = static_cast<io_t*>(p.y) + out;
#pragma unroll
          for (int n = 0; n < 4; ++n) {
            const float y0 = __uint_as_float(regs[4 * n + 2]) * p.scale;
            const float y1 = __uint_as_float(regs[4 * n + 3]) * p.scale;
            alignas(4) io_t packed[2] = {from_f32<io_t>(y0), from_f32<io_t>(y1)};
            *reinterpret_cast<uint32_t*>(yp + 8 * n) = *reinterpret_cast<const uint32_t*>(packed);
            if (p.y_f32 != nullptr) *reinterpret_cast<float2*>(p.y_f32 + out + 8 * n) = make_float2(y0, y1);
          }
        }
      }
      bad |= !mbar_wait(bar_state, (chunks_done + c) & 1);
      tcgen05_fence_after_sync();
      // ---- state rows (all quadrants): S is final.  Next chunk: S -> S0 operand (fp16), g_L(next) S -> TMEM ----
      {
        uint32_t regs[16];
        tmem_ld_frag16(tmem_lane + kColS + half * 32, regs);
        tmem_ld_wait();
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = __uint_as_float(regs[i]);
        if (more) {
          release_bl();  // S += Bl^T U, the last reader of this chunk's Bl, has retired
          const float gl[2] = {chunk_decay_of(frow0), chunk_decay_of(frow0 + 8)};  // g_L of the next chunk
#pragma unroll
          for (int i = 0; i < 16; ++i) regs[i] = __float_as_uint(x[i] * gl[(i >> 1) & 1]);
          tmem_st_frag16(tmem_lane + kColS + half * 32, regs);
          store_frag_f16_split(kOffOp, kTileK64, half * 4, x);
          tmem_st_wait();
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float* dst = state_g + (frow0 + 8 * h) * kHeadDim + half * 32 + 2 * fq;
#pragma unroll
            for (int n = 0; n < 4; ++n)
              __stcs(reinterpret_cast<float2*>(dst + 8 * n), make_float2(x[4 * n + 2 * h], x[4 * n + 2 * h + 1]));
          }
        }
      }
      if (more) {
        fence_proxy_async_smem();
        tcgen05_fence_before_sync();
        named_arrive(kBarState, kThreads);  // S0 of the next chunk is in place -> Q, then the load after next
        if (c + 2 < n_chunks) tma_in_flight = true;
      }
      failed = named_sync_or(kBarCompute, kComputeThreads, bad);
      if (failed) {
        if (tid == 0) *abort_flag = 1u;
        if (more) named_arrive(kBarMasks, kThreads);  // the issuer warp's next hand-off
        break;
      }
      FRWKV_PHASE(9)
    }
    // queue mode: the state of this segment is in the pool slot (stored by all compute threads before the barrier
    // that ended the last chunk): publish it
    if (QUEUE && !failed && segments_done != nullptr && tid == 0) {
      __threadfence();
      const int done = segment + 1;
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(segments_done), "r"(done) : "memory");
    }
  } else {
    // =====================================================================================================
    // Issuer warp: lane 0 issues every TMA load and every MMA, in the order the results are needed (the tensor
    // pipe runs them first in, first out).  An issuing thread stalls while the MMA queue is full, at about the
    // rate the MMAs execute, so none of the compute warps issues anything.  The warp waits on named barriers
    // only and leaves when it finds `abort_flag` set after one of them.
    // =====================================================================================================
    for (int c = 0; c < n_chunks; ++c) {
      named_sync(kBarOperands, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, true, 4>(tmem + kColP, op_x1, op_x2, idesc_p, false);
#ifdef FRWKV_TEST_HOOKS
        if (c != p.skip_commit_chunk)
#endif
          mma_commit(bar_p);  // P: queued behind the previous chunk's Y and S products
      }
      __syncwarp();
      named_sync(kBarState, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<false, true, 4>(tmem + kColQ, op_x1h, op_rows, idesc_kmn, false);  // Q = X1 S0: under the P read-back
      }
      __syncwarp();
      named_sync(kBarMasks, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, false, 2>(tmem + kColQ, op_x3, op_v, idesc_kmn, true);
        mma_commit(bar_mma);  // Q complete (commits track every earlier MMA of the thread)
        // S += Kl^T V does not need U: it runs now, while the compute warps invert and the pipe would be idle, instead
        // of at the end of the chunk where the state products are waited for
        issue_gemm<true, false, 2>(tmem + kColS, op_kl, op_v, idesc_mnmn, true);
        // the next chunk's tokens, most of a chunk ahead of their use; issued here because nothing waits for it,
        // whereas the products above and below are on the compute warps' critical path
        if (c + 1 < n_chunks) issue_tma(c + 1);
      }
      __syncwarp();
      named_sync(kBarInverse, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<false, false, 2>(tmem + kColU, op_x4, op_rows, idesc_kmn, false);
        mma_commit(bar_mma);
      }
      __syncwarp();
      named_sync(kBarU, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<false, false, 2>(tmem + kColQ, op_x4, op_rows, idesc_kmn, true);
        mma_commit(bar_mma);  // Y is complete when this one arrives ...
        issue_gemm<false, false, 2>(tmem + kColS, op_bl, op_rows, idesc_mnmn, true);
        mma_commit(bar_state);  // ... and S when this one does: the y read-back overlaps the state MMA
      }
      __syncwarp();
    }
  }
  chunks_done += static_cast<uint32_t>(n_chunks);
  }  // task loop

  // every MMA of this CTA has retired before anybody frees its TMEM (matters after an abort only: otherwise the
  // compute warps have waited for the last state update of every task)
  if (!compute_warp && lane == 0) {
    mma_commit(bar_drain);
    mbar_wait(bar_drain, 0);
  }
  __syncwarp();

  if (failed) {
    if (tid == 0 && p.error_flag != nullptr) atomicOr(p.error_flag, kErrorWait);
    if (tma_in_flight) mbar_wait(bar_tma, tma_parity, 200000u);  // bounded drain of the load in flight
    // fail closed even for a caller that passed no error flag: this (sequence, head)'s output rows become NaN (its
    // state slot keeps the value it had before the call: the state is only written after the last chunk)
    if (compute_warp) {
      const float qnan = __int_as_float(0x7fffffff);
      for (long long i = tid; i < static_cast<long long>(len) * kHeadDim; i += kComputeThreads) {
        const size_t at = (static_cast<size_t>(t_begin + i / kHeadDim) * p.heads + head) * kHeadDim + i % kHeadDim;
        static_cast<io_t*>(p.y)[at] = from_f32<io_t>(qnan);
        if (p.y_f32 != nullptr) p.y_f32[at] = qnan;
      }
    }
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *decay_flag != 0u && p.error_flag != nullptr) atomicOr(p.error_flag, kErrorDecay);
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// The shared-memory attribute is set once per device and kernel instance, not on every call.
template <typename io_t, bool LOGITS, bool FUSED, bool QUEUE>
int prepare_kernel() {
  static bool done[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return check_launch("cudaGetDevice");
  if (!done[device]) {
    if (cudaFuncSetAttribute(wkv7_chunk32_tc_kernel<io_t, LOGITS, FUSED, QUEUE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes) != cudaSuccess)
      return check_launch("wkv7_chunk32_tc_kernel shared-memory attribute");
    done[device] = true;  // benign race: two threads may both set the same attribute
  }
  return FRWKV_OK;
}

template <typename io_t, bool FUSED, bool QUEUE>
int launch_typed32(const ChunkParams& p, const Maps& maps, bool logits, cudaStream_t stream) {
  const int rc = logits ? prepare_kernel<io_t, true, FUSED, QUEUE>() : prepare_kernel<io_t, false, FUSED, QUEUE>();
  if (rc != FRWKV_OK) return rc;
  auto kernel = logits ? wkv7_chunk32_tc_kernel<io_t, true, FUSED, QUEUE> : wkv7_chunk32_tc_kernel<io_t, false, FUSED, QUEUE>;
  long long ctas = static_cast<long long>(p.n_seq) * p.heads;
  if (ctas > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "wkv7_prefill: too many (sequence, head) pairs");
  if constexpr (QUEUE) {  // persistent CTAs, two per SM
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    ctas = 2LL * sms;
  }
  kernel<<<static_cast<unsigned>(ctas), kThreads, kSmemBytes, stream>>>(p, maps);
  return check_launch("wkv7_chunk32_tc_kernel");
}

}  // namespace

#ifdef FRWKV_TEST_HOOKS
namespace chunk {
int& test_skip_commit_chunk() {
  static int chunk_index = -1;
  return chunk_index;
}
}  // namespace chunk
#endif

int launch_chunk32_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                      float scale, const int32_t* order, int len_from, int32_t* error_flag, const void* const* gate,
                      void* queue, cudaStream_t stream) {
  const bool bf16 = io_dtype == FRWKV_IO_BF16;
  chunk::Maps maps;
  const int map_rc = chunk::make_maps(&maps, r, w, k, v, a, gate != nullptr ? a : b, total_tokens, heads, bf16, kChunk);
  if (map_rc != FRWKV_OK) return map_rc;
  chunk::ChunkParams p{cu, slots, status, pool, bias, y, y_f32, error_flag, n_seq, total_tokens, heads, scale, order,
                       len_from, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (queue != nullptr) {  // header, then one flag per stream
    p.queue = static_cast<chunk::QueueHeader*>(queue);
    p.queue_flags = reinterpret_cast<int*>(p.queue + 1);
  }
  if (gate != nullptr) {
    p.gate_kk = gate[0];
    p.gate_a0 = gate[1];
    p.gate_ka = gate[2];
  }
#ifdef FRWKV_TEST_HOOKS
  p.skip_commit_chunk = chunk::test_skip_commit_chunk();
#endif
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  const bool queued = queue != nullptr;
  if (gate != nullptr) {
    if (bf16) return queued ? launch_typed32<__nv_bfloat16, true, true>(p, maps, logits, stream)
                            : launch_typed32<__nv_bfloat16, true, false>(p, maps, logits, stream);
    return queued ? launch_typed32<__half, true, true>(p, maps, logits, stream)
                  : launch_typed32<__half, true, false>(p, maps, logits, stream);
  }
  if (bf16) return queued ? launch_typed32<__nv_bfloat16, false, true>(p, maps, logits, stream)
                          : launch_typed32<__nv_bfloat16, false, false>(p, maps, logits, stream);
  return queued ? launch_typed32<__half, false, true>(p, maps, logits, stream)
                : launch_typed32<__half, false, false>(p, maps, logits, stream);
}

}  // namespace frwkv

#ifdef FRWKV_TEST_HOOKS
// Test build only: the chunk whose P commit the next prefill launches leave out (-1 = none).
extern "C" void frwkv_sm100_test_skip_commit(int chunk_index) { frwkv::chunk::test_skip_commit_chunk() = chunk_index; }
#endif
