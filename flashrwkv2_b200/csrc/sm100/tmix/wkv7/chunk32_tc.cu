// WKV7 chunked prefill on tcgen05 tensor cores, 32-row chunks, two CTAs resident per SM.
//
// Same algebra, precision scheme and data movement as the 64-row kernel in chunk_tc.cu (see the
// header there); what changes is the footprint.  With 32-row chunks the stacked operands
// [At; Rt], [Bt; Kt], [A_ak; A_rk] and [T; A_rb] have 64 rows, so every product is a natural
// M=64 MMA (no padding rows), one CTA needs 112 KB of shared memory and 256 TMEM columns, and
// two CTAs of 288 threads (96 registers) share an SM: while one waits for its MMAs or a
// barrier the other one's CUDA-core phases run.  A 64-row accumulator of an M=64 MMA puts row i
// in TMEM lane 32*(i/16) + i%16, i.e. every warp quadrant holds 16 rows in its lanes 0..15; the
// read-backs use the 16x256b fragment shape, which spreads those 16 rows over all 32 threads.
// Eight warps compute; a ninth issues every MMA and TMA load (see the loop below).  Inside the stacked operands the
// two kinds of rows alternate in groups of eight (token t: 16*(t/8) + t%8 and eight further), so that every
// thread's fragment holds one row of each kind and all eight warps share every read-back.
//
// Per chunk of L <= 32 rows (g_t = inclusive cumulative retention inside the chunk):
//     P  = [At; Rt] [Bt; Kt]^T  (64x64) -> A_ab, A_ak (strictly lower), A_rb, A_rk (lower), 32x32 each
//     Q  = [At; Rt] S0 + [A_ak; A_rk] V      (rows 0..31 = W, rows 32..63 = part of Y)
//     U  = (I - A_ab)^-1 W ;  Y = scale (Q[32..] + A_rb U) ;  S <- diag(g_L)(S0 + Bt^T U + Kt^T V)
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
constexpr uint32_t kTileK64 = 8 * kStride64;  // 64 rows x 64 columns, one bf16 part: 8320
constexpr uint32_t kTileK32 = 4 * kStride64;  // 64 rows x 32 columns, one bf16 part: 4160
constexpr uint32_t kStride32 = 4 * 128 + 16;  // stride between 16-byte chunks of a 32-row tile (padded)
constexpr uint32_t kTileV = 8 * kStride32;    // 32 rows x 64 columns, one bf16 part: 4224

constexpr uint32_t kRawTile = kChunk * 128;           // one [32][64] 16-bit tile as TMA writes it
constexpr uint32_t kOffRaw = 0;                       // r, w, k, v, a, b
constexpr uint32_t kOffX1 = kOffRaw + 6 * kRawTile;   // [At; Rt] hi, lo (64 x 64)
constexpr uint32_t kOffX2 = kOffX1 + 2 * kTileK64;    // [Bt; Kt] hi, lo (64 x 64)
constexpr uint32_t kOffX3 = kOffX2 + 2 * kTileK64;    // [A_ak; A_rk] hi, lo (64 x 32)
constexpr uint32_t kOffX4 = kOffX3 + 2 * kTileK32;    // [T; A_rb] hi, lo (64 x 32)
constexpr uint32_t kOffOp = kOffX4 + 2 * kTileK32;    // S0 (64 rows) / W / U (32 rows) operand hi, lo
constexpr uint32_t kOffV = kOffOp + 2 * kTileK64;     // V operand hi, lo (32 rows x 64)
constexpr uint32_t kOffMisc = kOffV + 2 * kTileV;     // gamma_L[2][64], group sums [8][64], barriers
constexpr uint32_t kMiscBytes = 2 * 64 * 4 + kWarps * 64 * 4 + 64;
// fp32 scratch of the 32x32 inverse.  It has its own area: the staging area must stay free for the next chunk's
// load, which is issued a whole chunk ahead.  The 16x16 block product of level 1 lives in T's upper-right block,
// which is zero and never stored.
constexpr int kInvLd = 36;
constexpr uint32_t kOffAb = kOffMisc + kMiscBytes;     // A_ab [32][36]
constexpr uint32_t kOffTi = kOffAb + 32 * kInvLd * 4;  // T    [32][36]
constexpr int kMbLd = kInvLd;
constexpr uint32_t kOffMb = kOffTi + 16 * 4;           // block product [16][16] at T[0..15][16..31]
constexpr uint32_t kSmemBytes = kOffTi + 32 * kInvLd * 4 + 128;
static_assert(2 * (kSmemBytes + 1024) <= 227 * 1024, "two CTAs must fit in one SM's shared memory");

// ---- TMEM map (columns) --------------------------------------------------------------------
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColP = 0, kColQ = 64, kColU = 128, kColS = 192;

template <typename io_t, bool LOGITS>
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
  const int rank = blockIdx.x / p.heads, head = blockIdx.x % p.heads;
  if (rank >= p.n_seq) return;
  const int seq = p.order != nullptr ? p.order[rank] : rank;
  if (seq >= active || seq < 0 || seq >= p.n_seq) return;
  const int t_begin = p.cu[seq], len = p.cu[seq + 1] - t_begin;
  if (len <= 0 || len < p.len_from) return;
  const int n_chunks = (len + kChunk - 1) / kChunk;
  const int slot = p.slots[seq];

  float* gamma_l = reinterpret_cast<float*>(smem + kOffMisc);
  float* group_sum = gamma_l + 2 * 64;  // [8][64] log2-decay sums of each 4-row group (gamma_l: [2][64] by chunk parity)
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(group_sum + kWarps * 64);
  uint64_t* bar_mma = bar_tma + 1;
  uint64_t* bar_state = bar_tma + 2;  // its own barrier: two commits may not complete two phases of one
  uint64_t* bar_drain = bar_tma + 3;  // the issuer warp's last commit: every MMA has retired before TMEM is freed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;  // set by the compute warps when a bounded wait gave up
  const uint32_t sbase = smem_u32(smem);

  if (tid == 0) {
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    mbar_init(bar_state, 1);
    mbar_init(bar_drain, 1);
    mbar_fence_init();
    *abort_flag = 0u;
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

  auto issue_tma = [&](int chunk_index) {  // one thread
    const int row = t_begin + chunk_index * kChunk;
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
  uint32_t tma_parity = 0;

  // 32 fp32 values (columns 32*half ..) of accumulator row `row` -> four 16-byte column chunks of the
  // row-operand tile (hi/lo, rows = contraction index, MN-major)
  auto store_operand_row = [&](int row, const uint32_t (&regs)[32]) {
    uint8_t* op = smem + kOffOp + (row & 7) * 16 + (row >> 3) * kRowGroup;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 hi, lo;
      split8(reinterpret_cast<const float*>(regs) + 8 * j, hi, lo);
      *reinterpret_cast<uint4*>(op + (half * 4 + j) * kStride64) = hi;
      *reinterpret_cast<uint4*>(op + kTileK64 + (half * 4 + j) * kStride64) = lo;
    }
  };

  // Fragment view of an accumulator block (tmem_ld_frag16): this thread holds rows frow0 and frow0 + 8 of its
  // quadrant and, of the 32 columns at 32*half, the pairs 8n + 2*fq + {0,1}, n = 0..3.
  const int fq = lane & 3;
  const int frow0 = quad * 16 + (lane >> 2);
  // fragment -> hi/lo operand tile at `tile` (rows = accumulator rows, 16-byte column chunks from `chunk0` on):
  // one 4-byte store per pair and part; the 32 lanes of a store cover 128 contiguous bytes
  auto store_operand_frag = [&](uint32_t tile, uint32_t lo_off, int chunk0, const float (&x)[16]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = frow0 + 8 * h;
      uint8_t* dst = smem + tile + (row >> 3) * kRowGroup + (row & 7) * 16 + fq * 4;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        uint32_t hi, lo;
        split2(x[4 * n + 2 * h], x[4 * n + 2 * h + 1], hi, lo);
        *reinterpret_cast<uint32_t*>(dst + (chunk0 + n) * kStride64) = hi;
        *reinterpret_cast<uint32_t*>(dst + lo_off + (chunk0 + n) * kStride64) = lo;
      }
    }
  };

  // ---- initial state: global -> TMEM (fp32) and -> S0 operand tile ----------------------------
  float* state_g = p.pool + (static_cast<size_t>(slot) * p.heads + head) * (kHeadDim * kHeadDim);
  const bool compute_warp = warp < kWarps;
  if (compute_warp) {
    uint32_t regs[32];
    if (row_lane) {
      const float4* src = reinterpret_cast<const float4*>(state_g + arow * kHeadDim + half * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 f = __ldcs(src + i);
        regs[4 * i] = __float_as_uint(f.x);
        regs[4 * i + 1] = __float_as_uint(f.y);
        regs[4 * i + 2] = __float_as_uint(f.z);
        regs[4 * i + 3] = __float_as_uint(f.w);
      }
      store_operand_row(arow, regs);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) regs[i] = 0u;
    }
    tmem_st32(tmem_lane + kColS + half * 32, regs);
    tmem_st_wait();
  }

  constexpr uint32_t idesc_kk = instr_desc_f16(64, 64, kMajorK, kMajorK);
  constexpr uint32_t idesc_kmn = instr_desc_f16(64, 64, kMajorK, kMajorMN);
  constexpr uint32_t idesc_mnmn = instr_desc_f16(64, 64, kMajorMN, kMajorMN);
  constexpr bool kVExact = std::is_same<io_t, __nv_bfloat16>::value;
  constexpr uint32_t v_lo_off = kVExact ? 0u : kTileV;

  // operand descriptors (fixed for the whole kernel); K-major tiles: chunk stride kStride64, row groups 128 B
  const Operand op_x1 = make_operand(sbase + kOffX1, kTileK64, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x2 = make_operand(sbase + kOffX2, kTileK64, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x3 = make_operand(sbase + kOffX3, kTileK32, 2 * kStride64, kStride64, kRowGroup);
  const Operand op_x4 = make_operand(sbase + kOffX4, kTileK32, 2 * kStride64, kStride64, kRowGroup);
  // MN-major tiles (rows = contraction index): row groups 128 B apart, 16-byte column chunks at the tile's stride
  const Operand op_rows = make_operand(sbase + kOffOp, kTileK64, 2 * kRowGroup, kRowGroup, kStride64);
  const Operand op_v = make_operand(sbase + kOffV, v_lo_off, 2 * kRowGroup, kRowGroup, kStride32);
  // [Bt; Kt] read MN-major: M = key channel, contraction = tile row (Bt rows 0..31, Kt rows 32..63)
  const Operand op_bt = make_operand(sbase + kOffX2, kTileK64, 2 * kRowGroup, kRowGroup, kStride64);
  const Operand op_kt = make_operand(sbase + kOffX2 + 4 * kRowGroup, kTileK64, 2 * kRowGroup, kRowGroup, kStride64);

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
    for (int n = 0; n < 4; ++n) {
      uint32_t hi, lo;
      split2(__uint_as_float(regs[4 * n]), __uint_as_float(regs[4 * n + 1]), hi, lo);
      *reinterpret_cast<uint32_t*>(dst + (half * 4 + n) * kStride64) = hi;
      *reinterpret_cast<uint32_t*>(dst + kTileK64 + (half * 4 + n) * kStride64) = lo;
    }
  };

  bool failed = false;
  bool bad = false;  // this thread saw a bounded wait give up; turned into `failed` at the next CTA barrier
#ifdef FRWKV_CHUNK_TIMING
  long long phase_t0 = clock64();
#endif
  const io_t* bias_g = LOGITS && p.bias != nullptr ? static_cast<const io_t*>(p.bias) + head * kHeadDim : nullptr;

  // ---- operand preparation of one chunk (decay products, scaled operands) -----------------------------------
  // It depends on the tokens only, so it runs for chunk c+1 while the tensor pipe works on chunk c's last
  // products.  [At; Rt] goes straight to its tile (free since Q was read); [Bt; Kt] and V, whose tiles the state
  // MMAs of chunk c still read, stay in these registers until release_operands().
  uint32_t held_x2[16];  // per row of this thread: Bt hi, Bt lo, Kt hi, Kt lo
  uint4 held_v_hi, held_v_lo = make_uint4(0u, 0u, 0u, 0u);
  float2 held_lg[kChunk / kWarps];  // log2 of the inclusive decay product of this thread's rows, scan -> scaling
  float2 held_off = make_float2(0.f, 0.f);  // ... and of the rows before them
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
    float2 run = make_float2(0.f, 0.f);
    float2 cum[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int t = tg * kRowsPerWarp + i;
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
      run.x += l.x;
      run.y += l.y;
      cum[i] = run;
    }
    reinterpret_cast<float2*>(group_sum + tg * 64)[kp] = run;
    // V operand: rows = token, 64 contiguous value columns (MN-major); bf16 is copied, fp16 is split
    {
      const uint8_t* raw_v = smem + kOffRaw + 3 * kRawTile;
      const int sr = tid >> 3, vc = tid & 7;  // 256 chunks of 8 values
      uint4 q = *reinterpret_cast<const uint4*>(raw_v + sr * 128 + vc * 16);
      if (sr >= rows) q = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (kVExact) {
        held_v_hi = q;
      } else {
        float x[8];
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack2<io_t>(words[e]);
          x[2 * e] = f.x;
          x[2 * e + 1] = f.y;
        }
        split8(x, held_v_hi, held_v_lo);
      }
    }
    named_sync(kBarCompute, kComputeThreads);
    float2 off = make_float2(0.f, 0.f);
#pragma unroll
    for (int g = 0; g < kWarps - 1; ++g) {  // loads issued together; only the adds are a chain
      const float2 sgrp = reinterpret_cast<const float2*>(group_sum + g * 64)[kp];
      if (g < tg) {
        off.x += sgrp.x;
        off.y += sgrp.y;
      }
    }
    held_off = off;
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) held_lg[i] = make_float2(off.x + cum[i].x, off.y + cum[i].y);
    return ok;
  };
  auto scale_operands = [&](int chunk, float* gamma_dst) {  // second half: no barrier inside
    const int rows = min(kChunk, len - chunk * kChunk);
    constexpr int kRowsPerWarp = kChunk / kWarps;
    const int kp = lane, tg = warp;
    const uint32_t* raw_r = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 0 * kRawTile);
    const uint32_t* raw_k = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 2 * kRawTile);
    const uint32_t* raw_a = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 4 * kRawTile);
    const uint32_t* raw_b = reinterpret_cast<const uint32_t*>(smem + kOffRaw + 5 * kRawTile);
    float2 g_prev = make_float2(fast_exp2(held_off.x), fast_exp2(held_off.y));
    uint8_t* x1 = smem + kOffX1 + (kp >> 2) * kStride64 + (kp & 3) * 4;
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const int t = tg * kRowsPerWarp + i;
      const bool live = t < rows;
      const float2 lg = held_lg[i];
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
      const uint32_t row_a = 2 * (t >> 3) * kRowGroup + (t & 7) * 16;  // At row of token t: 16*(t/8) + t%8
      const uint32_t row_r = row_a + kRowGroup;                        // Rt row: eight further
      uint32_t h, l;
      split2(a2.x * gx.x, a2.y * gx.y, h, l);
      *reinterpret_cast<uint32_t*>(x1 + row_a) = h;
      *reinterpret_cast<uint32_t*>(x1 + kTileK64 + row_a) = l;
      split2(r2.x * g.x, r2.y * g.y, h, l);
      *reinterpret_cast<uint32_t*>(x1 + row_r) = h;
      *reinterpret_cast<uint32_t*>(x1 + kTileK64 + row_r) = l;
      split2(b2.x * gi.x, b2.y * gi.y, held_x2[4 * i], held_x2[4 * i + 1]);
      split2(k2.x * gi.x, k2.y * gi.y, held_x2[4 * i + 2], held_x2[4 * i + 3]);
      if (t == kChunk - 1) reinterpret_cast<float2*>(gamma_dst)[kp] = g;
    }
  };
  auto release_operands = [&]() {  // [Bt; Kt] and V of the prepared chunk: registers -> tiles
    const int kp = lane, tg = warp;
    uint8_t* x2 = smem + kOffX2 + (kp >> 2) * kStride64 + (kp & 3) * 4;
#pragma unroll
    for (int i = 0; i < kChunk / kWarps; ++i) {
      const int t = tg * (kChunk / kWarps) + i;
      const uint32_t row_lo = (t >> 3) * kRowGroup + (t & 7) * 16;
      const uint32_t row_hi = ((t + 32) >> 3) * kRowGroup + (t & 7) * 16;
      *reinterpret_cast<uint32_t*>(x2 + row_lo) = held_x2[4 * i];
      *reinterpret_cast<uint32_t*>(x2 + kTileK64 + row_lo) = held_x2[4 * i + 1];
      *reinterpret_cast<uint32_t*>(x2 + row_hi) = held_x2[4 * i + 2];
      *reinterpret_cast<uint32_t*>(x2 + kTileK64 + row_hi) = held_x2[4 * i + 3];
    }
    const int sr = tid >> 3, vc = tid & 7;
    uint8_t* dst = smem + kOffV + vc * kStride32 + (sr & 7) * 16 + (sr >> 3) * kRowGroup;
    *reinterpret_cast<uint4*>(dst) = held_v_hi;
    if constexpr (!kVExact) *reinterpret_cast<uint4*>(dst + kTileV) = held_v_lo;
  };

  uint32_t mma_phase = 0;  // completed phases of bar_mma, counted the same way by every compute thread

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
    scale_operands(0, gamma_l);
    release_operands();
    fence_proxy_async_smem();
    tcgen05_fence_before_sync();
    failed = named_sync_or(kBarCompute, kComputeThreads, bad);
    if (failed && tid == 0) *abort_flag = 1u;
    named_arrive(kBarOperands, kThreads);  // [At; Rt], [Bt; Kt], V of chunk 0 are in place -> P
    if (!failed) {
      named_arrive(kBarState, kThreads);   // ... and so is S0 -> Q, then the next chunk's load
      if (n_chunks > 1) tma_in_flight = true;
    }

    for (int c = 0; c < n_chunks && !failed; ++c) {
      const int rows = min(kChunk, len - c * kChunk);
      const int row0 = t_begin + c * kChunk;
      FRWKV_PHASE(0)

      // ================= P = X1 X2^T (the issuer warp also starts Q = X1 S0, which runs under the read-back) ====
      bad |= !mbar_wait(bar_mma, mma_phase & 1);
      ++mma_phase;
      tcgen05_fence_after_sync();
      FRWKV_PHASE(2)
      // ================= read P: masks, A_ab -> fp32 scratch, others -> operand tiles =================
      {
        // this thread's rows: h = 0 the At row of token ftok (products with Bt: A_ab, with Kt: A_ak; strictly lower),
        // h = 1 its Rt row (A_rb, A_rk; lower); columns 32*half..: half 0 = products with Bt, half 1 = with Kt
        uint32_t regs[16];
        tmem_ld_frag16(tmem_lane + kColP + half * 32, regs);
        tmem_ld_wait();
        float vals[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int limit = ftok + h;  // keep columns s < limit
#pragma unroll
          for (int n = 0; n < 4; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e)
              vals[4 * n + 2 * h + e] = 8 * n + 2 * fq + e < limit ? __uint_as_float(regs[4 * n + 2 * h + e]) : 0.0f;
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
            uint32_t hi, lo;
            split2(vals[4 * n + 2], vals[4 * n + 3], hi, lo);
            *reinterpret_cast<uint32_t*>(rb + n * kStride64) = hi;
            *reinterpret_cast<uint32_t*>(rb + kTileK32 + n * kStride64) = lo;
          }
        } else {
          store_operand_frag(kOffX3, kTileK32, 0, vals);  // A_ak and A_rk rows, in accumulator order
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
        // T -> the At-kind rows of X4 (hi/lo, K-major): one 16-byte chunk per thread (128 threads)
        if (tid < 128) {
          const int t = tid & 31, cj = tid >> 5;  // a quarter-warp stores eight consecutive rows: 128 contiguous bytes
          float4 f0 = *reinterpret_cast<const float4*>(ti + t * kInvLd + cj * 8);
          float4 f1 = *reinterpret_cast<const float4*>(ti + t * kInvLd + cj * 8 + 4);
          if (t < 16 && cj >= 2) f0 = f1 = make_float4(0.f, 0.f, 0.f, 0.f);  // block above the diagonal (holds scratch)
          const float x[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
          uint4 hi, lo;
          split8(x, hi, lo);
          uint8_t* dst = smem + kOffX4 + 2 * (t >> 3) * kRowGroup + (t & 7) * 16 + cj * kStride64;  // At-kind row of token t
          *reinterpret_cast<uint4*>(dst) = hi;
          *reinterpret_cast<uint4*>(dst + kTileK32) = lo;
        }
      }
      FRWKV_PHASE(4)
      fence_proxy_async_smem();
      tcgen05_fence_before_sync();
      named_arrive(kBarInverse, kThreads);  // -> U = T W (rows 32..63 of this product are unused)
      FRWKV_PHASE(5)

      // while U is computed: first half of the next chunk's operand preparation (decay scan)
      if (c + 1 < n_chunks) bad |= !scan_decay(c + 1);
      bad |= !mbar_wait(bar_mma, mma_phase & 1);
      ++mma_phase;
      tcgen05_fence_after_sync();
      FRWKV_PHASE(6)
      rows_to_operand(kColU);
      fence_proxy_async_smem();
      tcgen05_fence_before_sync();
      named_arrive(kBarU, kThreads);  // -> Q[32..] += A_rb U ;  S += Bt^T U + Kt^T V
      FRWKV_PHASE(7)

      // the tensor pipe is busy with Y and S: second half of the next chunk's operand preparation meanwhile
      if (c + 1 < n_chunks) scale_operands(c + 1, gamma_l + ((c + 1) & 1) * 64);
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
      bad |= !mbar_wait(bar_state, c & 1);
      tcgen05_fence_after_sync();
      // This thread has seen the state MMAs finish: their [Bt; Kt] and V tiles take the next chunk's values, and
      // the next chunk's P = X1 X2^T, which does not need the state, starts while the state is read back.
      if (c + 1 < n_chunks) {
        release_operands();
        fence_proxy_async_smem();
        named_arrive(kBarOperands, kThreads);
      }
      // ---- state rows (all quadrants): S <- diag(g_L) S; keep in TMEM, refresh the S0 operand (or store) ----
      {
        uint32_t regs[16];
        tmem_ld_frag16(tmem_lane + kColS + half * 32, regs);
        tmem_ld_wait();
        const float* gamma_c = gamma_l + (c & 1) * 64;
        const float gl[2] = {gamma_c[frow0], gamma_c[frow0 + 8]};
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          x[i] = __uint_as_float(regs[i]) * gl[(i >> 1) & 1];
          regs[i] = __float_as_uint(x[i]);
        }
        if (c + 1 < n_chunks) {
          tmem_st_frag16(tmem_lane + kColS + half * 32, regs);
          store_operand_frag(kOffOp, kTileK64, half * 4, x);
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
      if (c + 1 < n_chunks) {
        fence_proxy_async_smem();
        tcgen05_fence_before_sync();
        named_arrive(kBarState, kThreads);  // S0 of the next chunk is in place -> Q, then the load after next
        if (c + 2 < n_chunks) tma_in_flight = true;
      }
      failed = named_sync_or(kBarCompute, kComputeThreads, bad);
      if (failed) {
        if (tid == 0) *abort_flag = 1u;
        if (c + 1 < n_chunks) named_arrive(kBarMasks, kThreads);  // the issuer warp's next hand-off
        break;
      }
      FRWKV_PHASE(9)
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
        issue_gemm<true, true, 4>(tmem + kColP, op_x1, op_x2, idesc_kk, false);
        if (c != p.skip_commit_chunk) mma_commit(bar_mma);  // P: runs while the previous chunk's state is read back
      }
      __syncwarp();
      named_sync(kBarState, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, true, 4>(tmem + kColQ, op_x1, op_rows, idesc_kmn, false);  // Q = X1 S0: under the P read-back
      }
      __syncwarp();
      named_sync(kBarMasks, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, !kVExact, 2>(tmem + kColQ, op_x3, op_v, idesc_kmn, true);
        mma_commit(bar_mma);  // Q complete (commits track every earlier MMA of the thread)
        // S += Kt^T V does not need U: it runs now, while the compute warps invert and the pipe would be idle, instead
        // of at the end of the chunk where the state products are waited for
        issue_gemm<true, !kVExact, 2>(tmem + kColS, op_kt, op_v, idesc_mnmn, true);
        // the next chunk's tokens, most of a chunk ahead of their use; issued here because nothing waits for it,
        // whereas the products above and below are on the compute warps' critical path
        if (c + 1 < n_chunks) issue_tma(c + 1);
      }
      __syncwarp();
      named_sync(kBarInverse, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, true, 2>(tmem + kColU, op_x4, op_rows, idesc_kmn, false);
        mma_commit(bar_mma);
      }
      __syncwarp();
      named_sync(kBarU, kThreads);
      if (*abort_flag != 0u) break;
      if (lane == 0) {
        tcgen05_fence_after_sync();
        issue_gemm<true, true, 2>(tmem + kColQ, op_x4, op_rows, idesc_kmn, true);
        mma_commit(bar_mma);  // Y is complete when this one arrives ...
        issue_gemm<true, true, 2>(tmem + kColS, op_bt, op_rows, idesc_mnmn, true);
        mma_commit(bar_state);  // ... and S when this one does: the y read-back overlaps the state MMAs
      }
      __syncwarp();
    }
    // every MMA of this CTA has retired before anybody frees its TMEM (matters after an abort only: otherwise the
    // compute warps have waited for the last state update)
    if (lane == 0) {
      mma_commit(bar_drain);
      mbar_wait(bar_drain, 0);
    }
    __syncwarp();
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
int launch_typed32(const ChunkParams& p, const Maps& maps, bool logits, cudaStream_t stream) {
  auto kernel = logits ? wkv7_chunk32_tc_kernel<io_t, true> : wkv7_chunk32_tc_kernel<io_t, false>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return check_launch("wkv7_chunk32_tc_kernel shared-memory attribute");
  const long long ctas = static_cast<long long>(p.n_seq) * p.heads;
  if (ctas > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "wkv7_prefill: too many (sequence, head) pairs");
  kernel<<<static_cast<unsigned>(ctas), kThreads, kSmemBytes, stream>>>(p, maps);
  return check_launch("wkv7_chunk32_tc_kernel");
}

}  // namespace

int launch_chunk32_tc(const int32_t* cu, const int32_t* slots, const int32_t* status, float* pool, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y_f32, int n_seq, int total_tokens, int heads, int io_dtype, int decay_mode,
                      float scale, const int32_t* order, int len_from, int32_t* error_flag, cudaStream_t stream) {
  const bool bf16 = io_dtype == FRWKV_IO_BF16;
  chunk::Maps maps;
  const int map_rc = chunk::make_maps(&maps, r, w, k, v, a, b, total_tokens, heads, bf16, kChunk);
  if (map_rc != FRWKV_OK) return map_rc;
  chunk::ChunkParams p{cu, slots, status, pool, bias, y, y_f32, error_flag, n_seq, total_tokens, heads, scale, order, len_from,
                       chunk::test_skip_commit_chunk()};
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  if (bf16) return launch_typed32<__nv_bfloat16>(p, maps, logits, stream);
  return launch_typed32<__half>(p, maps, logits, stream);
}

}  // namespace frwkv
