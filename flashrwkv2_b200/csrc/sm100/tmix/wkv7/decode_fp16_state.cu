// One-token decode step of the fp16-state contract, fed by TMA through a shared-memory ring.
//
// The register-streaming kernel (recurrent_stream.cu) keeps as many bytes in flight as its warps hold in
// registers; with an fp16 state a warp carries 4 KB, which leaves it latency-bound at about 0.58 of the HBM roof.
// Here the bytes in flight live in shared memory instead: persistent CTAs, one producer thread that issues, for
// every (sequence, head) item, one tiled TMA load of the 64 x 64 fp16 state (8 KB) and six 128-byte bulk copies of
// the token rows into a ring of kStages slots, and four consumer warps that take an item out of the ring into
// registers, hand the slot back at once and do the arithmetic while the loads of the following items are in the
// air.  Completion is tracked with mbarriers (full: transaction bytes; empty: one arrival per consumer warp).
//
// Layout in a slot.  A consumer warp owns 16 value columns and all 64 key rows; lane (j, c), c = lane % 4,
// holds key rows 8j .. 8j+7 and columns 4c .. 4c+3 of the warp's 16, so the token rows it needs are 16 contiguous
// bytes and both reductions over the key index end with three shuffles.  For the state reads to be free of bank
// conflicts, the rows that the eight j of one instruction touch (8j + i) must fall into different 16-byte column
// slots.  The tensor map therefore views an item as [i][j][64 columns] with the row strides swapped (j: 1024 B,
// i: 128 B): TMA then writes row 8j + i to line j + 8i of the slot, and its 128-byte swizzle XORs the 16-byte
// chunk index with line % 8 = j.
//
// Arithmetic and rounding points are those of recurrent_stream.cu's fp16-state path (reference:
// csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:244-340, tests/tmix/wkv7/test.py:88-149 of
// rwkv-rs/FlashRWKV2); the two kernels sum the key index in a different order, so they agree to a few fp16 units
// in the last place, not bit for bit.
#include <cstdlib>
#include "../../common.cuh"
#include "../../tcgen05.cuh"

#include <cstring>
#include <mutex>

namespace frwkv {
namespace {

using namespace tc;

constexpr int kStages = 4;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kStateBytes = 64 * 64 * 2;
constexpr uint32_t kRowBytes = 64 * 2;
constexpr uint32_t kSlotBytes = kStateBytes + 1024;  // state, six token rows, meta; keeps every state 1024-aligned
constexpr uint32_t kOffTokens = kStateBytes;          // r, w, k, v, a, b: 128 B each
constexpr uint32_t kOffMeta = kStateBytes + 6 * kRowBytes;
constexpr uint32_t kSmemBytes = kStages * kSlotBytes + 2 * kStages * 8 + 1024;
constexpr int kCtasPerSm = 4;

struct DecodeParams {
  const int* cu;
  const int* slots;
  const int* status;
  const int* elapsed;
  __half* pool;
  const __half *r, *w, *k, *v, *a, *b, *bias;
  __half* y;
  int* error_flag;
  int n_seq, total_tokens, heads;
  float scale;
};

__device__ __forceinline__ float dither_of(int phase) {
  const uint32_t bits = 2654435769u * static_cast<uint32_t>(phase);
  return 4.547473508864641e-13f * static_cast<float>(static_cast<int32_t>(bits));
}
__device__ __forceinline__ float to_half_and_back(float x) { return __half2float(__float2half_rn(x)); }

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(smem_u32(bar))
      : "memory");
}
// untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <bool LOGITS>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
wkv7_decode_fp16_state_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap state_map) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long n_items = static_cast<long long>(p.n_seq) * p.heads;

  // Programmatic dependent launch (see the launcher): this grid may be scheduled while the previous kernel of the
  // stream drains, but nothing is read before that kernel has completed.  Without the launch attribute both
  // instructions do nothing.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (p.status != nullptr && p.status[0] != 0) {
    const float qnan = __int_as_float(0x7fffffff);
    const long long elements = static_cast<long long>(p.total_tokens) * p.heads * kHeadDim;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + tid; i < elements;
         i += static_cast<long long>(gridDim.x) * kThreads)
      p.y[i] = __float2half_rn(qnan);
    return;
  }
  const int active = p.status != nullptr ? p.status[2] : p.n_seq;

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kSlotBytes);
  uint64_t* empty_bar = full_bar + kStages;
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, kConsumerWarps);
    }
    mbar_fence_init();
    tma_prefetch_descriptor(&state_map);
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ---- producer warp ----
    // The metadata of an item is a chain of dependent global loads (cu -> slot -> elapsed counter); done one item
    // at a time it would cost the producer two memory latencies per item.  The 32 lanes fetch the metadata of the
    // next 32 items of this CTA at once; lane 0 then walks them, waits for each ring slot and issues the copies.
    int it = 0;
    bool ok = true;
    for (long long base = blockIdx.x; base < n_items && ok; base += 32LL * gridDim.x) {
      const long long mine_item = base + static_cast<long long>(lane) * gridDim.x;
      int4 mine = make_int4(0, 0, 0, 0);
      int mine_head = 0;
      if (mine_item < n_items) {
        const unsigned item32 = static_cast<unsigned>(mine_item);  // the launcher checks that items fit 32 bits
        const int seq = static_cast<int>(item32 / static_cast<unsigned>(p.heads));
        mine_head = static_cast<int>(item32 % static_cast<unsigned>(p.heads));
        if (seq < active) {
          const int t = p.cu[seq], len = p.cu[seq + 1] - t, slot = p.slots[seq];
          if (len == 1) mine = make_int4(mine_head + 1, t, slot, p.elapsed[slot]);  // .x = head + 1; 0 = skip
        }
      }
      for (int l = 0; l < 32; ++l) {
        if (base + static_cast<long long>(l) * gridDim.x >= n_items) break;  // uniform across the warp
        int4 meta;
        meta.x = __shfl_sync(0xffffffffu, mine.x, l);
        meta.y = __shfl_sync(0xffffffffu, mine.y, l);
        meta.z = __shfl_sync(0xffffffffu, mine.z, l);
        meta.w = __shfl_sync(0xffffffffu, mine.w, l);
        const int head = __shfl_sync(0xffffffffu, mine_head, l);
        if (lane == 0) {
          const int stage = it % kStages;
          if (it >= kStages && !mbar_wait(empty_bar + stage, ((it / kStages) & 1) ^ 1)) {
            if (p.error_flag != nullptr) atomicOr(p.error_flag, 1);
            ok = false;  // the consumers' bounded waits run out in turn and report as well
          } else {
            uint8_t* slot_mem = smem + stage * kSlotBytes;
            *reinterpret_cast<int4*>(slot_mem + kOffMeta) = meta;
            if (meta.x != 0) {
              mbar_expect_tx(full_bar + stage, kStateBytes + 6 * kRowBytes);
              tma_load_4d(slot_mem, &state_map, full_bar + stage, 0, 0, 0, meta.z * p.heads + head);
              const size_t row = (static_cast<size_t>(meta.y) * p.heads + head) * kHeadDim;
              const __half* rows[6] = {p.r + row, p.w + row, p.k + row, p.v + row, p.a + row, p.b + row};
#pragma unroll
              for (int n = 0; n < 6; ++n)
                bulk_load(slot_mem + kOffTokens + n * kRowBytes, rows[n], kRowBytes, full_bar + stage);
            } else {
              mbar_arrive(full_bar + stage);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        ++it;
      }
    }
    return;
  }

  // ---- consumers ----
  // j = row group of this lane.  A 64-bit shared-memory access is served half a warp at a time, so the four row
  // groups of a half-warp must differ in more than the lowest bit for their swizzled chunks to be distinct:
  // lanes 0..15 take the even groups, lanes 16..31 the odd ones.
  const int c = lane & 3;
  const int j = (((lane >> 2) & 3) << 1) | (lane >> 4);
  const int col = warp * 16 + c * 4;          // first of this lane's four value columns
  const int chunk = col >> 3;                  // 16-byte chunk of a state line that holds them
  const uint32_t in_chunk = (col & 7) * 2;     // byte offset inside the chunk
  int it = 0;
  for (long long item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
    const int stage = it % kStages;
    const uint8_t* slot_mem = smem + stage * kSlotBytes;
    if (!mbar_wait(full_bar + stage, (it / kStages) & 1)) {
      if (lane == 0 && p.error_flag != nullptr) atomicOr(p.error_flag, 1);
      break;
    }
    const int4 meta = *reinterpret_cast<const int4*>(slot_mem + kOffMeta);
    if (meta.x == 0) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + stage);
      continue;
    }
    const int head = meta.x - 1;
    // state rows 8j + i: line j + 8i of the slot, chunk index swizzled with the line's low bits (= j).  Values
    // are kept as pairs: the arithmetic below runs on the packed fp32x2 FMA of sm_100 (two lanes per instruction).
    float2 S01[8], S23[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint2 q = *reinterpret_cast<const uint2*>(slot_mem + (j + 8 * i) * 128 + ((chunk ^ j) << 4) + in_chunk);
      S01[i] = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
      S23[i] = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
    }
    const uint8_t* tok = slot_mem + kOffTokens;
    const uint4 r8 = *reinterpret_cast<const uint4*>(tok + 0 * kRowBytes + j * 16);
    const uint4 k8 = *reinterpret_cast<const uint4*>(tok + 2 * kRowBytes + j * 16);
    const uint4 a8 = *reinterpret_cast<const uint4*>(tok + 4 * kRowBytes + j * 16);
    const uint4 b8 = *reinterpret_cast<const uint4*>(tok + 5 * kRowBytes + j * 16);
    const uint32_t w2 = *reinterpret_cast<const uint32_t*>(tok + 1 * kRowBytes + (8 * j + 2 * c) * 2);
    const uint2 v4raw = *reinterpret_cast<const uint2*>(tok + 3 * kRowBytes + col * 2);
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + stage);  // everything this warp needs is in registers

    // eight fp16 values of a token row -> fp32, value i at pairs[i / 2].{x, y}
    auto unpack8 = [](const uint4& q, float2 (&pairs)[4]) {
      pairs[0] = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
      pairs[1] = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
      pairs[2] = __half22float2(*reinterpret_cast<const __half2*>(&q.z));
      pairs[3] = __half22float2(*reinterpret_cast<const __half2*>(&q.w));
    };
    auto at = [](const float2 (&pairs)[4], int i) -> float { return (i & 1) ? pairs[i >> 1].y : pairs[i >> 1].x; };
    float2 ra[4], ka[4], aa[4], ba[4];
    unpack8(r8, ra);
    unpack8(k8, ka);
    unpack8(a8, aa);
    unpack8(b8, ba);
    // decay of rows 8j + 2c and 8j + 2c + 1, evaluated once per row group and handed round with shuffles
    float mine[2];
    {
      const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&w2));
      float2 bias2 = make_float2(0.f, 0.f);
      if (LOGITS && p.bias != nullptr)
        bias2 = __half22float2(*reinterpret_cast<const __half2*>(p.bias + head * kHeadDim + 8 * j + 2 * c));
      const int phase = meta.w + head * kHeadDim + 8 * j + 2 * c;
      float x0 = wf.x, x1 = wf.y;
      if constexpr (LOGITS) {  // SFU approximations (2^-22): far below the fp16 rounding of delta that follows
        x0 = retention_from_logit_fast(x0 + bias2.x);
        x1 = retention_from_logit_fast(x1 + bias2.y);
      }
      mine[0] = to_half_and_back(x0 - 1.0f + dither_of(phase));
      mine[1] = to_half_and_back(x1 - 1.0f + dither_of(phase + 1));
    }
    float2 sa01 = make_float2(0.f, 0.f), sa23 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float fa = at(aa, i);
      const float2 fa2 = make_float2(fa, fa);
      sa01 = __ffma2_rn(fa2, S01[i], sa01);
      sa23 = __ffma2_rn(fa2, S23[i], sa23);
    }
#pragma unroll
    for (int m = 4; m < 32; m <<= 1) {
      sa01.x += __shfl_xor_sync(0xffffffffu, sa01.x, m);
      sa01.y += __shfl_xor_sync(0xffffffffu, sa01.y, m);
      sa23.x += __shfl_xor_sync(0xffffffffu, sa23.x, m);
      sa23.y += __shfl_xor_sync(0xffffffffu, sa23.y, m);
    }
    const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&v4raw.x));
    const float2 v23 = __half22float2(*reinterpret_cast<const __half2*>(&v4raw.y));
    float2 acc01 = make_float2(0.f, 0.f), acc23 = make_float2(0.f, 0.f);
    __half* state_out = p.pool + (static_cast<size_t>(meta.z) * p.heads + head) * (kHeadDim * kHeadDim) +
                        static_cast<size_t>(8 * j) * kHeadDim + col;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float delta = __shfl_sync(0xffffffffu, mine[i & 1], (lane & ~3) | (i >> 1));
      const float fb = at(ba, i), fk = at(ka, i), fr = at(ra, i);
      const float2 d2 = make_float2(delta, delta), b2 = make_float2(fb, fb), k2 = make_float2(fk, fk),
                   r2 = make_float2(fr, fr);
      // S + S*delta + b*sa + k*v in fp32, then rounded to the stored precision; y reads the rounded state
      const float2 n01 = __ffma2_rn(k2, v01, __ffma2_rn(b2, sa01, __ffma2_rn(S01[i], d2, S01[i])));
      const float2 n23 = __ffma2_rn(k2, v23, __ffma2_rn(b2, sa23, __ffma2_rn(S23[i], d2, S23[i])));
      const __half2 lo = __floats2half2_rn(n01.x, n01.y), hi = __floats2half2_rn(n23.x, n23.y);
      acc01 = __ffma2_rn(r2, __half22float2(lo), acc01);
      acc23 = __ffma2_rn(r2, __half22float2(hi), acc23);
      uint2 q;
      q.x = *reinterpret_cast<const uint32_t*>(&lo);
      q.y = *reinterpret_cast<const uint32_t*>(&hi);
      __stcs(reinterpret_cast<uint2*>(state_out + i * kHeadDim), q);
    }
#pragma unroll
    for (int m = 4; m < 32; m <<= 1) {
      acc01.x += __shfl_xor_sync(0xffffffffu, acc01.x, m);
      acc01.y += __shfl_xor_sync(0xffffffffu, acc01.y, m);
      acc23.x += __shfl_xor_sync(0xffffffffu, acc23.x, m);
      acc23.y += __shfl_xor_sync(0xffffffffu, acc23.y, m);
    }
    if (j == 0) {
      const __half2 lo = __floats2half2_rn(acc01.x * p.scale, acc01.y * p.scale);
      const __half2 hi = __floats2half2_rn(acc23.x * p.scale, acc23.y * p.scale);
      uint2 q;
      q.x = *reinterpret_cast<const uint32_t*>(&lo);
      q.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(p.y + (static_cast<size_t>(meta.y) * p.heads + head) * kHeadDim + col) = q;
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [items][8 (i)][8 (j)][64 columns] view of the fp16 pool with the two row strides swapped (see the file header);
// cached per (address, item count): the same pool is used step after step.
int state_map_for(CUtensorMap* map, const void* pool, long long items) {
  constexpr int kEntries = 16;
  static std::mutex mutex;
  static const void* bases[kEntries];
  static long long counts[kEntries];
  static CUtensorMap maps[kEntries];
  static int used = 0, next = 0;
  static EncodeTiledFn encode = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  std::lock_guard<std::mutex> lock(mutex);
  for (int i = 0; i < used; ++i) {
    if (bases[i] == pool && counts[i] == items) {
      std::memcpy(map, &maps[i], sizeof(CUtensorMap));
      return FRWKV_OK;
    }
  }
  if (encode == nullptr) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_fp16_state: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[4] = {64, 8, 8, static_cast<cuuint64_t>(items)};
  const cuuint64_t strides[3] = {1024, 128, kStateBytes};  // j, i, item (bytes)
  const cuuint32_t box[4] = {64, 8, 8, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(pool), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_fp16_state: cuTensorMapEncodeTiled failed (%d)", int(rc));
  const int slot = used < kEntries ? used++ : (next = (next + 1) % kEntries);
  bases[slot] = pool;
  counts[slot] = items;
  std::memcpy(&maps[slot], map, sizeof(CUtensorMap));
  return FRWKV_OK;
}

template <bool LOGITS>
int prepare() {
  static bool done[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return check_launch("cudaGetDevice");
  if (!done[device]) {
    if (cudaFuncSetAttribute(wkv7_decode_fp16_state_kernel<LOGITS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemBytes) != cudaSuccess)
      return check_launch("wkv7_decode_fp16_state_kernel shared-memory attribute");
    done[device] = true;
  }
  return FRWKV_OK;
}

}  // namespace

// One-token rows only (the caller guarantees max_seqlen == 1); pool_slots = number of slots of the pool.
bool programmatic_launch_enabled();  // recurrent_stream.cu: FRWKV_PDL, read once

int launch_decode_fp16_state(const int32_t* cu, const int32_t* slots, const int32_t* status, const int32_t* elapsed,
                             void* pool, int pool_slots, const void* r, const void* w, const void* k, const void* v,
                             const void* a, const void* b, const void* bias, void* y, int n_seq, int total_tokens,
                             int heads, int decay_mode, float scale, int32_t* error_flag, cudaStream_t stream) {
  CUtensorMap map;
  int rc = state_map_for(&map, pool, static_cast<long long>(pool_slots) * heads);
  if (rc != FRWKV_OK) return rc;
  const bool logits = decay_mode == FRWKV_DECAY_LOGITS;
  rc = logits ? prepare<true>() : prepare<false>();
  if (rc != FRWKV_OK) return rc;
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long items = static_cast<long long>(n_seq) * heads;
  if (items > 0x7fffffffLL) return fail(FRWKV_ERR_ARGUMENT, "wkv7_recurrent_fp16_state: too many (sequence, head) pairs");
  // Grid: the CTAs stride over the items, so any grid works.  Exactly the resident CTAs would fix every SM's share
  // in advance, and SMs do not run equally fast; with up to 8 grids' worth of CTAs (at least 24 items each, so that
  // filling the ring stays a small part of a CTA's life) the hardware scheduler evens that out: 406 -> 389 us on
  // 2048 x 64 pairs.  FRWKV_FP16_GRID_MULT forces the multiple (tuning hook, read once).
  static const int forced = [] {
    const char* e = std::getenv("FRWKV_FP16_GRID_MULT");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  const long long resident = static_cast<long long>(sms) * kCtasPerSm;
  long long mult = forced > 0 ? forced : items / (resident * 24);
  mult = mult < 1 ? 1 : (mult > 8 && forced <= 0 ? 8 : mult);
  const long long want = resident * mult;
  const unsigned grid = static_cast<unsigned>(items < want ? items : want);
  DecodeParams p{cu, slots, status, elapsed, static_cast<__half*>(pool),
                 static_cast<const __half*>(r), static_cast<const __half*>(w), static_cast<const __half*>(k),
                 static_cast<const __half*>(v), static_cast<const __half*>(a), static_cast<const __half*>(b),
                 static_cast<const __half*>(bias), static_cast<__half*>(y), error_flag, n_seq, total_tokens, heads,
                 scale};
  // A decode step is this kernel and the counter kernel behind it, step after step on one stream: both are launched
  // with programmatic stream serialisation, so that each one's launch and ramp hide under its predecessor's tail
  // (every kernel of the chain waits for its predecessor's completion before it touches memory).
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = programmatic_launch_enabled() ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t err = logits ? cudaLaunchKernelEx(&config, wkv7_decode_fp16_state_kernel<true>, p, map)
                                 : cudaLaunchKernelEx(&config, wkv7_decode_fp16_state_kernel<false>, p, map);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_decode_fp16_state_kernel: %s", cudaGetErrorString(err));
  return check_launch("wkv7_decode_fp16_state_kernel");
}

}  // namespace frwkv
