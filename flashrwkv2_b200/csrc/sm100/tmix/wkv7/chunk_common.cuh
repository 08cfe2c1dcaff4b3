// Pieces of the tensor-core chunk kernel: parameters, the hi/lo operand splits (bf16 and fp16),
// operand descriptors and MMA issue, TMA tensor-map creation (cached per tensor).
#pragma once

#include "../../common.cuh"
#include "../../tcgen05.cuh"

#include <cstring>
#include <mutex>
#include <type_traits>

namespace frwkv {
namespace chunk {

using namespace tc;

constexpr uint32_t kRowGroup = 128;  // one core-matrix row group: 8 rows x 16 B

// Optional per-phase cycle counters of CTA 0 (development builds only).  The add is a reduction without a return
// value: a plain read-modify-write would stall the measuring warp for a global-memory round trip at every marker.
#ifdef FRWKV_CHUNK_TIMING
__device__ unsigned long long g_phase_ticks[16];
#define FRWKV_PHASE(i)                                                                  \
  if (tid == 255 && blockIdx.x == 0) {                                                  \
    const long long now = clock64();                                                    \
    atomicAdd(&g_phase_ticks[i], static_cast<unsigned long long>(now - phase_t0));      \
    phase_t0 = now;                                                                     \
  }
#else
#define FRWKV_PHASE(i)
#endif

// Test hook for the bounded waits, compiled only into the test build of the library (FRWKV_TEST_HOOKS):
// frwkv_sm100_test_skip_commit(chunk) makes the kernel leave out one tcgen05.commit, so that the wait on it
// runs out and the failure path (error flag, no hang) can be exercised.  The product library has neither
// the setter nor the check in its kernel.
#ifdef FRWKV_TEST_HOOKS
int& test_skip_commit_chunk();
#endif

// bits of *error_flag
constexpr int kErrorWait = 1;   // a bounded wait gave up
constexpr int kErrorDecay = 2;  // the decay product of one chunk left the fp32 range (retention mode only)

// Work queue of the persistent form of the chunk kernel (batches with more streams than CTA slots).  A stream
// (sequence, head) is cut into segments of `segment_chunks` chunks; tasks are numbered segment level by segment
// level, and within a level by the longest-first rank of the sequence and then by head, so a task's predecessor
// (the same stream, one segment earlier) always has a smaller number and has been handed out before it.
// level_end[g] = number of tasks in levels 0..g.  Filled on the device by sequence_order_kernel.
constexpr int kQueueLevels = 16;
struct QueueHeader {
  int next_task;       // handed out with atomicAdd
  int total_tasks;
  int segment_chunks;  // chunks per segment
  int level_end[kQueueLevels];
};

struct ChunkParams {
  const int* cu;
  const int* slots;
  const int* status;
  float* pool;
  const void* bias;
  void* y;
  float* y_f32;
  int* error_flag;
  int n_seq, total_tokens, heads;
  float scale;
  const int* order;  // CTA rank -> sequence, longest first (nullptr: natural order)
  int len_from;      // > 0: only sequences at least this long (shorter ones go to the recurrence kernel)
  // fused kk / a-gate producer (all null, or all three [H*64] parameter vectors in the token dtype): with them k is
  // the raw key projection, the `a` tensor holds the gate logits a12 and the `b` tensor is not read
  const void *gate_kk, *gate_a0, *gate_ka;
  QueueHeader* queue;  // nullptr: one stream per CTA
  int* queue_flags;    // [n_seq * heads] segments completed per stream (zeroed before the launch)
#ifdef FRWKV_TEST_HOOKS
  int skip_commit_chunk;  // chunk whose first MMA commit is left out, -1 = none
#endif
};

struct Maps {
  CUtensorMap r, w, k, v, a, b;
};

// SFU approximations (relative error about 2^-22, far below the bf16x2 operand precision)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo_elem, float hi_elem) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo_elem, hi_elem);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float bf16_lo_as_f32(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi_as_f32(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

// hi/lo split of two fp32 values into packed bf16 pairs
__device__ __forceinline__ void split2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16x2(x0, x1);
  lo = pack_bf16x2(x0 - bf16_lo_as_f32(hi), x1 - bf16_hi_as_f32(hi));
}

// hi/lo split of 8 consecutive fp32 values into two 16-byte vectors of bf16
__device__ __forceinline__ void split8(const float* x, uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
    l[i] = pack_bf16x2(x[2 * i] - bf16_lo_as_f32(h[i]), x[2 * i + 1] - bf16_hi_as_f32(h[i]));
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// fp16 operands: one rounding, or a hi/lo pair (22 significant bits).  A value beyond the fp16 range becomes
// inf (and the lo part -inf), so an overflow shows as NaN in the output instead of a silently saturated term.
__device__ __forceinline__ uint32_t pack_f16x2(float lo_elem, float hi_elem) {
  __half2 h = __floats2half2_rn(lo_elem, hi_elem);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void split2_f16(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  const __half2 h = __floats2half2_rn(x0, x1);
  const float2 back = __half22float2(h);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = pack_f16x2(x0 - back.x, x1 - back.y);
}

template <typename io_t> __device__ __forceinline__ float2 unpack2(uint32_t packed);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t packed) {
  return make_float2(bf16_lo_as_f32(packed), bf16_hi_as_f32(packed));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t packed) {
  return __half22float2(*reinterpret_cast<__half2*>(&packed));
}

// One dense contraction D (+)= A * B over KSTEPS steps of 16, as hi*hi (+ hi*lo) (+ lo*hi).
// The descriptors of step 0 are built once per kernel; a step only advances the 14-bit
// start-address field (units of 16 bytes), which cannot carry out of the low word.
struct Operand {
  uint64_t hi, lo;   // descriptors of the hi and lo parts at step 0 (lo == 0: no lo part)
  uint32_t kstep16;  // start-address advance per step of 16, in 16-byte units
};
__device__ __forceinline__ Operand make_operand(uint32_t addr, uint32_t lo_off, uint32_t kstep, uint32_t lbo,
                                                uint32_t sbo) {
  Operand o;
  o.hi = smem_desc(addr, lbo, sbo);
  o.lo = lo_off != 0 ? smem_desc(addr + lo_off, lbo, sbo) : 0ull;
  o.kstep16 = kstep >> 4;
  return o;
}
template <bool A_LO, bool B_LO, uint32_t KSTEPS = 4>
__device__ __forceinline__ void issue_gemm(uint32_t tmem_d, const Operand& a, const Operand& b, uint32_t idesc,
                                           bool accumulate) {
#pragma unroll
  for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
    const uint64_t a_hi = a.hi + ks * a.kstep16, b_hi = b.hi + ks * b.kstep16;
    mma_f16_ss(tmem_d, a_hi, b_hi, idesc, accumulate || ks > 0);
    if constexpr (B_LO) mma_f16_ss(tmem_d, a_hi, b.lo + ks * b.kstep16, idesc, true);
    if constexpr (A_LO) mma_f16_ss(tmem_d, a.lo + ks * a.kstep16, b_hi, idesc, true);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// [64, H, T] view of a packed [T, H, 64] 16-bit tensor; box = one head's `box_rows` rows x 64 columns.
inline int make_map(CUtensorMap* map, const void* base, int total_tokens, int heads, bool bf16, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(FRWKV_ERR_CUDA, "wkv7_prefill: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(total_tokens)};
  const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(heads) * 128};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                         const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(FRWKV_ERR_CUDA, "wkv7_prefill: cuTensorMapEncodeTiled failed (%d)", int(rc));
  return FRWKV_OK;
}


// Encoding a tensor map is a driver call of a few microseconds; a serving loop calls prefill with the same six
// buffers over and over, so the encoded maps are kept in a small cache keyed by (address, shape, dtype, box).
// A map depends on nothing else, so a stale entry for a freed and re-allocated address is still correct.
struct MapKey {
  const void* base;
  int total_tokens, heads, bf16, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && total_tokens == o.total_tokens && heads == o.heads && bf16 == o.bf16 &&
           box_rows == o.box_rows;
  }
};
inline int cached_map(CUtensorMap* map, const void* base, int total_tokens, int heads, bool bf16, int box_rows) {
  constexpr int kEntries = 96;
  static std::mutex mutex;
  static MapKey keys[kEntries];
  static CUtensorMap maps[kEntries];
  static int used = 0, next = 0;
  const MapKey key{base, total_tokens, heads, bf16 ? 1 : 0, box_rows};
  std::lock_guard<std::mutex> lock(mutex);
  for (int i = 0; i < used; ++i) {
    if (keys[i] == key) {
      std::memcpy(map, &maps[i], sizeof(CUtensorMap));
      return FRWKV_OK;
    }
  }
  const int rc = make_map(map, base, total_tokens, heads, bf16, box_rows);
  if (rc != FRWKV_OK) return rc;
  const int slot = used < kEntries ? used++ : (next = (next + 1) % kEntries);
  keys[slot] = key;
  std::memcpy(&maps[slot], map, sizeof(CUtensorMap));
  return FRWKV_OK;
}

inline int make_maps(Maps* maps, const void* r, const void* w, const void* k, const void* v, const void* a,
                     const void* b, int total_tokens, int heads, bool bf16, int box_rows) {
  const void* srcs[6] = {r, w, k, v, a, b};
  CUtensorMap* dsts[6] = {&maps->r, &maps->w, &maps->k, &maps->v, &maps->a, &maps->b};
  for (int i = 0; i < 6; ++i) {
    const int rc = cached_map(dsts[i], srcs[i], total_tokens, heads, bf16, box_rows);
    if (rc != FRWKV_OK) return rc;
  }
  return FRWKV_OK;
}

}  // namespace chunk
}  // namespace frwkv
