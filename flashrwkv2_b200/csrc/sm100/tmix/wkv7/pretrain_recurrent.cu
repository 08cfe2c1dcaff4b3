// WKV7 training operator: forward with state checkpoints, and the backward pass that consumes them.
//
// Contract of the reference's `pretrain_tmix_wkv7_recurrent_bf16` (rwkv-rs/FlashRWKV2 flashrwkv2/tmix/wkv7/pretrain.py:
// 52-116; kernels csrc/sm120/tmix/wkv7/pretrain_recurrent_bf16_forward.cu; oracle tests/tmix/wkv7/pretrain/test.py:44-65):
// dense bf16 [B, T, H, 64] tensors, T a multiple of 16, zero initial state, per token
//   rho = exp(-e^{-1/2} * sigmoid(w));  sa = a^T S;  S = diag(rho) S + b sa^T + k v^T;  y = r^T S.
// The forward stores, for the backward, sa of every token (fp32 [B, T, H, 64]) and the state after every 16th token
// (fp32 [B, H, T/16, 64, 64]).  The backward walks the tokens in reverse with the state gradient dS in registers and
// rebuilds the previous state from the current one, S_{t-1} = (S_t - b sa^T - k v^T) / rho (rho >= 0.545 by
// construction, so the division is benign), restarting from a checkpoint every 16 tokens so that the rebuilt state
// never drifts far.
//
// One CTA of 8 warps owns a (batch, head): warp w holds key rows 8w .. 8w+7, lane l value columns 2l, 2l+1, so a thread
// carries a 8 x 2 block of S (and of dS) in registers.  Sums over the key index cross the warps through shared
// memory (two barriers per token, buffers alternating); sums over the value index stay inside a warp as a
// reduce-scatter of the lane's eight row partials (nine shuffles instead of forty).  The token rows of a 16-token
// chunk are staged in shared memory as fp32.  This is a CUDA-core kernel bound by the per-token chain, like the
// reference's; it is here for completeness of the operator family, not as a tuned training kernel.
#include "../../common.cuh"

namespace frwkv {
namespace {

constexpr int kTrainChunk = 16;
constexpr int kTrainWarps = 8;
constexpr int kTrainThreads = kTrainWarps * 32;
constexpr float kDecayScale = -0.6065306597126334f;  // -e^{-1/2}

__device__ __forceinline__ float bf(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

// Sum over the 32 lanes of eight per-lane values at once: returns, in every lane, the total of value (lane >> 2) & 7.
__device__ __forceinline__ float row_reduce8(const float (&x)[8], int lane) {
  const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0, b2 = (lane & 4) != 0;
  float y4[4], y2[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = b4 ? x[i] : x[i + 4], keep = b4 ? x[i + 4] : x[i];
    y4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = b3 ? y4[i] : y4[i + 2], keep = b3 ? y4[i + 2] : y4[i];
    y2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  const float send = b2 ? y2[0] : y2[1], keep = b2 ? y2[1] : y2[0];
  float z = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  z += __shfl_xor_sync(0xffffffffu, z, 2);
  z += __shfl_xor_sync(0xffffffffu, z, 1);
  return z;
}

struct TrainParams {
  const __nv_bfloat16 *r, *w, *k, *v, *a, *b;
  int batch, tokens, heads;
};

__global__ void __launch_bounds__(kTrainThreads)
wkv7_pretrain_forward_kernel(const TrainParams p, __nv_bfloat16* __restrict__ y, float* __restrict__ boundary,
                             float* __restrict__ state_dot_a) {
  __shared__ float s_r[kTrainChunk][64], s_rho[kTrainChunk][64], s_k[kTrainChunk][64], s_v[kTrainChunk][64],
      s_a[kTrainChunk][64], s_b[kTrainChunk][64];
  __shared__ float s_part[2][2][kTrainWarps][64];  // [buffer][sa | y][warp][value column]
  const int head = blockIdx.x, batch = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = warp * 8, col = lane * 2;
  float S[8][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) S[i][0] = S[i][1] = 0.f;
  const long long chunks = p.tokens / kTrainChunk;
  float* my_boundary = boundary + (static_cast<long long>(batch) * p.heads + head) * chunks * 4096;

  for (int t0 = 0; t0 < p.tokens; t0 += kTrainChunk) {
    __syncthreads();  // the previous chunk's rows are no longer read
    for (int e = tid; e < kTrainChunk * 64; e += kTrainThreads) {
      const int tt = e >> 6, c = e & 63;
      const long long at = ((static_cast<long long>(batch) * p.tokens + t0 + tt) * p.heads + head) * 64 + c;
      s_r[tt][c] = bf(p.r, at);
      s_rho[tt][c] = __expf(kDecayScale / (1.0f + __expf(-bf(p.w, at))));
      s_k[tt][c] = bf(p.k, at);
      s_v[tt][c] = bf(p.v, at);
      s_a[tt][c] = bf(p.a, at);
      s_b[tt][c] = bf(p.b, at);
    }
    __syncthreads();
    for (int tt = 0; tt < kTrainChunk; ++tt) {
      const int buf = tt & 1;
      // sa = a^T S: own eight rows, then across the warps
      float2 part = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float av = s_a[tt][row0 + i];
        part.x = fmaf(av, S[i][0], part.x);
        part.y = fmaf(av, S[i][1], part.y);
      }
      *reinterpret_cast<float2*>(&s_part[buf][0][warp][col]) = part;
      __syncthreads();
      float2 sa = make_float2(0.f, 0.f);
#pragma unroll
      for (int wq = 0; wq < kTrainWarps; ++wq) {
        const float2 q = *reinterpret_cast<const float2*>(&s_part[buf][0][wq][col]);
        sa.x += q.x;
        sa.y += q.y;
      }
      const float2 vv = *reinterpret_cast<const float2*>(&s_v[tt][col]);
      float2 ypart = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float rho = s_rho[tt][row0 + i], bv = s_b[tt][row0 + i], kv = s_k[tt][row0 + i], rv = s_r[tt][row0 + i];
        S[i][0] = fmaf(rho, S[i][0], fmaf(bv, sa.x, kv * vv.x));
        S[i][1] = fmaf(rho, S[i][1], fmaf(bv, sa.y, kv * vv.y));
        ypart.x = fmaf(rv, S[i][0], ypart.x);
        ypart.y = fmaf(rv, S[i][1], ypart.y);
      }
      *reinterpret_cast<float2*>(&s_part[buf][1][warp][col]) = ypart;
      __syncthreads();
      if (warp == 0) {
        float2 yy = make_float2(0.f, 0.f);
#pragma unroll
        for (int wq = 0; wq < kTrainWarps; ++wq) {
          const float2 q = *reinterpret_cast<const float2*>(&s_part[buf][1][wq][col]);
          yy.x += q.x;
          yy.y += q.y;
        }
        const long long at = ((static_cast<long long>(batch) * p.tokens + t0 + tt) * p.heads + head) * 64 + col;
        *reinterpret_cast<__nv_bfloat162*>(y + at) = __floats2bfloat162_rn(yy.x, yy.y);
        *reinterpret_cast<float2*>(state_dot_a + at) = sa;
      }
    }
    // checkpoint: the state after the chunk's last token
    float* dst = my_boundary + static_cast<long long>(t0 / kTrainChunk) * 4096;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float2*>(dst + (row0 + i) * 64 + col) = make_float2(S[i][0], S[i][1]);
  }
}

__global__ void __launch_bounds__(kTrainThreads)  // 126 registers, two CTAs per SM; three (80 registers) measured slower
wkv7_pretrain_backward_kernel(const TrainParams p, const __nv_bfloat16* __restrict__ dy,
                              const float* __restrict__ boundary, const float* __restrict__ state_dot_a,
                              __nv_bfloat16* __restrict__ dr, __nv_bfloat16* __restrict__ dw,
                              __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                              __nv_bfloat16* __restrict__ da, __nv_bfloat16* __restrict__ db) {
  __shared__ float s_r[kTrainChunk][64], s_rho[kTrainChunk][64], s_k[kTrainChunk][64], s_v[kTrainChunk][64],
      s_a[kTrainChunk][64], s_b[kTrainChunk][64], s_dy[kTrainChunk][64], s_sa[kTrainChunk][64],
      s_dfac[kTrainChunk][64];  // d rho / d w
  __shared__ float s_part[2][2][kTrainWarps][64];  // [buffer][dv | dsa][warp][value column]
  const int head = blockIdx.x, batch = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row0 = warp * 8, col = lane * 2;
  const int my_row = row0 + ((lane >> 2) & 7);  // the row whose value-index sums land in this lane
  const bool writes_row = (lane & 3) == 0;
  float S[8][2], dS[8][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) S[i][0] = S[i][1] = dS[i][0] = dS[i][1] = 0.f;
  const long long chunks = p.tokens / kTrainChunk;
  const float* my_boundary = boundary + (static_cast<long long>(batch) * p.heads + head) * chunks * 4096;

  for (int t0 = p.tokens - kTrainChunk; t0 >= 0; t0 -= kTrainChunk) {
    __syncthreads();
    for (int e = tid; e < kTrainChunk * 64; e += kTrainThreads) {
      const int tt = e >> 6, c = e & 63;
      const long long at = ((static_cast<long long>(batch) * p.tokens + t0 + tt) * p.heads + head) * 64 + c;
      const float sig = 1.0f / (1.0f + __expf(-bf(p.w, at)));
      const float rho = __expf(kDecayScale * sig);
      s_r[tt][c] = bf(p.r, at);
      s_rho[tt][c] = rho;
      s_dfac[tt][c] = rho * kDecayScale * sig * (1.0f - sig);
      s_k[tt][c] = bf(p.k, at);
      s_v[tt][c] = bf(p.v, at);
      s_a[tt][c] = bf(p.a, at);
      s_b[tt][c] = bf(p.b, at);
      s_dy[tt][c] = bf(dy, at);
      s_sa[tt][c] = state_dot_a[at];
    }
    // the state after this chunk's last token
    const float* src = my_boundary + static_cast<long long>(t0 / kTrainChunk) * 4096;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 q = *reinterpret_cast<const float2*>(src + (row0 + i) * 64 + col);
      S[i][0] = q.x;
      S[i][1] = q.y;
    }
    __syncthreads();
    for (int tt = kTrainChunk - 1; tt >= 0; --tt) {
      const int buf = tt & 1;
      const long long row_at = ((static_cast<long long>(batch) * p.tokens + t0 + tt) * p.heads + head) * 64;
      const float2 dyv = *reinterpret_cast<const float2*>(&s_dy[tt][col]);
      const float2 vv = *reinterpret_cast<const float2*>(&s_v[tt][col]);
      const float2 sav = *reinterpret_cast<const float2*>(&s_sa[tt][col]);
      // y = r^T S_t:  dr_k = sum_v dy_v S_t[k][v];  dS += r dy^T.  Then S_{t-1} from S_t.
      float part_dr[8], part_dk[8], part_db[8], part_drho[8];
      float2 col_dv = make_float2(0.f, 0.f), col_dsa = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float rv = s_r[tt][row0 + i], kv = s_k[tt][row0 + i], bv = s_b[tt][row0 + i];
        const float inv_rho = __fdividef(1.0f, s_rho[tt][row0 + i]);  // rho in [0.545, 1): two units in the last place
        part_dr[i] = fmaf(dyv.x, S[i][0], dyv.y * S[i][1]);
        dS[i][0] = fmaf(rv, dyv.x, dS[i][0]);
        dS[i][1] = fmaf(rv, dyv.y, dS[i][1]);
        S[i][0] = (S[i][0] - bv * sav.x - kv * vv.x) * inv_rho;  // S_{t-1}
        S[i][1] = (S[i][1] - bv * sav.y - kv * vv.y) * inv_rho;
        part_dk[i] = fmaf(dS[i][0], vv.x, dS[i][1] * vv.y);
        part_db[i] = fmaf(dS[i][0], sav.x, dS[i][1] * sav.y);
        part_drho[i] = fmaf(dS[i][0], S[i][0], dS[i][1] * S[i][1]);
        col_dv.x = fmaf(dS[i][0], kv, col_dv.x);
        col_dv.y = fmaf(dS[i][1], kv, col_dv.y);
        col_dsa.x = fmaf(dS[i][0], bv, col_dsa.x);
        col_dsa.y = fmaf(dS[i][1], bv, col_dsa.y);
      }
      *reinterpret_cast<float2*>(&s_part[buf][0][warp][col]) = col_dv;
      *reinterpret_cast<float2*>(&s_part[buf][1][warp][col]) = col_dsa;
      const float g_r = row_reduce8(part_dr, lane), g_k = row_reduce8(part_dk, lane);
      const float g_b = row_reduce8(part_db, lane), g_rho = row_reduce8(part_drho, lane);
      __syncthreads();
      float2 dsa = make_float2(0.f, 0.f), dvv = make_float2(0.f, 0.f);
#pragma unroll
      for (int wq = 0; wq < kTrainWarps; ++wq) {
        const float2 q = *reinterpret_cast<const float2*>(&s_part[buf][1][wq][col]);
        dsa.x += q.x;
        dsa.y += q.y;
        if (warp == 0) {
          const float2 u = *reinterpret_cast<const float2*>(&s_part[buf][0][wq][col]);
          dvv.x += u.x;
          dvv.y += u.y;
        }
      }
      // sa = a^T S_{t-1}:  da_k = sum_v dsa_v S_{t-1}[k][v];  dS_{t-1} = rho dS + a dsa^T
      float part_da[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float rho = s_rho[tt][row0 + i], av = s_a[tt][row0 + i];
        part_da[i] = fmaf(dsa.x, S[i][0], dsa.y * S[i][1]);
        dS[i][0] = fmaf(rho, dS[i][0], av * dsa.x);
        dS[i][1] = fmaf(rho, dS[i][1], av * dsa.y);
      }
      const float g_a = row_reduce8(part_da, lane);
      // The five row gradients of this token replace the token's own rows in shared memory (this warp's eight rows
      // are read by this warp only, and every read of them is above) and leave for global memory, coalesced, when the
      // chunk is done.
      if (writes_row) {
        s_r[tt][my_row] = g_r;
        s_k[tt][my_row] = g_k;
        s_b[tt][my_row] = g_b;
        s_a[tt][my_row] = g_a;
        s_dfac[tt][my_row] = g_rho * s_dfac[tt][my_row];
      }
      if (warp == 0) *reinterpret_cast<__nv_bfloat162*>(dv + row_at + col) = __floats2bfloat162_rn(dvv.x, dvv.y);
    }
    __syncthreads();
    for (int e = tid; e < kTrainChunk * 32; e += kTrainThreads) {  // two channels per thread and row
      const int tt = e >> 5, c = (e & 31) * 2;
      const long long at = ((static_cast<long long>(batch) * p.tokens + t0 + tt) * p.heads + head) * 64 + c;
      *reinterpret_cast<__nv_bfloat162*>(dr + at) = __floats2bfloat162_rn(s_r[tt][c], s_r[tt][c + 1]);
      *reinterpret_cast<__nv_bfloat162*>(dk + at) = __floats2bfloat162_rn(s_k[tt][c], s_k[tt][c + 1]);
      *reinterpret_cast<__nv_bfloat162*>(db + at) = __floats2bfloat162_rn(s_b[tt][c], s_b[tt][c + 1]);
      *reinterpret_cast<__nv_bfloat162*>(da + at) = __floats2bfloat162_rn(s_a[tt][c], s_a[tt][c + 1]);
      *reinterpret_cast<__nv_bfloat162*>(dw + at) = __floats2bfloat162_rn(s_dfac[tt][c], s_dfac[tt][c + 1]);
    }
  }
}

int check_train_arguments(const char* who, const void* const* pointers, int count, int batch, int tokens, int heads) {
  for (int i = 0; i < count; ++i) {
    if (pointers[i] == nullptr) return fail(FRWKV_ERR_ARGUMENT, "%s: every tensor must be non-null", who);
    if ((reinterpret_cast<uintptr_t>(pointers[i]) & 15) != 0)
      return fail(FRWKV_ERR_ARGUMENT, "%s: tensors must be 16-byte aligned", who);
  }
  if (batch <= 0 || tokens <= 0 || heads <= 0 || batch > 65535)
    return fail(FRWKV_ERR_ARGUMENT, "%s: batch (<= 65535), tokens and heads must be positive", who);
  if (tokens % kTrainChunk != 0)
    return fail(FRWKV_ERR_ARGUMENT, "%s: the token count must be a multiple of %d", who, kTrainChunk);
  return FRWKV_OK;
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_sm100_wkv7_pretrain_forward(const void* r, const void* w, const void* k, const void* v,
                                                 const void* a, const void* b, void* y, float* boundary,
                                                 float* state_dot_a, int batch, int tokens, int heads, void* stream) {
  using namespace frwkv;
  const void* pointers[] = {r, w, k, v, a, b, y, boundary, state_dot_a};
  const int rc = check_train_arguments("wkv7_pretrain_forward", pointers, 9, batch, tokens, heads);
  if (rc != FRWKV_OK) return rc;
  const TrainParams p{static_cast<const __nv_bfloat16*>(r), static_cast<const __nv_bfloat16*>(w),
                      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
                      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), batch, tokens, heads};
  wkv7_pretrain_forward_kernel<<<dim3(heads, batch), kTrainThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      p, static_cast<__nv_bfloat16*>(y), boundary, state_dot_a);
  return check_launch("wkv7_pretrain_forward_kernel");
}

extern "C" int frwkv_sm100_wkv7_pretrain_backward(const void* r, const void* w, const void* k, const void* v,
                                                  const void* a, const void* b, const void* dy, const float* boundary,
                                                  const float* state_dot_a, void* dr, void* dw, void* dk, void* dv,
                                                  void* da, void* db, int batch, int tokens, int heads, void* stream) {
  using namespace frwkv;
  const void* pointers[] = {r, w, k, v, a, b, dy, boundary, state_dot_a, dr, dw, dk, dv, da, db};
  const int rc = check_train_arguments("wkv7_pretrain_backward", pointers, 15, batch, tokens, heads);
  if (rc != FRWKV_OK) return rc;
  const TrainParams p{static_cast<const __nv_bfloat16*>(r), static_cast<const __nv_bfloat16*>(w),
                      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
                      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), batch, tokens, heads};
  auto out = [](void* q) { return static_cast<__nv_bfloat16*>(q); };
  wkv7_pretrain_backward_kernel<<<dim3(heads, batch), kTrainThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      p, static_cast<const __nv_bfloat16*>(dy), boundary, state_dot_a, out(dr), out(dw), out(dk), out(dv), out(da),
      out(db));
  return check_launch("wkv7_pretrain_backward_kernel");
}
