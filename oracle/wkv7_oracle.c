/* CPU oracle for the WKV7 recurrence in plain C.  TEST INFRASTRUCTURE ONLY.
 *
 * Same recurrence as oracle/wkv7_oracle.py, which restates the reference's
 * parity definition (rwkv-rs/FlashRWKV2 tests/tmix/wkv7/test.py:29-85; decay
 * constant from csrc/sm120/tmix/wkv7/recurrent_decay.cuh:12).  It exists so the
 * parity tests and the benchmark's CPU baseline can cover sizes the Python loop
 * cannot finish in seconds.  The product never links or loads this file.
 *
 * Parity pin: tests/test_oracle.py checks this file against the Python oracle
 * and against the committed outputs of the reference's own function
 * (tests/golden/).
 *
 * Layout: token tensors [T, H, D] fp32 (the caller widens 16-bit inputs, as the
 * reference does at test.py:59-64); pool [slots, H, K, V] fp32, element (k, v)
 * at k*D+v, updated in place; cu_seqlens [n_seq+1]; slots [n_seq].
 * decay_mode 0: w holds raw decay logits (bias added before the sigmoid);
 * decay_mode 1: w holds the retention itself.
 * The *_f64 entry keeps the state and all sums in double (error analysis).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define WKV7_DECAY_RATE 0.6065306597126334

#define DEFINE_ORACLE(NAME, REAL, EXPF)                                          \
  int NAME(const float* r, const float* w, const float* k, const float* v,       \
           const float* a, const float* b, const float* decay_bias, REAL* y,     \
           REAL* pool, const int* cu_seqlens, const int* slots, int n_seq,       \
           int H, int D, double scale, int decay_mode, int n_threads) {          \
    if (D <= 0 || D > 256 || H <= 0 || n_seq < 0) return 1;                       \
    if (decay_mode != 0 && decay_mode != 1) return 2;                             \
    long pairs = (long)n_seq * H;                                                 \
    _Pragma("omp parallel for schedule(dynamic, 1) num_threads(n_threads)")       \
    for (long p = 0; p < pairs; ++p) {                                            \
      int seq = (int)(p / H), h = (int)(p % H);                                   \
      REAL* S = pool + ((size_t)slots[seq] * H + h) * D * D;                      \
      REAL sa[256], rho[256];                                                     \
      for (int t = cu_seqlens[seq]; t < cu_seqlens[seq + 1]; ++t) {               \
        size_t row = ((size_t)t * H + h) * D;                                     \
        for (int i = 0; i < D; ++i) {                                             \
          if (decay_mode == 0) {                                                  \
            REAL x = (REAL)w[row + i];                                            \
            if (decay_bias) x += (REAL)decay_bias[(size_t)h * D + i];             \
            REAL sig = (REAL)1 / ((REAL)1 + EXPF(-x));                            \
            rho[i] = EXPF(-(REAL)WKV7_DECAY_RATE * sig);                          \
          } else {                                                                \
            rho[i] = (REAL)w[row + i];                                            \
          }                                                                       \
        }                                                                         \
        for (int j = 0; j < D; ++j) sa[j] = 0;                                    \
        for (int i = 0; i < D; ++i) {                                             \
          REAL ai = (REAL)a[row + i];                                             \
          const REAL* Si = S + (size_t)i * D;                                     \
          for (int j = 0; j < D; ++j) sa[j] += ai * Si[j];                        \
        }                                                                         \
        REAL* yt = y + row;                                                       \
        for (int j = 0; j < D; ++j) yt[j] = 0;                                    \
        for (int i = 0; i < D; ++i) {                                             \
          REAL bi = (REAL)b[row + i], ki = (REAL)k[row + i];                      \
          REAL ri = (REAL)r[row + i], di = rho[i];                                \
          REAL* Si = S + (size_t)i * D;                                           \
          for (int j = 0; j < D; ++j) {                                           \
            REAL s = di * Si[j] + bi * sa[j] + ki * (REAL)v[row + j];             \
            Si[j] = s;                                                            \
            yt[j] += ri * s;                                                      \
          }                                                                       \
        }                                                                         \
        for (int j = 0; j < D; ++j) yt[j] *= (REAL)scale;                         \
      }                                                                           \
    }                                                                             \
    return 0;                                                                     \
  }

DEFINE_ORACLE(wkv7_oracle_f32, float, expf)
DEFINE_ORACLE(wkv7_oracle_f64, double, exp)

int wkv7_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
