/*
 * CPU restatement of the reference's banded contractions.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker for the CUDA kernels (tests/, the smoke check and bench.py's CPU-baseline leg); nothing in the
 * product path may call it.
 *
 * It follows the reference's defining loops in csrc/window_matmul/cpu/window_matmul_cpu.cpp:
 *   window forward     :35-46     window backward    :81-96
 *   unwindow forward   :129-140   unwindow backward  :175-190
 * including what makes the reference's results what they are, bit for bit:
 *   - every output element is accumulated IN THE ELEMENT TYPE, in place, starting from 0
 *     (`out += a * b`, :43, :92-93, :137, :186-187), one product at a time in ascending order of the
 *     reduction index; the product and the sum are rounded separately (the reference is built without
 *     FMA contraction, so build this file with -ffp-contract=off);
 *   - only in-sequence terms enter a sum (loop bounds max(0,s-w) .. min(M,s+w+1), :39, :85, :133, :179);
 *     out-of-sequence band slots of an output stay exactly 0 and those of an input are never read;
 *   - the band index is w_idx = key - query + window (:41 reduces to this);
 *   - fp16 accumulates in fp16: c10::Half's operators compute in float and round to half after every
 *     product and every sum.
 * Layouts are the reference's: src (B,M,N), other (B,N,M) for window_*, band (B,M,2w+1), all contiguous.
 *
 * Parity pin: tests/test_oracle.py checks these functions bit for bit against golden vectors produced
 * by the compiled reference itself (tests/golden/make_golden.py).
 */
#include <math.h>
#include <stddef.h>
#include <string.h>

#define WMM_MAX(a, b) ((a) > (b) ? (a) : (b))
#define WMM_MIN(a, b) ((a) < (b) ? (a) : (b))

#define WMM_DEFINE(T, SUF, MUL, ADD)                                                                   \
  /* window_matmul_cpu.cpp:35-46 */                                                                    \
  void wmm_oracle_window_fw_##SUF(const T *src, const T *other, T *out, int B, int M, int N, int w) { \
    const int W = 2 * w + 1;                                                                           \
    memset(out, 0, sizeof(T) * (size_t)B * M * W);                                                     \
    for (int b = 0; b < B; b++)                                                                        \
      for (int s = 0; s < M; s++)                                                                      \
        for (int k = WMM_MAX(0, s - w); k < WMM_MIN(M, s + w + 1); k++) {                              \
          const int j = k - s + w;                                                                     \
          T acc = out[((size_t)b * M + s) * W + j];                                                    \
          for (int h = 0; h < N; h++)                                                                  \
            acc = ADD(acc, MUL(src[((size_t)b * M + s) * N + h], other[((size_t)b * N + h) * M + k])); \
          out[((size_t)b * M + s) * W + j] = acc;                                                      \
        }                                                                                              \
  }                                                                                                    \
  /* window_matmul_cpu.cpp:81-96; grad_other has other's layout (B,N,M) */                             \
  void wmm_oracle_window_bw_##SUF(const T *src, const T *other, const T *gout, T *gsrc, T *gother,     \
                                  int B, int M, int N, int w) {                                        \
    const int W = 2 * w + 1;                                                                           \
    memset(gsrc, 0, sizeof(T) * (size_t)B * M * N);                                                    \
    memset(gother, 0, sizeof(T) * (size_t)B * M * N);                                                  \
    for (int b = 0; b < B; b++)                                                                        \
      for (int s = 0; s < M; s++)                                                                      \
        for (int k = WMM_MAX(0, s - w); k < WMM_MIN(M, s + w + 1); k++) {                              \
          const int j = k - s + w;                                                                     \
          for (int h = 0; h < N; h++) {                                                                \
            T *gs = &gsrc[((size_t)b * M + s) * N + h];                                                \
            *gs = ADD(*gs, MUL(other[((size_t)b * N + h) * M + k], gout[((size_t)b * M + s) * W + j])); \
            T *go = &gother[((size_t)b * N + h) * M + s];                                              \
            *go = ADD(*go, MUL(src[((size_t)b * M + k) * N + h],                                       \
                               gout[((size_t)b * M + k) * W + (2 * w - j)]));                          \
          }                                                                                            \
        }                                                                                              \
  }                                                                                                    \
  /* window_matmul_cpu.cpp:129-140 */                                                                  \
  void wmm_oracle_unwindow_fw_##SUF(const T *band, const T *other, T *out, int B, int M, int N,        \
                                    int w) {                                                           \
    const int W = 2 * w + 1;                                                                           \
    memset(out, 0, sizeof(T) * (size_t)B * M * N);                                                     \
    for (int b = 0; b < B; b++)                                                                        \
      for (int s = 0; s < M; s++)                                                                      \
        for (int k = WMM_MAX(0, s - w); k < WMM_MIN(M, s + w + 1); k++) {                              \
          const int j = k - s + w;                                                                     \
          const T a = band[((size_t)b * M + s) * W + j];                                               \
          for (int h = 0; h < N; h++) {                                                                \
            T *o = &out[((size_t)b * M + s) * N + h];                                                  \
            *o = ADD(*o, MUL(a, other[((size_t)b * M + k) * N + h]));                                  \
          }                                                                                            \
        }                                                                                              \
  }                                                                                                    \
  /* window_matmul_cpu.cpp:175-190 */                                                                  \
  void wmm_oracle_unwindow_bw_##SUF(const T *band, const T *other, const T *gout, T *gband,            \
                                    T *gother, int B, int M, int N, int w) {                           \
    const int W = 2 * w + 1;                                                                           \
    memset(gband, 0, sizeof(T) * (size_t)B * M * W);                                                   \
    memset(gother, 0, sizeof(T) * (size_t)B * M * N);                                                  \
    for (int b = 0; b < B; b++)                                                                        \
      for (int s = 0; s < M; s++)                                                                      \
        for (int k = WMM_MAX(0, s - w); k < WMM_MIN(M, s + w + 1); k++) {                              \
          const int j = k - s + w;                                                                     \
          for (int h = 0; h < N; h++) {                                                                \
            T *ga = &gband[((size_t)b * M + s) * W + j];                                               \
            *ga = ADD(*ga, MUL(other[((size_t)b * M + k) * N + h], gout[((size_t)b * M + s) * N + h])); \
            T *gv = &gother[((size_t)b * M + s) * N + h];                                              \
            *gv = ADD(*gv, MUL(band[((size_t)b * M + k) * W + (2 * w - j)],                            \
                               gout[((size_t)b * M + k) * N + h]));                                    \
          }                                                                                            \
        }                                                                                              \
  }

#define MUL_NATIVE(a, b) ((a) * (b))
#define ADD_NATIVE(a, b) ((a) + (b))
/* c10::Half arithmetic: operands widened to float, result rounded to half after each operation. */
#define MUL_HALF(a, b) ((_Float16)((float)(a) * (float)(b)))
#define ADD_HALF(a, b) ((_Float16)((float)(a) + (float)(b)))

WMM_DEFINE(float, f32, MUL_NATIVE, ADD_NATIVE)
WMM_DEFINE(double, f64, MUL_NATIVE, ADD_NATIVE)
WMM_DEFINE(_Float16, f16, MUL_HALF, ADD_HALF)

/*
 * Softmax over the band between the two operators, in double precision.  The reference ships no such
 * function: its callers compose it from torch ops (tests/test_attention.py:60-61, scores / sqrt(N), then
 * softmax over the last dimension); mask == 0 restates exactly that composition (every slot takes part
 * with the score stored there), mask != 0 is the same after setting the out-of-sequence slots (position
 * i + j - w outside [0, M)) to -inf, i.e. probability 0.  Pinned by tests/test_oracle.py against torch's
 * CPU softmax of the same composition.
 */
void wmm_oracle_band_softmax_f64(const double *scores, double *probs, long B, long M, long w, double scale,
                                 int mask) {
  const long W = 2 * w + 1;
  for (long r = 0; r < B * M; ++r) {
    const long i = r % M;
    const long jlo = mask ? WMM_MAX(0, w - i) : 0;
    const long jhi = mask ? WMM_MIN(W, M - i + w) : W;
    const double *x = scores + (size_t)r * W;
    double *p = probs + (size_t)r * W;
    double mx = -INFINITY, sum = 0.0;
    for (long j = jlo; j < jhi; ++j) mx = WMM_MAX(mx, x[j] * scale);
    for (long j = jlo; j < jhi; ++j) sum += exp(x[j] * scale - mx);
    for (long j = 0; j < W; ++j) p[j] = (j >= jlo && j < jhi) ? exp(x[j] * scale - mx) / sum : 0.0;
  }
}

/* grad_scores = scale * p * (grad_p - sum_j grad_p * p) over the slots that took part. */
void wmm_oracle_band_softmax_bw_f64(const double *probs, const double *gprobs, double *gscores, long B, long M,
                                    long w, double scale, int mask) {
  const long W = 2 * w + 1;
  for (long r = 0; r < B * M; ++r) {
    const long i = r % M;
    const long jlo = mask ? WMM_MAX(0, w - i) : 0;
    const long jhi = mask ? WMM_MIN(W, M - i + w) : W;
    const double *p = probs + (size_t)r * W, *g = gprobs + (size_t)r * W;
    double *o = gscores + (size_t)r * W;
    double dot = 0.0;
    for (long j = jlo; j < jhi; ++j) dot += p[j] * g[j];
    for (long j = 0; j < W; ++j) o[j] = (j >= jlo && j < jhi) ? scale * p[j] * (g[j] - dot) : 0.0;
  }
}

int wmm_oracle_abi_version(void) { return 2; }
