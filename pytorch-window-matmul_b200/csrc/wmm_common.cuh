// Shared declarations of the banded-contraction kernels (internal; the public surface is include/wmm_b200.h).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <atomic>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wmm_b200.h"

namespace wmm {

// One banded contraction, after validation.  `a` is the first operand in the order of the public
// entry point (X for band_nt, the band for band_n / band_t), `b` the second, `o` the output.  The band
// is always contiguous (batch, rows, 2w+1) and carries no strides.
struct Problem {
  const void *a;
  const void *b;
  void *o;
  int64_t a_sb, a_sr, a_sc;
  int64_t b_sb, b_sr, b_sc;
  int64_t o_sb, o_sr, o_sc;
  int32_t B, M, N, w;      // batch, rows of X / band, hidden size, window
  int32_t Mo, off, lo, hi; // rows of the other row space, its offset, in-sequence range
  int64_t band_sb;         // elements between batch entries of the band (M * (2w+1) when contiguous)
  int32_t dtype;
  uint32_t flags;
  // band_t on 16-bit types only: the first and the last `edge_rows` output rows (minus the outermost `edge_skip` at each
  // end) once more, unrounded, as fp32 rows of a (B, 2 * edge_rows, N) contiguous buffer; NULL = none
  float *edges;
  int32_t edge_rows, edge_skip;
};

enum Primitive { BAND_NT = 1, BAND_N = 2, BAND_T = 3 };

// Launchers.  Each returns cudaSuccess or the launch error; `launches` is incremented per kernel.
cudaError_t launch_generic(Primitive prim, const Problem &p, cudaStream_t stream, int *launches);

// Tensor-core (tcgen05) family: `eligible` is a pure host-side predicate on shape, dtype, strides and
// alignment; `launch_tensor` must only be called when it holds.
bool tensor_eligible(Primitive prim, const Problem &p);
cudaError_t launch_tensor(Primitive prim, const Problem &p, cudaStream_t stream, int *launches);
// band_n and band_t over the same band in ONE launch (the band is fetched from HBM once): `pn` and `pt`
// are the two problems; eligibility includes that they share band, geometry and dtype.
bool tensor_fused_pair_eligible(const Problem &pn, const Problem &pt);
cudaError_t launch_tensor_fused_pair(const Problem &pn, const Problem &pt, cudaStream_t stream, int *launches);

// Small-window family (w <= 32, 16-bit): warp-level MMAs fed from coalesced shared-memory tiles.
bool small_eligible(Primitive prim, const Problem &p);
cudaError_t launch_small(Primitive prim, const Problem &p, cudaStream_t stream, int *launches);

// Masked, scaled softmax over band rows (forward: in = scores; backward: in = probabilities, in2 = their gradient).
cudaError_t launch_band_softmax(bool backward, const void *in, const void *in2, void *out, const wmm_geometry &g,
                                int dtype, float scale, bool mask, cudaStream_t stream, int *launches);

// Neighbour exchange of halo rows through peer memory (wmm_halo.cu).
// `epoch_word`: one local word counting the completed exchanges; `scratch`: three local words (CTAs done, go word per side).
cudaError_t launch_halo_pull(const wmm_halo_buffer *bufs, int count, const wmm_halo_flags &flags, unsigned *epoch_word,
                             unsigned *scratch, int batch, int rows, int cols, int window, int dtype, bool accumulate,
                             cudaStream_t stream, int *launches, const wmm_halo_edges *edges = nullptr);

// The same exchange with its scratch words in a static device array of the library (lane < WMM_HALO_STATIC_LANES) and
// the exchange count in word 3 of flags.mine; no device memory is allocated.
cudaError_t launch_halo_pull_static(const wmm_halo_buffer *bufs, int count, const wmm_halo_flags &flags, int lane, int batch,
                                    int rows, int cols, int window, int dtype, bool accumulate, cudaStream_t stream,
                                    int *launches);

// Process-wide caps on the grid of the persistent tensor-core contractions and of the halo exchange (0 = none), set by
// wmm_set_cta_limits and read at launch time: a caller that runs an exchange beside a contraction gives each its SMs.
extern std::atomic<int> g_contraction_cta_limit;
extern std::atomic<int> g_exchange_cta_limit;

// Launchers describe a failure (which step, which driver code) here; the API layer appends it to the
// error string of the calling thread.
void set_launch_detail(const char *fmt, ...);
const char *launch_detail();

// Device-side status word: a kernel that abandons a bounded wait ORs a code into it.  Synchronises the
// current device, copies the word out and optionally clears it.
cudaError_t read_device_status(unsigned long long *word, bool clear);
// Address of that word on the current device (for kernels of other translation units); NULL on failure.
unsigned long long *device_status_word();

template <typename T> struct ElemTraits;
template <> struct ElemTraits<float> {
  using Acc = float;
  static __device__ __forceinline__ float load(const float *p) { return *p; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct ElemTraits<double> {
  using Acc = double;
  static __device__ __forceinline__ double load(const double *p) { return *p; }
  static __device__ __forceinline__ double store(double v) { return v; }
};
template <> struct ElemTraits<__half> {
  using Acc = float;
  static __device__ __forceinline__ float load(const __half *p) { return __half2float(*p); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};
template <> struct ElemTraits<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};

}  // namespace wmm
