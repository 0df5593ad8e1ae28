/*
 * wmm_b200 -- C ABI of the B200 (sm_100a) banded-contraction library.
 *
 * This is the native boundary that replaces the reference's pybind module `window_matmul_kernel`
 * (csrc/window_matmul/window_matmul.cpp:74-106: window_matmul_forward/backward,
 * unwindow_matmul_forward/backward) and the CUDA launchers behind it
 * (csrc/window_matmul/cuda/window_matmul_cuda.cu:224-416).  No torch, pybind or C++ types cross it:
 * device pointers, sizes, element strides, a dtype code and the caller's stream.
 *
 * Contract common to every compute entry point
 *   - All pointers are DEVICE pointers on the CUDA device that is current in the calling thread.
 *   - The caller owns every buffer (inputs, outputs): the library never allocates, frees or
 *     synchronises.  Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = default
 *     stream) and the call returns at once.
 *   - Every element of every output is written (out-of-sequence band entries as exact zeros), so
 *     outputs may be uninitialised memory.  The reference zero-fills its outputs first
 *     (window_matmul_cuda.cu:242,290-291,338,377-378); that extra pass is not needed here.
 *   - Return value: WMM_OK or a negative wmm_status; no exception or abort crosses the boundary.
 *     wmm_last_error_string() gives the reason for the calling thread's last failure.
 *   - Re-entrant and thread safe; no mutable global state besides the per-thread error string,
 *     a launch counter and a device-side status word (see wmm_device_status).
 *
 * The three primitives.  With W = 2*window+1 and, for a band entry (i, j), the position
 * p = i + j - window + other_off in the row space of the other operand:
 *
 *   band_nt:  Band[b,i,j] = sum_h X[b,i,h] * Y[b,p,h]        if seq_lo <= p < seq_hi, else exactly 0
 *   band_n :  Out [b,i,h] = sum_{j : seq_lo <= p < seq_hi} Band[b,i,j] * Y[b,p,h]
 *   band_t :  Out [b,p,h] = sum_{i in [0,rows), 0 <= j <= 2*window} Band[b,i,j] * X[b,i,h]
 *                           for seq_lo <= p < seq_hi; rows p of Out outside that range are zeros
 *
 * X and Band have `rows` rows (batch entries of the band `band_stride_b` elements apart, by default contiguous); Y
 * (band_nt, band_n) and Out of band_t have `other_rows` rows.  The
 * plain, unsharded operators use other_rows = rows, other_off = 0, seq_lo = 0, seq_hi = rows.  A
 * sequence-sharded caller passes its local rows plus a halo: other_rows = rows + 2*window,
 * other_off = window, and seq_lo/seq_hi clip at the ends of the global sequence.
 *
 * Arithmetic: products are accumulated in float (double for WMM_F64) and rounded once to the element
 * type.  For WMM_F32 and WMM_F64 every output element is one sequential chain over the ascending
 * reduction index, fused multiply-add by default, which is the order of the reference's kernels
 * (window_matmul_cuda.cu:24-35,64-83); WMM_FLAG_SPLIT_ROUNDING rounds product and sum separately, which
 * reproduces the reference's CPU loops (cpu/window_matmul_cpu.cpp:43,92-93,137,186-187) bit for bit.
 * Both statements hold for FINITE inputs: band elements that do not exist (outside the band of a dense tile, outside
 * the sequence) enter the chains as zero terms, so an Inf or NaN in an operand row reaches every output row whose
 * tile covers it (0 * Inf), where the reference's loops touch only rows within `window`, and a sum of -0.0 comes
 * out as +0.0.
 */
#ifndef WMM_B200_H
#define WMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WMM_ABI_VERSION 3

#if defined(__GNUC__)
#define WMM_API __attribute__((visibility("default")))
#else
#define WMM_API
#endif

typedef enum wmm_dtype { WMM_F16 = 0, WMM_BF16 = 1, WMM_F32 = 2, WMM_F64 = 3 } wmm_dtype;

typedef enum wmm_status {
  WMM_OK = 0,
  WMM_ERR_NULL = -1,        /* a required pointer is NULL */
  WMM_ERR_SHAPE = -2,       /* the reference's "Input mismatch" cases and non-positive sizes */
  WMM_ERR_DTYPE = -3,       /* unknown dtype code */
  WMM_ERR_STRIDE = -4,      /* a stride this library cannot address (negative, or overlapping output) */
  WMM_ERR_TOO_LARGE = -5,   /* an extent or element count beyond the 31-bit / grid limits */
  WMM_ERR_CUDA = -6,        /* a CUDA runtime/driver call failed; see wmm_last_error_string() */
  WMM_ERR_UNSUPPORTED = -7, /* a flag combination that no kernel implements */
  WMM_ERR_DEVICE = -8       /* a kernel gave up on a bounded wait (see wmm_device_status) */
} wmm_status;

enum {
  /* fp32/fp64 only: round product and sum separately (bit parity with the reference's CPU loops). */
  WMM_FLAG_SPLIT_ROUNDING = 1u << 0,
  /* never take a tensor-core kernel, whatever the shape (testing, and exact fp32 ordering). */
  WMM_FLAG_FORCE_GENERIC = 1u << 1,
  /* fail with WMM_ERR_UNSUPPORTED instead of taking the CUDA-core kernels (testing the fast paths:
   * families 1 and 2 of wmm_query_path). */
  WMM_FLAG_REQUIRE_TENSOR = 1u << 2,
  /* wmm_band_softmax / wmm_band_softmax_bwd only: out-of-sequence slots take part in the softmax with the score
   * stored there (window_matmul writes 0), which is what a plain torch softmax over the band does
   * (tests/test_attention.py:60-61).  Without this flag those slots get probability exactly 0. */
  WMM_FLAG_SOFTMAX_KEEP_PADDING = 1u << 3,
  /* wmm_window_bwd only: take the one-sweep kernel (each box of grad_A staged once for both products) whenever the
   * shape allows it, also for small problems where the library would choose the two-pass kernel because the boxes a
   * CTA replays at the start of its run outweigh the saving (testing the kernel on small cases). */
  WMM_FLAG_PREFER_SWEEP = 1u << 4,
  /* WMM_F32 only: multiply on the tensor cores with the operands rounded to tf32 (10-bit mantissa) and fp32 sums,
   * wherever a tensor-core kernel takes the problem (wmm_query_path says which); results are then within about 2e-3
   * relative of the exact fp32 result instead of 1e-5.  Without the flag fp32 always takes the exact-order kernels.
   * The reference has one fp32 path (window_matmul_cuda.cu:257, AT_DISPATCH_FLOATING_TYPES_AND_HALF), exact. */
  WMM_FLAG_TF32 = 1u << 5
};

/* A (batch, rows, cols) operand addressed by ELEMENT strides: either of the two inner strides may be
 * the unit one, so K of window_matmul can be passed as the (B,N,M) tensor it is
 * (window_matmul/window_matmul.py:36-37) or as a transposed view of a (B,M,N) tensor, without the
 * transposing copy of window_matmul_cuda.cu:236. */
typedef struct wmm_operand {
  const void *data;
  int64_t stride_b; /* between batch entries */
  int64_t stride_r; /* between rows (sequence positions) */
  int64_t stride_c; /* between columns (hidden features) */
} wmm_operand;

typedef struct wmm_geometry {
  int32_t batch;      /* B: batch x heads, flattened */
  int32_t rows;       /* M: rows of X and of the band */
  int32_t cols;       /* N: hidden size */
  int32_t window;     /* w >= 0; the band has 2*w+1 columns */
  int32_t other_rows; /* rows of Y (band_nt, band_n) / of Out (band_t) */
  int32_t other_off;  /* position of band entry (i=0, j=window) in that row space */
  int32_t seq_lo;     /* positions seq_lo <= p < seq_hi are inside the sequence */
  int32_t seq_hi;
  int64_t band_stride_b; /* elements between batch entries of the band tensor; 0 = rows * (2*window+1), i.e. contiguous.
                          * A larger stride addresses a range of rows of a longer band tensor (the interior rows of a
                          * sequence shard, say) in place; only the tensor-core kernels take it. */
} wmm_geometry;

/* ---- library / diagnostics ------------------------------------------------------------------- */

/* WMM_ABI_VERSION the library was built with. */
WMM_API int wmm_version(void);
/* Reason for the calling thread's most recent non-zero return (never NULL). */
WMM_API const char *wmm_last_error_string(void);
/* Static name of a status code. */
WMM_API const char *wmm_status_string(int status);
/* Number of kernels this library has launched in this process so far (all threads). */
WMM_API uint64_t wmm_launch_count(void);
/* Caps the grid of the launches that follow (process-wide, read when a launch is issued or captured; 0 = no cap, the
 * default): `contraction_ctas` for the persistent tensor-core kernels (one CTA per SM otherwise), `exchange_ctas` for
 * wmm_halo_pull / wmm_halo_pull_static (then one CTA per SM, large enough to keep the SM to itself, with eight times the
 * loads in flight).  For a caller that runs an exchange on one stream beside a contraction on another: with, say, 140 and
 * 8 on a 148-SM device the contraction leaves 8 SMs and the exchange runs there instead of waiting for an SM with room.  Results do not depend on the caps.  The reference
 * has no counterpart (it runs one kernel at a time).  Negative values fail with WMM_ERR_SHAPE. */
WMM_API int wmm_set_cta_limits(int contraction_ctas, int exchange_ctas);
/* Reads (and, if `clear` is non-zero, resets) the status word that a kernel sets when one of its bounded
 * waits runs out.  0 = clean.  Synchronises the current device.  Returns the word, or a negative status. */
WMM_API int64_t wmm_device_status(int clear);
/* Which kernel family the dispatcher picks for a problem: 0 = exact-order CUDA-core kernels, 1 = tcgen05
 * kernels, 2 = small-window kernels (w <= 32; warp-level MMAs fed from coalesced shared-memory tiles).  `primitive` is 1 (band_nt), 2 (band_n) or 3 (band_t); the operands carry the
 * strides and alignment that decide; pass the same arguments as to the compute call.  Negative = status. */
WMM_API int wmm_query_path(int primitive, const wmm_operand *a, const wmm_operand *b, const void *band,
                   const wmm_geometry *g, int dtype, unsigned flags);

/* ---- the three primitives --------------------------------------------------------------------- */

/* Band = band(X * Y^T): replaces the kernel window_matmul_kernel (window_matmul_cuda.cu:37-91), used by
 * window_matmul_fw_cuda (:224-270; X=Q, Y=K^T) and for grad_A in unwindow_matmul_bw_cuda (:403-408;
 * X=grad_O, Y=V).  `band` is a contiguous (batch, rows, 2w+1) output. */
WMM_API int wmm_band_nt(const wmm_operand *x, const wmm_operand *y, void *band, const wmm_geometry *g, int dtype,
                unsigned flags, void *stream);

/* Out = unskew(Band) * Y: replaces unwindow_matmul_kernel_A (window_matmul_cuda.cu:93-156), used by
 * unwindow_matmul_fw_cuda (:321-358; Y=V) and for grad_Q in window_matmul_bw_cuda (:308-312; Band=grad_A,
 * Y=K^T).  `band` is a contiguous (batch, rows, 2w+1) input; `out` is written through its strides. */
WMM_API int wmm_band_n(const void *band, const wmm_operand *y, const wmm_operand *out, const wmm_geometry *g,
               int dtype, unsigned flags, void *stream);

/* Out = unskew(Band)^T * X: replaces unwindow_matmul_kernel_B (window_matmul_cuda.cu:158-222), used for
 * grad_K in window_matmul_bw_cuda (:313-317; Band=grad_A, X=Q) and grad_V in unwindow_matmul_bw_cuda
 * (:409-414; Band=A, X=grad_O).  Out has g->other_rows rows. */
WMM_API int wmm_band_t(const void *band, const wmm_operand *x, const wmm_operand *out, const wmm_geometry *g,
               int dtype, unsigned flags, void *stream);

/* ---- the two backward passes ------------------------------------------------------------------- */

/* grad_Q = band_n(grad_A, K^T), grad_K^T = band_t(grad_A, Q): replaces window_matmul_bw_cuda
 * (window_matmul_cuda.cu:272-319).  kt / grad_kt are K and grad_K in (batch, rows, cols) index order
 * (pass a (B,N,M) tensor with its two inner strides swapped).  Plain geometry only
 * (other_rows = rows, other_off = 0); sharded callers use the primitives. */
WMM_API int wmm_window_bwd(const wmm_operand *q, const wmm_operand *kt, const void *grad_band,
                   const wmm_operand *grad_q, const wmm_operand *grad_kt, const wmm_geometry *g, int dtype,
                   unsigned flags, void *stream);

/* grad_A = band_nt(grad_O, V), grad_V = band_t(A, grad_O): replaces unwindow_matmul_bw_cuda
 * (window_matmul_cuda.cu:360-416).  Plain geometry only. */
WMM_API int wmm_unwindow_bwd(const void *band, const wmm_operand *v, const wmm_operand *grad_o, void *grad_band,
                     const wmm_operand *grad_v, const wmm_geometry *g, int dtype, unsigned flags,
                     void *stream);

/* ---- softmax over the band (between the two operators) ------------------------------------------ */

/* probs[b,i,:] = softmax_j(scale * scores[b,i,j]) over the slots j whose position i + j - window + other_off lies in
 * [seq_lo, seq_hi); the other slots get probability 0 (or take part, WMM_FLAG_SOFTMAX_KEEP_PADDING).  One pass over
 * HBM; `probs` may equal `scores`.  Both are contiguous (batch, rows, 2*window+1), 16-byte aligned; g->cols is not
 * used.  Replaces the torch ops a caller of the reference puts between the two operators
 * (tests/test_attention.py:60-61: `att_scores / sqrt(N)`, `softmax(att_scores, dim=-1)`), plus the -inf mask for
 * the out-of-sequence slots that the reference leaves to the caller. */
WMM_API int wmm_band_softmax(const void *scores, void *probs, const wmm_geometry *g, int dtype, float scale,
                             unsigned flags, void *stream);

/* grad_scores = scale * probs * (grad_probs - sum_j grad_probs * probs), slot rule as in the forward.
 * `grad_scores` may equal `grad_probs`. */
WMM_API int wmm_band_softmax_bwd(const void *probs, const void *grad_probs, void *grad_scores,
                                 const wmm_geometry *g, int dtype, float scale, unsigned flags, void *stream);

/* ---- sequence shards: neighbour exchange through peer memory ---------------------------------- */

/* A sharded operand in its "extended" buffer: contiguous (batch, rows + 2*window, cols) = w margin rows, the rank's own
 * rows, w margin rows.  `local` is this rank's buffer, `lower` / `upper` the SAME tensor's buffer on the rank that owns
 * the rows before / after (pointers that this device can load from: peer-mapped or symmetric memory), NULL at an end of
 * the global sequence.  All 16-byte aligned. */
typedef struct wmm_halo_buffer {
  void *local;
  const void *lower;
  const void *upper;
} wmm_halo_buffer;

/* Flag words of the hand-shake.  `mine`, `lower`, `upper`: this rank's and the neighbours' blocks of at least 4
 * 32-bit words in memory every neighbour can read AND write (word 0: ready epoch, word 1 / 2: acknowledgement written
 * by the lower / upper neighbour), zero before the first call; NULL for a missing neighbour.  `counters`: 4 words of
 * plain device memory of this rank, zero before the first call (word 0: exchanges completed; words 1-3: scratch of the
 * running launch). */
typedef struct wmm_halo_flags {
  unsigned *mine;
  unsigned *lower;
  unsigned *upper;
  unsigned *counters;
} wmm_halo_flags;

/* One neighbour exchange for up to 4 tensors of the same shape, in ONE kernel launch on `stream`:
 *   accumulate == 0: each buffer's lower margin <- the lower neighbour's last `window` own rows, upper margin <- the upper
 *                    neighbour's first `window` own rows (halo rows of K^T and V before the forward contractions);
 *   accumulate != 0: this rank's first `window` own rows += the lower neighbour's upper margin, its last `window` own rows
 *                    += the upper neighbour's lower margin (partial grad_K / grad_V rows after the backward contractions;
 *                    needs rows >= 2*window).
 * Every rank of the sequence group must issue the same sequence of these calls.  The kernel waits for the neighbours'
 * kernels of the same call: at most ~1 s for a neighbour to start (a side whose neighbour does not show up is skipped, the
 * other side is still served) and at most ~3 s for a neighbour to finish reading this rank's rows; a wait that runs out
 * sets bit 5 of wmm_device_status().  The
 * reference has no multi-GPU code; this replaces the send/recv pairs of a host communication library on that path. */
WMM_API int wmm_halo_pull(const wmm_halo_buffer *buffers, int count, const wmm_halo_flags *flags, int batch, int rows,
                          int cols, int window, int dtype, int accumulate, void *stream);

/* wmm_halo_pull for callers that cannot allocate device memory.  No counterpart in the reference (it has no multi-GPU
 * code).  Some users of this library run where cudaMalloc is not an option: an inference server that has handed all
 * device memory to its own pool at start-up, a plugin called from a host callback or in the middle of a stream capture,
 * where the runtime refuses allocations, or a real-time loop that must not take the allocator's lock.  wmm_halo_pull
 * asks such a caller for four words of device memory (`counters`) that it has no good way to provide.  This entry
 * point does the same exchange with those scratch words in a static device array inside the library instead:
 * WMM_HALO_STATIC_LANES lanes of 256 bytes (2 KB in all), which every GPU that loads the library holds until the
 * process exits.  It calls no allocation routine of any kind (no cudaMalloc / cudaFree, nothing of torch).
 *   - `flags->counters` is not used (pass NULL).  The count of completed exchanges lives in word 3 of the caller's own
 *     flag block `flags->mine` (which must therefore have its 4 words zeroed before the first call, like the rest of
 *     the block), so a fresh flag block starts a fresh count whatever the lane was used for before.
 *   - `lane` picks the scratch words: 0 <= lane < WMM_HALO_STATIC_LANES, anything else fails with WMM_ERR_TOO_LARGE.
 *     All calls on a lane share its words; the call clears them (stream-ordered) before its kernel runs, so nothing of
 *     an earlier call is carried over, but two calls on the SAME lane that overlap on the GPU (different streams,
 *     no ordering between them) race.  Give sequence groups that may run at the same time different lanes.
 *   - The first call on each device looks up the array's device address (with that device current).  Make that first
 *     call outside of any stream capture.
 * Everything else (buffers, flag hand-shake, waits, status bit 5) is as for wmm_halo_pull. */
#define WMM_HALO_STATIC_LANES 8
WMM_API int wmm_halo_pull_static(const wmm_halo_buffer *buffers, int count, const wmm_halo_flags *flags, int lane,
                                 int batch, int rows, int cols, int window, int dtype, int accumulate, void *stream);

/* ---- sequence shards: partial grad_K / grad_V rows summed with one rounding less ------------------------------ */

/* wmm_band_t for the 16-bit types that also writes output rows near both ends UNROUNDED, as fp32, into `edges`: a
 * contiguous (batch, 2 * edge_rows, cols) buffer whose rows [0, edge_rows) stand for output rows [0, edge_rows) and
 * whose rows [edge_rows, 2 * edge_rows) for output rows [other_rows - edge_rows, other_rows); the outermost `edge_skip`
 * rows at each end are not written.  A sequence shard computes partial grad_K / grad_V rows for its margins and for its
 * own rows next to them (edge_rows = 2 * window, edge_skip = window: the fp32 rows are its own first and last `window`
 * rows); adding a neighbour's partial row to an own row that was already rounded to 16 bits costs a rounding the
 * unsharded kernel does not have.  With the fp32 copy and wmm_halo_reduce_edges the own terms are not rounded before the
 * sum.  Only the tensor-core kernels write edge rows: other dtypes and shapes fail with WMM_ERR_UNSUPPORTED; needs
 * 2 * edge_rows <= other_rows, 0 <= edge_skip < edge_rows and `edges` 16-byte aligned.  No counterpart in the reference
 * (it has no multi-GPU code). */
WMM_API int wmm_band_t_edges(const void *band, const wmm_operand *x, const wmm_operand *out, float *edges, int edge_rows,
                             int edge_skip, const wmm_geometry *g, int dtype, unsigned flags, void *stream);

/* One tensor of wmm_halo_reduce_edges: `local` = this rank's extended (batch, rows + 2*window, cols) partial-row buffer
 * of the 16-bit type (its own rows are the result), `mine` = the fp32 edge rows (batch, 4*window, cols) that
 * wmm_band_t_edges wrote on this rank with edge_rows = 2*window, edge_skip = window, `lower` / `upper` = the neighbours'
 * extended 16-bit buffers of the same tensor as in wmm_halo_buffer (peer pointers; NULL at an end of the sequence). */
typedef struct wmm_halo_edges {
  void *local;
  const float *mine;
  const void *lower;
  const void *upper;
} wmm_halo_edges;

/* The reduction of wmm_halo_pull(accumulate != 0) with this rank's terms taken from its fp32 edge rows: its first
 * `window` own rows <- round(its unrounded rows + the lower neighbour's upper-margin rows), its last `window` own rows
 * likewise with the upper neighbour's lower-margin rows.  The neighbours' rows cross the link in 16 bits, as in
 * wmm_halo_pull.  Same hand-shake, waits and status bit; WMM_F16 / WMM_BF16 only, cols a multiple of 8,
 * rows >= 2*window. */
WMM_API int wmm_halo_reduce_edges(const wmm_halo_edges *tensors, int count, const wmm_halo_flags *flags, int batch,
                                  int rows, int cols, int window, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* WMM_B200_H */
