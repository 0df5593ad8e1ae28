// The C ABI (include/wmm_b200.h): argument validation, kernel-family dispatch, error reporting.
// Nothing here allocates device memory or synchronises, except wmm_device_status().
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "wmm_common.cuh"

namespace {

thread_local char tls_error[512] = "no error";
std::atomic<uint64_t> g_launches{0};
}  // namespace
namespace wmm {
std::atomic<int> g_contraction_cta_limit{0};
std::atomic<int> g_exchange_cta_limit{0};
}  // namespace wmm
namespace {

int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
  return status;
}

size_t elem_size(int dtype) {
  switch (dtype) {
    case WMM_F16:
    case WMM_BF16: return 2;
    case WMM_F32: return 4;
    case WMM_F64: return 8;
    default: return 0;
  }
}

int check_geometry(const wmm_geometry *g, int dtype, unsigned flags) {
  if (!g) return fail(WMM_ERR_NULL, "geometry is NULL");
  if (elem_size(dtype) == 0) return fail(WMM_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (g->batch < 0 || g->rows < 0 || g->cols < 0 || g->other_rows < 0 || g->window < 0)
    return fail(WMM_ERR_SHAPE, "Input mismatch: negative extent (batch %d rows %d cols %d other_rows %d window %d)",
                g->batch, g->rows, g->cols, g->other_rows, g->window);
  if (g->seq_lo < 0 || g->seq_lo > g->seq_hi || g->seq_hi > g->other_rows)
    return fail(WMM_ERR_SHAPE, "Input mismatch: sequence range [%d,%d) not inside [0,%d)", g->seq_lo, g->seq_hi,
                g->other_rows);
  if (g->window > (1 << 28) || (int64_t)g->rows + 2ll * g->window + 256 > 0x7fffffffLL ||
      (int64_t)g->other_rows + 2ll * g->window + 256 > 0x7fffffffLL ||
      (int64_t)(g->other_off < 0 ? -(int64_t)g->other_off : g->other_off) > (1ll << 30))
    return fail(WMM_ERR_TOO_LARGE, "extent beyond the 31-bit index range");
  if (g->band_stride_b != 0 && g->band_stride_b < (int64_t)g->rows * (2ll * g->window + 1))
    return fail(WMM_ERR_STRIDE, "band batch stride %lld is smaller than a batch entry (%d rows of %d)", (long long)g->band_stride_b,
                g->rows, 2 * g->window + 1);
  if ((flags & WMM_FLAG_FORCE_GENERIC) && (flags & WMM_FLAG_REQUIRE_TENSOR))
    return fail(WMM_ERR_UNSUPPORTED, "FORCE_GENERIC and REQUIRE_TENSOR exclude each other");
  if ((flags & WMM_FLAG_SPLIT_ROUNDING) && (flags & WMM_FLAG_REQUIRE_TENSOR))
    return fail(WMM_ERR_UNSUPPORTED, "split rounding exists only in the CUDA-core kernels");
  return WMM_OK;
}

int check_operand(const wmm_operand *op, const char *name, bool is_output, bool empty) {
  if (!op) return fail(WMM_ERR_NULL, "operand %s is NULL", name);
  if (!op->data && !empty) return fail(WMM_ERR_NULL, "operand %s has a NULL data pointer", name);
  if (op->stride_b < 0 || op->stride_r < 0 || op->stride_c < 0)
    return fail(WMM_ERR_STRIDE, "operand %s has a negative stride", name);
  if (is_output && (op->stride_r == 0 || op->stride_c == 0) && !empty)
    return fail(WMM_ERR_STRIDE, "output %s has a zero stride (overlapping elements)", name);
  return WMM_OK;
}

void fill(wmm::Problem &p, const wmm_geometry *g, int dtype, unsigned flags) {
  p.B = g->batch;
  p.M = g->rows;
  p.N = g->cols;
  p.w = g->window;
  p.Mo = g->other_rows;
  p.off = g->other_off;
  p.lo = g->seq_lo;
  p.hi = g->seq_hi;
  p.band_sb = g->band_stride_b ? g->band_stride_b : (int64_t)g->rows * (2ll * g->window + 1);
  p.dtype = dtype;
  p.flags = flags;
}

void set_a(wmm::Problem &p, const wmm_operand *x) {
  p.a = x->data;
  p.a_sb = x->stride_b;
  p.a_sr = x->stride_r;
  p.a_sc = x->stride_c;
}
void set_b(wmm::Problem &p, const wmm_operand *x) {
  p.b = x->data;
  p.b_sb = x->stride_b;
  p.b_sr = x->stride_r;
  p.b_sc = x->stride_c;
}
void set_o(wmm::Problem &p, const wmm_operand *x) {
  p.o = const_cast<void *>(x->data);
  p.o_sb = x->stride_b;
  p.o_sr = x->stride_r;
  p.o_sc = x->stride_c;
}
void set_band_a(wmm::Problem &p, const void *band) {
  p.a = band;
  p.a_sb = p.a_sr = p.a_sc = 0;
}
void set_band_o(wmm::Problem &p, void *band) {
  p.o = band;
  p.o_sb = p.o_sr = p.o_sc = 0;
}

// Kernel family for a problem: 0 = exact-order CUDA-core kernels, 1 = tcgen05 kernels, 2 = small-window kernels.
int pick_family(wmm::Primitive prim, const wmm::Problem &p) {
  if (p.flags & (WMM_FLAG_FORCE_GENERIC | WMM_FLAG_SPLIT_ROUNDING)) return 0;
  if (wmm::small_eligible(prim, p)) return 2;
  if (wmm::tensor_eligible(prim, p)) return 1;
  return 0;
}

bool wants_tensor(wmm::Primitive prim, const wmm::Problem &p) { return pick_family(prim, p) == 1; }

int dispatch(wmm::Primitive prim, const wmm::Problem &p, void *stream) {
  const int family = pick_family(prim, p);
  if (family == 0 && (p.flags & WMM_FLAG_REQUIRE_TENSOR))
    return fail(WMM_ERR_UNSUPPORTED, "no tensor-core kernel takes this problem (primitive %d)", (int)prim);
  if (family != 1 && p.band_sb != (int64_t)p.M * (2ll * p.w + 1))
    return fail(WMM_ERR_STRIDE, "a band with a batch stride is taken by the tensor-core kernels only (primitive %d)", (int)prim);
  int launches = 0;
  cudaError_t e = family == 1   ? wmm::launch_tensor(prim, p, (cudaStream_t)stream, &launches)
                  : family == 2 ? wmm::launch_small(prim, p, (cudaStream_t)stream, &launches)
                                : wmm::launch_generic(prim, p, (cudaStream_t)stream, &launches);
  g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
  if (e != cudaSuccess)
    return fail(WMM_ERR_CUDA, "CUDA error launching primitive %d: %s [%s]", (int)prim, cudaGetErrorString(e),
                family == 1 ? wmm::launch_detail() : family == 2 ? "small-window kernel launch" : "generic kernel launch");
  return WMM_OK;
}

// Problems with no output element need no launch; outputs with elements but an empty reduction are
// handled by the kernels (they write zeros).
bool nothing_to_write(wmm::Primitive prim, const wmm_geometry *g) {
  if (g->batch == 0 || g->cols == 0 && prim != wmm::BAND_NT) return true;
  if (prim == wmm::BAND_T) return g->other_rows == 0;
  return g->rows == 0;
}

int build(wmm::Primitive prim, wmm::Problem &p, const wmm_operand *x, const wmm_operand *y, const void *band_in,
          void *band_out, const wmm_operand *out, const wmm_geometry *g, int dtype, unsigned flags) {
  if (int s = check_geometry(g, dtype, flags)) return s;
  const bool empty = nothing_to_write(prim, g);
  fill(p, g, dtype, flags);
  switch (prim) {
    case wmm::BAND_NT:
      if (int s = check_operand(x, "x", false, empty || g->cols == 0)) return s;
      if (int s = check_operand(y, "y", false, empty || g->cols == 0 || g->other_rows == 0)) return s;
      if (!band_out && !empty) return fail(WMM_ERR_NULL, "band output is NULL");
      set_a(p, x);
      set_b(p, y);
      set_band_o(p, band_out);
      break;
    case wmm::BAND_N:
      if (!band_in && !empty) return fail(WMM_ERR_NULL, "band input is NULL");
      if (int s = check_operand(y, "y", false, empty || g->other_rows == 0)) return s;
      if (int s = check_operand(out, "out", true, empty)) return s;
      set_band_a(p, band_in);
      set_b(p, y);
      set_o(p, out);
      break;
    default:
      if (!band_in && !empty && g->rows > 0) return fail(WMM_ERR_NULL, "band input is NULL");
      if (int s = check_operand(x, "x", false, empty || g->rows == 0)) return s;
      if (int s = check_operand(out, "out", true, empty)) return s;
      set_band_a(p, band_in);
      set_b(p, x);
      set_o(p, out);
      break;
  }
  return empty ? 1 : WMM_OK;  // 1: valid, nothing to do
}

int plain_geometry(const wmm_geometry *g) {
  if (g && (g->other_rows != g->rows || g->other_off != 0))
    return fail(WMM_ERR_SHAPE, "Input mismatch: the fused backward entry points take the plain geometry only");
  return WMM_OK;
}

}  // namespace

extern "C" {

int wmm_version(void) { return WMM_ABI_VERSION; }

const char *wmm_last_error_string(void) { return tls_error; }

const char *wmm_status_string(int status) {
  switch (status) {
    case WMM_OK: return "WMM_OK";
    case WMM_ERR_NULL: return "WMM_ERR_NULL";
    case WMM_ERR_SHAPE: return "WMM_ERR_SHAPE";
    case WMM_ERR_DTYPE: return "WMM_ERR_DTYPE";
    case WMM_ERR_STRIDE: return "WMM_ERR_STRIDE";
    case WMM_ERR_TOO_LARGE: return "WMM_ERR_TOO_LARGE";
    case WMM_ERR_CUDA: return "WMM_ERR_CUDA";
    case WMM_ERR_UNSUPPORTED: return "WMM_ERR_UNSUPPORTED";
    case WMM_ERR_DEVICE: return "WMM_ERR_DEVICE";
    default: return "WMM_ERR_UNKNOWN";
  }
}

static int band_softmax_common(bool backward, const void *in, const void *in2, void *out, const wmm_geometry *g,
                               int dtype, float scale, unsigned flags, void *stream) {
  if (int s = check_geometry(g, dtype, 0u)) return s;
  if (flags & ~(unsigned)WMM_FLAG_SOFTMAX_KEEP_PADDING)
    return fail(WMM_ERR_UNSUPPORTED, "the band softmax takes no flag but WMM_FLAG_SOFTMAX_KEEP_PADDING");
  if ((int64_t)g->batch * g->rows == 0) return WMM_OK;
  if (g->band_stride_b != 0 && g->band_stride_b != (int64_t)g->rows * (2ll * g->window + 1))
    return fail(WMM_ERR_STRIDE, "the band softmax takes contiguous band tensors only");
  if (!in || !out || (backward && !in2)) return fail(WMM_ERR_NULL, "a band pointer is NULL");
  if (((uintptr_t)in | (uintptr_t)out | (uintptr_t)in2) & 15)
    return fail(WMM_ERR_STRIDE, "band tensors of the softmax must be 16-byte aligned");
  if (!(scale == scale)) return fail(WMM_ERR_SHAPE, "Input mismatch: scale is NaN");
  int launches = 0;
  cudaError_t e = wmm::launch_band_softmax(backward, in, in2, out, *g, dtype, scale,
                                           !(flags & WMM_FLAG_SOFTMAX_KEEP_PADDING), (cudaStream_t)stream, &launches);
  g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
  if (e != cudaSuccess) return fail(WMM_ERR_CUDA, "CUDA error launching the band softmax: %s", cudaGetErrorString(e));
  return WMM_OK;
}

int wmm_band_softmax(const void *scores, void *probs, const wmm_geometry *g, int dtype, float scale, unsigned flags,
                     void *stream) {
  return band_softmax_common(false, scores, nullptr, probs, g, dtype, scale, flags, stream);
}

int wmm_band_softmax_bwd(const void *probs, const void *grad_probs, void *grad_scores, const wmm_geometry *g,
                         int dtype, float scale, unsigned flags, void *stream) {
  return band_softmax_common(true, probs, grad_probs, grad_scores, g, dtype, scale, flags, stream);
}

int wmm_halo_pull(const wmm_halo_buffer *buffers, int count, const wmm_halo_flags *flags, int batch, int rows, int cols,
                  int window, int dtype, int accumulate, void *stream) {
  if (!buffers || !flags) return fail(WMM_ERR_NULL, "halo buffers or flags are NULL");
  if (count < 1 || count > 4) return fail(WMM_ERR_SHAPE, "Input mismatch: 1 to 4 buffers per exchange, got %d", count);
  const size_t e = elem_size(dtype);
  if (e == 0) return fail(WMM_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (batch < 0 || rows < 0 || cols < 0 || window < 0)
    return fail(WMM_ERR_SHAPE, "Input mismatch: negative extent (batch %d rows %d cols %d window %d)", batch, rows, cols, window);
  if (rows < (accumulate ? 2 : 1) * (int64_t)window)
    return fail(WMM_ERR_SHAPE, "Input mismatch: a shard of %d rows is too short for window %d", rows, window);
  if ((int64_t)batch * cols * window == 0) return WMM_OK;
  if (((int64_t)cols * e) % 16 != 0) return fail(WMM_ERR_STRIDE, "a row of %d elements is not a multiple of 16 bytes", cols);
  if (!flags->mine || !flags->counters) return fail(WMM_ERR_NULL, "flag block or counters are NULL");
  for (int i = 0; i < count; ++i) {
    if (!buffers[i].local) return fail(WMM_ERR_NULL, "buffer %d has a NULL local pointer", i);
    if (((uintptr_t)buffers[i].local | (uintptr_t)buffers[i].lower | (uintptr_t)buffers[i].upper) & 15)
      return fail(WMM_ERR_STRIDE, "buffer %d is not 16-byte aligned", i);
    if ((buffers[i].lower != nullptr) != (flags->lower != nullptr) || (buffers[i].upper != nullptr) != (flags->upper != nullptr))
      return fail(WMM_ERR_NULL, "buffer %d and the flags disagree on which neighbours exist", i);
  }
  int launches = 0;
  cudaError_t err = wmm::launch_halo_pull(buffers, count, *flags, flags->counters, flags->counters + 1, batch, rows, cols, window,
                                          dtype, accumulate != 0, (cudaStream_t)stream, &launches);
  g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
  if (err != cudaSuccess) return fail(WMM_ERR_CUDA, "CUDA error launching the halo exchange: %s", cudaGetErrorString(err));
  return WMM_OK;
}

// The neighbour exchange for callers that must not allocate: see include/wmm_b200.h.  Same checks as wmm_halo_pull, minus
// the counters (the scratch words are the library's own), plus the lane.
int wmm_halo_pull_static(const wmm_halo_buffer *buffers, int count, const wmm_halo_flags *flags, int lane, int batch,
                         int rows, int cols, int window, int dtype, int accumulate, void *stream) {
  if (!buffers || !flags) return fail(WMM_ERR_NULL, "halo buffers or flags are NULL");
  if (lane < 0 || lane >= WMM_HALO_STATIC_LANES)
    return fail(WMM_ERR_TOO_LARGE, "lane %d is outside the library's static scratch: it holds %d lanes (0 .. %d)", lane,
                WMM_HALO_STATIC_LANES, WMM_HALO_STATIC_LANES - 1);
  if (count < 1 || count > 4) return fail(WMM_ERR_SHAPE, "Input mismatch: 1 to 4 buffers per exchange, got %d", count);
  const size_t e = elem_size(dtype);
  if (e == 0) return fail(WMM_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (batch < 0 || rows < 0 || cols < 0 || window < 0)
    return fail(WMM_ERR_SHAPE, "Input mismatch: negative extent (batch %d rows %d cols %d window %d)", batch, rows, cols, window);
  if (rows < (accumulate ? 2 : 1) * (int64_t)window)
    return fail(WMM_ERR_SHAPE, "Input mismatch: a shard of %d rows is too short for window %d", rows, window);
  if ((int64_t)batch * cols * window == 0) return WMM_OK;
  if (((int64_t)cols * e) % 16 != 0) return fail(WMM_ERR_STRIDE, "a row of %d elements is not a multiple of 16 bytes", cols);
  if (!flags->mine) return fail(WMM_ERR_NULL, "flag block is NULL");
  for (int i = 0; i < count; ++i) {
    if (!buffers[i].local) return fail(WMM_ERR_NULL, "buffer %d has a NULL local pointer", i);
    if (((uintptr_t)buffers[i].local | (uintptr_t)buffers[i].lower | (uintptr_t)buffers[i].upper) & 15)
      return fail(WMM_ERR_STRIDE, "buffer %d is not 16-byte aligned", i);
    if ((buffers[i].lower != nullptr) != (flags->lower != nullptr) || (buffers[i].upper != nullptr) != (flags->upper != nullptr))
      return fail(WMM_ERR_NULL, "buffer %d and the flags disagree on which neighbours exist", i);
  }
  int launches = 0;
  cudaError_t err = wmm::launch_halo_pull_static(buffers, count, *flags, lane, batch, rows, cols, window, dtype, accumulate != 0,
                                                 (cudaStream_t)stream, &launches);
  g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
  if (err != cudaSuccess)
    return fail(WMM_ERR_CUDA, "CUDA error in the halo exchange on static scratch (lane %d): %s", lane, cudaGetErrorString(err));
  return WMM_OK;
}

// The reduction of partial rows from unrounded fp32 edge rows (see include/wmm_b200.h).
int wmm_halo_reduce_edges(const wmm_halo_edges *tensors, int count, const wmm_halo_flags *flags, int batch, int rows,
                          int cols, int window, int dtype, void *stream) {
  if (!tensors || !flags) return fail(WMM_ERR_NULL, "edge tensors or flags are NULL");
  if (count < 1 || count > 4) return fail(WMM_ERR_SHAPE, "Input mismatch: 1 to 4 tensors per reduction, got %d", count);
  if (dtype != WMM_F16 && dtype != WMM_BF16)
    return fail(WMM_ERR_UNSUPPORTED, "edge rows exist for the 16-bit types only (dtype code %d)", dtype);
  if (batch < 0 || rows < 0 || cols < 0 || window < 0)
    return fail(WMM_ERR_SHAPE, "Input mismatch: negative extent (batch %d rows %d cols %d window %d)", batch, rows, cols, window);
  if (rows < 2 * (int64_t)window)
    return fail(WMM_ERR_SHAPE, "Input mismatch: a shard of %d rows is too short for window %d", rows, window);
  if ((int64_t)batch * cols * window == 0) return WMM_OK;
  if (cols % 8 != 0) return fail(WMM_ERR_STRIDE, "a row of %d elements is not a multiple of 16 bytes", cols);
  if (!flags->mine || !flags->counters) return fail(WMM_ERR_NULL, "flag block or counters are NULL");
  for (int i = 0; i < count; ++i) {
    if (!tensors[i].local || !tensors[i].mine) return fail(WMM_ERR_NULL, "tensor %d has a NULL local pointer", i);
    if (((uintptr_t)tensors[i].local | (uintptr_t)tensors[i].mine | (uintptr_t)tensors[i].lower | (uintptr_t)tensors[i].upper) & 15)
      return fail(WMM_ERR_STRIDE, "tensor %d is not 16-byte aligned", i);
    if ((tensors[i].lower != nullptr) != (flags->lower != nullptr) || (tensors[i].upper != nullptr) != (flags->upper != nullptr))
      return fail(WMM_ERR_NULL, "tensor %d and the flags disagree on which neighbours exist", i);
  }
  int launches = 0;
  cudaError_t err = wmm::launch_halo_pull(nullptr, count, *flags, flags->counters, flags->counters + 1, batch, rows, cols, window,
                                          dtype, true, (cudaStream_t)stream, &launches, tensors);
  g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
  if (err != cudaSuccess) return fail(WMM_ERR_CUDA, "CUDA error launching the edge-row reduction: %s", cudaGetErrorString(err));
  return WMM_OK;
}

uint64_t wmm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int wmm_set_cta_limits(int contraction_ctas, int exchange_ctas) {
  if (contraction_ctas < 0 || exchange_ctas < 0)
    return fail(WMM_ERR_SHAPE, "CTA limits must be >= 0 (0 = no limit), got %d and %d", contraction_ctas, exchange_ctas);
  wmm::g_contraction_cta_limit.store(contraction_ctas, std::memory_order_relaxed);
  wmm::g_exchange_cta_limit.store(exchange_ctas, std::memory_order_relaxed);
  return WMM_OK;
}

int64_t wmm_device_status(int clear) {
  unsigned long long word = 0;
  cudaError_t e = wmm::read_device_status(&word, clear != 0);
  if (e != cudaSuccess) return fail(WMM_ERR_CUDA, "reading the device status word: %s", cudaGetErrorString(e));
  return (int64_t)word;
}

int wmm_query_path(int primitive, const wmm_operand *a, const wmm_operand *b, const void *band,
                   const wmm_geometry *g, int dtype, unsigned flags) {
  wmm::Problem p{};
  int s;
  switch (primitive) {
    case wmm::BAND_NT: s = build(wmm::BAND_NT, p, a, b, nullptr, const_cast<void *>(band), nullptr, g, dtype, flags); break;
    case wmm::BAND_N: s = build(wmm::BAND_N, p, nullptr, a, band, nullptr, b, g, dtype, flags); break;
    case wmm::BAND_T: s = build(wmm::BAND_T, p, a, nullptr, band, nullptr, b, g, dtype, flags); break;
    default: return fail(WMM_ERR_UNSUPPORTED, "unknown primitive %d", primitive);
  }
  if (s < 0) return s;
  if (s == 1) return 0;
  return pick_family((wmm::Primitive)primitive, p);
}

int wmm_band_nt(const wmm_operand *x, const wmm_operand *y, void *band, const wmm_geometry *g, int dtype,
                unsigned flags, void *stream) {
  wmm::Problem p{};
  const int s = build(wmm::BAND_NT, p, x, y, nullptr, band, nullptr, g, dtype, flags);
  if (s != WMM_OK) return s < 0 ? s : WMM_OK;
  return dispatch(wmm::BAND_NT, p, stream);
}

int wmm_band_n(const void *band, const wmm_operand *y, const wmm_operand *out, const wmm_geometry *g, int dtype,
               unsigned flags, void *stream) {
  wmm::Problem p{};
  const int s = build(wmm::BAND_N, p, nullptr, y, band, nullptr, out, g, dtype, flags);
  if (s != WMM_OK) return s < 0 ? s : WMM_OK;
  return dispatch(wmm::BAND_N, p, stream);
}

int wmm_band_t(const void *band, const wmm_operand *x, const wmm_operand *out, const wmm_geometry *g, int dtype,
               unsigned flags, void *stream) {
  wmm::Problem p{};
  const int s = build(wmm::BAND_T, p, x, nullptr, band, nullptr, out, g, dtype, flags);
  if (s != WMM_OK) return s < 0 ? s : WMM_OK;
  return dispatch(wmm::BAND_T, p, stream);
}

int wmm_band_t_edges(const void *band, const wmm_operand *x, const wmm_operand *out, float *edges, int edge_rows,
                     int edge_skip, const wmm_geometry *g, int dtype, unsigned flags, void *stream) {
  wmm::Problem p{};
  const int s = build(wmm::BAND_T, p, x, nullptr, band, nullptr, out, g, dtype, flags);
  if (s != WMM_OK) return s < 0 ? s : WMM_OK;
  if (!edges) return fail(WMM_ERR_NULL, "edges is NULL");
  if ((uintptr_t)edges & 15) return fail(WMM_ERR_STRIDE, "edges is not 16-byte aligned");
  if (edge_rows < 1 || 2 * (int64_t)edge_rows > g->other_rows || edge_skip < 0 || edge_skip >= edge_rows)
    return fail(WMM_ERR_SHAPE, "Input mismatch: %d edge rows (the outer %d skipped) at each end do not fit %d output rows",
                edge_rows, edge_skip, g->other_rows);
  if ((dtype != WMM_F16 && dtype != WMM_BF16) || pick_family(wmm::BAND_T, p) != 1)
    return fail(WMM_ERR_UNSUPPORTED, "only the tensor-core band_t of the 16-bit types writes edge rows");
  p.edges = edges;
  p.edge_rows = edge_rows;
  p.edge_skip = edge_skip;
  return dispatch(wmm::BAND_T, p, stream);
}

int wmm_window_bwd(const wmm_operand *q, const wmm_operand *kt, const void *grad_band, const wmm_operand *grad_q,
                   const wmm_operand *grad_kt, const wmm_geometry *g, int dtype, unsigned flags, void *stream) {
  if (int s = plain_geometry(g)) return s;
  // validate both halves before launching either, so a bad argument never leaves half a result
  wmm::Problem pq{}, pk{};
  const int sq = build(wmm::BAND_N, pq, nullptr, kt, grad_band, nullptr, grad_q, g, dtype, flags);
  if (sq < 0) return sq;
  const int sk = build(wmm::BAND_T, pk, q, nullptr, grad_band, nullptr, grad_kt, g, dtype, flags);
  if (sk < 0) return sk;
  if (sq == WMM_OK && sk == WMM_OK && wants_tensor(wmm::BAND_N, pq) && wants_tensor(wmm::BAND_T, pk) &&
      wmm::tensor_fused_pair_eligible(pq, pk)) {
    // both passes over grad_A in one launch: the band is read from HBM once
    int launches = 0;
    cudaError_t e = wmm::launch_tensor_fused_pair(pq, pk, (cudaStream_t)stream, &launches);
    g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
    if (e != cudaSuccess)
      return fail(WMM_ERR_CUDA, "CUDA error launching the fused window backward: %s [%s]", cudaGetErrorString(e), wmm::launch_detail());
    return WMM_OK;
  }
  if (sq == WMM_OK)
    if (int s = dispatch(wmm::BAND_N, pq, stream)) return s;
  if (sk == WMM_OK)
    if (int s = dispatch(wmm::BAND_T, pk, stream)) return s;
  return WMM_OK;
}

int wmm_unwindow_bwd(const void *band, const wmm_operand *v, const wmm_operand *grad_o, void *grad_band,
                     const wmm_operand *grad_v, const wmm_geometry *g, int dtype, unsigned flags, void *stream) {
  if (int s = plain_geometry(g)) return s;
  wmm::Problem pa{}, pv{};
  const int sa = build(wmm::BAND_NT, pa, grad_o, v, nullptr, grad_band, nullptr, g, dtype, flags);
  if (sa < 0) return sa;
  const int sv = build(wmm::BAND_T, pv, grad_o, nullptr, band, nullptr, grad_v, g, dtype, flags);
  if (sv < 0) return sv;
  if (sa == WMM_OK)
    if (int s = dispatch(wmm::BAND_NT, pa, stream)) return s;
  if (sv == WMM_OK)
    if (int s = dispatch(wmm::BAND_T, pv, stream)) return s;
  return WMM_OK;
}

}  // extern "C"
