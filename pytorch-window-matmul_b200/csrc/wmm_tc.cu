// tcgen05 / TMA kernels for the banded contractions on 16-bit inputs (fp16, bf16; fp32 accumulation in TMEM).
//
// Geometry shared by the three kernels.  A CTA owns tiles of 128 band rows.  In dense (row i, position p)
// coordinates a tile touches positions p0 .. p0 + 128 + 2w - 1, processed in chunks of 128.  The band
// tensor is contiguous (B, M, 2w+1); entry (i, j) sits at element i*(2w+1) + j = i*2w + (i + j) of its
// batch, so the band IS a dense row-major matrix with row pitch 2w (not 2w+1) in the coordinates
// (row i, x = i + j): a (128 rows x 128 positions) block of the dense product is a plain pitched 2-D
// box of the band tensor.  That makes band tiles TMA-addressable (3-D map: x, row, batch) although the
// true row length 2w+1 is odd; elements of a box outside 0 <= j <= 2w alias entries of neighbouring
// rows, so only boxes that lie wholly inside the band are moved by TMA, and the two triangular ends of
// a tile are moved with predicated vector accesses.
//
// Warp roles (persistent CTAs, one per SM, tiles taken round-robin with the sequence index fastest so
// that neighbouring CTAs share their halo rows in L2): warp 0 = TMA producer, warp 1 = MMA issuer and
// TMEM owner, warps 2-5 = epilogue (TMEM -> registers -> global / staging + TMA store).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <utility>

#include "wmm_common.cuh"
#include "wmm_ptx.cuh"

namespace wmm {

__device__ unsigned long long g_device_status = 0ull;

cudaError_t read_device_status(unsigned long long *word, bool clear) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(word, g_device_status, sizeof(*word));
  if (e == cudaSuccess && clear && *word) {
    const unsigned long long zero = 0;
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  }
  return e;
}

unsigned long long *device_status_word() {
  void *p = nullptr;
  return cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess ? static_cast<unsigned long long *>(p) : nullptr;
}

// Per-CTA timeline for tuning (build with -DWMM_TRACE): kernels store the global timer at a few points of their life;
// wmm_trace_read() copies the table out.  Compiled out of the normal library.
#ifdef WMM_TRACE
constexpr int kTraceSlots = 160;
__device__ unsigned long long g_trace[160 * kTraceSlots];
#define WMM_TRACE_POINT(id)                                                                     \
  do {                                                                                          \
    if (blockIdx.x < 160) g_trace[blockIdx.x * kTraceSlots + (id)] = ptx::globaltimer_ns();     \
  } while (0)
// time accumulated in a REGISTER by the caller (no memory traffic inside the loops), stored once with WMM_TRACE_STORE
#define WMM_TRACE_T0(var) const unsigned long long var = ptx::globaltimer_ns()
#define WMM_TRACE_ACC(acc, var) acc += ptx::globaltimer_ns() - var
#define WMM_TRACE_STORE(id, value)                                                  \
  do {                                                                              \
    if (blockIdx.x < 160) g_trace[blockIdx.x * kTraceSlots + (id)] = (value);       \
  } while (0)
extern "C" __attribute__((visibility("default"))) int wmm_trace_waits(unsigned long long *out, int clear) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, ptx::g_wait_tab, sizeof(ptx::g_wait_tab));
  if (e == cudaSuccess && clear) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, ptx::g_wait_tab);
    if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(ptx::g_wait_tab));
  }
  return e == cudaSuccess ? 160 * 20 : -1;
}
extern "C" __attribute__((visibility("default"))) int wmm_trace_read(unsigned long long *out, int clear) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(out + 159 * kTraceSlots, ptx::g_wait_info, sizeof(ptx::g_wait_info));   // (block 159 never exists)
  if (e == cudaSuccess && clear) {
    const unsigned long long zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(ptx::g_wait_info, zero, sizeof(zero));
  }
  if (e == cudaSuccess && clear) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_trace);
    if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(g_trace));
  }
  return e == cudaSuccess ? 160 * kTraceSlots : -1;
}
#else
#define WMM_TRACE_POINT(id) ((void)0)
#define WMM_TRACE_T0(var) ((void)0)
#define WMM_TRACE_ACC(acc, var) ((void)0)
#define WMM_TRACE_STORE(id, value) ((void)0)
#endif

namespace {
thread_local char tls_detail[256] = "";
}
void set_launch_detail(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_detail, sizeof(tls_detail), fmt, ap);
  va_end(ap);
}
const char *launch_detail() { return tls_detail; }

namespace {

using namespace ptx;

constexpr int TILE = 128;       // band rows per tile = MMA M
constexpr int CHUNK = 128;      // positions per chunk = MMA N of band_nt
constexpr int ACC_STAGES = 4;   // band_nt: 4 x 128 TMEM columns (one chunk each)
// Status codes OR-ed into g_device_status when a bounded wait runs out: bit 0 band_nt, bit 1 band_n / band_t.

// A (128 rows x NH) operand tile in shared memory, K-major, written by TMA with the hardware swizzle and read by
// tcgen05.mma through a matching descriptor.  ES = bytes per element (2: fp16 / bf16, 4: fp32 consumed as tf32).  Rows are
// SW_BYTES long; wider tiles are split into boxes of 128 bytes.  One k-step of the MMA is 32 bytes of a row (16 or 8
// elements) whatever the type.
template <int NH, int ES> struct KMajorTileE {
  static constexpr int BOXK = (NH * ES >= 128) ? 128 / ES : NH;
  static constexpr int SW_BYTES = BOXK * ES;
  static constexpr int NBOX = NH / BOXK;
  static constexpr int BOX_BYTES = 128 * SW_BYTES;
  static constexpr int BYTES = NBOX * BOX_BYTES;
  static constexpr uint32_t SWZ_CODE = SW_BYTES == 128 ? 2u : SW_BYTES == 64 ? 4u : 6u;
  static constexpr int KSTEPS = NH * ES / 32;
  static constexpr uint64_t DESC = smem_desc_base(16, 8 * SW_BYTES, SWZ_CODE);
  static __device__ __forceinline__ uint32_t kstep_offset(int ks) {
    return (uint32_t)((ks * 32 / SW_BYTES) * BOX_BYTES + (ks * 32 % SW_BYTES));
  }
};
template <int NH> using KMajorTile = KMajorTileE<NH, 2>;

template <bool BF16> __device__ __forceinline__ uint32_t pack2(uint32_t lo_bits, uint32_t hi_bits) {
  const float lo = __uint_as_float(lo_bits), hi = __uint_as_float(hi_bits);
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
}
template <bool BF16> __device__ __forceinline__ uint16_t pack1(uint32_t bits) {
  const float f = __uint_as_float(bits);
  if (BF16) {
    __nv_bfloat16 v = __float2bfloat16_rn(f);
    return *reinterpret_cast<uint16_t *>(&v);
  } else {
    __half v = __float2half_rn(f);
    return *reinterpret_cast<uint16_t *>(&v);
  }
}

#include "wmm_tc_nt.cuh"

#include "wmm_tc_mm.cuh"
#include "wmm_tc_sweep.cuh"
#include "wmm_tc_mm32.cuh"

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(ptr);
  });
  return fn;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

// Persistent grid: one CTA per SM (fewer if there are fewer work items).  The kernels are bandwidth-bound,
// so the SMs that run out of work early leave their share of the bandwidth to the others; launching fewer,
// evenly loaded CTAs measured slower.
int persistent_grid(int items) {
  int sms = sm_count();
  const int cap = g_contraction_cta_limit.load(std::memory_order_relaxed);   // SMs left to a concurrent exchange
  if (cap > 0 && cap < sms) sms = cap;
  return items < sms ? items : sms;
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its predecessor in the stream is
// still running; its prologue then overlaps the predecessor's tail and it blocks at griddepcontrol.wait (see wmm_ptx.cuh)
// before touching global memory.  Captured into CUDA graphs as a programmatic dependency edge.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = getenv("WMM_NO_PDL") != nullptr;
  // Under a CTA limit the free SMs belong to a kernel of another stream: an early-scheduled successor would sit on them
  // at its griddepcontrol.wait, so such launches keep plain stream order.
  cfg.numAttrs = no_pdl || g_contraction_cta_limit.load(std::memory_order_relaxed) > 0 ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

CUtensorMapSwizzle swizzle_for(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

// 3-D map (columns, rows, batch) over a 16-bit operand with unit column stride; box = (boxk x 128 x 1).
// `et`: 0 fp16, 1 bf16 (bool true), 2 fp32.
CUtensorMapDataType map_dtype(int et) {
  return et == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : et == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}
bool make_operand_map(CUtensorMap *m, int et, const void *data, int cols, int rows, int batch, int64_t stride_r,
                      int64_t stride_b, int boxk, int box_rows = 128, bool atom32 = false) {
  const int es = et == 2 ? 4 : 2;
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_r * es, (cuuint64_t)(batch > 1 ? stride_b : (int64_t)rows * stride_r) * es};
  const cuuint32_t box[3] = {(cuuint32_t)boxk, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(m, map_dtype(et), 3,
                                const_cast<void *>(data), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : swizzle_for(boxk * es), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    set_launch_detail("cuTensorMapEncodeTiled(operand %p, dims %d x %d x %d, strides %lld / %lld elements) returned %d", data, cols,
                      rows, batch, (long long)stride_r, (long long)stride_b, (int)r);
  return r == CUDA_SUCCESS;
}

// 3-D map (positions, hidden, batch) over a 16-bit operand stored with the positions contiguous
// (element (b, p, h) at b*stride_b + h*stride_c + p); box = (64 positions x `cols` hidden rows x 1), 128-byte swizzle.
bool make_operand_map_mn(CUtensorMap *m, bool bf16, const void *data, int cols, int rows, int batch, int64_t stride_c,
                         int64_t stride_b) {
  const cuuint64_t dims[3] = {(cuuint64_t)rows, (cuuint64_t)cols, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_c * 2, (cuuint64_t)(batch > 1 ? stride_b : (int64_t)cols * stride_c) * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)cols, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                                const_cast<void *>(data), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    set_launch_detail("cuTensorMapEncodeTiled(position-major operand %p, %d positions x %d, batch %d) returned %d", data, rows, cols,
                      batch, (int)r);
  return r == CUDA_SUCCESS;
}

// The band as a pitched matrix: x = i + j in [0, M + 2w), row i with pitch 2w elements, batch with
// pitch M*(2w+1).  Rows overlap in memory by design (pitch < extent); an in-range (x, i, b) never
// addresses memory outside the tensor.  Box = (64 x 128 x 1), 128-byte swizzle.
bool make_band_map(CUtensorMap *m, int et, const void *band, int M, int w, int batch, int64_t band_sb, int box_rows = 128,
                   bool atom32 = false) {
  const int es = et == 2 ? 4 : 2;
  const cuuint64_t dims[3] = {(cuuint64_t)M + 2ull * w, (cuuint64_t)M, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)(2 * w) * es, (cuuint64_t)band_sb * es};
  const cuuint32_t box[3] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1};   // 128-byte lines
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(m, map_dtype(et), 3,
                                const_cast<void *>(band), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    set_launch_detail("cuTensorMapEncodeTiled(band %p, rows %d, window %d, batch %d) returned %d", band, M, w, batch, (int)r);
  return r == CUDA_SUCCESS;
}

// an operand stored with the positions contiguous (stride_r == 1): hidden stride and batch stride 16-byte multiples
bool operand_mn_tma_ok(const void *data, int64_t sb, int64_t sr, int64_t sc, int batch) {
  return aligned16(data) && sr == 1 && sc > 0 && (sc % 8) == 0 && (batch <= 1 || (sb > 0 && (sb % 8) == 0));
}

bool operand_tma_ok(const void *data, int64_t sb, int64_t sr, int64_t sc, int batch) {
  return aligned16(data) && sc == 1 && sr > 0 && (sr % 8) == 0 && (batch <= 1 || (sb > 0 && (sb % 8) == 0));
}

// Y stored with the positions contiguous and usable through a (position, hidden, batch) map: chunk origins
// r0 - w + off + 64k must then be multiples of 8 elements.
bool y_position_major(const Problem &p) {
  return !operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) && operand_mn_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
         ((p.w - p.off) % 8) == 0;
}

// (the batch stride must be a multiple of 16 bytes: of 8 elements, which also covers fp32)
bool band_tma_ok(const void *band, int64_t band_sb, int w) { return aligned16(band) && (w % 4) == 0 && w >= 4 && (band_sb % 8) == 0; }

template <int ET, int NH, bool YMN, bool PAIRED> cudaError_t launch_nt(const Problem &p, cudaStream_t stream) {
  constexpr int BF16 = ET;   // (element type code of the tensor maps)
  using S = NtSmem<NH, ET == 2 ? 4 : 2>;
  using OT = KMajorTileE<NH, ET == 2 ? 4 : 2>;
  NtParams k;
  k.B = p.B; k.M = p.M; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  k.tiles_per_batch = (p.M + TILE - 1) / TILE;
  k.total_tiles = k.tiles_per_batch * p.B;
  k.nchunks = (TILE + 2 * p.w + CHUNK - 1) / CHUNK;
  k.paired = PAIRED ? 1 : 0;
  k.band = p.o;
  k.band_sb = p.band_sb;
  auto kern = band_nt_tc_kernel<ET, NH, YMN, PAIRED>;
  // the attribute is per device; setting it on every call is cheap and needs no per-device cache
  cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (attr_err != cudaSuccess) {
    set_launch_detail("cudaFuncSetAttribute(band_nt, %d bytes of shared memory)", S::ALLOC);
    return attr_err;
  }
  // The runtime call above has bound this thread to the device's primary context; the driver entry point
  // used for the tensor maps needs a current context (a fresh thread, e.g. an autograd worker, has none).
  CUtensorMap mx, my, mb;
  if (!make_operand_map(&mx, BF16, p.a, NH, p.M, p.B, p.a_sr, p.a_sb, OT::BOXK) ||
      !(YMN ? make_operand_map_mn(&my, BF16, p.b, NH, p.Mo, p.B, p.b_sc, p.b_sb)
            : make_operand_map(&my, BF16, p.b, NH, p.Mo, p.B, p.b_sr, p.b_sb, OT::BOXK)) ||
      !make_band_map(&mb, BF16, p.o, p.M, p.w, p.B, p.band_sb))
    return cudaErrorInvalidValue;
  const int grid = persistent_grid(k.total_tiles);
  set_launch_detail("band_nt launch, grid %d", grid);
  return launch_pdl(kern, grid, NT_THREADS, S::ALLOC, stream, mx, my, mb, k);
}

template <int NH> cudaError_t launch_nt_any(const Problem &p, cudaStream_t stream) {
  if (p.dtype == WMM_F32) {   // tf32 products, fp32 band
    if constexpr (NH <= 64) return (p.w % 64) == 0 ? launch_nt<2, NH, false, true>(p, stream) : launch_nt<2, NH, false, false>(p, stream);
    else return cudaErrorNotSupported;
  }
  const bool bf16 = p.dtype == WMM_BF16;
  const bool paired = (p.w % 64) == 0;   // 2w a multiple of 128
  if (y_position_major(p)) {
    if (paired) return bf16 ? launch_nt<1, NH, true, true>(p, stream) : launch_nt<0, NH, true, true>(p, stream);
    return bf16 ? launch_nt<1, NH, true, false>(p, stream) : launch_nt<0, NH, true, false>(p, stream);
  }
  if (paired) return bf16 ? launch_nt<1, NH, false, true>(p, stream) : launch_nt<0, NH, false, true>(p, stream);
  return bf16 ? launch_nt<1, NH, false, false>(p, stream) : launch_nt<0, NH, false, false>(p, stream);
}

// MODE 0 / 1: one problem (band_n / band_t).  MODE 2: `p` is the band_n problem and `pt` the band_t
// problem over the same band (same geometry, plain: other_rows = rows, other_off = 0).
template <bool BF16, int NH, int MODE, bool YMN> cudaError_t launch_mm(const Problem &p, const Problem *pt, cudaStream_t stream) {
  using S = MmSmem<NH>;
  using OT = KMajorTile<NH>;
  const bool tr = MODE == 1;
  const int out_rows = tr ? p.Mo : p.M;
  const int other_rows = tr ? p.M : p.Mo;
  MmParams k;
  k.B = p.B; k.M = p.M; k.Mo = p.Mo; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  k.tiles_per_batch = (out_rows + TILE - 1) / TILE;
  k.total_tiles = k.tiles_per_batch * p.B;
  k.nchunks = (TILE + 2 * p.w + 127) / 128;
  k.edges = MODE == 1 ? p.edges : nullptr;
  k.edge_rows = MODE == 1 ? p.edge_rows : 0;
  k.edge_skip = MODE == 1 ? p.edge_skip : 0;
  auto kern = band_mm_tc_kernel<BF16, NH, MODE, YMN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (e != cudaSuccess) {
    set_launch_detail("cudaFuncSetAttribute(band_mm mode %d, %d bytes of shared memory)", MODE, S::ALLOC);
    return e;
  }
  // (the tensor maps need the current context the runtime call above has bound to this thread)
  CUtensorMap mband, mother0, mout0, mother1, mout1;
  if (!make_band_map(&mband, BF16, p.a, p.M, p.w, p.B, p.band_sb) ||
      !(YMN ? make_operand_map_mn(&mother0, BF16, p.b, NH, other_rows, p.B, p.b_sc, p.b_sb)
            : make_operand_map(&mother0, BF16, p.b, NH, other_rows, p.B, p.b_sr, p.b_sb, OT::BOXK)) ||
      !make_operand_map(&mout0, BF16, p.o, NH, out_rows, p.B, p.o_sr, p.o_sb, OT::BOXK))
    return cudaErrorInvalidValue;
  if (MODE == 2) {
    if (!make_operand_map(&mother1, BF16, pt->b, NH, pt->M, pt->B, pt->b_sr, pt->b_sb, OT::BOXK) ||
        !make_operand_map(&mout1, BF16, pt->o, NH, pt->Mo, pt->B, pt->o_sr, pt->o_sb, OT::BOXK))
      return cudaErrorInvalidValue;
  } else {
    mother1 = mother0;
    mout1 = mout0;
  }
  const int items = MODE == 2 ? 2 * k.total_tiles : k.total_tiles;
  int grid = persistent_grid(items);
  if (MODE == 2 && (grid & 1) && grid > 1) --grid;  // even: each CTA keeps to one of the two passes
  set_launch_detail("band_mm mode %d launch, grid %d", MODE, grid);
  return launch_pdl(kern, grid, MM_THREADS, S::ALLOC, stream, mband, mother0, mout0, mother1, mout1, k);
}

template <int MODE, bool YMN> cudaError_t launch_mm_n(const Problem &p, const Problem *pt, cudaStream_t stream) {
  const bool bf16 = p.dtype == WMM_BF16;
  switch (p.N) {
    case 32: return bf16 ? launch_mm<true, 32, MODE, YMN>(p, pt, stream) : launch_mm<false, 32, MODE, YMN>(p, pt, stream);
    case 64: return bf16 ? launch_mm<true, 64, MODE, YMN>(p, pt, stream) : launch_mm<false, 64, MODE, YMN>(p, pt, stream);
    case 128: return bf16 ? launch_mm<true, 128, MODE, YMN>(p, pt, stream) : launch_mm<false, 128, MODE, YMN>(p, pt, stream);
    default: return cudaErrorNotSupported;
  }
}

// fp32 tensors, tf32 products (WMM_FLAG_TF32): band_n (TR = false) or band_t (TR = true)
template <int NH, bool TR> cudaError_t launch_mm32(const Problem &p, cudaStream_t stream) {
  using S = Mm32Smem<NH>;
  const int out_rows = TR ? p.Mo : p.M;
  const int other_rows = TR ? p.M : p.Mo;
  MmParams k;
  k.B = p.B; k.M = p.M; k.Mo = p.Mo; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  k.tiles_per_batch = (out_rows + TILE - 1) / TILE;
  k.total_tiles = k.tiles_per_batch * p.B;
  k.nchunks = (TILE + 2 * p.w + M32_RC - 1) / M32_RC;
  auto kern = band_mm_tf32_kernel<NH, TR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (e != cudaSuccess) {
    set_launch_detail("cudaFuncSetAttribute(band_mm tf32, %d bytes of shared memory)", S::ALLOC);
    return e;
  }
  CUtensorMap mband, mother, mout;
  // MN-major fp32 operands (the other operand; the band box of band_t) use the 128-byte swizzle with 32-byte atoms
  if (!make_band_map(&mband, 2, p.a, p.M, p.w, p.B, p.band_sb, TR ? M32_RC : 128, TR) ||
      !make_operand_map(&mother, 2, p.b, NH, other_rows, p.B, p.b_sr, p.b_sb, 32, M32_RC, true) ||
      !make_operand_map(&mout, 2, p.o, NH, out_rows, p.B, p.o_sr, p.o_sb, 32, 128))
    return cudaErrorInvalidValue;
  const int grid = persistent_grid(k.total_tiles);
  set_launch_detail("band_mm tf32 launch, grid %d", grid);
  return launch_pdl(kern, grid, MM_THREADS, S::ALLOC, stream, mband, mother, mout, k);
}

// band_n's other operand may be position-major (MODE 0 and the band_n half of MODE 2); band_t's never is here
template <int MODE> cudaError_t launch_mm_any(const Problem &p, const Problem *pt, cudaStream_t stream) {
  if (MODE != 1 && y_position_major(p)) return launch_mm_n<MODE, true>(p, pt, stream);
  return launch_mm_n<MODE, false>(p, pt, stream);
}

// grad_Q and grad_K^T of window_matmul in one sweep over grad_A (see wmm_tc_sweep.cuh for the conditions).
bool sweep_eligible(const Problem &pn, const Problem &pt) {
  if (pn.w < 128 || (pn.w % 128) != 0) return false;
  const int D = pn.w / 128;
  if (2 * D + 2 > SweepSmem<32>::MAX_SLOTS || (2 * D + 4) * pn.N > 512) return false;
  if (pn.lo != 0 || pn.hi != pn.M || y_position_major(pn)) return false;
  // A run that starts inside a sequence replays D (2D + 1) boxes; with short runs (few row tiles per CTA) that costs
  // more than the second pass of the two-pass kernel.
  const int64_t row_tiles = (int64_t)pn.B * ((pn.M + TILE - 1) / TILE);
  return (pn.flags & WMM_FLAG_PREFER_SWEEP) != 0 || row_tiles >= 8ll * sm_count();
}

template <bool BF16, int NH> cudaError_t launch_sweep(const Problem &pn, const Problem &pt, cudaStream_t stream) {
  using S = SweepSmem<NH>;
  using OT = KMajorTile<NH>;
  SweepParams k;
  k.B = pn.B; k.M = pn.M; k.w = pn.w; k.D = pn.w / 128;
  k.T = (pn.M + TILE - 1) / TILE;
  k.total_rows = k.B * k.T;
  auto kern = band_bwd_sweep_kernel<BF16, NH>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (e != cudaSuccess) {
    set_launch_detail("cudaFuncSetAttribute(band_bwd_sweep, %d bytes of shared memory)", S::ALLOC);
    return e;
  }
  k.gq = static_cast<uint16_t *>(pn.o); k.gq_sb = pn.o_sb; k.gq_sr = pn.o_sr;
  k.gk = static_cast<uint16_t *>(pt.o); k.gk_sb = pt.o_sb; k.gk_sr = pt.o_sr;
  CUtensorMap mband, my, mx;
  if (!make_band_map(&mband, BF16, pn.a, pn.M, pn.w, pn.B, pn.band_sb) ||
      !make_operand_map(&my, BF16, pn.b, NH, pn.Mo, pn.B, pn.b_sr, pn.b_sb, OT::BOXK) ||
      !make_operand_map(&mx, BF16, pt.b, NH, pt.M, pt.B, pt.b_sr, pt.b_sb, OT::BOXK))
    return cudaErrorInvalidValue;
  const int grid = persistent_grid(k.total_rows);
  set_launch_detail("band_bwd_sweep launch, grid %d", grid);
  return launch_pdl(kern, grid, SWP_THREADS, S::ALLOC, stream, mband, my, mx, k);
}

}  // namespace

bool tensor_eligible(Primitive prim, const Problem &p) {
  if (p.dtype == WMM_F32) {
    // fp32 operands go to the tensor cores only on request (WMM_FLAG_TF32: products of tf32-rounded values, fp32 sums)
    if (!(p.flags & WMM_FLAG_TF32) || !encode_fn()) return false;
    if (p.N != 32 && p.N != 64) return false;
    if ((int64_t)p.B * ((p.M + TILE - 1) / TILE) > 0x7fffffffLL) return false;
    // element strides of fp32 operands: multiples of 4 would do; the 16-bit rule (multiples of 8) is kept
    if (prim == BAND_NT)
      return band_tma_ok(p.o, p.band_sb, p.w) && operand_tma_ok(p.a, p.a_sb, p.a_sr, p.a_sc, p.B) &&
             operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) && p.Mo > 0;
    if (prim == BAND_N)
      return band_tma_ok(p.a, p.band_sb, p.w) && operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
             operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.Mo > 0;
    // band_t: the box of a tile starts at x = t0 - off + w, a multiple of 4 elements (16 bytes)
    return band_tma_ok(p.a, p.band_sb, p.w) && ((p.w - p.off) % 4) == 0 && operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
           operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.M > 0;
  }
  if (p.dtype != WMM_F16 && p.dtype != WMM_BF16) return false;
  if (!encode_fn()) return false;
  if (p.N != 32 && p.N != 64 && p.N != 128) return false;
  if ((int64_t)p.B * ((p.M + TILE - 1) / TILE) > 0x7fffffffLL) return false;
  switch (prim) {
    case BAND_NT:
      return band_tma_ok(p.o, p.band_sb, p.w) && operand_tma_ok(p.a, p.a_sb, p.a_sr, p.a_sc, p.B) &&
             (operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) || y_position_major(p)) && p.Mo > 0;
    case BAND_N:
      return band_tma_ok(p.a, p.band_sb, p.w) &&
             (operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) || (y_position_major(p) && p.lo == 0 && p.hi == p.Mo)) &&
             operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.Mo > 0;
    case BAND_T:
      // the box of a tile starts at x = t0 - off + w, which must be a multiple of 8 elements (16 bytes)
      return band_tma_ok(p.a, p.band_sb, p.w) && ((p.w - p.off) % 8) == 0 && operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
             operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.M > 0;
    default: return false;
  }
}

cudaError_t launch_tensor(Primitive prim, const Problem &p, cudaStream_t stream, int *launches) {
  cudaError_t e = cudaErrorNotSupported;
  if (prim == BAND_NT) {
    switch (p.N) {
      case 32: e = launch_nt_any<32>(p, stream); break;
      case 64: e = launch_nt_any<64>(p, stream); break;
      case 128: e = launch_nt_any<128>(p, stream); break;
    }
  }
  else if (p.dtype == WMM_F32) {
    if (prim == BAND_N) e = p.N == 32 ? launch_mm32<32, false>(p, stream) : launch_mm32<64, false>(p, stream);
    else if (prim == BAND_T) e = p.N == 32 ? launch_mm32<32, true>(p, stream) : launch_mm32<64, true>(p, stream);
  }
  else if (prim == BAND_N)
    e = launch_mm_any<0>(p, nullptr, stream);
  else if (prim == BAND_T)
    e = launch_mm_any<1>(p, nullptr, stream);
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

bool tensor_fused_pair_eligible(const Problem &pn, const Problem &pt) {
  if (pn.dtype == WMM_F32) return false;   // fp32 (tf32 products): the two single-product kernels
  return tensor_eligible(BAND_N, pn) && tensor_eligible(BAND_T, pt) && pn.a == pt.a && pn.Mo == pn.M && pt.Mo == pt.M &&
         pn.off == 0 && pt.off == 0 && pn.lo == pt.lo && pn.hi == pt.hi && pn.w == pt.w && pn.N == pt.N && pn.B == pt.B &&
         pn.M == pt.M && pn.dtype == pt.dtype && (int64_t)pn.B * ((pn.M + TILE - 1) / TILE) * 2 <= 0x7fffffffLL;
}

cudaError_t launch_tensor_fused_pair(const Problem &pn, const Problem &pt, cudaStream_t stream, int *launches) {
  cudaError_t e;
  if (sweep_eligible(pn, pt)) {
    const bool bf16 = pn.dtype == WMM_BF16;
    if (pn.N == 32) e = bf16 ? launch_sweep<true, 32>(pn, pt, stream) : launch_sweep<false, 32>(pn, pt, stream);
    else e = bf16 ? launch_sweep<true, 64>(pn, pt, stream) : launch_sweep<false, 64>(pn, pt, stream);
  } else {
    e = launch_mm_any<2>(pn, &pt, stream);
  }
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

}  // namespace wmm
