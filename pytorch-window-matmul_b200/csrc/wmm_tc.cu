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
#include <mutex>

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

namespace {

using namespace ptx;

constexpr int TILE = 128;       // band rows per tile = MMA M
constexpr int CHUNK = 128;      // positions per chunk = MMA N of band_nt
constexpr int ACC_STAGES = 8;   // band_nt: 8 x 64 TMEM columns
// Status codes OR-ed into g_device_status when a bounded wait runs out: bit 0 band_nt, bit 1 band_n / band_t.

// A (128 rows x NH) 16-bit operand tile in shared memory, K-major, written by TMA with the hardware
// swizzle and read by tcgen05.mma through a matching descriptor.  Rows are SW_BYTES long; wider tiles
// are split into boxes of 64 columns.
template <int NH> struct KMajorTile {
  static constexpr int BOXK = NH >= 64 ? 64 : NH;
  static constexpr int SW_BYTES = BOXK * 2;
  static constexpr int NBOX = NH / BOXK;
  static constexpr int BOX_BYTES = 128 * SW_BYTES;
  static constexpr int BYTES = NBOX * BOX_BYTES;
  static constexpr uint32_t SWZ_CODE = SW_BYTES == 128 ? 2u : SW_BYTES == 64 ? 4u : 6u;
  static constexpr int KSTEPS = NH / 16;
  static constexpr uint64_t DESC = smem_desc_base(16, 8 * SW_BYTES, SWZ_CODE);
  static __device__ __forceinline__ uint32_t kstep_offset(int ks) {
    return (uint32_t)((ks * 16 / BOXK) * BOX_BYTES + (ks * 16 % BOXK) * 2);
  }
};

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

// ---------------------------------------------------------------------------------------------------
// band_n (TRANSPOSED = false):  Out[i, :] = sum_p Band[i, p] Y[p, :]      tile = 128 band rows i
// band_t (TRANSPOSED = true):   Out[p, :] = sum_i Band[i, p] X[i, :]      tile = 128 positions p
//
// Both read (128 rows x 128 x-columns) boxes of the band through the pitched view and multiply them with
// 128-row slices of the other operand (hidden size contiguous, i.e. MN-major for the MMA).  band_n uses
// the box as a K-major A operand (rows = M, x = K); band_t uses the same bytes as an MN-major A operand
// (x = M, rows = K).  Box elements that are not band entries of their row (they alias neighbouring rows)
// or whose position is outside the sequence are zeroed in shared memory by the mask warps before the MMA
// reads them; only the first and last chunk of a tile, and tiles at the sequence ends, need that.
// ---------------------------------------------------------------------------------------------------

constexpr int MM_THREADS = 320;  // producer, MMA, 4 mask warps, 4 epilogue warps
constexpr uint32_t MM_EPI_BAR = 3;
constexpr unsigned long long ST_MM_TIMEOUT = 1ull << 1;

struct MmParams {
  int B, M, Mo, w, off, lo, hi;
  int tiles_per_batch, total_tiles, nchunks;
};

template <int NH> struct MmSmem {
  using BT = KMajorTile<128>;  // band box pair: 128 rows x 128 columns, two 64-column boxes
  using OT = KMajorTile<NH>;   // other operand / output: 128 rows x NH, boxes of OT::BOXK columns
  static constexpr int STAGES = NH >= 128 ? 3 : 4;
  static constexpr int STAGE_BYTES = BT::BYTES + OT::BYTES;
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int OFF_BARS = OFF_OUT + OT::BYTES;
  static constexpr int NBARS = 3 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BARS + NBARS * 8;
  static constexpr int BYTES = OFF_MISC + 32;
  static constexpr int ALLOC = BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * NH < 32 ? 32 : 2 * NH;  // two accumulator stages
};

template <bool BF16, int NH, bool TRANSPOSED>
__global__ void __launch_bounds__(MM_THREADS, 1)
band_mm_tc_kernel(const __grid_constant__ CUtensorMap map_band, const __grid_constant__ CUtensorMap map_other,
                  const __grid_constant__ CUtensorMap map_out, const MmParams p) {
  using S = MmSmem<NH>;
  using BT = typename S::BT;
  using OT = typename S::OT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + S::OFF_BARS;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (S::STAGES + s); };
  auto bar_masked = [&](int s) { return bars + 8u * (2 * S::STAGES + s); };
  auto bar_acc_full = [&](int s) { return bars + 8u * (3 * S::STAGES + s); };
  auto bar_acc_empty = [&](int s) { return bars + 8u * (3 * S::STAGES + 2 + s); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + S::OFF_MISC);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 4);
  volatile int *epi_ok = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; s++) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
      mbar_init(bar_masked(s), 128);
    }
    for (int s = 0; s < 2; s++) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), 128); }
    *abort_flag = 0;
    *epi_ok = 1;
    fence_mbar_init();
    prefetch_tmap(&map_band);
    prefetch_tmap(&map_other);
    prefetch_tmap(&map_out);
  }
  if (warp == 1) {
    tmem_alloc(base + S::OFF_MISC, S::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Tile / chunk geometry, identical in every role.  t0 = first row (band_n) or position (band_t) of the
  // tile.  Chunk c covers, along the reduction, 128 positions (band_n) or 128 band rows (band_t):
  //   band_n: box rows i = t0 .. t0+127, x = t0 + 128c + kk,         position of column kk: t0 - w + off + 128c + kk
  //   band_t: box rows i = t0 - off - w + 128c + ii, x = t0 - off + w + xx,   position of column xx: t0 + xx
  auto chunk_is_plain = [&](int t0, int c) -> bool {
    // true when no element of the box needs zeroing
    if (c < 1 || c * 128 + 127 > 2 * p.w) return false;
    if (!TRANSPOSED) {
      const int p0 = t0 - p.w + p.off + c * 128;
      return p0 >= p.lo && p0 + 128 <= p.hi;
    }
    return t0 >= p.lo && t0 + 128 <= p.hi;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        const int b = tile / p.tiles_per_batch, t0 = (tile % p.tiles_per_batch) * TILE;
        for (int c = 0; c < p.nchunks; ++c, ++it) {
          const int s = it % S::STAGES;
          if (!(ok = mbar_wait(bar_empty(s), ((it / S::STAGES) & 1) ^ 1, abort_flag))) break;
          mbar_expect_tx(bar_full(s), S::STAGE_BYTES);
          const uint32_t band_dst = base + s * S::STAGE_BYTES, other_dst = band_dst + BT::BYTES;
          const int x0 = TRANSPOSED ? t0 - p.off + p.w : t0 + c * 128;
          const int row0 = TRANSPOSED ? t0 - p.off - p.w + c * 128 : t0;
          const int orow0 = TRANSPOSED ? row0 : t0 - p.w + p.off + c * 128;
          tma_load_3d(band_dst, &map_band, bar_full(s), x0, row0, b);
          tma_load_3d(band_dst + BT::BOX_BYTES, &map_band, bar_full(s), x0 + 64, row0, b);
#pragma unroll
          for (int bx = 0; bx < OT::NBOX; bx++)
            tma_load_3d(other_dst + bx * OT::BOX_BYTES, &map_other, bar_full(s), bx * OT::BOXK, orow0, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC = instr_desc_f16(BF16, TRANSPOSED, true, TILE, NH);
      // A operand.  K-major (band_n): 8-row groups 1024 B apart, a k-step of 16 columns is 32 B further
      // along the 128-byte row (64 columns per box).  MN-major (band_t): 64 contiguous x per 128-byte row,
      // second 64 x in the next box (leading offset), 8-row k-groups 1024 B apart (stride offset), a k-step
      // of 16 rows is 2048 B further.
      constexpr uint64_t ADESC = TRANSPOSED ? smem_desc_base(BT::BOX_BYTES, 1024, 2u) : BT::DESC;
      // B operand, MN-major: OT::BOXK contiguous hidden columns per row, next box one leading offset away.
      constexpr uint64_t BDESC = smem_desc_base(OT::BOX_BYTES, 8 * OT::SW_BYTES, OT::SWZ_CODE);
      int it = 0, tit = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++tit) {
        const int as = tit & 1;
        if (!(ok = mbar_wait(bar_acc_empty(as), ((tit >> 1) & 1) ^ 1, abort_flag))) break;
        for (int c = 0; c < p.nchunks; ++c, ++it) {
          const int s = it % S::STAGES;
          // full: the TMA bytes have landed; masked: the mask warps are done with this stage.  The mask
          // warps arrive for EVERY chunk (also those they do not touch) so that no role ever runs more
          // than one barrier phase ahead of another, which parity waits cannot tell apart.
          if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
          if (!(ok = mbar_wait(bar_masked(s), (it / S::STAGES) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint32_t a_addr = base + s * S::STAGE_BYTES, b_addr = a_addr + BT::BYTES;
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const uint32_t a_off = TRANSPOSED ? (uint32_t)k * 2048u : BT::kstep_offset(k);
            const uint32_t b_off = (uint32_t)k * 16u * OT::SW_BYTES;
            umma_f16(tmem_base + as * NH, smem_desc(ADESC, a_addr + a_off), smem_desc(BDESC, b_addr + b_off), IDESC,
                     (c > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty(s));
        }
        if (ok) umma_commit(bar_acc_full(as));
      }
    }
  } else if (warp < 6) {
    // ---------------- mask warps: thread <-> row of the band box ----------------
    const int row = (warp - 2) * 32 + lane;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
      const int t0 = (tile % p.tiles_per_batch) * TILE;
      for (int c = 0; c < p.nchunks; ++c, ++it) {
        const int s = it % S::STAGES;
        if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
        if (chunk_is_plain(t0, c)) {
          mbar_arrive(bar_masked(s));
          continue;
        }
        // columns [col_lo, col_hi] of this row are band entries inside the sequence; the rest is zeroed
        int col_lo, col_hi;
        if (!TRANSPOSED) {
          const int p0 = t0 - p.w + p.off + c * 128;
          col_lo = max(row - c * 128, p.lo - p0);
          col_hi = min(row - c * 128 + 2 * p.w, p.hi - p0 - 1);
        } else {
          col_lo = max(row + c * 128 - 2 * p.w, p.lo - t0);
          col_hi = min(row + c * 128, p.hi - t0 - 1);
        }
        const uint32_t tile_addr = base + s * S::STAGE_BYTES;
#pragma unroll
        for (int g = 0; g < 16; g++) {
          const int c0 = g * 8;
          if (c0 >= col_lo && c0 + 7 <= col_hi) continue;
          const uint32_t a = tile_addr + (g >> 3) * BT::BOX_BYTES + row * 128 + (((g & 7) ^ (row & 7)) << 4);
          uint32_t v0 = 0, v1 = 0, v2 = 0, v3 = 0;
          if (c0 + 7 >= col_lo && c0 <= col_hi) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(a) : "memory");
            auto keep = [&](int col) { return col >= col_lo && col <= col_hi; };
            v0 &= (keep(c0 + 0) ? 0x0000ffffu : 0u) | (keep(c0 + 1) ? 0xffff0000u : 0u);
            v1 &= (keep(c0 + 2) ? 0x0000ffffu : 0u) | (keep(c0 + 3) ? 0xffff0000u : 0u);
            v2 &= (keep(c0 + 4) ? 0x0000ffffu : 0u) | (keep(c0 + 5) ? 0xffff0000u : 0u);
            v3 &= (keep(c0 + 6) ? 0x0000ffffu : 0u) | (keep(c0 + 7) ? 0xffff0000u : 0u);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v0), "r"(v1), "r"(v2), "r"(v3) : "memory");
        }
        if (!TRANSPOSED) {
          // rows of the other operand whose position is outside the sequence: zero them too, so that
          // whatever sits there (an unfilled halo, Inf, NaN) cannot reach the product as 0 * x
          const int pos = t0 - p.w + p.off + c * 128 + row;
          if (pos < p.lo || pos >= p.hi) {
            const uint32_t o_addr = tile_addr + BT::BYTES + row * OT::SW_BYTES;
#pragma unroll
            for (int bx = 0; bx < OT::NBOX; bx++)
#pragma unroll
              for (int q = 0; q < OT::SW_BYTES / 16; q++)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(o_addr + bx * OT::BOX_BYTES + q * 16), "r"(0u) : "memory");
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_masked(s));
      }
    }
  } else {
    // ---------------- epilogue: thread <-> output row of the tile ----------------
    const int quarter = warp & 3;
    const int rr = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 192;
    const uint32_t stage = base + S::OFF_OUT;
    int tit = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++tit) {
      const int b = tile / p.tiles_per_batch, t0 = (tile % p.tiles_per_batch) * TILE;
      const int as = tit & 1;
      if (epi_tid == 0) {
        int good = mbar_wait(bar_acc_full(as), (tit >> 1) & 1, abort_flag) ? 1 : 0;
        bulk_wait_read<0>();  // the previous tile's store has drained the staging buffer
        *epi_ok = good;
      }
      named_bar_sync(MM_EPI_BAR, 128);
      if (!(ok = (*epi_ok != 0))) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + as * NH + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
      for (int g = 0; g < NH / 32; g++) {
        uint32_t v[32];
        tmem_ld_x32(taddr + g * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
          const int col = g * 32 + q4 * 8;  // first hidden column of this 16-byte piece
          const int bx = col / OT::BOXK;
          const int cc = (col % OT::BOXK) / 8;
          const int sw = OT::SW_BYTES == 128 ? (rr & 7) : OT::SW_BYTES == 64 ? ((rr >> 1) & 3) : ((rr >> 2) & 1);
          const uint32_t a = stage + bx * OT::BOX_BYTES + rr * OT::SW_BYTES + ((cc ^ sw) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(pack2<BF16>(v[q4 * 8 + 0], v[q4 * 8 + 1])),
                       "r"(pack2<BF16>(v[q4 * 8 + 2], v[q4 * 8 + 3])), "r"(pack2<BF16>(v[q4 * 8 + 4], v[q4 * 8 + 5])),
                       "r"(pack2<BF16>(v[q4 * 8 + 6], v[q4 * 8 + 7]))
                       : "memory");
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar_acc_empty(as));
      fence_proxy_async_smem();
      named_bar_sync(MM_EPI_BAR, 128);
      if (epi_tid == 0) {
#pragma unroll
        for (int bx = 0; bx < OT::NBOX; bx++) tma_store_3d(&map_out, stage + bx * OT::BOX_BYTES, bx * OT::BOXK, t0, b);
        bulk_commit();
      }
    }
    if (epi_tid == 0) bulk_wait_all();
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_device_status, ST_MM_TIMEOUT);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, S::TMEM_COLS);
  }
}

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

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

CUtensorMapSwizzle swizzle_for(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

// 3-D map (columns, rows, batch) over a 16-bit operand with unit column stride; box = (boxk x 128 x 1).
bool make_operand_map(CUtensorMap *m, bool bf16, const void *data, int cols, int rows, int batch, int64_t stride_r,
                      int64_t stride_b, int boxk) {
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_r * 2, (cuuint64_t)(batch > 1 ? stride_b : (int64_t)rows * stride_r) * 2};
  const cuuint32_t box[3] = {(cuuint32_t)boxk, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_fn()(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void *>(data), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle_for(boxk * 2), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The band as a pitched matrix: x = i + j in [0, M + 2w), row i with pitch 2w elements, batch with
// pitch M*(2w+1).  Rows overlap in memory by design (pitch < extent); an in-range (x, i, b) never
// addresses memory outside the tensor.  Box = (64 x 128 x 1), 128-byte swizzle.
bool make_band_map(CUtensorMap *m, bool bf16, const void *band, int M, int w, int batch) {
  const cuuint64_t dims[3] = {(cuuint64_t)M + 2ull * w, (cuuint64_t)M, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)(2 * w) * 2, (cuuint64_t)M * (2ull * w + 1) * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_fn()(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void *>(band), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool operand_tma_ok(const void *data, int64_t sb, int64_t sr, int64_t sc, int batch) {
  return aligned16(data) && sc == 1 && sr > 0 && (sr % 8) == 0 && (batch <= 1 || (sb > 0 && (sb % 8) == 0));
}

bool band_tma_ok(const void *band, int M, int w) { return aligned16(band) && (w % 4) == 0 && w >= 4 && (M % 8) == 0; }

template <bool BF16, int NH> cudaError_t launch_nt(const Problem &p, cudaStream_t stream) {
  using S = NtSmem<NH>;
  using OT = KMajorTile<NH>;
  CUtensorMap mx, my, mb;
  if (!make_operand_map(&mx, BF16, p.a, NH, p.M, p.B, p.a_sr, p.a_sb, OT::BOXK) ||
      !make_operand_map(&my, BF16, p.b, NH, p.Mo, p.B, p.b_sr, p.b_sb, OT::BOXK) || !make_band_map(&mb, BF16, p.o, p.M, p.w, p.B))
    return cudaErrorInvalidValue;
  NtParams k;
  k.B = p.B; k.M = p.M; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  k.tiles_per_batch = (p.M + TILE - 1) / TILE;
  k.total_tiles = k.tiles_per_batch * p.B;
  k.nchunks = (TILE + 2 * p.w + CHUNK - 1) / CHUNK;
  k.paired = (p.w % 64 == 0) ? 1 : 0;
  k.band = p.o;
  auto kern = band_nt_tc_kernel<BF16, NH>;
  // the attribute is per device; setting it on every call is cheap and needs no per-device cache
  cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (attr_err != cudaSuccess) return attr_err;
  const int grid = k.total_tiles < sm_count() ? k.total_tiles : sm_count();
  kern<<<grid, NT_THREADS, S::ALLOC, stream>>>(mx, my, mb, k);
  return cudaGetLastError();
}

template <bool BF16, int NH, bool TRANSPOSED> cudaError_t launch_mm(const Problem &p, cudaStream_t stream) {
  using S = MmSmem<NH>;
  using OT = KMajorTile<NH>;
  CUtensorMap mband, mother, mout;
  const int out_rows = TRANSPOSED ? p.Mo : p.M;
  const int other_rows = TRANSPOSED ? p.M : p.Mo;
  if (!make_band_map(&mband, BF16, p.a, p.M, p.w, p.B) ||
      !make_operand_map(&mother, BF16, p.b, NH, other_rows, p.B, p.b_sr, p.b_sb, OT::BOXK) ||
      !make_operand_map(&mout, BF16, p.o, NH, out_rows, p.B, p.o_sr, p.o_sb, OT::BOXK))
    return cudaErrorInvalidValue;
  MmParams k;
  k.B = p.B; k.M = p.M; k.Mo = p.Mo; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  k.tiles_per_batch = (out_rows + TILE - 1) / TILE;
  k.total_tiles = k.tiles_per_batch * p.B;
  k.nchunks = (TILE + 2 * p.w + 127) / 128;
  auto kern = band_mm_tc_kernel<BF16, NH, TRANSPOSED>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC);
  if (e != cudaSuccess) return e;
  const int grid = k.total_tiles < sm_count() ? k.total_tiles : sm_count();
  kern<<<grid, MM_THREADS, S::ALLOC, stream>>>(mband, mother, mout, k);
  return cudaGetLastError();
}

template <bool TRANSPOSED> cudaError_t launch_mm_any(const Problem &p, cudaStream_t stream) {
  const bool bf16 = p.dtype == WMM_BF16;
  switch (p.N) {
    case 32: return bf16 ? launch_mm<true, 32, TRANSPOSED>(p, stream) : launch_mm<false, 32, TRANSPOSED>(p, stream);
    case 64: return bf16 ? launch_mm<true, 64, TRANSPOSED>(p, stream) : launch_mm<false, 64, TRANSPOSED>(p, stream);
    case 128: return bf16 ? launch_mm<true, 128, TRANSPOSED>(p, stream) : launch_mm<false, 128, TRANSPOSED>(p, stream);
    default: return cudaErrorNotSupported;
  }
}

}  // namespace

bool tensor_eligible(Primitive prim, const Problem &p) {
  if (p.dtype != WMM_F16 && p.dtype != WMM_BF16) return false;
  if (!encode_fn()) return false;
  if (p.N != 32 && p.N != 64 && p.N != 128) return false;
  if ((int64_t)p.B * ((p.M + TILE - 1) / TILE) > 0x7fffffffLL) return false;
  switch (prim) {
    case BAND_NT:
      return band_tma_ok(p.o, p.M, p.w) && operand_tma_ok(p.a, p.a_sb, p.a_sr, p.a_sc, p.B) &&
             operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) && p.Mo > 0;
    case BAND_N:
      return band_tma_ok(p.a, p.M, p.w) && operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
             operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.Mo > 0;
    case BAND_T:
      // the box of a tile starts at x = t0 - off + w, which must be a multiple of 8 elements (16 bytes)
      return band_tma_ok(p.a, p.M, p.w) && ((p.w - p.off) % 8) == 0 && operand_tma_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) &&
             operand_tma_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B) && p.M > 0;
    default: return false;
  }
}

cudaError_t launch_tensor(Primitive prim, const Problem &p, cudaStream_t stream, int *launches) {
  cudaError_t e = cudaErrorNotSupported;
  const bool bf16 = p.dtype == WMM_BF16;
  if (prim == BAND_NT) {
    switch (p.N) {
      case 32: e = bf16 ? launch_nt<true, 32>(p, stream) : launch_nt<false, 32>(p, stream); break;
      case 64: e = bf16 ? launch_nt<true, 64>(p, stream) : launch_nt<false, 64>(p, stream); break;
      case 128: e = bf16 ? launch_nt<true, 128>(p, stream) : launch_nt<false, 128>(p, stream); break;
    }
  }
  else if (prim == BAND_N)
    e = launch_mm_any<false>(p, stream);
  else if (prim == BAND_T)
    e = launch_mm_any<true>(p, stream);
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

}  // namespace wmm
