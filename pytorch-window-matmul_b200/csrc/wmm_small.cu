// Small-window kernels (w <= 32) for 16-bit inputs.
//
// With a narrow band the problem is purely HBM-bound (config 3: N=32, w=8 -> 7.5 flop/byte) and the pitched
// TMA view of the band used by the tcgen05 kernels degenerates (pitch 2w elements, boxes overlap 8-fold).
// Here a CTA owns 128 band rows; the packed band tile (128 x (2w+1), ONE contiguous span of global memory)
// and the (128 + 2w)-row slab of the other operand move between HBM and shared memory with coalesced
// 16-byte accesses, each HBM byte once.  The arithmetic is done per warp on 16 rows with warp-level
// m16n8k16 MMAs (fp32 accumulation) fed from shared memory: band_nt builds 16 x (16 + 2w) dense products
// and scatters them into the packed band image; band_n / band_t gather the un-skewed band fragments from
// the packed image.  Whole packed band tiles move with one untiled bulk copy where alignment allows (completion on an
// mbarrier with a bounded wait); everything else is cp.async and __syncthreads.  No waits on other CTAs.
#include "wmm_common.cuh"
#include "wmm_ptx.cuh"

namespace wmm {

namespace {

constexpr int SM_ROWS = 128;    // band rows (band_nt, band_n) or positions (band_t) per CTA
constexpr int SM_THREADS = 256; // 8 warps x 16 rows
constexpr int SM_MAX_W = 32;

struct SmallParams {
  const uint16_t *a;  // X (band_nt) or band (band_n, band_t)
  const uint16_t *b;  // Y (band_nt, band_n) or X (band_t)
  uint16_t *o;
  int64_t a_sb, a_sr, b_sb, b_sr, o_sb, o_sr;
  int B, M, Mo, w, off, lo, hi, tiles_per_batch;
  int total_tiles;
  unsigned long long *status;  // device status word (bit 3: a small-window kernel gave up on a bounded wait)
  int in_bytes;    // bytes of one input stage
  int slab_bytes;  // bytes of the slab inside an input stage
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool BF16> __device__ __forceinline__ uint16_t to16(float f) {
  if (BF16) {
    __nv_bfloat16 v = __float2bfloat16_rn(f);
    return *reinterpret_cast<uint16_t *>(&v);
  }
  __half v = __float2half_rn(f);
  return *reinterpret_cast<uint16_t *>(&v);
}

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid) {
  // 16 bytes global -> shared without passing through registers; !valid writes zeros and reads nothing
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// untiled bulk copy shared -> global (both 16-byte aligned, size a multiple of 16 bytes), tracked by bulk groups
__device__ __forceinline__ void bulk_store(void *dst, const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_addr(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// two floats -> two 16-bit values in one word (first in the low half)
template <bool BF16> __device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// The consecutive tiles a CTA owns, as (batch, tile in batch) of the first one and a count.
struct TileRange {
  int b, tb, count;
  __device__ TileRange(int total, int per_batch) {
    const int per = total / (int)gridDim.x, rem = total % (int)gridDim.x;
    const int first = (int)blockIdx.x * per + min((int)blockIdx.x, rem);
    count = per + ((int)blockIdx.x < rem ? 1 : 0);
    b = first / per_batch;
    tb = first % per_batch;
  }
};

template <int KEEP> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(KEEP) : "memory"); }

// Rows [row0, row0 + nrows) of a (batch, rows, N) operand with unit column stride -> shared memory with
// pitch PITCH bytes, asynchronously; rows outside [vlo, vhi) are zero-filled.  16-byte pieces, coalesced.
template <int N, int PITCH>
__device__ __forceinline__ void load_rows(uint8_t *dst, const uint16_t *src, int64_t sb, int64_t sr, int b, int row0, int nrows,
                                          int vlo, int vhi) {
  constexpr int PIECES = N / 8;  // 16-byte pieces per row
  for (int e = threadIdx.x; e < nrows * PIECES; e += SM_THREADS) {
    const int r = e / PIECES, pc = e % PIECES;
    const int row = row0 + r;
    const bool ok = row >= vlo && row < vhi;
    cp_async16(dst + r * PITCH + pc * 16, ok ? src + b * sb + row * sr + pc * 8 : src, ok);
  }
}

// The common case of load_rows: all nrows rows are in range and contiguous in global memory (row stride N), so 16-byte
// piece e of the block goes from src + 8e elements to dst + 16e + 16 (e / pieces-per-row) bytes: no per-piece row
// arithmetic, no range checks.
template <int N>
__device__ __forceinline__ void load_block(uint8_t *dst, const uint16_t *src, int nrows) {
  constexpr int PIECES = N / 8;
  const uint32_t d = smem_addr(dst);
  for (int e = threadIdx.x; e < nrows * PIECES; e += SM_THREADS)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + e * 16 + (e / PIECES) * 16), "l"(src + e * 8) : "memory");
}

// nelem contiguous 16-bit elements between global memory and shared memory.  `sm` holds the span at the
// same offset modulo 16 bytes as `gm`, so 16-byte accesses line up on both sides.  The body of the inbound
// copy is asynchronous; the (rare) unaligned head and tail elements are copied through registers.
__device__ __forceinline__ void copy_span_in(uint16_t *sm, const uint16_t *gm, int64_t nelem) {
  const int head = (int)(((16 - (reinterpret_cast<uintptr_t>(gm) & 15)) & 15) >> 1);
  const int64_t h = head < nelem ? head : nelem;
  for (int64_t e = threadIdx.x; e < h; e += SM_THREADS) sm[e] = gm[e];
  const int64_t nvec = (nelem - h) / 8;
  for (int64_t e = threadIdx.x; e < nvec; e += SM_THREADS) cp_async16(sm + h + e * 8, gm + h + e * 8, true);
  for (int64_t e = h + nvec * 8 + threadIdx.x; e < nelem; e += SM_THREADS) sm[e] = gm[e];
}
__device__ __forceinline__ void copy_span_out(uint16_t *gm, const uint16_t *sm, int64_t nelem) {
  const int head = (int)(((16 - (reinterpret_cast<uintptr_t>(gm) & 15)) & 15) >> 1);
  const int64_t h = head < nelem ? head : nelem;
  for (int64_t e = threadIdx.x; e < h; e += SM_THREADS) gm[e] = sm[e];
  const int64_t nvec = (nelem - h) / 8;
  for (int64_t e = threadIdx.x; e < nvec; e += SM_THREADS)
    *reinterpret_cast<uint4 *>(gm + h + e * 8) = *reinterpret_cast<const uint4 *>(sm + h + e * 8);
  for (int64_t e = h + nvec * 8 + threadIdx.x; e < nelem; e += SM_THREADS) gm[e] = sm[e];
}

template <int N> struct SmallLayout {
  static constexpr int PITCH = N * 2 + 16;              // bytes; keeps ldmatrix rows on distinct banks
  static constexpr int TILE_BYTES = SM_ROWS * PITCH;    // X tile / output staging
  // Shared memory is sized for the actual window (more CTAs per SM for narrow bands).  Pieces: the X tile /
  // output staging (TILE_BYTES), a slab of (128 + 2w) rows rounded up to 16, and the packed band image of up
  // to (128 + 2w) rows of 2w+1 elements plus 16 bytes of alignment slack.  Inputs are double-buffered.
  static int slab_bytes(int w) { return ((SM_ROWS + 2 * w + 15) & ~15) * PITCH; }
  static int img_bytes(int w) { return (((SM_ROWS + 2 * w) * (2 * w + 1) * 2 + 16 + 15) / 16) * 16; }
  static int nt_in(int w) { return TILE_BYTES + slab_bytes(w); }   // band_nt inputs: X tile, Y slab
  static int nt_bytes(int w) { return 2 * nt_in(w) + img_bytes(w); }
  static int mm_in(int w) { return slab_bytes(w) + img_bytes(w); }  // band_n / band_t inputs: slab, band image
  static int mm_bytes(int w) { return 2 * mm_in(w) + TILE_BYTES; }
};

// ---------------------------------------------------------------------------------------------------
// band_nt: Band[i, j] = X[i, :] . Y[i + j - w + off, :]
// ---------------------------------------------------------------------------------------------------
// NT_MAX = 8-column blocks of the dense product a warp may need: (16 + 2w) / 8 rounded up, compiled for
// w <= 8, w <= 16 and w <= 32 so that narrow windows do not carry the accumulators of wide ones.
template <bool BF16, int N, int NT_MAX> __global__ void __launch_bounds__(SM_THREADS, (NT_MAX <= 6 && N <= 64) ? 4 : 2) band_nt_small_kernel(const SmallParams p) {
  using L = SmallLayout<N>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint16_t *img = reinterpret_cast<uint16_t *>(smem + 2 * p.in_bytes);
  const int W = 2 * p.w + 1;
  const int slab = SM_ROWS + 2 * p.w;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nt_count = (16 + 2 * p.w + 7) / 8;

  // inputs of a tile -> stage buffer, asynchronously
  auto prefetch = [&](int b, int r0, int stage) {
    uint8_t *xs = smem + stage * p.in_bytes, *ys = xs + L::TILE_BYTES;
    const int yrows = (slab + 7) & ~7, y0 = r0 - p.w + p.off;
    if (p.a_sr == N && r0 + SM_ROWS <= p.M)
      load_block<N>(xs, p.a + b * p.a_sb + (int64_t)r0 * N, SM_ROWS);
    else
      load_rows<N, L::PITCH>(xs, p.a, p.a_sb, p.a_sr, b, r0, SM_ROWS, 0, p.M);
    if (p.b_sr == N && y0 >= p.lo && y0 + yrows <= p.hi)
      load_block<N>(ys, p.b + b * p.b_sb + (int64_t)y0 * N, yrows);
    else
      load_rows<N, L::PITCH>(ys, p.b, p.b_sb, p.b_sr, b, y0, yrows, p.lo, p.hi);
  };

  // this CTA's tiles are consecutive: (batch, tile-in-batch) advance without a division per tile
  TileRange tr(p.total_tiles, p.tiles_per_batch);
  int nb = tr.b, ntb = tr.tb;   // the tile being prefetched
  if (tr.count > 0) prefetch(nb, ntb * SM_ROWS, 0);
  cp_async_commit();
  for (int it = 0; it < tr.count; ++it) {
    const int stage = it & 1;
    const int b = nb, r0 = ntb * SM_ROWS;
    if (++ntb == p.tiles_per_batch) { ntb = 0; ++nb; }
    if (it + 1 < tr.count) prefetch(nb, ntb * SM_ROWS, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();  // this tile's inputs have landed (the next tile's may still be in flight)
    if (threadIdx.x == 0) bulk_wait_read0();  // the previous tile's image has left shared memory
    __syncthreads();     // ... for every thread

    const int vr = min(SM_ROWS, p.M - r0), p0 = r0 - p.w + p.off;  // slab row s <-> position p0 + s
    const uint8_t *xs = smem + stage * p.in_bytes, *ys = xs + L::TILE_BYTES;
    uint16_t *out = p.o + ((int64_t)b * p.M + r0) * W;
    uint16_t *im = img + ((reinterpret_cast<uintptr_t>(out) & 15) >> 1);  // same 16-byte phase as the destination

    float acc[NT_MAX][4];
#pragma unroll
    for (int nt = 0; nt < NT_MAX; nt++)
#pragma unroll
      for (int c = 0; c < 4; c++) acc[nt][c] = 0.f;
    const uint32_t xbase = smem_addr(xs) + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * L::PITCH + 16 * (lane >> 4);
    const uint32_t ybase = smem_addr(ys) + (warp * 16 + (lane & 7)) * L::PITCH + 16 * (lane >> 3);
#pragma unroll
    for (int ks = 0; ks < N / 32; ks++) {  // 32 hidden columns per pass: two k-steps
      uint32_t a0[4], a1[4];
      ldmatrix_x4(a0, xbase + ks * 64);
      ldmatrix_x4(a1, xbase + ks * 64 + 32);
#pragma unroll
      for (int nt = 0; nt < NT_MAX; nt++) {
        if (nt < nt_count) {
          uint32_t bb[4];  // keys 8nt..8nt+7 of the warp's slab x hidden 32ks..32ks+31
          ldmatrix_x4(bb, ybase + nt * 8 * L::PITCH + ks * 64);
          mma_16816<BF16>(acc[nt], a0, bb[0], bb[1]);
          mma_16816<BF16>(acc[nt], a1, bb[2], bb[3]);
        }
      }
    }
    // scatter into the packed image: dense (row rl, slab column col) -> band index j = col - rl
    const bool edge = vr < SM_ROWS || p0 < p.lo || p0 + slab > p.hi;
    if (!edge) {
      // interior tile: element (q, nt, e) of this lane sits at rowp[q] + 8nt + e and has j = jb[q] + 8nt + e
      uint16_t *rowp[2];
      int jb[2];
#pragma unroll
      for (int q = 0; q < 2; q++) {
        const int rl = g + 8 * q;
        jb[q] = 2 * t - rl;
        rowp[q] = im + (warp * 16 + rl) * W + jb[q];
      }
#pragma unroll
      for (int nt = 0; nt < NT_MAX; nt++) {
        if (nt < nt_count) {
#pragma unroll
          for (int q = 0; q < 2; q++) {
            const uint32_t pr = pack16<BF16>(acc[nt][2 * q], acc[nt][2 * q + 1]);
            if ((unsigned)(jb[q] + nt * 8) < (unsigned)W) rowp[q][nt * 8] = (uint16_t)pr;
            if ((unsigned)(jb[q] + nt * 8 + 1) < (unsigned)W) rowp[q][nt * 8 + 1] = (uint16_t)(pr >> 16);
          }
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT_MAX; nt++) {
        if (nt < nt_count) {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            const int rl = g + 8 * (c >> 1), col = nt * 8 + 2 * t + (c & 1);
            const int j = col - rl;
            bool ok = j >= 0 && j < W;
            float val = acc[nt][c];
            const int pos = p0 + warp * 16 + col;
            ok = ok && warp * 16 + rl < vr;
            if (pos < p.lo || pos >= p.hi) val = 0.f;
            if (ok) im[(warp * 16 + rl) * W + j] = to16<BF16>(val);
          }
        }
      }
    }
    // a full tile whose destination is 16-byte aligned leaves with one bulk copy (128 rows of 2w+1 16-bit elements are
    // a multiple of 16 bytes); ragged or unaligned tiles are copied out by all threads
    const bool bulk_out = vr == SM_ROWS && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (bulk_out) fence_async_smem();
    __syncthreads();
    if (bulk_out) {
      if (threadIdx.x == 0) {
        bulk_store(out, im, (uint32_t)(SM_ROWS * W * 2));
        bulk_commit_group();
      }
    } else {
      copy_span_out(out, im, (int64_t)vr * W);
    }
  }
  cp_async_wait<0>();
  if (threadIdx.x == 0) bulk_wait_all0();
}

// ---------------------------------------------------------------------------------------------------
// band_n (TR = false): Out[i, :] = sum_j Band[i, j] Y[i + j - w + off, :]          tile = 128 band rows
// band_t (TR = true):  Out[p, :] = sum_i Band[i, p - off - i + w] X[i, :]          tile = 128 positions
// ---------------------------------------------------------------------------------------------------
template <bool BF16, int N, bool TR, int KS_MAX> __global__ void __launch_bounds__(SM_THREADS, N <= 64 ? 4 : 2) band_mm_small_kernel(const SmallParams p) {
  using L = SmallLayout<N>;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *os = smem + 2 * p.in_bytes;  // output staging
  __shared__ __align__(8) uint64_t img_full[2];   // completion of a stage's bulk-loaded band image
  __shared__ int abort_flag;
  const int W = 2 * p.w + 1;
  const int slab = SM_ROWS + 2 * p.w;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ksteps = (16 + 2 * p.w + 15) / 16;
  const int out_rows = TR ? p.Mo : p.M;
  if (threadIdx.x == 0) {
    ptx::mbar_init(smem_addr(&img_full[0]), 1);
    ptx::mbar_init(smem_addr(&img_full[1]), 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();

  // Per tile: t0 = first band row (band_n) / position (band_t).  Slab row s of the other operand is
  // position t0 - w + off + s (band_n) or band row t0 - off - w + s (band_t).  The image holds band rows
  // [t0, t0 + 128) (band_n) or [s0, s0 + 128 + 2w) (band_t), clipped to [0, M).
  auto geometry = [&](int t0, int &s0, int &ilo, int &ihi) {
    s0 = TR ? t0 - p.off - p.w : t0 - p.w + p.off;
    const int img_row0 = TR ? s0 : t0;
    ilo = max(img_row0, 0);
    ihi = min(img_row0 + (TR ? slab : SM_ROWS), p.M);
  };
  auto image_of = [&](int stage, const uint16_t *band) -> uint16_t * {
    uint16_t *img = reinterpret_cast<uint16_t *>(smem + stage * p.in_bytes + p.slab_bytes);
    return img + ((reinterpret_cast<uintptr_t>(band) & 15) >> 1);  // same 16-byte phase as the source
  };
  // the image of a tile moves with one bulk copy when its source is 16-byte aligned and a multiple of 16 bytes long
  auto image_bulk = [&](const uint16_t *band, int rows) -> bool {
    return (reinterpret_cast<uintptr_t>(band) & 15) == 0 && ((rows * W * 2) & 15) == 0;
  };
  auto prefetch = [&](int b, int t0, int stage) {
    int s0, ilo, ihi;
    geometry(t0, s0, ilo, ihi);
    uint8_t *ys = smem + stage * p.in_bytes;
    const int yrows = (slab + 15) & ~15, vlo = TR ? 0 : p.lo, vhi = TR ? p.M : p.hi;
    if (p.b_sr == N && s0 >= vlo && s0 + yrows <= vhi)
      load_block<N>(ys, p.b + b * p.b_sb + (int64_t)s0 * N, yrows);
    else
      load_rows<N, L::PITCH>(ys, p.b, p.b_sb, p.b_sr, b, s0, yrows, vlo, vhi);
    if (ihi > ilo) {
      const uint16_t *band = p.a + ((int64_t)b * p.M + ilo) * W;
      if (image_bulk(band, ihi - ilo)) {
        if (threadIdx.x == 0) {
          const uint32_t bytes = (uint32_t)((ihi - ilo) * W * 2);
          ptx::mbar_expect_tx(smem_addr(&img_full[stage]), bytes);
          ptx::bulk_load_1d(smem_addr(image_of(stage, band)), band, bytes, smem_addr(&img_full[stage]));
        }
      } else {
        copy_span_in(image_of(stage, band), band, (int64_t)(ihi - ilo) * W);
      }
    }
  };

  TileRange tr(p.total_tiles, p.tiles_per_batch);
  int nb = tr.b, ntb = tr.tb;
  uint32_t full_phase[2] = {0u, 0u};
  bool aborted = false;
  if (tr.count > 0) prefetch(nb, ntb * SM_ROWS, 0);
  cp_async_commit();
  for (int it = 0; it < tr.count; ++it) {
    const int stage = it & 1;
    const int b = nb, t0 = ntb * SM_ROWS;
    if (++ntb == p.tiles_per_batch) { ntb = 0; ++nb; }
    if (it + 1 < tr.count) prefetch(nb, ntb * SM_ROWS, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();

    int s0, ilo, ihi;
    geometry(t0, s0, ilo, ihi);
    const uint16_t *band = p.a + ((int64_t)b * p.M + ilo) * W;
    if (ihi > ilo && image_bulk(band, ihi - ilo)) {
      if (!ptx::mbar_wait(smem_addr(&img_full[stage]), full_phase[stage], &abort_flag)) aborted = true;
      full_phase[stage] ^= 1u;
    }
    __syncthreads();  // this tile's inputs are visible to all; the previous tile's output staging is drained
    if (abort_flag) { aborted = true; break; }

    const uint8_t *ys = smem + stage * p.in_bytes;
    // the image starts at band row ilo; offsets below are relative to the unclipped first row
    const int img_row0 = TR ? s0 : t0;
    const uint16_t *im = image_of(stage, band) - (ilo - img_row0) * W;
    const bool edge = ilo != img_row0 || ihi != img_row0 + (TR ? slab : SM_ROWS) ||
                      (TR ? (t0 < p.lo || t0 + SM_ROWS > p.hi) : (s0 < p.lo || s0 + slab > p.hi));
    // image offset of dense element (ml, kc) = abase[ml] + kc (band_n) or abase[ml] + kc * 2w (band_t)
    int abase[2];
    // interior tiles: element with compile-time offset C = 16 ks + 8 (r >> 1) + e sits at ptr[q][C] (band_n) or
    // ptr[q][C * 2w] (band_t) and is inside the band iff (unsigned)(jd[q] + C) < W resp. (unsigned)(jd[q] - C) < W
    const uint16_t *ptr[2];
    int jd[2];
#pragma unroll
    for (int q = 0; q < 2; q++) {
      const int ml = g + 8 * q;
      abase[q] = TR ? warp * 16 * W + 2 * p.w + ml : (warp * 16 + ml) * W - ml;
      jd[q] = TR ? ml - 2 * t + 2 * p.w : 2 * t - ml;
      ptr[q] = im + abase[q] + (TR ? 2 * t * (W - 1) : 2 * t);
    }
    const int kstride = W - 1;

    float acc[N / 8][4];
#pragma unroll
    for (int nt = 0; nt < N / 8; nt++)
#pragma unroll
      for (int c = 0; c < 4; c++) acc[nt][c] = 0.f;
    // B fragments: rows (reduction index) of the slab starting at the warp's first one, hidden columns in n
    const uint32_t ybase = smem_addr(ys) + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * L::PITCH + 16 * (lane >> 4);
#pragma unroll
    for (int ks = 0; ks < KS_MAX; ks++) {
      if (ks < ksteps) {
        // A fragment gathered from the packed image.  Dense element (m = ml, k = kc) with kc counted from
        // the warp's first slab row:  band_n: row i = t0 + 16 warp + ml, j = kc - ml
        //                             band_t: position = t0 + 16 warp + ml, row i = s0 + 16 warp + kc, j = ml - kc + 2w
        uint32_t a[4];
        if (!edge) {
#pragma unroll
          for (int r = 0; r < 4; r++) {
            const int q = r & 1;
            uint32_t v = 0;
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int C = ks * 16 + 8 * (r >> 1) + e;
              if (!TR) {
                if ((unsigned)(jd[q] + C) < (unsigned)W) v |= (uint32_t)ptr[q][C] << (16 * e);
              } else {
                if ((unsigned)(jd[q] - C) < (unsigned)W) v |= (uint32_t)ptr[q][C * kstride] << (16 * e);
              }
            }
            a[r] = v;
          }
        } else {
#pragma unroll
          for (int r = 0; r < 4; r++) {
            const int ml = g + 8 * (r & 1), kc0 = ks * 16 + 2 * t + 8 * (r >> 1);
            uint32_t v = 0;
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int kc = kc0 + e;
              // band index and image offset: band_n j = kc - ml, offset row*W + j; band_t j = ml - kc + 2w, row kc
              const int j = TR ? ml - kc + 2 * p.w : kc - ml;
              const int idx = TR ? abase[r & 1] + kc * (W - 1) : abase[r & 1] + kc;
              bool ok = j >= 0 && j < W;
              // ragged or sequence-end tile: also check the band row and the position
              const int i = TR ? s0 + warp * 16 + kc : t0 + warp * 16 + ml;
              const int pos = TR ? t0 + warp * 16 + ml : s0 + warp * 16 + kc;
              ok = ok && i >= ilo && i < ihi && pos >= p.lo && pos < p.hi;
              if (ok) v |= (uint32_t)im[idx] << (16 * e);
            }
            a[r] = v;
          }
        }
#pragma unroll
        for (int np = 0; np < N / 16; np++) {  // two n-tiles (16 hidden columns) per ldmatrix
          uint32_t bb[4];
          ldmatrix_x4_trans(bb, ybase + ks * 16 * L::PITCH + np * 32);
          mma_16816<BF16>(acc[2 * np], a, bb[0], bb[1]);
          mma_16816<BF16>(acc[2 * np + 1], a, bb[2], bb[3]);
        }
      }
    }
    // stage the 128 x N output tile, then write whole rows with 16-byte stores
#pragma unroll
    for (int nt = 0; nt < N / 8; nt++)
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        const int row = warp * 16 + g + 4 * c, col = nt * 8 + 2 * t;
        *reinterpret_cast<uint32_t *>(os + row * L::PITCH + col * 2) = pack16<BF16>(acc[nt][c], acc[nt][c + 1]);
      }
    __syncthreads();
    constexpr int PIECES = N / 8;
    uint16_t *obase = p.o + b * p.o_sb + (int64_t)t0 * p.o_sr;
    const int vrows = min(SM_ROWS, out_rows - t0);
    if (p.o_sr == N) {  // contiguous output rows: piece e of the block
      for (int e = threadIdx.x; e < vrows * PIECES; e += SM_THREADS)
        *reinterpret_cast<uint4 *>(obase + e * 8) = *reinterpret_cast<const uint4 *>(os + e * 16 + (e / PIECES) * 16);
    } else {
      for (int e = threadIdx.x; e < vrows * PIECES; e += SM_THREADS) {
        const int r = e / PIECES, pc = e % PIECES;
        *reinterpret_cast<uint4 *>(obase + (int64_t)r * p.o_sr + pc * 8) = *reinterpret_cast<const uint4 *>(os + r * L::PITCH + pc * 16);
      }
    }
  }
  cp_async_wait<0>();
  if (aborted || abort_flag) {
    __syncthreads();
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, 8ull);
    // give a bulk copy that may still be in flight time to land before shared memory goes away
    const uint64_t t_begin = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t_begin < 2000000ull) __nanosleep(1000);
  }
}

// Persistent grid: as many CTAs as fit on the device at this shared-memory size (each loops over tiles).
template <typename K> cudaError_t launch(K kern, const SmallParams &k, int smem_bytes, cudaStream_t stream) {
  if (smem_bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
  }
  int per_sm = 0, dev = 0, sms = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, SM_THREADS, smem_bytes);
  if (e == cudaSuccess) e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorInvalidConfiguration;
  const int64_t resident = (int64_t)per_sm * sms;
  const int grid = (int)(k.total_tiles < resident ? k.total_tiles : resident);
  kern<<<grid, SM_THREADS, smem_bytes, stream>>>(k);
  return cudaGetLastError();
}

template <bool BF16, int N> cudaError_t launch_small_n(Primitive prim, SmallParams k, cudaStream_t stream) {
  using L = SmallLayout<N>;
  k.slab_bytes = L::slab_bytes(k.w);
  if (prim == BAND_NT) {
    k.in_bytes = L::nt_in(k.w);
    if (k.w <= 8) return launch(band_nt_small_kernel<BF16, N, 4>, k, L::nt_bytes(k.w), stream);
    if (k.w <= 16) return launch(band_nt_small_kernel<BF16, N, 6>, k, L::nt_bytes(k.w), stream);
    return launch(band_nt_small_kernel<BF16, N, 10>, k, L::nt_bytes(k.w), stream);
  }
  k.in_bytes = L::mm_in(k.w);
  const int smem = L::mm_bytes(k.w);
  if (prim == BAND_N) {
    if (k.w <= 8) return launch(band_mm_small_kernel<BF16, N, false, 2>, k, smem, stream);
    if (k.w <= 16) return launch(band_mm_small_kernel<BF16, N, false, 3>, k, smem, stream);
    return launch(band_mm_small_kernel<BF16, N, false, 5>, k, smem, stream);
  }
  if (k.w <= 8) return launch(band_mm_small_kernel<BF16, N, true, 2>, k, smem, stream);
  if (k.w <= 16) return launch(band_mm_small_kernel<BF16, N, true, 3>, k, smem, stream);
  return launch(band_mm_small_kernel<BF16, N, true, 5>, k, smem, stream);
}

bool rows_ok(const void *data, int64_t sb, int64_t sr, int64_t sc, int batch) {
  return (reinterpret_cast<uintptr_t>(data) & 15u) == 0 && sc == 1 && sr > 0 && (sr % 8) == 0 && (batch <= 1 || (sb % 8) == 0);
}

}  // namespace

bool small_eligible(Primitive prim, const Problem &p) {
  if (p.dtype != WMM_F16 && p.dtype != WMM_BF16) return false;
  if (p.w < 1 || p.w > SM_MAX_W) return false;
  if (p.N != 32 && p.N != 64 && p.N != 128) return false;
  const int tile_rows = prim == BAND_T ? p.Mo : p.M;
  if ((int64_t)p.B * ((tile_rows + SM_ROWS - 1) / SM_ROWS) > 0x7fffffffLL) return false;
  switch (prim) {
    case BAND_NT: return rows_ok(p.a, p.a_sb, p.a_sr, p.a_sc, p.B) && rows_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B);
    default: return rows_ok(p.b, p.b_sb, p.b_sr, p.b_sc, p.B) && rows_ok(p.o, p.o_sb, p.o_sr, p.o_sc, p.B);
  }
}

cudaError_t launch_small(Primitive prim, const Problem &p, cudaStream_t stream, int *launches) {
  SmallParams k;
  k.a = static_cast<const uint16_t *>(p.a);
  k.b = static_cast<const uint16_t *>(p.b);
  k.o = static_cast<uint16_t *>(p.o);
  k.a_sb = p.a_sb; k.a_sr = p.a_sr; k.b_sb = p.b_sb; k.b_sr = p.b_sr; k.o_sb = p.o_sb; k.o_sr = p.o_sr;
  k.status = device_status_word();
  k.B = p.B; k.M = p.M; k.Mo = p.Mo; k.w = p.w; k.off = p.off; k.lo = p.lo; k.hi = p.hi;
  const int tile_rows = prim == BAND_T ? p.Mo : p.M;
  k.tiles_per_batch = (tile_rows + SM_ROWS - 1) / SM_ROWS;
  k.total_tiles = k.tiles_per_batch * p.B;
  const bool bf16 = p.dtype == WMM_BF16;
  cudaError_t e;
  switch (p.N) {
    case 32: e = bf16 ? launch_small_n<true, 32>(prim, k, stream) : launch_small_n<false, 32>(prim, k, stream); break;
    case 64: e = bf16 ? launch_small_n<true, 64>(prim, k, stream) : launch_small_n<false, 64>(prim, k, stream); break;
    default: e = bf16 ? launch_small_n<true, 128>(prim, k, stream) : launch_small_n<false, 128>(prim, k, stream); break;
  }
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

}  // namespace wmm
