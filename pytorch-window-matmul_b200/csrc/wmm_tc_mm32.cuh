// band_n / band_t for fp32 tensors on the tensor cores (tcgen05.mma.kind::tf32: the operands' low 13 mantissa bits are
// ignored, sums are fp32).  Included by wmm_tc.cu (inside namespace wmm::<anon>).  Taken only with WMM_FLAG_TF32.
//
// Same plan as the 16-bit kernel (wmm_tc_mm.cuh) with the reduction cut into chunks of 64 instead of 128, so that a
// pipeline stage holds the same bytes: a band box of 32 KB and 64 rows of the other operand.
//   band_n (TR = false): box = 128 band rows x 64 x-columns, two TMA boxes of 32 columns (128-byte lines): a K-major A
//                        operand; B = 64 positions x NH of Y, hidden index contiguous: an MN-major B operand.
//   band_t (TR = true):  box = 64 band rows x 128 x-columns, four TMA boxes of 32 columns: the x index is the M
//                        dimension, so the same kind of bytes serve as an MN-major A operand; B = 64 rows x NH of X.
// MN-major fp32 operands need their own shared-memory layout (layout type 1 of the descriptor: 128-byte lines swizzled
// in 32-byte atoms, which TMA writes with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B): 32 elements (128 bytes) of the M / N
// index are contiguous, the 32-byte quarter of a line is XOR-ed with the line number modulo 4, four k-rows make a
// 512-byte group (the stride offset), the next 32 elements are one leading offset further; an instruction consumes
// eight k-rows, so a k-step advances the start address by 1024 bytes.
//
// Warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2-5 = mask, 6-9 = epilogue (as in the 16-bit kernel).

constexpr int M32_RC = 64;   // reduction elements per chunk

template <int NH> struct Mm32Smem {
  static constexpr int BAND_BYTES = 128 * M32_RC * 4;      // 32 KB either way round
  static constexpr int NBOX = NH / 32;                     // 32-column boxes of the other operand and of the output
  static constexpr int OTHER_BOX = M32_RC * 128;           // 64 rows of 128 bytes
  static constexpr int OTHER_BYTES = NBOX * OTHER_BOX;
  static constexpr int OUT_BOX = 128 * 128;                // 128 rows of 128 bytes
  static constexpr int OUT_BYTES = NBOX * OUT_BOX;
  static constexpr int STAGES = 4;
  static constexpr int STAGE_BYTES = BAND_BYTES + OTHER_BYTES;
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int OFF_BARS = OFF_OUT + OUT_BYTES;
  static constexpr int NBARS = 3 * STAGES + 4;
  static constexpr int OFF_MISC = OFF_BARS + NBARS * 8;
  static constexpr int BYTES = OFF_MISC + 32;
  static constexpr int ALLOC = BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = 2 * NH < 32 ? 32 : 2 * NH;  // two accumulator stages
};

template <int NH, bool TR>
__global__ void __launch_bounds__(MM_THREADS, 1)
band_mm_tf32_kernel(const __grid_constant__ CUtensorMap map_band, const __grid_constant__ CUtensorMap map_other,
                    const __grid_constant__ CUtensorMap map_out, const MmParams p) {
  using S = Mm32Smem<NH>;
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
  griddep_launch_dependents();
  griddep_wait();

  // Tile / chunk geometry.  t0 = first row (band_n) or position (band_t) of the tile; chunk c covers 64 steps of the
  // reduction:
  //   band_n: box rows i = t0 .. t0+127, x = t0 + 64c + kk,                  position of column kk: t0 - w + off + 64c + kk
  //   band_t: box rows i = t0 - off - w + 64c + ii (ii < 64), x = t0 - off + w + xx (xx < 128),  position of column xx: t0 + xx
  auto chunk_is_plain = [&](int t0, int c) -> bool {   // true when no element of the box needs zeroing
    if (c * M32_RC < 127 || c * M32_RC + (M32_RC - 1) > 2 * p.w) return false;
    if (!TR) {
      const int p0 = t0 - p.w + p.off + c * M32_RC;
      return p0 >= p.lo && p0 + M32_RC <= p.hi;
    }
    return t0 >= p.lo && t0 + 128 <= p.hi;
  };
  // the MMA thread waits for the mask warps only at sync points (see wmm_tc_mm.cuh)
  auto mask_sync = [&](bool plain, int &since) -> bool {
    if (!plain || since >= S::STAGES - 1) {
      since = 0;
      return true;
    }
    ++since;
    return false;
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
          const uint32_t band_dst = base + s * S::STAGE_BYTES, other_dst = band_dst + S::BAND_BYTES;
          const int x0 = TR ? t0 - p.off + p.w : t0 + c * M32_RC;
          const int row0 = TR ? t0 - p.off - p.w + c * M32_RC : t0;
          const int orow0 = TR ? row0 : t0 - p.w + p.off + c * M32_RC;
          if (TR) {
#pragma unroll
            for (int bx = 0; bx < 4; bx++) tma_load_3d(band_dst + bx * (M32_RC * 128), &map_band, bar_full(s), x0 + 32 * bx, row0, b);
          } else {
#pragma unroll
            for (int bx = 0; bx < 2; bx++) tma_load_3d(band_dst + bx * (128 * 128), &map_band, bar_full(s), x0 + 32 * bx, row0, b);
          }
#pragma unroll
          for (int bx = 0; bx < S::NBOX; bx++) tma_load_3d(other_dst + bx * S::OTHER_BOX, &map_other, bar_full(s), 32 * bx, orow0, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC = instr_desc_tf32(TR, true, TILE, NH);
      constexpr uint64_t ADESC_N = smem_desc_base(16, 1024, 2u);                 // K-major: 8-row groups 1024 B apart
      constexpr uint64_t ADESC_T = smem_desc_base(M32_RC * 128, 512, 1u);        // MN-major: next 32 x one box further
      constexpr uint64_t BDESC = smem_desc_base(S::OTHER_BOX, 512, 1u);          // MN-major: next 32 hidden columns one box further
      int it = 0, tit = 0, since = 0, mk[S::STAGES];
      for (int s = 0; s < S::STAGES; s++) mk[s] = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++tit) {
        const int t0 = (tile % p.tiles_per_batch) * TILE;
        const int as = tit & 1;
        if (!(ok = mbar_wait(bar_acc_empty(as), ((tit >> 1) & 1) ^ 1, abort_flag))) break;
        for (int c = 0; c < p.nchunks; ++c, ++it) {
          const int s = it % S::STAGES;
          if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
          if (mask_sync(chunk_is_plain(t0, c), since)) {
            if (!(ok = mbar_wait(bar_masked(s), mk[s] & 1, abort_flag))) break;
            ++mk[s];
          }
          tc_fence_after_sync();
          const uint32_t a_addr = base + s * S::STAGE_BYTES, b_addr = a_addr + S::BAND_BYTES;
#pragma unroll
          for (int k = 0; k < M32_RC / 8; k++) {
            // K-major A: a k-step of 8 columns is 32 B along the 128-byte line, the second 32 columns are the second box
            const uint32_t a_off = TR ? (uint32_t)k * 1024u : (uint32_t)(k >> 2) * (128u * 128u) + (uint32_t)(k & 3) * 32u;
            umma_tf32(tmem_base + as * NH, smem_desc(TR ? ADESC_T : ADESC_N, a_addr + a_off),
                      smem_desc(BDESC, b_addr + (uint32_t)k * 1024u), IDESC, (c > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty(s));
        }
        if (ok) umma_commit(bar_acc_full(as));
      }
    }
  } else if (warp < 6) {
    // ---------------- mask warps ----------------
    // band_n: thread <-> one of the 128 box rows, 16 pieces of 4 columns.  band_t: thread <-> (box row ii = t % 64, the
    // 64 columns of half t / 64): 16 pieces of 4 columns as well.
    const int mt = (warp - 2) * 32 + lane;
    const int row = TR ? (mt & 63) : mt;
    const int cbase = TR ? (mt >> 6) * 64 : 0;   // first column this thread looks after
    int it = 0, since = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
      const int t0 = (tile % p.tiles_per_batch) * TILE;
      for (int c = 0; c < p.nchunks; ++c, ++it) {
        const int s = it % S::STAGES;
        if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
        const bool plain = chunk_is_plain(t0, c);
        const bool sync = mask_sync(plain, since);
        if (plain) {
          if (sync) mbar_arrive(bar_masked(s));
          continue;
        }
        // columns [col_lo, col_hi] of this row are band entries inside the sequence; the rest is zeroed
        int col_lo, col_hi;
        if (!TR) {
          const int p0 = t0 - p.w + p.off + c * M32_RC;
          col_lo = max(row - c * M32_RC, p.lo - p0);
          col_hi = min(row - c * M32_RC + 2 * p.w, p.hi - p0 - 1);
        } else {
          col_lo = max(row + c * M32_RC - 2 * p.w, p.lo - t0);
          col_hi = min(row + c * M32_RC, p.hi - t0 - 1);
        }
        const uint32_t tile_addr = base + s * S::STAGE_BYTES;
        // 16-byte piece holding columns 4g .. 4g+3 of this row: box g / 8; band_n (K-major box): slot (g % 8) ^ (row % 8);
        // band_t (MN-major box, 32-byte atoms): 32-byte quarter ((g % 8) / 2) ^ (row % 4), half g % 2
        auto piece = [&](int g) -> uint32_t {
          if (TR) return tile_addr + (g >> 3) * (M32_RC * 128) + row * 128 + (((((g & 7) >> 1) ^ (row & 3)) << 5) | ((g & 1) << 4));
          return tile_addr + (g >> 3) * (128 * 128) + row * 128 + (((g & 7) ^ (row & 7)) << 4);
        };
        const int g0 = cbase >> 2;
        for (int g = g0; g < g0 + 16; g++) {
          const int c0 = g * 4;
          if (c0 >= col_lo && c0 + 3 <= col_hi) continue;              // wholly kept
          const uint32_t a = piece(g);
          if (c0 + 3 < col_lo || c0 > col_hi) {                         // wholly dropped
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(a), "r"(0u) : "memory");
            continue;
          }
          uint32_t v[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(a) : "memory");
#pragma unroll
          for (int k = 0; k < 4; k++)
            if (c0 + k < col_lo || c0 + k > col_hi) v[k] = 0u;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
        }
        if (!TR && mt < M32_RC) {
          // rows of the other operand whose position is outside the sequence: zero them too, so that whatever sits
          // there (an unfilled halo, Inf, NaN) cannot reach the product as 0 * x
          const int pos = t0 - p.w + p.off + c * M32_RC + mt;
          if (pos < p.lo || pos >= p.hi) {
            const uint32_t o_addr = tile_addr + S::BAND_BYTES + mt * 128;
#pragma unroll
            for (int bx = 0; bx < S::NBOX; bx++)
#pragma unroll
              for (int q = 0; q < 8; q++)
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(o_addr + bx * S::OTHER_BOX + q * 16), "r"(0u) : "memory");
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
      for (int g = 0; g < S::NBOX; g++) {
        uint32_t v[32];
        tmem_ld_x32(taddr + g * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 8; q8++) {
          const uint32_t a = stage + g * S::OUT_BOX + rr * 128 + ((q8 ^ (rr & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v[4 * q8]), "r"(v[4 * q8 + 1]), "r"(v[4 * q8 + 2]),
                       "r"(v[4 * q8 + 3])
                       : "memory");
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar_acc_empty(as));
      fence_proxy_async_smem();
      named_bar_sync(MM_EPI_BAR, 128);
      if (epi_tid == 0) {
#pragma unroll
        for (int bx = 0; bx < S::NBOX; bx++) tma_store_3d(&map_out, stage + bx * S::OUT_BOX, 32 * bx, t0, b);
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
