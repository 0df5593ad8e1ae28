// band_n / band_t on tensor cores.  Included by wmm_tc.cu (inside namespace wmm::<anon>).
//
//   band_n:  Out[i, :] = sum_p Band[i, p] Y[p, :]      tile = 128 band rows i
//   band_t:  Out[p, :] = sum_i Band[i, p] X[i, :]      tile = 128 positions p
//
// Both read (128 rows x 128 x-columns) boxes of the band through the pitched view and multiply them with
// 128-row slices of the other operand (hidden size contiguous, i.e. MN-major for the MMA).  band_n uses
// the box as a K-major A operand (rows = M, x = K); band_t uses the same bytes as an MN-major A operand
// (x = M, rows = K).  Box elements that are not band entries of their row (they alias neighbouring rows)
// or whose position is outside the sequence are zeroed in shared memory by the mask warps before the MMA
// reads them; only the first and last chunk of a tile, and tiles at the sequence ends, need that, and only
// for those chunks does the MMA thread wait for the mask warps.
//
// MODE 0 = band_n, 1 = band_t, 2 = both over the SAME band in one launch (the backward of window_matmul:
// grad_Q = band_n(grad_A, K^T), grad_K^T = band_t(grad_A, Q)).  In mode 2 the work items alternate
// (tile 0 band_n, tile 0 band_t, tile 1 band_n, ...), so the two passes over a region of the band run at
// the same time on neighbouring CTAs and the second one finds the boxes in L2: the band is fetched from
// HBM once.
//
// Warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2-5 = mask, 6-9 = epilogue.

constexpr int MM_THREADS = 320;
constexpr uint32_t MM_EPI_BAR = 5;
constexpr unsigned long long ST_MM_TIMEOUT = 1ull << 1;

struct MmParams {
  int B, M, Mo, w, off, lo, hi;
  int tiles_per_batch, total_tiles, nchunks;
  // band_t (MODE 1) only: unrounded fp32 copy of output rows [edge_skip, edge_rows) and [Mo - edge_rows, Mo - edge_skip)
  // of every batch entry, at the same row index of a (B, 2 * edge_rows, NH) contiguous buffer (row Mo - edge_rows is its
  // row edge_rows), for a sequence shard whose edge rows are summed with a neighbour's
  float *edges;
  int edge_rows, edge_skip;
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

// YMN: the other operand of the band_n pass is stored with the POSITIONS contiguous (K given as a contiguous
// (B, N, M) tensor): its 128-position slice is then two TMA boxes of (64 positions x NH rows), a K-major B operand.
template <bool BF16, int NH, int MODE, bool YMN>
__global__ void __launch_bounds__(MM_THREADS, 1)
band_mm_tc_kernel(const __grid_constant__ CUtensorMap map_band, const __grid_constant__ CUtensorMap map_other0,
                  const __grid_constant__ CUtensorMap map_out0, const __grid_constant__ CUtensorMap map_other1,
                  const __grid_constant__ CUtensorMap map_out1, const MmParams p) {
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
    prefetch_tmap(&map_other0);
    prefetch_tmap(&map_out0);
    if (MODE == 2) {
      prefetch_tmap(&map_other1);
      prefetch_tmap(&map_out1);
    }
  }
  if (warp == 1) {
    tmem_alloc(base + S::OFF_MISC, S::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, tensor memory, tensor-map prefetch) may run under the tail of the previous kernel of the
  // stream; from here on global memory is read and written.
  griddep_launch_dependents();
  griddep_wait();

  // Work items, identical in every role: item -> (tile, transposed?).
  const int total_items = MODE == 2 ? 2 * p.total_tiles : p.total_tiles;
  auto item_tile = [&](int wi) -> int { return MODE == 2 ? (wi >> 1) : wi; };
  auto item_tr = [&](int wi) -> bool { return MODE == 2 ? ((wi & 1) != 0) : (MODE == 1); };

  // Tile / chunk geometry.  t0 = first row (band_n) or position (band_t) of the tile.  Chunk c covers,
  // along the reduction, 128 positions (band_n) or 128 band rows (band_t):
  //   band_n: box rows i = t0 .. t0+127, x = t0 + 128c + kk,         position of column kk: t0 - w + off + 128c + kk
  //   band_t: box rows i = t0 - off - w + 128c + ii, x = t0 - off + w + xx,   position of column xx: t0 + xx
  auto chunk_is_plain = [&](bool tr, int t0, int c) -> bool {
    // true when no element of the box needs zeroing
    if (c < 1 || c * 128 + 127 > 2 * p.w) return false;
    if (!tr) {
      const int p0 = t0 - p.w + p.off + c * 128;
      return p0 >= p.lo && p0 + 128 <= p.hi;
    }
    return t0 >= p.lo && t0 + 128 <= p.hi;
  };

  // The MMA thread waits for the mask warps only at SYNC POINTS: every chunk that needs zeroing, and any
  // chunk that would otherwise be the STAGES-th in a row without one.  Both sides evaluate this rule on the
  // same chunk sequence.  Between two sync points fewer than STAGES chunks pass, so the producer can never
  // refill a stage twice while a mask thread is still waiting for its earlier phase.
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
      for (int wi = blockIdx.x; ok && wi < total_items; wi += gridDim.x) {
        const int tile = item_tile(wi);
        const bool tr = item_tr(wi);
        const CUtensorMap *map_other = (MODE == 2 && tr) ? &map_other1 : &map_other0;
        const int b = tile / p.tiles_per_batch, t0 = (tile % p.tiles_per_batch) * TILE;
        for (int c = 0; c < p.nchunks; ++c, ++it) {
          const int s = it % S::STAGES;
          if (!(ok = mbar_wait(bar_empty(s), ((it / S::STAGES) & 1) ^ 1, abort_flag))) break;
          mbar_expect_tx(bar_full(s), S::STAGE_BYTES);
          const uint32_t band_dst = base + s * S::STAGE_BYTES, other_dst = band_dst + BT::BYTES;
          const int x0 = tr ? t0 - p.off + p.w : t0 + c * 128;
          const int row0 = tr ? t0 - p.off - p.w + c * 128 : t0;
          const int orow0 = tr ? row0 : t0 - p.w + p.off + c * 128;
          tma_load_3d(band_dst, &map_band, bar_full(s), x0, row0, b);
          tma_load_3d(band_dst + BT::BOX_BYTES, &map_band, bar_full(s), x0 + 64, row0, b);
          if (YMN && !tr) {
#pragma unroll
            for (int hf = 0; hf < 2; hf++)  // map dims: (position, hidden, batch)
              tma_load_3d(other_dst + hf * (OT::BYTES / 2), map_other, bar_full(s), orow0 + hf * 64, 0, b);
          } else {
#pragma unroll
            for (int bx = 0; bx < OT::NBOX; bx++)
              tma_load_3d(other_dst + bx * OT::BOX_BYTES, map_other, bar_full(s), bx * OT::BOXK, orow0, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t IDESC_N = instr_desc_f16(BF16, false, true, TILE, NH);
      constexpr uint32_t IDESC_T = instr_desc_f16(BF16, true, true, TILE, NH);
      // A operand.  K-major (band_n): 8-row groups 1024 B apart, a k-step of 16 columns is 32 B further
      // along the 128-byte row (64 columns per box).  MN-major (band_t): 64 contiguous x per 128-byte row,
      // second 64 x in the next box (leading offset), 8-row k-groups 1024 B apart (stride offset), a k-step
      // of 16 rows is 2048 B further.
      constexpr uint64_t ADESC_N = BT::DESC;
      constexpr uint64_t ADESC_T = smem_desc_base(BT::BOX_BYTES, 1024, 2u);
      // B operand, MN-major: OT::BOXK contiguous hidden columns per row, next box one leading offset away.
      constexpr uint64_t BDESC = smem_desc_base(OT::BOX_BYTES, 8 * OT::SW_BYTES, OT::SWZ_CODE);
      // position-major Y (band_n pass only): K-major B, NH rows of 64 positions (128 B) per box, 8-row groups
      // 1024 B apart, a k-step of 16 positions is 32 B further along the row, second 64 positions = second box
      constexpr uint32_t IDESC_N_K = instr_desc_f16(BF16, false, false, TILE, NH);
      constexpr uint64_t BDESC_K = smem_desc_base(16, 1024, 2u);
      int it = 0, tit = 0, since = 0, mk[S::STAGES];
      for (int s = 0; s < S::STAGES; s++) mk[s] = 0;
      bool ok = true;
      for (int wi = blockIdx.x; ok && wi < total_items; wi += gridDim.x, ++tit) {
        const bool tr = item_tr(wi);
        const int t0 = (item_tile(wi) % p.tiles_per_batch) * TILE;
        const bool ymn = YMN && !tr;
        const uint32_t idesc = tr ? IDESC_T : (ymn ? IDESC_N_K : IDESC_N);
        const uint64_t bdesc = ymn ? BDESC_K : BDESC;
        const uint64_t adesc = tr ? ADESC_T : ADESC_N;
        const int as = tit & 1;
        if (!(ok = mbar_wait(bar_acc_empty(as), ((tit >> 1) & 1) ^ 1, abort_flag))) break;
        for (int c = 0; c < p.nchunks; ++c, ++it) {
          const int s = it % S::STAGES;
          // full: the TMA bytes have landed.  masked: the mask warps are done with this stage; waited for
          // only at sync points (see mask_sync below), i.e. for the chunks they had to touch.
          if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
          if (mask_sync(chunk_is_plain(tr, t0, c), since)) {
            if (!(ok = mbar_wait(bar_masked(s), mk[s] & 1, abort_flag))) break;
            ++mk[s];
          }
          tc_fence_after_sync();
          const uint32_t a_addr = base + s * S::STAGE_BYTES, b_addr = a_addr + BT::BYTES;
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const uint32_t a_off = tr ? (uint32_t)k * 2048u : BT::kstep_offset(k);
            const uint32_t b_off = ymn ? (uint32_t)(k >> 2) * (OT::BYTES / 2) + (uint32_t)(k & 3) * 32u : (uint32_t)k * 16u * OT::SW_BYTES;
            umma_f16(tmem_base + as * NH, smem_desc(adesc, a_addr + a_off), smem_desc(bdesc, b_addr + b_off), idesc,
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
    int it = 0, since = 0;
    bool ok = true;
    for (int wi = blockIdx.x; ok && wi < total_items; wi += gridDim.x) {
      const int tile = item_tile(wi);
      const bool tr = item_tr(wi);
      const int t0 = (tile % p.tiles_per_batch) * TILE;
      for (int c = 0; c < p.nchunks; ++c, ++it) {
        const int s = it % S::STAGES;
        // every phase of every stage is observed (a parity wait cannot tell phases two apart)
        if (!(ok = mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag))) break;
        const bool plain = chunk_is_plain(tr, t0, c);
        const bool sync = mask_sync(plain, since);
        if (plain) {
          if (sync) mbar_arrive(bar_masked(s));
          continue;
        }
        // columns [col_lo, col_hi] of this row are band entries inside the sequence; the rest is zeroed
        int col_lo, col_hi;
        if (!tr) {
          const int p0 = t0 - p.w + p.off + c * 128;
          col_lo = max(row - c * 128, p.lo - p0);
          col_hi = min(row - c * 128 + 2 * p.w, p.hi - p0 - 1);
        } else {
          col_lo = max(row + c * 128 - 2 * p.w, p.lo - t0);
          col_hi = min(row + c * 128, p.hi - t0 - 1);
        }
        const uint32_t tile_addr = base + s * S::STAGE_BYTES;
        // 16-byte piece g (8 columns) of this row: box g / 8, swizzled column (g % 8) ^ (row % 8)
        auto piece = [&](int g) -> uint32_t {
          return tile_addr + (g >> 3) * BT::BOX_BYTES + row * 128 + (((g & 7) ^ (row & 7)) << 4);
        };
        auto zero_piece = [&](int g) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(piece(g)), "r"(0u) : "memory");
        };
        // keep columns [col_lo, col_hi] of piece g, zero its other columns
        auto trim_piece = [&](int g) {
          const uint32_t a = piece(g);
          const int c0 = g * 8;
          uint32_t v[4];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(a) : "memory");
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const int ca = c0 + 2 * k, cb = ca + 1;
            v[k] &= ((ca >= col_lo && ca <= col_hi) ? 0x0000ffffu : 0u) | ((cb >= col_lo && cb <= col_hi) ? 0xffff0000u : 0u);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
        };
        if (col_lo > col_hi || col_hi < 0 || col_lo > 127) {
#pragma unroll 4
          for (int g = 0; g < 16; g++) zero_piece(g);
        } else {
          const int lo = max(col_lo, 0), hi = min(col_hi, 127);
          const int g_lo = lo >> 3, g_hi = hi >> 3;  // first / last piece with a column to keep
          for (int g = 0; g < g_lo; g++) zero_piece(g);
          for (int g = g_hi + 1; g < 16; g++) zero_piece(g);
          if ((lo & 7) != 0 || (g_lo == g_hi && (hi & 7) != 7)) trim_piece(g_lo);
          if (g_hi != g_lo && (hi & 7) != 7) trim_piece(g_hi);
        }
        if (!tr && !YMN) {  // (a position-major operand is only taken when the whole row range is in sequence)
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
    for (int wi = blockIdx.x; ok && wi < total_items; wi += gridDim.x, ++tit) {
      const int tile = item_tile(wi);
      const CUtensorMap *map_out = (MODE == 2 && item_tr(wi)) ? &map_out1 : &map_out0;
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
        if (MODE == 1 && p.edges != nullptr) {
          const int e = t0 + rr;   // output row of this thread
          const int er = e < p.edge_rows ? e : (e >= p.Mo - p.edge_rows && e < p.Mo ? e - (p.Mo - 2 * p.edge_rows) : -1);
          if (er >= p.edge_skip && er < 2 * p.edge_rows - p.edge_skip) {
            uint4 *dst = reinterpret_cast<uint4 *>(p.edges + ((size_t)b * 2 * p.edge_rows + er) * NH + g * 32);
#pragma unroll
            for (int q = 0; q < 8; q++) dst[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        }
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
        for (int bx = 0; bx < OT::NBOX; bx++) tma_store_3d(map_out, stage + bx * OT::BOX_BYTES, bx * OT::BOXK, t0, b);
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
