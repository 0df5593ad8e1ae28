// The backward of window_matmul in ONE sweep over the band: grad_Q = band_n(grad_A, K^T) and grad_K^T = band_t(grad_A, Q)
// with every (128 rows x 128 x-columns) box of grad_A brought into shared memory ONCE and used by both products.
// Included by wmm_tc.cu (inside namespace wmm::<anon>).
//
// Geometry (plain sequences only; w a multiple of 128, D = w / 128).  Row tile r = band rows 128r .. 128r+127.  In the
// pitched view (row i, x = i + j) its band entries lie in x-chunks c = r .. r + 2D; x-chunk c holds the positions of
// position tile pt = c - D.  So the boxes form a banded grid (r, pt), |r - pt| <= D, and
//     grad_Q  tile r   = sum over pt of  Box(r, pt)    . K^T[pt]     (a row of the grid:    accumulates over pt)
//     grad_K^T tile pt = sum over r  of  Box(r, pt)^T  . Q[r]       (a column of the grid: accumulates over r)
// A CTA owns a run of consecutive row tiles and walks them in order.  For each box it issues both MMAs: the box as a
// K-major A operand into the row accumulator, and the same bytes as an MN-major A operand into the accumulator of
// column pt.  2D+1 column accumulators are live at a time (plus one being drained), so tensor memory holds
// (2D + 2) column slots and 2 row slots of NH columns: (2D + 4) NH <= 512.  A column is complete after row pt + D;
// the CTA that owns that row writes it.  Rows before a CTA's run that feed its first columns are replayed (band_t
// product only): D (2D + 1) extra boxes per run that starts inside a sequence.
//
// Per box the SM takes in 32 KB of band + 16 KB of K^T rows (+ 16 KB of Q rows per row tile), against two full
// passes (2 x 48 KB per box) of the two-pass kernel.
//
// Warps: 0 = TMA producer, 1 = MMA issuer of the row products / TMEM owner, 2-5 = mask, 6-9 = epilogue, 10 = MMA issuer of
// the column products.  Waits are bounded as everywhere.

constexpr int SWP_THREADS = 352;
constexpr uint32_t SWP_EPI_BAR = 6;
constexpr unsigned long long ST_SWEEP_TIMEOUT = 1ull << 4;

struct SweepParams {
  int B, M, w, D, T;   // T = row tiles (= position tiles) per sequence
  int total_rows;      // B * T
  // outputs (element strides; unit column stride): written straight from registers, a 2 NH-byte row per thread
  uint16_t *gq, *gk;
  int64_t gq_sb, gq_sr, gk_sb, gk_sr;
};

template <int NH> struct SweepSmem {
  using BT = KMajorTile<128>;
  using OT = KMajorTile<NH>;
  static constexpr int STAGES = 4;
  static constexpr int MAX_SLOTS = 6;   // column accumulators (2D + 2 <= 6)
  static constexpr int STAGE_BYTES = BT::BYTES + OT::BYTES;
  static constexpr int OFF_X = STAGES * STAGE_BYTES;   // two Q tiles
  static constexpr int OFF_BARS = OFF_X + 2 * OT::BYTES;
  static constexpr int NBARS = 3 * STAGES + 8 + 2 * MAX_SLOTS;
  static constexpr int OFF_MISC = OFF_BARS + NBARS * 8;
  static constexpr int BYTES = OFF_MISC + 32;
  static constexpr int ALLOC = BYTES + 1024;
};

// The walk every role performs, in the same order.  Callbacks return false to stop (an abandoned wait).
//   row_begin(b, r, warm)                       a row tile starts (warm: replayed row, band_t product only)
//   box(b, r, pt, warm, t_pass, first_in_row)   one box; t_pass: this CTA owns column pt
//   flush_col(b, pt), flush_row(b, r)           an accumulator is complete (in this order after a main row)
//   row_end(warm)
template <typename RowBegin, typename Box, typename FlushCol, typename FlushRow, typename RowEnd>
__device__ __forceinline__ bool sweep_walk(const SweepParams &p, RowBegin row_begin, Box box, FlushCol flush_col, FlushRow flush_row,
                                           RowEnd row_end) {
  const int per = p.total_rows / (int)gridDim.x, rem = p.total_rows % (int)gridDim.x;
  int g = (int)blockIdx.x * per + min((int)blockIdx.x, rem);
  const int g_end = g + per + ((int)blockIdx.x < rem ? 1 : 0);
  while (g < g_end) {
    const int b = g / p.T, ra = g % p.T;
    const int rb = min(p.T, ra + (g_end - g));
    const int own_lo = ra - p.D, own_hi = rb == p.T ? p.T : rb - p.D;   // columns [own_lo, own_hi) are this run's
    for (int r = max(ra - 2 * p.D, 0); r < rb; ++r) {
      const bool warm = r < ra;
      int pt_lo = max(r - p.D, 0), pt_hi = min(r + p.D, p.T - 1);
      if (warm) {
        pt_lo = max(pt_lo, own_lo);
        pt_hi = min(pt_hi, own_hi - 1);
        if (pt_lo > pt_hi) continue;
      }
      if (!row_begin(b, r, warm)) return false;
      for (int pt = pt_lo; pt <= pt_hi; ++pt)
        if (!box(b, r, pt, warm, pt >= own_lo && pt < own_hi, pt == pt_lo)) return false;
      if (!row_end(warm)) return false;
      if (!warm) {
        if (r - p.D >= 0 && !flush_col(b, r - p.D)) return false;
        if (!flush_row(b, r)) return false;
        if (r == p.T - 1)
          for (int pt = max(p.T - p.D, 0); pt < p.T; ++pt)
            if (!flush_col(b, pt)) return false;
      }
    }
    g += rb - ra;
  }
  return true;
}

template <bool BF16, int NH>
__global__ void __launch_bounds__(SWP_THREADS, 1)
band_bwd_sweep_kernel(const __grid_constant__ CUtensorMap map_band, const __grid_constant__ CUtensorMap map_y,
                      const __grid_constant__ CUtensorMap map_x, const SweepParams p) {
  using S = SweepSmem<NH>;
  using BT = typename S::BT;
  using OT = typename S::OT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + S::OFF_BARS;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (S::STAGES + s); };
  auto bar_masked = [&](int s) { return bars + 8u * (2 * S::STAGES + s); };
  auto bar_xfull = [&](int s) { return bars + 8u * (3 * S::STAGES + s); };
  auto bar_xempty = [&](int s) { return bars + 8u * (3 * S::STAGES + 2 + s); };
  auto bar_nfull = [&](int s) { return bars + 8u * (3 * S::STAGES + 4 + s); };
  auto bar_nempty = [&](int s) { return bars + 8u * (3 * S::STAGES + 6 + s); };
  auto bar_tfull = [&](int s) { return bars + 8u * (3 * S::STAGES + 8 + s); };
  auto bar_tempty = [&](int s) { return bars + 8u * (3 * S::STAGES + 8 + S::MAX_SLOTS + s); };
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + S::OFF_MISC);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 4);
  volatile int *epi_ok = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslots = 2 * p.D + 2;
  if (threadIdx.x == 0) WMM_TRACE_POINT(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; s++) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 2);   // both MMA issuers
      mbar_init(bar_masked(s), 128);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_xfull(s), 1);
      mbar_init(bar_xempty(s), 1);
      mbar_init(bar_nfull(s), 1);
      mbar_init(bar_nempty(s), 128);
    }
    for (int s = 0; s < S::MAX_SLOTS; s++) {
      mbar_init(bar_tfull(s), 1);
      mbar_init(bar_tempty(s), 128);
    }
    *abort_flag = 0;
    *epi_ok = 1;
    fence_mbar_init();
    prefetch_tmap(&map_band);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(base + S::OFF_MISC, 512);
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
  // tensor memory columns: row accumulators at 0 and NH, column slot s at (2 + s) NH
  auto tmem_row = [&](int as) { return tmem_base + (uint32_t)(as * NH); };
  auto tmem_col = [&](int slot) { return tmem_base + (uint32_t)((2 + slot) * NH); };

  // chunk index of box (r, pt) inside the row's window, and whether the box needs no zeroing
  auto box_plain = [&](int r, int pt) -> bool {
    const int cc = pt + p.D - r;
    return cc >= 1 && cc * 128 + 127 <= 2 * p.w && pt * 128 + 128 <= p.M;
  };
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
      int it = 0, xrow = 0;
      sweep_walk(
          p,
          [&](int b, int r, bool) {
            const int xb = xrow & 1;
            if (!mbar_wait(bar_xempty(xb), ((xrow >> 1) & 1) ^ 1, abort_flag)) return false;
            mbar_expect_tx(bar_xfull(xb), OT::BYTES);
#pragma unroll
            for (int bx = 0; bx < OT::NBOX; bx++)
              tma_load_3d(base + S::OFF_X + xb * OT::BYTES + bx * OT::BOX_BYTES, &map_x, bar_xfull(xb), bx * OT::BOXK, r * TILE, b);
            ++xrow;
            return true;
          },
          [&](int b, int r, int pt, bool warm, bool, bool) {
            const int s = it % S::STAGES;
            if (!mbar_wait(bar_empty(s), ((it / S::STAGES) & 1) ^ 1, abort_flag)) return false;
            mbar_expect_tx(bar_full(s), warm ? BT::BYTES : S::STAGE_BYTES);
            const uint32_t band_dst = base + s * S::STAGE_BYTES, other_dst = band_dst + BT::BYTES;
            const int x0 = (pt + p.D) * 128;
            tma_load_3d(band_dst, &map_band, bar_full(s), x0, r * TILE, b);
            tma_load_3d(band_dst + BT::BOX_BYTES, &map_band, bar_full(s), x0 + 64, r * TILE, b);
            if (!warm) {
#pragma unroll
              for (int bx = 0; bx < OT::NBOX; bx++)
                tma_load_3d(other_dst + bx * OT::BOX_BYTES, &map_y, bar_full(s), bx * OT::BOXK, pt * 128, b);
            }
            ++it;
            return true;
          },
          [&](int, int) { return true; }, [&](int, int) { return true; }, [&](bool) { return true; });
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------- MMA issuers ----------------
    // Two threads issue the MMAs, each walking all boxes: warp 1 the row products (grad_Q = box . K^T rows, into the
    // row accumulators), warp 10 the column products (grad_K^T = box^T . Q rows, into the column slots).  Issuing an
    // MMA costs its thread about as much as the tensor core needs to execute it, and a box feeds sixteen of them: one
    // thread alone was busy three quarters of the kernel's time.  A stage is released when both have committed.
    if (lane == 0) {
      const bool rows = warp == 1;
      constexpr uint32_t IDESC_N = instr_desc_f16(BF16, false, true, TILE, NH);
      constexpr uint32_t IDESC_T = instr_desc_f16(BF16, true, true, TILE, NH);
      constexpr uint64_t ADESC_N = BT::DESC;
      constexpr uint64_t ADESC_T = smem_desc_base(BT::BOX_BYTES, 1024, 2u);
      constexpr uint64_t BDESC = smem_desc_base(OT::BOX_BYTES, 8 * OT::SW_BYTES, OT::SWZ_CODE);
      int it = 0, xrow = 0, nrow = 0, since = 0;
      uint32_t mk_bits = 0, col_bits = 0;   // parity of: masked-barrier uses per stage; column-slot uses
      int as = 0, xb = 0;
      unsigned long long w_wait = 0, w_issue = 0;   // (trace builds) time in waits / issuing MMAs and commits
      (void)w_wait; (void)w_issue;
      WMM_TRACE_POINT(rows ? 1 : 5);
      sweep_walk(
          p,
          [&](int, int, bool warm) {
            if (rows) {
              if (!warm) {
                as = nrow & 1;
                if (!mbar_wait(bar_nempty(as), ((nrow >> 1) & 1) ^ 1, abort_flag)) return false;
                ++nrow;
              }
            } else {
              xb = xrow & 1;
              if (!mbar_wait(bar_xfull(xb), (xrow >> 1) & 1, abort_flag)) return false;
              ++xrow;
            }
            return true;
          },
          [&](int, int r, int pt, bool warm, bool t_pass, bool first_in_row) {
            const int s = it % S::STAGES;
            WMM_TRACE_T0(t_w);
            if (!mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag)) return false;
            if (mask_sync(box_plain(r, pt), since)) {
              if (!mbar_wait(bar_masked(s), (mk_bits >> s) & 1u, abort_flag)) return false;
              mk_bits ^= 1u << s;
            }
            ++it;
            const int slot = pt % nslots;
            const bool col_first = t_pass && r == max(pt - p.D, 0);
            if (!rows && col_first) {  // a new column starts in this slot: the previous one must have been drained
              if (!mbar_wait(bar_tempty(slot), ((col_bits >> slot) & 1u) ^ 1u, abort_flag)) return false;
              col_bits ^= 1u << slot;
            }
            WMM_TRACE_ACC(w_wait, t_w);
            WMM_TRACE_T0(t_i);
            tc_fence_after_sync();
            const uint32_t a_addr = base + s * S::STAGE_BYTES, y_addr = a_addr + BT::BYTES;
            const uint32_t x_addr = base + S::OFF_X + xb * OT::BYTES;
            if (rows && !warm) {
#pragma unroll
              for (int k = 0; k < 8; k++)
                umma_f16(tmem_row(as), smem_desc(ADESC_N, a_addr + BT::kstep_offset(k)),
                         smem_desc(BDESC, y_addr + (uint32_t)k * 16u * OT::SW_BYTES), IDESC_N, (!first_in_row || k > 0) ? 1u : 0u);
            }
            if (!rows && t_pass) {
#pragma unroll
              for (int k = 0; k < 8; k++)
                umma_f16(tmem_col(slot), smem_desc(ADESC_T, a_addr + (uint32_t)k * 2048u),
                         smem_desc(BDESC, x_addr + (uint32_t)k * 16u * OT::SW_BYTES), IDESC_T, (!col_first || k > 0) ? 1u : 0u);
            }
            umma_commit(bar_empty(s));   // (arrives at once when this thread issued nothing from the stage)
            WMM_TRACE_ACC(w_issue, t_i);
            return true;
          },
          [&](int, int pt) {
            if (!rows) umma_commit(bar_tfull(pt % nslots));
            return true;
          },
          [&](int, int) {
            if (rows) umma_commit(bar_nfull(as));
            return true;
          },
          [&](bool) {
            if (!rows) umma_commit(bar_xempty(xb));
            return true;
          });
      WMM_TRACE_POINT(rows ? 2 : 6);
      WMM_TRACE_STORE(rows ? 3 : 7, w_wait);
      WMM_TRACE_STORE(rows ? 4 : 8, w_issue);
    }
  } else if (warp < 6) {
    // ---------------- mask warps: thread <-> row of the band box ----------------
    const int row = (warp - 2) * 32 + lane;
    int it = 0, since = 0;
    sweep_walk(
        p, [&](int, int, bool) { return true; },
        [&](int, int r, int pt, bool, bool, bool) {
          const int s = it % S::STAGES;
          if (!mbar_wait(bar_full(s), (it / S::STAGES) & 1, abort_flag)) return false;
          ++it;
          const bool plain = box_plain(r, pt);
          const bool sync = mask_sync(plain, since);
          if (plain) {
            if (sync) mbar_arrive(bar_masked(s));
            return true;
          }
          // columns [col_lo, col_hi] of this row are band entries inside the sequence; the rest is zeroed
          const int cc = pt + p.D - r;
          const int col_lo = max(row - cc * 128, 0);
          const int col_hi = min(row - cc * 128 + 2 * p.w, p.M - pt * 128 - 1);
          const uint32_t tile_addr = base + s * S::STAGE_BYTES;
          auto piece = [&](int g) -> uint32_t {
            return tile_addr + (g >> 3) * BT::BOX_BYTES + row * 128 + (((g & 7) ^ (row & 7)) << 4);
          };
          auto zero_piece = [&](int g) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(piece(g)), "r"(0u) : "memory");
          };
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
            const int g_lo = lo >> 3, g_hi = hi >> 3;
            for (int g = 0; g < g_lo; g++) zero_piece(g);
            for (int g = g_hi + 1; g < 16; g++) zero_piece(g);
            if ((lo & 7) != 0 || (g_lo == g_hi && (hi & 7) != 7)) trim_piece(g_lo);
            if (g_hi != g_lo && (hi & 7) != 7) trim_piece(g_hi);
          }
          fence_proxy_async_smem();
          mbar_arrive(bar_masked(s));
          return true;
        },
        [&](int, int) { return true; }, [&](int, int) { return true; }, [&](bool) { return true; });
  } else {
    // ---------------- epilogue: thread <-> output row of the tile ----------------
    // Each thread owns one output row of 2 NH bytes (a whole 128-byte line at NH = 64) and writes it from registers:
    // no staging buffer, which is what leaves room for the fourth pipeline stage.
    const int quarter = warp & 3;
    const int rr = quarter * 32 + lane;
    const int epi_tid = threadIdx.x - 192;
    int nrow = 0;
    uint32_t col_bits = 0;
    auto drain = [&](uint32_t full_bar, uint32_t parity, uint32_t empty_bar, uint32_t tcol, uint16_t *out, int64_t sr, int t0) -> bool {
      if (epi_tid == 0) *epi_ok = mbar_wait(full_bar, parity, abort_flag) ? 1 : 0;
      named_bar_sync(SWP_EPI_BAR, 128);
      const bool good = *epi_ok != 0;
      named_bar_sync(SWP_EPI_BAR, 128);   // everyone has read the verdict before the next drain overwrites it
      if (!good) return false;
      tc_fence_after_sync();
      const uint32_t taddr = tcol + ((uint32_t)(quarter * 32) << 16);
      uint16_t *dst = out + (int64_t)(t0 + rr) * sr;
      const bool in_range = t0 + rr < p.M;
#pragma unroll
      for (int g = 0; g < NH / 32; g++) {
        uint32_t v[32];
        tmem_ld_x32(taddr + g * 32, v);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++)
            *reinterpret_cast<uint4 *>(dst + g * 32 + q4 * 8) =
                make_uint4(pack2<BF16>(v[q4 * 8 + 0], v[q4 * 8 + 1]), pack2<BF16>(v[q4 * 8 + 2], v[q4 * 8 + 3]),
                           pack2<BF16>(v[q4 * 8 + 4], v[q4 * 8 + 5]), pack2<BF16>(v[q4 * 8 + 6], v[q4 * 8 + 7]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive(empty_bar);
      return true;
    };
    sweep_walk(
        p, [&](int, int, bool) { return true; }, [&](int, int, int, bool, bool, bool) { return true; },
        [&](int b, int pt) {
          const int slot = pt % nslots;
          const uint32_t parity = (col_bits >> slot) & 1u;
          col_bits ^= 1u << slot;
          return drain(bar_tfull(slot), parity, bar_tempty(slot), tmem_col(slot), p.gk + b * p.gk_sb, p.gk_sr, pt * 128);
        },
        [&](int b, int r) {
          const int as = nrow & 1;
          const uint32_t parity = (nrow >> 1) & 1;
          ++nrow;
          return drain(bar_nfull(as), parity, bar_nempty(as), tmem_row(as), p.gq + b * p.gq_sb, p.gq_sr, r * TILE);
        },
        [&](bool) { return true; });
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_device_status, ST_SWEEP_TIMEOUT);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}
