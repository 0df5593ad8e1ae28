// band_nt on tensor cores: Band = band(X Y^T).  Included by wmm_tc.cu (inside namespace wmm::<anon>).
//
// One MMA chunk = X tile (128 rows x NH) times 128 rows of Y -> a 128 x 128 fp32 accumulator in TMEM, issued as
// NH / 16 instructions of shape 128 x 128 x 16 (the issuing thread is the scarcest resource of this kernel: an
// instruction costs it about as much whatever its width, so chunks are not split into narrower MMAs).
// A tile of 128 band rows needs ceil((128 + 2w) / 128) chunks.  The epilogue turns accumulators into
// band storage:
//   * a chunk that lies wholly inside the band is converted, written to a swizzled staging buffer and
//     stored with two TMA box stores through the pitched view of the band (see wmm_tc.cu);
//   * the first and last chunk of a tile are triangular.  When 2w is a multiple of 128 the two triangles
//     are complementary: in the pitched view (pitch 2w) the last chunk of row i occupies the same line
//     as the first chunk of row i+1, so first-chunk row r goes to staging line r (columns >= r), last-
//     chunk row r to line r+1 (columns <= r), and the merged 128 x 128 box is stored by TMA like a full
//     chunk.  Only the last valid row's last-chunk piece (one row, <= 256 bytes) is written directly.
//   * for other windows the triangular chunks are written with predicated 16-byte stores from registers.
//
// Warps: 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2-17 = four epilogue groups of four warps that
// take work items (half a chunk = one 128 x 64 TMA box) round-robin, each with its own staging boxes: the
// conversion is latency-bound per warp, so it needs many warps.  Warp 18 = store issuer: it alone issues the TMA
// stores of all groups, in item order, and hands a staging box back once its store has read it.  (Issuing a
// tensor store holds the issuing thread for a few hundred nanoseconds; done by the groups' own threads that time
// sat on every item's critical path.)

constexpr int HALF = 64;        // positions per accumulator stage / per epilogue work item
constexpr int EPI_GROUPS = 4;
constexpr int EPI_THREADS = 128;
constexpr int NT_THREADS = 64 + EPI_GROUPS * EPI_THREADS + 32;
constexpr unsigned long long ST_NT_TIMEOUT = 1ull << 0;

struct NtParams {
  int B, M, w, off, lo, hi;
  int tiles_per_batch, total_tiles, nchunks;
  int paired;  // 2w is a multiple of 128: merge first and last chunk of a tile
  void *band;
  int64_t band_sb;   // elements between batch entries of the band (rows written without TMA)
};

template <int NH, int ES> struct NtSmem {
  using OT = KMajorTileE<NH, ES>;
  static constexpr bool BIG = OT::BYTES >= 32768;   // a 32 KB operand tile: N = 128 in 16 bits, N = 64 in fp32
  static constexpr int QS = 2;
  static constexpr int KS = BIG ? 3 : 4;
  static constexpr int STAGE_HALF = TILE * 128;  // one staging box: 128 lines of 128 bytes (64 16-bit or 32 fp32 positions)
  // Staging boxes: a pool shared by the four epilogue groups, used in item order (item n of the CTA goes through box
  // n % STAGE_BOXES).  With more boxes than groups a group converts its next item while the stores of earlier ones
  // still wait their turn in the SM's store queue.
  static constexpr int STAGE_BOXES = BIG ? 4 : 8;
  static constexpr int STORE_DEPTH = STAGE_BOXES / 2;   // stores whose shared-memory read may be pending when the next is issued
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + QS * OT::BYTES;
  static constexpr int OFF_STAGE = OFF_K + KS * OT::BYTES;  // STAGE_BOXES boxes of 16 KB
  static constexpr int OFF_BARS = OFF_STAGE + STAGE_BOXES * STAGE_HALF;
  static constexpr int NBARS = 2 * QS + 2 * KS + 2 * ACC_STAGES + STAGE_BOXES;
  static constexpr int OFF_MISC = OFF_BARS + NBARS * 8;
  static constexpr int BYTES = OFF_MISC + 64;
  static constexpr int ALLOC = BYTES + 1024;  // slack to align the base to 1024 B
};

// 8 packed 16-bit values (one 16-byte piece) from 8 fp32 accumulator bit patterns
template <bool BF16> __device__ __forceinline__ uint4 pack8(const uint32_t *v) {
  uint4 o;
  o.x = pack2<BF16>(v[0], v[1]);
  o.y = pack2<BF16>(v[2], v[3]);
  o.z = pack2<BF16>(v[4], v[5]);
  o.w = pack2<BF16>(v[6], v[7]);
  return o;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4 &o) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
}
__device__ __forceinline__ void st_shared_u16(uint32_t addr, uint16_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
// address of the 16-byte piece (line, column group cg = column / 8 in 0..7) of a 128-line x 64-column staging box
__device__ __forceinline__ uint32_t stage_addr(uint32_t stage, int line, int cg) {
  return stage + line * 128 + ((cg ^ (line & 7)) << 4);
}
// zero the accumulator values of 32 columns starting at column kbase whose position is outside [kk_lo, kk_hi)
__device__ __forceinline__ void mask_columns(uint32_t (&v)[32], int kbase, int kk_lo, int kk_hi) {
#pragma unroll
  for (int e = 0; e < 32; e++)
    if (kbase + e < kk_lo || kbase + e >= kk_hi) v[e] = 0u;
}

// YMN: Y is stored with the POSITIONS contiguous (K of window_matmul given as a contiguous (B, N, M) tensor, as
// in the reference's README).  A chunk is then two TMA boxes of (64 positions x NH rows), used as an
// MN-major B operand; otherwise Y rows are contiguous in the hidden index and the operand is K-major.
// PAIRED: 2w is a multiple of 128, so the first and the last chunk of a tile are merged (a compile-time switch: each
// variant carries only the epilogue paths it can reach, which keeps the loop body small).
// ET: 0 = fp16, 1 = bf16, 2 = fp32 operands multiplied as tf32 (fp32 band; K-major operands and unpaired epilogue only).
template <int ET, int NH, bool YMN, bool PAIRED>
__global__ void __launch_bounds__(NT_THREADS, 1)
band_nt_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                  const __grid_constant__ CUtensorMap map_band, const NtParams p) {
  constexpr bool F32 = ET == 2;
  constexpr bool BF16 = ET == 1;
  constexpr int ES = F32 ? 4 : 2;
  constexpr int ITEM = 128 / ES;      // positions per epilogue item = per staging box line: 64 or 32
  constexpr int IPC = CHUNK / ITEM;   // items per chunk: 2 or 4
  static_assert(!(F32 && YMN), "the fp32 variant takes hidden-contiguous operands only");
  using S = NtSmem<NH, ES>;
  using OT = KMajorTileE<NH, ES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + S::OFF_BARS;
  auto bar_q_full = [&](int s) { return bars + 8u * s; };
  auto bar_q_empty = [&](int s) { return bars + 8u * (S::QS + s); };
  auto bar_k_full = [&](int s) { return bars + 8u * (2 * S::QS + s); };
  auto bar_k_empty = [&](int s) { return bars + 8u * (2 * S::QS + S::KS + s); };
  auto bar_acc_full = [&](int s) { return bars + 8u * (2 * S::QS + 2 * S::KS + s); };
  auto bar_acc_empty = [&](int s) { return bars + 8u * (2 * S::QS + 2 * S::KS + ACC_STAGES + s); };
  // staging box x has been filled by an epilogue group (all its threads arrive)
  auto bar_st_full = [&](int x) { return bars + 8u * (2 * S::QS + 2 * S::KS + 2 * ACC_STAGES + x); };
  // Boxes come back in item order, so one counter says which are free again: the number of staged items whose store has
  // read its box.  Item n may fill box n % STAGE_BOXES once item n - STAGE_BOXES is among them.  (A counter, not an
  // mbarrier per box: a group may reach its wait for a box before the group of the box's previous item has reached its
  // own, and a parity wait cannot tell the phase it wants from the one two earlier.  Accumulator stages cannot be
  // overtaken like that: a stage is refilled only after both groups of its previous chunk have read it.)
  volatile int *st_freed = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 48);
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + S::OFF_MISC);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 4);
  volatile int *epi_ok = reinterpret_cast<volatile int *>(base_ptr + S::OFF_MISC + 8);  // two per group, used in turn

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr bool paired = PAIRED;
  if (threadIdx.x == 0) WMM_TRACE_POINT(0);
  // order in which the chunks of a tile are loaded and multiplied: with pairing the last chunk comes
  // second, so that both triangles are in TMEM together
  auto chunk_at = [&](int k) -> int { return !paired ? k : (k == 0 ? 0 : (k == 1 ? p.nchunks - 1 : k - 1)); };

  // Items of a tile whose box lies wholly inside the band go through a staging box and a TMA store: all of them with
  // pairing; otherwise the halves of chunks 1 .. floor((2w - 127) / 128).  They are consecutive: items st_first ..
  // st_first + st_count - 1 of every tile.
  const int st_first = paired ? 0 : IPC;
  const int st_count = paired ? IPC * (p.nchunks - 1) : IPC * max(0, (2 * p.w - (CHUNK - 1)) / CHUNK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::QS; s++) { mbar_init(bar_q_full(s), 1); mbar_init(bar_q_empty(s), 1); }
    for (int s = 0; s < S::KS; s++) { mbar_init(bar_k_full(s), 1); mbar_init(bar_k_empty(s), 1); }
    for (int s = 0; s < ACC_STAGES; s++) { mbar_init(bar_acc_full(s), 1); mbar_init(bar_acc_empty(s), IPC * EPI_THREADS); }
    for (int x = 0; x < S::STAGE_BOXES; x++) mbar_init(bar_st_full(x), EPI_THREADS);
    *st_freed = 0;
    *abort_flag = 0;
    for (int g = 0; g < 2 * EPI_GROUPS; g++) epi_ok[g] = 1;
    fence_mbar_init();
    prefetch_tmap(&map_x);
    prefetch_tmap(&map_y);
    prefetch_tmap(&map_band);
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
  if (threadIdx.x == 0) WMM_TRACE_POINT(1);
  griddep_launch_dependents();
  griddep_wait();
  if (threadIdx.x == 0) WMM_TRACE_POINT(2);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int qit = 0, kit = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++qit) {
        const int b = tile / p.tiles_per_batch, r0 = (tile % p.tiles_per_batch) * TILE;
        const int qs = qit % S::QS;
        if (!(ok = mbar_wait(bar_q_empty(qs), ((qit / S::QS) & 1) ^ 1, abort_flag))) break;
        mbar_expect_tx(bar_q_full(qs), OT::BYTES);
#pragma unroll
        for (int bx = 0; bx < OT::NBOX; bx++)
          tma_load_3d(base + S::OFF_Q + qs * OT::BYTES + bx * OT::BOX_BYTES, &map_x, bar_q_full(qs), bx * OT::BOXK, r0, b);
        if (qit == 0) WMM_TRACE_POINT(3);
        for (int k = 0; k < p.nchunks; ++k, ++kit) {
          const int ks = kit % S::KS;
          if (!(ok = mbar_wait(bar_k_empty(ks), ((kit / S::KS) & 1) ^ 1, abort_flag))) break;
          mbar_expect_tx(bar_k_full(ks), OT::BYTES);
          const int p0 = r0 - p.w + p.off + chunk_at(k) * CHUNK;
          if (YMN) {
#pragma unroll
            for (int hf = 0; hf < 2; hf++)  // map dims: (position, hidden, batch)
              tma_load_3d(base + S::OFF_K + ks * OT::BYTES + hf * (OT::BYTES / 2), &map_y, bar_k_full(ks), p0 + hf * HALF, 0, b);
          } else {
#pragma unroll
            for (int bx = 0; bx < OT::NBOX; bx++)
              tma_load_3d(base + S::OFF_K + ks * OT::BYTES + bx * OT::BOX_BYTES, &map_y, bar_k_full(ks), bx * OT::BOXK, p0, b);
          }
        }
      }
      WMM_TRACE_POINT(4);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // One accumulator stage = one chunk (128 rows x 128 positions, 128 TMEM columns); 4 stages.  The two halves of a
    // stage are converted by two epilogue groups; the stage is free again when both have read it.  With pairing the
    // first and the last chunk of a tile are multiplied back to back, so that both triangles are in TMEM together.
    if (lane == 0) {
      constexpr uint32_t IDESC = F32 ? instr_desc_tf32(false, false, TILE, CHUNK) : instr_desc_f16(BF16, false, YMN, TILE, CHUNK);
      // MN-major Y: one box = NH rows (hidden) of 64 positions (128 B); 8-row groups 1024 B apart, a k-step of
      // 16 hidden rows is 2048 B further; the second 64 positions of the chunk are the second box (leading offset).
      constexpr uint64_t YDESC = YMN ? smem_desc_base(OT::BYTES / 2, 1024, 2u) : OT::DESC;
      int qit = 0, kit = 0, ait = 0;
      bool ok = true;
      auto chunk_mma = [&](uint32_t q_addr, uint32_t k_addr) -> bool {
        const int as = ait % ACC_STAGES;
        if (!mbar_wait(bar_acc_empty(as), ((ait / ACC_STAGES) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int s = 0; s < OT::KSTEPS; s++) {
          const uint64_t da = smem_desc(OT::DESC, q_addr + OT::kstep_offset(s));
          const uint64_t db = smem_desc(YDESC, k_addr + (YMN ? (uint32_t)s * 2048u : OT::kstep_offset(s)));
          if (F32) umma_tf32(tmem_base + as * CHUNK, da, db, IDESC, s > 0 ? 1u : 0u);
          else umma_f16(tmem_base + as * CHUNK, da, db, IDESC, s > 0 ? 1u : 0u);
        }
        umma_commit(bar_acc_full(as));
        ++ait;
        return true;
      };
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++qit) {
        const int qs = qit % S::QS;
        if (!(ok = mbar_wait(bar_q_full(qs), (qit / S::QS) & 1, abort_flag))) break;
        if (qit == 0) WMM_TRACE_POINT(5);
        const uint32_t q_addr = base + S::OFF_Q + qs * OT::BYTES;
        int k = 0;
        if (paired) {
          const int ks0 = kit % S::KS, ks1 = (kit + 1) % S::KS;
          if (!(ok = mbar_wait(bar_k_full(ks0), (kit / S::KS) & 1, abort_flag))) break;
          if (!(ok = mbar_wait(bar_k_full(ks1), ((kit + 1) / S::KS) & 1, abort_flag))) break;
          const uint32_t k0_addr = base + S::OFF_K + ks0 * OT::BYTES, k1_addr = base + S::OFF_K + ks1 * OT::BYTES;
          if (!(ok = chunk_mma(q_addr, k0_addr) && chunk_mma(q_addr, k1_addr))) break;
          umma_commit(bar_k_empty(ks0));
          umma_commit(bar_k_empty(ks1));
          kit += 2;
          k = 2;
        }
        for (; k < p.nchunks; ++k, ++kit) {
          const int ks = kit % S::KS;
          if (!(ok = mbar_wait(bar_k_full(ks), (kit / S::KS) & 1, abort_flag))) break;
          const uint32_t k_addr = base + S::OFF_K + ks * OT::BYTES;
          if (!(ok = chunk_mma(q_addr, k_addr))) break;
          umma_commit(bar_k_empty(ks));
        }
        if (ok) umma_commit(bar_q_empty(qs));
      }
      WMM_TRACE_POINT(6);
    }
  } else if (warp < 2 + 4 * EPI_GROUPS) {
    // ---------------- epilogue groups: thread <-> band row of the tile ----------------
    // A work item is HALF a chunk: 128 rows x 64 columns = one TMA box of the band.  Items go to the
    // four groups round-robin; both halves of a chunk read the same accumulator stage.
    const int grp = (warp - 2) >> 2;   // 0 .. EPI_GROUPS-1
    const int quarter = warp & 3;      // TMEM lanes 32*quarter .. +31 belong to this warp
    const int rr = quarter * 32 + lane;
    const bool leader = (threadIdx.x == 64 + grp * EPI_THREADS);
    const uint32_t bar_id = 1 + grp;
    int seen = 0;   // items this group has taken so far: picks the verdict word
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const int W = 2 * p.w + 1;
    const int items_per_tile = IPC * (paired ? p.nchunks - 1 : p.nchunks);
    uint16_t *band = static_cast<uint16_t *>(p.band);
    int cit = 0, iit = 0, rot = 0;  // chunks (accumulator stages) of earlier tiles / half-chunk items seen so far / group rotation
    // Items go to the groups round-robin over the CTA's whole item sequence.  When a tile has a multiple of four items,
    // its first two (the merged ones, the costliest) would always land on groups 0 and 1: the assignment is then
    // shifted by two from tile to tile.
    const int rot_step = (paired && (items_per_tile % EPI_GROUPS) == 0) ? 2 : 0;
    int tl = 0;   // tiles of this CTA so far
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
      const int b = tile / p.tiles_per_batch, r0 = (tile % p.tiles_per_batch) * TILE;
      const int i = r0 + rr;
      const int vr = min(TILE, p.M - r0);  // valid rows of this tile
      const bool rows_ok = rr < vr;
      // A group visits only its own items: the loop body is large, and an iteration that merely skips an item still
      // costs two jumps across it.
      const int tile_iit = iit;   // items of earlier tiles
      if (threadIdx.x == 64 && tl == 0) WMM_TRACE_POINT(18);   // (18 -> 19 is 3.4 us in the first tile of a launch, 0.2 us later)
      for (int hitem = (grp - tile_iit - rot) & (EPI_GROUPS - 1); hitem < items_per_tile; hitem += EPI_GROUPS) {
        if (threadIdx.x == 64 && iit == 0) WMM_TRACE_POINT(19);
        const int item = hitem / IPC, h = hitem % IPC;
        const bool pair_item = paired && item == 0;
        // stage of this item's chunk: with pairing the tile's stages hold chunks 0, last, 1, 2, ... in this order
        const int a0 = cit + (paired ? (item == 0 ? 0 : item + 1) : item);
        const int as = a0 % ACC_STAGES, as2 = (a0 + 1) % ACC_STAGES;
        const int c = pair_item ? 0 : item;  // chunk index (with pairing, items 1.. are chunks 1..)
        // staged items (boxes wholly inside the band, stored by TMA) are numbered through the CTA's whole sequence
        const bool staged = hitem >= st_first && hitem < st_first + st_count;
        const int sidx = tl * st_count + (hitem - st_first);
        const int sx = sidx % S::STAGE_BOXES;
        const uint32_t stage = base + S::OFF_STAGE + (uint32_t)sx * S::STAGE_HALF;
        volatile int *verdict = epi_ok + 2 * grp + (seen & 1);
        ++seen;
        if (leader) {
          int good = mbar_wait(bar_acc_full(as), (a0 / ACC_STAGES) & 1, abort_flag) ? 1 : 0;
          if (good && pair_item) good = mbar_wait(bar_acc_full(as2), ((a0 + 1) / ACC_STAGES) & 1, abort_flag) ? 1 : 0;
          if (grp == 0 && iit == 0) WMM_TRACE_POINT(7);
          // the store that last used this staging box has read it
          if (good && staged) good = count_wait(st_freed, sidx - S::STAGE_BOXES + 1, abort_flag) ? 1 : 0;
          *verdict = good;
        }
        named_bar_sync(bar_id, EPI_THREADS);
        if (!(ok = (*verdict != 0))) break;
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + as * CHUNK + h * ITEM + lane_sel;  // columns ITEM*h .. of chunk c
        // positions of chunk c inside the sequence: columns kk in [kk_lo, kk_hi)
        const int p0 = r0 - p.w + p.off + c * CHUNK;
        const int kk_lo = p.lo - p0, kk_hi = p.hi - p0;
        const bool edge = kk_lo > 0 || kk_hi < CHUNK;

        if (PAIRED && pair_item) {
          // ---- merged first + last chunk ----
          // A warp owns rows 32*quarter .. +31.  Column blocks left of its diagonal block hold only
          // last-chunk entries of these rows, blocks right of it only first-chunk entries; the diagonal
          // block holds both, split per lane.
          const int cl = p.nchunks - 1;
          const uint32_t taddr_l = tmem_base + as2 * CHUNK + h * HALF + lane_sel;
          const int kl_lo = kk_lo - cl * CHUNK, kl_hi = kk_hi - cl * CHUNK;
          const bool edge_l = kl_lo > 0 || kl_hi < CHUNK;
          const bool direct_l = (rr == vr - 1);  // last valid row: its last-chunk piece has no staging line
          if constexpr (F32) {
            // fp32: an item is ONE 32-column block (g = h), a staging line holds its 32 values in eight 16-byte pieces
            const uint32_t taddr_lq = tmem_base + as2 * CHUNK + h * ITEM + lane_sel;
            float *row_lf = static_cast<float *>(p.band) + (int64_t)b * p.band_sb + (int64_t)i * W + (cl * CHUNK - rr);
            const int g = h;
            if (g < quarter) {
              uint32_t vl[32];
              tmem_ld_x32(taddr_lq, vl);
              tmem_ld_wait();
              if (edge_l) mask_columns(vl, g * 32, kl_lo, kl_hi);
              if (rows_ok) {
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++) {
                  const uint4 pc = make_uint4(vl[4 * q8], vl[4 * q8 + 1], vl[4 * q8 + 2], vl[4 * q8 + 3]);
                  if (!direct_l) st_shared_v4(stage_addr(stage, rr + 1, q8), pc);
                  else *reinterpret_cast<uint4 *>(row_lf + g * 32 + q8 * 4) = pc;
                }
              }
            } else if (g > quarter) {
              uint32_t v0[32];
              tmem_ld_x32(taddr, v0);
              tmem_ld_wait();
              if (edge) mask_columns(v0, g * 32, kk_lo, kk_hi);
              if (rows_ok) {
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++)
                  st_shared_v4(stage_addr(stage, rr, q8), make_uint4(v0[4 * q8], v0[4 * q8 + 1], v0[4 * q8 + 2], v0[4 * q8 + 3]));
              }
            } else {
              // diagonal block: line rr takes columns >= lane from this thread's first-chunk row and columns < lane from
              // the last-chunk row of the thread one lane below; lane 31 also writes its own last-chunk row (line rr + 1)
              uint32_t v0[32], vl[32];
              tmem_ld_x32(taddr, v0);
              tmem_ld_x32(taddr_lq, vl);
              tmem_ld_wait();
              if (edge) mask_columns(v0, g * 32, kk_lo, kk_hi);
              if (edge_l) mask_columns(vl, g * 32, kl_lo, kl_hi);
              uint32_t m[32];
#pragma unroll
              for (int k2 = 0; k2 < 32; k2++) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, vl[k2], 1);
                m[k2] = (k2 >= lane) ? v0[k2] : up;
              }
              if (rows_ok) {
#pragma unroll
                for (int q8 = 0; q8 < 8; q8++)
                  st_shared_v4(stage_addr(stage, rr, q8), make_uint4(m[4 * q8], m[4 * q8 + 1], m[4 * q8 + 2], m[4 * q8 + 3]));
                if (direct_l) {
                  // the last valid row of the tile: columns 32*quarter .. rr of its last-chunk row go straight to the band
#pragma unroll
                  for (int q8 = 0; q8 < 8; q8++) {
                    const int kk0 = g * 32 + q8 * 4;
                    if (kk0 + 3 <= rr) {
                      *reinterpret_cast<uint4 *>(row_lf + kk0) = make_uint4(vl[4 * q8], vl[4 * q8 + 1], vl[4 * q8 + 2], vl[4 * q8 + 3]);
                    } else if (kk0 <= rr) {
#pragma unroll
                      for (int e = 0; e < 4; e++)
                        if (kk0 + e <= rr) row_lf[kk0 + e] = __uint_as_float(vl[4 * q8 + e]);
                    }
                  }
                } else if (lane == 31) {
#pragma unroll
                  for (int q8 = 0; q8 < 8; q8++)
                    st_shared_v4(stage_addr(stage, rr + 1, q8), make_uint4(vl[4 * q8], vl[4 * q8 + 1], vl[4 * q8 + 2], vl[4 * q8 + 3]));
                }
              }
            }
          } else {
          uint16_t *row_l = band + (int64_t)b * p.band_sb + (int64_t)i * W + (cl * CHUNK - rr);
#pragma unroll
          for (int gb = 0; gb < 2; gb++) {
            const int g = 2 * h + gb;
            if (g < quarter) {
              uint32_t vl[32];
              tmem_ld_x32(taddr_l + gb * 32, vl);
              tmem_ld_wait();
              if (edge_l) mask_columns(vl, g * 32, kl_lo, kl_hi);
              if (rows_ok) {
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {
                  if (!direct_l)
                    st_shared_v4(stage_addr(stage, rr + 1, gb * 4 + q4), pack8<BF16>(&vl[q4 * 8]));
                  else
                    *reinterpret_cast<uint4 *>(row_l + g * 32 + q4 * 8) = pack8<BF16>(&vl[q4 * 8]);
                }
              }
            } else if (g > quarter) {
              uint32_t v0[32];
              tmem_ld_x32(taddr + gb * 32, v0);
              tmem_ld_wait();
              if (edge) mask_columns(v0, g * 32, kk_lo, kk_hi);
              if (rows_ok) {
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) st_shared_v4(stage_addr(stage, rr, gb * 4 + q4), pack8<BF16>(&v0[q4 * 8]));
              }
            } else {
              // diagonal block: line rr takes columns >= rr from this thread's first-chunk row and
              // columns < rr from the last-chunk row of the thread one lane below (row rr - 1); lane 31
              // also writes its own last-chunk row, which is all of line rr + 1 within this block.
              uint32_t v0[32], vl[32];
              tmem_ld_x32(taddr + gb * 32, v0);
              tmem_ld_x32(taddr_l + gb * 32, vl);
              tmem_ld_wait();
              if (edge) mask_columns(v0, g * 32, kk_lo, kk_hi);
              if (edge_l) mask_columns(vl, g * 32, kl_lo, kl_hi);
              uint32_t m[16], pl[16];
#pragma unroll
              for (int k2 = 0; k2 < 16; k2++) {
                pl[k2] = pack2<BF16>(vl[2 * k2], vl[2 * k2 + 1]);
                const uint32_t own = pack2<BF16>(v0[2 * k2], v0[2 * k2 + 1]);
                const uint32_t up = __shfl_up_sync(0xffffffffu, pl[k2], 1);
                m[k2] = (2 * k2 >= lane) ? own : ((2 * k2 + 1 < lane) ? up : ((up & 0x0000ffffu) | (own & 0xffff0000u)));
              }
              if (rows_ok) {
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++)
                  st_shared_v4(stage_addr(stage, rr, gb * 4 + q4), make_uint4(m[4 * q4], m[4 * q4 + 1], m[4 * q4 + 2], m[4 * q4 + 3]));
                if (direct_l) {
                  // the last valid row of the tile: columns 32*quarter .. rr of its last-chunk row go
                  // straight to the band (lane + 1 values)
#pragma unroll
                  for (int q4 = 0; q4 < 4; q4++) {
                    const int kk0 = g * 32 + q4 * 8;
                    if (kk0 + 7 <= rr) {
                      *reinterpret_cast<uint4 *>(row_l + kk0) = make_uint4(pl[4 * q4], pl[4 * q4 + 1], pl[4 * q4 + 2], pl[4 * q4 + 3]);
                    } else if (kk0 <= rr) {
#pragma unroll
                      for (int e = 0; e < 8; e++)
                        if (kk0 + e <= rr) row_l[kk0 + e] = (uint16_t)(pl[4 * q4 + (e >> 1)] >> ((e & 1) * 16));
                    }
                  }
                } else if (lane == 31) {
#pragma unroll
                  for (int q4 = 0; q4 < 4; q4++)
                    st_shared_v4(stage_addr(stage, rr + 1, gb * 4 + q4), make_uint4(pl[4 * q4], pl[4 * q4 + 1], pl[4 * q4 + 2], pl[4 * q4 + 3]));
                }
              }
            }
          }
          }
          tc_fence_before_sync();
          mbar_arrive(bar_acc_empty(as));
          mbar_arrive(bar_acc_empty(as2));
        } else if (staged) {
          // ---- an item (half or quarter of a chunk) that lies wholly inside the band ----
          if constexpr (F32) {
            uint32_t va[32];
            tmem_ld_x32(taddr, va);
            tmem_ld_wait();
            // the values are in registers: the accumulator columns are free for the next chunk before the staging starts
            tc_fence_before_sync();
            mbar_arrive(bar_acc_empty(as));
            if (edge) mask_columns(va, h * ITEM, kk_lo, kk_hi);
#pragma unroll
            for (int q8 = 0; q8 < 8; q8++)
              st_shared_v4(stage_addr(stage, rr, q8), make_uint4(va[4 * q8], va[4 * q8 + 1], va[4 * q8 + 2], va[4 * q8 + 3]));
          } else {
            uint32_t va[32], vb[32];
            tmem_ld_x32(taddr, va);
            tmem_ld_x32(taddr + 32, vb);
            tmem_ld_wait();
            // the values are in registers: the accumulator half is free for the next chunk before the conversion starts
            tc_fence_before_sync();
            mbar_arrive(bar_acc_empty(as));
            if (edge) {
              mask_columns(va, h * 64, kk_lo, kk_hi);
              mask_columns(vb, h * 64 + 32, kk_lo, kk_hi);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) st_shared_v4(stage_addr(stage, rr, q4), pack8<BF16>(&va[q4 * 8]));
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) st_shared_v4(stage_addr(stage, rr, 4 + q4), pack8<BF16>(&vb[q4 * 8]));
          }
        } else if (!PAIRED) {
          // ---- triangular / ragged chunk of an unpaired window: predicated stores from registers.
          // Groups of 8 columns start on 16-byte boundaries of the band tensor, so whole groups go out
          // as one 16-byte store.
          if constexpr (F32) {
            // (groups of 4 fp32 columns are the 16-byte units)
            float *row = static_cast<float *>(p.band) + (int64_t)b * p.band_sb + (int64_t)i * W;
            uint32_t v[32];
            tmem_ld_x32(taddr, v);
            tmem_ld_wait();
            if (edge) mask_columns(v, h * ITEM, kk_lo, kk_hi);
            if (rows_ok) {
#pragma unroll
              for (int q8 = 0; q8 < 8; q8++) {
                const int j0 = c * CHUNK + h * ITEM + q8 * 4 - rr;
                if (j0 >= 0 && j0 + 3 <= 2 * p.w) {
                  *reinterpret_cast<uint4 *>(row + j0) = make_uint4(v[4 * q8], v[4 * q8 + 1], v[4 * q8 + 2], v[4 * q8 + 3]);
                } else if (j0 + 3 >= 0 && j0 <= 2 * p.w) {
#pragma unroll
                  for (int e = 0; e < 4; e++)
                    if (j0 + e >= 0 && j0 + e <= 2 * p.w) row[j0 + e] = __uint_as_float(v[4 * q8 + e]);
                }
              }
            }
          } else {
          uint16_t *row = band + (int64_t)b * p.band_sb + (int64_t)i * W;
#pragma unroll
          for (int gb = 0; gb < 2; gb++) {
            const int g = 2 * h + gb;
            uint32_t v[32];
            tmem_ld_x32(taddr + gb * 32, v);
            tmem_ld_wait();
            if (edge) mask_columns(v, g * 32, kk_lo, kk_hi);
            if (rows_ok) {
#pragma unroll
              for (int q4 = 0; q4 < 4; q4++) {
                const int j0 = c * CHUNK + g * 32 + q4 * 8 - rr;
                if (j0 >= 0 && j0 + 7 <= 2 * p.w) {
                  *reinterpret_cast<uint4 *>(row + j0) = pack8<BF16>(&v[q4 * 8]);
                } else if (j0 + 7 >= 0 && j0 <= 2 * p.w) {
#pragma unroll
                  for (int e = 0; e < 8; e++)
                    if (j0 + e >= 0 && j0 + e <= 2 * p.w) row[j0 + e] = pack1<BF16>(v[q4 * 8 + e]);
                }
              }
            }
          }
          }
          tc_fence_before_sync();
          mbar_arrive(bar_acc_empty(as));
        }

        if (staged) {   // hand the box to the store issuer
          fence_proxy_async_smem();
          mbar_arrive(bar_st_full(sx));
        }
      }
      cit += p.nchunks;
      iit += items_per_tile;
      rot += rot_step;
      ++tl;
    }
    if (leader && grp == 0) WMM_TRACE_POINT(9);
  } else {
    // ---------------- store issuer: every staged item of the CTA, in item order ----------------
    if (lane == 0) {
      int sidx = 0;   // staged items so far
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        const int b = tile / p.tiles_per_batch, r0 = (tile % p.tiles_per_batch) * TILE;
        for (int k = 0; k < st_count; ++k, ++sidx) {
          const int hitem = st_first + k;
          const int c = (paired && hitem < IPC) ? 0 : (hitem / IPC), h = hitem % IPC;
          const int sx = sidx % S::STAGE_BOXES;
          if (!(ok = mbar_wait(bar_st_full(sx), (sidx / S::STAGE_BOXES) & 1, abort_flag))) break;
          tma_store_3d(&map_band, base + S::OFF_STAGE + (uint32_t)sx * S::STAGE_HALF, r0 + c * CHUNK + h * ITEM, r0, b);  // x = i + j of the box's first column
          bulk_commit();
          if (sidx == 0) WMM_TRACE_POINT(8);
          if (sidx >= S::STORE_DEPTH) {
            bulk_wait_read<S::STORE_DEPTH>();   // all but the newest STORE_DEPTH stores have read their boxes
            *st_freed = sidx - S::STORE_DEPTH + 1;
          }
        }
      }
      bulk_wait_all();
      WMM_TRACE_POINT(10);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(&g_device_status, ST_NT_TIMEOUT);
    // give copies and MMAs that may still be in flight time to land before shared and tensor memory go away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (threadIdx.x == 0) WMM_TRACE_POINT(11);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
    if (lane == 0) WMM_TRACE_POINT(12);
  }
}
