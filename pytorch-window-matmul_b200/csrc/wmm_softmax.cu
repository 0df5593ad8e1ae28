// Masked, scaled softmax over the rows of a band tensor (batch, rows, 2w+1), forward and backward, in ONE pass over HBM
// each: the step a windowed-attention block runs between window_matmul and unwindow_matmul (the reference composes it
// from torch ops, tests/test_attention.py:60-61: divide, softmax; a mask for the out-of-sequence slots is left to the
// caller).  HBM-bound: forward reads and writes the band once, backward reads two bands and writes one.
//
// A band row has an odd number of elements, so rows are only element-aligned.  One warp owns one row at a time and covers
// it with 16-byte vectors counted from the aligned address at or below the row start: the (at most two) vectors that
// straddle a neighbouring row are moved element by element, all others as one 16-byte access.  The whole row lives in
// registers between the load and the store, so the operation may run in place.
#include "wmm_common.cuh"
#include "wmm_ptx.cuh"

namespace wmm {
namespace {

constexpr int kWarpsPerBlock = 8;

struct SoftmaxArgs {
  const void *in;    // forward: scores; backward: probabilities
  const void *in2;   // backward: gradient of the probabilities
  void *out;
  long long rows_total;  // batch * rows
  long long row0;        // first row this launch handles
  int M, W, w;
  int off, lo, hi;   // slot j of row i is in sequence iff lo <= i + j - w + off < hi
  float scale;
  int mask;          // non-zero: out-of-sequence slots get probability 0; zero: they take part with their stored score
};

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, s));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
  return x;
}

template <typename T> struct alignas(16) AlignedVec { T v[16 / sizeof(T)]; };

// Row-in-registers kernels: VPL = 16-byte vectors per lane.
template <typename T, int VPL, bool BWD>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) band_softmax_kernel(const SoftmaxArgs a) {
  constexpr int E = 16 / (int)sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
  const float neg_inf = -INFINITY;
  for (long long r = a.row0 + warp0; r < a.rows_total; r += nwarps) {
    const int i = (int)(r % a.M);
    const T *row = static_cast<const T *>(a.in) + r * a.W;
    const int mis = (int)((reinterpret_cast<uintptr_t>(row) & 15) / sizeof(T));
    // slots j in [jlo, jhi) are in sequence
    const int jlo = max(0, a.lo - i + a.w - a.off);
    const int jhi = min(a.W, a.hi - i + a.w - a.off);
    float x[VPL][E];
    if (!BWD) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int e0 = (v * 32 + lane) * E - mis;
        if (e0 < a.W) {
          if (e0 >= 0 && e0 + E <= a.W) {
            AlignedVec<T> t = *reinterpret_cast<const AlignedVec<T> *>(row + e0);
#pragma unroll
            for (int k = 0; k < E; ++k) x[v][k] = ElemTraits<T>::load(&t.v[k]);
          } else {
#pragma unroll
            for (int k = 0; k < E; ++k) {
              const int idx = e0 + k;
              x[v][k] = (idx >= 0 && idx < a.W) ? ElemTraits<T>::load(row + idx) : neg_inf;
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < E; ++k) x[v][k] = neg_inf;
        }
      }
      float mx = neg_inf;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int e0 = (v * 32 + lane) * E - mis;
#pragma unroll
        for (int k = 0; k < E; ++k) {
          const int idx = e0 + k;
          const bool live = idx >= 0 && idx < a.W && (!a.mask || (idx >= jlo && idx < jhi));
          x[v][k] = live ? x[v][k] * a.scale : neg_inf;
          mx = fmaxf(mx, x[v][k]);
        }
      }
      mx = warp_max(mx);
      if (mx == neg_inf) mx = 0.f;   // a row with no live slot: all probabilities 0
      float sum = 0.f;
#pragma unroll
      for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int k = 0; k < E; ++k) {
          x[v][k] = sizeof(T) == 4 ? expf(x[v][k] - mx) : __expf(x[v][k] - mx);
          sum += x[v][k];
        }
      sum = warp_sum(sum);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      T *orow = static_cast<T *>(a.out) + r * a.W;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int e0 = (v * 32 + lane) * E - mis;
        if (e0 < a.W) {
          if (e0 >= 0 && e0 + E <= a.W) {
            AlignedVec<T> t;
#pragma unroll
            for (int k = 0; k < E; ++k) t.v[k] = ElemTraits<T>::store(x[v][k] * inv);
            *reinterpret_cast<AlignedVec<T> *>(orow + e0) = t;
          } else {
#pragma unroll
            for (int k = 0; k < E; ++k) {
              const int idx = e0 + k;
              if (idx >= 0 && idx < a.W) orow[idx] = ElemTraits<T>::store(x[v][k] * inv);
            }
          }
        }
      }
    } else {
      // grad_score = scale * P * (grad_P - sum_j grad_P * P); slots masked in the forward have P = 0 -> gradient 0
      const T *grow = static_cast<const T *>(a.in2) + r * a.W;
      float g[VPL][E];
      float dot = 0.f;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int e0 = (v * 32 + lane) * E - mis;
        if (e0 < a.W && e0 >= 0 && e0 + E <= a.W) {
          AlignedVec<T> t = *reinterpret_cast<const AlignedVec<T> *>(row + e0);
          AlignedVec<T> u = *reinterpret_cast<const AlignedVec<T> *>(grow + e0);
#pragma unroll
          for (int k = 0; k < E; ++k) {
            x[v][k] = ElemTraits<T>::load(&t.v[k]);
            g[v][k] = ElemTraits<T>::load(&u.v[k]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < E; ++k) {
            const int idx = e0 + k;
            const bool in = idx >= 0 && idx < a.W;
            x[v][k] = in ? ElemTraits<T>::load(row + idx) : 0.f;
            g[v][k] = in ? ElemTraits<T>::load(grow + idx) : 0.f;
          }
        }
#pragma unroll
        for (int k = 0; k < E; ++k) {
          const int idx = e0 + k;
          // masked slots: P is 0 there whatever the caller stored in grad_P (it may hold Inf/NaN)
          if (a.mask && !(idx >= jlo && idx < jhi)) { x[v][k] = 0.f; g[v][k] = 0.f; }
          dot += x[v][k] * g[v][k];
        }
      }
      dot = warp_sum(dot);
      T *orow = static_cast<T *>(a.out) + r * a.W;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int e0 = (v * 32 + lane) * E - mis;
        if (e0 < a.W) {
          if (e0 >= 0 && e0 + E <= a.W) {
            AlignedVec<T> t;
#pragma unroll
            for (int k = 0; k < E; ++k) t.v[k] = ElemTraits<T>::store(a.scale * x[v][k] * (g[v][k] - dot));
            *reinterpret_cast<AlignedVec<T> *>(orow + e0) = t;
          } else {
#pragma unroll
            for (int k = 0; k < E; ++k) {
              const int idx = e0 + k;
              if (idx >= 0 && idx < a.W) orow[idx] = ElemTraits<T>::store(a.scale * x[v][k] * (g[v][k] - dot));
            }
          }
        }
      }
    }
  }
}

// Any row length and fp64: one warp per row, three passes over the row (the second and third hit L1/L2).
template <typename T, bool BWD>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) band_softmax_loop_kernel(const SoftmaxArgs a) {
  using Acc = typename ElemTraits<T>::Acc;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
  for (long long r = a.row0 + warp0; r < a.rows_total; r += nwarps) {
    const int i = (int)(r % a.M);
    const T *row = static_cast<const T *>(a.in) + r * a.W;
    T *orow = static_cast<T *>(a.out) + r * a.W;
    const int jlo = a.mask ? max(0, a.lo - i + a.w - a.off) : 0;
    const int jhi = a.mask ? min(a.W, a.hi - i + a.w - a.off) : a.W;
    const Acc scale = (Acc)a.scale;
    if (!BWD) {
      Acc mx = -INFINITY;
      for (int j = jlo + lane; j < jhi; j += 32) mx = max(mx, (Acc)ElemTraits<T>::load(row + j) * scale);
      for (int s = 16; s > 0; s >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, s));
      Acc sum = 0;
      for (int j = jlo + lane; j < jhi; j += 32) sum += exp((Acc)ElemTraits<T>::load(row + j) * scale - mx);
      for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
      const Acc inv = sum > 0 ? (Acc)1 / sum : (Acc)0;
      for (int j = lane; j < a.W; j += 32) {
        // read before write at the same index: in-place use is safe
        const Acc p = (j >= jlo && j < jhi) ? exp((Acc)ElemTraits<T>::load(row + j) * scale - mx) * inv : (Acc)0;
        orow[j] = ElemTraits<T>::store(p);
      }
    } else {
      const T *grow = static_cast<const T *>(a.in2) + r * a.W;
      Acc dot = 0;
      for (int j = jlo + lane; j < jhi; j += 32)
        dot += (Acc)ElemTraits<T>::load(row + j) * (Acc)ElemTraits<T>::load(grow + j);
      for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
      for (int j = lane; j < a.W; j += 32) {
        const Acc v = (j >= jlo && j < jhi)
                          ? scale * (Acc)ElemTraits<T>::load(row + j) * ((Acc)ElemTraits<T>::load(grow + j) - dot)
                          : (Acc)0;
        orow[j] = ElemTraits<T>::store(v);
      }
    }
  }
}

int sm_count_cached();

// ---- ring kernels: the band streams through shared memory ----------------------------------------------------------
// Persistent CTAs.  A chunk is a whole number of band rows whose bytes are a multiple of 16, so it moves with one
// untiled bulk copy in each direction.  Warp 0 (one lane) keeps up to `stages` chunk loads in flight, warp 1 (one lane)
// stores finished chunks, 16 warps compute in place in shared memory: one row per warp (rows of 35 elements and more)
// or one row per thread (shorter rows).  The copy engines therefore run ahead of and behind the arithmetic, which a
// load-compute-store loop in registers cannot do.  Every wait is bounded; a wait that runs out sets the CTA's abort
// flag, all roles leave their loops, and the kernel reports through the device status word.
using namespace ptx;
constexpr int kRingComputeWarps = 16;
constexpr int kRingThreads = (kRingComputeWarps + 2) * 32;
constexpr int kRingMaxStages = 8;
constexpr int kRingHeader = 256;            // barriers (3 x 8 stages x 8 bytes) + abort flag
constexpr unsigned long long ST_SOFTMAX_TIMEOUT = 4ull;

struct RingArgs {
  SoftmaxArgs a;
  unsigned long long *status;
  long long chunks;
  int rows_per_chunk;
  int stages;
  unsigned chunk_bytes;   // rows_per_chunk * W * sizeof(T), a multiple of 16
  unsigned slot_bytes;    // chunk_bytes rounded up to 128
};

// slots [jlo, jlo + width) of row i are in sequence (all of them when the mask is off)
__device__ __forceinline__ void live_range(const SoftmaxArgs &a, int i, int &jlo, unsigned &width) {
  if (a.mask) {
    jlo = max(0, a.lo - i + a.w - a.off);
    const int jhi = min(a.W, a.hi - i + a.w - a.off);
    width = (unsigned)max(jhi - jlo, 0);
  } else {
    jlo = 0;
    width = (unsigned)a.W;
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NR rows at once (independent instruction streams for the scheduler).  prow[n] / grow[n]: the rows in shared memory;
// full[n]: every slot of the row is live, so only the last element of a lane needs a bound check.
template <typename T, int EPL, int NR, bool BWD, bool PER_THREAD>
__device__ __forceinline__ void ring_rows(T *const (&prow)[NR], T *const (&grow)[NR], int W, const int (&jlo)[NR],
                                          const unsigned (&width)[NR], float scale, int lane) {
  constexpr float kLog2e = 1.4426950408889634f;
  const int first = PER_THREAD ? 0 : lane;
  constexpr int STEP = PER_THREAD ? 1 : 32;
  bool all_full = true;
#pragma unroll
  for (int n = 0; n < NR; ++n) all_full = all_full && jlo[n] == 0 && width[n] == (unsigned)W;
  // elements below `safe` exist for every lane whatever the row (warp-per-row: all but the last step)
  constexpr int SAFE = PER_THREAD ? 0 : EPL - 1;
  if constexpr (!BWD) {
    const float c = scale * kLog2e;
    float x[NR][EPL];
    float mx[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) mx[n] = -INFINITY;
    if (all_full) {
#pragma unroll
      for (int k = 0; k < EPL; ++k)
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          const int idx = first + k * STEP;
          if (k < SAFE || idx < W) {
            x[n][k] = ElemTraits<T>::load(prow[n] + idx) * c;
          } else {
            x[n][k] = -INFINITY;
          }
          mx[n] = fmaxf(mx[n], x[n][k]);
        }
    } else {
#pragma unroll
      for (int k = 0; k < EPL; ++k)
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          const int idx = first + k * STEP;
          const bool live = (unsigned)(idx - jlo[n]) < width[n];
          x[n][k] = live ? ElemTraits<T>::load(prow[n] + idx) * c : -INFINITY;
          mx[n] = fmaxf(mx[n], x[n][k]);
        }
    }
    float sum[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) {
      if (!PER_THREAD) mx[n] = warp_max(mx[n]);
      if (mx[n] == -INFINITY) mx[n] = 0.f;
      sum[n] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k)
#pragma unroll
      for (int n = 0; n < NR; ++n) {
        x[n][k] = ex2_approx(x[n][k] - mx[n]);
        sum[n] += x[n][k];
      }
    float inv[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) {
      if (!PER_THREAD) sum[n] = warp_sum(sum[n]);
      inv[n] = sum[n] > 0.f ? 1.f / sum[n] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < EPL; ++k)
#pragma unroll
      for (int n = 0; n < NR; ++n) {
        const int idx = first + k * STEP;
        if (k < SAFE || idx < W) prow[n][idx] = ElemTraits<T>::store(x[n][k] * inv[n]);
      }
  } else {
    float p[NR][EPL], g[NR][EPL];
    float dot[NR];
#pragma unroll
    for (int n = 0; n < NR; ++n) dot[n] = 0.f;
    if (all_full) {
#pragma unroll
      for (int k = 0; k < EPL; ++k)
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          const int idx = first + k * STEP;
          if (k < SAFE || idx < W) {
            p[n][k] = ElemTraits<T>::load(prow[n] + idx);
            g[n][k] = ElemTraits<T>::load(grow[n] + idx);
          } else {
            p[n][k] = 0.f;
            g[n][k] = 0.f;
          }
          dot[n] += p[n][k] * g[n][k];
        }
    } else {
#pragma unroll
      for (int k = 0; k < EPL; ++k)
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          const int idx = first + k * STEP;
          const bool live = (unsigned)(idx - jlo[n]) < width[n];
          p[n][k] = live ? ElemTraits<T>::load(prow[n] + idx) : 0.f;
          g[n][k] = live ? ElemTraits<T>::load(grow[n] + idx) : 0.f;
          dot[n] += p[n][k] * g[n][k];
        }
    }
#pragma unroll
    for (int n = 0; n < NR; ++n)
      if (!PER_THREAD) dot[n] = warp_sum(dot[n]);
#pragma unroll
    for (int k = 0; k < EPL; ++k)
#pragma unroll
      for (int n = 0; n < NR; ++n) {
        const int idx = first + k * STEP;
        if (k < SAFE || idx < W) grow[n][idx] = ElemTraits<T>::store(scale * p[n][k] * (g[n][k] - dot[n]));
      }
  }
}

template <typename T, int EPL, int NR, bool BWD, bool PER_THREAD>
__global__ void __launch_bounds__(kRingThreads) band_softmax_ring_kernel(const RingArgs ra) {
  extern __shared__ __align__(128) uint8_t ring_smem[];
  const SoftmaxArgs &a = ra.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = ra.stages;
  const uint32_t bars = smem_u32(ring_smem);
  auto bar_full = [&](int s) { return bars + 8u * (uint32_t)s; };
  auto bar_done = [&](int s) { return bars + 8u * (uint32_t)(kRingMaxStages + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (uint32_t)(2 * kRingMaxStages + s); };
  volatile int *abort_flag = reinterpret_cast<volatile int *>(ring_smem + 3 * 8 * kRingMaxStages);
  uint8_t *stage0 = ring_smem + kRingHeader;
  const size_t stage_bytes = (size_t)ra.slot_bytes * (BWD ? 2 : 1);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_done(s), kRingComputeWarps);
      mbar_init(bar_empty(s), 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      const uint8_t *in = static_cast<const uint8_t *>(a.in);
      const uint8_t *in2 = static_cast<const uint8_t *>(a.in2);
      int it = 0;
      for (long long c = blockIdx.x; c < ra.chunks; c += gridDim.x, ++it) {
        const int s = it % S;
        if (!mbar_wait(bar_empty(s), ((it / S) & 1) ^ 1, abort_flag)) break;
        uint8_t *buf = stage0 + (size_t)s * stage_bytes;
        mbar_expect_tx(bar_full(s), BWD ? 2u * ra.chunk_bytes : ra.chunk_bytes);
        bulk_load_1d(smem_u32(buf), in + (size_t)c * ra.chunk_bytes, ra.chunk_bytes, bar_full(s));
        if (BWD) bulk_load_1d(smem_u32(buf + ra.slot_bytes), in2 + (size_t)c * ra.chunk_bytes, ra.chunk_bytes, bar_full(s));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint8_t *out = static_cast<uint8_t *>(a.out);
      int it = 0;
      for (long long c = blockIdx.x; c < ra.chunks; c += gridDim.x, ++it) {
        const int s = it % S;
        if (!mbar_wait(bar_done(s), (it / S) & 1, abort_flag)) break;
        uint8_t *buf = stage0 + (size_t)s * stage_bytes + (BWD ? ra.slot_bytes : 0u);
        bulk_store_1d(out + (size_t)c * ra.chunk_bytes, smem_u32(buf), ra.chunk_bytes);
        bulk_commit();
        if (it >= 1) {
          bulk_wait_read<1>();                     // the store before this one has read its stage
          mbar_arrive(bar_empty((it - 1) % S));
        }
      }
      bulk_wait_all();
    }
  } else {
    const int cw = warp - 2;
    const int R = ra.rows_per_chunk;
    int it = 0;
    for (long long c = blockIdx.x; c < ra.chunks; c += gridDim.x, ++it) {
      const int s = it % S;
      if (!mbar_wait(bar_full(s), (it / S) & 1, abort_flag)) break;
      uint8_t *buf = stage0 + (size_t)s * stage_bytes;
      T *pbuf = reinterpret_cast<T *>(buf);
      T *gbuf = reinterpret_cast<T *>(buf + ra.slot_bytes);
      const long long row_base = c * (long long)R;
      constexpr int RSTEP = PER_THREAD ? kRingComputeWarps * 32 : kRingComputeWarps;   // rows between a worker's rows
      const int r_first = PER_THREAD ? cw * 32 + lane : cw;
      int i = (int)((row_base + r_first) % a.M);
      const int istep = RSTEP % a.M;
      for (int r = r_first; r < R; r += RSTEP * NR) {
        T *prow[NR], *grow[NR];
        int jlo[NR];
        unsigned width[NR];
#pragma unroll
        for (int n = 0; n < NR; ++n) {
          live_range(a, i, jlo[n], width[n]);
          prow[n] = pbuf + (size_t)(r + n * RSTEP) * a.W;
          grow[n] = gbuf + (size_t)(r + n * RSTEP) * a.W;
          i += istep;
          if (i >= a.M) i -= a.M;
        }
        ring_rows<T, EPL, NR, BWD, PER_THREAD>(prow, grow, a.W, jlo, width, a.scale, lane);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_done(s));
    }
  }

  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && ra.status) atomicOr(ra.status, ST_SOFTMAX_TIMEOUT);
    // give copies that may still be in flight time to land before shared memory goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
}

template <typename T, int EPL, int NR, bool BWD, bool PER_THREAD>
cudaError_t launch_ring_one(const RingArgs &ra, size_t smem, int grid, cudaStream_t stream) {
  auto kern = band_softmax_ring_kernel<T, EPL, NR, BWD, PER_THREAD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<grid, kRingThreads, smem, stream>>>(ra);
  return cudaGetLastError();
}

// Launches the ring kernel over the whole chunks of the problem; *rows_done = rows it covers (0: not applicable).
template <typename T, bool BWD>
cudaError_t launch_ring(const SoftmaxArgs &a, cudaStream_t stream, long long *rows_done, int *launches) {
  *rows_done = 0;
  const bool per_thread = a.W <= 33;
  const int epl = per_thread ? a.W : (a.W + 31) / 32;
  if (epl > 33) return cudaSuccess;
  const size_t row_bytes = (size_t)a.W * sizeof(T);
  // two rows per worker at a time where registers and shared memory allow
  const int nr = (!per_thread && epl * (BWD ? 2 : 1) <= 34 && row_bytes * 32 * (BWD ? 2 : 1) * 3 <= 200 * 1024) ? 2 : 1;
  const int unit = (per_thread ? kRingComputeWarps * 32 : kRingComputeWarps) * nr;   // a multiple of 16 rows
  long long k = (long long)(16384 / (row_bytes * unit));
  if (k < 1) k = 1;
  if (k > 8) k = 8;
  RingArgs ra;
  ra.a = a;
  ra.rows_per_chunk = (int)(unit * k);
  ra.chunk_bytes = (unsigned)(row_bytes * ra.rows_per_chunk);
  ra.slot_bytes = (ra.chunk_bytes + 127u) & ~127u;
  const size_t stage_bytes = (size_t)ra.slot_bytes * (BWD ? 2 : 1);
  long long stages = (200 * 1024) / (long long)stage_bytes;
  if (stages > kRingMaxStages) stages = kRingMaxStages;
  if (stages < 3) return cudaSuccess;
  ra.stages = (int)stages;
  ra.chunks = (a.rows_total - a.row0) / ra.rows_per_chunk;
  if (ra.chunks < 1) return cudaSuccess;
  ra.status = device_status_word();
  const size_t smem = kRingHeader + stage_bytes * ra.stages;
  const int sms = sm_count_cached();
  const int grid = (int)(ra.chunks < sms ? ra.chunks : sms);
  cudaError_t e = cudaErrorInvalidValue;
#define WMM_RING_CASE(E, PT)                                                                        \
  if (per_thread == PT && epl <= E) {                                                               \
    if constexpr (!PT && E * (BWD ? 2 : 1) <= 34) {                                                  \
      e = nr == 2 ? launch_ring_one<T, E, 2, BWD, PT>(ra, smem, grid, stream)                        \
                  : launch_ring_one<T, E, 1, BWD, PT>(ra, smem, grid, stream);                       \
    } else {                                                                                        \
      e = launch_ring_one<T, E, 1, BWD, PT>(ra, smem, grid, stream);                                 \
    }                                                                                               \
  } else
  WMM_RING_CASE(5, true)
  WMM_RING_CASE(9, true)
  WMM_RING_CASE(17, true)
  WMM_RING_CASE(33, true)
  WMM_RING_CASE(2, false)
  WMM_RING_CASE(3, false)
  WMM_RING_CASE(5, false)
  WMM_RING_CASE(9, false)
  WMM_RING_CASE(13, false)
  WMM_RING_CASE(17, false)
  WMM_RING_CASE(25, false)
  WMM_RING_CASE(33, false)
  { return cudaSuccess; }
#undef WMM_RING_CASE
  if (e == cudaSuccess) {
    *rows_done = ra.chunks * ra.rows_per_chunk;
    if (launches) *launches += 1;
  }
  return e;
}

int sm_count_cached() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

template <typename T, bool BWD>
cudaError_t launch_typed(SoftmaxArgs a, cudaStream_t stream, int *launches) {
  constexpr int E = 16 / (int)sizeof(T);
  const bool bases_aligned = ((reinterpret_cast<uintptr_t>(a.in) | reinterpret_cast<uintptr_t>(a.out) |
                               reinterpret_cast<uintptr_t>(a.in2)) & 15) == 0;
  if (bases_aligned) {
    long long done = 0;
    cudaError_t e = launch_ring<T, BWD>(a, stream, &done, launches);
    if (e != cudaSuccess) return e;
    a.row0 += done;
    if (a.row0 >= a.rows_total) return cudaSuccess;
  }
  if (launches) *launches += 1;
  // vectors that cover a row at the worst misalignment
  const long long nvec = ((long long)a.W + 2 * (E - 1)) / E;
  const int vpl = (int)((nvec + 31) / 32);
  const long long blocks_needed = (a.rows_total - a.row0 + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = (long long)sm_count_cached() * 8;   // 8 resident blocks of 256 threads per SM
  const int grid = (int)(blocks_needed < cap ? blocks_needed : cap);
  const bool aligned = bases_aligned;
  const dim3 block(kWarpsPerBlock * 32);
#define WMM_SOFTMAX_CASE(V)                                                         \
  if (aligned && vpl <= V) {                                                        \
    band_softmax_kernel<T, V, BWD><<<grid, block, 0, stream>>>(a);                  \
    return cudaGetLastError();                                                      \
  }
  if (sizeof(T) <= 4) {
    WMM_SOFTMAX_CASE(1)
    WMM_SOFTMAX_CASE(2)
    WMM_SOFTMAX_CASE(3)
    WMM_SOFTMAX_CASE(4)
    WMM_SOFTMAX_CASE(6)
    WMM_SOFTMAX_CASE(8)
    if constexpr (!BWD) {
      WMM_SOFTMAX_CASE(12)
      WMM_SOFTMAX_CASE(16)
    }
  }
#undef WMM_SOFTMAX_CASE
  band_softmax_loop_kernel<T, BWD><<<grid, block, 0, stream>>>(a);
  return cudaGetLastError();
}

template <bool BWD>
cudaError_t launch_any(const SoftmaxArgs &a, int dtype, cudaStream_t stream, int *launches) {
  switch (dtype) {
    case WMM_F16: return launch_typed<__half, BWD>(a, stream, launches);
    case WMM_BF16: return launch_typed<__nv_bfloat16, BWD>(a, stream, launches);
    case WMM_F32: return launch_typed<float, BWD>(a, stream, launches);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_band_softmax(bool backward, const void *in, const void *in2, void *out, const wmm_geometry &g,
                                int dtype, float scale, bool mask, cudaStream_t stream, int *launches) {
  SoftmaxArgs a;
  a.in = in;
  a.in2 = in2;
  a.out = out;
  a.rows_total = (long long)g.batch * g.rows;
  a.row0 = 0;
  a.M = g.rows;
  a.W = 2 * g.window + 1;
  a.w = g.window;
  a.off = g.other_off;
  a.lo = g.seq_lo;
  a.hi = g.seq_hi;
  a.scale = scale;
  a.mask = mask ? 1 : 0;
  cudaError_t e;
  if (dtype == WMM_F64) {
    const long long blocks_needed = (a.rows_total + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const long long cap = (long long)sm_count_cached() * 8;
    const int grid = (int)(blocks_needed < cap ? blocks_needed : cap);
    if (backward)
      band_softmax_loop_kernel<double, true><<<grid, kWarpsPerBlock * 32, 0, stream>>>(a);
    else
      band_softmax_loop_kernel<double, false><<<grid, kWarpsPerBlock * 32, 0, stream>>>(a);
    e = cudaGetLastError();
    if (launches) *launches += 1;
  } else {
    e = backward ? launch_any<true>(a, dtype, stream, launches) : launch_any<false>(a, dtype, stream, launches);
  }
  return e;
}

}  // namespace wmm
