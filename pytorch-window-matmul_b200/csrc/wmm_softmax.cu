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

namespace wmm {
namespace {

constexpr int kWarpsPerBlock = 8;

struct SoftmaxArgs {
  const void *in;    // forward: scores; backward: probabilities
  const void *in2;   // backward: gradient of the probabilities
  void *out;
  long long rows_total;  // batch * rows
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
  for (long long r = warp0; r < a.rows_total; r += nwarps) {
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
  for (long long r = warp0; r < a.rows_total; r += nwarps) {
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
cudaError_t launch_typed(const SoftmaxArgs &a, cudaStream_t stream) {
  constexpr int E = 16 / (int)sizeof(T);
  // vectors that cover a row at the worst misalignment
  const long long nvec = ((long long)a.W + 2 * (E - 1)) / E;
  const int vpl = (int)((nvec + 31) / 32);
  const long long blocks_needed = (a.rows_total + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = (long long)sm_count_cached() * 8;   // 8 resident blocks of 256 threads per SM
  const int grid = (int)(blocks_needed < cap ? blocks_needed : cap);
  const bool aligned = ((reinterpret_cast<uintptr_t>(a.in) | reinterpret_cast<uintptr_t>(a.out) |
                         reinterpret_cast<uintptr_t>(a.in2)) & 15) == 0;
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
cudaError_t launch_any(const SoftmaxArgs &a, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case WMM_F16: return launch_typed<__half, BWD>(a, stream);
    case WMM_BF16: return launch_typed<__nv_bfloat16, BWD>(a, stream);
    case WMM_F32: return launch_typed<float, BWD>(a, stream);
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
  } else {
    e = backward ? launch_any<true>(a, dtype, stream) : launch_any<false>(a, dtype, stream);
  }
  if (e == cudaSuccess && launches) *launches += 1;
  return e;
}

}  // namespace wmm
