// CUDA-core kernels for the three banded contractions: any dtype, any shape, any strides.
//
// This family is (a) the exact-ordering path for fp32 / fp64 -- every output element is one sequential
// multiply-add chain over the ascending reduction index, one thread per output, no split-K and no
// cross-thread partial sums, which is the accumulation order of the reference's kernels
// (csrc/window_matmul/cuda/window_matmul_cuda.cu:24-35,64-83) and of its CPU loops
// (csrc/window_matmul/cpu/window_matmul_cpu.cpp:43,92-93,137,186-187) -- and (b) the path for shapes
// the tensor-core kernels cannot take (hidden size 3, one-row sequences, odd windows, unaligned
// pointers).
//
// All three primitives are the same register-tiled product C[64 x 64] += A[64 x 16] * B[16 x 64] in
// dense coordinates (row, position); they differ only in how a dense coordinate maps to memory:
//   band_nt  C(i, p) = sum_h X[i,h] Y[p,h]        stored at Band[i, p - off - i + w]
//   band_n   C(i, h) = sum_p Band[i, p-off-i+w] Y[p,h]
//   band_t   C(p, h) = sum_i Band[i, p-off-i+w] X[i,h]
// Entries of the dense operand that fall outside the band or outside the sequence are read as zeros;
// a zero term leaves a floating-point sum unchanged, so the chain equals the reference's shorter one.
#include "wmm_common.cuh"

namespace wmm {

namespace {

constexpr int TM = 64;   // output rows per CTA
constexpr int TN = 64;   // output columns per CTA
constexpr int TK = 16;   // reduction slice staged in shared memory
constexpr int PAD = 4;
constexpr int THREADS = 256;

template <bool SPLIT> __device__ __forceinline__ float mac(float a, float b, float c) {
  return SPLIT ? __fadd_rn(c, __fmul_rn(a, b)) : fmaf(a, b, c);
}
template <bool SPLIT> __device__ __forceinline__ double mac(double a, double b, double c) {
  return SPLIT ? __dadd_rn(c, __dmul_rn(a, b)) : fma(a, b, c);
}

struct Tile {
  int b, rt, ct;
};

// A-operand fetch: dense element (m, k) of the tile, already converted to the accumulator type.
template <typename T, int PRIM>
__device__ __forceinline__ typename ElemTraits<T>::Acc fetch_a(const Problem &p, const Tile &t, int m, int kidx) {
  using Acc = typename ElemTraits<T>::Acc;
  const int W = 2 * p.w + 1;
  if (PRIM == BAND_NT) {
    const int i = t.rt * TM + m, h = kidx;
    if (i >= p.M || h >= p.N) return Acc(0);
    const T *x = static_cast<const T *>(p.a);
    return ElemTraits<T>::load(x + t.b * p.a_sb + i * p.a_sr + h * p.a_sc);
  } else if (PRIM == BAND_N) {
    // kidx counts positions from the first one any row of the tile can reach
    const int i = t.rt * TM + m;
    const int pos = t.rt * TM - p.w + p.off + kidx;
    const int j = pos - p.off - i + p.w;
    if (i >= p.M || j < 0 || j >= W || pos < p.lo || pos >= p.hi) return Acc(0);
    const T *band = static_cast<const T *>(p.a);
    return ElemTraits<T>::load(band + ((int64_t)t.b * p.M + i) * W + j);
  } else {
    const int pos = t.rt * TM + m;
    const int i = t.rt * TM - p.off - p.w + kidx;
    const int j = pos - p.off - i + p.w;
    if (i < 0 || i >= p.M || j < 0 || j >= W || pos < p.lo || pos >= p.hi) return Acc(0);
    const T *band = static_cast<const T *>(p.a);
    return ElemTraits<T>::load(band + ((int64_t)t.b * p.M + i) * W + j);
  }
}

// B-operand fetch: dense element (k, n).
template <typename T, int PRIM>
__device__ __forceinline__ typename ElemTraits<T>::Acc fetch_b(const Problem &p, const Tile &t, int kidx, int n) {
  using Acc = typename ElemTraits<T>::Acc;
  const T *y = static_cast<const T *>(p.b);
  if (PRIM == BAND_NT) {
    const int pos = t.rt * TM - p.w + p.off + t.ct * TN + n, h = kidx;
    if (pos < p.lo || pos >= p.hi || h >= p.N) return Acc(0);
    return ElemTraits<T>::load(y + t.b * p.b_sb + pos * p.b_sr + h * p.b_sc);
  } else if (PRIM == BAND_N) {
    const int pos = t.rt * TM - p.w + p.off + kidx, h = t.ct * TN + n;
    if (pos < p.lo || pos >= p.hi || h >= p.N) return Acc(0);
    return ElemTraits<T>::load(y + t.b * p.b_sb + pos * p.b_sr + h * p.b_sc);
  } else {
    const int i = t.rt * TM - p.off - p.w + kidx, h = t.ct * TN + n;
    if (i < 0 || i >= p.M || h >= p.N) return Acc(0);
    return ElemTraits<T>::load(y + t.b * p.b_sb + i * p.b_sr + h * p.b_sc);
  }
}

// AKF / BKF: whether the reduction index is the fastest-varying one in memory for that operand, which
// picks the thread-to-element mapping of the staging loads (coalescing only; results do not depend on it).
template <typename T, int PRIM, bool SPLIT, bool AKF, bool BKF>
__global__ void __launch_bounds__(THREADS) band_generic_kernel(const Problem p, int nrt, int nct, int klen) {
  using Acc = typename ElemTraits<T>::Acc;
  __shared__ Acc As[TK][TM + PAD];
  __shared__ Acc Bs[TK][TN + PAD];

  Tile t;
  {
    int64_t lin = blockIdx.x;
    t.ct = (int)(lin % nct);
    lin /= nct;
    t.rt = (int)(lin % nrt);
    t.b = (int)(lin / nrt);
  }
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;

  Acc acc[4][4];
#pragma unroll
  for (int u = 0; u < 4; u++)
#pragma unroll
    for (int v = 0; v < 4; v++) acc[u][v] = Acc(0);

  for (int k0 = 0; k0 < klen; k0 += TK) {
#pragma unroll
    for (int r = 0; r < (TM * TK) / THREADS; r++) {
      const int e = tid + r * THREADS;
      const int m = AKF ? e / TK : e % TM;
      const int k = AKF ? e % TK : e / TM;
      As[k][m] = (k0 + k < klen) ? fetch_a<T, PRIM>(p, t, m, k0 + k) : Acc(0);
    }
#pragma unroll
    for (int r = 0; r < (TN * TK) / THREADS; r++) {
      const int e = tid + r * THREADS;
      const int n = BKF ? e / TK : e % TN;
      const int k = BKF ? e % TK : e / TN;
      Bs[k][n] = (k0 + k < klen) ? fetch_b<T, PRIM>(p, t, k0 + k, n) : Acc(0);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; k++) {
      Acc a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; u++) a[u] = As[k][ty * 4 + u];
#pragma unroll
      for (int v = 0; v < 4; v++) b[v] = Bs[k][tx * 4 + v];
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[u][v] = mac<SPLIT>(a[u], b[v], acc[u][v]);
    }
    __syncthreads();
  }

  T *out = static_cast<T *>(p.o);
  const int W = 2 * p.w + 1;
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int m = ty * 4 + u;
#pragma unroll
    for (int v = 0; v < 4; v++) {
      const int n = tx * 4 + v;
      if (PRIM == BAND_NT) {
        const int i = t.rt * TM + m;
        const int j = t.ct * TN + n - m;  // = pos - off - i + w
        const int pos = i + j - p.w + p.off;
        if (i < p.M && j >= 0 && j < W)
          out[((int64_t)t.b * p.M + i) * W + j] =
              ElemTraits<T>::store((pos >= p.lo && pos < p.hi) ? acc[u][v] : Acc(0));
      } else {
        const int r = t.rt * TM + m, h = t.ct * TN + n;
        const int rmax = (PRIM == BAND_N) ? p.M : p.Mo;
        if (r < rmax && h < p.N) out[t.b * p.o_sb + r * p.o_sr + h * p.o_sc] = ElemTraits<T>::store(acc[u][v]);
      }
    }
  }
}

template <typename T, int PRIM, bool SPLIT>
cudaError_t launch_typed(const Problem &p, cudaStream_t stream) {
  int nrt, nct, klen;
  bool akf, bkf;
  if (PRIM == BAND_NT) {
    nrt = (p.M + TM - 1) / TM;
    nct = (TM + 2 * p.w + TN - 1) / TN;
    klen = p.N;
    akf = p.a_sc <= p.a_sr;
    bkf = p.b_sc <= p.b_sr;
  } else if (PRIM == BAND_N) {
    nrt = (p.M + TM - 1) / TM;
    nct = (p.N + TN - 1) / TN;
    klen = TM + 2 * p.w;
    akf = true;
    bkf = p.b_sr < p.b_sc;
  } else {
    nrt = (p.Mo + TM - 1) / TM;
    nct = (p.N + TN - 1) / TN;
    klen = TM + 2 * p.w;
    akf = false;
    bkf = p.b_sr < p.b_sc;
  }
  const int64_t blocks = (int64_t)p.B * nrt * nct;
  if (blocks <= 0) return cudaSuccess;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const dim3 grid((unsigned)blocks), block(THREADS);
  if (akf && bkf)
    band_generic_kernel<T, PRIM, SPLIT, true, true><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else if (akf)
    band_generic_kernel<T, PRIM, SPLIT, true, false><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else if (bkf)
    band_generic_kernel<T, PRIM, SPLIT, false, true><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else
    band_generic_kernel<T, PRIM, SPLIT, false, false><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  return cudaGetLastError();
}

template <typename T, bool SPLIT> cudaError_t launch_prim(Primitive prim, const Problem &p, cudaStream_t s) {
  switch (prim) {
    case BAND_NT: return launch_typed<T, BAND_NT, SPLIT>(p, s);
    case BAND_N: return launch_typed<T, BAND_N, SPLIT>(p, s);
    default: return launch_typed<T, BAND_T, SPLIT>(p, s);
  }
}

}  // namespace

cudaError_t launch_generic(Primitive prim, const Problem &p, cudaStream_t stream, int *launches) {
  const bool split = (p.flags & WMM_FLAG_SPLIT_ROUNDING) != 0;
  cudaError_t e;
  switch (p.dtype) {
    case WMM_F16: e = launch_prim<__half, false>(prim, p, stream); break;
    case WMM_BF16: e = launch_prim<__nv_bfloat16, false>(prim, p, stream); break;
    case WMM_F32:
      e = split ? launch_prim<float, true>(prim, p, stream) : launch_prim<float, false>(prim, p, stream);
      break;
    default:
      e = split ? launch_prim<double, true>(prim, p, stream) : launch_prim<double, false>(prim, p, stream);
      break;
  }
  if (e == cudaSuccess && launches) ++*launches;
  return e;
}

}  // namespace wmm
