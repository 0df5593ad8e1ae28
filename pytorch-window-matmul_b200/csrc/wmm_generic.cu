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
// All three primitives are the same register-tiled product C[TM x TN] += A[TM x 16] * B[16 x TN] in
// dense coordinates (row, position) -- fp32: 128 x 128 tiles (band_nt) or 128 x 64 (band_n, band_t), 8 x 8 or
// 8 x 4 outputs per thread, next slice prefetched into registers -- and differ only in how a dense
// coordinate maps to memory:
//   band_nt  C(i, p) = sum_h X[i,h] Y[p,h]        stored at Band[i, p - off - i + w]
//   band_n   C(i, h) = sum_p Band[i, p-off-i+w] Y[p,h]
//   band_t   C(p, h) = sum_i Band[i, p-off-i+w] X[i,h]
// Entries of the dense operand that fall outside the band or outside the sequence are read as zeros;
// with finite operands a zero term leaves a floating-point sum unchanged (up to the sign of a zero sum), so the
// chain equals the reference's shorter one.  A non-finite operand row reaches every row of its tile (0 * Inf).
#include "wmm_common.cuh"

namespace wmm {

namespace {

constexpr int TK = 16;  // reduction slice staged in shared memory
constexpr int PAD = 4;
constexpr int THREADS = 256;

template <bool SPLIT> __device__ __forceinline__ float mac(float a, float b, float c) {
  return SPLIT ? __fadd_rn(c, __fmul_rn(a, b)) : fmaf(a, b, c);
}
template <bool SPLIT> __device__ __forceinline__ double mac(double a, double b, double c) {
  return SPLIT ? __dadd_rn(c, __dmul_rn(a, b)) : fma(a, b, c);
}

// Dense operand element (r, kidx) of a tile, r = output row (A operand) or output column (B operand),
// kidx = reduction index counted from the first one the tile can need.  Every case is an affine address
// plus a valid kidx range per r; outside the range the element is zero.
template <typename T, int PRIM, bool IS_A> struct OperandView {
  const T *base;          // element (r = 0, kidx = 0)
  int64_t r_stride, k_stride;
  int r_count;            // r < r_count exist
  int lo0, hi0;           // kidx range common to all r
  int w, W;
  // band operands: the valid range also depends on r (the band is 2w+1 wide around the diagonal)
  __device__ __forceinline__ void range(int r, int &lo, int &hi) const {
    lo = lo0;
    hi = hi0;
    if (IS_A && PRIM != BAND_NT) {  // j = kidx - r (band_n) resp. r - kidx + 2w (band_t) must lie in [0, W)
      lo = max(lo, r);
      hi = min(hi, r + W);
    }
    if (r >= r_count) hi = lo;
  }
  __device__ __forceinline__ const T *at(int r, int kidx) const { return base + r * r_stride + kidx * k_stride; }
};

template <typename T, int PRIM>
__device__ __forceinline__ void make_views(const Problem &p, int b, int rt, int ct, int TM, int TN, OperandView<T, PRIM, true> &A,
                                           OperandView<T, PRIM, false> &B) {
  const int W = 2 * p.w + 1;
  A.w = B.w = p.w;
  A.W = B.W = W;
  if (PRIM == BAND_NT) {
    const int i0 = rt * TM, p0 = rt * TM - p.w + p.off + ct * TN;
    A.base = static_cast<const T *>(p.a) + b * p.a_sb + (int64_t)i0 * p.a_sr;
    A.r_stride = p.a_sr; A.k_stride = p.a_sc; A.r_count = p.M - i0; A.lo0 = 0; A.hi0 = p.N;
    B.base = static_cast<const T *>(p.b) + b * p.b_sb + (int64_t)p0 * p.b_sr;
    B.r_stride = p.b_sr; B.k_stride = p.b_sc; A.w = p.w;
    // column n <-> position p0 + n: valid iff in [lo, hi)
    B.r_count = 0x7fffffff; B.lo0 = 0; B.hi0 = p.N;
    (void)B;
  } else if (PRIM == BAND_N) {
    const int i0 = rt * TM, c0 = ct * TN, pstart = i0 - p.w + p.off;  // kidx <-> position pstart + kidx
    // band[(b*M + i0 + r) * W + (kidx - r)]
    A.base = static_cast<const T *>(p.a) + ((int64_t)b * p.M + i0) * W;
    A.r_stride = W - 1; A.k_stride = 1; A.r_count = p.M - i0; A.lo0 = p.lo - pstart; A.hi0 = p.hi - pstart;
    B.base = static_cast<const T *>(p.b) + b * p.b_sb + (int64_t)pstart * p.b_sr + (int64_t)c0 * p.b_sc;
    B.r_stride = p.b_sc; B.k_stride = p.b_sr; B.r_count = p.N - c0; B.lo0 = p.lo - pstart; B.hi0 = p.hi - pstart;
  } else {
    const int p0 = rt * TM, c0 = ct * TN, istart = p0 - p.off - p.w;  // kidx <-> band row istart + kidx
    // band[(b*M + istart + kidx) * W + (r - kidx + 2w)]
    A.base = static_cast<const T *>(p.a) + ((int64_t)b * p.M + istart) * W + 2 * p.w;
    A.r_stride = 1; A.k_stride = W - 1;
    A.r_count = min(p.Mo, p.hi) - p0;  // positions beyond the sequence (or the output) produce zeros
    A.lo0 = max(-istart, 0); A.hi0 = p.M - istart;
    B.base = static_cast<const T *>(p.b) + b * p.b_sb + (int64_t)istart * p.b_sr + (int64_t)c0 * p.b_sc;
    B.r_stride = p.b_sc; B.k_stride = p.b_sr; B.r_count = p.N - c0; B.lo0 = max(-istart, 0); B.hi0 = p.M - istart;
  }
}

// AKF / BKF: whether the reduction index is the fastest-varying one in memory for that operand, which
// picks the thread-to-element mapping of the staging loads (coalescing only; results do not depend on it).
template <typename T, int PRIM, bool SPLIT, bool AKF, bool BKF, int TM, int TN>
__global__ void __launch_bounds__(THREADS) band_generic_kernel(const Problem p, int nrt, int nct, int klen) {
  using Acc = typename ElemTraits<T>::Acc;
  constexpr int MR = TM / 16, MC = TN / 16;          // outputs per thread
  constexpr int LA = TM * TK / THREADS, LB = TN * TK / THREADS;  // staged elements per thread and slice
  __shared__ Acc As[TK][TM + PAD];
  __shared__ Acc Bs[TK][TN + PAD];

  int b, rt, ct;
  {
    int64_t lin = blockIdx.x;
    ct = (int)(lin % nct);
    lin /= nct;
    rt = (int)(lin % nrt);
    b = (int)(lin / nrt);
  }
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;
  // Outputs of a thread: rows row_of(u), columns col_of(v).  Eight-wide micro-tiles are two groups of four,
  // half a tile apart, so that the 16-byte shared-memory reads of neighbouring threads are contiguous.
  auto row_of = [&](int u) -> int { return MR == 8 ? (u >> 2) * (TM / 2) + ty * 4 + (u & 3) : ty * MR + u; };
  auto col_of = [&](int v) -> int { return MC == 8 ? (v >> 2) * (TN / 2) + tx * 4 + (v & 3) : tx * MC + v; };

  OperandView<T, PRIM, true> A;
  OperandView<T, PRIM, false> B;
  make_views<T, PRIM>(p, b, rt, ct, TM, TN, A, B);
  // position bounds that depend on the output coordinate
  const int pos0 = (PRIM == BAND_NT) ? rt * TM - p.w + p.off + ct * TN : rt * TM;  // band_nt: column 0; band_t: row 0

  auto fetch_a = [&](int slot, int k0) -> Acc {
    const int e = tid + slot * THREADS;
    const int m = AKF ? e / TK : e % TM, k = AKF ? e % TK : e / TM;
    int lo, hi;
    A.range(m, lo, hi);
    if (PRIM == BAND_T && pos0 + m < p.lo) hi = lo;
    const int kidx = k0 + k;
    return (kidx >= lo && kidx < hi) ? ElemTraits<T>::load(A.at(m, kidx)) : Acc(0);
  };
  auto fetch_b = [&](int slot, int k0) -> Acc {
    const int e = tid + slot * THREADS;
    const int n = BKF ? e / TK : e % TN, k = BKF ? e % TK : e / TN;
    int lo, hi;
    B.range(n, lo, hi);
    if (PRIM == BAND_NT && (pos0 + n < p.lo || pos0 + n >= p.hi)) hi = lo;
    const int kidx = k0 + k;
    return (kidx >= lo && kidx < hi) ? ElemTraits<T>::load(B.at(n, kidx)) : Acc(0);
  };

  Acc acc[MR][MC];
#pragma unroll
  for (int u = 0; u < MR; u++)
#pragma unroll
    for (int v = 0; v < MC; v++) acc[u][v] = Acc(0);

  Acc ra[LA], rb[LB];  // the next slice, prefetched while the current one is multiplied
#pragma unroll
  for (int s = 0; s < LA; s++) ra[s] = fetch_a(s, 0);
#pragma unroll
  for (int s = 0; s < LB; s++) rb[s] = fetch_b(s, 0);

  for (int k0 = 0; k0 < klen; k0 += TK) {
#pragma unroll
    for (int s = 0; s < LA; s++) {
      const int e = tid + s * THREADS;
      As[AKF ? e % TK : e / TM][AKF ? e / TK : e % TM] = ra[s];
    }
#pragma unroll
    for (int s = 0; s < LB; s++) {
      const int e = tid + s * THREADS;
      Bs[BKF ? e % TK : e / TN][BKF ? e / TK : e % TN] = rb[s];
    }
    __syncthreads();
    if (k0 + TK < klen) {
#pragma unroll
      for (int s = 0; s < LA; s++) ra[s] = fetch_a(s, k0 + TK);
#pragma unroll
      for (int s = 0; s < LB; s++) rb[s] = fetch_b(s, k0 + TK);
    }
    const int kmax = min(TK, klen - k0);
#pragma unroll
    for (int k = 0; k < TK; k++) {
      if (k < kmax) {
        Acc a[MR], bb[MC];
#pragma unroll
        for (int u = 0; u < MR; u++) a[u] = As[k][row_of(u)];
#pragma unroll
        for (int v = 0; v < MC; v++) bb[v] = Bs[k][col_of(v)];
#pragma unroll
        for (int u = 0; u < MR; u++)
#pragma unroll
          for (int v = 0; v < MC; v++) acc[u][v] = mac<SPLIT>(a[u], bb[v], acc[u][v]);
      }
    }
    __syncthreads();
  }

  T *out = static_cast<T *>(p.o);
  const int W = 2 * p.w + 1;
#pragma unroll
  for (int u = 0; u < MR; u++) {
    const int m = row_of(u);
#pragma unroll
    for (int v = 0; v < MC; v++) {
      const int n = col_of(v);
      if (PRIM == BAND_NT) {
        const int i = rt * TM + m;
        const int j = ct * TN + n - m;  // = pos - off - i + w
        const int pos = i + j - p.w + p.off;
        if (i < p.M && j >= 0 && j < W)
          out[((int64_t)b * p.M + i) * W + j] = ElemTraits<T>::store((pos >= p.lo && pos < p.hi) ? acc[u][v] : Acc(0));
      } else {
        const int r = rt * TM + m, h = ct * TN + n;
        const int rmax = (PRIM == BAND_N) ? p.M : p.Mo;
        if (r < rmax && h < p.N) out[b * p.o_sb + r * p.o_sr + h * p.o_sc] = ElemTraits<T>::store(acc[u][v]);
      }
    }
  }
}

template <typename T, int PRIM, bool SPLIT, int TM, int TN>
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
    band_generic_kernel<T, PRIM, SPLIT, true, true, TM, TN><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else if (akf)
    band_generic_kernel<T, PRIM, SPLIT, true, false, TM, TN><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else if (bkf)
    band_generic_kernel<T, PRIM, SPLIT, false, true, TM, TN><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  else
    band_generic_kernel<T, PRIM, SPLIT, false, false, TM, TN><<<grid, block, 0, stream>>>(p, nrt, nct, klen);
  return cudaGetLastError();
}

// Tile shapes: fp32 with enough rows gets the large tiles; everything else (fp64: registers; 16-bit inputs:
// rarely here; short sequences: waste) the 64 x 64 ones.
template <typename T, bool SPLIT> cudaError_t launch_prim(Primitive prim, const Problem &p, cudaStream_t s) {
  constexpr bool F32 = sizeof(T) == 4;
  // large tiles only when there are enough of them to fill the device twice (B200: 148 SMs); a small problem is
  // spread over more CTAs with the 64 x 64 tiles
  const int64_t big_rows = (int64_t)p.B * (((prim == BAND_T ? p.Mo : p.M) + 127) / 128);
  const int64_t big_cols = prim == BAND_NT ? (128 + 2 * (int64_t)p.w + 127) / 128 : (p.N + 63) / 64;
  const bool big = F32 && p.M >= 512 && big_rows * big_cols >= 296;
  switch (prim) {
    case BAND_NT:
      if (F32 && big && p.w >= 32) return launch_typed<T, BAND_NT, SPLIT, F32 ? 128 : 64, F32 ? 128 : 64>(p, s);
      return launch_typed<T, BAND_NT, SPLIT, 64, 64>(p, s);
    case BAND_N:
      if (F32 && big && p.N > 32) return launch_typed<T, BAND_N, SPLIT, F32 ? 128 : 64, 64>(p, s);
      return launch_typed<T, BAND_N, SPLIT, 64, 64>(p, s);
    default:
      if (F32 && big && p.N > 32) return launch_typed<T, BAND_T, SPLIT, F32 ? 128 : 64, 64>(p, s);
      return launch_typed<T, BAND_T, SPLIT, 64, 64>(p, s);
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
