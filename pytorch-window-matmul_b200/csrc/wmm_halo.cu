// Neighbour exchange of sequence-shard halos through PEER MEMORY (one process per GPU, NVLink / NVSwitch): one kernel
// launch per exchange, no host-side communication library on the data path.
//
// Every rank keeps its sharded operands in "extended" buffers (batch, rows + 2w, cols): w margin rows, its own rows, w
// margin rows.  The buffers and a small block of flag words live in memory that the neighbours have mapped (symmetric
// memory).  Two operations:
//   exchange   (accumulate = 0): lower margin <- the lower neighbour's last w own rows, upper margin <- the upper
//                                neighbour's first w own rows            (forward halo of K^T and V rows)
//   reduction  (accumulate = 1): my first w own rows += the lower neighbour's upper margin, my last w own rows += the
//                                upper neighbour's lower margin          (reverse halo of partial grad_K / grad_V rows)
// Plain peer loads (16 bytes per thread and access), local stores: no TMA, no multicast.
//
// Hand-shake, per launch, with an epoch e that every rank counts in step (all ranks issue the same sequence of these
// launches): (1) a rank publishes ready = e when its kernel starts (everything earlier in its stream is complete, so its
// rows are final); (2) a CTA copies from a neighbour only after it has seen that neighbour's ready >= e; (3) when all
// CTAs are done the rank writes ack = e into both neighbours' flag blocks and waits for their acks, so nothing later in
// its own stream can overwrite rows a neighbour is still reading.  Every wait is bounded by wall clock (1 s): a wait
// that runs out sets the status word (bit 5) and the kernel returns without hanging.
#include "wmm_common.cuh"

namespace wmm {
namespace {

constexpr int kHaloThreads = 256;
constexpr int kHaloMaxBuffers = 4;
constexpr unsigned long long ST_HALO_TIMEOUT = 1ull << 5;
constexpr unsigned long long kHaloWaitNs = 1000ull * 1000ull * 1000ull;

struct HaloArgs {
  void *local[kHaloMaxBuffers];
  const void *lower[kHaloMaxBuffers];   // the lower neighbour's buffer of the same tensor (peer pointer) or NULL
  const void *upper[kHaloMaxBuffers];
  int count;
  int accumulate;
  int dtype;
  long long strip_vecs;    // 16-byte vectors of one (w x cols) strip of one batch entry
  long long row_vecs;      // 16-byte vectors of one batch entry of an extended buffer: (rows + 2w) x cols
  long long own_vecs;      // ... of the rows before the upper margin: (w + rows) x cols
  int batch;
  // flag words: [0] ready, [1] ack written by the lower neighbour, [2] ack written by the upper neighbour
  unsigned *mine;
  unsigned *lower_flags, *upper_flags;   // peer pointers or NULL
  unsigned *counters;                    // local: [0] epoch, [1] CTAs done
  unsigned long long *status;
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// waits until *p >= want (epochs only grow); false if the wait ran out
__device__ __forceinline__ bool wait_at_least(const unsigned *p, unsigned want) {
  if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
  const unsigned long long t0 = timer_ns();
  for (;;) {
    if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
    if (timer_ns() - t0 > kHaloWaitNs) return false;
    __nanosleep(200);
  }
}

template <typename T> __device__ __forceinline__ uint4 add16(uint4 a, uint4 b) {
  T *x = reinterpret_cast<T *>(&a);
  const T *y = reinterpret_cast<const T *>(&b);
#pragma unroll
  for (int k = 0; k < 16 / (int)sizeof(T); ++k)
    x[k] = ElemTraits<T>::store(ElemTraits<T>::load(x + k) + ElemTraits<T>::load(y + k));
  return a;
}

template <typename T>
__global__ void __launch_bounds__(kHaloThreads) halo_pull_kernel(const HaloArgs a) {
  __shared__ int ok_s;
  const unsigned e = *reinterpret_cast<volatile unsigned *>(a.counters) + 1u;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(a.mine, e);   // my rows are final: everything earlier in this stream has completed
    }
    bool ok = true;
    if (a.lower_flags) ok = wait_at_least(a.lower_flags, e);
    if (ok && a.upper_flags) ok = wait_at_least(a.upper_flags, e);
    ok_s = ok ? 1 : 0;
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  if (ok) {
    // work items: (buffer, side, batch entry, vector of the strip)
    const long long per_side = (long long)a.batch * a.strip_vecs;
    const long long total = (long long)a.count * 2 * per_side;
    for (long long it = (long long)blockIdx.x * kHaloThreads + threadIdx.x; it < total; it += (long long)gridDim.x * kHaloThreads) {
      const int t = (int)(it / (2 * per_side));
      const long long r = it % (2 * per_side);
      const int side = (int)(r / per_side);   // 0: lower neighbour, 1: upper neighbour
      const long long q = r % per_side;
      const long long b = q / a.strip_vecs, v = q % a.strip_vecs;
      const uint4 *src = static_cast<const uint4 *>(side == 0 ? a.lower[t] : a.upper[t]);
      if (!src) continue;
      uint4 *dst = static_cast<uint4 *>(a.local[t]);
      long long s_off, d_off;
      if (!a.accumulate) {
        // lower: neighbour's last w own rows (they end where its upper margin starts) -> my lower margin
        // upper: neighbour's first w own rows (they start after its lower margin)     -> my upper margin
        s_off = b * a.row_vecs + (side == 0 ? a.own_vecs - a.strip_vecs : a.strip_vecs) + v;
        d_off = b * a.row_vecs + (side == 0 ? 0 : a.own_vecs) + v;
        dst[d_off] = __ldcg(src + s_off);
      } else {
        // lower: neighbour's upper margin -> added to my first w own rows; upper: neighbour's lower margin -> my last w
        s_off = b * a.row_vecs + (side == 0 ? a.own_vecs : 0) + v;
        d_off = b * a.row_vecs + (side == 0 ? a.strip_vecs : a.own_vecs - a.strip_vecs) + v;
        dst[d_off] = add16<T>(dst[d_off], __ldcg(src + s_off));
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(a.counters + 1, 1u);
    if (prev == gridDim.x - 1) {   // the last CTA of this launch
      a.counters[1] = 0;
      bool fine = ok;
      __threadfence_system();
      // my reads of the neighbours' rows are done: tell them; then wait until they are done with mine
      if (a.lower_flags) st_release_sys(a.lower_flags + 2, e);   // I am the lower neighbour's UPPER neighbour
      if (a.upper_flags) st_release_sys(a.upper_flags + 1, e);
      if (a.lower_flags) fine = wait_at_least(a.mine + 1, e) && fine;
      if (a.upper_flags) fine = wait_at_least(a.mine + 2, e) && fine;
      a.counters[0] = e;
      if (!fine && a.status) atomicOr(a.status, ST_HALO_TIMEOUT);
      __threadfence();
    }
  }
}

}  // namespace

cudaError_t launch_halo_pull(const wmm_halo_buffer *bufs, int count, const wmm_halo_flags &flags, int batch, int rows,
                             int cols, int window, int dtype, bool accumulate, cudaStream_t stream, int *launches) {
  const size_t e = dtype == WMM_F32 ? 4 : dtype == WMM_F64 ? 8 : 2;
  HaloArgs a{};
  a.count = count;
  for (int i = 0; i < count; ++i) {
    a.local[i] = bufs[i].local;
    a.lower[i] = bufs[i].lower;
    a.upper[i] = bufs[i].upper;
  }
  a.accumulate = accumulate ? 1 : 0;
  a.dtype = dtype;
  a.batch = batch;
  a.strip_vecs = (long long)window * cols * e / 16;
  a.row_vecs = (long long)(rows + 2 * window) * cols * e / 16;
  a.own_vecs = (long long)(rows + window) * cols * e / 16;
  a.mine = flags.mine;
  a.lower_flags = flags.lower;
  a.upper_flags = flags.upper;
  a.counters = flags.counters;
  a.status = device_status_word();
  const long long total = (long long)count * 2 * batch * a.strip_vecs;
  long long blocks = (total + kHaloThreads * 8 - 1) / (kHaloThreads * 8);
  if (blocks < 1) blocks = 1;
  if (blocks > 128) blocks = 128;
  switch (dtype) {
    case WMM_F16: halo_pull_kernel<__half><<<(int)blocks, kHaloThreads, 0, stream>>>(a); break;
    case WMM_BF16: halo_pull_kernel<__nv_bfloat16><<<(int)blocks, kHaloThreads, 0, stream>>>(a); break;
    case WMM_F32: halo_pull_kernel<float><<<(int)blocks, kHaloThreads, 0, stream>>>(a); break;
    default: halo_pull_kernel<double><<<(int)blocks, kHaloThreads, 0, stream>>>(a); break;
  }
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess && launches) ++*launches;
  return err;
}

}  // namespace wmm
