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
// Plain peer loads (16 bytes per access, several in flight per thread), local stores: no TMA, no multicast.
//
// Hand-shake, per launch, with an epoch e that every rank counts in step (all ranks issue the same sequence of these
// launches).  The two sides (lower / upper neighbour) are independent of each other:
//   (1) the rank publishes ready = e when its kernel starts (everything earlier in its stream is complete, so its rows
//       are final);
//   (2) CTA 0 alone polls the neighbours' ready words over the link, one thread per side, for at most kReadyWaitNs, and
//       publishes the verdict of each side in a LOCAL go word; the other CTAs poll those local words.  A side whose
//       neighbour did not show up in time is skipped by every CTA (each one raises the status bit itself); the other side
//       is still copied;
//   (3) when all CTAs are done the rank writes ack = e into both neighbours' flag blocks, whether it copied from them or
//       gave up on them, and then waits for their acks, so that nothing later in its own stream can overwrite rows a
//       neighbour is still reading.  The ack wait (kAckWaitNs) is longer than a neighbour's ready wait plus its copy, so
//       a rank whose OTHER neighbour is absent still acknowledges in time: only the ranks next to an absent one report
//       a time-out.
// Every wait is bounded by wall clock: a wait that runs out sets the status word (bit 5) and the kernel returns.
#include <mutex>

#include "wmm_common.cuh"

namespace wmm {
namespace {

// 256 threads per CTA.  A CTA does not fit on an SM beside a CTA of the tensor-core contractions (those take nearly all of
// an SM's shared memory, band_nt nearly all registers too; two-warp CTAs would fit beside band_nt but take 49 us instead of
// 30 us for the C4 exchange at two ranks and bought 3 us).  An exchange that should run beside a contraction gets SMs of its
// own instead: wmm_set_cta_limits caps the contraction's grid and this kernel's, which then runs one 512-thread CTA per SM
// with 16 loads in flight per thread.
constexpr int kHaloThreads = 256;
constexpr int kHaloMaxBlocks = 128;
constexpr int kHaloMaxBuffers = 4;
constexpr int kHaloUnroll = 4;           // independent 16-byte peer loads in flight per thread
constexpr int kHaloUnrollFew = 16;       // ... when a CTA limit leaves the exchange a few SMs only
constexpr int kHaloThreadsFew = 512;     // ... in CTAs that take an SM's whole register file (512 x ~126 registers)
constexpr unsigned long long ST_HALO_TIMEOUT = 1ull << 5;
constexpr unsigned long long kReadyWaitNs = 1000ull * 1000ull * 1000ull;
constexpr unsigned long long kGoWaitNs = 1500ull * 1000ull * 1000ull;     // local wait for CTA 0's verdict
constexpr unsigned long long kAckWaitNs = 3000ull * 1000ull * 1000ull;

struct HaloArgs {
  void *local[kHaloMaxBuffers];
  const void *lower[kHaloMaxBuffers];   // the lower neighbour's buffer of the same tensor (peer pointer) or NULL
  const void *upper[kHaloMaxBuffers];
  // accumulate == 2 only: this rank's unrounded fp32 edge rows (B, 4w, cols) as band_t writes them with edge_rows = 2w,
  // edge_skip = w: rows [w,2w) = first own rows, [2w,3w) = last own rows (the margins' rows of the buffer are not used)
  const float *edge_mine[kHaloMaxBuffers];
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
  unsigned *epoch_word;                  // local: epochs completed so far
  unsigned *scratch;                     // local: [0] CTAs done, [1] go word of the lower side, [2] of the upper side
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
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned *p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// waits until *p >= want (epochs only grow); false if the wait ran out
__device__ __forceinline__ bool wait_at_least(const unsigned *p, unsigned want, unsigned long long limit_ns) {
  if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
  const unsigned long long t0 = timer_ns();
  for (;;) {
    if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
    if (timer_ns() - t0 > limit_ns) return false;
    __nanosleep(200);
  }
}
// A go word holds 2 * epoch + (1 if the neighbour was ready in time).  Returns that bit, 0 also if the wait ran out.
__device__ __forceinline__ bool wait_go(const unsigned *p, unsigned e) {
  const unsigned long long t0 = timer_ns();
  for (;;) {
    const unsigned v = ld_acquire_gpu(p);
    if ((int)((v >> 1) - e) >= 0) return (v & 1u) != 0;
    if (timer_ns() - t0 > kGoWaitNs) return false;
    __nanosleep(100);
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

template <typename T, int UNROLL, int THREADS>
__global__ void __launch_bounds__(THREADS, 1) halo_pull_kernel(const HaloArgs a) {
  __shared__ int ok_s[2];
  __shared__ int last_s;
  const unsigned e = *reinterpret_cast<volatile unsigned *>(a.epoch_word) + 1u;
  // threads 0 and 32 look after the lower and the upper side
  if (threadIdx.x == 0 || threadIdx.x == 32) {
    const int side = threadIdx.x >> 5;
    const unsigned *peer = side == 0 ? a.lower_flags : a.upper_flags;
    bool ok = false;
    if (blockIdx.x == 0) {
      if (side == 0) {
        __threadfence_system();
        st_release_sys(a.mine, e);   // my rows are final: everything earlier in this stream has completed
      }
      if (peer) ok = wait_at_least(peer, e, kReadyWaitNs);
      st_release_gpu(a.scratch + 1 + side, 2u * e + (ok ? 1u : 0u));   // the verdict on this side, for the other CTAs
    } else if (peer) {
      ok = wait_go(a.scratch + 1 + side, e);
    }
    ok_s[side] = ok ? 1 : 0;
    if (peer && !ok && a.status) atomicOr(a.status, ST_HALO_TIMEOUT);   // every CTA reports the share it skips
  }
  __syncthreads();

  // work items of one side: (buffer, batch entry, vector of the strip); UNROLL of them in flight per thread
  const long long per_buf = (long long)a.batch * a.strip_vecs;
  const long long per_side = (long long)a.count * per_buf;
  for (int side = 0; side < 2; ++side) {
    if (!ok_s[side]) continue;
    if (a.accumulate == 2) {
      // own edge rows = round(my UNROUNDED rows + the neighbour's margin rows): the neighbour's terms were rounded to 16
      // bits once (they cross the link as such), mine not at all before the sum.  8 elements (one 16-byte vector) per
      // item, 4 items per thread in flight.  Only the 16-bit types come here.
      if constexpr (sizeof(T) == 2) {
        constexpr int U = 4;
        const long long strip_elems = a.strip_vecs * 8;
        for (long long it0 = (long long)blockIdx.x * (THREADS * U) + threadIdx.x; it0 < per_side;
             it0 += (long long)gridDim.x * (THREADS * U)) {
          float4 mine[U][2];
          uint4 theirs[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long it = it0 + (long long)u * THREADS;
            if (it >= per_side) continue;
            const int t = (int)(it / per_buf);
            const long long q = it % per_buf;
            const long long b = q / a.strip_vecs, v = q % a.strip_vecs;
            const float *pm = a.edge_mine[t] + (b * 4 + (side == 0 ? 1 : 2)) * strip_elems + v * 8;
            const uint4 *src = static_cast<const uint4 *>(side == 0 ? a.lower[t] : a.upper[t]);
            theirs[u] = __ldcg(src + b * a.row_vecs + (side == 0 ? a.own_vecs : 0) + v);
            mine[u][0] = *reinterpret_cast<const float4 *>(pm);
            mine[u][1] = *(reinterpret_cast<const float4 *>(pm) + 1);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long it = it0 + (long long)u * THREADS;
            if (it >= per_side) continue;
            const int t = (int)(it / per_buf);
            const long long q = it % per_buf;
            const long long b = q / a.strip_vecs, v = q % a.strip_vecs;
            const long long d_off = b * a.row_vecs + (side == 0 ? a.strip_vecs : a.own_vecs - a.strip_vecs) + v;
            uint4 out;
            T *o = reinterpret_cast<T *>(&out);
            const float *m = reinterpret_cast<const float *>(mine[u]);
            const T *th = reinterpret_cast<const T *>(&theirs[u]);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = ElemTraits<T>::store(m[k] + ElemTraits<T>::load(th + k));
            static_cast<uint4 *>(a.local[t])[d_off] = out;
          }
        }
      }
      continue;
    }
    // where item `it` comes from (in the neighbour's buffer) and goes to (in mine)
    auto place = [&](long long it, const uint4 *&src, uint4 *&dst) {
      const int t = (int)(it / per_buf);
      const long long q = it % per_buf;
      const long long b = q / a.strip_vecs, v = q % a.strip_vecs;
      long long s_off, d_off;
      if (!a.accumulate) {
        // lower: neighbour's last w own rows (they end where its upper margin starts) -> my lower margin
        // upper: neighbour's first w own rows (they start after its lower margin)     -> my upper margin
        s_off = b * a.row_vecs + (side == 0 ? a.own_vecs - a.strip_vecs : a.strip_vecs) + v;
        d_off = b * a.row_vecs + (side == 0 ? 0 : a.own_vecs) + v;
      } else {
        // lower: neighbour's upper margin -> added to my first w own rows; upper: neighbour's lower margin -> my last w
        s_off = b * a.row_vecs + (side == 0 ? a.own_vecs : 0) + v;
        d_off = b * a.row_vecs + (side == 0 ? a.strip_vecs : a.own_vecs - a.strip_vecs) + v;
      }
      src = static_cast<const uint4 *>(side == 0 ? a.lower[t] : a.upper[t]) + s_off;
      dst = static_cast<uint4 *>(a.local[t]) + d_off;
    };
    for (long long it0 = (long long)blockIdx.x * (THREADS * UNROLL) + threadIdx.x; it0 < per_side;
         it0 += (long long)gridDim.x * (THREADS * UNROLL)) {
      uint4 val[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long it = it0 + (long long)u * THREADS;
        if (it >= per_side) continue;
        const uint4 *src;
        uint4 *dst;
        place(it, src, dst);
        val[u] = __ldcg(src);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long it = it0 + (long long)u * THREADS;
        if (it >= per_side) continue;
        const uint4 *src;
        uint4 *dst;
        place(it, src, dst);
        *dst = a.accumulate ? add16<T>(*dst, val[u]) : val[u];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    last_s = atomicAdd(a.scratch, 1u) == gridDim.x - 1 ? 1 : 0;   // the last CTA of this launch closes the hand-shake
  }
  __syncthreads();
  if (!last_s) return;
  if (threadIdx.x == 0 || threadIdx.x == 32) {
    const int side = threadIdx.x >> 5;
    unsigned *peer = side == 0 ? a.lower_flags : a.upper_flags;
    if (side == 0) a.scratch[0] = 0;
    __threadfence_system();
    if (peer) {
      // my reads of this neighbour's rows are done (or given up): tell it, then wait until it is done with mine.
      // (I am the lower neighbour's UPPER neighbour and the upper neighbour's LOWER one.)
      st_release_sys(peer + (side == 0 ? 2 : 1), e);
      if (!wait_at_least(a.mine + 1 + side, e, kAckWaitNs) && a.status) atomicOr(a.status, ST_HALO_TIMEOUT);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *a.epoch_word = e;
    __threadfence();
  }
}

}  // namespace

cudaError_t launch_halo_pull(const wmm_halo_buffer *bufs, int count, const wmm_halo_flags &flags, unsigned *epoch_word,
                             unsigned *scratch, int batch, int rows, int cols, int window, int dtype, bool accumulate,
                             cudaStream_t stream, int *launches, const wmm_halo_edges *edges) {
  const size_t e = dtype == WMM_F32 ? 4 : dtype == WMM_F64 ? 8 : 2;
  HaloArgs a{};
  a.count = count;
  for (int i = 0; i < count; ++i) {
    if (edges) {
      a.local[i] = edges[i].local;
      a.edge_mine[i] = edges[i].mine;
      a.lower[i] = edges[i].lower;
      a.upper[i] = edges[i].upper;
    } else {
      a.local[i] = bufs[i].local;
      a.lower[i] = bufs[i].lower;
      a.upper[i] = bufs[i].upper;
    }
  }
  a.accumulate = edges ? 2 : accumulate ? 1 : 0;
  a.dtype = dtype;
  a.batch = batch;
  a.strip_vecs = (long long)window * cols * e / 16;
  a.row_vecs = (long long)(rows + 2 * window) * cols * e / 16;
  a.own_vecs = (long long)(rows + window) * cols * e / 16;
  a.mine = flags.mine;
  a.lower_flags = flags.lower;
  a.upper_flags = flags.upper;
  a.epoch_word = epoch_word;
  a.scratch = scratch;
  a.status = device_status_word();
  const long long per_side = (long long)count * batch * a.strip_vecs;
  // With a CTA limit the exchange runs beside a contraction on the few SMs that one leaves free: one CTA per SM, sized
  // (threads x registers) so that nothing else fits on its SM whichever kernel the hardware places first, with eight times
  // the loads in flight per CTA.
  const int cap = g_exchange_cta_limit.load(std::memory_order_relaxed);
  const long long per_cta = cap > 0 ? (long long)kHaloThreadsFew * kHaloUnrollFew : (long long)kHaloThreads * kHaloUnroll;
  long long blocks = (per_side + per_cta - 1) / per_cta;
  if (blocks < 1) blocks = 1;
  if (blocks > kHaloMaxBlocks) blocks = kHaloMaxBlocks;
  if (cap > 0 && blocks > cap) blocks = cap;
#define WMM_HALO_LAUNCH(T)                                                                   \
  do {                                                                                       \
    if (cap > 0)                                                                             \
      halo_pull_kernel<T, kHaloUnrollFew, kHaloThreadsFew><<<(int)blocks, kHaloThreadsFew, 0, stream>>>(a); \
    else                                                                                     \
      halo_pull_kernel<T, kHaloUnroll, kHaloThreads><<<(int)blocks, kHaloThreads, 0, stream>>>(a); \
  } while (0)
  switch (dtype) {
    case WMM_F16: WMM_HALO_LAUNCH(__half); break;
    case WMM_BF16: WMM_HALO_LAUNCH(__nv_bfloat16); break;
    case WMM_F32: WMM_HALO_LAUNCH(float); break;
    default: WMM_HALO_LAUNCH(double); break;
  }
#undef WMM_HALO_LAUNCH
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess && launches) ++*launches;
  return err;
}

// ---------------------------------------------------------------------------------------------------------------------
// The exchange for callers that cannot allocate device memory (wmm_halo_pull_static).  The three scratch words of a
// launch (CTAs done, go word per side) live in this array, which every device that loads the library holds until the
// process ends: WMM_HALO_STATIC_LANES lanes of 256 bytes.  Calls on the same lane share their words; two such calls
// that overlap on the GPU race.  The count of completed exchanges is NOT kept here but in word 3 of the caller's own
// flag block, so it starts at zero with every new flag block, in step with the neighbours.
// ---------------------------------------------------------------------------------------------------------------------
namespace {
constexpr int kLaneWords = 64;   // 256 bytes per lane
static __device__ __align__(256) unsigned g_halo_static_scratch[WMM_HALO_STATIC_LANES * kLaneWords];

// The device address of the array on the CURRENT device.  In host code the array's name is only a handle for the
// runtime, not an address a kernel could use; the address is resolved once per device, with that device current.
cudaError_t halo_static_base(unsigned **out) {
  static std::mutex mu;
  static unsigned *base[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && base[dev]) {
    *out = base[dev];
    return cudaSuccess;
  }
  void *p = nullptr;
  e = cudaGetSymbolAddress(&p, g_halo_static_scratch);
  if (e != cudaSuccess) return e;
  if (!p) return cudaErrorInvalidSymbol;
  if (dev >= 0 && dev < 64) base[dev] = static_cast<unsigned *>(p);
  *out = static_cast<unsigned *>(p);
  return cudaSuccess;
}
}  // namespace

cudaError_t launch_halo_pull_static(const wmm_halo_buffer *bufs, int count, const wmm_halo_flags &flags, int lane, int batch,
                                    int rows, int cols, int window, int dtype, bool accumulate, cudaStream_t stream,
                                    int *launches) {
  unsigned *base = nullptr;
  cudaError_t e = halo_static_base(&base);
  if (e != cudaSuccess) return e;
  unsigned *scratch = base + lane * kLaneWords;
  // whatever the previous call on this lane left behind (another flag block's go words, a counter of a launch that was
  // cut short) must not be read as this launch's: the lane starts from zero, in stream order
  e = cudaMemsetAsync(scratch, 0, kLaneWords * sizeof(unsigned), stream);
  if (e != cudaSuccess) return e;
  return launch_halo_pull(bufs, count, flags, flags.mine + 3, scratch, batch, rows, cols, window, dtype, accumulate, stream,
                          launches);
}

}  // namespace wmm
