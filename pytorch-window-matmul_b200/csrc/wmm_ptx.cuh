// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels use: mbarriers, TMA
// (cp.async.bulk.tensor, no cluster multicast anywhere), tcgen05 MMA / TMEM, and the proxy fences between them.
// Every wait is bounded: a wait that runs out sets an abort flag that all roles of the CTA poll.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wmm {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wall-clock bound of any single wait.  Kernels of this library run for microseconds to milliseconds.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;

#ifdef WMM_TRACE
// (trace builds) the first wait of a kernel that ran out: barrier address, parity, block, thread
static __device__ unsigned long long g_wait_info[4] = {0, 0, 0, 0};
// ... and, for every warp of every block that abandoned a wait: (barrier address << 8) | (parity << 4) | 1
static __device__ unsigned long long g_wait_tab[160 * 20];
#endif

// Waits for the phase with the given parity to complete.  Returns false if the wait was abandoned,
// either because it ran out (then *abort_flag is set) or because another role of the CTA set the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
#ifdef WMM_SPIN_SLEEP
    __nanosleep(WMM_SPIN_SLEEP);
#endif
    if ((spin & 63u) == 0u) {
#ifdef WMM_TRACE
      if (*abort_flag) {
        if (blockIdx.x < 160 && (threadIdx.x >> 5) < 20)
          g_wait_tab[blockIdx.x * 20 + (threadIdx.x >> 5)] = ((unsigned long long)bar << 8) | (parity << 4) | 1ull;
        return false;
      }
#endif
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
#ifdef WMM_TRACE
        if (atomicCAS(&g_wait_info[0], 0ull, (unsigned long long)bar + 1ull) == 0ull) {
          g_wait_info[1] = parity;
          g_wait_info[2] = blockIdx.x;
          g_wait_info[3] = threadIdx.x;
        }
        if (blockIdx.x < 160 && (threadIdx.x >> 5) < 20)
          g_wait_tab[blockIdx.x * 20 + (threadIdx.x >> 5)] = ((unsigned long long)bar << 8) | (parity << 4) | 3ull;
#endif
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Waits until a counter in shared memory that another thread of the CTA only ever increases has reached `want`.  Bounded
// like mbar_wait.  The caller orders its later accesses behind the wait with a CTA barrier.
__device__ __forceinline__ bool count_wait(volatile int *counter, int want, volatile int *abort_flag) {
  if (*counter >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (*counter >= want) return true;
    if ((spin & 63u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ---- fences ---------------------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma operands)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- programmatic dependent launch ----------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the stream
// still runs.  launch_dependents: this CTA no longer minds the next kernel of the stream being scheduled (it gets SMs
// only as CTAs of this kernel exit).  wait: returns once the predecessor has completed and its memory is visible; nothing
// before it may touch global memory that the predecessor reads or writes.  Both are no-ops in a plain launch.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- TMA ------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// untiled bulk copies: both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void *dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tensor memory and tcgen05 --------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16/bf16 inputs, fp32 accumulation; issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with fp32 operands in shared memory read as tf32 (8 elements = 32 bytes of K per instruction).
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (lane field of taddr) + t.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------
// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets (all >> 4),
// descriptor version 1 at bit 46, swizzle mode at bits 61-63 (2 = 128 B, 4 = 64 B, 6 = 32 B).
__host__ __device__ constexpr uint64_t smem_desc_base(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle_code) {
  return ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) |
         ((uint64_t)swizzle_code << 61);
}
__device__ __forceinline__ uint64_t smem_desc(uint64_t base, uint32_t smem_addr) {
  return base | (uint64_t)((smem_addr >> 4) & 0x3fff);
}
// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, A/B format (0 = f16, 1 = bf16),
// operand majors (0 = K-major, 1 = MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc_f16(bool bf16, bool a_mn_major, bool b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Instruction descriptor of tcgen05.mma.kind::tf32: fp32 accumulator, A/B format 2 (tf32), the other fields as above.
__host__ __device__ constexpr uint32_t instr_desc_tf32(bool a_mn_major, bool b_mn_major, uint32_t m, uint32_t n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace ptx
}  // namespace wmm
