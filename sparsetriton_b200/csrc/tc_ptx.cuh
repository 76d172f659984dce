// Inline-PTX building blocks of the tensor-core kernels (sm_100a): mbarriers with bounded waits,
// cp.async, tcgen05 MMA / commit / TMEM load, TMEM allocation, shared-memory operand descriptors.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sparsetriton_b200.h"

namespace st {
namespace tc {

constexpr long long kWaitCycles = 4000000000ll;                // ~2 s at 2 GHz

// Sticky device-side status: [0] ST_DEV_* flags, [1] id of the wait that expired, [2] block, [3] spare.
// Defined here: this header belongs to the single translation unit that holds the tensor-core kernels.
__device__ int32_t g_status[4];

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.shared::cta.b64 t, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// Bounded wait.  Returns false if the limit expired or another role already gave up.
// `sleep_ns` > 0 backs off between polls: waiting warps must not take issue slots from the MMA
// and producer warps that share their scheduler.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where,
                                          unsigned sleep_ns = 0) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      if (atomicOr(&g_status[0], ST_DEV_TIMEOUT) == 0) {
        g_status[1] = where;
        g_status[2] = blockIdx.x;
      }
      return false;
    }
  }
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Ask for one line to be brought into L2 (no register result, nothing to wait for).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// ---- TMA (bulk tensor copies).  The descriptor lives in kernel parameter space (__grid_constant__).
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 t;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Four rows of a 2-D tensor (row coordinates r0..r3, first column `col`) -> four consecutive 128-byte
// lines at `dst`, written with the descriptor's swizzle; rows outside the tensor (e.g. -1) arrive as
// zeros.  Completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void* desc, uint32_t bar, int col, int r0, int r1,
                                            int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
      "l"(desc), "r"(bar), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
// A (cols x rows) box of a 2-D tensor starting at (col, row) -> dense lines at `dst`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* desc, uint32_t bar, int col, int row) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(desc), "r"(bar), "r"(col), "r"(row)
      : "memory");
}

// Lagged, warp-aggregated hand-over of cp.async stages.
//
// Having every producer thread arrive on a stage's mbarrier costs ~130 serialised shared-memory
// atomics per stage.  Instead each thread closes a stage with cp.async.commit_group, remembers the
// stage's mbarrier in a short queue, and once LAG newer groups have been committed
// (cp.async.wait_group LAG: the oldest one has landed) the warp syncs and one lane arrives for it.
// A longer lag keeps more copies in flight per thread but holds ring slots back from the consumer.
template <int LAG>
struct StageQueue {
  uint32_t bar[LAG + 1];    // 0 = empty slot; bar[LAG] is the oldest
  __device__ __forceinline__ void clear() {
#pragma unroll
    for (int i = 0; i <= LAG; ++i) bar[i] = 0;
  }
  // Call after commit_group of the stage whose barrier is `b`.
  __device__ __forceinline__ void push(uint32_t b, int lane) {
    cp_async_wait_group<LAG>();
    const uint32_t oldest = bar[LAG];
#pragma unroll
    for (int i = LAG; i > 0; --i) bar[i] = bar[i - 1];
    bar[0] = b;
    if (oldest) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(oldest);
    }
  }
  // Hand over everything still queued (end of the kernel's work).
  __device__ __forceinline__ void flush(int lane) {
    cp_async_wait_all();
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int i = LAG; i >= 0; --i)
        if (bar[i]) mbar_arrive(bar[i]);
    }
    clear();
  }
};

// Whole-warp bounded wait: lane 0 polls, the result is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int where,
                                               int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, where) ? 1 : 0;
  return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}

// Named barrier 1 among the `Threads` producer threads.
template <int Threads>
__device__ __forceinline__ void producer_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(Threads) : "memory");
}

// Shared-memory operand descriptor for rows of 128 bytes.
//   lbo_bytes  distance between 128-byte column blocks (MN-major operands); ignored for K-major
//   sbo_bytes  distance between row groups: 1024 (8 rows) for the 128-byte swizzle, 512 (4 rows) for
//              the 128-byte swizzle with 32-byte atoms
//   layout     2 = SWIZZLE_128B (16-byte chunk index ^= row % 8)
//              1 = SWIZZLE_128B_BASE32B (32-byte chunk index ^= row % 4): the only swizzled layout
//                  the tensor core accepts for an MN-major operand of 32-bit elements (tf32)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;   // descriptor version of sm_100
  d |= (uint64_t)layout << 61;
  return d;
}

// Position (in 16-byte units) at which logical chunk c of row r is stored inside its 128-byte row.
__device__ __forceinline__ int swz16(int c, int r) { return c ^ (r & 7); }
__device__ __forceinline__ int swz32(int c, int r) { return c ^ ((r & 3) << 1); }


}  // namespace tc
}  // namespace st
