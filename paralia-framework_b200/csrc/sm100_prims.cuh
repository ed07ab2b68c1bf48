// sm_100a device primitives shared by the tile kernels: mbarrier, TMA (bulk tensor
// copies, never with cluster multicast), and bounded waits.
//
// Every wait here gives up after a clock budget and reports through an error word so
// that a lost signal ends the kernel instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {
namespace prims {

// Error words written to the per-device status slot by a kernel that gave up.
enum : int {
  KERR_NONE = 0,
  KERR_FULL_WAIT_TIMEOUT = 1,   // a consumer never saw its stage arrive
  KERR_EMPTY_WAIT_TIMEOUT = 2,  // the producer never got a stage back
  KERR_DRAIN_TIMEOUT = 3,       // copies in flight did not land while bailing out
  KERR_TMEM_WAIT_TIMEOUT = 4    // an MMA-complete barrier never fired
};

// About two seconds at 2 GHz: far beyond any legitimate wait inside one tile.
constexpr long long WAIT_BUDGET_CLOCKS = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait for `parity` of `bar`. Returns false if the budget ran out or another thread of
// the CTA already raised *abort_flag (a shared-memory word).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag,
                                                  long long budget = WAIT_BUDGET_CLOCKS) {
  if (mbar_test(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t polls = 0;
  while (true) {
    if (mbar_test(bar, parity)) return true;
    if ((++polls & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget) return false;
    }
  }
}

// 3-D tiled TMA load global -> shared, completion on an mbarrier. No multicast.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace prims
}  // namespace paralia
