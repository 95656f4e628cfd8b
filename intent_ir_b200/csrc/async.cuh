// mbarrier + bulk-copy (TMA, untiled) helpers for kernels that stage contiguous row segments
// global -> shared asynchronously.  Every wait is bounded.
#pragma once
#include <stdint.h>

namespace ib200 {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbarrier_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarrier_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbarrier_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarrier_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// false when the (generous) try limit ran out; the caller records that and carries on so that
// no barrier shared with other threads or CTAs is abandoned
__device__ __forceinline__ bool mbarrier_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbarrier_try_wait(bar, parity)) return true;
  // back off between polls: a spinning warp would take issue slots from the warps doing the work
  for (uint32_t tries = 0; tries < (1u << 22); ++tries) {
    __nanosleep(tries < 8 ? 32 : 128);
    if (mbarrier_try_wait(bar, parity)) return true;
  }
  return false;
}
// contiguous copy; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // earlier generic reads of this buffer are done
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// address of `local` (a shared-memory object of this CTA) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(local)), "r"(rank));
  return r;
}
// asynchronous 4-byte store into a peer CTA's shared memory that also counts 4 bytes on the
// peer's mbarrier: data and notification travel together, no fence on this CTA's other stores
__device__ __forceinline__ void remote_store_signal(uint32_t remote_addr, float value, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(remote_addr), "r"(__float_as_uint(value)), "r"(remote_bar) : "memory");
}

}  // namespace ib200
