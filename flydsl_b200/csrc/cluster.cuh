// Thread-block-cluster helpers shared by the split-K kernels: cluster rank, cluster barrier, address
// mapping into another CTA's shared memory, bulk copy between CTAs' shared memories.
#pragma once
#include "common.cuh"

namespace flyb200 {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
// The two halves of cluster_sync_all, for work that fits between them.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// Bulk copy from this CTA's shared memory into the shared memory of a CTA of the cluster; the bytes
// are counted on an mbarrier of the destination CTA. (A copy engine transfer: no per-thread DSMEM
// stores, whose throughput is a few cycles per 4-byte access.)
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_local,
                                                 uint32_t bytes, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_cluster),
      "r"(src_local), "r"(bytes), "r"(bar_cluster)
      : "memory");
}

}  // namespace flyb200
