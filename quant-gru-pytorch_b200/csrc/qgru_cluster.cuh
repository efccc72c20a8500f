// qgru_cluster.cuh - inline-PTX helpers of the cluster recurrence kernels: cluster barrier,
// distributed-shared-memory addressing, the asynchronous remote store that counts its bytes on
// the receiver's mbarrier, and the byte offset of an element in a 128-byte-swizzled operand tile.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace qgru {
namespace clu {

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// 32-bit store into a peer CTA's shared memory that counts its 4 bytes on the peer's mbarrier when
// it lands: no fence and no acknowledgement on the sending side
__device__ __forceinline__ void st_async_u32(uint32_t peer_addr, uint32_t v, uint32_t peer_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(peer_addr),
                 "r"(v), "r"(peer_bar)
                 : "memory");
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_cta() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Byte offset of element (row b, byte k) inside a K-major tile of `rows` rows stored as 128-byte
// rows with the 128-byte swizzle: slabs of 128 K-bytes follow each other; inside a slab, groups
// of 8 rows take 1024 bytes and the 16-byte chunk index is XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t sw128_offset(int b, int k, int rows) {
    return (uint32_t)((k >> 7) * rows * 128 + (b >> 3) * 1024 + (b & 7) * 128 +
                      ((((k & 127) >> 4) ^ (b & 7)) << 4) + (k & 15));
}

}  // namespace clu
}  // namespace qgru
