// Thin wrappers over the Blackwell tensor-core PTX used by the grouped GEMM: tensor memory
// allocation, UMMA shared-memory / instruction descriptors, tcgen05.mma issue and commit,
// tensor-memory loads, and 2-D TMA tile loads (never multicast).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../a2a/ptx.cuh"

namespace pplx::tc {

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               :
               : "r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" : : "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_thread_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_thread_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ----
// K-major operand tile in shared memory with the 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart (what a TMA box of 128-byte rows with SWIZZLE_128B writes).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(const void* smem_tile) {
  const uint32_t addr = smem_u32(smem_tile);
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);   // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                // leading byte offset (unused with swizzle): 1
  d |= static_cast<uint64_t>(1024 >> 4) << 32;        // stride byte offset: 8 rows x 128 B
  d |= static_cast<uint64_t>(1) << 46;                // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor of kind::f8f6f4, e4m3 x e4m3 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_e4m3_f32(int m, int n) {
  return (1u << 4)                               // D format f32
         | (0u << 7) | (0u << 10)                // A, B format e4m3
         | (0u << 15) | (0u << 16)               // A, B K-major
         | (static_cast<uint32_t>(n >> 3) << 17) // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);// M / 16
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void mma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               :
               : "r"(smem_u32(bar))
               : "memory");
}

// ---- TMA ----
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" : : "l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" : : "r"(smem_u32(bar)) : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of one cluster, ranks 2i and 2i+1, work on one MMA ----
// The even CTA (the leader) issues the MMAs; each CTA holds its 128 rows of A, its half of B's
// rows, and its 128 rows of the accumulator in its own tensor memory.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `smem_ptr`'s counterpart in the shared memory of CTA `rank` of this cluster, for
// instructions that take a .shared::cluster address.
__device__ __forceinline__ uint32_t map_to_cta(const void* smem_ptr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(smem_ptr)), "r"(rank));
  return out;
}
// All threads of all CTAs of the cluster. Not bounded: every thread must get here on every path.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Executed by one warp in EACH CTA of the pair (as CUTLASS does in its 2-SM kernels).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               :
               : "r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" : : "r"(taddr), "r"(ncols) : "memory");
}
// 2-D tile load into this CTA's shared memory whose bytes are counted on the mbarrier at the
// .shared::cluster address `bar_cluster_addr` (the leader's). No multicast: each CTA loads its own.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// D[tmem of both CTAs] (+)= A * B^T over the pair: M 256 (128 rows per CTA), B's N rows split in
// halves between the CTAs. Issued by one thread of the leader; the descriptors are the leader's
// shared-memory addresses, which the peer mirrors.
__device__ __forceinline__ void mma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives on the mbarrier at `bar`'s offset in every CTA of `cta_mask` once the pair's MMAs issued
// so far have completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      :
      : "r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}
// Arrive on an mbarrier given by a .shared::cluster address (this CTA's or a peer's). Default
// semantics on purpose: a cluster-scope release would first drain every global store this thread
// has in flight, and the tensor-memory reads that the arrival publishes are ordered by
// tcgen05.fence::before_thread_sync, not by the memory model's release.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" : : "r"(bar_cluster_addr) : "memory");
}

// ---- block-scaled MMA (kind::mxf8f6f4.block_scale): one UE8M0 scale per operand row and 32
// elements of K, applied inside the tensor core. The scales live in tensor memory: 32 lanes x one
// 32-bit column hold the scales of 32 rows (row r of a 128-row block -> lane r % 32, column r / 32),
// repeated in each of the four lane quarters; the four bytes of a word are four scales along K,
// and the instruction descriptor's scale-factor id says which byte this MMA uses.

// Instruction descriptor: e4m3 x e4m3 -> f32, both K-major, UE8M0 scales; `sf_id` selects the
// byte of the scale words for A and for B.
__host__ __device__ constexpr uint32_t idesc_mx_e4m3_ue8m0(int m, int n, uint32_t sf_id = 0) {
  return (sf_id << 4)                              // B scale-factor id
         | (0u << 7) | (0u << 10)                  // A, B format e4m3
         | (0u << 15) | (0u << 16)                 // A, B K-major
         | (static_cast<uint32_t>(n >> 3) << 17)   // N / 8
         | (1u << 23)                              // scale format UE8M0
         | (static_cast<uint32_t>(m >> 4) << 24)   // M / 16
         | (sf_id << 29);                          // A scale-factor id
}

// Shared-memory descriptor of a block of scale words laid out for tcgen05.cp 32x128b: 32 rows of
// 16 bytes, rows 16 bytes apart (K-major, no swizzle: 8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_sf(const void* smem_block) {
  const uint32_t addr = smem_u32(smem_block);
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(128 >> 4) << 32;         // stride byte offset: 8 rows x 16 B
  d |= static_cast<uint64_t>(1) << 46;                // descriptor version (Blackwell)
  return d;
}

// Copies 32 rows x 16 bytes from shared memory into 4 tensor-memory columns of all four lane
// quarters (what the block-scaled MMA reads its scales from). Asynchronous, ordered with the
// tcgen05.mma and tcgen05.commit instructions of the issuing thread. With kCtas == 2 the copy
// happens in both CTAs of the pair, each from its own shared memory at the same offset.
template <int kCtas>
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  if constexpr (kCtas == 2) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" : : "r"(taddr), "l"(sdesc) : "memory");
  } else {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" : : "r"(taddr), "l"(sdesc) : "memory");
  }
}

// D[tmem] (+)= (A * 2^sfa) (B * 2^sfb)^T, one thread issues. M 128 (one CTA) or 256 (a pair).
template <int kCtas>
__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (kCtas == 2) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
  }
}

// Arrival that publishes this thread's earlier shared-memory writes to the other CTA of the
// cluster (cluster-scope release), and the matching bounded wait (cluster-scope acquire).
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" : : "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_timed_acquire_cluster(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
  if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
  const long long start = clock64();
  const long long limit = static_cast<long long>(timeout_ns) * 2;
  for (;;) {
    #pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
    }
    if (clock64() - start > limit) return false;
  }
}

}  // namespace pplx::tc
