// Memory-model and data-movement primitives used by the all-to-all kernels.
//
// Every cross-GPU handshake in this library is built from three things only:
//   * plain 16-byte stores to a peer mapping (payload),
//   * a release-scoped system-wide reduction on a flag word (arrival signal),
//   * an acquire-scoped system-wide load on the local copy of that flag (wait).
// The reference keeps the same vocabulary in
// p2p-all-to-all/a2a-kernels/src/core/memory.cuh:7-157; the MMIO host flags it
// also needs are absent here because no CPU proxy takes part in the protocol.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace pplx {

struct alignas(16) Vec16 {
  uint32_t x, y, z, w;
};

// Read-only input that no kernel in flight writes (user tensors): non-coherent
// path, do not pollute L1.
__device__ __forceinline__ Vec16 ld_input_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Data that a peer GPU wrote during this kernel's lifetime and that was made
// visible through an acquire: coherent (weak) load that skips L1 allocation.
__device__ __forceinline__ Vec16 ld_stream_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ void st_stream_v4(void* p, const Vec16& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
               :
               : "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void st_stream_u32(void* p, uint32_t v) {
  asm volatile("st.global.L1::no_allocate.u32 [%0], %1;" : : "l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" : : "l"(p), "r"(v) : "memory");
}

// Fire-and-forget arrival signal: orders every earlier write that this thread
// observed (its own and, through a preceding bar.sync, its block's) before the
// increment becomes visible anywhere in the system.
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" : : "l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t atom_acq_rel_gpu_add(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
               : "=r"(old)
               : "l"(p), "r"(v)
               : "memory");
  return old;
}

__device__ __forceinline__ uint32_t atom_relaxed_gpu_add(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.relaxed.gpu.global.add.u32 %0, [%1], %2;"
               : "=r"(old)
               : "l"(p), "r"(v)
               : "memory");
  return old;
}

__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Named barrier over `nthreads` threads (multiple of 32). Id 0 is __syncthreads.
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" : : "r"(id), "r"(nthreads) : "memory");
}

// Named barrier that also ORs a predicate over its participants; every thread gets the result.
__device__ __forceinline__ bool bar_red_or(int id, int nthreads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 p, %3, 0;\n"
      "bar.red.or.pred q, %1, %2, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(out)
      : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred;
}

// ---------------------------------------------------------------------------
// Bulk asynchronous copies (TMA engine, no tensor map, never multicast).
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" : : "r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
               :
               : "r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase. Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  uint32_t max_polls = (1u << 22)) {
  for (uint32_t i = 0; i < max_polls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Wait on an mbarrier phase for at most about `timeout_ns`. Returns false when the time ran
// out (the caller reports the failure and unwinds; it never spins forever). Time is taken
// from the SM's cycle counter (reading %globaltimer costs hundreds of cycles and would sit on
// the critical path of every wait that is not satisfied at once); 2 cycles per ns is an upper
// bound on the clock, so the real limit is at least `timeout_ns`.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  const long long limit = static_cast<long long>(timeout_ns) * 2;
  for (;;) {
    #pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (clock64() - start > limit) return false;
  }
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// global -> shared bulk copy; bytes and both addresses are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// shared -> global bulk store (the destination may be a peer mapping).
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               :
               : "l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until the smem sources of all committed bulk stores may be reused.
__device__ __forceinline__ void bulk_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Wait until all committed bulk stores are complete (writes performed).
__device__ __forceinline__ void bulk_wait0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

}  // namespace pplx
