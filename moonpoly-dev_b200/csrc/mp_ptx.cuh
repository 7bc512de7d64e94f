// Thin inline-PTX layer for sm_100a: mbarrier, TMA (non-multicast), tcgen05 / TMEM.
// Every wait in this file is bounded: after a wall-clock limit (or as soon as another
// thread has published an error) the wait gives up, records a code in the launch's
// status word and returns false, so a kernel can never spin forever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mp {

// Device-side status codes written to the status word (0 = ok).
enum : int {
  MP_DEV_OK = 0,
  MP_DEV_TIMEOUT_PRODUCER = 101,   // TMA producer waited too long for a free stage
  MP_DEV_TIMEOUT_MMA_FULL = 102,   // MMA issuer waited too long for a filled stage
  MP_DEV_TIMEOUT_MMA_TMEM = 103,   // MMA issuer waited too long for a drained accumulator
  MP_DEV_TIMEOUT_EPILOGUE = 104,   // epilogue waited too long for a finished accumulator
  MP_DEV_TIMEOUT_DRAIN = 105,      // teardown waited too long for copies in flight
  MP_DEV_BAD_CONFIG = 106,
  MP_DEV_TIMEOUT_CLUSTER = 107,    // a CTA waited too long for the other K slices of its thread-block cluster
  MP_DEV_TIMEOUT_PEER = 108,       // the cross-GPU flag barrier waited too long for another rank
};

static constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  Returns true when the phase with `parity` has completed.  Gives up (false)
// when the limit expires or when `*status` is already non-zero (another role failed); the first
// waiter to give up records `code`.  With status == nullptr only the time limit applies and
// nothing is recorded (used while draining copies in flight after an error).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xffu) == 0) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
      if (now - t0 > kWaitLimitNs) {
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// Short bounded wait until a global counter reaches `target` (acquire semantics); running out of
// time is not an error here, the caller just carries on without what it waited for.
constexpr unsigned long long kHelpWaitNs = 50000ull;
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool counter_wait_ge_for(const unsigned* ctr, unsigned target, unsigned long long limit_ns) {
  if (ld_acquire_u32(ctr) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (ld_acquire_u32(ctr) >= target) return true;
    if (globaltimer_ns() - t0 > limit_ns) return false;
  }
}

// ----------------------------------------------------------------------------- thread-block cluster
// Distributed shared memory between the CTAs of a cluster: plain loads from a peer's shared memory and
// mbarrier arrivals on a peer's barrier.  No load here is a TMA / bulk copy and none uses multicast.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `addr` in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrive on a barrier in any CTA of the cluster; release at cluster scope publishes this thread's earlier
// shared-memory writes (and, after a __syncwarp, its warp's) to whoever acquires the barrier.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}
// Bounded wait with acquire at cluster scope (same contract as mbar_wait).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  unsigned long long t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((it & 0xffu) == 0) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
      if (now - t0 > kWaitLimitNs) {
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ uint4 ld_dsmem_v4(uint32_t cluster_addr) {
  uint4 v;
  asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_smem_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// All threads of all CTAs of the cluster (must be reached by every thread, warps converged).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// 2-D tiled load, no multicast: global (c0 = innermost coordinate, c1 = row) -> this CTA's smem.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// 3-D tiled load, no multicast.  Used with the operand viewed as [K/kb][rows][kb elements]: one
// instruction then brings `kc` consecutive 128-byte K blocks of every row (kc * 128 contiguous
// bytes per row), which the TMA unit moves far faster than kc separate 128-byte-wide boxes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* tm, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// L2 prefetch of a box (no shared-memory destination, no barrier).  Harmless to issue for data
// another kernel may still overwrite: L2 is the point of coherence, a later write updates the line.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* tm, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* tm, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16 covers fp16/bf16 inputs with fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::i8: int8 x int8 -> int32 accumulate.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows of exactly 128 bytes,
// 8-row swizzle atoms 1024 bytes apart.  `saddr` must lie inside a 1024-byte-aligned tile; the
// K offset inside the 128-byte row is carried by the start address.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);        // start address      bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused, =1)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset  bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version 1 (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                        // layout type: SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 / kind::i8, both operands K-major, dense.
//   c_format: 1 = f32, 2 = s32;  ab_format: f16 kinds 0 = f16, 1 = bf16; i8 kind 1 = signed 8 bit.
__host__ __device__ __forceinline__ uint32_t umma_idesc(uint32_t c_format, uint32_t ab_format, uint32_t m,
                                                        uint32_t n) {
  return (c_format << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// TMEM -> registers: this warp's 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace mp
