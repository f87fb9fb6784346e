// Inline-PTX building blocks for the sm_100a kernels: mbarriers with bounded waits,
// TMA tile loads, shared-memory / instruction descriptors, tcgen05.mma / commit / ld.
#pragma once

#include "common.cuh"

namespace tc05 {

constexpr long long WAIT_BUDGET_CYCLES = 2000000000ll;  // ~1 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  // The last operand is a suspend-time hint in nanoseconds: the thread may sleep in
  // hardware until the phase completes or the hint expires, instead of burning issue
  // slots that the compute warps on the same scheduler need.
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(20000u)
      : "memory");
  return ok;
}

// Non-blocking test of the phase: for hand-offs that sit on a kernel's critical chain,
// where the wake-up delay of a suspended try_wait costs more than the polling does.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false when the wait gave up or another role already
// flagged an abort; the caller then leaves its loop.  SPIN polls instead of suspending.
// `budget` is the clock64 allowance (the kernels use WAIT_BUDGET_CYCLES; the wait self-test
// a millisecond's worth).
template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* err, uint32_t where,
                                          long long budget = WAIT_BUDGET_CYCLES) {
  if (SPIN ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (SPIN ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget) {
        *abort_flag = 1u;
        if (atomicCAS(err, 0u, VKG_ERR_WAIT_TIMEOUT) == 0u) err[1] = where;
        __threadfence_system();
        return false;
      }
    }
  }
}

// The same wait for a whole warp that goes on to a .sync.aligned instruction (tcgen05.ld) or
// a __syncwarp: all 32 lanes must call it.  Each lane polls on its own, then the warp votes, so
// either every lane carries on or every lane leaves -- a lane that ran out of budget at the
// very moment the phase completed for its neighbours cannot strand them in the aligned
// instruction that follows.
template <bool SPIN = false>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               uint32_t* err, uint32_t where,
                                               long long budget = WAIT_BUDGET_CYCLES) {
  const bool ok = mbar_wait<SPIN>(bar, parity, abort_flag, err, where, budget);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// Start fetching a tensor map (a kernel parameter) so the first TMA load does not wait for it.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version field.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// The same descriptor as two 32-bit halves.  The high word (stride between 8-row groups,
// version, swizzle) is constant per operand; the low word carries the start address (>> 4) and
// the leading-dimension offset, so stepping along K or to the next ring stage is ONE integer
// add on it.  The thread that issues tcgen05.mma is a single lane with nothing to hide its
// latencies behind: a descriptor rebuilt from shifts and masks per instruction costs that lane
// about 125 cycles per MMA, more than an N <= 128 instruction takes on the tensor core.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint32_t smem_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint64_t smem_desc_pack(uint32_t lo, uint32_t hi) {
  return ((uint64_t)hi << 32) | (uint64_t)lo;
}

// True in exactly one lane of a CONVERGED warp (all 32 lanes must execute it).  The warp that
// issues tcgen05.mma runs its loop converged and guards only the instruction itself with this:
// descriptors and loop state then live in uniform registers.  Issued instead from a branch only
// lane 0 takes, every operand is moved from a vector register per instruction, and with the
// schedulers busy (sixteen arithmetic-bound warps) sixteen N = 64 instructions took 1320 cycles
// against 800 for the converged form and 770 for the tensor core alone.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// NK instructions along K into one accumulator, called by a converged warp (one elected lane
// issues): the operands' descriptor low words advance by a_step / b_step (units of 16 bytes)
// per instruction, `hi` is their common high word; the first instruction overwrites the
// accumulator unless acc_first is set.
template <int NK>
__device__ __forceinline__ void umma_f16_chain(uint32_t tmem_d, uint32_t a_lo, uint32_t a_step,
                                               uint32_t b_lo, uint32_t b_step, uint32_t hi,
                                               uint32_t idesc, uint32_t acc_first) {
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (elect_one())
      umma_f16(tmem_d, smem_desc_pack(a_lo + k * a_step, hi), smem_desc_pack(b_lo + k * b_step, hi), idesc,
               k ? 1u : acc_first);
}

// The same instruction with the A operand in tensor memory: lane = row of A, two consecutive K
// elements of a 16-bit type per 32-bit column (even K in the low half), so one K = 16 step
// reads 8 columns.  A operand written there with tcgen05.st never passes through shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// NK such instructions along K: A advances 8 columns, B's descriptor low word by b_step.
template <int NK>
__device__ __forceinline__ void umma_f16_ts_chain(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo,
                                                  uint32_t b_step, uint32_t hi, uint32_t idesc,
                                                  uint32_t acc_first) {
#pragma unroll
  for (int k = 0; k < NK; ++k)
    if (elect_one())
      umma_f16_ts(tmem_d, tmem_a + 8 * k, smem_desc_pack(b_lo + k * b_step, hi), idesc, k ? 1u : acc_first);
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// the commit from a converged warp: one elected lane issues it
__device__ __forceinline__ void umma_commit_one(uint32_t bar) {
  if (elect_one()) umma_commit(bar);
}

// ---- CTA pairs (cta_group::2): one thread of the even-ranked CTA issues an MMA that spans
// the tensor cores, shared memory and TMEM of both CTAs of a 2-CTA cluster --------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// arrive on an mbarrier of another CTA of the cluster (address from mapa_shared)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

// Tile load whose completion bytes are counted on an mbarrier that may live in the peer CTA
// of the pair (bar is a shared::cluster address); the data lands in this CTA's shared memory.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// arrives on the mbarrier at this shared-memory offset in both CTAs of the pair once the
// MMAs issued so far have retired
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// registers -> TMEM, the mirror of tmem_ld16 (lane = TMEM lane, 16 consecutive columns)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}


__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"((uint64_t)map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// Tile store, shared memory -> global through the tensor map (no multicast): the box is
// clipped at the tensor's edges, so ragged last tiles need no predicates.  The copy joins
// the issuing thread's current bulk async-group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"((uint64_t)map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the issuing thread's bulk stores have finished READING shared memory (it may be reused);
// their global writes complete on their own, at the latest when the kernel ends
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA) that reads them next
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(volatile uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32((const void*)slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Instruction descriptor for kind::f16: fp32 accumulate, M = 128.
__host__ __device__ inline uint32_t make_idesc(int bf16, int a_mn, int b_mn, int n) {
  const uint32_t fmt = bf16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

}  // namespace tc05
