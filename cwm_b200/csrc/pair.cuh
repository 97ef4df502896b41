// Inline-PTX wrappers for kernels that run as clusters of two CTAs on neighbouring
// SMs and drive both tensor cores with one instruction stream (tcgen05 with
// cta_group::2): cluster rank and barrier, mbarrier operations on the partner's
// shared memory, TMA loads that report to the leader's mbarrier, paired tensor
// memory allocation, and the paired forms of tcgen05.mma / tcgen05.commit.
//
// In a pair, CTA rank 0 (the leader) issues every tcgen05.mma.  An instruction of
// shape M=256 x N computes rows 0-127 on the leader's SM (its TMEM lanes) and rows
// 128-255 on the partner's; each CTA supplies its own 128 rows of A (shared memory
// or TMEM, at the same address in both CTAs) and one half of the N extent of B
// from its own shared memory (rank 0 the first N/2 columns), so every B byte is
// read from shared memory once per pair instead of once per SM.
#pragma once

#include "common.cuh"

namespace cwm {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// All threads of all CTAs of the cluster; orders shared-memory writes (mbarrier
// initialisation included) before anything a partner does after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of `smem_addr` (a shared::cta address of this CTA) in CTA `rank` of the
// cluster, as a shared::cluster address.
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

// One arrival on an mbarrier of any CTA of the cluster (shared::cluster address).
// Release at CTA scope only: what the arrival hands over is tensor-memory data, which
// is ordered by tcgen05.wait / tcgen05.fence on both sides, not by the memory model's
// fences.  A cluster-scope release costs a full memory barrier (more than a thousand
// cycles on a busy SM) per arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Wait for arrivals that may come from the partner CTA (mbar_arrive_cluster()).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity,
                                                          long long limit) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait_cluster(bar, parity)) return true;
    }
    if (clock64() - t0 > limit) return false;
  }
}

// 2-D TMA tile load into this CTA's shared memory whose byte count is reported to
// an mbarrier of the pair's leader (`bar_cluster_addr` from cluster_map(.., 0)).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x,
                                                 int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}

namespace tc05 {

// ---- paired TMEM allocation: the same warp index of both CTAs executes these, with
// the same shared-memory slot offset; both CTAs get the same column range.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// The issuing warp runs its loop with all lanes (so that addresses and descriptors stay
// warp-uniform values) and one elected lane executes each tcgen05 instruction; the
// election picks the same lane every time, which keeps the instructions of one warp in
// issue order.
//
// One arrival on the mbarrier at this shared-memory offset in every CTA of
// `cta_mask`, when all tcgen05.mma issued so far by the elected lane have completed.
__device__ __forceinline__ void commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;\n\t}" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// A shared-memory matrix descriptor as its two 32-bit words: the start address is the
// low 14 bits of the low word in units of 16 bytes, so a loop steps it with one add.
struct Desc2 {
  uint32_t lo, hi;
};
__device__ __forceinline__ Desc2 split_desc(uint64_t d) {
  return Desc2{static_cast<uint32_t>(d), static_cast<uint32_t>(d >> 32)};
}

// The eight K=16 steps of one 128-deep product as a single block: one election, the
// descriptor start addresses stepped in place.  The issuing warp spends a few
// instructions per tcgen05.mma instead of an election, a predicate and two 64-bit
// moves each, which matters because every step keeps the tensor cores busy for only
// 64 cycles and the warp shares its scheduler with two softmax warps.
//
// D[tmem, both CTAs] (+)= A[smem, 128 rows per CTA] * B[smem, N/2 columns per CTA].
// A and B tiles are two 64-element halves of the K extent (128-byte swizzled rows);
// kAHalf / kBHalf = distance between the halves in 16-byte units.  Within a half the
// K=16 steps are 32 bytes (2 units) apart.
#define CWM_SS_NEXT(ainc, binc)                                                        \
  "add.u32 ra, ra, " ainc ";\n\tadd.u32 rb, rb, " binc ";\n\t"                         \
  "mov.b64 da, {ra, %2};\n\tmov.b64 db, {rb, %4};\n\t"                                 \
  "@e tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, t;\n\t"
template <uint32_t kAHalf, uint32_t kBHalf>
__device__ __forceinline__ void mma_ss_pair_x8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred e, t;\n\t.reg .b64 da, db;\n\t.reg .b32 ra, rb;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 t, %6, 0;\n\t"
      "mov.b32 ra, %1;\n\tmov.b32 rb, %3;\n\t"
      "mov.b64 da, {ra, %2};\n\tmov.b64 db, {rb, %4};\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, t;\n\t"
      "setp.eq.b32 t, %2, %2;\n\t"
      CWM_SS_NEXT("2", "2") CWM_SS_NEXT("2", "2") CWM_SS_NEXT("2", "2")
      CWM_SS_NEXT("%7", "%8")
      CWM_SS_NEXT("2", "2") CWM_SS_NEXT("2", "2") CWM_SS_NEXT("2", "2")
      "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate_first),
      "n"(kAHalf - 6), "n"(kBHalf - 6)
      : "memory");
}
#undef CWM_SS_NEXT

// The same for D[tmem] (+)= A[tmem, 128 rows per CTA] * B[smem, N/2 columns per CTA]: A advances by kAStep columns of tensor
// memory per step, B by kBStep units of 16 bytes.
#define CWM_TS_NEXT                                                                    \
  "add.u32 ra, ra, %6;\n\tadd.u32 rb, rb, %7;\n\tmov.b64 db, {rb, %3};\n\t"            \
  "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, t;\n\t"
template <uint32_t kAStep, uint32_t kBStep>
__device__ __forceinline__ void mma_ts_pair_x8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred e, t;\n\t.reg .b64 db;\n\t.reg .b32 ra, rb;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 t, %5, 0;\n\t"
      "mov.b32 ra, %1;\n\tmov.b32 rb, %2;\n\t"
      "mov.b64 db, {rb, %3};\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, t;\n\t"
      "setp.eq.b32 t, %3, %3;\n\t"
      CWM_TS_NEXT CWM_TS_NEXT CWM_TS_NEXT CWM_TS_NEXT CWM_TS_NEXT CWM_TS_NEXT CWM_TS_NEXT
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate_first), "n"(kAStep),
      "n"(kBStep)
      : "memory");
}
#undef CWM_TS_NEXT

}  // namespace tc05
}  // namespace cwm
