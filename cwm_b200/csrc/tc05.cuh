// Inline-PTX wrappers for the 5th-generation tensor core path of sm_100a: fences and
// waits of the tcgen05 family, shared-memory matrix descriptors, the instruction
// descriptor, and TMEM <-> register moves.  Allocation, tcgen05.mma and tcgen05.commit
// in their two-CTA forms are in pair.cuh.
#pragma once

#include "common.cuh"

namespace cwm {
namespace tc05 {

__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, for tiles written by TMA as
// rows of 128 bytes (8-row groups 1024 bytes apart, tile base 1024-aligned).
// K-major: the 128-byte row runs along K (Q and K tiles of S = Q K^T).
__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) /* LBO (unused) */ |
         (64ull << 32) /* SBO = 1024 B */ | (1ull << 46) /* descriptor version */ |
         (2ull << 61) /* SWIZZLE_128B */;
}
// MN-major: the 128-byte row runs along N (V tile of O = P V: rows are tokens = K,
// 64 head-dim elements per row; the next 64 elements live lbo_bytes further).
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) |
         (static_cast<uint64_t>(lbo_bytes >> 4) << 16) | (64ull << 32) /* SBO = 1024 B */ |
         (1ull << 46) | (2ull << 61);
}

// Instruction descriptor for kind::f16: fp32 accumulate, 16-bit A and B.
// ab_format: 0 = fp16, 1 = bf16.  b_mn_major: B is MN-major in shared memory.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int ab_format, bool b_mn_major) {
  return (1u << 4) /* D = f32 */ | (static_cast<uint32_t>(ab_format) << 7) |
         (static_cast<uint32_t>(ab_format) << 10) | (b_mn_major ? (1u << 16) : 0u) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- TMEM <-> registers: lane = thread of the warp, 32 / 16 consecutive columns ----
__device__ __forceinline__ void ld32(uint32_t (&r)[32], uint32_t taddr) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void ld8(uint32_t (&r)[8], uint32_t taddr) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(
                   taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ void st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

}  // namespace tc05
}  // namespace cwm
