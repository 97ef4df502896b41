// Argument blocks and launch entry points shared by the attention kernels.
#pragma once

#include <math.h>

#include "common.cuh"

namespace cwm {

constexpr int kHeadDim = 128;
// Upper bound on the persistent decode grid; sizes the split-KV workspace.
constexpr int kMaxDecodeCtas = 1024;

// Everything the attention kernels read besides the K/V tensor maps.
struct AttnArgs {
  const void* q;               // [total_q, hq, 128]
  void* out;                   // [total_q, hq, 128]
  float* lse;                  // [hq, total_q] or null
  const int32_t* cu_q;         // [batch + 1]
  const int32_t* seq_k;        // [batch]
  const int32_t* block_table;  // [batch, *], row stride bt_stride
  int batch;
  int hq;
  int hkv;
  int group;  // hq / hkv
  int page_size;
  int max_seqlen_q;
  int max_seqlen_k;
  long long num_pages;
  long long bt_stride;
  long long total_q;
  float scale_log2;  // softmax_scale * log2(e)
  int window_left;   // < 0: unbounded
  int* counters;     // workspace: int[batch * hkv], arrivals per (sequence, KV head); all zero
                     // between launches
  float* partial;    // workspace: split-KV partial states
  int* status;       // device status word
  long long wait_cycles;  // limit of every bounded wait, in SM clock cycles
  int decode_launched;    // the decode kernel runs in this call (prefill kernel: cross-check)
  int test_drop_last;     // self-test only: each producer withholds its last tile's loads
};
using DecodeArgs = AttnArgs;

// Split-KV workspace: two partial states per CTA (a size that depends on max_ctas
// only) followed by the arrival counters (one per sequence and KV head).  The
// counters must be zero when a launch starts; every launch leaves them zero again.
size_t decode_workspace_bytes(int batch, int hkv);
// max_ctas caps the persistent grid (the workspace holds two partials per CTA).
int launch_decode(const CUtensorMap& kmap, const CUtensorMap& vmap, AttnArgs a, bool bf16,
                  void* workspace, cudaStream_t stream, int max_ctas = kMaxDecodeCtas);
// Workspace bytes for a decode grid of at most max_ctas CTAs.
size_t decode_workspace_bytes_for(int batch, int hkv, int max_ctas);
// Bytes of the arrival counters, which start decode_partial_bytes(max_ctas) into the
// workspace.
size_t decode_counter_bytes(int batch, int hkv);
size_t decode_partial_bytes(int max_ctas);
// Values of the self-test hooks (cwm_test_hooks) for the next launches.
long long hook_wait_cycles();
int hook_drop_last_tile();
int launch_prefill(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                   AttnArgs a, bool bf16, cudaStream_t stream);

// mma.sync m16n8k16 where only rows 0..7 of the accumulator are kept: the two
// values of rows 8..15 go to scratch registers and enter as zero, so that
// independent products do not chain through them.
template <bool kBf16>
__device__ __forceinline__ void mma_16816_top(float (&c)[2], const uint32_t (&a)[4], uint32_t b0,
                                              uint32_t b1) {
  float j0, j1;
  if constexpr (kBf16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%10,%10};"
        : "+f"(c[0]), "+f"(c[1]), "=f"(j0), "=f"(j1)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%10,%10};"
        : "+f"(c[0]), "+f"(c[1]), "=f"(j0), "=f"(j1)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
  }
}

}  // namespace cwm
