// Chunked-prefill paged GQA attention on the sm_100a tensor cores, as a persistent
// grid of clusters of two CTAs that share every K and V tile (tcgen05.mma with
// cta_group::2).
//
// A work item is two query tiles of 128 rows that read the same KV head: the same
// 128 queries of two neighbouring query heads when the GQA group size is even,
// otherwise two consecutive 128-row blocks of one head.  One pair of CTAs on
// neighbouring SMs per two SMs of the GPU walks the list of items (heaviest query
// blocks first, the head pairs of a block on neighbouring clusters so that they meet
// in L2), and every ring below runs on across items: while the softmax warps finish
// an item and write its output, the copy warp is already fetching the next item's Q,
// K and V and the tensor cores compute its first scores.  Each CTA keeps its own
// query tile, loads one half of every 128-token K tile (64 keys) and one half of every
// V tile (64 of the 128 head-dim columns), and the leader CTA issues M=256
// instructions that compute both CTAs' rows while every K / V byte is read from
// shared memory once per pair.  Per CTA:
//   warp 0      TMA producer: the query tile of an item (two buffers), K halves and V
//               halves (4-stage rings) through the block table; byte counts are
//               reported to the leader's mbarriers
//   warp 1      leader only: issues O += P V (P read from tensor memory)
//   warp 2      leader only: issues S = Q K^T into one of two score slots in tensor
//               memory; completion of every product is multicast to both CTAs'
//               mbarriers with tcgen05.commit
//   warps 4-7   softmax of the even KV tiles   thread = query row; the two groups
//   warps 8-11  softmax of the odd KV tiles    work on different KV tiles of the
//               same rows at the same time and hand the running maximum of each
//               row to one another through shared memory.  A group takes the 128
//               scores of its row into registers and at once gives the score slot
//               back, so the next scores of that slot are computed while it works;
//               P (16-bit) goes to a buffer of its own; O is rescaled only when the
//               maximum grew by more than 2^8 (after waiting for the products
//               issued so far).
// (KV tiles are counted across items: "even" and "odd" refer to that count.)
// TMEM (512 columns per CTA): score slots at 0 and 128; P buffers at 256 and 320;
// O at 384.  KV tiles wholly above the causal diagonal or wholly left of the sliding
// window of both query tiles are never loaded; only edge tiles are masked.
// Every mbarrier wait is bounded.  Needs no scratch memory.
#include <atomic>
#include <type_traits>

#include "attn_common.cuh"
#include "pair.cuh"
#include "tc05.cuh"

namespace cwm {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kSlots = 2;        // score slots, one per softmax group
constexpr uint32_t kPCol = 256;  // two P buffers of 64 columns (16-bit pairs), one per group
// "S of tile g has completed" (barrier g % 4) both hands the scores to the softmax and
// frees K stage g % 4; "P V of tile g has completed" frees V stage g % 4 and the P
// buffer g % 2: one tcgen05.commit per product.
constexpr int kKStages = 4;
constexpr int kVStages = 4;
constexpr int kThreadsPair = 384;
constexpr int kQBytes = 128 * 256;  // [2 halves of 64 elements][128 rows][128 B]
constexpr int kQHalf = 128 * 128;
constexpr int kKBytes = 64 * 256;   // this CTA's 64 keys: [2 halves of 64 elements][64 rows][128 B]
constexpr int kKHalf = 64 * 128;
constexpr int kVBytes = 128 * 128;  // this CTA's 64 head-dim columns: [128 keys][128 B]
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kOCol = 384;
constexpr float kRescaleThreshold = 8.f;  // log2 domain
// Of every four pairs of scores, this many take the polynomial exp2.
constexpr int kPolyPairsOfFour = 1;
// Registers per thread after the roles split (launched with 168 x 384 threads):
// 128 x 56 + 256 x 224 = 64512.
constexpr int kRegsIssue = 56;
constexpr int kRegsSoftmax = 224;
constexpr uint16_t kBothCtas = 3;
constexpr int kPvBars = kVStages;

struct PairBars {
  uint64_t q_full[2];                           // leader: both query tiles of an item landed
  uint64_t q_free[2];                           // both CTAs: every S of the item has completed
  uint64_t k_full[kKStages], v_full[kVStages];  // leader: both halves landed
  uint64_t s_full[kKStages];  // both CTAs (multicast commit): S of tile g on bar g % 4
  uint64_t s_free[kSlots];    // leader: the scores of a tile are in registers (8 warps)
  uint64_t pv_done[kPvBars];  // both CTAs (multicast commit): P V of tile g on bar g % 4
  // leader: P of tile g is complete, on barrier g % 4; one arrival per softmax warp of
  // the group that took the tile, both CTAs.  Four barriers, not one per group: a warp
  // may finish tile g + 2 before a slower warp of its group has finished tile g, and
  // its second arrival must not count for tile g.  Tile g + 4 cannot be reached before
  // P V of tile g + 1 has been issued, which is after every arrival for tile g.
  uint64_t p_full[4];
  uint64_t o_free;  // leader: the output of an item has been read (16 warps)
};

struct QTile {
  int head;  // query head
  int r0;    // first query row within the sequence
  int lo;    // first KV tile
  int hi;    // last KV tile (hi < lo: nothing visible)
};

// One work item as every warp role needs it.
struct Item {
  int b;        // sequence
  int q0;       // first query row of the sequence in the packed query tensor
  int t;        // queries of the sequence in this call
  int n;        // keys of the sequence
  int pos0;     // position of query row 0
  int kv_head;
  int lo;       // first KV tile of the union of the two query tiles' ranges
  int n_tiles;  // <= 0: nothing visible for either tile
  QTile my;     // this CTA's query tile
};

__device__ __forceinline__ bool visible(int key, int pos, int window_left) {
  return key <= pos && (window_left < 0 || key >= pos - window_left);
}

// Item `item` of the list: query blocks from the heaviest (last) to the lightest, all
// head units of a block next to one another.
__device__ __forceinline__ Item make_item(const AttnArgs& a, const int* blk_prefix, int item,
                                          int total_units, int head_units, int pair_heads,
                                          int rank) {
  Item it;
  const int unit = total_units - 1 - item / head_units;
  const int head_unit = item % head_units;
  int lo_b = 0, hi_b = a.batch;
  while (hi_b - lo_b > 1) {
    const int mid = (lo_b + hi_b) >> 1;
    if (blk_prefix[mid] <= unit) lo_b = mid; else hi_b = mid;
  }
  it.b = lo_b;
  it.q0 = a.cu_q[it.b];
  it.t = a.cu_q[it.b + 1] - it.q0;
  int n = a.seq_k[it.b];
  it.n = n > a.max_seqlen_k ? a.max_seqlen_k : n;
  it.pos0 = it.n - it.t;
  const int unit_rows = pair_heads ? kBM : 2 * kBM;
  const int ur0 = (unit - blk_prefix[it.b]) * unit_rows;
  QTile qt[2];  // by CTA rank
  if (pair_heads) {
    qt[0].head = 2 * head_unit;
    qt[1].head = 2 * head_unit + 1;
    qt[0].r0 = qt[1].r0 = ur0;
  } else {
    qt[0].head = qt[1].head = head_unit;
    qt[0].r0 = ur0;
    qt[1].r0 = ur0 + kBM;
  }
  it.kv_head = qt[0].head / a.group;
  int lo = 0x7fffffff, hi = -1;
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int r0 = qt[x].r0;
    const int pmax = it.pos0 + min(r0 + kBM - 1, it.t - 1);
    if (r0 >= it.t || pmax < 0) {
      qt[x].lo = 0;
      qt[x].hi = -1;
    } else {
      const int kmin = a.window_left >= 0 ? max(0, it.pos0 + r0 - a.window_left) : 0;
      qt[x].lo = kmin / kBN;
      qt[x].hi = pmax / kBN;
      lo = min(lo, qt[x].lo);
      hi = max(hi, qt[x].hi);
    }
  }
  // Both CTAs walk the union of the two tiles' KV ranges; a tile outside a CTA's own
  // range is wholly masked there and contributes zeros.
  it.lo = lo;
  it.n_tiles = hi - lo + 1;
  it.my = qt[rank];
  return it;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreadsPair, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap, const AttnArgs a, const int pair_heads,
                    const int max_units) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* q_smem = smem_raw;  // two buffers
  uint8_t* k_smem = smem_raw + 2 * kQBytes;
  uint8_t* v_smem = k_smem + kKStages * kKBytes;
  PairBars* bars = reinterpret_cast<PairBars*>(v_smem + kVStages * kVBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  // set by the copy warp or an issuing warp whose wait ran out: those warps stop at
  // their next item (the softmax warps meet the consequence as waits that run out)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // [tile count % 4][128 rows] of {tile count + 1, reference maximum}: the hand-over
  // of a row's reference maximum from the group that took a tile to the group that
  // takes the next, thread to thread (a row belongs to the same lane in both groups).
  // A word is written again four tiles later, after P V of the tile two before that
  // has completed, which is after the word's reader has handed in its own tile.
  unsigned long long* mu_sh = reinterpret_cast<unsigned long long*>(tmem_slot + 2);
  float* fin_l = reinterpret_cast<float*>(mu_sh + 4 * kBM);  // [2 item parities][2 groups][128 rows]
  float* fin_m = fin_l + 4 * kBM;                            // [2 item parities][2 groups][128 rows]
  // [2 item parities]: a wait of a softmax warp ran out; written before the item's
  // barrier of the two groups and read after it, so that all eight warps leave together
  volatile int* sm_fail = reinterpret_cast<volatile int*>(fin_m + 4 * kBM);
  int* blk_prefix = reinterpret_cast<int*>(fin_m + 4 * kBM) + 2;  // [batch + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
  const int n_clusters = static_cast<int>(gridDim.x) >> 1;

  if (tid == 0) {
    *abort_flag = 0;
    sm_fail[0] = 0;
    sm_fail[1] = 0;
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_free[s], 1);
    }
    for (int s = 0; s < kKStages; ++s) mbar_init(&bars->k_full[s], 1);
    for (int s = 0; s < kVStages; ++s) mbar_init(&bars->v_full[s], 1);
    for (int s = 0; s < kKStages; ++s) mbar_init(&bars->s_full[s], 1);
    for (int s = 0; s < kSlots; ++s) mbar_init(&bars->s_free[s], 2 * 4);
    for (int s = 0; s < kPvBars; ++s) mbar_init(&bars->pv_done[s], 1);
    for (int x = 0; x < 4; ++x) mbar_init(&bars->p_full[x], 2 * 4);
    mbar_init(&bars->o_free, 2 * 8);
    fence_mbar_init();
    prefetch_tensormap(&qmap);
    prefetch_tensormap(&kmap);
    prefetch_tensormap(&vmap);
  }
  // Launched with programmatic serialization: resident early, but nothing another
  // kernel may have written is read before the previous kernel has completed.
  pdl_wait();
  pdl_launch_dependents();
  const long long wait_limit = a.wait_cycles;
  // work units per sequence: 128-row blocks (head pairs) or 256-row double blocks
  const int unit_rows = pair_heads ? kBM : 2 * kBM;
  const int head_units = pair_heads ? a.hq / 2 : a.hq;
  for (int b = tid; b < a.batch; b += kThreadsPair) {
    const int t = a.cu_q[b + 1] - a.cu_q[b];
    blk_prefix[b + 1] = t > 1 ? (t + unit_rows - 1) / unit_rows : 0;
    // a one-query sequence although the caller's bounds said there was none: the
    // decode kernel was not launched, so its output rows are not computed
    if (t == 1 && !a.decode_launched && blockIdx.x == 0) atomicOr(a.status, DEV_BAD_POS);
  }
  if (tid == 0) blk_prefix[0] = 0;
  for (int i = tid; i < 4 * kBM; i += kThreadsPair) mu_sh[i] = 0ull;  // count 0 matches no tile
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < a.batch; base += 32) {
      const int idx = base + lane;
      int v = idx < a.batch ? blk_prefix[idx + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      if (idx < a.batch) blk_prefix[idx + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  const int total_units = blk_prefix[a.batch];
  // more query blocks than the caller's max_seqlen_q allows: every block is still
  // computed here, but the bound is part of the interface and other kernels size
  // their grids by it, so the call is reported
  if (total_units > max_units && tid == 0 && blockIdx.x == 0) atomicOr(a.status, DEV_BAD_POS);
  const int total_items = total_units * head_units;

  // ---- tensor memory (both CTAs allocate the same columns) and barrier set-up ------
  if (warp == 1) {
    tc05::tmem_alloc_pair(tmem_slot, kTmemCols);
    tc05::tmem_relinquish_pair();
  }
  tc05::fence_before_sync();
  cluster_sync_all();
  tc05::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp < 4) {
    // the copy and issue warps give registers to the softmax warps, which hold a
    // whole row of 128 scores each
    reg_dealloc<kRegsIssue>();
    if (warp == 0) {
      // =================================================================== producer
      bool ok = true;
      int issued = 0;  // K/V tiles requested so far, over all items
      int ut = 0;      // items with any tile so far
      // the leader's "full" barriers, as addresses any CTA of the pair can signal
      const uint32_t kf0 = cluster_map(smem_u32(&bars->k_full[0]), 0);
      const uint32_t vf0 = cluster_map(smem_u32(&bars->v_full[0]), 0);
      const uint32_t qf0 = cluster_map(smem_u32(&bars->q_full[0]), 0);
      for (int item = cluster_id; item < total_items && ok; item += n_clusters) {
        if (*abort_flag) break;
        const Item it = make_item(a, blk_prefix, item, total_units, head_units, pair_heads, rank);
        if (it.n_tiles <= 0) continue;
        const int qb = ut & 1;
        if (lane == 0) {
          // the buffer's last user: the item two before this one
          if (ut >= 2 && !mbar_wait_bounded(&bars->q_free[qb], ((ut - 2) >> 1) & 1, wait_limit)) {
            ok = false;
          } else {
            if (rank == 0) mbar_arrive_expect_tx(&bars->q_full[qb], 2 * kQBytes);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              tma_load_2d_pair(q_smem + qb * kQBytes + half * kQHalf, &qmap,
                               it.my.head * kHeadDim + half * 64, it.q0 + it.my.r0, qf0 + qb * 8);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        ++ut;
        for (int i0 = 0; i0 < it.n_tiles && ok; i0 += 32) {
          const int i = i0 + lane;
          int row_a = 0, row_b = 0;
          if (i < it.n_tiles) {
            const int tok = (it.lo + i) * kBN;
            long long page =
                a.block_table[static_cast<long long>(it.b) * a.bt_stride + tok / a.page_size];
            if (page < 0 || page >= a.num_pages) {
              atomicOr(a.status, DEV_BAD_PAGE);
              page = 0;
            }
            row_a = static_cast<int>(page * a.page_size + tok % a.page_size);
            const int tok2 = tok + 64;
            row_b = row_a;  // second half without any needed key: reload the first
            if (tok2 < it.n) {
              long long page2 =
                  a.block_table[static_cast<long long>(it.b) * a.bt_stride + tok2 / a.page_size];
              if (page2 < 0 || page2 >= a.num_pages) {
                atomicOr(a.status, DEV_BAD_PAGE);
                page2 = 0;
              }
              row_b = static_cast<int>(page2 * a.page_size + tok2 % a.page_size);
            }
          }
          const int cnt = min(32, it.n_tiles - i0);
          const int x = it.kv_head * kHeadDim;
          for (int j = 0; j < cnt; ++j) {
            const int ra = __shfl_sync(0xffffffffu, row_a, j);
            const int rb = __shfl_sync(0xffffffffu, row_b, j);
            if (lane == 0) {
              const int sk = issued % kKStages;
              const int sv = issued % kVStages;
              // stage free: S of the tile that used it last has completed
              if (!mbar_wait_bounded(&bars->s_full[sk], ((issued / kKStages) & 1) ^ 1, wait_limit)) {
                ok = false;
              } else if (a.test_drop_last && i0 + j == it.n_tiles - 1) {
                // self-test: the item's last tile never arrives, so the waits for it run out
              } else {
                // K: this CTA's 64 keys, all 128 head-dim elements
                uint8_t* kd = k_smem + sk * kKBytes;
                const int rk = rank ? rb : ra;
                if (rank == 0) mbar_arrive_expect_tx(&bars->k_full[sk], 2 * kKBytes);
                tma_load_2d_pair(kd, &kmap, x, rk, kf0 + sk * 8);
                tma_load_2d_pair(kd + kKHalf, &kmap, x + 64, rk, kf0 + sk * 8);
                // stage free: P V of the tile that used it last has completed
                if (!mbar_wait_bounded(&bars->pv_done[sv], ((issued / kVStages) & 1) ^ 1, wait_limit)) {
                  ok = false;
                } else {
                  // V: all 128 keys, this CTA's 64 head-dim elements
                  uint8_t* vd = v_smem + sv * kVBytes;
                  if (rank == 0) mbar_arrive_expect_tx(&bars->v_full[sv], 2 * kVBytes);
                  tma_load_2d_pair(vd, &vmap, x + 64 * rank, ra, vf0 + sv * 8);
                  tma_load_2d_pair(vd + 64 * 128, &vmap, x + 64 * rank, rb, vf0 + sv * 8);
                }
              }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            ++issued;
          }
        }
      }
      if (lane == 0) {
        if (!ok) {
          atomicOr(a.status, DEV_WAIT_TIMEOUT);
          *abort_flag = 1;
        }
        // The leader's barriers count both CTAs' copies: it does not leave (and, by
        // the cluster barrier below, neither does its partner) while any is in flight.
        if (rank == 0) {
          bool drained = true;
          for (int u = max(0, ut - 2); u < ut && drained; ++u) {
            drained = mbar_wait_bounded(&bars->q_full[u & 1], (u >> 1) & 1, wait_limit);
          }
          for (int i = max(0, issued - kKStages); i < issued && drained; ++i) {
            drained = mbar_wait_bounded(&bars->k_full[i % kKStages], (i / kKStages) & 1, wait_limit);
          }
          for (int i = max(0, issued - kVStages); i < issued && drained; ++i) {
            drained = mbar_wait_bounded(&bars->v_full[i % kVStages], (i / kVStages) & 1, wait_limit);
          }
          if (!drained) atomicOr(a.status, DEV_WAIT_TIMEOUT);
        }
      }
    } else if (warp == 1) {
      // ======================================================= issuer of O += P V
      // All lanes run the loops and the waits; one elected lane executes the tcgen05
      // instructions.  The two products of a tile are issued by two warps on different
      // schedulers: a tcgen05.mma waits tens of cycles for its turn behind the
      // exponentials of the softmax warps that share the issuing warp's scheduler, so
      // one warp issuing all sixteen steps of a tile cannot keep up with the 1024
      // cycles the tensor cores need for them.
      if (rank == 0) {
        constexpr uint32_t kIdescPV = tc05::idesc_f16(2 * kBM, kHeadDim, kBf16 ? 1 : 0, true);
        const tc05::Desc2 vd = tc05::split_desc(tc05::desc_mnmajor_sw128(smem_u32(v_smem), kVBytes));
        bool ok = true;
        int g = 0;   // KV tiles so far, over all items
        int ut = 0;  // items with any tile so far
        for (int item = cluster_id; item < total_items && ok; item += n_clusters) {
          if (*abort_flag) break;
          const Item it = make_item(a, blk_prefix, item, total_units, head_units, pair_heads, rank);
          if (it.n_tiles <= 0) continue;
          // O still holds the item before until all sixteen softmax warps have read it
          if (ut >= 1) ok = mbar_wait_cluster_bounded(&bars->o_free, (ut - 1) & 1, wait_limit);
          ++ut;
          for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
            const int sv = g % kVStages;
            ok = mbar_wait_bounded(&bars->v_full[sv], (g / kVStages) & 1, wait_limit) &&
                 mbar_wait_cluster_bounded(&bars->p_full[g & 3], (g >> 2) & 1, wait_limit);
            if (!ok) break;
            tc05::fence_after_sync();
            tc05::mma_ts_pair_x8<8, (2048 >> 4)>(tmem_base + kOCol, tmem_base + kPCol + (g & 1) * 64,
                                                 vd.lo + sv * (kVBytes >> 4), vd.hi, kIdescPV,
                                                 j == 0 ? 0u : 1u);
            tc05::commit_pair(&bars->pv_done[sv], kBothCtas);
          }
        }
        if (!ok && lane == 0) {
          atomicOr(a.status, DEV_WAIT_TIMEOUT);
          *abort_flag = 1;
        }
      }
      __syncwarp();
    } else if (warp == 2) {
      // ======================================================= issuer of S = Q K^T
      // S of tile g goes to score slot g % 2 as soon as the softmax group that took
      // tile g - 2 holds those scores in registers.
      if (rank == 0) {
        constexpr uint32_t kIdescS = tc05::idesc_f16(2 * kBM, kBN, kBf16 ? 1 : 0, false);
        const tc05::Desc2 qd = tc05::split_desc(tc05::desc_kmajor_sw128(smem_u32(q_smem)));
        const tc05::Desc2 kd = tc05::split_desc(tc05::desc_kmajor_sw128(smem_u32(k_smem)));
        bool ok = true;
        int g = 0;
        int ut = 0;
        for (int item = cluster_id; item < total_items && ok; item += n_clusters) {
          if (*abort_flag) break;
          const Item it = make_item(a, blk_prefix, item, total_units, head_units, pair_heads, rank);
          if (it.n_tiles <= 0) continue;
          const int qb = ut & 1;
          ok = mbar_wait_bounded(&bars->q_full[qb], (ut >> 1) & 1, wait_limit);
          ++ut;
          for (int j = 0; j < it.n_tiles && ok; ++j, ++g) {
            const int sk = g % kKStages;
            if (g >= kSlots) {
              ok = mbar_wait_cluster_bounded(&bars->s_free[g & 1], ((g - kSlots) >> 1) & 1, wait_limit);
              if (!ok) break;
            }
            ok = mbar_wait_bounded(&bars->k_full[sk], (g / kKStages) & 1, wait_limit);
            if (!ok) break;
            tc05::fence_after_sync();
            tc05::mma_ss_pair_x8<(kQHalf >> 4), (kKHalf >> 4)>(
                tmem_base + (g & 1) * 128, qd.lo + qb * (kQBytes >> 4), qd.hi,
                kd.lo + sk * (kKBytes >> 4), kd.hi, kIdescS, 0u);
            tc05::commit_pair(&bars->s_full[sk], kBothCtas);
          }
          // the query buffer may be loaded again when every product that reads it is done
          if (ok) tc05::commit_pair(&bars->q_free[qb], kBothCtas);
        }
        if (!ok && lane == 0) {
          atomicOr(a.status, DEV_WAIT_TIMEOUT);
          *abort_flag = 1;
        }
      }
      __syncwarp();
    }
  } else {
    // ================================================================ softmax groups
    reg_alloc<kRegsSoftmax>();
    const int w = (warp - 4) >> 2;  // 0: even KV tiles, 1: odd KV tiles (counted over all items)
    const int quarter = warp & 3;   // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem_base + lane_base + kOCol;
    const uint32_t s_addr = tmem_base + lane_base + w * 128;
    const uint32_t p_addr = tmem_base + lane_base + kPCol + w * 64;
    const uint32_t pf_addr0 = cluster_map(smem_u32(&bars->p_full[0]), 0);
    const uint32_t sf_addr = cluster_map(smem_u32(&bars->s_free[w]), 0);
    const uint32_t of_addr = cluster_map(smem_u32(&bars->o_free), 0);
    const int wl = a.window_left;
    bool ok = true;
    int g0 = 0;  // KV tiles of the items so far
    int ic = 0;  // items so far

    for (int item = cluster_id; item < total_items; item += n_clusters, ++ic) {
      const Item it = make_item(a, blk_prefix, item, total_units, head_units, pair_heads, rank);
      const QTile my = it.my;
      const int t = it.t;
      const int n_tiles = it.n_tiles > 0 ? it.n_tiles : 0;
      const int r = my.r0 + row;
      const int pos = it.pos0 + min(r, t - 1);
      const int wpos_lo = it.pos0 + min(my.r0 + quarter * 32, t - 1);
      const int wpos_hi = it.pos0 + min(my.r0 + quarter * 32 + 31, t - 1);
      const bool row_live = my.hi >= my.lo;  // this CTA's tile sees any key at all
      float my_m = -INFINITY;  // reference maximum (log2 domain) this group last used
      float l = 0.f;           // sum of this group's P, relative to my_m

      // this group's tiles of the item: those whose count over all items has its parity
      for (int i = (g0 + w) & 1; i < n_tiles && ok; i += 2) {
        const int g = g0 + i;
        const int k0 = (it.lo + i) * kBN;
        if (!mbar_wait_bounded(&bars->s_full[g % kKStages], (g / kKStages) & 1, wait_limit)) {
          ok = false;
          break;
        }
        tc05::fence_after_sync();
        const bool full = row_live && k0 + kBN - 1 <= wpos_lo && (wl < 0 || k0 >= wpos_hi - wl);

        // ---- the 128 scores of the row: four loads in flight, one wait, kept in
        // registers for both the maximum and the exponentials
        float mx = -INFINITY;
        uint32_t sv[4][32];
        {
#pragma unroll
          for (int c = 0; c < 4; ++c) tc05::ld32(sv[c], s_addr + c * 32);
          tc05::wait_ld();
          // the slot may take the scores of the tile after the next
          tc05::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(sf_addr);
          if (!full) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                sv[c][e] = (row_live && visible(k0 + c * 32 + e, pos, wl)) ? sv[c][e]
                                                                           : 0xff800000u;  // -inf
              }
            }
          }
          // eight independent chains of three-input maxima
          float part[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) part[u] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int e = 0; e < 32; e += 16) {
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                part[u] = max3(part[u], __uint_as_float(sv[c][e + 2 * u]),
                               __uint_as_float(sv[c][e + 2 * u + 1]));
              }
            }
          }
          mx = fmaxf(max3(part[0], part[1], part[2]),
                     max3(max3(part[3], part[4], part[5]), part[6], part[7]));
        }

        // ---- the reference maximum the other group left after the tile before
        if (i > 0) {
          const volatile unsigned long long* src = mu_sh + ((g - 1) & 3) * kBM + row;
          unsigned long long word = *src;
          if (static_cast<uint32_t>(word >> 32) != static_cast<uint32_t>(g)) {
            const long long t0 = clock64();
            for (;;) {
              word = *src;
              if (static_cast<uint32_t>(word >> 32) == static_cast<uint32_t>(g)) break;
              if (clock64() - t0 > wait_limit) {
                ok = false;
                break;
              }
            }
          }
          // (a lane whose wait ran out leaves with its warp below)
          if (!__all_sync(0xffffffffu, ok)) {
            ok = false;
            break;
          }
          const float m_prev = __uint_as_float(static_cast<uint32_t>(word));
          if (m_prev != my_m) {
            l *= fast_exp2(my_m - m_prev);  // my_m = -inf: l is 0 and stays 0
            my_m = m_prev;
          }
        }
        // ---- running maximum, updated lazily; published before the exponentials so
        // that the other group can go on with the next tile
        const float m_new = fmaxf(my_m, mx * a.scale_log2);
        const bool grow = m_new - my_m > kRescaleThreshold;  // false when both are -inf
        const bool any_grow = __any_sync(0xffffffffu, grow);
        const float m_next = any_grow ? m_new : my_m;
        // this group's P buffer was last read by P V of the tile two before (that product
        // also stands between this tile's hand-over word and the reader of the word it
        // replaces)
        if (g >= 2 && !mbar_wait_bounded(&bars->pv_done[(g - 2) % kPvBars], ((g - 2) / kPvBars) & 1,
                                         wait_limit)) {
          ok = false;
          break;
        }
        *(volatile unsigned long long*)(mu_sh + (g & 3) * kBM + row) =
            (static_cast<unsigned long long>(g + 1) << 32) | __float_as_uint(m_next);
        if (any_grow) {
          if (i > 0) {
            const float mu_new = m_next == -INFINITY ? 0.f : m_next;
            const float alpha = fast_exp2(my_m - mu_new);
            l *= alpha;
            // rare (the maximum grew by more than 2^8): O must hold every product
            // issued so far and none that uses the new reference
            if (!mbar_wait_bounded(&bars->pv_done[(g - 1) % kPvBars], ((g - 1) / kPvBars) & 1,
                                   wait_limit)) {
              ok = false;
              break;
            }
            tc05::fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < 16; ++c) {
              uint32_t ov[8];
              tc05::ld8(ov, o_addr + c * 8);
              tc05::wait_ld();
#pragma unroll
              for (int e = 0; e < 8; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
              tc05::st8(o_addr + c * 8, ov);
            }
          }
          my_m = m_next;
        }
        const float mu = my_m == -INFINITY ? 0.f : my_m;

        // ---- P = exp2(S * scale - m), as packed 16-bit pairs into the group's P buffer
        float psum = 0.f;
        {
          float2 acc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] = make_float2(0.f, 0.f);
          const float2 scale2 = make_float2(a.scale_log2, a.scale_log2);
          const float2 nmu2 = make_float2(-mu, -mu);
          // On unmasked tiles a share of the exponentials runs on the FMA pipe to
          // unload the MUFU.  Masked tiles keep the MUFU for every score: it maps -inf
          // to an exact zero, which rows without any visible key rely on.
          auto write_p = [&](auto use_poly) {
            constexpr bool kPoly = decltype(use_poly)::value;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t packed[16];
#pragma unroll
              for (int e = 0; e < 32; e += 2) {
                float2 tt = fma2(
                    make_float2(__uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1])), scale2,
                    nmu2);
                if (kPoly && ((e >> 1) & 3) < kPolyPairsOfFour) {
                  tt = poly_exp2_pair(tt);
                } else {
                  tt.x = fast_exp2(tt.x);
                  tt.y = fast_exp2(tt.y);
                }
                acc[(e >> 1) & 3] = add2(acc[(e >> 1) & 3], tt);
                packed[e >> 1] = pack2<kBf16>(tt.x, tt.y);
              }
              tc05::st16(p_addr + c * 16, packed);
            }
          };
          if (full) {
            write_p(std::true_type{});
          } else {
            write_p(std::false_type{});
          }
          const float2 s01 = add2(add2(acc[0], acc[1]), add2(acc[2], acc[3]));
          psum = s01.x + s01.y;
        }
        l += psum;
        // one arrival per warp: arrivals at a barrier in another CTA's shared memory
        // are slow enough that 128 of them would cost more than the softmax itself
        tc05::wait_st();
        tc05::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(pf_addr0 + (g & 3) * 8);
      }

      // ---- the two groups' sums of the item, brought to the final reference maximum
      if (!ok) sm_fail[ic & 1] = 1;
      float* fl = fin_l + (ic & 1) * 2 * kBM;
      float* fm = fin_m + (ic & 1) * 2 * kBM;
      fl[w * kBM + row] = l;
      fm[w * kBM + row] = my_m;
      named_bar_sync(1, 2 * kBM);
      // a wait of one of the eight warps ran out: all of them see it here and leave
      if (sm_fail[ic & 1]) {
        ok = false;
        break;
      }
      const float l_other = fl[(1 - w) * kBM + row];
      const float m_other = fm[(1 - w) * kBM + row];
      const float m_fin = fmaxf(my_m, m_other);
      float l_tot = 0.f;
      if (m_fin != -INFINITY) {
        l_tot = l * fast_exp2(my_m - m_fin) + l_other * fast_exp2(m_other - m_fin);
      }

      // ---- epilogue: O / l -> global; each group stores one half of the head dim
      if (n_tiles > 0) {
        const int gl = g0 + n_tiles - 1;
        // (if this wait runs out the warp goes on to the next item's barrier, without
        // waiting or computing, and leaves there with the others)
        ok = mbar_wait_bounded(&bars->pv_done[gl % kPvBars], (gl / kPvBars) & 1, wait_limit);
        tc05::fence_after_sync();
      }
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      uint4* orow = reinterpret_cast<uint4*>(
          reinterpret_cast<uint16_t*>(a.out) +
          (static_cast<long long>(it.q0 + min(r, t - 1)) * a.hq + my.head) * kHeadDim + w * 64);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        if (n_tiles > 0 && ok) {
          tc05::ld32(v, o_addr + w * 64 + c * 32);
          tc05::wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (c == 1 && n_tiles > 0 && ok) {
          // O may take the next item's products
          tc05::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(of_addr);
        }
        if (r < t) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 o;
            o.x = pack2<kBf16>(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            o.y = pack2<kBf16>(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            o.z = pack2<kBf16>(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
            o.w = pack2<kBf16>(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
            orow[c * 4 + (e >> 3)] = o;
          }
        }
      }
      if (w == 0 && a.lse != nullptr && r < t) {
        a.lse[static_cast<long long>(my.head) * a.total_q + it.q0 + r] =
            l_tot > 0.f ? (m_fin + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
      }
      g0 += n_tiles;
    }
    if (!ok && lane == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
  }

  // ---- release tensor memory: neither CTA frees while its partner may still use it
  __syncwarp();
  tc05::fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

size_t prefill_smem_bytes(int batch) {
  return 2 * kQBytes + kKStages * kKBytes + kVStages * kVBytes + sizeof(PairBars) +
         2 * sizeof(uint32_t) + 4 * kBM * sizeof(unsigned long long) + 8 * kBM * sizeof(float) +
         2 * sizeof(int) +
         (static_cast<size_t>(batch) + 1) * sizeof(int);
}

int launch_prefill(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                        AttnArgs a, bool bf16, cudaStream_t stream) {
  if (a.max_seqlen_q <= 1) return CWM_OK;  // decode-only batch
  const size_t smem = prefill_smem_bytes(a.batch);
  if (smem > 227 * 1024) {
    set_error("paged_attn: batch %d too large for the prefill scheduler", a.batch);
    return CWM_ERR_UNSUPPORTED;
  }
  auto k = bf16 ? prefill_pair_kernel<true> : prefill_pair_kernel<false>;
  a.wait_cycles = hook_wait_cycles();
  a.test_drop_last = hook_drop_last_tile();
  static std::atomic<bool> attr_set[64][2];
  int dev = 0;
  CWM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev][bf16 ? 1 : 0].load(std::memory_order_acquire)) {
    CWM_CUDA_CHECK(
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev >= 0 && dev < 64) attr_set[dev][bf16 ? 1 : 0].store(true, std::memory_order_release);
  }
  const int pair_heads = a.group % 2 == 0 ? 1 : 0;
  const int unit_rows = pair_heads ? kBM : 2 * kBM;
  const int head_units = pair_heads ? a.hq / 2 : a.hq;
  // every sequence with t > 1 queries has ceil(t / unit_rows) <= t / unit_rows + 1 units
  long long max_units = a.total_q / unit_rows + a.batch;
  const long long by_max =
      static_cast<long long>(a.batch) * ((a.max_seqlen_q + unit_rows - 1) / unit_rows);
  if (by_max < max_units) max_units = by_max;
  if (max_units * head_units > 0x3fffffffLL) {
    set_error("paged_attn: too many query blocks (%lld)", max_units);
    return CWM_ERR_UNSUPPORTED;
  }
  // one pair of CTAs per two SMs, fewer when the call cannot have that many items
  long long clusters = sm_count() / 2;
  if (max_units * head_units < clusters) clusters = max_units * head_units;
  if (clusters < 1) clusters = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters), 1, 1);
  cfg.blockDim = dim3(kThreadsPair);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  CWM_CUDA_CHECK(cudaLaunchKernelEx(&cfg, k, qmap, kmap, vmap, a, pair_heads,
                                    static_cast<int>(max_units)));
  return CWM_OK;
}

}  // namespace cwm
