// Chunked-prefill paged GQA attention on the sm_100a tensor cores
// (tcgen05.mma, accumulators in tensor memory), for sequences with more than one
// query.
//
// One CTA owns two query tiles of 128 rows that share a KV head: the same 128
// queries of two neighbouring query heads when the GQA group size is even,
// otherwise two consecutive 128-row blocks of one head.  Roles by warp:
//   warp 0      TMA producer: the two Q tiles once, then 128-token K and V tiles
//               through the block table into 2-stage shared-memory rings
//   warp 1      one thread issues tcgen05.mma: S = Q K^T (M128 N128 K16 x 8, both
//               operands in swizzled shared memory) and O += P V (A = P read from
//               TMEM, B = V MN-major in shared memory), tracking completion with
//               tcgen05.commit on mbarriers
//   warps 4-7   softmax for tile A: thread = query row; reads S from TMEM, online
//   warps 8-11  softmax for tile B  softmax in fp32 with a lazily updated running
//               maximum, writes P (bf16) back over S in TMEM, rescales O in TMEM
//               only when the maximum grew by more than 2^8, normalises and stores
//               the output rows at the end
// TMEM (512 columns): S/P of tile A at 0, of tile B at 128, O of A at 256, of B at
// 384.  The tensor core alternates between the tiles, so the softmax of one tile
// overlaps the matrix products of the other.  KV tiles wholly above the causal
// diagonal or wholly left of the sliding window are never loaded; only edge tiles
// are masked.  Every mbarrier wait is bounded.  Needs no scratch memory.
#include <atomic>
#include <type_traits>

#include "attn_common.cuh"
#include "tc05.cuh"

namespace cwm {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kStages = 2;
constexpr int kThreadsTc = 384;
constexpr int kTileBytes = 128 * 256;  // [2 halves of 64 elements][128 rows][128 B]
constexpr int kHalfBytes = 128 * 128;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 domain
// Of every four pairs of scores, this many take the polynomial exp2 (more than one
// makes the softmax warps issue-bound).
constexpr int kPolyPairsOfFour = 1;

struct Bars {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], o_full[2];
};

// Query-tile bookkeeping shared by all roles.
struct QTile {
  int head;  // query head
  int r0;    // first query row within the sequence
  int lo;    // first KV tile
  int hi;    // last KV tile (hi < lo: nothing visible)
};

__device__ __forceinline__ bool visible(int key, int pos, int window_left) {
  return key <= pos && (window_left < 0 || key >= pos - window_left);
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreadsTc, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap, const AttnArgs a, const int pair_heads) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* q_smem = smem_raw;                              // 2 tiles
  uint8_t* k_smem = smem_raw + 2 * kTileBytes;             // kStages tiles
  uint8_t* v_smem = k_smem + kStages * kTileBytes;         // kStages tiles
  Bars* bars = reinterpret_cast<Bars*>(v_smem + kStages * kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  int* blk_prefix = reinterpret_cast<int*>(tmem_slot + 2);  // [batch + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&bars->s_full[x], 1);
      mbar_init(&bars->p_full[x], 128);
      mbar_init(&bars->o_full[x], 1);
    }
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
  for (int b = tid; b < a.batch; b += kThreadsTc) {
    const int t = a.cu_q[b + 1] - a.cu_q[b];
    blk_prefix[b + 1] = t > 1 ? (t + unit_rows - 1) / unit_rows : 0;
    // a one-query sequence although the caller's bounds said there was none: the
    // decode kernel was not launched, so its output rows are not computed
    if (t == 1 && !a.decode_launched && blockIdx.x == 0 && blockIdx.y == 0) {
      atomicOr(a.status, DEV_BAD_POS);
    }
  }
  if (tid == 0) blk_prefix[0] = 0;
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
  // more query blocks than the grid was sized for (max_seqlen_q below the true
  // maximum): the first blocks are not computed
  if (total_units > static_cast<int>(gridDim.y) && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
    atomicOr(a.status, DEV_BAD_POS);
  }
  const int unit = total_units - 1 - static_cast<int>(blockIdx.y);  // heavier blocks first
  if (unit < 0) return;
  int b;
  {
    int lo = 0, hi = a.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (blk_prefix[mid] <= unit) lo = mid; else hi = mid;
    }
    b = lo;
  }
  const int q0 = a.cu_q[b];
  const int t = a.cu_q[b + 1] - q0;
  int n = a.seq_k[b];
  n = n > a.max_seqlen_k ? a.max_seqlen_k : n;
  const int pos0 = n - t;  // position of query row 0
  const int ur0 = (unit - blk_prefix[b]) * unit_rows;

  QTile qt[2];
  if (pair_heads) {
    qt[0].head = 2 * blockIdx.x;
    qt[1].head = 2 * blockIdx.x + 1;
    qt[0].r0 = qt[1].r0 = ur0;
  } else {
    qt[0].head = qt[1].head = blockIdx.x;
    qt[0].r0 = ur0;
    qt[1].r0 = ur0 + kBM;
  }
  const int kv_head = qt[0].head / a.group;
  int lo = 0x7fffffff, hi = -1;
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int r0 = qt[x].r0;
    const int pmax = pos0 + min(r0 + kBM - 1, t - 1);
    if (r0 >= t || pmax < 0) {
      qt[x].lo = 0;
      qt[x].hi = -1;
    } else {
      const int kmin = a.window_left >= 0 ? max(0, pos0 + r0 - a.window_left) : 0;
      qt[x].lo = kmin / kBN;
      qt[x].hi = pmax / kBN;
      lo = min(lo, qt[x].lo);
      hi = max(hi, qt[x].hi);
    }
  }
  const int n_tiles = hi - lo + 1;  // <= 0: nothing visible for either tile

  // ---- tensor memory -------------------------------------------------------------
  if (warp == 1) {
    tc05::tmem_alloc(tmem_slot, kTmemCols);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ===================================================================== producer
    bool ok = true;
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->q_full, 2 * kTileBytes);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            tma_load_2d(q_smem + x * kTileBytes + half * kHalfBytes, &qmap,
                        qt[x].head * kHeadDim + half * 64, q0 + qt[x].r0, &bars->q_full);
          }
        }
      }
      int issued = 0;
      for (int i0 = 0; i0 < n_tiles && ok; i0 += 32) {
        const int i = i0 + lane;
        int row_a = 0, row_b = 0;
        if (i < n_tiles) {
          const int tok = (lo + i) * kBN;
          long long page = a.block_table[static_cast<long long>(b) * a.bt_stride + tok / a.page_size];
          if (page < 0 || page >= a.num_pages) {
            atomicOr(a.status, DEV_BAD_PAGE);
            page = 0;
          }
          row_a = static_cast<int>(page * a.page_size + tok % a.page_size);
          const int tok2 = tok + 64;
          row_b = row_a;  // second half without any needed key: reload the first
          if (tok2 < n) {
            long long page2 =
                a.block_table[static_cast<long long>(b) * a.bt_stride + tok2 / a.page_size];
            if (page2 < 0 || page2 >= a.num_pages) {
              atomicOr(a.status, DEV_BAD_PAGE);
              page2 = 0;
            }
            row_b = static_cast<int>(page2 * a.page_size + tok2 % a.page_size);
          }
        }
        const int cnt = min(32, n_tiles - i0);
        const int x = kv_head * kHeadDim;
        for (int j = 0; j < cnt; ++j) {
          const int ra = __shfl_sync(0xffffffffu, row_a, j);
          const int rb = __shfl_sync(0xffffffffu, row_b, j);
          if (lane == 0) {
            const int s = issued % kStages;
            const uint32_t ph = (issued / kStages) & 1;
            if (!mbar_wait_bounded(&bars->k_empty[s], ph ^ 1, wait_limit)) {
              ok = false;
            } else if (a.test_drop_last && i0 + j == n_tiles - 1) {
              // self-test: the last tile never arrives, so the waits for it run out
            } else {
              uint8_t* kd = k_smem + s * kTileBytes;
              mbar_arrive_expect_tx(&bars->k_full[s], kTileBytes);
              tma_load_2d(kd, &kmap, x, ra, &bars->k_full[s]);
              tma_load_2d(kd + 64 * 128, &kmap, x, rb, &bars->k_full[s]);
              tma_load_2d(kd + kHalfBytes, &kmap, x + 64, ra, &bars->k_full[s]);
              tma_load_2d(kd + kHalfBytes + 64 * 128, &kmap, x + 64, rb, &bars->k_full[s]);
              if (!mbar_wait_bounded(&bars->v_empty[s], ph ^ 1, wait_limit)) {
                ok = false;
              } else {
                uint8_t* vd = v_smem + s * kTileBytes;
                mbar_arrive_expect_tx(&bars->v_full[s], kTileBytes);
                tma_load_2d(vd, &vmap, x, ra, &bars->v_full[s]);
                tma_load_2d(vd + 64 * 128, &vmap, x, rb, &bars->v_full[s]);
                tma_load_2d(vd + kHalfBytes, &vmap, x + 64, ra, &bars->v_full[s]);
                tma_load_2d(vd + kHalfBytes + 64 * 128, &vmap, x + 64, rb, &bars->v_full[s]);
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          ++issued;
        }
      }
      if (lane == 0) {
        if (!ok) atomicOr(a.status, DEV_WAIT_TIMEOUT);
        // do not leave while copies are in flight
        const int first = issued > kStages ? issued - kStages : 0;
        bool drained = mbar_wait_bounded(&bars->q_full, 0, wait_limit);
        for (int i = first; i < issued && drained; ++i) {
          drained = mbar_wait_bounded(&bars->k_full[i % kStages], (i / kStages) & 1, wait_limit) &&
                    mbar_wait_bounded(&bars->v_full[i % kStages], (i / kStages) & 1, wait_limit);
        }
        if (!drained) atomicOr(a.status, DEV_WAIT_TIMEOUT);
      }
    }
  } else if (warp == 1) {
    // =================================================================== MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t kIdescS = tc05::idesc_f16(kBM, kBN, kBf16 ? 1 : 0, false);
      constexpr uint32_t kIdescPV = tc05::idesc_f16(kBM, kHeadDim, kBf16 ? 1 : 0, true);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t k_addr = smem_u32(k_smem);
      const uint32_t v_addr = smem_u32(v_smem);
      auto active = [&](int x, int j) { return lo + j >= qt[x].lo && lo + j <= qt[x].hi; };
      auto issue_s = [&](int x, int stage) {
        const uint32_t qb = q_addr + x * kTileBytes;
        const uint32_t kb = k_addr + stage * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t ofs = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          tc05::mma_ss(tmem_base + x * 128, tc05::desc_kmajor_sw128(qb + ofs),
                       tc05::desc_kmajor_sw128(kb + ofs), kIdescS, ks > 0 ? 1u : 0u);
        }
        tc05::commit(&bars->s_full[x]);
      };
      auto issue_pv = [&](int x, int stage, bool first) {
        const uint32_t vb = v_addr + stage * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc05::mma_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + kk * 8,
                       tc05::desc_mnmajor_sw128(vb + kk * 2048, kHalfBytes), kIdescPV,
                       (first && kk == 0) ? 0u : 1u);
        }
      };
      bool ok = mbar_wait_bounded(&bars->q_full, 0, wait_limit) && mbar_wait_bounded(&bars->k_full[0], 0, wait_limit);
      if (ok) {
        tc05::fence_after_sync();
        if (active(0, 0)) issue_s(0, 0);
        if (active(1, 0)) issue_s(1, 0);
        tc05::commit(&bars->k_empty[0]);
      }
      int pcnt[2] = {0, 0};
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        const int s1 = (j + 1) % kStages;
        const bool more = j + 1 < n_tiles;
        ok = mbar_wait_bounded(&bars->v_full[s], ph, wait_limit);
        if (ok && more) ok = mbar_wait_bounded(&bars->k_full[s1], ((j + 1) / kStages) & 1, wait_limit);
        if (!ok) break;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (active(x, j)) {
            if (!mbar_wait_bounded(&bars->p_full[x], pcnt[x] & 1, wait_limit)) {
              ok = false;
              break;
            }
            tc05::fence_after_sync();
            issue_pv(x, s, pcnt[x] == 0);
            ++pcnt[x];
            if (lo + j == qt[x].hi) tc05::commit(&bars->o_full[x]);
          }
          if (more && active(x, j + 1)) issue_s(x, s1);
        }
        if (!ok) break;
        tc05::commit(&bars->v_empty[s]);
        if (more) tc05::commit(&bars->k_empty[s1]);
      }
      if (!ok) atomicOr(a.status, DEV_WAIT_TIMEOUT);
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ================================================================ softmax groups
    const int x = (warp - 4) >> 2;
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const int r = qt[x].r0 + row;
    const int pos = pos0 + min(r, t - 1);
    const int wpos_lo = pos0 + min(qt[x].r0 + quarter * 32, t - 1);
    const int wpos_hi = pos0 + min(qt[x].r0 + quarter * 32 + 31, t - 1);
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + x * 128;
    const uint32_t o_addr = tmem_base + lane_base + 256 + x * 128;
    const int nx = qt[x].hi - qt[x].lo + 1;
    const int wl = a.window_left;
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;

    for (int i = 0; i < nx && ok; ++i) {
      const int k0 = (qt[x].lo + i) * kBN;
      if (!mbar_wait_bounded(&bars->s_full[x], i & 1, wait_limit)) {
        ok = false;
        break;
      }
      tc05::fence_after_sync();
      const bool full = k0 + kBN - 1 <= wpos_lo && (wl < 0 || k0 >= wpos_hi - wl);

      // ---- the 128 scores of the row: four loads in flight, one wait, kept in
      // registers for both the maximum and the exponentials
      float mx = -INFINITY;
      uint32_t sv[4][32];
      {
#pragma unroll
        for (int c = 0; c < 4; ++c) tc05::ld32(sv[c], s_addr + c * 32);
        tc05::wait_ld();
        if (!full) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              sv[c][e] = visible(k0 + c * 32 + e, pos, wl) ? sv[c][e] : 0xff800000u;  // -inf
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

      // ---- running maximum, updated lazily
      const float m_new = fmaxf(m_used, mx * a.scale_log2);
      const bool grow = m_new - m_used > kRescaleThreshold;  // false when both are -inf
      if (__any_sync(0xffffffffu, grow)) {
        if (i > 0) {
          const float mu_new = m_new == -INFINITY ? 0.f : m_new;
          const float alpha = fast_exp2(m_used - mu_new);
          l *= alpha;
          // rare (the maximum grew by more than 2^8): small pieces, so that the row
          // of scores can stay in registers meanwhile
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
        m_used = m_new;
      }
      const float mu = m_used == -INFINITY ? 0.f : m_used;

      // ---- P = exp2(S * scale - m), written over S as packed 16-bit pairs
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
              float2 t = fma2(
                  make_float2(__uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1])), scale2,
                  nmu2);
              if (kPoly && ((e >> 1) & 3) < kPolyPairsOfFour) {
                t = poly_exp2_pair(t);
              } else {
                t.x = fast_exp2(t.x);
                t.y = fast_exp2(t.y);
              }
              acc[(e >> 1) & 3] = add2(acc[(e >> 1) & 3], t);
              packed[e >> 1] = pack2<kBf16>(t.x, t.y);
            }
            tc05::st16(s_addr + c * 16, packed);
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
      tc05::wait_st();
      tc05::fence_before_sync();
      mbar_arrive(&bars->p_full[x]);
    }

    // ---- epilogue: O / l -> global
    if (ok && nx > 0) ok = mbar_wait_bounded(&bars->o_full[x], 0, wait_limit);
    if (!ok) {
      if (lane == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
    } else {
      if (nx > 0) tc05::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4* orow = reinterpret_cast<uint4*>(
          reinterpret_cast<uint16_t*>(a.out) +
          (static_cast<long long>(q0 + min(r, t - 1)) * a.hq + qt[x].head) * kHeadDim);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (nx > 0) {
          tc05::ld32(v, o_addr + c * 32);
          tc05::wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
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
      if (a.lse != nullptr && r < t) {
        a.lse[static_cast<long long>(qt[x].head) * a.total_q + q0 + r] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }

  // ---- release tensor memory
  tc05::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

size_t prefill_tc_smem_bytes(int batch) {
  return 2 * kTileBytes + 2 * kStages * kTileBytes + sizeof(Bars) + 2 * sizeof(uint32_t) +
         (static_cast<size_t>(batch) + 1) * sizeof(int);
}

int launch_prefill_tc(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                      AttnArgs a, bool bf16, cudaStream_t stream) {
  if (a.max_seqlen_q <= 1) return CWM_OK;  // decode-only batch
  const size_t smem = prefill_tc_smem_bytes(a.batch);
  if (smem > 227 * 1024) {
    set_error("paged_attn: batch %d too large for the prefill scheduler", a.batch);
    return CWM_ERR_UNSUPPORTED;
  }
  auto k = bf16 ? prefill_tc_kernel<true> : prefill_tc_kernel<false>;
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
  // every sequence with t > 1 queries has ceil(t / unit_rows) <= t / unit_rows + 1 units
  long long max_units = a.total_q / unit_rows + a.batch;
  const long long by_max =
      static_cast<long long>(a.batch) * ((a.max_seqlen_q + unit_rows - 1) / unit_rows);
  if (by_max < max_units) max_units = by_max;
  if (max_units > 65535) {
    set_error("paged_attn: too many query blocks (%lld)", max_units);
    return CWM_ERR_UNSUPPORTED;
  }
  dim3 grid(pair_heads ? a.hq / 2 : a.hq, static_cast<unsigned>(max_units), 1);
  CWM_CUDA_CHECK(launch_pdl(k, grid, dim3(kThreadsTc), smem, stream, qmap, kmap, vmap, a, pair_heads));
  return CWM_OK;
}

}  // namespace cwm
