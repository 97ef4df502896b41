// Chunked-prefill paged GQA attention, register-accumulator variant
// (mma.sync.m16n8k16, fp32 online softmax), for sequences with more than one
// query.  One CTA owns 128 queries of one query head: eight consumer warps of 16
// rows each, fed by a producer warp that streams 64-token K/V tiles through the
// block table with TMA tile loads into a shared-memory ring.  Tiles wholly above
// the causal diagonal or wholly left of the sliding window are never loaded;
// only edge tiles are masked.  Needs no scratch memory.
#include "attn_common.cuh"

namespace cwm {
namespace {

constexpr int kBM = 128;
constexpr int kTile = 64;
constexpr int kStages = 4;
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kBoxBytes = kTile * 128;
constexpr int kStageBytes = 4 * kBoxBytes;

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
prefill_mma_kernel(const __grid_constant__ CUtensorMap kmap,
                   const __grid_constant__ CUtensorMap vmap, const AttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* stages = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  int* blk_prefix = reinterpret_cast<int*>(empty_bar + kStages);  // [batch + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    fence_mbar_init();
    prefetch_tensormap(&kmap);
    prefetch_tensormap(&vmap);
  }
  // query blocks per sequence (sequences with one query belong to the decode kernel)
  for (int b = tid; b < a.batch; b += kThreads) {
    const int t = a.cu_q[b + 1] - a.cu_q[b];
    blk_prefix[b + 1] = t > 1 ? (t + kBM - 1) / kBM : 0;
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
  const int total_blocks = blk_prefix[a.batch];
  // heavier (later) query blocks first
  const int blk = total_blocks - 1 - static_cast<int>(blockIdx.y);
  if (blk < 0) return;
  int b;
  {
    int lo = 0, hi = a.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (blk_prefix[mid] <= blk) lo = mid; else hi = mid;
    }
    b = lo;
  }
  const int head = blockIdx.x;
  const int kv_head = head / a.group;
  const int q0 = a.cu_q[b];
  const int t = a.cu_q[b + 1] - q0;
  int n = a.seq_k[b];
  n = n > a.max_seqlen_k ? a.max_seqlen_k : n;
  const int r0 = (blk - blk_prefix[b]) * kBM;
  const int r1 = min(r0 + kBM, t);
  const int pos0 = n - t;  // position of query row 0
  // keys needed by this block
  const int kmax = pos0 + r1 - 1;
  const int kmin = a.window_left >= 0 ? max(0, pos0 + r0 - a.window_left) : 0;
  const int tile_lo = kmin / kTile;
  const int tile_hi = kmax >= 0 ? kmax / kTile : -1;
  const int n_tiles = tile_hi - tile_lo + 1;  // <= 0: nothing visible

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer warp
    int issued = 0;
    bool ok = true;
    for (int i0 = 0; i0 < n_tiles && ok; i0 += 32) {
      const int i = i0 + lane;
      int row = 0;
      if (i < n_tiles) {
        const int tok = (tile_lo + i) * kTile;
        long long page = a.block_table[static_cast<long long>(b) * a.bt_stride + tok / a.page_size];
        if (page < 0 || page >= a.num_pages) {
          atomicOr(a.status, DEV_BAD_PAGE);
          page = 0;
        }
        row = static_cast<int>(page * a.page_size + tok % a.page_size);
      }
      const int cnt = min(32, n_tiles - i0);
      const int x = kv_head * kHeadDim;
      for (int j = 0; j < cnt; ++j) {
        const int rj = __shfl_sync(0xffffffffu, row, j);
        if (lane == 0) {
          const int s = issued % kStages;
          const uint32_t ph = (issued / kStages) & 1;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1)) {
            ok = false;
          } else {
            uint8_t* st = stages + s * kStageBytes;
            mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
            tma_load_2d(st, &kmap, x, rj, &full_bar[s]);
            tma_load_2d(st + kBoxBytes, &kmap, x + 64, rj, &full_bar[s]);
            tma_load_2d(st + 2 * kBoxBytes, &vmap, x, rj, &full_bar[s]);
            tma_load_2d(st + 3 * kBoxBytes, &vmap, x + 64, rj, &full_bar[s]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        ++issued;
      }
    }
    if (lane == 0) {
      if (!ok) atomicOr(a.status, DEV_WAIT_TIMEOUT);
      const int first = issued > kStages ? issued - kStages : 0;
      for (int i = first; i < issued; ++i) {
        if (!mbar_wait_bounded(&full_bar[i % kStages], (i / kStages) & 1)) {
          atomicOr(a.status, DEV_WAIT_TIMEOUT);
          break;
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int c = lane & 3;
  const int wr0 = r0 + warp * 16;  // first query row of this warp
  // rows of this thread (clamped so that loads stay inside the sequence)
  const int row_a = min(wr0 + g, t - 1);
  const int row_b = min(wr0 + g + 8, t - 1);
  const int pos_a = pos0 + row_a;
  const int pos_b = pos0 + row_b;
  const int wpos_lo = pos0 + min(wr0, t - 1);
  const int wpos_hi = pos0 + min(wr0 + 15, t - 1);

  uint32_t qa[8][4];
  {
    const uint32_t* qa_row = reinterpret_cast<const uint32_t*>(a.q) +
                             (static_cast<long long>(q0 + row_a) * a.hq + head) * (kHeadDim / 2);
    const uint32_t* qb_row = reinterpret_cast<const uint32_t*>(a.q) +
                             (static_cast<long long>(q0 + row_b) * a.hq + head) * (kHeadDim / 2);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = qa_row[ks * 8 + c];
      qa[ks][1] = qb_row[ks * 8 + c];
      qa[ks][2] = qa_row[ks * 8 + 4 + c];
      qa[ks][3] = qb_row[ks * 8 + 4 + c];
    }
  }
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  bool ok = true;
  for (int it = 0; it < n_tiles; ++it) {
    const int s = it % kStages;
    const uint32_t ph = (it / kStages) & 1;
    if (!mbar_wait_bounded(&full_bar[s], ph)) {
      ok = false;
      break;
    }
    const uint32_t st = smem_u32(stages + s * kStageBytes);
    const int k0 = (tile_lo + it) * kTile;
    const bool visible = wr0 < t && k0 <= wpos_hi &&
                         (a.window_left < 0 || k0 + kTile - 1 >= wpos_lo - a.window_left);
    if (visible) {
      float sacc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      {
        const int mi = lane >> 3;
        const int r = lane & 7;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int chunk = ks * 2 + (mi & 1);
#pragma unroll
          for (int jp = 0; jp < 4; ++jp) {
            const int token = jp * 16 + (mi >> 1) * 8 + r;
            uint32_t kf[4];
            ldmatrix_x4(kf, st + (chunk >> 3) * kBoxBytes + swz128(token, chunk & 7));
            mma_16816<kBf16>(sacc[2 * jp], qa[ks], kf[0], kf[1]);
            mma_16816<kBf16>(sacc[2 * jp + 1], qa[ks], kf[2], kf[3]);
          }
        }
      }
      const bool full = k0 + kTile - 1 <= wpos_lo &&
                        (a.window_left < 0 || k0 >= wpos_hi - a.window_left);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sacc[j][e] * a.scale_log2;
          if (!full) {
            const int key = k0 + j * 8 + c * 2 + (e & 1);
            const int pos = (e & 2) ? pos_b : pos_a;
            const bool vis = key <= pos && (a.window_left < 0 || key >= pos - a.window_left);
            v = vis ? v : -INFINITY;
          }
          sacc[j][e] = v;
        }
      }
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mx_a = fmaxf(mx_a, fmaxf(sacc[j][0], sacc[j][1]));
        mx_b = fmaxf(mx_b, fmaxf(sacc[j][2], sacc[j][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float mu_a = mn_a == -INFINITY ? 0.f : mn_a;
      const float mu_b = mn_b == -INFINITY ? 0.f : mn_b;
      const float al_a = fast_exp2(m_a - mu_a), al_b = fast_exp2(m_b - mu_b);
      m_a = mn_a;
      m_b = mn_b;
      float ps_a = 0.f, ps_b = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sacc[j][0] = fast_exp2(sacc[j][0] - mu_a);
        sacc[j][1] = fast_exp2(sacc[j][1] - mu_a);
        sacc[j][2] = fast_exp2(sacc[j][2] - mu_b);
        sacc[j][3] = fast_exp2(sacc[j][3] - mu_b);
        ps_a += sacc[j][0] + sacc[j][1];
        ps_b += sacc[j][2] + sacc[j][3];
      }
      l_a = l_a * al_a + ps_a;
      l_b = l_b * al_b + ps_b;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        o[j][0] *= al_a;
        o[j][1] *= al_a;
        o[j][2] *= al_b;
        o[j][3] *= al_b;
      }
      {
        const int mi = lane >> 3;
        const int r = lane & 7;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t pfrag[4] = {
              pack2<kBf16>(sacc[2 * kk][0], sacc[2 * kk][1]),
              pack2<kBf16>(sacc[2 * kk][2], sacc[2 * kk][3]),
              pack2<kBf16>(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]),
              pack2<kBf16>(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3])};
          const int token = kk * 16 + (mi & 1) * 8 + r;
#pragma unroll
          for (int jn = 0; jn < 16; jn += 2) {
            const int chunk = jn + (mi >> 1);
            uint32_t vf[4];
            ldmatrix_x4_trans(vf, st + (2 + (chunk >> 3)) * kBoxBytes + swz128(token, chunk & 7));
            mma_16816<kBf16>(o[jn], pfrag, vf[0], vf[1]);
            mma_16816<kBf16>(o[jn + 1], pfrag, vf[2], vf[3]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }
  if (!ok) {
    if (lane == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
    return;
  }

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f;
  const float inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (wr0 + g < t) {
    uint32_t* orow = reinterpret_cast<uint32_t*>(a.out) +
                     (static_cast<long long>(q0 + wr0 + g) * a.hq + head) * (kHeadDim / 2);
#pragma unroll
    for (int j = 0; j < 16; ++j) orow[j * 4 + c] = pack2<kBf16>(o[j][0] * inv_a, o[j][1] * inv_a);
    if (a.lse != nullptr && c == 0) {
      a.lse[static_cast<long long>(head) * a.total_q + q0 + wr0 + g] =
          l_a > 0.f ? (m_a + log2f(l_a)) * 0.6931471805599453f : -INFINITY;
    }
  }
  if (wr0 + g + 8 < t) {
    uint32_t* orow = reinterpret_cast<uint32_t*>(a.out) +
                     (static_cast<long long>(q0 + wr0 + g + 8) * a.hq + head) * (kHeadDim / 2);
#pragma unroll
    for (int j = 0; j < 16; ++j) orow[j * 4 + c] = pack2<kBf16>(o[j][2] * inv_b, o[j][3] * inv_b);
    if (a.lse != nullptr && c == 0) {
      a.lse[static_cast<long long>(head) * a.total_q + q0 + wr0 + g + 8] =
          l_b > 0.f ? (m_b + log2f(l_b)) * 0.6931471805599453f : -INFINITY;
    }
  }
}

}  // namespace

int launch_prefill(const CUtensorMap& kmap, const CUtensorMap& vmap, AttnArgs a, bool bf16,
                   cudaStream_t stream) {
  if (a.max_seqlen_q <= 1) return CWM_OK;  // decode-only batch
  const size_t smem = static_cast<size_t>(kStages) * kStageBytes + 2 * kStages * sizeof(uint64_t) +
                      (static_cast<size_t>(a.batch) + 1) * sizeof(int);
  if (smem > 200 * 1024) {
    set_error("paged_attn: batch %d too large for the prefill scheduler", a.batch);
    return CWM_ERR_UNSUPPORTED;
  }
  auto k = bf16 ? prefill_mma_kernel<true> : prefill_mma_kernel<false>;
  CWM_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  // every sequence with t > 1 queries has ceil(t / 128) <= t / 128 + 1 blocks
  long long max_blocks = a.total_q / kBM + a.batch;
  const long long by_max = static_cast<long long>(a.batch) * ((a.max_seqlen_q + kBM - 1) / kBM);
  if (by_max < max_blocks) max_blocks = by_max;
  if (max_blocks > 65535) {
    set_error("paged_attn: too many query blocks (%lld)", max_blocks);
    return CWM_ERR_UNSUPPORTED;
  }
  dim3 grid(a.hq, static_cast<unsigned>(max_blocks), 1);
  k<<<grid, kThreads, smem, stream>>>(kmap, vmap, a);
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

}  // namespace cwm
