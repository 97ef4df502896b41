// Split-KV paged GQA decode attention for sm_100a (one query token per sequence).
//
// The kernel is HBM-bound: every K/V byte of the attended window is read once and
// serves all query heads of its GQA group.  Work is cut into tiles of 64 tokens
// of one (sequence, KV head); the flat list of tiles is divided evenly over a
// fixed, persistent grid (2 CTAs per SM), so the launch shape does not depend on
// the sequence lengths, which are read on the device (CUDA-graph friendly).
//
// Per CTA: one producer warp streams tiles into a 3-stage shared-memory ring with
// TMA tile loads (128-byte swizzle) through the block table; four consumer warps
// each take 16 tokens of a tile, compute S = Q K^T and O += P V with
// mma.sync.m16n8k16 (query heads on the M rows, fp32 online softmax with
// warp-shuffle row reductions), and keep their own running (max, sum, O).  When a
// (sequence, KV head) segment ends, the four warp states are merged through
// shared memory; a segment that lies wholly inside one CTA is written straight to
// the output, otherwise the CTA leaves a partial (max, sum, O) in the workspace and
// bumps the segment's arrival counter; the CTA that arrives last merges the partials
// of that segment, always in CTA order (so the result does not depend on timing),
// writes the output and resets the counter.  One launch, no second kernel.
#include <atomic>

#include "attn_common.cuh"

namespace cwm {
namespace {

constexpr int kTile = 64;
constexpr int kStages = 3;
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kBoxBytes = kTile * 128;       // one [64 rows x 128 B] TMA box
constexpr int kStageBytes = 4 * kBoxBytes;   // K lo, K hi, V lo, V hi
constexpr int kFragFloats = 34;              // 16 x 2 output values, max, sum
constexpr int kPartialFloats = kFragFloats * 32;

struct SeqInfo {
  int ctx;     // keys of the sequence
  int lo;      // first attended key
  int tile0;   // first attended tile (absolute tile index)
  int ntiles;  // attended tiles (0: not a decode sequence, or empty)
  int qtok;    // row of the query in q / out
};

__device__ __forceinline__ SeqInfo seq_info(const DecodeArgs& a, int b) {
  SeqInfo s;
  const int q0 = a.cu_q[b];
  const int q1 = a.cu_q[b + 1];
  int ctx = a.seq_k[b];
  ctx = ctx > a.max_seqlen_k ? a.max_seqlen_k : ctx;
  s.qtok = q0;
  s.ctx = ctx;
  if (q1 - q0 != 1 || ctx <= 0) {
    s.lo = 0;
    s.tile0 = 0;
    s.ntiles = 0;
    return s;
  }
  s.lo = a.window_left >= 0 ? max(0, ctx - 1 - a.window_left) : 0;
  s.tile0 = s.lo / kTile;
  s.ntiles = (ctx - 1) / kTile - s.tile0 + 1;
  return s;
}

// Largest b with prefix[b] <= g (prefix is non-decreasing, prefix[batch] > g).
__device__ __forceinline__ int find_seq(const int* prefix, int batch, int g) {
  int lo = 0, hi = batch;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= g) lo = mid; else hi = mid;
  }
  return lo;
}

// Per-thread slice of a warp's running state, in mma C-fragment layout: the
// thread with lane = 4 * head + c holds output columns 8 j + 2 c + {0, 1}.
struct Frag {
  float o[16][2];
  float m;  // running max (scaled, log2 domain); equal across the 4 lanes of a head
  float l;  // running sum (per-thread partial until quad_reduce_l)
};

__device__ __forceinline__ void frag_reset(Frag& f) {
#pragma unroll
  for (int j = 0; j < 16; ++j) f.o[j][0] = f.o[j][1] = 0.f;
  f.m = -INFINITY;
  f.l = 0.f;
}

__device__ __forceinline__ void frag_store(const Frag& f, float* buf, int lane) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    buf[(2 * j) * 32 + lane] = f.o[j][0];
    buf[(2 * j + 1) * 32 + lane] = f.o[j][1];
  }
  buf[32 * 32 + lane] = f.m;
  buf[33 * 32 + lane] = f.l;
}

// f <- merge(f, state stored at buf); both with fully reduced sums.
__device__ __forceinline__ void frag_merge(Frag& f, const float* buf, int lane) {
  const float mb = buf[32 * 32 + lane];
  const float lb = buf[33 * 32 + lane];
  const float mn = fmaxf(f.m, mb);
  const float mu = mn == -INFINITY ? 0.f : mn;
  const float sa = fast_exp2(f.m - mu);
  const float sb = fast_exp2(mb - mu);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    f.o[j][0] = f.o[j][0] * sa + buf[(2 * j) * 32 + lane] * sb;
    f.o[j][1] = f.o[j][1] * sa + buf[(2 * j + 1) * 32 + lane] * sb;
  }
  f.l = f.l * sa + lb * sb;
  f.m = mn;
}

// Normalise and store one finished (sequence, KV head) result.
template <bool kBf16>
__device__ __forceinline__ void frag_write_out(const Frag& f, const DecodeArgs& a, int qtok,
                                               int kv_head, int lane) {
  const int g = lane >> 2;
  if (g >= a.group) return;
  const int c = lane & 3;
  const int head = kv_head * a.group + g;
  const float inv = f.l > 0.f ? 1.f / f.l : 0.f;
  uint32_t* orow = reinterpret_cast<uint32_t*>(a.out) +
                   (static_cast<long long>(qtok) * a.hq + head) * (kHeadDim / 2);
#pragma unroll
  for (int j = 0; j < 16; ++j) orow[j * 4 + c] = pack2<kBf16>(f.o[j][0] * inv, f.o[j][1] * inv);
  if (a.lse != nullptr && c == 0) {
    a.lse[static_cast<long long>(head) * a.total_q + qtok] =
        f.l > 0.f ? (f.m + log2f(f.l)) * 0.6931471805599453f : -INFINITY;
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
              const DecodeArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // layout: stages | merge buffers (2 partials) | barriers | prefix
  uint8_t* stages = smem_raw;
  float* merge_buf = reinterpret_cast<float*>(smem_raw + kStages * kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(merge_buf + 2 * kPartialFloats);
  uint64_t* empty_bar = full_bar + kStages;
  int* prefix = reinterpret_cast<int*>(empty_bar + kStages);
  __shared__ int abort_flag;
  __shared__ int merge_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    fence_mbar_init();
    prefetch_tensormap(&kmap);
    prefetch_tensormap(&vmap);
  }
  // Launched with programmatic serialization: the CTAs may be resident while the
  // previous kernel (typically the rotary + cache write, or the previous attention
  // call, which still uses the workspace) is finishing.  Nothing that another kernel
  // may have written is read, and nothing is written, before this returns.
  pdl_wait();
  pdl_launch_dependents();
  const long long wait_limit = a.wait_cycles;
  // tiles per sequence -> exclusive prefix over sequences (times KV heads)
  for (int b = tid; b < a.batch; b += kThreads) {
    prefix[b + 1] = seq_info(a, b).ntiles * a.hkv;
  }
  if (tid == 0) prefix[0] = 0;
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < a.batch; base += 32) {
      const int idx = base + lane;
      int v = idx < a.batch ? prefix[idx + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
      }
      if (idx < a.batch) prefix[idx + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  // decode sequences without any key (padded lanes of a batch bucket): zero output
  for (int b = blockIdx.x; b < a.batch; b += gridDim.x) {
    if (prefix[b + 1] != prefix[b]) continue;
    const int q0 = a.cu_q[b];
    if (a.cu_q[b + 1] - q0 != 1) continue;
    uint32_t* orow = reinterpret_cast<uint32_t*>(a.out) +
                     static_cast<long long>(q0) * a.hq * (kHeadDim / 2);
    for (int i = tid; i < a.hq * (kHeadDim / 2); i += kThreads) orow[i] = 0u;
    if (a.lse != nullptr) {
      for (int hh = tid; hh < a.hq; hh += kThreads) {
        a.lse[static_cast<long long>(hh) * a.total_q + q0] = -INFINITY;
      }
    }
  }
  const int total = prefix[a.batch];
  const int per = (total + gridDim.x - 1) / gridDim.x;
  const int g_begin = min(total, static_cast<int>(blockIdx.x) * per);
  const int g_end = min(total, g_begin + per);
  if (g_begin >= g_end) return;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer warp
    int issued = 0;
    bool ok = true;
    for (int g0 = g_begin; g0 < g_end && ok; g0 += 32) {
      const int g = g0 + lane;
      int x = 0, row = 0;
      if (g < g_end) {
        const int b = find_seq(prefix, a.batch, g);
        const int r = g - prefix[b];
        const int nt = (prefix[b + 1] - prefix[b]) / a.hkv;
        const int h = r / nt;
        const int t = r - h * nt;
        const SeqInfo si = seq_info(a, b);
        const int tok = (si.tile0 + t) * kTile;
        long long page = a.block_table[static_cast<long long>(b) * a.bt_stride + tok / a.page_size];
        if (page < 0 || page >= a.num_pages) {
          atomicOr(a.status, DEV_BAD_PAGE);
          page = 0;
        }
        row = static_cast<int>(page * a.page_size + tok % a.page_size);
        x = h * kHeadDim;
      }
      const int cnt = min(32, g_end - g0);
      for (int j = 0; j < cnt; ++j) {
        const int xj = __shfl_sync(0xffffffffu, x, j);
        const int rj = __shfl_sync(0xffffffffu, row, j);
        if (lane == 0) {
          const int s = issued % kStages;
          const uint32_t ph = (issued / kStages) & 1;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1, wait_limit)) {
            ok = false;
          } else if (a.test_drop_last && g0 + j == g_end - 1) {
            // self-test: the last tile never arrives, so the consumers' wait runs out
          } else {
            uint8_t* st = stages + s * kStageBytes;
            mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
            tma_load_2d(st, &kmap, xj, rj, &full_bar[s]);
            tma_load_2d(st + kBoxBytes, &kmap, xj + 64, rj, &full_bar[s]);
            tma_load_2d(st + 2 * kBoxBytes, &vmap, xj, rj, &full_bar[s]);
            tma_load_2d(st + 3 * kBoxBytes, &vmap, xj + 64, rj, &full_bar[s]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        ++issued;
      }
    }
    if (!ok && lane == 0) {
      atomicOr(a.status, DEV_WAIT_TIMEOUT);
      atomicExch(&abort_flag, 1);
    }
    // Do not leave while copies are in flight: wait (bounded) for the stages
    // that were issued but possibly not consumed yet.
    if (lane == 0) {
      const int first = issued > kStages ? issued - kStages : 0;
      for (int i = first; i < issued; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (i / kStages) & 1;
        if (!mbar_wait_bounded(&full_bar[s], ph, wait_limit)) {
          atomicOr(a.status, DEV_WAIT_TIMEOUT);
          break;
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumer warps
  const int g = lane >> 2;  // query head within the group (rows 6, 7 are padding for CWM)
  const int c = lane & 3;
  int b = find_seq(prefix, a.batch, g_begin);
  SeqInfo si = seq_info(a, b);
  int rel = g_begin - prefix[b];
  int h = rel / si.ntiles;
  int t = rel - h * si.ntiles;
  int seg_start = g_begin - t;  // global tile index at which this segment starts

  Frag f;
  frag_reset(f);
  uint32_t qa[8][2];
  auto load_q = [&]() {
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(a.q) +
                           (static_cast<long long>(si.qtok) * a.hq + h * a.group + g) *
                               (kHeadDim / 2);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = g < a.group ? qrow[ks * 8 + c] : 0u;
      qa[ks][1] = g < a.group ? qrow[ks * 8 + 4 + c] : 0u;
    }
  };
  load_q();

  // Merge the four warp states and write the segment's result, or leave a partial
  // and, if this CTA is the last of the segment's CTAs to do so, merge them all.
  auto flush = [&](int seg_end) {
    // reduce the per-thread partial sums over the 4 lanes of a head
    f.l += __shfl_xor_sync(0xffffffffu, f.l, 1);
    f.l += __shfl_xor_sync(0xffffffffu, f.l, 2);
    named_bar_sync(1, kConsumerWarps * 32);  // merge buffers free (previous flush done)
    if (warp >= 2) frag_store(f, merge_buf + (warp - 2) * kPartialFloats, lane);
    named_bar_sync(1, kConsumerWarps * 32);
    if (warp < 2) frag_merge(f, merge_buf + warp * kPartialFloats, lane);
    named_bar_sync(1, kConsumerWarps * 32);
    if (warp == 1) frag_store(f, merge_buf, lane);
    named_bar_sync(1, kConsumerWarps * 32);
    const bool complete = seg_start >= g_begin && seg_end <= g_end;  // same in every warp
    // CTAs that hold a part of this segment: first .. last
    const int c_first = seg_start / per;
    const int c_last = (seg_start + si.ntiles - 1) / per;
    if (warp == 0) {
      frag_merge(f, merge_buf, lane);
      if (complete) {
        frag_write_out<kBf16>(f, a, si.qtok, h, lane);
      } else {
        const int slot = seg_start <= g_begin ? 0 : 1;
        frag_store(f, a.partial + (static_cast<long long>(blockIdx.x) * 2 + slot) * kPartialFloats,
                   lane);
        // The warp's stores are ordered before lane 0's arrival by the warp barrier, and
        // the arrival is a release (the partial is visible device-wide before it counts)
        // and an acquire (the CTA that arrives last sees every earlier partial): one
        // atomic instead of a fence on either side of it.
        __syncwarp();
        if (lane == 0) {
          int* counter = a.counters + b * a.hkv + h;
          int arrived;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                       : "=r"(arrived)
                       : "l"(counter)
                       : "memory");
          const int last = arrived == c_last - c_first ? 1 : 0;
          if (last) *counter = 0;  // every CTA of the segment has arrived: ready for the next launch
          merge_flag = last;
        }
      }
    }
    if (complete) return;
    named_bar_sync(1, kConsumerWarps * 32);
    if (merge_flag == 0) return;
    // This CTA arrived last: merge the partials of CTAs c_first .. c_last in that
    // order.  Warp w owns output columns 32 w .. 32 w + 31 of every head.  Two passes
    // (the maxima, then the weighted sums), past L1, each with the loads of up to
    // kMergeBatch CTAs in flight together: the merge of the last segment is the end
    // of the kernel, so its latency counts in full.
    auto partial_of = [&](int cta) {
      const int slot = seg_start <= cta * per ? 0 : 1;
      return a.partial + (static_cast<long long>(cta) * 2 + slot) * kPartialFloats;
    };
    constexpr int kMergeBatch = 8;
    float m = -INFINITY;
    for (int c0 = c_first; c0 <= c_last; c0 += kMergeBatch) {
      float mv[kMergeBatch];
#pragma unroll
      for (int k = 0; k < kMergeBatch; ++k) {
        mv[k] = c0 + k <= c_last ? __ldcg(partial_of(c0 + k) + 32 * 32 + lane) : -INFINITY;
      }
#pragma unroll
      for (int k = 0; k < kMergeBatch; ++k) m = fmaxf(m, mv[k]);
    }
    const float mu = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    float o[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j][0] = o[j][1] = 0.f;
    for (int c0 = c_first; c0 <= c_last; c0 += kMergeBatch) {
      float mv[kMergeBatch], lv[kMergeBatch], ov[kMergeBatch][4][2];
#pragma unroll
      for (int k = 0; k < kMergeBatch; ++k) {
        const bool in = c0 + k <= c_last;
        const float* buf = partial_of(in ? c0 + k : c_last);
        mv[k] = in ? __ldcg(buf + 32 * 32 + lane) : -INFINITY;
        lv[k] = in ? __ldcg(buf + 33 * 32 + lane) : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ov[k][j][0] = in ? __ldcg(buf + (2 * (4 * warp + j)) * 32 + lane) : 0.f;
          ov[k][j][1] = in ? __ldcg(buf + (2 * (4 * warp + j) + 1) * 32 + lane) : 0.f;
        }
      }
      // accumulated in CTA order, as before
#pragma unroll
      for (int k = 0; k < kMergeBatch; ++k) {
        if (c0 + k <= c_last) {
          const float w = fast_exp2(mv[k] - mu);
          l = fmaf(lv[k], w, l);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o[j][0] = fmaf(ov[k][j][0], w, o[j][0]);
            o[j][1] = fmaf(ov[k][j][1], w, o[j][1]);
          }
        }
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (g < a.group) {
      const int head = h * a.group + g;
      uint32_t* orow = reinterpret_cast<uint32_t*>(a.out) +
                       (static_cast<long long>(si.qtok) * a.hq + head) * (kHeadDim / 2);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        orow[(4 * warp + j) * 4 + c] = pack2<kBf16>(o[j][0] * inv, o[j][1] * inv);
      }
      if (a.lse != nullptr && warp == 0 && c == 0) {
        a.lse[static_cast<long long>(head) * a.total_q + si.qtok] =
            l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
  };

  // A wait that runs out (or a producer that gave up) must not strand the other
  // warps at the named barriers of flush(): the warp stops waiting and computing but
  // keeps walking its tile list, so every warp passes the same barriers and the CTA
  // ends; the status word tells the host that the output is not valid.
  bool ok = true;
  int it = 0;
  for (int gi = g_begin; gi < g_end; ++gi, ++it) {
    const int s = it % kStages;
    const uint32_t ph = (it / kStages) & 1;
    if (ok && (!mbar_wait_bounded(&full_bar[s], ph, wait_limit) || *((volatile int*)&abort_flag))) {
      ok = false;
      abort_flag = 1;
    }
    const uint32_t st = smem_u32(stages + s * kStageBytes);
    const int tok0 = (si.tile0 + t) * kTile + warp * 16;
    if (ok && tok0 + 16 > si.lo && tok0 < si.ctx) {
      if (tok0 + 16 > si.ctx) {
        // Rows at or beyond the end of the context hold whatever the page held before
        // (possibly Inf or NaN, which P = 0 would not cancel): clear their V values.
        const int r = lane & 15;
        if (tok0 + r >= si.ctx) {
          uint4* dst = reinterpret_cast<uint4*>(stages + s * kStageBytes +
                                                (2 + (lane >> 4)) * kBoxBytes +
                                                (warp * 16 + r) * 128);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();  // before the producer's next TMA write to this stage
        __syncwarp();
      }
      // ---- S = Q K^T for 16 tokens: two n-tiles of 8 tokens
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
      {
        const int mi = lane >> 3;
        const int r = lane & 7;
        const int token = warp * 16 + (mi >> 1) * 8 + r;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int chunk = ks * 2 + (mi & 1);
          uint32_t kf[4];
          ldmatrix_x4(kf, st + (chunk >> 3) * kBoxBytes + swz128(token, chunk & 7));
          const uint32_t afrag[4] = {qa[ks][0], 0u, qa[ks][1], 0u};
          mma_16816<kBf16>(sacc[0], afrag, kf[0], kf[1]);
          mma_16816<kBf16>(sacc[1], afrag, kf[2], kf[3]);
        }
      }
      // ---- online softmax on row g (values sacc[j][0..1]; rows 8..15 unused)
      float p[2][2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + j * 8 + c * 2 + e;
          const float v = sacc[j][e] * a.scale_log2;
          p[j][e] = (tok >= si.lo && tok < si.ctx) ? v : -INFINITY;
        }
      }
      float mx = fmaxf(fmaxf(p[0][0], p[0][1]), fmaxf(p[1][0], p[1][1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(f.m, mx);
      const float mu = mn == -INFINITY ? 0.f : mn;
      const float alpha = fast_exp2(f.m - mu);
      f.m = mn;
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[j][e] = fast_exp2(p[j][e] - mu);
          psum += p[j][e];
        }
      }
      f.l = f.l * alpha + psum;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        f.o[j][0] *= alpha;
        f.o[j][1] *= alpha;
      }
      // ---- O += P V
      const uint32_t pfrag[4] = {pack2<kBf16>(p[0][0], p[0][1]), 0u, pack2<kBf16>(p[1][0], p[1][1]),
                                 0u};
      {
        const int mi = lane >> 3;
        const int r = lane & 7;
        const int token = warp * 16 + (mi & 1) * 8 + r;
#pragma unroll
        for (int jn = 0; jn < 16; jn += 2) {
          const int chunk = jn + (mi >> 1);
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, st + (2 + (chunk >> 3)) * kBoxBytes + swz128(token, chunk & 7));
          mma_16816_top<kBf16>(f.o[jn], pfrag, vf[0], vf[1]);
          mma_16816_top<kBf16>(f.o[jn + 1], pfrag, vf[2], vf[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);

    // ---- advance to the next tile; close the segment when it ends
    ++t;
    if (t == si.ntiles) {
      flush(gi + 1);
      frag_reset(f);
      t = 0;
      seg_start = gi + 1;
      ++h;
      if (h == a.hkv) {
        h = 0;
        if (gi + 1 < g_end) {
          do {
            ++b;
            si = seq_info(a, b);
          } while (si.ntiles == 0 && b + 1 < a.batch);
        }
      }
      if (gi + 1 < g_end) load_q();
    }
  }
  if (t > 0) flush(seg_start + si.ntiles);
  if (!ok && lane == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
}

}  // namespace

size_t decode_smem_bytes(int batch) {
  return static_cast<size_t>(kStages) * kStageBytes + 2 * kPartialFloats * sizeof(float) +
         2 * kStages * sizeof(uint64_t) + (static_cast<size_t>(batch) + 1) * sizeof(int);
}

size_t decode_counter_bytes(int batch, int hkv) {
  return (static_cast<size_t>(batch) * static_cast<size_t>(hkv) * sizeof(int) + 255) / 256 * 256;
}

size_t decode_partial_bytes(int max_ctas) {
  return static_cast<size_t>(max_ctas) * 2 * kPartialFloats * sizeof(float);
}

size_t decode_workspace_bytes_for(int batch, int hkv, int max_ctas) {
  return decode_partial_bytes(max_ctas) + decode_counter_bytes(batch, hkv);
}

size_t decode_workspace_bytes(int batch, int hkv) {
  return decode_workspace_bytes_for(batch, hkv, kMaxDecodeCtas);
}

int launch_decode(const CUtensorMap& kmap, const CUtensorMap& vmap, DecodeArgs a, bool bf16,
                  void* workspace, cudaStream_t stream, int max_ctas) {
  // The partial states come first and their size does not depend on the batch, so
  // the counters sit at the same place for every call that shares the workspace
  // (a later, larger batch never finds an earlier call's partials under them).
  a.partial = static_cast<float*>(workspace);
  a.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) +
                                      decode_partial_bytes(max_ctas));
  a.wait_cycles = hook_wait_cycles();
  a.test_drop_last = hook_drop_last_tile();
  const size_t smem = decode_smem_bytes(a.batch);
  if (smem > 110 * 1024) {
    set_error("paged_attn: batch %d too large for the decode scheduler", a.batch);
    return CWM_ERR_UNSUPPORTED;
  }
  int grid = 2 * sm_count();
  if (grid > max_ctas) grid = max_ctas;
  // the opt-in to large dynamic shared memory is per device and per kernel
  static std::atomic<bool> attr_set[64][2];
  auto main_k = bf16 ? decode_kernel<true> : decode_kernel<false>;
  int dev = 0;
  CWM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev][bf16 ? 1 : 0].load(std::memory_order_acquire)) {
    CWM_CUDA_CHECK(cudaFuncSetAttribute(main_k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        110 * 1024));
    if (dev >= 0 && dev < 64) attr_set[dev][bf16 ? 1 : 0].store(true, std::memory_order_release);
  }
  CWM_CUDA_CHECK(launch_pdl(main_k, dim3(grid), dim3(kThreads), smem, stream, kmap, vmap, a));
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

}  // namespace cwm
