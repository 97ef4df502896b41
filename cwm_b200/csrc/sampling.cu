// Token sampling over a [rows, vocab] matrix of fp32 logits or probabilities:
// temperature softmax, nucleus (top-p) truncation, renormalisation and the draw, in
// one launch with one CTA per row and no sort.
//
// The reference sorts each row, takes the running sum, masks the entries whose
// exclusive running sum exceeds p, renormalises and draws (top_p in
// cwm/fastgen/utils/sampling.py:21-45); without top-p it draws in index order
// (sample, :6-18).  Here the set that survives the mask is found by a radix descent
// over the bit patterns of the probabilities: a histogram of probability mass per
// value bucket (11 + 11 + 9 bits) locates the smallest surviving value, and the
// same descent with the threshold u * (surviving mass) locates the entry that an
// inverse-CDF draw over the descending order would pick.  Mass is accumulated in
// 44-bit fixed point with integer atomics, so the result does not depend on the
// order in which threads add: the same inputs give the same token on every run and
// on every tensor-parallel rank.  Entries of equal probability are ordered by
// ascending index.
#include <atomic>

#include "common.cuh"

namespace cwm {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kFixShift = 44;   // probability 1.0 = 2^44 units
constexpr int kLoBits = 15;     // low part of a unit count; 2^17 entries cannot overflow 32 bits
constexpr int kBins1 = 1024;    // key bits 30..20 (sign is 0, values <= 1.0)
constexpr int kBins2 = 2048;    // key bits 19..9
constexpr int kBins3 = 512;     // key bits 8..0
constexpr int kChunk = kThreads * 4;  // entries per ordered chunk (one loop iteration)
constexpr int kMaxChunks = 2048;      // vocabularies up to 8M entries

struct Row {
  const float* x;
  long long n;
  float mx;       // maximum logit (logits only)
  float scale;    // log2(e) / temperature
  float inv_sum;  // 1 / sum of exponentials
  bool logits;
  bool vec4;
};

// Probability of one entry.  Written with explicit roundings so that every pass
// computes bit-identical values.
__device__ __forceinline__ float value_of(const Row& r, float x) {
  if (!r.logits) return x;
  const float e = fast_exp2(__fmul_rn(__fsub_rn(x, r.mx), r.scale));
  return __fmul_rn(e, r.inv_sum);
}

// Probability -> integer units of 2^-44 (exact shift of the mantissa; a positive
// probability is at least one unit, zero and negative values are zero units).
__device__ __forceinline__ unsigned long long to_units(float p) {
  const uint32_t bits = __float_as_uint(p);
  if (bits == 0u || (bits >> 31) != 0u) return 0ull;
  const int e = static_cast<int>(bits >> 23);
  if (e == 0) return 1ull;
  const unsigned long long m = (bits & 0x7fffffu) | 0x800000u;
  const int shift = e - (127 + 23 - kFixShift);
  unsigned long long u;
  if (shift >= 0) u = shift > 39 ? (m << 39) : (m << shift);
  else u = shift < -24 ? 0ull : (m >> -shift);
  return u == 0ull ? 1ull : u;
}

template <typename F>
__device__ __forceinline__ void for_each(const Row& r, F&& f) {
  // f(index, raw value); chunk c covers indices [c * kChunk, (c + 1) * kChunk)
  const int tid = threadIdx.x;
  if (r.vec4) {
    // four 16-byte loads in flight per thread before the first use: a row is streamed
    // by one CTA, so the loop is bound by memory latency unless loads are batched
    const float4* x4 = reinterpret_cast<const float4*>(r.x);
    const long long n4 = r.n >> 2;
    long long i = tid;
    for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = x4[i + u * kThreads];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long b = 4 * (i + u * kThreads);
        f(b, v[u].x);
        f(b + 1, v[u].y);
        f(b + 2, v[u].z);
        f(b + 3, v[u].w);
      }
    }
    for (; i < n4; i += kThreads) {
      const float4 v = x4[i];
      f(4 * i, v.x);
      f(4 * i + 1, v.y);
      f(4 * i + 2, v.z);
      f(4 * i + 3, v.w);
    }
    for (long long j = (n4 << 2) + tid; j < r.n; j += kThreads) f(j, r.x[j]);
  } else {
    for (long long base = 0; base < r.n; base += kChunk) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long i = base + 4 * tid + j;
        if (i < r.n) f(i, r.x[i]);
      }
    }
  }
}

struct Shared {
  uint32_t hi1[kBins1], lo1[kBins1];  // level-1 histogram, kept for the second descent
  uint32_t hi[kBins2], lo[kBins2];    // working histogram of levels 2 and 3
  unsigned long long warp_sums[kWarps];
  unsigned long long sel_before;
  unsigned long long sel_mass;
  unsigned long long bcast_u64;
  float red_f[kWarps];
  int sel_bin;
  int bcast_i;
  uint32_t chunk_hi[kMaxChunks], chunk_lo[kMaxChunks];
};

__device__ __forceinline__ void add_units(uint32_t* hi, uint32_t* lo, int bin,
                                          unsigned long long u) {
  const uint32_t l = static_cast<uint32_t>(u) & ((1u << kLoBits) - 1u);
  const uint32_t h = static_cast<uint32_t>(u >> kLoBits);
  if (l) atomicAdd(&lo[bin], l);
  if (h) atomicAdd(&hi[bin], h);
}

__device__ __forceinline__ unsigned long long bin_mass(const uint32_t* hi, const uint32_t* lo,
                                                       int bin) {
  return (static_cast<unsigned long long>(hi[bin]) << kLoBits) + lo[bin];
}

// Exclusive prefix over the threads of the block (thread order), 64-bit.
__device__ __forceinline__ unsigned long long block_exclusive(unsigned long long v, Shared& s,
                                                              unsigned long long* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();  // warp_sums free
  if (lane == 31) s.warp_sums[warp] = inc;
  __syncthreads();
  unsigned long long before = 0, all = 0;
  for (int w = 0; w < kWarps; ++w) {
    const unsigned long long t = s.warp_sums[w];
    if (w < warp) before += t;
    all += t;
  }
  if (total) *total = all;
  return before + inc - v;
}

// Among `nbins` value buckets (higher bucket = larger values), pick the lowest
// non-empty one whose mass of strictly higher buckets, plus `base`, is <= limit.
// Returns the bucket; *before = base + mass above it, *mass = its own mass.
// The highest non-empty bucket always qualifies when base <= limit.
__device__ __forceinline__ int pick_bucket(const uint32_t* hi, const uint32_t* lo, int nbins,
                                           unsigned long long base, unsigned long long limit,
                                           Shared& s, unsigned long long* before,
                                           unsigned long long* mass) {
  // thread t owns buckets nbins-1-2t and nbins-2-2t (descending order)
  const int b0 = nbins - 1 - 2 * static_cast<int>(threadIdx.x);
  const int b1 = b0 - 1;
  const unsigned long long m0 = b0 >= 0 ? bin_mass(hi, lo, b0) : 0ull;
  const unsigned long long m1 = b1 >= 0 ? bin_mass(hi, lo, b1) : 0ull;
  if (threadIdx.x == 0) s.sel_bin = 0x7fffffff;
  const unsigned long long ex = block_exclusive(m0 + m1, s, nullptr);  // syncs inside
  const unsigned long long above0 = base + ex;
  const unsigned long long above1 = above0 + m0;
  int cand = 0x7fffffff;
  if (m0 > 0 && above0 <= limit) cand = b0;
  if (m1 > 0 && above1 <= limit) cand = b1;  // lower bucket wins
  if (cand != 0x7fffffff) atomicMin(&s.sel_bin, cand);
  __syncthreads();
  const int sel = s.sel_bin;
  if (sel == b0) {
    s.sel_before = above0;
    s.sel_mass = m0;
  } else if (sel == b1) {
    s.sel_before = above1;
    s.sel_mass = m1;
  }
  __syncthreads();
  *before = s.sel_before;
  *mass = s.sel_mass;
  return sel;
}

__device__ __forceinline__ void clear_hist(uint32_t* hi, uint32_t* lo, int nbins) {
  for (int i = threadIdx.x; i < nbins; i += kThreads) hi[i] = lo[i] = 0u;
  __syncthreads();
}

// Descent from the level-1 histogram in s.hi1/lo1: the smallest present key whose
// mass of strictly larger keys is <= limit.  *before = that mass, *mass = total
// mass of the entries with exactly this key.  sel == 0x7fffffff: the row is empty.
__device__ __forceinline__ uint32_t descend(const Row& r, Shared& s, unsigned long long limit,
                                            unsigned long long* before,
                                            unsigned long long* mass) {
  unsigned long long bef, m;
  const int s1 = pick_bucket(s.hi1, s.lo1, kBins1, 0ull, limit, s, &bef, &m);
  if (s1 == 0x7fffffff) {
    *before = 0;
    *mass = 0;
    return 0xffffffffu;
  }
  clear_hist(s.hi, s.lo, kBins2);
  for_each(r, [&](long long, float x) {
    const float p = value_of(r, x);
    const uint32_t key = __float_as_uint(p);
    if ((key >> 20) == static_cast<uint32_t>(s1) && !(key >> 31)) {
      const unsigned long long u = to_units(p);
      if (u) add_units(s.hi, s.lo, (key >> 9) & (kBins2 - 1), u);
    }
  });
  __syncthreads();
  const int s2 = pick_bucket(s.hi, s.lo, kBins2, bef, limit, s, &bef, &m);
  const uint32_t prefix = (static_cast<uint32_t>(s1) << 11) | static_cast<uint32_t>(s2);
  clear_hist(s.hi, s.lo, kBins3);
  for_each(r, [&](long long, float x) {
    const float p = value_of(r, x);
    const uint32_t key = __float_as_uint(p);
    if ((key >> 9) == prefix) {
      const unsigned long long u = to_units(p);
      if (u) add_units(s.hi, s.lo, key & (kBins3 - 1), u);
    }
  });
  __syncthreads();
  const int s3 = pick_bucket(s.hi, s.lo, kBins3, bef, limit, s, &bef, &m);
  *before = bef;
  *mass = m;
  return (prefix << 9) | static_cast<uint32_t>(s3);
}

// Index of the rank-th (0-based, ascending index) entry for which pred holds.
template <typename Pred>
__device__ __forceinline__ long long kth_index(const Row& r, Shared& s, unsigned long long rank,
                                               Pred&& pred) {
  const int tid = threadIdx.x;
  const long long nchunks = (r.n + kChunk - 1) / kChunk;
  for (long long c = tid; c < nchunks; c += kThreads) s.chunk_lo[c] = 0u;
  __syncthreads();
  // matches per chunk of kChunk consecutive entries (matches are few: one atomic each)
  for_each(r, [&](long long i, float x) {
    if (pred(value_of(r, x))) atomicAdd(&s.chunk_lo[i / kChunk], 1u);
  });
  __syncthreads();
  if (tid == 0) {
    unsigned long long seen = 0;
    long long c = 0;
    for (; c < nchunks; ++c) {
      if (seen + s.chunk_lo[c] > rank) break;
      seen += s.chunk_lo[c];
    }
    s.bcast_i = static_cast<int>(c);
    s.bcast_u64 = rank - seen;
  }
  __syncthreads();
  const long long c = s.bcast_i;
  const unsigned long long local = s.bcast_u64;
  if (c >= nchunks) return -1;
  bool hit[4];
  uint32_t cnt = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const long long i = c * kChunk + 4 * tid + j;
    hit[j] = i < r.n && pred(value_of(r, r.x[i]));
    cnt += hit[j] ? 1u : 0u;
  }
  const unsigned long long ex = block_exclusive(cnt, s, nullptr);
  if (tid == 0) s.bcast_u64 = ~0ull;
  __syncthreads();
  if (local >= ex && local < ex + cnt) {
    unsigned long long k = local - ex;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (hit[j]) {
        if (k == 0) s.bcast_u64 = static_cast<unsigned long long>(c * kChunk + 4 * tid + j);
        --k;
      }
    }
  }
  __syncthreads();
  return static_cast<long long>(s.bcast_u64);
}

__device__ __forceinline__ float block_max(float v, Shared& s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) s.red_f[warp] = v;
  __syncthreads();
  float m = s.red_f[0];
  for (int w = 1; w < kWarps; ++w) m = fmaxf(m, s.red_f[w]);
  return m;
}

// Sum in a fixed order (per thread sequentially, butterfly within a warp, warps in
// order): the same value on every run.
__device__ __forceinline__ float block_sum(float v, Shared& s) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) s.red_f[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < kWarps; ++w) t = __fadd_rn(t, s.red_f[w]);
  return t;
}

struct SampleArgs {
  const float* x;         // [rows, vocab]
  const float* temps;     // [rows] or null (1.0)
  const float* top_ps;    // [rows] or null (no truncation)
  const float* uniforms;  // [rows], in [0, 1)
  long long* tokens;      // [rows]
  float* probs;           // [rows]: probability of the drawn token after renormalisation
  int* kept;              // [rows] or null: entries that survive the top-p mask
  long long vocab;
  long long row_stride;
  int is_logits;
  int mode;  // 0 greedy, 1 index order (no top-p), 2 descending order with top-p
};

__global__ void __launch_bounds__(kThreads, 1) sample_kernel(const SampleArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Shared& s = *reinterpret_cast<Shared*>(smem_raw);
  const int tid = threadIdx.x;
  const long long row = blockIdx.x;
  Row r;
  r.x = a.x + row * a.row_stride;
  r.n = a.vocab;
  r.logits = a.is_logits != 0;
  r.vec4 = (reinterpret_cast<uintptr_t>(r.x) & 15u) == 0;
  r.mx = 0.f;
  r.scale = 1.f;
  r.inv_sum = 1.f;

  if (a.mode == 0) {
    // greedy: the first index of the maximum
    unsigned long long best = 0ull;
    for_each(r, [&](long long i, float x) {
      uint32_t k = __float_as_uint(x);
      k = (k >> 31) ? ~k : (k | 0x80000000u);  // order-preserving map of floats
      if (x != x) k = 0u;                      // NaN never wins
      const unsigned long long cand =
          (static_cast<unsigned long long>(k) << 32) | (0xffffffffu - static_cast<uint32_t>(i));
      best = cand > best ? cand : best;
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
      best = t > best ? t : best;
    }
    if ((tid & 31) == 0) s.warp_sums[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kWarps; ++w) best = s.warp_sums[w] > best ? s.warp_sums[w] : best;
      a.tokens[row] = 0xffffffffu - static_cast<uint32_t>(best & 0xffffffffu);
      a.probs[row] = 1.f;
      if (a.kept) a.kept[row] = 1;
    }
    return;
  }

  if (r.logits) {
    float mx = -INFINITY;
    for_each(r, [&](long long, float x) { mx = fmaxf(mx, x); });
    r.mx = block_max(mx, s);
    const float t = a.temps ? a.temps[row] : 1.f;
    r.scale = __fdiv_rn(1.4426950408889634f, t);
    float sum = 0.f;
    for_each(r, [&](long long, float x) {
      sum = __fadd_rn(sum, fast_exp2(__fmul_rn(__fsub_rn(x, r.mx), r.scale)));
    });
    r.inv_sum = __fdiv_rn(1.f, block_sum(sum, s));
  }
  const float u01 = a.uniforms[row];

  if (a.mode == 1) {
    // index order: mass per chunk of consecutive entries, then inside one chunk
    const long long nchunks = (r.n + kChunk - 1) / kChunk;
    for (long long c = tid; c < nchunks; c += kThreads) s.chunk_hi[c] = s.chunk_lo[c] = 0u;
    __syncthreads();
    // four chunks per trip, their loads in flight together (one CTA streams the row,
    // so a trip per chunk would be bound by memory latency)
    for (long long c0 = 0; c0 < nchunks; c0 += 4) {
      float v[4][4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long i = (c0 + k) * kChunk + 4 * tid + j;
          v[k][j] = i < r.n ? r.x[i] : 0.f;
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        unsigned long long u = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long i = (c0 + k) * kChunk + 4 * tid + j;
          if (i < r.n) u += to_units(value_of(r, v[k][j]));
        }
        // per-warp sum first: 32 times fewer atomics
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) u += __shfl_xor_sync(0xffffffffu, u, o);
        if ((tid & 31) == 0 && u && c0 + k < nchunks) {
          atomicAdd(&s.chunk_lo[c0 + k], static_cast<uint32_t>(u) & ((1u << kLoBits) - 1u));
          atomicAdd(&s.chunk_hi[c0 + k], static_cast<uint32_t>(u >> kLoBits));
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      unsigned long long total = 0;
      for (long long c = 0; c < nchunks; ++c) total += bin_mass(s.chunk_hi, s.chunk_lo, c);
      unsigned long long target =
          static_cast<unsigned long long>(static_cast<double>(u01) * static_cast<double>(total));
      if (total > 0 && target >= total) target = total - 1;
      unsigned long long seen = 0;
      long long c = 0;
      for (; c < nchunks; ++c) {
        const unsigned long long m = bin_mass(s.chunk_hi, s.chunk_lo, c);
        if (seen + m > target) break;
        seen += m;
      }
      s.bcast_i = static_cast<int>(c);
      s.bcast_u64 = target - seen;
      s.sel_mass = total;
    }
    __syncthreads();
    const long long c = s.bcast_i;
    const unsigned long long local = s.bcast_u64;
    const unsigned long long total = s.sel_mass;
    if (c >= nchunks) {  // empty row
      if (tid == 0) {
        a.tokens[row] = 0;
        a.probs[row] = 0.f;
        if (a.kept) a.kept[row] = 0;
      }
      return;
    }
    unsigned long long uj[4], u = 0;
    float pj[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = c * kChunk + 4 * tid + j;
      pj[j] = i < r.n ? value_of(r, r.x[i]) : 0.f;
      uj[j] = to_units(pj[j]);
      u += uj[j];
    }
    unsigned long long ex = block_exclusive(u, s, nullptr);
    if (local >= ex && local < ex + u) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (local >= ex && local < ex + uj[j]) {
          a.tokens[row] = c * kChunk + 4 * tid + j;
          a.probs[row] = static_cast<float>(static_cast<double>(pj[j]) * 17592186044416.0 /
                                            static_cast<double>(total));
          if (a.kept) a.kept[row] = static_cast<int>(r.n);
        }
        ex += uj[j];
      }
    }
    return;
  }

  // ---- mode 2: descending order with the top-p mask
  clear_hist(s.hi1, s.lo1, kBins1);
  for_each(r, [&](long long, float x) {
    const float p = value_of(r, x);
    const unsigned long long u = to_units(p);
    if (u) add_units(s.hi1, s.lo1, min(__float_as_uint(p) >> 20, static_cast<uint32_t>(kBins1 - 1)), u);
  });
  __syncthreads();
  const float top_p = a.top_ps ? a.top_ps[row] : 1.f;
  // p >= 1 keeps everything (the exclusive running sum cannot exceed the total)
  const unsigned long long limit =
      top_p >= 1.f ? ~0ull
                   : (top_p <= 0.f ? 0ull
                                   : static_cast<unsigned long long>(static_cast<double>(top_p) *
                                                                     17592186044416.0));
  unsigned long long e0, tie_mass;
  const uint32_t kstar = descend(r, s, limit, &e0, &tie_mass);
  if (kstar == 0xffffffffu) {  // no positive entry
    if (tid == 0) {
      a.tokens[row] = 0;
      a.probs[row] = 0.f;
      if (a.kept) a.kept[row] = 0;
    }
    return;
  }
  const unsigned long long v_star = to_units(__uint_as_float(kstar));
  const unsigned long long ties = tie_mass / v_star;
  unsigned long long keep_ties = (limit - e0) / v_star + 1;
  if (keep_ties > ties) keep_ties = ties;
  const unsigned long long kept_mass = e0 + keep_ties * v_star;

  unsigned long long target =
      static_cast<unsigned long long>(static_cast<double>(u01) * static_cast<double>(kept_mass));
  if (target >= kept_mass) target = kept_mass - 1;
  unsigned long long e0s, mass_s;
  const uint32_t ksel = descend(r, s, target, &e0s, &mass_s);
  const unsigned long long v_sel = to_units(__uint_as_float(ksel));
  const unsigned long long rank = (target - e0s) / v_sel;
  const long long token = kth_index(r, s, rank, [&](float p) { return __float_as_uint(p) == ksel; });
  if (a.kept) {
    // entries above the threshold value plus the surviving ties
    uint32_t cnt = 0;
    for_each(r, [&](long long, float x) {
      const float p = value_of(r, x);
      if (!(__float_as_uint(p) >> 31) && __float_as_uint(p) > kstar) ++cnt;
    });
    unsigned long long total_cnt;
    block_exclusive(cnt, s, &total_cnt);
    if (tid == 0) a.kept[row] = static_cast<int>(total_cnt + keep_ties);
  }
  if (tid == 0) {
    a.tokens[row] = token < 0 ? 0 : token;
    a.probs[row] = static_cast<float>(static_cast<double>(__uint_as_float(ksel)) *
                                      17592186044416.0 / static_cast<double>(kept_mass));
  }
}

}  // namespace
}  // namespace cwm

using namespace cwm;

extern "C" int cwm_sample(const float* x, int is_logits, const float* temps, const float* top_ps,
                          const float* uniforms, int64_t rows, int64_t vocab, int64_t row_stride,
                          int mode, int64_t* tokens, float* probs, int32_t* kept, void* stream) {
  if (rows == 0) return CWM_OK;
  if (!x || !tokens || !probs || (mode != 0 && !uniforms)) {
    set_error("sample: null pointer");
    return CWM_ERR_INVALID;
  }
  if (rows < 0 || vocab <= 0 || row_stride < vocab || mode < 0 || mode > 2) {
    set_error("sample: bad size or mode argument");
    return CWM_ERR_INVALID;
  }
  if (vocab > static_cast<int64_t>(kMaxChunks) * kChunk) {
    set_error("sample: vocabulary of %lld entries is too large (at most %lld)",
              static_cast<long long>(vocab), static_cast<long long>(kMaxChunks) * kChunk);
    return CWM_ERR_UNSUPPORTED;
  }
  if (vocab > (1ll << 17) && mode != 0) {
    // 2^17 entries of 15-bit low parts fill a 32-bit histogram cell exactly
    set_error("sample: vocabularies above 131072 entries are not built for sampling");
    return CWM_ERR_UNSUPPORTED;
  }
  SampleArgs a;
  a.x = x;
  a.temps = temps;
  a.top_ps = top_ps;
  a.uniforms = uniforms;
  a.tokens = reinterpret_cast<long long*>(tokens);
  a.probs = probs;
  a.kept = kept;
  a.vocab = vocab;
  a.row_stride = row_stride;
  a.is_logits = is_logits;
  a.mode = mode;
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  CWM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    CWM_CUDA_CHECK(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(sizeof(Shared))));
    if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }
  sample_kernel<<<static_cast<unsigned>(rows), kThreads, sizeof(Shared),
                  static_cast<cudaStream_t>(stream)>>>(a);
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}
