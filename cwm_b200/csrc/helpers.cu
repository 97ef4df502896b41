// HBM-bound helpers of the attention path: paged row scatter, rotary embedding,
// RMS normalisation, and the fused rotate + page-write step.  All are plain
// coalesced 16-byte load/store kernels; none needs scratch memory.
#include "common.cuh"

namespace cwm {
namespace {

__device__ __forceinline__ long long load_batch_size(const void* p, int is_i64) {
  if (p == nullptr) return 0x7fffffffffffffffLL;
  return is_i64 ? *reinterpret_cast<const long long*>(p)
                : static_cast<long long>(*reinterpret_cast<const int*>(p));
}

// Destination row of token `n`, or -1 when the token is skipped.
// Addressing of cwm/fastgen/kernels/paged_memcpy.py:56-81, in 64-bit.
__device__ __forceinline__ long long paged_row(long long n, const int32_t* page_tbl,
                                               const int32_t* dst_pos, const int32_t* src_batch,
                                               long long batch_size, int page_size,
                                               long long tbl_stride, long long tbl_cols,
                                               long long dst_rows, int shard_idx, int shard_cnt,
                                               int* status) {
  if (n >= batch_size) return -1;
  int pos = dst_pos[n];
  if (pos < 0) return -1;  // padded lanes carry position -1
  if (shard_cnt > 1) {
    if (pos % shard_cnt != shard_idx) return -1;
    pos /= shard_cnt;
  }
  const long long b = src_batch ? static_cast<long long>(src_batch[n]) : n;
  const long long col = pos / page_size;
  if (col >= tbl_cols || b < 0) {
    atomicOr(status, DEV_BAD_POS);
    return -1;
  }
  const long long page = page_tbl[b * tbl_stride + col];
  const long long row = page * page_size + pos % page_size;
  if (page < 0 || row >= dst_rows) {
    atomicOr(status, DEV_BAD_PAGE);
    return -1;
  }
  return row;
}

// ---------------------------------------------------------------- paged_memcpy
// One group of `tpr` threads per source row; VecT is the widest type that the
// row size, strides and base addresses allow.
template <typename VecT>
__global__ void paged_memcpy_kernel(const VecT* __restrict__ src, VecT* __restrict__ dst,
                                    const int32_t* __restrict__ page_tbl,
                                    const int32_t* __restrict__ dst_pos,
                                    const int32_t* __restrict__ src_batch, const void* batch_size_p,
                                    int batch_size_is_i64, long long n_rows, long long row_vecs,
                                    int page_size, long long tbl_stride, long long tbl_cols,
                                    long long dst_stride_vecs, long long dst_rows, int shard_idx,
                                    int shard_cnt, int tpr, int* status) {
  const long long batch_size = load_batch_size(batch_size_p, batch_size_is_i64);
  const int rows_per_block = blockDim.x / tpr;
  const int sub = threadIdx.x / tpr;
  const int lane = threadIdx.x % tpr;
  for (long long n = static_cast<long long>(blockIdx.x) * rows_per_block + sub; n < n_rows;
       n += static_cast<long long>(gridDim.x) * rows_per_block) {
    const long long row = paged_row(n, page_tbl, dst_pos, src_batch, batch_size, page_size,
                                    tbl_stride, tbl_cols, dst_rows, shard_idx, shard_cnt, status);
    if (row < 0) continue;
    const VecT* s = src + n * row_vecs;
    VecT* d = dst + row * dst_stride_vecs;
    for (long long i = lane; i < row_vecs; i += tpr) d[i] = s[i];
  }
}

template <typename VecT>
int launch_paged_memcpy(const void* src, void* dst, const int32_t* page_tbl,
                        const int32_t* dst_pos, const int32_t* src_batch, const void* batch_size,
                        int is_i64, int64_t n, int64_t row_bytes, int page_size,
                        int64_t tbl_stride, int64_t tbl_cols, int64_t dst_stride_bytes,
                        int64_t dst_rows, int shard_idx, int shard_cnt, cudaStream_t stream) {
  const long long row_vecs = row_bytes / sizeof(VecT);
  int tpr = 1;
  while (tpr < 256 && tpr < row_vecs) tpr <<= 1;
  const int threads = 256;
  const int rows_per_block = threads / tpr;
  long long blocks = (n + rows_per_block - 1) / rows_per_block;
  const long long max_blocks = static_cast<long long>(sm_count()) * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  paged_memcpy_kernel<VecT><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      static_cast<const VecT*>(src), static_cast<VecT*>(dst), page_tbl, dst_pos, src_batch,
      batch_size, is_i64, n, row_vecs, page_size, tbl_stride, tbl_cols,
      dst_stride_bytes / static_cast<long long>(sizeof(VecT)), dst_rows, shard_idx, shard_cnt, tpr,
      status_word());
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

// ------------------------------------------------------------------------ rope

// Rotates the kElems/2 pairs held in one 16-byte vector.  cs holds (cos, sin)
// per pair.  Formula of cwm/fastgen/kernels/rope.py:84-85.
template <typename T>
__device__ __forceinline__ uint4 rotate_vec(uint4 raw, const float2* cs) {
  constexpr int kE = 16 / sizeof(T);
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < kE / 2; ++i) {
    const float re = to_f32(e[2 * i]);
    const float im = to_f32(e[2 * i + 1]);
    // products and sum as separate roundings, like the reference's fp32 math
    const float o_re = __fsub_rn(__fmul_rn(re, cs[i].x), __fmul_rn(im, cs[i].y));
    const float o_im = __fadd_rn(__fmul_rn(im, cs[i].x), __fmul_rn(re, cs[i].y));
    e[2 * i] = from_f32<T>(o_re);
    e[2 * i + 1] = from_f32<T>(o_im);
  }
  return raw;
}

constexpr int kMaxRopePairs = 1024;  // head_dim <= 2048

// Fills tab[i] = (cos, sin)(float(pos) * freqs[i]) for the pairs of one token, the
// block's threads sharing the work, and loads this thread's pairs (those covered by
// vector `v` of a head).  The angle and the accurate sine/cosine follow
// cwm/fastgen/kernels/rope.py:58,74-75.
template <typename T>
__device__ __forceinline__ void token_cos_sin(int pos, int v, int n_pairs,
                                              const float* __restrict__ freqs, float2* tab,
                                              float2* cs) {
  constexpr int kP = 8 / sizeof(T);  // pairs per 16-byte vector
  const float fpos = static_cast<float>(pos);
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const float a = __fmul_rn(fpos, freqs[i]);
    tab[i] = make_float2(cosf(a), sinf(a));
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kP; ++i) cs[i] = tab[v * kP + i];
}

// One block per token.  Thread (hslot, v) owns vector v of heads hslot,
// hslot + slots, ...; cos/sin are computed once per token in shared memory.
template <typename T>
__global__ void rope_kernel(uint4* __restrict__ x, const int32_t* __restrict__ pos,
                            const float* __restrict__ freqs, int n_heads, int vecs_per_head) {
  constexpr int kP = 8 / sizeof(T);
  const long long n = blockIdx.x;
  const int v = threadIdx.x % vecs_per_head;
  const int hslot = threadIdx.x / vecs_per_head;
  const int slots = blockDim.x / vecs_per_head;
  __shared__ float2 tab[kMaxRopePairs];
  float2 cs[kP];
  token_cos_sin<T>(pos[n], v, vecs_per_head * kP, freqs, tab, cs);
  if (hslot >= slots) return;
  uint4* row = x + n * n_heads * vecs_per_head;
  for (int h = hslot; h < n_heads; h += slots) {
    uint4* p = row + h * vecs_per_head + v;
    *p = rotate_vec<T>(*p, cs);
  }
}

// ----------------------------------------------------- fused rope + page write
template <typename T>
__global__ void rope_kv_write_kernel(uint4* __restrict__ xq, uint4* __restrict__ xk,
                                     const uint4* __restrict__ xv, uint4* __restrict__ cache_k,
                                     uint4* __restrict__ cache_v, const int32_t* __restrict__ pos,
                                     const float* __restrict__ freqs,
                                     const int32_t* __restrict__ page_tbl,
                                     const int32_t* __restrict__ src_batch,
                                     const void* batch_size_p, int batch_size_is_i64, int hq,
                                     int hkv, int vecs_per_head, int page_size,
                                     long long tbl_stride, long long tbl_cols,
                                     long long cache_stride_vecs, long long cache_rows,
                                     int* status, long long q_stride_vecs,
                                     long long k_stride_vecs, long long v_stride_vecs,
                                     uint4* __restrict__ q_out, int write_k_back) {
  // q_stride_vecs / k_stride_vecs / v_stride_vecs: distance between the rows of two
  // tokens (xq, xk and xv may be column blocks of one packed projection output).
  // q_out (nullable): contiguous [T, hq, D] destination of the rotated queries;
  // when null they are rotated in place.  write_k_back == 0: the rotated keys go to
  // the cache only.
  constexpr int kP = 8 / sizeof(T);
  const long long n = blockIdx.x;
  const int v = threadIdx.x % vecs_per_head;
  const int hslot = threadIdx.x / vecs_per_head;
  const int slots = blockDim.x / vecs_per_head;
  __shared__ float2 tab[kMaxRopePairs];
  float2 cs[kP];
  // Loads go out before the sines and cosines are computed, so that their latency
  // hides behind the arithmetic: up to four query vectors and one K/V vector per
  // thread are held in registers; further heads (wide models) take the loops below.
  constexpr int kHeld = 4;
  pdl_launch_dependents();  // the attention kernel may become resident now
  uint4* qrow = xq + n * q_stride_vecs;
  uint4* krow = xk + n * k_stride_vecs;
  const uint4* vrow = xv + n * v_stride_vecs;
  uint4* qdst = q_out != nullptr ? q_out + n * hq * vecs_per_head : qrow;
  uint4 qv[kHeld];
#pragma unroll
  for (int u = 0; u < kHeld; ++u) {
    const int h = hslot + u * slots;
    if (xq != nullptr && h < hq) qv[u] = qrow[h * vecs_per_head + v];
  }
  uint4 kv0 = make_uint4(0, 0, 0, 0), vv0 = make_uint4(0, 0, 0, 0);
  if (hslot < hkv) {
    kv0 = krow[hslot * vecs_per_head + v];
    vv0 = vrow[hslot * vecs_per_head + v];
  }
  const long long batch_size = load_batch_size(batch_size_p, batch_size_is_i64);
  const long long row = paged_row(n, page_tbl, pos, src_batch, batch_size, page_size, tbl_stride,
                                  tbl_cols, cache_rows, 0, 1, status);
  token_cos_sin<T>(pos[n], v, vecs_per_head * kP, freqs, tab, cs);
  if (xq != nullptr) {
#pragma unroll
    for (int u = 0; u < kHeld; ++u) {
      const int h = hslot + u * slots;
      if (h < hq) qdst[h * vecs_per_head + v] = rotate_vec<T>(qv[u], cs);
    }
    for (int h = hslot + kHeld * slots; h < hq; h += slots) {
      qdst[h * vecs_per_head + v] = rotate_vec<T>(qrow[h * vecs_per_head + v], cs);
    }
  }
  if (hslot < hkv) {
    const int idx = hslot * vecs_per_head + v;
    const uint4 kr = rotate_vec<T>(kv0, cs);
    if (write_k_back) krow[idx] = kr;
    if (row >= 0) {
      cache_k[row * cache_stride_vecs + idx] = kr;
      cache_v[row * cache_stride_vecs + idx] = vv0;
    }
  }
  for (int h = hslot + slots; h < hkv; h += slots) {
    const int idx = h * vecs_per_head + v;
    const uint4 kr = rotate_vec<T>(krow[idx], cs);
    if (write_k_back) krow[idx] = kr;
    if (row >= 0) {
      cache_k[row * cache_stride_vecs + idx] = kr;
      cache_v[row * cache_stride_vecs + idx] = vrow[idx];
    }
  }
}

// --------------------------------------------------------------------- rmsnorm
// One block per row; the row stays in registers between the sum of squares and
// the scaling, so HBM sees one read and one write per element.
// With `delta` the row is first updated in place, x <- round(x + delta) (the
// residual add of cwm/fastgen/forward.py:769,786, rounded to the storage type like
// the reference's add_), and the normalisation runs on the rounded sum.
template <typename T, int kVpt>
__global__ void rmsnorm_kernel(uint4* __restrict__ x, const uint4* __restrict__ delta,
                               const uint4* __restrict__ w, uint4* __restrict__ out,
                               int row_vecs, float inv_d, float eps) {
  constexpr int kE = 16 / sizeof(T);
  const long long n = blockIdx.x;
  uint4* xr = x + n * row_vecs;
  uint4 regs[kVpt];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVpt; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < row_vecs) {
      regs[i] = xr[idx];
      T* e = reinterpret_cast<T*>(&regs[i]);
      if (delta != nullptr) {
        const uint4 dv = delta[n * row_vecs + idx];
        const T* de = reinterpret_cast<const T*>(&dv);
#pragma unroll
        for (int j = 0; j < kE; ++j) e[j] = from_f32<T>(__fadd_rn(to_f32(e[j]), to_f32(de[j])));
        xr[idx] = regs[i];
      }
#pragma unroll
      for (int j = 0; j < kE; ++j) {
        const float a = to_f32(e[j]);
        ss = fmaf(a, a, ss);
      }
    }
  }
  __shared__ float warp_sums[32];
  __shared__ float rstd_s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) rstd_s = rsqrtf(t * inv_d + eps);
  }
  __syncthreads();
  const float rstd = rstd_s;
  uint4* orow = out + n * row_vecs;
#pragma unroll
  for (int i = 0; i < kVpt; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < row_vecs) {
      const uint4 wv = w[idx];
      const T* we = reinterpret_cast<const T*>(&wv);
      T* e = reinterpret_cast<T*>(&regs[i]);
#pragma unroll
      for (int j = 0; j < kE; ++j) {
        // (a * rstd) * w, cwm/fastgen/kernels/rmsnorm.py:61
        e[j] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(e[j]), rstd), to_f32(we[j])));
      }
      orow[idx] = regs[i];
    }
  }
}

// Any row length and alignment: scalar loads, two passes (the second pass hits L2).
template <typename T>
__global__ void rmsnorm_generic_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                       T* __restrict__ out, int d, float inv_d, float eps) {
  const long long n = blockIdx.x;
  const T* xr = x + n * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float a = to_f32(xr[i]);
    ss = fmaf(a, a, ss);
  }
  __shared__ float warp_sums[32];
  __shared__ float rstd_s;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) rstd_s = rsqrtf(t * inv_d + eps);
  }
  __syncthreads();
  const float rstd = rstd_s;
  T* orow = out + n * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    orow[i] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(xr[i]), rstd), to_f32(w[i])));
  }
}

template <typename T>
int launch_rmsnorm(const void* x, const void* delta, const void* w, void* out, int64_t n, int d,
                   float eps, cudaStream_t stream) {
  const float inv_d = 1.0f / static_cast<float>(d);
  const int64_t row_bytes = static_cast<int64_t>(d) * sizeof(T);
  const bool vec_ok = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                      reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const int row_vecs = static_cast<int>(row_bytes / 16);
  const unsigned grid = static_cast<unsigned>(n);
  if (vec_ok && row_vecs <= 256 * 8) {
    const int threads = row_vecs >= 512 ? 256 : 128;
    const int vpt = (row_vecs + threads - 1) / threads;
    auto xs = static_cast<uint4*>(const_cast<void*>(x));
    auto ds = static_cast<const uint4*>(delta);
    auto ws = static_cast<const uint4*>(w);
    auto os = static_cast<uint4*>(out);
#define CWM_RMS_CASE(V)                                                                       \
  case V:                                                                                     \
    rmsnorm_kernel<T, V><<<grid, threads, 0, stream>>>(xs, ds, ws, os, row_vecs, inv_d, eps); \
    break;
    switch (vpt) {
      CWM_RMS_CASE(1)
      CWM_RMS_CASE(2)
      CWM_RMS_CASE(3)
      CWM_RMS_CASE(4)
      CWM_RMS_CASE(5)
      CWM_RMS_CASE(6)
      CWM_RMS_CASE(7)
      CWM_RMS_CASE(8)
      default:
        set_error("rmsnorm: internal vector count %d", vpt);
        return CWM_ERR_INVALID;
    }
#undef CWM_RMS_CASE
  } else {
    if (delta != nullptr) {
      set_error("add_rmsnorm: rows must be 16-byte aligned multiples of 16 bytes, at most 32 KiB");
      return CWM_ERR_UNSUPPORTED;
    }
    rmsnorm_generic_kernel<T><<<grid, 256, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(w), static_cast<T*>(out), d, inv_d, eps);
  }
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

int rope_threads(int n_heads, int vecs_per_head) {
  int slots = 256 / vecs_per_head;
  if (slots > n_heads) slots = n_heads;
  if (slots < 1) slots = 1;
  return slots * vecs_per_head;
}

}  // namespace
}  // namespace cwm

using namespace cwm;

extern "C" int cwm_paged_memcpy(const void* src, void* dst, const int32_t* page_tbl,
                                const int32_t* dst_pos, const int32_t* src_batch,
                                const void* batch_size, int batch_size_is_i64, int64_t n,
                                int64_t e, int elem_bytes, int page_size, int64_t page_tbl_stride,
                                int64_t page_tbl_cols, int64_t dst_stride, int64_t dst_rows,
                                int shard_idx, int shard_cnt, void* stream) {
  if (n == 0 || e == 0) return CWM_OK;
  if (!src || !dst || !page_tbl || !dst_pos) {
    set_error("paged_memcpy: null pointer");
    return CWM_ERR_INVALID;
  }
  if (n < 0 || e < 0 || elem_bytes <= 0 || page_size <= 0 || shard_cnt < 1 || shard_idx < 0 ||
      shard_idx >= shard_cnt || dst_stride < e || page_tbl_cols < 0) {
    set_error("paged_memcpy: bad size argument");
    return CWM_ERR_INVALID;
  }
  const int64_t row_bytes = e * elem_bytes;
  const int64_t stride_bytes = dst_stride * elem_bytes;
  const uintptr_t align = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                          static_cast<uintptr_t>(row_bytes) | static_cast<uintptr_t>(stride_bytes);
  auto st = static_cast<cudaStream_t>(stream);
#define CWM_MC(V)                                                                              \
  return launch_paged_memcpy<V>(src, dst, page_tbl, dst_pos, src_batch, batch_size,            \
                                batch_size_is_i64, n, row_bytes, page_size, page_tbl_stride,   \
                                page_tbl_cols, stride_bytes, dst_rows, shard_idx, shard_cnt, st)
  if (align % 16 == 0) CWM_MC(uint4);
  if (align % 8 == 0) CWM_MC(uint2);
  if (align % 4 == 0) CWM_MC(uint32_t);
  if (align % 2 == 0) CWM_MC(uint16_t);
  CWM_MC(uint8_t);
#undef CWM_MC
}

extern "C" int cwm_rope(void* x, const int32_t* pos, const float* freqs, int64_t n, int h, int d,
                        int dtype, void* stream) {
  if (n == 0 || h == 0) return CWM_OK;
  if (!x || !pos || !freqs) {
    set_error("rope: null pointer");
    return CWM_ERR_INVALID;
  }
  const int esz = dtype == CWM_F32 ? 4 : 2;
  if (n < 0 || h < 0 || d <= 0 || d % 2 != 0) {
    set_error("rope: bad size argument");
    return CWM_ERR_INVALID;
  }
  if ((d * esz) % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 || d * esz / 16 > 256) {
    set_error("rope: head_dim %d (x %d bytes) must make 16-byte aligned heads of at most 4 KiB",
              d, esz);
    return CWM_ERR_UNSUPPORTED;
  }
  const int vph = d * esz / 16;
  const int threads = rope_threads(h, vph);
  auto st = static_cast<cudaStream_t>(stream);
  auto xv = static_cast<uint4*>(x);
  const unsigned grid = static_cast<unsigned>(n);
  switch (dtype) {
    case CWM_BF16:
      rope_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(xv, pos, freqs, h, vph);
      break;
    case CWM_F16:
      rope_kernel<__half><<<grid, threads, 0, st>>>(xv, pos, freqs, h, vph);
      break;
    case CWM_F32:
      rope_kernel<float><<<grid, threads, 0, st>>>(xv, pos, freqs, h, vph);
      break;
    default:
      set_error("rope: unknown dtype %d", dtype);
      return CWM_ERR_UNSUPPORTED;
  }
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

extern "C" int cwm_rmsnorm(const void* x, const void* w, void* out, int64_t n, int d, float eps,
                           int dtype, void* stream) {
  if (n == 0) return CWM_OK;
  if (!x || !w || !out) {
    set_error("rmsnorm: null pointer");
    return CWM_ERR_INVALID;
  }
  if (n < 0 || d <= 0) {
    set_error("rmsnorm: bad size argument");
    return CWM_ERR_INVALID;
  }
  auto st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CWM_BF16:
      return launch_rmsnorm<__nv_bfloat16>(x, nullptr, w, out, n, d, eps, st);
    case CWM_F16:
      return launch_rmsnorm<__half>(x, nullptr, w, out, n, d, eps, st);
    case CWM_F32:
      return launch_rmsnorm<float>(x, nullptr, w, out, n, d, eps, st);
    default:
      set_error("rmsnorm: unknown dtype %d", dtype);
      return CWM_ERR_UNSUPPORTED;
  }
}

extern "C" int cwm_add_rmsnorm(void* h, const void* delta, const void* w, void* out, int64_t n,
                               int d, float eps, int dtype, void* stream) {
  if (n == 0) return CWM_OK;
  if (!h || !delta || !w || !out) {
    set_error("add_rmsnorm: null pointer");
    return CWM_ERR_INVALID;
  }
  if (n < 0 || d <= 0) {
    set_error("add_rmsnorm: bad size argument");
    return CWM_ERR_INVALID;
  }
  if (reinterpret_cast<uintptr_t>(delta) % 16 != 0) {
    set_error("add_rmsnorm: delta must be 16-byte aligned");
    return CWM_ERR_UNSUPPORTED;
  }
  auto st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CWM_BF16:
      return launch_rmsnorm<__nv_bfloat16>(h, delta, w, out, n, d, eps, st);
    case CWM_F16:
      return launch_rmsnorm<__half>(h, delta, w, out, n, d, eps, st);
    case CWM_F32:
      return launch_rmsnorm<float>(h, delta, w, out, n, d, eps, st);
    default:
      set_error("add_rmsnorm: unknown dtype %d", dtype);
      return CWM_ERR_UNSUPPORTED;
  }
}

namespace cwm {
namespace {

int launch_rope_kv_write(const char* what, void* xq, void* xk, const void* xv, void* q_out,
                         int64_t q_stride, int64_t k_stride, int64_t v_stride, int write_k_back,
                         void* cache_k, void* cache_v, const int32_t* pos, const float* freqs,
                         const int32_t* page_tbl, const int32_t* src_batch,
                         const void* batch_size, int batch_size_is_i64, int64_t t, int hq,
                         int hkv, int d, int dtype, int page_size, int64_t page_tbl_stride,
                         int64_t page_tbl_cols, int64_t cache_stride, int64_t cache_rows,
                         void* stream) {
  if (t == 0) return CWM_OK;
  if (!xk || !xv || !cache_k || !cache_v || !pos || !freqs || !page_tbl) {
    set_error("%s: null pointer", what);
    return CWM_ERR_INVALID;
  }
  const int esz = dtype == CWM_F32 ? 4 : 2;
  if (t < 0 || hq < 0 || hkv <= 0 || d <= 0 || d % 2 != 0 || page_size <= 0 ||
      cache_stride < static_cast<int64_t>(hkv) * d || q_stride < static_cast<int64_t>(hq) * d ||
      k_stride < static_cast<int64_t>(hkv) * d || v_stride < static_cast<int64_t>(hkv) * d) {
    set_error("%s: bad size argument", what);
    return CWM_ERR_INVALID;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(xk) |
                          reinterpret_cast<uintptr_t>(xv) | reinterpret_cast<uintptr_t>(cache_k) |
                          reinterpret_cast<uintptr_t>(cache_v) | reinterpret_cast<uintptr_t>(q_out) |
                          static_cast<uintptr_t>(cache_stride * esz) |
                          static_cast<uintptr_t>(q_stride * esz) |
                          static_cast<uintptr_t>(k_stride * esz) |
                          static_cast<uintptr_t>(v_stride * esz) |
                          static_cast<uintptr_t>(d * esz);
  if (align % 16 != 0 || d * esz / 16 > 256) {
    set_error("%s: tensors, head size and row strides must be 16-byte aligned", what);
    return CWM_ERR_UNSUPPORTED;
  }
  const int vph = d * esz / 16;
  const int threads = rope_threads(hq > hkv ? hq : hkv, vph);
  auto st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(t);
#define CWM_RKW(T)                                                                              \
  rope_kv_write_kernel<T><<<grid, threads, 0, st>>>(                                            \
      static_cast<uint4*>(xq), static_cast<uint4*>(xk), static_cast<const uint4*>(xv),          \
      static_cast<uint4*>(cache_k), static_cast<uint4*>(cache_v), pos, freqs, page_tbl,         \
      src_batch, batch_size, batch_size_is_i64, hq, hkv, vph, page_size, page_tbl_stride,       \
      page_tbl_cols, cache_stride * esz / 16, cache_rows, status_word(), q_stride * esz / 16,   \
      k_stride * esz / 16, v_stride * esz / 16, static_cast<uint4*>(q_out), write_k_back)
  switch (dtype) {
    case CWM_BF16:
      CWM_RKW(__nv_bfloat16);
      break;
    case CWM_F16:
      CWM_RKW(__half);
      break;
    case CWM_F32:
      CWM_RKW(float);
      break;
    default:
      set_error("%s: unknown dtype %d", what, dtype);
      return CWM_ERR_UNSUPPORTED;
  }
#undef CWM_RKW
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

// out[t, i] = round(round(silu(x13[t, i])) * x13[t, ffn + i]): both roundings to the
// storage type, as the in-place silu followed by mul_ of the reference gives.
template <typename T>
__global__ void silu_mul_kernel(const uint4* __restrict__ x13, uint4* __restrict__ out,
                                long long rows, long long row_vecs) {
  constexpr int kE = 16 / sizeof(T);
  const long long total = rows * row_vecs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / row_vecs, c = i - r * row_vecs;
    uint4 a = x13[r * 2 * row_vecs + c];
    const uint4 b = x13[r * 2 * row_vecs + row_vecs + c];
    T* ea = reinterpret_cast<T*>(&a);
    const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int j = 0; j < kE; ++j) {
      const float x = to_f32(ea[j]);
      const T s = from_f32<T>(x / (1.f + expf(-x)));
      ea[j] = from_f32<T>(to_f32(s) * to_f32(eb[j]));
    }
    out[i] = a;
  }
}

// Copies n blocks of `rows` rows of `row_vecs` 16-byte vectors each; block i goes
// from src_ptrs[i] to dst_ptrs[i] with the row pitches given.  Either side may be
// pinned host memory (device-accessible under unified addressing): the copy then
// crosses the host link as plain 16-byte loads or stores issued by many CTAs.
// blockIdx.y = block, blockIdx.x strides over the block's vectors.
__global__ void block_copy_kernel(const unsigned long long* __restrict__ dst_ptrs,
                                  const unsigned long long* __restrict__ src_ptrs, int rows,
                                  int row_vecs, long long dst_pitch_vecs,
                                  long long src_pitch_vecs) {
  const uint4* src = reinterpret_cast<const uint4*>(src_ptrs[blockIdx.y]);
  uint4* dst = reinterpret_cast<uint4*>(dst_ptrs[blockIdx.y]);
  const long long total = static_cast<long long>(rows) * row_vecs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / row_vecs, c = i - r * row_vecs;
    dst[r * dst_pitch_vecs + c] = src[r * src_pitch_vecs + c];
  }
}

}  // namespace
}  // namespace cwm

extern "C" int cwm_block_copy(const uint64_t* dst_ptrs, const uint64_t* src_ptrs, int64_t n,
                              int64_t rows, int64_t row_bytes, int64_t dst_pitch_bytes,
                              int64_t src_pitch_bytes, void* stream) {
  if (n == 0 || rows == 0 || row_bytes == 0) return CWM_OK;
  if (!dst_ptrs || !src_ptrs) {
    set_error("block_copy: null pointer");
    return CWM_ERR_INVALID;
  }
  if (n < 0 || rows < 0 || row_bytes < 0 || dst_pitch_bytes < row_bytes ||
      src_pitch_bytes < row_bytes || n > 65535 || rows > 0x7fffffff) {
    set_error("block_copy: bad size argument (at most 65535 blocks per call)");
    return CWM_ERR_INVALID;
  }
  if (row_bytes % 16 != 0 || dst_pitch_bytes % 16 != 0 || src_pitch_bytes % 16 != 0) {
    set_error("block_copy: rows and pitches must be multiples of 16 bytes");
    return CWM_ERR_UNSUPPORTED;
  }
  const long long vecs = rows * (row_bytes / 16);
  const int threads = 256;
  long long gx = (vecs + threads * 8 - 1) / (threads * 8);  // about 8 vectors per thread
  if (gx < 1) gx = 1;
  if (gx > 64) gx = 64;
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(n), 1);
  block_copy_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const unsigned long long*>(dst_ptrs),
      reinterpret_cast<const unsigned long long*>(src_ptrs), static_cast<int>(rows),
      static_cast<int>(row_bytes / 16), dst_pitch_bytes / 16, src_pitch_bytes / 16);
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

extern "C" int cwm_rope_kv_write(void* xq, void* xk, const void* xv, void* cache_k, void* cache_v,
                                 const int32_t* pos, const float* freqs, const int32_t* page_tbl,
                                 const int32_t* src_batch, const void* batch_size,
                                 int batch_size_is_i64, int64_t t, int hq, int hkv, int d,
                                 int dtype, int page_size, int64_t page_tbl_stride,
                                 int64_t page_tbl_cols, int64_t cache_stride, int64_t cache_rows,
                                 void* stream) {
  return launch_rope_kv_write("rope_kv_write", xq, xk, xv, nullptr, static_cast<int64_t>(hq) * d,
                              static_cast<int64_t>(hkv) * d, static_cast<int64_t>(hkv) * d, 1,
                              cache_k, cache_v, pos, freqs, page_tbl, src_batch, batch_size,
                              batch_size_is_i64, t, hq, hkv, d, dtype, page_size, page_tbl_stride,
                              page_tbl_cols, cache_stride, cache_rows, stream);
}

extern "C" int cwm_qkv_rope_kv_write(const void* qkv, int64_t qkv_stride, void* q_out,
                                     void* cache_k, void* cache_v, const int32_t* pos,
                                     const float* freqs, const int32_t* page_tbl,
                                     const int32_t* src_batch, const void* batch_size,
                                     int batch_size_is_i64, int64_t t, int hq, int hkv, int d,
                                     int dtype, int page_size, int64_t page_tbl_stride,
                                     int64_t page_tbl_cols, int64_t cache_stride,
                                     int64_t cache_rows, void* stream) {
  if (t == 0) return CWM_OK;
  if (!qkv || !q_out) {
    set_error("qkv_rope_kv_write: null pointer");
    return CWM_ERR_INVALID;
  }
  const int esz = dtype == CWM_F32 ? 4 : 2;
  // the kernel only reads the packed rows (q_out given, keys not written back)
  char* base = static_cast<char*>(const_cast<void*>(qkv));
  void* xq = base;
  void* xk = base + static_cast<int64_t>(hq) * d * esz;
  void* xv = base + static_cast<int64_t>(hq + hkv) * d * esz;
  return launch_rope_kv_write("qkv_rope_kv_write", xq, xk, xv, q_out, qkv_stride, qkv_stride,
                              qkv_stride, 0, cache_k, cache_v, pos, freqs, page_tbl, src_batch,
                              batch_size, batch_size_is_i64, t, hq, hkv, d, dtype, page_size,
                              page_tbl_stride, page_tbl_cols, cache_stride, cache_rows, stream);
}

extern "C" int cwm_silu_mul(const void* x13, void* out, int64_t t, int64_t ffn, int dtype,
                            void* stream) {
  if (t == 0 || ffn == 0) return CWM_OK;
  if (!x13 || !out) {
    set_error("silu_mul: null pointer");
    return CWM_ERR_INVALID;
  }
  const int esz = dtype == CWM_F32 ? 4 : 2;
  if (t < 0 || ffn < 0) {
    set_error("silu_mul: bad size argument");
    return CWM_ERR_INVALID;
  }
  if ((ffn * esz) % 16 != 0 || reinterpret_cast<uintptr_t>(x13) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(out) % 16 != 0) {
    set_error("silu_mul: rows of %lld elements must be multiples of 16 bytes, 16-byte aligned",
              static_cast<long long>(ffn));
    return CWM_ERR_UNSUPPORTED;
  }
  const long long row_vecs = ffn * esz / 16;
  const long long total = t * row_vecs;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  const long long max_blocks = static_cast<long long>(sm_count()) * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  auto st = static_cast<cudaStream_t>(stream);
  auto in = static_cast<const uint4*>(x13);
  auto o = static_cast<uint4*>(out);
  switch (dtype) {
    case CWM_BF16:
      silu_mul_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), threads, 0, st>>>(in, o, t, row_vecs);
      break;
    case CWM_F16:
      silu_mul_kernel<__half><<<static_cast<unsigned>(blocks), threads, 0, st>>>(in, o, t, row_vecs);
      break;
    case CWM_F32:
      silu_mul_kernel<float><<<static_cast<unsigned>(blocks), threads, 0, st>>>(in, o, t, row_vecs);
      break;
    default:
      set_error("silu_mul: unknown dtype %d", dtype);
      return CWM_ERR_UNSUPPORTED;
  }
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}
