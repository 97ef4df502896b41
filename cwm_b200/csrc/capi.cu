// Host side of the C ABI: error reporting, the device status word, tensor-map
// construction for the paged K/V views, and the attention entry point that
// validates its arguments and launches the decode and prefill kernels.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "attn_common.cuh"

namespace cwm {

namespace {
thread_local char g_error[512] = "";
__device__ int g_status_word;
constexpr int kMaxDevices = 64;
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int* status_word() {
  static int* ptrs[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

int sm_count() {
  static std::atomic<int> counts[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = counts[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      n = 148;
    }
    counts[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

namespace {
std::atomic<long long> g_hook_wait_cycles{kDefaultWaitCycles};
std::atomic<int> g_hook_drop_last{0};
}  // namespace

long long hook_wait_cycles() { return g_hook_wait_cycles.load(std::memory_order_relaxed); }
int hook_drop_last_tile() { return g_hook_drop_last.load(std::memory_order_relaxed); }

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

struct MapKey {
  const void* base;
  long long inner, rows, stride_bytes;
  int dtype, box_rows, device;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && rows == o.rows &&
           stride_bytes == o.stride_bytes && dtype == o.dtype && box_rows == o.box_rows &&
           device == o.device;
  }
};

// Tensor map over a strided [rows, inner] 16-bit matrix, boxes of
// [box_rows x 64 elements] with the 128-byte swizzle.  Maps are cached: FastGen
// keeps one cache tensor per layer for the life of the engine.
int get_kv_map(const void* base, long long inner, long long rows, long long stride_bytes,
               int dtype, int box_rows, CUtensorMap* out, bool use_cache = true) {
  static std::mutex mu;
  static std::vector<std::pair<MapKey, CUtensorMap>> cache;
  int dev = 0;
  CWM_CUDA_CHECK(cudaGetDevice(&dev));
  const MapKey key{base, inner, rows, stride_bytes, dtype, box_rows, dev};
  if (use_cache) {
    std::lock_guard<std::mutex> lock(mu);
    for (auto& kv : cache) {
      if (kv.first == key) {
        *out = kv.second;
        return CWM_OK;
      }
    }
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return CWM_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(stride_bytes)};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap map;
  const CUresult r =
      fn(&map, dtype == CWM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
         2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (base %p, inner %lld, rows %lld, "
              "stride %lld B)", static_cast<int>(r), base, inner, rows, stride_bytes);
    return CWM_ERR_CUDA;
  }
  if (use_cache) {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() >= 1024) cache.erase(cache.begin());
    cache.emplace_back(key, map);
  }
  *out = map;
  return CWM_OK;
}

}  // namespace
}  // namespace cwm

using namespace cwm;

extern "C" int cwm_version(void) { return 1; }

extern "C" const char* cwm_strerror(int code) {
  switch (code) {
    case CWM_OK: return "ok";
    case CWM_ERR_INVALID: return "invalid argument";
    case CWM_ERR_UNSUPPORTED: return "unsupported configuration";
    case CWM_ERR_CUDA: return "CUDA call failed";
    case CWM_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* cwm_last_error(void) { return g_error; }

extern "C" int cwm_device_status(int32_t* host_out, void* stream) {
  if (host_out == nullptr) {
    set_error("device_status: null output");
    return CWM_ERR_INVALID;
  }
  int* p = status_word();
  if (p == nullptr) {
    set_error("device_status: no status word (no CUDA device?)");
    return CWM_ERR_CUDA;
  }
  auto st = static_cast<cudaStream_t>(stream);
  CWM_CUDA_CHECK(cudaMemcpyAsync(host_out, p, sizeof(int), cudaMemcpyDeviceToHost, st));
  CWM_CUDA_CHECK(cudaMemsetAsync(p, 0, sizeof(int), st));
  CWM_CUDA_CHECK(cudaStreamSynchronize(st));
  return CWM_OK;
}

extern "C" int cwm_test_hooks(long long wait_limit_cycles, int drop_last_tile) {
  g_hook_wait_cycles.store(wait_limit_cycles > 0 ? wait_limit_cycles : kDefaultWaitCycles,
                           std::memory_order_relaxed);
  g_hook_drop_last.store(drop_last_tile ? 1 : 0, std::memory_order_relaxed);
  return CWM_OK;
}

extern "C" size_t cwm_paged_attn_workspace_bytes(int batch, int64_t total_q, int hq, int hkv,
                                                 int d) {
  (void)total_q;
  (void)hq;
  (void)d;
  return decode_workspace_bytes(batch < 0 ? 0 : batch, hkv > 0 ? hkv : 1);
}

extern "C" int cwm_paged_attn_fwd(const void* q, const void* k, const void* v, void* out,
                                  float* lse, const int32_t* cu_seqlens_q,
                                  const int32_t* seqused_k, const int32_t* block_table, int batch,
                                  int64_t total_q, int hq, int hkv, int d, int dtype,
                                  int page_size, int64_t num_pages, int64_t kv_token_stride,
                                  int64_t bt_stride, int max_seqlen_q, int max_seqlen_k,
                                  float softmax_scale, int window_left, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  if (batch == 0 || total_q == 0) return CWM_OK;
  if (!q || !k || !v || !out || !cu_seqlens_q || !seqused_k || !block_table) {
    set_error("paged_attn: null pointer");
    return CWM_ERR_INVALID;
  }
  if (batch < 0 || total_q < 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || page_size <= 0 ||
      num_pages <= 0 || max_seqlen_q < 0 || max_seqlen_k < 0 || bt_stride < 0 ||
      kv_token_stride < static_cast<int64_t>(hkv) * d) {
    set_error("paged_attn: bad size argument");
    return CWM_ERR_INVALID;
  }
  if (d != kHeadDim) {
    set_error("paged_attn: head_dim %d is not built (128 only)", d);
    return CWM_ERR_UNSUPPORTED;
  }
  if (dtype != CWM_BF16 && dtype != CWM_F16) {
    set_error("paged_attn: dtype %d is not built (bf16 and fp16 only)", dtype);
    return CWM_ERR_UNSUPPORTED;
  }
  const int group = hq / hkv;
  if (group > 8) {
    set_error("paged_attn: %d query heads per KV head is not built (at most 8)", group);
    return CWM_ERR_UNSUPPORTED;
  }
  if (page_size % 64 != 0) {
    set_error("paged_attn: page_size %d must be a multiple of 64", page_size);
    return CWM_ERR_UNSUPPORTED;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out) |
                          static_cast<uintptr_t>(kv_token_stride * 2);
  if (align % 16 != 0) {
    set_error("paged_attn: q, k, v, out and the K/V token stride must be 16-byte aligned");
    return CWM_ERR_INVALID;
  }
  if (num_pages * page_size > 0x7fffffffLL) {
    set_error("paged_attn: cache of %lld rows is too large", (long long)(num_pages * page_size));
    return CWM_ERR_UNSUPPORTED;
  }
  int* status = status_word();
  if (status == nullptr) {
    set_error("paged_attn: cannot resolve the device status word");
    return CWM_ERR_CUDA;
  }
  // total_q == batch * max_seqlen_q with max_seqlen_q > 1 means that no sequence
  // has exactly one query, so the decode kernel has nothing to do.
  const bool may_decode = !(max_seqlen_q > 1 && total_q == static_cast<int64_t>(batch) * max_seqlen_q);
  if (may_decode) {
    const size_t need = decode_workspace_bytes(batch, hkv);
    if (workspace == nullptr || workspace_bytes < need) {
      set_error("paged_attn: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
      return CWM_ERR_WORKSPACE;
    }
    if (reinterpret_cast<uintptr_t>(workspace) % 16 != 0) {
      set_error("paged_attn: workspace must be 16-byte aligned");
      return CWM_ERR_INVALID;
    }
  }

  CUtensorMap kmap, vmap;
  const long long inner = static_cast<long long>(hkv) * d;
  const long long rows = num_pages * page_size;
  int rc = get_kv_map(k, inner, rows, kv_token_stride * 2, dtype, 64, &kmap);
  if (rc != CWM_OK) return rc;
  rc = get_kv_map(v, inner, rows, kv_token_stride * 2, dtype, 64, &vmap);
  if (rc != CWM_OK) return rc;

  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q;
  a.out = out;
  a.lse = lse;
  a.cu_q = cu_seqlens_q;
  a.seq_k = seqused_k;
  a.block_table = block_table;
  a.batch = batch;
  a.hq = hq;
  a.hkv = hkv;
  a.group = group;
  a.page_size = page_size;
  a.max_seqlen_q = max_seqlen_q;
  a.max_seqlen_k = max_seqlen_k;
  a.num_pages = num_pages;
  a.bt_stride = bt_stride;
  a.total_q = total_q;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.window_left = window_left;
  a.status = status;
  a.decode_launched = may_decode ? 1 : 0;
  auto st = static_cast<cudaStream_t>(stream);
  const bool bf16 = dtype == CWM_BF16;
  if (may_decode) {
    rc = launch_decode(kmap, vmap, a, bf16, workspace, st);
    if (rc != CWM_OK) return rc;
  }
  if (max_seqlen_q > 1) {
    // the query tensor changes from call to call: its map is built, not cached
    CUtensorMap qmap;
    rc = get_kv_map(q, static_cast<long long>(hq) * d, total_q, static_cast<long long>(hq) * d * 2,
                    dtype, 128, &qmap, false);
    if (rc != CWM_OK) return rc;
    rc = launch_prefill(qmap, kmap, vmap, a, bf16, st);
    if (rc != CWM_OK) return rc;
  }
  return CWM_OK;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some embedders of this library run where cudaMalloc is off the table: inside a
// serving loop whose memory is fully pre-planned, in a plugin that is handed
// fixed buffers by its host, or on a thread that must never block on the
// allocator.  They can still pass their own q / cache / output buffers, but they
// have nowhere to get the split-KV scratch from.  For them the scratch lives in
// the library image itself.
namespace cwm {
namespace {

// Sized for kNoAllocMaxBatch sequences with up to kNoAllocMaxKvHeads KV heads (the
// arrival counters) and a persistent grid of kNoAllocMaxCtas CTAs (two per SM on a
// 148-SM B200, with headroom to 152 SMs): about 2.7 MB that every GPU holds from
// the moment it loads the library until exit.
constexpr int kNoAllocMaxBatch = CWM_NOALLOC_MAX_BATCH;
constexpr int kNoAllocMaxKvHeads = 16;
constexpr int kNoAllocMaxCtas = 304;
constexpr size_t kNoAllocScratchBytes =
    static_cast<size_t>(kNoAllocMaxCtas) * 2 * 34 * 32 * sizeof(float) +
    static_cast<size_t>(kNoAllocMaxBatch) * kNoAllocMaxKvHeads * sizeof(int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the scratch array on the current device.  In host code the
// array's name is only a handle; the address the kernels need comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int noalloc_scratch(void** out) {
  static void* ptrs[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  CWM_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("paged_attn_decode_noalloc: device index %d out of range", dev);
    return CWM_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    CWM_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return CWM_OK;
}

}  // namespace
}  // namespace cwm

extern "C" int cwm_paged_attn_decode_noalloc(const void* q, const void* k, const void* v,
                                             void* out, float* lse,
                                             const int32_t* cu_seqlens_q,
                                             const int32_t* seqused_k,
                                             const int32_t* block_table, int batch, int hq,
                                             int hkv, int d, int dtype, int page_size,
                                             int64_t num_pages, int64_t kv_token_stride,
                                             int64_t bt_stride, int max_seqlen_k,
                                             float softmax_scale, int window_left,
                                             void* stream) {
  if (batch == 0) return CWM_OK;
  if (!q || !k || !v || !out || !cu_seqlens_q || !seqused_k || !block_table) {
    set_error("paged_attn_decode_noalloc: null pointer");
    return CWM_ERR_INVALID;
  }
  if (batch < 0 || batch > kNoAllocMaxBatch) {
    set_error("paged_attn_decode_noalloc: batch %d exceeds the built-in scratch (at most %d "
              "sequences per call)", batch, kNoAllocMaxBatch);
    return CWM_ERR_WORKSPACE;
  }
  if (hq <= 0 || hkv <= 0 || hq % hkv != 0 || page_size <= 0 || num_pages <= 0 ||
      max_seqlen_k < 0 || bt_stride < 0 || kv_token_stride < static_cast<int64_t>(hkv) * d) {
    set_error("paged_attn_decode_noalloc: bad size argument");
    return CWM_ERR_INVALID;
  }
  if (d != kHeadDim || (dtype != CWM_BF16 && dtype != CWM_F16) || hq / hkv > 8 ||
      page_size % 64 != 0) {
    set_error("paged_attn_decode_noalloc: only head_dim 128, bf16/fp16, at most 8 query heads "
              "per KV head and page sizes that are multiples of 64 are built");
    return CWM_ERR_UNSUPPORTED;
  }
  const uintptr_t align = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out) |
                          static_cast<uintptr_t>(kv_token_stride * 2);
  if (align % 16 != 0) {
    set_error("paged_attn_decode_noalloc: q, k, v, out and the K/V token stride must be "
              "16-byte aligned");
    return CWM_ERR_INVALID;
  }
  if (num_pages * page_size > 0x7fffffffLL) {
    set_error("paged_attn_decode_noalloc: cache of %lld rows is too large",
              (long long)(num_pages * page_size));
    return CWM_ERR_UNSUPPORTED;
  }
  void* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc != CWM_OK) return rc;
  if (decode_workspace_bytes_for(batch, hkv, kNoAllocMaxCtas) > kNoAllocScratchBytes) {
    set_error("paged_attn_decode_noalloc: %d sequences x %d KV heads exceed the built-in "
              "scratch (at most %d x %d)", batch, hkv, kNoAllocMaxBatch, kNoAllocMaxKvHeads);
    return CWM_ERR_WORKSPACE;
  }
  int* status = status_word();
  if (status == nullptr) {
    set_error("paged_attn_decode_noalloc: cannot resolve the device status word");
    return CWM_ERR_CUDA;
  }
  CUtensorMap kmap, vmap;
  const long long inner = static_cast<long long>(hkv) * d;
  const long long rows = num_pages * page_size;
  rc = get_kv_map(k, inner, rows, kv_token_stride * 2, dtype, 64, &kmap);
  if (rc != CWM_OK) return rc;
  rc = get_kv_map(v, inner, rows, kv_token_stride * 2, dtype, 64, &vmap);
  if (rc != CWM_OK) return rc;

  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q;
  a.out = out;
  a.lse = lse;
  a.cu_q = cu_seqlens_q;
  a.seq_k = seqused_k;
  a.block_table = block_table;
  a.batch = batch;
  a.hq = hq;
  a.hkv = hkv;
  a.group = hq / hkv;
  a.page_size = page_size;
  a.max_seqlen_q = 1;
  a.max_seqlen_k = max_seqlen_k;
  a.num_pages = num_pages;
  a.bt_stride = bt_stride;
  a.total_q = batch;
  a.scale_log2 = softmax_scale * 1.4426950408889634f;
  a.window_left = window_left;
  a.status = status;
  a.decode_launched = 1;
  // The arrival counters (behind the partial states) must be zero when the kernel
  // starts.  A launch that ran to its end leaves them zero, but the array is shared
  // by every caller on this device and outlives failed launches, so they are cleared
  // here on the caller's stream (a memset node, not an allocation).  The partial
  // states need no clearing: a launch reads only slots it wrote itself.
  CWM_CUDA_CHECK(cudaMemsetAsync(
      static_cast<unsigned char*>(scratch) + decode_partial_bytes(kNoAllocMaxCtas), 0,
      decode_counter_bytes(batch, hkv), static_cast<cudaStream_t>(stream)));
  return launch_decode(kmap, vmap, a, dtype == CWM_BF16, scratch,
                       static_cast<cudaStream_t>(stream), kNoAllocMaxCtas);
}
