// Sum all-reduce of a small activation tensor over the GPUs of one node, as one
// kernel over peer memory (NVLink / NVSwitch stores), for the row-parallel products
// of a tensor-parallel decoder layer.
//
// The reference engine sends these messages (batch x 6144 bf16 = 1.5 MB in decode)
// through a custom all-reduce below 8 MiB and through NCCL otherwise
// (cwm/fastgen/utils/collectives.py:28-45,73-88).  At this size the cost is latency,
// so the exchange is built from posted remote *stores* (one way across the switch)
// rather than remote loads (a round trip each):
//   1. every rank pushes slice p of its input into rank p's scratch (slot = sender),
//      then raises a flag at rank p;
//   2. rank p, once the flags of all senders are up, sums the slots of its scratch
//      in rank order with fp32 accumulation (local reads) and pushes the rounded
//      slice into every rank's result buffer, then raises a second flag everywhere;
//   3. a rank returns when the second flags of all ranks are up: its result buffer
//      is complete, and bit-identical to every other rank's.
// No "input ready" round is needed (a rank pushes its own data), and the flags carry
// an epoch that each launch advances, so nothing is ever reset and the launch can be
// replayed from a CUDA graph.  Each CTA synchronises with the CTA of the same index
// on the other ranks only, through its own flag slots.  Every wait is bounded; one
// that runs out sets status bit 2 and the kernel returns.  Buffer reuse is safe
// without further rounds: a rank starts its next call only after it has received
// every rank's reduced slice, i.e. after every rank has finished reading the
// scratch this rank will push into next.
#include <string.h>

#include <type_traits>

#include "common.cuh"

namespace cwm {
namespace {

constexpr int kArThreads = 256;
constexpr int kArMaxCtas = 128;
constexpr int kArMaxWorld = 8;
constexpr long long kArSpinLimit = 1ll << 24;  // polls of a flag before giving up

struct ArArgs {
  const uint4* in;                  // local input
  uint4* scratch[kArMaxWorld];      // every rank's scratch: [world slots][slice]
  uint4* result[kArMaxWorld];       // every rank's result buffer
  int* flags[kArMaxWorld];          // every rank's flags: [2 rounds][kArMaxCtas][kArMaxWorld]
  int* epoch;                       // local: [0] epoch of this launch, [1] CTAs finished
  int* status;
  long long slice_vecs;  // 16-byte vectors per rank's slice
  int rank;
  int world;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread t < world tells rank t "my part of this round is written", then waits for
// rank t's word.  Returns false (for the whole CTA) when a wait ran out.
__device__ __forceinline__ bool flag_round(const ArArgs& a, int round, int epoch) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __threadfence_system();  // this thread's pushes are ordered before the flags below
  __syncthreads();         // ... and so are every other thread's of the CTA
  if (threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    const int slot = (round * kArMaxCtas + blockIdx.x) * kArMaxWorld;
    st_release_sys(a.flags[peer] + slot + a.rank, epoch);
    const int* mine = a.flags[a.rank] + slot + peer;
    long long polls = 0;
    while (ld_acquire_sys(mine) != epoch) {
      if (++polls > kArSpinLimit) {
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  return failed == 0;
}

template <bool kBf16>
__device__ __forceinline__ void accumulate(float (&acc)[8], uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (kBf16) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      acc[2 * i] += __low2float(h);
      acc[2 * i + 1] += __high2float(h);
    }
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kArThreads) allreduce_kernel(const ArArgs a) {
  const int epoch = *a.epoch;
  const long long first = static_cast<long long>(blockIdx.x) * kArThreads + threadIdx.x;
  const long long step = static_cast<long long>(gridDim.x) * kArThreads;
  // ---- 1. push slice p of my input into rank p's scratch, slot = my rank
  for (long long i = first; i < a.slice_vecs; i += step) {
    uint4 v[kArMaxWorld];
#pragma unroll
    for (int p = 0; p < kArMaxWorld; ++p) {
      if (p < a.world) v[p] = a.in[static_cast<long long>(p) * a.slice_vecs + i];
    }
#pragma unroll
    for (int p = 0; p < kArMaxWorld; ++p) {
      if (p < a.world) a.scratch[p][static_cast<long long>(a.rank) * a.slice_vecs + i] = v[p];
    }
  }
  bool ok = flag_round(a, 0, epoch);
  // ---- 2. sum my slice over the senders in rank order, push the result everywhere
  if (ok) {
    const uint4* mine = a.scratch[a.rank];
    for (long long i = first; i < a.slice_vecs; i += step) {
      uint4 v[kArMaxWorld];
#pragma unroll
      for (int p = 0; p < kArMaxWorld; ++p) {
        if (p < a.world) v[p] = mine[static_cast<long long>(p) * a.slice_vecs + i];
      }
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int p = 0; p < kArMaxWorld; ++p) {
        if (p < a.world) accumulate<kBf16>(acc, v[p]);
      }
      uint4 r;
      r.x = pack2<kBf16>(acc[0], acc[1]);
      r.y = pack2<kBf16>(acc[2], acc[3]);
      r.z = pack2<kBf16>(acc[4], acc[5]);
      r.w = pack2<kBf16>(acc[6], acc[7]);
#pragma unroll
      for (int p = 0; p < kArMaxWorld; ++p) {
        if (p < a.world) a.result[p][static_cast<long long>(a.rank) * a.slice_vecs + i] = r;
      }
    }
    // ---- 3. my result buffer is complete when every rank's slice has landed
    ok = flag_round(a, 1, epoch);
  }
  if (!ok && threadIdx.x == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
  // ---- the last CTA to finish advances the epoch for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.epoch + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      a.epoch[1] = 0;
      a.epoch[0] = epoch + 1;
    }
  }
}


// ---- all-reduce fused with the residual add and the RMSNorm that follow it ------------
// In a tensor-parallel decoder layer the reduced product is used once: it is added to
// the residual stream and the sum is normalised (cwm/fastgen/forward.py:763-772,
// 782-789).  Rank p reduces whole rows here (rows p * R .. p * R + R - 1 of the
// message, R = rows / world), so it can do both on the spot: it adds the rounded sum
// to *its own rows* of the residual stream, normalises them and pushes the normalised
// rows to every rank.  Only the normalised activations are gathered; the residual
// stream stays sharded by rows (nothing else reads the other rows).  Roundings and
// the order of every sum are those of all-reduce, then add, then rmsnorm_kernel in
// helpers.cu (same thread-to-vector mapping, same reduction), so the result is bit
// for bit the one of the three separate steps.
struct ArNormArgs {
  ArArgs ar;
  uint4* h;        // local residual stream [rows, d]; rows of this rank's slice are updated
  const uint4* w;  // [d] norm weight
  int rows_per_rank;
  int row_vecs;  // 16-byte vectors per row
  float inv_d;
  float eps;
};

constexpr int kNormMaxVpt = 8;

template <bool kBf16>
__global__ void __launch_bounds__(256) allreduce_add_rmsnorm_kernel(const ArNormArgs n) {
  using T = typename std::conditional<kBf16, __nv_bfloat16, __half>::type;
  const ArArgs& a = n.ar;
  const int epoch = *a.epoch;
  const int rv = n.row_vecs;
  // ---- 1. push rows blockIdx.x, blockIdx.x + gridDim.x, ... of every slice to its owner
  for (int r = blockIdx.x; r < n.rows_per_rank; r += gridDim.x) {
    for (int idx = threadIdx.x; idx < rv; idx += blockDim.x) {
      uint4 v[kArMaxWorld];
#pragma unroll
      for (int p = 0; p < kArMaxWorld; ++p) {
        if (p < a.world) {
          v[p] = a.in[(static_cast<long long>(p) * n.rows_per_rank + r) * rv + idx];
        }
      }
#pragma unroll
      for (int p = 0; p < kArMaxWorld; ++p) {
        if (p < a.world) {
          a.scratch[p][(static_cast<long long>(a.rank) * n.rows_per_rank + r) * rv + idx] = v[p];
        }
      }
    }
  }
  bool ok = flag_round(a, 0, epoch);
  // ---- 2. my rows: sum over the senders in rank order, add to the residual stream,
  // normalise, push the normalised rows everywhere
  if (ok) {
    __shared__ float warp_sums[32];
    __shared__ float rstd_s;
    const uint4* mine = a.scratch[a.rank];
    for (int r = blockIdx.x; r < n.rows_per_rank; r += gridDim.x) {
      const long long grow = static_cast<long long>(a.rank) * n.rows_per_rank + r;
      uint4 regs[kNormMaxVpt];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kNormMaxVpt; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < rv) {
          uint4 v[kArMaxWorld];
#pragma unroll
          for (int p = 0; p < kArMaxWorld; ++p) {
            if (p < a.world) v[p] = mine[(static_cast<long long>(p) * n.rows_per_rank + r) * rv + idx];
          }
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int p = 0; p < kArMaxWorld; ++p) {
            if (p < a.world) accumulate<kBf16>(acc, v[p]);
          }
          uint4 d;  // the all-reduce result, rounded to the storage type
          d.x = pack2<kBf16>(acc[0], acc[1]);
          d.y = pack2<kBf16>(acc[2], acc[3]);
          d.z = pack2<kBf16>(acc[4], acc[5]);
          d.w = pack2<kBf16>(acc[6], acc[7]);
          regs[i] = n.h[grow * rv + idx];
          T* e = reinterpret_cast<T*>(&regs[i]);
          const T* de = reinterpret_cast<const T*>(&d);
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(__fadd_rn(to_f32(e[j]), to_f32(de[j])));
          n.h[grow * rv + idx] = regs[i];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float x = to_f32(e[j]);
            ss = fmaf(x, x, ss);
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      __syncthreads();  // warp_sums and rstd_s of the row before are no longer read
      if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) rstd_s = rsqrtf(t * n.inv_d + n.eps);
      }
      __syncthreads();
      const float rstd = rstd_s;
#pragma unroll
      for (int i = 0; i < kNormMaxVpt; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < rv) {
          const uint4 wv = n.w[idx];
          const T* we = reinterpret_cast<const T*>(&wv);
          T* e = reinterpret_cast<T*>(&regs[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            e[j] = from_f32<T>(__fmul_rn(__fmul_rn(to_f32(e[j]), rstd), to_f32(we[j])));
          }
#pragma unroll
          for (int p = 0; p < kArMaxWorld; ++p) {
            if (p < a.world) a.result[p][grow * rv + idx] = regs[i];
          }
        }
      }
    }
    // ---- 3. my result buffer is complete when every rank's rows have landed
    ok = flag_round(a, 1, epoch);
  }
  if (!ok && threadIdx.x == 0) atomicOr(a.status, DEV_WAIT_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.epoch + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      a.epoch[1] = 0;
      a.epoch[0] = epoch + 1;
    }
  }
}

}  // namespace
}  // namespace cwm

using namespace cwm;

extern "C" int cwm_allreduce_ctas(int64_t n_elems, int world) {
  if (n_elems <= 0 || world <= 0) return 0;
  const long long slice_vecs = n_elems / 8 / world;
  long long ctas = (slice_vecs + kArThreads - 1) / kArThreads;
  if (ctas < 1) ctas = 1;
  if (ctas > kArMaxCtas) ctas = kArMaxCtas;
  return static_cast<int>(ctas);
}

extern "C" int cwm_allreduce_flag_ints(void) { return 2 * kArMaxCtas * kArMaxWorld; }

extern "C" int cwm_allreduce(const void* in, const uint64_t* scratch_ptrs,
                             const uint64_t* result_ptrs, const uint64_t* flag_ptrs,
                             int32_t* epoch, int64_t n_elems, int dtype, int rank, int world,
                             void* stream) {
  if (n_elems == 0) return CWM_OK;
  if (!in || !scratch_ptrs || !result_ptrs || !flag_ptrs || !epoch) {
    set_error("allreduce: null pointer");
    return CWM_ERR_INVALID;
  }
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || n_elems < 0) {
    set_error("allreduce: bad rank / world (at most %d ranks)", kArMaxWorld);
    return CWM_ERR_INVALID;
  }
  if (dtype != CWM_BF16 && dtype != CWM_F16) {
    set_error("allreduce: bf16 and fp16 only");
    return CWM_ERR_UNSUPPORTED;
  }
  if (n_elems % (8ll * world) != 0 || reinterpret_cast<uintptr_t>(in) % 16 != 0) {
    set_error("allreduce: %lld elements must split into 16-byte vectors over %d ranks, and the "
              "input must be 16-byte aligned", static_cast<long long>(n_elems), world);
    return CWM_ERR_UNSUPPORTED;
  }
  ArArgs a;
  memset(&a, 0, sizeof(a));
  for (int p = 0; p < world; ++p) {
    if (scratch_ptrs[p] % 16 || result_ptrs[p] % 16 || flag_ptrs[p] % 4 || !scratch_ptrs[p] ||
        !result_ptrs[p] || !flag_ptrs[p]) {
      set_error("allreduce: peer buffer %d is null or misaligned", p);
      return CWM_ERR_INVALID;
    }
    a.scratch[p] = reinterpret_cast<uint4*>(scratch_ptrs[p]);
    a.result[p] = reinterpret_cast<uint4*>(result_ptrs[p]);
    a.flags[p] = reinterpret_cast<int*>(flag_ptrs[p]);
  }
  a.in = static_cast<const uint4*>(in);
  a.epoch = epoch;
  a.status = status_word();
  if (a.status == nullptr) {
    set_error("allreduce: cannot resolve the device status word");
    return CWM_ERR_CUDA;
  }
  a.slice_vecs = n_elems / 8 / world;
  a.rank = rank;
  a.world = world;
  const int ctas = cwm_allreduce_ctas(n_elems, world);
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == CWM_BF16) {
    allreduce_kernel<true><<<ctas, kArThreads, 0, st>>>(a);
  } else {
    allreduce_kernel<false><<<ctas, kArThreads, 0, st>>>(a);
  }
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

extern "C" int cwm_allreduce_add_rmsnorm(const void* in, void* h, const void* w,
                                         const uint64_t* scratch_ptrs, const uint64_t* result_ptrs,
                                         const uint64_t* flag_ptrs, int32_t* epoch, int64_t rows,
                                         int d, float eps, int dtype, int rank, int world,
                                         void* stream) {
  if (rows == 0) return CWM_OK;
  if (!in || !h || !w || !scratch_ptrs || !result_ptrs || !flag_ptrs || !epoch) {
    set_error("allreduce_add_rmsnorm: null pointer");
    return CWM_ERR_INVALID;
  }
  if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world || rows < 0 || d <= 0) {
    set_error("allreduce_add_rmsnorm: bad rank / world (at most %d ranks) or shape", kArMaxWorld);
    return CWM_ERR_INVALID;
  }
  if (dtype != CWM_BF16 && dtype != CWM_F16) {
    set_error("allreduce_add_rmsnorm: bf16 and fp16 only");
    return CWM_ERR_UNSUPPORTED;
  }
  const int row_vecs = d / 8;
  const int threads = row_vecs >= 512 ? 256 : 128;  // as rmsnorm_kernel, for the same sums
  if (rows % world != 0 || d % 8 != 0 || row_vecs > threads * kNormMaxVpt ||
      reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(h) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(w) % 16 != 0) {
    set_error("allreduce_add_rmsnorm: %lld rows must split evenly over %d ranks, rows must be "
              "16-byte multiples of at most 32 KiB, tensors 16-byte aligned",
              static_cast<long long>(rows), world);
    return CWM_ERR_UNSUPPORTED;
  }
  ArNormArgs n;
  memset(&n, 0, sizeof(n));
  ArArgs& a = n.ar;
  for (int p = 0; p < world; ++p) {
    if (scratch_ptrs[p] % 16 || result_ptrs[p] % 16 || flag_ptrs[p] % 4 || !scratch_ptrs[p] ||
        !result_ptrs[p] || !flag_ptrs[p]) {
      set_error("allreduce_add_rmsnorm: peer buffer %d is null or misaligned", p);
      return CWM_ERR_INVALID;
    }
    a.scratch[p] = reinterpret_cast<uint4*>(scratch_ptrs[p]);
    a.result[p] = reinterpret_cast<uint4*>(result_ptrs[p]);
    a.flags[p] = reinterpret_cast<int*>(flag_ptrs[p]);
  }
  a.in = static_cast<const uint4*>(in);
  a.epoch = epoch;
  a.status = status_word();
  if (a.status == nullptr) {
    set_error("allreduce_add_rmsnorm: cannot resolve the device status word");
    return CWM_ERR_CUDA;
  }
  a.rank = rank;
  a.world = world;
  n.rows_per_rank = static_cast<int>(rows / world);
  a.slice_vecs = static_cast<long long>(n.rows_per_rank) * row_vecs;
  n.row_vecs = row_vecs;
  n.h = static_cast<uint4*>(h);
  n.w = static_cast<const uint4*>(w);
  n.inv_d = 1.0f / static_cast<float>(d);
  n.eps = eps;
  const int ctas = n.rows_per_rank < kArMaxCtas ? n.rows_per_rank : kArMaxCtas;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == CWM_BF16) {
    allreduce_add_rmsnorm_kernel<true><<<ctas, threads, 0, st>>>(n);
  } else {
    allreduce_add_rmsnorm_kernel<false><<<ctas, threads, 0, st>>>(n);
  }
  CWM_CUDA_CHECK(cudaGetLastError());
  return CWM_OK;
}

// ---- buffers that other processes of the node can map (CUDA IPC) ---------------------
// Allocated with cudaMalloc outside any framework allocator, so that the IPC handle
// names exactly this allocation, and opened with the *caller's* device current, which
// is what makes the runtime enable peer access from the caller's GPU to the owner's.
extern "C" int cwm_peer_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) {
    set_error("peer_alloc: bad argument");
    return CWM_ERR_INVALID;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  CWM_CUDA_CHECK(cudaMalloc(&p, bytes));
  cudaError_t err = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err != cudaSuccess) {
    cudaFree(p);
    set_error("peer_alloc: %s", cudaGetErrorString(err));
    return CWM_ERR_CUDA;
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return CWM_OK;
}

extern "C" int cwm_peer_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) {
    set_error("peer_open: bad argument");
    return CWM_ERR_INVALID;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  CWM_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return CWM_OK;
}

extern "C" int cwm_peer_close(void* ptr) {
  if (ptr) CWM_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return CWM_OK;
}

extern "C" int cwm_peer_free(void* ptr) {
  if (ptr) CWM_CUDA_CHECK(cudaFree(ptr));
  return CWM_OK;
}
