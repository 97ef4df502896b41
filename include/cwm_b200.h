/*
 * C ABI of the B200 (sm_100a) implementation of the FastGen attention hot path.
 *
 * The reference (facebookresearch/cwm) has no FFI layer of its own: the boundary
 * of this path is the set of Python call signatures used by
 * cwm/fastgen/forward.py.  Each entry point below replaces one of them and cites
 * it.  All pointers are device pointers unless stated otherwise, all tensors are
 * owned by the caller, nothing here allocates device memory (except cwm_peer_alloc,
 * a set-up call), and every launch
 * goes to the stream given (a cudaStream_t passed as void*).  Calls are
 * asynchronous and may be captured in a CUDA graph unless stated otherwise.
 *
 * Return value: CWM_OK or a CWM_ERR_* code; cwm_last_error() gives a message for
 * the calling thread.  Conditions that the kernels detect on the device (a block
 * id outside the cache, a wait that ran out) are recorded in a status word that
 * cwm_device_status() reads back.
 */
#ifndef CWM_B200_H_
#define CWM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CWM_API __attribute__((visibility("default")))
#else
#define CWM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum cwm_status {
  CWM_OK = 0,
  CWM_ERR_INVALID = 1,     /* bad argument (shape, stride, alignment, null) */
  CWM_ERR_UNSUPPORTED = 2, /* valid but not built (head_dim, dtype, group size) */
  CWM_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed */
  CWM_ERR_WORKSPACE = 4    /* workspace missing or too small */
};

enum cwm_dtype { CWM_BF16 = 0, CWM_F16 = 1, CWM_F32 = 2 };

/* Library version (major * 100 + minor). */
CWM_API int cwm_version(void);
/* Text for a cwm_status code. */
CWM_API const char* cwm_strerror(int code);
/* Detailed message of the last failing call on this thread ("" if none). */
CWM_API const char* cwm_last_error(void);
/* Copies the device status word of the current device to *host_out and clears
 * it.  Synchronises the stream; not for use during graph capture.  Bits:
 * 1 = block id outside the cache, 2 = bounded wait ran out, 4 = bad position. */
CWM_API int cwm_device_status(int32_t* host_out, void* stream);

/* In-place rotary embedding on x[N, H, D] (interleaved pairs, fp32 math).
 * Replaces apply_rope(x, pos, freqs), cwm/fastgen/kernels/rope.py:93-163.
 * pos: int32[N]; freqs: float32[D/2]. */
CWM_API int cwm_rope(void* x, const int32_t* pos, const float* freqs, int64_t n, int h, int d, int dtype,
             void* stream);

/* out[N, D] = (x * rsqrt(mean(x^2) + eps)) * w, fp32 accumulation.
 * Replaces rmsnorm(x, w, eps), cwm/fastgen/kernels/rmsnorm.py:64-119 (and the
 * rms_norm calls of cwm/fastgen/forward.py:571,772,789).  x, w, out share dtype. */
CWM_API int cwm_rmsnorm(const void* x, const void* w, void* out, int64_t n, int d, float eps, int dtype,
                void* stream);

/* Residual add fused with the normalisation that follows it: h[N, D] += delta
 * (in place, rounded to the storage type) and out = rmsnorm(h, w, eps).  Replaces
 * the pairs h.add_(h_out); rms_norm(h, w, eps) at cwm/fastgen/forward.py:769-772
 * and :786-789 (and :571 of the next layer).  Rows must be multiples of 16 bytes,
 * 16-byte aligned, at most 32 KiB. */
CWM_API int cwm_add_rmsnorm(void* h, const void* delta, const void* w, void* out, int64_t n, int d,
                            float eps, int dtype, void* stream);

/* Scatter rows src[N, E] into a paged destination through a block table.
 * Replaces paged_memcpy(...), cwm/fastgen/kernels/paged_memcpy.py:90-228.
 * Row n goes to dst row page_tbl[b, pos / page_size] * page_size + pos % page_size
 * with b = src_batch[n] (n if null) and pos = dst_pos[n]; rows n >= *batch_size
 * are skipped when batch_size is given (an int32 or int64 device scalar).  With
 * shard_cnt > 1 only pos % shard_cnt == shard_idx is stored, at pos / shard_cnt.
 * Strides are in elements.  dst_rows bounds the destination: a row outside it is
 * not written and sets status bit 1. */
CWM_API int cwm_paged_memcpy(const void* src, void* dst, const int32_t* page_tbl, const int32_t* dst_pos,
                     const int32_t* src_batch /* nullable */, const void* batch_size /* nullable */,
                     int batch_size_is_i64, int64_t n, int64_t e, int elem_bytes, int page_size,
                     int64_t page_tbl_stride, int64_t page_tbl_cols, int64_t dst_stride,
                     int64_t dst_rows, int shard_idx, int shard_cnt, void* stream);

/* Fused form of the four calls at cwm/fastgen/forward.py:618-632: rotate
 * xq[T, Hq, D] and xk[T, Hkv, D] in place, then store the rotated k rows and the
 * xv rows into cache_k / cache_v (row stride cache_stride elements, heads
 * contiguous in a row) at the paged position of each token.  Same addressing and
 * batch_size rule as cwm_paged_memcpy (the rotation itself is unconditional, as
 * in the reference).  xq may be null (k/v only). */
CWM_API int cwm_rope_kv_write(void* xq, void* xk, const void* xv, void* cache_k, void* cache_v,
                      const int32_t* pos, const float* freqs, const int32_t* page_tbl,
                      const int32_t* src_batch /* nullable */,
                      const void* batch_size /* nullable */, int batch_size_is_i64, int64_t t,
                      int hq, int hkv, int d, int dtype, int page_size, int64_t page_tbl_stride,
                      int64_t page_tbl_cols, int64_t cache_stride, int64_t cache_rows,
                      void* stream);

/* The same step for a runner that computes the three projections as ONE product
 * (wq | wk | wv stacked): qkv[t, :] = [q heads | k heads | v heads] with row stride
 * qkv_stride elements.  Replaces the views, the two apply_rope calls and the two
 * paged_memcpy calls of cwm/fastgen/forward.py:608-632: the rotated queries go to
 * q_out[T, hq, d] (contiguous), the rotated keys and the values straight to their
 * pages; qkv itself is only read. */
CWM_API int cwm_qkv_rope_kv_write(const void* qkv, int64_t qkv_stride, void* q_out, void* cache_k,
                                  void* cache_v, const int32_t* pos, const float* freqs,
                                  const int32_t* page_tbl, const int32_t* src_batch /* nullable */,
                                  const void* batch_size /* nullable */, int batch_size_is_i64,
                                  int64_t t, int hq, int hkv, int d, int dtype, int page_size,
                                  int64_t page_tbl_stride, int64_t page_tbl_cols,
                                  int64_t cache_stride, int64_t cache_rows, void* stream);

/* out[t, i] = silu(x13[t, i]) * x13[t, ffn + i] for x13[T, 2 * ffn] (the stacked
 * w1 | w3 product), each step rounded to the storage type like the pair
 * F.silu(x1, inplace=True).mul_(x3) at cwm/fastgen/forward.py:776-781. */
CWM_API int cwm_silu_mul(const void* x13, void* out, int64_t t, int64_t ffn, int dtype,
                         void* stream);

/* Bytes of scratch that cwm_paged_attn_fwd needs for this problem size (split-KV
 * partial results and arrival counters of the decode kernel).  Depends on static
 * sizes only; grows with batch * hkv.  The workspace must be zero-filled once after
 * it is allocated.  Every call that completes leaves the part that matters (the
 * counters) zero again, so one workspace can serve later calls of any batch size
 * up to the one it was sized for (on one stream, or otherwise ordered) and
 * CUDA-graph replays, without clearing.  Zero-fill it again after a call for which
 * cwm_device_status reported bit 2. */
CWM_API size_t cwm_paged_attn_workspace_bytes(int batch, int64_t total_q, int hq, int hkv, int d);

/* Self-test hooks (process-wide, for the library's own tests; not part of the
 * reference's interface).  wait_limit_cycles: limit of the bounded waits inside the
 * attention kernels, in SM clock cycles (<= 0 restores the default of about two
 * seconds).  drop_last_tile != 0: the loader warp of every CTA withholds the loads
 * of its last K/V tile, so that the waits for that tile run out and the kernels take
 * their give-up path (status bit 2, output invalid) instead of computing; no memory
 * access is made that a normal launch would not make.  Applies to launches made
 * after the call. */
CWM_API int cwm_test_hooks(long long wait_limit_cycles, int drop_last_tile);

/* Variable-length paged-KV grouped-query attention, causal, with an optional
 * sliding window.  Replaces the call
 *   mha_fwd(query, key, value, cu_seqlens_q, None, seqused_k, None, max_seqlen_q,
 *           max_seqlen_k, 0, block_table, softmax_scale, True, window_left, -1)
 * at cwm/fastgen/forward.py:639-655 (xformers.ops.fmha.flash3.mha_fwd).
 *
 * q, out: [total_q, hq, d], contiguous.  k, v: element (page, tok, head, :) lives
 * at base + ((page * page_size + tok) * kv_token_stride + head * d) elements,
 * i.e. the strided views FastGen makes of its [K|V] cache rows.  Sequence b has
 * queries cu_seqlens_q[b] .. cu_seqlens_q[b+1] and seqused_k[b] keys; query j of
 * t sits at position seqused_k[b] - t + j and sees keys
 * max(0, pos - window_left) .. pos (window_left < 0: from 0).  Query head h uses
 * KV head h / (hq / hkv).  block_table: int32 [batch, *] with row stride
 * bt_stride; only the first ceil(seqused_k[b] / page_size) entries of a row are
 * read.  lse (nullable): float32 [hq, total_q], natural log.  All lengths are
 * read on the device, so the launch is valid for any lengths within the static
 * bounds max_seqlen_q / max_seqlen_k.  Sequences with one query are served by
 * the split-KV decode kernel, the others by the tensor-core prefill kernel.
 *
 * Limits (CWM_ERR_UNSUPPORTED otherwise): d == 128; bf16 or fp16; hq / hkv <= 8;
 * page_size a multiple of 64; num_pages * page_size < 2^31; batch up to about
 * 1300 sequences (the schedulers keep one int per sequence in shared memory).
 * max_seqlen_q must be at least the true maximum of the query counts: when
 * total_q == batch * max_seqlen_q > batch the decode kernel is not launched at
 * all, and the prefill kernel checks the number of query blocks against it.  A
 * call whose lengths break this promise sets status bit 4 and may have computed
 * only part of the output.  Keys at or beyond
 * seqused_k[b] are never used by the decode kernel, whatever their pages hold;
 * the prefill kernel multiplies the V rows of masked keys of a partly used tile
 * by zero, so the cache pages it touches must hold finite values (a cache that
 * starts zero-filled, as the reference's does, always qualifies).
 * workspace: see cwm_paged_attn_workspace_bytes for its one requirement. */
CWM_API int cwm_paged_attn_fwd(const void* q, const void* k, const void* v, void* out,
                       float* lse /* nullable */, const int32_t* cu_seqlens_q,
                       const int32_t* seqused_k, const int32_t* block_table, int batch,
                       int64_t total_q, int hq, int hkv, int d, int dtype, int page_size,
                       int64_t num_pages, int64_t kv_token_stride, int64_t bt_stride,
                       int max_seqlen_q, int max_seqlen_k, float softmax_scale, int window_left,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Largest batch cwm_paged_attn_decode_noalloc accepts. */
#define CWM_NOALLOC_MAX_BATCH 1024

/* Decode attention (one query per sequence) without any caller-provided scratch.
 * No counterpart in the reference: it exists for embedders that cannot allocate
 * device memory at call time -- a host application that hands a plugin a fixed
 * set of buffers, a serving loop whose memory plan is frozen, a thread that must
 * not touch the allocator.  Arguments are those of cwm_paged_attn_fwd with
 * total_q == batch and max_seqlen_q == 1 (cu_seqlens_q is 0, 1, ..., batch); the
 * split-KV scratch is a fixed array of about 2.7 MB inside the library image,
 * which every GPU that loads the library holds until the process exits.
 *
 * Limits: batch <= CWM_NOALLOC_MAX_BATCH and hkv <= 16, otherwise
 * CWM_ERR_WORKSPACE.  The call performs no cudaMalloc/cudaFree and calls no
 * allocating library routine; it clears the few KB of the array that must start
 * at zero with a memset on the caller's stream.  The
 * first call on each device looks up the address of the array (and, like any
 * first launch, lets the CUDA runtime load the kernels), so make that first
 * call before starting a stream capture.  All calls on a device share the one
 * array: two calls that can overlap on the GPU (different streams without an
 * ordering between them) race and give wrong results; calls on one stream are
 * safe.  The array keeps the previous call's contents, which no call relies on
 * (the part that must be zero is cleared by every call). */
CWM_API int cwm_paged_attn_decode_noalloc(const void* q, const void* k, const void* v, void* out,
                                          float* lse /* nullable */, const int32_t* cu_seqlens_q,
                                          const int32_t* seqused_k, const int32_t* block_table,
                                          int batch, int hq, int hkv, int d, int dtype,
                                          int page_size, int64_t num_pages,
                                          int64_t kv_token_stride, int64_t bt_stride,
                                          int max_seqlen_k, float softmax_scale, int window_left,
                                          void* stream);

/* Copies n cache blocks in one launch: block i is `rows` rows of row_bytes bytes, read
 * from src_ptrs[i] with row pitch src_pitch_bytes and written to dst_ptrs[i] with row
 * pitch dst_pitch_bytes.  dst_ptrs / src_ptrs are device-readable arrays of
 * addresses; the addresses may point into device memory or into pinned host memory
 * (the copy then runs over the host link without a copy-engine call per block).
 * Replaces the per-lane, per-block copy_ loops of DynCache.page_in / page_out,
 * cwm/fastgen/utils/cache.py:227-235 and :251-257.  Rows and pitches in multiples of
 * 16 bytes, 16-byte aligned addresses, n <= 65535. */
CWM_API int cwm_block_copy(const uint64_t* dst_ptrs, const uint64_t* src_ptrs, int64_t n,
                           int64_t rows, int64_t row_bytes, int64_t dst_pitch_bytes,
                           int64_t src_pitch_bytes, void* stream);

/* Sum all-reduce over the GPUs of one node through peer memory, for the row-parallel
 * products of a tensor-parallel layer (the custom all-reduce that
 * Collectives.all_reduce prefers below 8 MiB, cwm/fastgen/utils/collectives.py:28-45,
 * 73-88).  Every rank calls it with the same n_elems, in the same order, on a stream
 * that is behind the producer of its input.  in: n_elems local elements (left
 * unchanged).  scratch_ptrs / result_ptrs / flag_ptrs are HOST arrays of `world`
 * device addresses, entry p being rank p's buffer as this process can address it (its
 * own allocation for p == rank, an IPC mapping otherwise):
 *   scratch  n_elems elements;
 *   result   n_elems elements: when the call has run, result_ptrs[rank] holds the sum
 *            (the same bits on every rank); it is overwritten by the next call that
 *            is given the same buffers;
 *   flags    cwm_allreduce_flag_ints() int32, zero-filled once when allocated.
 * epoch: two local int32 {1, 0} set once at allocation and owned by the library
 * afterwards.  n_elems must be a multiple of 8 * world; bf16 or fp16 with fp32
 * accumulation in rank order.  Waits on peers are bounded; one that runs out sets
 * status bit 2.  Calls that share scratch and flags must not overlap (one stream, or
 * otherwise ordered). */
CWM_API int cwm_allreduce(const void* in, const uint64_t* scratch_ptrs,
                          const uint64_t* result_ptrs, const uint64_t* flag_ptrs, int32_t* epoch,
                          int64_t n_elems, int dtype, int rank, int world, void* stream);

/* The all-reduce above fused with what a tensor-parallel decoder layer does with its
 * result: h += sum (rounded to the storage type, as the reference's all_reduce then
 * add_ give), out = rmsnorm(h) * w.  Replaces
 *   all_reduce(h_out); h = h + h_out; x = rms_norm(h, w, eps)
 * of cwm/fastgen/forward.py:763-772 and :782-789 (collectives.py:73-88 for the
 * all-reduce).  in: [rows, d] local partial product.  Rank p sums rows
 * p * rows / world .. (p + 1) * rows / world - 1, adds them to THOSE rows of its local
 * h (the other rows of h are left as they are: with this entry point the residual
 * stream lives sharded by rows, each rank keeping its own rows current), normalises
 * them and writes the normalised rows into every rank's result buffer, which then
 * holds all of out = [rows, d], the same bits on every rank and the same bits as the
 * three separate calls give.  rows % world == 0; d * element size a multiple of 16
 * bytes and at most 32 KiB; buffers, epoch, bounded waits and ordering rules as for
 * cwm_allreduce (scratch and result need rows * d elements). */
CWM_API int cwm_allreduce_add_rmsnorm(const void* in, void* h, const void* w,
                                      const uint64_t* scratch_ptrs, const uint64_t* result_ptrs,
                                      const uint64_t* flag_ptrs, int32_t* epoch, int64_t rows,
                                      int d, float eps, int dtype, int rank, int world,
                                      void* stream);
CWM_API int cwm_allreduce_flag_ints(void);
CWM_API int cwm_allreduce_ctas(int64_t n_elems, int world);

/* Set-up of the buffers that cwm_allreduce shares between the processes of a node
 * (the only entry points of this library that allocate device memory; call them once
 * at start-up).  cwm_peer_alloc: cudaMalloc of `bytes` zero-filled bytes on the current
 * device plus its 64-byte CUDA IPC handle, to be sent to the other processes by any
 * host channel.  cwm_peer_open: maps a peer's buffer into this process with the
 * caller's device current (this is what enables peer access from the caller's GPU to
 * the owner's); the owner must outlive the mapping.  cwm_peer_close unmaps,
 * cwm_peer_free releases an own buffer: close every mapping on every process, meet at
 * a barrier, then free. */
CWM_API int cwm_peer_alloc(size_t bytes, void** ptr, void* handle64);
CWM_API int cwm_peer_open(const void* handle64, void** ptr);
CWM_API int cwm_peer_close(void* ptr);
CWM_API int cwm_peer_free(void* ptr);

/* Token sampling over x[rows, vocab] (fp32, row stride row_stride elements): one
 * launch does what FastGen._sample does with several torch calls,
 * cwm/fastgen/generate.py:996-1014 with cwm/fastgen/utils/sampling.py:6-45.
 *   is_logits != 0: x holds logits and the probabilities are
 *     softmax(x / temps[row]) (temps null: 1); otherwise x holds probabilities.
 *   mode 0: greedy, tokens[row] = first index of the row maximum (torch.argmax).
 *   mode 1: a draw in index order, the distribution of sample(probs)
 *     (sampling.py:6-18): the first index whose inclusive running sum exceeds
 *     uniforms[row] * total.
 *   mode 2: top_p(probs, top_ps) (sampling.py:21-45): entries in descending order
 *     (equal values by ascending index), those whose exclusive running sum exceeds
 *     top_ps[row] are dropped (top_ps null or >= 1: none), the rest renormalised,
 *     and the draw is the first survivor whose inclusive running sum exceeds
 *     uniforms[row] * (surviving mass).
 * uniforms[row] in [0, 1) stands in for torch.multinomial's generator, so that the
 * caller controls the stream of random numbers and every tensor-parallel rank
 * draws the same token.  probs[row] receives the probability of the drawn token
 * after renormalisation (1 for mode 0); kept (nullable) the number of surviving
 * entries.  Sums are kept in 2^-44 fixed point: results do not depend on thread
 * timing.  vocab <= 131072 for modes 1 and 2. */
CWM_API int cwm_sample(const float* x, int is_logits, const float* temps /* nullable */,
                       const float* top_ps /* nullable */, const float* uniforms, int64_t rows,
                       int64_t vocab, int64_t row_stride, int mode, int64_t* tokens, float* probs,
                       int32_t* kept /* nullable */, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CWM_B200_H_ */
