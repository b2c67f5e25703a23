/*
 * C ABI of the sm_100a (B200) FlashAttention launcher behind
 * atrex.flash_attn_varlen_func.
 *
 * This is the boundary a host-side binding links against.  It replaces, for the
 * ("nvidia", "sm100") target, what the reference reaches through its private
 * Python ABI `forward(**kwargs) -> (out, lse)` (python/atrex/api/flash_attn.py:395-421)
 * and follows the shape of the reference's only native launcher,
 *   int atrex_ppu_decode(void** pointers, int64_t* metadata, float scale, int splits, void* stream)
 *   int atrex_ppu_decode_resources(int* out)
 * (src/ppu/flash_attn/zwm890p/native_decode.cu:1032-1104, 1106-1120):
 * raw device pointers, a plain metadata block, a CUDA stream, an int status.
 *
 * Rules every entry point keeps:
 *   - plain C types only; no exceptions cross the boundary; 0 means success;
 *   - nothing is allocated or freed and the device is never synchronised;
 *   - all device work is enqueued on the caller's stream, so the call can be
 *     captured into a CUDA graph (lengths, page tables and descales are read on
 *     the device at every launch);
 *   - arguments are range-checked before anything is launched
 *     (native_decode.cu:1035-1043 does the same and returns InvalidValue).
 */
#ifndef ATREX_FA_SM100_H_
#define ATREX_FA_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATREX_FA_SM100_ABI_VERSION 5

#if defined(__GNUC__)
#define ATREX_FA_API __attribute__((visibility("default")))
#else
#define ATREX_FA_API
#endif

enum atrex_fa_status {
  ATREX_FA_OK = 0,
  ATREX_FA_INVALID_VALUE = 1,      /* malformed call            -> ValueError          */
  ATREX_FA_UNSUPPORTED = 2,        /* well formed, not served   -> NotImplementedError */
  ATREX_FA_WORKSPACE_TOO_SMALL = 3,
  ATREX_FA_CUDA_ERROR = 4,         /* a CUDA runtime/driver call failed -> RuntimeError */
  ATREX_FA_WRONG_DEVICE = 5,       /* current device is not compute capability 10.0     */
  ATREX_FA_ABI_MISMATCH = 6
};

enum atrex_fa_dtype { ATREX_FA_BF16 = 0, ATREX_FA_E4M3 = 1 };

/* Kernel family.  AUTO lets the launcher choose from graph-static sizes only. */
enum atrex_fa_route {
  ATREX_FA_ROUTE_AUTO = 0,
  ATREX_FA_ROUTE_MMA = 1,     /* split-KV mma.sync kernel (+ combine): short-Q decode, compatibility prefill */
  ATREX_FA_ROUTE_UMMA = 2     /* warp-specialised TMA + tcgen05 prefill                                       */
};

/*
 * One attention call.  Field meaning follows the keyword arguments of the
 * reference's private ABI (python/atrex/api/flash_attn.py:396-420) and the
 * fields of its native DecodeParams (native_decode.cu:28-74), widened to the
 * whole contract.  Strides are in ELEMENTS of the tensor they describe.
 * Unused pointers are NULL.
 */
typedef struct atrex_fa_sm100_params {
  uint32_t struct_bytes;   /* sizeof(atrex_fa_sm100_params) as the caller sees it */
  uint32_t abi_version;    /* ATREX_FA_SM100_ABI_VERSION                          */

  const void* q;           /* [total_q, Hq, D]                                              */
  const void* k;           /* paged [num_pages, page_size, Hkv, D] or packed [total_k,Hkv,D] */
  const void* v;
  void* out;               /* [total_q, Hq, D] BF16                                          */
  float* lse;              /* [Hq, total_q] natural log, or NULL                             */
  const int32_t* cu_seqlens_q;  /* [batch+1]                                                 */
  const int32_t* cu_seqlens_k;  /* [batch+1] packed K/V only, else NULL                      */
  const int32_t* seqused_k;     /* [batch]; required when paged.  Packed K/V: optional, and when  */
                                /* given the used length is min(cu_seqlens_k[b+1]-cu_seqlens_k[b], seqused_k[b]) */
  const int32_t* block_table;   /* [batch, max_pages_per_seq] or NULL for packed K/V         */
  const float* q_descale;       /* [batch, Hkv] FP8 only, or NULL                            */
  const float* k_descale;
  const float* v_descale;
  const void* sink;             /* BF16 [Hq] sink logits (s_aux) or NULL                     */
  int32_t* device_status;       /* optional: kernels store a nonzero code here if a bounded wait expires */
  void* profile_event_begin;    /* benchmark hook: optional cudaEvent_t pair recorded on the stream right    */
  void* profile_event_end;      /* before and after the dominant kernel of the call (not the plan or combine */
                                /* kernels).  Production callers pass NULL for both.                         */
  const int32_t* cp_tot_seqused_k;  /* [batch] total keys of each request over all context-parallel ranks;   */
                                    /* read only when cp_world_size > 1, else NULL                            */

  int64_t q_row_stride, q_head_stride;
  int64_t k_page_stride, k_row_stride, k_head_stride;   /* page stride ignored for packed K/V */
  int64_t v_page_stride, v_row_stride, v_head_stride;
  int64_t out_row_stride, out_head_stride;
  int64_t block_table_row_stride;
  int64_t q_descale_batch_stride, q_descale_head_stride;  /* may be 0 (broadcast views) */
  int64_t k_descale_batch_stride, k_descale_head_stride;
  int64_t v_descale_batch_stride, v_descale_head_stride;

  int32_t batch;
  int32_t total_q;
  int32_t total_k;             /* rows of packed K/V; 0 when paged */
  int32_t num_pages;           /* pool size when paged             */
  int32_t page_size;           /* 0 = packed K/V                   */
  int32_t max_pages_per_seq;   /* block_table width; a seqused_k above max_pages_per_seq * page_size is clamped to it */
  int32_t max_seqlen_q;        /* upper bounds only: real lengths are read on the device */
  int32_t max_seqlen_k;
  int32_t num_q_heads, num_kv_heads, head_dim;
  int32_t dtype;               /* enum atrex_fa_dtype of q/k/v     */
  int32_t causal;
  int32_t window_left, window_right;   /* -1 = unbounded                  */
  int32_t return_lse;
  int32_t num_splits;          /* 0 = launcher chooses, else 1..256 */
  int32_t route;               /* enum atrex_fa_route               */
  int32_t sm_count;            /* 0 = query the current device      */
  /* Context parallelism over the keys (no counterpart in the reference, which rejects these arguments:
   * python/atrex/api/flash_attn.py:128-135).  Rank r of W holds every W-th key of each request: its local key j
   * is the request's key j * W + r, seqused_k holds the LOCAL lengths and cp_tot_seqused_k the totals.  A query
   * row i of a request of q_len rows sits at position tot - q_len + i and sees local key j iff
   * j * W + r <= tot - q_len + i.  The caller merges the ranks' (out, lse) with atrex_fa_sm100_merge_parts.
   * cp_world_size 0 or 1 = off.  Causal calls without a sliding window only. */
  int32_t cp_world_size, cp_rank;
  float softmax_scale;
  float softcap;               /* 0 = off                           */
} atrex_fa_sm100_params;

/* What the launcher will do for a call: filled by atrex_fa_sm100_plan. */
typedef struct atrex_fa_sm100_plan_info {
  int32_t route;            /* resolved enum atrex_fa_route                     */
  int32_t num_splits;       /* resolved split count (>= 1)                      */
  int32_t kernel_launches;  /* kernels one forward call enqueues                */
  int32_t m_rows;           /* packed (query x group) rows per CTA tile         */
  uint64_t workspace_bytes; /* scratch the caller must pass to forward (may be 0) */
} atrex_fa_sm100_plan_info;

/* ABI handshake: callers compare these with their own header. */
ATREX_FA_API int atrex_fa_sm100_abi_version(void);
ATREX_FA_API size_t atrex_fa_sm100_params_bytes(void);

/* English text for a status code; never NULL. */
ATREX_FA_API const char* atrex_fa_sm100_status_string(int status);

/*
 * Detail of the last non-zero status returned on the calling thread (which check
 * failed, or which CUDA call with its error string); empty if there was none.
 * The reference reports launcher failures the same way, as text in the raised
 * RuntimeError (src/ppu/flash_attn/zwm890p/decode_runtime.py:108-113).
 */
ATREX_FA_API const char* atrex_fa_sm100_last_error(void);

/*
 * Pure host query (counterpart of atrex_ppu_decode_resources,
 * native_decode.cu:1106-1120): validates `p`, resolves route and split count
 * from graph-static sizes (batch, heads, max_seqlen_*, SM count) and reports the
 * scratch size.  Launches nothing.
 */
ATREX_FA_API int atrex_fa_sm100_plan(const atrex_fa_sm100_params* p, atrex_fa_sm100_plan_info* plan);

/*
 * Enqueue one attention call on `stream` (a cudaStream_t).  `workspace` is
 * caller-owned device scratch of at least plan.workspace_bytes, 256-byte
 * aligned; its contents on entry are irrelevant and may be NaN.  Replaces
 * `forward(**kwargs)` of the reference's per-arch launch modules
 * (src/nvidia/flash_attn/sm103/launch.py:282-311) and, in shape,
 * atrex_ppu_decode (native_decode.cu:1032-1104).
 */
ATREX_FA_API int atrex_fa_sm100_forward(const atrex_fa_sm100_params* p, void* workspace, uint64_t workspace_bytes,
                           void* stream);

/*
 * One-time per-device set-up (kernel attributes such as the dynamic shared
 * memory limit).  forward() does it on first use; calling it explicitly keeps
 * that work out of a latency-sensitive first call.  Counterpart of the
 * reference's compile-before-capture rule (src/nvidia/flash_attn/sm103/launch.py:155-241).
 */
ATREX_FA_API int atrex_fa_sm100_prewarm(void);

/*
 * Same as atrex_fa_sm100_forward, for callers that cannot provide scratch memory.
 * This entry point has no counterpart in the reference.  It exists for hosts that
 * cannot allocate on the device: an FFI binding that only receives device pointers
 * from another runtime and owns no allocator, a server whose HBM was handed
 * entirely to its KV-cache pool at start-up, or a latency-critical loop that must
 * not call cudaMalloc / cudaFree because they synchronise the device.
 *
 * The split-KV scratch comes from a fixed array inside the library
 * (ATREX_FA_SM100_STATIC_SCRATCH_BYTES per GPU, held by every GPU that loads the
 * library until the process exits).  A call whose plan needs more returns
 * ATREX_FA_WORKSPACE_TOO_SMALL and launches nothing; atrex_fa_sm100_last_error()
 * then names both sizes.  The call allocates and frees nothing, in this library or
 * through any other.
 *
 * The first call on a device looks up the array's device address; make that first
 * call (or any call of this function on that device) before starting a stream
 * capture.  The address is remembered per device for the life of the process: after
 * a cudaDeviceReset the remembered address is stale, so a process that resets a
 * device must not call this entry point on it again.  All calls on one device share the one array and it keeps the previous
 * call's contents: nothing in it needs clearing between calls, but two calls whose
 * kernels can overlap on the GPU (different streams without an ordering between
 * them) race on it and must be serialised by the caller.
 */
#define ATREX_FA_SM100_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
ATREX_FA_API uint64_t atrex_fa_sm100_static_scratch_bytes(void);
ATREX_FA_API int atrex_fa_sm100_forward_static_scratch(const atrex_fa_sm100_params* p, void* stream);

/*
 * KV-cache write path: the step before attention in the caller.  Scatters the new key / value rows
 * of a step, `key`, `value` [num_tokens, num_kv_heads, head_dim] BF16, into the paged pools that
 * atrex_fa_sm100_forward reads (`k`, `v` of atrex_fa_sm100_params with the same page / row / head
 * strides): token t goes to page slot_mapping[t] / page_size, row slot_mapping[t] % page_size; a
 * negative slot skips the token.  cache_dtype ATREX_FA_BF16 copies; ATREX_FA_E4M3 stores
 * e4m3(x / scale[head]) rounded to nearest even and saturated to +-448, where k_scale / v_scale are
 * device FP32 arrays indexed head * scale_head_stride (stride 0: one scale for the tensor; NULL: 1.0)
 * and are the descales the attention call is then given for that head.
 *
 * The reference has no writer: its tests fill caches by indexing
 * (op_test/utils/flash_attn_contract.py:40-51; op_test/nvidia/flash_attn/test_flash_attn_sm120.py:236-244)
 * and its stride rules (src/nvidia/flash_attn/sm120/launch.py:231-251) define the layouts a writer has
 * to produce; all of them are expressible with the strides below.
 *
 * All strides are in ELEMENTS of their tensor.  head_dim is a multiple of 8 (16 for an E4M3 cache);
 * every base pointer and every stride times its element size is 16-byte aligned for BF16 tensors and
 * 8-byte aligned for an E4M3 cache.  Nothing is allocated; one kernel is enqueued on `stream`.
 */
typedef struct atrex_fa_sm100_kv_write_params {
  uint32_t struct_bytes; /* sizeof(atrex_fa_sm100_kv_write_params) */
  uint32_t abi_version;  /* ATREX_FA_SM100_ABI_VERSION */
  const void* key;
  const void* value;
  void* key_cache;
  void* value_cache;
  const int64_t* slot_mapping; /* [num_tokens] */
  const float* k_scale;
  const float* v_scale;
  int64_t key_token_stride, key_head_stride, value_token_stride, value_head_stride;
  int64_t key_cache_page_stride, key_cache_row_stride, key_cache_head_stride;
  int64_t value_cache_page_stride, value_cache_row_stride, value_cache_head_stride;
  int64_t k_scale_head_stride, v_scale_head_stride;
  int32_t num_tokens, num_kv_heads, head_dim, page_size;
  int32_t cache_dtype; /* ATREX_FA_BF16 or ATREX_FA_E4M3 */
  int32_t num_pages;   /* pages in the pools: a slot >= num_pages * page_size is skipped like a negative one; 0 = unchecked */
} atrex_fa_sm100_kv_write_params;

ATREX_FA_API size_t atrex_fa_sm100_kv_write_params_bytes(void);
ATREX_FA_API int atrex_fa_sm100_kv_cache_write(const atrex_fa_sm100_kv_write_params* p, void* stream);

/*
 * Scales for an E4M3 cache, computed from the rows the write is about to store: k_scale_out[h] and
 * v_scale_out[h] (device FP32 [num_kv_heads]) = max |x| over the non-padding tokens of head h / 448, 1.0 for
 * a head without a finite non-zero value.  Only key, value, slot_mapping, their strides and the sizes of
 * `p` are read (the cache fields and cache_dtype are ignored).  `scratch` is 8 * num_kv_heads bytes of
 * device memory, 4-byte aligned, contents irrelevant.  Enqueues a memset and two kernels on `stream`;
 * allocates nothing.  The results feed atrex_fa_sm100_kv_cache_write (k_scale / v_scale, head stride 1)
 * and then the attention call's k_descale / v_descale.
 */
ATREX_FA_API int atrex_fa_sm100_kv_scales(const atrex_fa_sm100_kv_write_params* p, float* k_scale_out,
                                          float* v_scale_out, void* scratch, void* stream);

/*
 * Context parallelism, the merge step: `parts` [world, total_q, num_q_heads, head_dim] BF16 and `part_lse`
 * [world, num_q_heads, total_q] FP32 natural log are the outputs of atrex_fa_sm100_forward (with return_lse) of
 * `world` ranks that each attended a disjoint shard of every request's keys, gathered into this GPU's memory
 * (e.g. by an NCCL all-gather).  Writes out [total_q, num_q_heads, head_dim] BF16 and lse [num_q_heads, total_q]:
 * out = sum_w exp(lse_w - lse) out_w, lse = logsumexp_w lse_w; a part with lse = -inf is not read.  All tensors
 * dense; head_dim a multiple of 32 up to 256.  Same algebra as the split-KV combine
 * (src/nvidia/flash_attn/sm103/decode_reduce_cutedsl.py:71-152), across ranks instead of across splits.  The
 * reference rejects context parallelism (python/atrex/api/flash_attn.py:128-135); this has no counterpart there.
 */
ATREX_FA_API int atrex_fa_sm100_merge_parts(const void* parts, const float* part_lse, void* out, float* lse,
                                            int32_t world, int64_t total_q, int32_t num_q_heads, int32_t head_dim,
                                            void* stream);

/*
 * Context parallelism, exchange and merge as ONE kernel over peer memory (no counterpart in the reference).
 * Rank `rank` of `world` (<= 8) calls this after its attention call (atrex_fa_sm100_forward with cp_world_size,
 * return_lse) has been enqueued on `stream`.  parts[w] / part_lse[w] are rank w's O [total_q, num_q_heads,
 * head_dim] BF16 and LSE [num_q_heads, total_q] FP32 as THIS process addresses them (its own buffers for
 * w == rank, peer mappings - CUDA IPC, a symmetric-memory allocation - for the others); counters[w] is rank w's
 * array of 8 uint32 step counters in such memory too, zero before the first step.  `step` is the same on all
 * ranks for one exchange and grows by one per exchange.  The kernel stores `step` into slot `rank` of every
 * rank's counters, waits until all slots of its own array have reached `step`, then reads every rank's pair with
 * plain loads and writes out [total_q, num_q_heads, head_dim] BF16 and lse [num_q_heads, total_q]:
 * out = sum_w exp(lse_w - lse) out_w, lse = logsumexp_w lse_w; a part whose lse is -inf is not read.
 * The wait is bounded: if a peer never arrives, 106 is stored in *device_status and nothing is written.
 * The caller keeps the peers from overwriting parts[w] while slower ranks still read them: with two alternating
 * buffers a rank that has passed exchange n + 1 knows that exchange n was finished everywhere.
 * With all pointers on one GPU and every counter already at `step` the call is a plain merge (how a one-GPU
 * test emulates the ranks).  head_dim 128 or 256; parts and out 16-byte aligned.  Allocates nothing.
 */
typedef struct atrex_fa_sm100_cp_merge_params {
  uint32_t struct_bytes; /* sizeof(atrex_fa_sm100_cp_merge_params) */
  uint32_t abi_version;  /* ATREX_FA_SM100_ABI_VERSION */
  const void* parts[8];
  const float* part_lse[8];
  uint32_t* counters[8];
  void* out;
  float* lse;
  int32_t* device_status; /* optional */
  int64_t total_q;
  int32_t num_q_heads, head_dim, world, rank;
  uint32_t step;
  uint32_t reserved;
} atrex_fa_sm100_cp_merge_params;
ATREX_FA_API int atrex_fa_sm100_cp_merge(const atrex_fa_sm100_cp_merge_params* p, void* stream);

/*
 * Self-test of the bounded device-side wait (no counterpart in the reference; its precedent for a wait
 * with a limit is _tma_mbarrier_try_wait_parity(..., time_limit), src/nvidia/flash_attn/sm120/attention_cutedsl.py:2434).
 * Every wait inside the kernels gives up after an iteration limit, stores a code in
 * atrex_fa_sm100_params.device_status and lets its kernel return.  This entry point exercises exactly that
 * path: one thread waits at most `spin_limit` (1..65536) polls on a barrier that nobody arrives at, then
 * stores 104 (wait expired) in *device_status (may be NULL) and 0 in *result (1 would mean the barrier
 * completed), and the kernel returns normally.  One tiny kernel on `stream`; allocates nothing.
 */
ATREX_FA_API int atrex_fa_sm100_selftest_bounded_wait(int32_t* device_status, int32_t* result, uint32_t spin_limit,
                                                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATREX_FA_SM100_H_ */
