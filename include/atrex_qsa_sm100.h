/*
 * C ABI of the sm_100a (B200) compact sparse attention launcher behind atrex.qsa_compact.
 *
 * It replaces, for the ("nvidia", "sm100") target, what the reference reaches through
 *   forward(q, k_cache, v_cache, indexer_block_ids, query_positions, block_table, token_to_req,
 *           use_prefill_config, output_gate, out, sm_scale=, v_scale=)
 * of src/nvidia/qsa/sm100/runtime.py and decode_runtime.py (called from python/atrex/api/qsa.py:62-73), in the
 * shape of the reference's only native launcher ABI (raw device pointers, a plain metadata block, a stream, an
 * int status: src/ppu/flash_attn/zwm890p/native_decode.cu:1032-1104).  Same rules as atrex_fa_sm100.h: plain C
 * types, nothing allocated or synchronised, every kernel on the caller's stream, arguments checked before any
 * launch, all index data (block ids, positions, request ids, page table) read on the device at every launch.
 *
 * Semantics (python/atrex/api/qsa.py:19-47; op_test/nvidia/qsa/test_qsa_sm100.py:65-87,154-208): row t at
 * position p sees p + 1 tokens of request token_to_req[t]; with c = min((p + 1) / 4, 512) it attends the four
 * tokens 4b .. 4b + 3 of each of its first c listed blocks b (a negative id hides the block) and the (p + 1) % 4
 * tokens of the unfinished block, which start at ((p + 1) / 4) * 4.  A token counts when the request id is in
 * [0, batch), its logical page lies inside the table row and the physical page inside the pool.
 * out = bf16( bf16( softmax(q . k * sm_scale) v * v_scale ) * sigmoid(gate) ); rows that see nothing give 0.
 */
#ifndef ATREX_QSA_SM100_H_
#define ATREX_QSA_SM100_H_

#include <stddef.h>
#include <stdint.h>

#include "atrex_fa_sm100.h" /* status codes, dtype tags, ATREX_FA_API */

#ifdef __cplusplus
extern "C" {
#endif

#define ATREX_QSA_SM100_ABI_VERSION 1
#define ATREX_QSA_SM100_TOPK 512      /* block ids per row        */
#define ATREX_QSA_SM100_HEAD_DIM 256

/* Strides are in ELEMENTS of the tensor they describe.  K and V share one set of strides (the contract requires
 * identical shapes and strides, src/nvidia/qsa/common_utils/contract.py:44-45). */
typedef struct atrex_qsa_sm100_params {
  uint32_t struct_bytes; /* sizeof(atrex_qsa_sm100_params) */
  uint32_t abi_version;  /* ATREX_QSA_SM100_ABI_VERSION    */
  const void* q;                    /* [rows, Hq, 256] BF16 or E4M3                       */
  const void* k_cache;              /* [num_pages, page_size, Hkv, 256]                   */
  const void* v_cache;
  const int32_t* block_ids;         /* [rows, 512] contiguous                             */
  const void* query_positions;      /* [rows] int32 or int64 (positions_are_int64)        */
  const int32_t* block_table;       /* [batch, table_width] contiguous                    */
  const int32_t* token_to_req;      /* [rows]                                             */
  const void* output_gate;          /* [rows, Hq, 256] BF16 contiguous                    */
  void* out;                        /* [rows, Hq, 256] BF16 contiguous                    */
  int32_t* device_status;           /* optional, as in atrex_fa_sm100_params              */
  int64_t q_row_stride, q_head_stride;
  int64_t kv_page_stride, kv_row_stride, kv_head_stride;
  int32_t rows, num_q_heads, num_kv_heads;      /* Hkv 1 or 2; Hq / Hkv 8 or 12 */
  int32_t num_pages, page_size;                  /* page_size a positive multiple of 16 */
  int32_t batch, table_width;
  int32_t dtype;                    /* ATREX_FA_BF16 or ATREX_FA_E4M3 (Q, K and V alike)  */
  int32_t positions_are_int64;
  int32_t num_splits;               /* 0 = launcher chooses, else 1..16                   */
  int32_t sm_count;                 /* 0 = query the current device                       */
  float sm_scale;                   /* merged Q.K multiplier (> 0)                        */
  float v_scale;                    /* V's dequantisation multiplier (> 0)                */
} atrex_qsa_sm100_params;

typedef struct atrex_qsa_sm100_plan_info {
  int32_t num_splits;       /* resolved split count                */
  int32_t kernel_launches;  /* kernels one forward call enqueues   */
  uint64_t workspace_bytes; /* scratch forward needs (0 unsplit, and 0 when the 2 .. 8 splits of a row run as one
                               thread-block cluster and combine inside the attention kernel) */
} atrex_qsa_sm100_plan_info;

ATREX_FA_API int atrex_qsa_sm100_abi_version(void);
ATREX_FA_API size_t atrex_qsa_sm100_params_bytes(void);
/* Validates `p` and resolves the split count from graph-static sizes (rows, heads, SM count).  Launches nothing.
 * Whether the splits combine in a cluster depends on how many clusters the CURRENT device can hold at once, so plan
 * on the device that will run the call (without a device the plan assumes the scratch path). */
ATREX_FA_API int atrex_qsa_sm100_plan(const atrex_qsa_sm100_params* p, atrex_qsa_sm100_plan_info* plan);
/* Enqueues the call on `stream`; `workspace` is caller scratch of plan.workspace_bytes, 256-byte aligned, contents
 * irrelevant.  Detail of a failure: atrex_fa_sm100_last_error(). */
ATREX_FA_API int atrex_qsa_sm100_forward(const atrex_qsa_sm100_params* p, void* workspace, uint64_t workspace_bytes,
                                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATREX_QSA_SM100_H_ */
