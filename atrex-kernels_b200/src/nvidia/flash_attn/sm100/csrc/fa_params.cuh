// Device-side view of one attention call, shared by all kernels of the sm_100a tree.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace atrex_sm100 {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Everything a kernel needs, passed by value as a __grid_constant__ argument.
// The two tensor maps describe K and V as 4-D tensors (D, Hkv, rows, pages)
// with boxes of (64 elements x 1 head x box_rows x 1 page), 128-byte swizzled.
struct alignas(64) FwdParams {
  CUtensorMap k_map;
  CUtensorMap v_map;
  // Q as (D, Hq, total_q) with a box of (64 elements x group heads x 128/group rows): one box is
  // 128 packed GQA rows of one KV head.  Only encoded for the tcgen05 route.
  CUtensorMap q_map;

  const void* q;
  void* out;
  float* lse;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  const int32_t* seqused_k;
  const int32_t* block_table;
  const float* q_descale;
  const float* k_descale;
  const float* v_descale;
  const __nv_bfloat16* sink;
  const int32_t* cp_tot_seqused_k;   // total keys per request over all context-parallel ranks (cp_world_size > 1)
  int32_t* status;

  // split-KV scratch: normalised partial O [splits, total_q, Hq, D] f32 and
  // partial log2-domain LSE [splits, total_q, Hq] f32
  float* part_o;
  float* part_lse;
  // tile plan for calls with more than one row tile per request (else null):
  // order[i] = request served i-th (heaviest first), tile_prefix[i] = number of
  // row tiles of order[0..i)
  const int32_t* order;
  const int32_t* tile_prefix;

  int64_t q_row_stride, q_head_stride;
  int64_t out_row_stride, out_head_stride;
  int64_t block_table_row_stride;
  int64_t q_descale_bs, q_descale_hs;
  int64_t k_descale_bs, k_descale_hs;
  int64_t v_descale_bs, v_descale_hs;

  int32_t batch;
  int32_t total_q;
  int32_t total_k;
  int32_t num_pages;
  int32_t page_size;   // 0 = packed K/V
  int32_t box_rows;    // rows one TMA box covers (min(page_size, 64); 64 when packed)
  int32_t num_q_heads, num_kv_heads, group;
  int32_t causal;
  int32_t window_left, window_right;  // -1 = unbounded (after causal -> right = 0)
  int32_t num_splits;
  int32_t num_row_tiles;  // upper bound of row tiles (grid sizing); batch when order == null
  int32_t q_via_tma;      // single-tile tcgen05 kernel: Q tile arrives by TMA (GQA group divides 128)
  int32_t kv_cap;         // paged: block_table width x page_size, the most keys a request's table row can name
  int32_t cp_world_size;  // context-parallel ranks (1 = off): local key j is the request's key j * world + rank
  int32_t cp_rank;
  // Tail split of the single-tile tcgen05 kernel's decode path (0 / 1 = off): the items of requests
  // [tail_first, batch) are cut into tail_splits KV splits each, all earlier items run unsplit.  With equal items
  // on a persistent grid the last round is otherwise only partly filled (512 items on 148 CTAs: 4 rounds for 3.46
  // rounds of work); splitting just the last round's items fills it, and only their rows go through the combine.
  int32_t tail_first;
  int32_t tail_splits;
  float softmax_scale;
  float softcap;
  // position (1..3, minus 1) of the head / row / page coordinate in each tensor map
  int8_t k_perm[3];
  int8_t v_perm[3];
};

// KV length and the first K row (packed K/V) of request b.  Lengths are clamped to what the caller's buffers can
// hold, so a stale or corrupt length (a graph replayed after its metadata was overwritten) never becomes an
// out-of-range page-table or row index: paged, at most the table row's width in keys; packed, at most the rows
// left in the K/V tensor.
__device__ __forceinline__ void request_kv(const FwdParams& p, int b, int& kv_len, int& k_start) {
  k_start = 0;
  if (p.cu_seqlens_k != nullptr) {
    k_start = p.cu_seqlens_k[b];
    kv_len = p.cu_seqlens_k[b + 1] - k_start;
    if (p.seqused_k != nullptr) kv_len = min(kv_len, p.seqused_k[b]);
    if (k_start < 0 || k_start > p.total_k) kv_len = 0;
    else kv_len = min(kv_len, p.total_k - k_start);
  } else {
    kv_len = min(p.seqused_k[b], p.kv_cap);
  }
  if (kv_len < 0) kv_len = 0;
}

// Distance from a query index to the last key it may see: row i of a request sees keys up to i + off.  Without
// context parallelism off = kv_len - q_len (bottom-right alignment); with it, positions are the request's global
// ones and off = total keys - q_len.
__device__ __forceinline__ int request_off(const FwdParams& p, int b, int kv_len, int q_len) {
  return (p.cp_world_size > 1 ? p.cp_tot_seqused_k[b] : kv_len) - q_len;
}

// Exclusive upper bound of the LOCAL key indices row `qi` may see when the call has a right bound
// (window_right >= 0, which causal implies); the caller clamps it to [.., kv_len].  `pos` = qi + request_off().
__device__ __forceinline__ int right_bound(const FwdParams& p, int pos) {
  if (p.cp_world_size > 1) {
    const int t = pos - p.cp_rank;               // local key j is global key j * world + rank
    return t < 0 ? 0 : t / p.cp_world_size + 1;
  }
  return pos + p.window_right + 1;
}

}  // namespace atrex_sm100
