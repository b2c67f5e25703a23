// Entry points each kernel translation unit gives the C-ABI launcher.
#pragma once
#include <atomic>

#include <cuda_bf16.h>

#include "fa_params.cuh"

namespace atrex_sm100 {

// Launch through cudaLaunchKernelEx and report ITS status: the kernel<<<>>> +
// cudaGetLastError idiom would also pick up an unrelated stale error left in the
// calling thread by other code.
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

// ---- launcher.cu: shared by every entry point of the library ----
// Record the detail text of a failure for atrex_fa_sm100_last_error() on this thread and return `status`.
int report_failure(int status, const char* what, cudaError_t cuda = cudaSuccess);
void clear_failure();
// SM count of the current device; fails with ATREX_FA_WRONG_DEVICE unless it is compute capability 10.0.
int current_sm_count(int* sm_count);

// ---- fa_mma.cu: split-KV mma.sync kernel ----
int mma_rows_for(int packed_rows);            // 16, 32 or 64 rows per CTA
int mma_tile_n(int head_dim);                 // KV tokens per pipeline stage
cudaError_t mma_prepare();                    // per-device kernel attributes
cudaError_t mma_launch(const FwdParams& p, int head_dim, int m_rows, cudaStream_t stream);

// ---- fa_umma.cu: tcgen05 prefill kernel (BF16, head_dim 128) ----
bool umma_supports(int head_dim, int group, int dtype_is_bf16);
int umma_rows_per_item();                     // packed rows one work item covers (256)
cudaError_t umma_prepare();
cudaError_t umma_launch(const FwdParams& p, int sm_count, cudaStream_t stream);

// ---- fa_umma1.cu: single-row-tile tcgen05 kernel (head_dim 128 / 256, BF16 / FP8 E4M3, optional split-KV) ----
bool umma1_supports(int head_dim);
bool umma1_q_via_tma(int group);              // else the softmax warpgroup copies Q rows itself
int umma1_rows_per_item();                    // 128
int umma1_tile_n(int head_dim, bool fp8);     // keys per KV tile
cudaError_t umma1_prepare();
cudaError_t umma1_launch(const FwdParams& p, int head_dim, bool fp8, int sm_count, cudaStream_t stream);

// ---- fa_combine.cu: merge split partials; tile plan ----
cudaError_t combine_launch(const FwdParams& p, int head_dim, cudaStream_t stream);
// merge of per-rank (O, natural-log LSE) pairs computed over disjoint key sets (context parallelism)
cudaError_t merge_parts_launch(const void* parts, const float* part_lse, void* out, float* lse, int world,
                               int64_t total_q, int num_q_heads, int head_dim, cudaStream_t stream);
// order[batch], tile_prefix[batch + 1] for row tiles of m_rows packed rows
cudaError_t plan_launch(const FwdParams& p, int m_rows, int32_t* order, int32_t* tile_prefix,
                        cudaStream_t stream);

// ---- kv_write.cu: scatter of new K/V rows into the paged pools (optional BF16 -> E4M3 quantisation) ----
// Strides in elements of the respective tensor; scales are per KV head (head stride 0 = one scale per tensor).
struct KvWriteParams {
  const __nv_bfloat16* key;
  const __nv_bfloat16* value;
  void* key_cache;
  void* value_cache;
  const long long* slot_mapping;
  const float* k_scale;
  const float* v_scale;
  long long k_token_stride, k_head_stride, v_token_stride, v_head_stride;
  long long kc_page_stride, kc_row_stride, kc_head_stride, vc_page_stride, vc_row_stride, vc_head_stride;
  long long k_scale_head_stride, v_scale_head_stride;
  int num_tokens, num_kv_heads, head_dim, page_size;
  long long slot_limit;   // num_pages * page_size when the caller gave the pool size, else the largest value
};
cudaError_t kv_write_launch(const KvWriteParams& p, bool fp8, int sm_count, cudaStream_t stream);
// Per-head E4M3 scales (max |x| / 448) of the rows a write would store; `amax` is 2 * num_kv_heads words of scratch.
cudaError_t kv_scales_launch(const KvWriteParams& p, unsigned* amax, float* k_scale, float* v_scale, int sm_count,
                             cudaStream_t stream);

}  // namespace atrex_sm100
