// Split-KV combine and the row-tile plan.
//
// combine: O = sum_i w_i O_i / sum_i w_i with w_i = 2^(lse_i - max lse), where
// O_i are normalised FP32 partials and lse_i their log2-domain LSE; a split that
// saw no key publishes lse = -inf and its O is never read (it may be NaN
// scratch).  The sink logit joins as one more weight with O = 0.  Same algebra
// as the reference's reducers (src/nvidia/flash_attn/sm103/decode_reduce_cutedsl.py:71-152,
// src/nvidia/flash_attn/sm120/decode_reduce.py:63-176), one warp per output row.
//
// plan: orders requests by KV length (longest first) and prefix-sums their
// row-tile counts on the device, so grids never depend on lengths read by the
// host.  Counterpart of the reference's device-side split plan
// (src/ppu/flash_attn/zwm890p/native_decode.cu:714-900) and LPT tile order
// (src/nvidia/flash_attn/sm103/prefill_cutedsl.py:814-846).
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace atrex_sm100 {

namespace {

constexpr int kCombineWarps = 8;

template <int D>
__global__ void __launch_bounds__(kCombineWarps * 32)
atrex_sm100_combine_kernel(const __grid_constant__ FwdParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row_id = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);  // q_row * Hq + head
  const int64_t live_rows = (int64_t)min(p.cu_seqlens_q[p.batch], p.total_q) * p.num_q_heads;
  if (row_id >= live_rows) return;
  const int head = (int)(row_id % p.num_q_heads);
  const int64_t q_row = row_id / p.num_q_heads;
  // tail split: the rows of the requests before tail_first were written in final form by the attention kernel
  if (p.tail_splits > 1 && q_row < p.cu_seqlens_q[p.tail_first]) return;
  const int64_t split_stride = (int64_t)p.total_q * p.num_q_heads;

  float mx = -INFINITY;
  for (int s = lane; s < p.num_splits; s += 32) mx = fmaxf(mx, p.part_lse[s * split_stride + row_id]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sink_l2 = -INFINITY;
  if (p.sink != nullptr) sink_l2 = __bfloat162float(p.sink[head]) * kLog2e;
  const float m_f = fmaxf(mx, sink_l2);
  const float m_use = m_f == -INFINITY ? 0.f : m_f;

  constexpr int V = D / 32;  // contiguous floats per lane
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  float wsum = 0.f;
  for (int s = 0; s < p.num_splits; ++s) {
    const float lse = p.part_lse[s * split_stride + row_id];  // warp-uniform
    if (lse == -INFINITY) continue;
    const float w = fast_exp2(lse - m_use);
    wsum += w;
    const float* src = p.part_o + (s * split_stride + row_id) * D + lane * V;
#pragma unroll
    for (int i = 0; i < V; i += 4) {
      const float4 x = *reinterpret_cast<const float4*>(src + i);
      acc[i] += w * x.x; acc[i + 1] += w * x.y; acc[i + 2] += w * x.z; acc[i + 3] += w * x.w;
    }
  }
  if (sink_l2 != -INFINITY) wsum += fast_exp2(sink_l2 - m_use);
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + q_row * p.out_row_stride +
                       (int64_t)head * p.out_head_stride + lane * V;
#pragma unroll
  for (int i = 0; i < V; i += 4) {
    uint2 packed;
    packed.x = pack_bf16(acc[i] * inv, acc[i + 1] * inv);
    packed.y = pack_bf16(acc[i + 2] * inv, acc[i + 3] * inv);
    *reinterpret_cast<uint2*>(dst + i) = packed;
  }
  if (lane == 0 && p.lse != nullptr)
    p.lse[(int64_t)head * p.total_q + q_row] = wsum > 0.f ? (m_use + log2f(wsum)) * kLn2 : -INFINITY;
}

constexpr int kPlanThreads = 1024;
constexpr int kPlanSortMax = 4096;  // requests ordered by length up to this batch; identity order beyond

__global__ void __launch_bounds__(kPlanThreads)
atrex_sm100_plan_kernel(const __grid_constant__ FwdParams p, int m_rows, int32_t* order, int32_t* tile_prefix) {
  __shared__ unsigned long long keys[kPlanSortMax];
  __shared__ int scan[kPlanThreads];
  const int tid = threadIdx.x;
  const int B = p.batch;
  const bool sorted = B <= kPlanSortMax;
  if (sorted) {
    int n = 1;
    while (n < B) n <<= 1;
    for (int i = tid; i < n; i += kPlanThreads) {
      unsigned long long key = 0ull;  // padding sorts last
      if (i < B) {
        int kv_len, k_start;
        request_kv(p, i, kv_len, k_start);
        const int q_len = p.cu_seqlens_q[i + 1] - p.cu_seqlens_q[i];
        // cost class: keys a causal row tile walks, then query rows; index keeps the order stable
        key = ((unsigned long long)(unsigned)min(kv_len, 0xFFFFF) << 44) |
              ((unsigned long long)(unsigned)min(max(q_len, 0), 0xFFFFF) << 24) |
              (unsigned long long)(0xFFFFFF - i);
      }
      keys[i] = key;
    }
    __syncthreads();
    for (int k = 2; k <= n; k <<= 1) {       // bitonic sort, descending
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < n; i += kPlanThreads) {
          const int partner = i ^ j;
          if (partner > i) {
            const bool desc = (i & k) == 0;
            const unsigned long long a = keys[i], c = keys[partner];
            if (desc ? a < c : a > c) { keys[i] = c; keys[partner] = a; }
          }
        }
        __syncthreads();
      }
    }
    for (int i = tid; i < B; i += kPlanThreads) order[i] = 0xFFFFFF - (int)(keys[i] & 0xFFFFFFull);
  } else {
    for (int i = tid; i < B; i += kPlanThreads) order[i] = i;
  }
  __syncthreads();
  // exclusive prefix sum of row tiles in served order, kPlanThreads requests per pass
  int carry = 0;
  for (int base = 0; base < B; base += kPlanThreads) {
    const int i = base + tid;
    int tiles = 0;
    if (i < B) {
      const int b = order[i];
      const int rows = (p.cu_seqlens_q[b + 1] - p.cu_seqlens_q[b]) * p.group;
      tiles = rows > 0 ? (rows + m_rows - 1) / m_rows : 0;
    }
    scan[tid] = tiles;
    __syncthreads();
    for (int o = 1; o < kPlanThreads; o <<= 1) {
      const int add = tid >= o ? scan[tid - o] : 0;
      __syncthreads();
      scan[tid] += add;
      __syncthreads();
    }
    if (i < B) tile_prefix[i] = carry + scan[tid] - tiles;
    carry += scan[kPlanThreads - 1];
    __syncthreads();
  }
  if (tid == 0) tile_prefix[B] = carry;
}

// Merge of attention computed over disjoint key sets by different ranks (context parallelism): parts
// [W, total_q, Hq, D] BF16 with natural-log LSE [W, Hq, total_q] -> out [total_q, Hq, D] BF16, lse [Hq, total_q].
// One warp per (query row, head); same algebra as the split combine above, natural-log domain, BF16 partials.
// A part with LSE = -inf has weight 0 and its output row (possibly NaN) is not read.
__global__ void __launch_bounds__(kCombineWarps * 32)
atrex_sm100_merge_parts_kernel(const __nv_bfloat16* __restrict__ parts, const float* __restrict__ part_lse,
                               __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int world, int64_t total_q,
                               int num_q_heads, int head_dim) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);   // (query, head), head fastest
  if (row >= total_q * num_q_heads) return;
  const int64_t q = row / num_q_heads;
  const int h = (int)(row - q * num_q_heads);
  const int64_t lse_stride = (int64_t)num_q_heads * total_q, lse_off = (int64_t)h * total_q + q;
  float mx = -INFINITY;
  for (int w = 0; w < world; ++w) mx = fmaxf(mx, part_lse[w * lse_stride + lse_off]);
  float denom = 0.f;
  float acc[8];                                            // head_dim <= 256: 8 elements per lane
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const int per_lane = head_dim / 32;
  if (mx != -INFINITY) {
    for (int w = 0; w < world; ++w) {
      const float l = part_lse[w * lse_stride + lse_off];
      if (l == -INFINITY) continue;
      const float wgt = __expf(l - mx);
      denom += wgt;
      const __nv_bfloat16* src = parts + ((int64_t)w * total_q * num_q_heads + row) * head_dim + lane * per_lane;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < per_lane) acc[i] += wgt * __bfloat162float(src[i]);
    }
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  __nv_bfloat16* dst = out + row * head_dim + lane * per_lane;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < per_lane) dst[i] = __float2bfloat16(acc[i] * inv);
  if (lane == 0) lse[lse_off] = denom > 0.f ? mx + __logf(denom) : -INFINITY;
}

}  // namespace

cudaError_t combine_launch(const FwdParams& p, int head_dim, cudaStream_t stream) {
  const int64_t rows = (int64_t)p.total_q * p.num_q_heads;
  if (rows == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((rows + kCombineWarps - 1) / kCombineWarps);
  if (head_dim == 128)
    return launch_kernel(atrex_sm100_combine_kernel<128>, dim3(grid), dim3(kCombineWarps * 32), 0, stream, p);
  return launch_kernel(atrex_sm100_combine_kernel<256>, dim3(grid), dim3(kCombineWarps * 32), 0, stream, p);
}

cudaError_t plan_launch(const FwdParams& p, int m_rows, int32_t* order, int32_t* tile_prefix,
                        cudaStream_t stream) {
  return launch_kernel(atrex_sm100_plan_kernel, dim3(1), dim3(kPlanThreads), 0, stream, p, m_rows, order,
                       tile_prefix);
}

cudaError_t merge_parts_launch(const void* parts, const float* part_lse, void* out, float* lse, int world,
                               int64_t total_q, int num_q_heads, int head_dim, cudaStream_t stream) {
  const int64_t rows = total_q * num_q_heads;
  if (rows == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((rows + kCombineWarps - 1) / kCombineWarps);
  return launch_kernel(atrex_sm100_merge_parts_kernel, dim3(grid), dim3(kCombineWarps * 32), 0, stream,
                       static_cast<const __nv_bfloat16*>(parts), part_lse, static_cast<__nv_bfloat16*>(out), lse, world,
                       total_q, num_q_heads, head_dim);
}

}  // namespace atrex_sm100
