// KV-cache write path: scatter the new K and V rows of a step into the paged pools the attention
// kernels read, optionally quantising BF16 -> FP8 E4M3 on the way.
//
// This is the step immediately before attention in the caller.  The reference has no such operator:
// its tests build caches by indexing (op_test/utils/flash_attn_contract.py:40-51) and its stride
// rules (src/nvidia/flash_attn/sm120/launch.py:231-251) define the layouts a writer must produce --
// interleaved K|V pools, token-strided pages, head-major views -- all of which are "any page / row /
// head stride" here.  Semantics follow the serving engines' reshape-and-cache step: token t goes to
// slot slot_mapping[t] = page * page_size + row (negative: skip); with an FP8 cache,
// stored = e4m3_rn_satfinite(x / scale[head]) and `scale` is the descale the attention call is
// given for that head.
//
// HBM-bound byte work: one warp per (tensor, token), 16-byte vectors (8 BF16) on consecutive lanes so
// that loads and stores are whole 128-byte lines, four vectors per lane in flight.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fa_kernels.cuh"
#include "softmax_math.cuh"

namespace atrex_sm100 {

namespace {

constexpr int kWriteThreads = 256;
constexpr int kInFlight = 4;

// x / s correctly rounded, from the correctly rounded reciprocal r = RN(1/s) (Markstein's sequence: q0 = x r,
// remainder by one exact FMA, one corrective FMA), two elements per instruction (f32x2): three FMA-pipe
// instructions per PAIR instead of a full IEEE division per element, with one reciprocal per vector.  The
// cases the sequence does not cover -- quotients that overflow or are denormal -- are above E4M3's
// saturation point or below its smallest step either way; an overflowed first estimate is kept as it is
// (+-inf saturates; the correction would be inf - inf).
__device__ __forceinline__ uint32_t quotients_e4m3x2(uint32_t bf16_pair, f32x2 s2, f32x2 neg_s2, f32x2 r2) {
  const f32x2 x2 = pack2(__uint_as_float(bf16_pair << 16), __uint_as_float(bf16_pair & 0xffff0000u));
  const f32x2 q0 = mul2(x2, r2);
  const f32x2 rem = fma2(q0, neg_s2, x2);
  const f32x2 q = fma2(rem, r2, q0);
  float a0, a1, b0, b1;
  unpack2(q0, a0, a1);
  unpack2(q, b0, b1);
  b0 = fabsf(a0) <= 3.0e38f ? b0 : a0;
  b1 = fabsf(a1) <= 3.0e38f ? b1 : a1;
  return __nv_cvt_float2_to_fp8x2(make_float2(b0, b1), __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ uint2 quantise8(uint4 raw, float s) {
  const float r = __frcp_rn(s);
  const f32x2 s2 = pack2(s, s), neg_s2 = pack2(-s, -s), r2 = pack2(r, r);
  const uint32_t lo0 = quotients_e4m3x2(raw.x, s2, neg_s2, r2), hi0 = quotients_e4m3x2(raw.y, s2, neg_s2, r2);
  const uint32_t lo1 = quotients_e4m3x2(raw.z, s2, neg_s2, r2), hi1 = quotients_e4m3x2(raw.w, s2, neg_s2, r2);
  return make_uint2(lo0 | (hi0 << 16), lo1 | (hi1 << 16));
}

// One warp per (tensor, token): the slot lookup and the page arithmetic happen once per token, the
// lanes then move the token's num_kv_heads * head_dim / 8 vectors, kInFlight loads ahead of the stores.
template <bool kFp8>
__global__ void __launch_bounds__(kWriteThreads) atrex_sm100_kv_write_kernel(const KvWriteParams p) {
  const int lane = threadIdx.x & 31;
  const int vec_per_row = p.head_dim >> 3;                 // 16-byte vectors per (token, head) row
  const int vec_per_tok = p.num_kv_heads * vec_per_row;
  const int row_shift = (vec_per_row & (vec_per_row - 1)) == 0 ? __ffs(vec_per_row) - 1 : -1;   // power of two: shift
  const long long units = 2ll * p.num_tokens;              // K tokens, then V tokens
  const long long warps = (long long)gridDim.x * (kWriteThreads / 32);
  for (long long unit = (long long)blockIdx.x * (kWriteThreads / 32) + (threadIdx.x >> 5); unit < units; unit += warps) {
    const int which = unit >= p.num_tokens;
    const long long tok = unit - (which ? p.num_tokens : 0);
    const long long slot = __ldg(p.slot_mapping + tok);
    if (slot < 0) continue;                                // padding token (warp-uniform)
    const long long page = slot / p.page_size, in_page = slot - page * p.page_size;
    const __nv_bfloat16* src = (which ? p.value : p.key) + tok * (which ? p.v_token_stride : p.k_token_stride);
    const long long src_head = which ? p.v_head_stride : p.k_head_stride;
    const long long dst_head = which ? p.vc_head_stride : p.kc_head_stride;
    const long long dst_tok = which ? page * p.vc_page_stride + in_page * p.vc_row_stride
                                    : page * p.kc_page_stride + in_page * p.kc_row_stride;
    uint8_t* cache = reinterpret_cast<uint8_t*>(which ? p.value_cache : p.key_cache);
    const float* scales = which ? p.v_scale : p.k_scale;
    const long long scale_stride = which ? p.v_scale_head_stride : p.k_scale_head_stride;
    for (int v0 = lane; v0 < vec_per_tok; v0 += 32 * kInFlight) {
      uint4 raw[kInFlight];
      int head[kInFlight], vec[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int v = v0 + u * 32;
        head[u] = row_shift >= 0 ? v >> row_shift : v / vec_per_row;
        vec[u] = v - head[u] * vec_per_row;
        if (v < vec_per_tok) raw[u] = __ldg(reinterpret_cast<const uint4*>(src + head[u] * src_head + vec[u] * 8));
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        if (v0 + u * 32 >= vec_per_tok) continue;
        const long long off = dst_tok + head[u] * dst_head + vec[u] * 8;     // in cache elements
        if (kFp8) {
          const float scale = scales ? __ldg(scales + head[u] * scale_stride) : 1.f;
          *reinterpret_cast<uint2*>(cache + off) = quantise8(raw[u], scale);
        } else {
          *reinterpret_cast<uint4*>(cache + off * 2) = raw[u];
        }
      }
    }
  }
}

}  // namespace

cudaError_t kv_write_launch(const KvWriteParams& p, bool fp8, int sm_count, cudaStream_t stream) {
  const long long units = 2ll * p.num_tokens;
  if (units == 0) return cudaSuccess;
  const int warps_per_cta = kWriteThreads / 32;
  long long ctas = (units + warps_per_cta - 1) / warps_per_cta;
  const long long cap = (long long)sm_count * 8;   // 8 resident CTAs of 256 threads per SM, then the warps stride on
  if (ctas > cap) ctas = cap;
  if (fp8) return launch_kernel(atrex_sm100_kv_write_kernel<true>, dim3((unsigned)ctas), dim3(kWriteThreads), 0, stream, p);
  return launch_kernel(atrex_sm100_kv_write_kernel<false>, dim3((unsigned)ctas), dim3(kWriteThreads), 0, stream, p);
}

}  // namespace atrex_sm100
