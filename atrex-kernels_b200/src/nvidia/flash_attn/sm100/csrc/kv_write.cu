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

__device__ __forceinline__ uint2 quantise8(uint4 raw, float s, float r) {
  const f32x2 s2 = pack2(s, s), neg_s2 = pack2(-s, -s), r2 = pack2(r, r);
  const uint32_t lo0 = quotients_e4m3x2(raw.x, s2, neg_s2, r2), hi0 = quotients_e4m3x2(raw.y, s2, neg_s2, r2);
  const uint32_t lo1 = quotients_e4m3x2(raw.z, s2, neg_s2, r2), hi1 = quotients_e4m3x2(raw.w, s2, neg_s2, r2);
  return make_uint2(lo0 | (hi0 << 16), lo1 | (hi1 << 16));
}

// One warp per (tensor, token): the slot lookup and the page arithmetic happen once per token, the
// lanes then move the token's num_kv_heads * head_dim / 8 vectors, kInFlight loads ahead of the stores.
template <bool kFp8>
__global__ void __launch_bounds__(kWriteThreads) atrex_sm100_kv_write_kernel(const KvWriteParams p) {
  extern __shared__ float s_scale[];                       // E4M3 only: [tensor][head] scale, then reciprocal
  if (kFp8) {
    for (int i = threadIdx.x; i < 2 * p.num_kv_heads; i += kWriteThreads) {
      const int which = i >= p.num_kv_heads, head = i - which * p.num_kv_heads;
      const float* scales = which ? p.v_scale : p.k_scale;
      const float sc = scales ? __ldg(scales + head * (which ? p.v_scale_head_stride : p.k_scale_head_stride)) : 1.f;
      s_scale[i] = sc;
      s_scale[2 * p.num_kv_heads + i] = __frcp_rn(sc);     // correctly rounded, once per CTA and head
    }
    __syncthreads();
  }
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
    if (slot < 0 || slot >= p.slot_limit) continue;        // padding token, or a slot past the pools (warp-uniform)
    const long long page = slot / p.page_size, in_page = slot - page * p.page_size;
    const __nv_bfloat16* src = (which ? p.value : p.key) + tok * (which ? p.v_token_stride : p.k_token_stride);
    const long long src_head = which ? p.v_head_stride : p.k_head_stride;
    const long long dst_head = which ? p.vc_head_stride : p.kc_head_stride;
    const long long dst_tok = which ? page * p.vc_page_stride + in_page * p.vc_row_stride
                                    : page * p.kc_page_stride + in_page * p.kc_row_stride;
    uint8_t* cache = reinterpret_cast<uint8_t*>(which ? p.value_cache : p.key_cache);
    const float* head_scale = s_scale + which * p.num_kv_heads;
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
          *reinterpret_cast<uint2*>(cache + off) =
              quantise8(raw[u], head_scale[head[u]], head_scale[2 * p.num_kv_heads + head[u]]);
        } else {
          *reinterpret_cast<uint4*>(cache + off * 2) = raw[u];
        }
      }
    }
  }
}

// Per-KV-head scales for an E4M3 cache: scale[head] = max |x| over the step's rows of that head / 448, so that
// x / scale fills the format's range.  Pass 1 reduces |x| (BF16 magnitudes compare like their bit patterns, so
// the maximum is an integer max of 15-bit fields) per warp, then per CTA in shared memory, then with one
// atomicMax per head and CTA; pass 2 turns the maxima into FP32 scales.  `amax` must be zero on entry.
__global__ void __launch_bounds__(kWriteThreads) atrex_sm100_kv_amax_kernel(const KvWriteParams p, unsigned* amax) {
  extern __shared__ unsigned s_amax[];                     // [2][num_kv_heads]
  for (int i = threadIdx.x; i < 2 * p.num_kv_heads; i += kWriteThreads) s_amax[i] = 0u;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int vec_per_row = p.head_dim >> 3;
  const int vec_per_tok = p.num_kv_heads * vec_per_row;
  const int row_shift = (vec_per_row & (vec_per_row - 1)) == 0 ? __ffs(vec_per_row) - 1 : -1;
  const long long units = 2ll * p.num_tokens;
  const long long warps = (long long)gridDim.x * (kWriteThreads / 32);
  // A lane keeps the same (head, vector) slots for every token: kInFlight loads per token, their maxima kept per slot.
  for (int v0 = lane; v0 < vec_per_tok; v0 += 32 * kInFlight) {
    int head[kInFlight], vec[kInFlight];
    unsigned best[2][kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int v = v0 + u * 32;
      head[u] = row_shift >= 0 ? v >> row_shift : v / vec_per_row;
      vec[u] = v - head[u] * vec_per_row;
      best[0][u] = best[1][u] = 0u;
    }
    for (long long unit = (long long)blockIdx.x * (kWriteThreads / 32) + (threadIdx.x >> 5); unit < units; unit += warps) {
      const int which = unit >= p.num_tokens;
      const long long tok = unit - (which ? p.num_tokens : 0);
      const long long slot = __ldg(p.slot_mapping + tok);
      if (slot < 0 || slot >= p.slot_limit) continue;      // tokens that are not stored do not count
      const __nv_bfloat16* src = (which ? p.value : p.key) + tok * (which ? p.v_token_stride : p.k_token_stride);
      const long long src_head = which ? p.v_head_stride : p.k_head_stride;
      uint4 raw[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u)
        raw[u] = v0 + u * 32 < vec_per_tok ? __ldg(reinterpret_cast<const uint4*>(src + head[u] * src_head + vec[u] * 8))
                                           : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const unsigned w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        unsigned m = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) m = max(m, max(w[i] & 0x7fffu, (w[i] >> 16) & 0x7fffu));
        if (which) best[1][u] = max(best[1][u], m);
        else best[0][u] = max(best[0][u], m);
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      if (v0 + u * 32 >= vec_per_tok) continue;
      if (best[0][u]) atomicMax(&s_amax[head[u]], best[0][u]);
      if (best[1][u]) atomicMax(&s_amax[p.num_kv_heads + head[u]], best[1][u]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * p.num_kv_heads; i += kWriteThreads)
    if (s_amax[i]) atomicMax(&amax[i], s_amax[i]);
}

// amax (BF16 magnitude bits) -> scale = amax / 448 (IEEE division); a head without a finite non-zero value gets 1.
__global__ void atrex_sm100_kv_scale_kernel(const unsigned* amax, float* k_scale, float* v_scale, int num_kv_heads) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * num_kv_heads) return;
  const float a = __uint_as_float(amax[i] << 16);
  const float scale = (a > 0.f && a < __int_as_float(0x7f800000)) ? __fdiv_rn(a, 448.f) : 1.f;
  (i < num_kv_heads ? k_scale : v_scale)[i % num_kv_heads] = scale;
}

}  // namespace

cudaError_t kv_write_launch(const KvWriteParams& p, bool fp8, int sm_count, cudaStream_t stream) {
  const long long units = 2ll * p.num_tokens;
  if (units == 0) return cudaSuccess;
  const int warps_per_cta = kWriteThreads / 32;
  long long ctas = (units + warps_per_cta - 1) / warps_per_cta;
  const long long cap = (long long)sm_count * 8;   // 8 resident CTAs of 256 threads per SM, then the warps stride on
  if (ctas > cap) ctas = cap;
  if (fp8)
    return launch_kernel(atrex_sm100_kv_write_kernel<true>, dim3((unsigned)ctas), dim3(kWriteThreads),
                         sizeof(float) * 4 * p.num_kv_heads, stream, p);
  return launch_kernel(atrex_sm100_kv_write_kernel<false>, dim3((unsigned)ctas), dim3(kWriteThreads), 0, stream, p);
}

cudaError_t kv_scales_launch(const KvWriteParams& p, unsigned* amax, float* k_scale, float* v_scale, int sm_count,
                             cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(unsigned) * 2 * p.num_kv_heads, stream);
  if (e != cudaSuccess) return e;
  const long long units = 2ll * p.num_tokens;
  if (units > 0) {
    const int warps_per_cta = kWriteThreads / 32;
    long long ctas = (units + warps_per_cta - 1) / warps_per_cta;
    const long long cap = (long long)sm_count * 8;
    if (ctas > cap) ctas = cap;
    e = launch_kernel(atrex_sm100_kv_amax_kernel, dim3((unsigned)ctas), dim3(kWriteThreads),
                      sizeof(unsigned) * 2 * p.num_kv_heads, stream, p, amax);
    if (e != cudaSuccess) return e;
  }
  const int n = 2 * p.num_kv_heads;
  return launch_kernel(atrex_sm100_kv_scale_kernel, dim3((n + 127) / 128), dim3(128), 0, stream,
                       (const unsigned*)amax, k_scale, v_scale, p.num_kv_heads);
}

}  // namespace atrex_sm100
