// Context parallelism, the exchange step as ONE kernel: every rank attended its own share of each request's keys
// and left (O, natural-log LSE) in a buffer its peers can address; this kernel tells the peers that this rank's
// pair is ready, waits (bounded) until every peer has said the same, then reads all ranks' pairs with plain
// peer loads over NVLink and writes the merged (out, lse) into this GPU's memory.  No collective library call,
// no staging copy; the merge algebra is the split-KV combine's, across ranks instead of across splits
// (src/nvidia/flash_attn/sm103/decode_reduce_cutedsl.py:71-152).  The reference has no context parallelism
// (python/atrex/api/flash_attn.py:128-135 rejects the arguments).
//
// Protocol.  Each rank owns a small array of step counters, one per peer, in peer-addressable memory.  The
// launch of step n on rank r stores n into slot r of EVERY rank's array (system-scope release; the attention
// kernel that produced this rank's pair ran earlier on the same stream, so its writes are complete), then waits
// until all slots of its OWN array have reached n (system-scope acquire).  Counters only grow, so a rank that
// runs ahead is harmless.  The wait has an iteration limit: if a peer never arrives the kernel stores
// kWaitPeerTimeout in the status word and returns without writing the output.
//
// The waiting kernels of different ranks run on different GPUs; on one GPU the ranks are emulated by one launch
// over all ranks' buffers with the counters already set (see the C entry point).
#include "atrex_fa_sm100.h"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace atrex_sm100 {
namespace {

constexpr int kMaxCpWorld = 8;
constexpr int kCpWarps = 8;

struct CpMergeArgs {
  const __nv_bfloat16* parts[kMaxCpWorld];   // rank w's O [total_q, Hq, D]
  const float* lses[kMaxCpWorld];            // rank w's LSE [Hq, total_q]
  uint32_t* counters[kMaxCpWorld];           // rank w's counter array [kMaxCpWorld]
  __nv_bfloat16* out;
  float* lse;
  int32_t* status;
  long long total_q;
  int num_q_heads, head_dim, world, rank;
  uint32_t step;
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// LANES lanes of 16 bytes cover one row of head_dim BF16 (16 for head_dim 128, 32 for 256).
template <int LANES>
__global__ void __launch_bounds__(kCpWarps * 32)
atrex_sm100_cp_merge_kernel(const __grid_constant__ CpMergeArgs a) {
  __shared__ int s_ready;
  if (blockIdx.x == 0 && threadIdx.x < (unsigned)a.world) {
    __threadfence_system();
    store_release_sys(a.counters[threadIdx.x] + a.rank, a.step);
  }
  if (threadIdx.x == 0) {
    int ready = 1;
    for (int w = 0; w < a.world && ready; ++w) {
      const uint32_t* slot = a.counters[a.rank] + w;
      uint32_t spins = 0;
      while ((int32_t)(load_acquire_sys(slot) - a.step) < 0) {
        if (++spins > (1u << 21)) { ready = 0; break; }   // a second or two: far beyond any real skew
        if (spins > 256) __nanosleep(500);
      }
    }
    if (!ready && a.status != nullptr) atomicExch(a.status, (int)kWaitPeerTimeout);
    s_ready = ready;
  }
  __syncthreads();
  if (!s_ready) return;

  constexpr int kRowsPerWarp = 32 / LANES;
  const int lane = threadIdx.x & 31, sub = lane / LANES, l = lane % LANES;
  const long long rows = a.total_q * a.num_q_heads;
  const long long row = ((long long)blockIdx.x * kCpWarps + (threadIdx.x >> 5)) * kRowsPerWarp + sub;   // (query, head)
  if (row >= rows) return;
  const long long q = row / a.num_q_heads;
  const int h = (int)(row - q * a.num_q_heads);
  const long long lse_off = (long long)h * a.total_q + q;
  float part_l[kMaxCpWorld];
  float mx = -INFINITY;
#pragma unroll
  for (int w = 0; w < kMaxCpWorld; ++w) {
    part_l[w] = w < a.world ? __ldcg(a.lses[w] + lse_off) : -INFINITY;
    mx = fmaxf(mx, part_l[w]);
  }
  float acc[8], denom = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
  for (int w = 0; w < kMaxCpWorld; ++w) {
    if (w >= a.world || part_l[w] == -INFINITY) continue;   // a rank without keys for this row: weight 0, not read
    const float wgt = __expf(part_l[w] - mx);
    denom += wgt;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.parts[w] + row * a.head_dim) + l);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += wgt * __uint_as_float(u[i] << 16);
      acc[2 * i + 1] += wgt * __uint_as_float(u[i] & 0xFFFF0000u);
    }
  }
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
  uint4 o;
  o.x = pack_bf16(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  o.z = pack_bf16(acc[4] * inv, acc[5] * inv);
  o.w = pack_bf16(acc[6] * inv, acc[7] * inv);
  reinterpret_cast<uint4*>(a.out + row * a.head_dim)[l] = o;
  if (l == 0) a.lse[lse_off] = denom > 0.f ? mx + __logf(denom) : -INFINITY;
}

}  // namespace
}  // namespace atrex_sm100

extern "C" int atrex_fa_sm100_cp_merge(const atrex_fa_sm100_cp_merge_params* p, void* stream) {
  using namespace atrex_sm100;
  if (p == nullptr || p->struct_bytes != sizeof(atrex_fa_sm100_cp_merge_params) ||
      p->abi_version != ATREX_FA_SM100_ABI_VERSION)
    return ATREX_FA_ABI_MISMATCH;
  if (p->world < 1 || p->world > kMaxCpWorld || p->rank < 0 || p->rank >= p->world || p->total_q < 0 ||
      p->num_q_heads <= 0)
    return ATREX_FA_INVALID_VALUE;
  if (p->head_dim != 128 && p->head_dim != 256) return ATREX_FA_UNSUPPORTED;
  if (p->total_q == 0) return ATREX_FA_OK;
  if (p->out == nullptr || p->lse == nullptr) return ATREX_FA_INVALID_VALUE;
  CpMergeArgs a = {};
  for (int w = 0; w < p->world; ++w) {
    if (p->parts[w] == nullptr || p->part_lse[w] == nullptr || p->counters[w] == nullptr) return ATREX_FA_INVALID_VALUE;
    if ((reinterpret_cast<uintptr_t>(p->parts[w]) & 15u) != 0) return ATREX_FA_UNSUPPORTED;
    a.parts[w] = static_cast<const __nv_bfloat16*>(p->parts[w]);
    a.lses[w] = p->part_lse[w];
    a.counters[w] = p->counters[w];
  }
  if ((reinterpret_cast<uintptr_t>(p->out) & 15u) != 0) return ATREX_FA_UNSUPPORTED;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.lse = p->lse;
  a.status = p->device_status;
  a.total_q = p->total_q;
  a.num_q_heads = p->num_q_heads;
  a.head_dim = p->head_dim;
  a.world = p->world;
  a.rank = p->rank;
  a.step = p->step;
  const long long rows = a.total_q * a.num_q_heads;
  const int lanes = p->head_dim / 8;
  const long long rows_per_block = (long long)kCpWarps * (32 / lanes);
  const unsigned grid = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const cudaError_t e = lanes == 16 ? launch_kernel(atrex_sm100_cp_merge_kernel<16>, dim3(grid), dim3(kCpWarps * 32), 0, s, a)
                                    : launch_kernel(atrex_sm100_cp_merge_kernel<32>, dim3(grid), dim3(kCpWarps * 32), 0, s, a);
  return e == cudaSuccess ? ATREX_FA_OK : ATREX_FA_CUDA_ERROR;
}
