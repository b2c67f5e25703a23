// Thin inline-PTX wrappers used by the sm_100a attention kernels: mbarriers with
// BOUNDED waits, TMA tiled loads, ldmatrix / mma.sync, and small math helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace atrex_sm100 {

// Codes a kernel stores in params.device_status when a bounded wait gives up.
enum DeviceStatus : int {
  kDeviceOk = 0,
  kWaitFullTimeout = 101,   // consumer never saw a K/V tile arrive
  kWaitEmptyTimeout = 102,  // producer never saw a stage released
  kWaitMmaTimeout = 103,    // tcgen05 completion barrier never fired
  kWaitMiscTimeout = 104,
  kBadSmemAlignment = 105,
  kWaitPeerTimeout = 106    // context-parallel merge: a peer rank never reported its partial result
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false when the limit is reached; the caller then
// records a status code and leaves its loop, so a protocol mistake ends the
// kernel instead of hanging the GPU.  Every failed try_wait suspends the thread
// for up to kSuspendHintNs, so the limit is seconds, far above any real wait.
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t kSuspendHintNs = 1000;
// The loop holds one try_wait with a suspend-time hint, a count-down and nothing else.  Without the hint, and with
// the iteration test and a sleep in the loop, a waiting warp came back every ~240 cycles and the waits were 37 %
// of all instructions the head_dim-128 prefill kernel executed.  Effect on that kernel: +2.5 % in 10-step runs
// (1 012 -> 1 037 TFLOP/s), none in 40-step runs at the power cap (1 042 - 1 047 with or without the hint).  The
// opcode counters afterwards show SYNCS and NANOSLEEP in a loop: the hinted try_wait is itself a poll with a sleep,
// not a blocking wait, and the waits remain ~40 % of the executed instructions (from warps with nothing else to do).
// The spinning part is also kept out of line: a wait has a dozen call sites per kernel, and an inlined
// loop at each of them pushes the hot loops of the MMA-issuing and TMA-issuing warps out of the
// instruction cache.
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, uint32_t limit) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .u32 n;\n"
      "mov.u32 n, %3;\n"
      "ATREX_SPIN:\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %4;\n"
      "@p bra ATREX_SPIN_DONE;\n"
      "sub.u32 n, n, 1;\n"
      "setp.ne.u32 q, n, 0;\n"
      "@q bra ATREX_SPIN;\n"
      "ATREX_SPIN_DONE:\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity), "r"(limit == 0 ? 1u : limit), "r"(kSuspendHintNs)
      : "memory");
  return done != 0;
}
#ifdef ATREX_MBAR_SPIN_INLINE   // for kernels that use setmaxnreg: no calls with their own register ABI
__device__ __forceinline__
#else
static __device__ __noinline__   // one copy per translation unit
#endif
bool mbar_wait_slow(uint64_t* bar, uint32_t parity) { return mbar_spin(bar, parity, kSpinLimit); }
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}

// 16-byte asynchronous copy global -> shared (no registers held while in flight); zeros when !valid.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// 4-D tiled TMA load into this CTA only.  Coordinates are innermost first.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tensor_map, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// K/V tile load: the head, row and page coordinates sit where the host's
// ascending-stride ordering of the tensor map put them.
__device__ __forceinline__ void tma_load_kv(void* smem_dst, const void* tensor_map, uint64_t* bar, int d0,
                                            int head, int row, int page, const int8_t (&perm)[3]) {
  // selects instead of an indexed array: keeps the coordinates in registers
  const int c0 = perm[0] == 0 ? head : (perm[1] == 0 ? row : page);
  const int c1 = perm[0] == 1 ? head : (perm[1] == 1 ? row : page);
  const int c2 = perm[0] == 2 ? head : (perm[1] == 2 ? row : page);
  tma_load_4d(smem_dst, tensor_map, bar, d0, c0, c1, c2);
}
__device__ __forceinline__ void prefetch_tensormap(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                            uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 32-byte store (one full DRAM sector per thread); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
// Eight consecutive FP32 values times `scale`, as eight BF16, to 16 bytes / sixteen to 32 bytes.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi);
__device__ __forceinline__ void store_bf16_row32(__nv_bfloat16* dst, const uint32_t (&v)[32], float scale, bool vec32) {
  if (vec32) {
#pragma unroll
    for (int i = 0; i < 32; i += 16) {
      uint32_t pk[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        pk[u] = pack_bf16(__uint_as_float(v[i + 2 * u]) * scale, __uint_as_float(v[i + 2 * u + 1]) * scale);
      st_global_v8(dst + i, pk);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 pk;
      pk.x = pack_bf16(__uint_as_float(v[i]) * scale, __uint_as_float(v[i + 1]) * scale);
      pk.y = pack_bf16(__uint_as_float(v[i + 2]) * scale, __uint_as_float(v[i + 3]) * scale);
      pk.z = pack_bf16(__uint_as_float(v[i + 4]) * scale, __uint_as_float(v[i + 5]) * scale);
      pk.w = pack_bf16(__uint_as_float(v[i + 6]) * scale, __uint_as_float(v[i + 7]) * scale);
      *reinterpret_cast<uint4*>(dst + i) = pk;
    }
  }
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a tile whose rows
// are 128 bytes and that uses the TMA / UMMA 128-byte swizzle (tile base must
// be 1024-byte aligned).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace atrex_sm100
