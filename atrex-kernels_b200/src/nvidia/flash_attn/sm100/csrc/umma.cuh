// tcgen05 (5th-generation tensor core) and TMEM wrappers for sm_100a: shared-memory
// matrix descriptors, instruction descriptors, MMA issue, commit, TMEM allocation
// and TMEM <-> register moves.  Bit layouts follow the PTX ISA's "tcgen05
// shared memory descriptor" and "instruction descriptor" tables.
#pragma once

#include <stdint.h>

#include "ptx.cuh"

namespace atrex_sm100 {

// ---- shared-memory matrix descriptor, 128-byte swizzle -------------------------
// bits [0,14) start address >> 4, [16,30) leading byte offset >> 4,
// [32,46) stride byte offset >> 4, [46,48) version = 1, [61,64) layout (2 = SWIZZLE_128B).
//
// K-major operand (rows of 128 bytes, the contraction dimension contiguous):
//   8-row groups are `sbo` bytes apart (1024 for a dense tile); LBO is unused.
// MN-major operand (rows are contraction steps, 64 elements of the M/N
//   dimension contiguous per row): 8-row groups `sbo` bytes apart, successive
//   64-element column blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// ---- instruction descriptor for kind::f16 / kind::f8f6f4, FP32 accumulate --------
// [4,6) D format (1 = F32), [7,10) A format, [10,13) B format, bit 15 A major,
// bit 16 B major (0 = K-major, 1 = MN-major), [17,23) N >> 3, [24,29) M >> 4.
// Formats: kind::f16 -> 0 F16, 1 BF16; kind::f8f6f4 -> 0 E4M3, 1 E5M2.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Same two forms for 8-bit operands (kind::f8f6f4: E4M3 / E5M2, K = 32 per instruction).
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_f8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Warp-converged forms: every lane executes the call (so the compiler may keep the descriptors, which are
// the same in all lanes, in uniform registers and do their address arithmetic once per warp), and the
// lane whose `lead` is non-zero issues.  Exactly one lane of the warp must pass a non-zero `lead`.
// A shared-memory descriptor is passed as its two 32-bit halves: only the low half (start address >> 4 in
// bits 0-13) changes between the instructions of a tile, so stepping through a tile is one 32-bit add per
// operand instead of 64-bit arithmetic -- the issuing warp shares its scheduler with two softmax warps,
// and every instruction it needs per MMA delays the next MMA.
struct UmmaDesc {
  uint32_t lo, hi;
  __device__ __forceinline__ UmmaDesc operator+(uint32_t bytes_shr4) const { return UmmaDesc{lo + bytes_shr4, hi}; }
};
__device__ __forceinline__ UmmaDesc umma_desc_split(uint64_t d) { return UmmaDesc{(uint32_t)d, (uint32_t)(d >> 32)}; }

#define ATREX_UMMA_SS_LEAD(NAME, KIND)                                                                        \
  __device__ __forceinline__ void NAME(uint32_t lead, uint32_t d_tmem, UmmaDesc a, UmmaDesc b, uint32_t idesc, \
                                       uint32_t accumulate) {                                                 \
    asm volatile(                                                                                             \
        "{\n"                                                                                                 \
        ".reg .pred p, q;\n"                                                                                  \
        ".reg .b64 da, db;\n"                                                                                 \
        "mov.b64 da, {%1, %2};\n"                                                                             \
        "mov.b64 db, {%3, %4};\n"                                                                             \
        "setp.ne.b32 p, %6, 0;\n"                                                                             \
        "setp.ne.b32 q, %7, 0;\n"                                                                             \
        "@q tcgen05.mma.cta_group::1.kind::" KIND " [%0], da, db, %5, p;\n"                                   \
        "}\n" ::"r"(d_tmem),                                                                                  \
        "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accumulate), "r"(lead)                    \
        : "memory");                                                                                          \
  }
#define ATREX_UMMA_TS_LEAD(NAME, KIND)                                                                         \
  __device__ __forceinline__ void NAME(uint32_t lead, uint32_t d_tmem, uint32_t a_tmem, UmmaDesc b, uint32_t idesc, \
                                       uint32_t accumulate) {                                                  \
    asm volatile(                                                                                              \
        "{\n"                                                                                                  \
        ".reg .pred p, q;\n"                                                                                   \
        ".reg .b64 db;\n"                                                                                      \
        "mov.b64 db, {%2, %3};\n"                                                                              \
        "setp.ne.b32 p, %5, 0;\n"                                                                              \
        "setp.ne.b32 q, %6, 0;\n"                                                                              \
        "@q tcgen05.mma.cta_group::1.kind::" KIND " [%0], [%1], db, %4, p;\n"                                  \
        "}\n" ::"r"(d_tmem),                                                                                   \
        "r"(a_tmem), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(accumulate), "r"(lead)                              \
        : "memory");                                                                                           \
  }
ATREX_UMMA_SS_LEAD(umma_ss_f16_lead, "f16")
ATREX_UMMA_TS_LEAD(umma_ts_f16_lead, "f16")
ATREX_UMMA_SS_LEAD(umma_ss_f8_lead, "f8f6f4")
ATREX_UMMA_TS_LEAD(umma_ts_f8_lead, "f8f6f4")
#undef ATREX_UMMA_SS_LEAD
#undef ATREX_UMMA_TS_LEAD

__device__ __forceinline__ void umma_commit_lead(uint32_t lead, uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .pred q;\n"
      "setp.ne.b32 q, %1, 0;\n"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n" ::"r"(smem_u32(bar)),
      "r"(lead)
      : "memory");
}

// The mbarrier gets one arrival when every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMEM allocation (one full warp executes these) ------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_addr), "r"(columns) : "memory");
}

// ---- TMEM <-> registers: shape 32x32b, each thread of a warp owns one lane -------
// Warp w of a warpgroup may only touch lanes [32*(w%4), 32*(w%4)+32).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// ---- register budget per warpgroup ------------------------------------------------
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// 3-D tiled TMA load (Q tiles: D x heads x rows) into this CTA only.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tensor_map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(tensor_map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

}  // namespace atrex_sm100
