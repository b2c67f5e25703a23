// Compact sparse attention (atrex.qsa_compact) for sm_100a: gated attention of every query row over the tokens of
// its 512 selected four-token blocks, gathered through the page table.
//
// Native counterpart of the reference's sm100 kernels (src/nvidia/qsa/sm100/decode_fp8.py, prefill_bf16.py,
// prefill_fp8.py; contract python/atrex/api/qsa.py:19-47), designed for B200 rather than translated.  The operator
// is a gather: a row reads at most 2051 K and V rows of 256 elements per KV head (2.1 MB in BF16) and does
// 8 - 12 heads x 2051 x 256 x 4 FLOP on them, two FLOP per byte gathered, so the kernel is built around keeping
// many 512-byte row fetches in flight, not around tensor throughput:
//
//   * one CTA = (row, KV head, split of the row's token list); the 8 or 12 query heads of the KV head are the
//     rows of one 16-row MMA tile (pack-GQA: one fetch of a K/V row serves the whole group);
//   * the CTA first resolves its share of the row's blocks to cache addresses (block id -> first token -> page
//     table -> address; a four-token block never straddles a page) into shared memory: two dependent global
//     loads once per CTA instead of once per tile on every warp's critical path;
//   * each of the six or eight warps (eight for an E4M3 cache and for BF16 calls of one wave with long token
//     lists, which keep a ring of three operand tiles instead of two K + V stages) is then its own pipeline: it
//     takes every sixth / eighth 16-token tile (four blocks),
//     fetches K and V with 16-byte cp.async copies into its private double buffer (a row is one coalesced
//     512-byte request) and computes S = Q K^T, the online softmax (log2 domain) and O += P V with mma.sync
//     while the next tile's copies are in flight; no block-wide barrier inside the loop;
//   * tokens that do not count (hidden block, request id out of range, page outside the table or the pool) are
//     zero-filled in shared memory and masked in S, so no address is formed from them;
//   * E4M3 caches are copied as bytes (half the traffic) and nothing is widened in shared memory: S = Q K^T runs
//     on the E4M3 MMA (m16n8k32) straight from the raw K tile; for P V the transposing ldmatrix reads the raw V
//     tile, the bytes are widened to FP16 in registers (exact) and two FP16 MMAs per 16-byte chunk take its even
//     and its odd head dimensions (P stays 16-bit: three mantissa bits are too few for the probabilities);
//     sm_scale carries the Q and K scales, v_scale multiplies the result;
//   * the warps' partial states merge through shared memory; the epilogue rounds A to BF16, multiplies by
//     sigmoid(gate) and stores BF16 (or writes a normalised FP32 partial + log2 LSE for the split combine).
#include <cooperative_groups.h>
#include <cuda_fp8.h>

#include "atrex_qsa_sm100.h"
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace atrex_sm100 {
namespace {

constexpr int kD = ATREX_QSA_SM100_HEAD_DIM;
constexpr int kTopk = ATREX_QSA_SM100_TOPK;
constexpr int kTile = 16;                 // tokens per warp tile = four blocks
// Measured on B200 (64 decode rows / 2048 prefill rows, device time per call): 4 warps x 2 stages 32.0 / 510 us,
// 4 x 3 32.2 / 548 us, 6 x 2 33.1 / 496 us (E4M3 decode 41.6 / 40.7 / 36.9 us): six warps with double buffers.  The
// E4M3 decode then went 37.2 -> 31.4 us with S = Q K^T on the E4M3 MMA (K not widened) and -> 27.3 us with eight
// warps, and -> 23.0 us with P V from the raw V tile (bytes widened to FP16 in registers); a third raw stage
// (31.0), skipping the O rescale when no row maximum moved (32.6) and widening to FP16 instead of BF16 in shared
// memory (39.7 against 37.0 before the E4M3 MMA) did not help.
#ifndef ATREX_QSA_WARPS
#define ATREX_QSA_WARPS 6
#endif
#ifndef ATREX_QSA_STAGES
#define ATREX_QSA_STAGES 2
#endif
#ifndef ATREX_QSA_WARPS_FP8
#define ATREX_QSA_WARPS_FP8 8
#endif
constexpr int kMaxSplits = 16;
constexpr int kQBytes = 16 * kD * 2;      // Q tile: 16 rows (8 or 12 used) x 256 BF16 (E4M3: half of it)
constexpr int kOperandBytes = kTile * kD * 2;          // one K or V tile as BF16: 8 KB
constexpr int kStages = ATREX_QSA_STAGES;              // tiles resident per warp: one being consumed, the others in flight
constexpr int kBlockOffBytes = (kTopk + 4) * 8;        // element offset of every block's first row (-1 = does not count)
// Per cache type.  A warp's region holds kStages x (K + V) tiles as BF16 (32 KB), or for E4M3 the raw stages (16 KB;
// at least the 16.1 KB its share of the merge buffer needs): the E4M3 call, which moves half the bytes and is bound
// by the warps' own pace per tile rather than by memory, runs eight warps, as many as 255 registers per thread allow
// (ten or twelve warps at 168 registers spill: 29.4 / 26.2 us against 22.8).
constexpr int kRowTilesMax = (kTopk * 4 + 3 + kTile - 1) / kTile;   // tiles of the longest token list a row can have
constexpr int kMaxClusterSplits = 8;                   // portable cluster size
constexpr int kPartStride = kD + 4;                    // floats per (split, head) partial in the leader: A, then the LSE
// kRing: the warp's region is a ring of THREE operand tiles (K(i), V(i), K(i+1) -> V(i), K(i+1), V(i+1) -> ...) instead
// of two whole (K + V) stages: the same bytes in flight in a quarter less shared memory, so that the BF16 kernel runs
// eight warps as well.  It pays two waits, two barriers and two address passes per tile instead of one, which only
// the BF16 call of ONE wave (decode) wins back: 33.0 -> 30.7 us, against 0.499 -> 0.517 ms for a prefill chunk and
// 22.7 -> 25.4 us for the E4M3 decode, which has its eight warps anyway.  So the ring serves BF16 single-wave calls.
template <bool kFp8, bool kRing>
struct QsaCfg {
  static constexpr int kWarps = kFp8 ? ATREX_QSA_WARPS_FP8 : (kRing ? ATREX_QSA_WARPS_FP8 : ATREX_QSA_WARPS);
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kOpBytes = kTile * kD * (kFp8 ? 1 : 2);        // one K or V tile of 16 tokens
  static constexpr int kRawBytes = kStages * 2 * (kTile * kD);        // E4M3: kStages x (K + V) as bytes
  static constexpr int kMergeBytes = ((16 * (kD + 2) * 4 + 1023) / 1024) * 1024;
  static constexpr int kTileBytes = kRing ? 3 * kOpBytes : (kFp8 ? kRawBytes : kStages * 2 * kOperandBytes);
  static constexpr int kWarpBytes = kTileBytes > kMergeBytes ? kTileBytes : kMergeBytes;
  static constexpr int kMetaBytes = kWarps * kStages * kTile * 8;   // per warp, two tiles: 16 row offsets (int64, -1 = does not count)
  static constexpr int kSmemBytes = kQBytes + kWarps * kWarpBytes + kMetaBytes + kBlockOffBytes;
  static_assert(16 * (kD + 2) * 4 <= kWarpBytes, "merge buffer aliases the tile buffers");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static_assert(kMaxClusterSplits * 12 * kPartStride * 4 <= kWarps * kWarpBytes, "the cluster's partials fit the leader's tile buffers");
};

struct QsaParams {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* ids;
  const void* pos;
  const int32_t* table;
  const int32_t* req;
  const __nv_bfloat16* gate;
  __nv_bfloat16* out;
  float* part_o;      // [splits, rows, Hq, 256] normalised partial A (before v_scale)
  float* part_lse;    // [splits, rows, Hq] log2-domain LSE
  int32_t* status;
  long long q_row_stride, q_head_stride, kv_page_stride, kv_row_stride, kv_head_stride;
  int rows, hq, hkv, group, num_pages, page_size, batch, table_width, pos64, num_splits;
  int cluster_combine;   // the CTAs of one (row, KV head) are a thread-block cluster and combine their splits themselves
  float scale_log2, v_scale;
};


__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;   // 0: the destination is zero-filled and nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// Two E4M3 bytes of `word` (selected by a byte-permute pattern) -> two FP16, exact.
template <uint32_t kSelector>
__device__ __forceinline__ uint32_t e4m3_pair_to_f16x2(uint32_t word) {
  const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)__byte_perm(word, 0u, kSelector), __NV_E4M3);
  return (uint32_t)h2.x | ((uint32_t)h2.y << 16);
}

template <bool kFp8, bool kRing>
__global__ void __launch_bounds__(QsaCfg<kFp8, kRing>::kThreads, 1)
atrex_sm100_qsa_kernel(const __grid_constant__ QsaParams p) {
  using Cfg = QsaCfg<kFp8, kRing>;
  constexpr int kWarps = Cfg::kWarps, kThreads = Cfg::kThreads, kWarpBytes = Cfg::kWarpBytes;
  static_assert(kStages == 2, "two tiles of row offsets per warp");
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_smem = smem;
  uint8_t* tiles = smem + kQBytes;
  long long* meta = reinterpret_cast<long long*>(smem + kQBytes + kWarps * kWarpBytes);
  long long* block_off = meta + kWarps * kStages * kTile;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = blockIdx.x / p.hkv, h = blockIdx.x % p.hkv;
  const int split = blockIdx.y;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0 && p.status) atomicExch(p.status, kBadSmemAlignment);
    return;
  }

  // ---- the row's token list: complete blocks from the id list, then the unfinished block ----
  const long long position = p.pos64 ? reinterpret_cast<const long long*>(p.pos)[t]
                                     : (long long)reinterpret_cast<const int*>(p.pos)[t];
  const long long visible = position + 1;
  const int request = p.req[t];
  const bool live = visible > 0 && request >= 0 && request < p.batch;
  const int complete = live ? (int)min((long long)kTopk, visible / 4) : 0;
  const int n_tok = live ? complete * 4 + (int)(visible % 4) : 0;
  const long long tail_start = (visible / 4) * 4;
  const int n_tiles_row = (n_tok + kTile - 1) / kTile;
  const int tile_lo = (int)(((long long)n_tiles_row * split) / p.num_splits);
  const int tile_hi = (int)(((long long)n_tiles_row * (split + 1)) / p.num_splits);
  const int32_t* row_ids = p.ids + (long long)t * kTopk;
  const int32_t* table_row = p.table + (long long)(live ? request : 0) * p.table_width;

  // ---- Q rows of this KV head's group -> shared memory in the cache's own type (swizzled like K) ----
  {
    constexpr int kChunks = kFp8 ? kD / 16 : kD / 8;   // 16-byte chunks per row: 16 E4M3 or 8 BF16 each
    for (int idx = tid; idx < 16 * kChunks; idx += kThreads) {
      const int r = idx / kChunks, c = idx % kChunks;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < p.group) {
        const long long e = (long long)t * p.q_row_stride + (long long)(h * p.group + r) * p.q_head_stride;
        val = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.q) + e * (kFp8 ? 1 : 2) + c * 16));
      }
      *reinterpret_cast<uint4*>(q_smem + (c / 8) * (16 * 128) + swz128(r, c % 8)) = val;
    }
  }
  // ---- this split's blocks -> element offset of their first cache row ----
  // list block j < complete is the j-th listed block; list block `complete` is the unfinished last block
  for (int j = tile_lo * 4 + tid; j < tile_hi * 4 && j <= complete; j += kThreads) {
    long long tok = -1, off = -1;
    if (j < complete) {
      const int blk = row_ids[j];
      if (blk >= 0) tok = (long long)blk * 4;
    } else {
      tok = tail_start;
    }
    if (tok >= 0) {
      const long long lp = tok / p.page_size;
      if (lp < p.table_width) {
        const int phys = table_row[lp];
        if (phys >= 0 && phys < p.num_pages)
          off = (long long)phys * p.kv_page_stride + (tok - lp * p.page_size) * p.kv_row_stride +
                (long long)h * p.kv_head_stride;
      }
    }
    block_off[j - tile_lo * 4] = off;
  }
  __syncthreads();

  // ---- per-warp pipeline over its tiles ----
  uint8_t* my = tiles + warp * kWarpBytes;
  long long* my_meta = meta + warp * kStages * kTile;
  constexpr int kEsz = kFp8 ? 1 : 2;
  constexpr int kRowBytes = kD * kEsz;                 // bytes of one cache row for one head
  constexpr int kRawOperand = kTile * kRowBytes;       // raw bytes of one K or V tile
  // BF16: stage s holds K at s * 2 * kOperandBytes, V right behind.  E4M3: raw stage s at s * 2 * kRawOperand
  // (K then V); the widened tile (K then V) sits behind the raw stages.
  static_assert(!kFp8 || kStages * 2 * (kTile * kD) <= kWarpBytes, "the raw stages fit");
  auto raw_k = [&](int s) { return my + s * 2 * kRawOperand; };
  auto raw_v = [&](int s) { return my + s * 2 * kRawOperand + kRawOperand; };

  // the 16 tokens of tile `ti` (one lane per token: block base + row inside the block) and its copies into stage s
  auto issue_tile = [&](int ti, int s) {
    long long off = -1;
    if (lane < kTile) {
      const int i = ti * kTile + lane;
      if (i < n_tok) {
        const long long base = block_off[(i >> 2) - tile_lo * 4];
        if (base >= 0) off = base + (i & 3) * p.kv_row_stride;
      }
      my_meta[s * kTile + lane] = off;
    }
    const uint8_t* kbase = reinterpret_cast<const uint8_t*>(p.k);
    const uint8_t* vbase = reinterpret_cast<const uint8_t*>(p.v);
    if (kFp8) {
      // a row is 256 bytes = 16 chunks: two rows per warp instruction
#pragma unroll
      for (int j = 0; j < kTile / 2; ++j) {
        const int r = 2 * j + (lane >> 4), c = lane & 15;
        const long long row_off = __shfl_sync(0xffffffffu, off, r);
        const bool ok = row_off >= 0;
        const long long byte = ok ? row_off + c * 16 : 0;
        const uint32_t dst = (c / 8) * (kTile * 128) + swz128(r, c % 8);   // the MMA layout: both tiles are used raw
        cp_async16(raw_k(s) + dst, kbase + byte, ok);
        cp_async16(raw_v(s) + dst, vbase + byte, ok);
      }
    } else {
      // a row is 512 bytes = 32 chunks: one row per warp instruction, written in the swizzled MMA layout
#pragma unroll
      for (int r = 0; r < kTile; ++r) {
        const long long row_off = __shfl_sync(0xffffffffu, off, r);
        const bool ok = row_off >= 0;
        const long long byte = ok ? row_off * 2 + lane * 16 : 0;
        const uint32_t dst = (lane / 8) * (kTile * 128) + swz128(r, lane % 8);
        cp_async16(raw_k(s) + dst, kbase + byte, ok);
        cp_async16(raw_v(s) + dst, vbase + byte, ok);
      }
    }
    cp_async_commit();
  };

  // ---- the ring variant: operand 2i is K of the warp's i-th tile, 2i + 1 its V; operand n lives in buffer n % 3;
  // one copy group per operand (an empty one where no tile is left)
  auto ring = [&](int n) { return my + (n % 3) * Cfg::kOpBytes; };
  auto tile_offsets = [&](int ti, int slot) {   // the 16 tokens of tile `ti` -> row offsets in meta slot `slot`
    if (lane < kTile) {
      long long off = -1;
      const int i = ti * kTile + lane;
      if (ti < tile_hi && i < n_tok) {
        const long long base = block_off[(i >> 2) - tile_lo * 4];
        if (base >= 0) off = base + (i & 3) * p.kv_row_stride;
      }
      my_meta[slot * kTile + lane] = off;
    }
    __syncwarp();
  };
  auto issue_operand = [&](const void* tensor, int slot, uint8_t* dst_tile, bool exists) {
    if (exists) {
      const uint8_t* base = reinterpret_cast<const uint8_t*>(tensor);
      const long long off = lane < kTile ? my_meta[slot * kTile + lane] : -1;
      if (kFp8) {
#pragma unroll
        for (int j = 0; j < kTile / 2; ++j) {
          const int r = 2 * j + (lane >> 4), c = lane & 15;
          const long long row_off = __shfl_sync(0xffffffffu, off, r);
          const bool ok = row_off >= 0;
          cp_async16(dst_tile + (c / 8) * (kTile * 128) + swz128(r, c % 8), base + (ok ? row_off + c * 16 : 0), ok);
        }
      } else {
#pragma unroll
        for (int r = 0; r < kTile; ++r) {
          const long long row_off = __shfl_sync(0xffffffffu, off, r);
          const bool ok = row_off >= 0;
          cp_async16(dst_tile + (lane / 8) * (kTile * 128) + swz128(r, lane % 8), base + (ok ? row_off * 2 + lane * 16 : 0), ok);
        }
      }
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  const int g = lane >> 2, tq = lane & 3;
  const int mat = lane >> 3, mrow = lane & 7;
  const uint32_t q_addr = smem_u32(q_smem);
  const uint32_t q_lane_row = mrow + (mat & 1) * 8, q_lane_chunk = mat >> 1;
  const uint32_t k_lane_row = mrow + (mat >> 1) * 8, k_lane_chunk = mat & 1;
  const uint32_t v_lane_row = mrow + (mat & 1) * 8, v_lane_chunk = mat >> 1;

  // One copy group per tile, and an empty group where no tile is left, so that "all but the newest two groups
  // are complete" always means "this iteration's tile has landed".
  int stage = 0;
  const int first = tile_lo + warp;
  if constexpr (kRing) {
    // K and V of the warp's first tile, K of its second
    tile_offsets(first, 0);
    issue_operand(p.k, 0, ring(0), first < tile_hi);
    issue_operand(p.v, 0, ring(1), first < tile_hi);
    tile_offsets(first + kWarps, 1);
    issue_operand(p.k, 1, ring(2), first + kWarps < tile_hi);
  } else {
    if (first < tile_hi) issue_tile(first, 0);
#pragma unroll
    for (int d = 1; d < kStages - 1; ++d) {
      if (first + d * kWarps < tile_hi) issue_tile(first + d * kWarps, d);
      else cp_async_commit();
    }
  }
  int n_op = 0;   // ring: the operand about to be consumed (2i)
  for (int ti = first; ti < tile_hi; ti += kWarps, n_op += 2) {
    if constexpr (kRing) {
      cp_async_wait<2>();                                // all but the two newest groups: K(i) has landed
    } else {
      const int ahead = ti + (kStages - 1) * kWarps;
      if (ahead < tile_hi) issue_tile(ahead, (stage + kStages - 1) % kStages);
      else cp_async_commit();
      cp_async_wait<kStages - 1>();
    }
    __syncwarp();
    // which of the tile's 16 tokens count (bit r = token r); the ring keeps tile i's offsets in slot i & 1
    const unsigned live_mask = __ballot_sync(0xffffffffu, lane < kTile && my_meta[stage * kTile + lane] >= 0) & 0xFFFFu;

    // E4M3 tiles are multiplied from their raw stage: K by the E4M3 MMA, V converted in registers (below)
    const uint32_t k_addr = smem_u32(kRing ? ring(n_op) : raw_k(stage));
    const uint32_t v_addr = smem_u32(kRing ? ring(n_op + 1) : raw_v(stage));

    // ---- S = Q K^T : 16 rows x 16 tokens ----
    // four independent accumulator pairs (one per 64-element block of the head dimension) instead of one chain
    // of sixteen dependent MMAs: a warp is alone on its scheduler here, so only instruction-level parallelism
    // hides the MMA latency
    // An E4M3 cache is multiplied by the E4M3 Q with m16n8k32 (the byte layout of a tile is that of a 16-bit tile
    // of half the depth, so the same ldmatrix addressing serves both): half the instructions of the BF16 product.
    float s4[4][2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) s4[i][0][e] = s4[i][1][e] = 0.f;
    constexpr int kBlocks = kFp8 ? kD / 128 : kD / 64;     // 128-byte column blocks of a row
#pragma unroll
    for (int kb = 0; kb < kBlocks; ++kb) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4], b0, b1, b2, b3;
        ldmatrix_x4(a[0], a[1], a[2], a[3], q_addr + kb * (16 * 128) + swz128(q_lane_row, ks * 2 + q_lane_chunk));
        ldmatrix_x4(b0, b1, b2, b3, k_addr + kb * (kTile * 128) + swz128(k_lane_row, ks * 2 + k_lane_chunk));
        const int acc = kFp8 ? kb * 2 + (ks & 1) : kb;     // four independent chains either way
        if constexpr (kFp8) {
          mma_e4m3_16832(s4[acc][0], a, b0, b1);
          mma_e4m3_16832(s4[acc][1], a, b2, b3);
        } else {
          mma_bf16_16816(s4[acc][0], a, b0, b1);
          mma_bf16_16816(s4[acc][1], a, b2, b3);
        }
      }
    }
    if constexpr (kRing) {
      // K(i) is consumed: its buffer takes V of the next tile (operand 2i + 3), whose offsets are in the other slot
      __syncwarp();
      issue_operand(p.v, stage ^ 1, ring(n_op + 3), ti + kWarps < tile_hi);
    }
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = (s4[0][j][e] + s4[1][j][e]) + (s4[2][j][e] + s4[3][j][e]);
    // ---- scale, hide the tokens that do not count, online softmax (log2 domain) ----
    float alpha[2];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = j * 8 + 2 * tq + (e & 1);
        s[j][e] = (live_mask >> col) & 1u ? s[j][e] * p.scale_log2 : -INFINITY;
      }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float mx = fmaxf(fmaxf(s[0][2 * hh], s[0][2 * hh + 1]), fmaxf(s[1][2 * hh], s[1][2 * hh + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hh], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      alpha[hh] = fast_exp2(m_run[hh] - m_use);
      m_run[hh] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][2 * hh] = fast_exp2(s[j][2 * hh] - m_use);
        s[j][2 * hh + 1] = fast_exp2(s[j][2 * hh + 1] - m_use);
        sum += s[j][2 * hh] + s[j][2 * hh + 1];
      }
      l_run[hh] = l_run[hh] * alpha[hh] + sum;
    }
#pragma unroll
    for (int n = 0; n < kD / 8; ++n) {
      o_acc[n][0] *= alpha[0];
      o_acc[n][1] *= alpha[0];
      o_acc[n][2] *= alpha[1];
      o_acc[n][3] *= alpha[1];
    }
    // ---- O += P V : one 16-token step ----
    if constexpr (kRing) {
      cp_async_wait<2>();                                // all but the two newest groups: V(i) has landed
      __syncwarp();
    }
    {
      uint32_t a[4];
      if constexpr (kFp8) {
        // E4M3 V: the transposing 16-bit ldmatrix hands a thread, per 16-byte chunk (16 head dimensions) and token
        // half, the bytes V[2tq][2g], V[2tq][2g+1], V[2tq+1][2g], V[2tq+1][2g+1].  Bytes 0 and 2 are the B fragment
        // of an MMA over the chunk's EVEN dimensions, bytes 1 and 3 of one over its ODD dimensions; each pair is
        // widened to FP16 in registers (exact) and P is FP16 too.  No widened tile in shared memory; the accumulators
        // come out with the chunk's dimensions interleaved, which the merge below undoes when it stores them.
        a[0] = pack_f16(s[0][0], s[0][1]);
        a[1] = pack_f16(s[0][2], s[0][3]);
        a[2] = pack_f16(s[1][0], s[1][1]);
        a[3] = pack_f16(s[1][2], s[1][3]);
#pragma unroll
        for (int kb = 0; kb < kD / 128; ++kb) {
#pragma unroll
          for (int cp = 0; cp < 4; ++cp) {
            uint32_t r0, r1, r2, r3;   // chunk c: tokens 0-7, 8-15; chunk c + 1: tokens 0-7, 8-15
            ldmatrix_x4_trans(r0, r1, r2, r3, v_addr + kb * (kTile * 128) + swz128(v_lane_row, cp * 2 + v_lane_chunk));
            const int c = kb * 8 + cp * 2;
            mma_f16_16816(o_acc[2 * c], a, e4m3_pair_to_f16x2<0x4420>(r0), e4m3_pair_to_f16x2<0x4420>(r1));
            mma_f16_16816(o_acc[2 * c + 1], a, e4m3_pair_to_f16x2<0x4431>(r0), e4m3_pair_to_f16x2<0x4431>(r1));
            mma_f16_16816(o_acc[2 * c + 2], a, e4m3_pair_to_f16x2<0x4420>(r2), e4m3_pair_to_f16x2<0x4420>(r3));
            mma_f16_16816(o_acc[2 * c + 3], a, e4m3_pair_to_f16x2<0x4431>(r2), e4m3_pair_to_f16x2<0x4431>(r3));
          }
        }
      } else {
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int kb = 0; kb < kD / 64; ++kb) {
#pragma unroll
          for (int cp = 0; cp < 4; ++cp) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, v_addr + kb * (kTile * 128) + swz128(v_lane_row, cp * 2 + v_lane_chunk));
            mma_bf16_16816(o_acc[kb * 8 + cp * 2], a, b0, b1);
            mma_bf16_16816(o_acc[kb * 8 + cp * 2 + 1], a, b2, b3);
          }
        }
      }
    }
    __syncwarp();          // every lane is done with this stage before the next iteration's copies may land in it
    if constexpr (kRing) {
      // V(i) is consumed: its buffer takes K of the tile after next (operand 2i + 4), whose offsets replace this tile's
      tile_offsets(ti + 2 * kWarps, stage);
      issue_operand(p.k, stage, ring(n_op + 4), ti + 2 * kWarps < tile_hi);
    }
    stage = (stage + 1) % kStages;
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }

  // ---- merge the warps' states through shared memory (aliases the tile buffers) ----
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(tiles);           // [warp][16][256]
  float* red_m = red_o + kWarps * 16 * kD;                  // [warp][16]
  float* red_l = red_m + kWarps * 16;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = g + hh * 8;
    float* dst = red_o + ((size_t)warp * 16 + r) * kD;
    if constexpr (kFp8) {
      // accumulator 2c holds the even, 2c + 1 the odd dimensions of 16-dimension chunk c: this thread's four are
      // the consecutive dimensions 16c + 4tq .. + 3
#pragma unroll
      for (int c = 0; c < kD / 16; ++c)
        *reinterpret_cast<float4*>(dst + c * 16 + 4 * tq) =
            make_float4(o_acc[2 * c][2 * hh], o_acc[2 * c + 1][2 * hh], o_acc[2 * c][2 * hh + 1], o_acc[2 * c + 1][2 * hh + 1]);
    } else {
#pragma unroll
      for (int n = 0; n < kD / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + 2 * tq) = make_float2(o_acc[n][2 * hh], o_acc[n][2 * hh + 1]);
    }
    if (tq == 0) {
      red_m[warp * 16 + r] = m_run[hh];
      red_l[warp * 16 + r] = l_run[hh];
    }
  }
  __syncthreads();
  const bool split_mode = p.num_splits > 1;
  if (p.cluster_combine) {
    // The splits of this (row, KV head) are the CTAs of one cluster: each normalises its own partial, all of them
    // write theirs into the leader's shared memory (distributed shared memory; the leader's tile buffers are free
    // once every CTA of the cluster has passed the first cluster barrier), and the leader combines, gates and stores.
    // No second kernel and no scratch in global memory.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int kItems = (12 * (kD / 4) + kThreads - 1) / kThreads;   // (head, 4 dimensions) items per thread
    float4 o_loc[kItems];
    float lse_loc[kItems];
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const int idx = tid + k * kThreads;
      o_loc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      lse_loc[k] = -INFINITY;
      if (idx >= p.group * (kD / 4)) continue;
      const int r = idx / (kD / 4), c4 = idx % (kD / 4);
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red_m[w * 16 + r]);
      const float m_use = m == -INFINITY ? 0.f : m;
      float l = 0.f;
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float mw = red_m[w * 16 + r];
        if (mw == -INFINITY) continue;
        const float sc = fast_exp2(mw - m_use);
        l += red_l[w * 16 + r] * sc;
        const float4 ow = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + r) * kD + c4 * 4);
        o.x += ow.x * sc; o.y += ow.y * sc; o.z += ow.z * sc; o.w += ow.w * sc;
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      o_loc[k] = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
      lse_loc[k] = l > 0.f ? m_use + log2f(l) : -INFINITY;
    }
    __syncthreads();     // this CTA is done with its merge buffer
    cluster.sync();      // and so is every CTA of the row: the leader's buffers may be written
    float* part_local = reinterpret_cast<float*>(tiles);          // [split][12][kPartStride]
    float* part = cluster.map_shared_rank(part_local, 0);
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const int idx = tid + k * kThreads;
      if (idx >= p.group * (kD / 4)) continue;
      const int r = idx / (kD / 4), c4 = idx % (kD / 4);
      float* dst = part + ((size_t)split * 12 + r) * kPartStride;
      *reinterpret_cast<float4*>(dst + c4 * 4) = o_loc[k];
      if (c4 == 0) dst[kD] = lse_loc[k];
    }
    cluster.sync();      // all partials are in the leader's shared memory
    if (split == 0) {
#pragma unroll
      for (int k = 0; k < kItems; ++k) {
        const int idx = tid + k * kThreads;
        if (idx >= p.group * (kD / 4)) continue;
        const int r = idx / (kD / 4), c4 = idx % (kD / 4);
        const long long slot = (long long)t * p.hq + h * p.group + r;
        float mx = -INFINITY;
        for (int sp = 0; sp < p.num_splits; ++sp) mx = fmaxf(mx, part_local[((size_t)sp * 12 + r) * kPartStride + kD]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float denom = 0.f;
        if (mx != -INFINITY) {
          for (int sp = 0; sp < p.num_splits; ++sp) {
            const float* src = part_local + ((size_t)sp * 12 + r) * kPartStride;
            const float l = src[kD];
            if (l == -INFINITY) continue;
            const float w = fast_exp2(l - mx);
            denom += w;
            const float4 a = *reinterpret_cast<const float4*>(src + c4 * 4);
            acc.x += w * a.x; acc.y += w * a.y; acc.z += w * a.z; acc.w += w * a.w;
          }
        }
        const float inv = denom > 0.f ? p.v_scale / denom : 0.f;
        const uint2 graw = *reinterpret_cast<const uint2*>(p.gate + slot * kD + c4 * 4);
        const float gt[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xFFFF0000u),
                             __uint_as_float(graw.y << 16), __uint_as_float(graw.y & 0xFFFF0000u)};
        const float av[4] = {acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv};
        float res[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a_bf16 = __bfloat162float(__float2bfloat16(av[i]));     // A leaves the attention as BF16
          res[i] = a_bf16 * (1.f / (1.f + __expf(-gt[i])));
        }
        uint2 packed;
        packed.x = pack_bf16(res[0], res[1]);
        packed.y = pack_bf16(res[2], res[3]);
        *reinterpret_cast<uint2*>(p.out + slot * kD + c4 * 4) = packed;
      }
    }
    return;
  }
  for (int idx = tid; idx < p.group * (kD / 4); idx += kThreads) {
    const int r = idx / (kD / 4), c4 = idx % (kD / 4);
    const int head = h * p.group + r;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red_m[w * 16 + r]);
    const float m_use = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = red_m[w * 16 + r];
      if (mw == -INFINITY) continue;
      const float sc = fast_exp2(mw - m_use);
      l += red_l[w * 16 + r] * sc;
      const float4 ow = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + r) * kD + c4 * 4);
      o.x += ow.x * sc; o.y += ow.y * sc; o.z += ow.z * sc; o.w += ow.w * sc;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
    const long long slot = (long long)t * p.hq + head;
    if (split_mode) {
      const long long ps = (long long)split * p.rows * p.hq + slot;
      *reinterpret_cast<float4*>(p.part_o + ps * kD + c4 * 4) = o;
      if (c4 == 0) p.part_lse[ps] = l > 0.f ? m_use + log2f(l) : -INFINITY;
    } else {
      const uint2 graw = *reinterpret_cast<const uint2*>(p.gate + slot * kD + c4 * 4);
      const float gt[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xFFFF0000u),
                           __uint_as_float(graw.y << 16), __uint_as_float(graw.y & 0xFFFF0000u)};
      const float av[4] = {o.x * p.v_scale, o.y * p.v_scale, o.z * p.v_scale, o.w * p.v_scale};
      float res[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a_bf16 = __bfloat162float(__float2bfloat16(av[i]));       // A leaves the attention as BF16
        res[i] = a_bf16 * (1.f / (1.f + __expf(-gt[i])));
      }
      uint2 packed;
      packed.x = pack_bf16(res[0], res[1]);
      packed.y = pack_bf16(res[2], res[3]);
      *reinterpret_cast<uint2*>(p.out + slot * kD + c4 * 4) = packed;
    }
  }
}

// Split combine: out = bf16( bf16( sum_i w_i A_i / sum_i w_i * v_scale ) * sigmoid(gate) ), w_i = 2^(lse_i - max);
// a split that saw no token has lse = -inf and its partial is not read.  One warp per (row, head).
__global__ void __launch_bounds__(256)
atrex_sm100_qsa_combine_kernel(const __grid_constant__ QsaParams p) {
  const int lane = threadIdx.x & 31;
  const long long slot = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long slots = (long long)p.rows * p.hq;
  if (slot >= slots) return;
  float mx = -INFINITY;
  for (int s = 0; s < p.num_splits; ++s) mx = fmaxf(mx, p.part_lse[s * slots + slot]);
  float acc[8], denom = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < p.num_splits; ++s) {
      const float l = p.part_lse[s * slots + slot];
      if (l == -INFINITY) continue;
      const float w = fast_exp2(l - mx);
      denom += w;
      const float4* src = reinterpret_cast<const float4*>(p.part_o + (s * slots + slot) * kD + lane * 8);
      const float4 a = src[0], b = src[1];
      acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * a.z; acc[3] += w * a.w;
      acc[4] += w * b.x; acc[5] += w * b.y; acc[6] += w * b.z; acc[7] += w * b.w;
    }
  }
  const float inv = denom > 0.f ? p.v_scale / denom : 0.f;
  const uint4 graw = *reinterpret_cast<const uint4*>(p.gate + slot * kD + lane * 8);
  const uint32_t gw[4] = {graw.x, graw.y, graw.z, graw.w};
  uint32_t packed[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float g0 = __uint_as_float(gw[i] << 16), g1 = __uint_as_float(gw[i] & 0xFFFF0000u);
    const float a0 = __bfloat162float(__float2bfloat16(acc[2 * i] * inv));
    const float a1 = __bfloat162float(__float2bfloat16(acc[2 * i + 1] * inv));
    packed[i] = pack_bf16(a0 * (1.f / (1.f + __expf(-g0))), a1 * (1.f / (1.f + __expf(-g1))));
  }
  *reinterpret_cast<uint4*>(p.out + slot * kD + lane * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

struct QsaResolved {
  int splits, launches;
  int variant;          // QsaVariant
  bool cluster;         // the splits of a row combine inside the attention kernel (one cluster per row and KV head)
  uint64_t off_lse, off_o, bytes;
};

int qsa_check(const atrex_qsa_sm100_params* p) {
  if (p == nullptr) return report_failure(ATREX_FA_INVALID_VALUE, "parameter block is NULL");
  if (p->struct_bytes != sizeof(atrex_qsa_sm100_params) || p->abi_version != ATREX_QSA_SM100_ABI_VERSION)
    return report_failure(ATREX_FA_ABI_MISMATCH, "struct_bytes / abi_version do not match this library");
  if (p->rows < 0 || p->num_pages < 1 || p->batch < 1 || p->table_width < 1)
    return report_failure(ATREX_FA_INVALID_VALUE, "rows, num_pages, batch and table_width must be positive");
  if (p->page_size < 16 || p->page_size % 16)
    return report_failure(ATREX_FA_INVALID_VALUE, "page size must be a positive multiple of 16");
  if (p->num_kv_heads != 1 && p->num_kv_heads != 2)
    return report_failure(ATREX_FA_INVALID_VALUE, "Hkv must be 1 or 2");
  if (p->num_q_heads != 8 * p->num_kv_heads && p->num_q_heads != 12 * p->num_kv_heads)
    return report_failure(ATREX_FA_INVALID_VALUE, "GQA ratio must be 8 or 12");
  if (p->dtype != ATREX_FA_BF16 && p->dtype != ATREX_FA_E4M3)
    return report_failure(ATREX_FA_UNSUPPORTED, "dtype must be BF16 or E4M3");
  if (p->num_splits < 0 || p->num_splits > kMaxSplits)
    return report_failure(ATREX_FA_INVALID_VALUE, "num_splits must lie in [0, 16]");
  if (!(p->sm_scale > 0.f) || !(p->v_scale > 0.f) || p->sm_scale > 3.0e38f || p->v_scale > 3.0e38f)
    return report_failure(ATREX_FA_INVALID_VALUE, "sm_scale and v_scale must be positive and finite");
  if (p->rows > 0 && (!p->q || !p->k_cache || !p->v_cache || !p->block_ids || !p->query_positions ||
                      !p->block_table || !p->token_to_req || !p->output_gate || !p->out))
    return report_failure(ATREX_FA_INVALID_VALUE, "a tensor pointer is NULL");
  const uint64_t es = p->dtype == ATREX_FA_E4M3 ? 1 : 2;
  const int64_t strides[] = {p->q_row_stride, p->q_head_stride, p->kv_page_stride, p->kv_row_stride, p->kv_head_stride};
  for (int64_t st : strides)
    if (st < 0 || ((uint64_t)st * es) % 16) return report_failure(ATREX_FA_UNSUPPORTED, "a Q / K / V stride is not a multiple of 16 bytes");
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k_cache) |
                         reinterpret_cast<uintptr_t>(p->v_cache) | reinterpret_cast<uintptr_t>(p->output_gate) |
                         reinterpret_cast<uintptr_t>(p->out);
  if (ptrs & 15u) return report_failure(ATREX_FA_UNSUPPORTED, "Q, K, V, gate and out must be 16-byte aligned");
  return ATREX_FA_OK;
}

// The three instantiations: BF16 with two-stage buffers (six warps), BF16 with the operand ring (eight warps; calls of
// one wave), E4M3 (eight warps).
enum QsaVariant { kBf16Stages = 0, kBf16Ring = 1, kE4m3 = 2, kVariants = 3 };
struct QsaLaunchShape {
  const void* kernel;
  int threads, smem, warps;
};
QsaLaunchShape qsa_shape(int variant) {
  switch (variant) {
    case kBf16Ring:
      return {reinterpret_cast<const void*>(&atrex_sm100_qsa_kernel<false, true>), QsaCfg<false, true>::kThreads,
              QsaCfg<false, true>::kSmemBytes, QsaCfg<false, true>::kWarps};
    case kE4m3:
      return {reinterpret_cast<const void*>(&atrex_sm100_qsa_kernel<true, false>), QsaCfg<true, false>::kThreads,
              QsaCfg<true, false>::kSmemBytes, QsaCfg<true, false>::kWarps};
    default:
      return {reinterpret_cast<const void*>(&atrex_sm100_qsa_kernel<false, false>), QsaCfg<false, false>::kThreads,
              QsaCfg<false, false>::kSmemBytes, QsaCfg<false, false>::kWarps};
  }
}

// Kernel attributes, once per device.
cudaError_t qsa_prepare() {
  static std::atomic<int> prepared[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || prepared[dev].load(std::memory_order_acquire)) return cudaSuccess;
  for (int v = 0; v < kVariants && e == cudaSuccess; ++v) {
    const QsaLaunchShape sh = qsa_shape(v);
    e = cudaFuncSetAttribute(sh.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sh.smem);
  }
  if (e == cudaSuccess) prepared[dev].store(1, std::memory_order_release);
  return e;
}

// How many clusters of `splits` CTAs of the attention kernel this device can hold at once (one CTA of up to 214 KB per
// SM and a cluster inside one GPC); 0 when it cannot be asked (no device: the plan of a CPU-side test).  Asked once
// per size, variant and device.
int qsa_resident_clusters(int variant, int splits) {
  static std::atomic<int> cache[64][kVariants][kMaxClusterSplits + 1];   // value + 1; 0 = not asked yet
  int dev = 0;
  if (splits < 2 || splits > kMaxClusterSplits || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  const int seen = cache[dev][variant][splits].load(std::memory_order_acquire);
  if (seen > 0) return seen - 1;
  if (qsa_prepare() != cudaSuccess) return 0;
  const QsaLaunchShape sh = qsa_shape(variant);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, (unsigned)splits, 1);
  cfg.blockDim = dim3(sh.threads);
  cfg.dynamicSmemBytes = sh.smem;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 1;
  attr.val.clusterDim.y = (unsigned)splits;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, sh.kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();   // the query failed, nothing was launched: not this call's error
    clusters = 0;
  }
  cache[dev][variant][splits].store(clusters + 1, std::memory_order_release);
  return clusters;
}

void qsa_resolve(const atrex_qsa_sm100_params* p, int sm_count, QsaResolved* r) {
  int splits = p->num_splits;
  const bool fp8 = p->dtype == ATREX_FA_E4M3;
  const long long ctas = (long long)p->rows * p->num_kv_heads;
  // BF16 calls of one wave whose CTAs have long token lists (at most four splits of a row: 33 tiles or more per CTA)
  // take the operand ring with eight warps (see QsaCfg); with short lists the ring's longer start costs more than
  // the warps bring (16 rows: 15.8 us against 13.5 with the two-stage kernel).
  const long long upper = splits == 0 ? (ctas > 0 ? sm_count / ctas : 0) : splits;   // splits, or the most that fit
  const bool ring = !fp8 && ctas > 0 && upper >= 1 && upper <= 4 && ctas * (splits == 0 ? 1 : splits) <= sm_count;
  r->variant = fp8 ? kE4m3 : (ring ? kBf16Ring : kBf16Stages);
  if (splits == 0) {
    // rows x KV heads CTAs, one resident per SM: split the token lists while all CTAs still run in ONE wave
    // (measured on 64 decode rows: 2 splits = 128 CTAs 37 us, 3 splits = 192 CTAs in two waves 46 us)
    const long long want = ctas > 0 ? sm_count / ctas : 1;
    splits = (int)(want < 1 ? 1 : (want > kMaxSplits ? kMaxSplits : want));
    // A CTA's time is the number of rounds its warps make over its tiles (a full list has kRowTilesMax tiles): the
    // fewest splits that still give that many rounds leave less to combine (16 rows, six warps: 9 splits 14.4 us
    // per call, 8 splits 13.6, 7 splits - a fourth round - 15.8).
    const int warps = qsa_shape(r->variant).warps;
    auto rounds = [&](int n) { return ((kRowTilesMax + n - 1) / n + warps - 1) / warps; };
    while (splits > 1 && rounds(splits - 1) == rounds(splits)) --splits;
  }
  r->splits = splits;
  // The splits of a row combine inside the attention kernel when every row's cluster can be resident at once (one
  // wave, as for the split count itself); otherwise through scratch and the combine kernel.
  r->cluster = splits >= 2 && splits <= kMaxClusterSplits && qsa_resident_clusters(r->variant, splits) >= ctas;
  r->launches = splits > 1 && !r->cluster ? 2 : 1;
  const uint64_t slots = (uint64_t)p->rows * p->num_q_heads;
  r->off_lse = 0;
  const bool scratch = splits > 1 && !r->cluster;   // partials in global memory only for the combine kernel
  r->off_o = scratch ? (4ull * splits * slots + 255) / 256 * 256 : 0;
  r->bytes = scratch ? r->off_o + 4ull * splits * slots * kD : 0;
}

}  // namespace
}  // namespace atrex_sm100

using namespace atrex_sm100;

extern "C" {

int atrex_qsa_sm100_abi_version(void) { return ATREX_QSA_SM100_ABI_VERSION; }
size_t atrex_qsa_sm100_params_bytes(void) { return sizeof(atrex_qsa_sm100_params); }

int atrex_qsa_sm100_plan(const atrex_qsa_sm100_params* p, atrex_qsa_sm100_plan_info* plan) {
  clear_failure();
  if (plan == nullptr) return report_failure(ATREX_FA_INVALID_VALUE, "plan is NULL");
  int st = qsa_check(p);
  if (st != ATREX_FA_OK) return st;
  int sms = p->sm_count;
  if (sms <= 0 && (st = current_sm_count(&sms)) != ATREX_FA_OK) return st;
  QsaResolved r;
  qsa_resolve(p, sms, &r);
  plan->num_splits = r.splits;
  plan->kernel_launches = r.launches;
  plan->workspace_bytes = r.bytes;
  return ATREX_FA_OK;
}

int atrex_qsa_sm100_forward(const atrex_qsa_sm100_params* p, void* workspace, uint64_t workspace_bytes, void* stream_ptr) {
  clear_failure();
  int st = qsa_check(p);
  if (st != ATREX_FA_OK) return st;
  int sms = 0;
  if ((st = current_sm_count(&sms)) != ATREX_FA_OK) return st;   // also rejects devices that are not sm_100
  if (p->sm_count > 0) sms = p->sm_count;
  QsaResolved r;
  qsa_resolve(p, sms, &r);
  if (r.bytes > 0 && (workspace == nullptr || workspace_bytes < r.bytes || (reinterpret_cast<uintptr_t>(workspace) & 255u)))
    return report_failure(ATREX_FA_WORKSPACE_TOO_SMALL, "workspace missing, misaligned or too small");
  if (p->rows == 0) return ATREX_FA_OK;
  {
    const cudaError_t e = qsa_prepare();
    if (e != cudaSuccess) return report_failure(ATREX_FA_CUDA_ERROR, "cudaFuncSetAttribute (sparse attention kernels)", e);
  }
  QsaParams k = {};
  k.q = p->q; k.k = p->k_cache; k.v = p->v_cache; k.ids = p->block_ids; k.pos = p->query_positions;
  k.table = p->block_table; k.req = p->token_to_req;
  k.gate = static_cast<const __nv_bfloat16*>(p->output_gate);
  k.out = static_cast<__nv_bfloat16*>(p->out);
  k.status = p->device_status;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (r.bytes > 0) {
    k.part_lse = reinterpret_cast<float*>(ws + r.off_lse);
    k.part_o = reinterpret_cast<float*>(ws + r.off_o);
  }
  k.q_row_stride = p->q_row_stride; k.q_head_stride = p->q_head_stride;
  k.kv_page_stride = p->kv_page_stride; k.kv_row_stride = p->kv_row_stride; k.kv_head_stride = p->kv_head_stride;
  k.rows = p->rows; k.hq = p->num_q_heads; k.hkv = p->num_kv_heads; k.group = p->num_q_heads / p->num_kv_heads;
  k.num_pages = p->num_pages; k.page_size = p->page_size; k.batch = p->batch; k.table_width = p->table_width;
  k.pos64 = p->positions_are_int64 ? 1 : 0;
  k.num_splits = r.splits;
  k.cluster_combine = r.cluster ? 1 : 0;
  k.scale_log2 = p->sm_scale * kLog2e;
  k.v_scale = p->v_scale;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const dim3 grid((unsigned)((long long)p->rows * p->num_kv_heads), (unsigned)r.splits, 1);
  const QsaLaunchShape sh = qsa_shape(r.variant);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(sh.threads);
  cfg.dynamicSmemBytes = sh.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  if (r.cluster) {   // the CTAs (x, 0 .. splits - 1) of one row and KV head form a cluster
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 1;
    attr.val.clusterDim.y = (unsigned)r.splits;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
  }
  void* args[] = {&k};
  cudaError_t e = cudaLaunchKernelExC(&cfg, sh.kernel, args);
  if (e != cudaSuccess) return report_failure(ATREX_FA_CUDA_ERROR, "launch of the sparse attention kernel", e);
  if (r.splits > 1 && !r.cluster) {
    const long long slots = (long long)p->rows * p->num_q_heads;
    e = launch_kernel(atrex_sm100_qsa_combine_kernel, dim3((unsigned)((slots + 7) / 8)), dim3(256), 0, stream, k);
    if (e != cudaSuccess) return report_failure(ATREX_FA_CUDA_ERROR, "launch of the sparse attention combine kernel", e);
  }
  return ATREX_FA_OK;
}

}  // extern "C"
