// Single-row-tile attention kernel on tcgen05 tensor cores: one 128-row tile of packed GQA rows per
// work item, S double-buffered in TMEM, optional split-KV.  BF16 and FP8 E4M3 inputs, head_dim 128 and
// 256, BF16 output (or FP32 partials for the combine kernel).
//
// It serves (a) head_dim-256 prefill, the shape of the reference's Blackwell prefill
// (src/nvidia/flash_attn/sm103/prefill_cutedsl.py:146-4331: BF16 tile_n 64 / FP8 tile_n 128,
// S ping-pong + O = all 512 TMEM columns, :395-405), (b) every FP8 call, (c) BF16 prefill whose GQA
// group does not divide 128, and (d) short-query decode / speculative verify with 17..128 packed rows
// (the reference's tcgen05 decode, src/nvidia/flash_attn/sm103/decode_cutedsl.py:453-2873, keeps K as
// the M operand instead; here the packed rows are M and the spare rows are idle, which an HBM-bound
// call can afford):
//
//   * TMEM = S0 | S1 | O (tile_n + tile_n + head_dim columns); warp 8 issues QK^T for tile j+1 into
//     the other S buffer while the softmax warps work on tile j, then P V for tile j as soon as its P
//     is in TMEM, so the matrix work of one tile hides behind the softmax of the next;
//   * the score load and row maximum of tile j+1 stay in front of tile j+1 and are not run under the exponentials
//     of tile j: S(j+1) follows P V(j-1) on the tensor pipe (P lies over S, so the order is fixed) and is complete
//     only late in tile j's exponentials, and a wait for it there stalls longer than the load costs where it is
//     (E4M3 head_dim-256 prefill 1 497 against 1 602 TFLOP/s; with P in shared memory, which frees the order, 1 484);
//   * warps 0-7 are the softmax: TWO threads per row, each with half of the tile's key columns and half
//     of the O columns, exchanging their partial row maximum through shared memory (two warps per
//     scheduler keep the MUFU pipe busy where one cannot);
//   * warps 9 and 10 are the K (+Q) and V TMA producers over a 4-slot ring of 32 KB tiles; every CTA
//     loads its own copy; Q comes by TMA when the GQA group divides 128, otherwise warp 11 copies the rows
//     into the swizzled tile, one item ahead; warp 11 also resolves the next work item for the softmax warps;
//   * FP8: q_descale * k_descale ride in the softmax scale, P is written as E4M3 shifted up by 2^4
//     with a lazy-rescale threshold of 2^4 (P <= 256 < 448, prefill_cutedsl.py:2577-2593), V stays
//     MN-major E4M3 in shared memory, v_descale is applied in the epilogue;
//   * split-KV: each split takes a balanced share of the tile's KV tiles and writes a normalised
//     FP32 partial + log2 LSE; empty splits publish LSE = -inf.
#include <cuda_fp8.h>

#include "fa_kernels.cuh"
#include "softmax_math.cuh"
#include "umma.cuh"

namespace atrex_sm100 {

namespace {

constexpr int kRows = 128;          // packed rows per work item (UMMA M)
constexpr int kRing = 4;            // K/V ring slots of 32 KB
// Pairs of every 8 whose exponential runs on the FMA pipe.  FP8 head_dim-256 prefill, alternating builds in one call:
// 30-step runs 1 574 - 1 586 / 1 579 / 1 602 - 1 606 TFLOP/s with 0 / 1 / 2 of 8; 150-step runs at the power cap
// 1 540 - 1 550 / 1 559 / 1 504 - 1 510 with 1 / 2 / 3 of 8.
#ifndef ATREX_UMMA1_POLY_OF8
#define ATREX_UMMA1_POLY_OF8 2
#endif
constexpr int kPolyOf8_1 = ATREX_UMMA1_POLY_OF8;
constexpr int kSoftmaxWarps1 = 8;                 // two threads per row: 2 x 4 warps
constexpr int kMmaWarp1 = 8, kKWarp1 = 9, kVWarp1 = 10, kQWarp1 = 11;   // warp 11 copies Q where TMA cannot
constexpr int kThreads1 = (kSoftmaxWarps1 + 4) * 32;       // 384 threads, up to 168 registers each

template <int D, bool kFp8>
struct Cfg1 {
  static constexpr int kEsz = kFp8 ? 1 : 2;
  static constexpr int kRowBytes = D * kEsz;
  static constexpr int kSlotBytes = 32768;
  static constexpr int kBN = (kSlotBytes / kRowBytes) < 128 ? (kSlotBytes / kRowBytes) : 128;   // keys per tile
  static constexpr uint32_t kTmemCols = 512;
  static constexpr int kNKB = kRowBytes / 128;                // 128-byte column blocks per row
  static constexpr int kQBytes = kRows * kRowBytes;
  static constexpr int kQBlock = kRows * 128;                 // bytes of one Q column block
  static constexpr int kKVBlock = kBN * 128;                  // bytes of one K/V column block
  static constexpr int kKStepsQK = kNKB * 4;                  // 32 bytes of the head dimension per UMMA
  static constexpr int kKStepsPV = kBN * kEsz / 32;           // 32 bytes of P per row per UMMA
  static constexpr int kPVStepBytes = (32 / kEsz) * 128;      // V rows consumed per UMMA x 128 B
  static constexpr float kThreshold = kFp8 ? 4.f : 8.f;       // lazy-rescale threshold (log2 units)
  static constexpr float kShift = kFp8 ? 4.f : 0.f;           // P is stored as 2^shift * p
  static constexpr int kOffKV = kQBytes;
  static constexpr int kOffBar = kOffKV + kRing * kSlotBytes;
  static constexpr int kOffXchg = kOffBar + 256;              // [parity][half][row] floats for the row max / sum
  static constexpr int kOffItem = kOffXchg + 2 * 2 * kRows * 4;   // two ItemSlot
  static constexpr int kSmemBytes = kOffItem + 2 * 64;
  static constexpr uint32_t kFmt = kFp8 ? 0u : 1u;            // E4M3 (f8f6f4) / BF16 (f16)
  static_assert(2 * kBN + D <= 512, "S0 | S1 | O must fit the 512 TMEM columns");
  static_assert(kBN / 2 >= 32, "each softmax thread takes at least one 32-column chunk");
};

// Development timeline: with -DATREX_UMMA1_TRACE CTA 0 records clock64() at the marked points.
#ifdef ATREX_UMMA1_TRACE
__device__ long long g_umma1_trace[8192];
#define TRACE1(slot, idx) do { if (blockIdx.x == 0 && (idx) < 256) g_umma1_trace[(slot) * 256 + (idx)] = clock64(); } while (0)
#else
#define TRACE1(slot, idx) do { } while (0)
#endif

enum Bar256 { bQFull = 0, bQEmpty = 1, bKVFull = 2, bKVEmpty = 6, bSFull = 10, bPFull = 12, bOFull = 14, bOFinal = 15,
              bItemFull = 16, bItemEmpty = 18, bCount = 20 };

struct Item256 {
  int b, kvh, split, n_splits, row0, q_start, q_len, rows_total, kv_len, k_start, off, tile_lo, n_tiles;
};
// What warp 11 resolves one item ahead for the softmax warps (two slots in shared memory): the item, whether there
// is one, and the request's scales.
struct __align__(16) ItemSlot {
  Item256 it;
  int valid;
  float scale_log2, dv;
};
static_assert(sizeof(ItemSlot) == 64, "four 16-byte vectors");

// Work item `item` -> (row tile, KV head, KV split), split fastest.  Row tiles come from the device-side plan
// (heaviest request first, last row tile of a request first) or, when a request cannot have more than one
// row tile, are simply the requests.  False when past the end.
template <int BN>
__device__ __forceinline__ bool decode_item256(const FwdParams& p, int item, Item256& it) {
  int rest;
  if (p.tail_splits > 1) {
    // unsplit items of the first requests, then tail_splits items per (request, KV head) of the last ones
    const int n_unsplit = p.tail_first * p.num_kv_heads;
    if (item < n_unsplit) {
      rest = item;
      it.split = 0;
      it.n_splits = 1;
    } else {
      const int j = item - n_unsplit;
      it.split = j % p.tail_splits;
      rest = n_unsplit + j / p.tail_splits;
      it.n_splits = p.tail_splits;
    }
  } else {
    it.split = item % p.num_splits;
    rest = item / p.num_splits;
    it.n_splits = p.num_splits;
  }
  it.kvh = rest % p.num_kv_heads;
  const int tile_rank = rest / p.num_kv_heads;
  if (p.order == nullptr) {
    if (tile_rank >= p.batch) return false;
    it.b = tile_rank;
    it.row0 = 0;
  } else {
    if (tile_rank >= p.tile_prefix[p.batch]) return false;
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.tile_prefix[mid] <= tile_rank) lo = mid; else hi = mid;
    }
    it.b = p.order[lo];
    const int tiles_b = p.tile_prefix[lo + 1] - p.tile_prefix[lo];
    it.row0 = (tiles_b - 1 - (tile_rank - p.tile_prefix[lo])) * kRows;
  }
  it.q_start = p.cu_seqlens_q[it.b];
  it.q_len = p.cu_seqlens_q[it.b + 1] - it.q_start;
  it.rows_total = it.q_len * p.group;
  request_kv(p, it.b, it.kv_len, it.k_start);
  it.off = request_off(p, it.b, it.kv_len, it.q_len);
  it.tile_lo = 0;
  it.n_tiles = 0;
  if (it.row0 >= it.rows_total) return true;   // request without query rows: an item with no work
  const int qi_lo = it.row0 / p.group;
  const int qi_hi = min(it.q_len - 1, (it.row0 + kRows - 1) / p.group);
  int kv_end = it.kv_len, kv_begin = 0;
  if (p.window_right >= 0) kv_end = min(it.kv_len, right_bound(p, qi_hi + it.off));
  if (p.window_left >= 0) kv_begin = max(0, qi_lo + it.off - p.window_left);
  if (kv_end > kv_begin) {
    const int t0 = kv_begin / BN, n = (kv_end + BN - 1) / BN - t0;
    const int lo_t = (int)(((long long)n * it.split) / it.n_splits);
    const int hi_t = (int)(((long long)n * (it.split + 1)) / it.n_splits);
    it.tile_lo = t0 + lo_t;
    it.n_tiles = hi_t - lo_t;
  }
  return true;
}

// K or V tiles of one item, issued by one thread; NB boxes of (BN / NB) rows per tile, each box one
// copy per 128-byte column block.  Page ids of tile j+1 are fetched before the wait for tile j's slot.
template <int D, bool kFp8, int NB>
__device__ __forceinline__ bool produce_tiles256(const FwdParams& p, const Item256& it, int is_v, uint8_t* kv_smem,
                                                 uint64_t* bars, uint32_t& seq, int pshift) {
  using C = Cfg1<D, kFp8>;
  constexpr int kBoxRows = C::kBN / NB;
  constexpr uint32_t kBoxBytes = kBoxRows * 128u;
  constexpr int kInner = 128 / C::kEsz;   // elements per 128-byte block
  const CUtensorMap* map = is_v ? &p.v_map : &p.k_map;
  const int8_t(&perm)[3] = is_v ? p.v_perm : p.k_perm;
  const int32_t* table = p.page_size ? p.block_table + (int64_t)it.b * p.block_table_row_stride : nullptr;
  const int row_mask = p.page_size - 1;
  auto page_id = [&](int tok) -> int {
    if (table == nullptr) return 0;
    if (tok >= it.kv_len) return -1;
    const int pg = table[pshift >= 0 ? tok >> pshift : tok / p.page_size];
    return (pg >= 0 && pg < p.num_pages) ? pg : -1;
  };
  int cur[NB], nxt[NB];
  int tok0 = it.tile_lo * C::kBN;
#pragma unroll
  for (int x = 0; x < NB; ++x) cur[x] = page_id(tok0 + x * kBoxRows);
  for (int j = 0; j < it.n_tiles; ++j, tok0 += C::kBN) {
    if (j + 1 < it.n_tiles) {
#pragma unroll
      for (int x = 0; x < NB; ++x) nxt[x] = page_id(tok0 + C::kBN + x * kBoxRows);
    }
    const uint32_t slot = seq % kRing;
    if (seq >= (uint32_t)kRing && !mbar_wait(&bars[bKVEmpty + slot], ((seq / kRing) - 1) & 1u)) return false;
    uint8_t* dst = kv_smem + slot * C::kSlotBytes;
    int live = 0;
#pragma unroll
    for (int x = 0; x < NB; ++x) live += (cur[x] >= 0 && tok0 + x * kBoxRows < it.kv_len) ? 1 : 0;
    mbar_arrive_expect_tx(&bars[bKVFull + slot], (uint32_t)live * kBoxBytes * C::kNKB);
#pragma unroll
    for (int x = 0; x < NB; ++x) {
      const int tok = tok0 + x * kBoxRows;
      if (cur[x] < 0 || tok >= it.kv_len) continue;
      const int row = p.page_size ? (pshift >= 0 ? tok & row_mask : tok % p.page_size) : it.k_start + tok;
#pragma unroll
      for (int kb = 0; kb < C::kNKB; ++kb)
        tma_load_kv(dst + kb * C::kKVBlock + x * kBoxBytes, map, &bars[bKVFull + slot], kb * kInner, it.kvh, row,
                    cur[x], perm);
    }
#pragma unroll
    for (int x = 0; x < NB; ++x) cur[x] = nxt[x];
    seq += 2;
  }
  return true;
}

// One tile of keys for half a row: the 128 rows of a tile are served by 8 softmax warps, two threads per
// row with half of the tile's key columns each, so that two softmax warps per scheduler interleave on the
// MUFU pipe (one warp alone cannot keep it busy).  Step 1 loads the thread's scores from TMEM, masks
// them and returns their (unscaled) maximum.
template <int D, bool kFp8, bool kMask>
__device__ __forceinline__ float half_max(uint32_t s_tmem, uint32_t (&s)[Cfg1<D, kFp8>::kBN / 2], int col0, int vis_lo,
                                          int vis_hi) {
  constexpr int N = Cfg1<D, kFp8>::kBN / 2;
#pragma unroll
  for (int c = 0; c < N / 32; ++c) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
  tmem_ld_wait();
  if (kMask) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int col = col0 + i;
      if (col < vis_lo || col >= vis_hi) s[i] = 0xff800000u;  // -inf
    }
  }
  float mxv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < N; i += 8) {   // 3-input max: half the instructions of a pairwise reduction
    mxv[0] = fmax3(mxv[0], __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
    mxv[1] = fmax3(mxv[1], __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
    mxv[2] = fmax3(mxv[2], __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
    mxv[3] = fmax3(mxv[3], __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
  }
  return fmaxf(fmaxf(mxv[0], mxv[1]), fmaxf(mxv[2], mxv[3]));
}

// Step 2: P = 2^(s * scale + neg_m) (neg_m includes the FP8 shift) written over the first columns of the
// thread's OWN score columns (BF16 pairs, or four E4M3 per column); returns the sum of the probabilities.
template <int D, bool kFp8, int kPoly>
__device__ __forceinline__ float half_exp(uint32_t s_tmem, const uint32_t (&s)[Cfg1<D, kFp8>::kBN / 2], float scale_log2,
                                          float neg_m) {
  constexpr int N = Cfg1<D, kFp8>::kBN / 2;
  const f32x2 scale2 = pack2(scale_log2, scale_log2), negm2 = pack2(neg_m, neg_m);
  f32x2 sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
  for (int c = 0; c < N / 32; ++c) {
    if constexpr (kFp8) {
      uint32_t packed[8];
      exp32_e4m3<kPoly>(&s[c * 32], scale2, negm2, sum2, packed);
      tmem_st8(s_tmem + c * 8, packed);
    } else {
      uint32_t packed[16];
      exp32_bf16<kPoly>(&s[c * 32], scale2, negm2, sum2, packed);
      tmem_st16(s_tmem + c * 16, packed);
    }
  }
  return sum_of(sum2);
}

// Barrier that also ORs a predicate over the group: a bounded wait that expired in one thread takes the
// whole group out of its loop together (a plain bar.sync would strand the others).
__device__ __forceinline__ bool group_barrier_or(int id, int threads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.or.pred p, %2, %3, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(out)
      : "r"((uint32_t)pred), "r"(id), "r"(threads)
      : "memory");
  return out != 0;
}

#define WAIT256(bar_ptr, parity, code)                            \
  if (!mbar_wait((bar_ptr), (parity))) {                          \
    if (p.status) atomicExch(p.status, (code));                   \
    atomicExch(abort_flag, 1);                                    \
    break;                                                        \
  }

template <int D, bool kFp8>
__global__ void __launch_bounds__(kThreads1, 1)
atrex_sm100_fwd_umma1_kernel(const __grid_constant__ FwdParams p) {
  using C = Cfg1<D, kFp8>;
  constexpr int BN = C::kBN;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + C::kOffKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  int* abort_flag = reinterpret_cast<int*>(bars + 21);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0 && p.status) atomicExch(p.status, kBadSmemAlignment);
    return;
  }
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(&bars[bQFull], 1);   // the K warp's TMA transaction, or lane 0 of the Q-copying warp
    mbar_init(&bars[bQEmpty], 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&bars[bKVFull + s], 1);
      mbar_init(&bars[bKVEmpty + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars[bSFull + b], 1);
      mbar_init(&bars[bPFull + b], 2 * kRows);
    }
    mbar_init(&bars[bOFull], 1);
    mbar_init(&bars[bOFinal], 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars[bItemFull + s], 1);
      mbar_init(&bars[bItemEmpty + s], kSoftmaxWarps1);
    }
    fence_barrier_init();
  }
  if (warp == kMmaWarp1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t o_col = 2 * BN;
  const int step = gridDim.x;

  if (warp == kKWarp1 || warp == kVWarp1) {
    // ------------------------------- TMA producers: K (+Q) and V -------------------------------
    if (lane == 0) {
      const int is_v = warp == kVWarp1;
      if (!is_v) prefetch_tensormap(&p.q_map);
      prefetch_tensormap(is_v ? &p.v_map : &p.k_map);
      const int boxes = BN / p.box_rows;
      const int pshift = (p.page_size > 0 && (p.page_size & (p.page_size - 1)) == 0) ? __ffs(p.page_size) - 1 : -1;
      constexpr int kInner = 128 / C::kEsz;
      uint32_t it_count = 0, seq = (uint32_t)is_v;
      bool q_issued = false;
      for (int item = blockIdx.x;; item += step) {
        Item256 it;
        if (!decode_item256<BN>(p, item, it)) break;
        if (*(volatile int*)abort_flag) break;
        if (!is_v && p.q_via_tma) {
          if (it_count > 0) WAIT256(&bars[bQEmpty], (it_count - 1) & 1u, kWaitEmptyTimeout)
          mbar_arrive_expect_tx(&bars[bQFull], (uint32_t)C::kQBytes);
          q_issued = true;
#pragma unroll
          for (int kb = 0; kb < C::kNKB; ++kb)
            tma_load_3d(q_smem + kb * C::kQBlock, &p.q_map, &bars[bQFull], kb * kInner, it.kvh * p.group,
                        it.q_start + it.row0 / p.group);
        }
        bool ok;
        switch (boxes) {
          case 1: ok = produce_tiles256<D, kFp8, 1>(p, it, is_v, kv_smem, bars, seq, pshift); break;
          case 2: ok = produce_tiles256<D, kFp8, 2>(p, it, is_v, kv_smem, bars, seq, pshift); break;
          case 4: ok = produce_tiles256<D, kFp8, 4>(p, it, is_v, kv_smem, bars, seq, pshift); break;
          default: ok = produce_tiles256<D, kFp8, 8>(p, it, is_v, kv_smem, bars, seq, pshift); break;
        }
        if (!ok) {
          if (p.status) atomicExch(p.status, kWaitEmptyTimeout);
          atomicExch(abort_flag, 1);
          break;
        }
        ++it_count;
      }
      if (q_issued) mbar_wait(&bars[bQFull], (it_count > 0 ? it_count - 1 : 0) & 1u);
      for (uint32_t back = 2; back <= (uint32_t)kRing && back <= seq; back += 2) {
        const uint32_t n = seq - back;
        mbar_wait(&bars[bKVFull + n % kRing], (n / kRing) & 1u);
      }
    }
    __syncwarp();
  } else if (warp == kQWarp1) {
    // ------------------------------- item steward -------------------------------
    // One item ahead of the softmax warps this warp (a) resolves the item (request lookup, lengths, scales: seven
    // or eight dependent global loads, ~2 000 cycles that the 256 softmax threads used to spend at every item
    // boundary) into one of two shared-memory slots, and (b) when the GQA group does not tile the 128 rows as one
    // TMA box, copies the item's Q rows into the swizzled tile with asynchronous 16-byte copies (zeros past the
    // request's rows): the tile is free from the previous item's last S = Q K^T on, so the copy runs under that
    // item's last tiles and epilogue.
    constexpr int kChunksRow = C::kNKB * 8;          // 16-byte chunks per row
    static_assert(kChunksRow <= 32 && 32 % kChunksRow == 0, "a warp-wide copy covers whole rows");
    constexpr int kRpi = 32 / kChunksRow;            // rows per warp-wide copy
    const int sub = lane / kChunksRow, chunk = lane % kChunksRow;
    const uint8_t* q_base = reinterpret_cast<const uint8_t*>(p.q) + chunk * 16;
    uint8_t* dst0 = q_smem + (chunk >> 3) * C::kQBlock;
    ItemSlot* slots = reinterpret_cast<ItemSlot*>(smem + C::kOffItem);
    uint32_t n = 0;
    for (int item = blockIdx.x;; item += step, ++n) {
      ItemSlot* slot = slots + (n & 1u);
      // the softmax warps must have read what the slot held (item n - 2)
      if (n >= 2 && !mbar_wait(&bars[bItemEmpty + (n & 1u)], ((n >> 1) - 1u) & 1u)) {
        if (lane == 0) {
          if (p.status) atomicExch(p.status, kWaitEmptyTimeout);
          atomicExch(abort_flag, 1);
        }
        break;
      }
      if (lane == 0) {
        // resolved straight into the slot: no private copy of the item in this warp's registers
        const bool ok = decode_item256<BN>(p, item, slot->it) && *(volatile int*)abort_flag == 0;
        float dq = 1.f, dk = 1.f, dvs = 1.f;
        if (ok) {
          const int b = slot->it.b, kvh = slot->it.kvh;
          if (p.q_descale) dq = p.q_descale[b * p.q_descale_bs + kvh * p.q_descale_hs];
          if (p.k_descale) dk = p.k_descale[b * p.k_descale_bs + kvh * p.k_descale_hs];
          if (p.v_descale) dvs = p.v_descale[b * p.v_descale_bs + kvh * p.v_descale_hs];
        }
        slot->valid = ok ? 1 : 0;
        slot->scale_log2 = p.softmax_scale * dq * dk * kLog2e;   // > 0 on this route
        slot->dv = dvs;
        mbar_arrive(&bars[bItemFull + (n & 1u)]);                 // release: the slot is written before the arrival
      }
      __syncwarp();
      const Item256 it = slot->it;                              // all lanes, for the copy below
      if (!slot->valid) break;
      if (!p.q_via_tma) {
        if (n > 0 && !mbar_wait(&bars[bQEmpty], (n - 1u) & 1u)) {
          if (lane == 0) {
            if (p.status) atomicExch(p.status, kWaitEmptyTimeout);
            atomicExch(abort_flag, 1);
          }
          break;
        }
        // (query position, head inside the group) of this lane's row advance by kRpi rows per copy: no division
        // per chunk (with one, this copy was slower than the tiles it is meant to hide under)
        int row = it.row0 + sub;
        int pos = row / p.group, head = row - pos * p.group;
#pragma unroll 4
        for (int k = 0; k < kRows / kRpi; ++k) {
          const uint8_t* src = q_base + ((int64_t)(it.q_start + pos) * p.q_row_stride +
                                         (int64_t)(it.kvh * p.group + head) * p.q_head_stride) * C::kEsz;
          const bool valid = row < it.rows_total;
          cp_async_16(dst0 + swz128(k * kRpi + sub, chunk & 7), valid ? src : q_base, valid);
          row += kRpi;
          head += kRpi;
          while (head >= p.group) {
            head -= p.group;
            ++pos;
          }
        }
        cp_async_wait_all();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[bQFull]);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t kIdescQK = umma_idesc(kRows, BN, C::kFmt, C::kFmt, 0, 0);
    constexpr uint32_t kIdescPV = umma_idesc(kRows, D, C::kFmt, C::kFmt, 0, 1);
    const UmmaDesc q_desc0 = umma_desc_split(umma_desc_sw128(smem_u32(q_smem), 16, 1024));
    const UmmaDesc k_desc0 = umma_desc_split(umma_desc_sw128(smem_u32(kv_smem), 16, 1024));
    const UmmaDesc v_desc0 = umma_desc_split(umma_desc_sw128(smem_u32(kv_smem), C::kKVBlock, 1024));
    // ring numbering: tile t of the CTA's whole run has K number 2t and V number 2t + 1
    uint32_t it_count = 0, base = 0, cp[2] = {0, 0};
    [[maybe_unused]] uint32_t tt = 0;
    bool dead = false;
    // The whole warp runs the issue code and lane 0 issues: all operands are warp-uniform.
    const uint32_t lead = lane == 0;
    auto issue_qk = [&](int buf, uint32_t slot) {
      const UmmaDesc kd = k_desc0 + (uint32_t)((slot * C::kSlotBytes) >> 4);
#pragma unroll
      for (int ks = 0; ks < C::kKStepsQK; ++ks) {
        const uint32_t qoff = ((ks >> 2) * C::kQBlock + (ks & 3) * 32) >> 4;
        const uint32_t koff = ((ks >> 2) * C::kKVBlock + (ks & 3) * 32) >> 4;
        if constexpr (kFp8) umma_ss_f8_lead(lead, tmem_base + buf * BN, q_desc0 + qoff, kd + koff, kIdescQK, ks > 0);
        else umma_ss_f16_lead(lead, tmem_base + buf * BN, q_desc0 + qoff, kd + koff, kIdescQK, ks > 0);
      }
      umma_commit_lead(lead, &bars[bSFull + buf]);
      umma_commit_lead(lead, &bars[bKVEmpty + slot]);
    };
    for (int item = blockIdx.x; !dead; item += step) {
      Item256 it;
      if (!decode_item256<BN>(p, item, it)) break;
      if (*(volatile int*)abort_flag) break;
      if (!mbar_wait(&bars[bQFull], it_count & 1u)) { dead = true; break; }
      if (lane == 0) TRACE1(14, it_count);
      if (it.n_tiles == 0) {
        if (lane == 0) {
          mbar_arrive(&bars[bQEmpty]);
          mbar_arrive(&bars[bOFinal]);   // one phase per item, with or without tiles
        }
        ++it_count;
        continue;
      }
      {
        const uint32_t slot_k = base % kRing;   // K(0)
        if (!mbar_wait(&bars[bKVFull + slot_k], (base / kRing) & 1u)) { dead = true; break; }
        tcgen05_fence_after();
        issue_qk(0, slot_k);
        // Q is last read by the item's last S = Q K^T: releasing it there, not after the last P V, lets the
        // next item's Q load under this item's last tile and epilogue.
        if (it.n_tiles == 1) umma_commit_lead(lead, &bars[bQEmpty]);
      }
      for (int j = 0; j < it.n_tiles && !dead; ++j) {
        const uint32_t n_v = base + 2 * j + 1;   // V(j)
        if (j + 1 < it.n_tiles) {
          const uint32_t n_k = base + 2 * j + 2; // K(j+1)
          const uint32_t slot_k = n_k % kRing;
          if (!mbar_wait(&bars[bKVFull + slot_k], (n_k / kRing) & 1u)) { dead = true; break; }
          tcgen05_fence_after();
          if (lane == 0) TRACE1(8, tt);
          issue_qk((j + 1) & 1, slot_k);         // its S buffer held P(j-1), consumed by the earlier P V
          if (j + 2 == it.n_tiles) umma_commit_lead(lead, &bars[bQEmpty]);
        }
        if (lane == 0) TRACE1(15, tt);
        const uint32_t slot_v = n_v % kRing;
        if (!mbar_wait(&bars[bKVFull + slot_v], (n_v / kRing) & 1u)) { dead = true; break; }
        if (lane == 0) TRACE1(9, tt);
        const int tok0 = (it.tile_lo + j) * BN;
        if (tok0 + BN > it.kv_len) {
          // V rows past the end of the request may hold NaN: P is 0 there but 0 * NaN is NaN.
          const int first = max(0, it.kv_len - tok0);
          uint8_t* v_ptr = kv_smem + slot_v * C::kSlotBytes;
          constexpr int kChunks = C::kNKB * 8;   // 16-byte chunks per row
          for (int idx = lane; idx < (BN - first) * kChunks; idx += 32) {
            const int r = first + idx / kChunks, c = idx % kChunks;
            *reinterpret_cast<uint4*>(v_ptr + (c / 8) * C::kKVBlock + swz128(r, c % 8)) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async();
          __syncwarp();
        }
        const int buf = j & 1;
        if (!mbar_wait(&bars[bPFull + buf], cp[buf] & 1u)) { dead = true; break; }
        ++cp[buf];
        tcgen05_fence_after();
        if (lane == 0) TRACE1(10, tt);
        {
          const UmmaDesc vd = v_desc0 + (uint32_t)((slot_v * C::kSlotBytes) >> 4);
#pragma unroll
          for (int ks = 0; ks < C::kKStepsPV; ++ks) {
            const uint32_t voff = (ks * C::kPVStepBytes) >> 4;
            // P of key half h sits over the first columns of that half's own score columns
            constexpr int kPerHalf = C::kKStepsPV / 2;
            const uint32_t pcol = buf * BN + (ks / kPerHalf) * (BN / 2) + (ks % kPerHalf) * 8;
            if constexpr (kFp8)
              umma_ts_f8_lead(lead, tmem_base + o_col, tmem_base + pcol, vd + voff, kIdescPV, (j > 0) | (ks > 0));
            else
              umma_ts_f16_lead(lead, tmem_base + o_col, tmem_base + pcol, vd + voff, kIdescPV, (j > 0) | (ks > 0));
          }
          umma_commit_lead(lead, &bars[bOFull]);
          if (j + 1 == it.n_tiles) umma_commit_lead(lead, &bars[bOFinal]);   // one phase per item: O is final
          umma_commit_lead(lead, &bars[bKVEmpty + slot_v]);
          if (lane == 0) TRACE1(11, tt);
        }
        ++tt;
      }
      if (dead) break;
      base += 2u * (uint32_t)it.n_tiles;
      ++it_count;
    }
    if (dead && lane == 0) {
      if (p.status) atomicExch(p.status, kWaitMmaTimeout);
      atomicExch(abort_flag, 1);
    }
    __syncwarp();
  } else if (warp < kSoftmaxWarps1) {
    // ------------- softmax warps: two threads per row, half of each tile's key columns each -------------
    constexpr int N = BN / 2;                              // key columns per thread and tile
    const int h = warp >> 2;                               // which half of the key columns
    const int r = (warp & 3) * 32 + lane;                  // row = TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_off + o_col + h * (D / 2);   // this thread's half of the O columns
    float* xchg = reinterpret_cast<float*>(smem + C::kOffXchg);            // [parity][half][row]
    constexpr int kGroupBar = 1, kGroup = kSoftmaxWarps1 * 32;
    uint32_t cs[2] = {0, 0}, co = 0, it_count = 0, cx = 0;
    [[maybe_unused]] uint32_t tt = 0;   // tiles so far (trace index)
    bool dead = false;
    const ItemSlot* slots = reinterpret_cast<const ItemSlot*>(smem + C::kOffItem);
    for (; !dead; ++it_count) {
      if (tid == 0) TRACE1(20, it_count);
      // the item was resolved by warp 11 while the previous one was being worked on
      const ItemSlot* item_slot = slots + (it_count & 1u);
      const bool got = mbar_wait(&bars[bItemFull + (it_count & 1u)], (it_count >> 1) & 1u);
      // The slot stays this item's until the end of the epilogue, which reads the item again instead of keeping
      // its fields in registers across the tile loop.
      Item256 it;
      bool valid = false;
      float scale_log2 = 0.f;
      if (got) {
        it = item_slot->it;
        valid = item_slot->valid != 0;
        scale_log2 = item_slot->scale_log2;
      }
      if (tid == 0) TRACE1(22, it_count);
      // leave together: no more items, an abort seen by the steward, or a wait that expired in one thread
      if (group_barrier_or(kGroupBar, kGroup, !got || !valid || *(volatile int*)abort_flag != 0)) {
        if (!got) {
          if (p.status) atomicExch(p.status, kWaitFullTimeout);
          atomicExch(abort_flag, 1);
        }
        break;
      }
      if (tid == 0) TRACE1(12, it_count);
      const int qi = min((it.row0 + r) / p.group, max(it.q_len - 1, 0));
      const int vis_hi = p.window_right >= 0 ? min(it.kv_len, right_bound(p, qi + it.off)) : it.kv_len;
      const int vis_lo = p.window_left >= 0 ? max(0, qi + it.off - p.window_left) : 0;
      const int sqi_lo = it.row0 / p.group;
      const int sqi_hi = min(it.q_len - 1, (it.row0 + kRows - 1) / p.group);
      const int full_lo = p.window_left >= 0 ? max(0, sqi_hi + it.off - p.window_left) : 0;
      const int full_hi = p.window_right >= 0 ? min(it.kv_len, right_bound(p, sqi_lo + it.off)) : it.kv_len;
      float m_run = -INFINITY, l_run = 0.f;   // l_run: this thread's half of the row sum, in units of 2^kShift
      const int n_tiles = it.n_tiles, tile_lo = it.tile_lo;
      for (int j = 0; j < n_tiles; ++j) {
        if (tid == 0) TRACE1(17, tt);
        const int buf = j & 1;
        const uint32_t s_tmem = tmem_base + lane_off + buf * BN + h * N;   // own scores; P goes over them
        const int tok0 = (tile_lo + j) * BN;
        const bool need_mask = tok0 < full_lo || tok0 + BN > full_hi;
        if (tid == 0) TRACE1(16, tt);
        if (!mbar_wait(&bars[bSFull + buf], cs[buf] & 1u)) dead = true;
        if (tid == 0) TRACE1(18, tt);
        ++cs[buf];
        tcgen05_fence_after();
        if (tid == 0) TRACE1(0, tt);
        if (tid == 128) TRACE1(6, tt);
        uint32_t s[N];
        float mx = -INFINITY;
        if (!dead)
          mx = need_mask ? half_max<D, kFp8, true>(s_tmem, s, tok0 + h * N, vis_lo, vis_hi)
                         : half_max<D, kFp8, false>(s_tmem, s, tok0 + h * N, vis_lo, vis_hi);
        // row maximum = max of the two halves, exchanged through shared memory (double-buffered)
        if (tid == 0) TRACE1(1, tt);
        float* slot = xchg + (cx & 1u) * (2 * kRows);
        ++cx;
        slot[h * kRows + r] = mx;
        if (group_barrier_or(kGroupBar, kGroup, dead)) { dead = true; break; }
        if (tid == 0) TRACE1(2, tt);
        mx = fmaxf(mx, slot[(h ^ 1) * kRows + r]) * scale_log2;
        float alpha = 1.f;
        if (mx > m_run + C::kThreshold) {  // also the first finite maximum of the row
          alpha = fast_exp2(m_run - mx);
          m_run = mx;
        }
        const float neg_m = (m_run == -INFINITY ? 0.f : -m_run) + C::kShift;
        // masked scores are -inf and need ex2.approx's exact zero; elsewhere part of the work goes to the FMA pipe
        l_run = l_run * alpha + (need_mask ? half_exp<D, kFp8, 0>(s_tmem, s, scale_log2, neg_m)
                                           : half_exp<D, kFp8, kPolyOf8_1>(s_tmem, s, scale_log2, neg_m));
        if (tid == 0) TRACE1(3, tt);
        if (j > 0) {
          // O(j-1) must be complete before it is rescaled; the tensor pipe itself keeps P V(j) behind P V(j-1).
          // Without a rescale this phase of the O barrier is only counted (a satisfied wait and its fence cost
          // ~170 cycles per tile).  A later wait cannot mistake an older phase for its own: S(j), waited for above,
          // was committed after P V(j-2), so at most the phase being waited for is still open.  The end of the item
          // has no such guarantee (P V(n-2) may still be waiting for its V tile when the last softmax is done, in a
          // memory-bound decode), which is why it waits on a barrier of its own with one phase per item.
          const bool rescale = __any_sync(0xffffffffu, alpha != 1.f);
          if (rescale) {
            if (!mbar_wait(&bars[bOFull], co & 1u)) dead = true;   // reported at the next group barrier
            tcgen05_fence_after();
          }
          ++co;
          if (!dead && rescale) {
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
              uint32_t v[32];
              tmem_ld32(o_tmem + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st32(o_tmem + c * 32, v);
            }
          }
        }
        if (tid == 0) TRACE1(4, tt);
        tmem_st_wait();
        tcgen05_fence_before();
        mbar_arrive(&bars[bPFull + buf]);
        if (tid == 0) TRACE1(5, tt);
        if (tid == 128) TRACE1(7, tt);
        ++tt;
      }
      if (!dead) {
        if (!mbar_wait(&bars[bOFinal], it_count & 1u)) dead = true;   // one phase per item
        if (n_tiles > 0) ++co;
        tcgen05_fence_after();
      }
      if (tid == 0) TRACE1(21, it_count);
      // ---- epilogue: row sum = both halves; each thread normalises and stores its half of the O columns ----
      float* slot = xchg + (cx & 1u) * (2 * kRows);
      ++cx;
      slot[h * kRows + r] = l_run;
      if (group_barrier_or(kGroupBar, kGroup, dead)) {
        if (p.status) atomicExch(p.status, kWaitMmaTimeout);
        atomicExch(abort_flag, 1);
        dead = true;
        break;
      }
      const float l_row = l_run + slot[(h ^ 1) * kRows + r];
      const Item256 ie = item_slot->it;            // read again: see the top of the item loop
      const float dv = item_slot->dv;
      const int row = ie.row0 + r;
      const int hd = ie.kvh * p.group + row % p.group;
      const bool split_mode = ie.n_splits > 1;    // the combine kernel adds the sink and converts to BF16
      float sink_l2 = -INFINITY;
      if (p.sink != nullptr && !split_mode && row < ie.rows_total) sink_l2 = __bfloat162float(p.sink[hd]) * kLog2e;
      const float m_f = fmaxf(m_run, sink_l2);
      const float m_use = m_f == -INFINITY ? 0.f : m_f;
      const float resc = fast_exp2(m_run - m_use);
      float l = l_row * resc;                                        // in units of 2^kShift
      if (sink_l2 != -INFINITY) l += fast_exp2(sink_l2 - m_use + C::kShift);
      const float inv = (l > 0.f && ie.n_tiles > 0) ? dv * resc / l : 0.f;
      const int64_t q_row = ie.q_start + row / p.group;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + q_row * p.out_row_stride +
                           (int64_t)hd * p.out_head_stride + h * (D / 2);
      // Rows on 32-byte boundaries: one full sector per store (the epilogue is bound by the number of cache lines
      // its stores touch, since every lane writes another row).
      const bool out_vec32 = (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0 && (p.out_row_stride & 15) == 0 &&
                             (p.out_head_stride & 15) == 0;
      const int64_t part_slot = ((int64_t)ie.split * p.total_q + q_row) * p.num_q_heads + hd;
      float* part = split_mode ? p.part_o + part_slot * D + h * (D / 2) : nullptr;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t v[32];
        if (ie.n_tiles > 0) {
          tmem_ld32(o_tmem + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row < ie.rows_total && split_mode) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(part + c * 32 + i) =
                make_float4(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv,
                            __uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
        } else if (row < ie.rows_total) {
          store_bf16_row32(dst + c * 32, v, inv, out_vec32);
        }
      }
      if (h == 0 && row < ie.rows_total) {
        const float lse_l2 = l > 0.f ? m_use + log2f(l) - C::kShift : -INFINITY;
        if (split_mode) p.part_lse[part_slot] = lse_l2;
        else if (p.lse != nullptr) p.lse[(int64_t)hd * p.total_q + q_row] = lse_l2 * kLn2;
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bItemEmpty + (it_count & 1u)]);   // warp 11 may resolve item n + 2 into the slot
      if (tid == 0) TRACE1(13, it_count);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

}  // namespace

#ifdef ATREX_UMMA1_TRACE
extern "C" __attribute__((visibility("default"))) int atrex_fa_sm100_debug_trace1(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_umma1_trace, sizeof(long long) * n);
}
#endif

bool umma1_supports(int head_dim) { return head_dim == 128 || head_dim == 256; }
bool umma1_q_via_tma(int group) { return group >= 1 && group <= kRows && (kRows % group) == 0; }
int umma1_rows_per_item() { return kRows; }
int umma1_tile_n(int head_dim, bool fp8) {
  if (head_dim == 256) return fp8 ? Cfg1<256, true>::kBN : Cfg1<256, false>::kBN;
  return fp8 ? Cfg1<128, true>::kBN : Cfg1<128, false>::kBN;
}

#define ATREX_UMMA1_VARIANTS(X) X(128, false) X(128, true) X(256, false) X(256, true)

cudaError_t umma1_prepare() {
  cudaError_t e;
#define X(D, F)                                                                                               \
  if ((e = cudaFuncSetAttribute(atrex_sm100_fwd_umma1_kernel<D, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                Cfg1<D, F>::kSmemBytes)) != cudaSuccess)                                      \
    return e;
  ATREX_UMMA1_VARIANTS(X)
#undef X
  return cudaSuccess;
}

cudaError_t umma1_launch(const FwdParams& p, int head_dim, bool fp8, int sm_count, cudaStream_t stream) {
  long long items = (long long)p.num_row_tiles * p.num_kv_heads * p.num_splits;
  if (p.tail_splits > 1)
    items = (long long)p.num_kv_heads * (p.tail_first + (long long)(p.batch - p.tail_first) * p.tail_splits);
  const unsigned grid = (unsigned)(items < sm_count ? (items < 1 ? 1 : items) : sm_count);
#define X(D, F)                                                                                            \
  if (head_dim == D && fp8 == F)                                                                           \
    return launch_kernel(atrex_sm100_fwd_umma1_kernel<D, F>, dim3(grid), dim3(kThreads1), Cfg1<D, F>::kSmemBytes, \
                         stream, p);
  ATREX_UMMA1_VARIANTS(X)
#undef X
  return cudaErrorInvalidValue;
}

}  // namespace atrex_sm100
