// Warp-specialised prefill kernel on tcgen05 tensor cores (UMMA) with TMEM accumulators.
//
// Native counterpart of the reference's Blackwell prefill
// (src/nvidia/flash_attn/sm103/prefill_cutedsl.py:146-4331), designed for B200 and
// head_dim 128 (which the reference never runs on tcgen05):
//
//   * one CTA walks a static stripe of work items; an item is 256 packed GQA rows
//     (two 128-row Q subtiles) of one (request, KV head), heaviest requests first;
//   * warps 9 and 10 are the TMA producers, K (and the Q subtiles, once per item) and V: tiles of
//     128 tokens gathered page by page through the block table into a 4-slot ring of
//     128-byte-swizzled tiles (each CTA loads its own copy); the next tile's page ids are read
//     before the wait for the current slot, so the table lookup is off the issue path;
//   * warp 8 issues tcgen05.mma (the whole warp runs the issue code, lane 0's instruction is
//     predicated): S = Q K^T (both operands K-major in shared memory) into TMEM, then
//     O_tile = P V with P read straight from TMEM and V MN-major in shared memory, alternating
//     between the two subtiles so that one subtile's softmax overlaps the other's matrix work;
//   * warpgroups 0 and 1 (one thread per row) do the online softmax in the log2 domain and write
//     P as BF16 back into the S columns of TMEM, handing it to the issuer in two halves (after 64
//     and 128 keys) so that P V starts under the second half's exponentials; O accumulates in TMEM across
//     KV tiles and is rescaled in place only when a row maximum grows by more than 2^8 (the lazy
//     rescale of prefill_cutedsl.py:2589-2593), which after the first tiles is rare;
//   * TMEM: S0 | S1 | O0 | O1, 128 columns each (all 512).
//
// Every mbarrier wait is bounded; on expiry the CTA records a code, drains its
// copies, frees TMEM and returns.
#define ATREX_MBAR_SPIN_INLINE
#include "fa_kernels.cuh"
#include "softmax_math.cuh"
#include "umma.cuh"

namespace atrex_sm100 {

namespace {

constexpr int kBM = 128;                      // rows per Q subtile (UMMA M)
constexpr int kBN = 128;                      // KV tokens per tile (UMMA N of QK^T, K of PV)
constexpr int kHD = 128;                      // head dimension
constexpr int kTileBytes = kBN * kHD * 2;     // one K, V or Q tile: 32 KB
constexpr int kBlockBytes = kBN * 128;        // one 64-element column block of a tile: 16 KB
constexpr int kSlots = 4;                     // K/V ring: K(j), V(j), K(j+1), V(j+1)
constexpr int kUmmaThreads = 384;
constexpr int kRowsPerItem = 2 * kBM;
constexpr uint32_t kTmemCols = 512;

constexpr int kOffQ = 0;
constexpr int kOffKV = 2 * kTileBytes;
constexpr int kOffBar = kOffKV + kSlots * kTileBytes;
// barriers (8 bytes each)
enum Bar { kQFull = 0, kQEmpty = 1, kKVFull = 2, kKVEmpty = 6, kSFull = 10, kPFull = 12, kOFull = 14, kPLast = 16, kNumBars = 18 };
constexpr int kOffMisc = kOffBar + kNumBars * 8;   // tmem base (u32), abort flag (int)
constexpr int kUmmaSmemBytes = kOffMisc + 16;

#ifdef ATREX_UMMA_TRACE
__device__ long long g_umma_trace[8192];
#define TRACE(slot, idx) do { if (blockIdx.x == 0 && (idx) < 256) g_umma_trace[(slot) * 256 + (idx)] = clock64(); } while (0)
__device__ int g_trace_idx;
#else
#define g_trace_idx 0
#define TRACE(slot, idx) do { } while (0)
#endif

struct Item {
  int b, kvh, row0, q_start, q_len, rows_total, kv_len, k_start, off;
  int tile_lo, n_tiles;
};

// Work item `item` -> (KV head, row tile).  Items are KV-head-major: the CTAs in flight together take consecutive
// row tiles (heaviest request first, last row tile of a request first) of ONE KV head, so the K/V they stream is
// one head of one or two requests and stays in L2 however long the requests are.  (With the KV head as the
// fastest index the CTAs in flight covered every head of a request: 268 MB of K/V for two 32768-token requests
// with 8 KV heads, and the kernel then read 15x its algorithmic bytes from DRAM at an L2 hit rate of 76 %.)
// False when past the end.
__device__ __forceinline__ bool decode_item(const FwdParams& p, int item, Item& it) {
  const int total_tiles = p.tile_prefix[p.batch];
#ifdef ATREX_UMMA2_KVH_FASTEST
  const int tile_rank = item / p.num_kv_heads;
  if (tile_rank >= total_tiles) return false;
  it.kvh = item % p.num_kv_heads;
#else
  if (total_tiles <= 0) return false;
  it.kvh = item / total_tiles;
  if (it.kvh >= p.num_kv_heads) return false;
  const int tile_rank = item - it.kvh * total_tiles;
#endif
  int lo = 0, hi = p.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.tile_prefix[mid] <= tile_rank) lo = mid; else hi = mid;
  }
  it.b = p.order[lo];
  const int tiles_b = p.tile_prefix[lo + 1] - p.tile_prefix[lo];
  const int mt = tiles_b - 1 - (tile_rank - p.tile_prefix[lo]);  // last (heaviest causal) row tile first
  it.row0 = mt * kRowsPerItem;
  it.q_start = p.cu_seqlens_q[it.b];
  it.q_len = p.cu_seqlens_q[it.b + 1] - it.q_start;
  it.rows_total = it.q_len * p.group;
  request_kv(p, it.b, it.kv_len, it.k_start);
  it.off = request_off(p, it.b, it.kv_len, it.q_len);
  const int qi_lo = it.row0 / p.group;
  const int qi_hi = min(it.q_len - 1, (it.row0 + kRowsPerItem - 1) / p.group);
  int kv_end = it.kv_len, kv_begin = 0;
  if (p.window_right >= 0) kv_end = min(it.kv_len, right_bound(p, qi_hi + it.off));
  if (p.window_left >= 0) kv_begin = max(0, qi_lo + it.off - p.window_left);
  it.tile_lo = 0;
  it.n_tiles = 0;
  if (kv_end > kv_begin) {
    it.tile_lo = kv_begin / kBN;
    it.n_tiles = (kv_end + kBN - 1) / kBN - it.tile_lo;
  }
  return true;
}

#define UMMA_WAIT(bar_ptr, parity, code)                          \
  if (!mbar_wait((bar_ptr), (parity))) {                          \
    if (p.status) atomicExch(p.status, (code));                   \
    atomicExch(abort_flag, 1);                                    \
    break;                                                        \
  }

// K or V tiles of one work item, issued by one thread.  NB = TMA boxes per 128-token tile.  The page
// ids of tile j+1 are loaded before the wait for tile j's slot, so the table lookup is off the issue path.
// Copy issue is the serial part of the pipeline and this thread competes for issue slots with two
// softmax warps, so the loop is kept as short as it can be.  Returns false on a bounded-wait expiry.
template <int NB>
__device__ __forceinline__ bool produce_tiles(const FwdParams& p, const Item& it, int is_v, uint8_t* kv_smem,
                                              uint64_t* bars, uint32_t& seq, int pshift) {
  constexpr int kBoxRows = kBN / NB;
  constexpr uint32_t kBoxBytes = kBoxRows * 128u;
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
  int tok0 = it.tile_lo * kBN;
#pragma unroll
  for (int x = 0; x < NB; ++x) cur[x] = page_id(tok0 + x * kBoxRows);
  for (int j = 0; j < it.n_tiles; ++j, tok0 += kBN) {
    if (j + 1 < it.n_tiles) {
#pragma unroll
      for (int x = 0; x < NB; ++x) nxt[x] = page_id(tok0 + kBN + x * kBoxRows);
    }
    const uint32_t slot = seq % kSlots;
    if (seq >= (uint32_t)kSlots && !mbar_wait(&bars[kKVEmpty + slot], ((seq / kSlots) - 1) & 1u)) return false;
    uint8_t* dst = kv_smem + slot * kTileBytes;
    int live = 0;
#pragma unroll
    for (int x = 0; x < NB; ++x) live += (cur[x] >= 0 && tok0 + x * kBoxRows < it.kv_len) ? 1 : 0;
    mbar_arrive_expect_tx(&bars[kKVFull + slot], (uint32_t)live * kBoxBytes * 2u);
#pragma unroll
    for (int x = 0; x < NB; ++x) {
      const int tok = tok0 + x * kBoxRows;
      if (cur[x] < 0 || tok >= it.kv_len) continue;
      const int row = p.page_size ? (pshift >= 0 ? tok & row_mask : tok % p.page_size) : it.k_start + tok;
      tma_load_kv(dst + x * kBoxBytes, map, &bars[kKVFull + slot], 0, it.kvh, row, cur[x], perm);
      tma_load_kv(dst + kBlockBytes + x * kBoxBytes, map, &bars[kKVFull + slot], 64, it.kvh, row, cur[x], perm);
    }
#pragma unroll
    for (int x = 0; x < NB; ++x) cur[x] = nxt[x];
    seq += 2;
  }
  return true;
}

// Growth of the running row maximum (log2 units) below which the old maximum is kept: P then
// reaches at most 2^8, harmless in BF16 / FP32, and the TMEM-resident O needs no rescale.
constexpr float kRescaleThreshold = 8.f;

// Pairs of every 8 whose exponential is a polynomial on the FMA pipe (the rest use the MUFU pipe).
#ifndef ATREX_UMMA2_POLY_OF8
#define ATREX_UMMA2_POLY_OF8 0
#endif
constexpr int kPolyOf8 = ATREX_UMMA2_POLY_OF8;
constexpr int kPFirstChunks = 2;   // 32-key chunks of P in the first hand-over (of 4): the first 64 keys


// First step of a 128-key tile for one row (= one thread): the scores come from TMEM into registers,
// masked columns become -inf, and the running maximum follows the lazy-rescale rule.  Returns the
// factor the caller must apply to the O and the row sum accumulated so far (1 when the max was kept).
template <bool kMask>
__device__ __forceinline__ float tile_max(uint32_t s_tmem, uint32_t (&s)[kBN], float scale_log2, int tok0, int vis_lo,
                                          int vis_hi, float& m_run) {
  // The second half of the row loads while the first half is reduced.  Eight independent chains: with one
  // softmax warp per scheduler active at a time there is no thread-level parallelism to hide the latency of
  // a long dependency chain.
  float mxv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mxv[i] = -INFINITY;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (half == 0) {
#pragma unroll
      for (int c = 0; c < kBN / 64; ++c) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
    }
    tmem_ld_wait();
    if (half == 0) {
#pragma unroll
      for (int c = kBN / 64; c < kBN / 32; ++c)
        tmem_ld32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[c * 32]));
    }
    if (kMask) {
#pragma unroll
      for (int i = half * (kBN / 2); i < (half + 1) * (kBN / 2); ++i) {
        const int col = tok0 + i;
        if (col < vis_lo || col >= vis_hi) s[i] = 0xff800000u;  // -inf
      }
    }
#pragma unroll
    for (int i = half * (kBN / 2); i < (half + 1) * (kBN / 2); i += 16) {   // 3-input max: half the instructions
#pragma unroll
      for (int u = 0; u < 8; ++u)
        mxv[u] = fmax3(mxv[u], __uint_as_float(s[i + 2 * u]), __uint_as_float(s[i + 2 * u + 1]));
    }
  }
  if (threadIdx.x == 0) TRACE(24, g_trace_idx);
  mxv[0] = fmaxf(mxv[0], mxv[4]); mxv[1] = fmaxf(mxv[1], mxv[5]);
  mxv[2] = fmaxf(mxv[2], mxv[6]); mxv[3] = fmaxf(mxv[3], mxv[7]);
  float mx = fmaxf(fmaxf(mxv[0], mxv[1]), fmaxf(mxv[2], mxv[3]));
  mx *= scale_log2;
  float alpha = 1.f;
  if (mx > m_run + kRescaleThreshold) {  // also the first finite maximum of the row
    alpha = fast_exp2(m_run - mx);
    m_run = mx;
  }
  if (threadIdx.x == 0) TRACE(25, g_trace_idx);
  return alpha;
}

// Second step, for 64-key half `half` of the tile: P = 2^(s*scale - m) written over the S columns as BF16 pairs
// (64 keys = 32 packed registers = one TMEM store); the probabilities add into sum2.  64-key stores measured 1.5 %
// faster than 32-key ones on the 16-request prefill workload (1 055 - 1 057 against 1 039 - 1 042 TFLOP/s).
template <bool kMask>
__device__ __forceinline__ void tile_exp(uint32_t s_tmem, const uint32_t (&s)[kBN], int half, f32x2 scale2,
                                         f32x2 negm2, f32x2 (&sum2)[2]) {
  uint32_t packed[32];
  // masked scores are -inf and need ex2.approx's exact zero; elsewhere part of the work may go to the FMA pipe
  exp32_bf16<kMask ? 0 : kPolyOf8>(&s[half * 64], scale2, negm2, sum2, *reinterpret_cast<uint32_t(*)[16]>(&packed[0]));
  exp32_bf16<kMask ? 0 : kPolyOf8>(&s[half * 64 + 32], scale2, negm2, sum2,
                                   *reinterpret_cast<uint32_t(*)[16]>(&packed[16]));
  tmem_st32(s_tmem + half * 32, packed);
  if (threadIdx.x == 0) TRACE(26 + 2 * half, g_trace_idx);
}

}  // namespace

namespace {

__global__ void __launch_bounds__(kUmmaThreads, 1)
atrex_sm100_fwd_umma_kernel(const __grid_constant__ FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_smem = smem + kOffQ;
  uint8_t* kv_smem = smem + kOffKV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc);
  int* abort_flag = reinterpret_cast<int*>(smem + kOffMisc + 4);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0 && p.status) atomicExch(p.status, kBadSmemAlignment);
    return;
  }
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(&bars[kQFull], 1);
    mbar_init(&bars[kQEmpty], 1);
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&bars[kKVFull + s], 1);
      mbar_init(&bars[kKVEmpty + s], 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&bars[kSFull + w], 1);
      mbar_init(&bars[kPFull + w], kBM);
      mbar_init(&bars[kPLast + w], kBM);
      mbar_init(&bars[kOFull + w], 1);
    }
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_items_step = gridDim.x;

  if (warp >= 8) {
    // ============================ warpgroup 2: MMA issuer, TMA producer ============================
    setmaxnreg_dec<96>();
    if (warp == 9 || warp == 10) {
      // ------------------------------- TMA producers -------------------------------
      // Warp 9 loads Q and the K tiles (ring slots 0 and 2), warp 10 the V tiles (slots 1 and 3); one
      // thread of each issues everything.
      if (lane == 0) {
        const int is_v = warp == 10;
        if (!is_v) prefetch_tensormap(&p.q_map);
        prefetch_tensormap(is_v ? &p.v_map : &p.k_map);
        const int boxes = kBN / p.box_rows;
        const int pshift = (p.page_size > 0 && (p.page_size & (p.page_size - 1)) == 0) ? __ffs(p.page_size) - 1 : -1;
        uint32_t it_count = 0, seq = (uint32_t)is_v;
        bool q_issued = false;
        for (int item = blockIdx.x;; item += n_items_step) {
          Item it;
          if (!decode_item(p, item, it)) break;
          if (*(volatile int*)abort_flag) break;
          if (!is_v) {
            if (it_count > 0) UMMA_WAIT(&bars[kQEmpty], (it_count - 1) & 1u, kWaitEmptyTimeout)
            mbar_arrive_expect_tx(&bars[kQFull], 2u * kTileBytes);
            q_issued = true;
#pragma unroll
            for (int w = 0; w < 2; ++w)
#pragma unroll
              for (int kb = 0; kb < 2; ++kb)
                tma_load_3d(q_smem + w * kTileBytes + kb * kBlockBytes, &p.q_map, &bars[kQFull], kb * 64,
                            it.kvh * p.group, it.q_start + (it.row0 + w * kBM) / p.group);
          }
          bool ok;
          switch (boxes) {
            case 1: ok = produce_tiles<1>(p, it, is_v, kv_smem, bars, seq, pshift); break;
            case 2: ok = produce_tiles<2>(p, it, is_v, kv_smem, bars, seq, pshift); break;
            case 4: ok = produce_tiles<4>(p, it, is_v, kv_smem, bars, seq, pshift); break;
            default: ok = produce_tiles<8>(p, it, is_v, kv_smem, bars, seq, pshift); break;
          }
          if (!ok) {
            if (p.status) atomicExch(p.status, kWaitEmptyTimeout);
            atomicExch(abort_flag, 1);
            break;
          }
          ++it_count;
        }
        // Drain: every copy this thread issued must have landed before the CTA may exit.
        if (q_issued) mbar_wait(&bars[kQFull], (it_count > 0 ? it_count - 1 : 0) & 1u);
        for (uint32_t back = 2; back <= (uint32_t)kSlots && back <= seq; back += 2) {
          const uint32_t n = seq - back;   // this thread's last two tiles
          mbar_wait(&bars[kKVFull + n % kSlots], (n / kSlots) & 1u);
        }
      }
      __syncwarp();
    } else if (warp == 8) {
      // ------------------------------- MMA issuer -------------------------------
      constexpr uint32_t kIdescQK = umma_idesc(kBM, kBN, 1, 1, 0, 0);
      constexpr uint32_t kIdescPV = umma_idesc(kBM, kHD, 1, 1, 0, 1);
      const uint32_t q_addr = smem_u32(q_smem);
      const uint32_t kv_addr = smem_u32(kv_smem);
      uint32_t it_count = 0, seq = 0, cp[2] = {0, 0};
      bool dead = false;
      // Descriptors are built once; per instruction only the start-address field (bytes >> 4) moves.
      const UmmaDesc q_desc0 = umma_desc_split(umma_desc_sw128(q_addr, 16, 1024));
      const UmmaDesc k_desc0 = umma_desc_split(umma_desc_sw128(kv_addr, 16, 1024));
      const UmmaDesc v_desc0 = umma_desc_split(umma_desc_sw128(kv_addr, kBlockBytes, 1024));
      // The whole warp runs the issue code and lane 0 issues: all operands are warp-uniform.
      const uint32_t lead = lane == 0;
      auto issue_qk = [&](int w, uint32_t slot) {
        const UmmaDesc qd = q_desc0 + (uint32_t)((w * kTileBytes) >> 4);
        const UmmaDesc kd = k_desc0 + (uint32_t)((slot * kTileBytes) >> 4);
#pragma unroll
        for (int ks = 0; ks < kHD / 16; ++ks) {
          const uint32_t koff = ((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4;
          umma_ss_f16_lead(lead, tmem_base + w * kBN, qd + koff, kd + koff, kIdescQK, ks > 0);
        }
        umma_commit_lead(lead, &bars[kSFull + w]);
      };
      for (int item = blockIdx.x; !dead; item += n_items_step) {
        Item it;
        if (!decode_item(p, item, it)) break;
        if (*(volatile int*)abort_flag) break;
        if (it.n_tiles > 0) {
          do {  // single pass; UMMA_WAIT leaves it on a timeout
            UMMA_WAIT(&bars[kQFull], it_count & 1u, kWaitFullTimeout)
            uint32_t slot_k = seq % kSlots;
            UMMA_WAIT(&bars[kKVFull + slot_k], (seq / kSlots) & 1u, kWaitFullTimeout)
            ++seq;
            tcgen05_fence_after();
            issue_qk(0, slot_k);
            issue_qk(1, slot_k);
            umma_commit_lead(lead, &bars[kKVEmpty + slot_k]);
            // Q is last read by the item's last S = Q K^T: releasing it there, not after the last P V, lets the
            // next item's Q tiles load under this item's last tile and epilogue.
            if (it.n_tiles == 1) umma_commit_lead(lead, &bars[kQEmpty]);
            for (int j = 0; j < it.n_tiles && !dead; ++j) {
              const bool more = j + 1 < it.n_tiles;
              const uint32_t slot_v = seq % kSlots;
              if (lane == 0) TRACE(12, cp[0]);
              if (!mbar_wait(&bars[kKVFull + slot_v], (seq / kSlots) & 1u)) { dead = true; break; }
              ++seq;
              if (lane == 0) TRACE(13, cp[0]);
              // V rows past the end of the request may hold NaN: P is 0 there but 0 * NaN is NaN.
              const int tok0 = (it.tile_lo + j) * kBN;
              if (tok0 + kBN > it.kv_len) {
                const int first = max(0, it.kv_len - tok0);
                uint8_t* v_ptr = kv_smem + slot_v * kTileBytes;
                for (int idx = lane; idx < (kBN - first) * 16; idx += 32) {
                  const int r = first + idx / 16, c = idx % 16;
                  *reinterpret_cast<uint4*>(v_ptr + (c / 8) * kBlockBytes + swz128(r, c % 8)) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
                __syncwarp();
              }
              uint32_t slot_k2 = 0;
              if (more) {
                slot_k2 = seq % kSlots;
                if (!mbar_wait(&bars[kKVFull + slot_k2], (seq / kSlots) & 1u)) { dead = true; break; }
                ++seq;
                if (lane == 0) TRACE(14, cp[0]);
              }
              for (int w = 0; w < 2; ++w) {
                if (!mbar_wait(&bars[kPFull + w], cp[w] & 1u)) { dead = true; break; }
                if (lane == 0) TRACE(8 + 2 * w, cp[w]);
                ++cp[w];
                tcgen05_fence_after();
                {
                  const UmmaDesc vd = v_desc0 + (uint32_t)((slot_v * kTileBytes) >> 4);
#pragma unroll
                  for (int ks = 0; ks < kPFirstChunks * 2; ++ks)
                    umma_ts_f16_lead(lead, tmem_base + 2 * kBN + w * kHD, tmem_base + w * kBN + ks * 8,
                                     vd + (uint32_t)((ks * 2048) >> 4), kIdescPV, (j > 0) | (ks > 0));
                  if (!mbar_wait(&bars[kPLast + w], (cp[w] - 1) & 1u)) { dead = true; break; }
                  tcgen05_fence_after();
#pragma unroll
                  for (int ks = kPFirstChunks * 2; ks < kBN / 16; ++ks)
                    umma_ts_f16_lead(lead, tmem_base + 2 * kBN + w * kHD, tmem_base + w * kBN + ks * 8,
                                     vd + (uint32_t)((ks * 2048) >> 4), kIdescPV, 1u);
                  umma_commit_lead(lead, &bars[kOFull + w]);
                }
                if (more) issue_qk(w, slot_k2);
                if (lane == 0) TRACE(9 + 2 * w, cp[w] - 1);
              }
              if (dead) break;
              umma_commit_lead(lead, &bars[kKVEmpty + slot_v]);
              if (more) umma_commit_lead(lead, &bars[kKVEmpty + slot_k2]);
              if (j + 2 == it.n_tiles) umma_commit_lead(lead, &bars[kQEmpty]);
              if (lane == 0) TRACE(18, cp[0] - 1);
            }
          } while (false);
          if (dead || *(volatile int*)abort_flag) {
            if (dead && lane == 0) {
              if (p.status) atomicExch(p.status, kWaitMmaTimeout);
              atomicExch(abort_flag, 1);
            }
            break;
          }
        } else {
          // No key is visible: nothing to multiply, but the Q tiles were loaded and must be released.
          bool ok = mbar_wait(&bars[kQFull], it_count & 1u);
          if (!ok) { if (lane == 0) { if (p.status) atomicExch(p.status, kWaitFullTimeout); atomicExch(abort_flag, 1); } break; }
          if (lane == 0) mbar_arrive(&bars[kQEmpty]);
        }
        ++it_count;
      }
      __syncwarp();
    }
  } else {
    // ============================ warpgroups 0 and 1: softmax, O kept in TMEM ============================
    setmaxnreg_inc<200>();
    const int w = warp >> 2;                                   // subtile
    const int r = (warp & 3) * 32 + lane;                      // row inside the subtile = TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_off + w * kBN;
    const uint32_t o_tmem = tmem_base + lane_off + 2 * kBN + w * kHD;
    uint32_t cs = 0, co = 0;
    [[maybe_unused]] uint32_t itc = 0;   // items so far (trace index)
    bool dead = false;
    for (int item = blockIdx.x; !dead; item += n_items_step) {
      Item it;
      if (tid == 0) TRACE(30, itc);
      if (!decode_item(p, item, it)) break;
      if (tid == 0) TRACE(31, itc);
      if (*(volatile int*)abort_flag) break;
      const int sub_row0 = it.row0 + w * kBM;
      const int row = sub_row0 + r;
      const int qi = min(row / p.group, max(it.q_len - 1, 0));
      const int hd = it.kvh * p.group + row % p.group;
      const int vis_hi = p.window_right >= 0 ? min(it.kv_len, right_bound(p, qi + it.off)) : it.kv_len;
      const int vis_lo = p.window_left >= 0 ? max(0, qi + it.off - p.window_left) : 0;
      const int sqi_lo = sub_row0 / p.group;
      const int sqi_hi = min(it.q_len - 1, (sub_row0 + kBM - 1) / p.group);
      const int full_lo = p.window_left >= 0 ? max(0, sqi_hi + it.off - p.window_left) : 0;
      const int full_hi = p.window_right >= 0 ? min(it.kv_len, right_bound(p, sqi_lo + it.off)) : it.kv_len;
      float dq = 1.f, dk = 1.f, dv = 1.f;
      if (p.q_descale) dq = p.q_descale[it.b * p.q_descale_bs + it.kvh * p.q_descale_hs];
      if (p.k_descale) dk = p.k_descale[it.b * p.k_descale_bs + it.kvh * p.k_descale_hs];
      if (p.v_descale) dv = p.v_descale[it.b * p.v_descale_bs + it.kvh * p.v_descale_hs];
      const float scale_log2 = p.softmax_scale * dq * dk * kLog2e;   // > 0 on this route

      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < it.n_tiles; ++j) {
        const int tok0 = (it.tile_lo + j) * kBN;
        const bool need_mask = tok0 < full_lo || tok0 + kBN > full_hi;
        if (!mbar_wait(&bars[kSFull + w], cs & 1u)) { dead = true; break; }
        ++cs;
        tcgen05_fence_after();
#ifdef ATREX_UMMA_TRACE
        if (tid == 0 && blockIdx.x == 0) g_trace_idx = cs - 1;
#endif
        if (tid == 0) TRACE(0, cs - 1);
        if (tid == 128) TRACE(4, cs - 1);
        uint32_t s[kBN];
        const float alpha = need_mask ? tile_max<true>(s_tmem, s, scale_log2, tok0, vis_lo, vis_hi, m_run)
                                      : tile_max<false>(s_tmem, s, scale_log2, tok0, vis_lo, vis_hi, m_run);
        if (j > 0) {
          // O(j-1) must be complete before it is rescaled, and rescaled before the first part of P V(j) adds to it.
          // It is: the issuer issues Q K^T(j) of this subtile after its P V(j-1), and the commit behind S(j), waited
          // for above, covers every earlier MMA.  So this phase of the O barrier is only counted, not waited for
          // (a satisfied wait and its fence cost ~170 cycles per tile).
          ++co;
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            // narrow chunks: the tile's 128 scores stay in registers across this rare step
#pragma unroll
            for (int c = 0; c < kHD / 16; ++c) {
              uint32_t v[16];
              tmem_ld16(o_tmem + c * 16, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st16(o_tmem + c * 16, v);
            }
          }
        }
        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
        const f32x2 scale2 = pack2(scale_log2, scale_log2), negm2 = pack2(neg_m, neg_m);
        f32x2 sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
        // P is handed over in two halves of 64 keys (one 32-register TMEM store each), so that the tensor core
        // multiplies the first half by V while the second half's exponentials are still being computed.
        if (need_mask) tile_exp<true>(s_tmem, s, 0, scale2, negm2, sum2);
        else tile_exp<false>(s_tmem, s, 0, scale2, negm2, sum2);
        tmem_st_wait();
        tcgen05_fence_before();
        mbar_arrive(&bars[kPFull + w]);
        if (tid == 0) TRACE(1, cs - 1);
        if (need_mask) tile_exp<true>(s_tmem, s, 1, scale2, negm2, sum2);
        else tile_exp<false>(s_tmem, s, 1, scale2, negm2, sum2);
        l_run = l_run * alpha + sum_of(sum2);
        tmem_st_wait();
        if (tid == 0) TRACE(2, cs - 1);
        tcgen05_fence_before();
        mbar_arrive(&bars[kPLast + w]);
        if (tid == 0) TRACE(3, cs - 1);
        if (tid == 128) TRACE(7, cs - 1);
      }
      if (!dead && it.n_tiles > 0) {
        if (!mbar_wait(&bars[kOFull + w], co & 1u)) dead = true;
        ++co;
        tcgen05_fence_after();
      }
      if (dead) {
        if (p.status) atomicExch(p.status, kWaitMmaTimeout);
        atomicExch(abort_flag, 1);
        break;
      }
      // ---- epilogue: O from TMEM, normalise, store BF16 row and natural-log LSE ----
      if (tid == 0) TRACE(27, itc);
      float sink_l2 = -INFINITY;
      if (p.sink != nullptr && row < it.rows_total) sink_l2 = __bfloat162float(p.sink[hd]) * kLog2e;
      const float m_f = fmaxf(m_run, sink_l2);
      const float m_use = m_f == -INFINITY ? 0.f : m_f;
      const float resc = fast_exp2(m_run - m_use);
      float l = l_run * resc;
      if (sink_l2 != -INFINITY) l += fast_exp2(sink_l2 - m_use);
      const float inv = (l > 0.f && it.n_tiles > 0) ? dv * resc / l : 0.f;
      const int64_t q_row = it.q_start + row / p.group;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + q_row * p.out_row_stride +
                           (int64_t)hd * p.out_head_stride;
      // Rows on 32-byte boundaries: one full sector per store (the epilogue is bound by the number of cache lines
      // its stores touch, since every lane writes another row).
      const bool out_vec32 = (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0 && (p.out_row_stride & 15) == 0 &&
                             (p.out_head_stride & 15) == 0;
#pragma unroll
      for (int c = 0; c < kHD / 32; ++c) {
        uint32_t v[32];
        if (it.n_tiles > 0) {           // warp-uniform
          tmem_ld32(o_tmem + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row < it.rows_total) store_bf16_row32(dst + c * 32, v, inv, out_vec32);
      }
      if (row < it.rows_total && p.lse != nullptr)
        p.lse[(int64_t)hd * p.total_q + q_row] = l > 0.f ? (m_use + log2f(l)) * kLn2 : -INFINITY;
      // the next item's first P V overwrites O only after this warp's next P arrival, i.e. after these loads
      tcgen05_fence_before();
      if (tid == 0) TRACE(29, itc);
      ++itc;
    }
  }

  // All roles meet here (every wait above is bounded), then the allocating warp frees TMEM.
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 8) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool umma_supports(int head_dim, int group, int dtype_is_bf16) {
  return head_dim == kHD && dtype_is_bf16 && group >= 1 && group <= kBM && (kBM % group) == 0;
}

int umma_rows_per_item() { return kRowsPerItem; }

#ifdef ATREX_UMMA_TRACE
extern "C" __attribute__((visibility("default"))) int atrex_fa_sm100_debug_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_umma_trace, sizeof(long long) * n);
}
#endif

cudaError_t umma_prepare() {
  return cudaFuncSetAttribute(atrex_sm100_fwd_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kUmmaSmemBytes);
}

cudaError_t umma_launch(const FwdParams& p, int sm_count, cudaStream_t stream) {
  const long long items = (long long)p.num_row_tiles * p.num_kv_heads;
  const unsigned grid = (unsigned)(items < sm_count ? (items < 1 ? 1 : items) : sm_count);
  return launch_kernel(atrex_sm100_fwd_umma_kernel, dim3(grid), dim3(kUmmaThreads), kUmmaSmemBytes, stream, p);
}

}  // namespace atrex_sm100
