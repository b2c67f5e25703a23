// Split-KV attention kernel on mma.sync tensor cores with a TMA producer warp.
//
// Serves the HBM-bound short-query calls (decode and speculative verify, where
// the packed "query x GQA group" rows of one KV head fit one small row tile)
// and is the compatibility route for every BF16 call the tcgen05 prefill kernel
// does not take.  It is the native counterpart of the reference's paged decode
// (src/nvidia/flash_attn/sm103/decode_cutedsl.py:453-2873) and of its sm120
// split-KV kernel family (src/nvidia/flash_attn/sm120/attention_cutedsl.py:1210-1825),
// designed for B200 rather than translated:
//
//   * one CTA = one (request, row tile, KV head, KV split); rows are packed
//     GQA rows: row r <-> query r / group, head kv_head*group + r % group
//     (same order as decode_cutedsl.py:97-110);
//   * a producer warp walks the block table and issues one TMA box per page
//     slice into a ring of 128-byte-swizzled K/V stages (each CTA loads its own copy);
//   * WT warp groups of WM warps each take alternate KV tiles with private
//     online-softmax state (log2 domain) and merge once at the end, so there is
//     no per-tile block barrier;
//   * the result leaves through shared memory as coalesced stores: BF16 O and
//     natural-log LSE, or normalised FP32 partials + log2 LSE for the combine.
#include "fa_kernels.cuh"
#include "ptx.cuh"

namespace atrex_sm100 {

namespace {

// A consumer waits on a stage's "full" barrier by phase parity, which is only
// sound while it is at most one phase behind that barrier.  Every warp group
// therefore owns fixed stages (STAGES % WT == 0) and sees each of their phases
// in order.
template <int D, int WM, int WT, int STAGES, int TN>
struct MmaCfg {
  static_assert(STAGES % WT == 0, "each stage must have one fixed consumer group");
  static constexpr int kTileN = TN;                  // KV tokens per pipeline stage
  static constexpr int kM = 16 * WM;                 // packed rows per CTA
  static constexpr int kComputeWarps = WM * WT;
  static constexpr int kThreads = (kComputeWarps + 1) * 32;
  static constexpr int kKBlocks = D / 64;            // 128-byte swizzle blocks along D
  static constexpr int kOperandBytes = kTileN * D * 2;
  static constexpr int kStageBytes = 2 * kOperandBytes;
  static constexpr int kQBytes = kM * D * 2;
  static constexpr int kRedBytes = WT * kM * (D + 2) * 4;
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static_assert(kRedBytes <= kRingBytes, "merge buffer aliases the ring");
  static constexpr int kSmemBytes = kRingBytes + kQBytes + 2 * STAGES * 8 + 16;
  // CTAs per SM the shared memory allows (228 KB per SM, 1 KB reserved per CTA), at most 3
  static constexpr int kBySmem = (228 * 1024) / (kSmemBytes + 1024);
  static constexpr int kByRegs = D == 256 ? (kThreads <= 96 ? 2 : 1) : (kThreads <= 96 ? 3 : 2);
  static constexpr int kMinBlocks = kBySmem < 1 ? 1 : (kBySmem < kByRegs ? kBySmem : kByRegs);
};

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int D, int WM, int WT, int STAGES, int TN>
__global__ void __launch_bounds__((WM * WT + 1) * 32, MmaCfg<D, WM, WT, STAGES, TN>::kMinBlocks)
atrex_sm100_fwd_mma_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = MmaCfg<D, WM, WT, STAGES, TN>;
  constexpr int M = Cfg::kM;
  constexpr int KB = Cfg::kKBlocks;
  constexpr int kTileN = TN;

  // No static shared memory is declared, so the dynamic window starts at the
  // CTA's shared base; the swizzled tiles need 1024-byte alignment (checked below).
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* ring = smem;
  uint8_t* q_smem = smem + Cfg::kRingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(q_smem + Cfg::kQBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  int& s_abort = *reinterpret_cast<int*>(empty_bar + STAGES);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---- which work item ----
  const int kvh = blockIdx.x % p.num_kv_heads;
  const int item = blockIdx.x / p.num_kv_heads;
  const int split = blockIdx.y;
  int b, mt;
  if (p.order == nullptr) {
    b = item;
    mt = 0;
  } else {
    const int total_tiles = p.tile_prefix[p.batch];
    if (item >= total_tiles) return;
    int lo = 0, hi = p.batch;  // largest i with tile_prefix[i] <= item
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.tile_prefix[mid] <= item) lo = mid; else hi = mid;
    }
    b = p.order[lo];
    const int n_tiles = p.tile_prefix[lo + 1] - p.tile_prefix[lo];
    mt = n_tiles - 1 - (item - p.tile_prefix[lo]);  // heaviest (last) row tile of a causal request first
  }
  const int q_start = p.cu_seqlens_q[b];
  const int q_len = p.cu_seqlens_q[b + 1] - q_start;
  const int rows_total = q_len * p.group;
  const int row0 = mt * M;
  if (row0 >= rows_total) return;  // also covers q_len == 0
  int kv_len, k_start;
  request_kv(p, b, kv_len, k_start);

  // ---- key range this row tile can see, then this split's share of its tiles ----
  const int off = request_off(p, b, kv_len, q_len);
  const int qi_lo = row0 / p.group;
  const int qi_hi = min(q_len - 1, (row0 + M - 1) / p.group);
  int kv_end = kv_len, kv_begin = 0;
  if (p.window_right >= 0) kv_end = min(kv_len, right_bound(p, qi_hi + off));
  if (p.window_left >= 0) kv_begin = max(0, qi_lo + off - p.window_left);
  int tile_lo = 0, tile_hi = 0;
  if (kv_end > kv_begin) {
    const int t0 = kv_begin / kTileN, t1 = (kv_end + kTileN - 1) / kTileN;
    const int n = t1 - t0;
    tile_lo = t0 + (int)(((long long)n * split) / p.num_splits);
    tile_hi = t0 + (int)(((long long)n * (split + 1)) / p.num_splits);
  }
  const int n_tiles = tile_hi - tile_lo;

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (tid == 0 && p.status) atomicExch(p.status, kBadSmemAlignment);
    return;
  }
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WM);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const bool is_producer = warp == Cfg::kComputeWarps;
  const int wm = warp % WM;  // row slice inside the tile
  const int wt = warp / WM;  // which alternate KV tiles

  // softmax state of this thread's two rows (g and g+8 of the warp's 16)
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  if (is_producer) {
    // ===================== producer warp =====================
    if (lane == 0 && n_tiles > 0) {
      prefetch_tensormap(&p.k_map);
      prefetch_tensormap(&p.v_map);
      const int32_t* table = p.page_size ? p.block_table + (int64_t)b * p.block_table_row_stride : nullptr;
      const int boxes = kTileN / p.box_rows;
      const uint32_t box_bytes = (uint32_t)p.box_rows * 128u;
      for (int i = 0; i < n_tiles; ++i) {
        const int stage = i % STAGES;
        const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
        if (i >= STAGES && !mbar_wait(&empty_bar[stage], phase ^ 1u)) {
          if (p.status) atomicExch(p.status, kWaitEmptyTimeout);
          atomicExch(&s_abort, 1);
          break;
        }
        if (*(volatile int*)&s_abort) break;
        const int tok0 = (tile_lo + i) * kTileN;
        uint8_t* k_dst = ring + stage * Cfg::kStageBytes;
        uint8_t* v_dst = k_dst + Cfg::kOperandBytes;
        // decide the boxes first so the expected byte count is known before any copy lands
        int page_of[4], row_of[4];
        int live = 0;
        for (int x = 0; x < boxes; ++x) {
          const int tok = tok0 + x * p.box_rows;
          page_of[x] = -1;
          if (tok >= kv_len) continue;
          if (p.page_size) {
            const int pg = table[tok / p.page_size];
            if (pg < 0 || pg >= p.num_pages) continue;
            page_of[x] = pg;
            row_of[x] = tok % p.page_size;
          } else {
            page_of[x] = 0;
            row_of[x] = k_start + tok;
          }
          ++live;
        }
        mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)live * box_bytes * 2u * KB);
        for (int x = 0; x < boxes; ++x) {
          if (page_of[x] < 0) continue;
#pragma unroll
          for (int kb = 0; kb < KB; ++kb) {
            const uint32_t dst_off = kb * (kTileN * 128) + x * box_bytes;
            tma_load_kv(k_dst + dst_off, &p.k_map, &full_bar[stage], kb * 64, kvh, row_of[x], page_of[x], p.k_perm);
            tma_load_kv(v_dst + dst_off, &p.v_map, &full_bar[stage], kb * 64, kvh, row_of[x], page_of[x], p.v_perm);
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ===================== compute warps =====================
    // Q tile -> shared memory (swizzled like K so ldmatrix is conflict free).
    {
      const uint8_t* q_base = reinterpret_cast<const uint8_t*>(p.q);
      constexpr int kChunks = D / 8;  // 16-byte chunks per row
      for (int idx = tid; idx < M * kChunks; idx += Cfg::kComputeWarps * 32) {
        const int r = idx / kChunks, c = idx % kChunks;
        const int row = row0 + r;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < rows_total) {
          const int qi = row / p.group, hd = kvh * p.group + row % p.group;
          const int64_t e = (int64_t)(q_start + qi) * p.q_row_stride + (int64_t)hd * p.q_head_stride + c * 8;
          val = __ldg(reinterpret_cast<const uint4*>(q_base + e * 2));
        }
        const int kb = c / 8;
        *reinterpret_cast<uint4*>(q_smem + kb * (M * 128) + swz128(r, c % 8)) = val;
      }
      named_barrier(1, Cfg::kComputeWarps * 32);
    }

    const int g = lane >> 2, t = lane & 3;
    // per-row visibility bounds [lo, hi) in key index
    int vis_lo[2], vis_hi[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row0 + wm * 16 + g + h * 8;
      const int qi = min(row / p.group, q_len - 1);
      vis_hi[h] = p.window_right >= 0 ? min(kv_len, right_bound(p, qi + off)) : kv_len;
      vis_lo[h] = p.window_left >= 0 ? max(0, qi + off - p.window_left) : 0;
    }
    // tiles fully inside [full_lo, full_hi) need no mask
    const int full_lo = p.window_left >= 0 ? max(0, qi_hi + off - p.window_left) : 0;
    const int full_hi = p.window_right >= 0 ? min(kv_len, right_bound(p, qi_lo + off)) : kv_len;

    float dq = 1.f, dk = 1.f;
    if (p.q_descale) dq = p.q_descale[b * p.q_descale_bs + kvh * p.q_descale_hs];
    if (p.k_descale) dk = p.k_descale[b * p.k_descale_bs + kvh * p.k_descale_hs];
    const float scale = p.softmax_scale * dq * dk;
    const float scale_log2 = scale * kLog2e;
    const float cap_in = p.softcap > 0.f ? scale / p.softcap : 0.f;
    const float cap_out = p.softcap * kLog2e;

    const uint32_t q_addr = smem_u32(q_smem);
    // lane roles for ldmatrix
    const int mat = lane >> 3, mrow = lane & 7;
    const uint32_t q_lane_row = wm * 16 + mrow + (mat & 1) * 8;
    const uint32_t q_lane_chunk = mat >> 1;
    const uint32_t k_lane_row = mrow + (mat >> 1) * 8;
    const uint32_t k_lane_chunk = mat & 1;
    const uint32_t v_lane_row = mrow + (mat & 1) * 8;
    const uint32_t v_lane_chunk = mat >> 1;

    for (int i = wt; i < n_tiles; i += WT) {
      const int stage = i % STAGES;
      const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase))) {
        if (lane == 0) {
          if (p.status) atomicExch(p.status, kWaitFullTimeout);
          atomicExch(&s_abort, 1);
        }
        break;
      }
      const int tok0 = (tile_lo + i) * kTileN;
      const uint32_t k_addr = smem_u32(ring + stage * Cfg::kStageBytes);
      const uint32_t v_addr = k_addr + Cfg::kOperandBytes;

      // Rows past the end of the request may hold anything (unused page tail,
      // stale shared memory): P is 0 there but 0 * NaN is NaN, so zero V rows.
      if (tok0 + kTileN > kv_len) {
        const int first = max(0, kv_len - tok0);
        uint8_t* v_ptr = ring + stage * Cfg::kStageBytes + Cfg::kOperandBytes;
        for (int idx = wm * 32 + lane; idx < (kTileN - first) * (D / 8); idx += WM * 32) {
          const int r = first + idx / (D / 8), c = idx % (D / 8);
          *reinterpret_cast<uint4*>(v_ptr + (c / 8) * (kTileN * 128) + swz128(r, c % 8)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        if (WM == 1) __syncwarp(); else named_barrier(2 + wt, WM * 32);
      }

      // ---- S = Q K^T ----
      float s[TN / 8][4];
#pragma unroll
      for (int j = 0; j < TN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t a[4];
          ldmatrix_x4(a[0], a[1], a[2], a[3],
                      q_addr + kb * (M * 128) + swz128(q_lane_row, ks * 2 + q_lane_chunk));
#pragma unroll
          for (int jp = 0; jp < TN / 16; ++jp) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3,
                        k_addr + kb * (kTileN * 128) + swz128(jp * 16 + k_lane_row, ks * 2 + k_lane_chunk));
            mma_bf16_16816(s[2 * jp], a, b0, b1);
            mma_bf16_16816(s[2 * jp + 1], a, b2, b3);
          }
        }
      }

      // ---- scale, softcap, mask ----
      const bool need_mask = tok0 < full_lo || tok0 + kTileN > full_hi;
#pragma unroll
      for (int j = 0; j < TN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = s[j][e];
          x = p.softcap > 0.f ? cap_out * fast_tanh(x * cap_in) : x * scale_log2;
          if (need_mask) {
            const int col = tok0 + j * 8 + 2 * t + (e & 1);
            const int h = e >> 1;
            if (col < vis_lo[h] || col >= vis_hi[h]) x = -INFINITY;
          }
          s[j][e] = x;
        }
      }

      // ---- online softmax (log2 domain) ----
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < TN / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * h], s[j][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[h], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = fast_exp2(m_run[h] - m_use);
        m_run[h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < TN / 8; ++j) {
          s[j][2 * h] = fast_exp2(s[j][2 * h] - m_use);
          s[j][2 * h + 1] = fast_exp2(s[j][2 * h + 1] - m_use);
          sum += s[j][2 * h] + s[j][2 * h + 1];
        }
        l_run[h] = l_run[h] * alpha[h] + sum;
      }
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        o_acc[n][0] *= alpha[0];
        o_acc[n][1] *= alpha[0];
        o_acc[n][2] *= alpha[1];
        o_acc[n][3] *= alpha[1];
      }

      // ---- O += P V ----
#pragma unroll
      for (int kk = 0; kk < TN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
          for (int cp = 0; cp < 4; ++cp) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3,
                              v_addr + kb * (kTileN * 128) + swz128(kk * 16 + v_lane_row, cp * 2 + v_lane_chunk));
            mma_bf16_16816(o_acc[kb * 8 + cp * 2], a, b0, b1);
            mma_bf16_16816(o_acc[kb * 8 + cp * 2 + 1], a, b2, b3);
          }
        }
      }

      // ---- release the stage ----
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }

    // row sums: add the four lanes of a quad
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
      l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
  }

  // Every TMA copy that was issued has been waited for by its consumer, so the
  // ring can be reused as the merge buffer once all warps are here.
  __syncthreads();
  if (*(volatile int*)&s_abort) return;

  float* red_o = reinterpret_cast<float*>(ring);                 // [WT][M][D]
  float* red_m = red_o + WT * M * D;                             // [WT][M]
  float* red_l = red_m + WT * M;                                 // [WT][M]
  if (!is_producer) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = wm * 16 + g + h * 8;
      float* dst = red_o + ((size_t)wt * M + r) * D;
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + 2 * t) = make_float2(o_acc[n][2 * h], o_acc[n][2 * h + 1]);
      if (t == 0) {
        red_m[wt * M + r] = m_run[h];
        red_l[wt * M + r] = l_run[h];
      }
    }
  }
  __syncthreads();

  // ---- merge the WT partial states, finalise, store ----
  float dv = 1.f;
  if (p.v_descale) dv = p.v_descale[b * p.v_descale_bs + kvh * p.v_descale_hs];
  const bool split_mode = p.num_splits > 1;
  for (int idx = tid; idx < M * (D / 4); idx += Cfg::kThreads) {
    const int r = idx / (D / 4), c4 = idx % (D / 4);
    const int row = row0 + r;
    if (row >= rows_total) continue;
    const int qi = row / p.group, hd = kvh * p.group + row % p.group;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WT; ++w) m = fmaxf(m, red_m[w * M + r]);
    float sink_l2 = -INFINITY;
    if (p.sink != nullptr && !split_mode) sink_l2 = __bfloat162float(p.sink[hd]) * kLog2e;
    const float m_f = fmaxf(m, sink_l2);
    const float m_use = m_f == -INFINITY ? 0.f : m_f;
    float l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WT; ++w) {
      const float mw = red_m[w * M + r];
      if (mw == -INFINITY) continue;  // that warp group saw no visible key: its O is all zero
      const float sc = fast_exp2(mw - m_use);
      l += red_l[w * M + r] * sc;
      const float4 ow = *reinterpret_cast<const float4*>(red_o + ((size_t)w * M + r) * D + c4 * 4);
      o.x += ow.x * sc; o.y += ow.y * sc; o.z += ow.z * sc; o.w += ow.w * sc;
    }
    if (sink_l2 != -INFINITY) l += fast_exp2(sink_l2 - m_use);
    const float inv = l > 0.f ? dv / l : 0.f;
    o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
    const float lse_l2 = l > 0.f ? m_use + log2f(l) : -INFINITY;
    const int64_t q_row = q_start + qi;
    if (split_mode) {
      const int64_t slot = ((int64_t)split * p.total_q + q_row) * p.num_q_heads + hd;
      *reinterpret_cast<float4*>(p.part_o + slot * D + c4 * 4) = o;
      if (c4 == 0) p.part_lse[slot] = lse_l2;
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + q_row * p.out_row_stride +
                           (int64_t)hd * p.out_head_stride + c4 * 4;
      uint2 packed;
      packed.x = pack_bf16(o.x, o.y);
      packed.y = pack_bf16(o.z, o.w);
      *reinterpret_cast<uint2*>(dst) = packed;
      if (c4 == 0 && p.lse != nullptr) p.lse[(int64_t)hd * p.total_q + q_row] = lse_l2 * kLn2;
    }
  }
}

template <int D, int WM, int WT, int STAGES, int TN>
cudaError_t launch_one(const FwdParams& p, cudaStream_t stream) {
  using Cfg = MmaCfg<D, WM, WT, STAGES, TN>;
  auto kernel = atrex_sm100_fwd_mma_kernel<D, WM, WT, STAGES, TN>;
  dim3 grid((unsigned)p.num_row_tiles * p.num_kv_heads, (unsigned)p.num_splits, 1);
  return launch_kernel(kernel, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, p);
}

template <int D, int WM, int WT, int STAGES, int TN>
cudaError_t prepare_one() {
  using Cfg = MmaCfg<D, WM, WT, STAGES, TN>;
  return cudaFuncSetAttribute(atrex_sm100_fwd_mma_kernel<D, WM, WT, STAGES, TN>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
}

}  // namespace

int mma_rows_for(int packed_rows) { return packed_rows <= 16 ? 16 : (packed_rows <= 32 ? 32 : 64); }

// KV tokens per stage: a stage is 32 KB (K + V) for both head dimensions.
int mma_tile_n(int head_dim) { return head_dim == 128 ? 64 : 32; }

#define ATREX_MMA_VARIANTS(X)  \
  X(128, 1, 2, 2, 64)          \
  X(128, 2, 2, 2, 64)          \
  X(128, 4, 1, 3, 64)          \
  X(256, 1, 2, 2, 32)          \
  X(256, 2, 2, 4, 32)          \
  X(256, 4, 1, 3, 32)

cudaError_t mma_prepare() {
  cudaError_t e;
#define X(D, WM, WT, ST, TN) \
  if ((e = prepare_one<D, WM, WT, ST, TN>()) != cudaSuccess) return e;
  ATREX_MMA_VARIANTS(X)
#undef X
  return cudaSuccess;
}

cudaError_t mma_launch(const FwdParams& p, int head_dim, int m_rows, cudaStream_t stream) {
#define X(D, WM, WT, ST, TN) \
  if (head_dim == D && m_rows == 16 * WM) return launch_one<D, WM, WT, ST, TN>(p, stream);
  ATREX_MMA_VARIANTS(X)
#undef X
  return cudaErrorInvalidValue;
}

}  // namespace atrex_sm100
