// C-ABI launcher of the sm_100a attention kernels (declared in include/atrex_fa_sm100.h).
//
// Host-only logic: argument checks, the route / split policy (from graph-static
// sizes only, as the reference's decode policy insists,
// src/nvidia/flash_attn/sm103/decode_runtime.py:443-470), TMA descriptor
// encoding, workspace carving and the launches.  Nothing here allocates,
// synchronises or reads device memory.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "atrex_fa_sm100.h"
#include "fa_kernels.cuh"

namespace atrex_sm100 {
namespace {

thread_local char g_last_error[256] = "";

int fail(int status, const char* what, cudaError_t cuda = cudaSuccess) {
  if (cuda != cudaSuccess)
    std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(cuda));
  else
    std::snprintf(g_last_error, sizeof(g_last_error), "%s", what);
  return status;
}

constexpr int kMaxDevices = 64;
constexpr int kMaxSplits = 256;

struct DeviceInfo {
  std::atomic<int> state{0};  // 0 unknown, 1 usable, -1 wrong architecture
  std::atomic<int> prepared{0};
  int sm_count = 0;
};
DeviceInfo g_devices[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::atomic<EncodeTiledFn> g_encode{nullptr};

EncodeTiledFn encode_fn() {
  EncodeTiledFn fn = g_encode.load(std::memory_order_acquire);
  if (fn != nullptr) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess || sym == nullptr)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  g_encode.store(fn, std::memory_order_release);
  return fn;
}

int current_device(DeviceInfo** info) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(ATREX_FA_UNSUPPORTED, "device ordinal out of range");
  DeviceInfo& d = g_devices[dev];
  int st = d.state.load(std::memory_order_acquire);
  if (st == 0) {
    int major = 0, minor = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return fail(ATREX_FA_CUDA_ERROR, "cudaDeviceGetAttribute failed");
    d.sm_count = sms;
    st = (major == 10 && minor == 0) ? 1 : -1;
    d.state.store(st, std::memory_order_release);
  }
  *info = &d;
  return st == 1 ? ATREX_FA_OK : fail(ATREX_FA_WRONG_DEVICE, "current device is not compute capability 10.0");
}

int prepare_device(DeviceInfo& d) {
  if (d.prepared.load(std::memory_order_acquire)) return ATREX_FA_OK;
  cudaError_t e = mma_prepare();
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "cudaFuncSetAttribute (mma kernels)", e);
  e = umma_prepare();
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "cudaFuncSetAttribute (tcgen05 kernel)", e);
  e = umma1_prepare();
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "cudaFuncSetAttribute (tcgen05 single-tile kernels)", e);
  d.prepared.store(1, std::memory_order_release);
  return ATREX_FA_OK;
}

inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

struct Resolved {
  int route, kernel, m_rows, tile_n, splits, launches;
  int tail_first, tail_splits;   // single-tile tcgen05 decode: split only the last round's items (0 = off)
  bool tiled;          // more than one row tile per request possible -> device plan
  int num_row_tiles;   // grid upper bound
  uint64_t off_order, off_prefix, off_lse, off_o, bytes;
};

int check_params(const atrex_fa_sm100_params* p) {
  if (p == nullptr) return fail(ATREX_FA_INVALID_VALUE, "parameter block is NULL");
  if (p->struct_bytes != sizeof(atrex_fa_sm100_params) || p->abi_version != ATREX_FA_SM100_ABI_VERSION)
    return fail(ATREX_FA_ABI_MISMATCH, "struct_bytes / abi_version do not match this library");
  if (p->batch < 0 || p->total_q < 0 || p->total_k < 0 || p->num_pages < 0 || p->page_size < 0 ||
      p->max_seqlen_q < 0 || p->max_seqlen_k < 0 || p->max_pages_per_seq < 0)
    return fail(ATREX_FA_INVALID_VALUE, "negative size (batch, total_q, total_k, num_pages, page_size, max_seqlen_*, max_pages_per_seq)");
  if (p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->num_q_heads % p->num_kv_heads != 0)
    return fail(ATREX_FA_INVALID_VALUE, "num_q_heads must be a positive multiple of num_kv_heads");
  if (p->num_splits < 0) return fail(ATREX_FA_INVALID_VALUE, "num_splits is negative");
  if (p->cu_seqlens_q == nullptr || p->out == nullptr) return fail(ATREX_FA_INVALID_VALUE, "cu_seqlens_q or out is NULL");
  if (p->total_q > 0 && p->q == nullptr) return fail(ATREX_FA_INVALID_VALUE, "q is NULL");
  if (p->page_size > 0) {
    if (p->block_table == nullptr || p->seqused_k == nullptr)
      return fail(ATREX_FA_INVALID_VALUE, "paged K/V needs block_table and seqused_k");
  } else if (p->cu_seqlens_k == nullptr) {
    return fail(ATREX_FA_INVALID_VALUE, "packed K/V needs cu_seqlens_k");
  }
  if (p->return_lse && p->lse == nullptr) return fail(ATREX_FA_INVALID_VALUE, "return_lse without an lse buffer");
  if (p->softcap < 0.f) return fail(ATREX_FA_INVALID_VALUE, "softcap is negative");
  if (p->cp_world_size < 0 || (p->cp_world_size > 1 && (p->cp_rank < 0 || p->cp_rank >= p->cp_world_size)))
    return fail(ATREX_FA_INVALID_VALUE, "cp_rank outside [0, cp_world_size)");
  if (p->cp_world_size > 1) {
    if (p->cp_tot_seqused_k == nullptr) return fail(ATREX_FA_INVALID_VALUE, "cp_world_size > 1 needs cp_tot_seqused_k");
    if (!p->causal || p->window_left >= 0 || p->window_right > 0)
      return fail(ATREX_FA_UNSUPPORTED, "context parallelism serves causal calls without a sliding window");
  }
  if (p->head_dim != 128 && p->head_dim != 256) return fail(ATREX_FA_UNSUPPORTED, "head_dim must be 128 or 256");
  if (p->dtype != ATREX_FA_BF16 && p->dtype != ATREX_FA_E4M3) return fail(ATREX_FA_UNSUPPORTED, "dtype must be BF16 or E4M3");
  if (p->num_splits > kMaxSplits) return fail(ATREX_FA_UNSUPPORTED, "num_splits above 256");
  if (p->page_size > 0 && p->page_size % 64 != 0 && p->page_size != 16 && p->page_size != 32)
    return fail(ATREX_FA_UNSUPPORTED, "page_size must be 16, 32 or a multiple of 64");
  if (p->route != ATREX_FA_ROUTE_AUTO && p->route != ATREX_FA_ROUTE_MMA && p->route != ATREX_FA_ROUTE_UMMA)
    return fail(ATREX_FA_INVALID_VALUE, "unknown route");
  // 16-byte alignment of everything the kernels touch with vectors or TMA
  const uint64_t es = p->dtype == ATREX_FA_E4M3 ? 1 : 2;
  auto misaligned = [&](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) != 0; };
  if (misaligned(p->q) || misaligned(p->k) || misaligned(p->v) || misaligned(p->out))
    return fail(ATREX_FA_UNSUPPORTED, "q, k, v and out must be 16-byte aligned");
  const int64_t strides[] = {p->q_row_stride, p->q_head_stride, p->k_row_stride, p->k_head_stride,
                             p->v_row_stride, p->v_head_stride, p->out_row_stride, p->out_head_stride,
                             p->page_size ? p->k_page_stride : 0, p->page_size ? p->v_page_stride : 0};
  for (int64_t s : strides)
    if (s < 0 || (static_cast<uint64_t>(s) * es) % 16 != 0)
      return fail(ATREX_FA_UNSUPPORTED, "a q / k / v / out stride is negative or not a multiple of 16 bytes");
  if ((static_cast<uint64_t>(p->out_row_stride) * 2) % 16 != 0 || (static_cast<uint64_t>(p->out_head_stride) * 2) % 16 != 0)
    return fail(ATREX_FA_UNSUPPORTED, "an out stride is not a multiple of 16 bytes");
  return ATREX_FA_OK;
}

enum Kernel { kKernelMma = 0, kKernelUmma2 = 1, kKernelUmma1 = 2 };

// Which kernel, how many splits, how much scratch - from graph-static sizes only.
//   mma.sync kernel   : BF16 calls with at most 16 packed rows per (request, KV head) (plain decode), softcap,
//                       a non-positive scale, or a caller that pins the route;
//   tcgen05, 2 subtiles: BF16 head_dim-128 prefill whose GQA group divides 128, no explicit KV split;
//   tcgen05, 1 tile    : everything else - FP8, head_dim 256, other groups, 17..128 packed rows (speculative
//                       decode, wide GQA decode) with split-KV, prefill with an explicit split count.
int resolve(const atrex_fa_sm100_params* p, int sm_count, Resolved* r) {
  const int group = p->num_q_heads / p->num_kv_heads;
  const int64_t packed_max = (int64_t)p->max_seqlen_q * group;
  const bool fp8 = p->dtype == ATREX_FA_E4M3;
  const bool tensor_ok = p->softcap == 0.f && p->softmax_scale > 0.f && umma1_supports(p->head_dim);
  const bool umma2_ok = tensor_ok && umma_supports(p->head_dim, group, !fp8) && p->q_head_stride <= p->q_row_stride;
  if ((p->route == ATREX_FA_ROUTE_UMMA || fp8) && !tensor_ok)
    return fail(ATREX_FA_UNSUPPORTED, fp8 ? "E4M3 calls run on the tcgen05 kernels only: no softcap, softmax_scale > 0"
                                          : "the tcgen05 route takes no softcap and needs softmax_scale > 0");
  if (fp8 && p->route == ATREX_FA_ROUTE_MMA)   // the mma.sync kernel is BF16 only
    return fail(ATREX_FA_UNSUPPORTED, "E4M3 calls cannot take the mma.sync route");
  int kernel;
  if (p->route == ATREX_FA_ROUTE_MMA) kernel = kKernelMma;
  else if (fp8) kernel = kKernelUmma1;
  else if (p->route == ATREX_FA_ROUTE_AUTO && (!tensor_ok || packed_max <= 16)) kernel = kKernelMma;
  else if (packed_max > 128 && umma2_ok && p->num_splits <= 1) kernel = kKernelUmma2;
  else kernel = kKernelUmma1;
  r->kernel = kernel;
  r->route = kernel == kKernelMma ? ATREX_FA_ROUTE_MMA : ATREX_FA_ROUTE_UMMA;

  int tile_n;
  if (kernel == kKernelMma) {
    r->m_rows = mma_rows_for((int)(packed_max > 64 ? 64 : packed_max));
    tile_n = mma_tile_n(p->head_dim);
  } else if (kernel == kKernelUmma2) {
    r->m_rows = umma_rows_per_item();
    tile_n = 128;
  } else {
    r->m_rows = umma1_rows_per_item();
    tile_n = umma1_tile_n(p->head_dim, fp8);
  }
  r->tile_n = tile_n;
  r->tiled = kernel == kKernelUmma2 || packed_max > r->m_rows;
  const int64_t tiles_bound =
      r->tiled ? ((int64_t)p->total_q * group) / r->m_rows + p->batch : (int64_t)p->batch;
  if (tiles_bound * p->num_kv_heads * kMaxSplits > 0x7FFFFFFFll)
    return fail(ATREX_FA_UNSUPPORTED, "row tiles x KV heads x splits exceeds the 32-bit work-item range");
  r->num_row_tiles = (int)tiles_bound;

  // keys one row tile can see, at the upper bound (a two-sided window limits it)
  int64_t span = p->max_seqlen_k;
  if (p->window_left >= 0 && (p->causal || p->window_right >= 0)) {
    const int64_t rows_q = r->tiled ? (r->m_rows + group - 1) / group + 1 : p->max_seqlen_q;
    const int64_t w = (int64_t)p->window_left + rows_q + (p->causal ? 0 : p->window_right) + 1 + tile_n;
    if (w < span) span = w;  // + one tile above: the window need not start on a tile edge
  }
  const int kv_tiles = (int)((span + tile_n - 1) / tile_n);
  int splits = 1;
  if (kernel == kKernelUmma2) {
    splits = 1;
  } else if (p->num_splits > 0) {
    splits = p->num_splits;
  } else if (kernel == kKernelMma || !r->tiled) {
    // decode-shaped: enough CTAs to fill the machine several times over, at least 512 keys per split
    const int64_t items = (int64_t)r->num_row_tiles * p->num_kv_heads;
    const int64_t slots = kernel == kKernelMma
                              ? (int64_t)sm_count * (p->head_dim == 128 ? (r->m_rows == 16 ? 3 : 2) : 1)
                              : (int64_t)sm_count;
    // The tcgen05 kernel is persistent and its split partials are wide (128 rows): split only to fill the SMs.
    const int64_t waves = kernel == kKernelMma ? 8 : 2;
    const int64_t want = items > 0 ? (slots * waves + items - 1) / items : 1;
    const int64_t cap = (int64_t)kv_tiles * tile_n / 512;
    splits = (int)(want < cap ? want : cap);
  }
  if (splits > kv_tiles) splits = kv_tiles;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits < 1) splits = 1;
  r->tail_first = r->tail_splits = 0;
  if (kernel == kKernelUmma1 && !r->tiled && p->num_splits == 0 && splits == 1) {
    // Persistent grid, one item per (request, KV head): when the items do not fill the last round, cut the
    // last round's items (whole requests) so that they do.  512 items on 148 SMs: 444 unsplit + 68 x 2.
    const int64_t items = (int64_t)p->batch * p->num_kv_heads;
    const int64_t grid = items < sm_count ? items : sm_count;
    const int64_t rem = grid > 0 && items > grid ? items % grid : 0;
    if (rem > 0) {
      const int64_t rem_req = (rem + p->num_kv_heads - 1) / p->num_kv_heads;
      int64_t ts = grid / (rem_req * p->num_kv_heads);
      if (ts > 4) ts = 4;
      if (ts > kv_tiles) ts = kv_tiles;
      if (ts >= 2) {
        r->tail_first = (int)(p->batch - rem_req);
        r->tail_splits = (int)ts;
        splits = (int)ts;   // sizes the partial buffers; only the tail requests' rows use them
      }
    }
  }
  r->splits = splits;
  r->launches = 1 + (r->tiled ? 1 : 0) + (splits > 1 ? 1 : 0);

  uint64_t off = 0;
  r->off_order = off;
  if (r->tiled) off = align_up(off + 4ull * p->batch, 256);
  r->off_prefix = off;
  if (r->tiled) off = align_up(off + 4ull * (p->batch + 1), 256);
  r->off_lse = off;
  if (splits > 1) off = align_up(off + 4ull * splits * p->total_q * p->num_q_heads, 256);
  r->off_o = off;
  if (splits > 1) off = align_up(off + 4ull * splits * p->total_q * p->num_q_heads * p->head_dim, 256);
  r->bytes = off;
  return ATREX_FA_OK;
}

// K or V as a 4-D tensor (D, heads, rows, pages).  The three outer dimensions
// are handed to the encoder in ascending-stride order (HND cache views have the
// head stride above the row stride); perm[] tells the kernel where each went.
int encode_kv_map(CUtensorMap* map, const void* base, int64_t head_stride, int64_t row_stride,
                  int64_t page_stride, int heads, int64_t rows, int64_t pages, int head_dim, int box_rows,
                  int8_t perm[3], int es = 2) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(ATREX_FA_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not found");
  struct Dim { uint64_t extent, stride; uint32_t box; int which; };
  Dim dims[3] = {{(uint64_t)heads, (uint64_t)head_stride * es, 1u, 0},
                 {(uint64_t)rows, (uint64_t)row_stride * es, (uint32_t)box_rows, 1},
                 {(uint64_t)pages, (uint64_t)page_stride * es, 1u, 2}};
  for (int i = 0; i < 3; ++i)       // extent-1 dimensions never move: give them a harmless stride
    if (dims[i].extent <= 1) { dims[i].extent = 1; }
  for (int i = 0; i < 3; ++i)
    for (int j = i + 1; j < 3; ++j)
      if (dims[j].stride < dims[i].stride) { Dim t = dims[i]; dims[i] = dims[j]; dims[j] = t; }
  cuuint64_t extent[4] = {(cuuint64_t)head_dim, dims[0].extent, dims[1].extent, dims[2].extent};
  cuuint64_t stride[3] = {dims[0].stride, dims[1].stride, dims[2].stride};
  cuuint32_t box[4] = {(cuuint32_t)(128 / es), dims[0].box, dims[1].box, dims[2].box};   // 128 bytes wide
  cuuint32_t elem[4] = {1u, 1u, 1u, 1u};
  for (int i = 0; i < 3; ++i) {
    if (stride[i] == 0) stride[i] = 16;  // extent-1 dimension with a zero stride
    if (stride[i] % 16 != 0 || stride[i] >= (1ull << 40))
      return fail(ATREX_FA_UNSUPPORTED, "K/V stride is not a multiple of 16 bytes below 2^40");
    perm[dims[i].which] = (int8_t)i;
  }
  const CUresult res = fn(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 4,
                          const_cast<void*>(base), extent, stride, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return res == CUDA_SUCCESS ? ATREX_FA_OK : fail(ATREX_FA_UNSUPPORTED, "cuTensorMapEncodeTiled rejected the K/V layout");
}

// Q as (D, Hq, total_q); one box = 64 elements x `group` heads x 128/group rows = 128 packed GQA rows.
int encode_q_map(CUtensorMap* map, const void* base, int64_t head_stride, int64_t row_stride, int heads,
                 int64_t rows, int head_dim, int group, int es) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(ATREX_FA_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t extent[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)(rows > 0 ? rows : 1)};
  cuuint64_t stride[2] = {(cuuint64_t)head_stride * es, (cuuint64_t)row_stride * es};
  cuuint32_t box[3] = {(cuuint32_t)(128 / es), (cuuint32_t)group, (cuuint32_t)(128 / group)};
  cuuint32_t elem[3] = {1u, 1u, 1u};
  const CUresult res = fn(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                          const_cast<void*>(base), extent, stride, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return res == CUDA_SUCCESS ? ATREX_FA_OK : fail(ATREX_FA_UNSUPPORTED, "cuTensorMapEncodeTiled rejected the Q layout");
}

}  // namespace

int report_failure(int status, const char* what, cudaError_t cuda) { return fail(status, what, cuda); }
void clear_failure() { g_last_error[0] = 0; }
int current_sm_count(int* sm_count) {
  DeviceInfo* info = nullptr;
  const int st = current_device(&info);
  if (st == ATREX_FA_OK) *sm_count = info->sm_count;
  return st;
}

}  // namespace atrex_sm100

using namespace atrex_sm100;

extern "C" {

const char* atrex_fa_sm100_last_error(void) { return g_last_error; }

int atrex_fa_sm100_abi_version(void) { return ATREX_FA_SM100_ABI_VERSION; }

size_t atrex_fa_sm100_params_bytes(void) { return sizeof(atrex_fa_sm100_params); }

const char* atrex_fa_sm100_status_string(int status) {
  switch (status) {
    case ATREX_FA_OK: return "ok";
    case ATREX_FA_INVALID_VALUE: return "invalid value in attention parameters";
    case ATREX_FA_UNSUPPORTED: return "well-formed call that the sm100 kernels do not serve (dtype, head_dim, page_size, alignment or route)";
    case ATREX_FA_WORKSPACE_TOO_SMALL: return "workspace is missing, misaligned or smaller than the plan requires";
    case ATREX_FA_CUDA_ERROR: return "a CUDA runtime or driver call failed";
    case ATREX_FA_WRONG_DEVICE: return "current CUDA device is not compute capability 10.0 (sm_100a)";
    case ATREX_FA_ABI_MISMATCH: return "parameter block does not match this library's ABI version or size";
    default: return "unknown status";
  }
}

int atrex_fa_sm100_plan(const atrex_fa_sm100_params* p, atrex_fa_sm100_plan_info* plan) {
  if (plan == nullptr) return fail(ATREX_FA_INVALID_VALUE, "plan is NULL");
  g_last_error[0] = 0;
  int st = check_params(p);
  if (st != ATREX_FA_OK) return st;
  int sm_count = p->sm_count;
  if (sm_count <= 0) {
    DeviceInfo* info = nullptr;
    st = current_device(&info);
    if (st != ATREX_FA_OK) return st;
    sm_count = info->sm_count;
  }
  Resolved r;
  st = resolve(p, sm_count, &r);
  if (st != ATREX_FA_OK) return st;
  plan->route = r.route;
  plan->num_splits = r.splits;
  plan->kernel_launches = r.launches;
  plan->m_rows = r.m_rows;
  plan->workspace_bytes = r.bytes;
  return ATREX_FA_OK;
}

int atrex_fa_sm100_prewarm(void) {
  g_last_error[0] = 0;
  DeviceInfo* info = nullptr;
  const int st = current_device(&info);
  if (st != ATREX_FA_OK) return st;
  return prepare_device(*info);
}

// The TMA descriptors of a call and what was decided with them.
struct EncodedMaps {
  CUtensorMap k_map, v_map, q_map;
  int8_t k_perm[3], v_perm[3];
  int32_t box_rows, q_via_tma, num_pages;
};

static int encode_maps(const atrex_fa_sm100_params* p, const Resolved& r, EncodedMaps& m) {
  int st = ATREX_FA_OK;
  const bool paged = p->page_size > 0;
  const int64_t rows = paged ? p->page_size : p->total_k;
  const int64_t pages = paged ? p->num_pages : 1;
  const int es = p->dtype == ATREX_FA_E4M3 ? 1 : 2;
  // Rows one TMA box covers: a whole KV tile of the chosen kernel, or less where pages are smaller.  A box never
  // crosses a page: with pages of 192, 320, ... rows a 128-key tile straddles pages at 64-row granularity, so
  // the box is the largest power of two dividing both (page sizes are 16, 32 or multiples of 64).
  int box_rows = r.tile_n;
  if (paged) while (p->page_size % box_rows != 0) box_rows >>= 1;
  const bool empty_kv = rows == 0 || pages == 0 || p->k == nullptr || p->v == nullptr;
  int8_t kperm[3] = {0, 1, 2}, vperm[3] = {0, 1, 2};
  if (empty_kv) {
    // No key exists: the kernels will not issue a copy, but the descriptors must still be valid.
    st = encode_kv_map(&m.k_map, p->q, p->head_dim, p->head_dim, p->head_dim, 1, 1, 1, p->head_dim, box_rows, kperm, es);
    if (st == ATREX_FA_OK)
      st = encode_kv_map(&m.v_map, p->q, p->head_dim, p->head_dim, p->head_dim, 1, 1, 1, p->head_dim, box_rows, vperm, es);
  } else {
    st = encode_kv_map(&m.k_map, p->k, p->k_head_stride, p->k_row_stride,
                       paged ? p->k_page_stride : p->k_row_stride * rows, p->num_kv_heads, rows, pages,
                       p->head_dim, box_rows, kperm, es);
    if (st == ATREX_FA_OK)
      st = encode_kv_map(&m.v_map, p->v, p->v_head_stride, p->v_row_stride,
                         paged ? p->v_page_stride : p->v_row_stride * rows, p->num_kv_heads, rows, pages,
                         p->head_dim, box_rows, vperm, es);
  }
  if (st != ATREX_FA_OK) return st;
  for (int i = 0; i < 3; ++i) { m.k_perm[i] = kperm[i]; m.v_perm[i] = vperm[i]; }
  m.q_via_tma = r.kernel == kKernelUmma2 || (r.kernel == kKernelUmma1 && umma1_q_via_tma(p->num_q_heads / p->num_kv_heads) &&
                                             p->q_head_stride <= p->q_row_stride);
  if (m.q_via_tma) {
    st = encode_q_map(&m.q_map, p->q, p->q_head_stride, p->q_row_stride, p->num_q_heads, p->total_q, p->head_dim,
                      p->num_q_heads / p->num_kv_heads, es);
    if (st != ATREX_FA_OK) return st;
  }
  m.box_rows = box_rows;
  m.num_pages = empty_kv ? 0 : (int)pages;
  return ATREX_FA_OK;
}

// A serving loop repeats the same call shape over the same Q buffer and KV pools step after step, and
// encoding two or three TMA descriptors through the driver is the largest single cost on the host side
// of a launch.  Each host thread keeps the descriptors of its last few distinct (Q, K, V layout, kernel)
// combinations.  The key holds every input of the encoding, so a hit returns descriptors that are
// bit-identical to a fresh encoding; nothing that lives in device memory (lengths, page tables,
// descales) is cached, and every other kernel argument is rebuilt from the caller's block on each call.
namespace {
struct MapKey {
  const void *q, *k, *v;
  int64_t q_row_stride, q_head_stride, k_page_stride, k_row_stride, k_head_stride, v_page_stride, v_row_stride,
      v_head_stride;
  int32_t total_q, total_k, num_pages, page_size, num_q_heads, num_kv_heads, head_dim, dtype, kernel, tile_n, device,
      pad;
};
constexpr int kMapCacheSlots = 16;
struct CachedMaps {
  bool valid = false;
  uint64_t stamp = 0;
  MapKey key;
  EncodedMaps maps;
};
thread_local CachedMaps g_maps[kMapCacheSlots];
thread_local uint64_t g_map_stamp = 0;
}  // namespace

static int maps_for(const atrex_fa_sm100_params* p, const Resolved& r, int device, const EncodedMaps** out) {
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.q = p->q; key.k = p->k; key.v = p->v;
  key.q_row_stride = p->q_row_stride; key.q_head_stride = p->q_head_stride;
  key.k_page_stride = p->k_page_stride; key.k_row_stride = p->k_row_stride; key.k_head_stride = p->k_head_stride;
  key.v_page_stride = p->v_page_stride; key.v_row_stride = p->v_row_stride; key.v_head_stride = p->v_head_stride;
  key.total_q = p->total_q; key.total_k = p->total_k; key.num_pages = p->num_pages; key.page_size = p->page_size;
  key.num_q_heads = p->num_q_heads; key.num_kv_heads = p->num_kv_heads; key.head_dim = p->head_dim;
  key.dtype = p->dtype; key.kernel = r.kernel; key.tile_n = r.tile_n; key.device = device;
  CachedMaps* victim = &g_maps[0];
  for (CachedMaps& c : g_maps) {
    if (c.valid && std::memcmp(&c.key, &key, sizeof(key)) == 0) {
      c.stamp = ++g_map_stamp;
      *out = &c.maps;
      return ATREX_FA_OK;
    }
    if (victim->valid && (!c.valid || c.stamp < victim->stamp)) victim = &c;
  }
  victim->valid = false;
  const int st = encode_maps(p, r, victim->maps);
  if (st != ATREX_FA_OK) return st;
  victim->key = key;
  victim->stamp = ++g_map_stamp;
  victim->valid = true;
  *out = &victim->maps;
  return ATREX_FA_OK;
}

int atrex_fa_sm100_forward(const atrex_fa_sm100_params* p, void* workspace, uint64_t workspace_bytes,
                           void* stream_ptr) {
  g_last_error[0] = 0;
  int st = check_params(p);
  if (st != ATREX_FA_OK) return st;
  DeviceInfo* info = nullptr;
  st = current_device(&info);
  if (st != ATREX_FA_OK) return st;
  Resolved r;
  st = resolve(p, p->sm_count > 0 ? p->sm_count : info->sm_count, &r);
  if (st != ATREX_FA_OK) return st;
  if (r.bytes > 0 && (workspace == nullptr || workspace_bytes < r.bytes ||
                      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0))
    return fail(ATREX_FA_WORKSPACE_TOO_SMALL, "workspace missing, misaligned or too small");
  if (p->batch == 0 || p->total_q == 0) return ATREX_FA_OK;
  st = prepare_device(*info);
  if (st != ATREX_FA_OK) return st;
  const EncodedMaps* maps = nullptr;
  st = maps_for(p, r, (int)(info - g_devices), &maps);
  if (st != ATREX_FA_OK) return st;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const bool paged = p->page_size > 0;
  const bool fp8 = p->dtype == ATREX_FA_E4M3;
  FwdParams f;
  std::memset(&f, 0, sizeof(f));
  f.k_map = maps->k_map; f.v_map = maps->v_map; f.q_map = maps->q_map;
  for (int i = 0; i < 3; ++i) { f.k_perm[i] = maps->k_perm[i]; f.v_perm[i] = maps->v_perm[i]; }
  f.q_via_tma = maps->q_via_tma;
  f.q = p->q; f.out = p->out; f.lse = p->return_lse ? p->lse : nullptr;
  f.cu_seqlens_q = p->cu_seqlens_q;
  f.cu_seqlens_k = paged ? nullptr : p->cu_seqlens_k;
  f.seqused_k = p->seqused_k;
  f.block_table = p->block_table;
  f.q_descale = p->q_descale; f.k_descale = p->k_descale; f.v_descale = p->v_descale;
  // with context parallelism the sink logit joins the softmax once, on rank 0; the merge across ranks carries it
  f.sink = (p->cp_world_size > 1 && p->cp_rank != 0) ? nullptr : static_cast<const __nv_bfloat16*>(p->sink);
  f.status = p->device_status;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  if (r.tiled) {
    f.order = reinterpret_cast<int32_t*>(ws + r.off_order);
    f.tile_prefix = reinterpret_cast<int32_t*>(ws + r.off_prefix);
  }
  if (r.splits > 1) {
    f.part_lse = reinterpret_cast<float*>(ws + r.off_lse);
    f.part_o = reinterpret_cast<float*>(ws + r.off_o);
  }
  f.q_row_stride = p->q_row_stride; f.q_head_stride = p->q_head_stride;
  f.out_row_stride = p->out_row_stride; f.out_head_stride = p->out_head_stride;
  f.block_table_row_stride = p->block_table_row_stride;
  f.q_descale_bs = p->q_descale_batch_stride; f.q_descale_hs = p->q_descale_head_stride;
  f.k_descale_bs = p->k_descale_batch_stride; f.k_descale_hs = p->k_descale_head_stride;
  f.v_descale_bs = p->v_descale_batch_stride; f.v_descale_hs = p->v_descale_head_stride;
  f.batch = p->batch; f.total_q = p->total_q; f.total_k = p->total_k;
  f.num_pages = maps->num_pages;
  f.page_size = p->page_size; f.box_rows = maps->box_rows;
  f.num_q_heads = p->num_q_heads; f.num_kv_heads = p->num_kv_heads;
  f.group = p->num_q_heads / p->num_kv_heads;
  f.causal = p->causal ? 1 : 0;
  f.window_left = p->window_left < 0 ? -1 : p->window_left;
  f.window_right = p->causal ? 0 : (p->window_right < 0 ? -1 : p->window_right);
  f.num_splits = r.splits;
  f.num_row_tiles = r.num_row_tiles;
  {
    const int64_t cap = paged ? (int64_t)p->max_pages_per_seq * p->page_size : 0;
    f.kv_cap = (int32_t)(cap > 0x7FFFFFFFll ? 0x7FFFFFFFll : cap);
  }
  f.cp_world_size = p->cp_world_size > 1 ? p->cp_world_size : 1;
  f.cp_rank = p->cp_world_size > 1 ? p->cp_rank : 0;
  f.cp_tot_seqused_k = p->cp_world_size > 1 ? p->cp_tot_seqused_k : nullptr;
  f.tail_first = r.tail_first;
  f.tail_splits = r.tail_splits;
  f.softmax_scale = p->softmax_scale;
  f.softcap = p->softcap;

  cudaError_t e;
  if (r.tiled && (e = plan_launch(f, r.m_rows, const_cast<int32_t*>(f.order), const_cast<int32_t*>(f.tile_prefix),
                                  stream)) != cudaSuccess)
    return fail(ATREX_FA_CUDA_ERROR, "launch of the plan kernel", e);
  if (p->profile_event_begin != nullptr &&
      (e = cudaEventRecord(static_cast<cudaEvent_t>(p->profile_event_begin), stream)) != cudaSuccess)
    return fail(ATREX_FA_CUDA_ERROR, "cudaEventRecord(profile_event_begin)", e);
  const int sms = p->sm_count > 0 ? p->sm_count : info->sm_count;
  if (r.kernel == kKernelUmma2) e = umma_launch(f, sms, stream);
  else if (r.kernel == kKernelUmma1) e = umma1_launch(f, p->head_dim, fp8, sms, stream);
  else e = mma_launch(f, p->head_dim, r.m_rows, stream);
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "launch of the attention kernel", e);
  if (p->profile_event_end != nullptr &&
      (e = cudaEventRecord(static_cast<cudaEvent_t>(p->profile_event_end), stream)) != cudaSuccess)
    return fail(ATREX_FA_CUDA_ERROR, "cudaEventRecord(profile_event_end)", e);
  if (r.splits > 1 && (e = combine_launch(f, p->head_dim, stream)) != cudaSuccess)
    return fail(ATREX_FA_CUDA_ERROR, "launch of the combine kernel", e);
  return ATREX_FA_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Entry point that allocates nothing (no counterpart in the reference).
//
// Some hosts of this library have no way to hand it scratch memory: a serving
// process that binds the C ABI over FFI and only ever receives device pointers
// from another runtime owns no device allocator; an engine that reserved all of
// HBM for its KV-cache pool at start-up makes any later cudaMalloc fail; and a
// latency-critical loop cannot afford cudaMalloc / cudaFree, which synchronise
// the whole device.  For them the split-KV scratch (partial O and partial LSE,
// plus the row-tile plan) lives in the fixed array below, which every GPU that
// loads this library holds until the process exits.
// ---------------------------------------------------------------------------
namespace atrex_sm100 {
namespace {

constexpr uint64_t kStaticScratchBytes = ATREX_FA_SM100_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device.  In host code the array's
// name is only a stand-in for the symbol, never a device address, so it is
// resolved with cudaGetSymbolAddress once per device, with that device current.
std::atomic<void*> g_static_scratch_ptr[kMaxDevices];

int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail(ATREX_FA_UNSUPPORTED, "device ordinal out of range");
  void* ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(ATREX_FA_CUDA_ERROR, "cudaGetSymbolAddress(static scratch)", e);
    g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return ATREX_FA_OK;
}

}  // namespace
}  // namespace atrex_sm100

extern "C" {

uint64_t atrex_fa_sm100_static_scratch_bytes(void) { return kStaticScratchBytes; }

int atrex_fa_sm100_forward_static_scratch(const atrex_fa_sm100_params* p, void* stream) {
  atrex_fa_sm100_plan_info info;
  int st = atrex_fa_sm100_plan(p, &info);
  if (st != ATREX_FA_OK) return st;
  if (info.workspace_bytes > kStaticScratchBytes) {
    char text[200];
    std::snprintf(text, sizeof(text),
                  "call needs %llu bytes of scratch but the built-in scratch holds %llu: lower num_splits or "
                  "use atrex_fa_sm100_forward with caller scratch",
                  (unsigned long long)info.workspace_bytes, (unsigned long long)kStaticScratchBytes);
    return fail(ATREX_FA_WORKSPACE_TOO_SMALL, text);
  }
  void* scratch = nullptr;
  st = static_scratch_for_current_device(&scratch);
  if (st != ATREX_FA_OK) return st;
  // Nothing in the scratch has to start at zero: every partial a combine reads
  // was written by the attention kernel of the same call, and a split without
  // keys publishes LSE = -inf so its (stale) partial O is never read.
  return atrex_fa_sm100_forward(p, scratch, kStaticScratchBytes, stream);
}


size_t atrex_fa_sm100_kv_write_params_bytes(void) { return sizeof(atrex_fa_sm100_kv_write_params); }

static int kv_fill(const atrex_fa_sm100_kv_write_params* p, bool need_cache, atrex_sm100::KvWriteParams* k, bool* fp8_out,
                   int* sm_count) {
  using namespace atrex_sm100;
  g_last_error[0] = 0;
  if (p == nullptr) return fail(ATREX_FA_INVALID_VALUE, "null parameter block");
  if (p->struct_bytes != sizeof(atrex_fa_sm100_kv_write_params) || p->abi_version != ATREX_FA_SM100_ABI_VERSION)
    return fail(ATREX_FA_ABI_MISMATCH, "kv-write parameter block does not match this library");
  if (p->num_tokens < 0 || p->num_kv_heads <= 0 || p->head_dim <= 0 || p->page_size <= 0 || p->num_pages < 0)
    return fail(ATREX_FA_INVALID_VALUE, "negative or zero size");
  if (p->num_kv_heads > 1024) return fail(ATREX_FA_UNSUPPORTED, "more than 1024 KV heads");   // per-head shared-memory tables
  bool fp8 = false;
  if (need_cache) {
    if (p->cache_dtype != ATREX_FA_BF16 && p->cache_dtype != ATREX_FA_E4M3)
      return fail(ATREX_FA_UNSUPPORTED, "cache dtype must be BF16 or E4M3");
    fp8 = p->cache_dtype == ATREX_FA_E4M3;
  }
  if (p->head_dim % (fp8 ? 16 : 8)) return fail(ATREX_FA_UNSUPPORTED, "head_dim must be a multiple of 8 (16 for E4M3)");
  if (p->num_tokens > 0) {
    if (!p->key || !p->value || !p->slot_mapping) return fail(ATREX_FA_INVALID_VALUE, "null tensor pointer");
    if (need_cache && (!p->key_cache || !p->value_cache)) return fail(ATREX_FA_INVALID_VALUE, "null cache pointer");
    // 16-byte source vectors; 16-byte (BF16) or 8-byte (E4M3) destination vectors
    const int64_t src_strides[] = {p->key_token_stride, p->key_head_stride, p->value_token_stride, p->value_head_stride};
    for (int64_t st : src_strides)
      if ((st * 2) % 16) return fail(ATREX_FA_UNSUPPORTED, "key / value strides must be multiples of 16 bytes");
    if (((uintptr_t)p->key | (uintptr_t)p->value) % 16) return fail(ATREX_FA_UNSUPPORTED, "key / value are not 16-byte aligned");
    if (need_cache) {
      const int64_t dst_strides[] = {p->key_cache_page_stride,   p->key_cache_row_stride,   p->key_cache_head_stride,
                                     p->value_cache_page_stride, p->value_cache_row_stride, p->value_cache_head_stride};
      const int dst_align = fp8 ? 8 : 16, dst_es = fp8 ? 1 : 2;
      for (int64_t st : dst_strides)
        if ((st * dst_es) % dst_align) return fail(ATREX_FA_UNSUPPORTED, "cache strides are not vector aligned");
      if (((uintptr_t)p->key_cache | (uintptr_t)p->value_cache) % dst_align)
        return fail(ATREX_FA_UNSUPPORTED, "cache pointers are not vector aligned");
    }
  }
  DeviceInfo* dev = nullptr;
  int st = current_device(&dev);
  if (st != ATREX_FA_OK) return st;
  *sm_count = dev->sm_count;
  *fp8_out = fp8;
  k->key = static_cast<const __nv_bfloat16*>(p->key);
  k->value = static_cast<const __nv_bfloat16*>(p->value);
  k->key_cache = p->key_cache;
  k->value_cache = p->value_cache;
  k->slot_mapping = reinterpret_cast<const long long*>(p->slot_mapping);
  k->k_scale = p->k_scale;
  k->v_scale = p->v_scale;
  k->k_token_stride = p->key_token_stride, k->k_head_stride = p->key_head_stride;
  k->v_token_stride = p->value_token_stride, k->v_head_stride = p->value_head_stride;
  k->kc_page_stride = p->key_cache_page_stride, k->kc_row_stride = p->key_cache_row_stride;
  k->kc_head_stride = p->key_cache_head_stride;
  k->vc_page_stride = p->value_cache_page_stride, k->vc_row_stride = p->value_cache_row_stride;
  k->vc_head_stride = p->value_cache_head_stride;
  k->k_scale_head_stride = p->k_scale_head_stride, k->v_scale_head_stride = p->v_scale_head_stride;
  k->num_tokens = p->num_tokens, k->num_kv_heads = p->num_kv_heads, k->head_dim = p->head_dim, k->page_size = p->page_size;
  k->slot_limit = p->num_pages > 0 ? (long long)p->num_pages * p->page_size : 0x7FFFFFFFFFFFFFFFll;
  return ATREX_FA_OK;
}

int atrex_fa_sm100_kv_cache_write(const atrex_fa_sm100_kv_write_params* p, void* stream) {
  using namespace atrex_sm100;
  KvWriteParams k;
  bool fp8 = false;
  int sms = 0;
  int st = kv_fill(p, true, &k, &fp8, &sms);
  if (st != ATREX_FA_OK) return st;
  if (p->num_tokens == 0) return ATREX_FA_OK;
  cudaError_t e = kv_write_launch(k, fp8, sms, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "kv-cache write kernel launch", e);
  return ATREX_FA_OK;
}

int atrex_fa_sm100_kv_scales(const atrex_fa_sm100_kv_write_params* p, float* k_scale_out, float* v_scale_out,
                             void* scratch, void* stream) {
  using namespace atrex_sm100;
  if (k_scale_out == nullptr || v_scale_out == nullptr || scratch == nullptr || ((uintptr_t)scratch % 4))
    return fail(ATREX_FA_INVALID_VALUE, "null or misaligned output / scratch pointer");
  KvWriteParams k;
  bool fp8 = false;
  int sms = 0;
  int st = kv_fill(p, false, &k, &fp8, &sms);
  if (st != ATREX_FA_OK) return st;
  cudaError_t e = kv_scales_launch(k, static_cast<unsigned*>(scratch), k_scale_out, v_scale_out, sms,
                                   static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "kv-scales kernel launch", e);
  return ATREX_FA_OK;
}

int atrex_fa_sm100_merge_parts(const void* parts, const float* part_lse, void* out, float* lse, int32_t world,
                               int64_t total_q, int32_t num_q_heads, int32_t head_dim, void* stream) {
  using namespace atrex_sm100;
  g_last_error[0] = 0;
  if (world <= 0 || total_q < 0 || num_q_heads <= 0) return fail(ATREX_FA_INVALID_VALUE, "negative or zero size");
  if (head_dim <= 0 || head_dim % 32 || head_dim > 256) return fail(ATREX_FA_UNSUPPORTED, "head_dim must be a multiple of 32 up to 256");
  if (total_q == 0) return ATREX_FA_OK;
  if (!parts || !part_lse || !out || !lse) return fail(ATREX_FA_INVALID_VALUE, "null tensor pointer");
  DeviceInfo* dev = nullptr;
  int st = current_device(&dev);
  if (st != ATREX_FA_OK) return st;
  cudaError_t e = merge_parts_launch(parts, part_lse, out, lse, world, total_q, num_q_heads, head_dim,
                                     static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(ATREX_FA_CUDA_ERROR, "merge kernel launch", e);
  return ATREX_FA_OK;
}

}  // extern "C"
