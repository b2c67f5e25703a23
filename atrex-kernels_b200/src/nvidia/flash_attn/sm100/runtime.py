"""Torch custom op over the C-ABI launcher of the sm_100a attention kernels.

The op ``atrex_sm100::fa_fwd`` mutates caller-owned ``out`` / ``lse`` / ``workspace``
tensors and enqueues on torch's current stream; its CUDA implementation fills the
plain-C parameter block declared in ``include/atrex_fa_sm100.h`` and calls
``atrex_fa_sm100_forward`` through ctypes.  This is the counterpart of the
reference's per-family runtimes, which allocate outputs and call-local scratch and
launch a prebuilt kernel (src/nvidia/flash_attn/sm103/decode_runtime.py:637-890,
src/ppu/flash_attn/zwm890p/decode_runtime.py:99-113 for the ctypes C-ABI form).

There is no fallback of any kind: if ``libatrex_fa_sm100.so`` is missing or its
ABI does not match, the first call raises ``RuntimeError``.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

ABI_VERSION = 5
ROUTE_AUTO, ROUTE_MMA, ROUTE_UMMA = 0, 1, 2
_STATUS_EXCEPTIONS = {1: ValueError, 2: NotImplementedError}

_i64, _i32, _u32, _f32, _ptr = ctypes.c_int64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_float, ctypes.c_void_p


class Params(ctypes.Structure):
    """Mirror of ``atrex_fa_sm100_params`` (include/atrex_fa_sm100.h); order and types must match."""

    _fields_ = (
        [("struct_bytes", _u32), ("abi_version", _u32)]
        + [(n, _ptr) for n in ("q", "k", "v", "out", "lse", "cu_seqlens_q", "cu_seqlens_k", "seqused_k",
                               "block_table", "q_descale", "k_descale", "v_descale", "sink", "device_status",
                               "profile_event_begin", "profile_event_end", "cp_tot_seqused_k")]
        + [(n, _i64) for n in ("q_row_stride", "q_head_stride",
                               "k_page_stride", "k_row_stride", "k_head_stride",
                               "v_page_stride", "v_row_stride", "v_head_stride",
                               "out_row_stride", "out_head_stride", "block_table_row_stride",
                               "q_descale_batch_stride", "q_descale_head_stride",
                               "k_descale_batch_stride", "k_descale_head_stride",
                               "v_descale_batch_stride", "v_descale_head_stride")]
        + [(n, _i32) for n in ("batch", "total_q", "total_k", "num_pages", "page_size", "max_pages_per_seq",
                               "max_seqlen_q", "max_seqlen_k", "num_q_heads", "num_kv_heads", "head_dim",
                               "dtype", "causal", "window_left", "window_right", "return_lse", "num_splits",
                               "route", "sm_count", "cp_world_size", "cp_rank")]
        + [("softmax_scale", _f32), ("softcap", _f32)]
    )


class PlanInfo(ctypes.Structure):
    """Mirror of ``atrex_fa_sm100_plan_info``."""

    _fields_ = [("route", _i32), ("num_splits", _i32), ("kernel_launches", _i32), ("m_rows", _i32),
                ("workspace_bytes", ctypes.c_uint64)]


LIBRARY_PATH = Path(__file__).resolve().parent / "libatrex_fa_sm100.so"
_lib = None
_lib_lock = threading.Lock()
_status_tensors: dict[int, torch.Tensor] = {}


def load_library():
    """Load the native library once; raise ``RuntimeError`` when it is absent or incompatible."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not LIBRARY_PATH.is_file():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python {LIBRARY_PATH.parent / 'build.py'}` "
                "(there is no fallback path)"
            )
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        lib.atrex_fa_sm100_abi_version.restype = ctypes.c_int
        lib.atrex_fa_sm100_params_bytes.restype = ctypes.c_size_t
        lib.atrex_fa_sm100_status_string.restype = ctypes.c_char_p
        lib.atrex_fa_sm100_status_string.argtypes = [ctypes.c_int]
        lib.atrex_fa_sm100_last_error.restype = ctypes.c_char_p
        lib.atrex_fa_sm100_plan.restype = ctypes.c_int
        lib.atrex_fa_sm100_plan.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(PlanInfo)]
        lib.atrex_fa_sm100_forward.restype = ctypes.c_int
        lib.atrex_fa_sm100_forward.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        lib.atrex_fa_sm100_prewarm.restype = ctypes.c_int
        if lib.atrex_fa_sm100_abi_version() != ABI_VERSION or lib.atrex_fa_sm100_params_bytes() != ctypes.sizeof(Params):
            raise RuntimeError("libatrex_fa_sm100.so does not match this Python binding (ABI version or struct size)")
        _lib = lib
    return _lib


def raise_for_status(status: int) -> None:
    if status == 0:
        return
    lib = load_library()
    text = lib.atrex_fa_sm100_status_string(status).decode()
    detail = lib.atrex_fa_sm100_last_error().decode()
    raise _STATUS_EXCEPTIONS.get(status, RuntimeError)(f"atrex sm100 attention: {text} (status {status}; {detail})")


def _ptr_of(t):
    return None if t is None else t.data_ptr()


def device_status(device) -> torch.Tensor | None:
    """Per-device int32 word that kernels set if a bounded wait expires; None while a graph is being captured
    and the word does not exist yet (it is allocated eagerly, never inside a capture)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_tensors.get(index)
    if word is None and not torch.cuda.is_current_stream_capturing():
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_tensors[index] = word
    return word


def check_device_status(device) -> int:
    """Synchronise and return the device status word (0 = no bounded wait ever expired); resets it."""
    word = device_status(torch.device(device))
    if word is None:
        return 0
    value = int(word.item())
    if value:
        word.zero_()
    return value


def set_pointers(p: Params, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, q_descale,
                 k_descale, v_descale, sink, status, cp_tot_seqused_k=None) -> None:
    """The part of a parameter block that changes from call to call for one layout: the addresses."""
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _ptr_of(lse)
    p.cu_seqlens_q, p.cu_seqlens_k = cu_seqlens_q.data_ptr(), _ptr_of(cu_seqlens_k)
    p.seqused_k, p.block_table = _ptr_of(seqused_k), _ptr_of(block_table)
    p.q_descale, p.k_descale, p.v_descale = _ptr_of(q_descale), _ptr_of(k_descale), _ptr_of(v_descale)
    p.sink, p.device_status = _ptr_of(sink), _ptr_of(status)
    p.cp_tot_seqused_k = _ptr_of(cp_tot_seqused_k)


def layout_key(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, q_descale, k_descale,
               v_descale, sink, status, max_seqlen_q, max_seqlen_k, softmax_scale, softcap, causal,
               window_left, window_right, num_splits, route, cp_world_size=1, cp_rank=0, cp_tot_seqused_k=None):
    """Everything ``build_params`` reads except the addresses: two calls with equal keys differ only in pointers.
    No tensor contents, identities or version counters enter it."""
    return (q.shape, q.stride(), q.dtype, k.shape, k.stride(), v.stride(), out.stride(), lse is not None,
            cu_seqlens_q.shape[0], cu_seqlens_k is None, seqused_k is None,
            None if block_table is None else (block_table.shape[1], block_table.stride(0)),
            None if q_descale is None else q_descale.stride(), None if k_descale is None else k_descale.stride(),
            None if v_descale is None else v_descale.stride(), sink is None, status is None,
            max_seqlen_q, max_seqlen_k, softmax_scale, softcap, causal, window_left, window_right, num_splits, route,
            cp_world_size, cp_rank)


def build_params(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, q_descale, k_descale,
                 v_descale, sink, status, max_seqlen_q, max_seqlen_k, softmax_scale, softcap, causal,
                 window_left, window_right, num_splits, route, cp_world_size=1, cp_rank=0,
                 cp_tot_seqused_k=None) -> Params:
    p = Params()
    p.struct_bytes, p.abi_version = ctypes.sizeof(Params), ABI_VERSION
    p.q, p.k, p.v, p.out, p.lse = _ptr_of(q), _ptr_of(k), _ptr_of(v), _ptr_of(out), _ptr_of(lse)
    p.cu_seqlens_q, p.cu_seqlens_k = _ptr_of(cu_seqlens_q), _ptr_of(cu_seqlens_k)
    p.seqused_k, p.block_table = _ptr_of(seqused_k), _ptr_of(block_table)
    p.q_descale, p.k_descale, p.v_descale = _ptr_of(q_descale), _ptr_of(k_descale), _ptr_of(v_descale)
    p.sink, p.device_status = _ptr_of(sink), _ptr_of(status)
    p.cp_tot_seqused_k = _ptr_of(cp_tot_seqused_k)
    p.cp_world_size, p.cp_rank = cp_world_size, cp_rank
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    paged = block_table is not None
    if paged:
        p.k_page_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
        p.v_page_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
        p.num_pages, p.page_size, p.total_k = k.shape[0], k.shape[1], 0
        p.max_pages_per_seq, p.block_table_row_stride = block_table.shape[1], block_table.stride(0)
    else:
        p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1)
        p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1)
        p.total_k = k.shape[0]
    p.out_row_stride, p.out_head_stride = out.stride(0), out.stride(1)
    for name, scale in (("q", q_descale), ("k", k_descale), ("v", v_descale)):
        if scale is not None:
            setattr(p, f"{name}_descale_batch_stride", scale.stride(0))
            setattr(p, f"{name}_descale_head_stride", scale.stride(1))
    p.batch, p.total_q = cu_seqlens_q.shape[0] - 1, q.shape[0]
    p.max_seqlen_q, p.max_seqlen_k = max_seqlen_q, max_seqlen_k
    p.num_q_heads, p.num_kv_heads, p.head_dim = q.shape[1], k.shape[-2], q.shape[2]
    p.dtype = 0 if q.dtype == torch.bfloat16 else 1
    p.causal, p.window_left, p.window_right = int(causal), window_left, window_right
    p.return_lse, p.num_splits, p.route, p.sm_count = int(lse is not None), num_splits, route, 0
    p.softmax_scale, p.softcap = softmax_scale, softcap
    return p


def plan(params: Params) -> PlanInfo:
    """Resolve route, split count and scratch size for a call (host only; launches nothing)."""
    info = PlanInfo()
    raise_for_status(load_library().atrex_fa_sm100_plan(ctypes.byref(params), ctypes.byref(info)))
    return info


def prewarm(device=None) -> None:
    """Load the library and set kernel attributes on ``device`` so no first-call work lands in a graph capture."""
    lib = load_library()
    with torch.cuda.device(device):
        raise_for_status(lib.atrex_fa_sm100_prewarm())
        device_status(torch.device("cuda", torch.cuda.current_device()))


_SCHEMA = (
    "fa_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) out, Tensor(b!)? lse, Tensor(c!)? workspace, "
    "Tensor cu_seqlens_q, Tensor? cu_seqlens_k, Tensor? seqused_k, Tensor? block_table, "
    "Tensor? q_descale, Tensor? k_descale, Tensor? v_descale, Tensor? sink, Tensor(d!)? status, "
    "int max_seqlen_q, int max_seqlen_k, float softmax_scale, float softcap, bool causal, "
    "int window_left, int window_right, int num_splits, int route, int cp_world_size=1, int cp_rank=0, "
    "Tensor? cp_tot_seqused_k=None) -> ()"
)
_op_library = torch.library.Library("atrex_sm100", "DEF")
_op_library.define(_SCHEMA)


def _fa_fwd_cuda(q, k, v, out, lse, workspace, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, q_descale,
                 k_descale, v_descale, sink, status, max_seqlen_q, max_seqlen_k, softmax_scale, softcap, causal,
                 window_left, window_right, num_splits, route, cp_world_size=1, cp_rank=0, cp_tot_seqused_k=None):
    params = build_params(q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, q_descale,
                          k_descale, v_descale, sink, status, max_seqlen_q, max_seqlen_k, softmax_scale, softcap,
                          causal, window_left, window_right, num_splits, route, cp_world_size, cp_rank,
                          cp_tot_seqused_k)
    ws_ptr = None if workspace is None else workspace.data_ptr()
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    stream = torch.cuda.current_stream(q.device).cuda_stream
    raise_for_status(load_library().atrex_fa_sm100_forward(ctypes.byref(params), ws_ptr, ws_bytes, stream))


def launch_params(params: Params, workspace, device) -> None:
    """Enqueue a call whose parameter block is already built (eager path: no dispatcher round trip, the block
    that was planned is the block that runs)."""
    ws_ptr = None if workspace is None else workspace.data_ptr()
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    stream = _raw_stream(device)
    status = (_lib or load_library()).atrex_fa_sm100_forward(ctypes.byref(params), ws_ptr, ws_bytes, stream)
    if status:
        raise_for_status(status)


def _raw_stream(device) -> int:
    """cudaStream_t of torch's current stream on ``device`` as an integer."""
    index = device.index
    if _get_raw_stream is not None and index is not None:
        return _get_raw_stream(index)
    return torch.cuda.current_stream(device).cuda_stream


# torch's own fast accessor (no Stream object is built); the public API is the fallback
_get_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _fa_fwd_meta(*args, **kwargs):
    return None


_op_library.impl("fa_fwd", _fa_fwd_cuda, "CUDA")
_op_library.impl("fa_fwd", _fa_fwd_meta, "Meta")

fa_fwd = torch.ops.atrex_sm100.fa_fwd
