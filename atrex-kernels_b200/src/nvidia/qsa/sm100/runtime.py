"""Runtime of the sm_100a compact sparse attention: ``forward(...)`` fills the plain-C parameter block of
``include/atrex_qsa_sm100.h`` and calls the native launcher through ctypes on torch's current stream.

Counterpart of the reference's src/nvidia/qsa/sm100/runtime.py and decode_runtime.py (``forward`` with the same
positional arguments, called from python/atrex/api/qsa.py:62-73).  The kernels live in the library the attention
path loads (built ahead of time; a missing library raises ``RuntimeError`` - there is no fallback).  Scratch for
the split combine comes from the torch allocator per call, so a CUDA-graph pool owns it during capture; block
ids, positions, request ids and the page table are read on the device at every launch.
"""

from __future__ import annotations

import ctypes
import threading

import torch

from atrex.src.nvidia.flash_attn.sm100 import runtime as fa_runtime

ABI_VERSION = 1
_ptr, _i64, _i32, _u32, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_float


class Params(ctypes.Structure):
    """Mirror of ``atrex_qsa_sm100_params``; order and types must match the header."""

    _fields_ = (
        [("struct_bytes", _u32), ("abi_version", _u32)]
        + [(n, _ptr) for n in ("q", "k_cache", "v_cache", "block_ids", "query_positions", "block_table",
                               "token_to_req", "output_gate", "out", "device_status")]
        + [(n, _i64) for n in ("q_row_stride", "q_head_stride", "kv_page_stride", "kv_row_stride", "kv_head_stride")]
        + [(n, _i32) for n in ("rows", "num_q_heads", "num_kv_heads", "num_pages", "page_size", "batch", "table_width",
                               "dtype", "positions_are_int64", "num_splits", "sm_count")]
        + [("sm_scale", _f32), ("v_scale", _f32)]
    )


class PlanInfo(ctypes.Structure):
    _fields_ = [("num_splits", _i32), ("kernel_launches", _i32), ("workspace_bytes", ctypes.c_uint64)]


_bound = False


def library():
    global _bound
    lib = fa_runtime.load_library()
    if not _bound:
        lib.atrex_qsa_sm100_abi_version.restype = ctypes.c_int
        lib.atrex_qsa_sm100_params_bytes.restype = ctypes.c_size_t
        lib.atrex_qsa_sm100_plan.restype = ctypes.c_int
        lib.atrex_qsa_sm100_plan.argtypes = [ctypes.POINTER(Params), ctypes.POINTER(PlanInfo)]
        lib.atrex_qsa_sm100_forward.restype = ctypes.c_int
        lib.atrex_qsa_sm100_forward.argtypes = [ctypes.POINTER(Params), ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
        if lib.atrex_qsa_sm100_abi_version() != ABI_VERSION or lib.atrex_qsa_sm100_params_bytes() != ctypes.sizeof(Params):
            raise RuntimeError("libatrex_fa_sm100.so does not match this Python binding (sparse attention block)")
        _bound = True
    return lib


def build_params(q, k, v, ids, pos, table, req, gate, out, sm_scale, v_scale, num_splits=0, status=None) -> Params:
    p = Params()
    p.struct_bytes, p.abi_version = ctypes.sizeof(Params), ABI_VERSION
    p.q, p.k_cache, p.v_cache = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.block_ids, p.query_positions = ids.data_ptr(), pos.data_ptr()
    p.block_table, p.token_to_req = table.data_ptr(), req.data_ptr()
    p.output_gate, p.out = gate.data_ptr(), out.data_ptr()
    p.device_status = None if status is None else status.data_ptr()
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    p.kv_page_stride, p.kv_row_stride, p.kv_head_stride = k.stride(0), k.stride(1), k.stride(2)
    p.rows, p.num_q_heads, p.num_kv_heads = q.shape[0], q.shape[1], k.shape[2]
    p.num_pages, p.page_size = k.shape[0], k.shape[1]
    p.batch, p.table_width = table.shape
    p.dtype = 0 if q.dtype == torch.bfloat16 else 1
    p.positions_are_int64 = int(pos.dtype == torch.int64)
    p.num_splits, p.sm_count = num_splits, 0
    p.sm_scale, p.v_scale = sm_scale, v_scale
    return p


def plan(params: Params) -> PlanInfo:
    info = PlanInfo()
    fa_runtime.raise_for_status(library().atrex_qsa_sm100_plan(ctypes.byref(params), ctypes.byref(info)))
    return info


_LAYOUT_LIMIT = 128
_local = threading.local()


def forward(q, k_cache, v_cache, indexer_block_ids, query_positions, block_table, token_to_req, use_prefill_config,
            output_gate, out=None, *, sm_scale, v_scale, num_splits=0):
    """Enqueue one call on the current stream of ``q``'s device; returns ``out`` (allocated here when None).

    A decode loop repeats one layout (shapes, strides, scales) with fresh addresses: the filled parameter block and
    its planned scratch size are kept per layout and host thread, and only the ten addresses are patched.  No
    tensor contents, identities or version counters enter the key."""
    if out is None:
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    status = fa_runtime.device_status(q.device)
    key = (q.shape, q.stride(), q.dtype, k_cache.shape, k_cache.stride(), block_table.shape, query_positions.dtype,
           sm_scale, v_scale, num_splits, status is None)
    layouts = getattr(_local, "layouts", None)
    if layouts is None:
        layouts = _local.layouts = {}
    entry = layouts.get(key)
    if entry is None:
        params = build_params(q, k_cache, v_cache, indexer_block_ids, query_positions, block_table, token_to_req,
                              output_gate, out, sm_scale, v_scale, num_splits, status)
        entry = (params, plan(params).workspace_bytes)
        if len(layouts) >= _LAYOUT_LIMIT:
            layouts.clear()
        layouts[key] = entry
    else:
        p = entry[0]
        p.q, p.k_cache, p.v_cache = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
        p.block_ids, p.query_positions = indexer_block_ids.data_ptr(), query_positions.data_ptr()
        p.block_table, p.token_to_req = block_table.data_ptr(), token_to_req.data_ptr()
        p.output_gate, p.out = output_gate.data_ptr(), out.data_ptr()
        p.device_status = None if status is None else status.data_ptr()
    params, workspace_bytes = entry
    info = PlanInfo(workspace_bytes=workspace_bytes)
    workspace = torch.empty(info.workspace_bytes, dtype=torch.uint8, device=q.device) if info.workspace_bytes else None
    stream = fa_runtime._raw_stream(q.device)
    status = library().atrex_qsa_sm100_forward(ctypes.byref(params), None if workspace is None else workspace.data_ptr(),
                                               info.workspace_bytes, stream)
    if status:
        fa_runtime.raise_for_status(status)
    return out
