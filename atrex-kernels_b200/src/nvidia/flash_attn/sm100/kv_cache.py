"""KV-cache write path of the sm_100a attention: ``write_kv_cache`` scatters a step's new K/V rows into the
paged pools ``flash_attn_varlen_func`` reads, optionally quantising BF16 -> FP8 E4M3.

The reference has no writer (its tests fill caches by indexing, op_test/utils/flash_attn_contract.py:40-51);
the argument names and semantics follow the serving engines' reshape-and-cache step so that a caller can swap
it in: ``slot_mapping[t] = page * page_size + row`` (negative: padding token, skipped), FP8 caches store
``e4m3(x / scale)``, and ``scale`` is what the attention call then receives as ``k_descale`` / ``v_descale``
(a per-head ``[num_kv_heads]`` scale expands over the batch with stride 0).

There is no CPU fallback: without the native library the call raises ``RuntimeError``.
"""

from __future__ import annotations

import ctypes

import torch

from . import runtime


class KvWriteParams(ctypes.Structure):
    """Mirror of ``atrex_fa_sm100_kv_write_params`` (include/atrex_fa_sm100.h)."""

    _fields_ = [
        ("struct_bytes", ctypes.c_uint32), ("abi_version", ctypes.c_uint32),
        ("key", ctypes.c_void_p), ("value", ctypes.c_void_p),
        ("key_cache", ctypes.c_void_p), ("value_cache", ctypes.c_void_p),
        ("slot_mapping", ctypes.c_void_p), ("k_scale", ctypes.c_void_p), ("v_scale", ctypes.c_void_p),
        ("key_token_stride", ctypes.c_int64), ("key_head_stride", ctypes.c_int64),
        ("value_token_stride", ctypes.c_int64), ("value_head_stride", ctypes.c_int64),
        ("key_cache_page_stride", ctypes.c_int64), ("key_cache_row_stride", ctypes.c_int64),
        ("key_cache_head_stride", ctypes.c_int64),
        ("value_cache_page_stride", ctypes.c_int64), ("value_cache_row_stride", ctypes.c_int64),
        ("value_cache_head_stride", ctypes.c_int64),
        ("k_scale_head_stride", ctypes.c_int64), ("v_scale_head_stride", ctypes.c_int64),
        ("num_tokens", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("page_size", ctypes.c_int32),
        ("cache_dtype", ctypes.c_int32), ("num_pages", ctypes.c_int32),
    ]


def _bind(lib):
    if getattr(lib, "_atrex_kv_write_bound", False):
        return
    lib.atrex_fa_sm100_kv_write_params_bytes.restype = ctypes.c_size_t
    lib.atrex_fa_sm100_kv_cache_write.restype = ctypes.c_int
    lib.atrex_fa_sm100_kv_cache_write.argtypes = [ctypes.POINTER(KvWriteParams), ctypes.c_void_p]
    lib.atrex_fa_sm100_kv_scales.restype = ctypes.c_int
    lib.atrex_fa_sm100_kv_scales.argtypes = [ctypes.POINTER(KvWriteParams), ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p]
    if lib.atrex_fa_sm100_kv_write_params_bytes() != ctypes.sizeof(KvWriteParams):
        raise RuntimeError("libatrex_fa_sm100.so does not match this Python binding (kv-write struct size)")
    lib._atrex_kv_write_bound = True


def _scale_args(scale, num_kv_heads, device, name):
    if scale is None:
        return None, 0
    if not isinstance(scale, torch.Tensor) or scale.dtype != torch.float32 or scale.device != device:
        raise ValueError(f"{name} must be an FP32 tensor on the cache device")
    if scale.numel() == 1:
        return scale.data_ptr(), 0
    if scale.shape != (num_kv_heads,):
        raise ValueError(f"{name} must have 1 or num_kv_heads elements")
    return scale.data_ptr(), scale.stride(0)


def validate(key, value, key_cache, value_cache, slot_mapping, k_scale=None, v_scale=None):
    """Shape / dtype / layout checks; ``ValueError`` for malformed calls, ``NotImplementedError`` for unsupported."""
    if key.ndim != 3 or value.shape != key.shape:
        raise ValueError("key and value must be [num_tokens, num_kv_heads, head_dim] of one shape")
    if key_cache.ndim != 4 or value_cache.shape != key_cache.shape:
        raise ValueError("key_cache and value_cache must be [num_pages, page_size, num_kv_heads, head_dim] of one shape")
    tokens, heads, dim = key.shape
    if key_cache.shape[2] != heads or key_cache.shape[3] != dim:
        raise ValueError("cache heads / head_dim do not match key")
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise NotImplementedError("key and value must be bfloat16")
    if key_cache.dtype != value_cache.dtype or key_cache.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise NotImplementedError("caches must both be bfloat16 or both float8_e4m3fn")
    if slot_mapping.shape != (tokens,) or slot_mapping.dtype != torch.int64 or slot_mapping.stride(0) != 1:
        raise ValueError("slot_mapping must be a contiguous int64 [num_tokens]")
    if (k_scale is not None or v_scale is not None) and key_cache.dtype != torch.float8_e4m3fn:
        raise ValueError("scales apply to FP8 caches only")
    if not (key.device == value.device == key_cache.device == value_cache.device == slot_mapping.device):
        raise ValueError("all tensors must be on one device")
    if key.device.type != "cuda":
        raise NotImplementedError("Atrex sm100 KV-cache write runs on CUDA devices only")
    fp8 = key_cache.dtype == torch.float8_e4m3fn
    if dim % (16 if fp8 else 8):
        raise NotImplementedError("head_dim must be a multiple of 8 (16 for an FP8 cache)")
    if key.stride(2) != 1 or value.stride(2) != 1 or key_cache.stride(3) != 1 or value_cache.stride(3) != 1:
        raise NotImplementedError("the head dimension must be contiguous")


def write_kv_cache(key, value, key_cache, value_cache, slot_mapping, k_scale=None, v_scale=None) -> None:
    """Scatter ``key`` / ``value`` into the paged caches in place, on the current stream of their device."""
    validate(key, value, key_cache, value_cache, slot_mapping, k_scale, v_scale)
    lib = runtime.load_library()
    _bind(lib)
    tokens, heads, dim = key.shape
    p = KvWriteParams()
    p.struct_bytes, p.abi_version = ctypes.sizeof(KvWriteParams), runtime.ABI_VERSION
    p.key, p.value = key.data_ptr(), value.data_ptr()
    p.key_cache, p.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    p.slot_mapping = slot_mapping.data_ptr()
    p.k_scale, p.k_scale_head_stride = _scale_args(k_scale, heads, key.device, "k_scale")
    p.v_scale, p.v_scale_head_stride = _scale_args(v_scale, heads, key.device, "v_scale")
    p.key_token_stride, p.key_head_stride = key.stride(0), key.stride(1)
    p.value_token_stride, p.value_head_stride = value.stride(0), value.stride(1)
    p.key_cache_page_stride, p.key_cache_row_stride, p.key_cache_head_stride = key_cache.stride()[:3]
    p.value_cache_page_stride, p.value_cache_row_stride, p.value_cache_head_stride = value_cache.stride()[:3]
    p.num_tokens, p.num_kv_heads, p.head_dim, p.page_size = tokens, heads, dim, key_cache.shape[1]
    p.cache_dtype = 1 if key_cache.dtype == torch.float8_e4m3fn else 0
    p.num_pages = key_cache.shape[0]     # slots past the pools are skipped like padding, never written
    with torch.cuda.device(key.device):
        stream = torch.cuda.current_stream(key.device).cuda_stream
        runtime.raise_for_status(lib.atrex_fa_sm100_kv_cache_write(ctypes.byref(p), stream))


def compute_kv_scales(key, value, slot_mapping):
    """Per-KV-head scales for an FP8 E4M3 cache from the rows about to be written: ``(k_scale, v_scale)``, FP32
    ``[num_kv_heads]`` on the device, ``max |x| / 448`` over the non-padding tokens of each head (1.0 for a head
    with no finite non-zero value).  Pass them to ``write_kv_cache`` and, expanded over the batch, to the
    attention call as ``k_descale`` / ``v_descale``."""
    if key.ndim != 3 or value.shape != key.shape:
        raise ValueError("key and value must be [num_tokens, num_kv_heads, head_dim] of one shape")
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise NotImplementedError("key and value must be bfloat16")
    tokens, heads, dim = key.shape
    if slot_mapping.shape != (tokens,) or slot_mapping.dtype != torch.int64 or slot_mapping.stride(0) != 1:
        raise ValueError("slot_mapping must be a contiguous int64 [num_tokens]")
    if not (key.device == value.device == slot_mapping.device):
        raise ValueError("all tensors must be on one device")
    if key.device.type != "cuda":
        raise NotImplementedError("Atrex sm100 KV-cache scales run on CUDA devices only")
    if dim % 8 or key.stride(2) != 1 or value.stride(2) != 1:
        raise NotImplementedError("head_dim must be a contiguous multiple of 8")
    lib = runtime.load_library()
    _bind(lib)
    p = KvWriteParams()
    p.struct_bytes, p.abi_version = ctypes.sizeof(KvWriteParams), runtime.ABI_VERSION
    p.key, p.value, p.slot_mapping = key.data_ptr(), value.data_ptr(), slot_mapping.data_ptr()
    p.key_token_stride, p.key_head_stride = key.stride(0), key.stride(1)
    p.value_token_stride, p.value_head_stride = value.stride(0), value.stride(1)
    p.num_tokens, p.num_kv_heads, p.head_dim, p.page_size = tokens, heads, dim, 1
    scales = torch.empty(2, heads, dtype=torch.float32, device=key.device)
    scratch = torch.empty(2 * heads, dtype=torch.int32, device=key.device)
    with torch.cuda.device(key.device):
        stream = torch.cuda.current_stream(key.device).cuda_stream
        runtime.raise_for_status(lib.atrex_fa_sm100_kv_scales(ctypes.byref(p), scales[0].data_ptr(),
                                                              scales[1].data_ptr(), scratch.data_ptr(), stream))
    return scales[0], scales[1]
