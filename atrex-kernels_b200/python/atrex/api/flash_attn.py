"""vLLM-compatible varlen / paged attention: the public contract and its fail-fast checks.

This is the sm_100a (B200) counterpart of the reference's
python/atrex/api/flash_attn.py.  The two public functions keep the reference's
signature, argument meaning, return convention and exception types
(python/atrex/api/flash_attn.py:280-421); the validation is the reference's
(:98-277) restated for the one target this build serves, ``("nvidia", "sm100")``,
with the features the reference's NVIDIA targets refuse but this build runs:
head_dim 128 and 256, sliding windows, ``s_aux`` sinks in prefill and decode,
softcap, ``num_splits`` up to 256, and context parallelism over the keys
(``cp_world_size``, ``cp_rank``, ``cp_tot_seqused_k``; the reference rejects all
three, python/atrex/api/flash_attn.py:128-135).

Context parallelism: rank ``r`` of ``W`` holds every ``W``-th key of each request
(its local key ``j`` is the request's key ``j * W + r``, the layout serving engines
use for decode context parallelism); ``seqused_k`` gives the LOCAL lengths and
``cp_tot_seqused_k`` the totals.  Query row ``i`` of a request with ``q_len`` rows
sits at position ``tot - q_len + i`` and sees local key ``j`` iff
``j * W + r <= tot - q_len + i``.  Each rank's call returns its partial ``(out,
lse)``; ``atrex.src.nvidia.flash_attn.sm100.sharding`` merges them across ranks.

Conventions: a malformed call raises ``ValueError``; a well-formed call that this
build does not run raises ``NotImplementedError``; the message names the offending
argument.  ``can_use_flash_attn_varlen_func`` runs the same checks and nothing
else: it never loads the native library, allocates or launches.
"""

import contextlib

from atrex.utils.device_target import detect_device_target

_NO_DEVICE_SWITCH = contextlib.nullcontext()

# One target only.  4 is the reference's number for its datacenter-Blackwell
# generation (python/atrex/api/flash_attn.py:6-10 uses {4} for sm103).
_TARGET_FA_VERSIONS = {("nvidia", "sm100"): frozenset({4})}

_HEAD_DIMS = (128, 256)
# E4M3 runs on the single-tile tcgen05 kernel (the mma.sync kernel is BF16 only, and it is the one with softcap).
_FP8_ROUTE_BUILT = True
_MAX_SPLITS = 256

# (argument, value that means "not used", message) for vLLM arguments that no
# ATREX target consumes (python/atrex/api/flash_attn.py:109-151).
_UNSUPPORTED_ARGUMENTS = (
    ("deterministic", False, "Atrex attention does not support deterministic=True"),
    ("scheduler_metadata", None, "Atrex owns its kernel schedule and does not consume vendor scheduler_metadata"),
    ("num_prefill", -1, "Atrex does not consume provider-specific prefill/decode counters (num_prefill)"),
    ("max_seqlen_k_decode", 0, "Atrex does not consume provider-specific prefill/decode counters (max_seqlen_k_decode)"),
    ("max_seqlen_k_prefill", 0, "Atrex does not consume provider-specific prefill/decode counters (max_seqlen_k_prefill)"),
    ("dropout_p", 0, "Atrex attention supports inference without dropout (dropout_p)"),
    ("return_attn_probs", False, "Atrex attention does not return probabilities (return_attn_probs)"),
    ("alibi_slopes", None, "Atrex attention does not support ALiBi (alibi_slopes)"),
    ("q_v", None, "Atrex standard attention does not support auxiliary Q/MLA (q_v)"),
    ("qv", None, "Atrex standard attention does not support auxiliary Q/MLA (qv)"),
    ("output_scale", None, "Atrex attention does not support quantized output (output_scale)"),
    ("mask_mod", None, "Atrex attention does not support custom mask modifiers (mask_mod)"),
    ("aux_tensors", None, "Atrex attention does not support custom mask modifiers (aux_tensors)"),
    ("dynamic_causal", None, "Atrex attention does not support per-sequence causal masks (dynamic_causal)"),
)


def _is_unused(value, neutral):
    if neutral is None:
        return value is None
    if neutral is False:
        return value is False
    return value == neutral


def _validate_out(call, torch):
    """``out`` must look like Q, in the output dtype, with unit stride on the head dimension.

    FP8 inputs produce BF16 (python/atrex/api/flash_attn.py:13-28).
    """
    out, q = call["out"], call["q"]
    if out is None:
        return
    want = torch.bfloat16 if q.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else q.dtype
    if out.shape != q.shape or out.dtype != want or out.device != q.device:
        raise ValueError("out must have Q's shape/device and the backend output dtype")
    if out.stride(-1) != 1 or (out.stride(-2) * out.element_size()) % 16 or (out.stride(0) * out.element_size()) % 16 \
            or out.data_ptr() % 16:
        raise ValueError("out has an unsupported layout")


def _validate_descales(call, torch, batch, num_kv_heads):
    """FP32 ``[batch, num_kv_heads]`` on Q's device, any strides (stride 0 included); BF16 takes none.

    Follows python/atrex/api/flash_attn.py:31-48.
    """
    q = call["q"]
    given = [call[name] for name in ("q_descale", "k_descale", "v_descale")]
    if q.dtype == torch.bfloat16:
        if any(scale is not None for scale in given):
            raise NotImplementedError("BF16 attention does not consume FP8 descales")
        return
    for scale in given:
        if scale is None:
            continue
        if scale.shape != (batch, num_kv_heads) or scale.dtype != torch.float32 or scale.device != q.device:
            raise ValueError("FP8 descales must be float32 [batch,num_kv_heads] on the Q device")


def _validate_context_parallel(call, torch, batch, window):
    """``cp_world_size`` ranks each hold every ``cp_world_size``-th key; see the module docstring."""
    world, rank, total = call["cp_world_size"], call["cp_rank"], call["cp_tot_seqused_k"]
    if not isinstance(world, int) or not isinstance(rank, int) or isinstance(world, bool) or isinstance(rank, bool):
        raise ValueError("cp_world_size and cp_rank must be Python ints")
    if world < 1 or not 0 <= rank < world:
        raise ValueError("cp_rank must lie in [0, cp_world_size) and cp_world_size must be positive")
    if world == 1:
        if total is not None:
            raise ValueError("cp_tot_seqused_k is only meaningful with cp_world_size > 1")
        return
    q = call["q"]
    if total is None:
        raise ValueError("context parallelism (cp_world_size > 1) requires cp_tot_seqused_k")
    if total.shape != (batch,) or total.dtype != torch.int32 or total.device != q.device or total.stride(0) != 1:
        raise ValueError("cp_tot_seqused_k must be a contiguous int32 [batch] on the Q device")
    if call["seqused_k"] is None:
        raise ValueError("context parallelism requires seqused_k (the local key counts)")
    if not call["causal"]:
        raise NotImplementedError("Atrex sm100 context parallelism serves causal attention only (causal)")
    if window[0] >= 0 or window[1] > 0:
        raise NotImplementedError("Atrex sm100 context parallelism does not support a sliding window (window_size)")


def _validate_sm100_call(call, torch, batch, window, softcap):
    """Checks specific to the sm_100a kernels (the reference's per-target block is :51-88)."""
    q, k, v = call["q"], call["k"], call["v"]
    block_table = call["block_table"]
    if q.dtype == torch.float8_e5m2:
        raise NotImplementedError("Atrex sm100 attention supports dtype bfloat16 and float8_e4m3fn, not float8_e5m2")
    sink = call["s_aux"]
    if sink is not None:
        if sink.shape != (q.shape[-2],) or sink.dtype != torch.bfloat16 or sink.device != q.device:
            raise ValueError("s_aux must be BF16 [num_q_heads] on the Q device")
        if sink.stride(0) != 1:
            raise ValueError("s_aux must be contiguous")
    _validate_out(call, torch)
    _validate_descales(call, torch, batch, k.shape[-2])
    if call["num_splits"] > _MAX_SPLITS:
        raise NotImplementedError(f"Atrex sm100 attention supports num_splits <= {_MAX_SPLITS}")
    if softcap < 0:
        raise ValueError("softcap must be nonnegative")
    if block_table is not None:
        page = k.shape[1]
        if page % 64 and page not in (16, 32):
            raise NotImplementedError(
                "Atrex sm100 paged attention requires page_size 16, 32 or a multiple of 64"
            )
    # The kernels move K/V with TMA and Q/O with 16-byte vectors: every stride
    # above the head dimension and every base address must be 16-byte aligned.
    for name, tensor in (("q", q), ("k", k), ("v", v)):
        size = tensor.element_size()
        if tensor.data_ptr() % 16 or any((tensor.stride(d) * size) % 16 for d in range(tensor.ndim - 1)):
            raise NotImplementedError(f"{name} has an unsupported layout: strides and base must be 16-byte aligned")
    for name in ("max_seqlen_q", "max_seqlen_k"):
        if not isinstance(call[name], int):
            raise ValueError(f"{name} must be a Python int")
    if q.shape[0] >= 2**31 or k.shape[0] >= 2**31:
        raise NotImplementedError("Atrex sm100 attention indexes rows and pages with 32 bits")
    if block_table is None and call["cu_seqlens_k"] is None:
        raise NotImplementedError("Atrex sm100 packed K/V requires cu_seqlens_k")
    _validate_context_parallel(call, torch, batch, window)
    if q.dtype == torch.float8_e4m3fn:
        if not _FP8_ROUTE_BUILT:
            raise NotImplementedError("Atrex sm100 attention does not serve float8_e4m3fn yet (BF16 only)")
        if softcap:
            raise NotImplementedError("Atrex sm100 float8_e4m3fn attention does not support softcap")
        scale = call["softmax_scale"]
        if scale is not None and scale <= 0:
            raise NotImplementedError("Atrex sm100 float8_e4m3fn attention requires a positive softmax_scale")


def _validate_flash_attn_call(call):
    """Check one call against the contract without compiling, allocating or launching.

    Returns ``(target, window, softcap)`` as the reference's validator does
    (python/atrex/api/flash_attn.py:98-277).
    """
    import torch

    for name, neutral, message in _UNSUPPORTED_ARGUMENTS:
        if not _is_unused(call[name], neutral):
            raise NotImplementedError(message)

    q, k, v = call["q"], call["k"], call["v"]
    cu_seqlens_q, cu_seqlens_k = call["cu_seqlens_q"], call["cu_seqlens_k"]
    seqused_k, block_table = call["seqused_k"], call["block_table"]

    if (cu_seqlens_k is None) == (seqused_k is None):
        raise ValueError("Provide exactly one of cu_seqlens_k and seqused_k")
    if block_table is not None and seqused_k is None:
        raise ValueError("Paged KV requires seqused_k")
    if q.ndim != 3 or k.ndim != (3 if block_table is None else 4):
        raise ValueError("Expected packed Q and packed or paged K/V")
    if v.ndim != k.ndim:
        raise ValueError("K/V must have the same rank")
    if not (q.device == k.device == v.device):
        raise ValueError("Q/K/V must share one device")
    if not (q.dtype == k.dtype == v.dtype):
        raise NotImplementedError("Atrex attention requires matching Q/K/V dtypes")
    if q.dtype not in (torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
        raise NotImplementedError(f"Unsupported attention dtype {q.dtype}")

    target = detect_device_target(q.device)
    head_dim = q.shape[-1]
    if head_dim not in _HEAD_DIMS or k.shape[-1] != head_dim or v.shape[-1] != head_dim:
        raise NotImplementedError(
            f"Atrex {target.family}/{target.arch} attention requires matching head dimensions in {_HEAD_DIMS}"
        )
    if k.shape[:-1] != v.shape[:-1]:
        raise ValueError("Incompatible K/V dimensions")
    if k.shape[-2] <= 0 or q.shape[-2] % k.shape[-2]:
        raise ValueError("Q heads must be divisible by KV heads")
    if q.shape[-2] <= 0:
        raise ValueError("Q must contain at least one attention head")
    if any(t.stride(-1) != 1 for t in (q, k, v)):
        raise ValueError("Q/K/V head dimensions must be contiguous")
    if q.dtype != torch.bfloat16 and any(t.requires_grad for t in (q, k, v)):
        raise NotImplementedError("Atrex FP8 attention is forward-only")
    if call["num_splits"] < 0:
        raise ValueError("num_splits must be nonnegative")
    if cu_seqlens_q is None:
        raise ValueError("Atrex varlen attention requires cu_seqlens_q")

    for name in ("cu_seqlens_q", "cu_seqlens_k", "seqused_k", "block_table"):
        meta = call[name]
        if meta is None:
            continue
        if meta.device != q.device or meta.dtype != torch.int32:
            raise ValueError(f"{name} must be int32 on the Q device")
        if meta.ndim not in (1, 2) or meta.stride(-1) != 1:
            raise ValueError(f"{name} must have contiguous rows")

    window = (-1, -1) if call["window_size"] is None else tuple(call["window_size"])
    if len(window) != 2:
        raise ValueError("window_size must contain two values")
    window = tuple(-1 if w is None else int(w) for w in window)
    softcap, logits_soft_cap = call["softcap"], call["logits_soft_cap"]
    if logits_soft_cap is not None:
        if softcap not in (0, 0.0, logits_soft_cap):
            raise ValueError("softcap and logits_soft_cap disagree")
        softcap = logits_soft_cap

    key = (target.family, target.arch)
    versions = _TARGET_FA_VERSIONS.get(key)
    if versions is None:
        raise NotImplementedError(
            f"Atrex attention supports only nvidia/sm100 in this build; detected {target.family}/{target.arch}"
        )
    fa_version = call["fa_version"]
    if fa_version is not None and fa_version not in versions:
        listed = ", ".join(str(x) for x in sorted(versions))
        raise NotImplementedError(
            f"Atrex {target.family}/{target.arch} supports fa_version {listed}; received {fa_version}"
        )

    if cu_seqlens_q.ndim != 1:
        raise ValueError("cu_seqlens_q must be one-dimensional")
    batch = cu_seqlens_q.shape[0] - 1
    if batch < 0:
        raise ValueError("Invalid cu_seqlens_q")
    if q.shape[0] and batch == 0:
        raise ValueError("Nonempty Q requires sequence metadata")
    if cu_seqlens_k is not None and cu_seqlens_k.shape != (batch + 1,):
        raise ValueError("cu_seqlens_k must have shape [batch+1]")
    if seqused_k is not None and seqused_k.shape != (batch,):
        raise ValueError("seqused_k must have shape [batch]")
    if block_table is not None and (block_table.ndim != 2 or block_table.shape[0] != batch):
        raise ValueError("block_table must have shape [batch,max_pages]")
    if block_table is not None and k.shape[1] <= 0:
        raise ValueError("Paged K/V requires a positive page size")
    if call["max_seqlen_q"] < 0 or call["max_seqlen_k"] < 0:
        raise ValueError("maximum sequence lengths must be nonnegative")

    _validate_sm100_call(call, torch, batch, window, softcap)
    return target, window, softcap


_TENSOR_ARGUMENTS = ("q", "k", "v", "cu_seqlens_q", "cu_seqlens_k", "seqused_k", "block_table", "out", "q_descale",
                     "k_descale", "v_descale", "s_aux", "cp_tot_seqused_k")
_ALIGNED_ARGUMENTS = ("q", "k", "v", "out")
_VALIDATED_LIMIT = 512
_validated = {}   # call signature -> (window, softcap) of a call that passed _validate_flash_attn_call


def _call_signature(call):
    """Everything the validator reads, as one hashable value, or None when the call is not of the usual form.

    The checks of ``_validate_flash_attn_call`` look at argument VALUES for scalars and at shape, strides, dtype,
    device (plus 16-byte alignment of Q, K, V and out, and ``requires_grad``) for tensors; they never read tensor
    contents.  A serving loop repeats one signature step after step, so a call whose signature already passed
    skips the 60-odd checks.  Tensor identity, version counters and device data never enter the signature.
    """
    try:
        parts = []
        for name, value in call.items():
            if name in _TENSOR_ARGUMENTS and value is not None:
                parts.append((value.shape, value.stride(), value.dtype, value.device, value.requires_grad,
                              value.data_ptr() % 16 if name in _ALIGNED_ARGUMENTS else 0))
            elif name == "window_size" and value is not None:
                parts.append(tuple(value))
            else:
                parts.append(value)
        signature = tuple(parts)
        hash(signature)
        return signature
    except (AttributeError, TypeError, RuntimeError):
        return None


def can_use_flash_attn_varlen_func(
    q,
    k,
    v,
    max_seqlen_q,
    cu_seqlens_q,
    max_seqlen_k,
    cu_seqlens_k=None,
    seqused_k=None,
    q_v=None,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=None,
    softcap=0.0,
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    block_table=None,
    return_softmax_lse=False,
    out=None,
    scheduler_metadata=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    num_splits=0,
    output_scale=None,
    fa_version=None,
    s_aux=None,
    cp_world_size=1,
    cp_rank=0,
    cp_tot_seqused_k=None,
    mask_mod=None,
    aux_tensors=None,
    dynamic_causal=None,
    *,
    qv=None,
    logits_soft_cap=None,
    num_prefill=-1,
    max_seqlen_k_decode=0,
    max_seqlen_k_prefill=0,
):
    """True iff ``flash_attn_varlen_func`` would accept exactly this call.  No side effects."""
    try:
        _validate_flash_attn_call(locals())
    except (AttributeError, ImportError, NotImplementedError, RuntimeError, TypeError, ValueError):
        return False
    return True


def flash_attn_varlen_func(
    q,
    k,
    v,
    max_seqlen_q,
    cu_seqlens_q,
    max_seqlen_k,
    cu_seqlens_k=None,
    seqused_k=None,
    q_v=None,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=None,
    softcap=0.0,
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    block_table=None,
    return_softmax_lse=False,
    out=None,
    scheduler_metadata=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    num_splits=0,
    output_scale=None,
    fa_version=None,
    s_aux=None,
    cp_world_size=1,
    cp_rank=0,
    cp_tot_seqused_k=None,
    mask_mod=None,
    aux_tensors=None,
    dynamic_causal=None,
    *,
    qv=None,
    logits_soft_cap=None,
    num_prefill=-1,
    max_seqlen_k_decode=0,
    max_seqlen_k_prefill=0,
):
    """Run attention on the current stream; return ``out`` or ``(out, lse)``.

    ``lse`` is FP32 ``[num_q_heads, total_q]`` in natural log.  When ``out`` is
    supplied it is written in place and returned.
    """
    call = locals()
    import torch
    from atrex.src.nvidia.flash_attn.sm100.launch import forward

    signature = _call_signature(call)
    known = _validated.get(signature) if signature is not None else None
    if known is None:
        target, window, softcap = _validate_flash_attn_call(call)
        if (target.family, target.arch) != ("nvidia", "sm100"):  # exhaustive with _TARGET_FA_VERSIONS
            raise AssertionError(f"unhandled validated target {target}")
        if signature is not None:
            if len(_validated) >= _VALIDATED_LIMIT:
                _validated.clear()
            _validated[signature] = (window, softcap)
    else:
        window, softcap = known

    # the reference enters the tensors' device around the launch (python/atrex/api/flash_attn.py:395); switching
    # is skipped when that device is current already
    index = q.device.index
    guard = torch.cuda.device(q.device) if index is not None and index != torch.cuda.current_device() \
        else _NO_DEVICE_SWITCH
    with guard:
        output, lse = forward(
            q=q,
            k=k,
            v=v,
            cu_seqlens_q=cu_seqlens_q,
            cu_seqlens_k=cu_seqlens_k,
            seqused_k=seqused_k,
            max_seqlen_q=max_seqlen_q,
            max_seqlen_k=max_seqlen_k,
            page_table=block_table,
            softmax_scale=q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale,
            causal=causal,
            softcap=softcap,
            window_size_left=window[0] if window[0] >= 0 else None,
            window_size_right=window[1] if window[1] >= 0 else None,
            learnable_sink=s_aux,
            out=out,
            return_lse=return_softmax_lse,
            q_descale=q_descale,
            k_descale=k_descale,
            v_descale=v_descale,
            num_splits=num_splits,
            cp_world_size=cp_world_size,
            cp_rank=cp_rank,
            cp_tot_seqused_k=cp_tot_seqused_k,
            layout_token=signature,
        )
    return (output, lse) if return_softmax_lse else output


__all__ = ("can_use_flash_attn_varlen_func", "flash_attn_varlen_func")
