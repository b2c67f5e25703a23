"""CPU FP32 restatement of ATREX varlen / paged attention.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the sm_100a kernels.  Only the test suite, the
smoke check and the benchmark's CPU-baseline leg may import it; the product
path never does.

What it follows (paths are relative to the alibaba/atrex-kernels tree):

* ``op_test/utils/flash_attn_contract.py:81-111`` (``reference``): per request,
  gather pages through the block table, widen to FP32, apply the per
  ``[request, kv_head]`` descales to Q, K and V, scores = Q.K^T * softmax_scale,
  bottom-right aligned causal mask (query row ``i`` of a request sees key ``j``
  iff ``j <= i + kv_len - q_len``), natural-log LSE laid out ``[Hq, total_q]``,
  softmax with rows that see no key giving zeros, O laid out ``[total_q, Hq, D]``.
* ``op_test/nvidia/flash_attn/test_flash_attn_sm120.py:316-332`` (contiguous K/V
  packed by ``cu_seqlens_k``), ``:335-357`` (non-causal), ``:360-385`` and
  ``:732-771`` (descales + bottom-right alignment for q_len > 1).
* ``src/nvidia/flash_attn/sm103/prefill_runtime.py:121-141``
  (``_resolve_causal_local_window``): ``causal`` forces right = 0; a window whose
  left + right < 0 is no window; ``(None, 0)`` is plain causal; otherwise key
  ``j`` is visible iff ``i + off - left <= j <= i + off + right`` with
  ``off = kv_len - q_len``.
* ``src/nvidia/flash_attn/sm103/prefill_cutedsl.py:3365-3375,3579-3583`` (sink):
  the per-query-head sink logit joins the softmax denominator un-scaled
  (``row_sum += exp(sink - row_max)``) and is included in the LSE; it adds
  nothing to O.
* softcap: ``scores = cap * tanh(scores * softmax_scale / cap)`` before masking
  (``src/nvidia/flash_attn/sm120/runtime.py:575-577`` delegates this to
  flash-attn-4's ``create_softcap_scoremod``, which is not vendored).

* context parallelism over the keys (``cp_world_size``, ``cp_rank``, ``cp_tot_seqused_k``): the reference
  rejects these arguments (``python/atrex/api/flash_attn.py:128-135``), so the definition is this file's: rank
  ``r`` of ``W`` holds the keys ``r, r + W, r + 2W, ...`` of each request, a query row ``i`` of ``q_len`` rows sits
  at position ``tot - q_len + i`` and sees local key ``j`` iff ``j * W + r <= tot - q_len + i`` (causal only).

Parity status.  Causal / non-causal, paged / contiguous, varlen, GQA, descales
and LSE are PINNED: ``tests/golden`` holds outputs of the reference's own
``reference()`` and ``_fp32_prefill_ref`` run on CPU, and ``tests/test_oracle.py``
checks this module against them.  Sliding window, sinks and softcap are
PARITY UNPINNED: no reference test exercises their numerics (the reference
rejects windows on NVIDIA and never runs a sink or softcap case), so for those
three this file is the definition; context parallelism likewise.
"""

from __future__ import annotations

import math

import numpy as np

__all__ = [
    "attention",
    "resolve_window",
    "bf16_round",
    "e4m3_round",
    "algorithmic_flops",
    "algorithmic_decode_bytes",
]


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round FP32 to the nearest BF16 (ties to even), returned as FP32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def _e4m3_table() -> np.ndarray:
    vals = []
    for code in range(128):
        e, m = code >> 3, code & 7
        if e == 15 and m == 7:
            continue  # NaN encoding
        vals.append((m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7))
    return np.array(vals, dtype=np.float64)


_E4M3 = _e4m3_table()


def e4m3_round(x: np.ndarray) -> np.ndarray:
    """Round FP32 to the nearest E4M3 value (ties to even mantissa, saturating at 448)."""
    x64 = np.asarray(x, dtype=np.float64)
    mag = np.minimum(np.abs(x64), 448.0)
    hi = np.clip(np.searchsorted(_E4M3, mag, side="left"), 0, len(_E4M3) - 1)
    lo = np.clip(hi - 1, 0, len(_E4M3) - 1)
    d_hi, d_lo = np.abs(_E4M3[hi] - mag), np.abs(mag - _E4M3[lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & (lo % 2 == 0))
    out = np.where(pick_lo, _E4M3[lo], _E4M3[hi])
    return (np.sign(x64) * out).astype(np.float32)


def resolve_window(causal, left, right):
    """Canonical (left, right) visibility bounds; ``None`` means unbounded.

    Follows ``_resolve_causal_local_window``
    (src/nvidia/flash_attn/sm103/prefill_runtime.py:121-141).  Negative inputs
    mean "unbounded" as in the public ``window_size=(-1, -1)`` convention.
    """
    left = None if left is None or left < 0 else int(left)
    right = None if right is None or right < 0 else int(right)
    if causal:
        right = 0
    return left, right


def _request_attention(q, k, v, scale, left, right, softcap, sink, key_pos=None, total=None):
    """q [nq,Hq,D], k/v [nk,Hq,D] (already head-expanded, FP32).  Returns O, LSE.

    ``key_pos`` / ``total``: positions of the local keys inside the whole request and its total key count
    (context parallelism); default is keys 0..nk-1 of a request of nk keys."""
    nq, hq, _ = q.shape
    nk = k.shape[0]
    out = np.zeros_like(q)
    lse = np.full((hq, nq), -np.inf, dtype=np.float32)
    off = (nk if total is None else total) - nq
    rows = np.arange(nq)[:, None] + off
    cols = (np.arange(nk) if key_pos is None else np.asarray(key_pos))[None, :]
    hidden = np.zeros((nq, nk), dtype=bool)
    if right is not None:
        hidden |= cols > rows + right
    if left is not None:
        hidden |= cols < rows - left
    for h in range(hq):
        s = (q[:, h, :] @ k[:, h, :].T).astype(np.float32) * np.float32(scale) if nk else np.zeros((nq, 0), np.float32)
        if softcap:
            s = (np.float32(softcap) * np.tanh(s / np.float32(softcap))).astype(np.float32)
        s = np.where(hidden, -np.inf, s)
        m = s.max(axis=1) if nk else np.full((nq,), -np.inf, np.float32)
        if sink is not None:
            m = np.maximum(m, np.float32(sink[h]))
        safe_m = np.where(np.isfinite(m), m, 0.0).astype(np.float32)
        p = np.exp(s - safe_m[:, None]).astype(np.float32)
        denom = p.sum(axis=1, dtype=np.float32)
        if sink is not None:
            denom = denom + np.exp(np.float32(sink[h]) - safe_m)
        with np.errstate(divide="ignore"):
            lse[h] = np.where(denom > 0, safe_m + np.log(denom), -np.inf)
        inv = np.where(denom > 0, 1.0 / np.where(denom > 0, denom, 1.0), 0.0).astype(np.float32)
        if nk:
            out[:, h, :] = (p @ v[:, h, :]) * inv[:, None]
    return out, lse


def attention(
    q,
    k,
    v,
    cu_seqlens_q,
    *,
    seqused_k=None,
    cu_seqlens_k=None,
    block_table=None,
    softmax_scale=None,
    causal=False,
    window=(-1, -1),
    softcap=0.0,
    sink=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    cp_world_size=1,
    cp_rank=0,
    cp_tot_seqused_k=None,
):
    """FP32 attention over packed varlen Q and paged or packed K/V.

    ``q`` is ``[total_q, Hq, D]``.  Paged: ``k``/``v`` are ``[pages, page, Hkv, D]``
    with ``block_table [B, max_pages]`` and ``seqused_k [B]``.  Packed: ``k``/``v``
    are ``[total_k, Hkv, D]`` with ``cu_seqlens_k [B+1]`` (or ``seqused_k`` giving a
    shorter used length per request).  All inputs are value arrays already
    decoded to FP32 (FP8/BF16 storage is the caller's business); descales are
    ``[B, Hkv]``.  Returns ``(O [total_q,Hq,D] f32, LSE [Hq,total_q] f32)``.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    cu_q = [int(x) for x in np.asarray(cu_seqlens_q).tolist()]
    batch = len(cu_q) - 1
    hq, dim = q.shape[1], q.shape[2]
    hkv = k.shape[-2]
    group = hq // hkv
    scale = dim ** -0.5 if softmax_scale is None else softmax_scale
    left, right = resolve_window(causal, window[0], window[1])
    out = np.zeros_like(q)
    lse = np.full((hq, q.shape[0]), -np.inf, dtype=np.float32)
    cu_k = None if cu_seqlens_k is None else [int(x) for x in np.asarray(cu_seqlens_k).tolist()]
    used = None if seqused_k is None else [int(x) for x in np.asarray(seqused_k).tolist()]
    for b in range(batch):
        nq = cu_q[b + 1] - cu_q[b]
        if nq == 0:
            continue
        if block_table is not None:
            length = used[b]
            page = k.shape[1]
            ids = np.asarray(block_table)[b, : math.ceil(length / page)].astype(np.int64)
            kr = k[ids].reshape(-1, hkv, dim)[:length]
            vr = v[ids].reshape(-1, hkv, dim)[:length]
        else:
            start = cu_k[b] if cu_k is not None else 0
            length = used[b] if used is not None else cu_k[b + 1] - cu_k[b]
            kr = k[start : start + length]
            vr = v[start : start + length]
        qr = q[cu_q[b] : cu_q[b + 1]]
        if q_descale is not None:
            qr = qr * np.repeat(np.asarray(q_descale, np.float32)[b], group).reshape(1, hq, 1)
        if k_descale is not None:
            kr = kr * np.asarray(k_descale, np.float32)[b].reshape(1, hkv, 1)
        if v_descale is not None:
            vr = vr * np.asarray(v_descale, np.float32)[b].reshape(1, hkv, 1)
        kr = np.repeat(kr, group, axis=1)
        vr = np.repeat(vr, group, axis=1)
        key_pos = total = None
        if cp_world_size > 1:   # this rank's local key j is the request's key j * W + r; the sink joins on rank 0 only
            key_pos = np.arange(kr.shape[0]) * cp_world_size + cp_rank
            total = int(np.asarray(cp_tot_seqused_k)[b])
        o_b, lse_b = _request_attention(qr.astype(np.float32), kr.astype(np.float32), vr.astype(np.float32),
                                        scale, left, right, softcap,
                                        sink if cp_world_size <= 1 or cp_rank == 0 else None, key_pos, total)
        out[cu_q[b] : cu_q[b + 1]] = o_b
        lse[:, cu_q[b] : cu_q[b + 1]] = lse_b
    return out, lse


def visible_pairs(q_len, kv_len, causal, window=(-1, -1)):
    """Number of (query, key) pairs that are not masked for one request."""
    left, right = resolve_window(causal, window[0], window[1])
    off = kv_len - q_len
    total = 0
    if left is None and right is None:
        return q_len * kv_len
    if left is None and right == 0 and off >= 0:
        return q_len * off + q_len * (q_len + 1) // 2
    for i in range(q_len):
        hi = kv_len - 1 if right is None else min(kv_len - 1, i + off + right)
        lo = 0 if left is None else max(0, i + off - left)
        total += max(0, hi - lo + 1)
    return total


def algorithmic_flops(q_lens, kv_lens, num_q_heads, head_dim, causal, window=(-1, -1)):
    """4 * D * Hq * sum(visible pairs): 2 FLOP per MAC for QK^T and for PV."""
    pairs = sum(visible_pairs(a, b, causal, window) for a, b in zip(q_lens, kv_lens))
    return 4 * head_dim * num_q_heads * pairs


def algorithmic_decode_bytes(q_lens, kv_lens, num_q_heads, num_kv_heads, head_dim, kv_elem_bytes,
                             page_size, window=(-1, -1), q_elem_bytes=None, out_elem_bytes=2):
    """K+V bytes of the keys any query row can see, plus Q read, O write and the page-table entries."""
    q_elem_bytes = kv_elem_bytes if q_elem_bytes is None else q_elem_bytes
    total = 0
    for nq, nk in zip(q_lens, kv_lens):
        left = window[0]
        span = nk if left is None or left < 0 else min(nk, left + nq)
        total += span * num_kv_heads * head_dim * 2 * kv_elem_bytes
        total += 4 * math.ceil(span / page_size) if page_size else 0
        total += nq * num_q_heads * head_dim * (q_elem_bytes + out_elem_bytes)
    return total
