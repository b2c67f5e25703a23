"""CPU FP32 restatement of ATREX compact sparse attention (``qsa_compact``).  TEST INFRASTRUCTURE ONLY.

Only the test suite and the benchmark's CPU-baseline leg may import this module; the product path never does.

What it follows (paths relative to the alibaba/atrex-kernels tree):

* ``python/atrex/api/qsa.py:19-47`` (the contract): Q ``[T, Hq, 256]``, K / V caches ``[P, S, Hkv, 256]``, compact
  int32 block ids ``[T, 512]`` (each selected block is four request-local tokens), explicit query positions and
  request ids, a page table, a BF16 output gate; FP8 calls carry ``sm_scale`` (the merged Q.K multiplier) and
  ``v_scale``.
* ``op_test/nvidia/qsa/test_qsa_sm100.py:65-87`` (``expand_torch``): a row at position ``p`` sees ``p + 1`` tokens;
  with ``c = min((p + 1) // 4, 512)`` it attends the four tokens of each of the FIRST ``c`` listed blocks (a
  negative id hides that block) plus the ``(p + 1) % 4`` tokens of the unfinished last block, which start at
  ``((p + 1) // 4) * 4``.
* ``op_test/nvidia/qsa/test_qsa_sm100.py:154-208`` (``oracle``): a token is valid when its row's request id is in
  range, its logical page lies inside the table row and the physical page inside the pool; scores =
  ``(q * sq) . (k * sk) * 256 ** -0.5`` over the valid tokens, softmax with all-hidden rows giving zeros,
  ``A = P (v * sv)`` rounded to BF16, ``out = bf16(A * sigmoid(gate))``.

Parity status: PINNED.  ``tests/golden/qsa_*.npz`` hold outputs of the reference's own ``oracle`` run on CPU
tensors by ``tests/golden/make_qsa_golden.py``; ``tests/test_qsa_oracle.py`` checks this module against them.
"""

from __future__ import annotations

import numpy as np

from .fa_oracle import bf16_round

__all__ = ["expand", "qsa_compact", "gathered_tokens", "algorithmic_bytes"]

TOPK = 512


def expand(block_ids, positions):
    """Token list per row: ``(tokens [T, 2051] int64, -1 where hidden; count [T])`` as ``expand_torch`` builds it."""
    ids = np.asarray(block_ids).astype(np.int64)
    pos = np.asarray(positions).astype(np.int64)
    rows, topk = ids.shape
    cols = np.arange(topk * 4 + 3)
    visible = pos + 1
    complete = np.clip(visible // 4, 0, topk)
    count = complete * 4
    rank = np.minimum(cols // 4, topk - 1)
    selected = ids[:, rank] * 4 + cols % 4
    tail_start = (visible // 4) * 4
    tail_count = visible % 4
    token = np.where(cols[None, :] < count[:, None], selected, tail_start[:, None] + cols[None, :] - count[:, None])
    valid = (cols[None, :] < (count + tail_count)[:, None]) & (token >= 0)
    return np.where(valid, token, -1), count + tail_count


def qsa_compact(q, k_cache, v_cache, block_ids, positions, block_table, token_to_req, gate, *, sm_scale=None,
                v_scale=1.0, q_scale=1.0, k_scale=1.0):
    """FP32 gated sparse attention over value arrays (already decoded from BF16 / E4M3).  ``sm_scale`` is the
    merged multiplier of the public API; when it is None the multiplier is ``256 ** -0.5 * q_scale * k_scale``.
    Returns ``out [T, Hq, 256]`` as FP32 values that are exactly representable in BF16."""
    q = np.asarray(q, np.float32)
    k = np.asarray(k_cache, np.float32)
    v = np.asarray(v_cache, np.float32)
    gate = np.asarray(gate, np.float32)
    table = np.asarray(block_table).astype(np.int64)
    req = np.asarray(token_to_req).astype(np.int64)
    rows, hq, dim = q.shape
    pages, page, hkv, _ = k.shape
    group = hq // hkv
    scale = np.float32(dim ** -0.5 * q_scale * k_scale if sm_scale is None else sm_scale)
    tokens, count = expand(block_ids, positions)
    width = tokens.shape[1]
    out = np.zeros_like(q)
    for r in range(rows):
        tok = tokens[r]
        safe = np.maximum(tok, 0)
        lp, off = safe // page, safe % page
        in_req = 0 <= req[r] < table.shape[0]
        phys = table[np.clip(req[r], 0, table.shape[0] - 1), np.clip(lp, 0, table.shape[1] - 1)]
        valid = (np.arange(width) < count[r]) & (tok >= 0) & in_req & (lp < table.shape[1]) & (phys >= 0) & (phys < pages)
        if not valid.any():
            continue
        sel = np.nonzero(valid)[0]
        keys = k[phys[sel], off[sel]]                      # [n, Hkv, D]
        vals = v[phys[sel], off[sel]] * np.float32(v_scale)
        for h in range(hkv):
            qh = q[r, h * group:(h + 1) * group]           # [G, D]
            s = (qh @ keys[:, h, :].T).astype(np.float32) * scale
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            p /= p.sum(axis=1, keepdims=True, dtype=np.float32)
            a = bf16_round((p @ vals[:, h, :]).astype(np.float32))
            g = gate[r, h * group:(h + 1) * group]
            out[r, h * group:(h + 1) * group] = bf16_round(a * (1.0 / (1.0 + np.exp(-g))).astype(np.float32))
    return out


def gathered_tokens(block_ids, positions):
    """Tokens each row attends (before page-table validity): the unit of the path's algorithmic traffic."""
    return expand(block_ids, positions)[1]


def algorithmic_bytes(block_ids, positions, num_q_heads, num_kv_heads, kv_elem_bytes, head_dim=256):
    """K and V rows every (row, KV head) gathers, the row's Q and gate read and out written, its 512 block ids and
    its position / request id."""
    n = int(np.asarray(gathered_tokens(block_ids, positions)).sum())
    rows = np.asarray(positions).shape[0]
    return (n * num_kv_heads * head_dim * 2 * kv_elem_bytes
            + rows * num_q_heads * head_dim * (kv_elem_bytes + 2 + 2) + rows * (TOPK * 4 + 12))
