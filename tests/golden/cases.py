"""Seeded input generator shared by the fixture script and the tests (numpy only).

Every case is rebuilt bit-for-bit from its seed (numpy's PCG64 stream is
platform independent), so the fixtures only store reference OUTPUTS.  Values are
held as FP32 arrays that are exactly representable in the storage type (BF16 or
E4M3), which is what both the reference's torch oracle and the kernels consume.
The layout follows ``build_case`` in op_test/utils/flash_attn_contract.py:40-78:
a page pool, a block table that is a random permutation of the pool padded with
-1, and per-request / per-kv-head descales 0.75.., 1.25.., 0.5.. for FP8.
"""

from __future__ import annotations

import math
import os
import sys

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from oracle.fa_oracle import bf16_round, e4m3_round  # noqa: E402

GOLDEN_CASES = {
    # name: dict(page, q_lens, kv_lens, hq, hkv, d, fp8, causal)
    "c1_varlen_causal": dict(page=128, q_lens=[128, 256, 384, 512], kv_lens=[128, 256, 384, 512],
                             hq=16, hkv=2, d=128, fp8=False, causal=True, identity=True, std=1.0),
    "paged_decode_bf16": dict(page=64, q_lens=[1, 1, 1], kv_lens=[70, 129, 300],
                              hq=8, hkv=2, d=128, fp8=False, causal=True),
    "paged_prefill_fp8_hd256": dict(page=128, q_lens=[65, 3], kv_lens=[257, 513],
                                    hq=8, hkv=1, d=256, fp8=True, causal=True),
    "ragged_q_page16": dict(page=16, q_lens=[0, 1, 3, 4, 2], kv_lens=[5, 64, 65, 200, 2],
                            hq=4, hkv=2, d=128, fp8=False, causal=True),
    "noncausal_bf16": dict(page=32, q_lens=[5, 1], kv_lens=[37, 96],
                           hq=4, hkv=1, d=128, fp8=False, causal=False),
    "short_q_fp8_hd128": dict(page=64, q_lens=[4, 2, 1], kv_lens=[100, 64, 300],
                              hq=16, hkv=2, d=128, fp8=True, causal=True),
}


def build(name_or_spec, seed=1729):
    spec = GOLDEN_CASES[name_or_spec] if isinstance(name_or_spec, str) else dict(name_or_spec)
    rng = np.random.Generator(np.random.PCG64(seed))
    page, q_lens, kv_lens = spec["page"], spec["q_lens"], spec["kv_lens"]
    hq, hkv, d, fp8 = spec["hq"], spec["hkv"], spec["d"], spec["fp8"]
    std = spec.get("std", 0.4)
    rnd = e4m3_round if fp8 else bf16_round
    counts = [math.ceil(n / page) for n in kv_lens]
    pages = sum(counts)
    k = rnd(rng.standard_normal((pages, page, hkv, d), dtype=np.float32) * std)
    v = rnd(rng.standard_normal((pages, page, hkv, d), dtype=np.float32) * std)
    table = np.full((len(counts), max(counts)), -1, dtype=np.int32)
    perm = np.arange(pages, dtype=np.int32) if spec.get("identity") else rng.permutation(pages).astype(np.int32)
    o = 0
    for r, n in enumerate(counts):
        table[r, :n] = perm[o:o + n]
        o += n
    cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    q = rnd(rng.standard_normal((int(cu[-1]), hq, d), dtype=np.float32) * std)
    case = dict(q=q, k=k, v=v, block_table=table, cu_seqlens_q=cu,
                seqused_k=np.asarray(kv_lens, dtype=np.int32),
                max_seqlen_q=max(q_lens), max_seqlen_k=max(kv_lens),
                softmax_scale=d ** -0.5, causal=spec["causal"], fp8=fp8,
                q_descale=None, k_descale=None, v_descale=None)
    if fp8:
        b = len(counts)
        head = np.arange(hkv, dtype=np.float32)[None, :] * 0.0625
        for key, base, step in (("q_descale", 0.75, 0.125), ("k_descale", 1.25, 0.125), ("v_descale", 0.5, 0.25)):
            case[key] = (base + step * np.arange(b, dtype=np.float32))[:, None] + head
    return case


def sample_rows(total_q, limit=20):
    """Row subset stored in a fixture (all rows when the case is small)."""
    if total_q <= limit:
        return np.arange(total_q)
    return np.unique(np.concatenate([np.arange(0, total_q, max(1, total_q // limit)), [total_q - 1]]))
