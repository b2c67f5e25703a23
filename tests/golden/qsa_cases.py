"""Seeded inputs of the compact-sparse-attention fixtures (numpy only; rebuilt bit-for-bit from the seed).

Shapes follow the reference's own small cases (op_test/nvidia/qsa/test_qsa_sm100.py:363-436): head_dim 256, one or
two KV heads, GQA ratio 8 or 12, 512 block ids per row drawn without replacement from the blocks a row can see,
positions at page and block boundaries, request ids with padding entries (-1), a page table with holes (-1) and
out-of-pool entries.  Values are FP32 arrays exactly representable in the storage type.
"""

from __future__ import annotations

import os
import sys

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from oracle.fa_oracle import bf16_round, e4m3_round  # noqa: E402

QSA_CASES = {
    # positions cover: nothing visible (-1), less than one block, block / page boundaries, more than 512 blocks
    "qsa_bf16_ratio8": dict(page=128, hkv=1, ratio=8, fp8=False, batch=3, width=40,
                            positions=[-1, 0, 1, 2, 3, 7, 127, 128, 1022, 1023, 2047, 2050, 3001, 4094],
                            bad_requests=[5], holes=True),
    "qsa_fp8_ratio12": dict(page=64, hkv=2, ratio=12, fp8=True, batch=2, width=70,
                            positions=[3, 62, 63, 64, 255, 2048, 4095, 4097], bad_requests=[2], holes=True),
    "qsa_bf16_page16": dict(page=16, hkv=2, ratio=8, fp8=False, batch=2, width=140,
                            positions=[15, 16, 17, 100, 2049, 2200], bad_requests=[], holes=False),
}


def build(name_or_spec, seed=20261110):
    spec = QSA_CASES[name_or_spec] if isinstance(name_or_spec, str) else dict(name_or_spec)
    rng = np.random.Generator(np.random.PCG64(seed))
    page, hkv, ratio, fp8 = spec["page"], spec["hkv"], spec["ratio"], spec["fp8"]
    batch, width = spec["batch"], spec["width"]
    rnd = e4m3_round if fp8 else bf16_round
    pages = batch * width
    heads = hkv * ratio
    positions = np.asarray(spec["positions"], dtype=np.int64)
    rows = positions.shape[0]
    k = rnd(rng.standard_normal((pages, page, hkv, 256), dtype=np.float32) * (1.0 if fp8 else 0.5))
    v = rnd(rng.standard_normal((pages, page, hkv, 256), dtype=np.float32))
    q = rnd(rng.standard_normal((rows, heads, 256), dtype=np.float32) * (1.0 if fp8 else 0.5))
    gate = bf16_round(rng.standard_normal((rows, heads, 256), dtype=np.float32))
    table = rng.permutation(pages).astype(np.int32).reshape(batch, width)
    if spec["holes"]:
        table[:, 3::11] = -1                # unmapped logical pages
        table[:, 5::13] = pages + 2         # entries outside the pool
    ids = np.full((rows, 512), -1, dtype=np.int32)
    for r, p in enumerate(positions.tolist()):
        blocks = max(0, (p + 1) // 4)
        n = min(512, blocks)
        if n:
            ids[r, :n] = rng.permutation(blocks)[:n].astype(np.int32)
            ids[r, : n : 17] = -1 if r % 3 == 2 else ids[r, : n : 17]     # some rows hide a few listed blocks
    req = (np.arange(rows) % batch).astype(np.int32)
    for r in spec["bad_requests"]:
        req[r] = -1
    case = dict(q=q, k_cache=k, v_cache=v, indexer_block_ids=ids, query_positions=positions, block_table=table,
                token_to_req=req, output_gate=gate, fp8=fp8)
    if fp8:
        case["scales"] = dict(q=0.75, k_cache=0.5, v_cache=1.25)
    return case
