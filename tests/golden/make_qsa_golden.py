"""Regenerates the compact-sparse-attention fixtures from the reference's own FP32 oracle.

    python tests/golden/make_qsa_golden.py /path/to/atrex-kernels

``oracle`` and ``expand_torch`` are taken from op_test/nvidia/qsa/test_qsa_sm100.py (:154-208, :65-87) by source
text - importing that module needs an installed wheel and a GPU - and run on CPU tensors built from the seeded
inputs of ``qsa_cases.py``.  The fixtures hold outputs only (BF16 bit patterns); inputs are rebuilt from seeds.
"""

from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import qsa_cases  # noqa: E402


def _load_functions(ref_root, rel, names):
    tree = ast.parse(open(os.path.join(ref_root, rel)).read())
    ns = {"torch": torch}
    nodes = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert len(nodes) == len(names), [n.name for n in nodes]
    exec(compile(ast.Module(nodes, []), rel, "exec"), ns)
    return [ns[n] for n in names]


def to_torch(case):
    dt = torch.float8_e4m3fn if case["fp8"] else torch.bfloat16
    d = {}
    for key in ("q", "k_cache", "v_cache"):
        d[key] = torch.from_numpy(case[key]).to(dt)
        assert torch.equal(d[key].float(), torch.from_numpy(case[key])), key
    d["output_gate"] = torch.from_numpy(case["output_gate"]).bfloat16()
    for key in ("indexer_block_ids", "query_positions", "block_table", "token_to_req"):
        d[key] = torch.from_numpy(case[key])
    return d


def main(ref_root):
    expand_torch, oracle = _load_functions(ref_root, "op_test/nvidia/qsa/test_qsa_sm100.py", ["expand_torch", "oracle"])
    oracle.__globals__["expand_torch"] = expand_torch
    for name in qsa_cases.QSA_CASES:
        case = qsa_cases.build(name)
        out = oracle(to_torch(case), case.get("scales", {}))
        bits = out.view(torch.int16).numpy().view(np.uint16)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), out_bf16_bits=bits)
        print(name, tuple(out.shape), "abs max", float(out.float().abs().max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_qsa_golden.py <path to an alibaba/atrex-kernels checkout>")
    main(sys.argv[1])
