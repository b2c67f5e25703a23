"""Regenerate tests/golden/*.npz from the reference's own FP32 attention.

Run in a checkout that has the alibaba/atrex-kernels tree available:

    python tests/golden/make_golden.py /path/to/atrex-kernels

It loads ``op_test/utils/flash_attn_contract.py`` by file path (so the
reference's conftest, which wants an installed wheel, is not triggered), feeds
its ``reference(case)`` the seeded CPU inputs from ``cases.py`` and stores the
outputs.  For the contiguous four-request case it also runs ``_fp32_prefill_ref``
from ``op_test/nvidia/flash_attn/test_flash_attn_sm120.py:316-332`` (extracted
by source text, since importing that test module needs a GPU wheel).
The fixtures are outputs only; inputs are rebuilt from seeds.
"""

from __future__ import annotations

import ast
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def _load_contract(ref_root):
    path = os.path.join(ref_root, "op_test", "utils", "flash_attn_contract.py")
    spec = importlib.util.spec_from_file_location("ref_flash_attn_contract", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _load_function(ref_root, rel, name):
    src = open(os.path.join(ref_root, rel)).read()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            ns = {"torch": torch}
            exec(compile(ast.Module([node], []), rel, "exec"), ns)
            return ns[name]
    raise KeyError(name)


def _to_torch(case):
    dt = torch.float8_e4m3fn if case["fp8"] else torch.bfloat16
    t = {}
    for key in ("q", "k", "v"):
        t[key] = torch.from_numpy(case[key]).to(dt)
        assert torch.equal(t[key].float(), torch.from_numpy(case[key])), key
    for key in ("block_table", "cu_seqlens_q", "seqused_k"):
        t[key] = torch.from_numpy(case[key])
    for key in ("q_descale", "k_descale", "v_descale"):
        t[key] = None if case[key] is None else torch.from_numpy(case[key])
    t["softmax_scale"] = case["softmax_scale"]
    t["causal"] = case["causal"]
    return t


def main(ref_root):
    contract = _load_contract(ref_root)
    prefill_ref = _load_function(ref_root, "op_test/nvidia/flash_attn/test_flash_attn_sm120.py", "_fp32_prefill_ref")
    for name in cases.GOLDEN_CASES:
        case = cases.build(name)
        tc = _to_torch(case)
        out, lse = contract.reference(tc)
        rows = cases.sample_rows(out.shape[0])
        # rows of q_len-0 requests are left uninitialised by the reference: none exist in LSE/O slices we keep
        payload = dict(rows=rows, out=out[rows].numpy(), lse=lse.numpy())
        if name == "c1_varlen_causal":
            hkv, d = case["k"].shape[2], case["k"].shape[3]
            kc = torch.cat([tc["k"][tc["block_table"][r, : -(-int(n) // 128)].long()].reshape(-1, hkv, d)[: int(n)]
                            for r, n in enumerate(case["seqused_k"])])
            vc = torch.cat([tc["v"][tc["block_table"][r, : -(-int(n) // 128)].long()].reshape(-1, hkv, d)[: int(n)]
                            for r, n in enumerate(case["seqused_k"])])
            out2 = prefill_ref(tc["q"], kc, vc, tc["cu_seqlens_q"], list(case["seqused_k"]), case["softmax_scale"])
            payload["out_contiguous_ref"] = out2[rows].numpy()
            payload["checksum"] = np.array([out.double().sum().item(), out.double().abs().sum().item(),
                                            lse.double().sum().item()])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **payload)
        print(name, out.shape, "rows kept", len(rows))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to an alibaba/atrex-kernels checkout>")
    main(sys.argv[1])
