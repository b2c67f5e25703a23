"""The compact-sparse-attention oracle against outputs of the reference's own FP32 oracle (tests/golden/qsa_*.npz,
written by tests/golden/make_qsa_golden.py from op_test/nvidia/qsa/test_qsa_sm100.py:154-208)."""

import os

import numpy as np
import pytest

from golden import qsa_cases
from oracle import qsa_oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_output(name):
    bits = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))["out_bf16_bits"]
    return (bits.astype(np.uint32) << 16).view(np.float32)


def run_oracle(case):
    s = case.get("scales", {})
    return qsa_oracle.qsa_compact(case["q"], case["k_cache"], case["v_cache"], case["indexer_block_ids"],
                                  case["query_positions"], case["block_table"], case["token_to_req"],
                                  case["output_gate"], q_scale=s.get("q", 1.0), k_scale=s.get("k_cache", 1.0),
                                  v_scale=s.get("v_cache", 1.0))


@pytest.mark.parametrize("name", sorted(qsa_cases.QSA_CASES))
def test_oracle_matches_reference_outputs(name):
    case = qsa_cases.build(name)
    want = golden_output(name)
    got = run_oracle(case)
    assert got.shape == want.shape
    # both round A and the gated product to BF16: allow one BF16 step where FP32 summation order differs
    diff = np.abs(got - want)
    assert np.all(diff <= 2.0 ** -7 * np.maximum(np.abs(want), 2.0 ** -10)), float(diff.max())
    assert np.mean(diff == 0) > 0.98
    # rows that see nothing (position -1, padding request id) are exactly zero in both
    dead = [r for r, (p, q) in enumerate(zip(case["query_positions"], case["token_to_req"])) if p < 0 or q < 0]
    assert np.all(want[dead] == 0) and np.all(got[dead] == 0)
    assert dead or name == "qsa_bf16_page16"


def test_expansion_rules():
    ids = np.full((4, 512), -1, np.int32)
    ids[1, :2] = [5, 0]
    ids[2, :3] = [7, -1, 2]
    ids[3, :512] = np.arange(512)[::-1]
    tokens, count = qsa_oracle.expand(ids, np.array([-1, 9, 14, 4000]))
    assert count.tolist() == [0, 10, 15, 512 * 4 + 1]
    assert tokens[0].max() == -1
    # position 9: ten visible tokens = two listed blocks (5 -> 20..23, 0 -> 0..3) + the two tokens 8, 9 of block 2
    assert tokens[1][:10].tolist() == [20, 21, 22, 23, 0, 1, 2, 3, 8, 9] and tokens[1][10:].max() == -1
    # a negative id hides its block but keeps its slots; the tail follows the three complete ranks
    assert tokens[2][:15].tolist() == [28, 29, 30, 31, -1, -1, -1, -1, 8, 9, 10, 11, 12, 13, 14]
    # more than 512 visible blocks: only the first 512 ranks, then the tail of the unfinished block
    assert tokens[3][0] == 511 * 4 and tokens[3][2047] == 3 and tokens[3][2048] == 4000 and tokens[3][2049] == -1
    assert qsa_oracle.algorithmic_bytes(ids, np.array([-1, 9, 14, 4000]), 8, 1, 2) == \
        (10 + 15 + 2049) * 1024 + 4 * 8 * 256 * 6 + 4 * (2048 + 12)
