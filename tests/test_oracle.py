"""The CPU oracle against outputs of the reference's own FP32 attention (tests/golden/*.npz)."""

import os

import numpy as np
import pytest

from golden import cases
from oracle import fa_oracle

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _oracle(case, **extra):
    return fa_oracle.attention(
        case["q"], case["k"], case["v"], case["cu_seqlens_q"], seqused_k=case["seqused_k"],
        block_table=case["block_table"], softmax_scale=case["softmax_scale"], causal=case["causal"],
        q_descale=case["q_descale"], k_descale=case["k_descale"], v_descale=case["v_descale"], **extra)


@pytest.mark.parametrize("name", sorted(cases.GOLDEN_CASES))
def test_oracle_matches_reference_outputs(name):
    case = cases.build(name)
    gold = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out, lse = _oracle(case)
    rows = gold["rows"]
    np.testing.assert_allclose(out[rows], gold["out"], atol=2e-6, rtol=1e-5)
    live = np.concatenate([np.arange(case["cu_seqlens_q"][b], case["cu_seqlens_q"][b + 1])
                           for b in range(len(case["seqused_k"]))]).astype(int)
    np.testing.assert_allclose(lse[:, live], gold["lse"][:, live], atol=5e-6, rtol=1e-5)
    if "out_contiguous_ref" in gold.files:
        np.testing.assert_allclose(out[rows], gold["out_contiguous_ref"], atol=2e-6, rtol=1e-5)
        total = np.array([out.astype(np.float64).sum(), np.abs(out.astype(np.float64)).sum(),
                          lse.astype(np.float64).sum()])
        np.testing.assert_allclose(total, gold["checksum"], rtol=1e-6)


def test_packed_kv_equals_identity_pages():
    case = cases.build("c1_varlen_causal")
    out_paged, lse_paged = _oracle(case)
    hkv, d = case["k"].shape[2:]
    k = case["k"].reshape(-1, hkv, d)
    v = case["v"].reshape(-1, hkv, d)
    # identity pages of 128 hold each request back to back only when lengths are page multiples
    cu_k = np.concatenate([[0], np.cumsum(case["seqused_k"])]).astype(np.int32)
    out, lse = fa_oracle.attention(case["q"], k, v, case["cu_seqlens_q"], cu_seqlens_k=cu_k,
                                   softmax_scale=case["softmax_scale"], causal=True)
    np.testing.assert_array_equal(out, out_paged)
    np.testing.assert_array_equal(lse, lse_paged)


def test_window_semantics():
    case = cases.build(dict(page=16, q_lens=[4], kv_lens=[40], hq=2, hkv=1, d=128, fp8=False, causal=True))
    # a left window wider than the sequence is plain causal
    a = _oracle(case)
    b = _oracle(case, window=(1000, 0))
    np.testing.assert_array_equal(a[0], b[0])
    # window (0, 0): each row sees exactly its own diagonal key, so O is that V row and LSE the single score
    out, lse = _oracle(case, window=(0, 0))
    off = 40 - 4
    ids = case["block_table"][0]
    v = case["v"][ids].reshape(-1, 1, 128)[:40]
    k = case["k"][ids].reshape(-1, 1, 128)[:40]
    for i in range(4):
        np.testing.assert_allclose(out[i, 0], v[off + i, 0], atol=1e-6)
        score = float(case["q"][i, 1] @ k[off + i, 0]) * case["softmax_scale"]
        np.testing.assert_allclose(lse[1, i], score, rtol=1e-5, atol=1e-6)


def test_sink_only_changes_normalisation():
    case = cases.build(dict(page=16, q_lens=[3], kv_lens=[20], hq=2, hkv=1, d=128, fp8=False, causal=True))
    out0, lse0 = _oracle(case)
    sink = np.array([0.3, -1.2], dtype=np.float32)
    out1, lse1 = _oracle(case, sink=sink)
    for h in range(2):
        expect_lse = np.logaddexp(lse0[h], sink[h])
        np.testing.assert_allclose(lse1[h], expect_lse, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(out1[:, h], out0[:, h] * np.exp(lse0[h] - expect_lse)[:, None], rtol=1e-5, atol=1e-6)


def test_context_parallel_shards_merge_to_the_unsharded_result():
    """Every W-th key on each rank (local key j = global key j * W + r): the ranks' partial (O, LSE), merged with the
    split-KV algebra, equal the oracle over all keys - for decode (q_len 1), ragged prefill rows, a request whose
    early rows see no key on some ranks, and a sink that must be counted once."""
    rng = np.random.default_rng(7)
    hq, hkv, d, world = 4, 2, 128, 3
    q_lens, kv_lens = [1, 5, 7, 2], [50, 9, 7, 1]
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    q = fa_oracle.bf16_round(rng.standard_normal((cu[-1], hq, d), dtype=np.float32))
    k = fa_oracle.bf16_round(rng.standard_normal((cu_k[-1], hkv, d), dtype=np.float32))
    v = fa_oracle.bf16_round(rng.standard_normal((cu_k[-1], hkv, d), dtype=np.float32))
    sink = np.array([0.5, -0.25, 1.5, 0.0], dtype=np.float32)
    for use_sink in (None, sink):
        full_o, full_l = fa_oracle.attention(q, k, v, cu, cu_seqlens_k=cu_k, causal=True, sink=use_sink)
        parts_o, parts_l = [], []
        for r in range(world):
            ks = np.concatenate([k[cu_k[b]:cu_k[b + 1]][r::world] for b in range(4)])
            vs = np.concatenate([v[cu_k[b]:cu_k[b + 1]][r::world] for b in range(4)])
            local = [len(range(r, n, world)) for n in kv_lens]
            cu_l = np.concatenate([[0], np.cumsum(local)]).astype(np.int32)
            o, l = fa_oracle.attention(q, ks, vs, cu, cu_seqlens_k=cu_l, causal=True, sink=use_sink,
                                       cp_world_size=world, cp_rank=r,
                                       cp_tot_seqused_k=np.array(kv_lens, np.int32))
            parts_o.append(o)
            parts_l.append(l)
        parts_o, parts_l = np.stack(parts_o), np.stack(parts_l)            # [W, T, H, D], [W, H, T]
        with np.errstate(invalid="ignore"):
            lse = np.logaddexp.reduce(parts_l, axis=0)
            w = np.where(np.isfinite(parts_l), np.exp(parts_l - np.where(np.isfinite(lse), lse, 0.0)), 0.0)
        merged = (parts_o * w.transpose(0, 2, 1)[..., None]).sum(axis=0)
        np.testing.assert_allclose(merged, full_o, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(lse, full_l, rtol=1e-5, atol=1e-5)
        # rank 2 holds key 2 of request 2 (7 keys, 7 rows): rows 0 and 1 sit before it and see nothing there
        assert np.all(np.isneginf(parts_l[2][:, cu[2]:cu[2] + 2])) and np.all(parts_o[2][cu[2]:cu[2] + 2] == 0)


def test_rows_without_keys():
    case = cases.build(dict(page=16, q_lens=[5, 2], kv_lens=[3, 0], hq=2, hkv=1, d=128, fp8=False, causal=True))
    out, lse = _oracle(case)
    # request 0: q_len 5 > kv_len 3 -> the first two rows sit before key 0 (bottom-right alignment)
    assert np.all(out[:2] == 0) and np.all(np.isneginf(lse[:, :2]))
    assert np.all(np.isfinite(lse[:, 2:5]))
    assert np.all(out[5:] == 0) and np.all(np.isneginf(lse[:, 5:]))


def test_rounding_helpers():
    x = np.array([1.0, 1.00390625, 1.001953125, 448.0, 500.0, -0.3, 2.0 ** -9 * 1.5, 0.0], dtype=np.float32)
    import torch

    np.testing.assert_array_equal(fa_oracle.bf16_round(x), torch.from_numpy(x).bfloat16().float().numpy())
    y = np.linspace(-460, 460, 20001, dtype=np.float32)
    ref = torch.from_numpy(np.clip(y, -448, 448)).to(torch.float8_e4m3fn).float().numpy()
    np.testing.assert_array_equal(fa_oracle.e4m3_round(y), ref)


def test_work_counters():
    # 4 requests of 128, 256, 384 and 512 tokens, 16 query heads, head_dim 128: 4*128*16*246400 FLOP
    assert fa_oracle.algorithmic_flops([128, 256, 384, 512], [128, 256, 384, 512], 16, 128, True) == 2018508800
    assert fa_oracle.visible_pairs(4, 100, True) == 4 * 96 + 10
    assert fa_oracle.visible_pairs(4, 100, True, (9, 0)) == 40
    nbytes = fa_oracle.algorithmic_decode_bytes([1], [1000], 32, 8, 128, 2, 64)
    assert nbytes == 1000 * 8 * 128 * 4 + 4 * 16 + 32 * 128 * 4
