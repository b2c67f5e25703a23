"""Helpers for the GPU parity tests: seeded cases in the cache layouts callers use, and the oracle check.

Layouts follow the reference's case builders (op_test/utils/flash_attn_contract.py:40-78,
op_test/nvidia/flash_attn/test_flash_attn_sm120.py:236-244): K and V as the two
halves of one interleaved pool, token-strided pages, the vLLM head-major cache
viewed as ``[pages, page, Hkv, D]``, a block table that is a view of a wider
parent filled with -1, and a random page permutation.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from oracle import fa_oracle

BF16_O_ATOL = 2e-2     # max-abs on O for BF16 inputs
FP8_O_ATOL = 6e-2      # max-abs on O for E4M3 inputs
LSE_RTOL = 1e-3        # relative on LSE (plus the same absolute floor near zero)


def make_case(page, q_lens, kv_lens, *, hq=8, hkv=2, d=128, fp8=False, layout="plain", seed=1729, std=1.0,
              spare_pages=2, poison_tail=False, device="cuda"):
    """Paged case on ``device``.  ``poison_tail`` fills unused pool rows with NaN (BF16) / 0x7F (E4M3)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    counts = [math.ceil(n / page) for n in kv_lens]
    pages = sum(counts) + spare_pages

    def pool(shape):
        return (torch.randn(shape, generator=g) * std).to(dtype)

    if layout == "plain":
        k, v = pool((pages, page, hkv, d)), pool((pages, page, hkv, d))
    elif layout == "interleaved":
        cache = pool((pages, 2, page, hkv, d))
        k, v = cache[:, 0], cache[:, 1]
    elif layout == "strided":
        cache = pool((pages, 2, page * 2, hkv, d))
        k, v = cache[:, 0, ::2], cache[:, 1, ::2]
    elif layout == "hnd":  # vLLM head-major cache [P, Hkv, page, 2D] viewed as [P, page, Hkv, D]
        cache = pool((pages, hkv, page, 2 * d))
        k, v = cache[..., :d].permute(0, 2, 1, 3), cache[..., d:].permute(0, 2, 1, 3)
    else:
        raise ValueError(layout)
    parent = torch.full((len(counts), max(counts + [1]) + 3), -1, dtype=torch.int32)
    table = parent[:, : max(counts + [1])]
    perm = torch.randperm(pages, generator=g).to(torch.int32)
    o = 0
    for r, n in enumerate(counts):
        table[r, :n] = perm[o:o + n]
        o += n
    if poison_tail:
        used = torch.zeros(pages, page, dtype=torch.bool)
        for r, n in enumerate(kv_lens):
            for j in range(counts[r]):
                used[table[r, j], : min(page, n - j * page)] = True
        if fp8:  # masked writes are not implemented for float8: poke the NaN encoding 0x7F through a byte view
            k.view(torch.uint8)[~used] = 0x7F
            v.view(torch.uint8)[~used] = 0x7F
        else:
            k[~used] = float("nan")
            v[~used] = float("nan")
    cu = torch.zeros(len(q_lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(q_lens, dtype=torch.int64), 0)
    q = pool((int(cu[-1]), hq, d))
    case = dict(q=q, k=k, v=v, block_table=table, cu_seqlens_q=cu,
                seqused_k=torch.tensor(kv_lens, dtype=torch.int32),
                max_seqlen_q=max(q_lens + [0]), max_seqlen_k=max(counts + [1]) * page,
                softmax_scale=d ** -0.5, causal=True,
                q_descale=None, k_descale=None, v_descale=None)
    if fp8:
        b = len(counts)
        head = torch.arange(hkv, dtype=torch.float32)[None, :] * 0.0625
        for key, base, step in (("q_descale", 0.75, 0.125), ("k_descale", 1.25, 0.125), ("v_descale", 0.5, 0.25)):
            case[key] = (base + step * torch.arange(b, dtype=torch.float32))[:, None] + head
    # move to the device preserving views/strides
    dev = {}
    for key, val in case.items():
        if not torch.is_tensor(val):
            dev[key] = val
    if layout == "plain":
        dev["k"], dev["v"] = k.to(device), v.to(device)
    else:
        cache_d = cache.to(device)
        if layout == "interleaved":
            dev["k"], dev["v"] = cache_d[:, 0], cache_d[:, 1]
        elif layout == "strided":
            dev["k"], dev["v"] = cache_d[:, 0, ::2], cache_d[:, 1, ::2]
        else:
            dev["k"], dev["v"] = cache_d[..., :d].permute(0, 2, 1, 3), cache_d[..., d:].permute(0, 2, 1, 3)
    parent_d = parent.to(device)
    dev["block_table"] = parent_d[:, : table.shape[1]]
    for key in ("q", "cu_seqlens_q", "seqused_k", "q_descale", "k_descale", "v_descale"):
        dev[key] = None if case[key] is None else case[key].to(device)
    return dev


def to_numpy(t):
    return None if t is None else t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def oracle_for(case, *, requests=None, window=(-1, -1), softcap=0.0, sink=None, cu_seqlens_k=None):
    """Run the CPU oracle on a device case (optionally only on the listed requests; other rows stay zero)."""
    cu = to_numpy(case["cu_seqlens_q"]).astype(np.int64)
    q = to_numpy(case["q"])
    kwargs = dict(softmax_scale=case["softmax_scale"], causal=case["causal"], window=window, softcap=softcap,
                  sink=None if sink is None else to_numpy(sink))
    paged = case.get("block_table") is not None
    if requests is None:
        requests = range(len(cu) - 1)
    out = np.zeros(q.shape, np.float32)
    lse = np.full((q.shape[1], q.shape[0]), -np.inf, np.float32)
    k_np, v_np = to_numpy(case["k"]), to_numpy(case["v"])
    for b in requests:
        sub_cu = np.array([0, cu[b + 1] - cu[b]], dtype=np.int32)
        descales = {name: None if case.get(name) is None else to_numpy(case[name])[b:b + 1]
                    for name in ("q_descale", "k_descale", "v_descale")}
        if paged:
            o, l = fa_oracle.attention(q[cu[b]:cu[b + 1]], k_np, v_np, sub_cu,
                                       seqused_k=to_numpy(case["seqused_k"])[b:b + 1],
                                       block_table=to_numpy(case["block_table"])[b:b + 1], **descales, **kwargs)
        else:
            ck = to_numpy(cu_seqlens_k if cu_seqlens_k is not None else case["cu_seqlens_k"]).astype(np.int64)
            o, l = fa_oracle.attention(q[cu[b]:cu[b + 1]], k_np[ck[b]:ck[b + 1]], v_np[ck[b]:ck[b + 1]], sub_cu,
                                       cu_seqlens_k=np.array([0, ck[b + 1] - ck[b]], dtype=np.int32),
                                       **descales, **kwargs)
        out[cu[b]:cu[b + 1]] = o
        lse[:, cu[b]:cu[b + 1]] = l
    return out, lse


def compare(actual_out, actual_lse, expect_out, expect_lse, cu, requests=None, *, fp8=False):
    """North-star gate: max-abs on O, relative on LSE, only over rows of the checked requests."""
    cu = np.asarray(cu).astype(np.int64)
    if requests is None:
        requests = range(len(cu) - 1)
    rows = np.concatenate([np.arange(cu[b], cu[b + 1]) for b in requests] + [np.zeros(0, np.int64)]).astype(np.int64)
    a = actual_out.detach().float().cpu().numpy()[rows]
    e = expect_out[rows]
    assert np.isfinite(a).all(), "non-finite values in O"
    err = np.abs(a - e).max() if a.size else 0.0
    assert err <= (FP8_O_ATOL if fp8 else BF16_O_ATOL), f"O max-abs error {err}"
    if actual_lse is not None:
        la = actual_lse.detach().cpu().numpy()[:, rows]
        le = expect_lse[:, rows]
        inf_e = np.isneginf(le)
        assert np.array_equal(np.isneginf(la), inf_e), "LSE -inf pattern differs"
        fin = ~inf_e
        if fin.any():
            lerr = np.abs(la[fin] - le[fin]) / np.maximum(np.abs(le[fin]), 1.0)
            assert lerr.max() <= LSE_RTOL, f"LSE relative error {lerr.max()}"
    return err


def run(case, *, return_lse=True, out=None, **knobs):
    from atrex import flash_attn_varlen_func

    kwargs = dict(case)
    kwargs.update(knobs)
    kwargs.update(return_softmax_lse=return_lse, out=out)
    result = flash_attn_varlen_func(**kwargs)
    return result if return_lse else (result, None)


def check(case, *, requests=None, fp8=False, **knobs):
    """Call the public API and compare with the oracle under the same knobs."""
    out, lse = run(case, **knobs)
    torch.cuda.synchronize()
    window = knobs.get("window_size") or (-1, -1)
    window = tuple(-1 if w is None else w for w in window)
    eo, el = oracle_for(dict(case, causal=knobs.get("causal", case["causal"])), requests=requests,
                        window=window, softcap=knobs.get("softcap", 0.0), sink=knobs.get("s_aux"))
    return compare(out, lse, eo, el, to_numpy(case["cu_seqlens_q"]), requests, fp8=fp8)
