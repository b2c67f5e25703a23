"""KV-cache write path (the step before attention): oracle properties on CPU, bit-exact parity on the GPU.

The cache layouts are the ones the reference's tests read from (op_test/utils/flash_attn_contract.py:40-51,
op_test/nvidia/flash_attn/test_flash_attn_sm120.py:236-244): K|V interleaved pools, token-strided pages, the
head-major cache viewed as [pages, page, heads, dim]; here they are WRITTEN through the native path and then
compared byte for byte with the oracle, and attention over the written cache is compared with the pinned
attention oracle.
"""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from atrex.src.nvidia.flash_attn.sm100 import kv_cache
from oracle import fa_oracle, kv_cache_oracle


def _slots(kv_lens, page, pages, generator, pad_every=0):
    """Slot ids of all tokens of all requests, pages drawn from a random permutation (as a block table would)."""
    counts = [math.ceil(n / page) for n in kv_lens]
    perm = torch.randperm(pages, generator=generator).tolist()
    table, slots, o = [], [], 0
    for n, c in zip(kv_lens, counts):
        mine = perm[o:o + c]
        o += c
        table.append(mine)
        slots += [mine[t // page] * page + t % page for t in range(n)]
    slots = torch.tensor(slots, dtype=torch.int64)
    if pad_every:
        slots[::pad_every] = -1
    return slots, table


def _empty_caches(layout, pages, page, heads, dim, dtype, device, fill):
    def pool(shape):
        t = torch.empty(shape, dtype=torch.uint8 if dtype == torch.float8_e4m3fn else dtype, device=device)
        t.fill_(fill)
        return t.view(dtype) if dtype == torch.float8_e4m3fn else t

    if layout == "plain":
        return pool((pages, page, heads, dim)), pool((pages, page, heads, dim)), None
    if layout == "interleaved":
        cache = pool((pages, 2, page, heads, dim))
        return cache[:, 0], cache[:, 1], cache
    if layout == "strided":
        cache = pool((pages, 2, page * 2, heads, dim))
        return cache[:, 0, ::2], cache[:, 1, ::2], cache
    if layout == "hnd":
        cache = pool((pages, heads, page, 2 * dim))
        return cache[..., :dim].permute(0, 2, 1, 3), cache[..., dim:].permute(0, 2, 1, 3), cache
    raise ValueError(layout)


# ------------------------------------------------------------------ CPU: oracle and host logic

def test_oracle_scatter_and_skip():
    g = torch.Generator().manual_seed(7)
    page, pages, heads, dim = 16, 9, 2, 8
    slots, _ = _slots([20, 5, 33], page, pages, g, pad_every=7)
    tokens = slots.numel()
    key = torch.randn(tokens, heads, dim, generator=g).bfloat16().float().numpy()
    value = torch.randn(tokens, heads, dim, generator=g).bfloat16().float().numpy()
    kc = np.full((pages, page, heads, dim), -7.0, dtype=np.float32)
    vc = np.full_like(kc, -7.0)
    kv_cache_oracle.write_kv_cache(key, value, kc, vc, slots.numpy())
    touched = np.zeros((pages, page), dtype=bool)
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert np.array_equal(kc[s // page, s % page], key[t]) and np.array_equal(vc[s // page, s % page], value[t])
        touched[s // page, s % page] = True
    assert np.all(kc[~touched] == -7.0) and np.all(vc[~touched] == -7.0)


def test_oracle_fp8_matches_torch_conversion():
    """The oracle's quotient + E4M3 rounding equals torch's own float32 -> float8_e4m3fn conversion."""
    g = torch.Generator().manual_seed(11)
    tokens, heads, dim, page = 64, 3, 16, 16
    key = (torch.randn(tokens, heads, dim, generator=g) * 40).bfloat16().float()
    value = (torch.randn(tokens, heads, dim, generator=g) * 600).bfloat16().float()   # saturates
    ks = torch.tensor([0.5, 1.25, 3.0])
    vs = torch.tensor([2.0])
    slots = torch.arange(tokens, dtype=torch.int64)
    kc = np.zeros((tokens // page, page, heads, dim), dtype=np.float32)
    vc = np.zeros_like(kc)
    kv_cache_oracle.write_kv_cache(key.numpy(), value.numpy(), kc, vc, slots.numpy(), ks.numpy(), vs.numpy(), fp8=True)
    want_k = (key / ks[None, :, None]).to(torch.float8_e4m3fn).float().view(-1, page, heads, dim).numpy()
    want_v = (value / vs).clamp(-448, 448).to(torch.float8_e4m3fn).float().view(-1, page, heads, dim).numpy()
    assert np.array_equal(kc, want_k)
    assert np.array_equal(vc, want_v)
    assert np.abs(vc).max() == 448.0


def test_validate_rejects_malformed_calls():
    key = torch.zeros(4, 2, 16, dtype=torch.bfloat16)
    cache = torch.zeros(3, 16, 2, 16, dtype=torch.bfloat16)
    slots = torch.zeros(4, dtype=torch.int64)
    with pytest.raises(ValueError):
        kv_cache.validate(key, key[:3], cache, cache, slots)
    with pytest.raises(ValueError):
        kv_cache.validate(key, key, cache, cache[:, :, :1], slots)
    with pytest.raises(ValueError):
        kv_cache.validate(key, key, cache, cache, slots.int())
    with pytest.raises(NotImplementedError):
        kv_cache.validate(key.float(), key.float(), cache, cache, slots)
    with pytest.raises(NotImplementedError):   # CPU tensors: no fallback path exists
        kv_cache.validate(key, key, cache, cache, slots)
    with pytest.raises(ValueError):
        kv_cache.validate(key, key, cache, cache, slots, k_scale=torch.ones(1))


def test_binding_struct_matches_library():
    import ctypes
    from atrex.src.nvidia.flash_attn.sm100 import runtime
    lib = runtime.load_library()
    kv_cache._bind(lib)
    assert lib.atrex_fa_sm100_kv_write_params_bytes() == ctypes.sizeof(kv_cache.KvWriteParams)
    p = kv_cache.KvWriteParams()
    assert lib.atrex_fa_sm100_kv_cache_write(ctypes.byref(p), None) == 6      # ABI mismatch: struct_bytes is 0
    assert lib.atrex_fa_sm100_kv_cache_write(None, None) == 1


# ------------------------------------------------------------------ GPU: parity through the C ABI

def _run_write(layout, fp8, kv_lens, page, heads, dim, seed, pad_every=0, scales="head", std=None):
    g = torch.Generator().manual_seed(seed)
    pages = sum(math.ceil(n / page) for n in kv_lens) + 2
    slots, table = _slots(kv_lens, page, pages, g, pad_every)
    tokens = slots.numel()
    if std is None:
        std = 3.0 if fp8 else 1.0     # FP8: use the format's range (values up to ~ +-20 before scaling)
    # sources are views of a wider buffer: row strides differ from the logical width
    parent_k = (torch.randn(tokens, heads + 1, dim, generator=g) * std).bfloat16()
    parent_v = (torch.randn(tokens, heads, 2 * dim, generator=g) * std).bfloat16()
    key, value = parent_k[:, :heads], parent_v[..., :dim]
    dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    fill = 0x55 if fp8 else 0                        # untouched bytes must stay as they were
    kc, vc, _ = _empty_caches(layout, pages, page, heads, dim, dtype, "cuda", fill)
    if not fp8:
        kc.fill_(-3.0)
        vc.fill_(-3.0)
    ks = vs = None
    if fp8:
        if scales == "head":
            ks = (0.5 + 0.25 * torch.arange(heads, dtype=torch.float32)).cuda()
            vs = (1.5 - 0.125 * torch.arange(heads, dtype=torch.float32)).cuda()
        elif scales == "tensor":
            ks, vs = torch.tensor([0.75]).cuda(), torch.tensor([2.0]).cuda()
    kv_cache.write_kv_cache(key.cuda(), value.cuda(), kc, vc, slots.cuda(), ks, vs)
    torch.cuda.synchronize()
    init = np.float32(torch.tensor([fill], dtype=torch.uint8).view(dtype).float().item()) if fp8 else np.float32(-3.0)
    want_k = np.full((pages, page, heads, dim), init, dtype=np.float32)
    want_v = np.full_like(want_k, init)
    kv_cache_oracle.write_kv_cache(key.float().numpy(), value.float().numpy(), want_k, want_v, slots.numpy(),
                                   None if ks is None else ks.cpu().numpy(), None if vs is None else vs.cpu().numpy(),
                                   fp8=fp8)
    got_k, got_v = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    assert np.array_equal(got_k, want_k), f"K differs in {(got_k != want_k).sum()} elements"
    assert np.array_equal(got_v, want_v), f"V differs in {(got_v != want_v).sum()} elements"
    return dict(kc=kc, vc=vc, table=table, ks=ks, vs=vs, key=key, value=value)


@pytest.mark.gpu
@pytest.mark.parametrize("layout", ["plain", "interleaved", "strided", "hnd"])
@pytest.mark.parametrize("fp8", [False, True])
def test_write_is_bit_exact(layout, fp8):
    _run_write(layout, fp8, [300, 1, 77, 64], page=64, heads=2, dim=128, seed=3, pad_every=5)


@pytest.mark.gpu
@pytest.mark.parametrize("page,heads,dim", [(16, 1, 256), (32, 8, 128), (128, 3, 64)])
def test_write_shapes(page, heads, dim):
    _run_write("plain", False, [page * 2 + 1, 5], page, heads, dim, seed=5)
    _run_write("interleaved", True, [page * 2 + 1, 5], page, heads, dim, seed=6, scales="tensor")


@pytest.mark.gpu
def test_fp8_quotients_are_correctly_rounded():
    """Every BF16 bit pattern divided by awkward scales (significand all ones, just above a power of two, tiny,
    huge): the stored E4M3 byte equals the oracle's for all of them."""
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16)
    x = bits.view(torch.bfloat16)
    x = x[torch.isfinite(x.float())]
    n = x.numel() // 16 * 16
    x = x[:n]
    scales = torch.tensor([float(np.nextafter(np.float32(1.0), np.float32(0.0))), float(np.nextafter(np.float32(2.0), np.float32(3.0))),
                           3.0, 0.3333333432674408, 1e-3, 977.0, float(np.nextafter(np.float32(0.5), np.float32(0.0))), 1.7],
                          dtype=torch.float32)
    heads = scales.numel()
    key = x.view(-1, 1, 16).expand(-1, heads, 16).contiguous()      # [tokens, heads, 16]: every head sees every value
    tokens = key.shape[0]
    page = 16
    pages = math.ceil(tokens / page)
    kc = torch.zeros(pages, page, heads, 16, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    vc = torch.zeros_like(kc)
    slots = torch.arange(tokens, dtype=torch.int64)
    kv_cache.write_kv_cache(key.cuda(), key.cuda(), kc, vc, slots.cuda(), scales.cuda(), scales.flip(0).contiguous().cuda())
    torch.cuda.synchronize()
    want_k = np.zeros((pages, page, heads, 16), dtype=np.float32)
    want_v = np.zeros_like(want_k)
    kv_cache_oracle.write_kv_cache(key.float().numpy(), key.float().numpy(), want_k, want_v, slots.numpy(),
                                   scales.numpy(), scales.flip(0).numpy(), fp8=True)
    assert np.array_equal(kc.float().cpu().numpy(), want_k)
    assert np.array_equal(vc.float().cpu().numpy(), want_v)


def test_oracle_scales():
    key = np.zeros((5, 3, 8), dtype=np.float32)
    value = np.zeros_like(key)
    key[1, 0, 3] = -896.0
    key[2, 1, 0] = 7.0
    key[4, 1, 1] = 100.0            # padding token: ignored
    value[0, 2, 7] = np.inf
    ks, vs = kv_cache_oracle.kv_scales(key, value, np.array([0, 1, 2, 3, -1]))
    assert ks.tolist() == [2.0, np.float32(7.0) / np.float32(448.0), 1.0] and vs.tolist() == [1.0, 1.0, 1.0]


@pytest.mark.gpu
@pytest.mark.parametrize("heads,dim,tokens", [(2, 128, 777), (8, 128, 4096), (3, 64, 50), (1, 256, 1)])
def test_scales_match_oracle_and_fill_the_range(heads, dim, tokens):
    g = torch.Generator().manual_seed(tokens)
    parent = (torch.randn(tokens, heads + 1, dim, generator=g) * 5).bfloat16()
    key = parent[:, :heads]
    value = (torch.randn(tokens, heads, dim, generator=g) * 0.01).bfloat16()
    if tokens > 10:
        value[:, 0] = 0                       # a head of zeros gets scale 1
    slots = torch.arange(tokens, dtype=torch.int64)
    if tokens > 10:
        slots[::3] = -1                       # padding tokens do not count
        key[0] = 1e30                         # ... even when they are huge (token 0 is padding)
    ks, vs = kv_cache.compute_kv_scales(key.cuda(), value.cuda(), slots.cuda())
    torch.cuda.synchronize()
    want_k, want_v = kv_cache_oracle.kv_scales(key.float().numpy(), value.float().numpy(), slots.numpy())
    assert np.array_equal(ks.cpu().numpy(), want_k) and np.array_equal(vs.cpu().numpy(), want_v)
    # writing with these scales uses the whole E4M3 range and never saturates
    page = 16
    pages = math.ceil(tokens / page)
    kc = torch.zeros(pages, page, heads, dim, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    vc = torch.zeros_like(kc)
    kv_cache.write_kv_cache(key.cuda().contiguous(), value.cuda(), kc, vc, slots.cuda(), ks, vs)
    torch.cuda.synchronize()
    assert float(kc.float().abs().max()) == 448.0


@pytest.mark.gpu
def test_write_empty_and_all_padding():
    kc = torch.full((2, 16, 2, 64), 1.0, dtype=torch.bfloat16, device="cuda")
    vc = kc.clone()
    empty = torch.zeros(0, 2, 64, dtype=torch.bfloat16, device="cuda")
    kv_cache.write_kv_cache(empty, empty, kc, vc, torch.zeros(0, dtype=torch.int64, device="cuda"))
    rows = torch.randn(5, 2, 64, device="cuda").bfloat16()
    kv_cache.write_kv_cache(rows, rows, kc, vc, torch.full((5,), -1, dtype=torch.int64, device="cuda"))
    torch.cuda.synchronize()
    assert bool((kc == 1.0).all()) and bool((vc == 1.0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_slots_past_the_pools_are_skipped(fp8):
    """A slot id at or beyond num_pages * page_size (a corrupt slot mapping) is skipped like a padding token: the
    caches here are the first 3 pages of a 5-page buffer, slots aimed at pages 3 and 4 must leave those pages (and
    everything else) untouched."""
    pages, page, heads, dim = 5, 16, 2, 64
    dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    big_k = torch.full((pages, page, heads, dim), 1.0, device="cuda").to(dtype)
    big_v = big_k.clone()
    kc, vc = big_k[:3], big_v[:3]
    g = torch.Generator().manual_seed(4)
    rows = torch.randn(6, heads, dim, generator=g).bfloat16().cuda()
    loud = rows.clone()
    loud[3:] *= 100.0                                   # the out-of-range tokens carry the largest magnitudes
    slots = torch.tensor([0, 17, 47, 48, 79, 1 << 40], dtype=torch.int64, device="cuda")
    kv_cache.write_kv_cache(loud, loud, kc, vc, slots)
    torch.cuda.synchronize()
    assert bool((big_k[3:].float() == 1.0).all()) and bool((big_v[3:].float() == 1.0).all())
    flat = kc.reshape(-1, heads, dim).float()
    want = rows[:3].float().to(dtype).float() if fp8 else rows[:3].float()
    assert torch.equal(flat[[0, 17, 47]], want)
    untouched = torch.ones(3 * page, dtype=torch.bool, device="cuda")
    untouched[[0, 17, 47]] = False
    assert bool((flat[untouched] == 1.0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_attention_over_written_cache(fp8):
    """Write dense K/V through the native path, then attend: equals the attention oracle over the same rows."""
    import atrex
    kv_lens, q_lens, page, heads, hq, dim = [200, 513], [7, 130], 64, 2, 8, 128
    w = _run_write("interleaved", fp8, kv_lens, page, heads, dim, seed=9, std=1.0)   # unit-scale values: the
    # attention tolerances are absolute
    g = torch.Generator().manual_seed(10)
    dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    q = (torch.randn(sum(q_lens), hq, dim, generator=g) * (0.6 if fp8 else 1.0)).to(dtype)
    width = max(len(t) for t in w["table"])
    table = torch.full((len(kv_lens), width), -1, dtype=torch.int32)
    for r, t in enumerate(w["table"]):
        table[r, :len(t)] = torch.tensor(t, dtype=torch.int32)
    cu = torch.tensor([0, q_lens[0], sum(q_lens)], dtype=torch.int32)
    call = dict(q=q.cuda(), k=w["kc"], v=w["vc"], block_table=table.cuda(), cu_seqlens_q=cu.cuda(),
                seqused_k=torch.tensor(kv_lens, dtype=torch.int32).cuda(), max_seqlen_q=max(q_lens),
                max_seqlen_k=width * page, softmax_scale=dim ** -0.5, causal=True, return_softmax_lse=True)
    qd = None
    if fp8:
        qd = torch.full((len(kv_lens), heads), 0.875, dtype=torch.float32)
        call.update(q_descale=qd.cuda(), k_descale=w["ks"][None, :].expand(len(kv_lens), heads),
                    v_descale=w["vs"][None, :].expand(len(kv_lens), heads))
    out, lse = atrex.flash_attn_varlen_func(**call)
    torch.cuda.synchronize()
    # oracle inputs: what the cache decodes to, request by request, packed
    key, value = w["key"].float().numpy(), w["value"].float().numpy()
    if fp8:
        ks, vs = w["ks"].cpu().numpy(), w["vs"].cpu().numpy()
        key = fa_oracle.e4m3_round(key / ks[None, :, None]) * ks[None, :, None]
        value = fa_oracle.e4m3_round(value / vs[None, :, None]) * vs[None, :, None]
    qf = q.float().numpy() * (0.875 if fp8 else 1.0)
    cu_k = np.concatenate([[0], np.cumsum(kv_lens)])
    want_o, want_l = fa_oracle.attention(qf, key, value, cu.numpy(), cu_seqlens_k=cu_k, softmax_scale=dim ** -0.5,
                                         causal=True)
    tol = 6e-2 if fp8 else 2e-2
    assert np.abs(out.float().cpu().numpy() - want_o).max() <= tol
    got_l = lse.cpu().numpy()
    assert np.all(np.abs(got_l - want_l) <= 1e-3 * np.maximum(1.0, np.abs(want_l)))


@pytest.mark.gpu
def test_write_in_cuda_graph():
    page, heads, dim, tokens = 64, 4, 128, 256
    kc = torch.zeros(8, page, heads, dim, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    key = torch.zeros(tokens, heads, dim, dtype=torch.bfloat16, device="cuda")
    value = torch.zeros_like(key)
    slots = torch.arange(tokens, dtype=torch.int64, device="cuda")
    kv_cache.write_kv_cache(key, value, kc, vc, slots)     # loads the library outside the capture
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        kv_cache.write_kv_cache(key, value, kc, vc, slots)
    for step in range(3):
        key.copy_(torch.randn(tokens, heads, dim, device="cuda").bfloat16())
        value.copy_(key * 2)
        slots.copy_(torch.randperm(8 * page, device="cuda")[:tokens])
        graph.replay()
        torch.cuda.synchronize()
        s = slots.cpu()
        assert torch.equal(kc.view(-1, heads, dim)[s.cuda()], key) and torch.equal(vc.view(-1, heads, dim)[s.cuda()], value)


@pytest.mark.gpu
def test_write_full_size_round_trip():
    """Full-size step (128K new tokens, 8 KV heads, head_dim 128): gather(write(x)) == x, nothing else touched."""
    tokens, heads, dim, page = 131072, 8, 128, 64
    pages = tokens // page + 16
    g = torch.Generator(device="cuda").manual_seed(1)
    key = torch.randn(tokens, heads, dim, device="cuda", generator=g).bfloat16()
    value = torch.randn(tokens, heads, dim, device="cuda", generator=g).bfloat16()
    kc = torch.full((pages, page, heads, dim), 5.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full_like(kc, 5.0)
    slots = torch.randperm(pages * page, device="cuda", generator=g)[:tokens]
    kv_cache.write_kv_cache(key, value, kc, vc, slots)
    torch.cuda.synchronize()
    assert torch.equal(kc.view(-1, heads, dim)[slots], key)
    assert torch.equal(vc.view(-1, heads, dim)[slots], value)
    untouched = torch.ones(pages * page, dtype=torch.bool, device="cuda")
    untouched[slots] = False
    assert bool((kc.view(-1, heads, dim)[untouched] == 5.0).all())
