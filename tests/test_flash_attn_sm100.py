"""GPU parity tests for atrex.flash_attn_varlen_func on sm_100a, against the CPU oracle.

Modelled on the reference's per-target test modules
(op_test/nvidia/flash_attn/test_flash_attn_sm103.py, test_flash_attn_sm120.py):
seeded random cases through the public API, compared with the FP32 oracle.
Tolerances (tests/fa_testlib.py): BF16 O max-abs <= 2e-2, E4M3 O <= 6e-2, LSE
<= 1e-3 relative.  Sliding window, sinks and softcap have no reference test that
pins their numerics; for them the oracle in oracle/fa_oracle.py is the definition.
"""

import os
import re

import math

import numpy as np
import pytest
import torch

import fa_testlib as T
from golden import cases as golden_cases

pytestmark = pytest.mark.gpu
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(autouse=True)
def _no_device_timeouts():
    yield
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    assert runtime.check_device_status("cuda") == 0, "a kernel's bounded wait expired"


@pytest.fixture(params=["auto", "mma"])
def route(request, monkeypatch):
    """Run a test once with the launcher's own routing (tcgen05 kernel where eligible) and once pinned to the
    mma.sync kernel."""
    from atrex.src.nvidia.flash_attn.sm100 import launch, runtime

    if request.param == "mma":
        monkeypatch.setattr(launch, "DEFAULT_ROUTE", runtime.ROUTE_MMA)
    return request.param


def _planned_route(case, **knobs):
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    out = torch.empty_like(case["q"])
    params = runtime.build_params(case["q"], case["k"], case["v"], out, None, case["cu_seqlens_q"],
                                  case.get("cu_seqlens_k"), case.get("seqused_k"), case.get("block_table"), None,
                                  None, None, None, None, case["max_seqlen_q"], case["max_seqlen_k"],
                                  case["softmax_scale"], 0.0, knobs.get("causal", True), -1, -1, 0, 0)
    return runtime.plan(params).route


def _golden_to_device(case):
    dev = {}
    for key, val in case.items():
        if isinstance(val, np.ndarray):
            t = torch.from_numpy(val)
            if key in ("q", "k", "v"):
                t = t.to(torch.float8_e4m3fn if case["fp8"] else torch.bfloat16)
            dev[key] = t.cuda()
        elif key != "fp8":
            dev[key] = val
    return dev


@pytest.mark.parametrize("name", sorted(golden_cases.GOLDEN_CASES))
def test_golden_fixtures(name):
    """Kernel output against the stored outputs of the reference's own FP32 attention."""
    case = golden_cases.build(name)
    gold = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out, lse = T.run(_golden_to_device(case))
    torch.cuda.synchronize()
    rows = gold["rows"]
    err = np.abs(out.float().cpu().numpy()[rows] - gold["out"]).max()
    assert err <= (T.FP8_O_ATOL if case["fp8"] else T.BF16_O_ATOL), err
    cu = case["cu_seqlens_q"]
    live = np.concatenate([np.arange(cu[b], cu[b + 1]) for b in range(len(cu) - 1)]).astype(int)
    la, le = lse.cpu().numpy()[:, live], gold["lse"][:, live]
    assert (np.abs(la - le) / np.maximum(np.abs(le), 1.0)).max() <= T.LSE_RTOL


@pytest.mark.parametrize("page", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("layout", ["plain", "interleaved", "strided", "hnd"])
def test_decode_q1_layouts(page, layout):
    case = T.make_case(page, [1, 1, 1, 1, 1], [1, 63, 64, 65, 1000], hq=8, hkv=2, layout=layout, poison_tail=True)
    T.check(case)


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (16, 1, 128), (8, 8, 128), (64, 4, 128), (16, 2, 256), (8, 1, 256)])
@pytest.mark.parametrize("q_len", [1, 2, 3, 4])
def test_short_q_gqa(hq, hkv, d, q_len):
    """Q1..Q4 with the GQA shapes of the headline configs (packed rows 4..64)."""
    kv = [300, 17, 2049, 128]
    case = T.make_case(64, [q_len] * 4, kv, hq=hq, hkv=hkv, d=d)
    T.check(case)


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 8, 64])
def test_split_kv(splits):
    """Explicit and automatic split counts, including more splits than some requests have tiles."""
    case = T.make_case(64, [1, 2, 4, 1], [5000, 64, 129, 1], hq=16, hkv=2, poison_tail=True)
    T.check(case, num_splits=splits)


def test_ragged_q_with_empty_requests():
    """cu_seqlens_q = [0,0,1,3,6,10,15]-style raggedness, q_len 0 and kv_len 0 (reference: test_flash_attn_sm103.py:430-441)."""
    case = T.make_case(128, [0, 1, 2, 3, 4, 5, 0, 2], [77, 1, 300, 1000, 129, 640, 50, 0], hq=16, hkv=1, d=256)
    out, lse = T.run(case)
    torch.cuda.synchronize()
    eo, el = T.oracle_for(case)
    T.compare(out, lse, eo, el, T.to_numpy(case["cu_seqlens_q"]))
    # the last request has no keys: zeros and -inf written by the kernel itself
    assert torch.all(out[-2:] == 0) and torch.all(torch.isneginf(lse[:, -2:]))


def test_q_longer_than_kv(route):
    """Bottom-right alignment when q_len > kv_len: leading rows see nothing."""
    case = T.make_case(64, [5, 70], [3, 20], hq=4, hkv=2)
    T.check(case)


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_paged(d, causal, route):
    case = T.make_case(64, [200, 1, 333, 64], [200, 900, 500, 64], hq=8, hkv=2, d=d, std=0.6)
    T.check(case, causal=causal)


@pytest.mark.parametrize("group", [1, 3, 8])
def test_prefill_group_sizes(group, route):
    """Row tiles that straddle query rows when the group does not divide the tile."""
    case = T.make_case(128, [130, 77], [130, 400], hq=2 * group, hkv=2, std=0.6)
    T.check(case)


def test_prefill_packed_kv(route):
    """Contiguous K/V packed by cu_seqlens_k: four requests of 128, 256, 384 and 512 tokens, 16 query / 2 KV heads."""
    from atrex import flash_attn_varlen_func

    lens = [128, 256, 384, 512]
    g = torch.Generator().manual_seed(7)
    total = sum(lens)
    q = torch.randn(total, 16, 128, generator=g).bfloat16().cuda()
    k = torch.randn(total, 2, 128, generator=g).bfloat16().cuda()
    v = torch.randn(total, 2, 128, generator=g).bfloat16().cuda()
    cu = torch.tensor([0, 128, 384, 768, 1280], dtype=torch.int32).cuda()
    out, lse = flash_attn_varlen_func(q, k, v, 512, cu, 512, cu_seqlens_k=cu, causal=True,
                                      softmax_scale=128 ** -0.5, return_softmax_lse=True)
    torch.cuda.synchronize()
    case = dict(q=q, k=k, v=v, cu_seqlens_q=cu, cu_seqlens_k=cu, softmax_scale=128 ** -0.5, causal=True)
    eo, el = T.oracle_for(case)
    T.compare(out, lse, eo, el, [0, 128, 384, 768, 1280])


@pytest.mark.parametrize("window", [(0, 0), (5, 0), (63, 0), (64, 0), (200, 0), (4095, 0), (10, 10), (-1, 7), (30, -1)])
def test_sliding_window(window, route):
    """Parity unpinned by the reference (it rejects windows on NVIDIA): the oracle defines the expected result."""
    case = T.make_case(64, [4, 1, 130, 2], [700, 300, 260, 5000], hq=8, hkv=2, std=0.6)
    causal = window[1] == 0
    T.check(case, causal=causal, window_size=window)
    if window == (4095, 0):
        T.check(case, causal=True, window_size=window, num_splits=4)


def test_sinks_and_lse(route):
    """Per-head sink logits join the denominator un-scaled; split and unsplit paths agree with the oracle."""
    case = T.make_case(128, [4, 4, 1, 100], [3000, 129, 50, 228], hq=16, hkv=1)
    sink = (torch.randn(16, generator=torch.Generator().manual_seed(3))).bfloat16().cuda()
    for splits in (1, 0, 5):
        T.check(case, s_aux=sink, num_splits=splits)
    T.check(case, s_aux=sink, window_size=(127, 0))


def test_sink_with_no_visible_key():
    case = T.make_case(64, [2], [0], hq=4, hkv=1)
    sink = torch.tensor([0.5, -2.0, 0.0, 3.0]).bfloat16().cuda()
    out, lse = T.run(case, s_aux=sink)
    torch.cuda.synchronize()
    assert torch.all(out == 0)
    np.testing.assert_allclose(lse.cpu().numpy(), sink.float().cpu().numpy()[:, None].repeat(2, 1), rtol=1e-3)


@pytest.mark.parametrize("softcap", [5.0, 30.0])
def test_softcap(softcap):
    case = T.make_case(64, [3, 100], [400, 100], hq=8, hkv=2, std=1.5)
    T.check(case, softcap=softcap)
    T.check(dict(case, logits_soft_cap=softcap), softcap=softcap)


def test_out_is_written_in_place_and_inputs_untouched():
    case = T.make_case(64, [1, 4], [500, 80], hq=8, hkv=2)
    before = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in case.items()}
    big = torch.full((5, 16, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    out = big[:, ::2]  # head-strided view: last dim contiguous, 16-byte aligned
    got, _ = T.run(case, out=out)
    torch.cuda.synchronize()
    assert got.data_ptr() == out.data_ptr()
    eo, el = T.oracle_for(case)
    T.compare(got, None, eo, el, T.to_numpy(case["cu_seqlens_q"]))
    assert torch.all(big[:, 1::2] == 7.0), "rows outside the view were written"
    for key, val in before.items():
        if torch.is_tensor(val):
            assert torch.equal(val.view(torch.uint8) if val.dtype == torch.float8_e4m3fn else val,
                               case[key].view(torch.uint8) if val.dtype == torch.float8_e4m3fn else case[key]), key


def test_padding_rows_after_last_request_are_left_alone():
    """vLLM pads q for CUDA graphs: rows past cu_seqlens_q[-1] belong to nobody."""
    case = T.make_case(64, [1, 1], [100, 3000], hq=8, hkv=2)
    q_pad = torch.cat([case["q"], torch.randn(3, 8, 128, device="cuda").bfloat16()])
    out = torch.full_like(q_pad, 9.0)
    for splits in (1, 4):
        got, _ = T.run(dict(case, q=q_pad), out=out, num_splits=splits)
        torch.cuda.synchronize()
        assert torch.all(got[2:] == 9.0)
        eo, el = T.oracle_for(case)
        T.compare(got[:2], None, eo, el, [0, 1, 2])


def test_graph_replay_rereads_metadata():
    """Capture once, then change lengths, page table rows and Q in place (reference: flash_attn_contract.py:125-142)."""
    from atrex import flash_attn_varlen_func

    case = T.make_case(64, [1, 1, 1, 1], [900, 64, 2000, 301], hq=16, hkv=2)
    out = torch.empty_like(case["q"])
    kwargs = dict(case, out=out, return_softmax_lse=True, num_splits=0)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            flash_attn_varlen_func(**kwargs)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_out, g_lse = flash_attn_varlen_func(**kwargs)
    case["seqused_k"].copy_(torch.tensor([10, 1, 1999, 64], dtype=torch.int32))
    case["q"].copy_(torch.randn_like(case["q"].float()).bfloat16())
    case["block_table"][1, 0], case["block_table"][3, 0] = case["block_table"][3, 0].clone(), case["block_table"][1, 0].clone()
    graph.replay()
    torch.cuda.synchronize()
    eo, el = T.oracle_for(case)
    T.compare(g_out, g_lse, eo, el, T.to_numpy(case["cu_seqlens_q"]))


def test_poisoned_scratch_is_never_read():
    """Free a NaN-filled block of the workspace size so the allocator hands it to the next call
    (reference: test_flash_attn_sm103.py:194-206,498-591)."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    case = T.make_case(64, [1, 4, 2], [4000, 10, 0], hq=8, hkv=2)
    args = dict(case)
    out = torch.empty_like(case["q"])
    params = runtime.build_params(case["q"], case["k"], case["v"], out, None, case["cu_seqlens_q"], None,
                                  case["seqused_k"], case["block_table"], None, None, None, None, None,
                                  case["max_seqlen_q"], case["max_seqlen_k"], case["softmax_scale"], 0.0, True,
                                  -1, -1, 16, 0)
    nbytes = runtime.plan(params).workspace_bytes
    assert nbytes > 0
    poison = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")
    del poison
    T.check(args, num_splits=16)


def test_umma_route_is_taken_and_matches_mma_route():
    """The launcher sends BF16 head_dim-128 prefill to the tcgen05 kernel; its result agrees with the mma.sync
    kernel's on the same inputs (both are checked against the oracle elsewhere)."""
    from atrex.src.nvidia.flash_attn.sm100 import launch, runtime

    case = T.make_case(64, [700, 33, 256, 1], [900, 33, 1000, 77], hq=16, hkv=2, std=0.6, poison_tail=True)
    assert _planned_route(case) == runtime.ROUTE_UMMA
    a, la = T.run(case)
    launch.DEFAULT_ROUTE = runtime.ROUTE_MMA
    try:
        b, lb = T.run(case)
    finally:
        launch.DEFAULT_ROUTE = runtime.ROUTE_AUTO
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max().item() <= T.BF16_O_ATOL
    assert torch.allclose(la, lb, rtol=1e-3, atol=1e-3)
    eo, el = T.oracle_for(case)
    T.compare(a, la, eo, el, T.to_numpy(case["cu_seqlens_q"]))


@pytest.mark.parametrize("page,layout", [(16, "plain"), (32, "interleaved"), (64, "hnd"), (128, "strided"), (256, "plain")])
def test_umma_prefill_page_sizes_and_layouts(page, layout):
    case = T.make_case(page, [300, 129], [300, 1500], hq=8, hkv=1, layout=layout, std=0.6, poison_tail=True)
    T.check(case)


def test_umma_prefill_long_causal():
    """Several row tiles per request and many KV tiles; oracle on the whole (small-head) case."""
    case = T.make_case(64, [2048, 513], [2048, 3000], hq=4, hkv=1, std=0.5)
    T.check(case)


@pytest.mark.parametrize("page", [16, 64, 128])
def test_fp8_prefill_hd256(page):
    """E4M3 inputs with per-(request, KV head) descales, BF16 output (head_dim 256, 12 query heads on 1 KV
    head, cached prefix)."""
    case = T.make_case(page, [300, 70, 1, 513], [300, 900, 64, 513], hq=12, hkv=1, d=256, fp8=True, std=0.8,
                       poison_tail=True)
    T.check(case, fp8=True)


@pytest.mark.parametrize("d,fp8,hq,hkv", [(256, False, 24, 2), (128, True, 12, 1), (256, True, 24, 2), (128, True, 3, 1),
                                          (128, True, 10, 2)])
def test_q_rows_copied_by_the_steward_warp(d, fp8, hq, hkv):
    """GQA groups that do not tile 128 rows as one TMA box (12, 3, 5): warp 11 of the single-tile kernel copies the
    item's Q rows into the swizzled tile one item ahead, one, two or four rows per warp-wide copy depending on the
    row size (512 / 256 / 128 bytes).  Empty requests, a request of one row, many row tiles per request (several
    items per CTA: the two item slots wrap), zeros past a request's rows; oracle on every request."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    case = T.make_case(64, [0, 5, 1400, 130, 0, 1], [40, 700, 1400, 1000, 0, 9], hq=hq, hkv=hkv, d=d, fp8=fp8,
                       std=0.6, poison_tail=True, seed=d + hq)
    assert _planned_route(case) == runtime.ROUTE_UMMA     # head_dim 256 or E4M3: the single-tile tcgen05 kernel
    T.check(case, fp8=fp8)


def test_fp8_descales_matter_and_are_reread():
    """A non-unit descale must change the result, and a descale mutated in place between calls must be read
    again (reference: op_test/ppu/flash_attn/test_flash_attn_zwm890p.py:268-309)."""
    case = T.make_case(128, [40, 200], [400, 200], hq=8, hkv=2, d=256, fp8=True, std=0.8)
    T.check(case, fp8=True)
    base, _ = T.run(case)
    with torch.inference_mode():
        case["v_descale"].mul_(2.0)
        case["k_descale"][0, 1] = 0.3
    T.check(case, fp8=True)
    again, _ = T.run(case)
    torch.cuda.synchronize()
    assert not torch.allclose(base.float(), again.float(), atol=1e-2)
    # broadcast (stride-0) descales are accepted without copying
    flat = dict(case, q_descale=torch.full((1, 1), 0.5, device="cuda").expand(2, 2),
                k_descale=torch.full((1, 1), 1.5, device="cuda").expand(2, 2),
                v_descale=torch.full((1, 1), 0.75, device="cuda").expand(2, 2))
    T.check(flat, fp8=True)


def test_fp8_short_q_and_window_sink():
    case = T.make_case(64, [1, 4, 2], [700, 64, 3000], hq=16, hkv=2, d=256, fp8=True, std=0.8)
    T.check(case, fp8=True)
    sink = torch.randn(16, generator=torch.Generator().manual_seed(9)).bfloat16().cuda()
    T.check(case, fp8=True, s_aux=sink, window_size=(511, 0))


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_fp8_decode_with_splits(d, splits):
    """FP8 short-query calls run on the single-tile tcgen05 kernel, with or without split-KV."""
    case = T.make_case(64, [1, 4, 2, 1], [3000, 64, 700, 1], hq=16, hkv=2, d=d, fp8=True, std=0.8, poison_tail=True)
    T.check(case, fp8=True, num_splits=splits)


def test_fp8_is_rejected_where_no_kernel_serves_it():
    from atrex import can_use_flash_attn_varlen_func, flash_attn_varlen_func

    case = T.make_case(64, [4], [100], hq=8, hkv=2, d=128, fp8=True)
    assert not can_use_flash_attn_varlen_func(**case, softcap=5.0)
    with pytest.raises(NotImplementedError, match="softcap"):
        flash_attn_varlen_func(**case, softcap=5.0)


@pytest.mark.parametrize("hq,hkv,q_len", [(64, 4, 4), (24, 2, 3), (32, 2, 2), (40, 8, 5)])
@pytest.mark.parametrize("splits", [0, 1, 5])
def test_bf16_wide_short_q_on_tcgen05(hq, hkv, q_len, splits):
    """17..128 packed rows per KV head (speculative decode, wide GQA): single-tile tcgen05 kernel, any group."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    case = T.make_case(128, [q_len, 1, q_len, q_len], [5000, 300, 128, 2100], hq=hq, hkv=hkv, poison_tail=True)
    assert _planned_route(case) == runtime.ROUTE_UMMA
    sink = torch.randn(hq, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    T.check(case, num_splits=splits)
    T.check(case, num_splits=splits, s_aux=sink, window_size=(1023, 0))


def test_baseline_decode_config_subsample():
    """Decode batch of 64 requests, 32 query / 8 KV heads, head_dim 128, page 64, KV lengths uniform in
    [1024, 16384]; oracle on 6 requests."""
    rng = np.random.default_rng(1729)
    kv = rng.integers(1024, 16385, size=64).tolist()
    case = T.make_case(64, [1] * 64, kv, hq=32, hkv=8, spare_pages=16)
    T.check(case, requests=[0, 7, 21, 40, 63, int(np.argmax(kv))])


def test_baseline_spec_decode_config_subsample():
    """Speculative decode: 4 query tokens, 64 query / 4 KV heads, page 128, 32768 keys, window (4095, 0), sinks and
    LSE, at a batch of 6; oracle on two requests."""
    case = T.make_case(128, [4] * 6, [32768] * 6, hq=64, hkv=4, spare_pages=4)
    sink = torch.randn(64, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    T.check(case, requests=[0, 5], window_size=(4095, 0), s_aux=sink)


def test_linearity_in_v_at_full_size():
    """Size-independent property: attention is linear in V, so O(V1 + V2) = O(V1) + O(V2) at a decode batch
    too large for the oracle."""
    rng = np.random.default_rng(3)
    kv = rng.integers(1024, 8193, size=32).tolist()
    case = T.make_case(64, [1] * 32, kv, hq=32, hkv=8, std=0.5)
    v1 = case["v"]
    v2 = torch.randn_like(v1.float()).mul_(0.5).bfloat16()
    o1, l1 = T.run(case)
    o2, l2 = T.run(dict(case, v=v2))
    o12, l12 = T.run(dict(case, v=(v1.float() + v2.float()).bfloat16()))
    torch.cuda.synchronize()
    assert torch.equal(l1, l2) and torch.equal(l1, l12)
    assert (o12.float() - (o1.float() + o2.float())).abs().max().item() <= 3e-2


# ------------------------------------------------------------------ cross-kernel and operational checks
def test_prefill_last_row_equals_decode_at_full_length():
    """Size-independent property at lengths too large for the oracle: the last query row of a causal prefill
    (tcgen05 kernel) sees exactly the keys a Q1 decode call (mma.sync split-KV kernel + combine) sees."""
    from atrex import flash_attn_varlen_func

    lens = [16384, 9000, 4097]
    case = T.make_case(64, lens, lens, hq=32, hkv=8, std=0.7, spare_pages=4)
    out_p, lse_p = T.run(case)
    cu = T.to_numpy(case["cu_seqlens_q"])
    last = torch.tensor([int(cu[i + 1]) - 1 for i in range(len(lens))], device="cuda")
    decode = dict(case, q=case["q"][last].contiguous(), max_seqlen_q=1,
                  cu_seqlens_q=torch.arange(len(lens) + 1, dtype=torch.int32, device="cuda"))
    out_d, lse_d = T.run(decode)
    torch.cuda.synchronize()
    assert (out_p[last].float() - out_d.float()).abs().max().item() <= T.BF16_O_ATOL
    assert torch.allclose(lse_p[:, last], lse_d, rtol=1e-3, atol=1e-3)


def test_baseline_multi_gpu_prefill_shape_subsample():
    """Full-length prefill (query length = KV length) with 64 query / 8 KV heads, head_dim 128, page 64 on a few
    requests; oracle on the shortest one (the others are covered by the cross-kernel property above)."""
    lens = [1024, 6000, 2500]
    case = T.make_case(64, lens, lens, hq=64, hkv=8, std=0.7)
    T.check(case, requests=[0])


@pytest.mark.parametrize("kind", ["umma2", "umma1_fp8", "umma1_splits"])
def test_graph_replay_on_tcgen05_routes(kind):
    """Capture once; then change lengths, Q and (FP8) descales in place and replay: everything is re-read on the
    device (reference: op_test/utils/flash_attn_contract.py:125-142, test_flash_attn_zwm890p.py:884-905)."""
    from atrex import flash_attn_varlen_func

    if kind == "umma2":
        case, extra, fp8 = T.make_case(64, [300, 150], [700, 150], hq=8, hkv=2, std=0.6), {}, False
    elif kind == "umma1_fp8":
        case, extra, fp8 = T.make_case(128, [300, 4], [700, 900], hq=12, hkv=1, d=256, fp8=True, std=0.8), {}, True
    else:
        case, extra, fp8 = T.make_case(128, [4, 4, 2], [3000, 500, 128], hq=64, hkv=4), dict(num_splits=3), False
    out = torch.empty(case["q"].shape, dtype=torch.bfloat16, device="cuda")
    kwargs = dict(case, out=out, return_softmax_lse=True, **extra)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            flash_attn_varlen_func(**kwargs)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_out, g_lse = flash_attn_varlen_func(**kwargs)
    q_lens = case["cu_seqlens_q"][1:] - case["cu_seqlens_q"][:-1]
    case["seqused_k"].copy_(torch.maximum(case["seqused_k"] - 37, q_lens))
    if fp8:
        with torch.inference_mode():
            case["k_descale"].mul_(0.5)
            case["v_descale"].add_(0.25)
    else:
        case["q"].copy_(torch.randn_like(case["q"].float()).mul_(0.6).bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    eo, el = T.oracle_for(case)
    T.compare(g_out, g_lse, eo, el, T.to_numpy(case["cu_seqlens_q"]), fp8=fp8)


def test_scratch_is_call_local():
    """Repeated calls of several shapes keep allocated memory flat: scratch comes from the allocator per call and
    nothing is cached per layer (reference: op_test/utils/flash_attn_contract.py:145-175)."""
    from atrex import flash_attn_varlen_func

    shapes = [T.make_case(64, [1] * 8, [2000] * 8, hq=32, hkv=8),
              T.make_case(64, [300, 100], [300, 400], hq=8, hkv=2),
              T.make_case(128, [4] * 4, [3000] * 4, hq=64, hkv=4)]
    calls = [dict(c, out=torch.empty_like(c["q"]), return_softmax_lse=False) for c in shapes]
    for kw in calls:
        for _ in range(3):
            flash_attn_varlen_func(**kw)
    torch.cuda.synchronize()
    baseline = torch.cuda.memory_allocated()
    for _ in range(50):
        for kw in calls:
            flash_attn_varlen_func(**kw)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() <= baseline + 256 * 1024


def test_custom_op_path_matches_the_eager_path():
    """Eager calls go straight to the C ABI; under a tracer the same call is the operator atrex_sm100::fa_fwd.
    Both enqueue the same kernels: identical output for a decode and a prefill case."""
    from atrex import flash_attn_varlen_func
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    for case in (T.make_case(64, [1] * 4, [3000, 17, 640, 2049], hq=32, hkv=8),
                 T.make_case(64, [300, 100], [300, 400], hq=8, hkv=2)):
        out, lse = flash_attn_varlen_func(**case, return_softmax_lse=True)
        out2, lse2 = torch.empty_like(out), torch.empty_like(lse)
        args = (case["q"], case["k"], case["v"], out2, lse2, case["cu_seqlens_q"], None, case["seqused_k"],
                case["block_table"], None, None, None, None, runtime.device_status(out.device),
                case["max_seqlen_q"], case["max_seqlen_k"], case["softmax_scale"], 0.0, True, -1, -1, 0,
                runtime.ROUTE_AUTO)
        info = runtime.plan(runtime.build_params(*args))
        ws = torch.empty(max(1, info.workspace_bytes), dtype=torch.uint8, device=out.device)
        torch.ops.atrex_sm100.fa_fwd(*args[:5], ws, *args[5:])
        torch.cuda.synchronize()
        assert torch.equal(out, out2) and torch.equal(lse, lse2)


def test_decode_context_parallel_merge_of_two_shards():
    """Decode context parallelism emulated on one GPU: every request's pages are dealt alternately to two shards,
    each shard is attended on its own (with LSE) and the two (O, LSE) pairs are merged the way
    sharding.gather_context_parallel merges ranks; equals attention over the whole cache."""
    from atrex import flash_attn_varlen_func
    from atrex.src.nvidia.flash_attn.sm100 import sharding

    page = 64
    kv_lens = [1000, 64, 333, 5000, 1]
    case = T.make_case(page, [1] * len(kv_lens), kv_lens, hq=32, hkv=8)
    full_o, full_l = flash_attn_varlen_func(**case, return_softmax_lse=True)
    table = case["block_table"].cpu()
    outs, lses = [], []
    for shard in range(2):
        width = (table.shape[1] + 1) // 2
        sub = torch.full((len(kv_lens), max(width, 1)), -1, dtype=torch.int32)
        used = []
        for b, n in enumerate(kv_lens):
            pages = math.ceil(n / page)
            mine = list(range(shard, pages, 2))
            tokens = sum(min(page, n - j * page) for j in mine)
            # a shard's pages are all full except possibly the request's last page, which must come last
            order = sorted(mine, key=lambda j: (j == pages - 1))
            for slot, j in enumerate(order):
                sub[b, slot] = table[b, j]
            used.append(tokens)
        part = dict(case, block_table=sub.cuda(), seqused_k=torch.tensor(used, dtype=torch.int32).cuda(),
                    max_seqlen_k=sub.shape[1] * page)
        o, l = flash_attn_varlen_func(**part, return_softmax_lse=True)
        outs.append(o)
        lses.append(l)
    got_o, got_l = sharding.merge_partial_attention(torch.stack(outs), torch.stack(lses))
    torch.cuda.synchronize()
    assert (got_o.float() - full_o.float()).abs().max().item() <= T.BF16_O_ATOL
    assert torch.allclose(got_l, full_l, rtol=T.LSE_RTOL, atol=T.LSE_RTOL)
    assert float(lses[1][0, 4]) == float("-inf")          # the one-key request has nothing on shard 1
    # the library's merge kernel (what gather_context_parallel uses on CUDA) against the torch formulation
    nat_o, nat_l = sharding._merge_parts_native(torch.stack(outs), torch.stack(lses))
    torch.cuda.synchronize()
    assert (nat_o.float() - got_o.float()).abs().max().item() <= 2e-2 * max(1.0, got_o.float().abs().max().item()) / 4
    assert torch.allclose(nat_l, got_l, rtol=1e-5, atol=1e-5)
    assert (nat_o.float() - full_o.float()).abs().max().item() <= T.BF16_O_ATOL
    poisoned = torch.stack(outs).clone()
    poisoned[1, 4] = float("nan")                          # the empty shard's row must not be read
    nat_o2, _ = sharding._merge_parts_native(poisoned, torch.stack(lses))
    assert torch.equal(nat_o2, nat_o)


def test_only_atrex_kernels_run():
    """Every compute kernel the public call launches carries the atrex_ prefix (reference:
    op_test/utils/flash_attn_contract.py:178-212)."""
    from atrex import flash_attn_varlen_func

    cases = [T.make_case(64, [1] * 4, [3000] * 4, hq=32, hkv=8),                     # mma.sync + combine
             T.make_case(64, [400, 100], [400, 400], hq=8, hkv=2),                    # plan + tcgen05 two-subtile
             T.make_case(128, [300, 4], [700, 900], hq=12, hkv=1, d=256, fp8=True)]   # plan + tcgen05 single tile
    seen = set()
    for case in cases:
        kw = dict(case, out=torch.empty(case["q"].shape, dtype=torch.bfloat16, device="cuda"))
        for _ in range(2):
            flash_attn_varlen_func(**kw)
        torch.cuda.synchronize()
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            flash_attn_varlen_func(**kw)
            torch.cuda.synchronize()
        names = [e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        kernels = [n for n in names if not n.lower().startswith(("memcpy", "memset"))]
        assert kernels, "profiler exposed no kernels"
        assert all("atrex_" in n for n in kernels), kernels
        seen.update(re.search(r"atrex_sm100_[a-z0-9_]+", n).group(0) for n in kernels)
    assert {"atrex_sm100_fwd_mma_kernel", "atrex_sm100_combine_kernel", "atrex_sm100_plan_kernel",
            "atrex_sm100_fwd_umma_kernel", "atrex_sm100_fwd_umma1_kernel"} <= seen, seen


def test_poisoned_scratch_on_split_tcgen05_path():
    """Split partials of the single-tile tcgen05 kernel: splits without keys publish -inf and their (NaN) scratch
    is never read."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    case = T.make_case(128, [4, 4, 1], [6000, 10, 0], hq=64, hkv=4)
    poison = torch.full((64 << 20,), 0xFF, dtype=torch.uint8, device="cuda")
    del poison
    T.check(case, num_splits=8)


# ------------------------------------------------------------------ pages that straddle KV tiles, clamped lengths
@pytest.mark.parametrize("page,d,fp8", [(192, 128, False), (320, 128, False), (192, 256, True), (448, 256, False)])
def test_pages_that_are_not_a_multiple_of_the_kv_tile(page, d, fp8):
    """A 128-key tile over pages of 192 / 320 / 448 rows starts in one page and ends in the next: it must be
    fetched as two 64-row boxes (one 128-row box would read past the page and miss the next page's first rows).
    Prefill on the tcgen05 kernels and decode on the mma.sync kernel, unused rows poisoned."""
    case = T.make_case(page, [300, 129], [300, 1500], hq=8, hkv=1, d=d, fp8=fp8, std=0.6, poison_tail=True)
    assert _planned_route(case) == 2
    T.check(case, fp8=fp8)
    decode = T.make_case(page, [1, 2, 1], [1500, 193, 5000], hq=8, hkv=2, d=d, fp8=fp8, poison_tail=True)
    T.check(decode, fp8=fp8)


def test_lengths_beyond_the_block_table_are_clamped():
    """A stale seqused_k larger than the table row can address (a graph replayed over overwritten metadata) is
    clamped to max_pages * page_size on the device: the request then reads exactly its table row, never past it."""
    page, lens = 64, [256, 512]
    case = T.make_case(page, [1, 3], lens, hq=8, hkv=2, spare_pages=0)
    assert case["block_table"].shape[1] * page == 512
    want_o, want_l = T.run(case)
    stale = dict(case, seqused_k=torch.tensor([256, 1 << 30], dtype=torch.int32, device="cuda"))
    got_o, got_l = T.run(stale)
    torch.cuda.synchronize()
    assert torch.equal(got_o, want_o) and torch.equal(got_l, want_l)
    prefill = T.make_case(page, [200, 512], lens, hq=8, hkv=2, spare_pages=0, seed=3)
    want_o, want_l = T.run(prefill)
    got_o, got_l = T.run(dict(prefill, seqused_k=torch.tensor([256, 2 ** 31 - 1], dtype=torch.int32, device="cuda")))
    torch.cuda.synchronize()
    assert torch.equal(got_o, want_o) and torch.equal(got_l, want_l)


def test_packed_kv_with_both_cu_seqlens_k_and_seqused_k_through_the_c_abi():
    """The C ABI (unlike the Python API) accepts packed K/V with both arrays: the used length of a request is the
    smaller of its cu_seqlens_k extent and seqused_k, as the oracle defines it."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime
    from oracle import fa_oracle

    lens, used = [128, 300, 77], [100, 300, 0]
    g = torch.Generator().manual_seed(11)
    total = sum(lens)
    q = torch.randn(9, 8, 128, generator=g).bfloat16().cuda()
    k = torch.randn(total, 2, 128, generator=g).bfloat16().cuda()
    v = torch.randn(total, 2, 128, generator=g).bfloat16().cuda()
    cu_q = torch.tensor([0, 3, 6, 9], dtype=torch.int32).cuda()
    cu_k = torch.tensor([0, 128, 428, 505], dtype=torch.int32).cuda()
    su = torch.tensor(used, dtype=torch.int32).cuda()
    eo, el = fa_oracle.attention(T.to_numpy(q), T.to_numpy(k), T.to_numpy(v), T.to_numpy(cu_q),
                                 cu_seqlens_k=T.to_numpy(cu_k), seqused_k=np.array(used), softmax_scale=128 ** -0.5,
                                 causal=True)
    for route in (runtime.ROUTE_MMA, runtime.ROUTE_UMMA):
        out = torch.full_like(q, float("nan"))
        lse = torch.full((8, 9), float("nan"), dtype=torch.float32, device="cuda")
        params = runtime.build_params(q, k, v, out, lse, cu_q, cu_k, su, None, None, None, None, None,
                                      runtime.device_status(q.device), 3, 300, 128 ** -0.5, 0.0, True, -1, -1, 1, route)
        need = runtime.plan(params).workspace_bytes
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
        runtime.launch_params(params, ws, q.device)
        torch.cuda.synchronize()
        T.compare(out, lse, eo, el, [0, 3, 6, 9])


# ------------------------------------------------------------------ the benchmark's own shapes
def test_fp8_prefill_at_the_benchmark_heads_with_amax_descales():
    """FP8 E4M3 causal paged prefill with a cached prefix at 24 query / 2 KV heads, head_dim 256, page 128, each
    request quantised with its own scales (max |x| / 448 per request and KV head, the way a serving stack fills an
    FP8 cache); oracle on two of the four requests."""
    hq, hkv, d, page = 24, 2, 256, 128
    q_lens, prefix = [512, 700, 2048, 1500], [300, 0, 4096, 2000]
    kv_lens = [a + b for a, b in zip(q_lens, prefix)]
    case = T.make_case(page, q_lens, kv_lens, hq=hq, hkv=hkv, d=d, seed=21)      # BF16 draw, quantised below
    table = case["block_table"].long()
    cu = case["cu_seqlens_q"].tolist()
    kq, vq = torch.zeros_like(case["k"], dtype=torch.float8_e4m3fn), torch.zeros_like(case["v"], dtype=torch.float8_e4m3fn)
    qq = torch.empty_like(case["q"], dtype=torch.float8_e4m3fn)
    scales = {n: torch.empty(len(q_lens), hkv, dtype=torch.float32, device="cuda")
              for n in ("q_descale", "k_descale", "v_descale")}
    for r, n in enumerate(kv_lens):
        ids = table[r, : math.ceil(n / page)]
        for src, dst, name in ((case["k"], kq, "k_descale"), (case["v"], vq, "v_descale")):
            block = src[ids].float()
            scale = block.abs().amax(dim=(0, 1, 3)).clamp_min(1e-6) / 448.0
            dst[ids] = (block / scale[None, None, :, None]).to(torch.float8_e4m3fn)
            scales[name][r] = scale
        rows = case["q"][cu[r]:cu[r + 1]].float().view(q_lens[r], hkv, hq // hkv, d)
        scale = rows.abs().amax(dim=(0, 2, 3)).clamp_min(1e-6) / 448.0
        qq[cu[r]:cu[r + 1]] = (rows / scale[None, :, None, None]).view(q_lens[r], hq, d).to(torch.float8_e4m3fn)
        scales["q_descale"][r] = scale
    fp8_case = dict(case, q=qq, k=kq, v=vq, **scales)
    T.check(fp8_case, requests=[0, 1], fp8=True, return_lse=False)


def test_prefill_of_131072_keys():
    """One request at the longest length the multi-GPU prefill workload draws (131072 tokens, query = keys), 8 query
    / 1 KV head, head_dim 128, page 64.  Size-independent property: the last prefill row equals a query-length-1
    decode over the same cache (another kernel: mma.sync split-KV + combine); oracle on the first and the last 256
    rows (the oracle takes a row slice as a request of its own: bottom-right alignment puts the last rows at the
    end of the keys, and the first 256 rows see the first 256 keys only)."""
    n, hq, page = 131072, 8, 64
    case = T.make_case(page, [n], [n], hq=hq, hkv=1, std=0.7, spare_pages=2, seed=5)
    out, lse = T.run(case)
    decode = dict(case, q=case["q"][-1:].contiguous(), max_seqlen_q=1,
                  cu_seqlens_q=torch.tensor([0, 1], dtype=torch.int32, device="cuda"))
    out_d, lse_d = T.run(decode)
    torch.cuda.synchronize()
    assert (out[-1:].float() - out_d.float()).abs().max().item() <= T.BF16_O_ATOL
    assert torch.allclose(lse[:, -1:], lse_d, rtol=T.LSE_RTOL, atol=T.LSE_RTOL)
    cu256 = torch.tensor([0, 256], dtype=torch.int32, device="cuda")
    tail = dict(case, q=case["q"][-256:], cu_seqlens_q=cu256)
    eo, el = T.oracle_for(tail)
    T.compare(out[-256:], lse[:, -256:], eo, el, [0, 256])
    head = dict(case, q=case["q"][:256], cu_seqlens_q=cu256,
                seqused_k=torch.tensor([256], dtype=torch.int32, device="cuda"))
    eo, el = T.oracle_for(head)
    T.compare(out[:256], lse[:, :256], eo, el, [0, 256])


# ------------------------------------------------------------------ context parallelism over the keys
def _cp_shards(case, kv_lens, world, page):
    """Deal every request's keys round-robin to `world` caches (rank r gets keys r, r + W, ...), each with its own
    pool and block table; returns one call dict per rank."""
    table = case["block_table"].long().cpu()
    hkv, d = case["k"].shape[2:]
    dtype = case["k"].dtype
    raw = torch.bfloat16 if dtype == torch.bfloat16 else torch.uint8     # move FP8 values as bytes
    src_k, src_v = case["k"].view(raw), case["v"].view(raw)
    shards = []
    for r in range(world):
        local = [len(range(r, n, world)) for n in kv_lens]
        counts = [math.ceil(n / page) for n in local]
        pool_k = torch.zeros(sum(counts) + 1, page, hkv, d, dtype=raw, device="cuda")
        pool_v = torch.zeros_like(pool_k)
        sub = torch.full((len(kv_lens), max(counts + [1])), -1, dtype=torch.int32)
        nxt = 0
        for b, n in enumerate(kv_lens):
            ids = table[b, : math.ceil(n / page)].cuda()
            keys = src_k[ids].reshape(-1, hkv, d)[:n][r::world]
            vals = src_v[ids].reshape(-1, hkv, d)[:n][r::world]
            for j in range(counts[b]):
                rows = keys[j * page:(j + 1) * page]
                pool_k[nxt, : rows.shape[0]] = rows
                pool_v[nxt, : rows.shape[0]] = vals[j * page:(j + 1) * page]
                sub[b, j] = nxt
                nxt += 1
        pool_k, pool_v = pool_k.view(dtype), pool_v.view(dtype)
        shards.append(dict(case, k=pool_k, v=pool_v, block_table=sub.cuda(),
                           seqused_k=torch.tensor(local, dtype=torch.int32, device="cuda"),
                           max_seqlen_k=sub.shape[1] * page, cp_world_size=world, cp_rank=r,
                           cp_tot_seqused_k=torch.tensor(kv_lens, dtype=torch.int32, device="cuda")))
    return shards


def _cp_oracle(shard, sink):
    from oracle import fa_oracle

    descales = {n: None if shard.get(n) is None else T.to_numpy(shard[n]) for n in ("q_descale", "k_descale", "v_descale")}
    return fa_oracle.attention(T.to_numpy(shard["q"]), T.to_numpy(shard["k"]), T.to_numpy(shard["v"]),
                               T.to_numpy(shard["cu_seqlens_q"]), seqused_k=T.to_numpy(shard["seqused_k"]),
                               block_table=T.to_numpy(shard["block_table"]), softmax_scale=shard["softmax_scale"],
                               causal=True, sink=T.to_numpy(sink), cp_world_size=shard["cp_world_size"],
                               cp_rank=shard["cp_rank"], cp_tot_seqused_k=T.to_numpy(shard["cp_tot_seqused_k"]),
                               **descales)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("shape", ["decode", "spec_decode", "prefill", "prefill_hd256_fp8"])
def test_context_parallel_ranks_on_one_gpu(world, shape):
    """Context parallelism emulated on one GPU: rank r's cache holds keys r, r + W, ... of every request; each
    rank's call (cp_world_size, cp_rank, cp_tot_seqused_k) is checked against the oracle for that rank (the mask
    uses the keys' positions in the whole request; the sink joins on rank 0 only), and the merged (O, LSE) against
    the oracle over all keys."""
    from atrex.src.nvidia.flash_attn.sm100 import sharding

    page, fp8, d, hq, hkv = 64, False, 128, 32, 8
    if shape == "decode":
        q_lens, kv_lens = [1, 1, 1, 1], [1000, 3, 333, 1]
    elif shape == "spec_decode":
        q_lens, kv_lens, hq, hkv = [4, 4, 2], [900, 5, 64], 64, 4
    elif shape == "prefill":
        q_lens, kv_lens, hq, hkv = [300, 40, 129], [300, 700, 129], 8, 2
    else:
        q_lens, kv_lens, hq, hkv, d, fp8, page = [200, 30], [200, 500], 12, 1, 256, True, 128
    case = T.make_case(page, q_lens, kv_lens, hq=hq, hkv=hkv, d=d, fp8=fp8, std=0.7, seed=13)
    sink = torch.randn(hq, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    full_o, full_l = T.oracle_for(case, sink=sink)
    cu = T.to_numpy(case["cu_seqlens_q"])
    outs, lses = [], []
    for shard in _cp_shards(case, kv_lens, world, page):
        o, l = T.run(shard, s_aux=sink)
        torch.cuda.synchronize()
        eo, el = _cp_oracle(shard, sink)
        T.compare(o, l, eo, el, cu, fp8=fp8)
        outs.append(o)
        lses.append(l)
    got_o, got_l = sharding._merge_parts_native(torch.stack(outs), torch.stack(lses))
    torch.cuda.synchronize()
    T.compare(got_o, got_l, full_o, full_l, cu, fp8=fp8)


# ------------------------------------------------------------------ the bounded wait, seen to expire
def test_a_bounded_wait_that_expires_reports_and_returns():
    """Every device-side wait gives up after a limit, stores a code in the status word and lets its kernel return.
    The self-test kernel waits (256 polls) on a barrier nobody arrives at: it must return normally with result 0
    and code 104 in the status word, which the host-side check reports once and clears.  Nothing traps; the
    context stays usable (an attention call afterwards is still correct)."""
    import ctypes

    from atrex.src.nvidia.flash_attn.sm100 import runtime

    lib = runtime.load_library()
    fn = lib.atrex_fa_sm100_selftest_bounded_wait
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
    device = torch.device("cuda", torch.cuda.current_device())
    assert runtime.check_device_status(device) == 0
    word = runtime.device_status(device)
    result = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(word.data_ptr(), result.data_ptr(), 256, stream) == 0
    torch.cuda.synchronize()
    assert int(result) == 0
    assert runtime.check_device_status(device) == 104
    assert runtime.check_device_status(device) == 0
    assert fn(word.data_ptr(), None, 256, stream) == 1          # a result pointer is required
    T.check(T.make_case(64, [1, 2], [300, 70], hq=8, hkv=2))


def test_tail_split_of_the_last_round():
    """80 requests x 4 KV heads = 320 work items on a 148-SM persistent grid: the planner cuts the last round's items
    (6 requests, 24 items) into four KV splits and only their rows go through the combine; rows before and inside
    the tail, with a window, sinks and LSE, against the oracle; scratch poisoned beforehand."""
    kv = [700 + 17 * i for i in range(80)]
    case = T.make_case(128, [4] * 79 + [3], kv, hq=64, hkv=4, spare_pages=2, seed=31)
    sink = torch.randn(64, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    poison = torch.full((64 << 20,), 0xFF, dtype=torch.uint8, device="cuda")
    del poison
    T.check(case, requests=[0, 40, 73, 74, 75, 79], window_size=(511, 0), s_aux=sink)
    T.check(case, requests=[0, 73, 74, 79])
