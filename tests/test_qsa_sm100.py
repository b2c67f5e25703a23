"""Compact sparse attention (atrex.qsa_compact) on sm_100a: contract checks on CPU, parity on a B200.

Modelled on the reference's op_test/nvidia/qsa/test_qsa_sm100.py: seeded cases through the public API compared with
the FP32 oracle under its tolerance (|err| <= 0.003 + 0.02 |ref|, :21,438-451), the golden fixtures (outputs of the
reference's own oracle), metadata refreshed between calls and between CUDA-graph replays (:474-500, 716-781),
strided Q and int32 positions (:611-631), an interleaved K|V pool with gaps between pages (:238-289).
"""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import atrex
from atrex.utils.device_target import DeviceTarget
from golden import qsa_cases
from oracle import qsa_oracle
from test_qsa_oracle import golden_output, run_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ATOL, RTOL = 0.003, 0.02


# ------------------------------------------------------------------ CPU: contract
@pytest.fixture
def as_b200(monkeypatch):
    from atrex.api import qsa

    monkeypatch.setattr(qsa, "detect_device_target", lambda device: DeviceTarget("nvidia", "sm100", "12.9", 0))
    yield qsa
    qsa._validated.clear()


def _call(rows=3, hkv=1, ratio=8, page=64, fp8=False, device="cpu"):
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    q = torch.zeros(rows, hkv * ratio, 256, device=device).to(dt)
    k = torch.zeros(6, page, hkv, 256, device=device).to(dt)
    return dict(q=q, k_cache=k, v_cache=torch.zeros_like(k),
                indexer_block_ids=torch.full((rows, 512), -1, dtype=torch.int32, device=device),
                query_positions=torch.zeros(rows, dtype=torch.int64, device=device),
                block_table=torch.zeros(2, 3, dtype=torch.int32, device=device),
                token_to_req=torch.zeros(rows, dtype=torch.int32, device=device), use_prefill_config=False,
                output_gate=torch.zeros(rows, hkv * ratio, 256, dtype=torch.bfloat16, device=device))


def test_lazy_export():
    assert "qsa_compact" in atrex.__all__


def test_other_devices_are_rejected():
    with pytest.raises(NotImplementedError, match="nvidia/sm100"):
        atrex.qsa_compact(**_call())
    with pytest.raises(ValueError, match="q must be a tensor"):
        atrex.qsa_compact(**dict(_call(), q=None))


BAD = [
    (lambda d: d.update(v_cache=d["v_cache"][:, :32]), "identical four-dimensional"),
    (lambda d: d.update(k_cache=d["k_cache"][:, :24], v_cache=d["v_cache"][:, :24]), "positive multiple of 16"),
    (lambda d: d.update(q=torch.zeros(3, 10, 256, dtype=torch.bfloat16)), "GQA ratio"),
    (lambda d: d.update(q=d["q"].float()), "BF16 or all be FP8"),
    (lambda d: d.update(output_gate=d["output_gate"].float()), "gate must be BF16"),
    (lambda d: d.update(q=torch.zeros(3, 8, 512, dtype=torch.bfloat16)[..., ::2]), "contiguous D"),
    (lambda d: d.update(indexer_block_ids=torch.zeros(3, 1024, dtype=torch.int32)[:, ::2]), "block IDs"),
    (lambda d: d.update(indexer_block_ids=d["indexer_block_ids"].long()), "block IDs"),
    (lambda d: d.update(query_positions=d["query_positions"].float()), "positions"),
    (lambda d: d.update(token_to_req=d["token_to_req"].long()), "request IDs"),
    (lambda d: d.update(block_table=d["block_table"].long()), "page table"),
    (lambda d: d.update(block_table=torch.zeros(3, 16385, dtype=torch.int32)), "1M tokens"),
    (lambda d: d.update(output_gate=torch.zeros(3, 8, 256 + 1, dtype=torch.bfloat16)[..., 1:]), "gate must"),
    (lambda d: d.update(out=d["q"]), "share storage"),
    (lambda d: d.update(out=torch.zeros(3, 8, 256)), "out must be"),
    (lambda d: d["q"].requires_grad_(True), "inference-only"),
    (lambda d: d.update(sm_scale=0.1), "only for NVIDIA FP8"),
    (lambda d: d.update(v_scale=2.0), "only for NVIDIA FP8"),
]


@pytest.mark.parametrize("index", range(len(BAD)))
def test_malformed_calls_fail_fast(as_b200, index, monkeypatch):
    from atrex.src.nvidia.qsa.sm100 import runtime

    monkeypatch.setattr(runtime, "forward", lambda *a, **k: pytest.fail("a malformed call reached the launcher"))
    mutate, match = BAD[index]
    call = _call()
    mutate(call)
    with pytest.raises(ValueError, match=re.escape(match)):
        atrex.qsa_compact(**call)


def test_fp8_scales_are_checked(as_b200, monkeypatch):
    from atrex.src.nvidia.qsa.sm100 import runtime

    seen = []
    monkeypatch.setattr(runtime, "forward", lambda *a, **k: seen.append((k["sm_scale"], k["v_scale"])))
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    call = _call(fp8=True)
    for bad in (0.0, -1.0, float("inf"), float("nan"), 1e-50, 1e50, True, []):
        with pytest.raises((TypeError, ValueError)):
            atrex.qsa_compact(**call, sm_scale=bad)
        with pytest.raises((TypeError, ValueError)):
            atrex.qsa_compact(**call, sm_scale=0.0625, v_scale=bad)
    atrex.qsa_compact(**call)
    atrex.qsa_compact(**call, sm_scale=0.03, v_scale=1.5)
    atrex.qsa_compact(**_call())
    assert seen == [(256 ** -0.5, 1.0), (0.03, 1.5), (256 ** -0.5, 1.0)]


def test_library_exports_the_sparse_attention_abi():
    from atrex.src.nvidia.qsa.sm100 import runtime

    lib = runtime.library()
    header = open(os.path.join(ROOT, "include", "atrex_qsa_sm100.h")).read()
    declared = re.findall(r"ATREX_FA_API\s+[\w\s\*]+?\b(atrex_qsa_sm100_\w+)\s*\(", header)
    assert len(declared) == 4
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.atrex_qsa_sm100_abi_version() == int(re.search(r"ATREX_QSA_SM100_ABI_VERSION (\d+)", header).group(1))


def test_launcher_checks_the_block_and_plans_from_static_sizes():
    from atrex.src.nvidia.flash_attn.sm100 import runtime as fa_runtime
    from atrex.src.nvidia.qsa.sm100 import runtime

    def block(rows, **over):
        d = _call(rows=rows)
        p = runtime.build_params(d["q"], d["k_cache"], d["v_cache"], d["indexer_block_ids"], d["query_positions"],
                                 d["block_table"], d["token_to_req"], d["output_gate"], torch.zeros_like(d["q"]),
                                 256 ** -0.5, 1.0)
        p.sm_count = 148
        for key, value in over.items():
            setattr(p, key, value)
        return p

    # 8 rows on 148 SMs could take 16 splits of 9 tiles: two rounds of the six warps, which 11 splits of 12 tiles
    # also are, with less to combine (and 10 splits of 13 tiles would be three)
    few, many = runtime.plan(block(8)), runtime.plan(block(4096))
    assert few.num_splits == 11 and few.kernel_launches == 2 and few.workspace_bytes >= 11 * 8 * 8 * 257 * 4
    assert runtime.plan(block(16)).num_splits == 8      # 9 would fit the SMs; 8 are the same three rounds
    assert runtime.plan(block(64)).num_splits == 2 and runtime.plan(block(100)).num_splits == 1
    assert many.num_splits == 1 and many.kernel_launches == 1 and many.workspace_bytes == 0
    assert runtime.plan(block(8, num_splits=3)).num_splits == 3
    for over, exc, match in ((dict(page_size=24), ValueError, "multiple of 16"), (dict(num_kv_heads=3), ValueError, "Hkv"),
                             (dict(num_q_heads=10), ValueError, "GQA ratio"), (dict(sm_scale=0.0), ValueError, "sm_scale"),
                             (dict(num_splits=17), ValueError, "num_splits"), (dict(q_row_stride=3), NotImplementedError, "stride"),
                             (dict(dtype=5), NotImplementedError, "dtype")):
        with pytest.raises(exc, match=match):
            runtime.plan(block(8, **over))
    p = block(8)
    p.abi_version = 99
    assert runtime.library().atrex_qsa_sm100_plan(ctypes.byref(p), ctypes.byref(runtime.PlanInfo())) == 6
    del fa_runtime


# ------------------------------------------------------------------ GPU: parity
def _to_device(case):
    dt = torch.float8_e4m3fn if case["fp8"] else torch.bfloat16
    d = {key: torch.from_numpy(case[key]).to(dt).cuda() for key in ("q", "k_cache", "v_cache")}
    d["output_gate"] = torch.from_numpy(case["output_gate"]).bfloat16().cuda()
    for key in ("indexer_block_ids", "query_positions", "block_table", "token_to_req"):
        d[key] = torch.from_numpy(case[key]).cuda()
    d["use_prefill_config"] = True
    kwargs = {}
    if case["fp8"]:
        s = case["scales"]
        kwargs = dict(sm_scale=256 ** -0.5 * s["q"] * s["k_cache"], v_scale=s["v_cache"])
    return d, kwargs


def _check(actual, expected):
    a = actual.float().cpu().numpy()
    assert np.isfinite(a).all()
    err = np.abs(a - expected)
    bad = err > ATOL + RTOL * np.abs(expected)
    assert not bad.any(), dict(failed=int(bad.sum()), max_abs=float(err.max()))
    return float(err.max())


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(qsa_cases.QSA_CASES))
def test_golden_fixtures(name):
    """The reference's own oracle outputs (positions at block / page boundaries, hidden blocks, holes in the page
    table, padding request ids, more than 512 visible blocks), through the public API."""
    case = qsa_cases.build(name)
    data, kwargs = _to_device(case)
    out = atrex.qsa_compact(**data, **kwargs)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and out.shape == data["q"].shape
    _check(out, golden_output(name))
    given = torch.full_like(out, float("nan"))
    assert atrex.qsa_compact(**data, out=given, **kwargs) is given
    torch.cuda.synchronize()
    assert torch.equal(given, out)


def _random_case(rows, page, hkv, ratio, fp8, seed, *, full=False, pool_gap=False, q_padded=False, pos_int32=False):
    """Rows at random positions of three requests of up to 4100 tokens; `full`: every row lists 512 blocks."""
    rng = np.random.Generator(np.random.PCG64(seed))
    spec = dict(page=page, hkv=hkv, ratio=ratio, fp8=fp8, batch=3, width=-(-4100 // page), holes=True, bad_requests=[],
                positions=(rng.integers(2050, 4100, rows) if full else rng.integers(-1, 4100, rows)).tolist())
    case = qsa_cases.build(spec, seed=seed)
    data, kwargs = _to_device(case)
    if pool_gap:      # K and V as the two halves of one pool with the heads interleaved and a gap between pages
        pool = torch.zeros((data["k_cache"].shape[0], page * 2, hkv, 512), dtype=data["k_cache"].dtype, device="cuda")
        pool[:, :page, :, :256] = data["k_cache"]
        pool[:, :page, :, 256:] = data["v_cache"]
        data["k_cache"], data["v_cache"] = pool[:, :page, :, :256], pool[:, :page, :, 256:]
    if q_padded:      # Q rows inside a wider allocation: 16-byte but not 32-byte aligned base, padded head stride
        storage = torch.zeros((rows, hkv * ratio, 256 + 16 // data["q"].element_size()), dtype=data["q"].dtype, device="cuda")
        storage[:, :, 16 // data["q"].element_size():] = data["q"]
        data["q"] = storage[:, :, 16 // data["q"].element_size():]
    if pos_int32:
        data["query_positions"] = data["query_positions"].int()
    return case, data, kwargs


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("page,hkv,ratio", [(128, 1, 8), (16, 2, 12), (64, 2, 8), (4224, 1, 12)])
def test_ragged_prefill_rows(page, hkv, ratio, fp8):
    case, data, kwargs = _random_case(70, page, hkv, ratio, fp8, seed=page + ratio + fp8, pool_gap=page == 128,
                                      q_padded=page == 64, pos_int32=page == 16)
    out = atrex.qsa_compact(**data, **kwargs)
    torch.cuda.synchronize()
    _check(out, run_oracle(case))


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("rows,splits", [(1, 0), (4, 0), (8, 5), (32, 16), (7, 1), (8, 8), (6, 3), (20, 7), (33, 0)])
def test_decode_rows_with_split_token_lists(rows, splits, fp8):
    """Few rows, every row with a full list of 512 blocks (2048+ tokens): the token list is split over CTAs.  Up
    to eight splits of a row run as one thread-block cluster and combine in the leader's shared memory when every
    row's cluster can be resident at once (2, 3, 5 and 8 splits here); otherwise (16 splits, or 40 clusters of 7)
    the partials go through scratch and the combine kernel; automatic and explicit split counts, scratch poisoned
    beforehand."""
    from atrex.src.nvidia.qsa.sm100 import runtime

    case, data, kwargs = _random_case(rows, 128, 2, 12, fp8, seed=rows + splits, full=True)
    poison = torch.full((32 << 20,), 0xFF, dtype=torch.uint8, device="cuda")
    del poison
    scale = kwargs.get("sm_scale", 256 ** -0.5)
    out = runtime.forward(data["q"], data["k_cache"], data["v_cache"], data["indexer_block_ids"],
                          data["query_positions"], data["block_table"], data["token_to_req"], False,
                          data["output_gate"], None, sm_scale=scale, v_scale=kwargs.get("v_scale", 1.0), num_splits=splits)
    torch.cuda.synchronize()
    _check(out, run_oracle(case))


@pytest.mark.gpu
@pytest.mark.parametrize("fp8", [False, True])
def test_graph_replay_rereads_metadata(fp8):
    """Capture once; then change block ids, positions, request ids, the page table and the gate in place and replay:
    everything is read on the device at every launch (reference: test_qsa_sm100.py:716-781)."""
    case, data, kwargs = _random_case(8, 64, 1, 8, fp8, seed=77, full=True)
    data["out"] = torch.empty(data["q"].shape, dtype=torch.bfloat16, device="cuda")
    atrex.qsa_compact(**data, **kwargs)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        atrex.qsa_compact(**data, **kwargs)
    for step in range(3):
        case["indexer_block_ids"][:, ::7 + step] = -1
        case["query_positions"] = np.maximum(case["query_positions"] - 300 * step, -1)
        case["token_to_req"] = np.roll(case["token_to_req"], 1)
        case["token_to_req"][-1] = -1
        case["block_table"] = np.ascontiguousarray(case["block_table"][::-1])
        case["output_gate"] = np.roll(case["output_gate"], 5, axis=2)
        for key in ("indexer_block_ids", "query_positions", "token_to_req", "block_table"):
            data[key].copy_(torch.from_numpy(case[key]))
        data["output_gate"].copy_(torch.from_numpy(case["output_gate"]).bfloat16())
        data["out"].fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        _check(data["out"], run_oracle(case))


@pytest.mark.gpu
def test_only_atrex_kernels_run_and_inputs_are_untouched():
    case, data, kwargs = _random_case(6, 128, 1, 8, False, seed=5, full=True)
    before = {k: v.clone() for k, v in data.items() if torch.is_tensor(v)}
    atrex.qsa_compact(**data)
    torch.cuda.synchronize()
    kernels = []
    for _ in range(3):       # a profiler session that follows another one in the same process can come back empty
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            atrex.qsa_compact(**data)
            torch.cuda.synchronize()
        names = [e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        kernels = [n for n in names if not n.lower().startswith(("memcpy", "memset"))]
        if kernels:
            break
    if not kernels:
        pytest.skip("the profiler reported no device events in this process")
    assert all("atrex_sm100_qsa" in n for n in kernels), kernels
    for key, value in before.items():
        assert torch.equal(value.view(torch.uint8), data[key].view(torch.uint8)), key
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    assert runtime.check_device_status("cuda") == 0
