"""CPU-only tests of the public boundary: lazy import, device classification, fail-fast validation,
and the C-ABI library's exports and host-side planning.

The validation is exercised on CPU tensors by making ``detect_device_target`` report a B200, the way the
reference's own infrastructure tests swap in fakes (op_test/test_lazy_import.py, op_test/test_device_target.py).
Cases follow the reference's eligibility tests (op_test/nvidia/flash_attn/test_flash_attn_sm103.py:837-880,
op_test/nvidia/flash_attn/test_flash_attn_sm120.py:36-68).
"""

import ctypes
import re
import subprocess
import sys
import os
from types import SimpleNamespace

import pytest
import torch

import atrex
from atrex.utils.device_target import DeviceTarget, detect_device_target

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---------------------------------------------------------------- lazy public API
def test_import_is_lazy():
    code = ("import sys; sys.path.insert(0, %r); import atrex; "
            "assert 'torch' not in sys.modules and 'atrex.api.flash_attn' not in sys.modules; "
            "assert callable(atrex.flash_attn_varlen_func) and callable(atrex.can_use_flash_attn_varlen_func)"
            % os.path.join(ROOT, "atrex-kernels_b200", "python"))
    subprocess.check_call([sys.executable, "-c", code])


def test_lazy_proxy_rebinds_after_first_call(monkeypatch):
    imports = []

    def implementation(value, *, increment=1):
        return value + increment

    def fake_import(name):
        imports.append(name)
        return SimpleNamespace(implementation=implementation)

    monkeypatch.setattr(atrex, "_import_module", fake_import)
    proxy = atrex._lazy_import_and_call("implementation", "atrex.api.example", public_name="example")
    monkeypatch.setattr(atrex, "example", proxy, raising=False)
    assert imports == [] and proxy.__name__ == "example"
    assert atrex.example(3, increment=2) == 5
    assert atrex.example is implementation
    assert atrex.example(4) == 5 and imports == ["atrex.api.example"]


def test_lazy_proxy_keeps_proxy_when_import_fails(monkeypatch):
    proxy = atrex._lazy_import_and_call("missing", "atrex.api.missing")
    monkeypatch.setattr(atrex, "missing", proxy, raising=False)

    def fail_import(name):
        raise ModuleNotFoundError(name)

    monkeypatch.setattr(atrex, "_import_module", fail_import)
    with pytest.raises(ModuleNotFoundError):
        atrex.missing()
    assert atrex.missing is proxy


# ---------------------------------------------------------------- device classification
class _FakeCuda:
    def __init__(self, name, capability, gfx=""):
        self._props = SimpleNamespace(name=name, gcnArchName=gfx)
        self._cap = capability

    def get_device_properties(self, index):
        return self._props

    def get_device_capability(self, index):
        return self._cap

    def is_available(self):
        return True

    def current_device(self):
        return 0


def _fake_torch(monkeypatch, name, capability=(10, 0), cuda="12.9", hip=None, gfx=""):
    fake = SimpleNamespace(cuda=_FakeCuda(name, capability, gfx), version=SimpleNamespace(cuda=cuda, hip=hip))
    monkeypatch.setitem(sys.modules, "torch", fake)


@pytest.mark.parametrize("name,cap,kwargs,expect", [
    ("NVIDIA B200", (10, 0), {}, ("nvidia", "sm100")),
    ("NVIDIA B300 SXM6", (10, 3), {}, ("nvidia", "sm103")),
    ("NVIDIA L40S", (8, 9), {}, ("nvidia", "sm89")),
    ("ZW-M890P", (8, 9), {"cuda": "13.0"}, ("alibaba_ppu", "zwm890p")),
    ("AMD Instinct MI308X", (9, 4), {"hip": "7.2", "gfx": "gfx942:sramecc+:xnack-"}, ("amd", "gfx942")),
    ("Mystery Accelerator", (9, 0), {}, ("unknown", "unknown")),
])
def test_device_classification(monkeypatch, name, cap, kwargs, expect):
    _fake_torch(monkeypatch, name, cap, **kwargs)
    target = detect_device_target(0)
    assert (target.family, target.arch) == expect


def test_cpu_device_is_not_a_target():
    target = detect_device_target(torch.device("cpu"))
    assert (target.family, target.arch) == ("cpu", "cpu")


# ---------------------------------------------------------------- validation on CPU tensors
@pytest.fixture
def as_b200(monkeypatch):
    from atrex.api import flash_attn

    monkeypatch.setattr(flash_attn, "detect_device_target",
                        lambda device: DeviceTarget("nvidia", "sm100", "12.9", 0))
    yield flash_attn
    flash_attn._validated.clear()   # signatures accepted under the stand-in target must not outlive it


def _call(fp8=False, paged=True, hq=8, hkv=2, d=128, page=64):
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    q = torch.zeros(6, hq, d).to(dt)
    if paged:
        k = torch.zeros(10, page, hkv, d).to(dt)
        v = torch.zeros(10, page, hkv, d).to(dt)
        extra = dict(seqused_k=torch.tensor([100, 200], dtype=torch.int32),
                     block_table=torch.zeros(2, 4, dtype=torch.int32))
    else:
        k = torch.zeros(300, hkv, d).to(dt)
        v = torch.zeros(300, hkv, d).to(dt)
        extra = dict(cu_seqlens_k=torch.tensor([0, 100, 300], dtype=torch.int32))
    call = dict(q=q, k=k, v=v, max_seqlen_q=4, cu_seqlens_q=torch.tensor([0, 2, 6], dtype=torch.int32),
                max_seqlen_k=256, causal=True, **extra)
    if fp8:
        for name in ("q_descale", "k_descale", "v_descale"):
            call[name] = torch.ones(2, hkv)
    return call


def test_good_calls_are_eligible(as_b200):
    fp8_ok = as_b200._FP8_ROUTE_BUILT
    assert atrex.can_use_flash_attn_varlen_func(**_call(fp8=True, d=256)) == fp8_ok
    assert atrex.can_use_flash_attn_varlen_func(**_call(fp8=True, d=128)) == fp8_ok
    assert atrex.can_use_flash_attn_varlen_func(**_call(fp8=True, d=256, hq=6, hkv=2)) == fp8_ok
    # FP8 runs on the tcgen05 kernel, which has no softcap and needs a positive scale
    assert not atrex.can_use_flash_attn_varlen_func(**dict(_call(fp8=True, d=256), softcap=10.0))
    assert not atrex.can_use_flash_attn_varlen_func(**dict(_call(fp8=True, d=256), softmax_scale=-1.0))
    for kwargs in (dict(), dict(paged=False), dict(d=256), dict(page=16), dict(page=4224),
                   dict(hq=64, hkv=4)):
        assert atrex.can_use_flash_attn_varlen_func(**_call(**kwargs)), kwargs
    good = _call()
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, fa_version=4))
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, window_size=(4095, 0)))
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, s_aux=torch.zeros(8, dtype=torch.bfloat16)))
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, softcap=30.0, num_splits=256, causal=False))
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, logits_soft_cap=30.0))
    # context parallelism over the keys: local lengths in seqused_k, totals in cp_tot_seqused_k
    total = torch.tensor([400, 800], dtype=torch.int32)
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, cp_world_size=4, cp_rank=3, cp_tot_seqused_k=total))
    assert atrex.can_use_flash_attn_varlen_func(**dict(good, cp_world_size=4, cp_rank=0, cp_tot_seqused_k=total,
                                                       s_aux=torch.zeros(8, dtype=torch.bfloat16)))
    assert atrex.can_use_flash_attn_varlen_func(
        **dict(_call(fp8=True, d=256), k_descale=torch.ones(1, 1).expand(2, 2))) == fp8_ok


BAD = [
    (dict(fa_version=3), NotImplementedError, "fa_version"),
    (dict(fa_version=2), NotImplementedError, "fa_version"),
    (dict(deterministic=True), NotImplementedError, "deterministic"),
    (dict(scheduler_metadata=torch.zeros(1)), NotImplementedError, "scheduler_metadata"),
    (dict(num_prefill=3), NotImplementedError, "num_prefill"),
    (dict(max_seqlen_k_decode=1), NotImplementedError, "max_seqlen_k_decode"),
    (dict(dropout_p=0.1), NotImplementedError, "dropout"),
    (dict(return_attn_probs=True), NotImplementedError, "return_attn_probs"),
    (dict(cp_world_size=2), ValueError, "cp_tot_seqused_k"),
    (dict(cp_tot_seqused_k=torch.zeros(2, dtype=torch.int32)), ValueError, "cp_tot_seqused_k"),
    (dict(cp_world_size=2, cp_rank=2, cp_tot_seqused_k=torch.zeros(2, dtype=torch.int32)), ValueError, "cp_rank"),
    (dict(cp_world_size=0), ValueError, "cp_world_size"),
    (dict(cp_world_size=2, cp_tot_seqused_k=torch.zeros(2, dtype=torch.int64)), ValueError, "cp_tot_seqused_k"),
    (dict(cp_world_size=2, cp_tot_seqused_k=torch.zeros(3, dtype=torch.int32)), ValueError, "cp_tot_seqused_k"),
    (dict(cp_world_size=2, cp_tot_seqused_k=torch.zeros(2, dtype=torch.int32), causal=False), NotImplementedError,
     "causal"),
    (dict(cp_world_size=2, cp_tot_seqused_k=torch.zeros(2, dtype=torch.int32), window_size=(64, 0)),
     NotImplementedError, "window_size"),
    (dict(alibi_slopes=torch.zeros(8)), NotImplementedError, "ALiBi"),
    (dict(q_v=torch.zeros(1)), NotImplementedError, "q_v"),
    (dict(qv=torch.zeros(1)), NotImplementedError, "qv"),
    (dict(output_scale=torch.zeros(1)), NotImplementedError, "output_scale"),
    (dict(mask_mod=lambda *a: True), NotImplementedError, "mask_mod"),
    (dict(dynamic_causal=torch.zeros(1)), NotImplementedError, "dynamic_causal"),
    (dict(cu_seqlens_k=torch.tensor([0, 1, 2], dtype=torch.int32)), ValueError, "exactly one"),
    (dict(seqused_k=None), ValueError, "exactly one"),
    (dict(num_splits=-1), ValueError, "num_splits"),
    (dict(num_splits=257), NotImplementedError, "num_splits"),
    (dict(window_size=(1, 2, 3)), ValueError, "window_size"),
    (dict(softcap=1.0, logits_soft_cap=2.0), ValueError, "softcap"),
    (dict(cu_seqlens_q=None), ValueError, "cu_seqlens_q"),
    (dict(cu_seqlens_q=torch.tensor([0, 2, 6], dtype=torch.int64)), ValueError, "cu_seqlens_q"),
    (dict(block_table=torch.zeros(3, 4, dtype=torch.int32)), ValueError, "block_table"),
    (dict(seqused_k=torch.zeros(3, dtype=torch.int32)), ValueError, "seqused_k"),
    (dict(max_seqlen_k=-1), ValueError, "maximum sequence lengths"),
    (dict(s_aux=torch.zeros(8)), ValueError, "s_aux"),
    (dict(s_aux=torch.zeros(4, dtype=torch.bfloat16)), ValueError, "s_aux"),
    (dict(q_descale=torch.ones(2, 2)), NotImplementedError, "descales"),
    (dict(out=torch.zeros(6, 8, 128)), ValueError, "out"),
    (dict(out=torch.zeros(7, 8, 128, dtype=torch.bfloat16)), ValueError, "out"),
    (dict(out=torch.zeros(6, 8, 256, dtype=torch.bfloat16)[..., ::2]), ValueError, "out"),
]


@pytest.mark.parametrize("update,exc,match", BAD, ids=[f"{i}-{m}" for i, (_, _, m) in enumerate(BAD)])
def test_ineligible_calls_fail_fast(as_b200, update, exc, match):
    kwargs = dict(_call(), **update)
    assert not atrex.can_use_flash_attn_varlen_func(**kwargs)
    with pytest.raises(exc, match=re.escape(match)):
        atrex.flash_attn_varlen_func(**kwargs)


def test_shape_and_dtype_rejections(as_b200):
    base = _call()
    cases = [
        (dict(q=base["q"].float(), k=base["k"].float(), v=base["v"].float()), NotImplementedError, "dtype"),
        (dict(k=base["k"].to(torch.float8_e4m3fn)), NotImplementedError, "matching Q/K/V dtypes"),
        (dict(q=torch.zeros(6, 8, 64, dtype=torch.bfloat16)), NotImplementedError, "head dimensions"),
        (dict(q=torch.zeros(6, 7, 128, dtype=torch.bfloat16)), ValueError, "divisible"),
        (dict(v=torch.zeros(10, 64, 1, 128, dtype=torch.bfloat16)), ValueError, "K/V"),
        (dict(k=torch.zeros(10, 64, 2, 256, dtype=torch.bfloat16)[..., ::2]), ValueError, "contiguous"),
        (dict(k=torch.zeros(10, 48, 2, 128, dtype=torch.bfloat16),
              v=torch.zeros(10, 48, 2, 128, dtype=torch.bfloat16)), NotImplementedError, "page_size"),
        (dict(q=torch.zeros(6, 8, 128, dtype=torch.float8_e5m2), k=base["k"].to(torch.float8_e5m2),
              v=base["v"].to(torch.float8_e5m2)), NotImplementedError, "float8_e5m2"),
    ]
    for update, exc, match in cases:
        kwargs = dict(base, **update)
        assert not atrex.can_use_flash_attn_varlen_func(**kwargs), match
        with pytest.raises(exc, match=re.escape(match)):
            atrex.flash_attn_varlen_func(**kwargs)
    fp8 = _call(fp8=True, d=256)
    for bad in (torch.ones(2, 3), torch.ones(2, 2, dtype=torch.float64)):
        with pytest.raises(ValueError, match="descales"):
            atrex.flash_attn_varlen_func(**dict(fp8, v_descale=bad))
    with pytest.raises(NotImplementedError, match="softcap"):
        atrex.flash_attn_varlen_func(**dict(_call(fp8=True, d=128), softcap=5.0))


def test_other_devices_are_rejected():
    """Without the B200 stand-in a CPU call names the detected target, as the reference does for unknown targets
    (python/atrex/api/flash_attn.py:239-244)."""
    with pytest.raises(NotImplementedError, match="nvidia/sm100"):
        atrex.flash_attn_varlen_func(**_call())
    assert not atrex.can_use_flash_attn_varlen_func(**_call())


def test_can_use_never_reaches_the_launcher(as_b200, monkeypatch):
    """Eligibility must not load, build or launch anything (reference: op_test/ppu/flash_attn/test_flash_attn_zwm890p.py:686-708)."""
    from atrex.src.nvidia.flash_attn.sm100 import launch, runtime

    def boom(*a, **k):
        raise AssertionError("eligibility check reached the native path")

    monkeypatch.setattr(runtime, "load_library", boom)
    monkeypatch.setattr(launch, "forward", boom)
    assert atrex.can_use_flash_attn_varlen_func(**_call())
    assert not atrex.can_use_flash_attn_varlen_func(**dict(_call(), fa_version=3))


def test_runtime_errors_propagate_without_fallback(as_b200, monkeypatch):
    """An exception from the selected runtime is the caller's answer; nothing else is tried
    (reference: op_test/ppu/flash_attn/test_flash_attn_zwm890p.py:375-395)."""
    from atrex.src.nvidia.flash_attn.sm100 import launch

    for exc in (ValueError, RuntimeError, NotImplementedError):
        def raiser(**kwargs):
            raise exc("from the runtime")

        monkeypatch.setattr(launch, "forward", raiser)
        monkeypatch.setattr(torch.cuda, "device", lambda d: __import__("contextlib").nullcontext())
        with pytest.raises(exc, match="from the runtime"):
            atrex.flash_attn_varlen_func(**_call())


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    monkeypatch.setattr(runtime, "_lib", None)
    monkeypatch.setattr(runtime, "LIBRARY_PATH", tmp_path / "libatrex_fa_sm100.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        runtime.load_library()


# ---------------------------------------------------------------- C ABI: exports and host-side planning
HEADER = os.path.join(ROOT, "include", "atrex_fa_sm100.h")


def test_library_exports_every_declared_symbol():
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    lib = runtime.load_library()
    declared = re.findall(r"ATREX_FA_API\s+[\w\s\*]+?\b(atrex_fa_sm100_\w+)\s*\(", open(HEADER).read())
    assert len(declared) >= 7
    for name in declared:
        assert hasattr(lib, name), name
    version = int(re.search(r"#define ATREX_FA_SM100_ABI_VERSION (\d+)", open(HEADER).read()).group(1))
    assert lib.atrex_fa_sm100_abi_version() == version == runtime.ABI_VERSION
    assert lib.atrex_fa_sm100_params_bytes() == ctypes.sizeof(runtime.Params)
    assert lib.atrex_fa_sm100_status_string(2).decode().startswith("well-formed")


def _plan(call, **over):
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    out = torch.empty(call["q"].shape, dtype=torch.bfloat16)
    p = runtime.build_params(call["q"], call["k"], call["v"], out, None, call["cu_seqlens_q"],
                             call.get("cu_seqlens_k"), call.get("seqused_k"), call.get("block_table"),
                             None, None, None, None, None, over.pop("max_seqlen_q", call["max_seqlen_q"]),
                             over.pop("max_seqlen_k", call["max_seqlen_k"]), 0.1, 0.0, True,
                             over.pop("window_left", -1), -1, over.pop("num_splits", 0), 0)
    p.sm_count = 148
    for key, val in over.items():
        setattr(p, key, val)
    return runtime, p


def test_plan_is_a_pure_function_of_static_sizes():
    """Split counts come from batch, heads, upper bounds and the SM count, never from device data
    (reference policy tests: op_test/nvidia/flash_attn/test_flash_attn_sm120.py:116-163)."""
    call = _call(hq=32, hkv=8)
    runtime, p = _plan(call, max_seqlen_q=1, max_seqlen_k=16384)
    info = runtime.plan(p)
    assert info.route == runtime.ROUTE_MMA and info.m_rows == 16 and info.num_splits > 1
    assert info.kernel_launches == 2
    assert info.workspace_bytes >= info.num_splits * 6 * 32 * (128 + 1) * 4
    again = runtime.plan(p)
    assert (again.num_splits, again.workspace_bytes) == (info.num_splits, info.workspace_bytes)
    # an explicit request is honoured, clamped to the number of KV tiles
    assert runtime.plan(_plan(call, max_seqlen_q=1, max_seqlen_k=16384, num_splits=7)[1]).num_splits == 7
    assert runtime.plan(_plan(call, max_seqlen_q=1, max_seqlen_k=64, num_splits=7)[1]).num_splits == 1
    one = runtime.plan(_plan(call, max_seqlen_q=1, max_seqlen_k=16384, num_splits=1)[1])
    assert one.kernel_launches == 1 and one.workspace_bytes == 0
    # a window bounds the keys a row can see, hence the useful splits
    wide = runtime.plan(_plan(call, max_seqlen_q=1, max_seqlen_k=1 << 20)[1]).num_splits
    narrow = runtime.plan(_plan(call, max_seqlen_q=1, max_seqlen_k=1 << 20, window_left=1023)[1]).num_splits
    assert narrow < wide
    # long queries: several row tiles per request -> device-side tile plan kernel + scratch for it
    tiled = runtime.plan(_plan(call, max_seqlen_q=4, max_seqlen_k=256, num_splits=1)[1])
    assert tiled.m_rows == 16 and tiled.kernel_launches == 1
    tiled = runtime.plan(_plan(call, max_seqlen_q=64, max_seqlen_k=256, num_splits=1, route=runtime.ROUTE_MMA)[1])
    assert tiled.m_rows == 64 and tiled.kernel_launches == 2 and tiled.workspace_bytes > 0
    # prefill-shaped BF16 head_dim-128 calls go to the tcgen05 kernel: 256 packed rows per item, no KV split
    umma = runtime.plan(_plan(call, max_seqlen_q=64, max_seqlen_k=256)[1])
    assert umma.route == runtime.ROUTE_UMMA and umma.m_rows == 256 and umma.num_splits == 1
    assert umma.kernel_launches == 2 and umma.workspace_bytes > 0
    # explicit splits, other GQA groups and head_dim 256 run on the single-tile tcgen05 kernel (128 rows per item)
    split4 = runtime.plan(_plan(call, max_seqlen_q=64, max_seqlen_k=4096, num_splits=4)[1])
    assert split4.route == runtime.ROUTE_UMMA and split4.m_rows == 128 and split4.num_splits == 4
    assert split4.kernel_launches == 3
    odd = runtime.plan(_plan(_call(hq=12, hkv=4), max_seqlen_q=64, max_seqlen_k=256)[1])
    assert odd.route == runtime.ROUTE_UMMA and odd.m_rows == 128
    hd256 = runtime.plan(_plan(_call(d=256), max_seqlen_q=64, max_seqlen_k=256)[1])
    assert hd256.route == runtime.ROUTE_UMMA and hd256.m_rows == 128
    # speculative decode (17..128 packed rows) goes there too, with automatic splits and no plan kernel
    spec = runtime.plan(_plan(_call(hq=64, hkv=4), max_seqlen_q=4, max_seqlen_k=32768)[1])
    assert spec.route == runtime.ROUTE_UMMA and spec.m_rows == 128 and spec.num_splits > 1
    assert spec.kernel_launches == 2
    # softcap keeps a call on the mma.sync kernel
    _, capped = _plan(call, max_seqlen_q=64, max_seqlen_k=256)
    capped.softcap = 10.0
    assert runtime.plan(capped).route == runtime.ROUTE_MMA
    # FP8 always runs there, whatever the query length; the mma.sync kernel cannot take it
    fp8 = _call(fp8=True, d=256)
    assert runtime.plan(_plan(fp8, max_seqlen_q=1, max_seqlen_k=4096)[1]).route == runtime.ROUTE_UMMA
    with pytest.raises(NotImplementedError):
        runtime.plan(_plan(fp8, max_seqlen_q=1, max_seqlen_k=4096, route=runtime.ROUTE_MMA)[1])
    assert runtime.plan(_plan(_call(fp8=True, d=128), max_seqlen_q=64, max_seqlen_k=256)[1]).route == runtime.ROUTE_UMMA


def test_launcher_rejects_bad_blocks_before_any_launch():
    call = _call()
    runtime, p = _plan(call)
    lib = runtime.load_library()
    info = runtime.PlanInfo()
    p.abi_version = 1
    assert lib.atrex_fa_sm100_plan(ctypes.byref(p), ctypes.byref(info)) == 6
    runtime, p = _plan(call, head_dim=96)
    with pytest.raises(NotImplementedError):
        runtime.plan(p)
    runtime, p = _plan(call, num_kv_heads=3)
    with pytest.raises(ValueError):
        runtime.plan(p)
    runtime, p = _plan(call, page_size=48)
    with pytest.raises(NotImplementedError):
        runtime.plan(p)
    runtime, p = _plan(call, k_row_stride=3)
    with pytest.raises(NotImplementedError, match="status 2"):
        runtime.plan(p)
    assert lib.atrex_fa_sm100_plan(None, ctypes.byref(info)) == 1


def test_launcher_errors_name_the_failed_check_and_never_repeat_an_older_one():
    """Every non-zero status comes with its own text; a later failure without text would otherwise show the
    previous call's message on that thread."""
    call = _call()
    runtime, p = _plan(call, k_row_stride=3)
    with pytest.raises(NotImplementedError, match="stride"):
        runtime.plan(p)
    fp8 = _call(fp8=True, d=256)
    with pytest.raises(NotImplementedError, match="mma.sync route"):
        runtime.plan(_plan(fp8, max_seqlen_q=1, max_seqlen_k=4096, route=runtime.ROUTE_MMA)[1])
    _, capped = _plan(call, max_seqlen_q=64, max_seqlen_k=256, route=runtime.ROUTE_UMMA)
    capped.softcap = 10.0
    with pytest.raises(NotImplementedError, match="softcap"):
        runtime.plan(capped)
    with pytest.raises(ValueError, match="num_q_heads"):
        runtime.plan(_plan(call, num_kv_heads=3)[1])
    # a good call clears the text
    runtime.plan(_plan(call)[1])
    assert runtime.load_library().atrex_fa_sm100_last_error() == b""
    # context-parallel blocks: rank range, totals pointer, causal only
    with pytest.raises(ValueError, match="cp_rank"):
        runtime.plan(_plan(call, cp_world_size=2, cp_rank=2, cp_tot_seqused_k=64)[1])
    with pytest.raises(ValueError, match="cp_tot_seqused_k"):
        runtime.plan(_plan(call, cp_world_size=2, cp_rank=1)[1])
    with pytest.raises(NotImplementedError, match="context parallelism"):
        runtime.plan(_plan(call, cp_world_size=2, cp_rank=1, cp_tot_seqused_k=64, causal=0)[1])
    runtime.plan(_plan(call, cp_world_size=2, cp_rank=1, cp_tot_seqused_k=64)[1])


@pytest.mark.parametrize("page", [192, 320, 448, 4224])
def test_pages_that_are_not_a_multiple_of_the_kv_tile_are_planned(page):
    """Page sizes that are multiples of 64 but not of the 128-key tile are served (a tile then straddles pages
    and is fetched in 64-row boxes); the plan is the same as for a 128-row page."""
    call = _call(page=page)
    runtime, p = _plan(call, max_seqlen_q=64, max_seqlen_k=4 * page)
    info = runtime.plan(p)
    assert info.route == runtime.ROUTE_UMMA and info.m_rows == 256


def test_kv_write_block_is_checked_on_the_host():
    from atrex.src.nvidia.flash_attn.sm100 import kv_cache, runtime

    lib = runtime.load_library()
    kv_cache._bind(lib)
    p = kv_cache.KvWriteParams()
    p.struct_bytes, p.abi_version = ctypes.sizeof(kv_cache.KvWriteParams), runtime.ABI_VERSION
    p.num_tokens, p.num_kv_heads, p.head_dim, p.page_size, p.num_pages = 4, 2, 128, 64, -1
    assert lib.atrex_fa_sm100_kv_cache_write(ctypes.byref(p), None) == 1
    assert b"negative" in lib.atrex_fa_sm100_last_error()


def test_device_status_word_is_reported_once_and_reset(monkeypatch):
    """A kernel whose bounded wait expired leaves a code in the per-device status word; the host reads it,
    reports it and clears it (CPU stand-in for the word, no kernel involved)."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    word = torch.tensor([103], dtype=torch.int32)
    monkeypatch.setitem(runtime._status_tensors, 0, word)
    assert runtime.check_device_status(torch.device("cuda", 0)) == 103
    assert int(word) == 0
    assert runtime.check_device_status(torch.device("cuda", 0)) == 0


def test_repeated_layouts_reuse_the_filled_block_but_never_addresses(as_b200, monkeypatch):
    """The eager path keeps one filled parameter block per layout and patches addresses into it: a second call with
    other tensors of the same layout must reach the launcher with the NEW addresses and must not plan again."""
    from atrex.src.nvidia.flash_attn.sm100 import launch, runtime

    seen, plans = [], []
    monkeypatch.setattr(runtime, "device_status", lambda device: None)
    monkeypatch.setattr(runtime, "launch_params", lambda params, ws, dev: seen.append(
        (params.q, params.k, params.out, params.seqused_k, params.block_table)))
    real_plan = runtime.plan
    # (no GPU here: give the planner the SM count it would otherwise ask the device for)
    monkeypatch.setattr(runtime, "plan", lambda params: (plans.append(1), setattr(params, "sm_count", 148),
                                                         real_plan(params))[2])
    monkeypatch.setattr(torch.cuda, "device", lambda d: __import__("contextlib").nullcontext())
    monkeypatch.setattr(launch, "_local", __import__("threading").local())
    empty = torch.empty
    monkeypatch.setattr(torch, "empty", lambda *a, **k: empty(*a, **{**k, "device": "cpu"}))
    a, b = _call(), _call()
    b["seqused_k"] = torch.tensor([7, 9], dtype=torch.int32)
    out_a, out_b = torch.zeros(6, 8, 128, dtype=torch.bfloat16), torch.zeros(6, 8, 128, dtype=torch.bfloat16)
    atrex.flash_attn_varlen_func(**a, num_splits=1, out=out_a)
    atrex.flash_attn_varlen_func(**b, num_splits=1, out=out_b)
    assert len(plans) == 1 and len(seen) == 2
    assert seen[0][0] == a["q"].data_ptr() and seen[1][0] == b["q"].data_ptr()
    assert seen[1][3] == b["seqused_k"].data_ptr() and seen[1][4] == b["block_table"].data_ptr()
    assert (seen[0][2], seen[1][2]) == (out_a.data_ptr(), out_b.data_ptr())
    # another layout (a wider block table) is planned on its own
    c = _call()
    c["block_table"] = torch.zeros(2, 8, dtype=torch.int32)
    atrex.flash_attn_varlen_func(**c, num_splits=1, out=out_a)
    assert len(plans) == 2


def test_tail_split_plan_of_the_speculative_decode_shape():
    """One work item per (request, KV head) on a persistent grid: 128 requests x 4 KV heads = 512 items on 148 SMs
    would run 4 rounds for 3.46 rounds of work; the planner cuts the last 68 items (17 requests) in two, so the
    call needs scratch and a combine launch, and a batch that fills its rounds does not."""
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    def spec(batch):
        q = torch.zeros(4 * batch, 64, 128, dtype=torch.bfloat16)
        k = torch.zeros(4, 128, 4, 128, dtype=torch.bfloat16)
        cu = torch.arange(0, 4 * batch + 1, 4, dtype=torch.int32)
        p = runtime.build_params(q, k, k, torch.empty_like(q), None, cu, None, torch.zeros(batch, dtype=torch.int32),
                                 torch.zeros(batch, 256, dtype=torch.int32), None, None, None, None, None, 4, 32768,
                                 0.1, 0.0, True, 4095, 0, 0, 0)
        p.sm_count = 148
        return runtime.plan(p)

    tail = spec(128)
    assert tail.route == runtime.ROUTE_UMMA and tail.num_splits == 2 and tail.kernel_launches == 2
    assert tail.workspace_bytes >= 2 * 512 * 64 * 129 * 4
    full = spec(74)                                     # 296 items: exactly two rounds
    assert full.num_splits == 1 and full.kernel_launches == 1 and full.workspace_bytes == 0
    assert spec(80).num_splits == 4                     # 320 items: the last 24 (6 requests) cut in four (the cap)
    assert spec(37).num_splits == 2                     # fewer than two rounds of items: every item is split
