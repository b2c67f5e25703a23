"""The allocation-free entry point of the C ABI, checked against the regular one.

``atrex_fa_sm100_forward_static_scratch`` serves hosts that cannot give the launcher
scratch memory (an FFI binding with no device allocator of its own, a server whose
HBM is fully reserved by its KV-cache pool, a loop that must avoid the device-wide
synchronisation of cudaMalloc / cudaFree).  Its split-KV scratch is a fixed array
inside the library, so the only question is whether it computes what
``atrex_fa_sm100_forward`` computes.  The file name makes pytest collect it last.
"""

import ctypes
import gc

import pytest
import torch

import fa_testlib as T

_STATIC_CALLS = {"n": 0}     # calls of the allocation-free entry point made by this process so far

pytestmark = pytest.mark.gpu


def _entry_points():
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    lib = runtime.load_library()
    fn = lib.atrex_fa_sm100_forward_static_scratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(runtime.Params), ctypes.c_void_p]
    lib.atrex_fa_sm100_static_scratch_bytes.restype = ctypes.c_uint64
    return runtime, lib, fn


def _params(runtime, case, out, lse, num_splits):
    return runtime.build_params(case["q"], case["k"], case["v"], out, lse, case["cu_seqlens_q"], None,
                                case["seqused_k"], case["block_table"], None, None, None, None, None,
                                case["max_seqlen_q"], case["max_seqlen_k"], case["softmax_scale"], 0.0, True,
                                -1, -1, num_splits, 0)


def _compare_entry_points(runtime, lib, static_forward, case, splits, limit, *, expect_launches):
    """One call through atrex_fa_sm100_forward with caller scratch, the same call through the allocation-free
    entry point; both against each other and against the oracle."""
    stream = torch.cuda.current_stream().cuda_stream
    shape_lse = (case["q"].shape[1], case["q"].shape[0])
    out_ref = torch.empty_like(case["q"])
    lse_ref = torch.empty(shape_lse, dtype=torch.float32, device="cuda")
    p_ref = _params(runtime, case, out_ref, lse_ref, splits)
    info = runtime.plan(p_ref)
    need = info.workspace_bytes
    assert 0 < need <= limit
    assert info.kernel_launches == expect_launches
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    runtime.raise_for_status(lib.atrex_fa_sm100_forward(ctypes.byref(p_ref), workspace.data_ptr(), need, stream))

    out_new = torch.full_like(case["q"], float("nan"))
    lse_new = torch.full(shape_lse, float("nan"), dtype=torch.float32, device="cuda")
    p_new = _params(runtime, case, out_new, lse_new, splits)
    gc.collect()                                        # garbage of earlier tests must not be freed inside the window
    free_before = torch.cuda.mem_get_info()[0]          # the driver's view: catches cudaMalloc in the library itself
    before = torch.cuda.memory_stats()["allocation.all.allocated"]   # torch's allocator: a count that only grows
    runtime.raise_for_status(static_forward(ctypes.byref(p_new), stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    # The first call of a process may load the library's module image, the 16 MiB array included (that is the CUDA
    # runtime's own doing, and why the header asks for one call before a capture); from the second call on the
    # device's free memory must not shrink at all.
    if _STATIC_CALLS["n"] > 0:
        assert torch.cuda.mem_get_info()[0] >= free_before
    _STATIC_CALLS["n"] += 1

    assert (out_new.float() - out_ref.float()).abs().max().item() <= T.BF16_O_ATOL
    # rows that see no key carry LSE = -inf in both; compare the rest relatively
    assert torch.equal(torch.isneginf(lse_new), torch.isneginf(lse_ref))
    seen = torch.isfinite(lse_ref)
    rel = (lse_new[seen] - lse_ref[seen]).abs() / lse_ref[seen].abs().clamp_min(1.0)
    assert rel.max().item() <= T.LSE_RTOL
    # and both agree with the oracle
    eo, el = T.oracle_for(case)
    T.compare(out_new, lse_new, eo, el, T.to_numpy(case["cu_seqlens_q"]))
    return info


def test_static_scratch_entry_point_matches_regular_entry_point():
    runtime, lib, static_forward = _entry_points()
    torch.cuda.set_device(0)
    limit = lib.atrex_fa_sm100_static_scratch_bytes()
    assert limit == 16 * 1024 * 1024

    # two different decode batches back to back: the second call finds the first call's partials in the array
    for seed, kv_lens, splits in ((11, [3000, 64, 517, 1], 6), (12, [40, 2100, 900, 1300], 4)):
        case = T.make_case(64, [1, 2, 2, 1], kv_lens, hq=16, hkv=2, seed=seed, poison_tail=True)
        info = _compare_entry_points(runtime, lib, static_forward, case, splits, limit, expect_launches=2)
        assert info.route == runtime.ROUTE_MMA      # at most 16 packed rows: the mma.sync split-KV kernel
    assert runtime.check_device_status("cuda") == 0


def test_static_scratch_entry_point_on_the_planned_and_the_tcgen05_split_routes():
    """The array also holds the row-tile plan of calls with several row tiles per request (plan kernel +
    attention kernel + combine), and the wide FP32 partials of the tcgen05 single-tile kernel's split-KV path;
    two calls in a row on each, the second over the first one's leftovers."""
    runtime, lib, static_forward = _entry_points()
    torch.cuda.set_device(0)
    limit = lib.atrex_fa_sm100_static_scratch_bytes()
    # several row tiles per request (max_seqlen_q * group > rows per tile) with an explicit split: plan kernel,
    # tcgen05 single-tile kernel, combine
    for seed, q_lens, kv_lens in ((3, [200, 40], [700, 40]), (4, [64, 300], [900, 300])):
        case = T.make_case(64, q_lens, kv_lens, hq=8, hkv=2, seed=seed, std=0.6, poison_tail=True)
        info = _compare_entry_points(runtime, lib, static_forward, case, 2, limit, expect_launches=3)
        assert info.route == runtime.ROUTE_UMMA and info.m_rows == 128
    # speculative decode: 64 packed rows per KV head on the tcgen05 single-tile kernel, three KV splits
    for seed, kv_lens in ((5, [5000, 300, 128]), (6, [64, 4000, 2500])):
        case = T.make_case(128, [4, 4, 3], kv_lens, hq=64, hkv=4, seed=seed, poison_tail=True)
        info = _compare_entry_points(runtime, lib, static_forward, case, 3, limit, expect_launches=2)
        assert info.route == runtime.ROUTE_UMMA and info.num_splits == 3
    assert runtime.check_device_status("cuda") == 0


def test_static_scratch_entry_point_rejects_oversized_calls():
    runtime, lib, static_forward = _entry_points()
    torch.cuda.set_device(0)
    # 64 requests x 64 heads x 256 splits of FP32 partials is far beyond the built-in array
    case = T.make_case(64, [1] * 64, [128] * 64, hq=64, hkv=8, seed=5)
    case["max_seqlen_k"] = 64 * 1024
    out = torch.full_like(case["q"], 3.0)
    params = _params(runtime, case, out, None, 256)
    assert runtime.plan(params).workspace_bytes > lib.atrex_fa_sm100_static_scratch_bytes()
    status = static_forward(ctypes.byref(params), torch.cuda.current_stream().cuda_stream)
    assert status == 3
    assert b"built-in scratch" in lib.atrex_fa_sm100_last_error()
    torch.cuda.synchronize()
    assert torch.all(out == 3.0), "a rejected call must not launch anything"
