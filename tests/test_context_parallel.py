"""Context parallelism: the fused exchange + merge kernel.

On one GPU the ranks are emulated by ONE launch over all ranks' buffers with the step counters already set (two
kernels that wait for each other must never share a GPU); with two or more GPUs a torchrun job runs the real
protocol: symmetric-memory buffers, per-rank attention with ``cp_world_size`` / ``cp_rank`` /
``cp_tot_seqused_k``, the merge kernel reading the peers' results over NVLink.
"""

import ctypes
import math
import os
import subprocess
import sys

import pytest
import torch

import fa_testlib as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from atrex.src.nvidia.flash_attn.sm100 import runtime, sharding

    lib = runtime.load_library()
    sharding._bind_cp_merge(lib)
    return runtime, sharding, lib


def test_cp_merge_block_is_checked_on_the_host():
    runtime, sharding, lib = _lib()
    p = sharding.CpMergeParams()
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), None) == 6               # struct_bytes 0: ABI mismatch
    p.struct_bytes, p.abi_version = ctypes.sizeof(sharding.CpMergeParams), runtime.ABI_VERSION
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), None) == 1               # world 0
    p.world, p.rank, p.num_q_heads, p.head_dim, p.total_q = 9, 0, 8, 128, 4
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), None) == 1               # more than 8 ranks
    p.world, p.head_dim = 2, 96
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), None) == 2               # head_dim
    p.head_dim, p.total_q = 128, 0
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), None) == 0               # nothing to do


def _emulated(world, total_q, heads, dim, *, rank, step, counters_at, seed):
    runtime, sharding, lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(seed)
    parts = torch.randn(world, total_q, heads, dim, generator=g, device="cuda").bfloat16()
    lses = torch.randn(world, heads, total_q, generator=g, device="cuda") * 3
    if world > 1:
        lses[1, :, ::3] = float("-inf")                   # a rank without keys for some rows
        parts[1, ::3] = float("nan")                      # ... whose O must not be read
    if world > 2:
        lses[:, 0, 1] = float("-inf")                     # a row no rank has keys for
    counters = torch.full((world, 8), counters_at, dtype=torch.int32, device="cuda")
    out = torch.full((total_q, heads, dim), 7.0, dtype=torch.bfloat16, device="cuda")
    lse = torch.full((heads, total_q), 7.0, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = sharding.CpMergeParams()
    p.struct_bytes, p.abi_version = ctypes.sizeof(sharding.CpMergeParams), runtime.ABI_VERSION
    for w in range(world):
        p.parts[w], p.part_lse[w], p.counters[w] = parts[w].data_ptr(), lses[w].data_ptr(), counters[w].data_ptr()
    p.out, p.lse, p.device_status = out.data_ptr(), lse.data_ptr(), status.data_ptr()
    p.total_q, p.num_q_heads, p.head_dim, p.world, p.rank, p.step = total_q, heads, dim, world, rank, step
    assert lib.atrex_fa_sm100_cp_merge(ctypes.byref(p), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    return sharding, parts, lses, counters, out, lse, int(status)


@pytest.mark.gpu
@pytest.mark.parametrize("world,dim", [(2, 128), (4, 256), (8, 128), (1, 256)])
def test_cp_merge_of_emulated_ranks(world, dim):
    """All ranks' buffers on one GPU, every counter already at the step: the launch is a plain merge and must equal
    the torch formulation of the same algebra; the launching rank's own slot is stamped in every rank's array."""
    total_q, heads, step, rank = 37, 12, 5, world - 1
    sharding, parts, lses, counters, out, lse, status = _emulated(world, total_q, heads, dim, rank=rank, step=step,
                                                                 counters_at=step, seed=world)
    assert status == 0
    clean = torch.where(torch.isnan(parts.float()), torch.zeros((), device="cuda"), parts.float()).bfloat16()
    want_o, want_l = sharding.merge_partial_attention(clean, lses)
    assert torch.equal(torch.isneginf(lse), torch.isneginf(want_l))
    fin = torch.isfinite(want_l)
    assert torch.allclose(lse[fin], want_l[fin], rtol=1e-5, atol=1e-5)
    assert (out.float() - want_o.float()).abs().max().item() <= 2e-2
    assert bool((counters[:, rank] == step).all())


@pytest.mark.gpu
def test_cp_merge_gives_up_when_a_peer_never_arrives():
    """A counter that nothing advances: the bounded wait expires (a second or two), the kernel stores 106 in the
    status word, writes no output and returns; the context stays usable."""
    sharding, parts, lses, counters, out, lse, status = _emulated(2, 5, 4, 128, rank=0, step=3, counters_at=2, seed=9)
    assert status == 106
    assert bool((out == 7.0).all()) and bool((lse == 7.0).all())
    assert int(counters[0, 0]) == 3 and int(counters[1, 0]) == 3 and int(counters[0, 1]) == 2
    T.check(T.make_case(64, [1, 2], [300, 70], hq=8, hkv=2))


@pytest.mark.gpu
def test_exchange_on_one_rank_is_the_identity():
    from atrex import flash_attn_varlen_func
    from atrex.src.nvidia.flash_attn.sm100 import sharding

    case = T.make_case(64, [1, 1, 1], [500, 64, 3], hq=32, hkv=8)
    exchange = sharding.ContextParallelExchange(8, 32, 128, "cuda")
    want_o, want_l = flash_attn_varlen_func(**case, return_softmax_lse=True)
    for _ in range(3):                                    # both slots get used
        o, l = flash_attn_varlen_func(**case, return_softmax_lse=True, out=exchange.out_buffer(3))
        got_o, got_l = exchange.merge(3, l)
        torch.cuda.synchronize()
        assert torch.equal(got_o, want_o) and torch.equal(got_l, want_l)
    with pytest.raises(ValueError, match="capacity"):
        exchange.out_buffer(9)


@pytest.mark.gpu
def test_exchange_between_two_gpus():
    """Two ranks, two GPUs: see tests/cp_worker.py (skipped on a one-GPU box)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "cp_worker.py")]
    done = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "cp_worker ok" in done.stdout
