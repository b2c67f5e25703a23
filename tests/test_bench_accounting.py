"""bench.py's own work accounting (algorithmic bytes / FLOPs) agrees with the oracle's definitions."""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np

from oracle import fa_oracle, kv_cache_oracle, qsa_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("atrex_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(mod)
    finally:
        sys.argv = argv
    return mod


def test_flops_and_bytes_match_the_oracle():
    b = _bench()
    rng = np.random.default_rng(5)
    for left in (-1, 0, 7, 4095):
        q = rng.integers(1, 40, 12).tolist()
        kv = [a + int(x) for a, x in zip(q, rng.integers(0, 60, 12))]
        assert b.algorithmic_flops(q, kv, 8, 128, left) == fa_oracle.algorithmic_flops(q, kv, 8, 128, True, (left, 0))
        assert b.algorithmic_decode_bytes(q, kv, 32, 8, 128, 2, 64, left) == \
            fa_oracle.algorithmic_decode_bytes(q, kv, 32, 8, 128, 2, 64, window=(left, 0))
        for nq, nk in zip(q, kv):
            assert b.causal_visible_pairs(nq, nk, left) == fa_oracle.visible_pairs(nq, nk, True, (left, 0))
    for fp8 in (False, True):
        assert b.kv_write_bytes(1000, 8, 128, fp8) == kv_cache_oracle.algorithmic_bytes(1000, 8, 128, fp8)


def test_every_workload_has_work_units():
    b = _bench()
    for name, spec in b.WORKLOADS.items():
        if spec["kind"] == "kv_write":
            assert b.kv_write_bytes(spec["tokens"], spec["hkv"], spec["d"], spec["fp8"]) > 0
            continue
        if spec["kind"] == "qsa":
            pos = np.array([-1, 9, 14, 4000])
            ids = np.zeros((4, 512), np.int32)
            assert b.qsa_work_bytes(dict(spec, fp8=False, hq=8, hkv=1), ids, pos) == \
                qsa_oracle.algorithmic_bytes(ids, pos, 8, 1, 2)
            continue
        small = dict(spec, batch=2)
        q, kv = b.draw_lengths(small, 1)
        assert b.work_units(small, q, kv) > 0, name


def test_pooled_partition_balances_the_ranks():
    """With N ranks the benchmark pools the N seeded batches and deals the requests by cost, longest first: every
    request is served exactly once, every rank derives the same partition, the one-rank job is the plain seeded
    batch, and the ranks' work is level (decode: within 0.1 % at 8 ranks, where independent per-rank batches
    differ by more than 10 %)."""
    b = _bench()
    spec = b.WORKLOADS["decode_q1"]
    q1, kv1, loads1 = b.shard_requests(spec, 1, 0)
    assert (q1, kv1) == b.draw_lengths(spec, 1729) and len(loads1) == 1
    for world in (2, 4, 8):
        pooled = sorted(kv for r in range(world) for kv in b.draw_lengths(spec, 1729 + 1000 * r)[1])
        served, loads = [], None
        for rank in range(world):
            q, kv, loads_r = b.shard_requests(spec, world, rank)
            assert loads is None or loads == loads_r
            loads = loads_r
            assert b.work_units(spec, q, kv) == loads[rank]
            served += kv
        assert sorted(served) == pooled
        assert max(loads) / (sum(loads) / world) < 1.001
    # the strong prefill set: one fixed draw, the same 256 requests whatever the rank count
    strong = b.WORKLOADS["prefill_sharded"]
    all_kv = sorted(b.draw_lengths(strong, 1729)[1])
    for world in (1, 2, 8):
        served, loads = [], None
        for rank in range(world):
            _, kv, loads = b.shard_requests(strong, world, rank)
            served += kv
        assert sorted(served) == all_kv
        assert max(loads) / (sum(loads) / world) < 1.02
