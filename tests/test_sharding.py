"""Request sharding and the KV-head split, on CPU (single process and two gloo ranks)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from atrex.src.nvidia.flash_attn.sm100 import sharding
from oracle import fa_oracle


def test_request_cost_matches_oracle_pair_count():
    for q, k, causal, left in [(1, 100, True, -1), (7, 7, True, -1), (5, 3, True, -1), (4, 50, True, 9), (3, 9, False, -1)]:
        assert sharding.request_cost(q, k, causal, left) == fa_oracle.visible_pairs(q, k, causal, (left, 0 if causal else -1))


def test_partition_is_complete_balanced_and_deterministic():
    rng = np.random.default_rng(1729)
    lens = np.clip(np.round(np.exp(rng.normal(np.log(8192), 0.75, 256))), 1024, 131072).astype(int)
    costs = [sharding.request_cost(int(n), int(n)) for n in lens]
    for world in (1, 2, 4, 8):
        shards = sharding.partition_requests(costs, world)
        assert sorted(i for s in shards for i in s) == list(range(256))
        loads = sharding.shard_loads(costs, shards)
        # LPT bound: no rank exceeds the mean by more than the largest single request
        assert max(loads) <= sum(costs) / world + max(costs)
        if world > 1:
            assert max(loads) / (sum(costs) / world) < 1.25
        assert shards == sharding.partition_requests(costs, world)
    with pytest.raises(ValueError):
        sharding.partition_requests(costs, 0)


def test_split_heads():
    q, kv = sharding.split_heads(64, 8, 8, 3)
    assert (q.start, q.stop, kv.start, kv.stop) == (24, 32, 3, 4)
    with pytest.raises(ValueError):
        sharding.split_heads(64, 8, 3, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        q_lens = [3, 1, 4, 2, 5, 1]
        kv_lens = [40, 64, 7, 100, 5, 33]
        hq, hkv, d = 4, 2, 128
        cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        q = rng.standard_normal((cu[-1], hq, d)).astype(np.float32)
        k = [rng.standard_normal((n, hkv, d)).astype(np.float32) for n in kv_lens]
        v = [rng.standard_normal((n, hkv, d)).astype(np.float32) for n in kv_lens]

        def attend(ids, q_heads=slice(None), kv_heads=slice(None)):
            out = {}
            for b in ids:
                o, _ = fa_oracle.attention(q[cu[b]:cu[b + 1], q_heads], k[b][:, kv_heads], v[b][:, kv_heads],
                                           np.array([0, q_lens[b]], np.int32),
                                           cu_seqlens_k=np.array([0, kv_lens[b]], np.int32), causal=True)
                out[b] = o
            return out

        full = attend(range(len(q_lens)))
        # (1) request sharding: each rank computes its shard, no collective; the union is the full result
        costs = [sharding.request_cost(a, b) for a, b in zip(q_lens, kv_lens)]
        mine = sharding.partition_requests(costs, world)[rank]
        part = attend(mine)
        for b in mine:
            np.testing.assert_array_equal(part[b], full[b])
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        assert sorted(i for s in everyone for i in s) == list(range(len(q_lens)))
        # (2) KV-head split: each rank computes its heads for all requests, then one all-gather of O
        q_sl, kv_sl = sharding.split_heads(hq, hkv, world, rank)
        local = attend(range(len(q_lens)), q_sl, kv_sl)
        local_out = torch.from_numpy(np.concatenate([local[b] for b in range(len(q_lens))]))
        gathered = sharding.gather_heads(local_out, world)
        expect = np.concatenate([full[b] for b in range(len(q_lens))])
        np.testing.assert_allclose(gathered.numpy(), expect, rtol=0, atol=0)
        # (3) decode context parallelism: query length 1, each rank holds every world-th key of every request
        #     (one request's local shard is empty on rank 1), partial (O, LSE) all-gathered and merged
        dq = rng.standard_normal((len(kv_lens), hq, d)).astype(np.float32)
        dkv = [1 if b == 2 else n for b, n in enumerate(kv_lens)]          # request 2 has a single key
        cu1 = np.arange(len(kv_lens) + 1, dtype=np.int32)
        want_o = np.zeros_like(dq)
        want_l = np.zeros((hq, len(kv_lens)), np.float32)
        loc_o = np.zeros_like(dq)
        loc_l = np.full((hq, len(kv_lens)), -np.inf, np.float32)
        for b, n in enumerate(dkv):
            o, l = fa_oracle.attention(dq[b:b + 1], k[b][:n], v[b][:n], np.array([0, 1], np.int32),
                                       cu_seqlens_k=np.array([0, n], np.int32), causal=True)
            want_o[b], want_l[:, b] = o[0], l[:, 0]
            mine_k, mine_v = k[b][:n][rank::world], v[b][:n][rank::world]
            if len(mine_k):
                o, l = fa_oracle.attention(dq[b:b + 1], mine_k, mine_v, np.array([0, 1], np.int32),
                                           cu_seqlens_k=np.array([0, len(mine_k)], np.int32), causal=True)
                loc_o[b], loc_l[:, b] = o[0], l[:, 0]
            else:
                loc_o[b] = np.nan                                           # must never be read
        assert cu1[-1] == len(dkv)
        got_o, got_l = sharding.gather_context_parallel(torch.from_numpy(loc_o), torch.from_numpy(loc_l), world)
        np.testing.assert_allclose(got_o.numpy(), want_o, rtol=0, atol=2e-6)
        np.testing.assert_allclose(got_l.numpy(), want_l, rtol=0, atol=2e-6)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_request_sharding_and_head_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_merge_partial_attention_handles_empty_parts():
    out = torch.tensor([[[[1.0, 2.0]]], [[[float("nan"), float("nan")]]], [[[3.0, 6.0]]]])      # [W=3, T=1, H=1, D=2]
    lse = torch.tensor([[[0.0]], [[float("-inf")]], [[0.0]]])                                      # [W, H, T]
    merged, total = sharding.merge_partial_attention(out, lse)
    assert torch.allclose(merged, torch.tensor([[[2.0, 4.0]]])) and torch.allclose(total, torch.log(torch.tensor([[2.0]])))
    merged, total = sharding.merge_partial_attention(out[1:2], lse[1:2])                            # no key anywhere
    assert torch.equal(merged, torch.zeros(1, 1, 2)) and total.item() == float("-inf")

