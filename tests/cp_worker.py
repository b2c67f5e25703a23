"""torchrun worker of tests/test_context_parallel.py: context-parallel attention over W GPUs.

Every rank builds the same seeded case, keeps keys rank, rank + W, ... of each request in its own paged cache,
attends them with the public call (cp_world_size, cp_rank, cp_tot_seqused_k) into the exchange's symmetric-memory
slot and merges with the fused exchange kernel; the result is checked against the CPU oracle over all keys, for
decode (query length 1), speculative decode with a sink, and a ragged prefill batch, several steps each so that
both slots and growing step counters are exercised.
"""

import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for path in (os.path.join(ROOT, "atrex-kernels_b200", "python"), ROOT, os.path.join(ROOT, "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import fa_testlib as T  # noqa: E402


def shard_case(case, kv_lens, world, rank, page):
    table = case["block_table"].long().cpu()
    hkv, d = case["k"].shape[2:]
    local = [len(range(rank, n, world)) for n in kv_lens]
    counts = [math.ceil(n / page) for n in local]
    pool_k = torch.zeros(sum(counts) + 1, page, hkv, d, dtype=torch.bfloat16, device="cuda")
    pool_v = torch.zeros_like(pool_k)
    sub = torch.full((len(kv_lens), max(counts + [1])), -1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(kv_lens):
        ids = table[b, : math.ceil(n / page)].cuda()
        keys = case["k"][ids].reshape(-1, hkv, d)[:n][rank::world]
        vals = case["v"][ids].reshape(-1, hkv, d)[:n][rank::world]
        for j in range(counts[b]):
            rows = keys[j * page:(j + 1) * page]
            pool_k[nxt, : rows.shape[0]] = rows
            pool_v[nxt, : rows.shape[0]] = vals[j * page:(j + 1) * page]
            sub[b, j] = nxt
            nxt += 1
    return dict(case, k=pool_k, v=pool_v, block_table=sub.cuda(),
                seqused_k=torch.tensor(local, dtype=torch.int32, device="cuda"), max_seqlen_k=sub.shape[1] * page,
                cp_world_size=world, cp_rank=rank,
                cp_tot_seqused_k=torch.tensor(kv_lens, dtype=torch.int32, device="cuda"))


def main():
    from atrex import flash_attn_varlen_func
    from atrex.src.nvidia.flash_attn.sm100 import runtime, sharding

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    runtime.prewarm(device)
    shapes = [dict(q_lens=[1, 1, 1, 1], kv_lens=[1000, 3, 333, 1], hq=32, hkv=8, sink=False),
              dict(q_lens=[4, 4, 2], kv_lens=[900, 5, 64], hq=64, hkv=4, sink=True),
              dict(q_lens=[300, 40, 129], kv_lens=[300, 700, 129], hq=8, hkv=2, sink=False)]
    exchange = sharding.ContextParallelExchange(512, 64, 128, device)
    for shape in shapes:
        if shape["hq"] != exchange.heads:
            exchange = sharding.ContextParallelExchange(512, shape["hq"], 128, device)
        case = T.make_case(64, shape["q_lens"], shape["kv_lens"], hq=shape["hq"], hkv=shape["hkv"], std=0.7, seed=13,
                           device=device)
        sink = torch.randn(shape["hq"], generator=torch.Generator().manual_seed(2)).bfloat16().to(device) \
            if shape["sink"] else None
        want_o, want_l = T.oracle_for(case, sink=sink)
        mine = shard_case(case, shape["kv_lens"], world, rank, 64)
        total_q = case["q"].shape[0]
        for _ in range(4):
            o, l = flash_attn_varlen_func(**mine, s_aux=sink, return_softmax_lse=True, out=exchange.out_buffer(total_q))
            got_o, got_l = exchange.merge(total_q, l)
            torch.cuda.synchronize()
            T.compare(got_o, got_l, want_o, want_l, T.to_numpy(case["cu_seqlens_q"]))
        # the collective formulation (two all-gathers + the merge kernel) gives the same answer
        o, l = flash_attn_varlen_func(**mine, s_aux=sink, return_softmax_lse=True)
        ref_o, ref_l = sharding.gather_context_parallel(o, l, world)
        torch.cuda.synchronize()
        assert (ref_o.float() - got_o.float()).abs().max().item() <= 1e-2
    assert runtime.check_device_status(device) == 0
    dist.barrier()
    if rank == 0:
        print("cp_worker ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
