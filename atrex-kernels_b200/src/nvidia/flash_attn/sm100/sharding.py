"""Sharding one attention batch over the GPUs of a box.

Attention for one request (and one KV head) never reads another request's data, so the natural unit is the
request: every rank owns whole requests (their Q rows, their pages, their O rows) and the data path needs no
collective.  ``partition_requests`` balances the ranks by cost (visible (query, key) pairs for prefill, keys read
for decode) with the longest-processing-time-first rule.  ``split_heads`` / ``gather_heads`` are the optional
KV-head split: rank r computes KV heads [r*Hkv/G, (r+1)*Hkv/G) and their query heads for ALL requests, then one
all-gather assembles O.  The reference has no multi-GPU code at all (its API rejects context-parallel arguments,
python/atrex/api/flash_attn.py:128-135); this module is new surface that sits above the unchanged operator.
"""

from __future__ import annotations

import heapq
from typing import Sequence


def request_cost(q_len: int, kv_len: int, causal: bool = True, window_left: int = -1) -> int:
    """Visible (query, key) pairs of one request: proportional to its FLOPs (prefill) or its keys read (q_len 1)."""
    if q_len <= 0 or kv_len <= 0:
        return 0
    off = kv_len - q_len
    total = 0
    if not causal and window_left < 0:
        return q_len * kv_len
    if window_left < 0 and off >= 0:
        return q_len * off + q_len * (q_len + 1) // 2
    for i in range(q_len):
        hi = min(kv_len - 1, i + off) if causal else kv_len - 1
        lo = max(0, i + off - window_left) if window_left >= 0 else 0
        total += max(0, hi - lo + 1)
    return total


def partition_requests(costs: Sequence[int], world_size: int) -> list[list[int]]:
    """Greedy LPT: requests in descending cost, each to the currently lightest rank.  Returns request ids per rank
    (each list ascending).  Deterministic, so every rank can compute the same partition without communicating."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    shards: list[list[int]] = [[] for _ in range(world_size)]
    heap = [(0, r) for r in range(world_size)]
    heapq.heapify(heap)
    for idx in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
        load, rank = heapq.heappop(heap)
        shards[rank].append(idx)
        heapq.heappush(heap, (load + costs[idx], rank))
    return [sorted(s) for s in shards]


def shard_loads(costs: Sequence[int], shards: Sequence[Sequence[int]]) -> list[int]:
    return [sum(costs[i] for i in shard) for shard in shards]


def split_heads(num_q_heads: int, num_kv_heads: int, world_size: int, rank: int) -> tuple[slice, slice]:
    """Query-head and KV-head slices rank ``rank`` computes in the KV-head-split variant."""
    if num_kv_heads % world_size:
        raise ValueError("num_kv_heads must be divisible by the number of ranks for a KV-head split")
    kv_per = num_kv_heads // world_size
    group = num_q_heads // num_kv_heads
    return (slice(rank * kv_per * group, (rank + 1) * kv_per * group), slice(rank * kv_per, (rank + 1) * kv_per))


def gather_heads(local_out, world_size: int, group=None):
    """All-gather ``local_out [total_q, Hq/G, D]`` from every rank into ``[total_q, Hq, D]`` (rank-major heads).

    One ``all_gather_into_tensor`` over NCCL / NVLink followed by a local transpose; with ``world_size == 1`` it is
    the identity.  The tensors are this GPU's own memory on both sides of the collective.
    """
    import torch
    import torch.distributed as dist

    if world_size == 1:
        return local_out
    total_q, heads, dim = local_out.shape
    staged = torch.empty((world_size * total_q, heads, dim), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(staged, local_out.contiguous(), group=group)
    return staged.view(world_size, total_q, heads, dim).permute(1, 0, 2, 3).reshape(total_q, world_size * heads, dim)


def merge_partial_attention(partial_out, partial_lse):
    """Merge attention computed over disjoint key sets: ``partial_out [W, total_q, Hq, D]``, ``partial_lse
    [W, Hq, total_q]`` (natural log, ``-inf`` where a part saw no key) -> ``(out [total_q, Hq, D], lse [Hq, total_q])``.

    ``out = sum_w exp(lse_w - lse) * out_w`` with ``lse = logsumexp_w lse_w``: the same algebra as the split-KV
    combine kernel (and the reference's, src/nvidia/flash_attn/sm103/decode_reduce_cutedsl.py:71-152), here across
    ranks instead of across splits.  Parts without keys get weight 0 and their (arbitrary) output is not read.
    """
    import torch

    lse = torch.logsumexp(partial_lse.float(), dim=0)                               # [Hq, total_q]
    weight = torch.exp(partial_lse.float() - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse)))
    weight = torch.where(torch.isfinite(partial_lse), weight, torch.zeros_like(weight))      # [W, Hq, total_q]
    contrib = torch.where(weight.permute(0, 2, 1).unsqueeze(-1) > 0, partial_out.float(), torch.zeros((), device=partial_out.device))
    out = (contrib * weight.permute(0, 2, 1).unsqueeze(-1)).sum(dim=0)
    return out.to(partial_out.dtype), lse


def gather_context_parallel(local_out, local_lse, world_size: int, group=None):
    """Decode context parallelism: every rank holds a disjoint shard of each request's KV cache, attends its own
    shard (``return_softmax_lse=True``; for a query length of 1 every local key is visible) and this function
    all-gathers the ``(O, LSE)`` pairs over NCCL and merges them.  Returns the full ``(out, lse)`` on every rank.
    Two ``all_gather_into_tensor`` calls on this GPU's own tensors; with ``world_size == 1`` it is the identity."""
    import torch
    import torch.distributed as dist

    if world_size == 1:
        return local_out, local_lse
    outs = torch.empty((world_size,) + tuple(local_out.shape), dtype=local_out.dtype, device=local_out.device)
    lses = torch.empty((world_size,) + tuple(local_lse.shape), dtype=local_lse.dtype, device=local_lse.device)
    dist.all_gather_into_tensor(outs.view(-1, *local_out.shape[1:]), local_out.contiguous(), group=group)
    dist.all_gather_into_tensor(lses.view(-1, *local_lse.shape[1:]), local_lse.contiguous(), group=group)
    if local_out.is_cuda and local_out.dtype == torch.bfloat16 and local_lse.dtype == torch.float32:
        return _merge_parts_native(outs, lses)              # one kernel instead of a chain of element-wise ones
    return merge_partial_attention(outs, lses)


def _merge_parts_native(outs, lses):
    """``merge_partial_attention`` as one launch of the library's merge kernel (BF16 parts, FP32 LSE, CUDA)."""
    import ctypes

    import torch

    from . import runtime

    lib = runtime.load_library()
    fn = lib.atrex_fa_sm100_merge_parts
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                   ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    world, total_q, heads, dim = outs.shape
    outs, lses = outs.contiguous(), lses.contiguous()
    out = torch.empty((total_q, heads, dim), dtype=torch.bfloat16, device=outs.device)
    lse = torch.empty((heads, total_q), dtype=torch.float32, device=outs.device)
    with torch.cuda.device(outs.device):
        stream = torch.cuda.current_stream(outs.device).cuda_stream
        runtime.raise_for_status(fn(outs.data_ptr(), lses.data_ptr(), out.data_ptr(), lse.data_ptr(), world, total_q,
                                    heads, dim, stream))
    return out, lse



class ContextParallelExchange:
    """Context parallelism with the exchange and the merge as ONE kernel over peer memory.

    Every rank attends its share of each request's keys (``flash_attn_varlen_func(..., cp_world_size, cp_rank,
    cp_tot_seqused_k, return_softmax_lse=True, out=exchange.out_buffer(total_q))``) and then calls
    ``merge(total_q, lse)``: one launch of ``atrex_sm100_cp_merge_kernel`` announces this rank's ``(O, LSE)`` to
    the peers, waits (bounded) for theirs and reads them with plain peer loads over NVLink; no collective library
    call and no staging copy sit on the data path.  The partial results live in a symmetric-memory allocation
    (``torch.distributed._symmetric_memory``: the same virtual layout on every rank, mapped into every rank's
    address space), two alternating slots so that a rank that runs ahead never overwrites a slot a slower rank is
    still reading.  ``world_size == 1`` needs no peer memory and ``merge`` just hands the local pair back.

    Capacity is fixed at construction (``max_total_q`` query tokens); nothing is allocated per step except the
    result tensors.
    """

    _COUNTER_BYTES = 256

    def __init__(self, max_total_q: int, num_q_heads: int, head_dim: int, device, group=None):
        import os

        import torch
        import torch.distributed as dist

        self.torch, self.device = torch, torch.device(device)
        self.heads, self.dim, self.capacity = int(num_q_heads), int(head_dim), int(max_total_q)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.step = 0
        self._o_bytes = self.capacity * self.heads * self.dim * 2
        self._lse_bytes = self.capacity * self.heads * 4
        slot = (self._o_bytes + 255) // 256 * 256 + (self._lse_bytes + 255) // 256 * 256
        self._slot_bytes = slot
        total = self._COUNTER_BYTES + 2 * slot
        if self.world > 1:
            # plain peer mappings only: no multicast object is bound to these buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            self._buffer = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self._buffer.zero_()
            handle = symm_mem.rendezvous(self._buffer, dist.group.WORLD if group is None else group)
            self._peer_base = [int(ptr) for ptr in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(self.device)
            dist.barrier(group)            # every rank's counters are zero before anyone signals
        else:
            self._buffer = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self._peer_base = [self._buffer.data_ptr()]

    def _slot_offset(self, step: int) -> int:
        return self._COUNTER_BYTES + (step & 1) * self._slot_bytes

    def out_buffer(self, total_q: int):
        """The BF16 ``[total_q, Hq, D]`` tensor this step's attention call must write (pass it as ``out=``)."""
        if total_q > self.capacity:
            raise ValueError(f"{total_q} query tokens exceed the exchange capacity of {self.capacity}")
        begin = self._slot_offset(self.step)
        flat = self._buffer[begin: begin + total_q * self.heads * self.dim * 2]
        return flat.view(self.torch.bfloat16).view(total_q, self.heads, self.dim)

    def merge(self, total_q: int, lse):
        """Exchange and merge this step's partial results; returns ``(out, lse)`` over all keys on every rank.
        ``lse`` is the FP32 ``[Hq, total_q]`` tensor the attention call returned."""
        import ctypes

        from . import runtime

        torch = self.torch
        local_out = self.out_buffer(total_q)
        if self.world == 1:
            self.step += 1
            return local_out.clone(), lse
        begin = self._slot_offset(self.step)
        lse_off = begin + (self._o_bytes + 255) // 256 * 256
        self._buffer[lse_off: lse_off + total_q * self.heads * 4].view(torch.float32).view(self.heads, total_q).copy_(lse)
        self.step += 1
        out = torch.empty((total_q, self.heads, self.dim), dtype=torch.bfloat16, device=self.device)
        merged_lse = torch.empty((self.heads, total_q), dtype=torch.float32, device=self.device)
        params = CpMergeParams()
        params.struct_bytes, params.abi_version = ctypes.sizeof(CpMergeParams), runtime.ABI_VERSION
        for w, base in enumerate(self._peer_base):
            params.parts[w] = base + begin
            params.part_lse[w] = base + lse_off
            params.counters[w] = base
        params.out, params.lse = out.data_ptr(), merged_lse.data_ptr()
        status = runtime.device_status(self.device)
        params.device_status = None if status is None else status.data_ptr()
        params.total_q, params.num_q_heads, params.head_dim = total_q, self.heads, self.dim
        params.world, params.rank, params.step = self.world, self.rank, self.step
        lib = runtime.load_library()
        _bind_cp_merge(lib)
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            runtime.raise_for_status(lib.atrex_fa_sm100_cp_merge(ctypes.byref(params), stream))
        return out, merged_lse


def _cp_merge_struct():
    import ctypes

    class CpMergeParams(ctypes.Structure):
        """Mirror of ``atrex_fa_sm100_cp_merge_params`` (include/atrex_fa_sm100.h)."""

        _fields_ = [("struct_bytes", ctypes.c_uint32), ("abi_version", ctypes.c_uint32),
                    ("parts", ctypes.c_void_p * 8), ("part_lse", ctypes.c_void_p * 8),
                    ("counters", ctypes.c_void_p * 8),
                    ("out", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("device_status", ctypes.c_void_p),
                    ("total_q", ctypes.c_int64),
                    ("num_q_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("world", ctypes.c_int32),
                    ("rank", ctypes.c_int32), ("step", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]

    return CpMergeParams


CpMergeParams = _cp_merge_struct()


def _bind_cp_merge(lib):
    import ctypes

    if getattr(lib, "_atrex_cp_merge_bound", False):
        return
    lib.atrex_fa_sm100_cp_merge.restype = ctypes.c_int
    lib.atrex_fa_sm100_cp_merge.argtypes = [ctypes.POINTER(CpMergeParams), ctypes.c_void_p]
    lib._atrex_cp_merge_bound = True
