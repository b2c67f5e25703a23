"""Benchmark of the sm_100a attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode_q1]

One "step" is one call of ``atrex.flash_attn_varlen_func`` over one synthetic batch.
The default workload is the BF16 Q1 paged decode configuration (batch 64, 32 query /
8 KV heads, head_dim 128, page 64, KV lengths uniform in [1024, 16384], block table =
seeded permutation of a 20000-page pool, N(0,1) inputs, num_splits = 0).  The metric
is achieved HBM GB/s on ALGORITHMIC bytes: the K and V rows every query can see, plus
Q, O and the page-table entries read.  With N > 1 every rank runs its own batch of
the same shape (weak scaling, no collective on the data path); time is the maximum
over ranks, value the sum of bytes over ranks divided by it.

``--impl reference`` times the CPU FP32 attention (the oracle port of the reference's
``reference()`` in op_test/utils/flash_attn_contract.py:81-111) on the host cores on a
bounded sample of the same workload and prints the same JSON shape.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "atrex-kernels_b200", "python"), ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

WORKLOADS = {
    # BF16 paged decode, query length 1
    "decode_q1": dict(batch=64, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=1024, kv_hi=16384, pool=20000,
                      window=None, sink=False, lse=False, metric="paged_decode_hbm_bandwidth", unit="GB/s"),
    # same shape at a quarter of the batch and a small pool: the case profiler captures run on
    "decode_q1_small": dict(batch=16, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=1024, kv_hi=16384, pool=2500,
                            window=None, sink=False, lse=False, metric="paged_decode_hbm_bandwidth", unit="GB/s"),
    # BF16 speculative decode, query length 4, sliding window, sinks, LSE
    "decode_q4_window": dict(batch=128, q_len=4, hq=64, hkv=4, d=128, page=128, kv_lo=32768, kv_hi=32768,
                             pool=128 * 256 + 64, window=(4095, 0), sink=True, lse=True,
                             metric="paged_decode_hbm_bandwidth", unit="GB/s"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            data = json.load(f)
        return dict(hbm_gbs=float(data["hbm_gbs"]), source="measured")
    return dict(hbm_gbs=6650.0, source="fallback")


def draw_lengths(spec, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(spec["kv_lo"], spec["kv_hi"] + 1, size=spec["batch"]).tolist()


def algorithmic_bytes(spec, kv_lens):
    from oracle.fa_oracle import algorithmic_decode_bytes

    window = spec["window"] or (-1, -1)
    total = algorithmic_decode_bytes([spec["q_len"]] * spec["batch"], kv_lens, spec["hq"], spec["hkv"], spec["d"], 2,
                                     spec["page"], window=window)
    if spec["lse"]:
        total += 4 * spec["batch"] * spec["q_len"] * spec["hq"]
    return total


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def run(self):
        if self.nvml is None:
            return
        n = self.nvml
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.02)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return dict(sm_mhz=statistics.median(self.samples) if self.samples else None, sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons), samples=len(self.samples))


def physical_gpu_index(local_index):
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_index])
        except (ValueError, IndexError):
            return local_index
    return local_index


def build_device_case(spec, kv_lens, seed, device):
    """Synthetic batch resident on ``device`` plus pinned host copies of the per-step inputs."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    pool, page, hkv, d = spec["pool"], spec["page"], spec["hkv"], spec["d"]
    k = torch.randn((pool, page, hkv, d), generator=g, device=device, dtype=torch.bfloat16)
    v = torch.randn((pool, page, hkv, d), generator=g, device=device, dtype=torch.bfloat16)
    batch, q_len = spec["batch"], spec["q_len"]
    q = torch.randn((batch * q_len, spec["hq"], d), generator=g, device=device, dtype=torch.bfloat16)
    counts = [-(-n // page) for n in kv_lens]
    width = max(counts)
    rng = np.random.default_rng(seed + 1)
    perm = rng.permutation(pool).astype(np.int32)
    table = np.full((batch, width), -1, dtype=np.int32)
    o = 0
    for r, n in enumerate(counts):
        table[r, :n] = perm[o:o + n]
        o += n
    assert o <= pool
    host = dict(
        q=q.cpu().pin_memory(),
        cu_seqlens_q=(torch.arange(batch + 1, dtype=torch.int32) * q_len).pin_memory(),
        seqused_k=torch.tensor(kv_lens, dtype=torch.int32).pin_memory(),
        block_table=torch.from_numpy(table).pin_memory(),
    )
    case = dict(q=q, k=k, v=v, max_seqlen_q=q_len, cu_seqlens_q=host["cu_seqlens_q"].to(device),
                max_seqlen_k=width * page, seqused_k=host["seqused_k"].to(device),
                block_table=host["block_table"].to(device), softmax_scale=d ** -0.5, causal=True,
                window_size=spec["window"], num_splits=0, return_softmax_lse=spec["lse"],
                out=torch.empty_like(q))
    if spec["sink"]:
        case["s_aux"] = torch.randn(spec["hq"], generator=g, device=device).bfloat16()
    return case, host


def cpu_baseline(spec, kv_lens, seed, budget_s=12.0):
    """The CPU FP32 oracle on the first requests of the workload until about ``budget_s`` seconds are used."""
    from oracle import fa_oracle

    rng = np.random.default_rng(seed)
    hq, hkv, d, page = spec["hq"], spec["hkv"], spec["d"], spec["page"]
    done_bytes, used, n_req, t_total = 0, 0.0, 0, 0.0
    window = spec["window"] or (-1, -1)
    for b, n in enumerate(kv_lens):
        pages = -(-n // page)
        k = fa_oracle.bf16_round(rng.standard_normal((pages, page, hkv, d), dtype=np.float32))
        v = fa_oracle.bf16_round(rng.standard_normal((pages, page, hkv, d), dtype=np.float32))
        q = fa_oracle.bf16_round(rng.standard_normal((spec["q_len"], hq, d), dtype=np.float32))
        table = np.arange(pages, dtype=np.int32)[None, :]
        sink = rng.standard_normal(hq).astype(np.float32) if spec["sink"] else None
        t0 = time.perf_counter()
        fa_oracle.attention(q, k, v, np.array([0, spec["q_len"]], np.int32), seqused_k=np.array([n], np.int32),
                            block_table=table, softmax_scale=d ** -0.5, causal=True, window=window, sink=sink)
        t_total += time.perf_counter() - t0
        done_bytes += algorithmic_bytes(dict(spec, batch=1), [n])
        n_req += 1
        if t_total >= budget_s or n_req >= 16:
            break
    try:
        from threadpoolctl import threadpool_info

        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count() or 1
    return dict(value=done_bytes / t_total / 1e9, unit=spec["unit"], cores=cores, kind="port",
                sample=f"first {n_req} of {spec['batch']} requests of the workload, one pass, {t_total:.1f} s"), t_total


def run_reference(args, spec, rank, world):
    """CPU arm: each step is the oracle over a bounded sample of the batch."""
    if rank != 0:
        return
    kv_lens = draw_lengths(spec, 1729)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    per_step = max(2.0, min(20.0, 120.0 / (steps + warm)))
    for _ in range(min(warm, 1)):
        cpu_baseline(spec, kv_lens, 1729, budget_s=1.0)
    values, samples, total_t = [], None, 0.0
    for _ in range(min(steps, 8)):
        base, t = cpu_baseline(spec, kv_lens, 1729, budget_s=per_step)
        values.append(base["value"])
        samples, total_t = base, total_t + t
    value = statistics.median(values)
    line = dict(impl="reference", metric=spec["metric"], value=value, unit=spec["unit"], n_gpus=args.gpus,
                steps=len(values), warmup=min(warm, 1), ms_per_step=total_t / len(values) * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, **{k: spec[k] for k in ("batch", "q_len", "hq", "hkv", "d", "page")}),
                cpu_baseline=dict(samples, value=value),
                e2e=dict(value=value, unit=spec["unit"], h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_q1", choices=sorted(WORKLOADS))
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    spec = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, spec, rank, world)
        return

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    import atrex
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    runtime.prewarm(device)
    warmup = max(3, args.warmup)
    seed = 1729 + 1000 * rank
    kv_lens = draw_lengths(spec, seed)
    case, host = build_device_case(spec, kv_lens, seed, device)
    case["num_splits"] = args.num_splits
    my_bytes = algorithmic_bytes(spec, kv_lens)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        atrex.flash_attn_varlen_func(**case)

    # ---------------- kernel-resident timing ----------------
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    clocks = sampler.stop()
    elapsed_ms = start.elapsed_time(stop)

    # ---------------- dominant kernel alone (events recorded by the launcher around it) ----------------
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(); ev1.record()
    torch.cuda.synchronize()
    plan_args = (case["q"], case["k"], case["v"], case["out"], None, case["cu_seqlens_q"], None, case["seqused_k"],
                 case["block_table"], None, None, None, case.get("s_aux"), None, case["max_seqlen_q"],
                 case["max_seqlen_k"], case["softmax_scale"], 0.0, True,
                 spec["window"][0] if spec["window"] else -1, spec["window"][1] if spec["window"] else -1,
                 args.num_splits, 0)
    params = runtime.build_params(*plan_args)
    info = runtime.plan(params)
    lse_buf = torch.empty((spec["hq"], case["q"].shape[0]), dtype=torch.float32, device=device) if spec["lse"] else None
    params = runtime.build_params(*plan_args[:4], lse_buf, *plan_args[5:])
    params.profile_event_begin, params.profile_event_end = ev0.cuda_event, ev1.cuda_event
    workspace = torch.empty(max(1, info.workspace_bytes), dtype=torch.uint8, device=device)
    lib = runtime.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    # Calls are queued back to back, each with its own event pair, so that an event is recorded when the previous
    # call's last kernel retires and the attention kernel starts right behind it (no idle-GPU launch latency inside
    # the measured interval).
    n_timed = min(args.steps, 50)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_timed)]
    for a, b in pairs:
        a.record(); b.record()
    torch.cuda.synchronize()
    for i in range(warmup + n_timed):
        if i >= warmup:
            a, b = pairs[i - warmup]
            params.profile_event_begin, params.profile_event_end = a.cuda_event, b.cuda_event
        runtime.raise_for_status(lib.atrex_fa_sm100_forward(ctypes.byref(params), workspace.data_ptr(),
                                                             workspace.numel(), stream))
    torch.cuda.synchronize()
    kernel_ms = [a.elapsed_time(b) for a, b in pairs]
    kernel_ms_avg = sum(kernel_ms) / len(kernel_ms)

    # ---------------- end to end: host inputs in, host result out ----------------
    dev_in = {name: case[name] for name in host}
    out_host = torch.empty(case["out"].shape, dtype=case["out"].dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        for name, src in host.items():
            dev_in[name].copy_(src, non_blocking=True)
        out = atrex.flash_attn_varlen_func(**case)
        out = out[0] if isinstance(out, tuple) else out
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(warmup):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(args.steps):
        e2e_step()
    e2.record()
    barrier()
    # every step ends with a host-side stream synchronise, so wall clock and device events bracket the same work
    e2e_ms = max(s2.elapsed_time(e2), (time.perf_counter() - t0) * 1e3)

    status = runtime.check_device_status(device)

    # ---------------- reduce over ranks ----------------
    stats = torch.tensor([elapsed_ms, e2e_ms, kernel_ms_avg], dtype=torch.float64, device=device)
    total_bytes = torch.tensor([float(my_bytes)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms, kernel_ms_avg = stats.tolist()
    total = total_bytes.item()

    if rank == 0:
        peaks = measured_peaks()
        value = total * args.steps / (elapsed_ms * 1e-3) / 1e9
        achieved = my_bytes / (kernel_ms_avg * 1e-3) / 1e9
        line = dict(
            metric=spec["metric"], value=value, unit=spec["unit"], n_gpus=world, steps=args.steps, warmup=warmup,
            ms_per_step=elapsed_ms / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
            dtype="bf16", data="synthetic",
            config=dict(workload=args.workload, batch_per_gpu=spec["batch"], q_len=spec["q_len"],
                        num_q_heads=spec["hq"], num_kv_heads=spec["hkv"], head_dim=spec["d"],
                        page_size=spec["page"], kv_len_range=[spec["kv_lo"], spec["kv_hi"]], pool_pages=spec["pool"],
                        num_splits=info.num_splits, sharding="one batch per rank, no collective",
                        l2="inputs larger than L2 (K/V touched per step >> 126 MB)",
                        algorithmic_bytes_per_step_per_gpu=my_bytes),
            roofline=dict(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s",
                          frac=achieved / peaks["hbm_gbs"], traffic=None, peak_source=peaks["source"],
                          frac_of_nominal_8tbs=achieved / 8000.0, kernel="atrex_sm100_fwd_mma_kernel",
                          kernel_ms=kernel_ms_avg),
            e2e=dict(value=total * args.steps / (e2e_ms * 1e-3) / 1e9, unit=spec["unit"], h2d_bytes_per_step=h2d,
                     d2h_bytes_per_step=d2h,
                     note="per-step inputs (q, cu_seqlens_q, seqused_k, block_table) copied from pinned host memory, "
                          "O copied back; the paged KV cache is resident device state"),
            gpu_launches=info.kernel_launches * args.steps,
            clocks=dict(sm_mhz=clocks["sm_mhz"], sm_max_mhz=clocks["sm_max_mhz"], reasons=clocks["reasons"]),
            device_status=status,
        )
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(spec, kv_lens, seed)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
